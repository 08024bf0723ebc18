// bfloat16 matrix products on the 5th-generation tensor cores (sm_100a): TMA loads into
// 128-byte-swizzled shared memory, tcgen05.mma issued by one thread with the accumulator in
// tensor memory, tcgen05.ld for the epilogue.
//
//   D[m, n] = sum_k X[m, k] * W[n, k]        X: [M, K] activations, W: [N, K] weights, both K-major
//
// Two orientations share the kernel.  "tokens as rows" (prefill): the 128 accumulator lanes
// are token rows, a CTA owns a 128 x BN tile of D.  "weights as rows" (decode, few tokens):
// the 128 lanes are weight rows and the tokens are the MMA's N (16..64), so that a step with
// 1..64 tokens still streams every weight once with full 128-row MMAs; K may be split
// across CTAs (grid.z), each split writing its own 32-bit partial sums, which the next
// add+RMSNorm kernel adds in index order (no atomics: the result never depends on timing).
// Epilogues: + bias, 32-bit output, accumulate into the 32-bit residual stream, and
// SwiGLU on row-interleaved gate/up weights.
//
// maeddesg/ROCmForge's counterparts are its RDNA-WMMA prefill GEMMs (hip_kernels/wmma/
// wmma_gemm_tiled.hip:57-195: 64x64x16 tiles, FP16 operands, FP32 accumulate) and its decode
// GEMV family (hip_kernels/quant/q4_0_gemv.hip, fused variants per src/gpu/ops.rs:509-880);
// the fusion pattern (bias in the QKV product, gate+up+SiLU in one launch, residual in the
// O and down products) is kept, the tiling and the instruction path are sm_100a's own.
//
// Every wait on an mbarrier is bounded: when it runs out the CTA records a code in the
// global status word, all roles leave their loops, tensor memory is freed and the kernel
// returns; the host reads the word and raises.
#include <cuda.h>
#include "common.cuh"

#define TC_BM 128
#define TC_BK 64
#define TC_THREADS 192
#define TC_WAIT_LIMIT_NS 2000000000ULL      // 2 s

enum { EPI_STORE = 0, EPI_F32 = 1, EPI_RESIDUAL = 2, EPI_SWIGLU = 3, EPI_PARTIAL = 4 };

struct TcParams {
    void* out;              // see the epilogue
    const void* bias;       // [N] or null
    int bias_is_f32;
    int M, N, K;            // tokens, weight rows, inner size
    int ldo;                // row stride of out, in elements
    int mode;
    int k_blocks_per_split; // in units of TC_BK
    long long partial_stride;   // elements between the partial sums of two splits
    int* status;            // device word: 0 = fine
};

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait: false when the limit ran out or another role gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    for (;;) {
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (global_ns() - t0 > TC_WAIT_LIMIT_NS) { *abort_flag = 1; return false; }
    }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
__device__ __forceinline__ void tcgen05_alloc(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tcgen05_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tcgen05_mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                 uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tcgen05_ld32(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tcgen05_ld16(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tcgen05_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (64 bf16) wide,
// written by TMA with the 128-byte swizzle: 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);          // start address, 16-byte units
    d |= (uint64_t)1 << 16;                          // leading-dimension byte offset (unused with swizzle): 1
    d |= (uint64_t)(1024 >> 4) << 32;                // stride between 8-row groups
    d |= (uint64_t)1 << 46;                          // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                          // 128-byte swizzle
    return d;
}
// Instruction descriptor: bf16 x bf16 -> f32, both operands K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t make_idesc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
}

// ---------------------------------------------------------------- the kernel
// SWAP = false: map A = X (rows are tokens), map B = W;  SWAP = true: map A = W, map B = X.
template <int BN, bool SWAP, int STAGES>
__global__ void __launch_bounds__(TC_THREADS, SWAP ? 2 : 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, TcParams p) {
    constexpr uint32_t A_BYTES = TC_BM * TC_BK * 2;
    constexpr uint32_t B_BYTES = BN * TC_BK * 2;
    constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);     // full[S], empty[S], tmem_full
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 1);
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile_a = blockIdx.y, tile_b = blockIdx.x, split = blockIdx.z;
    const int kb_total = (p.K + TC_BK - 1) / TC_BK;
    const int kb_begin = split * p.k_blocks_per_split;
    int kb_end = kb_begin + p.k_blocks_per_split;
    if (kb_end > kb_total) kb_end = kb_total;
    const int n_kb = kb_end - kb_begin;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&bars[s]), 1);
            mbar_init(smem_u32(&bars[STAGES + s]), 1);
        }
        mbar_init(smem_u32(&bars[2 * STAGES]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
    }
    if (warp == 1) {
        tcgen05_alloc(smem_u32(tmem_slot), TMEM_COLS);
        tcgen05_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- producer: one thread feeds the ring of stages
        if (lane == 0) {
            for (int i = 0; i < n_kb; ++i) {
                const int s = i % STAGES;
                const uint32_t parity = ((i / STAGES) & 1) ^ 1;
                if (!mbar_wait(smem_u32(&bars[STAGES + s]), parity, &abort_flag)) break;
                const uint32_t full = smem_u32(&bars[s]);
                mbar_expect_tx(full, STAGE_BYTES);
                const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
                const int k0 = (kb_begin + i) * TC_BK;
                tma_load_2d(sa, &map_a, k0, tile_a * TC_BM, full);
                tma_load_2d(sa + A_BYTES, &map_b, k0, tile_b * BN, full);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: one thread, accumulator in tensor memory
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(BN);
            bool ok = true;
            for (int i = 0; i < n_kb && ok; ++i) {
                const int s = i % STAGES;
                ok = mbar_wait(smem_u32(&bars[s]), (i / STAGES) & 1, &abort_flag);
                if (!ok) break;
                tcgen05_fence_after();
                const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
                const uint64_t da = make_smem_desc(sa), db = make_smem_desc(sa + A_BYTES);
#pragma unroll
                for (int k = 0; k < TC_BK / 16; ++k)         // 16 bf16 = 32 bytes = 2 descriptor units per step
                    tcgen05_mma_bf16(tmem_base, da + 2 * k, db + 2 * k, idesc, (i | k) ? 1u : 0u);
                tcgen05_commit(smem_u32(&bars[STAGES + s]));  // frees the stage when these MMAs are done
            }
            tcgen05_commit(smem_u32(&bars[2 * STAGES]));      // accumulator complete
        }
    } else {
        // ---------------- epilogue: four warps, one quarter of the 128 lanes each
        const int quarter = warp & 3;
        const bool ok = mbar_wait(smem_u32(&bars[2 * STAGES]), 0, &abort_flag);
        tcgen05_fence_after();
        if (ok && n_kb > 0) {
            const int row_a = tile_a * TC_BM + quarter * 32 + lane;        // index along map A's rows
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16);
            constexpr int CH = BN < 32 ? 16 : 32;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += CH) {
                uint32_t r[32];
                if (CH == 32) tcgen05_ld32(taddr + c0, r); else tcgen05_ld16(taddr + c0, r);
                tcgen05_wait_ld();
                if (!SWAP) {
                    // lane = token m, registers = 32 consecutive weight rows n
                    const int m = row_a, n0 = tile_b * BN + c0;
                    if (m < p.M) {
                        if (p.mode == EPI_SWIGLU) {
                            __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)m * p.ldo + (n0 >> 1);
#pragma unroll
                            for (int j = 0; j < CH; j += 2)
                                if (n0 + j + 1 < p.N) {
                                    const float g = __uint_as_float(r[j]), u = __uint_as_float(r[j + 1]);
                                    o[j >> 1] = __float2bfloat16_rn(g / (1.f + expf(-g)) * u);
                                }
                        } else {
#pragma unroll
                            for (int j = 0; j < CH; ++j) {
                                const int n = n0 + j;
                                if (n < p.N) {
                                    float v = __uint_as_float(r[j]);
                                    if (p.bias) v += load_vec(p.bias, p.bias_is_f32, n);
                                    const size_t o = (size_t)m * p.ldo + n;
                                    if (p.mode == EPI_STORE) reinterpret_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(v);
                                    else if (p.mode == EPI_F32) reinterpret_cast<float*>(p.out)[o] = v;
                                    else reinterpret_cast<float*>(p.out)[o] += v;
                                }
                            }
                        }
                    }
                } else {
                    // lane = weight row n, registers = consecutive tokens m
                    const int n = row_a, m0 = tile_b * BN + c0;
                    const float b = (p.bias && n < p.N) ? load_vec(p.bias, p.bias_is_f32, n) : 0.f;
#pragma unroll
                    for (int j = 0; j < CH; ++j) {
                        const int m = m0 + j;
                        float v = __uint_as_float(r[j]) + b;
                        if (p.mode == EPI_SWIGLU) {
                            // gate in even lanes, up in the odd lane beside it
                            const float u = __shfl_down_sync(0xffffffffu, v, 1);
                            if (!(lane & 1) && m < p.M && n + 1 < p.N)
                                reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)m * p.ldo + (n >> 1)] =
                                    __float2bfloat16_rn(v / (1.f + expf(-v)) * u);
                        } else if (m < p.M && n < p.N) {
                            const size_t o = (size_t)m * p.ldo + n;
                            if (p.mode == EPI_STORE) reinterpret_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(v);
                            else if (p.mode == EPI_F32) reinterpret_cast<float*>(p.out)[o] = v;
                            else if (p.mode == EPI_RESIDUAL) reinterpret_cast<float*>(p.out)[o] += v;
                            else reinterpret_cast<float*>(p.out)[(size_t)split * p.partial_stride + o] = v;
                        }
                    }
                }
            }
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        tcgen05_dealloc(tmem_base, TMEM_COLS);
    }
    if (threadIdx.x == 0 && abort_flag && p.status) atomicExch(p.status, 1);
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

// 2-D map of a row-major bf16 matrix [rows, cols] with row stride ld (elements); box = [box_rows, 64].
static int make_map(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return RF_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(base) & 15) || (ld * 2) % 16) return RF_ERR_BAD_ARG;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {TC_BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : RF_ERR_BAD_ARG;
}

template <int BN, bool SWAP, int STAGES>
static int launch_cfg(const CUtensorMap& ma, const CUtensorMap& mb, const TcParams& p, dim3 grid, cudaStream_t st) {
    constexpr size_t smem = (size_t)STAGES * (TC_BM * TC_BK * 2 + BN * TC_BK * 2) + (2 * STAGES + 1) * 8 + 16 + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, SWAP, STAGES>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    gemm_tc_kernel<BN, SWAP, STAGES><<<grid, TC_THREADS, smem, st>>>(ma, mb, p);
    RF_LAUNCH_CHECK();
    return 0;
}

extern "C" {

// Whether the tensor-core kernel takes this product (else the caller uses the CUDA-core kernel).
int rf_gemm_tc_supported(int M, int N, int K, int mode) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if (K % 8) return 0;                              // TMA needs 16-byte row strides
    if (mode == EPI_SWIGLU && (N % 2)) return 0;
    return encode_fn() != nullptr;
}

// Tokens as rows: out[M, N] (mode STORE / F32 / RESIDUAL) or out[M, N/2] (SWIGLU).
int rf_gemm_tc(const void* X, int ldx, const void* W, const void* bias, int bias_is_f32, void* out, int ldo,
               int M, int N, int K, int mode, int* status, cudaStream_t st) {
    if (!rf_gemm_tc_supported(M, N, K, mode) || mode == EPI_PARTIAL) return RF_ERR_UNSUPPORTED;
    CUtensorMap ma, mb;
    int e;
    TcParams p{out, bias, bias_is_f32, M, N, K, ldo, mode, (K + TC_BK - 1) / TC_BK, 0, status};
    if (N > 128) {
        if ((e = make_map(&ma, X, M, K, ldx, TC_BM)) || (e = make_map(&mb, W, N, K, K, 256))) return e;
        dim3 grid((N + 255) / 256, (M + TC_BM - 1) / TC_BM, 1);
        return launch_cfg<256, false, 4>(ma, mb, p, grid, st);
    }
    if ((e = make_map(&ma, X, M, K, ldx, TC_BM)) || (e = make_map(&mb, W, N, K, K, 128))) return e;
    dim3 grid((N + 127) / 128, (M + TC_BM - 1) / TC_BM, 1);
    return launch_cfg<128, false, 6>(ma, mb, p, grid, st);
}

// Weights as rows, for M <= 64 tokens.  splits > 1 requires mode PARTIAL: out is then
// [splits, M, N] float32 (partial_stride = M * N) and holds the partial sums of each K range.
int rf_gemm_tc_skinny(const void* X, int ldx, const void* W, const void* bias, int bias_is_f32, void* out, int ldo,
                      int M, int N, int K, int mode, int splits, int* status, cudaStream_t st) {
    if (!rf_gemm_tc_supported(M, N, K, mode) || M > 64 || splits < 1) return RF_ERR_UNSUPPORTED;
    if (splits > 1 && mode != EPI_PARTIAL) return RF_ERR_BAD_ARG;
    const int kb = (K + TC_BK - 1) / TC_BK;
    const int per = (kb + splits - 1) / splits;
    if ((splits - 1) * per >= kb) return RF_ERR_BAD_ARG;          // an empty split would leave its partial unwritten
    TcParams p{out, bias, bias_is_f32, M, N, K, ldo, mode, per, (long long)M * ldo, status};
    CUtensorMap ma, mb;
    int e;
    const int bn = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
    if ((e = make_map(&ma, W, N, K, K, TC_BM)) || (e = make_map(&mb, X, M, K, ldx, bn))) return e;
    dim3 grid(1, (N + TC_BM - 1) / TC_BM, splits);
    // stage counts chosen so that two CTAs share an SM: their pipelines overlap each other's
    // start-up and epilogue, and 2 x stages x 16 KB of weight bytes are in flight per SM
    if (bn == 16) return launch_cfg<16, true, 6>(ma, mb, p, grid, st);
    if (bn == 32) return launch_cfg<32, true, 5>(ma, mb, p, grid, st);
    return launch_cfg<64, true, 4>(ma, mb, p, grid, st);
}

}
