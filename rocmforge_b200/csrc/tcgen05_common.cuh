// Shared pieces of the tcgen05 matrix-product kernels: tile constants, the parameter block, inline-PTX
// wrappers (mbarrier, TMA, tensor memory, tcgen05.mma / ld / commit), descriptor builders and the
// epilogue of the "tokens as rows" orientation.
#pragma once
#include <cuda.h>
#include "common.cuh"

#define TC_BM 128
#define TC_BK 64
#define TC_THREADS 192
#define TC_WAIT_LIMIT_NS 2000000000ULL      // 2 s

enum { EPI_STORE = 0, EPI_F32 = 1, EPI_RESIDUAL = 2, EPI_SWIGLU = 3, EPI_PARTIAL = 4, EPI_RESNORM = 5 };

// What the weights-as-rows kernel needs to finish a residual update and prepare the norm that follows it
// (mode EPI_RESNORM), and to apply a norm that was prepared that way to its own input (ss_in).
struct TcNorm {             // 56 bytes: with TcParams and two tensor maps the kernel's parameters are 384 bytes, no more
    // EPI_RESNORM: the K splits of an output tile add their partial sums (in rank order) and the bias into the residual
    // stream (TcParams.out: [M, N] float32, updated in place), and write stream * norm weight in bfloat16 for the next
    // product and the tile's share of every token's sum of squares
    const void* norm_w;         // [N] weight of the norm that follows
    __nv_bfloat16* normed;      // [M, N] out: (stream after the update) * norm weight, not yet divided by the RMS
    float* ss_out;              // [ceil(N/128)][ss_out_stride] out: sum over the tile's columns of stream^2
    // input side: this product's activations are stream * norm weight of a norm prepared as above; row m is
    // scaled by rsqrt(sum_t ss_in[t][m] * ss_inv_width + ss_eps) in the epilogue (the product is linear in it)
    const float* ss_in;         // null: the activations are already normalised
    int norm_w_is_f32;
    int ss_out_stride;
    int ss_in_tiles, ss_in_stride;
    float ss_eps, ss_inv_width;
};

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
    int splits;             // clustered kernel: K parts of the residual epilogue, added in order (1 = none)
};
// (TcNorm travels as a kernel parameter of its own, and only to the kernel variant that uses it.  Inside TcParams it
// took the kernel's parameters from 328 to 416 bytes, and every product of few tokens then needed about 4 us longer:
// measured on the 0.5B shape, a decode step of 1.14 ms became 1.45 ms; up to 384 bytes nothing changes, from 400 on
// the time is lost.)
struct TcNoNorm {};

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


// Epilogue of one 32-column (or 16-column) chunk in the "tokens as rows" orientation: lane = token m,
// registers = CH consecutive weight rows starting at n0.  A thread owns a contiguous piece of its
// output row, so it writes 16 bytes at a time wherever the row and the chunk are aligned for it
// (scalar stores of 2 bytes from 32 lanes to 32 different rows would make the epilogue, not the
// tensor cores, the limit of the kernel).
__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// silu for a bfloat16 result: the hardware exponential and reciprocal are 32-bit with a relative
// error near 1e-6, three orders below the rounding of the output
__device__ __forceinline__ float silu_fast(float g) { return __fdividef(g, 1.f + __expf(-g)); }

// v[0 .. CH) += bias[n0 .. n0 + CH): the bias of CH consecutive output columns (the same values in every lane of a warp
// whose lanes are rows).  Decided once per call and fetched 16 bytes at a time where the piece is whole and aligned: a
// test of pointer and bound per element (32 predicated scalar loads) made the epilogue of a 128 x 256 tile take 8 us
// instead of 2, with or without a bias.
template <int CH>
__device__ __forceinline__ void add_bias_columns(float* v, const void* bias, int is_f32, int n0, int N) {
    if (n0 + CH <= N) {
        if (is_f32) {
            const float* b = reinterpret_cast<const float*>(bias) + n0;
            if (!(reinterpret_cast<uintptr_t>(b) & 15)) {
#pragma unroll
                for (int j = 0; j < CH; j += 4) {
                    const float4 t = *reinterpret_cast<const float4*>(b + j);
                    v[j] += t.x; v[j + 1] += t.y; v[j + 2] += t.z; v[j + 3] += t.w;
                }
                return;
            }
        } else {
            const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(bias) + n0;
            if (!(reinterpret_cast<uintptr_t>(b) & 15)) {
#pragma unroll
                for (int j = 0; j < CH; j += 8) {
                    const uint4 t = *reinterpret_cast<const uint4*>(b + j);       // a bfloat16 is the upper half of a float
                    v[j] += __uint_as_float(t.x << 16);     v[j + 1] += __uint_as_float(t.x & 0xffff0000u);
                    v[j + 2] += __uint_as_float(t.y << 16); v[j + 3] += __uint_as_float(t.y & 0xffff0000u);
                    v[j + 4] += __uint_as_float(t.z << 16); v[j + 5] += __uint_as_float(t.z & 0xffff0000u);
                    v[j + 6] += __uint_as_float(t.w << 16); v[j + 7] += __uint_as_float(t.w & 0xffff0000u);
                }
                return;
            }
        }
    }
#pragma unroll
    for (int j = 0; j < CH; ++j)
        if (n0 + j < N) v[j] += load_vec(bias, is_f32, n0 + j);
}

template <int CH>
__device__ __forceinline__ void epilogue_rows(const TcParams& p, const uint32_t* r, int m, int n0) {
    if (m >= p.M) return;
    const bool whole = n0 + CH <= p.N;
    if (p.mode == EPI_SWIGLU) {
        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)m * p.ldo + (n0 >> 1);
        if (whole && !(reinterpret_cast<uintptr_t>(o) & 15)) {
#pragma unroll
            for (int j = 0; j < CH; j += 16) {
                uint32_t w[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float g0 = __uint_as_float(r[j + 4 * q]), u0 = __uint_as_float(r[j + 4 * q + 1]);
                    const float g1 = __uint_as_float(r[j + 4 * q + 2]), u1 = __uint_as_float(r[j + 4 * q + 3]);
                    w[q] = pack_bf16x2(silu_fast(g0) * u0, silu_fast(g1) * u1);
                }
                *reinterpret_cast<uint4*>(o + (j >> 1)) = make_uint4(w[0], w[1], w[2], w[3]);
            }
            return;
        }
#pragma unroll
        for (int j = 0; j < CH; j += 2)
            if (n0 + j + 1 < p.N) {
                const float g = __uint_as_float(r[j]), u = __uint_as_float(r[j + 1]);
                o[j >> 1] = __float2bfloat16_rn(g / (1.f + expf(-g)) * u);
            }
        return;
    }
    float v[CH];
#pragma unroll
    for (int j = 0; j < CH; ++j) v[j] = __uint_as_float(r[j]);
    if (p.bias) add_bias_columns<CH>(v, p.bias, p.bias_is_f32, n0, p.N);
    const size_t o = (size_t)m * p.ldo + n0;
    if (p.mode == EPI_STORE) {
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + o;
        if (whole && !(reinterpret_cast<uintptr_t>(dst) & 15)) {
#pragma unroll
            for (int j = 0; j < CH; j += 8)
                *reinterpret_cast<uint4*>(dst + j) = make_uint4(pack_bf16x2(v[j], v[j + 1]), pack_bf16x2(v[j + 2], v[j + 3]),
                                                                 pack_bf16x2(v[j + 4], v[j + 5]), pack_bf16x2(v[j + 6], v[j + 7]));
            return;
        }
#pragma unroll
        for (int j = 0; j < CH; ++j) if (n0 + j < p.N) dst[j] = __float2bfloat16_rn(v[j]);
        return;
    }
    float* dst = reinterpret_cast<float*>(p.out) + o;
    if (whole && !(reinterpret_cast<uintptr_t>(dst) & 15)) {
#pragma unroll
        for (int j = 0; j < CH; j += 4) {
            float4 t = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            if (p.mode == EPI_RESIDUAL) {
                const float4 old = *reinterpret_cast<const float4*>(dst + j);
                t.x += old.x; t.y += old.y; t.z += old.z; t.w += old.w;
            }
            *reinterpret_cast<float4*>(dst + j) = t;
        }
        return;
    }
#pragma unroll
    for (int j = 0; j < CH; ++j)
        if (n0 + j < p.N) dst[j] = (p.mode == EPI_RESIDUAL ? dst[j] : 0.f) + v[j];
}

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against libcuda).
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
