// bfloat16 matrix products on the 5th-generation tensor cores (sm_100a): TMA loads into
// 128-byte-swizzled shared memory, tcgen05.mma issued by one thread with the accumulator in
// tensor memory, tcgen05.ld for the epilogue.
//
//   D[m, n] = sum_k X[m, k] * W[n, k]        X: [M, K] activations, W: [N, K] weights, both K-major
//
// Two orientations share the kernel.  "tokens as rows" (prefill): the 128 accumulator lanes
// are token rows, a CTA owns a 128 x BN tile of D.  "weights as rows" (decode, few tokens):
// the 128 lanes are weight rows and the tokens are the MMA's N (16..64), so that a step with
// few tokens (tiles of up to 64) still streams every weight once with full 128-row MMAs; K may be split
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
#include <type_traits>
#include "tcgen05_common.cuh"

// ---------------------------------------------------------------- the kernel
// SWAP = false: map A = X (rows are tokens), map B = W;  SWAP = true: map A = W, map B = X.
// NORM = true (weights-as-rows only): the variant that applies a deferred norm to its input rows (pn.ss_in)
// and/or finishes the residual update and prepares the next norm (EPI_RESNORM); it needs more registers, so the
// ordinary products do not carry it.
template <int BN, bool SWAP, int STAGES, bool NORM = false>
__global__ void __launch_bounds__(TC_THREADS, SWAP ? (STAGES <= 4 && BN == 16 ? 3 : 2) : 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, TcParams p,
               typename std::conditional<NORM, TcNorm, TcNoNorm>::type norm_arg) {
    // the variant without the norm never looks at this (every use below sits behind ``NORM &&``)
    const TcNorm& pn = *reinterpret_cast<const TcNorm*>(&norm_arg);
    constexpr uint32_t A_BYTES = TC_BM * TC_BK * 2;
    constexpr uint32_t B_BYTES = BN * TC_BK * 2;
    constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);     // full[S], empty[S], tmem_full
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 1);
    __shared__ int abort_flag;
    __shared__ float rstd_s[NORM ? BN : 1];                    // 1 / RMS of this tile's tokens (deferred norm of the input)
    __shared__ float ss_w[NORM ? 4 * BN : 1];                  // EPI_RESNORM: the four epilogue warps' sums of squares

    pdl_trigger();
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
            // The weight operand does not depend on the kernel before this one: fill the ring with it at
            // once, wait for that kernel, then add the activation operand to the same stages.
            const int pre = n_kb < STAGES ? n_kb : STAGES;
            for (int i = 0; i < pre; ++i) {
                const uint32_t full = smem_u32(&bars[i]);
                mbar_expect_tx(full, STAGE_BYTES);
                const uint32_t sa = smem_u32(smem + i * STAGE_BYTES);
                const int k0 = (kb_begin + i) * TC_BK;
                if (SWAP) tma_load_2d(sa, &map_a, k0, tile_a * TC_BM, full);
                else tma_load_2d(sa + A_BYTES, &map_b, k0, tile_b * BN, full);
            }
            pdl_wait();
            for (int i = 0; i < pre; ++i) {
                const uint32_t full = smem_u32(&bars[i]);
                const uint32_t sa = smem_u32(smem + i * STAGE_BYTES);
                const int k0 = (kb_begin + i) * TC_BK;
                if (SWAP) tma_load_2d(sa + A_BYTES, &map_b, k0, tile_b * BN, full);
                else tma_load_2d(sa, &map_a, k0, tile_a * TC_BM, full);
            }
            for (int i = pre; i < n_kb; ++i) {
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
        pdl_wait();                                      // the output may still be read by the kernel before us
        if (NORM && pn.ss_in) {
            // the input's norm was left unfinished by the product before us: 1 / RMS of each token of this tile, from
            // the tiles' sums of squares in index order
            const int t = threadIdx.x - 64;
            if (t < BN) {
                const int m = tile_b * BN + t;
                float ss = 0.f;
                if (m < p.M)
                    for (int i = 0; i < pn.ss_in_tiles; ++i) ss += pn.ss_in[(size_t)i * pn.ss_in_stride + m];
                rstd_s[t] = rsqrtf(ss * pn.ss_inv_width + pn.ss_eps);
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
        }
        const bool ok = mbar_wait(smem_u32(&bars[2 * STAGES]), 0, &abort_flag);
        tcgen05_fence_after();
        if (ok && n_kb > 0 && !(NORM && p.mode == EPI_RESNORM)) {
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
                    epilogue_rows<CH>(p, r, row_a, tile_b * BN + c0);
                } else {
                    // lane = weight row n, registers = consecutive tokens m
                    const int n = row_a, m0 = tile_b * BN + c0;
                    const float b = (p.bias && n < p.N && p.mode != EPI_RESNORM) ? load_vec(p.bias, p.bias_is_f32, n) : 0.f;
                    if (m0 >= p.M) break;                // the tile's other columns are padding, not tokens
                    if (NORM && pn.ss_in) {
#pragma unroll
                        for (int j = 0; j < CH; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * rstd_s[c0 + j]);
                    }
                    if (p.mode == EPI_SWIGLU) {
                        // gate in even lanes, up in the odd lane beside it.  Two tokens at a time: the even lane
                        // finishes token j (it gets that token's up), the odd lane token j + 1 (it gets its gate),
                        // so every lane evaluates one silu per pair of tokens and every lane stores.
                        const bool odd = lane & 1;
#pragma unroll
                        for (int j = 0; j < CH; j += 2) {
                            const float v0 = __uint_as_float(r[j]) + b, v1 = __uint_as_float(r[j + 1]) + b;
                            const float got = __shfl_xor_sync(0xffffffffu, odd ? v0 : v1, 1);
                            const float g = odd ? got : v0, u = odd ? v1 : got;
                            const int m = m0 + j + (odd ? 1 : 0);
                            if (m < p.M && (n | 1) < p.N)
                                reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)m * p.ldo + (n >> 1)] =
                                    __float2bfloat16_rn(silu_fast(g) * u);
                        }
                    } else if (n < p.N) {
                        // the mode, the output's base and the number of tokens that exist are settled once per chunk: a
                        // token then costs an add and a store (settling them per element made a chunk of 32 tokens take
                        // 1.2 us, half of a small product's time at 64 tokens)
                        const int m_cnt = min(CH, p.M - m0);
                        const size_t o0 = (size_t)m0 * p.ldo + n;
                        if (p.mode == EPI_STORE) {
                            __nv_bfloat16* ob = reinterpret_cast<__nv_bfloat16*>(p.out) + o0;
#pragma unroll
                            for (int j = 0; j < CH; ++j)
                                if (j < m_cnt) ob[(size_t)j * p.ldo] = __float2bfloat16_rn(__uint_as_float(r[j]) + b);
                        } else if (p.mode == EPI_RESIDUAL) {
                            float* of = reinterpret_cast<float*>(p.out) + o0;
#pragma unroll
                            for (int j = 0; j < CH; ++j)
                                if (j < m_cnt) of[(size_t)j * p.ldo] += __uint_as_float(r[j]) + b;
                        } else {                         // F32, or a split's partial sums (PARTIAL, RESNORM)
                            float* of = reinterpret_cast<float*>(p.out) + o0 +
                                        (p.mode == EPI_F32 ? (size_t)0 : (size_t)split * p.partial_stride);
#pragma unroll
                            for (int j = 0; j < CH; ++j)
                                if (j < m_cnt) of[(size_t)j * p.ldo] = __uint_as_float(r[j]) + b;
                        }
                    }
                }
            }
        }
    }
    if (NORM && p.mode == EPI_RESNORM) {
        // ---- the K splits of an output tile are one thread-block cluster (along grid.z).  Every CTA owns BN / S of the
        // tile's tokens: the others push their partial sums of those tokens into its shared memory, it adds them in
        // rank order to the 32-bit stream and prepares the norm.  Nothing goes through global memory, and the order of
        // the sum is the ranks', whatever the timing.
        const int S = (int)gridDim.z, TS = BN / S;
        uint32_t rank;
        asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
        float* recv = reinterpret_cast<float*>(smem);                // [S senders][TS tokens][128 rows], where the ring lay
        // 1. every CTA of the cluster has finished its products: its ring is free to receive
        tcgen05_fence_before();
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        tcgen05_fence_after();
        const int quarter = warp & 3, row = quarter * 32 + lane;
        if (warp >= 2 && !abort_flag && n_kb > 0) {
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16);
            constexpr int CH = BN < 32 ? 16 : 32;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += CH) {
                uint32_t r[32];
                if (CH == 32) tcgen05_ld32(taddr + c0, r); else tcgen05_ld16(taddr + c0, r);
                tcgen05_wait_ld();
#pragma unroll
                for (int j = 0; j < CH; ++j) {
                    const int tok = c0 + j, owner = tok / TS;
                    float v = __uint_as_float(r[j]);
                    if (pn.ss_in) v *= rstd_s[tok];
                    uint32_t raddr;
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(raddr)
                                 : "r"(smem_u32(recv + ((size_t)(rank * TS + (tok - owner * TS)) * TC_BM + row))), "r"(owner));
                    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(raddr), "f"(v) : "memory");
                }
            }
        }
        // 2. every push has landed
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        if (warp >= 2) {
            const int n = tile_a * TC_BM + row, m0 = tile_b * BN + (int)rank * TS;
            const bool n_ok = n < p.N;
            const float b = (p.bias && n_ok) ? load_vec(p.bias, p.bias_is_f32, n) : 0.f;
            const float wn = n_ok ? load_vec(pn.norm_w, pn.norm_w_is_f32, n) : 0.f;
            float* stream = reinterpret_cast<float*>(p.out);
            for (int t0 = 0; t0 < TS; t0 += 8) {                         // eight tokens' stream values in flight at once
                float hv[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int m = m0 + t0 + u;
                    hv[u] = (t0 + u < TS && m < p.M && n_ok) ? stream[(size_t)m * p.ldo + n] : 0.f;
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int tk = t0 + u, m = m0 + tk;
                    if (tk >= TS) break;                                 // uniform over the CTA
                    float sq = 0.f;
                    if (m < p.M && n_ok && !abort_flag) {
                        const size_t o = (size_t)m * p.ldo + n;
                        float v = hv[u];
                        for (int s2 = 0; s2 < S; ++s2) v += recv[((size_t)s2 * TS + tk) * TC_BM + row];      // ranks in order
                        v += b;
                        stream[o] = v;
                        pn.normed[o] = __float2bfloat16_rn(v * wn);
                        sq = v * v;
                    }
                    sq = warp_sum(sq);
                    if (lane == 0) ss_w[quarter * BN + tk] = sq;
                }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            const int t = threadIdx.x - 64;
            if (t < TS && m0 + t < p.M)
                pn.ss_out[(size_t)tile_a * pn.ss_out_stride + m0 + t] = (ss_w[t] + ss_w[BN + t]) + (ss_w[2 * BN + t] + ss_w[3 * BN + t]);
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
template <int BN, bool SWAP, int STAGES, bool NORM = false>
static int launch_cfg(const CUtensorMap& ma, const CUtensorMap& mb, const TcParams& p, dim3 grid, cudaStream_t st,
                      const TcNorm* norm = nullptr, int cluster_z = 1) {
    constexpr size_t smem = (size_t)STAGES * (TC_BM * TC_BK * 2 + BN * TC_BK * 2) + (2 * STAGES + 1) * 8 + 16 + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, SWAP, STAGES, NORM>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    typename std::conditional<NORM, TcNorm, TcNoNorm>::type extra{};
    if constexpr (NORM) extra = *norm;
    if (cluster_z > 1) {                             // the K splits of a tile as one cluster
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(TC_THREADS);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = st;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = cluster_z;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = g_rf_pdl ? 2 : 1;
        cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc_kernel<BN, SWAP, STAGES, NORM>, ma, mb, p, extra);
        if (e != cudaSuccess) return (int)e;
        RF_LAUNCH_CHECK();
        return 0;
    }
    rf_launch(gemm_tc_kernel<BN, SWAP, STAGES, NORM>, grid, dim3(TC_THREADS), smem, st, ma, mb, p, extra);
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
    if (!rf_gemm_tc_supported(M, N, K, mode) || mode == EPI_PARTIAL || mode == EPI_RESNORM) return RF_ERR_UNSUPPORTED;
    CUtensorMap ma, mb;
    int e;
    TcParams p{out, bias, bias_is_f32, M, N, K, ldo, mode, (K + TC_BK - 1) / TC_BK, 0, status, 1};
    if (N > 128) {
        if ((e = make_map(&ma, X, M, K, ldx, TC_BM)) || (e = make_map(&mb, W, N, K, K, 256))) return e;
        dim3 grid((N + 255) / 256, (M + TC_BM - 1) / TC_BM, 1);
        return launch_cfg<256, false, 4>(ma, mb, p, grid, st);
    }
    if ((e = make_map(&ma, X, M, K, ldx, TC_BM)) || (e = make_map(&mb, W, N, K, K, 128))) return e;
    dim3 grid((N + 127) / 128, (M + TC_BM - 1) / TC_BM, 1);
    return launch_cfg<128, false, 6>(ma, mb, p, grid, st);
}

// Weights as rows, for M <= 256 tokens in tiles of up to 128 (the tiles of one weight tile are neighbours in the grid,
// so the weight comes from memory once and from L2 after that).  splits > 1 requires mode PARTIAL or RESNORM: out is then
// [splits, M, N] float32 (partial_stride = M * N) and holds the partial sums of each K range.
//
// ss_in (optional): the activations X are (residual stream * norm weight) of a norm that the product before left
// unfinished; ss_in [ss_in_tiles][ss_in_stride] holds the tiles' sums of squares of the stream, and every output row m
// is scaled by rsqrt(sum_t ss_in[t][m] / K + ss_eps).
// Mode RESNORM (splits = 1, 2, 4 or 8: the splits of an output tile are one thread-block cluster and add their
// partial sums through each other's shared memory): resid [M, N] += the product (+ bias), normed [M, N] = resid *
// norm_w in bfloat16, ss_out [ceil(N/128)][ss_out_stride] = each weight tile's sum of resid^2 per token; out is not used.
int rf_gemm_tc_skinny_ex(const void* X, int ldx, const void* W, const void* bias, int bias_is_f32, void* out, int ldo,
                         int M, int N, int K, int mode, int splits, const float* ss_in, int ss_in_tiles,
                         int ss_in_stride, float ss_eps, float* resid, const void* norm_w, int norm_w_is_f32,
                         void* normed, float* ss_out, int ss_out_stride, int* status, cudaStream_t st) {
    if (!rf_gemm_tc_supported(M, N, K, mode) || M > 256 || splits < 1) return RF_ERR_UNSUPPORTED;
    if (splits > 1 && mode != EPI_PARTIAL && mode != EPI_RESNORM) return RF_ERR_BAD_ARG;
    if (mode == EPI_RESNORM && (!resid || !norm_w || !normed || !ss_out || ldo != N || ss_out_stride < M))
        return RF_ERR_BAD_ARG;
    // the splits of a tile form a cluster whose CTAs share the tile's tokens: 1, 2, 4 or 8 of them
    if (mode == EPI_RESNORM && splits != 1 && splits != 2 && splits != 4 && splits != 8) return RF_ERR_BAD_ARG;
    if (ss_in && (ss_in_tiles <= 0 || ss_in_stride < M)) return RF_ERR_BAD_ARG;
    const int kb = (K + TC_BK - 1) / TC_BK;
    const int per = (kb + splits - 1) / splits;
    if ((splits - 1) * per >= kb) return RF_ERR_BAD_ARG;          // an empty split would leave its partial unwritten
    TcParams p{mode == EPI_RESNORM ? (void*)resid : out, bias, bias_is_f32, M, N, K, ldo, mode, per, (long long)M * ldo, status, 1};
    const TcNorm nrm = TcNorm{norm_w, reinterpret_cast<__nv_bfloat16*>(normed), ss_out, ss_in, norm_w_is_f32, ss_out_stride,
                              ss_in_tiles, ss_in_stride, ss_eps, 1.0f / (float)K};
    static_assert(sizeof(TcParams) + sizeof(TcNorm) <= 128, "two tensor maps and these must stay within 384 bytes");
    CUtensorMap ma, mb;
    int e;
    const int bn = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
    if ((e = make_map(&ma, W, N, K, K, TC_BM)) || (e = make_map(&mb, X, M, K, ldx, bn))) return e;
    dim3 grid((M + bn - 1) / bn, (N + TC_BM - 1) / TC_BM, splits);      // token tiles fastest: they share a weight tile in L2
    // stage counts chosen so that two CTAs share an SM (three with up to 16 tokens: 3 x 4 stages hold as many weight
    // bytes as 2 x 6, and the third place takes a CTA of the next product while this one still runs: 2.791 against
    // 2.802 ms a decode step of the 7B shape at batch 8, 2.737 against 2.756 ms at batch 1): their pipelines overlap each
    // other's start-up and epilogue, and 2 x stages x 16 KB of weight bytes are in flight per SM.  (128 tokens:
    // two CTAs with three 32 KB stages each, 5.09 ms a decode step of the 7B shape; one CTA with six
    // stages 6.46 ms; two tiles of 64 tokens sharing the weight tile through L2 5.65 ms.)
    if (ss_in || mode == EPI_RESNORM) {
        const int cz = mode == EPI_RESNORM ? splits : 1;
        if (bn == 16) return launch_cfg<16, true, 6, true>(ma, mb, p, grid, st, &nrm, cz);
        if (bn == 32) return launch_cfg<32, true, 5, true>(ma, mb, p, grid, st, &nrm, cz);
        if (bn == 64) return launch_cfg<64, true, 4, true>(ma, mb, p, grid, st, &nrm, cz);
        return launch_cfg<128, true, 3, true>(ma, mb, p, grid, st, &nrm, cz);
    }
    if (bn == 16) return launch_cfg<16, true, 4>(ma, mb, p, grid, st);
    if (bn == 32) return launch_cfg<32, true, 5>(ma, mb, p, grid, st);
    if (bn == 64) return launch_cfg<64, true, 4>(ma, mb, p, grid, st);
    return launch_cfg<128, true, 3>(ma, mb, p, grid, st);
}

int rf_gemm_tc_skinny(const void* X, int ldx, const void* W, const void* bias, int bias_is_f32, void* out, int ldo,
                      int M, int N, int K, int mode, int splits, int* status, cudaStream_t st) {
    if (mode == EPI_RESNORM) return RF_ERR_BAD_ARG;
    return rf_gemm_tc_skinny_ex(X, ldx, W, bias, bias_is_f32, out, ldo, M, N, K, mode, splits, nullptr, 0, 0, 0.f,
                                nullptr, nullptr, 0, nullptr, nullptr, 0, status, st);
}

}
