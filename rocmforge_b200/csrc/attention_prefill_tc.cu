// Prefill attention on the 5th-generation tensor cores: both products of the tiled, causal,
// grouped-query attention run as tcgen05.mma with their accumulators in tensor memory.
//
// A CTA owns 128 consecutive new tokens of one sequence and one query head.  Per cache page (64 keys,
// brought in by TMA with the 128-byte swizzle, two stages):
//     S[128 x 64]   = Q K^T              tcgen05.mma, A = Q tile, B = key tile, both K-major
//     softmax       : four warps, one thread per query row: the row of S comes out of tensor memory
//                     with tcgen05.ld, so its maximum and sum need no shuffles; 32-bit throughout
//     P (bfloat16)  -> tensor memory, in place of the scores it was made from: the A operand of the next product
//     O[128 x hd]  += P V                tcgen05.mma, B = value tile read as an MN-major operand
// O stays in tensor memory for the whole row tile.  The reference point of the exponentials is only
// moved when a row's maximum has grown by more than 8 (in log2 units): weights then stay below 2^8,
// far inside bfloat16 and float32 range, and O has to be rescaled (read from tensor memory, scaled,
// written back) only on those rare steps instead of on every one.  Shared and tensor memory are sized so
// that two CTAs share an SM: while one is in its softmax the other keeps the tensor cores busy.
//
// Same mathematics and page skipping as attention_prefill.cu (the mma.sync kernel, which stays for
// comparison and as the fallback); counterpart in maeddesg/ROCmForge:
// hip_kernels/wmma/wmma_attention_prefill.hip:386-671.
#include "tcgen05_common.cuh"

#define AT_THREADS 192
#define AT_BM 128
#define AT_BN 64

__device__ __forceinline__ float at_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Weights are rounded to bfloat16 with integer arithmetic (add half an ulp, keep the upper 16 bits): the
// conversion instruction shares the special-function unit with ex2.  Two variants that measured SLOWER here
// and were dropped: a share of the exponentials as a polynomial on the FMA pipe (763 -> 734 TFLOP/s at 8,192
// tokens), and two softmax threads per row (763 -> 435): the softmax warps lack neither ex2 throughput nor
// threads; what helped was letting the next page's scores be computed while they work (see issue_s).
__device__ __forceinline__ uint32_t at_pack_bf16x2(float a, float b) {      // a, b >= 0 and finite
    return __byte_perm(__float_as_uint(a) + 0x8000u, __float_as_uint(b) + 0x8000u, 0x7632);
}

__device__ __forceinline__ void tcgen05_st32(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
// A operand in tensor memory (128 lanes = rows, two bfloat16 per 32-bit column), B through a shared-memory descriptor.
__device__ __forceinline__ void tcgen05_mma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                                    uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tcgen05_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void at_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Descriptor of an MN-major operand tile with the 128-byte swizzle: rows are K (keys), 128 bytes = 64
// elements of N (head dimensions) per row; 8-row groups 1024 bytes apart (stride byte offset), the next
// block of 64 N-elements `lbo_bytes` further (leading byte offset).
__device__ __forceinline__ uint64_t make_smem_desc_mn(uint32_t addr, uint32_t lbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// bf16 x bf16 -> f32, M = 128, N = n, A K-major, B K-major (b_mn = 0) or MN-major (b_mn = 1)
__host__ __device__ constexpr uint32_t at_idesc(int n, int b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(AT_BM >> 4) << 24);
}

template <int HD>
__global__ void __launch_bounds__(AT_THREADS, 2)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out, int out_stride,
                            const int* __restrict__ tiles, const int* __restrict__ seq_slot,
                            const int* __restrict__ seq_start, const int* __restrict__ seq_nnew,
                            const int* __restrict__ cu_q, const int* __restrict__ block_table, int max_pages,
                            int nh, int nkv, float scale, int window, int* __restrict__ status) {
    constexpr int HALVES = HD / 64;                     // 128-byte column blocks of a head
    constexpr uint32_t QH_BYTES = AT_BM * 128;          // one column block of the Q tile (also the P tile)
    constexpr uint32_t Q_BYTES = HALVES * QH_BYTES;
    constexpr uint32_t KH_BYTES = AT_BN * 128;          // one column block of a page of keys (or values)
    constexpr uint32_t KV_BYTES = HALVES * KH_BYTES;
    constexpr uint32_t TMEM_COLS = 256;                 // S (two buffers): columns 0..127, O: columns 128..128+HD-1
    extern __shared__ __align__(1024) uint8_t smem[];   // no static shared memory: the window starts aligned
    uint8_t* q_s = smem;                                 // [HALVES][128][128 B]
    uint8_t* kv_s = q_s + Q_BYTES;                       // [2 stages][K | V][HALVES][64][128 B]
    uint64_t* bars = reinterpret_cast<uint64_t*>(kv_s + 4 * KV_BYTES);
    // q_full, k_full[2], k_free[2], s_full[2], p_ready[2], pv_done[2], v_full[2], v_free[2].  Keys and values of a stage have
    // barriers of their own: a page's keys are done with when its scores are computed, a whole softmax before its values
    // are, and the next-but-one page's keys can be on their way that much earlier (with one barrier for both, the softmax
    // warps waited a third of every step for scores whose keys had been asked for too late).
    // p_ready and pv_done alternate between two barriers from page to page.  A wait names a phase by its parity alone, so
    // a barrier must never complete two phases between two looks of one of its waiters.  A softmax thread hands P(t) over
    // BEFORE it looks at the P V of page t - 1 (unless it has to rescale O), so with one barrier each, a warp that was slow
    // between those two instructions found P V(t - 1) and P V(t) both complete, read the parity as "not yet" and waited
    // for a product that needed its own next arrival (and the MMA thread the same with the arrivals of pages t and t + 1):
    // once in some thousand launches a CTA stood still until its wait ran out.  With two barriers the next phase of the
    // one a thread waits on needs that thread's arrival of the page after next, which comes after the wait.
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
    int& abort_flag = *reinterpret_cast<int*>(tmem_slot + 1);
    const uint32_t b_q = smem_u32(&bars[0]), b_kfull = smem_u32(&bars[1]), b_kfree = smem_u32(&bars[3]);
    const uint32_t b_sfull = smem_u32(&bars[5]), b_pready = smem_u32(&bars[7]), b_pvdone = smem_u32(&bars[9]);
    const uint32_t b_vfull = smem_u32(&bars[11]), b_vfree = smem_u32(&bars[13]);

    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // heavy tiles first: the table is sorted by the keys a tile sees and walked backwards, and the heads are the
    // fast grid dimension, so the tiles with the most keys of ALL heads are handed out before any light one
    // (tiles fastest, a head after the other, left the heavy tiles of the last heads to the end of the kernel)
    const int tile_idx = gridDim.y - 1 - blockIdx.y;
    const int seq = tiles[2 * tile_idx], q0 = tiles[2 * tile_idx + 1];
    const int head = blockIdx.x, kvh = head / (nh / nkv);
    const int start = seq_start[seq], n_new = seq_nnew[seq];
    const int* bt = block_table + (size_t)seq_slot[seq] * max_pages;
    const int row_base = cu_q[seq] + q0;
    int rows_here = n_new - q0; if (rows_here > AT_BM) rows_here = AT_BM;
    const int pos_first = start + q0, pos_last = pos_first + rows_here - 1, seq_last = start + n_new - 1;
    const int lo_first = (window > 0 && pos_first - window + 1 > 0) ? pos_first - window + 1 : 0;
    const int kt_lo = lo_first / AT_BN, kt_hi = pos_last / AT_BN;      // AT_BN == RF_PAGE: a tile is a page
    const int n_kt = kt_hi - kt_lo + 1;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(b_q, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(b_kfull + 8 * s, 1); mbar_init(b_kfree + 8 * s, 1);
            mbar_init(b_vfull + 8 * s, 1); mbar_init(b_vfree + 8 * s, 1);
        }
        mbar_init(b_sfull, 1);
        mbar_init(b_sfull + 8, 1);
        mbar_init(b_pready, 128); mbar_init(b_pready + 8, 128);
        mbar_init(b_pvdone, 1); mbar_init(b_pvdone + 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
    }
    if (warp == 1) {
        tcgen05_alloc(smem_u32(tmem_slot), TMEM_COLS);
        tcgen05_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 2 * AT_BN;
    pdl_wait();                                         // queries, keys and values come from the kernel before us

    if (warp == 0) {
        // ---------------- producer
        if (lane == 0) {
            mbar_expect_tx(b_q, Q_BYTES);
            for (int h = 0; h < HALVES; ++h)
                tma_load_2d(smem_u32(q_s + h * QH_BYTES), &map_q, head * HD + h * 64, row_base, b_q);
            for (int t = 0; t < n_kt; ++t) {
                const int st = t & 1;
                uint8_t* kd = kv_s + (size_t)st * 2 * KV_BYTES;
                const int row = (bt[kt_lo + t] * nkv + kvh) * RF_PAGE;
                if (!mbar_wait(b_kfree + 8 * st, ((t >> 1) & 1) ^ 1, &abort_flag)) break;
                mbar_expect_tx(b_kfull + 8 * st, KV_BYTES);
                for (int h = 0; h < HALVES; ++h)
                    tma_load_2d(smem_u32(kd + h * KH_BYTES), &map_k, h * 64, row, b_kfull + 8 * st);
                if (!mbar_wait(b_vfree + 8 * st, ((t >> 1) & 1) ^ 1, &abort_flag)) break;
                mbar_expect_tx(b_vfull + 8 * st, KV_BYTES);
                for (int h = 0; h < HALVES; ++h)
                    tma_load_2d(smem_u32(kd + KV_BYTES + h * KH_BYTES), &map_v, h * 64, row, b_vfull + 8 * st);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_s = at_idesc(AT_BN, 0), idesc_o = at_idesc(HD, 1);
            // S has two buffers in tensor memory: the scores of page t + 1 are computed while the softmax
            // warps are still busy with page t, so they find their next input ready when they come back.
            auto issue_s = [&](int t) -> bool {
                const int st = t & 1;
                if (!mbar_wait(b_kfull + 8 * st, (t >> 1) & 1, &abort_flag)) return false;
                tcgen05_fence_after();
                const uint32_t k_t = smem_u32(kv_s + (size_t)st * 2 * KV_BYTES);
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks)      // S = Q K^T over the head dimension
                    tcgen05_mma_bf16(tmem_s + st * AT_BN, make_smem_desc(smem_u32(q_s) + (ks >> 2) * QH_BYTES + (ks & 3) * 32),
                                     make_smem_desc(k_t + (ks >> 2) * KH_BYTES + (ks & 3) * 32), idesc_s, ks ? 1u : 0u);
                tcgen05_commit(b_sfull + 8 * st);
                tcgen05_commit(b_kfree + 8 * st);          // the keys of this stage are consumed
                return true;
            };
            bool ok = mbar_wait(b_q, 0, &abort_flag);
            if (ok && n_kt > 0) ok = issue_s(0);
            for (int t = 0; t < n_kt && ok; ++t) {
                const int st = t & 1;
                if (t + 1 < n_kt) { ok = issue_s(t + 1); if (!ok) break; }
                ok = mbar_wait(b_pready + 8 * st, (t >> 1) & 1, &abort_flag);      // P(t) is in tensor memory, S(t) has been read
                if (!ok) break;
                ok = mbar_wait(b_vfull + 8 * st, (t >> 1) & 1, &abort_flag);
                if (!ok) break;
                tcgen05_fence_after();
                const uint32_t v_t = smem_u32(kv_s + (size_t)st * 2 * KV_BYTES) + KV_BYTES;
#pragma unroll
                for (int ks = 0; ks < AT_BN / 16; ++ks)   // O += P V over the page's 64 keys
                    tcgen05_mma_bf16_ts(tmem_o, tmem_s + st * AT_BN + ks * 8,
                                     make_smem_desc_mn(v_t + ks * 16 * 128, KH_BYTES), idesc_o, (t | ks) ? 1u : 0u);
                tcgen05_commit(b_vfree + 8 * st);         // the values of this stage are consumed
                tcgen05_commit(b_pvdone + 8 * st);
            }
        }
    } else {
        // ---------------- softmax, correction, epilogue: one thread per query row
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const int pos_i = pos_first + row;
        const int lo_i = (window > 0 && pos_i - window + 1 > 0) ? pos_i - window + 1 : 0;
        const bool row_ok = row < rows_here;
        const float sl2 = scale * 1.4426950408889634f;
        float m_ref = -INFINITY, l = 0.f;
        bool ok = true;
        for (int t = 0; t < n_kt; ++t) {
            const int st = t & 1;
            const int key0 = (kt_lo + t) * AT_BN;
            ok = mbar_wait(b_sfull + 8 * st, (t >> 1) & 1, &abort_flag);
            if (!ok) break;
            tcgen05_fence_after();
            // the value rows past the sequence's end were never written (or belong to a page that was not
            // loaded): their weights are zero, but 0 * (whatever bits lie there) must be 0
            const bool cleared = key0 + AT_BN - 1 > seq_last;
            if (cleared) {
                ok = mbar_wait(b_vfull + 8 * st, (t >> 1) & 1, &abort_flag);      // the page's values have landed
                if (!ok) break;
                uint8_t* v_t = kv_s + (size_t)st * 2 * KV_BYTES + KV_BYTES;
                const int first_bad = seq_last + 1 - key0;
                for (int i = threadIdx.x - 64; i < (AT_BN - first_bad) * HALVES * 8; i += 128) {
                    const int r = first_bad + i / (HALVES * 8), c = i % (HALVES * 8);
                    const uint32_t a = smem_u32(v_t + (c >> 3) * KH_BYTES) + r * 128 + (((c & 7) ^ (r & 7)) << 4);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(a), "r"(0u) : "memory");
                }
            }
            const bool no_mask = key0 + AT_BN - 1 <= pos_first && rows_here == AT_BM &&
                                 (window <= 0 || key0 >= pos_last - window + 1);
            // the row of S, once, into registers (raw products; masked ones -inf).  Maximum and sum are kept
            // in four independent partial results each: one warp per scheduler cannot hide a chain of 64
            // dependent operations
            float sc[AT_BN];
            {
                uint32_t r[32];
#pragma unroll
                for (int c0 = 0; c0 < AT_BN; c0 += 32) {
                    tcgen05_ld32(tmem_s + st * AT_BN + lane_base + c0, r);
                    tcgen05_wait_ld();
#pragma unroll
                    for (int j = 0; j < 32; ++j) sc[c0 + j] = __uint_as_float(r[j]);
                }
            }
            if (!no_mask) {
#pragma unroll
                for (int j = 0; j < AT_BN; ++j) {
                    const int key = key0 + j;
                    if (!(row_ok && key <= pos_i && key >= lo_i)) sc[j] = -INFINITY;
                }
            }
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < AT_BN; j += 4) {
                mx4[0] = fmaxf(mx4[0], sc[j]); mx4[1] = fmaxf(mx4[1], sc[j + 1]);
                mx4[2] = fmaxf(mx4[2], sc[j + 2]); mx4[3] = fmaxf(mx4[3], sc[j + 3]);
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * sl2;      // in units of log2 e (sl2 > 0)
            // move the reference only when the maximum has grown by more than 8: then O and l are rescaled
            float corr = 1.f;
            if (mx > m_ref + 8.f) {
                corr = (m_ref == -INFINITY) ? 0.f : at_exp2(m_ref - mx);
                m_ref = mx;
            }
            const float nref = (m_ref == -INFINITY) ? 0.f : -m_ref;
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t pk[AT_BN / 2];
#pragma unroll
            for (int j = 0; j < AT_BN; j += 4) {
                // weight = 2^(raw * scale * log2 e - reference): one FMA and one ex2 each; ex2(-inf) = 0
                const float p0 = at_exp2(fmaf(sc[j], sl2, nref)), p1 = at_exp2(fmaf(sc[j + 1], sl2, nref));
                const float p2 = at_exp2(fmaf(sc[j + 2], sl2, nref)), p3 = at_exp2(fmaf(sc[j + 3], sl2, nref));
                sum4[0] += p0; sum4[1] += p1; sum4[2] += p2; sum4[3] += p3;
                pk[j >> 1] = at_pack_bf16x2(p0, p1);
                pk[(j >> 1) + 1] = at_pack_bf16x2(p2, p3);
            }
            const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            // P takes the place of this page's scores in tensor memory: 64 bfloat16 = 32 columns of this thread's lane, the
            // A operand of P V as they lie (no way through shared memory, no proxy fence, and nothing of the previous P V
            // is overwritten, so P need not wait for it)
            tcgen05_st32(tmem_s + st * AT_BN + lane_base, pk);
            bool seen = false;                           // whether this step has looked at the previous P V's barrier
            if (t > 0 && __any_sync(0xffffffffu, corr != 1.f)) {
                ok = mbar_wait(b_pvdone + 8 * ((t - 1) & 1), ((t - 1) >> 1) & 1, &abort_flag);   // O is touched: that product must be complete
                if (!ok) break;
                seen = true;
                tcgen05_fence_after();
#pragma unroll 1
                for (int c0 = 0; c0 < HD; c0 += 32) {
                    uint32_t r[32];
                    tcgen05_ld32(tmem_o + lane_base + c0, r);
                    tcgen05_wait_ld();
#pragma unroll
                    for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * corr);
                    tcgen05_st32(tmem_o + lane_base + c0, r);
                }
            }
            tcgen05_wait_st();
            l = l * corr + sum;
            if (cleared) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the cleared value rows are for the MMA to read
            tcgen05_fence_before();
            at_arrive(b_pready + 8 * st);
            if (t > 0 && !seen) {                        // every phase of a barrier is seen once, or its parity says nothing
                ok = mbar_wait(b_pvdone + 8 * ((t - 1) & 1), ((t - 1) >> 1) & 1, &abort_flag);
                if (!ok) break;
            }
        }
        if (ok && n_kt > 0) ok = mbar_wait(b_pvdone + 8 * ((n_kt - 1) & 1), ((n_kt - 1) >> 1) & 1, &abort_flag);
        if (ok) {
            tcgen05_fence_after();
            const float inv = l > 0.f ? 1.f / l : 0.f;
            __nv_bfloat16* orow = out + (size_t)(row_base + row) * out_stride + (size_t)head * HD;
#pragma unroll 1
            for (int c0 = 0; c0 < HD; c0 += 32) {
                uint32_t r[32];
                tcgen05_ld32(tmem_o + lane_base + c0, r);
                tcgen05_wait_ld();
                if (row_ok) {
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        *reinterpret_cast<uint4*>(orow + c0 + 8 * q) = make_uint4(
                            pack_bf16x2(__uint_as_float(r[8 * q]) * inv, __uint_as_float(r[8 * q + 1]) * inv),
                            pack_bf16x2(__uint_as_float(r[8 * q + 2]) * inv, __uint_as_float(r[8 * q + 3]) * inv),
                            pack_bf16x2(__uint_as_float(r[8 * q + 4]) * inv, __uint_as_float(r[8 * q + 5]) * inv),
                            pack_bf16x2(__uint_as_float(r[8 * q + 6]) * inv, __uint_as_float(r[8 * q + 7]) * inv));
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
    if (threadIdx.x == 0 && abort_flag && status) atomicExch(status, 6);
}

// ---------------------------------------------------------------- host side
// rows x cols bf16 matrix with row stride ld (elements); box = box_rows x 64 columns, 128-byte swizzle
static int at_map(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, int box_rows) {
    return make_map(map, base, rows, cols, ld, box_rows);
}

template <int HD>
static int at_launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, void* out, int out_stride,
                     const int* tiles, int n_tiles, const int* seq_slot, const int* seq_start, const int* seq_nnew,
                     const int* cu_q, const int* block_table, int max_pages, int nh, int nkv, float scale, int window,
                     int* status, cudaStream_t st) {
    constexpr size_t smem = (size_t)(HD / 64) * AT_BM * 128 + 4 * (size_t)(HD / 64) * AT_BN * 128 + 15 * 8 + 16;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    cudaError_t e = rf_launch(attention_prefill_tc_kernel<HD>, dim3(nh, n_tiles), dim3(AT_THREADS), smem, st, mq, mk, mv,
                              reinterpret_cast<__nv_bfloat16*>(out), out_stride, tiles, seq_slot, seq_start, seq_nnew, cu_q,
                              block_table, max_pages, nh, nkv, scale, window, status);
    if (e != cudaSuccess) return (int)e;
    RF_LAUNCH_CHECK();
    return 0;
}

extern "C" {

int rf_attention_prefill_tc_supported(int nh, int nkv, int hd) {
    if (nkv <= 0 || nh % nkv || nh > 65535) return 0;
    return (hd == 64 || hd == 128) && encode_fn() != nullptr;
}

// tiles: n_tiles pairs (sequence index, first new-token row of the tile within the sequence), 128 rows a tile.
// q: [T, q_stride] with the heads' columns first; T is needed for the map's extent.
int rf_attention_prefill_tc(const void* q, int q_stride, int T, void* out, int out_stride, const void* k_pages,
                            const void* v_pages, long long n_pages, const int* tiles, int n_tiles, const int* seq_slot,
                            const int* seq_start, const int* seq_nnew, const int* cu_q, const int* block_table,
                            int max_pages, int nh, int nkv, int hd, float scale, int window, int* status,
                            cudaStream_t st) {
    if (n_tiles <= 0) return 0;
    if (n_tiles > 65535) return RF_ERR_UNSUPPORTED;      // tiles are the grid's y dimension (8 million prompt tokens)
    if (!rf_attention_prefill_tc_supported(nh, nkv, hd)) return RF_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(out) & 15) || (out_stride % 8)) return RF_ERR_BAD_ARG;
    CUtensorMap mq, mk, mv;
    int e;
    const long long rows = n_pages * nkv * RF_PAGE;
    if ((e = at_map(&mq, q, T, (long long)nh * hd, q_stride, AT_BM)) || (e = at_map(&mk, k_pages, rows, hd, hd, RF_PAGE)) ||
        (e = at_map(&mv, v_pages, rows, hd, hd, RF_PAGE)))
        return e;
    if (hd == 64)
        return at_launch<64>(mq, mk, mv, out, out_stride, tiles, n_tiles, seq_slot, seq_start, seq_nnew, cu_q, block_table,
                             max_pages, nh, nkv, scale, window, status, st);
    return at_launch<128>(mq, mk, mv, out, out_stride, tiles, n_tiles, seq_slot, seq_start, seq_nnew, cu_q, block_table,
                          max_pages, nh, nkv, scale, window, status, st);
}

}
