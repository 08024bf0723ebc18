// Decode attention over the paged cache: one new token per sequence, bfloat16 cache.
//
// The context is cut into chunks of 128 keys (two cache pages); a CTA owns (chunk, kv head,
// sequence) and serves ALL query heads of that kv head's group from one pass over the
// chunk's keys and values (maeddesg/ROCmForge's flash_attn_decode_gqa_kernel has the same idea
// with 32-key tiles in LDS and one block per kv head, hip_kernels/attention.hip:633-798; its
// dispatched decode kernel keeps all scores of a head in LDS, :148-213).  A page's keys (or
// values) of one kv head are one contiguous slab, so the whole chunk is brought into shared
// memory by four bulk async copies that are all in flight at once.  Both products run on the
// tensor cores (mma.sync m16n8k16, bf16 in, 32-bit accumulate) with the group's query heads
// as the 16 rows: Q K^T into 32-bit scores, the softmax in 32-bit, the weights rounded to
// bfloat16 as the operand of P V (as maeddesg/ROCmForge's WMMA attention rounds them to FP16,
// hip_kernels/wmma/wmma_attention_prefill.hip:574).  Each CTA writes its chunk's (max, sum, unnormalised
// output) to scratch memory; the CTA that finishes last for a (sequence, kv head) merges
// the chunks in index order, so the result does not depend on which CTA that was.  The grid
// may be larger than the context needs (a replayed CUDA graph keeps its launch shape): CTAs
// beyond the sequence's last chunk, or wholly before its window, leave at once.
#include <cuda.h>
#include "common.cuh"

#define DEC_THREADS 128
#define DEC_WARPS 4
#define DEC_CHUNK 128
#define DEC_GP 8                      // query heads per kv head, padded
#define DEC_WAIT_LIMIT_NS 2000000000ULL

__device__ __forceinline__ uint32_t dec_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

template <int EPL>
__global__ void __launch_bounds__(DEC_THREADS)
attention_decode_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, __nv_bfloat16* __restrict__ out,
                        int out_stride, const __nv_bfloat16* __restrict__ k_pages,
                        const __nv_bfloat16* __restrict__ v_pages, const int* __restrict__ tok_seq,
                        const int* __restrict__ tok_pos, const int* __restrict__ seq_slot,
                        const int* __restrict__ block_table, int max_pages, int nh, int nkv, float scale,
                        int window, int max_chunks, float* __restrict__ part_o, float* __restrict__ part_ml,
                        int* __restrict__ counters, int* __restrict__ status) {
    constexpr int HD = EPL * 32;
    constexpr uint32_t SLAB = RF_PAGE * HD * 2;                 // bytes of one page's keys of one kv head
    extern __shared__ __align__(1024) uint8_t dec_smem[];
    __nv_bfloat16* k_s = reinterpret_cast<__nv_bfloat16*>(dec_smem);                   // [128][HD]
    __nv_bfloat16* v_s = k_s + DEC_CHUNK * HD;                                          // [128][HD]
    float* p_s = reinterpret_cast<float*>(v_s + DEC_CHUNK * HD);                        // [GP][128] scores, then weights
    float* wred = p_s + DEC_GP * DEC_CHUNK;                                             // [4 warps][GP]
    uint64_t* bar = reinterpret_cast<uint64_t*>(wred + DEC_WARPS * DEC_GP);
    float* o_red = reinterpret_cast<float*>(dec_smem);                                 // [4][GP][HD], over k_s when done
    __shared__ int is_last, gave_up;

    pdl_trigger();
    const int G = nh / nkv;
    const int c = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z, tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const int pos = tok_pos[b];
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int c_lo = lo / DEC_CHUNK, c_hi = pos / DEC_CHUNK;
    if (c_hi >= max_chunks) {           // the launch has no CTA for the sequence's last chunk: say so, touch nothing
        if (c == 0 && tid == 0 && status) atomicExch(status, 3);
        return;
    }
    if (c < c_lo || c > c_hi) return;
    const int n_act = c_hi - c_lo + 1;
    const int slot = seq_slot[tok_seq[b]];
    const int* bt = block_table + (size_t)slot * max_pages;
    const int k_first = c * DEC_CHUNK;
    int k_begin = lo - k_first; if (k_begin < 0) k_begin = 0;                  // chunk-relative valid range
    int k_last = pos - k_first; if (k_last > DEC_CHUNK - 1) k_last = DEC_CHUNK - 1;

    // positions, slots and block tables are not written by any kernel of the step; the queries and the
    // newest keys and values are: wait for the kernel before us
    pdl_wait();
    // ---- bring the chunk's pages in: all copies in flight at once
    const uint32_t bar_a = dec_smem_u32(bar);
    if (tid == 0) {
        gave_up = 0;
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_a));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        uint32_t bytes = 0;
        for (int pg = 0; pg < DEC_CHUNK / RF_PAGE; ++pg)
            if (pg * RF_PAGE <= k_last && pg * RF_PAGE + RF_PAGE - 1 >= k_begin) bytes += 2 * SLAB;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar_a), "r"(bytes) : "memory");
        for (int pg = 0; pg < DEC_CHUNK / RF_PAGE; ++pg) {
            if (!(pg * RF_PAGE <= k_last && pg * RF_PAGE + RF_PAGE - 1 >= k_begin)) continue;
            const int page = bt[k_first / RF_PAGE + pg];
            const size_t off = ((size_t)page * nkv + kvh) * RF_PAGE * HD;
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(dec_smem_u32(k_s + pg * RF_PAGE * HD)), "l"(k_pages + off), "r"(SLAB), "r"(bar_a) : "memory");
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(dec_smem_u32(v_s + pg * RF_PAGE * HD)), "l"(v_pages + off), "r"(SLAB), "r"(bar_a) : "memory");
        }
    }
    // the group's queries as the A operand of mma.m16n8k16 (row = query head of the group, rows >= G are
    // zero; with at most 8 heads per group the upper 8 rows are always zero): two registers per 16 dims
    const int gid = lane >> 2, tig = lane & 3;
    uint32_t qa[HD / 16][2];
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
        qa[ks][0] = qa[ks][1] = 0u;
        if (gid < G) {
            const __nv_bfloat16* qrow = q + (size_t)b * q_stride + (size_t)(kvh * G + gid) * HD + ks * 16 + tig * 2;
            qa[ks][0] = *reinterpret_cast<const uint32_t*>(qrow);
            qa[ks][1] = *reinterpret_cast<const uint32_t*>(qrow + 8);
        }
    }
    __syncthreads();                                   // the barrier is initialised for everyone
    {   // bounded wait for the copies
        uint32_t ok = 0;
        unsigned long long t0 = 0;
        for (long long it = 0; !ok; ++it) {
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n\t"
                         "selp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(bar_a) : "memory");
            if (ok) break;
            if ((it & 63) == 63) {
                unsigned long long now;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
                if (t0 == 0) t0 = now;
                if (now - t0 > DEC_WAIT_LIMIT_NS || gave_up) { gave_up = 1; break; }
            }
        }
    }
    __syncthreads();
    if (gave_up) {                                      // record it and leave; the output stays unwritten
        if (tid == 0 && status) atomicExch(status, 2);
        return;
    }

    // value rows outside the sequence (the rest of a half-filled page) get weight zero below, but
    // 0 * (whatever bits lie there) must be 0: clear those rows
    for (int i = tid; i < DEC_CHUNK * (HD / 8); i += DEC_THREADS) {
        const int row = i / (HD / 8);
        if (row < k_begin || row > k_last) reinterpret_cast<uint4*>(v_s)[i] = make_uint4(0u, 0u, 0u, 0u);
    }

    // ---- scores on the tensor cores: a warp owns 32 keys = 4 tiles of 8; S[head][key] = q . k
    const int kbase = warp * 32;
    const bool warp_active = kbase <= k_last && kbase + 31 >= k_begin;
    float sc[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
    if (warp_active) {
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                const __nv_bfloat16* kr = k_s + (kbase + nt * 8 + gid) * HD + ks * 16 + tig * 2;
                const uint32_t b0 = *reinterpret_cast<const uint32_t*>(kr);
                const uint32_t b1 = *reinterpret_cast<const uint32_t*>(kr + 8);
                asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                             : "+f"(sc[nt][0]), "+f"(sc[nt][1]), "+f"(sc[nt][2]), "+f"(sc[nt][3])
                             : "r"(qa[ks][0]), "r"(0u), "r"(qa[ks][1]), "r"(0u), "r"(b0), "r"(b1));
            }
        }
    }
    // this thread: head gid, keys kbase + nt*8 + tig*2 + {0,1}; 32-bit from here on
    float mloc = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int kk = kbase + nt * 8 + tig * 2 + e;
            const bool ok = warp_active && kk >= k_begin && kk <= k_last;     // garbage beyond the sequence is masked here
            sc[nt][e] = ok ? sc[nt][e] * scale : -INFINITY;
            mloc = fmaxf(mloc, sc[nt][e]);
        }
    mloc = fmaxf(mloc, __shfl_xor_sync(0xffffffffu, mloc, 1));
    mloc = fmaxf(mloc, __shfl_xor_sync(0xffffffffu, mloc, 2));
    if (tig == 0) wred[warp * DEC_GP + gid] = mloc;
    __syncthreads();
    const float mrow = fmaxf(fmaxf(wred[gid], wred[DEC_GP + gid]), fmaxf(wred[2 * DEC_GP + gid], wred[3 * DEC_GP + gid]));
    __syncthreads();
    float lloc = 0.f;
    uint32_t pa[2][2];                                  // P as the A operand of the second product, two 16-key steps
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
        const float p0 = sc[nt][0] == -INFINITY ? 0.f : expf(sc[nt][0] - mrow);
        const float p1 = sc[nt][1] == -INFINITY ? 0.f : expf(sc[nt][1] - mrow);
        lloc += p0 + p1;
        const __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
        pa[nt >> 1][nt & 1] = *reinterpret_cast<const uint32_t*>(&pk);
    }
    lloc += __shfl_xor_sync(0xffffffffu, lloc, 1);
    lloc += __shfl_xor_sync(0xffffffffu, lloc, 2);
    if (tig == 0) wred[warp * DEC_GP + gid] = lloc;
    __syncthreads();
    const float lrow = (wred[gid] + wred[DEC_GP + gid]) + (wred[2 * DEC_GP + gid] + wred[3 * DEC_GP + gid]);
    // every thread needs m and l of the heads it writes later: park them in shared memory
    if (warp == 0 && tig == 0) { p_s[gid] = mrow; p_s[DEC_GP + gid] = lrow; }

    // ---- values on the tensor cores: O[head][dim] += P[head][key] * V[key][dim]
    float oc[HD / 8][4];
#pragma unroll
    for (int nt = 0; nt < HD / 8; ++nt) oc[nt][0] = oc[nt][1] = oc[nt][2] = oc[nt][3] = 0.f;
    if (warp_active) {
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
            // a tile of 16 keys wholly outside the sequence holds garbage: skip it (its weights are zero, but 0 * NaN is not)
            const int t0 = kbase + ks * 16;
            if (t0 > k_last || t0 + 15 < k_begin) continue;
#pragma unroll
            for (int nt = 0; nt < HD / 8; nt += 2) {
                const int mi = lane >> 3, r = lane & 7;
                const __nv_bfloat16* vr = v_s + (t0 + (mi & 1) * 8 + r) * HD + (nt + (mi >> 1)) * 8;
                uint32_t v0, v1, v2, v3;
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(v0), "=r"(v1), "=r"(v2), "=r"(v3) : "r"(dec_smem_u32(vr)));
                asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                             : "+f"(oc[nt][0]), "+f"(oc[nt][1]), "+f"(oc[nt][2]), "+f"(oc[nt][3])
                             : "r"(pa[ks][0]), "r"(0u), "r"(pa[ks][1]), "r"(0u), "r"(v0), "r"(v1));
                asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                             : "+f"(oc[nt + 1][0]), "+f"(oc[nt + 1][1]), "+f"(oc[nt + 1][2]), "+f"(oc[nt + 1][3])
                             : "r"(pa[ks][0]), "r"(0u), "r"(pa[ks][1]), "r"(0u), "r"(v2), "r"(v3));
            }
        }
    }
    __syncthreads();                                   // everyone is done with k_s / v_s
#pragma unroll
    for (int nt = 0; nt < HD / 8; ++nt) {
        o_red[(warp * DEC_GP + gid) * HD + nt * 8 + tig * 2] = oc[nt][0];
        o_red[(warp * DEC_GP + gid) * HD + nt * 8 + tig * 2 + 1] = oc[nt][1];
    }
    __syncthreads();

    // ---- this chunk's result: final if it is the only chunk, else a partial in scratch memory
    for (int i = tid; i < G * HD; i += DEC_THREADS) {
        const int g = i / HD, d = i - g * HD;
        const float o = (o_red[g * HD + d] + o_red[(DEC_GP + g) * HD + d])
                      + (o_red[(2 * DEC_GP + g) * HD + d] + o_red[(3 * DEC_GP + g) * HD + d]);
        const int head = kvh * G + g;
        if (n_act == 1) {
            const float lg = p_s[DEC_GP + g];
            out[(size_t)b * out_stride + (size_t)head * HD + d] = __float2bfloat16_rn(lg > 0.f ? o / lg : 0.f);
        } else {
            part_o[(((size_t)b * nh + head) * max_chunks + c) * HD + d] = o;
        }
    }
    if (n_act == 1) return;
    if (tid < G) {
        float* ml = part_ml + (((size_t)b * nh + kvh * G + tid) * max_chunks + c) * 2;
        ml[0] = p_s[tid]; ml[1] = p_s[DEC_GP + tid];
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const int done = atomicAdd(&counters[b * nkv + kvh], 1);
        is_last = (done == n_act - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    // weights of the chunks, once per head: w[g][cc] = exp(m_cc - M) / L.  All loads of this phase are
    // independent of one another (p_s and o_red are free by now).
    float* w_s = p_s;                                    // [GP][DEC_CHUNK]: max, then weight, of chunk cc
    float* l_s = o_red;                                  // [GP][DEC_CHUNK]: sum of chunk cc
    for (int i = tid; i < G * n_act; i += DEC_THREADS) {
        const int g = i / n_act, cc = i - g * n_act;
        const float2 ml = __ldcg(reinterpret_cast<const float2*>(
            part_ml + (((size_t)b * nh + kvh * G + g) * max_chunks + c_lo + cc) * 2));
        w_s[g * DEC_CHUNK + cc] = ml.x;
        l_s[g * DEC_CHUNK + cc] = ml.y;
    }
    __syncthreads();
    if (tid < G) {
        float M = -INFINITY;
        for (int cc = 0; cc < n_act; ++cc) M = fmaxf(M, w_s[tid * DEC_CHUNK + cc]);
        float L = 0.f;
        for (int cc = 0; cc < n_act; ++cc) {             // chunks in index order
            const float w = expf(w_s[tid * DEC_CHUNK + cc] - M);
            L += w * l_s[tid * DEC_CHUNK + cc];
            w_s[tid * DEC_CHUNK + cc] = w;
        }
        const float inv = L > 0.f ? 1.f / L : 0.f;
        for (int cc = 0; cc < n_act; ++cc) w_s[tid * DEC_CHUNK + cc] *= inv;
    }
    __syncthreads();
    for (int i = tid; i < G * (HD / 4); i += DEC_THREADS) {
        const int g = i / (HD / 4), d4 = i - g * (HD / 4);
        const int head = kvh * G + g;
        const float4* po = reinterpret_cast<const float4*>(part_o + (((size_t)b * nh + head) * max_chunks + c_lo) * HD) + d4;
        float4 O = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
        for (int cc = 0; cc < n_act; ++cc) {
            const float w = w_s[g * DEC_CHUNK + cc];
            const float4 v = __ldcg(po + (size_t)cc * (HD / 4));
            O.x = fmaf(w, v.x, O.x); O.y = fmaf(w, v.y, O.y); O.z = fmaf(w, v.z, O.z); O.w = fmaf(w, v.w, O.w);
        }
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(out + (size_t)b * out_stride + (size_t)head * HD + 4 * d4);
        o2[0] = __floats2bfloat162_rn(O.x, O.y);
        o2[1] = __floats2bfloat162_rn(O.z, O.w);
    }
    if (tid == 0) counters[b * nkv + kvh] = 0;          // ready for the next launch
}

// ---------------------------------------------------------------- thread-block clusters
__device__ __forceinline__ uint32_t dcl_cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void dcl_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// ---------------------------------------------------------------- a warp per tile of keys
// For contexts of ordinary length the merge through global memory above costs more than the attention
// itself (write partials, fence, count arrivals, fence, read them back: five trips to L2).  Here the CTAs
// that share a (sequence, kv head) form a thread-block cluster of `splits` CTAs; CTA r takes the pages
// r, r + splits, ... of the context, brought in by TMA with the 128-byte swizzle so that ldmatrix reads
// them without bank conflicts.  No scratch memory, no atomics; the launch shape depends on the batch
// alone, so a captured graph stays valid while the context grows.  Inside a CTA every warp works alone: the
// CTA's pages are cut into tiles of ROWS keys, warp w takes the tiles w, w + WARPS, ... and has a buffer for
// one tile of keys and one of values, each with its own mbarrier.  A warp computes all scores of a tile,
// releases the key buffer to the copy of its next tile, rescales once per tile and multiplies by the values,
// then releases the value buffer: the copy of the next keys runs under the value product and the copy
// of the next values under the next score product, and no barrier of the whole CTA lies on the way.  With
// contexts of a few hundred keys every warp has one tile, all copies are in flight at once (those of pages
// older than the newest position even before the kernel ahead of this one has finished).
//
// mma.sync is the slow tensor path of this GPU, so the products are turned to need as few of them as
// possible: the 16 rows of an instruction hold keys (scores, S^T = K Q^T) or output dimensions (O^T = V^T P^T)
// and its 8 columns the up to 8 query heads of the kv head, instead of 16 rows of which 7 or 8 are heads.
// K is the A operand as it lies in shared memory, V^T comes from ldmatrix.trans, Q^T is the B operand straight
// from the query's registers, and P^T becomes a B operand by transposing the 8x8 blocks of the score
// accumulators with movmatrix.  A thread then holds two heads' running maximum and sum.
//
// The merge: warps leave their states in shared memory, the CTA folds them, and every CTA pushes to each peer
// the slice of output dimensions that this peer owns (remote stores into a slot per sender); after ONE cluster
// barrier each CTA folds the slots of its slice in rank order and writes it.  No CTA reads a peer's memory,
// so none has to wait for its peers before it exits.
template <int EPL, int ROWS, int WARPS>
__global__ void __launch_bounds__(WARPS * 32)
attention_decode_warps_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                              const __nv_bfloat16* __restrict__ q, int q_stride, __nv_bfloat16* __restrict__ out,
                              int out_stride, const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                              const int* __restrict__ seq_slot, const int* __restrict__ block_table, int max_pages,
                              int nh, int nkv, float scale, int window, int splits, int* __restrict__ status) {
    constexpr int HD = EPL * 32;
    constexpr int NT = WARPS * 32;
    constexpr int HALVES = HD / 64;                             // 128-byte column blocks of a row
    constexpr uint32_t HALF_BYTES = ROWS * 128;                 // one column block of a tile: [ROWS][128 B], swizzled
    constexpr uint32_t TILE = ROWS * HD * 2;                    // a tile's keys (or values)
    constexpr int UPP = RF_PAGE / ROWS;                         // tiles per page
    constexpr int NB = ROWS / 16;                               // blocks of 16 keys per tile
    constexpr int SP = HD + 4;                                  // floats between two heads of a warp's state
    static_assert(HALF_BYTES % 1024 == 0, "a column block must keep the swizzle pattern's 1024-byte period");
    static_assert((2 * DEC_GP + DEC_GP * SP) * 4 <= 2 * TILE, "a warp's state lies where its tiles lay");
    extern __shared__ __align__(1024) uint8_t dec_smem[];
    uint8_t* ring = dec_smem + ((1024u - (dec_smem_u32(dec_smem) & 1023u)) & 1023u);    // [warp][K | V][HALVES][ROWS][128 B]
    float* f_w = reinterpret_cast<float*>(ring + (size_t)WARPS * 2 * TILE);             // [WARPS][GP] weights of the warps
    float* c_m = f_w + WARPS * DEC_GP;                                                  // this CTA: [GP]
    float* c_l = c_m + DEC_GP;                                                          // [GP]
    float* slots = c_l + DEC_GP;                                // [splits][2*GP + GP * HD/splits]: what the peers push
    uint64_t* bars = reinterpret_cast<uint64_t*>(slots + splits * 2 * DEC_GP + DEC_GP * HD);     // [warp][K | V]
    __shared__ int gave_up;

    pdl_trigger();
    const int G = nh / nkv;
    const int kvh = blockIdx.y, b = blockIdx.z, tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5, gid = lane >> 2, tig = lane & 3;
    const int rank = splits > 1 ? (int)dcl_cluster_rank() : 0;
    const int pos = tok_pos[b];
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int p_lo = lo / RF_PAGE, p_hi = pos / RF_PAGE;
    const int n_my = (p_hi - p_lo - rank) >= 0 ? (p_hi - p_lo - rank) / splits + 1 : 0;     // pages of this CTA
    const int n_units = n_my * UPP;
    const int* bt = block_table + (size_t)seq_slot[tok_seq[b]] * max_pages;
    uint8_t* my_k = ring + (size_t)warp * 2 * TILE;
    const uint32_t k_t = dec_smem_u32(my_k), v_t = k_t + TILE;
    const uint32_t bar_k = dec_smem_u32(&bars[warp * 2]), bar_v = bar_k + 8;

    if (tid == 0) gave_up = 0;
    if (lane == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_k));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_v));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
    }
    __syncthreads();
    // a store into a peer's shared memory needs that peer to have started: arrive here, wait just before the first
    // push (every CTA has long arrived by then, so the wait costs nothing)
    if (splits > 1) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");

    // tile u of this CTA: page p_lo + rank + (u / UPP) * splits, rows (u % UPP) * ROWS ... of it
    auto first_key = [&](int u) { return (p_lo + rank + (u / UPP) * splits) * RF_PAGE + (u % UPP) * ROWS; };
    auto next_tile = [&](int u) {                     // the next of this warp's tiles that holds a key in [lo, pos]
        for (u += WARPS; u < n_units; u += WARPS) {
            const int k0 = first_key(u);
            if (k0 <= pos && k0 + ROWS - 1 >= lo) break;
        }
        return u;
    };
    auto issue = [&](int u, bool keys) {              // lane 0: the keys or the values of tile u into this warp's buffer
        const int page = bt[p_lo + rank + (u / UPP) * splits];
        const int row = (page * nkv + kvh) * RF_PAGE + (u % UPP) * ROWS;
        const uint32_t bar = keys ? bar_k : bar_v, dst = keys ? k_t : v_t;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(TILE) : "memory");
#pragma unroll
        for (int h = 0; h < HALVES; ++h)
            asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                         ::"r"(dst + h * HALF_BYTES), "l"(keys ? &map_k : &map_v), "r"(h * 64), "r"(row), "r"(bar) : "memory");
    };
    auto wait = [&](uint32_t bar, uint32_t parity) -> bool {          // bounded; the whole warp gets one verdict
        uint32_t ok = 0;
        unsigned long long t0 = 0;
        for (long long it = 0; !ok; ++it) {
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                         "selp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
            if (ok) break;
            if ((it & 63) == 63) {
                unsigned long long now;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
                if (t0 == 0) t0 = now;
                if (now - t0 > DEC_WAIT_LIMIT_NS) break;
            }
        }
        return __all_sync(0xffffffffu, ok != 0);
    };

    // Only the page of the newest position is written in this step (by the kernel before this one); the
    // older pages were written by earlier steps, which are complete: their copies start before the wait.
    int u = next_tile(warp - WARPS);
    const bool early = u < n_units && first_key(u) / RF_PAGE < p_hi;
    if (lane == 0 && early) { issue(u, true); issue(u, false); }
    pdl_wait();                                         // queries and the newest keys/values come from the kernel before us
    if (lane == 0 && !early && u < n_units) { issue(u, true); issue(u, false); }

    uint32_t qb[HD / 16][2];                            // Q^T as the B operand: head gid, dims ks*16 + tig*2 (+8)
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
        qb[ks][0] = qb[ks][1] = 0u;
        if (gid < G) {
            const __nv_bfloat16* qrow = q + (size_t)b * q_stride + (size_t)(kvh * G + gid) * HD + ks * 16 + tig * 2;
            qb[ks][0] = *reinterpret_cast<const uint32_t*>(qrow);
            qb[ks][1] = *reinterpret_cast<const uint32_t*>(qrow + 8);
        }
    }
    // O^T: block mt of 16 dimensions: [0] (dim gid, head tig*2), [1] (dim gid, head tig*2+1), [2], [3] the same for dim gid + 8
    float oc[HD / 16][4];
#pragma unroll
    for (int mt = 0; mt < HD / 16; ++mt) oc[mt][0] = oc[mt][1] = oc[mt][2] = oc[mt][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};        // heads tig*2 and tig*2 + 1
    const int mi = lane >> 3, r8 = lane & 7;
    bool failed = false;

    for (uint32_t it = 0; u < n_units; ++it) {
        const int un = next_tile(u);
        const int key0 = first_key(u);
        int k_begin = lo - key0; if (k_begin < 0) k_begin = 0;                    // valid rows of this tile
        int k_last = pos - key0; if (k_last > ROWS - 1) k_last = ROWS - 1;
        if (!wait(bar_k, it & 1)) { failed = true; break; }
        // ---- scores, transposed: [0] (key gid, head tig*2), [1] (key gid, head tig*2+1), [2], [3] the same for key gid + 8
        float sc[NB][4];
#pragma unroll
        for (int kb = 0; kb < NB; ++kb) sc[kb][0] = sc[kb][1] = sc[kb][2] = sc[kb][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
            for (int kb = 0; kb < NB; ++kb) {
                // matrices: (keys + 0..7, dims ks*16 + 0..7), (keys + 8.., same dims), (keys + 0..7, dims + 8), (keys + 8.., dims + 8)
                const int krow = kb * 16 + (mi & 1) * 8 + r8;
                const int gc = ks * 2 + (mi >> 1);                                 // 16-byte chunk along the row
                const uint32_t a = k_t + (gc >> 3) * HALF_BYTES + krow * 128 + (((gc & 7) ^ (krow & 7)) << 4);
                uint32_t a0, a1, a2, a3;
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(a0), "=r"(a1), "=r"(a2), "=r"(a3) : "r"(a));
                asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                             : "+f"(sc[kb][0]), "+f"(sc[kb][1]), "+f"(sc[kb][2]), "+f"(sc[kb][3])
                             : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(qb[ks][0]), "r"(qb[ks][1]));
            }
        }
        __syncwarp();                                    // every lane has read the keys: the buffer may be refilled
        if (lane == 0 && un < n_units) issue(un, true);
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int kb = 0; kb < NB; ++kb)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int kk = kb * 16 + gid + (e >> 1) * 8;
                sc[kb][e] = (kk >= k_begin && kk <= k_last) ? sc[kb][e] * scale : -INFINITY;
                mx[e & 1] = fmaxf(mx[e & 1], sc[kb][e]);
            }
        float corr[2], psum[2] = {0.f, 0.f};
#pragma unroll
        for (int h = 0; h < 2; ++h) {                    // the tile's keys lie across the lanes of equal tig
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 4));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 8));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 16));
            const float m_new = fmaxf(m_run[h], mx[h]);  // finite: the tile holds a key of the sequence
            corr[h] = (m_run[h] == -INFINITY) ? 0.f : expf(m_run[h] - m_new);
            m_run[h] = m_new;
        }
        uint32_t pb[NB][2];                              // P^T as the B operand: head gid, keys tig*2.. (+8) of block kb
#pragma unroll
        for (int kb = 0; kb < NB; ++kb) {
            float p[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                p[e] = sc[kb][e] == -INFINITY ? 0.f : expf(sc[kb][e] - m_run[e & 1]);
                psum[e & 1] += p[e];
            }
            const __nv_bfloat162 lo8 = __floats2bfloat162_rn(p[0], p[1]), hi8 = __floats2bfloat162_rn(p[2], p[3]);
            // an 8x8 block (row = key gid, columns = heads tig*2, tig*2+1) transposed: row = head gid, columns = keys tig*2, tig*2+1
            asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(pb[kb][0]) : "r"(*reinterpret_cast<const uint32_t*>(&lo8)));
            asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(pb[kb][1]) : "r"(*reinterpret_cast<const uint32_t*>(&hi8)));
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            psum[h] += __shfl_xor_sync(0xffffffffu, psum[h], 4);
            psum[h] += __shfl_xor_sync(0xffffffffu, psum[h], 8);
            psum[h] += __shfl_xor_sync(0xffffffffu, psum[h], 16);
            l_run[h] = l_run[h] * corr[h] + psum[h];
        }
#pragma unroll
        for (int mt = 0; mt < HD / 16; ++mt) {
            oc[mt][0] *= corr[0]; oc[mt][1] *= corr[1]; oc[mt][2] *= corr[0]; oc[mt][3] *= corr[1];
        }
        if (!wait(bar_v, it & 1)) { failed = true; break; }
        if (k_begin > 0 || k_last < ROWS - 1) {
            // rows outside the sequence get weight zero, but 0 * (whatever bits lie there) must be 0
            // (the swizzle permutes 16-byte pieces inside a row: clearing whole rows needs no address math)
            for (int i = lane; i < ROWS * HALVES * 8; i += 32) {
                const int row = (i >> 3) % ROWS, h = i / (ROWS * 8);
                if (row < k_begin || row > k_last)
                    asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(v_t + h * HALF_BYTES + row * 128 + (i & 7) * 16),
                                 "r"(0u) : "memory");
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");       // before a later copy overwrites them
            __syncwarp();
        }
#pragma unroll
        for (int kb = 0; kb < NB; ++kb) {
            if (kb * 16 > k_last || kb * 16 + 15 < k_begin) continue;             // a block without a key of the sequence
#pragma unroll
            for (int mt = 0; mt < HD / 16; ++mt) {
                // V^T: matrices (keys + 0..7, dims mt*16 + 0..7), (same keys, dims + 8), (keys + 8.., dims), (keys + 8.., dims + 8)
                const int vrow = kb * 16 + (mi >> 1) * 8 + r8, gc = mt * 2 + (mi & 1);
                const uint32_t va = v_t + (gc >> 3) * HALF_BYTES + vrow * 128 + (((gc & 7) ^ (vrow & 7)) << 4);
                uint32_t a0, a1, a2, a3;
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(a0), "=r"(a1), "=r"(a2), "=r"(a3) : "r"(va));
                asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                             : "+f"(oc[mt][0]), "+f"(oc[mt][1]), "+f"(oc[mt][2]), "+f"(oc[mt][3])
                             : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(pb[kb][0]), "r"(pb[kb][1]));
            }
        }
        __syncwarp();                                    // the values have been read
        if (lane == 0 && un < n_units) issue(un, false);
        u = un;
    }
    if (failed) gave_up = 1;

    // ---- a warp leaves its state where its tiles lay: max [GP] | sum [GP] | output [GP][SP]
    {
        float* st = reinterpret_cast<float*>(my_k);
        if (gid == 0) {
            st[tig * 2] = m_run[0]; st[tig * 2 + 1] = m_run[1];
            st[DEC_GP + tig * 2] = l_run[0]; st[DEC_GP + tig * 2 + 1] = l_run[1];
        }
        float* o0 = st + 2 * DEC_GP + (tig * 2) * SP, *o1 = o0 + SP;
#pragma unroll
        for (int mt = 0; mt < HD / 16; ++mt) {
            o0[mt * 16 + gid] = oc[mt][0]; o1[mt * 16 + gid] = oc[mt][1];
            o0[mt * 16 + gid + 8] = oc[mt][2]; o1[mt * 16 + gid + 8] = oc[mt][3];
        }
    }
    __syncthreads();
    if (tid < WARPS * DEC_GP) {
        // the warps' weights for every head, and the CTA's maximum and sum: thread (head g, warp w) with the warps of a head
        // in neighbouring lanes, so that maximum and sum are shuffles over WARPS lanes instead of one thread's loops
        const int g = tid / WARPS, w = tid % WARPS;
        const float* st = reinterpret_cast<const float*>(ring + (size_t)w * 2 * TILE);
        const float m = st[g];
        float M = m;
#pragma unroll
        for (int o = 1; o < WARPS; o <<= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
        const float f = m == -INFINITY ? 0.f : expf(m - M);
        f_w[w * DEC_GP + g] = f;
        // the sum in the warps' index order, whatever the lanes' timing: lane (g, 0) adds its neighbours' terms one by one
        const float term = f * st[DEC_GP + g];
        float L = 0.f;
#pragma unroll
        for (int k = 0; k < WARPS; ++k) L += __shfl_sync(0xffffffffu, term, (tid & 31) - w + k);
        if (w == 0) { c_m[g] = M; c_l[g] = L; }
    }
    __syncthreads();
    const int DS = HD / splits;                          // output dimensions per CTA of the cluster
    const int slot_floats = 2 * DEC_GP + DEC_GP * DS;
    if (splits > 1) asm volatile("barrier.cluster.wait.aligned;" ::: "memory");      // all peers run (see the arrive above)
    // four neighbouring dimensions per thread: eight 16-byte loads from the warps' states and one 16-byte (remote) store
    // instead of four times as many scalar ones (the scalar form took 0.9 us of a 6 us kernel)
    for (int i = tid; i < G * (HD / 4); i += NT) {
        const int g = i / (HD / 4), d = (i - g * (HD / 4)) * 4;
        float O[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            const float f = f_w[w * DEC_GP + g];
            const float4 v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(ring + (size_t)w * 2 * TILE) + 2 * DEC_GP + g * SP + d);
            O[0] += f * v.x; O[1] += f * v.y; O[2] += f * v.z; O[3] += f * v.w;
        }
        if (splits == 1) {
            if (!gave_up) {
                __nv_bfloat16* o = out + (size_t)b * out_stride + (size_t)(kvh * G + g) * HD + d;
#pragma unroll
                for (int u = 0; u < 4; ++u) o[u] = __float2bfloat16_rn(c_l[g] > 0.f ? O[u] / c_l[g] : 0.f);
            }
        } else {                                         // to the CTA that owns these dimensions, into this CTA's slot there
            const int t = d / DS;
            uint32_t raddr;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(raddr)
                         : "r"(dec_smem_u32(slots + rank * slot_floats + 2 * DEC_GP + g * DS + (d - t * DS))), "r"(t));
            asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(raddr), "f"(O[0]), "f"(O[1]), "f"(O[2]), "f"(O[3]) : "memory");
        }
    }
    if (splits > 1) {
        for (int i = tid; i < splits * 2 * DEC_GP; i += NT) {       // this CTA's maxima and sums to every peer
            const int t = i / (2 * DEC_GP), j = i - t * 2 * DEC_GP;
            uint32_t raddr;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(raddr)
                         : "r"(dec_smem_u32(slots + rank * slot_floats + j)), "r"(t));
            asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(raddr), "f"(j < DEC_GP ? c_m[j] : c_l[j - DEC_GP]) : "memory");
        }
        dcl_cluster_sync();                              // every push has landed; nobody reads a peer's memory after it
        if (!gave_up)
            for (int i = tid; i < G * DS; i += NT) {
                const int g = i / DS, dd = i - g * DS;
                float M = -INFINITY;
#pragma unroll 4
                for (int r = 0; r < splits; ++r) M = fmaxf(M, slots[r * slot_floats + g]);
                float L = 0.f, O = 0.f;
#pragma unroll 4
                for (int r = 0; r < splits; ++r) {       // CTAs in rank order
                    const float* sl = slots + r * slot_floats;
                    const float f = sl[g] == -INFINITY ? 0.f : expf(sl[g] - M);
                    L += f * sl[DEC_GP + g];
                    O += f * sl[2 * DEC_GP + g * DS + dd];
                }
                out[(size_t)b * out_stride + (size_t)(kvh * G + g) * HD + rank * DS + dd] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
            }
    }
    if (gave_up && tid == 0 && status) atomicExch(status, 5);
}

// pages [n_pages, nkv, 64, hd] seen as a matrix [n_pages * nkv * 64, hd]; box = 64 rows x 64 columns, 128-byte swizzle
typedef CUresult (*DecEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int dec_make_map(CUtensorMap* map, const void* pages, long long rows, int hd, int box_rows = 64) {
    static DecEncodeFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qr) != cudaSuccess ||
            qr != cudaDriverEntryPointSuccess)
            return RF_ERR_UNSUPPORTED;
        fn = reinterpret_cast<DecEncodeFn>(ptr);
    }
    if (reinterpret_cast<uintptr_t>(pages) & 15) return RF_ERR_BAD_ARG;
    cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pages), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : RF_ERR_BAD_ARG;
}

template <int EPL, int ROWS, int WARPS>
static int launch_warps(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                        const void* v_pages, long long n_pages, const int* tok_seq, const int* tok_pos,
                        const int* seq_slot, const int* block_table, int max_pages, int nh, int nkv, float scale,
                        int window, int B, int splits, int* status, cudaStream_t st) {
    constexpr int HD = EPL * 32;
    const size_t smem = (size_t)WARPS * 2 * ROWS * HD * 2 +
                        (size_t)(WARPS * DEC_GP + 2 * DEC_GP + 16 * 2 * DEC_GP + DEC_GP * HD) * sizeof(float) + WARPS * 2 * 8 + 16 + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_decode_warps_kernel<EPL, ROWS, WARPS>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        // clusters of 16 (one sequence with a long context: 4 kv heads x 16 CTAs) are beyond the portable size
        e = cudaFuncSetAttribute(attention_decode_warps_kernel<EPL, ROWS, WARPS>,
                                 cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(splits, nkv, B);
    cfg.blockDim = dim3(WARPS * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (splits > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = splits; attr[n].val.clusterDim.y = 1; attr[n].val.clusterDim.z = 1;
        ++n;
    }
    if (g_rf_pdl) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    CUtensorMap mk, mv;
    int me;
    if ((me = dec_make_map(&mk, k_pages, n_pages * nkv * RF_PAGE, HD, ROWS)) ||
        (me = dec_make_map(&mv, v_pages, n_pages * nkv * RF_PAGE, HD, ROWS)))
        return me;
    cudaError_t e = cudaLaunchKernelEx(&cfg, attention_decode_warps_kernel<EPL, ROWS, WARPS>, mk, mv,
        reinterpret_cast<const __nv_bfloat16*>(q), q_stride, reinterpret_cast<__nv_bfloat16*>(out), out_stride, tok_seq,
        tok_pos, seq_slot, block_table, max_pages, nh, nkv, scale, window, splits, status);
    if (e != cudaSuccess) return (int)e;
    RF_LAUNCH_CHECK();
    return 0;
}

template <int EPL>
static int launch(const void* q, int q_stride, void* out, int out_stride, const void* k_pages, const void* v_pages,
                  const int* tok_seq, const int* tok_pos, const int* seq_slot, const int* block_table,
                  int max_pages, int nh, int nkv, float scale, int window, int B, int max_chunks,
                  float* part_o, float* part_ml, int* counters, int* status, cudaStream_t st) {
    constexpr int HD = EPL * 32;
    const size_t smem = (size_t)2 * DEC_CHUNK * HD * 2 + (DEC_GP * DEC_CHUNK + DEC_WARPS * DEC_GP) * sizeof(float) + 16;
    static bool configured = false;
    if (!configured && smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<EPL>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(max_chunks, nkv, B);
    rf_launch(attention_decode_kernel<EPL>, grid, dim3(DEC_THREADS), smem, st,
        reinterpret_cast<const __nv_bfloat16*>(q), q_stride, reinterpret_cast<__nv_bfloat16*>(out), out_stride,
        reinterpret_cast<const __nv_bfloat16*>(k_pages), reinterpret_cast<const __nv_bfloat16*>(v_pages), tok_seq,
        tok_pos, seq_slot, block_table, max_pages, nh, nkv, scale, window, max_chunks, part_o, part_ml, counters, status);
    RF_LAUNCH_CHECK();
    return 0;
}

extern "C" {

// What this kernel takes: head sizes whose rows split evenly over 32 lanes, up to 8 query heads per kv head,
// and at most DEC_CHUNK chunks (16,384 keys) per sequence: the merge keeps one weight per chunk in shared memory.
int rf_attention_decode_supported(int nh, int nkv, int hd) {
    if (nkv <= 0 || nh % nkv || nh / nkv > DEC_GP) return 0;
    return hd == 64 || hd == 128 || hd == 256;
}

int rf_attention_decode_chunk() { return DEC_CHUNK; }

// Scratch sizes in elements for B sequences: part_o, part_ml (floats), counters (ints, zero before the first launch).
void rf_attention_decode_scratch(int B, int nh, int nkv, int hd, int max_chunks, long long* n_part_o,
                                 long long* n_part_ml, long long* n_counters) {
    *n_part_o = (long long)B * nh * max_chunks * hd;
    *n_part_ml = (long long)B * nh * max_chunks * 2;
    *n_counters = (long long)B * nkv;
}

// A warp per tile of keys, `warps` (4 or 8) warps per CTA.
int rf_attention_decode_warps(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                              const void* v_pages, long long n_pages, const int* tok_seq, const int* tok_pos,
                              const int* seq_slot, const int* block_table, int max_pages, int nh, int nkv, int hd,
                              float scale, int window, int B, int splits, int warps, int* status, cudaStream_t st) {
    if (B <= 0) return 0;
    if (!rf_attention_decode_supported(nh, nkv, hd)) return RF_ERR_UNSUPPORTED;
    if (nkv > 65535 || B > 65535) return RF_ERR_UNSUPPORTED;
    if (splits != 1 && splits != 2 && splits != 4 && splits != 8 && splits != 16) return RF_ERR_BAD_ARG;
    if (warps != 4 && warps != 8) return RF_ERR_BAD_ARG;
    if ((reinterpret_cast<uintptr_t>(q) & 15) || (q_stride * 2) % 16) return RF_ERR_BAD_ARG;
#define GOW(EPL, ROWS, WARPS) return launch_warps<EPL, ROWS, WARPS>(q, q_stride, out, out_stride, k_pages, v_pages, n_pages, tok_seq, \
                              tok_pos, seq_slot, block_table, max_pages, nh, nkv, scale, window, B, splits, status, st)
    if (hd == 64) { if (warps == 8) GOW(2, 32, 8); GOW(2, 32, 4); }
    if (hd == 128) { if (warps == 8) GOW(4, 32, 8); GOW(4, 32, 4); }
    if (warps == 8) GOW(8, 16, 8);
    GOW(8, 16, 4);
#undef GOW
}

int rf_attention_decode(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                        const void* v_pages, const int* tok_seq, const int* tok_pos, const int* seq_slot,
                        const int* block_table, int max_pages, int nh, int nkv, int hd, float scale, int window,
                        int B, int max_chunks, float* part_o, float* part_ml, int* counters, int* status,
                        cudaStream_t st) {
    if (B <= 0) return 0;
    if (!rf_attention_decode_supported(nh, nkv, hd) || max_chunks <= 0 || max_chunks > DEC_CHUNK || B > 65535)
        return RF_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(q) & 15) || (q_stride * 2) % 16) return RF_ERR_BAD_ARG;
#define GO(EPL) return launch<EPL>(q, q_stride, out, out_stride, k_pages, v_pages, tok_seq, tok_pos, seq_slot, \
                                   block_table, max_pages, nh, nkv, scale, window, B, max_chunks, part_o, part_ml, \
                                   counters, status, st)
    if (hd == 64) GO(2);
    if (hd == 128) GO(4);
    GO(8);
#undef GO
}

}
