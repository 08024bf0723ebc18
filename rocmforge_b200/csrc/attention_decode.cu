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

// ---------------------------------------------------------------- the clustered variant
// For contexts of ordinary length the merge through global memory above costs more than the attention
// itself (write partials, fence, count arrivals, fence, read them back: five trips to L2).  Here the
// CTAs that share a (sequence, kv head) form a thread-block cluster of `splits` CTAs instead.  CTA r
// walks the pages r, r + splits, r + 2*splits, ... of the context with a ring of TMA copies (128-byte
// swizzle, so that ldmatrix reads the key and value fragments without bank conflicts; with plain
// 256-byte rows the fragment loads were 8-way conflicted and took most of a page's time); each warp
// owns 16 of a page's 64 keys and keeps its own running maximum, sum and output
// across pages (the online softmax, as in the prefill kernel), so a page costs one mbarrier wait and
// one CTA barrier.  At the end the four warps' states are merged in shared memory, and CTA 0 reads its
// peers' states through distributed shared memory, in rank order, and writes the result.  No scratch
// memory, no atomics; the launch shape depends on the batch alone, so a captured graph stays valid
// while the context grows.
#define DCL_MAX_STAGES 6
#define DCL_MAX_PAGES 256             // pages one CTA may walk (16,384 keys)

__device__ __forceinline__ uint32_t dcl_cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void dcl_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float dcl_ld_remote(const float* local, uint32_t rank) {
    uint32_t raddr;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(raddr) : "r"(dec_smem_u32(local)), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(raddr) : "memory");
    return v;
}

template <int EPL>
__global__ void __launch_bounds__(DEC_THREADS)
attention_decode_cluster_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                                const __nv_bfloat16* __restrict__ q, int q_stride, __nv_bfloat16* __restrict__ out,
                                int out_stride, const int* __restrict__ tok_seq,
                                const int* __restrict__ tok_pos, const int* __restrict__ seq_slot,
                                const int* __restrict__ block_table, int max_pages, int nh, int nkv, float scale,
                                int window, int splits, int stages, int* __restrict__ status) {
    constexpr int HD = EPL * 32;
    constexpr uint32_t SLAB = RF_PAGE * HD * 2;                 // one page's keys (or values) of one kv head
    constexpr int HALVES = HD / 64;                             // 128-byte column blocks of a row
    constexpr uint32_t HALF_BYTES = RF_PAGE * 128;              // one column block of a page: [64 rows][128 B], swizzled
    extern __shared__ __align__(1024) uint8_t dec_smem[];
    // the swizzle pattern is a function of the address: the ring starts on a 1024-byte boundary (the same in every CTA)
    uint8_t* ring = dec_smem + ((1024u - (dec_smem_u32(dec_smem) & 1023u)) & 1023u);    // [stage][K | V][HALVES][64][128 B]
    float* w_m = reinterpret_cast<float*>(ring);                                       // [4 warps][GP]: over the ring,
    float* w_l = w_m + DEC_WARPS * DEC_GP;                                              // [4][GP]        once the last
    float* w_o = w_l + DEC_WARPS * DEC_GP;                                              // [4][GP][HD]    page is done
    float* c_m = reinterpret_cast<float*>(ring + (size_t)stages * 2 * SLAB);            // this CTA: [GP]
    float* c_l = c_m + DEC_GP;                                                          // [GP]
    float* c_o = c_l + DEC_GP;                                                          // [GP][HD]
    uint64_t* bars = reinterpret_cast<uint64_t*>(c_o + DEC_GP * HD);                   // [stages]
    __shared__ int gave_up;
    __shared__ int page_of[DCL_MAX_PAGES];              // this CTA's pages, read from the block table once

    pdl_trigger();
    const int G = nh / nkv;
    const int kvh = blockIdx.y, b = blockIdx.z, tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5, gid = lane >> 2, tig = lane & 3;
    const int rank = splits > 1 ? (int)dcl_cluster_rank() : 0;
    const int pos = tok_pos[b];
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int p_lo = lo / RF_PAGE, p_hi = pos / RF_PAGE;
    const int n_my = (p_hi - p_lo - rank) >= 0 ? (p_hi - p_lo - rank) / splits + 1 : 0;     // pages of this CTA
    const int* bt = block_table + (size_t)seq_slot[tok_seq[b]] * max_pages;
    if (p_hi - p_lo + 1 > DCL_MAX_PAGES * splits) {     // more pages than a CTA's table holds: the same verdict in
        if (tid == 0 && status) atomicExch(status, 7);  // every CTA of the cluster; the caller bounds the context
        return;
    }
    // the block table is not written by any kernel of the step: fetch this CTA's entries now, all at once,
    // instead of one dependent global load per page on the copy-issuing thread's critical path
    for (int k = tid; k < n_my && k < DCL_MAX_PAGES; k += DEC_THREADS) page_of[k] = bt[p_lo + rank + k * splits];

    if (tid == 0) {
        gave_up = 0;
        for (int s = 0; s < stages; ++s)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(dec_smem_u32(&bars[s])));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
    }
    __syncthreads();

    auto issue = [&](int k) {                           // thread 0: page p_lo + rank + k*splits into stage k % stages
        const int stage = k % stages;
        const uint32_t bar = dec_smem_u32(&bars[stage]);
        const int row = (page_of[k] * nkv + kvh) * RF_PAGE;      // first row of the page in the [pages*kv*64, HD] view
        const uint32_t dst = dec_smem_u32(ring + (size_t)stage * 2 * SLAB);
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(2 * SLAB) : "memory");
#pragma unroll
        for (int h = 0; h < HALVES; ++h) {
            asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                         ::"r"(dst + h * HALF_BYTES), "l"(&map_k), "r"(h * 64), "r"(row), "r"(bar) : "memory");
            asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                         ::"r"(dst + SLAB + h * HALF_BYTES), "l"(&map_v), "r"(h * 64), "r"(row), "r"(bar) : "memory");
        }
    };
    // Only the page of the newest position is written in this step (by the kernel before this one); the
    // older pages were written by earlier steps, which are complete: their copies start before the wait.
    int early = 0;
    if (tid == 0)
        for (; early < n_my && early < stages - 1 && p_lo + rank + early * splits < p_hi; ++early) issue(early);
    pdl_wait();                                         // queries and the newest keys/values come from the kernel before us
    if (tid == 0)
        for (int k = early; k < n_my && k < stages - 1; ++k) issue(k);

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
    float oc[HD / 8][2];                                 // this thread: head gid, dims nt*8 + tig*2 + {0,1}
#pragma unroll
    for (int nt = 0; nt < HD / 8; ++nt) oc[nt][0] = oc[nt][1] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;

    for (int k = 0; k < n_my; ++k) {
        const int stage = k % stages;
        if (tid == 0 && k + stages - 1 < n_my) issue(k + stages - 1);              // its stage was released by the last sync
        {
            const uint32_t bar = dec_smem_u32(&bars[stage]);
            const uint32_t parity = (k / stages) & 1;
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
                    if (now - t0 > DEC_WAIT_LIMIT_NS || gave_up) { gave_up = 1; break; }
                }
            }
        }
        __syncthreads();                                 // one verdict for everyone
        if (gave_up) break;
        const uint32_t k_t = dec_smem_u32(ring + (size_t)stage * 2 * SLAB), v_t = k_t + SLAB;
        const int key0 = (p_lo + rank + k * splits) * RF_PAGE;
        int k_begin = lo - key0; if (k_begin < 0) k_begin = 0;                    // valid rows of this page
        int k_last = pos - key0; if (k_last > RF_PAGE - 1) k_last = RF_PAGE - 1;
        if (k_begin > 0 || k_last < RF_PAGE - 1) {
            // rows outside the sequence get weight zero, but 0 * (whatever bits lie there) must be 0
            // (the swizzle permutes 16-byte pieces inside a row: clearing whole rows needs no address math)
            for (int i = tid; i < RF_PAGE * HALVES * 8; i += DEC_THREADS) {
                const int row = (i >> 3) % RF_PAGE, h = i / (RF_PAGE * 8);
                if (row < k_begin || row > k_last)
                    asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(v_t + h * HALF_BYTES + row * 128 + (i & 7) * 16),
                                 "r"(0u) : "memory");
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncthreads();
        }
        // ---- scores of this warp's 16 keys: two tiles of 8, both from one ldmatrix.x4 per 16 dimensions
        const int kb = warp * 16;
        float sc[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
        const bool warp_active = kb <= k_last && kb + 15 >= k_begin;
        if (warp_active) {
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) {
                // matrices: (keys kb + 0..7, dims ks*16 + 0..7), (same keys, dims + 8), (keys + 8, dims), (keys + 8, dims + 8)
                const int mi = lane >> 3, r = lane & 7;
                const int krow = kb + (mi >> 1) * 8 + r;
                const int gc = ks * 2 + (mi & 1);                                  // 16-byte chunk along the row
                const uint32_t a = k_t + (gc >> 3) * HALF_BYTES + krow * 128 + (((gc & 7) ^ (krow & 7)) << 4);
                uint32_t b0, b1, b2, b3;
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(a));
                asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                             : "+f"(sc[0][0]), "+f"(sc[0][1]), "+f"(sc[0][2]), "+f"(sc[0][3])
                             : "r"(qa[ks][0]), "r"(0u), "r"(qa[ks][1]), "r"(0u), "r"(b0), "r"(b1));
                asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                             : "+f"(sc[1][0]), "+f"(sc[1][1]), "+f"(sc[1][2]), "+f"(sc[1][3])
                             : "r"(qa[ks][0]), "r"(0u), "r"(qa[ks][1]), "r"(0u), "r"(b2), "r"(b3));
            }
        }
        float mx = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int kk = kb + nt * 8 + tig * 2 + e;
                const bool ok = warp_active && kk >= k_begin && kk <= k_last;
                sc[nt][e] = ok ? sc[nt][e] * scale : -INFINITY;
                mx = fmaxf(mx, sc[nt][e]);
            }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run, mx);
        const float corr = (m_run == -INFINITY) ? 0.f : expf(m_run - m_new);
        float psum = 0.f;
        uint32_t pa[2];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            const float p0 = sc[nt][0] == -INFINITY ? 0.f : expf(sc[nt][0] - m_new);
            const float p1 = sc[nt][1] == -INFINITY ? 0.f : expf(sc[nt][1] - m_new);
            psum += p0 + p1;
            const __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
            pa[nt] = *reinterpret_cast<const uint32_t*>(&pk);
        }
        psum += __shfl_xor_sync(0xffffffffu, psum, 1);
        psum += __shfl_xor_sync(0xffffffffu, psum, 2);
        l_run = l_run * corr + psum;
        m_run = m_new;
#pragma unroll
        for (int nt = 0; nt < HD / 8; ++nt) { oc[nt][0] *= corr; oc[nt][1] *= corr; }
        if (warp_active) {
#pragma unroll
            for (int nt = 0; nt < HD / 8; nt += 2) {
                const int mi = lane >> 3, r = lane & 7;
                const int vrow = kb + (mi & 1) * 8 + r, gc = nt + (mi >> 1);
                const uint32_t va = v_t + (gc >> 3) * HALF_BYTES + vrow * 128 + (((gc & 7) ^ (vrow & 7)) << 4);
                uint32_t v0, v1, v2, v3;
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(v0), "=r"(v1), "=r"(v2), "=r"(v3) : "r"(va));
                float d0[4] = {oc[nt][0], oc[nt][1], 0.f, 0.f}, d1[4] = {oc[nt + 1][0], oc[nt + 1][1], 0.f, 0.f};
                asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                             : "+f"(d0[0]), "+f"(d0[1]), "+f"(d0[2]), "+f"(d0[3])
                             : "r"(pa[0]), "r"(0u), "r"(pa[1]), "r"(0u), "r"(v0), "r"(v1));
                asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                             : "+f"(d1[0]), "+f"(d1[1]), "+f"(d1[2]), "+f"(d1[3])
                             : "r"(pa[0]), "r"(0u), "r"(pa[1]), "r"(0u), "r"(v2), "r"(v3));
                oc[nt][0] = d0[0]; oc[nt][1] = d0[1]; oc[nt + 1][0] = d1[0]; oc[nt + 1][1] = d1[1];
            }
        }
        __syncthreads();                                 // the stage may be refilled
    }

    // ---- the four warps' states -> this CTA's state
    if (tig == 0) { w_m[warp * DEC_GP + gid] = m_run; w_l[warp * DEC_GP + gid] = l_run; }
#pragma unroll
    for (int nt = 0; nt < HD / 8; ++nt) {
        w_o[(warp * DEC_GP + gid) * HD + nt * 8 + tig * 2] = oc[nt][0];
        w_o[(warp * DEC_GP + gid) * HD + nt * 8 + tig * 2 + 1] = oc[nt][1];
    }
    __syncthreads();
    for (int i = tid; i < DEC_GP * HD; i += DEC_THREADS) {
        const int g = i / HD, d = i - g * HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, w_m[w * DEC_GP + g]);
        float L = 0.f, O = 0.f;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) {            // warps in index order
            const float mw = w_m[w * DEC_GP + g];
            const float f = mw == -INFINITY ? 0.f : expf(mw - M);
            L += f * w_l[w * DEC_GP + g];
            O += f * w_o[(w * DEC_GP + g) * HD + d];
        }
        c_o[g * HD + d] = O;
        if (d == 0) { c_m[g] = M; c_l[g] = L; }
    }
    __syncthreads();
    if (splits > 1) dcl_cluster_sync();                  // every CTA's state is complete and visible in the cluster
    if (rank == 0 && !gave_up) {
        // Bring the peers' states (max | sum | output, contiguous) into this CTA's memory first: batches of
        // independent 16-byte remote loads, so that their latencies overlap instead of adding up.
        constexpr int STATE4 = (2 * DEC_GP + DEC_GP * HD) / 4;            // float4 per CTA state
        float4* stage = reinterpret_cast<float4*>(ring);                    // [splits - 1][STATE4], over the ring
        const int total = (splits - 1) * STATE4;
        for (int i0 = tid; i0 < total; i0 += DEC_THREADS * 4) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + u * DEC_THREADS;
                if (i < total) {
                    const int r = 1 + i / STATE4, j = i - (r - 1) * STATE4;
                    uint32_t raddr;
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(raddr) : "r"(dec_smem_u32(c_m) + 16 * j), "r"(r));
                    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                                 : "=f"(v[u].x), "=f"(v[u].y), "=f"(v[u].z), "=f"(v[u].w) : "r"(raddr) : "memory");
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + u * DEC_THREADS;
                if (i < total) stage[i] = v[u];
            }
        }
        __syncthreads();
        const float* st = reinterpret_cast<const float*>(stage);
        for (int i = tid; i < G * HD; i += DEC_THREADS) {
            const int g = i / HD, d = i - g * HD;
            float M = c_m[g];
            for (int r = 1; r < splits; ++r) M = fmaxf(M, st[(r - 1) * STATE4 * 4 + g]);
            float L = 0.f, O = 0.f;
            for (int r = 0; r < splits; ++r) {           // CTAs in rank order
                const float* base = st + (r - 1) * STATE4 * 4;
                const float mr = r ? base[g] : c_m[g];
                const float f = mr == -INFINITY ? 0.f : expf(mr - M);
                L += f * (r ? base[DEC_GP + g] : c_l[g]);
                O += f * (r ? base[2 * DEC_GP + g * HD + d] : c_o[g * HD + d]);
            }
            out[(size_t)b * out_stride + (size_t)(kvh * G + g) * HD + d] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
        }
    }
    if (splits > 1) dcl_cluster_sync();                  // peers stay until their state has been read
    if (gave_up && tid == 0 && status) atomicExch(status, 5);
}

// pages [n_pages, nkv, 64, hd] seen as a matrix [n_pages * nkv * 64, hd]; box = 64 rows x 64 columns, 128-byte swizzle
typedef CUresult (*DecEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int dec_make_map(CUtensorMap* map, const void* pages, long long rows, int hd) {
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
    cuuint32_t box[2] = {64, 64};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pages), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : RF_ERR_BAD_ARG;
}

template <int EPL>
static int launch_cluster(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                          const void* v_pages, long long n_pages, const int* tok_seq, const int* tok_pos, const int* seq_slot,
                          const int* block_table, int max_pages, int nh, int nkv, float scale, int window, int B,
                          int splits, int stages, int* status, cudaStream_t st) {
    constexpr int HD = EPL * 32;
    auto bytes = [](int n) {
        return (size_t)n * 2 * RF_PAGE * HD * 2 + (size_t)(2 * DEC_GP + DEC_GP * HD) * sizeof(float) + DCL_MAX_STAGES * 8 + 16 + 1024;
    };
    while (stages > 2 && bytes(stages) > 200 * 1024) --stages;        // head_dim 256: fewer stages fit
    const size_t smem = bytes(stages);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_decode_cluster_kernel<EPL>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(200 * 1024));
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(splits, nkv, B);
    cfg.blockDim = dim3(DEC_THREADS);
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
    if ((me = dec_make_map(&mk, k_pages, n_pages * nkv * RF_PAGE, HD)) || (me = dec_make_map(&mv, v_pages, n_pages * nkv * RF_PAGE, HD)))
        return me;
    cudaError_t e = cudaLaunchKernelEx(&cfg, attention_decode_cluster_kernel<EPL>, mk, mv,
        reinterpret_cast<const __nv_bfloat16*>(q), q_stride, reinterpret_cast<__nv_bfloat16*>(out), out_stride, tok_seq,
        tok_pos, seq_slot, block_table, max_pages, nh, nkv, scale, window, splits, stages, status);
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

// The clustered variant: `splits` (1, 2, 4 or 8) CTAs share a (sequence, kv head); no scratch memory.
// `stages` (2..6) pages of keys and values are in flight per CTA: 3 lets two CTAs share an SM (many
// sequences), 6 hides the copy latency when a single CTA walks a whole context (few sequences).
int rf_attention_decode_cluster(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                                const void* v_pages, long long n_pages, const int* tok_seq, const int* tok_pos,
                                const int* seq_slot,
                                const int* block_table, int max_pages, int nh, int nkv, int hd, float scale,
                                int window, int B, int splits, int stages, int* status, cudaStream_t st) {
    if (B <= 0) return 0;
    if (!rf_attention_decode_supported(nh, nkv, hd) || B > 65535) return RF_ERR_UNSUPPORTED;
    if (stages < 2 || stages > DCL_MAX_STAGES) return RF_ERR_BAD_ARG;
    if (splits != 1 && splits != 2 && splits != 4 && splits != 8) return RF_ERR_BAD_ARG;
    if ((reinterpret_cast<uintptr_t>(q) & 15) || (q_stride * 2) % 16) return RF_ERR_BAD_ARG;
#define GOC(EPL) return launch_cluster<EPL>(q, q_stride, out, out_stride, k_pages, v_pages, n_pages, tok_seq, tok_pos, seq_slot, \
                                            block_table, max_pages, nh, nkv, scale, window, B, splits, stages, status, st)
    if (hd == 64) GOC(2);
    if (hd == 128) GOC(4);
    GOC(8);
#undef GOC
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
