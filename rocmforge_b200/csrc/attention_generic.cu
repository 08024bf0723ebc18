// Attention of new tokens over the paged cache, for every head size, group size and
// window: the plain kernel that the true 32-bit path always uses and that the
// bfloat16 path uses for whatever the tuned kernels refuse.
//
// One block of 128 threads per (query token, kv head): the query heads that share the kv head (eight at a
// time) are served from one pass over the keys and values, so the cache is read once per group instead of
// once per head.  Keys are taken a chunk (128, or 64 for head sizes above 256) at a time: the chunk is
// copied into shared memory with coalesced loads and widened to 32-bit, a thread scores one key against
// every head of the group, the block keeps each head's running maximum and sum (online softmax, all in
// 32-bit), the values replace the keys in shared memory, and every thread accumulates its (head, output
// dimension) pairs over the chunk.  The order of the sums depends on the query's position alone, never on
// the batch.
//
// What it computes is maeddesg/ROCmForge's flash_attn_verify_all_heads_kernel
// ("N new rows attend over the cache", hip_kernels/attention.hip:1121-1287) with the
// formulas of src/cpu/ops.rs:195-303: kv head = head / (heads / kv_heads), score =
// dot(q,k) / sqrt(head_dim), a query at position p sees keys 0..=p.
#include "common.cuh"

#define ATT_THREADS 128
#define ATT_WARPS 4
#define ATT_MAX_HD 512
#define ATT_GB 8                                    // query heads of a group served by one pass

template <typename T> struct Vec4;
template <> struct Vec4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
};
template <> struct Vec4<__nv_bfloat16> {
    static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);           // a bfloat16 is the upper half of a float
        return make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                           __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
    }
};

template <typename T, int CK>
__global__ void __launch_bounds__(ATT_THREADS)
attention_generic_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride,
                         const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                         const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                         const int* __restrict__ seq_slot, const int* __restrict__ block_table,
                         int max_pages, int nh, int nkv, int hd, float scale, int window, int hpb) {
    constexpr int ACC = ATT_GB * (CK == 128 ? 256 : ATT_MAX_HD) / ATT_THREADS;     // (head, dim) pairs of a thread at most
    pdl_trigger();
    pdl_wait();
    extern __shared__ float smem[];
    const int ldk = hd + 1;                         // a key row per thread: odd stride, no bank conflicts
    float* qs = smem;                               // [GB][hd]
    float* kv = qs + ATT_GB * hd;                   // [CK][hd + 1]: the chunk's keys, then its values
    float* probs = kv + CK * ldk;                   // [GB][CK]
    float* red = probs + ATT_GB * CK;               // [ATT_WARPS][GB]

    const int t = blockIdx.x, kvh = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = nh / nkv;
    const int pos = tok_pos[t];
    const int slot = seq_slot[tok_seq[t]];
    const int* bt = block_table + (size_t)slot * max_pages;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;

    const bool vec = (hd & 3) == 0;                 // rows of whole 4-element groups: 16-byte (8-byte) loads
    const int hq = hd >> 2;
    auto load_chunk = [&](const T* __restrict__ pages, int c0, int cnt) {
        if (vec) {
            // the chunk as cnt * hd/4 groups of four elements, eight independent loads per thread in flight
            const int total = cnt * hq;
            for (int base = tid; base < total; base += 8 * ATT_THREADS) {
                float4 got[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int idx = base + u * ATT_THREADS;
                    if (idx < total) {
                        const int r = idx / hq, c = (idx - r * hq) * 4, j = c0 + r;
                        got[u] = Vec4<T>::load(pages + (((size_t)bt[j / RF_PAGE] * nkv + kvh) * RF_PAGE + (j % RF_PAGE)) * hd + c);
                    }
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int idx = base + u * ATT_THREADS;
                    if (idx < total) {
                        const int r = idx / hq, c = (idx - r * hq) * 4;
                        float* dst = kv + r * ldk + c;
                        dst[0] = got[u].x; dst[1] = got[u].y; dst[2] = got[u].z; dst[3] = got[u].w;
                    }
                }
            }
            return;
        }
        for (int r = warp; r < cnt; r += ATT_WARPS) {           // a warp copies whole rows: coalesced
            const int j = c0 + r;
            const T* src = pages + (((size_t)bt[j / RF_PAGE] * nkv + kvh) * RF_PAGE + (j % RF_PAGE)) * hd;
            for (int i = lane; i < hd; i += 32) kv[r * ldk + i] = Cvt<T>::to_f32(src[i]);
        }
    };

    // heads per block (hpb <= 8): the host spreads a group over several blocks when there are few tokens
    for (int g0 = blockIdx.z * hpb; g0 < G; g0 += gridDim.z * hpb) {
        const int gb = min(hpb, G - g0);
        __syncthreads();                            // the previous pass is done with shared memory
        for (int i = tid; i < gb * hd; i += ATT_THREADS) {
            const int g = i / hd, d = i - g * hd;
            qs[i] = Cvt<T>::to_f32(q[(size_t)t * q_stride + (size_t)(kvh * G + g0 + g) * hd + d]);
        }
        float m_run[ATT_GB], l_run[ATT_GB], acc[ACC];
#pragma unroll
        for (int g = 0; g < ATT_GB; ++g) { m_run[g] = -INFINITY; l_run[g] = 0.f; }
#pragma unroll
        for (int i = 0; i < ACC; ++i) acc[i] = 0.f;

        for (int c0 = lo; c0 <= pos; c0 += CK) {
            const int cnt = min(CK, pos - c0 + 1);
            __syncthreads();                        // the values of the chunk before are used up (and qs is written)
            load_chunk(k_pages, c0, cnt);
            __syncthreads();
            // ---- scores of key tid against every head of the pass
            float s[ATT_GB];
#pragma unroll
            for (int g = 0; g < ATT_GB; ++g) s[g] = -INFINITY;
            if (tid < cnt) {
                float d[ATT_GB];
#pragma unroll
                for (int g = 0; g < ATT_GB; ++g) d[g] = 0.f;
                const float* kr = kv + tid * ldk;
                for (int i = 0; i < hd; ++i) {
                    const float kk = kr[i];
#pragma unroll
                    for (int g = 0; g < ATT_GB; ++g)
                        if (g < gb) d[g] = fmaf(qs[g * hd + i], kk, d[g]);
                }
#pragma unroll
                for (int g = 0; g < ATT_GB; ++g)
                    if (g < gb) s[g] = d[g] * scale;
            }
            // ---- the chunk's maximum per head: warps, then the block
#pragma unroll
            for (int g = 0; g < ATT_GB; ++g) {
                const float w = warp_max(s[g]);
                if (lane == 0) red[warp * ATT_GB + g] = w;
            }
            __syncthreads();
            float corr[ATT_GB], p[ATT_GB];
#pragma unroll
            for (int g = 0; g < ATT_GB; ++g) {
                float cm = red[g];
#pragma unroll
                for (int w = 1; w < ATT_WARPS; ++w) cm = fmaxf(cm, red[w * ATT_GB + g]);
                const float m_new = fmaxf(m_run[g], cm);
                p[g] = (tid < cnt && g < gb) ? expf(s[g] - m_new) : 0.f;
                corr[g] = (m_run[g] == -INFINITY) ? 0.f : expf(m_run[g] - m_new);
                m_run[g] = m_new;
                if (tid < CK) probs[g * CK + tid] = p[g];
            }
            __syncthreads();                        // every thread has read the maxima; the keys are used up
            // ---- the chunk's sums (warps in index order), and the values into shared memory
#pragma unroll
            for (int g = 0; g < ATT_GB; ++g) {
                const float w = warp_sum(p[g]);
                if (lane == 0) red[warp * ATT_GB + g] = w;
            }
            load_chunk(v_pages, c0, cnt);
            __syncthreads();
#pragma unroll
            for (int g = 0; g < ATT_GB; ++g) {
                float cs = red[g];
#pragma unroll
                for (int w = 1; w < ATT_WARPS; ++w) cs += red[w * ATT_GB + g];
                l_run[g] = l_run[g] * corr[g] + cs;
            }
            // ---- output: this thread's (head, dimension) pairs over the chunk's keys in order
#pragma unroll
            for (int i = 0; i < ACC; ++i) {
                const int e = tid + i * ATT_THREADS;
                if (e < gb * hd) {
                    const int g = e / hd, d = e - g * hd;
                    float c = 0.f;
#pragma unroll
                    for (int gg = 0; gg < ATT_GB; ++gg) if (gg == g) c = corr[gg];
                    // four interleaved sums (keys j, j+1, j+2, j+3 of every four), combined pairwise: the order is fixed
                    // by the chunk alone, and four chains hide the latency of one
                    const float* pr = probs + g * CK;
                    const float* vv = kv + d;
                    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
                    int j = 0;
                    for (; j + 3 < cnt; j += 4) {
                        a0 = fmaf(pr[j], vv[j * ldk], a0);
                        a1 = fmaf(pr[j + 1], vv[(j + 1) * ldk], a1);
                        a2 = fmaf(pr[j + 2], vv[(j + 2) * ldk], a2);
                        a3 = fmaf(pr[j + 3], vv[(j + 3) * ldk], a3);
                    }
                    for (; j < cnt; ++j) a0 = fmaf(pr[j], vv[j * ldk], a0);
                    acc[i] = acc[i] * c + ((a0 + a1) + (a2 + a3));
                }
            }
        }
#pragma unroll
        for (int i = 0; i < ACC; ++i) {
            const int e = tid + i * ATT_THREADS;
            if (e < gb * hd) {
                const int g = e / hd, d = e - g * hd;
                float l = 0.f;
#pragma unroll
                for (int gg = 0; gg < ATT_GB; ++gg) if (gg == g) l = l_run[gg];
                out[(size_t)t * out_stride + (size_t)(kvh * G + g0 + g) * hd + d] = Cvt<T>::from_f32(l > 0.f ? acc[i] / l : 0.f);
            }
        }
    }
}

template <typename T, int CK>
static int launch_ck(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                     const void* v_pages, const int* tok_seq, const int* tok_pos, const int* seq_slot,
                     const int* block_table, int max_pages, int nh, int nkv, int hd, float scale, int window,
                     int T_, cudaStream_t st) {
    const size_t smem = ((size_t)ATT_GB * hd + (size_t)CK * (hd + 1) + ATT_GB * CK + ATT_WARPS * ATT_GB) * sizeof(float);
    static size_t configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_generic_kernel<T, CK>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    // tokens along x: no 65,535 limit on a step's tokens.  All heads of a group in one block (the cache is read once per
    // group) when the tokens alone give every SM a block; with fewer tokens fewer heads per block, down to one (a block
    // per SM and not two: 64 sequences of 2 kv heads x 7 heads took 225 us in 512 blocks of 2 heads, 127 us in 256 of 4)
    const int G = nh / nkv;
    int hpb = ATT_GB;
    while (hpb > 1 && (long long)T_ * nkv * ((G + hpb - 1) / hpb) < 148) hpb >>= 1;
    const int zb = (G + hpb - 1) / hpb;
    if (zb > 65535) return RF_ERR_UNSUPPORTED;
    dim3 grid(T_, nkv, zb);
    rf_launch(attention_generic_kernel<T, CK>, grid, dim3(ATT_THREADS), smem, st,
        reinterpret_cast<const T*>(q), q_stride, reinterpret_cast<T*>(out), out_stride,
        reinterpret_cast<const T*>(k_pages), reinterpret_cast<const T*>(v_pages), tok_seq, tok_pos, seq_slot,
        block_table, max_pages, nh, nkv, hd, scale, window, hpb);
    RF_LAUNCH_CHECK();
    return 0;
}

template <typename T>
static int launch(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                  const void* v_pages, const int* tok_seq, const int* tok_pos, const int* seq_slot,
                  const int* block_table, int max_pages, int nh, int nkv, int hd, float scale, int window,
                  int T_, cudaStream_t st) {
    if (T_ <= 0) return 0;
    if (hd <= 0 || hd > ATT_MAX_HD || nkv <= 0 || nh % nkv || nkv > 65535) return RF_ERR_UNSUPPORTED;
    if (hd <= 256)
        return launch_ck<T, 128>(q, q_stride, out, out_stride, k_pages, v_pages, tok_seq, tok_pos, seq_slot, block_table,
                                 max_pages, nh, nkv, hd, scale, window, T_, st);
    return launch_ck<T, 64>(q, q_stride, out, out_stride, k_pages, v_pages, tok_seq, tok_pos, seq_slot, block_table,
                            max_pages, nh, nkv, hd, scale, window, T_, st);
}

extern "C" int rf_attention_generic(int dtype, const void* q, int q_stride, void* out, int out_stride,
                                    const void* k_pages, const void* v_pages, const int* tok_seq,
                                    const int* tok_pos, const int* seq_slot, const int* block_table,
                                    int max_pages, int nh, int nkv, int hd, float scale, int window, int T_,
                                    cudaStream_t st) {
    return dtype == 0
        ? launch<float>(q, q_stride, out, out_stride, k_pages, v_pages, tok_seq, tok_pos, seq_slot, block_table,
                        max_pages, nh, nkv, hd, scale, window, T_, st)
        : launch<__nv_bfloat16>(q, q_stride, out, out_stride, k_pages, v_pages, tok_seq, tok_pos, seq_slot,
                                block_table, max_pages, nh, nkv, hd, scale, window, T_, st);
}
