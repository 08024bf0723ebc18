// Attention of new tokens over the paged cache, for every head size, group size and
// window: the plain kernel that the true 32-bit path always uses and that the
// bfloat16 path uses for whatever the tuned kernels refuse.
//
// One block per (query token, query head).  Keys are taken 128 at a time: a thread
// scores one key, the block keeps the running maximum and sum (online softmax, all in
// 32-bit), then every thread accumulates its output dimensions over the chunk.
// The order of the sums depends on the query's position alone, never on the batch.
//
// What it computes is maeddesg/ROCmForge's flash_attn_verify_all_heads_kernel
// ("N new rows attend over the cache", hip_kernels/attention.hip:1121-1287) with the
// formulas of src/cpu/ops.rs:195-303: kv head = head / (heads / kv_heads), score =
// dot(q,k) / sqrt(head_dim), a query at position p sees keys 0..=p.
#include "common.cuh"

#define ATT_THREADS 128
#define ATT_MAX_HD 512

template <typename T>
__global__ void __launch_bounds__(ATT_THREADS)
attention_generic_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride,
                         const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                         const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                         const int* __restrict__ seq_slot, const int* __restrict__ block_table,
                         int max_pages, int nh, int nkv, int hd, float scale, int window) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float smem[];
    float* qs = smem;                               // hd
    float* probs = qs + hd;                         // ATT_THREADS
    float* red = probs + ATT_THREADS;               // 33
    long long* voff = reinterpret_cast<long long*>(red + 34);   // ATT_THREADS, 8-byte aligned by layout below

    const int head = blockIdx.x, t = blockIdx.y, tid = threadIdx.x;
    const int pos = tok_pos[t];
    const int slot = seq_slot[tok_seq[t]];
    const int kvh = head / (nh / nkv);
    const int* bt = block_table + (size_t)slot * max_pages;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;

    const T* qrow = q + (size_t)t * q_stride + (size_t)head * hd;
    for (int i = tid; i < hd; i += ATT_THREADS) qs[i] = Cvt<T>::to_f32(qrow[i]);
    __syncthreads();

    float m = -INFINITY, l = 0.f;
    float acc[ATT_MAX_HD / ATT_THREADS];
#pragma unroll
    for (int i = 0; i < ATT_MAX_HD / ATT_THREADS; ++i) acc[i] = 0.f;

    for (int c0 = lo; c0 <= pos; c0 += ATT_THREADS) {
        const int j = c0 + tid;
        float s = -INFINITY;
        long long off = 0;
        if (j <= pos) {
            const int page = bt[j / RF_PAGE];
            off = ((long long)page * nkv + kvh) * RF_PAGE * hd + (long long)(j % RF_PAGE) * hd;
            const T* kr = k_pages + off;
            float d = 0.f;
            for (int i = 0; i < hd; ++i) d = fmaf(qs[i], Cvt<T>::to_f32(kr[i]), d);
            s = d * scale;
        }
        const float cm = block_max(s, red);
        const float m_new = fmaxf(m, cm);
        const float p = (j <= pos) ? expf(s - m_new) : 0.f;
        probs[tid] = p;
        voff[tid] = off;
        const float csum = block_sum(p, red);       // also makes probs/voff visible
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * corr + csum;
        const int cnt = (pos - c0 + 1 < ATT_THREADS) ? pos - c0 + 1 : ATT_THREADS;
#pragma unroll
        for (int i = 0; i < ATT_MAX_HD / ATT_THREADS; ++i) {
            const int d = tid + i * ATT_THREADS;
            if (d < hd) {
                float a = acc[i] * corr;
                for (int jj = 0; jj < cnt; ++jj)
                    a = fmaf(probs[jj], Cvt<T>::to_f32(v_pages[voff[jj] + d]), a);
                acc[i] = a;
            }
        }
        m = m_new;
        __syncthreads();
    }
    T* orow = out + (size_t)t * out_stride + (size_t)head * hd;
#pragma unroll
    for (int i = 0; i < ATT_MAX_HD / ATT_THREADS; ++i) {
        const int d = tid + i * ATT_THREADS;
        if (d < hd) orow[d] = Cvt<T>::from_f32(l > 0.f ? acc[i] / l : 0.f);
    }
}

template <typename T>
static int launch(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                  const void* v_pages, const int* tok_seq, const int* tok_pos, const int* seq_slot,
                  const int* block_table, int max_pages, int nh, int nkv, int hd, float scale, int window,
                  int T_, cudaStream_t st) {
    if (T_ <= 0) return 0;
    if (hd <= 0 || hd > ATT_MAX_HD || nkv <= 0 || nh % nkv) return RF_ERR_UNSUPPORTED;
    if (T_ > 65535) return RF_ERR_UNSUPPORTED;
    // qs[hd] + probs[128] + red[34] floats, then 128 8-byte offsets; (hd + 162) must be even for alignment
    const int hd_pad = hd + (hd & 1);
    const size_t smem = (size_t)(hd_pad + ATT_THREADS + 34) * sizeof(float) + ATT_THREADS * sizeof(long long);
    if (hd & 1) return RF_ERR_UNSUPPORTED;
    dim3 grid(nh, T_);
    rf_launch(attention_generic_kernel<T>, grid, dim3(ATT_THREADS), smem, st,
        reinterpret_cast<const T*>(q), q_stride, reinterpret_cast<T*>(out), out_stride,
        reinterpret_cast<const T*>(k_pages), reinterpret_cast<const T*>(v_pages), tok_seq, tok_pos, seq_slot,
        block_table, max_pages, nh, nkv, hd, scale, window);
    RF_LAUNCH_CHECK();
    return 0;
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
