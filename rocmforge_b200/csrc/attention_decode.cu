// Decode attention over the paged cache: one new token per sequence, bfloat16 cache.
//
// The context is cut into chunks of 256 keys; a CTA owns (chunk, kv head, sequence) and
// serves ALL query heads of that kv head's group from one pass over the chunk's keys and
// values (maeddesg/ROCmForge's flash_attn_decode_gqa_kernel has the same idea with 32-key
// tiles in LDS and one block per kv head, hip_kernels/attention.hip:633-798; its dispatched
// decode kernel keeps all scores of a head in LDS, :148-213).  Scores, softmax and the
// output sums are 32-bit.  Each CTA writes its chunk's (max, sum, unnormalised output) to
// scratch memory; the CTA that finishes last for a (sequence, kv head) merges the chunks in
// index order, so the result does not depend on which CTA that was.  The grid may be larger
// than the context needs (a replayed CUDA graph keeps its launch shape): CTAs beyond the
// sequence's last chunk, or wholly before its window, leave at once.
#include "common.cuh"

#define DEC_THREADS 256
#define DEC_CHUNK 256

template <int GP>
__global__ void __launch_bounds__(DEC_THREADS)
attention_decode_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, __nv_bfloat16* __restrict__ out,
                        int out_stride, const __nv_bfloat16* __restrict__ k_pages,
                        const __nv_bfloat16* __restrict__ v_pages, const int* __restrict__ tok_seq,
                        const int* __restrict__ tok_pos, const int* __restrict__ seq_slot,
                        const int* __restrict__ block_table, int max_pages, int nh, int nkv, int hd, float scale,
                        int window, int max_chunks, float* __restrict__ part_o, float* __restrict__ part_ml,
                        int* __restrict__ counters) {
    extern __shared__ float sm[];
    const int G = nh / nkv;
    float* q_s = sm;                                   // [GP][hd]
    float* p_s = q_s + GP * hd;                        // [GP][DEC_CHUNK]
    float* wred = p_s + GP * DEC_CHUNK;                // [8 warps][GP]
    float* o_red = wred + 8 * GP;                      // [n_ks][GP][hd]
    __shared__ int is_last;

    const int c = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z, tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const int pos = tok_pos[b];
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int c_lo = lo / DEC_CHUNK, c_hi = pos / DEC_CHUNK;
    if (c < c_lo || c > c_hi) return;
    const int n_act = c_hi - c_lo + 1;
    const int slot = seq_slot[tok_seq[b]];
    const int* bt = block_table + (size_t)slot * max_pages;

    const __nv_bfloat16* qrow = q + (size_t)b * q_stride + (size_t)kvh * G * hd;
    for (int i = tid; i < G * hd; i += DEC_THREADS) q_s[i] = __bfloat162float(qrow[i]) * scale;
    __syncthreads();

    // ---- scores: one key per thread, all heads of the group
    const int j = c * DEC_CHUNK + tid;
    const bool valid = j >= lo && j <= pos;
    float s[GP];
#pragma unroll
    for (int g = 0; g < GP; ++g) s[g] = 0.f;
    if (valid) {
        const int page = bt[j / RF_PAGE];
        const uint4* kr = reinterpret_cast<const uint4*>(
            k_pages + ((size_t)page * nkv + kvh) * RF_PAGE * hd + (size_t)(j % RF_PAGE) * hd);
        for (int v8 = 0; v8 < hd / 8; ++v8) {
            const uint4 raw = kr[v8];
            const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
            float kf[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __bfloat1622float2(h2[i]);
                kf[2 * i] = f.x; kf[2 * i + 1] = f.y;
            }
#pragma unroll
            for (int g = 0; g < GP; ++g) {
                if (g < G) {
                    const float4 qa = *reinterpret_cast<const float4*>(q_s + g * hd + v8 * 8);
                    const float4 qb = *reinterpret_cast<const float4*>(q_s + g * hd + v8 * 8 + 4);
                    s[g] += kf[0] * qa.x + kf[1] * qa.y + kf[2] * qa.z + kf[3] * qa.w
                          + kf[4] * qb.x + kf[5] * qb.y + kf[6] * qb.z + kf[7] * qb.w;
                }
            }
        }
    }
    // ---- chunk maximum per head
    float m[GP], l[GP];
#pragma unroll
    for (int g = 0; g < GP; ++g) {
        float v = valid ? s[g] : -INFINITY;
        v = warp_max(v);
        if (lane == 0) wred[warp * GP + g] = v;
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < GP; ++g) {
        float v = wred[g];
#pragma unroll
        for (int w = 1; w < 8; ++w) v = fmaxf(v, wred[w * GP + g]);
        m[g] = v;
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < GP; ++g) {
        const float p = valid ? expf(s[g] - m[g]) : 0.f;
        p_s[g * DEC_CHUNK + tid] = p;
        const float v = warp_sum(p);
        if (lane == 0) wred[warp * GP + g] = v;
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < GP; ++g) {
        float v = wred[g];
#pragma unroll
        for (int w = 1; w < 8; ++w) v += wred[w * GP + g];
        l[g] = v;
    }

    // ---- values: thread = (pair of dimensions, subset of keys), all heads of the group
    const int half = hd >> 1, n_ks = DEC_THREADS / half;
    const int dp = tid % half, ks = tid / half;
    float acc[GP][2];
#pragma unroll
    for (int g = 0; g < GP; ++g) acc[g][0] = acc[g][1] = 0.f;
    const int k_first = c * DEC_CHUNK;
    int k_last = pos - k_first;                         // last valid key of the chunk, chunk-relative
    if (k_last > DEC_CHUNK - 1) k_last = DEC_CHUNK - 1;
    int k_begin = lo - k_first;
    if (k_begin < 0) k_begin = 0;
    for (int kk = k_begin + ks; kk <= k_last; kk += n_ks) {
        const int jj = k_first + kk;
        const int page = bt[jj / RF_PAGE];
        const __nv_bfloat162 v2 = *reinterpret_cast<const __nv_bfloat162*>(
            v_pages + ((size_t)page * nkv + kvh) * RF_PAGE * hd + (size_t)(jj % RF_PAGE) * hd + 2 * dp);
        const float2 vf = __bfloat1622float2(v2);
#pragma unroll
        for (int g = 0; g < GP; ++g) {
            if (g < G) {
                const float p = p_s[g * DEC_CHUNK + kk];
                acc[g][0] = fmaf(p, vf.x, acc[g][0]);
                acc[g][1] = fmaf(p, vf.y, acc[g][1]);
            }
        }
    }
#pragma unroll
    for (int g = 0; g < GP; ++g) {
        if (g < G) {
            o_red[(ks * GP + g) * hd + 2 * dp] = acc[g][0];
            o_red[(ks * GP + g) * hd + 2 * dp + 1] = acc[g][1];
        }
    }
    __syncthreads();

    // ---- this chunk's result: final if it is the only chunk, else a partial in scratch memory
    for (int i = tid; i < G * hd; i += DEC_THREADS) {
        const int g = i / hd, d = i - g * hd;
        float o = 0.f;
        for (int k2 = 0; k2 < n_ks; ++k2) o += o_red[(k2 * GP + g) * hd + d];     // fixed order
        const int head = kvh * G + g;
        if (n_act == 1) {
            float lg = 0.f;                              // l[g] lives in registers indexed at compile time
#pragma unroll
            for (int gg = 0; gg < GP; ++gg) if (gg == g) lg = l[gg];
            out[(size_t)b * out_stride + (size_t)head * hd + d] = __float2bfloat16_rn(lg > 0.f ? o / lg : 0.f);
        } else {
            part_o[(((size_t)b * nh + head) * max_chunks + c) * hd + d] = o;
        }
    }
    if (n_act == 1) return;
    if (tid < G) {
        float mg = 0.f, lg = 0.f;
#pragma unroll
        for (int gg = 0; gg < GP; ++gg) if (gg == tid) { mg = m[gg]; lg = l[gg]; }
        float* ml = part_ml + (((size_t)b * nh + kvh * G + tid) * max_chunks + c) * 2;
        ml[0] = mg; ml[1] = lg;
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
    for (int i = tid; i < G * hd; i += DEC_THREADS) {
        const int g = i / hd, d = i - g * hd;
        const int head = kvh * G + g;
        const size_t base = ((size_t)b * nh + head) * max_chunks;
        float M = -INFINITY;
        for (int cc = c_lo; cc <= c_hi; ++cc) M = fmaxf(M, __ldcg(part_ml + (base + cc) * 2));
        float L = 0.f, O = 0.f;
        for (int cc = c_lo; cc <= c_hi; ++cc) {          // chunks in index order
            const float w = expf(__ldcg(part_ml + (base + cc) * 2) - M);
            L += w * __ldcg(part_ml + (base + cc) * 2 + 1);
            O += w * __ldcg(part_o + (base + cc) * hd + d);
        }
        out[(size_t)b * out_stride + (size_t)head * hd + d] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
    }
    if (tid == 0) counters[b * nkv + kvh] = 0;          // ready for the next launch
}

static size_t smem_bytes(int gp, int hd) {
    const int n_ks = DEC_THREADS / (hd / 2);
    return (size_t)(gp * hd + gp * DEC_CHUNK + 8 * gp + n_ks * gp * hd) * sizeof(float);
}

template <int GP>
static int launch(const void* q, int q_stride, void* out, int out_stride, const void* k_pages, const void* v_pages,
                  const int* tok_seq, const int* tok_pos, const int* seq_slot, const int* block_table,
                  int max_pages, int nh, int nkv, int hd, float scale, int window, int B, int max_chunks,
                  float* part_o, float* part_ml, int* counters, cudaStream_t st) {
    const size_t smem = smem_bytes(GP, hd);
    if (smem > 200 * 1024) return RF_ERR_UNSUPPORTED;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<GP>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    dim3 grid(max_chunks, nkv, B);
    attention_decode_kernel<GP><<<grid, DEC_THREADS, smem, st>>>(
        reinterpret_cast<const __nv_bfloat16*>(q), q_stride, reinterpret_cast<__nv_bfloat16*>(out), out_stride,
        reinterpret_cast<const __nv_bfloat16*>(k_pages), reinterpret_cast<const __nv_bfloat16*>(v_pages), tok_seq,
        tok_pos, seq_slot, block_table, max_pages, nh, nkv, hd, scale, window, max_chunks, part_o, part_ml, counters);
    RF_LAUNCH_CHECK();
    return 0;
}

extern "C" {

// head sizes this kernel takes: hd/2 must divide the 256 threads, rows must allow 16-byte loads
int rf_attention_decode_supported(int nh, int nkv, int hd) {
    if (nkv <= 0 || nh % nkv || nh / nkv > 16) return 0;
    return hd == 16 || hd == 32 || hd == 64 || hd == 128 || hd == 256;
}

// Scratch sizes in elements for B sequences: part_o, part_ml (floats), counters (ints, zero before the first launch).
void rf_attention_decode_scratch(int B, int nh, int nkv, int hd, int max_chunks, long long* n_part_o,
                                 long long* n_part_ml, long long* n_counters) {
    *n_part_o = (long long)B * nh * max_chunks * hd;
    *n_part_ml = (long long)B * nh * max_chunks * 2;
    *n_counters = (long long)B * nkv;
}

int rf_attention_decode(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                        const void* v_pages, const int* tok_seq, const int* tok_pos, const int* seq_slot,
                        const int* block_table, int max_pages, int nh, int nkv, int hd, float scale, int window,
                        int B, int max_chunks, float* part_o, float* part_ml, int* counters, cudaStream_t st) {
    if (B <= 0) return 0;
    if (!rf_attention_decode_supported(nh, nkv, hd) || max_chunks <= 0 || B > 65535) return RF_ERR_UNSUPPORTED;
    const int G = nh / nkv;
#define GO(GP) return launch<GP>(q, q_stride, out, out_stride, k_pages, v_pages, tok_seq, tok_pos, seq_slot, \
                                 block_table, max_pages, nh, nkv, hd, scale, window, B, max_chunks, part_o, part_ml, \
                                 counters, st)
    if (G <= 1) GO(1);
    if (G <= 2) GO(2);
    if (G <= 4) GO(4);
    if (G <= 8) GO(8);
    GO(16);
#undef GO
}

}
