// Picking the next token on the device: argmax, and temperature / top-k / top-p
// sampling with one seeded draw per row.
//
// Rules follow maeddesg/ROCmForge: of equal maxima the highest index wins
// (hip_kernels/elementwise.hip:154-155, src/cpu/ops.rs:2244-2250); temperature is
// clamped to >= 1e-6 and divides the logits before the softmax, top-k keeps the k
// largest, the nucleus is the shortest prefix of the descending order whose
// probabilities reach top_p, and the token is the first whose running sum reaches
// u * (nucleus sum), u being one LCG step of the seed (src/cpu/sampler.rs:22-185).
// The reference sorts on the host; here the prefix is found without sorting, by a
// radix descent over the bits of the logits (see sample_kernel).
#include "common.cuh"

// ---------------------------------------------------------------- argmax
__global__ void __launch_bounds__(1024)
argmax_kernel(const float* __restrict__ logits, int V, long long row_stride, int* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    __shared__ float sval[32];
    __shared__ int sidx[32];
    const float* x = logits + (size_t)blockIdx.x * row_stride;
    float best = -INFINITY;
    int bi = -1;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = x[i];
        if (v > best || (v == best && i > bi) || bi < 0) { best = v; bi = i; }
    }
    // NaN never wins a comparison: a row of NaNs yields its first scanned index per thread
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (oi >= 0 && (bi < 0 || ov > best || (ov == best && oi > bi))) { best = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { sval[warp] = best; sidx[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        const int nwarp = (blockDim.x + 31) >> 5;
        best = lane < nwarp ? sval[lane] : -INFINITY;
        bi = lane < nwarp ? sidx[lane] : -1;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi >= 0 && (bi < 0 || ov > best || (ov == best && oi > bi))) { best = ov; bi = oi; }
        }
        if (lane == 0) out[blockIdx.x] = bi < 0 ? 0 : bi;
    }
}

extern "C" int rf_argmax(const float* logits, int rows, int V, long long row_stride, int* out, cudaStream_t st) {
    if (rows <= 0) return 0;
    if (V <= 0) return RF_ERR_BAD_ARG;
    rf_launch(argmax_kernel, dim3(rows), dim3(1024), 0, st, logits, V, row_stride, out);
    RF_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- temperature / top-k / top-p
// Order of the vocabulary: descending logit, ascending index among equal logits.  A logit's
// position in that order is found through the order-preserving 32-bit key of its bits, eight
// bits at a time (four passes over the row per search), with probability mass counted in
// 2^-40 fixed point so that the sums are exact integers and do not depend on thread timing.
#define SMP_THREADS 1024

__device__ __forceinline__ unsigned key_of(float x) {
    const unsigned b = __float_as_uint(x);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

struct SampleShared;

struct SampleShared {
    unsigned long long mass[256];
    unsigned cnt[256];
    float red[34];
    double red64[34];
    unsigned scan[33];
    // results broadcast by thread 0
    unsigned prefix, mask;
    unsigned long long acc, mass_eq;
    unsigned n_eq;
    int chosen, index;
};

// Sum of one double per thread, in a tree fixed by the block size; every thread gets it.
__device__ __forceinline__ double block_sum_f64(double v, double* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        double t = lane < nwarp ? red[lane] : 0.0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

// n-th (1-based) smallest index i with in-set key(i) == K; every thread returns it.
__device__ int nth_index_with_key(const float* x, int V, unsigned K, int limit_index, unsigned n, SampleShared& s) {
    const int chunk = (V + SMP_THREADS - 1) / SMP_THREADS;
    const int lo = threadIdx.x * chunk, hi = min(V, lo + chunk);
    unsigned c = 0;
    for (int i = lo; i < hi; ++i) c += (key_of(x[i]) == K && i <= limit_index);
    // exclusive scan of c over the block
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned inc = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned v = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += v;
    }
    __syncthreads();
    if (lane == 31) s.scan[warp] = inc;
    if (threadIdx.x == 0) s.index = -1;
    __syncthreads();
    if (warp == 0) {
        unsigned w = s.scan[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned v = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += v;
        }
        s.scan[lane] = w - s.scan[lane];           // exclusive per-warp offset
    }
    __syncthreads();
    const unsigned before = s.scan[warp] + inc - c;
    if (c > 0 && before < n && n <= before + c) {
        unsigned seen = before;
        for (int i = lo; i < hi; ++i)
            if (key_of(x[i]) == K && i <= limit_index && ++seen == n) { s.index = i; break; }
    }
    __syncthreads();
    return s.index;
}

__global__ void __launch_bounds__(SMP_THREADS)
sample_kernel(const float* __restrict__ logits, int V, long long row_stride, float temperature, float top_p,
              int top_k, const unsigned long long* __restrict__ seeds, const int* __restrict__ draw_counter,
              int* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    __shared__ SampleShared s;
    const float* x = logits + (size_t)blockIdx.x * row_stride;
    const int tid = threadIdx.x;
    const float t = fmaxf(temperature, 1e-6f);

    float mx = -INFINITY;
    for (int i = tid; i < V; i += SMP_THREADS) mx = fmaxf(mx, x[i]);
    mx = block_max(mx, s.red);
    const float mx_t = mx / t;

    // ---- top-k: key Kk of the k-th largest logit and the largest index Ik still inside among its equals
    unsigned Kk = 0;
    int Ik = V;
    if (top_k > 0 && top_k < V) {
        if (tid == 0) { s.prefix = 0; s.mask = 0; s.acc = (unsigned long long)top_k; }
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            if (tid < 256) s.cnt[tid] = 0;
            __syncthreads();
            const unsigned prefix = s.prefix, mask = s.mask;
            for (int i = tid; i < V; i += SMP_THREADS) {
                const unsigned k = key_of(x[i]);
                if ((k & mask) == prefix) atomicAdd(&s.cnt[(k >> shift) & 255], 1u);
            }
            __syncthreads();
            if (tid == 0) {
                unsigned long long remaining = s.acc;
                int chosen = 0;
                for (int b = 255; b >= 0; --b) {
                    if (s.cnt[b] >= remaining) { chosen = b; break; }
                    remaining -= s.cnt[b];
                }
                s.acc = remaining;
                s.n_eq = s.cnt[chosen];
                s.prefix = prefix | ((unsigned)chosen << shift);
                s.mask = mask | (0xffu << shift);
            }
            __syncthreads();
        }
        Kk = s.prefix;
        const unsigned need = (unsigned)s.acc, n_eq = s.n_eq;
        __syncthreads();
        if (need < n_eq) Ik = nth_index_with_key(x, V, Kk, V, need, s);
    }
#define IN_SET(k, i) ((k) > Kk || ((k) == Kk && (i) <= Ik))

    // ---- softmax denominator over the set
    double part = 0.0;
    for (int i = tid; i < V; i += SMP_THREADS) {
        const unsigned k = key_of(x[i]);
        if (IN_SET(k, i)) part += (double)expf(x[i] / t - mx_t);
    }
    const double total = block_sum_f64(part, s.red64);
#define WEIGHT(i) ((unsigned long long)((double)expf(x[i] / t - mx_t) / total * 1099511627776.0))

    // descent: the key at which the running mass (descending order) reaches `target`
    unsigned long long target, C;
    unsigned Kp = Kk;
    int Ip = Ik;
    for (int phase = 0; phase < 2; ++phase) {
        if (phase == 0) {
            if (top_p >= 1.f) {                      // the nucleus is the whole set: C = its mass
                unsigned long long m = 0;
                for (int i = tid; i < V; i += SMP_THREADS) {
                    const unsigned k = key_of(x[i]);
                    if (IN_SET(k, i)) m += WEIGHT(i);
                }
                if (tid == 0) s.acc = 0;
                __syncthreads();
                atomicAdd(&s.acc, m);
                __syncthreads();
                C = s.acc;
                __syncthreads();
                continue;
            }
            target = (unsigned long long)((double)top_p * 1099511627776.0);
        } else {
            unsigned long long seed = seeds[blockIdx.x];
            if (draw_counter) seed += (unsigned long long)(*draw_counter);
            const unsigned long long v = seed * 6364136223846793005ULL + 1442695040888963407ULL;
            const float u = (float)(v >> 11) / 9007199254740992.0f;
            target = (unsigned long long)((double)u * (double)C);
            if (target > C) target = C;
        }
        if (tid == 0) { s.prefix = 0; s.mask = 0; s.acc = 0; }
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            if (tid < 256) { s.cnt[tid] = 0; s.mass[tid] = 0; }
            __syncthreads();
            const unsigned prefix = s.prefix, mask = s.mask;
            for (int i = tid; i < V; i += SMP_THREADS) {
                const unsigned k = key_of(x[i]);
                if ((k & mask) == prefix && IN_SET(k, i)) {
                    const int b = (k >> shift) & 255;
                    atomicAdd(&s.cnt[b], 1u);
                    atomicAdd(&s.mass[b], WEIGHT(i));
                }
            }
            __syncthreads();
            if (tid == 0) {
                unsigned long long acc = s.acc;
                int chosen = -1, last = -1;
                for (int b = 255; b >= 0; --b) {
                    if (s.cnt[b] == 0) continue;
                    last = b;
                    if (acc + s.mass[b] >= target) { chosen = b; break; }
                    acc += s.mass[b];
                }
                if (chosen < 0) { chosen = last < 0 ? 0 : last; acc -= (last < 0 ? 0 : s.mass[chosen]); }
                s.acc = acc;
                s.n_eq = s.cnt[chosen];
                s.mass_eq = s.mass[chosen];
                s.prefix = prefix | ((unsigned)chosen << shift);
                s.mask = mask | (0xffu << shift);
            }
            __syncthreads();
        }
        const unsigned K = s.prefix, n_eq = s.n_eq;
        const unsigned long long acc = s.acc, w = n_eq ? s.mass_eq / n_eq : 0;
        __syncthreads();
        // how many of the equal logits at K are needed to reach the target (at least one)
        unsigned long long n = 1;
        if (w > 0 && target > acc) n = (target - acc + w - 1) / w;
        if (n < 1) n = 1;
        if (n > n_eq) n = n_eq;
        if (phase == 0) {
            C = acc + n * w;
            Kp = K;
            Ip = (n < n_eq) ? nth_index_with_key(x, V, K, (K == Kk) ? Ik : V, (unsigned)n, s) : ((K == Kk) ? Ik : V);
            // the nucleus narrows the set for the draw
            Kk = Kp;
            Ik = Ip;
        } else {
            const int idx = nth_index_with_key(x, V, K, (K == Kk) ? Ik : V, (unsigned)n, s);
            if (tid == 0) out[blockIdx.x] = idx < 0 ? 0 : idx;
        }
    }
#undef IN_SET
#undef WEIGHT
}

extern "C" int rf_sample(const float* logits, int rows, int V, long long row_stride, float temperature,
                         float top_p, int top_k, const unsigned long long* seeds, const int* draw_counter,
                         int* out, cudaStream_t st) {
    if (rows <= 0) return 0;
    if (V <= 0 || !seeds) return RF_ERR_BAD_ARG;
    rf_launch(sample_kernel, dim3(rows), dim3(SMP_THREADS), 0, st, logits, V, row_stride, temperature, top_p, top_k, seeds,
              draw_counter, out);
    RF_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- feeding a replayed decode step
// After a decode step that is replayed without host work: the sampled ids become the next
// step's tokens and every sequence moves one position on (the reference's
// increment_decode_state_kernel, hip_kernels/elementwise.hip:721-753).
__global__ void advance_decode_kernel(int* tokens, int* tok_pos, int* seq_start, const int* sampled, int B) {
    pdl_trigger();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < B) {
        tokens[i] = sampled[i];
        tok_pos[i] += 1;
        seq_start[i] += 1;
    }
}

extern "C" int rf_advance_decode(int* tokens, int* tok_pos, int* seq_start, const int* sampled, int B,
                                 cudaStream_t st) {
    if (B <= 0) return 0;
    rf_launch(advance_decode_kernel, dim3((B + 127) / 128), dim3(128), 0, st, tokens, tok_pos, seq_start, sampled, B);
    RF_LAUNCH_CHECK();
    return 0;
}
