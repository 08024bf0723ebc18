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
// The largest logit of a row; among equal logits the largest index; NaN never wins (a row of NaNs yields 0).
// A row is scanned by a thread-block cluster of 1 to 16 CTAs, each on its slice of the vocabulary with 16-byte
// loads where the row allows them: a decode step has a handful of rows of 150,000 logits, and one CTA per row
// (64 rows: 65 us of a step) leaves most of the GPU idle.  Every CTA hands its winner to the cluster's first CTA
// through distributed shared memory; that one merges them in rank order.
__device__ __forceinline__ void argmax_take(float& best, int& bi, float v, int i) {
    if (i >= 0 && (bi < 0 || v > best || (v == best && i > bi))) { best = v; bi = i; }
}

__global__ void __launch_bounds__(1024)
argmax_kernel(const float* __restrict__ logits, int V, long long row_stride, int* __restrict__ out, int slices) {
    pdl_trigger();
    __shared__ float sval[32];
    __shared__ int sidx[32];
    __shared__ float cval[16];          // the cluster's winners, filled in the first CTA only
    __shared__ int cidx[16];
    const int row = blockIdx.x / slices, rank = blockIdx.x % slices;      // cluster dimension = slices along x
    const float* x = logits + (size_t)row * row_stride;
    int per = (V + slices - 1) / slices;
    per = (per + 3) & ~3;                                                 // slices start on 16-byte borders of the row
    const int i0 = min(V, rank * per), i1 = min(V, i0 + per);
    pdl_wait();
    float best = -INFINITY;
    int bi = -1;
    if ((reinterpret_cast<uintptr_t>(x) & 15) == 0) {
        const int n4 = (i1 - i0) >> 2;
        const float4* x4 = reinterpret_cast<const float4*>(x + i0);
        for (int j = threadIdx.x; j < n4; j += blockDim.x) {
            const float4 v = x4[j];
            const int i = i0 + 4 * j;
            // a NaN fails every comparison: it is taken only as a thread's first candidate, and loses to any number later
            if (v.x == v.x) argmax_take(best, bi, v.x, i);
            if (v.y == v.y) argmax_take(best, bi, v.y, i + 1);
            if (v.z == v.z) argmax_take(best, bi, v.z, i + 2);
            if (v.w == v.w) argmax_take(best, bi, v.w, i + 3);
        }
        for (int i = i0 + 4 * n4 + threadIdx.x; i < i1; i += blockDim.x)
            if (x[i] == x[i]) argmax_take(best, bi, x[i], i);
    } else {
        for (int i = i0 + threadIdx.x; i < i1; i += blockDim.x)
            if (x[i] == x[i]) argmax_take(best, bi, x[i], i);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        argmax_take(best, bi, ov, oi);
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
            argmax_take(best, bi, ov, oi);
        }
        if (lane == 0) {
            if (slices == 1) {
                out[row] = bi < 0 ? 0 : bi;
            } else {                                 // into the first CTA's shared memory
                uint32_t va, ia;
                asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(va) : "r"((uint32_t)__cvta_generic_to_shared(&cval[rank])));
                asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(ia) : "r"((uint32_t)__cvta_generic_to_shared(&cidx[rank])));
                asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(va), "f"(best) : "memory");
                asm volatile("st.shared::cluster.s32 [%0], %1;" ::"r"(ia), "r"(bi) : "memory");
            }
        }
    }
    if (slices > 1) {
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        if (rank == 0 && threadIdx.x == 0) {
            best = cval[0]; bi = cidx[0];
            for (int r = 1; r < slices; ++r) argmax_take(best, bi, cval[r], cidx[r]);
            out[row] = bi < 0 ? 0 : bi;
        }
    }
}

extern "C" int rf_argmax(const float* logits, int rows, int V, long long row_stride, int* out, cudaStream_t st) {
    if (rows <= 0) return 0;
    if (V <= 0) return RF_ERR_BAD_ARG;
    // as many CTAs per row as fill the GPU about twice over, each with at least 4,096 logits
    int slices = 16;
    while (slices > 1 && ((long long)rows * slices > 320 || V / slices < 4096)) slices >>= 1;
    if (row_stride % 4) slices = 1;                  // rows that do not start on 16-byte borders: one CTA, scalar loads
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(argmax_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(rows * slices);
    cfg.blockDim = dim3(1024);
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = slices; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_rf_pdl ? 2 : 1;
    cudaError_t err = cudaLaunchKernelEx(&cfg, argmax_kernel, logits, V, row_stride, out, slices);
    if (err != cudaSuccess) return (int)err;
    RF_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- temperature / top-k / top-p
// Order of the vocabulary: descending logit, ascending index among equal logits.  A logit's
// position in that order is found through the order-preserving 32-bit key of its bits, eight
// bits at a time (four passes over the row per search), with probability mass counted in
// 2^-40 fixed point so that the sums are exact integers and do not depend on thread timing.
//
// A row is worked on by a thread-block cluster of 16, 8, 4, 2 or 1 CTAs (the more, the fewer rows), each on its slice of the
// vocabulary (a step samples a handful of rows while 148 SMs are idle; one CTA per row spent 3.7 ms on 152,064 logits).
// Every pass ends in a collective: each CTA leaves its histogram (or partial sum, or count) in its own
// shared memory, one cluster barrier, then EVERY CTA reads all contributions through distributed
// shared memory, adds them in rank order and takes the same decision; the buffers alternate, so a CTA may
// start its next pass while a peer still reads the last one.  Inside a CTA the lanes of a warp that hit the
// same histogram bin are found with match.any and added as one atomic (logits share their upper key bits:
// without this nearly all atomics of the first passes hit one address).
#define SMP_THREADS 1024

__device__ __forceinline__ unsigned key_of(float x) {
    const unsigned b = __float_as_uint(x);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

struct SampleShared {
    unsigned long long mass[2][256];    // this CTA's histograms, two buffers
    unsigned cnt[2][256];
    unsigned long long all_mass[256];   // the cluster's, summed by this CTA
    unsigned all_cnt[256];
    unsigned long long grp_mass[32];    // ... in groups of eight bins
    unsigned grp_cnt[32];
    double part64[2];                   // this CTA's partial sum
    float part32[2];                    // ... maximum
    unsigned count[2];                  // ... number of matches
    int found[2];                       // an index that its owner pushes to every CTA
    float red[34];
    double red64[34];
    unsigned scan[33];
    unsigned prefix, mask;              // the descent's state: the same in every CTA
    unsigned long long acc, mass_eq;
    unsigned n_eq;
    int index;
};

__device__ __forceinline__ unsigned smp_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ unsigned smp_nranks() {
    unsigned n;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(n));
    return n;
}
__device__ __forceinline__ void smp_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t smp_remote(const void* local, unsigned rank) {
    uint32_t a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
    return a;
}
__device__ __forceinline__ unsigned smp_ld_u32(const void* local, unsigned rank) {
    unsigned v;
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(smp_remote(local, rank)) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long smp_ld_u64(const void* local, unsigned rank) {
    unsigned long long v;
    asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(v) : "r"(smp_remote(local, rank)) : "memory");
    return v;
}

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

// ---- collectives of the cluster; `e` counts them and picks the buffer
__device__ float cluster_max(float v, SampleShared& s, int& e) {
    const int b = e++ & 1;
    v = block_max(v, s.red);
    if (threadIdx.x == 0) s.part32[b] = v;
    smp_cluster_sync();
    if (threadIdx.x == 0) {
        float m = -INFINITY;
        for (unsigned r = 0; r < smp_nranks(); ++r) m = fmaxf(m, __uint_as_float(smp_ld_u32(&s.part32[b], r)));
        s.red[33] = m;
    }
    __syncthreads();
    return s.red[33];
}
__device__ double cluster_sum_f64(double v, SampleShared& s, int& e) {
    const int b = e++ & 1;
    v = block_sum_f64(v, s.red64);
    if (threadIdx.x == 0) s.part64[b] = v;
    smp_cluster_sync();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (unsigned r = 0; r < smp_nranks(); ++r) t += __longlong_as_double((long long)smp_ld_u64(&s.part64[b], r));   // rank order
        s.red64[33] = t;
    }
    __syncthreads();
    return s.red64[33];
}
// the CTAs' histograms of buffer b (complete in each CTA) -> all_cnt / all_mass in every CTA
__device__ void cluster_histogram(SampleShared& s, int b, bool with_mass) {
    __syncthreads();
    smp_cluster_sync();
    if (threadIdx.x < 256) {
        unsigned c = 0;
        unsigned long long m = 0;
        for (unsigned r = 0; r < smp_nranks(); ++r) {
            c += smp_ld_u32(&s.cnt[b][threadIdx.x], r);
            if (with_mass) m += smp_ld_u64(&s.mass[b][threadIdx.x], r);
        }
        s.all_cnt[threadIdx.x] = c;
        s.all_mass[threadIdx.x] = m;
        // sums of groups of eight bins, so that the one thread that walks the histogram takes 32 + 8 steps, not 256
        unsigned gc = c;
        unsigned long long gm = m;
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) {
            gc += __shfl_xor_sync(0xffffffffu, gc, o);
            gm += __shfl_xor_sync(0xffffffffu, gm, o);
        }
        if ((threadIdx.x & 7) == 0) { s.grp_cnt[threadIdx.x >> 3] = gc; s.grp_mass[threadIdx.x >> 3] = gm; }
    }
    __syncthreads();
}
// one element into buffer b's histogram: the lanes of a warp with the same bin add as one
__device__ __forceinline__ void histogram_add(SampleShared& s, int b, bool valid, int bin, unsigned long long w, bool with_mass) {
    const unsigned act = __ballot_sync(0xffffffffu, valid);
    if (!valid) return;
    const unsigned peers = __match_any_sync(act, bin);
    // a weight is below 2^40 (+ rounding): halves of 20 and 21 bits, 32 of which add up inside 32 bits
    const unsigned lo = __reduce_add_sync(peers, (unsigned)(w & 0xfffffu));
    const unsigned hi = __reduce_add_sync(peers, (unsigned)(w >> 20));
    if ((threadIdx.x & 31) == __ffs(peers) - 1) {
        atomicAdd(&s.cnt[b][bin], (unsigned)__popc(peers));
        if (with_mass) atomicAdd(&s.mass[b][bin], ((unsigned long long)hi << 20) + lo);
    }
}

// n-th (1-based) smallest index i of the row with key(i) == K and i <= limit_index; every thread of every CTA returns it.
__device__ int nth_index_with_key(const float* x, int lo, int hi, unsigned K, int limit_index, unsigned n,
                                  SampleShared& s, int& e) {
    const int b = e++ & 1;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = SMP_THREADS / 32;
    // a warp owns a contiguous piece of the CTA's slice, in steps of 32 indices
    const int seg = ((hi - lo + nwarp - 1) / nwarp + 31) / 32 * 32;
    const int wlo = lo + warp * seg, whi = min(hi, wlo + seg);
    unsigned c = 0;
    for (int i = wlo + lane; i < whi; i += 32) c += (key_of(x[i]) == K && i <= limit_index);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
    __syncthreads();
    if (lane == 0) s.scan[warp] = c;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned t = 0;
        for (int w = 0; w < nwarp; ++w) { const unsigned v = s.scan[w]; s.scan[w] = t; t += v; }     // exclusive
        s.count[b] = t;
        s.found[b] = -1;
    }
    __syncthreads();
    smp_cluster_sync();
    // matches in the CTAs before this one
    unsigned before_cta = 0, mine = 0;
    const unsigned rank = smp_rank();
    for (unsigned r = 0; r < smp_nranks(); ++r) {
        const unsigned v = smp_ld_u32(&s.count[b], r);
        if (r < rank) before_cta += v;
        if (r == rank) mine = v;
    }
    if (before_cta < n && n <= before_cta + mine) {      // the n-th lies in this CTA: which warp, which index
        const unsigned before = before_cta + s.scan[warp];
        if (c > 0 && before < n && n <= before + c) {
            unsigned seen = before;
            for (int base = wlo; base < whi; base += 32) {
                const int i = base + lane;
                const bool m = i < whi && key_of(x[i]) == K && i <= limit_index;
                const unsigned bal = __ballot_sync(0xffffffffu, m);
                const unsigned k = __popc(bal);
                if (seen + k >= n) {
                    const int idx = base + __fns(bal, 0, n - seen);
                    if (lane == 0)
                        for (unsigned r = 0; r < smp_nranks(); ++r)
                            asm volatile("st.shared::cluster.s32 [%0], %1;" ::"r"(smp_remote(&s.found[b], r)), "r"(idx) : "memory");
                    break;
                }
                seen += k;
            }
        }
    }
    smp_cluster_sync();
    return s.found[b];
}

__global__ void __launch_bounds__(SMP_THREADS)
sample_kernel(const float* __restrict__ logits, int V, long long row_stride, float temperature, float top_p,
              int top_k, const unsigned long long* __restrict__ seeds, const int* __restrict__ draw_counter,
              int* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    __shared__ SampleShared s;
    const int cl = (int)smp_nranks();
    const int row = blockIdx.x / cl;
    const unsigned rank = smp_rank();
    const float* x = logits + (size_t)row * row_stride;
    const int tid = threadIdx.x;
    const float t = fmaxf(temperature, 1e-6f);
    const int slice = (V + cl - 1) / cl;
    const int lo = min(V, (int)rank * slice), hi = min(V, lo + slice);       // this CTA's indices
    int e = 0;                                                               // collectives so far

    float mx = -INFINITY;
    for (int i = lo + tid; i < hi; i += SMP_THREADS) mx = fmaxf(mx, x[i]);
    mx = cluster_max(mx, s, e);
    const float mx_t = mx / t;

    // ---- top-k: key Kk of the k-th largest logit and the largest index Ik still inside among its equals
    unsigned Kk = 0;
    int Ik = V;
    if (top_k > 0 && top_k < V) {
        if (tid == 0) { s.prefix = 0; s.mask = 0; s.acc = (unsigned long long)top_k; }
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass, b = e++ & 1;
            if (tid < 256) s.cnt[b][tid] = 0;
            __syncthreads();
            const unsigned prefix = s.prefix, mask = s.mask;
            for (int i0 = lo; i0 < hi; i0 += SMP_THREADS) {
                const int i = i0 + tid;
                const unsigned k = i < hi ? key_of(x[i]) : 0u;
                histogram_add(s, b, i < hi && (k & mask) == prefix, (k >> shift) & 255, 0, false);
            }
            cluster_histogram(s, b, false);
            if (tid == 0) {
                unsigned long long remaining = s.acc;
                int chosen = 0;
                for (int g = 31; g >= 0; --g) {                  // bins from 255 down, a group of eight at a time
                    if (s.grp_cnt[g] < remaining) { remaining -= s.grp_cnt[g]; continue; }
                    for (int bin = g * 8 + 7; bin >= g * 8; --bin) {
                        if (s.all_cnt[bin] >= remaining) { chosen = bin; break; }
                        remaining -= s.all_cnt[bin];
                    }
                    break;
                }
                s.acc = remaining;
                s.n_eq = s.all_cnt[chosen];
                s.prefix = prefix | ((unsigned)chosen << shift);
                s.mask = mask | (0xffu << shift);
            }
            __syncthreads();
        }
        Kk = s.prefix;
        const unsigned need = (unsigned)s.acc, n_eq = s.n_eq;
        __syncthreads();
        if (need < n_eq) Ik = nth_index_with_key(x, lo, hi, Kk, V, need, s, e);
    }
#define IN_SET(k, i) ((k) > Kk || ((k) == Kk && (i) <= Ik))

    // ---- softmax denominator over the set
    double part = 0.0;
    for (int i = lo + tid; i < hi; i += SMP_THREADS) {
        const unsigned k = key_of(x[i]);
        if (IN_SET(k, i)) part += (double)expf(x[i] / t - mx_t);
    }
    const double total = cluster_sum_f64(part, s, e);
    const double to_fixed = 1099511627776.0 / total;                         // probabilities in units of 2^-40
#define WEIGHT(i) ((unsigned long long)((double)expf(x[i] / t - mx_t) * to_fixed))

    // descent: the key at which the running mass (descending order) reaches `target`
    unsigned long long target, C = 0;
    unsigned Kp = Kk;
    int Ip = Ik;
    for (int phase = 0; phase < 2; ++phase) {
        if (phase == 0) {
            if (top_p >= 1.f) {                      // the nucleus is the whole set: C = its mass
                const int b = e++ & 1;
                unsigned long long m = 0;
                for (int i = lo + tid; i < hi; i += SMP_THREADS) {
                    const unsigned k = key_of(x[i]);
                    if (IN_SET(k, i)) m += WEIGHT(i);
                }
                if (tid == 0) s.mass[b][0] = 0;
                __syncthreads();
                atomicAdd(&s.mass[b][0], m);
                __syncthreads();
                smp_cluster_sync();
                if (tid == 0) {
                    unsigned long long c = 0;
                    for (unsigned r = 0; r < smp_nranks(); ++r) c += smp_ld_u64(&s.mass[b][0], r);
                    s.acc = c;
                }
                __syncthreads();
                C = s.acc;
                __syncthreads();
                continue;
            }
            target = (unsigned long long)((double)top_p * 1099511627776.0);
        } else {
            unsigned long long seed = seeds[row];
            if (draw_counter) seed += (unsigned long long)(*draw_counter);
            const unsigned long long v = seed * 6364136223846793005ULL + 1442695040888963407ULL;
            const float u = (float)(v >> 11) / 9007199254740992.0f;
            target = (unsigned long long)((double)u * (double)C);
            if (target > C) target = C;
        }
        if (tid == 0) { s.prefix = 0; s.mask = 0; s.acc = 0; }
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass, b = e++ & 1;
            if (tid < 256) { s.cnt[b][tid] = 0; s.mass[b][tid] = 0; }
            __syncthreads();
            const unsigned prefix = s.prefix, mask = s.mask;
            for (int i0 = lo; i0 < hi; i0 += SMP_THREADS) {
                const int i = i0 + tid;
                const unsigned k = i < hi ? key_of(x[i]) : 0u;
                const bool valid = i < hi && (k & mask) == prefix && IN_SET(k, i);
                histogram_add(s, b, valid, (k >> shift) & 255, valid ? WEIGHT(i) : 0ull, true);
            }
            cluster_histogram(s, b, true);
            if (tid == 0) {
                unsigned long long acc = s.acc;
                int chosen = -1, last = -1;
                for (int g = 31; g >= 0 && chosen < 0; --g) {    // bins from 255 down, a group of eight at a time
                    if (s.grp_cnt[g] == 0) continue;
                    if (acc + s.grp_mass[g] < target) {          // the whole group lies before the target
                        acc += s.grp_mass[g];
                        for (int bin = g * 8; bin < g * 8 + 8; ++bin)
                            if (s.all_cnt[bin]) { last = bin; break; }       // its lowest bin in use
                        continue;
                    }
                    for (int bin = g * 8 + 7; bin >= g * 8; --bin) {
                        if (s.all_cnt[bin] == 0) continue;
                        last = bin;
                        if (acc + s.all_mass[bin] >= target) { chosen = bin; break; }
                        acc += s.all_mass[bin];
                    }
                }
                if (chosen < 0) { chosen = last < 0 ? 0 : last; acc -= (last < 0 ? 0 : s.all_mass[chosen]); }
                s.acc = acc;
                s.n_eq = s.all_cnt[chosen];
                s.mass_eq = s.all_mass[chosen];
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
            Ip = (n < n_eq) ? nth_index_with_key(x, lo, hi, K, (K == Kk) ? Ik : V, (unsigned)n, s, e) : ((K == Kk) ? Ik : V);
            // the nucleus narrows the set for the draw
            Kk = Kp;
            Ik = Ip;
        } else {
            const int idx = nth_index_with_key(x, lo, hi, K, (K == Kk) ? Ik : V, (unsigned)n, s, e);
            if (tid == 0 && rank == 0) out[row] = idx < 0 ? 0 : idx;
        }
    }
    smp_cluster_sync();                              // no CTA leaves while a peer may still read its shared memory
#undef IN_SET
#undef WEIGHT
}

extern "C" int rf_sample(const float* logits, int rows, int V, long long row_stride, float temperature,
                         float top_p, int top_k, const unsigned long long* seeds, const int* draw_counter,
                         int* out, cudaStream_t st) {
    if (rows <= 0) return 0;
    if (V <= 0 || !seeds) return RF_ERR_BAD_ARG;
    // CTAs per row: as many as keep the whole batch resident at once (two CTAs of 1,024 threads fit an SM)
    // 16 is beyond the portable cluster size and pays for a few rows only (8 rows of 152,064 logits: 0.29 ms
    // in clusters of 16, 0.19 ms in clusters of 8; one row 0.14 against 0.19 ms)
    int cl = rows <= 4 ? 16 : 8;
    while (cl > 1 && (long long)rows * cl > 160) cl >>= 1;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(rows * cl);
    cfg.blockDim = dim3(SMP_THREADS);
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cl; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_rf_pdl ? 2 : 1;
    cudaError_t err = cudaLaunchKernelEx(&cfg, sample_kernel, logits, V, row_stride, temperature, top_p, top_k, seeds,
                                         draw_counter, out);
    if (err != cudaSuccess) return (int)err;
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

// tokens[i] = ids[row_map[i]]: the tokens of a step that is launched before the host has seen the ids the step
// before it sampled (the batch may have shrunk in between: row_map names each sequence's row in that step).
__global__ void gather_tokens_kernel(int* tokens, const int* ids, const int* row_map, int B) {
    pdl_trigger();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < B) tokens[i] = ids[row_map[i]];
}

extern "C" int rf_gather_tokens(int* tokens, const int* ids, const int* row_map, int B, cudaStream_t st) {
    if (B <= 0) return 0;
    rf_launch(gather_tokens_kernel, dim3((B + 127) / 128), dim3(128), 0, st, tokens, ids, row_map, B);
    RF_LAUNCH_CHECK();
    return 0;
}

extern "C" int rf_advance_decode(int* tokens, int* tok_pos, int* seq_start, const int* sampled, int B,
                                 cudaStream_t st) {
    if (B <= 0) return 0;
    rf_launch(advance_decode_kernel, dim3((B + 127) / 128), dim3(128), 0, st, tokens, tok_pos, seq_start, sampled, B);
    RF_LAUNCH_CHECK();
    return 0;
}
