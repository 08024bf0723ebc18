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
// A value of every CTA, fetched by the lanes of one warp at once (lane r asks CTA r: one round trip through the cluster's
// shared memory instead of one per CTA) and folded in rank order.
__device__ float cluster_max(float v, SampleShared& s, int& e) {
    const int b = e++ & 1;
    v = block_max(v, s.red);
    if (threadIdx.x == 0) s.part32[b] = v;
    smp_cluster_sync();
    if (threadIdx.x < 32) {
        const unsigned n = smp_nranks();
        float m = threadIdx.x < n ? __uint_as_float(smp_ld_u32(&s.part32[b], threadIdx.x)) : -INFINITY;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (threadIdx.x == 0) s.red[33] = m;
    }
    __syncthreads();
    return s.red[33];
}
__device__ double cluster_sum_f64(double v, SampleShared& s, int& e) {
    const int b = e++ & 1;
    v = block_sum_f64(v, s.red64);
    if (threadIdx.x == 0) s.part64[b] = v;
    smp_cluster_sync();
    if (threadIdx.x < 32) {
        const unsigned n = smp_nranks();
        const double mine = threadIdx.x < n ? __longlong_as_double((long long)smp_ld_u64(&s.part64[b], threadIdx.x)) : 0.0;
        double t = 0.0;
        for (unsigned r = 0; r < n; ++r) t += __shfl_sync(0xffffffffu, mine, r);           // rank order
        if (threadIdx.x == 0) s.red64[33] = t;
    }
    __syncthreads();
    return s.red64[33];
}
// the CTAs' histograms of buffer b (complete in each CTA) -> all_cnt / all_mass in every CTA
__device__ void cluster_histogram(SampleShared& s, int b, bool with_mass) {
    __syncthreads();
    smp_cluster_sync();
    if (threadIdx.x < 256) {
        // every CTA's value of this bin: all loads under way before the first is used
        unsigned cs[16];
        unsigned long long ms[16];
        const unsigned n = smp_nranks();
#pragma unroll
        for (unsigned r = 0; r < 16; ++r) {
            cs[r] = 0; ms[r] = 0;
            if (r < n) {
                cs[r] = smp_ld_u32(&s.cnt[b][threadIdx.x], r);
                if (with_mass) ms[r] = smp_ld_u64(&s.mass[b][threadIdx.x], r);
            }
        }
        unsigned c = 0;
        unsigned long long m = 0;
#pragma unroll
        for (unsigned r = 0; r < 16; ++r) { c += cs[r]; m += ms[r]; }
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

// The bin at which a running sum over a 256-bin histogram reaches `target`, found by one warp (every lane takes eight
// bins; a shuffle scan gives each lane the sum before its bins) instead of one thread walking the bins.  Bins are visited
// from 255 down (`desc`) or from 0 up, positions from `limit` on are left out, empty bins (count 0) are passed over.
// The sum starts at acc0; the first bin with sum + its mass >= target is chosen and `acc` is the sum before it.  If the
// sum never gets there (rounding), the last bin in use is chosen.  `mass` null: the counts are the masses.
// Called by all 32 lanes of a warp; every lane gets the result.
__device__ void warp_choose_bin(const unsigned* cnt, const unsigned long long* mass, bool desc, int limit,
                                unsigned long long acc0, unsigned long long target, int& chosen, unsigned long long& acc) {
    const int lane = threadIdx.x & 31;
    unsigned c[8];
    unsigned long long m[8], sum = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int p = lane * 8 + j, bin = desc ? 255 - p : p;
        c[j] = p < limit ? cnt[bin] : 0u;
        m[j] = c[j] ? (mass ? mass[bin] : (unsigned long long)c[j]) : 0ull;
        sum += m[j];
    }
    unsigned long long incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
    }
    unsigned long long run = acc0 + incl - sum, m_last = 0;
    int j_found = -1, j_last = -1;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        if (c[j] == 0) continue;
        j_last = j;
        m_last = m[j];
        if (j_found < 0) {
            if (run + m[j] >= target) j_found = j;
            else run += m[j];
        }
    }
    const unsigned found = __ballot_sync(0xffffffffu, j_found >= 0), used = __ballot_sync(0xffffffffu, j_last >= 0);
    int p;
    if (found) {
        const int src = __ffs(found) - 1;
        p = src * 8 + __shfl_sync(0xffffffffu, j_found, src);
        acc = __shfl_sync(0xffffffffu, run, src);
    } else if (used) {
        const int src = 31 - __clz(used);
        p = src * 8 + __shfl_sync(0xffffffffu, j_last, src);
        acc = acc0 + __shfl_sync(0xffffffffu, incl, 31) - __shfl_sync(0xffffffffu, m_last, src);
    } else {
        chosen = 0;
        acc = acc0;
        return;
    }
    chosen = desc ? 255 - p : p;
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
    {
        const unsigned got = (unsigned)lane < smp_nranks() ? smp_ld_u32(&s.count[b], lane) : 0u;      // lane r asks CTA r
        for (unsigned r = 0; r < smp_nranks(); ++r) {
            const unsigned v = __shfl_sync(0xffffffffu, got, r);
            if (r < rank) before_cta += v;
            if (r == rank) mine = v;
        }
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
            if (tid < 32) {                                      // bins from 255 down until `remaining` tokens are passed
                const unsigned long long remaining = s.acc;
                int chosen;
                unsigned long long passed;
                warp_choose_bin(s.all_cnt, nullptr, true, 256, 0, remaining, chosen, passed);
                __syncwarp();
                if (tid == 0) {
                    s.acc = remaining - passed;
                    s.n_eq = s.all_cnt[chosen];
                    s.prefix = prefix | ((unsigned)chosen << shift);
                    s.mask = mask | (0xffu << shift);
                }
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
            if (tid < 32) {                                      // bins from 255 down until the running mass reaches the target
                int chosen;
                unsigned long long acc;
                warp_choose_bin(s.all_cnt, s.all_mass, true, 256, s.acc, target, chosen, acc);
                __syncwarp();
                if (tid == 0) {
                    s.acc = acc;
                    s.n_eq = s.all_cnt[chosen];
                    s.mass_eq = s.all_mass[chosen];
                    s.prefix = prefix | ((unsigned)chosen << shift);
                    s.mask = mask | (0xffu << shift);
                }
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

// ---------------------------------------------------------------- the same sampler with the slice in shared memory
// The kernel above walks the row twelve times or more, and every visit of a logit pays for its key, a division, an
// exponential and a conversion to fixed point again (about 60 instructions; the kernel is bound by instructions, not by
// memory).  Here a CTA reads its slice ONCE into shared memory (logit and exponential, 8 bytes a token), and the two
// searches in descending order (the nucleus' edge, the draw) share one histogram over 256 LINEAR bins of
// (maximum - logit): float subtraction, multiplication by a positive factor and truncation are all monotone, so a lower
// bin never holds a smaller logit than a higher one, and logits spread far more evenly over linear bins than over the
// upper bits of their keys (which are sign and exponent: most of a row shares two or three of those).  The bin that a
// search ends in holds a few per cent of the row; its tokens are gathered into a list (offsets into the slice) and only
// they go through the four 8-bit passes over the key bits that order them exactly.  Definitions (order, fixed-point
// masses, ties by index) are those of the kernel above, so both give the same token.
#define SMP2_CAP 19200            // tokens of a CTA's slice (152,064 / 8 = 19,008): 10 bytes each in shared memory

struct Sample2Shared : SampleShared {
    unsigned long long lin_mass[256];   // the cluster's histogram over the linear bins (kept for the second search)
    unsigned lin_cnt[256];
    unsigned long long lin_grp_mass[32];
    unsigned lin_grp_cnt[32];
    unsigned list_n;                    // tokens of this CTA in the gathered bin
    int bin;                            // a search's linear bin: the same in every CTA
    unsigned long long bin_acc;         // mass of the bins before it
};

// Tokens of the slice whose linear bin is `bin` -> list (their offsets in the slice, in no particular order: what is done
// with them does not depend on it).
__device__ void gather_bin(Sample2Shared& s, const float* xs, int n_mine, float mx, float bscale, int bin, unsigned short* list) {
    if (threadIdx.x == 0) s.list_n = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31;
    for (int j0 = 0; j0 < n_mine; j0 += SMP_THREADS) {
        const int j = j0 + threadIdx.x;
        const bool member = j < n_mine && min(255, (int)((mx - xs[j]) * bscale)) == bin;
        const unsigned bal = __ballot_sync(0xffffffffu, member);
        if (bal == 0) continue;
        unsigned base = 0;
        if (lane == 0) base = atomicAdd(&s.list_n, (unsigned)__popc(bal));
        base = __shfl_sync(0xffffffffu, base, 0);
        if (member) list[base + __popc(bal & ((1u << lane) - 1u))] = (unsigned short)j;
    }
    __syncthreads();
}

__global__ void __launch_bounds__(SMP_THREADS)
sample_cached_kernel(const float* __restrict__ logits, int V, long long row_stride, float temperature, float top_p,
                     int top_k, const unsigned long long* __restrict__ seeds, const int* __restrict__ draw_counter,
                     int* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) uint8_t smp_dyn[];
    __shared__ Sample2Shared s;
    float* xs = reinterpret_cast<float*>(smp_dyn);                       // the slice's logits
    float* ps = xs + SMP2_CAP;                                           // ... exponentials (0 outside the top-k set)
    unsigned short* list = reinterpret_cast<unsigned short*>(ps + SMP2_CAP);
    const int cl = (int)smp_nranks();
    const int row = blockIdx.x / cl;
    const unsigned rank = smp_rank();
    const float* x = logits + (size_t)row * row_stride;
    const int tid = threadIdx.x;
    const float t = fmaxf(temperature, 1e-6f);
    const int slice = (V + cl - 1) / cl;
    const int lo = min(V, (int)rank * slice), hi = min(V, lo + slice);       // this CTA's indices
    const int n_mine = hi - lo;
    const float* xv = xs - lo;                                               // xv[i] = logit of index i, lo <= i < hi
    int e = 0;                                                               // collectives so far

    float mx = -INFINITY, mn = INFINITY;
    for (int i = lo + tid; i < hi; i += SMP_THREADS) {
        const float v = x[i];
        xs[i - lo] = v;
        mx = fmaxf(mx, v);
        if (v > -INFINITY) mn = fminf(mn, v);         // masked-out tokens (-inf) go to the last bin whatever the span
    }
    mx = cluster_max(mx, s, e);
    mn = -cluster_max(-mn, s, e);
    const float mx_t = mx / t;
    // linear bins over [maximum - range, maximum]; what lies below (weights under e^-24 of the largest) shares the last
    // bin.  A row without a finite span (all equal, or not finite) goes into bin 0 as a whole: the key passes order it.
    const bool spans = mx > mn && mx - mn < INFINITY;
    const float bscale = spans ? 256.f / fminf(mx - mn, 24.f * t) : 0.f;
#define LBIN(v) min(255, (int)((mx - (v)) * bscale))

    // ---- top-k: key Kk of the k-th largest logit and the largest index Ik still inside among its equals
    unsigned Kk = 0;
    int Ik = V;
    int listed = -1;                                 // the linear bin whose tokens `list` holds
    if (top_k > 0 && top_k < V) {
        // the linear bin that holds the k-th largest logit (counts only), then its tokens through the key passes
        {
            const int b = e++ & 1;
            if (tid < 256) s.cnt[b][tid] = 0;
            __syncthreads();
            for (int j = tid; j < n_mine; j += SMP_THREADS) atomicAdd(&s.cnt[b][LBIN(xs[j])], 1u);
            cluster_histogram(s, b, false);
            if (tid < 32) {
                int chosen;
                unsigned long long passed;
                warp_choose_bin(s.all_cnt, nullptr, false, 256, 0, (unsigned long long)top_k, chosen, passed);
                __syncwarp();
                if (tid == 0) { s.bin = chosen; s.bin_acc = passed; }
            }
            __syncthreads();
        }
        const int kbin = s.bin;
        const unsigned long long kbefore = s.bin_acc;
        __syncthreads();
        gather_bin(s, xs, n_mine, mx, bscale, kbin, list);
        listed = kbin;
        const int n_klist = (int)s.list_n;
        if (tid == 0) { s.prefix = 0; s.mask = 0; s.acc = (unsigned long long)top_k - kbefore; }
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass, b = e++ & 1;
            if (tid < 256) s.cnt[b][tid] = 0;
            __syncthreads();
            const unsigned prefix = s.prefix, mask = s.mask;
            for (int q0 = 0; q0 < n_klist; q0 += SMP_THREADS) {
                const int q = q0 + tid;
                const unsigned k = key_of(xs[q < n_klist ? (int)list[q] : 0]);
                histogram_add(s, b, q < n_klist && (k & mask) == prefix, (k >> shift) & 255, 0, false);
            }
            cluster_histogram(s, b, false);
            if (tid < 32) {                                      // bins from 255 down until `remaining` tokens are passed
                const unsigned long long remaining = s.acc;
                int chosen;
                unsigned long long passed;
                warp_choose_bin(s.all_cnt, nullptr, true, 256, 0, remaining, chosen, passed);
                __syncwarp();
                if (tid == 0) {
                    s.acc = remaining - passed;
                    s.n_eq = s.all_cnt[chosen];
                    s.prefix = prefix | ((unsigned)chosen << shift);
                    s.mask = mask | (0xffu << shift);
                }
            }
            __syncthreads();
        }
        Kk = s.prefix;
        const unsigned need = (unsigned)s.acc, n_eq = s.n_eq;
        __syncthreads();
        if (need < n_eq) Ik = nth_index_with_key(xv, lo, hi, Kk, V, need, s, e);
    }
#define IN_SET(k, i) ((k) > Kk || ((k) == Kk && (i) <= Ik))

    // ---- exponentials, once, and the softmax denominator over the set
    double part = 0.0;
    for (int j = tid; j < n_mine; j += SMP_THREADS) {
        const float v = xs[j];
        const unsigned k = key_of(v);
        const float p = IN_SET(k, lo + j) ? expf(v / t - mx_t) : 0.f;
        ps[j] = p;
        part += (double)p;
    }
    const double total = cluster_sum_f64(part, s, e);
    const double to_fixed = 1099511627776.0 / total;                         // probabilities in units of 2^-40
#define WEIGHT(j) ((unsigned long long)((double)ps[j] * to_fixed))

    // ---- the histogram over the linear bins: counts and masses of the set.  Neighbouring tokens fall into different
    // bins here, so every token adds on its own (finding the lanes of equal bin first, as the key passes do, took 88 us
    // of this kernel's 137 when every lane had a bin of its own): one 64-bit add, the count in the upper 16 bits
    // (a slice has fewer than 65,536 tokens and its mass is below 2^41).
    {
        const int b = e++ & 1;
        unsigned long long* packed = s.mass[b];
        if (tid < 256) packed[tid] = 0;
        __syncthreads();
        for (int j = tid; j < n_mine; j += SMP_THREADS) {
            const float v = xs[j];
            const unsigned k = key_of(v);
            if (IN_SET(k, lo + j)) atomicAdd(&packed[LBIN(v)], (1ull << 48) | WEIGHT(j));
        }
        __syncthreads();
        if (tid < 256) {
            const unsigned long long pk = packed[tid];
            s.cnt[b][tid] = (unsigned)(pk >> 48);
            s.mass[b][tid] = pk & ((1ull << 48) - 1);
        }
        cluster_histogram(s, b, true);
        if (tid < 256) { s.lin_cnt[tid] = s.all_cnt[tid]; s.lin_mass[tid] = s.all_mass[tid]; }
        if (tid < 32) { s.lin_grp_cnt[tid] = s.grp_cnt[tid]; s.lin_grp_mass[tid] = s.grp_mass[tid]; }
        __syncthreads();
    }

    unsigned long long target, C = 0;
    unsigned Kp = Kk;
    int Ip = Ik;
    int edge_bin = 256;                              // the nucleus' last linear bin (256: no nucleus, every bin is inside)
    unsigned long long edge_before = 0;              // mass of the bins before it
    for (int phase = 0; phase < 2; ++phase) {
        if (phase == 0) {
            if (top_p >= 1.f) {                      // the nucleus is the whole set: C = its mass
                if (tid == 0) {
                    unsigned long long c = 0;
                    for (int g = 0; g < 32; ++g) c += s.lin_grp_mass[g];
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
        // ---- the linear bin in which the running mass (from the largest logits down) reaches the target
        if (tid < 32) {
            int chosen;
            unsigned long long acc;
            if (phase == 1 && edge_bin < 256 && target > edge_before) {      // inside the nucleus' last bin
                chosen = edge_bin;
                acc = edge_before;
            } else {                                 // the bins before the nucleus' last one are wholly inside
                const int limit = (phase == 1 && edge_bin < 256) ? edge_bin : 256;
                warp_choose_bin(s.lin_cnt, s.lin_mass, false, limit, 0, target, chosen, acc);
            }
            __syncwarp();
            if (tid == 0) { s.bin = chosen; s.bin_acc = acc; }
        }
        __syncthreads();
        const int bin = s.bin;
        const unsigned long long bin_acc = s.bin_acc;
        __syncthreads();
        if (listed != bin) { gather_bin(s, xs, n_mine, mx, bscale, bin, list); listed = bin; }
        const int n_list = (int)s.list_n;
        // ---- inside the bin: the key at which the running mass reaches the target, eight key bits at a time
        if (tid == 0) { s.prefix = 0; s.mask = 0; s.acc = bin_acc; }
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass, b = e++ & 1;
            if (tid < 256) { s.cnt[b][tid] = 0; s.mass[b][tid] = 0; }
            __syncthreads();
            const unsigned prefix = s.prefix, mask = s.mask;
            for (int q0 = 0; q0 < n_list; q0 += SMP_THREADS) {
                const int q = q0 + tid;
                const int j = q < n_list ? (int)list[q] : 0;
                const unsigned k = key_of(xs[j]);
                const bool valid = q < n_list && (k & mask) == prefix && IN_SET(k, lo + j);
                histogram_add(s, b, valid, (k >> shift) & 255, valid ? WEIGHT(j) : 0ull, true);
            }
            cluster_histogram(s, b, true);
            if (tid < 32) {                                      // bins from 255 down until the running mass reaches the target
                int chosen;
                unsigned long long acc;
                warp_choose_bin(s.all_cnt, s.all_mass, true, 256, s.acc, target, chosen, acc);
                __syncwarp();
                if (tid == 0) {
                    s.acc = acc;
                    s.n_eq = s.all_cnt[chosen];
                    s.mass_eq = s.all_mass[chosen];
                    s.prefix = prefix | ((unsigned)chosen << shift);
                    s.mask = mask | (0xffu << shift);
                }
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
            Ip = (n < n_eq) ? nth_index_with_key(xv, lo, hi, K, (K == Kk) ? Ik : V, (unsigned)n, s, e) : ((K == Kk) ? Ik : V);
            // the nucleus narrows the set for the draw
            Kk = Kp;
            Ik = Ip;
            edge_bin = bin;
            edge_before = bin_acc;
        } else {
            const int idx = nth_index_with_key(xv, lo, hi, K, (K == Kk) ? Ik : V, (unsigned)n, s, e);
            if (tid == 0 && rank == 0) out[row] = idx < 0 ? 0 : idx;
        }
    }
    smp_cluster_sync();                              // no CTA leaves while a peer may still read its shared memory
#undef IN_SET
#undef WEIGHT
#undef LBIN
}

static int g_sample_cached = 1;
extern "C" int rf_sample_set_cached(int on) { g_sample_cached = on ? 1 : 0; return 0; }

static int launch_sample_cached(const float* logits, int rows, int V, long long row_stride, float temperature, float top_p,
                                int top_k, const unsigned long long* seeds, const int* draw_counter, int* out, int cl,
                                cudaStream_t st) {
    const size_t smem = (size_t)SMP2_CAP * 10;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(sample_cached_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e != cudaSuccess) return (int)e;
        e = cudaFuncSetAttribute(sample_cached_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(rows * cl);
    cfg.blockDim = dim3(SMP_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cl; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_rf_pdl ? 2 : 1;
    cudaError_t err = cudaLaunchKernelEx(&cfg, sample_cached_kernel, logits, V, row_stride, temperature, top_p, top_k, seeds,
                                         draw_counter, out);
    if (err != cudaSuccess) return (int)err;
    RF_LAUNCH_CHECK();
    return 0;
}

extern "C" int rf_sample(const float* logits, int rows, int V, long long row_stride, float temperature,
                         float top_p, int top_k, const unsigned long long* seeds, const int* draw_counter,
                         int* out, cudaStream_t st) {
    if (rows <= 0) return 0;
    if (V <= 0 || !seeds) return RF_ERR_BAD_ARG;
    if (g_sample_cached) {
        // the slice in shared memory: clusters of 8 (16 for vocabularies beyond 153,600; fewer CTAs for small ones), one
        // CTA per SM; more rows than SMs / 8 run one cluster after the other
        int c2 = 1;
        while (c2 < 8 && V > c2 * 4096) c2 <<= 1;
        if ((V + c2 - 1) / c2 > SMP2_CAP) c2 = 16;
        if ((V + c2 - 1) / c2 <= SMP2_CAP)
            return launch_sample_cached(logits, rows, V, row_stride, temperature, top_p, top_k, seeds, draw_counter, out, c2, st);
    }
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
