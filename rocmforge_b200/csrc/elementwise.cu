// Embedding gather, residual-add + RMSNorm, rotary position encoding fused with the
// cache write, and SwiGLU.  Each kernel is templated on the compute dtype (float for
// the true 32-bit path, bfloat16 for serving); the residual stream is 32-bit in both.
//
// What they compute follows maeddesg/ROCmForge's hip_kernels/norm.hip:18-84 (RMSNorm),
// rope.hip:48-91 and attention.hip:1561-1621 (NeoX rotation fused with the cache
// write), elementwise.hip:72-82 (SiLU, multiply) and the embedding gathers of
// elementwise.hip:243-445; how they are launched and laid out is this library's own.
#include "common.cuh"

// Four neighbouring elements as one access.
template <typename T> struct Four;
template <> struct Four<float> {
    static __device__ __forceinline__ void load(const float* p, float* v) {
        const float4 x = *reinterpret_cast<const float4*>(p);
        v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
    }
    static __device__ __forceinline__ void store(float* p, const float* v) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <> struct Four<__nv_bfloat16> {
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) {
        const uint2 x = *reinterpret_cast<const uint2*>(p);
        v[0] = __uint_as_float(x.x << 16); v[1] = __uint_as_float(x.x & 0xffff0000u);
        v[2] = __uint_as_float(x.y << 16); v[3] = __uint_as_float(x.y & 0xffff0000u);
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* v) {
        const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
        uint2 x;
        x.x = *reinterpret_cast<const uint32_t*>(&a); x.y = *reinterpret_cast<const uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = x;
    }
};

// ---------------------------------------------------------------- embedding
// out[t, :] = table[ids[t], :] widened to 32-bit (the residual stream).
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                             float* __restrict__ out, int H, int V) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    int id = ids[t];
    id = id < 0 ? 0 : (id >= V ? V - 1 : id);   // ids are validated on the host; never read outside
    const T* row = table + (size_t)id * H;
    float* o = out + (size_t)t * H;
    // four elements per access where rows allow it: a decode step starts with this kernel, and 14 rounds of 2-byte
    // loads from a table row that lies in DRAM took 10 us
    if (H % 4 == 0 && (reinterpret_cast<uintptr_t>(table) % (4 * sizeof(T))) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
        for (int i = 4 * threadIdx.x; i < H; i += 4 * blockDim.x) {
            float v[4];
            Four<T>::load(row + i, v);
            *reinterpret_cast<float4*>(o + i) = make_float4(v[0], v[1], v[2], v[3]);
        }
        return;
    }
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = Cvt<T>::to_f32(row[i]);
}

// ---------------------------------------------------------------- add + RMSNorm
// v = h[row] + sum_s pending[s][row];  y = v * rsqrt(mean(v^2) + eps) * w.
// pending_kind: 0 none, 1 = n_pending 32-bit partial sums [S, T, H] (split-K outputs,
// added in index order), 2 = one [T, H] tensor in the compute dtype.
// rows == nullptr: one block per token, h is updated in place.
// rows != nullptr: block r reads token rows[r], writes y[r] and leaves h alone.
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const void* __restrict__ pending,
                                   int pending_kind, int n_pending, size_t pending_stride,
                                   const void* __restrict__ w, int w_is_f32, float eps,
                                   T* __restrict__ y, const int* __restrict__ rows, int H) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float row_buf[];          // H floats + 33 for the reduction
    float* red = row_buf + H;
    const int r = blockIdx.x;
    const int t = rows ? rows[r] : r;
    float* hrow = h + (size_t)t * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = hrow[i];
        if (pending_kind == 1) {
            const float* p = reinterpret_cast<const float*>(pending) + (size_t)t * H + i;
            for (int s = 0; s < n_pending; ++s) v += p[(size_t)s * pending_stride];
        } else if (pending_kind == 2) {
            v += Cvt<T>::to_f32(reinterpret_cast<const T*>(pending)[(size_t)t * H + i]);
        }
        row_buf[i] = v;
        ss += v * v;
    }
    const float total = block_sum(ss, red);
    const float inv = rsqrtf(total / (float)H + eps);
    T* yrow = y + (size_t)r * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = row_buf[i];
        if (!rows && pending_kind != 0) hrow[i] = v;
        yrow[i] = Cvt<T>::from_f32(v * inv * load_vec(w, w_is_f32, i));
    }
}

// The same for rows whose length is a multiple of 4: the row lives in registers (at most NV float4 per
// thread), every load is 16 bytes wide and independent of the others, so a short row costs a few
// memory round trips instead of a chain of them.  Sums are formed in the same order as above
// (h first, then the partial sums in index order), element by element.
//
// A row may be shared by a thread-block cluster of `cl` CTAs (few rows: a decode step's norm reads the K-split
// partial sums of the product before it, 150 KB a row at width 3,584 with ten splits, and one CTA per row leaves a
// handful of SMs pulling all of that from L2).  The CTAs' threads are numbered through (rank * blockDim + thread)
// and work exactly as the threads of one large block would; the warps' sums of squares are pushed into every
// CTA's shared memory and folded by the same tree as in block_sum, so the result is bit for bit that of one CTA.
// The pushes are st.async stores that report their bytes to the receiving CTA's mbarrier, set up before the cluster's
// one barrier at the kernel's top (which the dependency wait hides): a CTA waits for the words it expects and for
// nothing else.  With plain remote stores and a second cluster barrier (arrive.release, wait.acquire) behind them
// the exchange cost 0.9 us of a kernel that otherwise takes 1.3 (a decode step of the 7B shape at batch 8 2.59 -> 2.54
// ms, at batch 1 2.51 -> 2.45 ms).  The wait is bounded: status 7 when a peer's words never come.
__device__ __forceinline__ float cluster_block_sum(float v, float* red, uint64_t* bar, int vt, int n_warps, int cl,
                                                    int* status) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");     // every peer has started and set up its barrier
    if (lane == 0) {
        // a warp's sum goes into every CTA's array by a store that reports its bytes to that CTA's mbarrier: a CTA
        // then waits for the words it expects and for nothing else (no second cluster barrier, no release fence)
        const uint32_t mine = (uint32_t)__cvta_generic_to_shared(&red[vt >> 5]);
        const uint32_t mbar = (uint32_t)__cvta_generic_to_shared(bar);
        for (int r = 0; r < cl; ++r) {
            uint32_t remote, remote_bar;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(mine), "r"(r));
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote_bar) : "r"(mbar), "r"(r));
            asm volatile("st.async.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];"
                         ::"r"(remote), "r"(__float_as_uint(v)), "r"(remote_bar) : "memory");
        }
    }
    {
        const uint32_t mbar = (uint32_t)__cvta_generic_to_shared(bar);
        uint32_t ok = 0;
        unsigned long long t0 = 0;
        for (long long it = 0; !ok; ++it) {
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                         "selp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(mbar), "r"(0u) : "memory");
            if (ok) break;
            if ((it & 63) == 63) {
                unsigned long long now;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
                if (t0 == 0) t0 = now;
                if (now - t0 > 2000000000ull) break;     // 2 s: a peer's words never came; the row is invalid
            }
        }
        if (!ok && threadIdx.x == 0 && status) atomicExch(status, 7);
    }
    if (warp == 0) {
        float t = lane < n_warps ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

// INF: partial sums of one element group asked for at once.  A decode step's norm is a chain of L2 round trips and
// nothing else; ten or fifteen K splits read four at a time (and the rest one by one) were four to six trips, sixteen at
// a time they are one.  The wide form needs its registers: it is compiled for blocks of at most 256 threads.
template <typename T, int NV, int INF, int MAXT>
__global__ void __launch_bounds__(MAXT)
add_rmsnorm_vec_kernel(float* __restrict__ h, const void* __restrict__ pending, int pending_kind, int n_pending,
                       size_t pending_stride, const void* __restrict__ w, int w_is_f32, float eps,
                       T* __restrict__ y, const int* __restrict__ rows, int H, int cl, int* __restrict__ status) {
    pdl_trigger();
    __shared__ float red[34];
    __shared__ __align__(8) uint64_t sum_bar;
    if (cl > 1) {
        if (threadIdx.x == 0) {                          // this CTA expects a word from every warp of the row's cluster
            const uint32_t mbar = (uint32_t)__cvta_generic_to_shared(&sum_bar);
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(mbar));
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(mbar), "r"((uint32_t)(cl * blockDim.x / 32 * 4)) : "memory");
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");            // "started": peers may store here
    }
    const int r = blockIdx.x / cl;
    const int t = rows ? rows[r] : r;
    const int nvec = H >> 2;
    int rank = 0;
    if (cl > 1) asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const int vt = rank * blockDim.x + threadIdx.x, VT = cl * blockDim.x;       // this thread among the row's threads
    uint4 wraw[NV];                              // the norm's weights (four floats, or four bfloat16 in x and y):
#pragma unroll                                   // no kernel writes them, so they are fetched while the kernel
    for (int i = 0; i < NV; ++i) {               // before this one still runs
        const int c = vt + i * VT;
        wraw[i] = make_uint4(0u, 0u, 0u, 0u);
        if (c < nvec) {
            if (w_is_f32) {
                wraw[i] = reinterpret_cast<const uint4*>(w)[c];
            } else {
                const uint2 two = reinterpret_cast<const uint2*>(w)[c];
                wraw[i].x = two.x; wraw[i].y = two.y;
            }
        }
    }
    pdl_wait();
    float4* hrow = reinterpret_cast<float4*>(h + (size_t)t * H);
    float4 v[NV];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = vt + i * VT;
        if (c < nvec) {
            float4 a = hrow[c];
            if (pending_kind == 1) {
                const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(pending) + (size_t)t * H) + c;
                if constexpr (INF > 4) {
                    for (int s2 = 0; s2 < n_pending; s2 += INF) {    // INF loads in flight, added in index order
                        float4 b[INF];
#pragma unroll
                        for (int u = 0; u < INF; ++u)
                            if (s2 + u < n_pending)
                                b[u] = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + (size_t)(s2 + u) * pending_stride);
#pragma unroll
                        for (int u = 0; u < INF; ++u)
                            if (s2 + u < n_pending) { a.x += b[u].x; a.y += b[u].y; a.z += b[u].z; a.w += b[u].w; }
                    }
                } else {
                    int s2 = 0;
                    for (; s2 + 4 <= n_pending; s2 += 4) {   // four loads in flight, added in index order
                        float4 b[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u)
                            b[u] = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + (size_t)(s2 + u) * pending_stride);
#pragma unroll
                        for (int u = 0; u < 4; ++u) { a.x += b[u].x; a.y += b[u].y; a.z += b[u].z; a.w += b[u].w; }
                    }
                    for (; s2 < n_pending; ++s2) {
                        const float4 b = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + (size_t)s2 * pending_stride);
                        a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
                    }
                }
            } else if (pending_kind == 2) {
                const T* p = reinterpret_cast<const T*>(pending) + (size_t)t * H + 4 * c;
                a.x += Cvt<T>::to_f32(p[0]); a.y += Cvt<T>::to_f32(p[1]);
                a.z += Cvt<T>::to_f32(p[2]); a.w += Cvt<T>::to_f32(p[3]);
            }
            v[i] = a;
            ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
        }
    }
    const float total = cl > 1 ? cluster_block_sum(ss, red, &sum_bar, vt, VT >> 5, cl, status) : block_sum(ss, red);
    const float inv = rsqrtf(total / (float)H + eps);
    T* yrow = y + (size_t)r * H;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = vt + i * VT;
        if (c < nvec) {
            if (!rows && pending_kind != 0) hrow[c] = v[i];
            float w0, w1, w2, w3;
            if (w_is_f32) {
                w0 = __uint_as_float(wraw[i].x); w1 = __uint_as_float(wraw[i].y);
                w2 = __uint_as_float(wraw[i].z); w3 = __uint_as_float(wraw[i].w);
            } else {                             // a bfloat16 is the upper half of a float
                w0 = __uint_as_float(wraw[i].x << 16); w1 = __uint_as_float(wraw[i].x & 0xffff0000u);
                w2 = __uint_as_float(wraw[i].y << 16); w3 = __uint_as_float(wraw[i].y & 0xffff0000u);
            }
            const float o0 = v[i].x * inv * w0, o1 = v[i].y * inv * w1;
            const float o2 = v[i].z * inv * w2, o3 = v[i].w * inv * w3;
            const float ov[4] = {o0, o1, o2, o3};
            Four<T>::store(yrow + 4 * c, ov);              // one 16-byte (8-byte) store: the row is aligned for it
        }
    }
}

// The norm of many rows without a pending update (a prompt step: the products add into the stream themselves).  The
// kernel above keeps a row in registers, and 56 registers a thread leave room for four rows per SM: 56 KB in flight,
// which one L2 round trip turns into 4 TB/s over the GPU (12 us for 2,048 rows of 3,584).  Here a row is read twice,
// the second time from L1 (8 rows of 14 KB per SM fit it), so a thread needs 20-odd registers, eight CTAs share an SM
// and twice the bytes are in flight.  Same sums in the same order as above (block_sum over one float4 per step).
template <typename T>
__global__ void __launch_bounds__(256, 8)
rmsnorm_rows_kernel(const float* __restrict__ h, const void* __restrict__ w, int w_is_f32, float eps, T* __restrict__ y,
                    int H) {
    pdl_trigger();
    __shared__ float red[34];
    const int r = blockIdx.x, nvec = H >> 2;
    pdl_wait();
    const float4* hrow = reinterpret_cast<const float4*>(h + (size_t)r * H);
    float ss = 0.f;
    for (int c0 = threadIdx.x; c0 < nvec; c0 += 4 * blockDim.x) {          // four loads in flight per thread
        float4 a[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int c = c0 + i * blockDim.x;
            a[i] = c < nvec ? hrow[c] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) ss += a[i].x * a[i].x + a[i].y * a[i].y + a[i].z * a[i].z + a[i].w * a[i].w;
    }
    const float total = block_sum(ss, red);
    const float inv = rsqrtf(total / (float)H + eps);
    T* yrow = y + (size_t)r * H;
#pragma unroll 4
    for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
        const float4 a = hrow[c];
        float w0, w1, w2, w3;
        if (w_is_f32) {
            const float4 t = reinterpret_cast<const float4*>(w)[c];
            w0 = t.x; w1 = t.y; w2 = t.z; w3 = t.w;
        } else {                                 // a bfloat16 is the upper half of a float
            const uint2 two = reinterpret_cast<const uint2*>(w)[c];
            w0 = __uint_as_float(two.x << 16); w1 = __uint_as_float(two.x & 0xffff0000u);
            w2 = __uint_as_float(two.y << 16); w3 = __uint_as_float(two.y & 0xffff0000u);
        }
        const float ov[4] = {a.x * inv * w0, a.y * inv * w1, a.z * inv * w2, a.w * inv * w3};
        Four<T>::store(yrow + 4 * c, ov);
    }
}

// ---------------------------------------------------------------- rotation + cache write
// Rows of q | k | v, [T, (nh + 2*nkv) * hd], come either in the compute dtype (src, one tensor)
// or as n_partials 32-bit partial sums of a K-split product plus a bias (the sum is formed here,
// in index order).  q is rotated and written to q_out (which may be the source itself); k is
// rotated and v copied into the page of (slot, position): pages are [n_pages, nkv, RF_PAGE, hd].
// The angle is float(pos) * inv_freq[i] in 32-bit; sincosf is the accurate one.
template <typename T, bool PARTIALS>
__global__ void rope_kv_write_kernel(const void* __restrict__ src, int row_stride, int n_partials,
                                     size_t partial_stride, const void* __restrict__ bias, int bias_is_f32,
                                     T* __restrict__ q_out, int q_out_stride, int nh, int nkv, int hd,
                                     const float* __restrict__ inv_freq,
                                     const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                     const int* __restrict__ seq_slot,
                                     const int* __restrict__ block_table, int max_pages,
                                     T* __restrict__ k_pages, T* __restrict__ v_pages, int write_kv,
                                     int rot_dim, int interleaved) {
    // grid: (token, block of pairs).  Pair index space: nh + nkv rotated heads, then nkv value heads,
    // hd/2 pairs each (a value "pair" is two neighbouring elements, copied).
    // Position, slot, page, frequency, bias and the angle's sine and cosine do not depend on the kernel
    // before this one (no kernel of a step writes them): all of that is done before pdl_wait(), so that
    // after it only the loads of the product's sums and the stores remain.
    pdl_trigger();
    const int t = blockIdx.x;
    const int half = hd >> 1;
    const int idx = blockIdx.y * blockDim.x + threadIdx.x;
    const int n_pairs = (nh + 2 * nkv) * half;
    if (idx >= n_pairs) return;
    const int head = idx / half, i = idx - head * half;
    if (head >= nh && !write_kv) return;
    const int pos = tok_pos[t];
    // which two elements of the head this pair is, and whether they turn: the first rot_dim elements of a query or
    // key head are rotated, as pairs (i, i + rot_dim/2) or (2i, 2i+1); the rest, and values, pass through
    const int rh = rot_dim >> 1;
    bool rotated = head < nh + nkv;
    int e0, e1;
    if (rotated && interleaved) { e0 = 2 * i; e1 = e0 + 1; rotated = e0 < rot_dim; }
    else if (rotated && i < rh) { e0 = i; e1 = i + rh; }
    else if (rotated) { e0 = rot_dim + 2 * (i - rh); e1 = e0 + 1; rotated = false; }
    else { e0 = 2 * i; e1 = e0 + 1; }
    const int col0 = head * hd + e0, col1 = head * hd + e1;
    float b0 = 0.f, b1 = 0.f;
    if (PARTIALS && bias) { b0 = load_vec(bias, bias_is_f32, col0); b1 = load_vec(bias, bias_is_f32, col1); }
    size_t page_base = 0;
    if (head >= nh) {
        const int slot = seq_slot[tok_seq[t]];
        const int page = block_table[(size_t)slot * max_pages + pos / RF_PAGE];
        page_base = (size_t)page * nkv * RF_PAGE * hd + (size_t)(pos % RF_PAGE) * hd;
    }
    float s = 0.f, c = 1.f;
    if (rotated) sincosf((float)pos * inv_freq[i], &s, &c);
    pdl_wait();
    float x0, x1;
    if (PARTIALS) {
        const float* p = reinterpret_cast<const float*>(src) + (size_t)t * row_stride;
        x0 = b0; x1 = b1;
        for (int sp = 0; sp < n_partials; sp += 8) {    // eight pairs of loads in flight at once, added in index order
            float u0[8], u1[8];
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (sp + u < n_partials) {
                    u0[u] = p[(size_t)(sp + u) * partial_stride + col0];
                    u1[u] = p[(size_t)(sp + u) * partial_stride + col1];
                }
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (sp + u < n_partials) { x0 += u0[u]; x1 += u1[u]; }
        }
    } else {
        x0 = Cvt<T>::to_f32(reinterpret_cast<const T*>(src)[(size_t)t * row_stride + col0]);
        x1 = Cvt<T>::to_f32(reinterpret_cast<const T*>(src)[(size_t)t * row_stride + col1]);
    }
    if (rotated) {
        const float r0 = x0 * c - x1 * s, r1 = x0 * s + x1 * c;
        x0 = r0; x1 = r1;
    }
    T* dst = head < nh ? q_out + (size_t)t * q_out_stride + (size_t)head * hd
           : head < nh + nkv ? k_pages + page_base + (size_t)(head - nh) * RF_PAGE * hd
                             : v_pages + page_base + (size_t)(head - nh - nkv) * RF_PAGE * hd;
    dst[e0] = Cvt<T>::from_f32(x0);
    dst[e1] = Cvt<T>::from_f32(x1);
}

// The same for many tokens (prompts) whose q | k | v rows are one tensor in the compute dtype: a block per
// token; a thread takes four neighbouring pair indices, computes their sines and cosines once and walks
// over the heads in steps of blockDim.x / (hd/8) with loads and stores of four elements, so the
// trigonometry is shared by the heads and every access is 8 or 16 bytes wide.
template <typename T>
__global__ void __launch_bounds__(256)
rope_kv_write_rows_kernel(const T* __restrict__ src, int row_stride, T* __restrict__ q_out, int q_out_stride,
                          int nh, int nkv, int hd, const float* __restrict__ inv_freq,
                          const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                          const int* __restrict__ seq_slot, const int* __restrict__ block_table, int max_pages,
                          T* __restrict__ k_pages, T* __restrict__ v_pages, int write_kv) {
    pdl_trigger();
    const int t = blockIdx.x;
    const int half = hd >> 1, groups = half >> 2;        // groups of four pairs per head
    const int g = threadIdx.x % groups, lane_head = threadIdx.x / groups, head_step = blockDim.x / groups;
    if (lane_head >= head_step) return;                  // threads beyond the last whole row of groups
    const int pos = tok_pos[t];
    size_t page_base = 0;
    if (write_kv) {
        const int slot = seq_slot[tok_seq[t]];
        const int page = block_table[(size_t)slot * max_pages + pos / RF_PAGE];
        page_base = (size_t)page * nkv * RF_PAGE * hd + (size_t)(pos % RF_PAGE) * hd;
    }
    float sn[4], cs[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) sincosf((float)pos * inv_freq[4 * g + j], &sn[j], &cs[j]);
    pdl_wait();
    const T* row = src + (size_t)t * row_stride;
    const int rotated = write_kv ? nh + nkv : nh;
    for (int head = lane_head; head < rotated; head += head_step) {
        float x0[4], x1[4], r0[4], r1[4];
        Four<T>::load(row + (size_t)head * hd + 4 * g, x0);
        Four<T>::load(row + (size_t)head * hd + half + 4 * g, x1);
#pragma unroll
        for (int j = 0; j < 4; ++j) { r0[j] = x0[j] * cs[j] - x1[j] * sn[j]; r1[j] = x0[j] * sn[j] + x1[j] * cs[j]; }
        T* dst = head < nh ? q_out + (size_t)t * q_out_stride + (size_t)head * hd
                           : k_pages + page_base + (size_t)(head - nh) * RF_PAGE * hd;
        Four<T>::store(dst + 4 * g, r0);
        Four<T>::store(dst + half + 4 * g, r1);
    }
    if (write_kv)
        for (int vh = lane_head; vh < nkv; vh += head_step) {
            float a[4], b[4];
            const T* sv = row + (size_t)(nh + nkv + vh) * hd;
            Four<T>::load(sv + 4 * g, a);
            Four<T>::load(sv + half + 4 * g, b);
            T* dst = v_pages + page_base + (size_t)vh * RF_PAGE * hd;
            Four<T>::store(dst + 4 * g, a);
            Four<T>::store(dst + half + 4 * g, b);
        }
}

// ---------------------------------------------------------------- SwiGLU
// gu: [T, 2I] with gate_j at column 2j and up_j at column 2j+1 (the fused weight is
// interleaved row by row at load time); a[t, j] = silu(gate) * up, evaluated in 32-bit.
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ a, size_t n_out, int I) {
    pdl_trigger();
    pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n_out;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / I, j = idx - t * I;
        const float g = Cvt<T>::to_f32(gu[t * 2 * I + 2 * j]);
        const float u = Cvt<T>::to_f32(gu[t * 2 * I + 2 * j + 1]);
        a[idx] = Cvt<T>::from_f32(g / (1.f + expf(-g)) * u);
    }
}

// ---------------------------------------------------------------- launchers
template <typename T>
static int launch_embed(const void* table, const int* ids, float* out, int T_, int H, int V, cudaStream_t st) {
    if (T_ <= 0) return 0;
    rf_launch(embed_kernel<T>, dim3(T_), dim3(256), 0, st, reinterpret_cast<const T*>(table), ids, out, H, V);
    RF_LAUNCH_CHECK();
    return 0;
}

template <typename T>
static int launch_add_rmsnorm(float* h, const void* pending, int kind, int n_pending, size_t pstride,
                              const void* w, int w_is_f32, float eps, void* y, const int* rows,
                              int n_rows, int H, int* status, cudaStream_t st) {
    if (n_rows <= 0) return 0;
    if (H % 4 == 0 && H <= 4 * 4 * 1024 && (pstride % 4) == 0 &&
        !(reinterpret_cast<uintptr_t>(h) & 15) && !(reinterpret_cast<uintptr_t>(w) & 15) && !(reinterpret_cast<uintptr_t>(y) & 15) &&
        !(kind == 1 && (reinterpret_cast<uintptr_t>(pending) & 15))) {
        const int nvec = H / 4;
        if (kind == 0 && !rows && n_rows >= 512) {       // a prompt step's norm: rows read twice, eight CTAs per SM
            rf_launch(rmsnorm_rows_kernel<T>, dim3(n_rows), dim3(256), 0, st, (const float*)h, w, w_is_f32, eps, reinterpret_cast<T*>(y), H);
            RF_LAUNCH_CHECK();
            return 0;
        }
        // few rows (decode): one 16-byte vector per thread, the shortest chain per row;
        // many rows (prompts): 256 threads a row, so that eight rows per SM are in flight
        int threads = ((nvec + 31) / 32) * 32;
        if (threads > 1024) threads = 1024;
        if (n_rows >= 512 && nvec > 256 && nvec <= 1024) threads = 256;
        const int per = (nvec + threads - 1) / threads;
        T* yy = reinterpret_cast<T*>(y);
        // few rows: the row's threads as a cluster of up to 8 CTAs of whole warps, while that makes no more CTAs than
        // two per SM
        int cl = 1;
        for (int c = 8; c >= 2; --c)
            if ((threads / 32) % c == 0 && (long long)n_rows * c <= 296) { cl = c; break; }
        const dim3 grid(n_rows * cl), block(threads / cl);
        auto go = [&](auto kernel) {
            if (cl > 1) rf_launch_cluster(kernel, grid, block, 0, st, cl, h, pending, kind, n_pending, pstride, w, w_is_f32, eps, yy, rows, H, cl, status);
            else rf_launch(kernel, grid, block, 0, st, h, pending, kind, n_pending, pstride, w, w_is_f32, eps, yy, rows, H, cl, status);
        };
        const bool wide = block.x <= 256 && kind == 1 && n_pending > 4;      // K splits to add up, and room for the registers
        if (per <= 1 && wide) go(add_rmsnorm_vec_kernel<T, 1, 16, 256>);
        else if (per <= 2 && wide) go(add_rmsnorm_vec_kernel<T, 2, 8, 256>);
        else if (per <= 1) go(add_rmsnorm_vec_kernel<T, 1, 4, 1024>);
        else if (per <= 2) go(add_rmsnorm_vec_kernel<T, 2, 4, 1024>);
        else go(add_rmsnorm_vec_kernel<T, 4, 4, 1024>);
        RF_LAUNCH_CHECK();
        return 0;
    }
    const size_t smem = (size_t)(H + 33) * sizeof(float);
    if (smem > 200 * 1024) return RF_ERR_UNSUPPORTED;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(add_rmsnorm_kernel<T>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    const int threads = H >= 2048 ? 512 : 256;
    rf_launch(add_rmsnorm_kernel<T>, dim3(n_rows), dim3(threads), smem, st, h, pending, kind, n_pending, pstride, w,
              w_is_f32, eps, reinterpret_cast<T*>(y), rows, H);
    RF_LAUNCH_CHECK();
    return 0;
}

template <typename T>
static int launch_rope_kv_write(const void* src, int row_stride, int n_partials, size_t partial_stride,
                                const void* bias, int bias_is_f32, void* q_out, int q_out_stride, int nh, int nkv,
                                int hd, const float* inv_freq, const int* tok_seq, const int* tok_pos,
                                const int* seq_slot, const int* block_table, int max_pages, void* k_pages,
                                void* v_pages, int write_kv, int T_, int rot_dim, int interleaved, cudaStream_t st) {
    if (T_ <= 0) return 0;
    if (hd % 2 || rot_dim % 2 || rot_dim < 0 || rot_dim > hd) return RF_ERR_BAD_ARG;
    const int n_pairs = (nh + 2 * nkv) * (hd / 2);
    const dim3 grid(T_, (n_pairs + 255) / 256);
    if (T_ > 2147483647 || grid.y > 65535) return RF_ERR_UNSUPPORTED;
    // prompts: rows of one tensor, everything aligned for accesses of four elements
    const size_t four = 4 * sizeof(T);
    auto aligned = [&](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) % four) == 0; };
    if (n_partials == 0 && rot_dim == hd && !interleaved && T_ >= 64 && hd % 8 == 0 && hd / 8 <= 256 && row_stride % 4 == 0 && q_out_stride % 4 == 0 &&
        aligned(src) && aligned(q_out) && (!write_kv || (aligned(k_pages) && aligned(v_pages)))) {
        const int groups = hd / 8;
        int threads = ((nh + 2 * nkv) * groups + 31) / 32 * 32;        // a row of groups per head, at most 256 threads
        if (threads > 256) threads = 256;
        if (threads < groups) threads = (groups + 31) / 32 * 32;
        rf_launch(rope_kv_write_rows_kernel<T>, dim3(T_), dim3(threads), 0, st, reinterpret_cast<const T*>(src), row_stride,
            reinterpret_cast<T*>(q_out), q_out_stride, nh, nkv, hd, inv_freq, tok_seq, tok_pos, seq_slot, block_table,
            max_pages, reinterpret_cast<T*>(k_pages), reinterpret_cast<T*>(v_pages), write_kv);
        RF_LAUNCH_CHECK();
        return 0;
    }
    if (n_partials > 0)
        rf_launch(rope_kv_write_kernel<T, true>, grid, dim3(256), 0, st, src, row_stride, n_partials, partial_stride, bias,
            bias_is_f32, reinterpret_cast<T*>(q_out), q_out_stride, nh, nkv, hd, inv_freq, tok_seq, tok_pos, seq_slot,
            block_table, max_pages, reinterpret_cast<T*>(k_pages), reinterpret_cast<T*>(v_pages), write_kv, rot_dim,
            interleaved);
    else
        rf_launch(rope_kv_write_kernel<T, false>, grid, dim3(256), 0, st, src, row_stride, 0, (size_t)0, (const void*)nullptr, 0,
            reinterpret_cast<T*>(q_out), q_out_stride, nh, nkv, hd, inv_freq, tok_seq, tok_pos, seq_slot,
            block_table, max_pages, reinterpret_cast<T*>(k_pages), reinterpret_cast<T*>(v_pages), write_kv, rot_dim,
            interleaved);
    RF_LAUNCH_CHECK();
    return 0;
}

template <typename T>
static int launch_swiglu(const void* gu, void* a, int T_, int I, cudaStream_t st) {
    const size_t n = (size_t)T_ * I;
    if (n == 0) return 0;
    const int blocks = (int)((n + 255) / 256 > 148 * 16 ? 148 * 16 : (n + 255) / 256);
    rf_launch(swiglu_kernel<T>, dim3(blocks), dim3(256), 0, st, reinterpret_cast<const T*>(gu), reinterpret_cast<T*>(a), n, I);
    RF_LAUNCH_CHECK();
    return 0;
}

// dtype: 0 = float32, 1 = bfloat16
extern "C" {
int rf_embed(int dtype, const void* table, const int* ids, float* out, int T_, int H, int V, cudaStream_t st) {
    return dtype == 0 ? launch_embed<float>(table, ids, out, T_, H, V, st)
                      : launch_embed<__nv_bfloat16>(table, ids, out, T_, H, V, st);
}
int rf_add_rmsnorm(int dtype, float* h, const void* pending, int kind, int n_pending, long long pstride,
                   const void* w, int w_is_f32, float eps, void* y, const int* rows, int n_rows, int H,
                   int* status, cudaStream_t st) {
    // status: the device word that a cluster's bounded wait sets to 7 when it runs out (may be null)
    return dtype == 0
        ? launch_add_rmsnorm<float>(h, pending, kind, n_pending, (size_t)pstride, w, w_is_f32, eps, y, rows, n_rows, H, status, st)
        : launch_add_rmsnorm<__nv_bfloat16>(h, pending, kind, n_pending, (size_t)pstride, w, w_is_f32, eps, y, rows, n_rows, H, status, st);
}
int rf_rope_kv_write(int dtype, const void* src, int row_stride, int n_partials, long long partial_stride,
                     const void* bias, int bias_is_f32, void* q_out, int q_out_stride, int nh, int nkv, int hd,
                     const float* inv_freq, const int* tok_seq, const int* tok_pos, const int* seq_slot,
                     const int* block_table, int max_pages, void* k_pages, void* v_pages, int write_kv, int T_,
                     int rot_dim, int interleaved, cudaStream_t st) {
    return dtype == 0
        ? launch_rope_kv_write<float>(src, row_stride, n_partials, (size_t)partial_stride, bias, bias_is_f32, q_out,
                                      q_out_stride, nh, nkv, hd, inv_freq, tok_seq, tok_pos, seq_slot, block_table,
                                      max_pages, k_pages, v_pages, write_kv, T_, rot_dim, interleaved, st)
        : launch_rope_kv_write<__nv_bfloat16>(src, row_stride, n_partials, (size_t)partial_stride, bias, bias_is_f32,
                                              q_out, q_out_stride, nh, nkv, hd, inv_freq, tok_seq, tok_pos, seq_slot,
                                              block_table, max_pages, k_pages, v_pages, write_kv, T_, rot_dim, interleaved, st);
}
int rf_swiglu(int dtype, const void* gu, void* a, int T_, int I, cudaStream_t st) {
    return dtype == 0 ? launch_swiglu<float>(gu, a, T_, I, st) : launch_swiglu<__nv_bfloat16>(gu, a, T_, I, st);
}
}
