// CUDA-core matrix product  Y[M,N] = X[M,K] * W[N,K]^T (+ bias), any M, N, K.
//
// It is the whole matrix path of the true 32-bit model (FFMA only: the tensor cores'
// 32-bit mode rounds operands to TF32, which is what that path must not do) and the
// fallback of the bfloat16 path for shapes the tensor-core kernel refuses.
//
// A CTA of 256 threads owns a BM x 128 tile of Y (BM = 16, 32, 64 or 128 tokens, chosen from M) and
// walks K in blocks of 16: the next block's operands travel from global memory into registers
// (16-byte loads) while the current block is multiplied out of shared memory, where both operands lie
// k-major so that a thread fetches its 8 weight columns and its BM/16 token rows with 16-byte loads and
// spends 8 * BM/16 FFMAs on them.  With few tokens the small BM keeps the arithmetic per weight byte low
// enough for the weight stream to be the limit, and K may be split over grid.z (mode 3): each split writes
// its own 32-bit partial sums [split, M, N], which the consumer adds in index order.
// A token's sums are formed in ascending k inside a split whatever BM is, and the number of splits is
// the caller's function of N and K alone, so a row's result does not depend on the other rows of its
// batch.  Counterpart in maeddesg/ROCmForge: the scalar GEMM at the end of its dispatch chain
// (src/gpu/ops.rs:1591-1973) and src/cpu/ops.rs:342-352.
#include "common.cuh"

#define GS_BN 128
#define GS_BK 16
#define GS_THREADS 256

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

// Four consecutive k of one row, zero beyond the row count or K; 16-byte (8-byte for bfloat16) loads where
// the row is aligned for them.
template <typename T>
__device__ __forceinline__ float4 load_k4(const T* __restrict__ base, int row, int rows, int ld, int k, int k_end, bool vec) {
    if (row >= rows || k >= k_end) return make_float4(0.f, 0.f, 0.f, 0.f);
    const T* p = base + (size_t)row * ld + k;
    if (vec && k + 3 < k_end) return Vec4<T>::load(p);
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = (k + j < k_end) ? Cvt<T>::to_f32(p[j]) : 0.f;
    return make_float4(v[0], v[1], v[2], v[3]);
}

// mode 0: Y (compute dtype) = acc + bias;  1: Y (float) = acc + bias;  2: Y (float) += acc + bias;
// 3: Y (float) [split, M, N] = acc (partial sums of this split's K range; the bias is the consumer's)
template <typename T, int BM>
__global__ void __launch_bounds__(GS_THREADS)
gemm_simt_kernel(const T* __restrict__ X, const T* __restrict__ W, const void* __restrict__ bias,
                 int bias_is_f32, void* __restrict__ Y, int M, int N, int K, int ldx, int ldy, int mode,
                 int k_per_split, int vec_x, int vec_w) {
    constexpr int TM = BM / 16;                                  // token rows of a thread
    constexpr int XV = (BM * GS_BK / 4 + GS_THREADS - 1) / GS_THREADS;     // 16-byte loads of X per thread and block
    constexpr int WV = GS_BN * GS_BK / 4 / GS_THREADS;                      // ... of W (2)
    constexpr int LDX = BM + 4, LDW = GS_BN + 4;
    __shared__ __align__(16) float Xs[2][GS_BK][LDX];
    __shared__ __align__(16) float Ws[2][GS_BK][LDW];
    pdl_trigger();
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * GS_BN;
    const int k_begin = blockIdx.z * k_per_split;
    const int k_end = min(K, k_begin + k_per_split);
    const int lr = tid >> 2, lk = (tid & 3) * 4;                 // this thread's row and k offset inside a block load

    float4 xr[XV], wr[WV];
    auto fetch_w = [&](int k0) {
#pragma unroll
        for (int i = 0; i < WV; ++i) wr[i] = load_k4(W, n0 + lr + 64 * i, N, K, k0 + lk, k_end, vec_w);
    };
    auto fetch_x = [&](int k0) {
#pragma unroll
        for (int i = 0; i < XV; ++i)
            xr[i] = (lr + 64 * i < BM) ? load_k4(X, m0 + lr + 64 * i, M, ldx, k0 + lk, k_end, vec_x)
                                       : make_float4(0.f, 0.f, 0.f, 0.f);
    };
    auto stash = [&](int buf) {                                  // registers -> shared memory, transposed to k-major
#pragma unroll
        for (int i = 0; i < WV; ++i) {
            const int r = lr + 64 * i;
            Ws[buf][lk][r] = wr[i].x; Ws[buf][lk + 1][r] = wr[i].y; Ws[buf][lk + 2][r] = wr[i].z; Ws[buf][lk + 3][r] = wr[i].w;
        }
#pragma unroll
        for (int i = 0; i < XV; ++i) {
            const int r = lr + 64 * i;
            if (r < BM) {
                Xs[buf][lk][r] = xr[i].x; Xs[buf][lk + 1][r] = xr[i].y; Xs[buf][lk + 2][r] = xr[i].z; Xs[buf][lk + 3][r] = xr[i].w;
            }
        }
    };

    float acc[TM][8];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
    // weights do not depend on the kernel before this one; activations (and the output) do
    if (k_begin < k_end) fetch_w(k_begin);
    pdl_wait();
    if (k_begin < k_end) {
        fetch_x(k_begin);
        stash(0);
    }
    __syncthreads();
    int buf = 0;
    for (int k0 = k_begin; k0 < k_end; k0 += GS_BK) {
        const bool more = k0 + GS_BK < k_end;
        if (more) { fetch_w(k0 + GS_BK); fetch_x(k0 + GS_BK); }   // in flight while this block is multiplied
#pragma unroll
        for (int k = 0; k < GS_BK; ++k) {
            // weight columns tx*4 .. +3 and 64 + tx*4 .. +3: sixteen lanes read 256 contiguous bytes
            const float4 b0 = *reinterpret_cast<const float4*>(&Ws[buf][k][tx * 4]);
            const float4 b1 = *reinterpret_cast<const float4*>(&Ws[buf][k][64 + tx * 4]);
            const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
            float a[TM];
            if constexpr (TM == 8) {
                const float4 a0 = *reinterpret_cast<const float4*>(&Xs[buf][k][ty * 4]);
                const float4 a1 = *reinterpret_cast<const float4*>(&Xs[buf][k][64 + ty * 4]);
                a[0] = a0.x; a[1] = a0.y; a[2] = a0.z; a[3] = a0.w;
                a[4] = a1.x; a[5] = a1.y; a[6] = a1.z; a[7] = a1.w;
            } else if constexpr (TM == 4) {
                const float4 a0 = *reinterpret_cast<const float4*>(&Xs[buf][k][ty * 4]);
                a[0] = a0.x; a[1] = a0.y; a[2] = a0.z; a[3] = a0.w;
            } else if constexpr (TM == 2) {
                const float2 a0 = *reinterpret_cast<const float2*>(&Xs[buf][k][ty * 2]);
                a[0] = a0.x; a[1] = a0.y;
            } else {
                a[0] = Xs[buf][k][ty];
            }
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        if (more) stash(buf ^ 1);
        __syncthreads();
        buf ^= 1;
    }

    // this thread's rows and columns (the same interleaving as the operand loads above)
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + (TM == 8 ? (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4)) : ty * TM + i);
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int n = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias && mode != 3) v += load_vec(bias, bias_is_f32, n);
            const size_t o = (size_t)m * ldy + n;
            if (mode == 0) reinterpret_cast<T*>(Y)[o] = Cvt<T>::from_f32(v);
            else if (mode == 1) reinterpret_cast<float*>(Y)[o] = v;
            else if (mode == 2) reinterpret_cast<float*>(Y)[o] += v;
            else reinterpret_cast<float*>(Y)[(size_t)blockIdx.z * M * ldy + o] = v;
        }
    }
}

template <typename T, int BM>
static int launch_bm(const void* X, const void* W, const void* bias, int bias_is_f32, void* Y, int M, int N,
                     int K, int ldx, int ldy, int mode, int splits, cudaStream_t st) {
    dim3 grid((N + GS_BN - 1) / GS_BN, (M + BM - 1) / BM, splits);
    if (grid.y > 65535 || grid.z > 65535) return RF_ERR_UNSUPPORTED;
    // K range of a split: whole blocks of 16, the same for every split but the last
    const int kb = (K + GS_BK - 1) / GS_BK;
    const int per = (kb + splits - 1) / splits * GS_BK;
    if ((long long)(splits - 1) * per >= K && splits > 1) return RF_ERR_BAD_ARG;       // an empty split
    const size_t es = sizeof(T);
    const int vec_x = (reinterpret_cast<uintptr_t>(X) % (4 * es) == 0) && (ldx % 4 == 0);
    const int vec_w = (reinterpret_cast<uintptr_t>(W) % (4 * es) == 0) && (K % 4 == 0);
    rf_launch(gemm_simt_kernel<T, BM>, grid, dim3(GS_THREADS), 0, st, reinterpret_cast<const T*>(X),
              reinterpret_cast<const T*>(W), bias, bias_is_f32, Y, M, N, K, ldx, ldy, mode, per, vec_x, vec_w);
    RF_LAUNCH_CHECK();
    return 0;
}

template <typename T>
static int launch(const void* X, const void* W, const void* bias, int bias_is_f32, void* Y, int M, int N,
                  int K, int ldx, int ldy, int mode, int splits, cudaStream_t st) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || mode < 0 || mode > 3 || splits < 1) return RF_ERR_BAD_ARG;
    if (splits > 1 && mode != 3) return RF_ERR_BAD_ARG;
    if (M <= 16) return launch_bm<T, 16>(X, W, bias, bias_is_f32, Y, M, N, K, ldx, ldy, mode, splits, st);
    if (M <= 32) return launch_bm<T, 32>(X, W, bias, bias_is_f32, Y, M, N, K, ldx, ldy, mode, splits, st);
    if (M <= 64) return launch_bm<T, 64>(X, W, bias, bias_is_f32, Y, M, N, K, ldx, ldy, mode, splits, st);
    return launch_bm<T, 128>(X, W, bias, bias_is_f32, Y, M, N, K, ldx, ldy, mode, splits, st);
}

extern "C" int rf_gemm_simt(int dtype, const void* X, const void* W, const void* bias, int bias_is_f32,
                            void* Y, int M, int N, int K, int ldx, int ldy, int mode, int splits, cudaStream_t st) {
    return dtype == 0 ? launch<float>(X, W, bias, bias_is_f32, Y, M, N, K, ldx, ldy, mode, splits, st)
                      : launch<__nv_bfloat16>(X, W, bias, bias_is_f32, Y, M, N, K, ldx, ldy, mode, splits, st);
}
