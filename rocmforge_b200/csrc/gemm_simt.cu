// Plain CUDA-core matrix product  Y[M,N] = X[M,K] * W[N,K]^T (+ bias), any M, N, K.
//
// It is the whole matrix path of the true 32-bit model (FFMA only: the tensor cores'
// 32-bit mode rounds operands to TF32, which is what that path must not do) and the
// fallback of the bfloat16 path for shapes the tensor-core kernel refuses.
// Products are summed in 32-bit in ascending k by one thread per output element, so
// a row's result does not depend on how many other rows the batch has.
// Counterpart in maeddesg/ROCmForge: the scalar GEMM at the end of its dispatch chain
// (src/gpu/ops.rs:1591-1973) and src/cpu/ops.rs:342-352.
#include "common.cuh"

#define BM 64
#define BN 64
#define BK 16

// mode 0: Y (compute dtype) = acc + bias;  1: Y (float) = acc + bias;  2: Y (float) += acc + bias
template <typename T>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const T* __restrict__ X, const T* __restrict__ W, const void* __restrict__ bias,
                 int bias_is_f32, void* __restrict__ Y, int M, int N, int K, int ldx, int ldy, int mode) {
    pdl_trigger();
    pdl_wait();
    __shared__ float Xs[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int i = threadIdx.x; i < BM * BK; i += 256) {
            const int r = i / BK, c = i - r * BK;
            const int m = m0 + r, n = n0 + r, k = k0 + c;
            Xs[c][r] = (m < M && k < K) ? Cvt<T>::to_f32(X[(size_t)m * ldx + k]) : 0.f;
            Ws[c][r] = (n < N && k < K) ? Cvt<T>::to_f32(W[(size_t)n * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = Xs[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += load_vec(bias, bias_is_f32, n);
            const size_t o = (size_t)m * ldy + n;
            if (mode == 0) reinterpret_cast<T*>(Y)[o] = Cvt<T>::from_f32(v);
            else if (mode == 1) reinterpret_cast<float*>(Y)[o] = v;
            else reinterpret_cast<float*>(Y)[o] += v;
        }
    }
}

template <typename T>
static int launch(const void* X, const void* W, const void* bias, int bias_is_f32, void* Y, int M, int N,
                  int K, int ldx, int ldy, int mode, cudaStream_t st) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || mode < 0 || mode > 2) return RF_ERR_BAD_ARG;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) return RF_ERR_UNSUPPORTED;
    rf_launch(gemm_simt_kernel<T>, grid, dim3(256), 0, st, reinterpret_cast<const T*>(X), reinterpret_cast<const T*>(W), bias,
              bias_is_f32, Y, M, N, K, ldx, ldy, mode);
    RF_LAUNCH_CHECK();
    return 0;
}

extern "C" int rf_gemm_simt(int dtype, const void* X, const void* W, const void* bias, int bias_is_f32,
                            void* Y, int M, int N, int K, int ldx, int ldy, int mode, cudaStream_t st) {
    return dtype == 0 ? launch<float>(X, W, bias, bias_is_f32, Y, M, N, K, ldx, ldy, mode, st)
                      : launch<__nv_bfloat16>(X, W, bias, bias_is_f32, Y, M, N, K, ldx, ldy, mode, st);
}
