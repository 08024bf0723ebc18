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
    argmax_kernel<<<rows, 1024, 0, st>>>(logits, V, row_stride, out);
    RF_LAUNCH_CHECK();
    return 0;
}
