// Random weights on the device: element i of a tensor gets a value that depends on (key, i) alone, the key
// being made from the seed and the tensor's name on the host.  The same arithmetic exists on the host
// (weights/random_init.py), operation for operation, so that a model made on the device and a model folder
// written on the host hold the same bits for one seed.
//
//   h = mix64(key + (i + 1) * 0x9E3779B97F4A7C15)              (the splitmix64 finaliser)
//   u = h >> 32;  cell = u >> 16;  frac = (u & 0xffff) / 65536
//   z = table[cell] + frac * (table[cell + 1] - table[cell])   (float64, each operation rounded on its own)
//   value = float32(z * std), then rounded to the tensor's dtype
//
// ``table`` holds the standard normal quantiles at 65,537 evenly spaced probabilities (the caller computes
// it once and passes the same table to both sides): a piecewise linear inverse distribution function,
// without any transcendental function that two machines could round differently.
// maeddesg/ROCmForge has no random-weights mode (its model tests need downloaded files,
// tests/gpu_decode_real.rs:20-21); this kernel exists for this library's tests and measurements.
#include "common.cuh"

__device__ __forceinline__ unsigned long long rf_mix64(unsigned long long z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    return z ^ (z >> 31);
}

template <typename T>
__global__ void fill_normal_kernel(T* __restrict__ out, size_t n, unsigned long long key, double std,
                                   const double* __restrict__ table) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const unsigned long long h = rf_mix64(key + (unsigned long long)(i + 1) * 0x9E3779B97F4A7C15ULL);
        const unsigned int u = (unsigned int)(h >> 32);
        const unsigned int cell = u >> 16;
        const double frac = (double)(u & 0xffffu) * (1.0 / 65536.0);
        const double lo = table[cell], hi = table[cell + 1];
        const double z = __dadd_rn(lo, __dmul_rn(frac, __dadd_rn(hi, -lo)));       // no fused multiply-add: the host has none
        out[i] = Cvt<T>::from_f32((float)__dmul_rn(z, std));
    }
}

extern "C" int rf_fill_normal(int dtype, void* out, long long n, unsigned long long key, double std,
                              const double* table, cudaStream_t st) {
    if (n <= 0) return 0;
    if (!out || !table) return RF_ERR_BAD_ARG;
    const long long want = (n + 255) / 256;
    const int blocks = (int)(want > 148 * 32 ? 148 * 32 : want);
    if (dtype == 0)
        fill_normal_kernel<float><<<blocks, 256, 0, st>>>(reinterpret_cast<float*>(out), (size_t)n, key, std, table);
    else
        fill_normal_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(reinterpret_cast<__nv_bfloat16*>(out), (size_t)n, key, std, table);
    RF_LAUNCH_CHECK();
    return 0;
}
