// The allocation-free variant of the decode attention: see attention_decode_noalloc.h for who it is
// for and what it promises.  The kernel is the one of attention_decode.cu, compiled into this
// library a second time; only the home of its scratch memory differs.
#include "attention_decode_noalloc.h"
#include "attention_decode.cu"

// Scratch of every call on this GPU.  In host code this name is only a handle for the runtime's
// symbol lookup, not a device address: a kernel must be given the pointer that
// cudaGetSymbolAddress returns, never `rf_noalloc_scratch` itself.
static __device__ __align__(256) unsigned char rf_noalloc_scratch[RF_NOALLOC_SCRATCH_BYTES];

#define RF_NOALLOC_MAX_DEVICES 64
static void* g_scratch_of_device[RF_NOALLOC_MAX_DEVICES];

// The array's address on the current device, looked up once per device.
static int scratch_address(void** ptr) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= RF_NOALLOC_MAX_DEVICES) return RF_ERR_UNSUPPORTED;
    if (!g_scratch_of_device[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, rf_noalloc_scratch);
        if (e != cudaSuccess) return (int)e;
        if (!p) return RF_ERR_UNSUPPORTED;
        g_scratch_of_device[dev] = p;
    }
    *ptr = g_scratch_of_device[dev];
    return 0;
}

extern "C" int rf_attention_decode_noalloc(const void* q, int q_stride, void* out, int out_stride,
                                           const void* k_pages, const void* v_pages, const int* tok_seq,
                                           const int* tok_pos, const int* seq_slot, const int* block_table,
                                           int max_pages, int nh, int nkv, int hd, float scale, int window, int B,
                                           int max_chunks, int* status, cudaStream_t st) {
    if (B <= 0) return 0;
    if (!rf_attention_decode_supported(nh, nkv, hd) || max_chunks <= 0) return RF_ERR_UNSUPPORTED;
    long long n_o = 0, n_ml = 0, n_c = 0;
    rf_attention_decode_scratch(B, nh, nkv, hd, max_chunks, &n_o, &n_ml, &n_c);
    // layout inside the array: partial outputs | partial (max, sum) | counters, each 256-byte aligned
    const size_t off_ml = ((size_t)n_o * sizeof(float) + 255) & ~(size_t)255;
    const size_t off_c = (off_ml + (size_t)n_ml * sizeof(float) + 255) & ~(size_t)255;
    const size_t need = off_c + (size_t)n_c * sizeof(int);
    if (need > RF_NOALLOC_SCRATCH_BYTES) return RF_ERR_UNSUPPORTED;      // larger than the fixed array: refuse
    void* base = nullptr;
    const int rc = scratch_address(&base);
    if (rc) return rc;
    unsigned char* b8 = static_cast<unsigned char*>(base);
    int* counters = reinterpret_cast<int*>(b8 + off_c);
    // the array keeps the previous call's contents; the counters must start at zero
    cudaError_t e = cudaMemsetAsync(counters, 0, (size_t)n_c * sizeof(int), st);
    if (e != cudaSuccess) return (int)e;
    return rf_attention_decode(q, q_stride, out, out_stride, k_pages, v_pages, tok_seq, tok_pos, seq_slot,
                               block_table, max_pages, nh, nkv, hd, scale, window, B, max_chunks,
                               reinterpret_cast<float*>(b8), reinterpret_cast<float*>(b8 + off_ml), counters,
                               status, st);
}
