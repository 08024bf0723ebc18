// Attention of many new tokens over the paged bfloat16 cache (prompts, and chunks appended to a
// context): tiled, causal, grouped-query, ragged.
//
// A CTA owns 64 consecutive new tokens of one sequence and one query head; its four warps hold 16
// query rows each.  Keys and values come a cache page (64 positions) at a time: TMA copies the
// page's [64 x head_dim] slab of the head's kv head into shared memory with the 128-byte swizzle
// (two stages, the next page in flight while this one is used), ldmatrix reads it without bank
// conflicts, and both products run on the tensor cores (mma.sync m16n8k16, bf16 in, 32-bit
// accumulate).  The softmax is the online one in 32-bit (running maximum and sum per row, the
// output rescaled when the maximum moves); the weights are rounded to bfloat16 only as the
// operand of the second product.  Pages wholly above a tile's last query, or wholly below its
// window, are skipped; the page on the diagonal is masked element-wise.
//
// Same structure as maeddesg/ROCmForge's wmma_attention_prefill_online_kernel (64-query x 64-key
// tiles, causal tile skip, diagonal mask, P rounded to 16-bit, final division by the row sum;
// hip_kernels/wmma/wmma_attention_prefill.hip:386-671), but it reads the cache, so earlier
// context and other sequences of a ragged batch need no separate path, and head sizes 64 and 128
// are both taken.  Which tiles exist is decided on the host (a table of (sequence, first row)),
// so the device never searches.
#include <cuda.h>
#include "common.cuh"

#define PF_THREADS 128
#define PF_BM 64
#define PF_WAIT_LIMIT_NS 2000000000ULL

__device__ __forceinline__ uint32_t pf_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void pf_mma(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Address of the 16-byte chunk `chunk` (0..7) of row `row` in a [64 rows x 128 bytes] tile written by TMA
// with the 128-byte swizzle (the tile starts on a 1024-byte boundary).
// 2^x on the special-function unit (32-bit, relative error about 2^-22): the softmax weights are
// rounded to bfloat16 right after, and their sum is formed from the same values
__device__ __forceinline__ float pf_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t pf_swz(uint32_t tile, int row, int chunk) {
    return tile + row * 128 + ((chunk ^ (row & 7)) << 4);
}

template <int HD>
__global__ void __launch_bounds__(PF_THREADS)
attention_prefill_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                         const __nv_bfloat16* __restrict__ q, int q_stride, __nv_bfloat16* __restrict__ out,
                         int out_stride, const int* __restrict__ tiles, const int* __restrict__ seq_slot,
                         const int* __restrict__ seq_start, const int* __restrict__ seq_nnew,
                         const int* __restrict__ cu_q, const int* __restrict__ block_table, int max_pages,
                         int nh, int nkv, float scale, int window, int* __restrict__ status) {
    constexpr int HALVES = HD / 64;                     // 128-byte column blocks per row
    constexpr uint32_t TILE_BYTES = 64 * 128;           // one column block of one page
    constexpr uint32_t STAGE_BYTES = 2 * HALVES * TILE_BYTES;      // K and V
    extern __shared__ uint8_t pf_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(pf_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 2 * STAGE_BYTES);
    __shared__ int gave_up;

    pdl_trigger();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gid = lane >> 2, tig = lane & 3;
    // heavy tiles first: the table is sorted by the keys a tile sees and walked backwards, heads fastest
    const int tile_idx = gridDim.y - 1 - blockIdx.y;
    const int seq = tiles[2 * tile_idx], q0 = tiles[2 * tile_idx + 1];
    const int head = blockIdx.x, kvh = head / (nh / nkv);
    const int start = seq_start[seq], n_new = seq_nnew[seq];
    const int* bt = block_table + (size_t)seq_slot[seq] * max_pages;
    const int row_base = cu_q[seq] + q0;                // first packed token row of the tile
    int rows_here = n_new - q0; if (rows_here > PF_BM) rows_here = PF_BM;
    const int pos_first = start + q0, pos_last = start + q0 + rows_here - 1, seq_last = start + n_new - 1;
    const int lo_first = (window > 0 && pos_first - window + 1 > 0) ? pos_first - window + 1 : 0;
    const int kt_lo = lo_first / RF_PAGE, kt_hi = pos_last / RF_PAGE;
    const int n_kt = kt_hi - kt_lo + 1;

    if (tid == 0) {
        gave_up = 0;
        for (int s = 0; s < 2; ++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(pf_smem_u32(&bars[s])));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
    }
    __syncthreads();
    pdl_wait();                                        // queries, keys and values come from the kernel before us

    auto issue = [&](int it) {                          // thread 0: bring page kt_lo + it into stage it & 1
        const int stage = it & 1;
        const uint32_t bar = pf_smem_u32(&bars[stage]);
        const uint32_t dst = pf_smem_u32(smem + stage * STAGE_BYTES);
        const int page = bt[kt_lo + it];
        const int row = (page * nkv + kvh) * RF_PAGE;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(STAGE_BYTES) : "memory");
#pragma unroll
        for (int h = 0; h < HALVES; ++h) {
            asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                         ::"r"(dst + h * TILE_BYTES), "l"(&map_k), "r"(h * 64), "r"(row), "r"(bar) : "memory");
            asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                         ::"r"(dst + (HALVES + h) * TILE_BYTES), "l"(&map_v), "r"(h * 64), "r"(row), "r"(bar) : "memory");
        }
    };
    if (tid == 0) issue(0);

    // ---- this warp's 16 query rows as A fragments (rows beyond the tile's end are zero)
    const int r0 = warp * 16 + gid, r1 = r0 + 8;        // tile-relative rows of this thread
    uint32_t qa[HD / 16][4];
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
        const int col = head * HD + ks * 16 + tig * 2;
        const __nv_bfloat16* p0 = q + (size_t)(row_base + r0) * q_stride + col;
        const __nv_bfloat16* p1 = q + (size_t)(row_base + r1) * q_stride + col;
        qa[ks][0] = r0 < rows_here ? *reinterpret_cast<const uint32_t*>(p0) : 0u;
        qa[ks][1] = r1 < rows_here ? *reinterpret_cast<const uint32_t*>(p1) : 0u;
        qa[ks][2] = r0 < rows_here ? *reinterpret_cast<const uint32_t*>(p0 + 8) : 0u;
        qa[ks][3] = r1 < rows_here ? *reinterpret_cast<const uint32_t*>(p1 + 8) : 0u;
    }
    const int pos0 = pos_first + r0, pos1 = pos_first + r1;
    const int lo0 = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
    const int lo1 = (window > 0 && pos1 - window + 1 > 0) ? pos1 - window + 1 : 0;

    float oc[HD / 8][4];
#pragma unroll
    for (int nt = 0; nt < HD / 8; ++nt) oc[nt][0] = oc[nt][1] = oc[nt][2] = oc[nt][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    for (int it = 0; it < n_kt; ++it) {
        const int stage = it & 1;
        if (tid == 0 && it + 1 < n_kt) issue(it + 1);    // the other stage was released by the sync below
        {   // bounded wait for this stage
            const uint32_t bar = pf_smem_u32(&bars[stage]);
            const uint32_t parity = (it >> 1) & 1;
            uint32_t ok = 0;
            unsigned long long t0 = 0;
            for (long long spin = 0; !ok; ++spin) {
                asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                             "selp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
                if (ok) break;
                if ((spin & 63) == 63) {
                    unsigned long long now;
                    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
                    if (t0 == 0) t0 = now;
                    if (now - t0 > PF_WAIT_LIMIT_NS || gave_up) { gave_up = 1; break; }
                }
            }
        }
        __syncthreads();                                 // everyone sees the same verdict
        if (gave_up) break;
        const uint32_t k_tile = pf_smem_u32(smem + stage * STAGE_BYTES);
        const uint32_t v_tile = k_tile + HALVES * TILE_BYTES;
        const int key0 = (kt_lo + it) * RF_PAGE;
        if (key0 + RF_PAGE - 1 > seq_last) {
            // the rest of the sequence's last page was never written: its value rows get weight zero,
            // but 0 * (whatever bits lie there) must be 0, so clear them
            const int first_bad = seq_last + 1 - key0;
            for (int i = tid; i < (RF_PAGE - first_bad) * HALVES * 8; i += PF_THREADS) {
                const int row = first_bad + i / (HALVES * 8), c = i % (HALVES * 8);
                const uint32_t a = pf_swz(v_tile + (c >> 3) * TILE_BYTES, row, c & 7);
                asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(a), "r"(0u) : "memory");
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // a later TMA write must come after these
            __syncthreads();
        }
        const bool warp_needed = key0 <= pos_first + warp * 16 + 15;         // some row of the warp sees this page

        // ---- S = Q K^T for 64 keys: 8 tiles of 8 keys
        float sc[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
        if (warp_needed) {
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
                for (int np = 0; np < 4; ++np) {         // a pair of key tiles per ldmatrix.x4
                    // matrices: (keys np*16 + 0..7, dims ks*16 + 0..7), (same keys, dims + 8), (keys + 8, dims), (keys + 8, dims + 8)
                    const int mi = lane >> 3, r = lane & 7;
                    const int krow = np * 16 + (mi >> 1) * 8 + r;
                    const int chunk = (ks * 2 + (mi & 1)) & 7;
                    const uint32_t a = pf_swz(k_tile + ((ks * 2) >> 3) * TILE_BYTES, krow, chunk);
                    uint32_t b0, b1, b2, b3;
                    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                                 : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(a));
                    pf_mma(sc[np * 2], qa[ks], b0, b1);
                    pf_mma(sc[np * 2 + 1], qa[ks], b2, b3);
                }
            }
        }
        // ---- mask, running maximum, weights (32-bit; scores in units of log2 e so that exp is one ex2)
        const float sl2 = scale * 1.4426950408889634f;
        // a page wholly inside every row's range of this warp (below the diagonal, inside the window) needs no mask
        const bool no_mask = warp_needed && key0 + RF_PAGE - 1 <= pos_first + warp * 16 && warp * 16 + 15 < rows_here &&
                             (window <= 0 || key0 >= pos_first + warp * 16 + 15 - window + 1);
        float mx0 = -INFINITY, mx1 = -INFINITY;
        if (no_mask) {
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) sc[nt][e] *= sl2;
                mx0 = fmaxf(mx0, fmaxf(sc[nt][0], sc[nt][1]));
                mx1 = fmaxf(mx1, fmaxf(sc[nt][2], sc[nt][3]));
            }
        } else {
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int j = key0 + nt * 8 + tig * 2 + e;
                    const bool ok0 = warp_needed && j <= pos0 && j >= lo0 && r0 < rows_here;
                    const bool ok1 = warp_needed && j <= pos1 && j >= lo1 && r1 < rows_here;
                    sc[nt][e] = ok0 ? sc[nt][e] * sl2 : -INFINITY;
                    sc[nt][2 + e] = ok1 ? sc[nt][2 + e] * sl2 : -INFINITY;
                    mx0 = fmaxf(mx0, sc[nt][e]);
                    mx1 = fmaxf(mx1, sc[nt][2 + e]);
                }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        // ex2(-inf) = 0 covers masked scores and the first page; a row that has seen no key yet keeps mn = -inf,
        // where (-inf) - (-inf) would be NaN: such rows use 0 as the reference instead
        const float ref0 = mn0 == -INFINITY ? 0.f : mn0, ref1 = mn1 == -INFINITY ? 0.f : mn1;
        const float cr0 = pf_exp2(m0 - ref0), cr1 = pf_exp2(m1 - ref1);
        m0 = mn0; m1 = mn1;
        float s0 = 0.f, s1 = 0.f;
        uint32_t pa[4][4];                               // P as A fragments: 4 steps of 16 keys
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            const float p00 = pf_exp2(sc[nt][0] - ref0), p01 = pf_exp2(sc[nt][1] - ref0);
            const float p10 = pf_exp2(sc[nt][2] - ref1), p11 = pf_exp2(sc[nt][3] - ref1);
            s0 += p00 + p01; s1 += p10 + p11;
            const __nv_bfloat162 x = __floats2bfloat162_rn(p00, p01), y = __floats2bfloat162_rn(p10, p11);
            pa[nt >> 1][(nt & 1) * 2] = *reinterpret_cast<const uint32_t*>(&x);
            pa[nt >> 1][(nt & 1) * 2 + 1] = *reinterpret_cast<const uint32_t*>(&y);
        }
        s0 += __shfl_xor_sync(0xffffffffu, s0, 1); s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
        s1 += __shfl_xor_sync(0xffffffffu, s1, 1); s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
        l0 = l0 * cr0 + s0; l1 = l1 * cr1 + s1;
#pragma unroll
        for (int nt = 0; nt < HD / 8; ++nt) { oc[nt][0] *= cr0; oc[nt][1] *= cr0; oc[nt][2] *= cr1; oc[nt][3] *= cr1; }

        // ---- O += P V
        if (warp_needed) {
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {             // 16 keys per step
#pragma unroll
                for (int nt = 0; nt < HD / 8; nt += 2) {
                    // matrices: (keys ks*16 + 0..7, dims nt*8..), (keys + 8, same dims), (keys, dims + 8), (keys + 8, dims + 8)
                    const int mi = lane >> 3, r = lane & 7;
                    const int vrow = ks * 16 + (mi & 1) * 8 + r;
                    const int dchunk = nt + (mi >> 1);                       // 16-byte chunk index along the row
                    const uint32_t a = pf_swz(v_tile + (dchunk >> 3) * TILE_BYTES, vrow, dchunk & 7);
                    uint32_t v0, v1, v2, v3;
                    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                                 : "=r"(v0), "=r"(v1), "=r"(v2), "=r"(v3) : "r"(a));
                    pf_mma(oc[nt], pa[ks], v0, v1);
                    pf_mma(oc[nt + 1], pa[ks], v2, v3);
                }
            }
        }
        __syncthreads();                                 // the stage may be refilled
    }
    if (gave_up) {
        if (tid == 0 && status) atomicExch(status, 3);
        return;
    }
    // ---- O / l -> bfloat16
    const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
#pragma unroll
    for (int nt = 0; nt < HD / 8; ++nt) {
        const int col = head * HD + nt * 8 + tig * 2;
        if (r0 < rows_here)
            *reinterpret_cast<__nv_bfloat162*>(out + (size_t)(row_base + r0) * out_stride + col) =
                __floats2bfloat162_rn(oc[nt][0] * i0, oc[nt][1] * i0);
        if (r1 < rows_here)
            *reinterpret_cast<__nv_bfloat162*>(out + (size_t)(row_base + r1) * out_stride + col) =
                __floats2bfloat162_rn(oc[nt][2] * i1, oc[nt][3] * i1);
    }
}

// ---------------------------------------------------------------- host side
typedef CUresult (*PfEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static PfEncodeFn pf_encode_fn() {
    static PfEncodeFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qr) == cudaSuccess &&
            qr == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<PfEncodeFn>(ptr);
    }
    return fn;
}

// pages [n_pages, nkv, 64, hd] seen as a matrix [n_pages * nkv * 64, hd]; box = 64 rows x 64 columns
static int pf_make_map(CUtensorMap* map, const void* pages, long long rows, int hd) {
    PfEncodeFn fn = pf_encode_fn();
    if (!fn) return RF_ERR_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(pages) & 15) return RF_ERR_BAD_ARG;
    cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
    cuuint32_t box[2] = {64, 64};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pages), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : RF_ERR_BAD_ARG;
}

template <int HD>
static int pf_launch(const CUtensorMap& mk, const CUtensorMap& mv, const void* q, int q_stride, void* out,
                     int out_stride, const int* tiles, int n_tiles, const int* seq_slot, const int* seq_start,
                     const int* seq_nnew, const int* cu_q, const int* block_table, int max_pages, int nh, int nkv,
                     float scale, int window, int* status, cudaStream_t st) {
    constexpr size_t smem = 2 * 2 * (HD / 64) * 64 * 128 + 2 * 8 + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    if (n_tiles > 65535) return RF_ERR_UNSUPPORTED;     // tiles are the grid's y dimension
    dim3 grid(nh, n_tiles);
    rf_launch(attention_prefill_kernel<HD>, grid, dim3(PF_THREADS), smem, st,
        mk, mv, reinterpret_cast<const __nv_bfloat16*>(q), q_stride, reinterpret_cast<__nv_bfloat16*>(out), out_stride,
        tiles, seq_slot, seq_start, seq_nnew, cu_q, block_table, max_pages, nh, nkv, scale, window, status);
    RF_LAUNCH_CHECK();
    return 0;
}

extern "C" {

int rf_attention_prefill_supported(int nh, int nkv, int hd) {
    if (nkv <= 0 || nh % nkv || nh > 65535) return 0;
    return (hd == 64 || hd == 128) && pf_encode_fn() != nullptr;
}

// tiles: n_tiles pairs (sequence index, first new-token row of the tile within the sequence), 64 rows a tile.
int rf_attention_prefill(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                         const void* v_pages, long long n_pages, const int* tiles, int n_tiles, const int* seq_slot,
                         const int* seq_start, const int* seq_nnew, const int* cu_q, const int* block_table,
                         int max_pages, int nh, int nkv, int hd, float scale, int window, int* status,
                         cudaStream_t st) {
    if (n_tiles <= 0) return 0;
    if (!rf_attention_prefill_supported(nh, nkv, hd)) return RF_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(q) & 3) || (q_stride & 1) || (out_stride & 1)) return RF_ERR_BAD_ARG;
    CUtensorMap mk, mv;
    int e;
    const long long rows = n_pages * nkv * RF_PAGE;
    if ((e = pf_make_map(&mk, k_pages, rows, hd)) || (e = pf_make_map(&mv, v_pages, rows, hd))) return e;
    if (hd == 64)
        return pf_launch<64>(mk, mv, q, q_stride, out, out_stride, tiles, n_tiles, seq_slot, seq_start, seq_nnew, cu_q,
                             block_table, max_pages, nh, nkv, scale, window, status, st);
    return pf_launch<128>(mk, mv, q, q_stride, out, out_stride, tiles, n_tiles, seq_slot, seq_start, seq_nnew, cu_q,
                          block_table, max_pages, nh, nkv, scale, window, status, st);
}

}
