// The large-M bfloat16 matrix product: persistent, clustered, with a double-buffered accumulator.
//
//   D[m, n] = sum_k X[m, k] * W[n, k]      tokens as accumulator rows, 128 x 256 tiles per CTA
//
// What it adds to gemm_tcgen05.cu, and why (B200: 148 SMs, ~2.25 PFLOP/s dense bf16, one L2):
//   * A 128 x 256 x 64 step needs 48 KB of operands for 4.2 MFLOP; 148 SMs at full tensor rate would
//     pull more from L2 than it delivers.  CTAs are therefore launched as clusters of CL along M:
//     the CL CTAs of a cluster work on the same 256 weight rows, each loads 256/CL of them and
//     multicasts its part into every CTA of the cluster, so a weight tile crosses L2 -> SM once per
//     cluster instead of once per CTA.  (This GPU's own memory only; this file is used by
//     single-GPU runs alone.)
//   * CTAs are persistent: each cluster walks a list of (row group, column tile) work items, rows
//     fastest, so that neighbouring clusters share a weight tile in L2.
//   * The accumulator has two buffers in tensor memory (2 x 256 columns): while the four epilogue
//     warps drain tile i, the MMA thread is already accumulating tile i + 1, and the TMA ring runs
//     ahead across tile borders.
//   * The epilogue leaves through shared memory and TMA: a thread owns one output row, so direct stores
//     would scatter 16-byte pieces over 32 rows per instruction; instead the four epilogue warps write a
//     128-row x 128-byte slab into a swizzled staging buffer (two of them, alternating) and one thread
//     hands it to TMA, which writes full lines, clips at the matrix edge, and for the residual epilogue
//     ADDS in L2 (cp.reduce.async.bulk .add.f32), so the 32-bit stream is never read back into the SM.
// A stage of a CTA's ring is written by its own loads and by its peers' multicasts, so it may be
// refilled only when every CTA of the cluster has finished reading it: the "empty" barrier of a
// stage counts CL arrivals, and each CTA's MMA thread signals all of them with one multicast
// tcgen05.commit.  Waits are bounded as everywhere; a cluster-wide barrier at both ends keeps a
// CTA's shared memory alive while peers can still write to it.
//
// Counterpart in maeddesg/ROCmForge: the prefill GEMMs of hip_kernels/wmma/ (64x64x16 tiles, one
// tile per block, single-buffered LDS, wmma_gemm_tiled.hip:57-195).
#include "tcgen05_common.cuh"

#define CG_BN 256
#define CG_STAGES 4
#define CG_THREADS 192

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tma_load_2d_multicast(uint32_t dst, const CUtensorMap* map, int c0, int c1,
                                                      uint32_t bar, uint16_t mask) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.multicast::cluster"
        " [%0], [%1, {%2, %3}], [%4], %5;"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar), "h"(mask) : "memory");
}
__device__ __forceinline__ void tcgen05_commit_multicast(uint32_t bar, uint16_t mask) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(mask) : "memory");
}
// ---- two CTAs as one MMA unit (cta_group::2).  The even CTA of a pair issues 256-row products that read both
// CTAs' shared memory (each holds its own 128 activation rows and its half of the weight rows) and write both
// CTAs' tensor memory; loads of either CTA report their bytes to the even CTA's barrier.
__device__ __forceinline__ uint32_t cluster_addr_of(uint32_t local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t cluster_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void tcgen05_alloc_pair(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tcgen05_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tcgen05_mma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                      uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tcgen05_commit_pair(uint32_t bar, uint16_t mask) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(mask) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
// M = 256 over the pair, N = n
__host__ __device__ constexpr uint32_t make_idesc_pair(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int c0, int c1, uint32_t src) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];"
                 ::"l"(map), "r"(c0), "r"(c1), "r"(src) : "memory");
}
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, int c0, int c1, uint32_t src) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2}], [%3];"
                 ::"l"(map), "r"(c0), "r"(c1), "r"(src) : "memory");
}
__device__ __forceinline__ void epi_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }   // the 4 epilogue warps

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// grid.x = n_clusters * CL (cluster dimension CL along x).  Work item w -> row group w % groups_m,
// column tile (w / groups_m) % tiles_n, K part w / (groups_m * tiles_n); CTA `rank` of the cluster owns
// row tile group * CL + rank.
//
// K parts (p.splits > 1, residual epilogue only).  The persistent clusters work in rounds, and a last round
// that is half empty costs as much as a full one (2,048 x 3,584 outputs: 112 tiles on 74 clusters).  The
// host may therefore cut K into P parts: P times as many, shorter work items fill the rounds better
// (112 x 5 items: 8 rounds of a fifth = 1.6 instead of 2).  Every part adds its sums into the 32-bit
// stream with TMA's reduce-add, and so that the sum of a tile is formed in ONE order, whatever the timing,
// part q of a tile waits (bounded) until part q - 1 of that tile has been added: `flags[tile]` counts the
// parts that are in; the last part sets it back to zero for the next launch.  Parts are scheduled
// part-major (all first parts, then all second parts, ...), and all clusters of the grid are resident, so a
// wait is always for work that was handed out earlier: it cannot deadlock, and in practice it never spins.
// PAIR (CL = 2 only): the two CTAs of a cluster form one MMA unit.  A stage then holds this CTA's activation tile and
// only its own half of the weight tile (32 KB instead of 48 KB, so the ring has six stages), nothing is multicast,
// and per 64-deep step an SM reads 32 KB of operands from its shared memory instead of 48 KB for the same flops.
template <bool PAIR> struct ClusterLayout {
    static constexpr int stages = PAIR ? 6 : CG_STAGES;
    static constexpr uint32_t a_bytes = TC_BM * TC_BK * 2;
    static constexpr uint32_t b_bytes = (PAIR ? CG_BN / 2 : CG_BN) * TC_BK * 2;
    static constexpr size_t smem = (size_t)stages * (a_bytes + b_bytes) + 2 * 16384 + (2 * stages + 4) * 8 + 16 + 1024;
};

template <int CL, bool PAIR>
__global__ void __launch_bounds__(CG_THREADS, 1)
gemm_tc_cluster_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                       const __grid_constant__ CUtensorMap map_out, TcParams p, int groups_m, int tiles_n, int bn,
                       int* __restrict__ flags) {
    // bn: columns of a tile (a multiple of 32, at most CG_BN; the host picks the width that wastes least of the last
    // round of clusters); the ring and the accumulators are laid out for CG_BN
    static_assert(!PAIR || CL == 2, "a pair is two CTAs");
    constexpr uint32_t A_BYTES = ClusterLayout<PAIR>::a_bytes;
    constexpr uint32_t B_BYTES = ClusterLayout<PAIR>::b_bytes;
    constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
    const uint32_t b_part = (uint32_t)(bn / CL) * TC_BK * 2;            // bytes of the weight rows this CTA loads
    // bytes that a stage's "full" barrier expects: as a pair, both CTAs' loads report to the even CTA's barrier
    const uint32_t stage_tx = (PAIR ? 2 * A_BYTES : A_BYTES) + (uint32_t)bn * TC_BK * 2;
    constexpr int S = ClusterLayout<PAIR>::stages;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* staging = smem + S * STAGE_BYTES;                       // 2 x [128 rows x 128 bytes], swizzled
    uint64_t* bars = reinterpret_cast<uint64_t*>(staging + 2 * 16384);
    // full[S], empty[S], acc_full[2], acc_empty[2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S + 4);
    __shared__ int abort_flag;

    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int cluster_id = blockIdx.x / CL, n_clusters = gridDim.x / CL;
    const int n_tiles = groups_m * tiles_n;
    const int n_work = n_tiles * p.splits;
    const int kb_all = (p.K + TC_BK - 1) / TC_BK;
    const int kb_part = (kb_all + p.splits - 1) / p.splits;         // k blocks per K part (the host leaves none empty)
    const uint16_t all = (uint16_t)((1u << CL) - 1);

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < S; ++s) {
            mbar_init(smem_u32(&bars[s]), 1);
            mbar_init(smem_u32(&bars[S + s]), PAIR ? 1 : CL);         // as a pair: one commit of the even CTA frees both
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&bars[2 * S + b]), 1);
            mbar_init(smem_u32(&bars[2 * S + 2 + b]), PAIR ? 2 : 128);  // as a pair: one arrival per CTA, at the even CTA
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
    }
    if (warp == 1) {
        if constexpr (PAIR) {                            // the same warp of both CTAs allocates for the pair
            tcgen05_alloc_pair(smem_u32(tmem_slot), 512);
            tcgen05_relinquish_pair();
        } else {
            tcgen05_alloc(smem_u32(tmem_slot), 512);
            tcgen05_relinquish();
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();                                  // every CTA's barriers exist before anyone signals them
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            // The weights do not depend on the kernel before this one: the ring's first lap gets its weight
            // tiles at once; the activations follow into the same stages after the dependency wait.
            int pre = 0;
            // where a stage's loads report their bytes: this CTA's barrier, as a pair the even CTA's
            auto full_of = [&](int s) -> uint32_t {
                const uint32_t local = smem_u32(&bars[s]);
                if constexpr (PAIR) return cluster_addr_of(local, 0);
                return local;
            };
            auto load_weights = [&](uint32_t sa, int kb, int tile_n, uint32_t full) {
                if constexpr (PAIR)
                    tma_load_2d_pair(sa + A_BYTES, &map_b, kb * TC_BK, tile_n * bn + (int)rank * (bn / CL), full);
                else
                    tma_load_2d_multicast(sa + A_BYTES + rank * b_part, &map_b, kb * TC_BK,
                                          tile_n * bn + (int)rank * (bn / CL), full, all);
            };
            auto load_rows = [&](uint32_t sa, int kb, int tile_m, uint32_t full) {
                if constexpr (PAIR) tma_load_2d_pair(sa, &map_a, kb * TC_BK, tile_m * TC_BM, full);
                else tma_load_2d(sa, &map_a, kb * TC_BK, tile_m * TC_BM, full);
            };
            const bool arms = !PAIR || rank == 0;        // who tells the barrier how many bytes to expect
            if (cluster_id < n_work) {
                const int tile_n = (cluster_id / groups_m) % tiles_n;
                const int kb0 = (cluster_id / n_tiles) * kb_part, kb1 = min(kb_all, kb0 + kb_part);
                pre = min(S, kb1 - kb0);
                for (int i = 0; i < pre; ++i) {
                    if (arms) mbar_expect_tx(smem_u32(&bars[i]), stage_tx);
                    load_weights(smem_u32(smem + i * STAGE_BYTES), kb0 + i, tile_n, full_of(i));
                }
            }
            pdl_wait();
            int it = 0;                                  // running k-block count across work items
            for (int w = cluster_id; w < n_work && !abort_flag; w += n_clusters) {
                const int tile_m = (w % groups_m) * CL + (int)rank, tile_n = (w / groups_m) % tiles_n;
                const int kb0 = (w / n_tiles) * kb_part, kb1 = min(kb_all, kb0 + kb_part);
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % S;
                    const uint32_t full = full_of(s);
                    const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
                    if (it < pre) {                      // armed above, the weights are on their way
                        load_rows(sa, kb, tile_m, full);
                        continue;
                    }
                    if (!mbar_wait(smem_u32(&bars[S + s]), ((it / S) & 1) ^ 1, &abort_flag)) break;
                    if (arms) mbar_expect_tx(smem_u32(&bars[s]), stage_tx);
                    load_rows(sa, kb, tile_m, full);
                    load_weights(sa, kb, tile_n, full);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && (!PAIR || rank == 0)) {          // as a pair, the even CTA issues the products of both
            const uint32_t idesc = PAIR ? make_idesc_pair(bn) : make_idesc(bn);
            int it = 0, local = 0;
            for (int w = cluster_id; w < n_work && !abort_flag; w += n_clusters, ++local) {
                const int buf = local & 1;
                if (!mbar_wait(smem_u32(&bars[2 * S + 2 + buf]), ((local >> 1) & 1) ^ 1, &abort_flag)) break;
                tcgen05_fence_after();
                const uint32_t acc = tmem_base + buf * CG_BN;
                bool ok = true;
                const int kb_total = min(kb_all, (w / n_tiles + 1) * kb_part) - (w / n_tiles) * kb_part;
                for (int kb = 0; kb < kb_total; ++kb, ++it) {
                    const int s = it % S;
                    ok = mbar_wait(smem_u32(&bars[s]), (it / S) & 1, &abort_flag);
                    if (!ok) break;
                    tcgen05_fence_after();
                    const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
                    const uint64_t da = make_smem_desc(sa), db = make_smem_desc(sa + A_BYTES);
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k) {
                        if constexpr (PAIR) tcgen05_mma_bf16_pair(acc, da + 2 * k, db + 2 * k, idesc, (kb | k) ? 1u : 0u);
                        else tcgen05_mma_bf16(acc, da + 2 * k, db + 2 * k, idesc, (kb | k) ? 1u : 0u);
                    }
                    // the stage is free in every CTA that fed it
                    if constexpr (PAIR) tcgen05_commit_pair(smem_u32(&bars[S + s]), all);
                    else tcgen05_commit_multicast(smem_u32(&bars[S + s]), all);
                }
                if (!ok) break;
                // this accumulator is complete (as a pair: both halves, and both CTAs' epilogues are told)
                if constexpr (PAIR) tcgen05_commit_pair(smem_u32(&bars[2 * S + buf]), all);
                else tcgen05_commit(smem_u32(&bars[2 * S + buf]));
            }
        }
    } else {
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;             // this thread's row of the tile
        pdl_wait();                                      // the output may still be read by the kernel before this one
        const bool leader = (warp == 2 && lane == 0);    // hands the slabs to TMA
        int local = 0, slab = 0;
        for (int w = cluster_id; w < n_work; w += n_clusters, ++local) {
            const int buf = local & 1;
            const int tile_m = (w % groups_m) * CL + (int)rank, tile_n = (w / groups_m) % tiles_n;
            const int part = w / n_tiles;                // K part: only the first one adds the bias
            const int mode = p.mode;
            const CUtensorMap* omap = &map_out;
            int* flag = flags + tile_m * tiles_n + tile_n;
            bool ordered = part == 0;                    // whether the parts before this one are known to be in
            if (!mbar_wait(smem_u32(&bars[2 * S + buf]), (local >> 1) & 1, &abort_flag)) break;
            tcgen05_fence_after();
            const uint32_t taddr = tmem_base + buf * CG_BN + ((uint32_t)(quarter * 32) << 16);
            // accumulator columns per 128-byte slab row: 32 as float, 64 as bfloat16, 128 through SwiGLU
            const int cols_per_slab = (mode == EPI_F32 || mode == EPI_RESIDUAL) ? 32 : (mode == EPI_STORE ? 64 : 128);
            // The accumulator leaves tensor memory 32 columns at a time, and the load of the next 32 is under way while
            // these are converted and written (the last tile's epilogue hides behind nothing).
            const bool with_bias = part == 0 && p.bias != nullptr;
            auto put_chunk = [&](int c, const uint32_t* r) {
                const int cc = c % cols_per_slab, c0 = c - cc;
                uint8_t* st = staging + (slab & 1) * 16384;
                if (cc == 0) {
                    // the slab before last used this buffer: TMA must have read it
                    if (leader) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                    epi_barrier();
                }
                const uint32_t srow = smem_u32(st) + row * 128;
                const int n0 = tile_n * bn + c;
                if (mode == EPI_SWIGLU) {            // 32 accumulators -> 16 bfloat16 = 2 chunks of 16 bytes
#pragma unroll
                    for (int h8 = 0; h8 < 2; ++h8) {
                        uint32_t wv[4];
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const int j = h8 * 16 + 4 * q;
                            wv[q] = pack_bf16x2(silu_fast(__uint_as_float(r[j])) * __uint_as_float(r[j + 1]),
                                                silu_fast(__uint_as_float(r[j + 2])) * __uint_as_float(r[j + 3]));
                        }
                        const int chunk = (cc >> 4) + h8;
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(srow + ((chunk ^ (row & 7)) << 4)),
                                     "r"(wv[0]), "r"(wv[1]), "r"(wv[2]), "r"(wv[3]) : "memory");
                    }
                } else {
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                    if (with_bias) add_bias_columns<32>(v, p.bias, p.bias_is_f32, n0, p.N);
                    if (mode == EPI_STORE) {         // 32 accumulators -> 4 chunks of 8 bfloat16
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const int chunk = (cc >> 3) + q;
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(srow + ((chunk ^ (row & 7)) << 4)),
                                         "r"(pack_bf16x2(v[8 * q], v[8 * q + 1])), "r"(pack_bf16x2(v[8 * q + 2], v[8 * q + 3])),
                                         "r"(pack_bf16x2(v[8 * q + 4], v[8 * q + 5])), "r"(pack_bf16x2(v[8 * q + 6], v[8 * q + 7]))
                                         : "memory");
                        }
                    } else {                         // 32 floats = the whole slab row
#pragma unroll
                        for (int q = 0; q < 8; ++q)
                            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(srow + ((q ^ (row & 7)) << 4)),
                                         "f"(v[4 * q]), "f"(v[4 * q + 1]), "f"(v[4 * q + 2]), "f"(v[4 * q + 3]) : "memory");
                    }
                }
                if (cc + 32 < cols_per_slab) return;                               // the slab is not complete yet
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");       // the slab is for TMA to read
                epi_barrier();
                if (leader) {
                    // output column of the slab's first element, in elements of the output matrix
                    const int oc0 = (mode == EPI_SWIGLU) ? (tile_n * bn + c0) / 2 : tile_n * bn + c0;
                    if (!ordered) {                      // the tile's earlier K parts must have been added
                        unsigned long long t0 = 0;
                        for (long long spin = 0; !abort_flag; ++spin) {
                            int seen;
                            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
                            if (seen >= part) { ordered = true; break; }
                            if ((spin & 63) == 63) {
                                unsigned long long now;
                                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
                                if (t0 == 0) t0 = now;
                                if (now - t0 > 2000000000ull) { abort_flag = 1; break; }
                            }
                        }
                        asm volatile("fence.proxy.async;" ::: "memory");
                    }
                    if (ordered) {
                        if (mode == EPI_RESIDUAL) tma_reduce_add_2d(omap, oc0, tile_m * TC_BM, smem_u32(st));
                        else tma_store_2d(omap, oc0, tile_m * TC_BM, smem_u32(st));
                    }
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                }
                ++slab;
            };
            {
                uint32_t ra[32], rb[32];
                tcgen05_ld32(taddr, ra);
#pragma unroll 1
                for (int c = 0; c < bn; c += 64) {
                    tcgen05_wait_ld();
                    if (c + 32 < bn) tcgen05_ld32(taddr + c + 32, rb);
                    put_chunk(c, ra);
                    if (c + 32 < bn) {
                        tcgen05_wait_ld();
                        if (c + 64 < bn) tcgen05_ld32(taddr + c + 64, ra);
                        put_chunk(c + 32, rb);
                    }
                }
            }
            tcgen05_fence_before();
            if constexpr (PAIR) {                        // one arrival per CTA at the even CTA, where the products are issued
                epi_barrier();
                if (leader) mbar_arrive_cluster(cluster_addr_of(smem_u32(&bars[2 * S + 2 + buf]), 0));
            } else {
                mbar_arrive(smem_u32(&bars[2 * S + 2 + buf]));               // 128 arrivals hand the buffer back
            }
            if (leader && p.splits > 1) {
                // this part's additions are complete in memory before the next part of the tile may start
                asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
                asm volatile("fence.proxy.async;" ::: "memory");
                __threadfence();
                if (ordered) {
                    if (part == p.splits - 1) atomicExch(flag, 0);           // ready for the next launch
                    else atomicAdd(flag, 1);
                }
            }
        }
        if (leader) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // all output has left before the CTA ends
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();                                  // no peer may still write here or signal our barriers
    if (warp == 1) {
        tcgen05_fence_after();
        if constexpr (PAIR) tcgen05_dealloc_pair(tmem_base, 512);
        else tcgen05_dealloc(tmem_base, 512);
    }
    if (threadIdx.x == 0 && abort_flag && p.status) atomicExch(p.status, 4);
}

// Map of an output matrix [rows, cols] (bfloat16 or float32, row stride ld elements); box = 128 rows x 128 bytes.
static int make_out_map(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, bool f32) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return RF_ERR_UNSUPPORTED;
    const int esz = f32 ? 4 : 2;
    if ((reinterpret_cast<uintptr_t>(base) & 15) || (ld * esz) % 16) return RF_ERR_BAD_ARG;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * esz};
    cuuint32_t box[2] = {(cuuint32_t)(128 / esz), TC_BM};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                    const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : RF_ERR_BAD_ARG;
}

template <int CL, bool PAIR>
static int cluster_width() {
    constexpr size_t smem = ClusterLayout<PAIR>::smem;
    static int max_clusters = -1;
    if (max_clusters < 0) {
        cudaLaunchConfig_t cfg = {};
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = CL; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        cfg.blockDim = dim3(CG_THREADS);
        cfg.dynamicSmemBytes = smem;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        cfg.gridDim = dim3(CL);
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_cluster_kernel<CL, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return -(int)e - 100;
        int n = 0;
        e = cudaOccupancyMaxActiveClusters(&n, gemm_tc_cluster_kernel<CL, PAIR>, &cfg);
        if (e != cudaSuccess) return -(int)e - 100;
        if (n <= 0) return RF_ERR_UNSUPPORTED;
        max_clusters = n;
    }
    return max_clusters;
}

template <int CL, bool PAIR>
static int launch_cluster(const void* X, int ldx, const void* W, TcParams p, int parts, int* flags, int n_flags,
                          cudaStream_t st) {
    constexpr size_t smem = ClusterLayout<PAIR>::smem;
    const int max_clusters = cluster_width<CL, PAIR>();
    if (max_clusters <= 0) return max_clusters < -100 ? -(max_clusters + 100) : RF_ERR_UNSUPPORTED;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CL; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.blockDim = dim3(CG_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // Tile width and K parts: the persistent clusters work in rounds, and a last round that is half empty
    // costs as much as a full one (N = 3584 in 256-column tiles on 74 clusters: 112 tiles, 1.5 rounds).  Among
    // the widths the epilogue can cut into slabs, and (residual epilogue) 1..5 K parts, take the pair with the
    // least estimated time: rounds x (blocks per part x time of a block, which goes with the bytes a CTA loads
    // for it, + 2 us per round when there are parts: their epilogues and restarts).  Parts must keep 48 blocks
    // (an epilogue, eight slabs through shared memory, hides behind the next part's products only if those
    // take longer: with parts of 19 blocks the o projection took 66 us instead of 54), the output must stay in
    // L2 (each part reads and writes it once more: 8,192 x 3,584 outputs got 18 % slower with 5 parts), and the
    // estimate must promise a twentieth, or K stays whole.  Parts are for a last round that is badly filled
    // (two or more rounds) or for a GPU that is not half used; one round that nearly fills it is left alone
    // (1,024 x 3,584 x 18,944: 152 us whole, 156 in parts).  Measured: 2,048 rows 224 -> 205 us, 512 rows 130 -> 108 us.
    const int tiles_m = (p.M + TC_BM - 1) / TC_BM, groups_m = (tiles_m + CL - 1) / CL;
    const int unit = (p.mode == EPI_F32 || p.mode == EPI_RESIDUAL) ? 32 : (p.mode == EPI_STORE ? 64 : 128);
    const int kb_all = (p.K + TC_BK - 1) / TC_BK;
    const bool parts_allowed = p.mode == EPI_RESIDUAL && flags && (long long)p.M * p.N * 4 <= (32ll << 20);
    int bn = CG_BN;
    double best = -1, best_whole = -1;
    int bn_whole = CG_BN;
    p.splits = 1;
    for (int cand = CG_BN; cand >= 128; cand -= unit) {
        const long long tiles = (long long)groups_m * ((p.N + cand - 1) / cand);
        for (int P = 1; P <= 5; ++P) {
            if (parts > 0 && P != parts) continue;                               // the caller's choice
            if (parts == 0 && P > 1 && (!parts_allowed || kb_all / P < 48)) break;
            const int per = (kb_all + P - 1) / P;
            if ((P - 1) * per >= kb_all) continue;                               // a part would be empty
            if (P > 1 && tiles * CL > n_flags) continue;
            const long long rounds = (tiles * P + max_clusters - 1) / max_clusters;
            const double cost = rounds * (per * 0.39 * (TC_BM + cand / CL) / 256.0 + (P > 1 ? 2.0 : 0.0));
            if (best < 0 || cost < best) { best = cost; bn = cand; p.splits = P; }
            if (P == 1 && (best_whole < 0 || cost < best_whole)) { best_whole = cost; bn_whole = cand; }
        }
    }
    if (best < 0) return RF_ERR_BAD_ARG;
    if (parts == 0 && p.splits > 1) {
        const long long tiles_whole = (long long)groups_m * ((p.N + CG_BN - 1) / CG_BN);       // in full-width tiles
        const bool badly_filled = tiles_whole > max_clusters || tiles_whole * 2 <= max_clusters;
        if (best > 0.95 * best_whole || !badly_filled) { p.splits = 1; bn = bn_whole; }
    }
    if (best < 0) return RF_ERR_BAD_ARG;
    if (p.splits > 1 && (p.mode != EPI_RESIDUAL || !flags)) return RF_ERR_BAD_ARG;
    CUtensorMap ma, mb, mo;
    int e;
    if ((e = make_map(&ma, X, p.M, p.K, ldx, TC_BM)) || (e = make_map(&mb, W, p.N, p.K, p.K, bn / CL))) return e;
    const bool f32_out = p.mode == EPI_F32 || p.mode == EPI_RESIDUAL;
    const long long out_cols = p.mode == EPI_SWIGLU ? p.N / 2 : p.N;
    if ((e = make_out_map(&mo, p.out, p.M, out_cols, p.ldo, f32_out))) return e;
    const int tiles_n = (p.N + bn - 1) / bn;
    int n_clusters = groups_m * tiles_n * p.splits;
    if (n_clusters > max_clusters) n_clusters = max_clusters;
    cfg.gridDim = dim3(n_clusters * CL);
    cfg.numAttrs = g_rf_pdl ? 2 : 1;
    cudaError_t le = cudaLaunchKernelEx(&cfg, gemm_tc_cluster_kernel<CL, PAIR>, ma, mb, mo, p, groups_m, tiles_n, bn, flags);
    if (le != cudaSuccess) return (int)le;
    RF_LAUNCH_CHECK();
    return 0;
}

// Whether clusters of two run as one MMA unit (cta_group::2) or as two CTAs that multicast their weight halves.
static int g_pair = 1;

extern "C" {

int rf_gemm_tc_cluster_set_pair(int on) { g_pair = on ? 1 : 0; return 0; }
int rf_gemm_tc_cluster_pair() { return g_pair; }

int rf_gemm_tc_cluster_supported(int M, int N, int K, int mode) {
    // more tokens than the skinny kernel takes: below 256 rows a cluster's second CTA works on an empty tile, which
    // still beats 14 unclustered CTAs streaming a 3,584-row weight (decode at batch 128: 8.0 ms a step without)
    if (M <= 64 || N < CG_BN || K <= 0 || K % 8) return 0;
    if (mode == EPI_SWIGLU && (N % 2)) return 0;
    if (mode == EPI_PARTIAL) return 0;
    const int out_cols = mode == EPI_SWIGLU ? N / 2 : N;
    if (out_cols % 8) return 0;                      // TMA stores need 16-byte row strides
    return encode_fn() != nullptr;
}

// Same contract as rf_gemm_tc (tokens as rows), for M > 64 and N >= 256.  cluster = 2 or 4 CTAs along M.
// parts: K parts of the residual epilogue (0 = chosen here); flags: n_flags zeroed ints that stay with the
// device between launches (the kernel leaves them zeroed), or null for no K parts.
// How many clusters of `cluster` CTAs run at once (what the persistent grid is sized to), or a negative code.
int rf_gemm_tc_cluster_width(int cluster);

int rf_gemm_tc_cluster(const void* X, int ldx, const void* W, const void* bias, int bias_is_f32, void* out, int ldo,
                       int M, int N, int K, int mode, int cluster, int parts, int* flags, int n_flags, int* status,
                       cudaStream_t st) {
    if (!rf_gemm_tc_cluster_supported(M, N, K, mode)) return RF_ERR_UNSUPPORTED;
    if (parts < 0 || parts > 5) return RF_ERR_BAD_ARG;
    TcParams p{out, bias, bias_is_f32, M, N, K, ldo, mode, (K + TC_BK - 1) / TC_BK, 0, status, 1};
    if (cluster == 2 && g_pair) return launch_cluster<2, true>(X, ldx, W, p, parts, flags, n_flags, st);
    if (cluster == 2) return launch_cluster<2, false>(X, ldx, W, p, parts, flags, n_flags, st);
    if (cluster == 4) return launch_cluster<4, false>(X, ldx, W, p, parts, flags, n_flags, st);
    return RF_ERR_BAD_ARG;
}

int rf_gemm_tc_cluster_width(int cluster) {
    if (cluster == 2 && g_pair) return cluster_width<2, true>();
    if (cluster == 2) return cluster_width<2, false>();
    if (cluster == 4) return cluster_width<4, false>();
    return RF_ERR_BAD_ARG;
}

}
