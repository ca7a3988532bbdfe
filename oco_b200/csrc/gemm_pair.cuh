// Paired tile kernel: two CTAs of a cluster (an SM pair) work on one route tile of up to 512 routes.
//
// Same product as grouped_gemm_wide_kernel (half operands, fp32 accumulators in tensor memory), with the
// operands' roles exchanged so that the expensive operand is the shared one:
//
//   * The routes are the M side. CTA r of the pair fetches, per K slice, route rows
//     [256 h + 128 r, + 128) of the tile for h = 0, 1 (TMA, as before) and owns their accumulators: its
//     128 tensor-memory lanes are routes, columns [256 h, 256 h + 256) belong to half h.
//   * The decoded weights are the N side. Per K slice each CTA decodes 128 weight rows (64 of each of
//     the item's two matrices) into its own shared memory; one thread of the even CTA issues
//     tcgen05.mma.cta_group::2 instructions of M = 256, N = 256: each SM multiplies its own routes with
//     the decoded rows of BOTH CTAs. A decoded weight row therefore serves up to 512 routes instead of
//     256, which halves the decode work per product (the decode, not the tensor pipe, bounds the
//     one-CTA kernel), and experts with 257..512 routes no longer pay a second, thinly filled tile.
//   * The sixteen producer warps form two groups of eight: group q decodes the K slices of parity q, so
//     a warp still owns 16 rows of a slice and one group's waits overlap the other's arithmetic.
//   * The epilogue reads accumulators with routes in the lanes: a thread holds consecutive features of
//     one route and writes them as 64-byte (activation) or 32-byte (bf16 output) runs of its row.
//
// Status: opt-in (OCO_MOE_PAIR_TILES=1). At the gpt-oss-20b prefill shape it measured 0.470 / 0.272 ms for
// the up / down tiles against 0.344 / 0.177 ms for grouped_gemm_wide_kernel: the decode still sets the pace, and
// a third of the M = 256 products multiply padding rows where the one-CTA kernel sizes N to the live routes.
//
// Signals that cross the pair: the TMA loads of both CTAs complete on the even CTA's `full_b` barriers;
// the MMA thread commits to the `empty` and accumulator barriers of both CTAs; in the odd CTA one
// otherwise idle thread forwards "A stage full" and "accumulators drained" to the even CTA (producer
// warps arrive on their own CTA's barriers: a remote arrival with cluster-scope release costs a warp
// far more). Every load has one destination CTA. All mbarrier waits are bounded (see mbar_wait); the two cluster
// barriers (after set-up, before the end) are reached by every thread on every path.
#pragma once
#include "gemm_wide.cuh"

namespace oco {

// ---- what crosses the pair ------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// The address, in the cluster's shared window, of CTA `rank`'s copy of this CTA's shared address.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void st_cluster_u32(uint32_t cluster_addr, uint32_t v) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// mbar_wait for a barrier on which the other CTA of the pair arrives: the same bound, cluster-scope acquire.
__device__ __forceinline__ void mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                                  uint32_t* status_word) {
    if (mbar_try_wait_cluster(bar, parity)) return;
    long long start = clock64();
    while (!mbar_try_wait_cluster(bar, parity)) {
        if (*abort_flag) return;
        if (clock64() - start > kWaitCycles) {
            *abort_flag = 1u;
            atomicExch(status_word, (uint32_t)kDevBarrierTimeout);
            return;
        }
    }
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D (256 rows: 128 in each CTA's tensor memory) += A (128 rows in each CTA) x B (N / 2 rows in each CTA)
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                              uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ uint32_t umma_idesc_f16_pair(uint32_t n) {
    return (1u << 4) | ((n >> 3) << 17) | ((256u >> 4) << 24);
}
// One arrival, when the MMAs issued so far have retired, on the barrier at `bar` of both CTAs (one instruction
// per CTA; a single instruction that signals both measured the same).
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    const uint32_t b0 = map_to_cta(bar, 0), b1 = map_to_cta(bar, 1);
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(b0) : "memory");
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(b1) : "memory");
}
// This CTA's box of route rows into its own shared memory; the bytes are counted on the barrier at `cluster_bar`
// (an address in the cluster's shared window: the even CTA's).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t smem_dst, const CUtensorMap* map, int c0, int c1, uint32_t cluster_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_dst), "l"(map), "r"(c0), "r"(c1), "r"(cluster_bar)
        : "memory");
}

template <int FMT>
struct PairShapeT {
    using W = WideShapeT<FMT>;
    static constexpr bool kSuper = W::kSuper;
    static constexpr int kMaxRoutes = 512;            // routes per tile: two halves of 256 (128 per CTA each)
    static constexpr int kProducerWarps = 16;
    static constexpr int kGroupWarps = 8;             // warps of one producer group: 8 x 16 = 128 weight rows
    static constexpr int kMmaWarp = 16, kTmaWarp = 17;
    static constexpr int kThreads = 18 * 32;
    static constexpr int kAStage = 128 * 128;         // decoded rows of one K slice: 2 matrices x 64 rows x 64 halves
    static constexpr int kAStages = 4;
    static constexpr int kBHalf = 128 * 128;          // 128 routes x 64 halves
    static constexpr int kBStage = 2 * kBHalf;
    static constexpr int kBStages = kSuper ? 2 : 3;
    static constexpr int kChunkSlices = W::kChunkSlices;
    static constexpr int kChunkBytes = W::kChunkBytes;
    static constexpr int kRowChunks = W::kRowChunks;
    static constexpr int kPitch = W::kPitch;
    static constexpr int kCopies = W::kCopies;
    static constexpr int kRingWarp = W::kRingWarp;
    static constexpr int kRing = W::kRing;
    static constexpr int kCtrl = 512 + 256 * 4 + 2 * 256 * 4;   // barriers and flags, row map of 256 routes, two bias rows
    static constexpr int kSmemBytes = kAStages * kAStage + kBStages * kBStage + kRing + kCtrl + 1024;
    static constexpr int kTmemCols = 512;
    static_assert(8 * (3 * kAStages + 2 * kBStages + 3) <= 256, "barriers fit below the flags");
    static_assert(kSmemBytes <= 232448, "shared memory of one CTA");
};

// FMT: MXFP4, Q4_0 or Q4_K. EPI as in gemm.cuh. Launched in clusters of two CTAs; persistent: pair c takes
// work items c, c + pairs, ... where an item is (route tile, feature block) with the feature block running
// fastest. A feature block is 128 features of both matrices (gated) or 256 features (one matrix, taken as
// two blocks of 128); CTA r decodes features [64 r, 64 r + 64) of each block of 128. Accumulator column
// 128 j + 64 m + i of a half holds feature 64 j + i of matrix (block) m. Tiles come from the route plan made
// with `p.tile_rows` (<= 512) routes per tile.
template <int FMT, int EPI>
__global__ void __launch_bounds__(PairShapeT<FMT>::kThreads, 1)
grouped_gemm_pair_kernel(const GemmParams p, const __grid_constant__ CUtensorMap tmap_b32,
                         const __grid_constant__ CUtensorMap tmap_b64, const __grid_constant__ CUtensorMap tmap_b128) {
    pdl_launch_dependents();   // the next kernel of the step may be set up beside this one
    pdl_wait();                // the kernel before has completed and its writes are visible
    using S = PairShapeT<FMT>;
    constexpr bool GATED = epi_gated(EPI);
    constexpr bool SUPER = S::kSuper;                                  // Q4_K: 144-byte super-blocks of four K slices
    constexpr int kBlockBytes = FMT == OCO_FMT_MXFP4 ? 17 : 18;        // the 32-element formats
    constexpr int kSliceBytes = 2 * kBlockBytes;
    constexpr int kFeatPerItem = GATED ? 128 : 256;
    extern __shared__ unsigned char smem_raw[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = cluster_rank();                              // 0: the CTA that issues the MMAs
    const int cid = (int)(blockIdx.x >> 1), ncl = (int)(gridDim.x >> 1);   // this pair, pairs in the grid

    // ---- the work list ---------------------------------------------------------------------------
    const uint32_t tile_rows = p.tile_rows;
    const int nfeat = (p.n + kFeatPerItem - 1) / kFeatPerItem;
    const int ntiles = p.tiles ? (int)*p.tile_count : (int)((p.dense_rows + tile_rows - 1) / tile_rows);
    const int total = nfeat * ntiles;
    struct Item { uint32_t expert, row0, nv; int f0; };                // f0: first feature of the item
    auto load_item = [&](int item) {
        Item r;
        const int tile = item / nfeat;
        r.f0 = (item - tile * nfeat) * kFeatPerItem;
        uint32_t begin, count;
        if (p.tiles) {
            r.expert = p.tiles[2 * tile];
            begin = p.tiles[2 * tile + 1];
            r.row0 = p.offsets[r.expert] + begin;
            count = p.offsets[r.expert + 1] - p.offsets[r.expert];
        } else {
            r.expert = 0; begin = (uint32_t)tile * tile_rows; r.row0 = begin; count = (uint32_t)p.dense_rows;
        }
        r.nv = min(tile_rows, count - begin);
        return r;
    };
    // live routes of this CTA's part of half h of a tile with nv routes
    auto live_rows = [&](uint32_t nv, uint32_t h, uint32_t r) -> uint32_t {
        const uint32_t first = 256u * h + 128u * r;
        return nv > first ? min(128u, nv - first) : 0u;
    };
    const int nkb = (p.K + 63) / 64;
    const int nblk = p.K >> 5;

    // ---- shared memory carve-up ----------------------------------------------------------------
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char* gen_base = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t a_base = base, b_base = base + S::kAStages * S::kAStage;
    const uint32_t ring_base = b_base + S::kBStages * S::kBStage;
    const uint32_t ctrl = ring_base + S::kRing;
    unsigned char* ctrl_gen = gen_base + (ctrl - base);
    auto full_a = [&](int s) { return ctrl + 8u * s; };
    auto empty_a = [&](int s) { return ctrl + 8u * (S::kAStages + s); };
    auto peer_a = [&](int s) { return ctrl + 8u * (2 * S::kAStages + s); };   // even CTA: the odd CTA's stage s is full
    auto full_b = [&](int s) { return ctrl + 8u * (3 * S::kAStages + s); };
    auto empty_b = [&](int s) { return ctrl + 8u * (3 * S::kAStages + S::kBStages + s); };
    const uint32_t accum_bar = ctrl + 8u * (3 * S::kAStages + 2 * S::kBStages);
    const uint32_t tmem_free = accum_bar + 8u;
    const uint32_t peer_free = accum_bar + 16u;                         // even CTA: the odd CTA's accumulators are drained
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ctrl_gen + 256);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    volatile uint32_t* stop_flag = tmem_slot + 2;                      // the status word as the even CTA saw it
    uint32_t* out_rows = reinterpret_cast<uint32_t*>(ctrl_gen + 512);  // [2][128]: output row of this CTA's route l of half h
    float* bias_s = reinterpret_cast<float*>(ctrl_gen + 512 + 1024);   // [2][256]: bias of accumulator column c, first / second matrix
    const uint32_t lead = map_to_cta(ctrl, 0);                         // the even CTA's control block
    auto at_lead = [&](uint32_t bar) { return lead + (bar - ctrl); };

    if (tid == 0) {
        for (int s = 0; s < S::kAStages; s++) { mbar_init(full_a(s), S::kGroupWarps); mbar_init(empty_a(s), 1); mbar_init(peer_a(s), 1); }
        for (int s = 0; s < S::kBStages; s++) { mbar_init(full_b(s), 1); mbar_init(empty_b(s), 1); }
        mbar_init(accum_bar, 1);
        mbar_init(tmem_free, S::kProducerWarps);
        mbar_init(peer_free, 1);
        *abort_flag = 0;
        fence_barrier_init();
        if (rank == 0) {       // one reading of the status word decides for the pair
            const uint32_t st = *reinterpret_cast<volatile uint32_t*>(p.status);
            st_cluster_u32(map_to_cta(smem_u32((const void*)stop_flag), 0), st);
            st_cluster_u32(map_to_cta(smem_u32((const void*)stop_flag), 1), st);
        }
    }
    if (warp == S::kMmaWarp) {
        tmem_alloc_pair(smem_u32(tmem_slot), S::kTmemCols);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();        // both CTAs' barriers exist before anything arrives on them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const bool stop = *stop_flag != 0u;

    if (stop) {
        // an earlier kernel of the step gave up: nothing runs
    } else if (warp < S::kProducerWarps) {
        // ===== producers ==========================================================================
        // Group q = warp >> 3 takes the K slices of parity q; row group rg = warp & 7 is stage rows
        // [16 rg, 16 rg + 16): matrix (block) rg >> 2, its rows 16 (rg & 3) .. of this CTA's 64.
        const int q = warp >> 3, rg = warp & 7, mat = rg >> 2;
        const uint8_t* wmat = (GATED && mat) ? p.w1 : p.w0;
        const uint8_t* w_end = (GATED && mat) ? p.w1_end : p.w0_end;
        constexpr uint32_t kChunkBytes = S::kChunkBytes;                     // packed bytes per row per buffer
        constexpr int NC = S::kCopies;
        constexpr uint32_t kBufBytes = 16 * S::kPitch;
        const uint32_t ring = ring_base + (uint32_t)warp * S::kRingWarp;
        const int nchunks = (nkb + S::kChunkSlices - 1) / S::kChunkSlices;
        // packed bytes of row r of this warp's 16 for an item
        auto row_ptr = [&](const Item& it, int r) -> const uint8_t* {
            int f = it.f0 + (GATED ? 0 : 128 * mat) + 64 * (int)rank + 16 * (rg & 3) + r;
            f = min(f, p.n - 1);
            return wmat + ((size_t)it.expert * p.n + f) * p.row_bytes;
        };
        // copy role: NC 16-byte pieces per buffer: piece index (lane + 32 i) -> (row, column)
        uint32_t cdst[NC];
        int crow[NC];
#pragma unroll
        for (int i = 0; i < NC; i++) {
            int idx = lane + 32 * i;
            crow[i] = idx / S::kRowChunks;
            cdst[i] = ring + (uint32_t)(crow[i] * S::kPitch + (idx % S::kRowChunks) * 16);
        }
        auto issue = [&](const uint8_t* const (&csrc)[NC], int chunk) {      // the K slices of ring chunk `chunk`
            if (chunk < nchunks) {
                const uint32_t bsel = (uint32_t)(chunk & 1) * kBufBytes;
#pragma unroll
                for (int i = 0; i < NC; i++) {
                    const uint8_t* a16 = (const uint8_t*)(((uintptr_t)(csrc[i] + (size_t)chunk * kChunkBytes)) & ~(uintptr_t)15) +
                                         ((cdst[i] - ring) % S::kPitch);
                    if (a16 < w_end) cp_async16(cdst[i] + bsel, a16);
                }
            }
            cp_async_commit();
        };
        // decode role: lane -> (row r = lane >> 1, half-slice h = lane & 1)
        const int r = lane >> 1, h = lane & 1;
        const int prow = 16 * rg + r;                                        // row of the 128-row stage
        const uint32_t ring_row = ring + (uint32_t)r * S::kPitch + (SUPER ? 0u : (uint32_t)h * kBlockBytes);
        const uint32_t sw = (uint32_t)(prow & 7);
        const uint32_t a_row = (uint32_t)(prow >> 3) * 1024u + (uint32_t)(prow & 7) * 128u;
        uint32_t st_off[4];
#pragma unroll
        for (int c = 0; c < 4; c++) st_off[c] = a_base + a_row + ((((uint32_t)(4 * h + c)) ^ sw) << 4);
        const bool ragged = !SUPER && (nblk & 1) != 0;                       // K is not a multiple of 64

        const uint8_t* csrc[NC];
        Item cur;
        bool started = false;                 // the first ring buffer of `cur` is already on its way
        int seq = 0;
        for (int item = cid; item < total; item += ncl, seq++) {
            if (!started) {
                cur = load_item(item);
#pragma unroll
                for (int i = 0; i < NC; i++) csrc[i] = row_ptr(cur, crow[i]);
                issue(csrc, 0);
            }
            const uint32_t a_lo = (uint32_t)(uintptr_t)row_ptr(cur, r) & 15u;   // alignment of the row start
            const int g0 = seq * nkb;                                           // slices of earlier items
            for (int chunk = 0; chunk < nchunks; chunk++) {
                issue(csrc, chunk + 1);                                          // other buffer: decoded one chunk ago
                cp_async_wait<1>();                                              // this chunk's copies have landed
                __syncwarp();
                const uint32_t rbuf = ring_row + (uint32_t)(chunk & 1) * kBufBytes + ((a_lo + (uint32_t)chunk * kChunkBytes) & 15u);
                uint32_t hdr[4];
                if (SUPER) {
                    const uint32_t a4 = rbuf & ~3u, sh = (rbuf & 3u) * 8u;
                    uint32_t w[5];
#pragma unroll
                    for (int i = 0; i < 5; i++) asm volatile("ld.shared.b32 %0, [%1];" : "=r"(w[i]) : "r"(a4 + 4u * i));
#pragma unroll
                    for (int i = 0; i < 4; i++) hdr[i] = __funnelshift_r(w[i], w[i + 1], sh);
                }
#pragma unroll
                for (int k2 = 0; k2 < S::kChunkSlices / 2; k2++) {
                    const int kk = 2 * k2 + q;                                   // this group's slices of the chunk
                    const int kb = chunk * S::kChunkSlices + kk;
                    if (kb < nkb) {
                        uint32_t v[16];
                        if (SUPER) {
                            const uint32_t at = rbuf + 16u + 32u * (uint32_t)kk + 16u * (uint32_t)h;
                            const uint32_t a4 = at & ~3u, sh = (at & 3u) * 8u;
                            uint32_t w[5], codes[4];
#pragma unroll
                            for (int i = 0; i < 5; i++) asm volatile("ld.shared.b32 %0, [%1];" : "=r"(w[i]) : "r"(a4 + 4u * i));
#pragma unroll
                            for (int i = 0; i < 4; i++) codes[i] = __funnelshift_r(w[i], w[i + 1], sh);
                            decode_q4_k_half(hdr, codes, kk, v);
                        } else {
                            const uint32_t at = rbuf + (uint32_t)kk * kSliceBytes;
                            const uint32_t a4 = at & ~3u, sh = (at & 3u) * 8u;
                            uint32_t w[6];
#pragma unroll
                            for (int i = 0; i < (FMT == OCO_FMT_MXFP4 ? 5 : 6); i++)
                                asm volatile("ld.shared.b32 %0, [%1];" : "=r"(w[i]) : "r"(a4 + 4u * i));
                            if (FMT == OCO_FMT_MXFP4) decode_mxfp4_block(w, sh, v);
                            else decode_q4_0_block(w, sh, v);
                        }
                        if (ragged && h && kb == nkb - 1) {                      // the slice's second block is past K
#pragma unroll
                            for (int i = 0; i < 16; i++) v[i] = 0;
                        }
                        const int g = g0 + kb, s = g % S::kAStages;
                        if (lane == 0) mbar_wait(empty_a(s), ((uint32_t)(g / S::kAStages) & 1u) ^ 1u, abort_flag, p.status);
                        __syncwarp();
                        const uint32_t soff = (uint32_t)s * S::kAStage;
#pragma unroll
                        for (int c = 0; c < 4; c++)
                            asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(st_off[c] + soff), "r"(v[4 * c]),
                                         "r"(v[4 * c + 1]), "r"(v[4 * c + 2]), "r"(v[4 * c + 3]) : "memory");
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(full_a(s));
                    }
                }
            }
            cp_async_wait<0>();
            // the next item's first bytes travel while this item's accumulators are drained
            const Item done = cur;
            started = item + ncl < total;
            if (started) {
                cur = load_item(item + ncl);
#pragma unroll
                for (int i = 0; i < NC; i++) csrc[i] = row_ptr(cur, crow[i]);
                issue(csrc, 0);
            }
            // ===== epilogue of `done` ================================================================
            const uint32_t nh = done.nv > 256u ? 2u : 1u;
            asm volatile("bar.sync 1, %0;" ::"n"(S::kProducerWarps * 32) : "memory");   // nobody still reads the maps of the item before
            if (tid < 256) {
                const uint32_t hh = (uint32_t)tid >> 7, l = (uint32_t)tid & 127u;
                const uint32_t ri = 256u * hh + 128u * rank + l;                // route of the tile
                if (ri < done.nv) out_rows[tid] = (EPI == kEpiDownBf16 && p.route_of_row) ? p.route_of_row[done.row0 + ri] : done.row0 + ri;
            } else {
                // accumulator column c = 128 j + 64 m + i: feature f0 + (GATED ? 0 : 128 m) + 64 j + i of matrix (block) m
                const int c = tid - 256, j = c >> 7, m = (c >> 6) & 1, i = c & 63;
                const int f = done.f0 + (GATED ? 0 : 128 * m) + 64 * j + i;
                float ba = 0.f;
                if (f < p.n) {
                    if (GATED) {
                        if (m == 0) { if (p.b0) ba = bf16_round(p.b0[((size_t)done.expert * p.n + f) * p.bias_stride]); }
                        else if (EPI == kEpiSwigluF16) ba = bf16_round(__fadd_rn(p.b1[((size_t)done.expert * p.n + f) * p.bias_stride], 1.0f));
                    } else if (p.b0) {
                        ba = bf16_round(p.b0[((size_t)done.expert * p.n + f) * p.bias_stride]);
                    }
                }
                bias_s[c] = ba;
            }
            asm volatile("bar.sync 1, %0;" ::"n"(S::kProducerWarps * 32) : "memory");
            if (lane == 0) mbar_wait(accum_bar, (uint32_t)seq & 1u, abort_flag, p.status);
            __syncwarp();
            tc_fence_after();
            // warp -> lanes 32 (warp & 3) (routes), decoded rows of CTA j = (warp >> 2) & 1, and half (two halves) or
            // feature group (one half) u2 = warp >> 3
            const uint32_t quad = (uint32_t)(warp & 3), j = (uint32_t)(warp >> 2) & 1u, u2 = (uint32_t)warp >> 3;
            const uint32_t hh = nh == 2u ? u2 : 0u;
            const uint32_t l = 32u * quad + (uint32_t)lane;
            const uint32_t ri = 256u * hh + 128u * rank + l;
            const bool live = ri < done.nv;
            const size_t orow = live ? (size_t)out_rows[128u * hh + l] * p.n : 0;
            const uint32_t taddr = tmem_base + ((32u * quad) << 16) + 256u * hh + 128u * j;
            const int fj = done.f0 + 64 * (int)j;                              // first feature of this warp's columns (matrix 0)
            const float* bias0 = bias_s + 128 * j;                              // columns 128 j + [0, 64): first matrix, + 64: second
            // Work units: GATED: two 32-feature groups u (features fj + 32 u ..): gate and up columns of the group's low
            // and high 16 (or 32) features; plain: four 16-column chunks of each block. With one half the two warps
            // that share (quad, j) split the units.
            if (GATED) {
                constexpr int SPAN = FMT == OCO_FMT_Q4_K ? 32 : 16;            // features whose codes share a byte lie SPAN apart
#pragma unroll 1
                for (uint32_t u = 0; u < 2; u++) {
                    const bool mine = nh == 2u || u == u2;
                    const uint32_t a = FMT == OCO_FMT_Q4_K ? 16u * u : 32u * u;   // low features a .. a + 15, high a + SPAN ..
                    uint32_t packed[16];
                    if (mine) {
                        uint32_t g0r[16], u0r[16], g1r[16], u1r[16];
                        tmem_ld16(taddr + a, g0r);
                        tmem_ld16(taddr + 64u + a, u0r);
                        tmem_ld16(taddr + a + SPAN, g1r);
                        tmem_ld16(taddr + 64u + a + SPAN, u1r);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 16; i++) {
                            const float ga = __fadd_rn(__uint_as_float(g0r[i]), bias0[a + i]);
                            const float ua = __fadd_rn(__uint_as_float(u0r[i]), bias0[64 + a + i]);
                            const float gb = __fadd_rn(__uint_as_float(g1r[i]), bias0[a + SPAN + i]);
                            const float ub = __fadd_rn(__uint_as_float(u1r[i]), bias0[64 + a + SPAN + i]);
                            packed[i] = (uint32_t)epilogue_value<EPI>(ga, ua) | ((uint32_t)epilogue_value<EPI>(gb, ub) << 16);
                        }
                    }
                    if ((nh == 2u && u == 1u) || (nh == 1u && u == u2)) {      // last read of this warp's columns
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(tmem_free);
                    }
                    // operand order: features a + i and a + SPAN + i sit side by side, from the position of feature a on
                    const int opos = operand_pos(FMT, fj + (int)a);
                    if (mine && live && fj + (int)a < p.n) {
                        uint16_t* dst = p.out + orow + opos;
                        if (fj + (int)a + SPAN + 16 <= p.n && (((uintptr_t)dst) & 15u) == 0) {
#pragma unroll
                            for (int v4 = 0; v4 < 4; v4++)
                                *reinterpret_cast<uint4*>(dst + 8 * v4) = make_uint4(packed[4 * v4], packed[4 * v4 + 1], packed[4 * v4 + 2], packed[4 * v4 + 3]);
                        } else {
#pragma unroll
                            for (int i = 0; i < 16; i++) {
                                if (fj + (int)a + i < p.n) dst[2 * i] = (uint16_t)(packed[i] & 0xffffu);
                                if (fj + (int)a + SPAN + i < p.n) dst[2 * i + 1] = (uint16_t)(packed[i] >> 16);
                            }
                        }
                    }
                }
            } else {
#pragma unroll 1
                for (uint32_t u = 0; u < 8; u++) {                             // chunk u: block m = u >> 2, columns 16 (u & 3) ..
                    const bool mine = nh == 2u || (u >> 2) == u2;
                    const uint32_t m = u >> 2, c0 = 16u * (u & 3u);
                    uint32_t acc[16];
                    if (mine) {
                        tmem_ld16(taddr + 64u * m + c0, acc);
                        tmem_ld_wait();
                    }
                    if ((nh == 2u && u == 7u) || (nh == 1u && u == 4u * u2 + 3u)) {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(tmem_free);
                    }
                    const int f = fj + 128 * (int)m + (int)c0;
                    if (mine && live && f < p.n) {
                        uint32_t packed[8];
#pragma unroll
                        for (int i = 0; i < 8; i++) {
                            const float x0 = __fadd_rn(__uint_as_float(acc[2 * i]), bias0[64 * m + c0 + 2 * i]);
                            const float x1 = __fadd_rn(__uint_as_float(acc[2 * i + 1]), bias0[64 * m + c0 + 2 * i + 1]);
                            packed[i] = (uint32_t)epilogue_value<EPI>(x0, 0.f) | ((uint32_t)epilogue_value<EPI>(x1, 0.f) << 16);
                        }
                        uint16_t* dst = p.out + orow + (EPI == kEpiDownBf16 ? f : operand_pos(FMT, f));
                        if (EPI == kEpiDownBf16 && f + 16 <= p.n && (((uintptr_t)dst) & 15u) == 0) {
                            *reinterpret_cast<uint4*>(dst) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                            *reinterpret_cast<uint4*>(dst + 8) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                        } else {
#pragma unroll
                            for (int i = 0; i < 16; i++) {
                                const int fi = f + i;
                                if (fi < p.n) p.out[orow + (EPI == kEpiDownBf16 ? fi : operand_pos(FMT, fi))] = (uint16_t)((packed[i >> 1] >> (16 * (i & 1))) & 0xffffu);
                            }
                        }
                    }
                }
            }
        }
    } else if (warp == S::kMmaWarp) {
        if (lane == 0 && rank == 0) {
            // ===== MMA issue ======================================================================
            const uint32_t idesc = umma_idesc_f16_pair(256u);
            int seq = 0;
            for (int item = cid; item < total; item += ncl, seq++) {
                const Item it = load_item(item);
                const uint32_t nh = it.nv > 256u ? 2u : 1u;
                if (seq > 0) {                                                // the accumulators of the item before are drained, in both CTAs
                    mbar_wait(tmem_free, (uint32_t)(seq - 1) & 1u, abort_flag, p.status);
                    mbar_wait_cluster(peer_free, (uint32_t)(seq - 1) & 1u, abort_flag, p.status);
                    tc_fence_after();
                }
                const int g0 = seq * nkb;
                for (int kb = 0; kb < nkb; kb++) {
                    const int g = g0 + kb, sa = g % S::kAStages, sb = g % S::kBStages;
                    mbar_wait(full_a(sa), (uint32_t)(g / S::kAStages) & 1u, abort_flag, p.status);
                    mbar_wait_cluster(peer_a(sa), (uint32_t)(g / S::kAStages) & 1u, abort_flag, p.status);
                    mbar_wait(full_b(sb), (uint32_t)(g / S::kBStages) & 1u, abort_flag, p.status);
                    tc_fence_after();
                    const uint64_t wdesc = umma_desc(a_base + (uint32_t)sa * S::kAStage);          // decoded rows: the N side
                    const uint64_t x0 = umma_desc(b_base + (uint32_t)sb * S::kBStage);             // routes of half 0: the M side
                    const uint64_t x1 = umma_desc(b_base + (uint32_t)sb * S::kBStage + S::kBHalf);
#pragma unroll
                    for (int kk = 0; kk < 4; kk++) {
                        const uint32_t acc = (kb | kk) != 0 ? 1u : 0u;
                        umma_f16_pair(tmem_base, x0 + 2u * kk, wdesc + 2u * kk, idesc, acc);
                        if (nh == 2u) umma_f16_pair(tmem_base + 256u, x1 + 2u * kk, wdesc + 2u * kk, idesc, acc);
                    }
                    umma_commit_pair(empty_a(sa));
                    umma_commit_pair(empty_b(sb));
                }
                umma_commit_pair(accum_bar);
            }
            if (seq > 0) mbar_wait(accum_bar, (uint32_t)(seq - 1) & 1u, abort_flag, p.status);   // every MMA has retired
            tc_fence_before();
        } else if (lane == 0) {
            // ===== odd CTA: forward "A stage full" and "accumulators drained" to the even CTA ===========
            int seq = 0;
            for (int item = cid; item < total; item += ncl, seq++) {
                if (seq > 0) {
                    mbar_wait(tmem_free, (uint32_t)(seq - 1) & 1u, abort_flag, p.status);
                    mbar_arrive_cluster(at_lead(peer_free));
                }
                const int g0 = seq * nkb;
                for (int kb = 0; kb < nkb; kb++) {
                    const int g = g0 + kb, sa = g % S::kAStages;
                    mbar_wait(full_a(sa), (uint32_t)(g / S::kAStages) & 1u, abort_flag, p.status);
                    mbar_arrive_cluster(at_lead(peer_a(sa)));
                }
            }
        }
    } else if (lane == 0) {
        // ===== route rows by TMA =====================================================================
        int seq = 0;
        for (int item = cid; item < total; item += ncl, seq++) {
            const Item it = load_item(item);
            const int g0 = seq * nkb;
            // per half: the smallest box (32, 64 or 128 rows of 64 halves) that holds this CTA's live routes
            uint32_t mine[2], bytes_all = 0;
#pragma unroll
            for (uint32_t hh = 0; hh < 2; hh++) {
                mine[hh] = live_rows(it.nv, hh, rank);
                for (uint32_t rr = 0; rr < 2; rr++) {
                    const uint32_t lv = live_rows(it.nv, hh, rr);
                    bytes_all += lv == 0 ? 0u : (lv <= 32u ? 32u : lv <= 64u ? 64u : 128u) * 128u;
                }
            }
            for (int kb = 0; kb < nkb; kb++) {
                const int g = g0 + kb, sb = g % S::kBStages;
                mbar_wait(empty_b(sb), ((uint32_t)(g / S::kBStages) & 1u) ^ 1u, abort_flag, p.status);
                if (rank == 0) mbar_arrive_expect_tx(full_b(sb), bytes_all);              // the boxes of both CTAs
#pragma unroll
                for (uint32_t hh = 0; hh < 2; hh++) {
                    if (mine[hh] == 0) continue;
                    const CUtensorMap* box = mine[hh] <= 32u ? &tmap_b32 : mine[hh] <= 64u ? &tmap_b64 : &tmap_b128;
                    tma_load_2d_pair(b_base + (uint32_t)sb * S::kBStage + hh * S::kBHalf, box, kb * 64,
                                     (int)(it.row0 + 256u * hh + 128u * rank), at_lead(full_b(sb)));
                }
            }
        }
    }
    __syncthreads();
    if (*abort_flag) {
        for (int i = 0; i < 64; i++) __nanosleep(1000);   // let copies in flight land before the CTA retires
        __syncthreads();
    }
    tc_fence_before();
    cluster_sync_all();        // neither CTA retires, or gives its tensor memory back, while the other may still signal or multiply
    if (warp == S::kMmaWarp) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, S::kTmemCols);
    }
}

}  // namespace oco
