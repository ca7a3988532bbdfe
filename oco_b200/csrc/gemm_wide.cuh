// Wide grouped tile kernel: 256 routes x 256 weight rows per work item.
//
// Same product as grouped_gemm_tc_kernel (D[feature, route] = sum_k W[feature, k] * X[row, k], half
// operands, fp32 accumulators in tensor memory), reorganised around what limits it on B200:
//
//   * Two A tiles share one B tile. Gated layers pair the gate rows with the up rows of the same
//     128 features; the down projection pairs two neighbouring 128-feature tiles. Both
//     accumulators (2 x 256 columns) fill the SM's 512 tensor-memory columns; one CTA per SM.
//   * Weight bytes are fetched coalesced. A thread-per-row load touches 32 different cache lines
//     per request and the L1 tag stage, not DRAM, becomes the limit. Here every producer warp
//     owns 16 consecutive weight rows and streams their packed bytes through a private
//     shared-memory ring with 16-byte cp.async copies, consecutive lanes taking consecutive chunks
//     of a row; each lane then decodes one 32-element block per 64-wide K slice from the ring.
//   * A and B stages are separate rings: A tiles are produced in the SM just in time, B tiles travel
//     from L2 by TMA (the smallest box that holds the tile's live routes). A dedicated warp issues
//     the TMA loads, one thread issues the MMAs, each barrier has one arrival per warp.
//   * The grid is persistent: one CTA per SM takes (route tile, feature tile) items from the list, the first by
//     its index, the following ones from a counter in global memory as it becomes free: items cost between 0.6
//     (a thinly filled tile) and 1 (a full one) of the same time, and a fixed deal leaves some CTAs with a fifth
//     more work than the average. Items are still handed out in list order, so CTAs that run at the same time
//     work on neighbouring items (one route tile's rows in L2, one expert's weight rows in DRAM pages).
//
// All waits are bounded (see mbar_wait); a wait that gives up sets the status word.
#pragma once
#include "gemm.cuh"

namespace oco {

// Per format: MXFP4 / Q4_0 rows are 32-element blocks of 17 / 18 bytes and a ring buffer holds two
// K slices of a row; a Q4_K row is 144-byte super-blocks of 256 elements and a ring buffer holds one
// super-block (four K slices), which leaves room for two A stages instead of three.
template <int FMT>
struct WideShapeT {
    static constexpr bool kSuper = FMT == OCO_FMT_Q4_K;
    static constexpr int kNT = 256;                   // routes per tile (MMA N)
    static constexpr int kProducerWarps = 16;         // 256 row streams / 16 rows per warp
    static constexpr int kMmaWarp = 16, kTmaWarp = 17;
    static constexpr int kThreads = 18 * 32;
    static constexpr int kATile = 128 * 128;          // one A tile: 128 rows x 64 halves
    static constexpr int kAStage = 2 * kATile;        // both A tiles
    static constexpr int kAStages = kSuper ? 2 : 3;
    static constexpr int kBStage = kNT * 128;
    static constexpr int kBStages = 2;
    static constexpr int kChunkSlices = kSuper ? 4 : 2;   // K slices per raw-ring buffer
    static constexpr int kChunkBytes = kSuper ? 144 : 4 * (FMT == OCO_FMT_MXFP4 ? 17 : 18);   // packed bytes of them, per row
    static constexpr int kRowChunks = (kChunkBytes + 15 + 15) / 16;   // 16-byte pieces fetched per row per buffer (any alignment)
    static constexpr int kPitch = 16 * (kRowChunks | 1);  // ring bytes per row: an odd number of pieces spreads the rows over the banks
    static constexpr int kCopies = 16 * kRowChunks / 32;  // pieces per lane per buffer
    static constexpr int kRingBufs = 2;
    static constexpr int kRingWarp = kRingBufs * 16 * kPitch;
    static constexpr int kRing = kProducerWarps * kRingWarp;
    static constexpr int kCtrl = 512 + kNT * 4;       // barriers, tmem slot, abort flag, row map
    static constexpr int kSmemBytes = kAStages * kAStage + kBStages * kBStage + kRing + kCtrl + 1024;
    static constexpr int kTmemCols = 512;
    static_assert(16 * kRowChunks % 32 == 0, "pieces of a buffer divide over the lanes");
    static_assert(kSmemBytes <= 232448, "shared memory of one CTA");
};

// FMT: MXFP4, Q4_0 or Q4_K. EPI as in gemm.cuh.
// Persistent: grid = number of SMs; CTA c takes work items c, c + grid, ... where an item is
// (route tile, feature tile) with the feature tile running fastest, so that the CTAs running at
// the same time share a route tile's B rows in L2. Barriers, tensor memory and rings are set up
// once; their phases run on across items. Between two items the producers start the next item's
// weight bytes on their way before they drain the accumulators of the finished one, and the MMA
// warp waits for the drain (`tmem_free`) before it overwrites them. `w_end`: first byte past the
// 16-byte-aligned envelope of the weight tensors (no copy starts at or beyond it).
template <int FMT, int EPI>
__global__ void __launch_bounds__(WideShapeT<FMT>::kThreads, 1)
grouped_gemm_wide_kernel(const GemmParams p, const __grid_constant__ CUtensorMap tmap_b32,
                         const __grid_constant__ CUtensorMap tmap_b64, const __grid_constant__ CUtensorMap tmap_b128,
                         const __grid_constant__ CUtensorMap tmap_b) {
    pdl_launch_dependents();   // the next kernel of the step may be set up beside this one
    pdl_wait();                // the kernel before has completed and its writes are visible
    using S = WideShapeT<FMT>;
    constexpr bool GATED = epi_gated(EPI);
    constexpr int NT = S::kNT;
    constexpr bool SUPER = S::kSuper;                                  // Q4_K: 144-byte super-blocks of four K slices
    constexpr int kBlockBytes = FMT == OCO_FMT_MXFP4 ? 17 : 18;        // the 32-element formats
    constexpr int kSliceBytes = 2 * kBlockBytes;
    constexpr int kFeatPerItem = GATED ? 128 : 256;
    extern __shared__ unsigned char smem_raw[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool dyn = p.sched != nullptr;
    // The last CTA to leave puts the two scheduling words back to zero for the next launch.
    auto leave = [&]() {
        if (dyn && tid == 0) {
            __threadfence();
            if (atomicAdd(p.sched + 1, 1u) == gridDim.x - 1) { p.sched[0] = 0u; p.sched[1] = 0u; __threadfence(); }
        }
    };
    if (__syncthreads_or(tid == 0 && *reinterpret_cast<volatile uint32_t*>(p.status) != 0u)) { leave(); return; }

    // ---- the work list ---------------------------------------------------------------------------
    const int nfeat = (p.n + kFeatPerItem - 1) / kFeatPerItem;
    const int ntiles = p.tiles ? (int)*p.tile_count : (p.dense_rows + NT - 1) / NT;
    const int total = nfeat * ntiles;
    struct Item { uint32_t expert, row0, nv; int f0; };
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
            r.expert = 0; begin = (uint32_t)tile * NT; r.row0 = begin; count = (uint32_t)p.dense_rows;
        }
        r.nv = min((uint32_t)NT, count - begin);
        return r;
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
    auto full_b = [&](int s) { return ctrl + 8u * (2 * S::kAStages + s); };
    auto empty_b = [&](int s) { return ctrl + 8u * (2 * S::kAStages + S::kBStages + s); };
    const uint32_t accum_bar = ctrl + 8u * (2 * S::kAStages + 2 * S::kBStages);
    const uint32_t tmem_free = accum_bar + 8u;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ctrl_gen + 128);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    // item of step `seq` of this CTA: slot seq & 1, published by lane 0 of producer warp 0 (one arrival on item_full)
    volatile uint32_t* item_slot = tmem_slot + 4;
    auto item_full = [&](int q) { return ctrl + 8u * (2 * S::kAStages + 2 * S::kBStages + 2 + q); };
    // read by one thread of a role: waits for the item of step seq; the end of the list once a wait has given up
    auto item_of = [&](int seq) -> int {
        mbar_wait(item_full(seq & 1), (uint32_t)(seq >> 1) & 1u, abort_flag, p.status);
        return *abort_flag ? total : (int)item_slot[seq & 1];
    };
    uint32_t* out_rows = reinterpret_cast<uint32_t*>(ctrl_gen + 512);

    if (tid == 0) {
        for (int s = 0; s < S::kAStages; s++) { mbar_init(full_a(s), S::kProducerWarps); mbar_init(empty_a(s), 1); }
        for (int s = 0; s < S::kBStages; s++) { mbar_init(full_b(s), 1); mbar_init(empty_b(s), 1); }
        mbar_init(accum_bar, 1);
        mbar_init(tmem_free, S::kProducerWarps);
        mbar_init(item_full(0), 1); mbar_init(item_full(1), 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == S::kMmaWarp) {
        tmem_alloc(smem_u32(tmem_slot), S::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < S::kProducerWarps) {
        // ===== producers ==========================================================================
        // Row stream rs = 16 * warp + r: A tile (rs >> 7), tile row (rs & 127).
        const int tile = warp >> 3;                                  // which A tile this warp feeds
        const uint8_t* wmat = (GATED && tile) ? p.w1 : p.w0;
        const int trow0 = (warp & 7) * 16;                           // first tile row of this warp
        const uint8_t* w_end = (GATED && tile) ? p.w1_end : p.w0_end;
        constexpr uint32_t kChunkBytes = S::kChunkBytes;                     // packed bytes per row per buffer
        constexpr int NC = S::kCopies;
        constexpr uint32_t kBufBytes = 16 * S::kPitch;
        const uint32_t ring = ring_base + (uint32_t)warp * S::kRingWarp;
        const int nchunks = (nkb + S::kChunkSlices - 1) / S::kChunkSlices;
        // packed bytes of tile row trow0 + r of an item
        auto row_ptr = [&](const Item& it, int r) -> const uint8_t* {
            const int feat0 = GATED ? it.f0 : it.f0 + 128 * tile;
            int f = min(feat0 + trow0 + r, p.n - 1);
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
                    // 16-byte-aligned envelope of the row's bytes for this chunk, column (cdst offset)
                    const uint8_t* a16 = (const uint8_t*)(((uintptr_t)(csrc[i] + (size_t)chunk * kChunkBytes)) & ~(uintptr_t)15) +
                                         ((cdst[i] - ring) % S::kPitch);
                    if (a16 < w_end) cp_async16(cdst[i] + bsel, a16);
                }
            }
            cp_async_commit();
        };
        // decode role: lane -> (row r = lane >> 1, half-slice h = lane & 1)
        const int r = lane >> 1, h = lane & 1;
        const int prow = trow0 + r;
        const uint32_t ring_row = ring + (uint32_t)r * S::kPitch + (SUPER ? 0u : (uint32_t)h * kBlockBytes);
        const uint32_t sw = (uint32_t)(prow & 7);
        const uint32_t a_row = (uint32_t)tile * S::kATile + (uint32_t)(prow >> 3) * 1024u + (uint32_t)(prow & 7) * 128u;
        uint32_t st_off[4];
#pragma unroll
        for (int c = 0; c < 4; c++) st_off[c] = a_base + a_row + ((((uint32_t)(4 * h + c)) ^ sw) << 4);
        const bool ragged = !SUPER && (nblk & 1) != 0;                       // K is not a multiple of 64
        // epilogue role: warp -> tensor-memory lanes 32 * (warp & 3) (tile rows), columns [64 * (warp >> 2), +64)
        const int erow = (warp & 3) * 32 + lane;
        const uint32_t taddr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
        const uint32_t c_begin = (uint32_t)(warp >> 2) * 64u;

        const uint8_t* csrc[NC];
        Item cur;
        bool started = false;                 // the first ring buffer of `cur` is already on its way
        int seq = 0;
        const bool fetcher = warp == 0 && lane == 0;
        if (fetcher) { item_slot[0] = blockIdx.x; mbar_arrive(item_full(0)); }
        // the chunk during which the fetcher asks for the CTA's next item: late, so that a CTA holds no item it
        // will not start soon, yet a few slices before the end, so that the answer is there when the item ends
        const int fetch_chunk = max(0, nchunks - 4);
        uint32_t fetched = 0;
        int next = 0;
        for (int item = blockIdx.x; item < total; item = next, seq++) {
            if (!started) {
                cur = load_item(item);
#pragma unroll
                for (int i = 0; i < NC; i++) csrc[i] = row_ptr(cur, crow[i]);
                issue(csrc, 0);
            }
            const uint32_t a_lo = (uint32_t)(uintptr_t)row_ptr(cur, r) & 15u;   // alignment of the row start
            const int g0 = seq * nkb;                                           // slices of earlier items
            for (int chunk = 0; chunk < nchunks; chunk++) {
                if (fetcher) {
                    if (chunk == fetch_chunk) fetched = dyn ? gridDim.x + atomicAdd(p.sched, 1u) : (uint32_t)item + gridDim.x;
                    if (chunk == min(fetch_chunk + 2, nchunks - 1)) {
                        item_slot[(seq + 1) & 1] = min(fetched, (uint32_t)total);
                        mbar_arrive(item_full((seq + 1) & 1));
                    }
                }
                issue(csrc, chunk + 1);                                          // other buffer: decoded one chunk ago
                cp_async_wait<1>();                                              // this chunk's copies have landed
                __syncwarp();
                // the row's bytes for this chunk start ((a_lo + chunk * kChunkBytes) & 15) into its ring slot
                const uint32_t rbuf = ring_row + (uint32_t)(chunk & 1) * kBufBytes + ((a_lo + (uint32_t)chunk * kChunkBytes) & 15u);
                // Q4_K: the super-block's header (d, dmin, twelve scale bytes) serves its four slices
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
                for (int kk = 0; kk < S::kChunkSlices; kk++) {
                    const int kb = chunk * S::kChunkSlices + kk;
                    if (kb < nkb) {
                        uint32_t v[16];
                        if (SUPER) {
                            // code bytes 16 h .. 16 h + 15 of the slice's sub-block pair
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
            if (lane == 0) next = item_of(seq + 1);
            next = __shfl_sync(0xffffffffu, next, 0);
            started = next < total;
            if (started) {
                cur = load_item(next);
#pragma unroll
                for (int i = 0; i < NC; i++) csrc[i] = row_ptr(cur, crow[i]);
                issue(csrc, 0);
            }
            // ===== epilogue of `done` ================================================================
            asm volatile("bar.sync 1, %0;" ::"n"(S::kProducerWarps * 32) : "memory");                    // nobody still reads the row map of the item before
            for (uint32_t i = tid; i < done.nv; i += S::kProducerWarps * 32)
                out_rows[i] = (EPI == kEpiDownBf16 && p.route_of_row) ? p.route_of_row[done.row0 + i] : done.row0 + i;
            asm volatile("bar.sync 1, %0;" ::"n"(S::kProducerWarps * 32) : "memory");
            if (lane == 0) mbar_wait(accum_bar, (uint32_t)seq & 1u, abort_flag, p.status);
            __syncwarp();
            tc_fence_after();
            const uint32_t c_end = min(done.nv, c_begin + 64u);
            const int fa = done.f0 + erow, fb = GATED ? fa : fa + 128;        // features of accumulator 0 / 1
            float bias_a = 0.f, bias_b = 0.f;
            if (fa < p.n && p.b0) bias_a = bf16_round(p.b0[((size_t)done.expert * p.n + fa) * p.bias_stride]);
            if (GATED) {
                if (EPI == kEpiSwigluF16 && fa < p.n) bias_b = bf16_round(__fadd_rn(p.b1[((size_t)done.expert * p.n + fa) * p.bias_stride], 1.0f));
            } else if (fb < p.n && p.b0) {
                bias_b = bf16_round(p.b0[((size_t)done.expert * p.n + fb) * p.bias_stride]);
            }
            const int col_a = EPI == kEpiDownBf16 ? fa : operand_pos(FMT, fa);
            const int col_b = EPI == kEpiDownBf16 ? fb : operand_pos(FMT, fb);
            for (uint32_t c = c_begin; c < c_end; c += 16) {
                uint32_t ra[16], rb[16];
                tmem_ld16(taddr + c, ra);
                tmem_ld16(taddr + NT + c, rb);
                tmem_ld_wait();
                if (c + 16 >= c_end) {                                        // last read of this warp's columns:
                    tc_fence_before();                                        // the MMA warp may overwrite them while
                    __syncwarp();                                             // the values are finished in registers
                    if (lane == 0) mbar_arrive(tmem_free);
                }
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    if (c + j < done.nv) {
                        const size_t orow = (size_t)out_rows[c + j] * p.n;
                        const float a = __fadd_rn(__uint_as_float(ra[j]), bias_a);
                        const float b = __fadd_rn(__uint_as_float(rb[j]), bias_b);
                        if (GATED) {
                            if (fa < p.n) p.out[orow + col_a] = epilogue_value<EPI>(a, b);
                        } else {
                            if (fa < p.n) p.out[orow + col_a] = epilogue_value<EPI>(a, 0.f);
                            if (fb < p.n) p.out[orow + col_b] = epilogue_value<EPI>(b, 0.f);
                        }
                    }
                }
            }
            if (c_begin >= c_end) {                                           // no live column in this warp's range
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tmem_free);
            }
        }
    } else if (warp == S::kMmaWarp) {
        if (lane == 0) {
            // ===== MMA issue ======================================================================
            int seq = 0;
            for (int item = item_of(0); item < total; item = item_of(++seq)) {
                const Item it = load_item(item);
                const uint32_t n_mma = max(16u, (it.nv + 15u) & ~15u);
                const uint32_t idesc = umma_idesc_f16(n_mma);
                if (seq > 0) {                                                // the accumulators of the item before are drained
                    mbar_wait(tmem_free, (uint32_t)(seq - 1) & 1u, abort_flag, p.status);
                    tc_fence_after();
                }
                const int g0 = seq * nkb;
                for (int kb = 0; kb < nkb; kb++) {
                    const int g = g0 + kb, sa = g % S::kAStages, sb = g % S::kBStages;
                    mbar_wait(full_a(sa), (uint32_t)(g / S::kAStages) & 1u, abort_flag, p.status);
                    mbar_wait(full_b(sb), (uint32_t)(g / S::kBStages) & 1u, abort_flag, p.status);
                    tc_fence_after();
                    const uint32_t a_stage = a_base + (uint32_t)sa * S::kAStage;
                    const uint64_t a0 = umma_desc(a_stage), a1 = umma_desc(a_stage + S::kATile);
                    const uint64_t b = umma_desc(b_base + (uint32_t)sb * S::kBStage);
#pragma unroll
                    for (int kk = 0; kk < 4; kk++) {
                        const uint32_t acc = (kb | kk) != 0 ? 1u : 0u;
                        umma_f16(tmem_base, a0 + 2u * kk, b + 2u * kk, idesc, acc);
                        umma_f16(tmem_base + NT, a1 + 2u * kk, b + 2u * kk, idesc, acc);
                    }
                    umma_commit(empty_a(sa));
                    umma_commit(empty_b(sb));
                }
                umma_commit(accum_bar);
            }
            if (seq > 0) mbar_wait(accum_bar, (uint32_t)(seq - 1) & 1u, abort_flag, p.status);   // every MMA has retired
            tc_fence_before();
        }
    } else if (lane == 0) {
        // ===== B tiles by TMA =========================================================================
        int seq = 0;
        for (int item = item_of(0); item < total; item = item_of(++seq)) {
            const Item it = load_item(item);
            const int g0 = seq * nkb;
            // the smallest box (32, 64, 128 or 256 rows of 64 halves) that holds the tile's live rows
            const CUtensorMap* box = it.nv <= 32 ? &tmap_b32 : it.nv <= 64 ? &tmap_b64 : it.nv <= 128 ? &tmap_b128 : &tmap_b;
            const uint32_t box_bytes = (it.nv <= 32 ? 32u : it.nv <= 64 ? 64u : it.nv <= 128 ? 128u : 256u) * 128u;
            for (int kb = 0; kb < nkb; kb++) {
                const int g = g0 + kb, sb = g % S::kBStages;
                mbar_wait(empty_b(sb), ((uint32_t)(g / S::kBStages) & 1u) ^ 1u, abort_flag, p.status);
                mbar_arrive_expect_tx(full_b(sb), box_bytes);
                tma_load_2d(b_base + (uint32_t)sb * S::kBStage, box, kb * 64, (int)it.row0, full_b(sb));
            }
        }
    }
    __syncthreads();
    if (*abort_flag) {
        for (int i = 0; i < 64; i++) __nanosleep(1000);   // let copies in flight land before the CTA retires
        __syncthreads();
    }
    if (warp == S::kMmaWarp) {
        tc_fence_after();
        tmem_dealloc(tmem_base, S::kTmemCols);
    }
    leave();
}

}  // namespace oco
