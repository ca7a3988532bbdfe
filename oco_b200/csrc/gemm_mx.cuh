// Grouped expert products for many tokens on the block-scaled tensor-core path: tcgen05.mma
// kind::mxf4 with UE8M0 scales per 32 elements, fp32 accumulators in tensor memory.
//
// An opt-in numerics mode (oco_moe_desc.numerics = 2), not the reference's arithmetic: the reference
// multiplies half weights with half activations (shaders/experts/projections.metal:192-346); here the
// MXFP4 weights enter the MMA exactly as the GGUF file holds them (e2m1 codes and E8M0 scales: nothing is
// decoded or rounded) and the ACTIVATIONS are quantised to MXFP4 as well, one UE8M0 scale per 32
// elements (mx_quantize_kernel), which is what costs accuracy. In exchange the MMA runs at four times
// the f16 rate and the producers only move bytes.
//
//   * A work item is one 128-route tile of an expert x 128 features x two weight tiles that share the B
//     tile (gate and up rows of the same features, or two neighbouring feature tiles of the down
//     projection): two accumulators of 128 columns.
//   * 16 producer warps: warp w feeds matrix w / 8 with the weight rows of class c = w mod 8, rows f0 + c + 8 i
//     (rows eight apart start at the same byte of a 16-byte word, so one warp's sixteen rows need the same
//     shifts); they are the tile rows 16 c + i, consecutive, so that the lanes' 16-byte stores into the
//     swizzled tile fall into distinct banks. Each warp streams its rows' packed bytes through a private ring
//     (16-byte cp.async, consecutive lanes taking consecutive pieces of a row, one K group of 256 elements per
//     stage) and moves every block's sixteen code bytes into the K-major 128-byte-swizzled A tile and its
//     scale byte into the scale tile (mx_move_row, mx.cuh). (Loading through registers one step ahead and
//     storing to the ring measured slower: 0.38 against 0.29 ms for the up tiles of the 20b-shaped prefill.)
//   * B tiles (quantised activation rows, 128 bytes = 256 e2m1 per row and K group) arrive by TMA, their
//     scales as one 1 KB bulk copy per K group: the quantiser wrote them in the layout tcgen05.cp wants.
//   * One thread issues per K group: the scale copies into tensor memory, then 4 MMAs (K = 64) per tile.
//   * The producer warps drain the accumulators (bias, activation, store) as in the f16 tile kernels.
// Persistent grid, bounded waits (mbar_wait), no multicast.
#pragma once
#include "gemm.cuh"
#include "mx.cuh"

namespace oco {

struct MxGemmShape {
    static constexpr int kNT = 128;                   // routes per tile (MMA N)
    static constexpr int kProducerWarps = 16;
    static constexpr int kMmaWarp = 16, kTmaWarp = 17;
    static constexpr int kThreads = 18 * 32;
    static constexpr int kATile = 128 * 128;          // 128 rows x 128 bytes (256 e2m1)
    static constexpr int kAStage = 2 * kATile + 2 * 1024;   // both A tiles, then their scale tiles (two 512-byte tiles each)
    static constexpr int kAStages = 3;
    static constexpr int kBStage = kNT * 128 + 1024;  // the B tile, then its scales
    static constexpr int kBStages = 2;
    static constexpr int kRingStages = 2;
    static constexpr int kRingWarp = kRingStages * 16 * kMxSlot;
    static constexpr int kRing = kProducerWarps * kRingWarp;
    static constexpr int kCtrl = 512 + kNT * 4;       // barriers, tmem slot, abort flag, row map
    static constexpr int kSmemBytes = kAStages * kAStage + kBStages * kBStage + kRing + kCtrl + 1024;
    static constexpr int kTmemCols = 512;
    static constexpr int kColSfa = 256, kColSfb = 320;
    static_assert(kSmemBytes <= 232448, "shared memory of one CTA");
};

// MXFP4 quantiser of activation rows for the block-scaled tile kernel. One CTA per route tile; a thread
// takes one block of 32 values of one row: scale 2^e with the smallest e such that 6 * 2^e >= max |v|
// (no clipping), codes rounded to nearest even, packed two per byte in the tiles' operand order, and
// the scale byte written where tcgen05.cp expects it: tile t, K group g, 512-byte tile (blk >> 2) & 1,
// byte (n & 31) * 16 + (n >> 5) * 4 + (blk & 3) for row n of the tile.
//   GATHER: rows are token rows (bf16, element order), row n of the tile is token route_of_row[..] / per_row;
//   else rows are the expert-sorted half rows the up kernel wrote (already in operand order).
template <bool GATHER>
__global__ void __launch_bounds__(256) mx_quantize_kernel(const uint16_t* __restrict__ src, const uint32_t* __restrict__ tiles,
                                                          const uint32_t* __restrict__ tile_count, const uint32_t* __restrict__ offsets,
                                                          const uint32_t* __restrict__ route_of_row, int per_row, int K,
                                                          unsigned char* __restrict__ q, unsigned char* __restrict__ sf, uint32_t tile_rows) {
    // four CTAs per tile, 32 rows each (gridDim.x = 4 x the tiles the launch was sized for)
    const uint32_t tile = blockIdx.x >> 2, part = blockIdx.x & 3u;
    if (tile >= *tile_count) return;
    const uint32_t expert = tiles[2 * tile], begin = tiles[2 * tile + 1];
    const uint32_t row0 = offsets[expert] + begin;
    const uint32_t nv = min(tile_rows, offsets[expert + 1] - offsets[expert] - begin);       // tile_rows <= 128
    const int nkb = K >> 5, nkg = (nkb + 7) >> 3, nblk = nkg * 8;
    for (uint32_t i = threadIdx.x; i < 32u * (uint32_t)nblk; i += 256) {
        const uint32_t n = part * 32u + i / (uint32_t)nblk, blk = i % (uint32_t)nblk;
        unsigned char* sfp = sf + ((size_t)tile * nkg + (blk >> 3)) * 1024 + ((blk >> 2) & 1u) * 512 + (n & 31u) * 16 + (n >> 5) * 4 + (blk & 3u);
        if (n >= nv || blk >= (uint32_t)nkb) { *sfp = 127; continue; }    // rows and blocks past the end: operand zeros, scale one
        const uint16_t* row = GATHER ? src + (size_t)(route_of_row[row0 + n] / (uint32_t)per_row) * K : src + (size_t)(row0 + n) * K;
        float v[32];
        const uint4* p4 = reinterpret_cast<const uint4*>(row + blk * 32);
#pragma unroll
        for (int c = 0; c < 4; c++) {
            const uint4 w = p4[c];
            const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int k = 0; k < 4; k++) {
                if (GATHER) {
                    v[8 * c + 2 * k] = bf16_bits_to_f32((uint16_t)(ws[k] & 0xffffu));
                    v[8 * c + 2 * k + 1] = bf16_bits_to_f32((uint16_t)(ws[k] >> 16));
                } else {
                    v[8 * c + 2 * k] = f16_bits_to_f32((uint16_t)(ws[k] & 0xffffu));
                    v[8 * c + 2 * k + 1] = f16_bits_to_f32((uint16_t)(ws[k] >> 16));
                }
            }
        }
        float amax = 0.f;
        bool bad = false;
#pragma unroll
        for (int k = 0; k < 32; k++) { amax = fmaxf(amax, fabsf(v[k])); bad |= nonfinite(v[k]); }
        const uint32_t ab = __float_as_uint(amax);
        int s0 = (int)((ab >> 23) & 0xffu) - 2 + ((ab & 0x7fffffu) > 0x400000u ? 1 : 0);
        s0 = max(0, min(254, s0));
        const float inv = __uint_as_float(s0 >= 254 ? 0x00400000u : (uint32_t)(254 - s0) << 23);
        uint32_t words[4];
#pragma unroll
        for (int c = 0; c < 4; c++) {
            uint32_t w = 0;
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const int j = 4 * c + k;                 // byte j: operand positions 2j, 2j + 1
                // element order (token rows): positions 2j, 2j + 1 are elements j, j + 16; operand order: 2j, 2j + 1
                const float lo = GATHER ? v[j] : v[2 * j], hi = GATHER ? v[j + 16] : v[2 * j + 1];
                const uint32_t b = (uint32_t)__nv_cvt_float2_to_fp4x2(make_float2(__fmul_rn(lo, inv), __fmul_rn(hi, inv)), __NV_E2M1, cudaRoundNearest);
                w |= (b & 0xffu) << (8 * k);
            }
            words[c] = w;
        }
        *reinterpret_cast<uint4*>(q + (size_t)(row0 + n) * (K / 2) + blk * 16) = make_uint4(words[0], words[1], words[2], words[3]);
        *sfp = (unsigned char)(bad ? 255 : s0);
    }
}

// EPI as in gemm.cuh. `tmap_b`: the quantised activation rows as bytes [rows][K / 2], box 128 bytes x 128 rows,
// 128-byte swizzle. p.sfb: the scale tiles the quantiser wrote. p.xs is unused.
template <int EPI>
__global__ void __launch_bounds__(MxGemmShape::kThreads, 1)
grouped_gemm_mx_kernel(const GemmParams p, const __grid_constant__ CUtensorMap tmap_b) {
    using S = MxGemmShape;
    constexpr bool GATED = epi_gated(EPI);
    constexpr int NT = S::kNT;
    constexpr int kFeatPerItem = GATED ? 128 : 256;
    extern __shared__ unsigned char smem_raw[];
    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    if (__syncthreads_or(tid == 0 && *reinterpret_cast<volatile uint32_t*>(p.status) != 0u)) return;

    // ---- the work list ---------------------------------------------------------------------------
    const int nfeat = (p.n + kFeatPerItem - 1) / kFeatPerItem;
    const int ntiles = (int)*p.tile_count;
    const int total = nfeat * ntiles;
    struct Item { uint32_t expert, row0, nv; int f0, tile; };
    auto load_item = [&](int item) {
        Item r;
        r.tile = item / nfeat;
        r.f0 = (item - r.tile * nfeat) * kFeatPerItem;
        r.expert = p.tiles[2 * r.tile];
        const uint32_t begin = p.tiles[2 * r.tile + 1];
        r.row0 = p.offsets[r.expert] + begin;
        r.nv = min((uint32_t)NT, p.offsets[r.expert + 1] - p.offsets[r.expert] - begin);
        return r;
    };
    const int nkb = p.K >> 5, nkg = (nkb + 7) >> 3;

    // ---- shared memory carve-up ----------------------------------------------------------------
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char* gen = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t a_base = base, b_base = base + S::kAStages * S::kAStage;
    const uint32_t ring_base = b_base + S::kBStages * S::kBStage;
    const uint32_t ctrl = ring_base + S::kRing;
    unsigned char* ctrl_gen = gen + (ctrl - base);
    auto full_a = [&](int s) { return ctrl + 8u * s; };
    auto empty_a = [&](int s) { return ctrl + 8u * (S::kAStages + s); };
    auto full_b = [&](int s) { return ctrl + 8u * (2 * S::kAStages + s); };
    auto empty_b = [&](int s) { return ctrl + 8u * (2 * S::kAStages + S::kBStages + s); };
    const uint32_t accum_bar = ctrl + 8u * (2 * S::kAStages + 2 * S::kBStages);
    const uint32_t tmem_free = accum_bar + 8u;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ctrl_gen + 128);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    uint32_t* out_rows = reinterpret_cast<uint32_t*>(ctrl_gen + 512);

    if (tid == 0) {
        for (int s = 0; s < S::kAStages; s++) { mbar_init(full_a(s), S::kProducerWarps); mbar_init(empty_a(s), 1); }
        for (int s = 0; s < S::kBStages; s++) { mbar_init(full_b(s), 1); mbar_init(empty_b(s), 1); }
        mbar_init(accum_bar, 1);
        mbar_init(tmem_free, S::kProducerWarps);
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
        const int mat = warp >> 3, cls = warp & 7;
        const uint8_t* wmat = (GATED && mat) ? p.w1 : p.w0;
        const uint8_t* w_end = (GATED && mat) ? p.w1_end : p.w0_end;
        const uint32_t ring = ring_base + (uint32_t)warp * S::kRingWarp;
        const unsigned char* ring_gen = gen + (ring - base);
        // packed bytes of the row with offset d (0..127) from the item's first feature
        auto row_ptr = [&](const Item& it, int d) -> const uint8_t* {
            const int feat0 = GATED ? it.f0 : it.f0 + 128 * mat;
            const int f = min(feat0 + d, p.n - 1);
            return wmat + ((size_t)it.expert * p.n + f) * p.row_bytes;
        };
        // move role: lane i < 16 moves the row with offset cls + 8 i into tile row 16 cls + i
        const int t = 16 * cls + (lane & 15), doff = cls + 8 * (lane & 15);
        const uint32_t a_off = (uint32_t)mat * S::kATile + (uint32_t)(t >> 3) * 1024u + (uint32_t)(t & 7) * 128u, sw = (uint32_t)(t & 7) << 4;
        const uint32_t sf_off = 2u * S::kATile + (uint32_t)mat * 1024u + (uint32_t)(t & 31) * 16u + (uint32_t)(t >> 5) * 4u;
        // epilogue role: warp -> tensor-memory lanes 32 * (warp & 3) (tile rows), columns [32 * (warp >> 2), +32);
        // tile row L holds the feature with offset (L >> 4) + 8 * (L & 15)
        const int etile = (warp & 3) * 32 + lane, erow = (etile >> 4) + 8 * (etile & 15);
        const uint32_t taddr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
        const uint32_t c_begin = (uint32_t)(warp >> 2) * 32u;

        // fetch role: 160 pieces per stage, piece (lane + 32 k) -> row i = / 10, piece % 10
        const uint8_t* row16[5];
        uint32_t fdst[5], r15[5];
        auto prepare = [&](const Item& it) {
#pragma unroll
            for (int k = 0; k < 5; k++) {
                const int idx = lane + 32 * k, ri = idx / kMxPiecesPerRow, piece = idx - ri * kMxPiecesPerRow;
                const uint8_t* rp = row_ptr(it, cls + 8 * ri);
                row16[k] = (const uint8_t*)((uintptr_t)rp & ~(uintptr_t)15) + piece * 16;
                r15[k] = (uint32_t)((uintptr_t)rp & 15u);
                fdst[k] = (uint32_t)(ri * kMxSlot + piece * 16);
            }
        };
        auto issue = [&](int g, int slice) {             // K group g of the prepared item into ring stage slice % 2
            if (g < nkg) {
                const uint32_t st = ring + (uint32_t)(slice % S::kRingStages) * (16 * kMxSlot);
#pragma unroll
                for (int k = 0; k < 5; k++) {
                    const uint8_t* a16 = row16[k] + ((r15[k] + (uint32_t)g * kMxGroupBytes) & ~15u);
                    if (a16 < w_end) cp_async16(st + fdst[k], a16);
                }
            }
            cp_async_commit();
        };

        Item cur;
        bool started = false;                 // the first ring stage of `cur` is already on its way
        int seq = 0;
        for (int item = blockIdx.x; item < total; item += gridDim.x, seq++) {
            if (!started) {
                cur = load_item(item);
                prepare(cur);
                issue(0, seq * nkg);
            }
            const uint8_t* mrow = row_ptr(cur, doff);
            const int g0 = seq * nkg;
            for (int g = 0; g < nkg; g++) {
                const int G = g0 + g, sa = G % S::kAStages;
                issue(g + 1, G + 1);                                             // other ring stage: moved one step ago
                cp_async_wait<1>();                                              // this K group has landed
                if (lane == 0) mbar_wait(empty_a(sa), ((uint32_t)(G / S::kAStages) & 1u) ^ 1u, abort_flag, p.status);
                __syncwarp();
                const uint32_t dl = (uint32_t)((uintptr_t)(mrow + (size_t)g * kMxGroupBytes) & 15u);
                const uint32_t dl_first = __shfl_sync(0xffffffffu, dl, 0);
                const bool same = __all_sync(0xffffffffu, lane >= 16 || dl == dl_first);
                if (lane < 16) {
                    const unsigned char* slot = ring_gen + (size_t)(G % S::kRingStages) * (16 * kMxSlot) + lane * kMxSlot;
                    unsigned char* stage = gen + (size_t)sa * S::kAStage;
                    const int nb = min(8, nkb - g * 8);
                    uint32_t c[40];
#pragma unroll
                    for (int i = 0; i < 10; i++) {
                        const uint4 v = *reinterpret_cast<const uint4*>(slot + 16 * i);
                        c[4 * i] = v.x; c[4 * i + 1] = v.y; c[4 * i + 2] = v.z; c[4 * i + 3] = v.w;
                    }
                    unsigned char* a_row = stage + a_off;
                    unsigned char* sf_dst = stage + sf_off;
                    if (same && nb == 8) {
                        switch (dl) {
                            case 0: mx_move_row<0>(c, a_row, sw, sf_dst); break;
                            case 1: mx_move_row<1>(c, a_row, sw, sf_dst); break;
                            case 2: mx_move_row<2>(c, a_row, sw, sf_dst); break;
                            case 3: mx_move_row<3>(c, a_row, sw, sf_dst); break;
                            case 4: mx_move_row<4>(c, a_row, sw, sf_dst); break;
                            case 5: mx_move_row<5>(c, a_row, sw, sf_dst); break;
                            case 6: mx_move_row<6>(c, a_row, sw, sf_dst); break;
                            case 7: mx_move_row<7>(c, a_row, sw, sf_dst); break;
                            case 8: mx_move_row<8>(c, a_row, sw, sf_dst); break;
                            case 9: mx_move_row<9>(c, a_row, sw, sf_dst); break;
                            case 10: mx_move_row<10>(c, a_row, sw, sf_dst); break;
                            case 11: mx_move_row<11>(c, a_row, sw, sf_dst); break;
                            case 12: mx_move_row<12>(c, a_row, sw, sf_dst); break;
                            case 13: mx_move_row<13>(c, a_row, sw, sf_dst); break;
                            case 14: mx_move_row<14>(c, a_row, sw, sf_dst); break;
                            default: mx_move_row<15>(c, a_row, sw, sf_dst); break;
                        }
                    } else {
                        mx_move_row_any(dl, c, a_row, sw, sf_dst, nb);
                    }
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(full_a(sa));
            }
            cp_async_wait<0>();
            // the next item's first bytes travel while this item's accumulators are drained
            const Item done = cur;
            started = item + (int)gridDim.x < total;
            if (started) {
                cur = load_item(item + gridDim.x);
                prepare(cur);
                issue(0, (seq + 1) * nkg);
            }
            // ===== epilogue of `done` ================================================================
            asm volatile("bar.sync 1, %0;" ::"n"(S::kProducerWarps * 32) : "memory");                    // nobody still reads the row map of the item before
            for (uint32_t i = tid; i < done.nv; i += S::kProducerWarps * 32)
                out_rows[i] = (EPI == kEpiDownBf16 && p.route_of_row) ? p.route_of_row[done.row0 + i] : done.row0 + i;
            asm volatile("bar.sync 1, %0;" ::"n"(S::kProducerWarps * 32) : "memory");
            if (lane == 0) mbar_wait(accum_bar, (uint32_t)seq & 1u, abort_flag, p.status);
            __syncwarp();
            tc_fence_after();
            const uint32_t c_end = min(done.nv, c_begin + 32u);
            const int fa = done.f0 + erow, fb = GATED ? fa : fa + 128;        // features of accumulator 0 / 1
            float bias_a = 0.f, bias_b = 0.f;
            if (fa < p.n && p.b0) bias_a = bf16_round(p.b0[((size_t)done.expert * p.n + fa) * p.bias_stride]);
            if (GATED) {
                if (EPI == kEpiSwigluF16 && fa < p.n) bias_b = bf16_round(__fadd_rn(p.b1[((size_t)done.expert * p.n + fa) * p.bias_stride], 1.0f));
            } else if (fb < p.n && p.b0) {
                bias_b = bf16_round(p.b0[((size_t)done.expert * p.n + fb) * p.bias_stride]);
            }
            const int col_a = EPI == kEpiDownBf16 ? fa : operand_pos(OCO_FMT_MXFP4, fa);
            const int col_b = EPI == kEpiDownBf16 ? fb : operand_pos(OCO_FMT_MXFP4, fb);
            for (uint32_t c = c_begin; c < c_begin + 32u; c += 16) {
                uint32_t ra[16], rb[16];
                tmem_ld16(taddr + c, ra);
                tmem_ld16(taddr + NT + c, rb);
                tmem_ld_wait();
                if (c + 16 >= c_begin + 32u) {                                // last read of this warp's columns
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(tmem_free);
                }
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    if (c + j < c_end) {
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
        }
    } else if (warp == S::kMmaWarp) {
        if (lane == 0) {
            // ===== MMA issue ======================================================================
            int seq = 0;
            for (int item = blockIdx.x; item < total; item += gridDim.x, seq++) {
                const Item it = load_item(item);
                const uint32_t n_mma = max(16u, (it.nv + 15u) & ~15u);
                if (seq > 0) {                                                // the accumulators of the item before are drained
                    mbar_wait(tmem_free, (uint32_t)(seq - 1) & 1u, abort_flag, p.status);
                    tc_fence_after();
                }
                const int g0 = seq * nkg;
                for (int g = 0; g < nkg; g++) {
                    const int G = g0 + g, sa = G % S::kAStages, sb = G % S::kBStages;
                    mbar_wait(full_a(sa), (uint32_t)(G / S::kAStages) & 1u, abort_flag, p.status);
                    mbar_wait(full_b(sb), (uint32_t)(G / S::kBStages) & 1u, abort_flag, p.status);
                    tc_fence_after();
                    const uint32_t a_stage = a_base + (uint32_t)sa * S::kAStage, b_stage = b_base + (uint32_t)sb * S::kBStage;
                    const uint32_t sfb_t = tmem_base + S::kColSfb + 8u * (uint32_t)sb;
                    mx_cp_scales(sfb_t, mx_sf_desc(b_stage + NT * 128u));
                    mx_cp_scales(sfb_t + 4u, mx_sf_desc(b_stage + NT * 128u + 512u));
                    const uint64_t bd = umma_desc(b_stage);
#pragma unroll
                    for (int mat = 0; mat < 2; mat++) {
                        const uint32_t sfa_t = tmem_base + S::kColSfa + (uint32_t)(sa * 2 + mat) * 8u;
                        const uint32_t sfa_smem = a_stage + 2u * S::kATile + (uint32_t)mat * 1024u;
                        mx_cp_scales(sfa_t, mx_sf_desc(sfa_smem));
                        mx_cp_scales(sfa_t + 4u, mx_sf_desc(sfa_smem + 512u));
                        const uint64_t ad = umma_desc(a_stage + (uint32_t)mat * S::kATile);
#pragma unroll
                        for (int kk = 0; kk < 4; kk++)
                            umma_mxf4(tmem_base + (uint32_t)mat * NT, ad + 2u * kk, bd + 2u * kk, mx_idesc(n_mma, (uint32_t)(kk & 1) * 2u),
                                      sfa_t + 4u * (kk >> 1), sfb_t + 4u * (kk >> 1), (g | kk) ? 1u : 0u);
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
        // ===== B tiles by TMA, their scales by one bulk copy =============================================
        int seq = 0;
        for (int item = blockIdx.x; item < total; item += gridDim.x, seq++) {
            const Item it = load_item(item);
            const int g0 = seq * nkg;
            for (int g = 0; g < nkg; g++) {
                const int G = g0 + g, sb = G % S::kBStages;
                const uint32_t b_stage = b_base + (uint32_t)sb * S::kBStage;
                mbar_wait(empty_b(sb), ((uint32_t)(G / S::kBStages) & 1u) ^ 1u, abort_flag, p.status);
                mbar_arrive_expect_tx(full_b(sb), NT * 128u + 1024u);
                tma_load_2d(b_stage, &tmap_b, g * 128, (int)it.row0, full_b(sb));
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(b_stage + NT * 128u),
                             "l"(p.sfb + ((size_t)it.tile * nkg + g) * 1024), "r"(1024u), "r"(full_b(sb)) : "memory");
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
}

// ---- the same product over REPACKED weights: every operand by TMA, no producer warps ----------------------
// The GGUF layout (17-byte blocks) is what forces the producers above. A host that can afford a second form
// of the expert tensors (made once, oco_moe_bind_repacked) gets them as two planes per tensor:
//   codes   [expert][feature tile][K group][16384]  the code bytes of 128 rows x 256 elements as the MMA reads
//                                                   them from shared memory (K-major, 128-byte swizzle: row r,
//                                                   16-byte piece c at (r / 8) * 1024 + (r % 8) * 128 + ((c ^ (r % 8)) * 16))
//   scales  [expert][feature tile][K group][1024]   the blocks' scale bytes in the layout tcgen05.cp wants
//                                                   (two 512-byte tiles of four blocks each per K group)
// so that a weight tile is one contiguous 16 KB and arrives with ONE bulk copy (a tensor copy of 128 rows of 128
// bytes from a row-major plane runs at the copy engine's rate per row, several times slower). A stage of the
// pipeline is then five copies issued by one thread: two weight tiles, their scale tiles and the activation
// tile (TMA) with its scales. Nothing in the SM touches the weight bytes. mx_repack_kernel makes the planes
// (zeroed first: rows of a feature tile past the expert's last row and blocks past K hold zero codes and a zero
// scale byte; their products land in accumulator lanes nobody reads, or add zero).
__global__ void __launch_bounds__(256) mx_repack_kernel(const uint8_t* __restrict__ w, size_t row_stride, int n, int experts, int K,
                                                        unsigned char* __restrict__ codes, unsigned char* __restrict__ sf) {
    const int nkb = K >> 5, nkg = (nkb + 7) >> 3, nt = (n + 127) >> 7;
    const size_t total = (size_t)experts * n * nkb;
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (size_t)gridDim.x * 256) {
        const size_t row = i / nkb;
        const uint32_t blk = (uint32_t)(i - row * nkb);
        const uint32_t e = (uint32_t)(row / n), r = (uint32_t)(row - (size_t)e * n);
        const uint8_t* b = w + row * row_stride + (size_t)blk * 17;
        uint32_t words[4];
#pragma unroll
        for (int c = 0; c < 4; c++)
            words[c] = (uint32_t)b[1 + 4 * c] | ((uint32_t)b[2 + 4 * c] << 8) | ((uint32_t)b[3 + 4 * c] << 16) | ((uint32_t)b[4 + 4 * c] << 24);
        const uint32_t t = r >> 7, rr = r & 127u;
        unsigned char* tile = codes + ((((size_t)e * nt + t) * nkg + (blk >> 3)) << 14);
        *reinterpret_cast<uint4*>(tile + (rr >> 3) * 1024u + (rr & 7u) * 128u + (((blk & 7u) ^ (rr & 7u)) << 4)) = make_uint4(words[0], words[1], words[2], words[3]);
        sf[(((size_t)e * nt + t) * nkg + (blk >> 3)) * 1024 + ((blk >> 2) & 1u) * 512 + (rr & 31u) * 16 + (rr >> 5) * 4 + (blk & 3u)] = b[0];
    }
}

struct MxrGemmShape {
    static constexpr int kNT = 112;                            // routes per tile: two accumulator sets of 2 x 112 columns and
                                                               // 32 scale columns fill the 512 columns of tensor memory
    static constexpr int kBRows = 128;                         // rows of the B box (the tile's rows and 16 that are not read)
    static constexpr int kEpilogueWarps = 16;
    static constexpr int kMmaWarp = 16, kTmaWarp = 17, kMmaWarp2 = 18;   // one issuing thread per weight tile
    static constexpr int kThreads = 19 * 32;
    static constexpr int kATile = 128 * 128;
    static constexpr int kOffSfa = 2 * kATile;                 // the two A tiles, their scale tiles (1 KB each),
    static constexpr int kOffB = kOffSfa + 2 * 1024;           // the B tile, its scales
    static constexpr int kOffSfb = kOffB + kBRows * 128;
    static constexpr int kStage = kOffSfb + 1024;              // 52224 bytes
    static constexpr int kStages = 4;
    static constexpr int kCtrl = 512 + 2 * 128 * 4;            // barriers, tmem slot, abort flag, two row maps
    static constexpr int kSmemBytes = kStages * kStage + kCtrl + 1024;
    static constexpr int kTmemCols = 512;
    static constexpr int kColSf = 4 * kNT;                      // 16 scale columns per issuing thread from here
    static_assert(kSmemBytes <= 232448, "shared memory of one CTA");
    static_assert(kStage % 1024 == 0, "stages keep the tiles' 1024-byte alignment");
};

// EPI as in gemm.cuh. p.w0 / p.w1: the code planes of the two matrices (for the down projection both are the same
// plane: the item's two feature tiles), p.sfa0 / p.sfa1 their scale tiles; tmap_b: the quantised activation rows,
// p.sfb their scale tiles.
template <int EPI>
__global__ void __launch_bounds__(MxrGemmShape::kThreads, 1)
grouped_gemm_mxr_kernel(const GemmParams p, const __grid_constant__ CUtensorMap tmap_b) {
    using S = MxrGemmShape;
    constexpr bool GATED = epi_gated(EPI);
    constexpr int NT = S::kNT;
    constexpr int kFeatPerItem = GATED ? 128 : 256;
    extern __shared__ unsigned char smem_raw[];
    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    if (__syncthreads_or(tid == 0 && *reinterpret_cast<volatile uint32_t*>(p.status) != 0u)) return;

    const int nfeat = (p.n + kFeatPerItem - 1) / kFeatPerItem;
    const int ntiles = (int)*p.tile_count;
    const int total = nfeat * ntiles;
    struct Item { uint32_t expert, row0, nv; int f0, tile; };
    auto load_item = [&](int item) {
        Item r;
        r.tile = item / nfeat;
        r.f0 = (item - r.tile * nfeat) * kFeatPerItem;
        r.expert = p.tiles[2 * r.tile];
        const uint32_t begin = p.tiles[2 * r.tile + 1];
        r.row0 = p.offsets[r.expert] + begin;
        r.nv = min((uint32_t)NT, p.offsets[r.expert + 1] - p.offsets[r.expert] - begin);
        return r;
    };
    const int nkb = p.K >> 5, nkg = (nkb + 7) >> 3;

    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char* gen = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t ctrl = base + S::kStages * S::kStage;
    unsigned char* ctrl_gen = gen + (ctrl - base);
    auto full = [&](int s) { return ctrl + 8u * s; };
    auto empty = [&](int s) { return ctrl + 8u * (S::kStages + s); };
    // two accumulator sets: while the epilogue warps drain one, the MMAs of the next item fill the other
    auto accum_bar = [&](uint32_t set) { return ctrl + 8u * (2 * S::kStages + set); };
    auto tmem_free = [&](uint32_t set) { return ctrl + 8u * (2 * S::kStages + 2 + set); };
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ctrl_gen + 128);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    uint32_t* out_rows = reinterpret_cast<uint32_t*>(ctrl_gen + 512);

    if (tid == 0) {
        for (int s = 0; s < S::kStages; s++) { mbar_init(full(s), 1); mbar_init(empty(s), 2); }   // both issuing threads commit
        for (uint32_t b = 0; b < 2; b++) { mbar_init(accum_bar(b), 2); mbar_init(tmem_free(b), S::kEpilogueWarps); }
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

    if (warp < S::kEpilogueWarps) {
        // ===== epilogue: warp -> tensor-memory lanes 32 * (warp & 3) (tile rows = features), columns [28 * (warp >> 2), +28)
        const int erow = (warp & 3) * 32 + lane;
        const uint32_t taddr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
        constexpr uint32_t kColsPerWarp = NT / 4;
        const uint32_t c_begin = (uint32_t)(warp >> 2) * kColsPerWarp;
        int seq = 0;
        for (int item = blockIdx.x; item < total; item += gridDim.x, seq++) {
            const Item done = load_item(item);
            asm volatile("bar.sync 1, %0;" ::"n"(S::kEpilogueWarps * 32) : "memory");     // nobody still reads the row map of the item before
            for (uint32_t i = tid; i < done.nv; i += S::kEpilogueWarps * 32)
                out_rows[i] = (EPI == kEpiDownBf16 && p.route_of_row) ? p.route_of_row[done.row0 + i] : done.row0 + i;
            asm volatile("bar.sync 1, %0;" ::"n"(S::kEpilogueWarps * 32) : "memory");
            const uint32_t set = (uint32_t)seq & 1u, use = (uint32_t)seq >> 1;
            const uint32_t tset = taddr + set * 2u * NT;
            if (lane == 0) mbar_wait(accum_bar(set), use & 1u, abort_flag, p.status);
            __syncwarp();
            tc_fence_after();
            const uint32_t c_end = min(done.nv, c_begin + kColsPerWarp);
            const int fa = done.f0 + erow, fb = GATED ? fa : fa + 128;
            float bias_a = 0.f, bias_b = 0.f;
            if (fa < p.n && p.b0) bias_a = bf16_round(p.b0[((size_t)done.expert * p.n + fa) * p.bias_stride]);
            if (GATED) {
                if (EPI == kEpiSwigluF16 && fa < p.n) bias_b = bf16_round(__fadd_rn(p.b1[((size_t)done.expert * p.n + fa) * p.bias_stride], 1.0f));
            } else if (fb < p.n && p.b0) {
                bias_b = bf16_round(p.b0[((size_t)done.expert * p.n + fb) * p.bias_stride]);
            }
            const int col_a = EPI == kEpiDownBf16 ? fa : operand_pos(OCO_FMT_MXFP4, fa);
            const int col_b = EPI == kEpiDownBf16 ? fb : operand_pos(OCO_FMT_MXFP4, fb);
            for (uint32_t c = c_begin; c < c_begin + kColsPerWarp; c += 16) {      // the second read runs past the warp's columns: unused
                uint32_t ra[16], rb[16];
                tmem_ld16(tset + c, ra);
                tmem_ld16(tset + NT + c, rb);
                tmem_ld_wait();
                if (c + 16 >= c_begin + kColsPerWarp) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(tmem_free(set));
                }
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    if (c + j < c_end) {
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
        }
    } else if (warp == S::kMmaWarp || warp == S::kMmaWarp2) {
        if (lane == 0) {
            // ===== MMA issue: one thread per weight tile and accumulator =====================================
            // A tcgen05 instruction costs its issuing thread about 80 cycles whatever it does, and a K group is
            // six scale copies, eight MMAs and a commit: one thread would spend 1.8 times the MMAs' tensor time
            // issuing them. Each thread copies the activation scales into columns of its own (the order of two
            // threads' tcgen05 operations is not defined) and its weight tile's scales, then issues its four MMAs.
            const int mat = warp == S::kMmaWarp ? 0 : 1;
            int seq = 0;
            for (int item = blockIdx.x; item < total; item += gridDim.x, seq++) {
                const Item it = load_item(item);
                const uint32_t n_mma = max(16u, (it.nv + 15u) & ~15u);
                const uint32_t set = (uint32_t)seq & 1u, use = (uint32_t)seq >> 1;
                if (use > 0) {                                                // this set's item before last is drained
                    mbar_wait(tmem_free(set), (use - 1u) & 1u, abort_flag, p.status);
                    tc_fence_after();
                }
                const int g0 = seq * nkg;
                for (int g = 0; g < nkg; g++) {
                    const int G = g0 + g, s = G % S::kStages;
                    mbar_wait(full(s), (uint32_t)(G / S::kStages) & 1u, abort_flag, p.status);
                    tc_fence_after();
                    const uint32_t stage = base + (uint32_t)s * S::kStage;
                    // one set of scale columns per issuing thread, rewritten every K group: a thread's tcgen05.cp and
                    // tcgen05.mma execute in the order it issued them
                    const uint32_t sfb_t = tmem_base + S::kColSf + 16u * (uint32_t)mat;                      // SFB 8 columns, then SFA 8
                    const uint32_t sfa_t = sfb_t + 8u;
                    mx_cp_scales(sfb_t, mx_sf_desc(stage + S::kOffSfb));
                    mx_cp_scales(sfb_t + 4u, mx_sf_desc(stage + S::kOffSfb + 512u));
                    const uint32_t sfa_smem = stage + S::kOffSfa + (uint32_t)mat * 1024u;
                    mx_cp_scales(sfa_t, mx_sf_desc(sfa_smem));
                    mx_cp_scales(sfa_t + 4u, mx_sf_desc(sfa_smem + 512u));
                    const uint64_t bd = umma_desc(stage + S::kOffB);
                    const uint64_t ad = umma_desc(stage + (uint32_t)mat * S::kATile);
#pragma unroll
                    for (int kk = 0; kk < 4; kk++)
                        umma_mxf4(tmem_base + set * 2u * NT + (uint32_t)mat * NT, ad + 2u * kk, bd + 2u * kk, mx_idesc(n_mma, (uint32_t)(kk & 1) * 2u),
                                  sfa_t + 4u * (kk >> 1), sfb_t + 4u * (kk >> 1), (g | kk) ? 1u : 0u);
                    umma_commit(empty(s));
                }
                umma_commit(accum_bar(set));
            }
            if (seq > 0) mbar_wait(accum_bar((uint32_t)(seq - 1) & 1u), ((uint32_t)(seq - 1) >> 1) & 1u, abort_flag, p.status);   // every MMA has retired
            tc_fence_before();
        }
    } else if (lane == 0) {
        // ===== every operand of a stage: five copies ======================================================
        int seq = 0;
        for (int item = blockIdx.x; item < total; item += gridDim.x, seq++) {
            const Item it = load_item(item);
            const int g0 = seq * nkg;
            const int ft0 = it.f0 >> 7, ft1 = GATED ? ft0 : min(ft0 + 1, p.sfa_tiles - 1);
            const size_t t0 = ((size_t)it.expert * p.sfa_tiles + ft0) * nkg, t1 = ((size_t)it.expert * p.sfa_tiles + ft1) * nkg;
            const unsigned char* sf0 = p.sfa0 + t0 * 1024;
            const unsigned char* sf1 = (GATED ? p.sfa1 : p.sfa0) + t1 * 1024;
            const uint8_t* c0 = p.w0 + (t0 << 14);
            const uint8_t* c1 = (GATED ? p.w1 : p.w0) + (t1 << 14);
            for (int g = 0; g < nkg; g++) {
                const int G = g0 + g, s = G % S::kStages;
                const uint32_t stage = base + (uint32_t)s * S::kStage;
                mbar_wait(empty(s), ((uint32_t)(G / S::kStages) & 1u) ^ 1u, abort_flag, p.status);
                mbar_arrive_expect_tx(full(s), 2u * S::kATile + 2u * 1024u + S::kBRows * 128u + 1024u);
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(stage),
                             "l"(c0 + ((size_t)g << 14)), "r"(16384u), "r"(full(s)) : "memory");
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(stage + S::kATile),
                             "l"(c1 + ((size_t)g << 14)), "r"(16384u), "r"(full(s)) : "memory");
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(stage + S::kOffSfa),
                             "l"(sf0 + (size_t)g * 1024), "r"(1024u), "r"(full(s)) : "memory");
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(stage + S::kOffSfa + 1024u),
                             "l"(sf1 + (size_t)g * 1024), "r"(1024u), "r"(full(s)) : "memory");
                tma_load_2d(stage + S::kOffB, &tmap_b, g * 128, (int)it.row0, full(s));
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(stage + S::kOffSfb),
                             "l"(p.sfb + ((size_t)it.tile * nkg + g) * 1024), "r"(1024u), "r"(full(s)) : "memory");
            }
        }
    }
    __syncthreads();
    if (*abort_flag) {
        for (int i = 0; i < 64; i++) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == S::kMmaWarp) {
        tc_fence_after();
        tmem_dealloc(tmem_base, S::kTmemCols);
    }
}

}  // namespace oco
