// MXFP4 expert rows on the block-scaled tensor-core path (tcgen05.mma kind::mxf4, UE8M0 scales per 32
// elements, fp32 accumulators in tensor memory), for one token.
//
// A GGUF MXFP4 block is already what this MMA kind multiplies: sixteen bytes of e2m1 pairs and one
// E8M0 scale. Nothing is decoded: the packed rows stream from HBM into shared memory, producer warps
// move each block's sixteen code bytes to the 16-byte-aligned position the MMA descriptor wants and
// its scale byte into the scale-factor tile, and one thread issues the MMAs. A code byte holds
// elements j and j + 16 of its block while the tensor core reads a byte as two consecutive
// contraction positions, so the activation operand is laid out in the same "operand order"
// (position 2j = element j, position 2j + 1 = element j + 16); a dot product does not care in which
// order k is visited.
//
// The activations stay at full precision although the B operand is e2m1 too: a value is split into
// pieces x = sum_p q_p * 2^(e_p), every q_p an e2m1 number, e_p a scale shared by the 32 elements of
// the block (the first piece takes two bits of the block's largest magnitude, every further piece
// three more). The pieces of one activation vector are different columns of the B operand, so one
// MMA multiplies the weight rows with all of them; the epilogue adds the columns in fp32. Eight
// pieces carry 23 bits below the block's largest element, all products are exact and the
// accumulation is fp32, which is the reference's single-token arithmetic (f32 activations times
// decoded weights, shaders/experts/projections.metal:78-182) up to summation order.
//
// The rows of a GGUF tensor start at any byte address and are not a multiple of 16 bytes long, so
// they are fetched as the 16-byte pieces that cover them (cp.async, consecutive lanes taking
// consecutive pieces of a row): every producer warp streams its own 16 rows through a private ring,
// one K group (256 elements, 136 packed bytes) per stage, and nothing but the MMA barriers is
// shared between warps.
#pragma once
#include "gemm.cuh"
#include "mx_pieces.cuh"

namespace oco {

constexpr int kMxGroupBlocks = 8;                    // blocks per K group: one 128-byte swizzle row of e2m1 codes
constexpr int kMxGroupBytes = kMxGroupBlocks * 17;   // packed bytes of a K group in a row
constexpr int kMxSlot = 176;                         // ring bytes per row and K group: 136 + 15 of misalignment, 16 x 11
constexpr int kMxPiecesPerRow = 10;                  // 16-byte pieces fetched per row and K group
constexpr int kMxWarpRows = 16;                      // tile rows of a producer warp (two units of eight rows)
constexpr int kMxRingStages = 4;
// ring bytes of one producer warp: a stage holds one K group of its row of every unit of a pass
__host__ __device__ constexpr uint32_t mx_ring_bytes(int pass_units) { return (uint32_t)(kMxRingStages * pass_units * kMxSlot); }
constexpr int kMxProducerWarps = 16;                 // 2 matrices x 128 tile rows / 16
constexpr int kMxMmaWarp = kMxProducerWarps;
constexpr int kMxThreads = (kMxProducerWarps + 2) * 32;   // + one MMA-issuing warp per matrix
constexpr int kMxAStages = 2;
constexpr int kMxTmemCols = 512;
constexpr int kMxColD = 0, kMxColSfa = 64, kMxColSfb = 128;   // scale addresses are multiples of four columns

__device__ __forceinline__ uint64_t mx_sf_desc(uint32_t smem_addr) {   // 32 rows x 16 bytes, no swizzle, 8-row groups 128 bytes apart
    uint32_t lo = (smem_addr & 0x3ffffu) >> 4;
    uint32_t hi = (128u >> 4) | (1u << 14);
    return ((uint64_t)hi << 32) | lo;
}
__device__ __forceinline__ void mx_cp_scales(uint32_t taddr, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void umma_mxf4(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t sfa, uint32_t sfb, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc), "r"(sfa), "r"(sfb) : "memory");
}
// kind::mxf4: A and B e2m1 (format 1), UE8M0 scales, M = 128, N = n; scale ids pick bytes 0-1 or 2-3 of a scale column.
__device__ __forceinline__ uint32_t mx_idesc(uint32_t n, uint32_t sf_id) {
    return (sf_id << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | (1u << 23) | ((128u >> 4) << 24) | (sf_id << 29);
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}

struct MxParams {
    const uint8_t* w[2];          // first packed row of each matrix (expand: gate, up; down: down)
    const uint8_t* w_end[2];      // first byte past the 16-byte envelope of each matrix (no piece starts there or beyond)
    uint32_t row_stride;          // bytes between consecutive rows of a matrix
    int K;                        // contraction length
    int rows_per_route;           // output rows of one expert's matrix
    int routes;
    int pass_units;               // units (eight rows of one route, of every matrix) a CTA takes per pass
    const uint32_t* ids;          // [routes] expert of each route; null = expert 0
    // B operand: e2m1 pieces and their scales. expand: of the token (one image for all routes);
    // down: of each route's activations, `b_route_bytes` / `sfb_route_bytes` apart
    const unsigned char* b_img;
    const unsigned char* sfb_img;
    uint32_t b_route_bytes, sfb_route_bytes;
    // epilogue
    const float* b0;              // expand: gate bias; down: bias (or null)
    const float* b1;              // expand: up bias
    int bias_stride;
    float* act_out;               // expand: f32 [routes][rows_per_route]
    unsigned char* act_b;         // expand: the down kernel's B images, one per route, and their scales, written
    unsigned char* act_sfb;       //         by whoever completes a block of 32 activations last
    uint32_t act_b_route_bytes, act_sfb_route_bytes;
    uint32_t* blk_arrivals;       // expand: one zeroed counter per route and block of 32 activations
    uint16_t* y;                  // down: bf16 [routes][rows_per_route]
    uint32_t* arrivals;           // down: one zeroed counter per output row
    const float* probs;
    uint16_t* residual;
    int round_sum;
    uint32_t* status;
};

constexpr uint32_t kMxCtrlBytes = 1024;              // barriers | tensor-memory slot, flags, queue
// Shared memory: A stages | SFA tiles | B image | SFB tiles | control | one ring per live producer warp.
__host__ __device__ inline uint32_t mx_fixed_smem(int n_mat, uint32_t nkb) {
    return (uint32_t)kMxAStages * n_mat * (16384u + 1024u) + mx_b_bytes(8, nkb) + mx_sfb_bytes(nkb) + kMxCtrlBytes + 1024u;
}
// Units of a pass that starts at u0 for a CTA whose share ends at u_end: `pass_units` at most, and (down)
// units of one route only, since a pass multiplies with one activation vector.
__host__ __device__ inline int mx_pass_end(int u0, int u_end, int upr, int pass_units, bool one_route) {
    int u1 = u0 + pass_units;
    if (u1 > u_end) u1 = u_end;
    if (one_route && u1 > (u0 / upr + 1) * upr) u1 = (u0 / upr + 1) * upr;
    return u1;
}

// Moves the eight blocks of one K group of ONE raw row (this lane's) into its A tile row and scale tiles.
// c[0..39]: the row's ring slot as 16-byte pieces; the row's data starts at byte D of the slot. With D a
// compile-time constant every word index and shift below is static: a block's sixteen code bytes are
// four funnel shifts away from their aligned place, its scale byte one byte permute. (A row's last K
// group, when it is not full, takes mx_move_row_any, which zeroes the blocks past the end of the row.)
template <int D>
__device__ __forceinline__ void mx_move_row(const uint32_t (&c)[40], unsigned char* a_row, uint32_t sw, unsigned char* sf_dst) {
    uint32_t sfw[2] = {0u, 0u};
#pragma unroll
    for (int b = 0; b < 8; b++) {
        const int o = D + 17 * b;                  // the block's scale byte; its codes follow
        const int q = (o + 1) >> 2, t = ((o + 1) & 3) * 8;
        uint4 k;
        if (t == 0) k = make_uint4(c[q], c[q + 1], c[q + 2], c[q + 3]);
        else k = make_uint4(__funnelshift_r(c[q], c[q + 1], t), __funnelshift_r(c[q + 1], c[q + 2], t),
                            __funnelshift_r(c[q + 2], c[q + 3], t), __funnelshift_r(c[q + 3], c[q + 4], t));
        *reinterpret_cast<uint4*>(a_row + (((uint32_t)b << 4) ^ sw)) = k;
        // the scale byte into byte b & 3 of its word: one byte permute
        sfw[b >> 2] = __byte_perm(sfw[b >> 2], c[o >> 2], (0x3210u & ~(0xfu << (4 * (b & 3)))) | ((4u + (uint32_t)(o & 3)) << (4 * (b & 3))));
    }
    *reinterpret_cast<uint32_t*>(sf_dst) = sfw[0];
    *reinterpret_cast<uint32_t*>(sf_dst + 512) = sfw[1];
}
// The same with a start byte known only at run time (rows whose pointers differ in their low four bits:
// matrices with an odd row stride) and with blocks past `nb` zeroed (scale byte zero): the words are
// selected with conditional moves.
__device__ __forceinline__ void mx_move_row_any(uint32_t dl, const uint32_t (&c)[40], unsigned char* a_row, uint32_t sw, unsigned char* sf_dst, int nb) {
    uint32_t sfw[2] = {0u, 0u};
#pragma unroll
    for (int b = 0; b < 8; b++) {
        const uint32_t o = dl + (uint32_t)b;                 // block b starts at byte dl + 17 b = 16 b + o
        const bool hi = o >= 16u;
        const uint32_t sh = o & 15u, qw = sh >> 2, tb = (sh & 3u) * 8u;
        uint32_t w[8], y[6], x[5];
#pragma unroll
        for (int i = 0; i < 8; i++) w[i] = hi ? c[4 * (b + 1) + i] : c[4 * b + i];
#pragma unroll
        for (int i = 0; i < 6; i++) y[i] = (qw & 2u) ? w[i + 2] : w[i];
#pragma unroll
        for (int i = 0; i < 5; i++) x[i] = (qw & 1u) ? y[i + 1] : y[i];
        uint32_t scale = (x[0] >> tb) & 0xffu;
        uint4 k = make_uint4(__funnelshift_rc(x[0], x[1], tb + 8u), __funnelshift_rc(x[1], x[2], tb + 8u),
                             __funnelshift_rc(x[2], x[3], tb + 8u), __funnelshift_rc(x[3], x[4], tb + 8u));
        if (b >= nb) { k = make_uint4(0u, 0u, 0u, 0u); scale = 0u; }
        *reinterpret_cast<uint4*>(a_row + (((uint32_t)b << 4) ^ sw)) = k;
        sfw[b >> 2] |= scale << (8 * (b & 3));
    }
    *reinterpret_cast<uint32_t*>(sf_dst) = sfw[0];
    *reinterpret_cast<uint32_t*>(sf_dst + 512) = sfw[1];
}

// EXPAND: two matrices (gate, up), one activation vector for all routes, fused clipped SwiGLU, f32
// activations out; whoever completes a block of 32 activations last also splits it into the pieces the
// down kernel multiplies with. Otherwise: one matrix, one route per pass, bf16 expert outputs and, by
// whoever completes an output row last, the weighted sum onto the residual.
// Grid: one CTA per SM; CTA c owns the units [c U / G, (c + 1) U / G) where a unit is eight consecutive
// rows of one route (of both matrices), U = routes * rows_per_route / 8. Tile row t of a pass is row j = t / 16
// of the pass's unit t mod 16, and producer warp j of a matrix serves the rows j of all units: rows eight
// apart start at the same byte of a 16-byte word (unless the row stride is odd), so one warp's rows
// need the same shifts.
template <bool EXPAND>
__global__ void __launch_bounds__(kMxThreads, 1) mx_rows_kernel(const MxParams p) {
    constexpr int NMAT = EXPAND ? 2 : 1;
    constexpr uint32_t NCOL = 8u;
    extern __shared__ unsigned char smem_raw[];
    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const int nkb = p.K >> 5, nkg = (nkb + 7) >> 3;
    const int upr = p.rows_per_route >> 3;                      // units per route
    const int units_total = p.routes * upr;
    const int u_begin = (int)((long long)blockIdx.x * units_total / gridDim.x);
    const int u_end = (int)((long long)(blockIdx.x + 1) * units_total / gridDim.x);

    // ---- shared memory carve-up ------------------------------------------------------------------
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char* gen = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t a_base = base;                                               // [stage][mat] 16 KB tiles
    const uint32_t sfa_base = a_base + kMxAStages * NMAT * 16384u;              // [stage][mat] two 512-byte tiles
    const uint32_t b_base = sfa_base + kMxAStages * NMAT * 1024u;
    const uint32_t b_bytes = mx_b_bytes(NCOL, nkb), sfb_bytes = mx_sfb_bytes(nkb);
    const uint32_t sfb_base = b_base + b_bytes;
    const uint32_t ctrl = sfb_base + sfb_bytes;
    const uint32_t ring_base = ctrl + kMxCtrlBytes;
    unsigned char* ctrl_gen = gen + (ctrl - base);
    auto a_full = [&](int s) { return ctrl + 8u * s; };
    auto a_empty = [&](int s) { return ctrl + 8u * (2 + s); };
    const uint32_t accum_bar = ctrl + 8u * 4, b_bar = ctrl + 8u * 5, tmem_free = ctrl + 8u * 6, sfb_ready = ctrl + 8u * 7;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ctrl_gen + 64);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    uint32_t* queue_len = tmem_slot + 2;                                        // expand: completed activation blocks
    uint32_t* queue = reinterpret_cast<uint32_t*>(ctrl_gen + 128);              //         (route << 16 | block), up to 64

    pdl_launch_dependents();
    if (tid == 0) {
        for (int s = 0; s < kMxAStages; s++) { mbar_init(a_full(s), 8 * NMAT); mbar_init(a_empty(s), NMAT); }
        mbar_init(accum_bar, NMAT);
        mbar_init(sfb_ready, 1);
        mbar_init(b_bar, 1);
        mbar_init(tmem_free, 4);
        *abort_flag = 0;
        *queue_len = 0;
        fence_barrier_init();
    }
    if (warp == kMxMmaWarp) {
        tmem_alloc(smem_u32(tmem_slot), kMxTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();                       // ids, activations and pieces written by the kernels before are complete

    int step0 = 0;            // K groups of earlier passes (barrier phases run on)
    int pass = 0;
    int b_loads = 0;          // B images fetched so far (phase of b_bar)
    int b_route = -1;
    for (int u0 = u_begin; u0 < u_end; pass++) {
        const int u1 = mx_pass_end(u0, u_end, upr, p.pass_units, !EXPAND);
        const int r_first = u0 / upr;
        __syncthreads();      // the pass before is finished with the B image
        const bool load_b = EXPAND ? pass == 0 : r_first != b_route;
        if (tid == 0 && load_b) {
            // the activation vector's pieces and their scales (made by the router or the expand kernel)
            const size_t r = EXPAND ? 0 : (size_t)r_first;
            mbar_arrive_expect_tx(b_bar, b_bytes + sfb_bytes);
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(b_base), "l"(p.b_img + r * p.b_route_bytes), "r"(b_bytes), "r"(b_bar) : "memory");
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(sfb_base), "l"(p.sfb_img + r * p.sfb_route_bytes), "r"(sfb_bytes), "r"(b_bar) : "memory");
        }
        if (load_b) { b_route = r_first; b_loads++; }

        if (warp < kMxProducerWarps) {
            const int mat = warp >> 3, wi = warp & 7;
            if (mat < NMAT) {
                // ===== producers ========================================================================
                // Warp wi serves row wi of every unit of the pass: lane s < 16 is unit u0 + s (tile row 16 wi + s).
                const int j = wi;
                const uint32_t stage_bytes = (uint32_t)(p.pass_units * kMxSlot);
                const uint32_t ring = ring_base + (uint32_t)(mat * 8 + wi) * mx_ring_bytes(p.pass_units);
                const unsigned char* ring_gen = gen + (ring - base);
                auto row_ptr = [&](int s) -> const uint8_t* {
                    const int unit = u0 + s;
                    if (unit >= u1) return nullptr;
                    const int route = unit / upr;
                    const uint32_t e = p.ids ? p.ids[route] : 0u;
                    return p.w[mat] + ((size_t)e * p.rows_per_route + (size_t)(unit - route * upr) * 8 + j) * p.row_stride;
                };
                // fetch role: 160 pieces per stage, piece (lane + 32 k) -> row s = / 10, piece % 10
                // (row16: the row's pointer rounded down to 16 bytes plus the piece; r15: its low four bits)
                const uint8_t* row16[5];
                uint32_t fdst[5], r15[5];
                bool guard = false;         // some piece of some K group may start at or past the end of the tensor's envelope
#pragma unroll
                for (int k = 0; k < 5; k++) {
                    const int idx = lane + 32 * k, sr = idx / kMxPiecesPerRow, piece = idx - sr * kMxPiecesPerRow;
                    const uint8_t* rp = row_ptr(sr);
                    row16[k] = rp ? (const uint8_t*)((uintptr_t)rp & ~(uintptr_t)15) + piece * 16 : nullptr;
                    r15[k] = (uint32_t)((uintptr_t)rp & 15u);
                    fdst[k] = (uint32_t)(sr * kMxSlot + piece * 16);
                    if (rp && row16[k] + (size_t)nkg * kMxGroupBytes + 16 > p.w_end[mat]) guard = true;
                }
                guard = __any_sync(0xffffffffu, guard);
                auto issue = [&](int g) {
                    if (g < nkg) {
                        const uint32_t st = ring + (uint32_t)((step0 + g) % kMxRingStages) * stage_bytes;
#pragma unroll
                        for (int k = 0; k < 5; k++) {
                            if (row16[k]) {
                                // this lane's piece of the 16-byte envelope of the row's K group g
                                const uint8_t* a16 = row16[k] + ((r15[k] + (uint32_t)g * kMxGroupBytes) & ~15u);
                                if (!guard || a16 < p.w_end[mat]) cp_async16(st + fdst[k], a16);
                            }
                        }
                    }
                    cp_async_commit();
                };
                // move role: lane s < 16 moves its row
                const int t = j * 16 + (lane & 15);
                const uint8_t* mrow = lane < 16 ? row_ptr(lane) : nullptr;
                const uint32_t a_off = (uint32_t)(t >> 3) * 1024u + (uint32_t)(t & 7) * 128u, sw = (uint32_t)(t & 7) << 4;
                const uint32_t sf_off = (uint32_t)(t & 31) * 16u + (uint32_t)(t >> 5) * 4u;
#pragma unroll
                for (int sI = 0; sI < kMxRingStages - 1; sI++) issue(sI);
                for (int g = 0; g < nkg; g++) {
                    const int n = step0 + g, as = n & (kMxAStages - 1);
                    issue(g + kMxRingStages - 1);
                    cp_async_wait<kMxRingStages - 1>();                            // K group g has landed
                    if (lane == 0) mbar_wait(a_empty(as), ((uint32_t)(n / kMxAStages) & 1u) ^ 1u, abort_flag, p.status);
                    __syncwarp();
                    const uint32_t dl = (uint32_t)((uintptr_t)(mrow + (size_t)g * kMxGroupBytes) & 15u);   // where the row's data starts in its slot
                    const uint32_t dl_first = __shfl_sync(0xffffffffu, dl, 0);              // every lane takes part in the shuffle
                    const bool same = __all_sync(0xffffffffu, !mrow || dl == dl_first);
                    if (mrow) {
                        const unsigned char* slot = ring_gen + (size_t)(n % kMxRingStages) * stage_bytes + (lane & 15) * kMxSlot;
                        unsigned char* a_row = gen + (a_base - base) + (size_t)(as * NMAT + mat) * 16384u + a_off;
                        unsigned char* sf_dst = gen + (sfa_base - base) + (size_t)(as * NMAT + mat) * 1024u + sf_off;
                        const int nb = min(8, nkb - g * 8);
                        uint32_t c[40];
#pragma unroll
                        for (int i = 0; i < 10; i++) {
                            const uint4 v = *reinterpret_cast<const uint4*>(slot + 16 * i);
                            c[4 * i] = v.x; c[4 * i + 1] = v.y; c[4 * i + 2] = v.z; c[4 * i + 3] = v.w;
                        }
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
                    if (lane == 0) mbar_arrive(a_full(as));
                }
                cp_async_wait<0>();
            }
            // ===== epilogue (warps 0-3, one quadrant of tensor-memory lanes each) ======================
            if (warp < 4) {
                const int q = warp;
                if (lane == 0) mbar_wait(accum_bar, (uint32_t)pass & 1u, abort_flag, p.status);
                __syncwarp();
                tc_fence_after();
                const int t = q * 32 + lane;
                const int unit = u0 + (t & 15);
                const bool live = unit < u1;
                const int route = unit / upr, row = (unit - route * upr) * 8 + (t >> 4);   // row within the route's matrix
                const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + kMxColD;
                uint32_t d0[8], d1[8];
                tmem_ld8(taddr, d0);
                if (EXPAND) tmem_ld8(taddr + 32u, d1);
                tmem_ld_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tmem_free);
                if (EXPAND) {
                    if (live) {
                        float sg = 0.f, su = 0.f;
#pragma unroll
                        for (int i = 7; i >= 0; i--) { sg = __fadd_rn(sg, __uint_as_float(d0[i])); su = __fadd_rn(su, __uint_as_float(d1[i])); }
                        const uint32_t e = p.ids ? p.ids[route] : 0u;
                        const size_t bi = ((size_t)e * p.rows_per_route + row) * p.bias_stride;
                        const float gate = __fadd_rn(sg, bf16_round(p.b0[bi]));
                        const float up = __fadd_rn(su, bf16_round(__fadd_rn(p.b1[bi], 1.0f)));
                        p.act_out[(size_t)route * p.rows_per_route + row] = swiglu_clipped(gate, up);
                        // whoever writes the last of a block's 32 activations queues the block for splitting
                        __threadfence();
                        const uint32_t blk = (uint32_t)row >> 5;
                        uint32_t* counter = p.blk_arrivals + (size_t)route * (p.rows_per_route >> 5) + blk;
                        if (atomicAdd(counter, 1u) == 31u) {
                            *counter = 0;                                                 // ready for the next call
                            const uint32_t at = atomicAdd(queue_len, 1u);
                            if (at < 64u) queue[at] = ((uint32_t)route << 16) | blk;
                        }
                    }
                } else if (live) {
                    float sy = 0.f;
#pragma unroll
                    for (int i = 7; i >= 0; i--) sy = __fadd_rn(sy, __uint_as_float(d0[i]));
                    const uint32_t e = p.ids ? p.ids[route] : 0u;
                    if (p.b0) sy = __fadd_rn(sy, bf16_round(p.b0[((size_t)e * p.rows_per_route + row) * p.bias_stride]));
                    p.y[(size_t)route * p.rows_per_route + row] = f32_to_bf16_bits(sy);
                    if (p.residual) {
                        // Whoever completes an output row last (the routes' rows are spread over CTAs) adds the
                        // weighted expert outputs to the residual (moe_sum, routing.metal:154-168). Nobody waits.
                        __threadfence();
                        const uint32_t seen = atomicAdd(p.arrivals + row, 1u);
                        if (seen == (uint32_t)(p.routes - 1)) {
                            p.arrivals[row] = 0;                                            // ready for the next call
                            if (*reinterpret_cast<volatile uint32_t*>(p.status) == 0u) {
                                __threadfence();
                                float sres = 0.0f;
                                for (int r = 0; r < p.routes; r++)
                                    sres = __fmaf_rn(bf16_bits_to_f32(__ldcg(p.y + (size_t)r * p.rows_per_route + row)), p.probs[r], sres);
                                if (p.round_sum) sres = bf16_round(sres);
                                p.residual[row] = f32_to_bf16_bits(__fadd_rn(bf16_bits_to_f32(p.residual[row]), sres));
                            }
                        }
                    }
                }
            }
        } else if (lane == 0 && warp - kMxMmaWarp < NMAT) {
            // ===== MMA issue: one thread per matrix (issuing an MMA costs tens of cycles) ================
            const int mat = warp - kMxMmaWarp;
            if (pass > 0) mbar_wait(tmem_free, (uint32_t)(pass - 1) & 1u, abort_flag, p.status);   // accumulators of the pass before are read
            if (load_b) {
                if (mat == 0) {
                    mbar_wait(b_bar, (uint32_t)(b_loads - 1) & 1u, abort_flag, p.status);
                    tc_fence_after();
                    // scales of the B operand: four blocks per copy, up to the end of the last K group (the MMAs of
                    // a partly filled group read them too; their blocks hold zeros with a zero scale byte)
                    for (int i = 0; i < 2 * nkg; i++) mx_cp_scales(tmem_base + kMxColSfb + 4u * i, mx_sf_desc(sfb_base + 512u * i));
                    if (NMAT > 1) umma_commit(sfb_ready);
                } else {
                    mbar_wait(sfb_ready, (uint32_t)(b_loads - 1) & 1u, abort_flag, p.status);
                    mbar_wait(b_bar, (uint32_t)(b_loads - 1) & 1u, abort_flag, p.status);
                }
            }
            tc_fence_after();
            for (int g = 0; g < nkg; g++) {
                const int n = step0 + g, as = n & (kMxAStages - 1);
                mbar_wait(a_full(as), (uint32_t)(n / kMxAStages) & 1u, abort_flag, p.status);
                tc_fence_after();
                const uint32_t sfa_smem = sfa_base + (uint32_t)(as * NMAT + mat) * 1024u;
                const uint32_t sfa_t = tmem_base + kMxColSfa + (uint32_t)(as * NMAT + mat) * 8u;
                mx_cp_scales(sfa_t, mx_sf_desc(sfa_smem));
                mx_cp_scales(sfa_t + 4u, mx_sf_desc(sfa_smem + 512u));
                const uint64_t ad = umma_desc(a_base + (uint32_t)(as * NMAT + mat) * 16384u);
                const uint64_t bd = umma_desc(b_base + (uint32_t)g * (NCOL * 128u));
#pragma unroll
                for (int kk = 0; kk < 4; kk++) {
                    const uint32_t sfid = (uint32_t)(kk & 1) * 2u;
                    umma_mxf4(tmem_base + kMxColD + 32u * mat, ad + 2u * kk, bd + 2u * kk, mx_idesc(NCOL, sfid),
                              sfa_t + 4u * (kk >> 1), tmem_base + kMxColSfb + 4u * (2u * g + (kk >> 1)), (g | kk) ? 1u : 0u);
                }
                umma_commit(a_empty(as));
            }
            umma_commit(accum_bar);
        }
        step0 += nkg;
        u0 = u1;
    }
    __syncthreads();
    if (EXPAND) {
        // the blocks of 32 activations this CTA completed: split them for the down kernel
        __threadfence();
        const uint32_t nq = min(*queue_len, 64u);
        for (uint32_t k = (uint32_t)warp; k < nq; k += kMxThreads / 32) {
            const uint32_t route = queue[k] >> 16, blk = queue[k] & 0xffffu;
            const float v = __ldcg(p.act_out + (size_t)route * p.rows_per_route + blk * 32u + (uint32_t)(lane >> 1) + 16u * (uint32_t)(lane & 1));
            mx_split_block(v, lane, p.act_b + (size_t)route * p.act_b_route_bytes, p.act_sfb + (size_t)route * p.act_sfb_route_bytes, 8u, 0u, blk);
        }
    }
    if (*abort_flag) {
        for (int i = 0; i < 64; i++) __nanosleep(1000);   // let copies in flight land before the CTA retires
        __syncthreads();
    }
    if (warp == kMxMmaWarp) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kMxTmemCols);
    }
}

// ---- the same products over REPACKED weights (oco_moe_bind_repacked): every operand by TMA ---------------------
// With the code bytes in a plane of 16-byte-aligned rows and the scale bytes as ready-made tiles (gemm_mx.cuh,
// mx_repack_kernel) nothing has to be moved inside the SM: a copy thread brings a tile of 128 weight rows and its
// scale tile per K group, the MMA threads multiply it with the activation's pieces as above. A pass is one tile of
// 128 consecutive rows of one route (of both matrices for the expand kernel); CTA c takes the tiles
// [c T / G, (c + 1) T / G). Tile row t is row 128 * tile + t of the expert's matrix, so a block of 32 activations is
// exactly one epilogue warp's 32 lanes of one pass: the warp that computed it splits it into pieces for the down
// kernel on the spot (no counters, no queue). The down kernel's weighted sum onto the residual is the one above.
struct MxTmaParams {
    const unsigned char* codes[2];   // code tiles of each matrix, [expert][row tile][K group][16384], as shared memory wants them
    const unsigned char* sf[2];      // scale tiles of each matrix, [expert][row tile][K group][1024]
    int row_tiles;                   // row tiles per expert (ceil(rows_per_route / 128))
};
constexpr int kMxTmaStages = 4;
constexpr int kMxTmaSplit = 4;                       // MMA-issuing threads per matrix: thread i takes the K groups g = i mod 4 into
                                                     // accumulator columns of its own (a tcgen05 instruction costs its thread 70-90
                                                     // cycles and a tile's K groups in one thread were the longest part of the kernel)
__host__ __device__ constexpr int mx_tma_warps(int n_mat) { return 4 + n_mat * kMxTmaSplit + 1; }   // epilogue, issuers, copy
__host__ __device__ inline uint32_t mx_tma_smem(int n_mat, uint32_t nkb) {
    return (uint32_t)kMxTmaStages * n_mat * (16384u + 1024u) + mx_b_bytes(8, nkb) + mx_sfb_bytes(nkb) + kMxCtrlBytes + 1024u;
}

template <bool EXPAND>
__global__ void __launch_bounds__(mx_tma_warps(EXPAND ? 2 : 1) * 32, 1)
mx_rows_tma_kernel(const MxParams p, const MxTmaParams q) {
    constexpr int NMAT = EXPAND ? 2 : 1;
    constexpr int kIssuers = NMAT * kMxTmaSplit, kCopyWarp = 4 + kIssuers;
    constexpr uint32_t kColMat = 8u * kMxTmaSplit;               // accumulator columns of one matrix: eight per issuing thread
    constexpr uint32_t NCOL = 8u;
    constexpr uint32_t kStage = NMAT * (16384u + 1024u);       // the matrices' tiles, then their scale tiles
    extern __shared__ unsigned char smem_raw[];
    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const int nkb = p.K >> 5, nkg = (nkb + 7) >> 3;
    const int tpr = q.row_tiles;                               // tiles per route
    const int tiles_total = p.routes * tpr;
    const int t_begin = (int)((long long)blockIdx.x * tiles_total / gridDim.x);
    const int t_end = (int)((long long)(blockIdx.x + 1) * tiles_total / gridDim.x);

    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char* gen = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t a_base = base;                                               // [stage] NMAT tiles of 16 KB, NMAT scale tiles of 1 KB
    const uint32_t b_base = a_base + kMxTmaStages * kStage;
    const uint32_t b_bytes = mx_b_bytes(NCOL, nkb), sfb_bytes = mx_sfb_bytes(nkb);
    const uint32_t sfb_base = b_base + b_bytes;
    const uint32_t ctrl = sfb_base + sfb_bytes;
    unsigned char* ctrl_gen = gen + (ctrl - base);
    auto a_full = [&](int s) { return ctrl + 8u * s; };
    auto a_empty = [&](int s) { return ctrl + 8u * (kMxTmaStages + s); };
    const uint32_t accum_bar = ctrl + 8u * (2 * kMxTmaStages), b_bar = accum_bar + 8u, tmem_free = accum_bar + 16u, sfb_ready = accum_bar + 24u;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ctrl_gen + 128);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    pdl_launch_dependents();
    if (tid == 0) {
        for (int s = 0; s < kMxTmaStages; s++) { mbar_init(a_full(s), 1); mbar_init(a_empty(s), NMAT); }
        mbar_init(accum_bar, kIssuers);
        mbar_init(sfb_ready, 1);
        mbar_init(b_bar, 1);
        mbar_init(tmem_free, 4);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 4) {
        tmem_alloc(smem_u32(tmem_slot), kMxTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();                       // ids, activations and pieces written by the kernels before are complete

    int step0 = 0, pass = 0, b_loads = 0, b_route = -1;
    (void)sfb_ready;
    for (int tile = t_begin; tile < t_end; tile++, pass++) {
        const int route = tile / tpr, rt = tile - route * tpr;          // row tile rt of this route's expert
        const uint32_t e = p.ids ? p.ids[route] : 0u;
        __syncthreads();      // the pass before is finished with the B image
        const bool load_b = EXPAND ? pass == 0 : route != b_route;
        if (tid == 0 && load_b) {
            const size_t r = EXPAND ? 0 : (size_t)route;
            mbar_arrive_expect_tx(b_bar, b_bytes + sfb_bytes);
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(b_base), "l"(p.b_img + r * p.b_route_bytes), "r"(b_bytes), "r"(b_bar) : "memory");
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(sfb_base), "l"(p.sfb_img + r * p.sfb_route_bytes), "r"(sfb_bytes), "r"(b_bar) : "memory");
        }
        if (load_b) { b_route = route; b_loads++; }

        if (warp < 4) {
            // ===== epilogue: tile row t = 32 * warp + lane =================================================
            if (lane == 0) mbar_wait(accum_bar, (uint32_t)pass & 1u, abort_flag, p.status);
            __syncwarp();
            tc_fence_after();
            const int row = rt * 128 + warp * 32 + lane;                 // row within the route's matrix
            const bool live = row < p.rows_per_route;
            const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + kMxColD;
            // the pieces' columns (smallest piece first within a thread's eight) of the issuing threads' partial sums
            float s0 = 0.f, s1 = 0.f;
#pragma unroll
            for (int i = kMxTmaSplit - 1; i >= 0; i--) {
                if (i >= nkg) continue;                                  // fewer K groups than issuing threads: nothing was accumulated there
                uint32_t d0[8], d1[8];
                tmem_ld8(taddr + 8u * i, d0);
                if (EXPAND) tmem_ld8(taddr + kColMat + 8u * i, d1);
                tmem_ld_wait();
                float t0 = 0.f, t1 = 0.f;
#pragma unroll
                for (int c = 7; c >= 0; c--) { t0 = __fadd_rn(t0, __uint_as_float(d0[c])); if (EXPAND) t1 = __fadd_rn(t1, __uint_as_float(d1[c])); }
                s0 = __fadd_rn(s0, t0); s1 = __fadd_rn(s1, t1);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tmem_free);
            if (EXPAND) {
                float a = 0.f;
                if (live) {
                    const float sg = s0, su = s1;
                    const size_t bi = ((size_t)e * p.rows_per_route + row) * p.bias_stride;
                    const float gate = __fadd_rn(sg, bf16_round(p.b0[bi]));
                    const float up = __fadd_rn(su, bf16_round(__fadd_rn(p.b1[bi], 1.0f)));
                    a = swiglu_clipped(gate, up);
                    p.act_out[(size_t)route * p.rows_per_route + row] = a;
                }
                // this warp's 32 rows are one block of the down kernel's contraction: split it into pieces here
                // (lane l of the split holds element (l >> 1) + 16 * (l & 1) of the block)
                const int first = rt * 128 + warp * 32;
                if (first < p.rows_per_route) {                          // rows_per_route is a multiple of 32: the block is whole or absent
                    const float v = __shfl_sync(0xffffffffu, a, (lane >> 1) + 16 * (lane & 1));
                    mx_split_block(v, lane, p.act_b + (size_t)route * p.act_b_route_bytes, p.act_sfb + (size_t)route * p.act_sfb_route_bytes, 8u, 0u,
                                   (uint32_t)first >> 5);
                }
            } else if (live) {
                float sy = s0;
                if (p.b0) sy = __fadd_rn(sy, bf16_round(p.b0[((size_t)e * p.rows_per_route + row) * p.bias_stride]));
                p.y[(size_t)route * p.rows_per_route + row] = f32_to_bf16_bits(sy);
                if (p.residual) {
                    __threadfence();
                    const uint32_t seen = atomicAdd(p.arrivals + row, 1u);
                    if (seen == (uint32_t)(p.routes - 1)) {
                        p.arrivals[row] = 0;                                            // ready for the next call
                        if (*reinterpret_cast<volatile uint32_t*>(p.status) == 0u) {
                            __threadfence();
                            float sres = 0.0f;
                            for (int r = 0; r < p.routes; r++)
                                sres = __fmaf_rn(bf16_bits_to_f32(__ldcg(p.y + (size_t)r * p.rows_per_route + row)), p.probs[r], sres);
                            if (p.round_sum) sres = bf16_round(sres);
                            p.residual[row] = f32_to_bf16_bits(__fadd_rn(bf16_bits_to_f32(p.residual[row]), sres));
                        }
                    }
                }
            }
        } else if (warp < kCopyWarp) {
            if (lane == 0) {
                // ===== MMA issue: kMxTmaSplit threads per matrix, thread ki takes the K groups g = ki mod kMxTmaSplit =====
                const int mat = (warp - 4) / kMxTmaSplit, ki = (warp - 4) % kMxTmaSplit;
                if (pass > 0) mbar_wait(tmem_free, (uint32_t)(pass - 1) & 1u, abort_flag, p.status);
                if (load_b) {
                    mbar_wait(b_bar, (uint32_t)(b_loads - 1) & 1u, abort_flag, p.status);
                    tc_fence_after();
                }
                const uint32_t d_t = tmem_base + kMxColD + (uint32_t)mat * kColMat + 8u * (uint32_t)ki;
                // scale columns of this thread alone (a thread's tcgen05.cp and mma run in the order it issued them): 8 of the
                // weights, 8 of the activation's pieces, rewritten every K group
                const uint32_t sfa_t = tmem_base + kMxColSfa + 16u * (uint32_t)(warp - 4), sfb_t = sfa_t + 8u;
                bool first = true;
                for (int g = ki; g < nkg; g += kMxTmaSplit) {
                    const int n = step0 + g, as = n % kMxTmaStages;
                    mbar_wait(a_full(as), (uint32_t)(n / kMxTmaStages) & 1u, abort_flag, p.status);
                    tc_fence_after();
                    const uint32_t stage = a_base + (uint32_t)as * kStage;
                    const uint32_t sfa_smem = stage + NMAT * 16384u + (uint32_t)mat * 1024u;
                    mx_cp_scales(sfa_t, mx_sf_desc(sfa_smem));
                    mx_cp_scales(sfa_t + 4u, mx_sf_desc(sfa_smem + 512u));
                    mx_cp_scales(sfb_t, mx_sf_desc(sfb_base + 1024u * (uint32_t)g));
                    mx_cp_scales(sfb_t + 4u, mx_sf_desc(sfb_base + 1024u * (uint32_t)g + 512u));
                    const uint64_t ad = umma_desc(stage + (uint32_t)mat * 16384u);
                    const uint64_t bd = umma_desc(b_base + (uint32_t)g * (NCOL * 128u));
#pragma unroll
                    for (int kk = 0; kk < 4; kk++) {
                        const uint32_t sfid = (uint32_t)(kk & 1) * 2u;
                        umma_mxf4(d_t, ad + 2u * kk, bd + 2u * kk, mx_idesc(NCOL, sfid), sfa_t + 4u * (kk >> 1), sfb_t + 4u * (kk >> 1),
                                  (!first || kk) ? 1u : 0u);
                    }
                    first = false;
                    umma_commit(a_empty(as));
                }
                umma_commit(accum_bar);
            }
        } else if (warp == kCopyWarp && lane == 0) {
            // ===== the weight tiles and their scale tiles, one K group per stage ================================
            const size_t t0 = ((size_t)e * tpr + rt) * nkg;
            const unsigned char* sf0 = q.sf[0] + t0 * 1024;
            const unsigned char* sf1 = NMAT > 1 ? q.sf[1] + t0 * 1024 : nullptr;
            const unsigned char* c0 = q.codes[0] + (t0 << 14);
            const unsigned char* c1 = NMAT > 1 ? q.codes[1] + (t0 << 14) : nullptr;
            for (int g = 0; g < nkg; g++) {
                const int n = step0 + g, as = n % kMxTmaStages;
                const uint32_t stage = a_base + (uint32_t)as * kStage;
                mbar_wait(a_empty(as), ((uint32_t)(n / kMxTmaStages) & 1u) ^ 1u, abort_flag, p.status);
                mbar_arrive_expect_tx(a_full(as), kStage);
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(stage),
                             "l"(c0 + ((size_t)g << 14)), "r"(16384u), "r"(a_full(as)) : "memory");
                if (NMAT > 1)
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(stage + 16384u),
                                 "l"(c1 + ((size_t)g << 14)), "r"(16384u), "r"(a_full(as)) : "memory");
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(stage + NMAT * 16384u),
                             "l"(sf0 + (size_t)g * 1024), "r"(1024u), "r"(a_full(as)) : "memory");
                if (NMAT > 1)
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(stage + NMAT * 16384u + 1024u),
                                 "l"(sf1 + (size_t)g * 1024), "r"(1024u), "r"(a_full(as)) : "memory");
            }
        }
        step0 += nkg;
    }
    __syncthreads();
    if (*abort_flag) {
        for (int i = 0; i < 64; i++) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 4) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kMxTmemCols);
    }
}

}  // namespace oco
