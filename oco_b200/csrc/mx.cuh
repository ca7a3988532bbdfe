// MXFP4 expert rows on the block-scaled tensor-core path (tcgen05.mma kind::mxf4, UE8M0 scales per 32
// elements, fp32 accumulators in tensor memory), for one token and for a few tokens.
//
// A GGUF MXFP4 block is already what this MMA kind multiplies: sixteen bytes of e2m1 pairs and one
// E8M0 scale. Nothing is decoded: the packed rows stream from HBM into shared memory (TMA tensor
// copies), producer warps move each block's sixteen code bytes to the 16-byte-aligned position the
// MMA descriptor wants and its scale byte into the scale-factor tile, and one thread issues the
// MMAs. A code byte holds elements j and j + 16 of its block while the tensor core reads a byte as
// two consecutive contraction positions, so the activation operand is laid out in the same
// "operand order" (position 2j = element j, position 2j + 1 = element j + 16); a dot product does
// not care in which order k is visited.
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
// The rows of a GGUF tensor are `row_bytes` apart, not a multiple of 16 bytes, so no single tensor
// map covers them. Rows PR apart (PR = 8, or 16 when 8 rows are not a multiple of 16 bytes) start at
// the same offset within a 16-byte word: there is one tensor map per residue j = row mod PR, a 2-D
// view [row / PR][16-byte envelope of the row] with pitch PR * row_bytes, and one copy brings the
// same K range of every PR-th row of a CTA's share. Reads past a row's end are out of the view's
// bounds and come back as zeros.
#pragma once
#include "gemm.cuh"
#include "mx_pieces.cuh"

namespace oco {

constexpr int kMxGroupBlocks = 8;                    // blocks per K group: one 128-byte swizzle row of e2m1 codes
constexpr int kMxGroupBytes = kMxGroupBlocks * 17;   // packed bytes of a K group in a row
constexpr int kMxSlot = 176;                         // raw bytes per row and K group: 136 + 15 of misalignment, 16 x odd
constexpr int kMxMapSizes = 5;                       // tensor maps with 1, 2, 4, 8, 16 rows per box
constexpr int kMxMaxResidues = 16;
constexpr int kMxThreads = 10 * 32;                  // 8 producer / epilogue warps, the MMA warp, the TMA warp
constexpr int kMxMmaWarp = 8, kMxTmaWarp = 9;
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
__device__ __forceinline__ void tma_load_2d_gmap(uint32_t smem_dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_dst), "l"(map), "r"(c0), "r"(c1), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}

struct MxParams {
    const CUtensorMap* maps;      // device memory: [tensor][kMxMaxResidues][kMxMapSizes]
    const uint8_t* w[2];          // first packed row of each matrix (expand: gate, up; down: down)
    int tensor[2];                // which tensor's maps each matrix uses
    int n_mat;
    uint32_t row_stride;          // bytes between consecutive rows of a matrix
    int PR;                       // rows per tensor-map period
    int K;                        // contraction length
    int rows_per_route;           // output rows of one expert's matrix
    int routes;
    int region;                   // raw bytes per residue, matrix and stage (a multiple of 128, see mx_region_bytes)
    int raw_stages;
    const uint32_t* ids;          // [routes] expert of each route; null = expert 0
    // B operand
    const unsigned char* b_img;   // expand: the token's pieces, mx_b_bytes(8, nkb)
    const unsigned char* sfb_img; //         and their scales, mx_sfb_bytes(nkb)
    const float* act;             // down: f32 [routes][K] activations, split by the kernel itself
    // epilogue
    const float* b0;              // expand: gate bias; down: bias (or null)
    const float* b1;              // expand: up bias
    int bias_stride;
    float* act_out;               // expand: f32 [routes][rows_per_route]
    uint16_t* y;                  // down: bf16 [routes][rows_per_route]
    uint32_t* arrivals;           // down: one zeroed counter per output row
    const float* probs;
    uint16_t* residual;
    int round_sum;
    uint32_t* status;
};

// Shared memory: A stages | SFA atoms | B image | SFB image | down: nothing more | control | raw ring.
constexpr uint32_t kMxCtrlBytes = 3072;             // barriers | tensor-memory slot, flags | copy list | row offsets
__host__ __device__ inline uint32_t mx_fixed_smem(int n_mat, uint32_t n_cols, uint32_t nkb) {
    return (uint32_t)kMxAStages * n_mat * (16384u + 1024u) + mx_b_bytes(n_cols, nkb) + mx_sfb_bytes(nkb) + kMxCtrlBytes + 1024u;
}
__host__ __device__ inline uint32_t mx_raw_stage_bytes(int n_mat, int PR, int region) { return (uint32_t)n_mat * PR * region; }

// The copies that bring units [u0, u1) (one row per unit and residue) into a residue's raw region: runs of
// units inside one route are cut into boxes of 16, 8, 4, 2, 1 rows; a box holds its rows kMxSlot bytes
// apart and starts on a 128-byte boundary, as a TMA destination must. Calls emit(y offset within the
// route, log2 rows, byte offset) per box and row(s, byte offset) per unit; returns the bytes used.
template <class Emit, class Row>
__host__ __device__ inline uint32_t mx_plan_copies(int u0, int u1, int upr, Emit emit, Row row) {
    uint32_t off = 0;
    for (int u = u0; u < u1;) {
        const int r = u / upr, su = u - r * upr;
        int left = min(u1 - u, upr - su), y = su;
        for (int lg = kMxMapSizes - 1; lg >= 0; lg--) {
            if (left & (1 << lg)) {
                off = (off + 127u) & ~127u;
                emit(r, y, lg, off);
                for (int i = 0; i < (1 << lg); i++) row(u - u0 + (y - su) + i, off + (uint32_t)i * kMxSlot);
                off += (uint32_t)(1 << lg) * kMxSlot;
                y += 1 << lg; left -= 1 << lg;
            }
        }
        u += min(u1 - u, upr - su);
    }
    return (off + 127u) & ~127u;
}
// The units of a pass that starts at u0 for a CTA whose share ends at u_end.
__host__ __device__ inline int mx_pass_end(int u0, int u_end, int upr, int PR, bool two_routes_at_most) {
    int u1 = min(u_end, u0 + 128 / PR);
    if (two_routes_at_most) u1 = min(u1, (u0 / upr + 2) * upr);
    return u1;
}

// EXPAND: two matrices (gate, up), one activation vector for all routes (8 columns), fused clipped SwiGLU,
// f32 activations out. Otherwise: one matrix, the activations of up to two routes per pass (16 columns),
// bf16 expert outputs and, by whoever completes an output-row block last, the weighted sum onto the residual.
// Grid: one CTA per SM; CTA c owns the units [c U / G, (c + 1) U / G) where a unit is PR consecutive
// rows of one route (and of both matrices), U = routes * rows_per_route / PR.
template <bool EXPAND>
__global__ void __launch_bounds__(kMxThreads, 1) mx_rows_kernel(const MxParams p) {
    constexpr int NMAT = EXPAND ? 2 : 1;
    constexpr uint32_t NCOL = EXPAND ? 8u : 16u;
    extern __shared__ unsigned char smem_raw[];
    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const int PR = p.PR;
    const int nkb = p.K >> 5, nkg = (nkb + 7) >> 3;
    const int upr = p.rows_per_route / PR;                      // units per route
    const int units_total = p.routes * upr;
    const int u_begin = (int)((long long)blockIdx.x * units_total / gridDim.x);
    const int u_end = (int)((long long)(blockIdx.x + 1) * units_total / gridDim.x);
    const int units_pass = 128 / PR;

    // ---- shared memory carve-up ------------------------------------------------------------------
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char* gen = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t a_base = base;                                               // [stage][mat] 16 KB tiles
    const uint32_t sfa_base = a_base + kMxAStages * NMAT * 16384u;              // [stage][mat] two 512-byte atoms
    const uint32_t b_base = sfa_base + kMxAStages * NMAT * 1024u;
    const uint32_t sfb_base = b_base + mx_b_bytes(NCOL, nkb);
    const uint32_t ctrl = sfb_base + mx_sfb_bytes(nkb);
    const uint32_t raw_base = ctrl + kMxCtrlBytes;
    const uint32_t raw_stage_bytes = mx_raw_stage_bytes(NMAT, PR, p.region);
    unsigned char* ctrl_gen = gen + (ctrl - base);
    auto raw_full = [&](int s) { return ctrl + 8u * s; };
    auto raw_empty = [&](int s) { return ctrl + 8u * (16 + s); };
    auto a_full = [&](int s) { return ctrl + 8u * (32 + s); };
    auto a_empty = [&](int s) { return ctrl + 8u * (34 + s); };
    const uint32_t accum_bar = ctrl + 8u * 36, b_bar = ctrl + 8u * 37, tmem_free = ctrl + 8u * 38;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ctrl_gen + 512);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    // per pass: the copy list of a residue (the same for every residue and matrix) and each unit's place
    struct Copy { int y, lg; uint32_t off, pad; };
    Copy* copies = reinterpret_cast<Copy*>(ctrl_gen + 1024);                    // at most 64 entries
    uint32_t* row_off = reinterpret_cast<uint32_t*>(ctrl_gen + 2048);           // [units of a pass]
    int* ncopies = reinterpret_cast<int*>(ctrl_gen + 520);

    pdl_launch_dependents();
    if (tid == 0) {
        for (int s = 0; s < p.raw_stages; s++) { mbar_init(raw_full(s), 1); mbar_init(raw_empty(s), 4 * NMAT); }
        for (int s = 0; s < kMxAStages; s++) { mbar_init(a_full(s), 4 * NMAT); mbar_init(a_empty(s), 1); }
        mbar_init(accum_bar, 1);
        mbar_init(b_bar, 1);
        mbar_init(tmem_free, 4);
        *abort_flag = 0;
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

    if (EXPAND && u_begin < u_end) {
        // the token's pieces and their scales, prepared by the router kernel
        if (tid == 0) {
            const uint32_t bb = mx_b_bytes(NCOL, nkb), sb = mx_sfb_bytes(nkb);
            mbar_arrive_expect_tx(b_bar, bb + sb);
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(b_base), "l"(p.b_img), "r"(bb), "r"(b_bar) : "memory");
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(sfb_base), "l"(p.sfb_img), "r"(sb), "r"(b_bar) : "memory");
        }
    }

    int step0 = 0;            // K groups of earlier passes (ring and barrier phases run on)
    int pass = 0;
    int b_routes_first = -1;  // down: the routes whose pieces are in the B image
    for (int u0 = u_begin; u0 < u_end; pass++) {
        // a pass: up to 128 rows, and (down) units of at most two routes
        const int u1 = mx_pass_end(u0, u_end, upr, PR, !EXPAND);
        const int r_first = u0 / upr;
        const int n_units = u1 - u0;
        __syncthreads();      // the pass before is finished with the copy list and (down) the B image
        if (tid == 0) {
            int n = 0;
            mx_plan_copies(u0, u1, upr,
                           [&](int r, int y, int lg, uint32_t off) {
                               const uint32_t e = p.ids ? p.ids[r] : 0u;
                               if (n < 64) { copies[n].y = (int)e * upr + y; copies[n].lg = lg; copies[n].off = off; n++; }
                           },
                           [&](int s, uint32_t off) { row_off[s] = off; });
            *ncopies = n;
        }
        if (!EXPAND && r_first != b_routes_first) {
            // split the f32 activations of routes r_first, r_first + 1 into pieces (columns 0-7, 8-15)
            unsigned char* bimg = gen + (b_base - base);
            unsigned char* sfimg = gen + (sfb_base - base);
            const int nwarps = kMxThreads / 32;
            for (int i = warp; i < 2 * nkg * 8; i += nwarps) {
                const int rr = i / (nkg * 8), blk = i - rr * (nkg * 8);
                const int route = r_first + rr;
                float v = 0.0f;
                if (route < p.routes && blk < nkb) v = p.act[(size_t)route * p.K + blk * 32 + (lane >> 1) + 16 * (lane & 1)];
                mx_split_block(v, lane, bimg, sfimg, NCOL, 8u * rr, (uint32_t)blk);
            }
            b_routes_first = r_first;
            fence_proxy_async_smem();
        }
        __syncthreads();

        if (warp < 4 * NMAT) {
            // ===== producers: raw slot -> A tile row + scale bytes =================================
            const int mat = warp >> 2, q = warp & 3;
            const int t = q * 32 + lane;                                  // tile row
            // eight consecutive lanes hold eight consecutive units of one residue: their raw rows lie
            // kMxSlot = 16 x 11 bytes apart, so a 16-byte load per lane has no bank conflict
            const int j = t / units_pass, s = t - j * units_pass;
            const bool live = s < n_units;
            const uint32_t off0 = (uint32_t)((uintptr_t)(p.w[mat] + (size_t)j * p.row_stride) & 15u);
            const uint32_t slot_off = (uint32_t)((mat * PR + j) * p.region) + (live ? row_off[s] : 0u);
            const uint32_t a_row = (uint32_t)(t >> 3) * 1024u + (uint32_t)(t & 7) * 128u, sw = (uint32_t)(t & 7);
            for (int g = 0; g < nkg; g++) {
                const int n = step0 + g, rs = n % p.raw_stages, as = n % kMxAStages;
                if (lane == 0) {
                    mbar_wait(raw_full(rs), (uint32_t)(n / p.raw_stages) & 1u, abort_flag, p.status);
                    mbar_wait(a_empty(as), ((uint32_t)(n / kMxAStages) & 1u) ^ 1u, abort_flag, p.status);
                }
                __syncwarp();
                if (live) {
                    const uint32_t slot = raw_base + (uint32_t)rs * raw_stage_bytes + slot_off;
                    const uint32_t dl = (off0 + 8u * (uint32_t)g) & 15u;      // where the row's bytes start in the slot
                    uint32_t c[40];
#pragma unroll
                    for (int i = 0; i < 10; i++)
                        asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(c[4 * i]), "=r"(c[4 * i + 1]), "=r"(c[4 * i + 2]), "=r"(c[4 * i + 3]) : "r"(slot + 16u * i));
                    const uint32_t a_dst = a_base + (uint32_t)(as * NMAT + mat) * 16384u + a_row;
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
                        const uint32_t scale = (x[0] >> tb) & 0xffu;
                        const uint32_t k0 = __funnelshift_rc(x[0], x[1], tb + 8u), k1 = __funnelshift_rc(x[1], x[2], tb + 8u),
                                       k2 = __funnelshift_rc(x[2], x[3], tb + 8u), k3 = __funnelshift_rc(x[3], x[4], tb + 8u);
                        asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(a_dst + (((uint32_t)b ^ sw) << 4)), "r"(k0), "r"(k1), "r"(k2), "r"(k3) : "memory");
                        sfw[b >> 2] |= scale << (8 * (b & 3));
                    }
                    const uint32_t sf_dst = sfa_base + (uint32_t)(as * NMAT + mat) * 1024u + (uint32_t)lane * 16u + (uint32_t)q * 4u;
                    asm volatile("st.shared.b32 [%0], %1;" ::"r"(sf_dst), "r"(sfw[0]) : "memory");
                    asm volatile("st.shared.b32 [%0], %1;" ::"r"(sf_dst + 512u), "r"(sfw[1]) : "memory");
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) { mbar_arrive(a_full(as)); mbar_arrive(raw_empty(rs)); }
            }
            // ===== epilogue =============================================================================
            if (mat == 0) {
                if (lane == 0) mbar_wait(accum_bar, (uint32_t)pass & 1u, abort_flag, p.status);
                __syncwarp();
                tc_fence_after();
                const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + kMxColD;
                const int unit = u0 + s, route = unit / upr, row = (unit - route * upr) * PR + j;   // row within the route's matrix
                if (EXPAND) {
                    uint32_t dg[8], du[8];
                    tmem_ld8(taddr, dg);
                    tmem_ld8(taddr + 32u, du);
                    tmem_ld_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(tmem_free);
                    if (live) {
                        float sg = 0.f, su = 0.f;
#pragma unroll
                        for (int i = 7; i >= 0; i--) { sg = __fadd_rn(sg, __uint_as_float(dg[i])); su = __fadd_rn(su, __uint_as_float(du[i])); }
                        const uint32_t e = p.ids ? p.ids[route] : 0u;
                        const size_t bi = ((size_t)e * p.rows_per_route + row) * p.bias_stride;
                        const float gate = __fadd_rn(sg, bf16_round(p.b0[bi]));
                        const float up = __fadd_rn(su, bf16_round(__fadd_rn(p.b1[bi], 1.0f)));
                        p.act_out[(size_t)route * p.rows_per_route + row] = swiglu_clipped(gate, up);
                    }
                } else {
                    // both routes' columns; each lane keeps the eight of its own route
                    uint32_t d16[16], d[8];
                    tmem_ld16(taddr, d16);
                    tmem_ld_wait();
                    const bool second = live && route != r_first;
#pragma unroll
                    for (int i = 0; i < 8; i++) d[i] = second ? d16[8 + i] : d16[i];
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(tmem_free);
                    if (live) {
                        float sy = 0.f;
#pragma unroll
                        for (int i = 7; i >= 0; i--) sy = __fadd_rn(sy, __uint_as_float(d[i]));
                        const uint32_t e = p.ids ? p.ids[route] : 0u;
                        if (p.b0) sy = __fadd_rn(sy, bf16_round(p.b0[((size_t)e * p.rows_per_route + row) * p.bias_stride]));
                        p.y[(size_t)route * p.rows_per_route + row] = f32_to_bf16_bits(sy);
                    }
                    if (p.residual) {
                        // Whoever completes an output row last (the routes' rows are spread over CTAs) adds the
                        // weighted expert outputs to the residual (moe_sum, routing.metal:154-168). Nobody waits.
                        if (live) {
                            __threadfence();
                            const uint32_t seen = atomicAdd(p.arrivals + row, 1u);
                            if (seen == (uint32_t)(p.routes - 1)) {
                                p.arrivals[row] = 0;                                        // ready for the next call
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
            }
        } else if (warp == kMxMmaWarp) {
            if (lane == 0) {
                // ===== MMA issue ========================================================================
                if (pass == 0) {
                    if (EXPAND) mbar_wait(b_bar, 0u, abort_flag, p.status);
                } else {
                    mbar_wait(tmem_free, (uint32_t)(pass - 1) & 1u, abort_flag, p.status);   // accumulators of the pass before are read
                }
                tc_fence_after();
                if (EXPAND ? pass == 0 : true) {
                    // scales of the B operand: four blocks per copy
                    for (int i = 0; i < (nkb + 3) / 4; i++) mx_cp_scales(tmem_base + kMxColSfb + 4u * i, mx_sf_desc(sfb_base + 512u * i));
                }
                for (int g = 0; g < nkg; g++) {
                    const int n = step0 + g, as = n % kMxAStages;
                    mbar_wait(a_full(as), (uint32_t)(n / kMxAStages) & 1u, abort_flag, p.status);
                    tc_fence_after();
#pragma unroll
                    for (int mat = 0; mat < NMAT; mat++) {
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
                    }
                    umma_commit(a_empty(as));
                }
                umma_commit(accum_bar);
            }
        } else if (warp == kMxTmaWarp) {
            // ===== packed rows by TMA: lane j copies the rows with residue j =======================
            const int nc = *ncopies;
            // the tensor maps live in global memory (written by a host copy): acquire them for the TMA unit
            if (pass == 0 && lane < PR) {
#pragma unroll
                for (int mat = 0; mat < NMAT; mat++)
                    for (int lg = 0; lg < kMxMapSizes; lg++)
                        asm volatile("fence.proxy.tensormap::generic.acquire.gpu [%0], 128;" ::"l"(p.maps + ((size_t)p.tensor[mat] * kMxMaxResidues + lane) * kMxMapSizes + lg) : "memory");
            }
            uint32_t off0[NMAT];
#pragma unroll
            for (int mat = 0; mat < NMAT; mat++) off0[mat] = (uint32_t)((uintptr_t)(p.w[mat] + (size_t)lane * p.row_stride) & 15u);
            const uint32_t stage_tx = (uint32_t)(NMAT * PR * n_units * kMxSlot);
            for (int g = 0; g < nkg; g++) {
                const int n = step0 + g, rs = n % p.raw_stages;
                if (lane == 0) {
                    mbar_wait(raw_empty(rs), ((uint32_t)(n / p.raw_stages) & 1u) ^ 1u, abort_flag, p.status);
                    mbar_arrive_expect_tx(raw_full(rs), stage_tx);
                }
                __syncwarp();
                if (lane < PR && !*abort_flag) {
#pragma unroll
                    for (int mat = 0; mat < NMAT; mat++) {
                        const int x0 = (int)(((off0[mat] + (uint32_t)g * kMxGroupBytes) >> 4) * 2u);   // 8-byte elements, 16-byte aligned
                        const CUtensorMap* mj = p.maps + ((size_t)p.tensor[mat] * kMxMaxResidues + lane) * kMxMapSizes;
                        const uint32_t dst = raw_base + (uint32_t)rs * raw_stage_bytes + (uint32_t)((mat * PR + lane) * p.region);
                        for (int i = 0; i < nc; i++) tma_load_2d_gmap(dst + copies[i].off, mj + copies[i].lg, x0, copies[i].y, raw_full(rs));
                    }
                }
            }
        }
        step0 += nkg;
        u0 = u1;
    }
    __syncthreads();
    if (*abort_flag) {
        for (int i = 0; i < 64; i++) __nanosleep(1000);   // let copies in flight land before the CTA retires
        __syncthreads();
    }
    if (warp == kMxMmaWarp) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kMxTmemCols);
    }
}

}  // namespace oco
