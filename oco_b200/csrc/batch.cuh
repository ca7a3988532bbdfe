// Expert products for a few tokens (about two routes per expert, e.g. a decode batch of 64 over
// 128 experts). The work is still memory-bound, and a 32-route tile would decode every weight
// block for two live columns, so the rows are streamed as in the single-token kernels
// (decode.cuh) with the eight columns of the MMA's B operand holding up to eight routes of the
// same expert. Numerics are the tile kernels': half operands, fp32 accumulation, the same
// epilogues (reference expert_up_tensor / expert_down_tensor, shaders/experts/projections.metal:
// 185-420, taken at a tile height of eight).
//
//   route_plan_kernel (tile_rows = 8)  ->  groups of up to 8 routes of one expert
//   batch_fragments_kernel             ->  each group's token rows as B fragments
//   batch_expand_kernel                ->  activations (half, expert-sorted) + the down stage's fragments
//   batch_down_kernel                  ->  bf16 expert outputs in route order
#pragma once
#include "decode.cuh"
#include "gemm.cuh"

namespace oco {

constexpr int kBatchWarps = 16;                     // one CTA per SM; the group's fragments take 512 bytes a block
constexpr int kBatchThreads = kBatchWarps * 32;
constexpr int kBatchCols = 8;
constexpr int kBatchFragBlock = kBatchCols * 64;    // bytes of one block's B fragments

__host__ __device__ inline size_t batch_smem_bytes(int nkb) {
    return (size_t)nkb * kBatchFragBlock + kMiscBytes + (size_t)kBatchWarps * kScaleBytes +
           (size_t)kBatchWarps * 2 * kStageBytes + 16;
}

// Position (in halves) of element k of column `col` in a group's fragments:
// frag[((kb * 8 + col) * 4 + tig) * 4 + slot] is a half2 (element 4*tig+slot, element 4*tig+slot+16).
__host__ __device__ inline size_t batch_frag_pos(int k, int col) {
    const int kb = k >> 5, j = k & 31, jj = j & 15, sel = j >> 4, tig = jj >> 2, slot = jj & 3;
    return ((((size_t)kb * kBatchCols + col) * 4 + tig) * 4 + slot) * 2 + sel;
}

// The token rows of every route group as B fragments (bf16 -> half, zero in unused columns).
// grid: max groups; one thread per 16-byte fragment piece (block, column, tig).
__global__ void __launch_bounds__(256) batch_fragments_kernel(const uint16_t* __restrict__ x,
                                                              const uint32_t* __restrict__ tiles,
                                                              const uint32_t* __restrict__ tile_count,
                                                              const uint32_t* __restrict__ offsets,
                                                              const uint32_t* __restrict__ route_of_row, int per_row,
                                                              int H, uint4* __restrict__ frag) {
    if (blockIdx.x >= *tile_count) return;
    const uint32_t expert = tiles[2 * blockIdx.x], begin = tiles[2 * blockIdx.x + 1];
    const uint32_t row0 = offsets[expert] + begin, count = offsets[expert + 1] - offsets[expert];
    const int n = (int)min((uint32_t)kBatchCols, count - begin);
    const int nkb = H / 32;
    uint4* out = frag + (size_t)blockIdx.x * nkb * (kBatchFragBlock / 16);
    for (int i = threadIdx.x; i < nkb * 32; i += 256) {
        const int kb = i >> 5, col = (i >> 2) & 7, tig = i & 3;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (col < n) {
            const uint32_t token = route_of_row[row0 + col] / (uint32_t)per_row;
            const uint16_t* src = x + (size_t)token * H + kb * 32 + 4 * tig;
            const uint2 lo = *reinterpret_cast<const uint2*>(src), hi = *reinterpret_cast<const uint2*>(src + 16);
            auto pair = [](uint32_t a, uint32_t b) {          // (bf16 a, bf16 b) -> half2
                __half2 h = __floats2half2_rn(__uint_as_float(a << 16), __uint_as_float(b << 16));
                return *reinterpret_cast<uint32_t*>(&h);
            };
            v.x = pair(lo.x & 0xffffu, hi.x & 0xffffu);
            v.y = pair(lo.x >> 16, hi.x >> 16);
            v.z = pair(lo.y & 0xffffu, hi.y & 0xffffu);
            v.w = pair(lo.y >> 16, hi.y >> 16);
        }
        out[i] = v;
    }
}

struct BatchParams {
    const uint8_t* w0;        // expand: gate rows (up rows when not gated); down: the down rows
    const uint8_t* w1;        // expand, gated: up rows
    const float* b0;
    const float* b1;
    const uint32_t* tiles;    // (expert, first row within the expert) per route group
    const uint32_t* tile_count;
    const uint32_t* offsets;
    const uint32_t* route_of_row;
    const __half* frag_in;    // [group][n_in / 32] blocks of 512 bytes
    __half* frag_out;         // expand: the down stage's fragments, [group][n_out / 32] blocks
    uint16_t* out;            // expand: half [R, n_out] expert-sorted, operand order; down: bf16 [R, n_out] route order
    int n_in, n_out;          // contraction length, output features
    int parts;                // CTAs per group
    uint32_t row_bytes;       // bytes from one weight row of a matrix to its next row
    int bias_stride;          // floats from one feature's bias to the next
    uint32_t* status;
};

// EPI as in gemm.cuh. grid: parts * max groups, CTA = (group, part); the part's units (16 weight
// rows each) go round the warps.
template <int FMT, int EPI>
__global__ void __launch_bounds__(kBatchThreads, 1) batch_rows_kernel(const BatchParams p) {
    constexpr bool GATED = epi_gated(EPI);
    constexpr bool DOWN = EPI == kEpiDownBf16;
    constexpr int ROWS = GATED ? 8 : 16;              // output features per unit
    extern __shared__ __align__(16) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, g = lane >> 2, tig = lane & 3;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const int group = blockIdx.x / p.parts, part = blockIdx.x - group * p.parts;
    if ((uint32_t)group >= *p.tile_count) return;
    const uint32_t expert = p.tiles[2 * group], begin = p.tiles[2 * group + 1];
    const uint32_t row0 = p.offsets[expert] + begin, count = p.offsets[expert + 1] - p.offsets[expert];
    const int n = (int)min((uint32_t)kBatchCols, count - begin);
    const int nkb = p.n_in / 32;
    const uint32_t part_off = (uint32_t)nkb * kBatchFragBlock;
    float* misc = reinterpret_cast<float*>(smem + part_off);
    volatile uint32_t* give_up = reinterpret_cast<volatile uint32_t*>(misc) + 496;
    const uint32_t xbar = smem_u32(smem) + part_off + 1920u;
    const uint32_t stab = part_off + kMiscBytes + (uint32_t)warp * kScaleBytes;
    const uint32_t ring = part_off + kMiscBytes + (uint32_t)kBatchWarps * kScaleBytes + (uint32_t)warp * 2 * kStageBytes;
    if (tid == 0) *give_up = 0u;
    fetch_fragments(smem, p.frag_in + (size_t)group * nkb * (kBatchFragBlock / 2), (uint32_t)nkb * kBatchFragBlock, xbar, warp, lane);

    RowStream<FMT, 2, kBatchCols> rs;
    rs.init(smem, ring, stab, part_off + 1280u + (uint32_t)warp * 16u, give_up, p.status, lane);
    rs.ncols = n;
    __syncthreads();          // the mbarriers exist
    const uint32_t xlane = (uint32_t)((g * 4 + tig) * 16);
    const int units = p.n_out / ROWS;
    const int per_part = (units + p.parts - 1) / p.parts;
    const int u_end = min(units, (part + 1) * per_part);
    // the routes of this lane's two columns
    const int c0 = 2 * tig, c1 = 2 * tig + 1;
    uint32_t orow0 = 0, orow1 = 0;
    if (c0 < n) orow0 = DOWN ? p.route_of_row[row0 + c0] : row0 + c0;
    if (c1 < n) orow1 = DOWN ? p.route_of_row[row0 + c1] : row0 + c1;
    __half* fout = DOWN ? nullptr : p.frag_out + (size_t)group * (p.n_out / 32) * (kBatchFragBlock / 2);
    bool fetched = false;
    for (int u = part * per_part + warp; u < u_end; u += kBatchWarps) {
        const int f0 = u * ROWS;
        const size_t off = ((size_t)expert * p.n_out + f0) * p.row_bytes;
        if (GATED) rs.begin(p.w0 + off, p.w1 + off, p.row_bytes, 0, nkb);
        else rs.begin(p.w0 + off, p.w0 + off + (size_t)8 * p.row_bytes, p.row_bytes, 0, nkb);
        // biases travel while the rows stream: accumulator rows g (span A) and g (span B)
        const int fa = f0 + g, fb = GATED ? fa : fa + 8;
        float bias_a = 0.f, bias_b = 0.f;
        if (p.b0) bias_a = bf16_round(__ldg(p.b0 + ((size_t)expert * p.n_out + fa) * p.bias_stride));
        if (GATED) {
            if (EPI == kEpiSwigluF16) bias_b = bf16_round(__fadd_rn(__ldg(p.b1 + ((size_t)expert * p.n_out + fa) * p.bias_stride), 1.0f));
        } else if (p.b0) {
            bias_b = bf16_round(__ldg(p.b0 + ((size_t)expert * p.n_out + fb) * p.bias_stride));
        }
        float sum[4] = {0.f, 0.f, 0.f, 0.f};
        if (!fetched) { mbar_wait(xbar, 0u, give_up, p.status); fetched = true; }
        rs.run(xlane, sum);
        // sum[0..1]: row g of span A x columns c0, c1; sum[2..3]: row g of span B
        auto put = [&](int col, uint32_t orow, int f, uint16_t h) {
            if (DOWN) {
                p.out[(size_t)orow * p.n_out + f] = h;
            } else {
                p.out[(size_t)orow * p.n_out + operand_pos(FMT, f)] = h;
                reinterpret_cast<uint16_t*>(fout)[batch_frag_pos(f, col)] = h;
            }
        };
        if (GATED) {
            if (c0 < n) put(c0, orow0, fa, epilogue_value<EPI>(__fadd_rn(sum[0], bias_a), __fadd_rn(sum[2], bias_b)));
            if (c1 < n) put(c1, orow1, fa, epilogue_value<EPI>(__fadd_rn(sum[1], bias_a), __fadd_rn(sum[3], bias_b)));
        } else {
            if (c0 < n) {
                put(c0, orow0, fa, epilogue_value<EPI>(__fadd_rn(sum[0], bias_a), 0.f));
                put(c0, orow0, fb, epilogue_value<EPI>(__fadd_rn(sum[2], bias_b), 0.f));
            }
            if (c1 < n) {
                put(c1, orow1, fa, epilogue_value<EPI>(__fadd_rn(sum[1], bias_a), 0.f));
                put(c1, orow1, fb, epilogue_value<EPI>(__fadd_rn(sum[3], bias_b), 0.f));
            }
        }
    }
}

}  // namespace oco
