// Single-token expert products: memory-bound streaming of the packed weight rows.
//
// Each CTA walks a list of work items. An item is 16 weight rows (8 gate + 8 up rows of one
// expert, or 8 rows each of two experts for the down projection) over the whole contraction
// length: two contiguous byte spans in the GGUF tensor. The spans are brought into a shared
// memory ring with 16-byte cp.async copies (coalesced, several items in flight per SM), the
// eight warps split the 32-element blocks of the item between them, and each warp multiplies its
// blocks with m16n8k16 tensor-core MMAs: the A fragment is the block's e2m1 codes converted to
// half in registers (one cvt per code byte), the B fragment is the activation vector split into
// hi + lo half parts in two of the eight columns, so the product is exact to f32 rounding. The
// block scale multiplies the block's partial sum afterwards in f32, as the reference's
// single-token kernels do (shaders/experts/projections.metal:57-59). A byte holds elements j and
// j + 16 of its block; the contraction index is permuted accordingly on the activation side
// instead of shuffling weights.
//
// FP32 FMA pipes cannot keep up with 4.25-bit weights at HBM rate (one FMA plus decode per weight
// needs more issue slots than an SM has per byte delivered), which is why the dot products ride
// on the tensor pipe even though the kernel is bandwidth-bound.
#pragma once
#include "common.cuh"
#include "router.cuh"

namespace oco {

constexpr int kDecodeThreads = 256;
constexpr int kDecodeWarps = 8;
constexpr int kExpandStages = 4;  // ring depth of the up/gate kernel
constexpr int kDownStages = 3;    // the down kernel also holds four fragment columns per block

// D = A * B with a zero accumulator, then D += A * B (fp32 accumulate, half operands).
__device__ __forceinline__ void mma16816_first(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds8(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

// Block codecs for the 32-element formats whose code byte j holds elements j (low nibble) and
// j + 16 (high nibble): MXFP4 (17 bytes, E8M0 scale) and Q4_0 (18 bytes, f16 scale, code - 8).
// `block` is the shared-memory byte address of the block; quads() turns a word of four code
// bytes into four half2 (element j, element j + 16).
template <int FMT>
struct Block32;
template <>
struct Block32<OCO_FMT_MXFP4> {
    static constexpr int kBytes = 17, kHeader = 1;
    __device__ static __forceinline__ float scale(uint32_t block) { return e8m0_scale(lds8(block)); }
    __device__ static __forceinline__ void quads(uint32_t w, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
        cvt_e2m1x2_x4(w, r0, r1, r2, r3);
    }
};
template <>
struct Block32<OCO_FMT_Q4_0> {
    static constexpr int kBytes = 18, kHeader = 2;
    __device__ static __forceinline__ float scale(uint32_t block) {
        return f16_bits_to_f32((uint16_t)(lds8(block) | (lds8(block + 1) << 8)));
    }
    __device__ static __forceinline__ uint32_t pair(uint32_t byte) {
        // 0x6400 | q is the half 1024 + q; subtracting 1032 leaves q - 8 exactly.
        uint32_t v = (byte & 0xfu) | ((byte & 0xf0u) << 12) | 0x64006400u;
        __half2 h = __hsub2(*reinterpret_cast<__half2*>(&v), __half2half2(__ushort_as_half((unsigned short)0x6408)));
        return *reinterpret_cast<uint32_t*>(&h);
    }
    __device__ static __forceinline__ void quads(uint32_t w, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
        r0 = pair(w); r1 = pair(w >> 8); r2 = pair(w >> 16); r3 = pair(w >> 24);
    }
};

// Dot products of 16 packed rows with the activation fragments, for the blocks kb = warp, warp + 8, ...
// rowA / rowB: shared-memory byte addresses of this lane's row g of the first / second span;
// xlane: address of this lane's fragment (uint4) for block 0; xstride: fragment bytes per block.
// sum[0..1] accumulate row g (two columns), sum[2..3] row g + 8. The warp's blocks are 8 apart, so
// every address advances by a multiple of four bytes per step and the word alignment of the code
// bytes is fixed for the whole loop.
template <int FMT>
__device__ __forceinline__ void rows_dot(uint32_t rowA, uint32_t rowB, uint32_t xlane, uint32_t xstride, int nkb,
                                         int warp, int tig, float (&sum)[4]) {
    using B = Block32<FMT>;
    constexpr uint32_t kStep = kDecodeWarps * B::kBytes;                 // 136 or 144 bytes
    uint32_t ba = rowA + (uint32_t)warp * B::kBytes, bb = rowB + (uint32_t)warp * B::kBytes;
    const uint32_t ca = ba + B::kHeader + 4u * tig, cb = bb + B::kHeader + 4u * tig;
    const uint32_t shA = (ca & 3u) * 8u, shB = (cb & 3u) * 8u;
    uint32_t a4 = ca & ~3u, b4 = cb & ~3u;
    uint32_t xa = xlane + (uint32_t)warp * xstride;
    const uint32_t xstep = kDecodeWarps * xstride;
#pragma unroll 2
    for (int kb = warp; kb < nkb; kb += kDecodeWarps) {
        const uint32_t wa = __funnelshift_r(lds32(a4), lds32(a4 + 4), shA);
        const uint32_t wb = __funnelshift_r(lds32(b4), lds32(b4 + 4), shB);
        const float sa = B::scale(ba), sb = B::scale(bb);
        const uint4 xf = lds128(xa);
        uint32_t qa0, qa1, qa2, qa3, qb0, qb1, qb2, qb3;
        B::quads(wa, qa0, qa1, qa2, qa3);
        B::quads(wb, qb0, qb1, qb2, qb3);
        float acc[4];
        mma16816_first(acc, qa0, qb0, qa1, qb1, xf.x, xf.y);
        mma16816(acc, qa2, qb2, qa3, qb3, xf.z, xf.w);
        sum[0] = __fmaf_rn(acc[0], sa, sum[0]);
        sum[1] = __fmaf_rn(acc[1], sa, sum[1]);
        sum[2] = __fmaf_rn(acc[2], sb, sum[2]);
        sum[3] = __fmaf_rn(acc[3], sb, sum[3]);
        a4 += kStep; b4 += kStep; ba += kStep; bb += kStep; xa += xstep;
    }
}

// Issues the cp.async copies of one byte span [src, src + bytes) into `dst` (16-byte aligned),
// widened to whole 16-byte chunks. Returns nothing; the span's first byte lands at dst + (src & 15).
__device__ __forceinline__ void copy_span_async(uint8_t* dst, const uint8_t* src, uint32_t bytes, int tid) {
    uintptr_t a = (uintptr_t)src;
    const uint8_t* base = (const uint8_t*)(a & ~(uintptr_t)15);
    uint32_t chunks = (((uint32_t)a & 15u) + bytes + 15u) >> 4;
    uint32_t d = smem_u32(dst);
    for (uint32_t i = tid; i < chunks; i += kDecodeThreads) cp_async16(d + i * 16u, base + (size_t)i * 16u);
}

// Splits f32 values into hi + lo halves and scatters them into the B-fragment layout:
// frag[((kb * COLS + col) * 4 + tig) * 4 + slot] is a half2 (element 4*tig+slot, element 4*tig+slot+16)
// of block kb; hi goes to column `col`, lo to column `col + 1`.
__device__ __forceinline__ void frag_store(__half* frag, int cols, int col, int k, float v) {
    __half hi = __float2half_rn(v);
    float rem = nonfinite(v) ? 0.0f : v - __half2float(hi);
    __half lo = __float2half_rn(rem);
    int kb = k >> 5, j = k & 31, jj = j & 15, sel = j >> 4, tig = jj >> 2, slot = jj & 3;
    size_t at = ((((size_t)kb * cols + col) * 4 + tig) * 4 + slot) * 2 + sel;
    frag[at] = hi;
    frag[at + (size_t)16 * 2] = lo;  // next column: 4 tig * 4 slots * 2 halves further
}

struct DecodeExpandParams {
    const uint8_t* gate_w;   // null when not gated
    const uint8_t* up_w;
    const float* gate_b;
    const float* up_b;
    const uint16_t* x;       // bf16 [H]
    const float* logits;     // f32 [E]
    const float* sel_bias;
    uint32_t* ids;           // out [K]
    float* probs;            // out [K]
    float* act;              // out f32 [K, F] (for inspection)
    __half* actfrag;         // out: B fragments of the down projection, [ceil(K/2)][F/32][4][4][4] half2
    int H, F, E, K, normalize;
    float scale;
    uint32_t row_bytes;      // bytes of one packed row of length H
    uint32_t span_cap;       // shared-memory bytes reserved per span
};

// Up (and gate) products of the K selected experts for one token, with the activation fused
// (reference expert_expand, projections.metal:78-137; matvec_q4 + relu^2, vector.metal:155-228).
// Every CTA repeats the top-k selection from the logits, as the reference does per SIMD group.
// GATED: item = 8 gate rows + 8 up rows (columns c0..c0+7); otherwise 16 up rows.
template <int ARCH, int FMT>
__global__ void __launch_bounds__(kDecodeThreads) decode_expand_kernel(const DecodeExpandParams p) {
    constexpr int kDecodeStages = kExpandStages;
    constexpr bool GATED = ARCH != OCO_ARCH_NEMOTRON;
    constexpr int COLS_PER_ITEM = GATED ? 8 : 16;
    using B = Block32<FMT>;
    extern __shared__ __align__(16) unsigned char smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tig = lane & 3;
    const int nkb = p.H / 32;
    // shared layout: xfrag [nkb][2][4] uint4 | partial [2][8 warps][16][2] f32 | ring
    uint4* xfrag = reinterpret_cast<uint4*>(smem);
    float* partial = reinterpret_cast<float*>(smem + (size_t)nkb * 2 * 4 * 16);
    uint8_t* ring = reinterpret_cast<uint8_t*>(partial) + 2 * kDecodeWarps * 16 * 2 * 4;
    const uint32_t stage_bytes = 2 * p.span_cap;

    // ---- selection (all warps, identical) -----------------------------------------------------
    uint32_t ids[kMaxTopK];
    float probs[kMaxTopK];
    if (p.logits) {
        float lv[4];
        load_logits(p.logits, p.E, lane, lv);
        select_experts<ARCH>(lv, p.E, p.K, p.sel_bias, p.normalize, p.scale, lane, ids, probs);
    } else {  // a one-expert bank (the always-on shared expert): nothing to select
#pragma unroll
        for (int r = 0; r < kMaxTopK; r++) { ids[r] = 0; probs[r] = 1.0f; }
    }
    if (blockIdx.x == 0 && warp == 0) {
#pragma unroll
        for (int r = 0; r < kMaxTopK; r++)
            if (r < p.K && lane == r) { p.ids[r] = ids[r]; p.probs[r] = probs[r]; }
    }
    // ---- activation vector into B fragments (hi, lo columns) ----------------------------------
    for (int k = tid; k < p.H; k += kDecodeThreads)
        frag_store(reinterpret_cast<__half*>(xfrag), 2, 0, k, bf16_bits_to_f32(p.x[k]));

    const int col_blocks = (p.F + COLS_PER_ITEM - 1) / COLS_PER_ITEM;
    const int items = p.K * col_blocks;
    auto issue = [&](int item, int stage) {
        if (item < items) {
            int r = item / col_blocks, c0 = (item % col_blocks) * COLS_PER_ITEM;
            uint32_t e = 0;
#pragma unroll
            for (int q = 0; q < kMaxTopK; q++)
                if (q == r) e = ids[q];
            int rows = min(COLS_PER_ITEM, p.F - c0);
            size_t off = ((size_t)e * p.F + c0) * p.row_bytes;
            uint8_t* s0 = ring + (size_t)stage * stage_bytes;
            if (GATED) {
                copy_span_async(s0, p.gate_w + off, rows * p.row_bytes, tid);
                copy_span_async(s0 + p.span_cap, p.up_w + off, rows * p.row_bytes, tid);
            } else {
                int r0 = min(8, rows);
                copy_span_async(s0, p.up_w + off, r0 * p.row_bytes, tid);
                if (rows > 8)
                    copy_span_async(s0 + p.span_cap, p.up_w + off + (size_t)8 * p.row_bytes, (rows - 8) * p.row_bytes, tid);
            }
        }
        cp_async_commit();
    };
    int it = 0;
    const int first = blockIdx.x, step = gridDim.x;
#pragma unroll
    for (int s = 0; s < kDecodeStages - 1; s++) issue(first + s * step, s);

    for (int item = first; item < items; item += step, it++) {
        issue(item + (kDecodeStages - 1) * step, (it + kDecodeStages - 1) % kDecodeStages);
        cp_async_wait<kDecodeStages - 1>();
        __syncthreads();
        int r = item / col_blocks, c0 = (item % col_blocks) * COLS_PER_ITEM;
        uint32_t e = 0;
#pragma unroll
        for (int q = 0; q < kMaxTopK; q++)
            if (q == r) e = ids[q];
        size_t off = ((size_t)e * p.F + c0) * p.row_bytes;
        const uint32_t s0 = smem_u32(ring) + (uint32_t)(it % kDecodeStages) * stage_bytes;
        // rows g (first span) and g + 8 (second span)
        uint32_t rowA, rowB;
        if (GATED) {
            rowA = s0 + ((uint32_t)(uintptr_t)(p.gate_w + off) & 15u) + (uint32_t)g * p.row_bytes;
            rowB = s0 + p.span_cap + ((uint32_t)(uintptr_t)(p.up_w + off) & 15u) + (uint32_t)g * p.row_bytes;
        } else {
            rowA = s0 + ((uint32_t)(uintptr_t)(p.up_w + off) & 15u) + (uint32_t)g * p.row_bytes;
            rowB = s0 + p.span_cap + ((uint32_t)(uintptr_t)(p.up_w + off + (size_t)8 * p.row_bytes) & 15u) + (uint32_t)g * p.row_bytes;
        }
        float sum[4] = {0.f, 0.f, 0.f, 0.f};
        // columns 0 / 1 of the fragments hold the token's hi / lo halves; lanes of other columns
        // re-read them (their products are never looked at)
        rows_dot<FMT>(rowA, rowB, smem_u32(xfrag) + (uint32_t)(((g & 1) * 4 + tig) * 16), 2 * 4 * 16, nkb, warp, tig, sum);
        float* part = partial + (size_t)(it & 1) * kDecodeWarps * 32;
        if (tig == 0) {
            part[(warp * 16 + g) * 2 + 0] = __fadd_rn(sum[0], sum[1]);      // row g: hi + lo columns
            part[(warp * 16 + g + 8) * 2 + 0] = __fadd_rn(sum[2], sum[3]);  // row g + 8
        }
        __syncthreads();
        if (tid < COLS_PER_ITEM && c0 + tid < p.F) {
            int col = c0 + tid;
            float a = 0.f, b = 0.f;
            for (int w = 0; w < kDecodeWarps; w++) {
                if (GATED) {
                    a = __fadd_rn(a, part[(w * 16 + tid) * 2]);
                    b = __fadd_rn(b, part[(w * 16 + tid + 8) * 2]);
                } else {
                    a = __fadd_rn(a, part[(w * 16 + tid) * 2]);
                }
            }
            float v;
            if (ARCH == OCO_ARCH_GPT_OSS) {
                float gate = __fadd_rn(a, bf16_round(p.gate_b[(size_t)e * p.F + col]));
                float up = __fadd_rn(b, bf16_round(__fadd_rn(p.up_b[(size_t)e * p.F + col], 1.0f)));
                v = swiglu_clipped(gate, up);
            } else if (ARCH == OCO_ARCH_QWEN) {
                v = silu_gate_bf16(bf16_round(a), bf16_round(b));
            } else {
                float u = fmaxf(bf16_round(a), 0.0f);
                v = bf16_round(a) != bf16_round(a) ? qnan() : __fmul_rn(u, u);
            }
            p.act[(size_t)r * p.F + col] = v;
            frag_store(p.actfrag + (size_t)(r >> 1) * (p.F / 32) * 4 * 4 * 4 * 2, 4, (r & 1) * 2, col, v);
        }
    }
    cp_async_wait<0>();
}

struct DecodeDownParams {
    const uint8_t* down_w;
    const float* down_b;      // null when the family has no bias
    const uint32_t* ids;      // [K]
    const __half* actfrag;    // [ceil(K/2)][F/32][4][4] uint4
    uint16_t* y;              // out bf16 [K, H]
    int H, F, K;
    uint32_t row_bytes;       // bytes of one packed row of length F
    uint32_t span_cap;
    // Fused combine (null residual = off): the CTA that completes the last route pair of a block
    // of eight output rows adds the weighted expert outputs to the residual
    // (reference moe_sum, routing.metal:154-168; moe_add, nemotron.metal:222-236).
    uint32_t* arrivals;       // one zeroed counter per block of eight output rows; left at zero again
    const float* probs;       // [K]
    uint16_t* residual;       // bf16 [H], in place
    const uint16_t* shared;   // bf16 [H] shared-expert output joining the sum, or null
    int round_sum;            // 1: the expert sum is rounded to bf16 before the residual add
};

// Down products for one token: item = 8 output rows of route 2p and the same 8 rows of route 2p+1
// (reference matvec_mxfp4, projections.metal:140-182; matvec_q4, vector.metal:155-228).
// CTA c serves route pair c % P.
template <int FMT>
__global__ void __launch_bounds__(kDecodeThreads) decode_down_kernel(const DecodeDownParams p) {
    constexpr int kDecodeStages = kDownStages;
    using B = Block32<FMT>;
    extern __shared__ __align__(16) unsigned char smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tig = lane & 3;
    const int nkb = p.F / 32;
    const int P = (p.K + 1) / 2;
    const int pair = blockIdx.x % P;
    uint4* xfrag = reinterpret_cast<uint4*>(smem);                       // [nkb][4][4] uint4
    float* partial = reinterpret_cast<float*>(smem + (size_t)nkb * 4 * 4 * 16);
    uint8_t* ring = reinterpret_cast<uint8_t*>(partial) + 2 * kDecodeWarps * 16 * 2 * 4;
    const uint32_t stage_bytes = 2 * p.span_cap;
    const int r0 = 2 * pair, r1 = min(2 * pair + 1, p.K - 1);
    const uint32_t e0 = p.ids[r0], e1 = p.ids[r1];

    // the pair's activation fragments (written by the expand kernel) -> shared memory
    {
        const uint4* src = reinterpret_cast<const uint4*>(p.actfrag) + (size_t)pair * nkb * 16;
        uint32_t d = smem_u32(xfrag);
        for (int i = tid; i < nkb * 16; i += kDecodeThreads) cp_async16(d + i * 16u, src + i);
        cp_async_commit();
    }
    const int row_blocks = (p.H + 7) / 8;
    const int ctas = gridDim.x / P;          // CTAs serving this pair
    const int first = blockIdx.x / P;
    auto issue = [&](int rb, int stage) {
        if (rb < row_blocks && first < ctas) {
            int d0 = rb * 8, rows = min(8, p.H - d0);
            uint8_t* s0 = ring + (size_t)stage * stage_bytes;
            copy_span_async(s0, p.down_w + ((size_t)e0 * p.H + d0) * p.row_bytes, rows * p.row_bytes, tid);
            copy_span_async(s0 + p.span_cap, p.down_w + ((size_t)e1 * p.H + d0) * p.row_bytes, rows * p.row_bytes, tid);
        }
        cp_async_commit();
    };
    int it = 0;
#pragma unroll
    for (int s = 0; s < kDecodeStages - 1; s++) issue(first + s * ctas, s);
    if (first >= ctas) { cp_async_wait<0>(); return; }

    for (int rb = first; rb < row_blocks; rb += ctas, it++) {
        issue(rb + (kDecodeStages - 1) * ctas, (it + kDecodeStages - 1) % kDecodeStages);
        cp_async_wait<kDecodeStages - 1>();
        __syncthreads();
        const int d0 = rb * 8;
        const uint32_t s0 = smem_u32(ring) + (uint32_t)(it % kDecodeStages) * stage_bytes;
        const uint8_t* ga = p.down_w + ((size_t)e0 * p.H + d0) * p.row_bytes;
        const uint8_t* gb = p.down_w + ((size_t)e1 * p.H + d0) * p.row_bytes;
        const uint32_t rowA = s0 + ((uint32_t)(uintptr_t)ga & 15u) + (uint32_t)g * p.row_bytes;
        const uint32_t rowB = s0 + p.span_cap + ((uint32_t)(uintptr_t)gb & 15u) + (uint32_t)g * p.row_bytes;
        float sum[4] = {0.f, 0.f, 0.f, 0.f};
        rows_dot<FMT>(rowA, rowB, smem_u32(xfrag) + (uint32_t)(((g & 3) * 4 + tig) * 16), 4 * 4 * 16, nkb, warp, tig, sum);
        // route r0: rows g, columns 0,1 (tig 0: acc 0,1); route r1: rows g+8, columns 2,3 (tig 1: acc 2,3)
        float* part = partial + (size_t)(it & 1) * kDecodeWarps * 32;
        if (tig == 0) part[(warp * 16 + g) * 2] = __fadd_rn(sum[0], sum[1]);
        if (tig == 1) part[(warp * 16 + g + 8) * 2] = __fadd_rn(sum[2], sum[3]);
        __syncthreads();
        if (tid < 16) {
            int q = tid >> 3, row = d0 + (tid & 7), route = 2 * pair + q;
            if (row < p.H && route < p.K) {
                float a = 0.f;
                for (int w = 0; w < kDecodeWarps; w++) a = __fadd_rn(a, part[(w * 16 + tid) * 2]);
                uint32_t e = q ? e1 : e0;
                if (p.down_b) a = __fadd_rn(a, bf16_round(p.down_b[(size_t)e * p.H + row]));
                p.y[(size_t)route * p.H + row] = f32_to_bf16_bits(a);
            }
        }
        if (p.residual) {
            // Whoever finishes a row block last combines it. No CTA waits for another.
            __shared__ int is_last;
            __threadfence();
            __syncthreads();
            if (tid == 0) {
                is_last = atomicAdd(p.arrivals + rb, 1u) == (uint32_t)(P - 1);
                if (is_last) p.arrivals[rb] = 0;      // ready for the next call on this stream
            }
            __syncthreads();
            if (is_last && tid < 8 && d0 + tid < p.H) {
                __threadfence();
                const int row = d0 + tid;
                float sres = p.shared ? bf16_bits_to_f32(p.shared[row]) : 0.0f;
                for (int r = 0; r < p.K; r++)
                    sres = __fmaf_rn(bf16_bits_to_f32(__ldcg(p.y + (size_t)r * p.H + row)), p.probs[r], sres);
                if (p.round_sum) sres = bf16_round(sres);
                p.residual[row] = f32_to_bf16_bits(__fadd_rn(bf16_bits_to_f32(p.residual[row]), sres));
            }
        }
    }
    cp_async_wait<0>();
}

}  // namespace oco
