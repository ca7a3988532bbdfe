// Grouped expert products for many tokens on the 5th-generation tensor cores.
//
// One CTA computes, for one tile of an expert's routes, 128 output features:
//     D[feature, route] = sum_k W[expert][feature, k] * X[route_row, k]
// with the weights as the A operand (M = 128 features) and the expert-sorted activation rows as
// the B operand (N = up to NT routes), so an expert's packed weights are decoded once per NT
// routes and small experts cost a narrow N, not a padded 128-row tile.
//
//   * B tiles (activation rows, half) arrive by TMA (cp.async.bulk.tensor, 128-byte swizzle) from
//     the expert-sorted row buffer; rows past the buffer read as zero.
//   * A tiles are produced by four warps: each thread owns one weight row, reads its packed GGUF
//     blocks from global memory where they lie (any byte alignment), decodes them to half in
//     registers and writes the K-major 128-byte-swizzled layout the MMA descriptors expect.
//   * One thread issues tcgen05.mma (kind::f16, fp32 accumulators in tensor memory) per 16-wide K
//     step and commits to mbarriers that hand the stage back to the producers.
//   * The producer warps then become the epilogue: tcgen05.ld the accumulators (thread = feature,
//     column = route), add the bf16-rounded bias, apply the activation, store.
// Gated layers keep two accumulators (gate and up) over the same B tile, so the activation is
// applied in registers and the f32 projections never travel to memory (the reference stores both
// and runs a separate pass, shaders/experts/projections.metal:192-271 + routing.metal:44-64).
//
// Operand precision is the reference's: decoded weight -> half, activation -> half, fp32
// accumulation (projections.metal:223-233,305-326; shaders/nemotron.metal:309-335).
#pragma once
#include "common.cuh"

namespace oco {

enum GemmEpilogue : int {
    kEpiSwigluF16 = 0,  // gated, biases, clipped SwiGLU -> half rows (expert-sorted)
    kEpiSiluF16 = 1,    // gated, SiLU gate over bf16-rounded projections -> half rows
    kEpiRelu2F16 = 2,   // bf16-rounded projection, relu^2 in f32 -> half rows
    kEpiDownBf16 = 3,   // (+ bias) -> bf16, scattered to each route's row
    kEpiRelu2Bf16F16 = 4  // dense shared expert: relu^2 stored as bf16, then to half
};
__host__ __device__ constexpr bool epi_gated(int epi) { return epi == kEpiSwigluF16 || epi == kEpiSiluF16; }

struct GemmParams {
    const uint8_t* w0;   // gate (gated) or the single matrix, [experts][n][row_bytes]
    const uint8_t* w1;   // up (gated)
    const float* b0;     // bias of w0 (f32 [experts, n]) or null
    const float* b1;     // bias of w1
    int n;               // output features per expert
    int K;               // contraction length
    uint32_t row_bytes;  // bytes from one weight row of a matrix to its next row (the packed row length, or twice
                         // that when gate and up rows are interleaved in one tensor)
    int bias_stride;     // floats from one feature's bias to the next (1, or 2 when interleaved)
    const uint32_t* tiles;       // (expert, first row within expert) pairs; null = dense
    const uint32_t* tile_count;
    const uint32_t* offsets;     // exclusive expert offsets into the sorted rows
    const uint32_t* route_of_row;  // null = identity
    const uint16_t* xs;  // B operand rows, half [rows, K] (used by the CUDA-core variant)
    uint16_t* out;       // half [rows, n] sorted, or bf16 [routes, n]
    uint32_t* status;
    int dense_rows;      // dense mode: number of rows (single expert 0)
    int tile_rows;       // NT
    const uint8_t* w0_end;  // first byte past the 16-byte-aligned envelope of w0 / w1 (wide kernel)
    const uint8_t* w1_end;
    const unsigned char* sfb;  // block-scaled kernel: the B rows' scale tiles, [tile][K group][1024]
    const unsigned char* sfa0; // repacked weights (grouped_gemm_mxr_kernel): the scale tiles of w0 / w1,
    const unsigned char* sfa1; //   [expert][feature tile][K group][1024]
    int sfa_tiles;             //   feature tiles per expert
    uint32_t* sched;           // wide kernel: two zeroed words (items handed out, CTAs finished) for handing out work
                               //   items as CTAs become free; null = item c, c + grid, ... for CTA c
};

// ---- operand order ---------------------------------------------------------------------------------
// A code byte holds two elements of its block: byte j of an MXFP4 / Q4_0 block holds elements j and
// j + 16, byte i of a Q4_K 64-element chunk holds elements i and i + 32. Decoding a byte yields the
// two as one half2, and the tiles keep them adjacent: within every block the contraction index runs
// in "operand order" (byte 0 low nibble, byte 0 high nibble, byte 1 low nibble, ...). The activation
// rows are written in the same order, so no decoded value is ever moved to another lane or
// register before it is stored; a dot product does not care in which order k is visited.
__host__ __device__ inline int operand_pos(int fmt, int k) {
    if (fmt == OCO_FMT_Q4_K) return (k & ~63) + (((k & 31) << 1) | ((k >> 5) & 1));
    return (k & ~31) + (((k & 15) << 1) | ((k >> 4) & 1));
}

__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
    __half2 r = __hmul2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
}
// Two copies of an f32 rounded to half (round to nearest even, subnormals kept).
__device__ __forceinline__ uint32_t f32_to_half2_dup(float f) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %1;" : "=r"(r) : "f"(f));
    return r;
}

// Raw words of one half-slice (32 operand positions = four 16-byte chunks of the A tile) of a
// packed row, fetched ahead of use so global-load latency hides behind the decode of earlier ones.
//   MXFP4: block 2*kb64 + h, 5 aligned words;  Q4_0: likewise, 6 aligned words;
//   Q4_K : 4 header words (d, dmin, 12 scale bytes) + code bytes 16h..16h+15 of the sub-block pair.
template <int FMT>
struct RawHalf {
    static constexpr int kWords = FMT == OCO_FMT_MXFP4 ? 5 : (FMT == OCO_FMT_Q4_0 ? 6 : 8);
    uint32_t w[kWords];
};

template <int FMT>
__device__ __forceinline__ void load_half(const uint8_t* row, int kb64, int h, int K, RawHalf<FMT>& raw) {
    if (FMT == OCO_FMT_Q4_K) {
        // Super-blocks are 144 bytes; rows are whole super-blocks, so 4-byte alignment of the
        // tensor base carries to every word read here. Unaligned bases take the byte path.
        const uint8_t* b = row + (size_t)(kb64 >> 2) * 144;
        const uint8_t* codes = b + 16 + (kb64 & 3) * 32 + 16 * h;
        if ((((uintptr_t)b) & 3u) == 0) {
            const uint32_t* hw = reinterpret_cast<const uint32_t*>(b);
            const uint32_t* cw = reinterpret_cast<const uint32_t*>(codes);
#pragma unroll
            for (int i = 0; i < 4; i++) raw.w[i] = __ldg(hw + i);
#pragma unroll
            for (int i = 0; i < 4; i++) raw.w[4 + i] = __ldg(cw + i);
        } else {
#pragma unroll
            for (int i = 0; i < 4; i++) raw.w[i] = ldg_u32_unaligned(b + 4 * i);
#pragma unroll
            for (int i = 0; i < 4; i++) raw.w[4 + i] = ldg_u32_unaligned(codes + 4 * i);
        }
    } else {
        constexpr int kBytes = FMT == OCO_FMT_MXFP4 ? 17 : 18;
        const int blk = 2 * kb64 + h;
        if (blk < (K >> 5)) {
            uintptr_t a = (uintptr_t)(row + (size_t)blk * kBytes);
            const uint32_t* w = (const uint32_t*)(a & ~(uintptr_t)3);
#pragma unroll
            for (int i = 0; i < RawHalf<FMT>::kWords; i++) raw.w[i] = __ldg(w + i);
        } else {
#pragma unroll
            for (int i = 0; i < RawHalf<FMT>::kWords; i++) raw.w[i] = 0;
        }
    }
}

// MXFP4 block (17 bytes starting `sh` bits into w[0]) -> 16 half2 in operand order, each
// half( e2m1 * 2^(e-127) ) (reference decoder: shaders/matrix/weights.metal:40-46; half rounding:
// projections.metal:227). Scales 2^-24..2^15 are halves themselves and one multiply rounds once.
// Any other header (including 0, the reserved 255 and powers beyond the half range) takes two
// multiplies: the first by a power of two that keeps every product a normal half (exact), the
// second carrying the single rounding, so the result equals rounding the exact product once.
__device__ __forceinline__ void decode_mxfp4_block(const uint32_t* w, uint32_t sh, uint32_t* out) {
    const uint32_t e = (w[0] >> sh) & 0xffu;
    const uint32_t s1 = sh + 8u;
    const uint32_t q[4] = {__funnelshift_rc(w[0], w[1], s1), __funnelshift_rc(w[1], w[2], s1),
                           __funnelshift_rc(w[2], w[3], s1), __funnelshift_rc(w[3], w[4], s1)};
    const bool plain = (e - 103u) <= 39u;
    if (__all_sync(__activemask(), plain)) {
        const uint32_t sc = f32_to_half2_dup(__uint_as_float(e << 23));
#pragma unroll
        for (int i = 0; i < 4; i++) {
            uint32_t r0, r1, r2, r3;
            cvt_e2m1x2_x4(q[i], r0, r1, r2, r3);
            out[4 * i] = hmul2_u32(r0, sc); out[4 * i + 1] = hmul2_u32(r1, sc);
            out[4 * i + 2] = hmul2_u32(r2, sc); out[4 * i + 3] = hmul2_u32(r3, sc);
        }
    } else {
        const int t = (int)e - 127;
        const int t1 = max(-13, min(13, t));
        const int t2 = t - t1;
        const uint32_t h1 = (uint32_t)(t1 + 15) << 10;
        const uint32_t sa = h1 | (h1 << 16);
        uint32_t sb;
        if (e == 255u) sb = 0x7e007e00u;                                   // NaN
        else if (t2 > 15) sb = 0x7bff7bffu;                                // 65504: any non-zero product overflows
        else sb = f32_to_half2_dup(t2 < -126 ? 0.0f : __uint_as_float((uint32_t)(t2 + 127) << 23));
#pragma unroll
        for (int i = 0; i < 4; i++) {
            uint32_t r0, r1, r2, r3;
            cvt_e2m1x2_x4(q[i], r0, r1, r2, r3);
            out[4 * i] = hmul2_u32(hmul2_u32(r0, sa), sb); out[4 * i + 1] = hmul2_u32(hmul2_u32(r1, sa), sb);
            out[4 * i + 2] = hmul2_u32(hmul2_u32(r2, sa), sb); out[4 * i + 3] = hmul2_u32(hmul2_u32(r3, sa), sb);
        }
    }
}

// Q4_0 block (18 bytes starting `sh` bits into w[0]) -> 16 half2 in operand order:
// half( d * (q - 8) ) (reference q4_decode, shaders/matrix/q4_tile.metal:24-37). q - 8 is exact as
// a half and d is a half, so one half multiply rounds the exact product once.
__device__ __forceinline__ void decode_q4_0_block(const uint32_t* w, uint32_t sh, uint32_t* out) {
    const uint32_t hd = __funnelshift_rc(w[0], w[1], sh) & 0xffffu;  // sh <= 24
    const uint32_t d2 = hd | (hd << 16);
    const uint32_t s2 = sh + 16u;  // 16..40
    uint32_t q[4];
    if (s2 <= 32u) {
        q[0] = __funnelshift_rc(w[0], w[1], s2); q[1] = __funnelshift_rc(w[1], w[2], s2);
        q[2] = __funnelshift_rc(w[2], w[3], s2); q[3] = __funnelshift_rc(w[3], w[4], s2);
    } else {
        const uint32_t s3 = s2 - 32u;
        q[0] = __funnelshift_rc(w[1], w[2], s3); q[1] = __funnelshift_rc(w[2], w[3], s3);
        q[2] = __funnelshift_rc(w[3], w[4], s3); q[3] = __funnelshift_rc(w[4], w[5], s3);
    }
    const uint32_t bias = 0x64086408u;  // 1032 as halves: (1024 + q) - 1032 = q - 8
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t lo = q[i] & 0x0f0f0f0fu, hi = (q[i] >> 4) & 0x0f0f0f0fu;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            // byte j of lo -> bits 0..7, byte j of hi -> bits 16..23, 0x64 above each: halves 1024 + q
            uint32_t v = (__byte_perm(lo, hi, (uint32_t)(j | ((4 + j) << 8))) & 0x00ff00ffu) | 0x64006400u;
            __half2 h = __hsub2(*reinterpret_cast<__half2*>(&v), *reinterpret_cast<const __half2*>(&bias));
            __half2 o = __hmul2(h, *reinterpret_cast<const __half2*>(&d2));
            out[4 * i + j] = *reinterpret_cast<uint32_t*>(&o);
        }
    }
}

// Q4_K: code bytes 16h..16h+15 of sub-blocks 2c and 2c+1 of one super-block -> 16 half2 in operand
// order: each byte gives half2( d*sc0*q_lo - dmin*m0 , d*sc1*q_hi - dmin*m1 ), with one f32 rounding
// in the subtraction before the half rounding (weights.metal:67-77).
__device__ __forceinline__ void decode_q4_k_half(const uint32_t* hdr, const uint32_t* codes, int c, uint32_t* out) {
    const float d = f16_bits_to_f32((uint16_t)(hdr[0] & 0xffffu)), dm = f16_bits_to_f32((uint16_t)(hdr[0] >> 16));
    auto sbyte = [&](int i) -> uint32_t {  // scale byte i of 12 (hdr words 1..3)
        uint32_t word = i < 4 ? hdr[1] : (i < 8 ? hdr[2] : hdr[3]);
        return (word >> (8 * (i & 3))) & 0xffu;
    };
    float scale[2], minimum[2];
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const int s = 2 * c + h;
        uint32_t sc, mn;
        if (s < 4) {
            sc = sbyte(s) & 63u;
            mn = sbyte(s + 4) & 63u;
        } else {
            sc = (sbyte(s + 4) & 15u) | ((sbyte(s - 4) >> 6) << 4);
            mn = (sbyte(s + 4) >> 4) | ((sbyte(s) >> 6) << 4);
        }
        scale[h] = __fmul_rn(d, (float)sc);
        minimum[h] = __fmul_rn(dm, (float)mn);
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t word = codes[i];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint32_t b = (word >> (8 * j)) & 0xffu;
            __half2 v = __floats2half2_rn(__fsub_rn(__fmul_rn(scale[0], (float)(b & 15u)), minimum[0]),
                                          __fsub_rn(__fmul_rn(scale[1], (float)(b >> 4)), minimum[1]));
            out[4 * i + j] = *reinterpret_cast<uint32_t*>(&v);
        }
    }
}

// Decodes a fetched half-slice into `out` (16 half2 in operand order); positions at or past K are zero.
template <int FMT>
__device__ __forceinline__ void decode_half(const RawHalf<FMT>& raw, const uint8_t* row, int kb64, int h, int K,
                                            uint32_t (&out)[16]) {
    if (FMT == OCO_FMT_Q4_K) {
        decode_q4_k_half(raw.w, raw.w + 4, kb64 & 3, out);
    } else {
        constexpr int kBytes = FMT == OCO_FMT_MXFP4 ? 17 : 18;
        const int blk = 2 * kb64 + h;
        if (blk < (K >> 5)) {
            const uint32_t sh = ((uint32_t)(uintptr_t)(row + (size_t)blk * kBytes) & 3u) * 8u;
            if (FMT == OCO_FMT_MXFP4) decode_mxfp4_block(raw.w, sh, out);
            else decode_q4_0_block(raw.w, sh, out);
        } else {
#pragma unroll
            for (int i = 0; i < 16; i++) out[i] = 0;
        }
    }
}

// Decodes the 64 weights [64*kb64, 64*kb64 + 64) of one packed row (fetch + decode), operand order.
template <int FMT>
__device__ __forceinline__ void decode_row_k64(const uint8_t* row, int kb64, int K, uint32_t (&out)[32]) {
#pragma unroll
    for (int h = 0; h < 2; h++) {
        RawHalf<FMT> raw;
        uint32_t v[16];
        load_half<FMT>(row, kb64, h, K, raw);
        decode_half<FMT>(raw, row, kb64, h, K, v);
#pragma unroll
        for (int i = 0; i < 16; i++) out[16 * h + i] = v[i];
    }
}

// ---- epilogue arithmetic -------------------------------------------------------------------------
// Tile epilogues evaluate the activations with the hardware exp2 / reciprocal approximations
// (relative error about 1e-6, far inside the half rounding of the stored value). Routing never
// goes through these: ids and weights use the exact sequence shared with the host checker.
__device__ __forceinline__ float sigmoid_times(float g, float scale) {   // sigmoid(scale * g), g finite
    float e = __expf(-fabsf(g) * scale);
    return __fdividef(g < 0 ? e : 1.0f, 1.0f + e);
}
__device__ __forceinline__ float swiglu_clipped_fast(float g, float u) {
    if (nonfinite(g) || nonfinite(u)) return qnan();
    g = fminf(g, 7.0f);
    u = fminf(fmaxf(u, -6.0f), 8.0f);
    return sigmoid_times(g, 1.702f) * g * u;
}
__device__ __forceinline__ float silu_gate_bf16_fast(float a, float b) {
    if (nonfinite(a) || nonfinite(b)) return qnan();
    return bf16_round(bf16_round(sigmoid_times(a, 1.0f) * a) * b);
}

// a: accumulator of w0 (+ bias), b: accumulator of w1 (+ bias); returns the stored 16-bit pattern.
template <int EPI>
__device__ __forceinline__ uint16_t epilogue_value(float a, float b) {
    if (EPI == kEpiSwigluF16) return f32_to_f16_bits(swiglu_clipped_fast(a, b));
    if (EPI == kEpiSiluF16) return f32_to_f16_bits(silu_gate_bf16_fast(bf16_round(a), bf16_round(b)));
    if (EPI == kEpiRelu2F16 || EPI == kEpiRelu2Bf16F16) {
        float r = bf16_round(a);
        float u = fmaxf(r, 0.0f);
        float v = r != r ? qnan() : __fmul_rn(u, u);
        if (EPI == kEpiRelu2Bf16F16) v = bf16_round(v);
        return f32_to_f16_bits(v);
    }
    return f32_to_bf16_bits(a);
}

// ---- tcgen05 / TMA wrappers ----------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_dst), "l"(map), "r"(c0), "r"(c1), "r"(bar)
        : "memory");
}

// K-major, 128-byte swizzle: 8-row groups of 1024 bytes (stride byte offset), descriptor version 1.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    uint32_t lo = ((smem_addr & 0x3ffffu) >> 4) | (1u << 16);
    uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
    return ((uint64_t)hi << 32) | lo;
}
// kind::f16: D f32, A and B half, both K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t umma_idesc_f16(uint32_t n) {
    return (1u << 4) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}

// Thread layout: producer warps first (they turn into the epilogue), then one warp that owns the
// tensor memory allocation and issues the MMAs. A 64-element slice of the tile's weight rows is
// (matrices x 2) half-slices per row; the 128 rows x kParts producer threads share them so that a
// thread decodes one or two 32-element blocks per slice. Many light producer warps hide the
// decode's dependent-instruction latency better than few heavy ones.
//   gated, NT = 256: 4 parts (16 producer warps): part = matrix + 2 * half; both accumulators fill
//                    all 512 tensor-memory columns, one CTA per SM.
//   otherwise:       2 parts (8 producer warps), two CTAs per SM; gated: part = matrix (both
//                    halves), single matrix: part = half.
template <int EPI, int NT>
struct GemmShape {
    static constexpr bool kGated = epi_gated(EPI);
    static constexpr int kMats = kGated ? 2 : 1;
    static constexpr bool kWide = kGated && NT == 256;
    static constexpr int kParts = kWide ? 4 : 2;
    static constexpr int kHalvesPerThread = kMats * 2 / kParts;       // 1 or 2
    static constexpr int kProducerWarps = 4 * kParts;
    static constexpr int kThreads = (kProducerWarps + 1) * 32;
    static constexpr int kABytes = 128 * 128;                          // 128 rows x 64 halves
    static constexpr int kBBytes = NT * 128;
    static constexpr int kStageBytes = kMats * kABytes + kBBytes;
    static constexpr int kCtasPerSm = kWide ? 1 : 2;
    static constexpr int kBudget = kWide ? 200 * 1024 : 110 * 1024;
    static constexpr int kStagesRaw = kBudget / kStageBytes;
    static constexpr int kStages = kStagesRaw > 4 ? 4 : kStagesRaw;
    static constexpr int kTmemCols = kMats * NT;
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment*/ + 256 /*barriers*/ + NT * 4 /*row map*/;
};

// Decodes one half-slice of a weight row and stores it as four 16-byte chunks of the K-major,
// 128-byte-swizzled A tile (chunk c of row r lives at chunk c ^ (r & 7)).
template <int FMT>
__device__ __forceinline__ void produce_half(const RawHalf<FMT>& raw, const uint8_t* row, int kb, int h, int K,
                                             uint32_t tile_row_addr, uint32_t sw) {
    uint32_t v[16];
    decode_half<FMT>(raw, row, kb, h, K, v);
#pragma unroll
    for (int c = 0; c < 4; c++) {
        const uint32_t addr = tile_row_addr + ((((uint32_t)(4 * h + c)) ^ sw) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v[4 * c]), "r"(v[4 * c + 1]),
                     "r"(v[4 * c + 2]), "r"(v[4 * c + 3]) : "memory");
    }
}

template <int FMT, int EPI, int NT>
__global__ void __launch_bounds__(GemmShape<EPI, NT>::kThreads, GemmShape<EPI, NT>::kCtasPerSm)
grouped_gemm_tc_kernel(const GemmParams p, const __grid_constant__ CUtensorMap tmap_b) {
    using S = GemmShape<EPI, NT>;
    constexpr bool GATED = S::kGated;
    constexpr int PW = S::kProducerWarps;
    extern __shared__ unsigned char smem_raw[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // ---- which tile ----------------------------------------------------------------------------
    uint32_t expert, begin, count, row0;
    if (p.tiles) {
        if (blockIdx.y >= *p.tile_count) return;
        expert = p.tiles[2 * blockIdx.y];
        begin = p.tiles[2 * blockIdx.y + 1];
        row0 = p.offsets[expert] + begin;
        count = p.offsets[expert + 1] - p.offsets[expert];
    } else {
        expert = 0; begin = blockIdx.y * NT; row0 = begin; count = (uint32_t)p.dense_rows;
        if (begin >= count) return;
    }
    // An earlier wait gave up somewhere: drain the grid. The decision is made CTA-uniform.
    if (__syncthreads_or(tid == 0 && *reinterpret_cast<volatile uint32_t*>(p.status) != 0u)) return;
    const uint32_t nv = min((uint32_t)NT, count - begin);           // live routes in this tile
    const uint32_t n_mma = max(16u, (nv + 15u) & ~15u);
    const int f0 = blockIdx.x * 128;
    const int nkb = (p.K + 63) / 64;

    // ---- shared memory carve-up ----------------------------------------------------------------
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char* gen_base = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + S::kStages * S::kStageBytes;        // full[S], empty[S], accum, then tmem slot, abort
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (S::kStages + s); };
    const uint32_t accum_bar = bars + 8u * (2 * S::kStages);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen_base + S::kStages * S::kStageBytes + 8 * (2 * S::kStages + 1));
    volatile uint32_t* abort_flag = tmem_slot + 1;
    // Destination row of every live column of the tile (the scatter of the down projection).
    uint32_t* out_rows = reinterpret_cast<uint32_t*>(gen_base + S::kStages * S::kStageBytes + 256);
    for (uint32_t i = tid; i < nv; i += S::kThreads)
        out_rows[i] = (EPI == kEpiDownBf16 && p.route_of_row) ? p.route_of_row[row0 + i] : row0 + i;

    if (tid == 0) {
        // full: one arrival per producer warp plus the thread that announces the TMA bytes
        for (int s = 0; s < S::kStages; s++) { mbar_init(full_bar(s), PW + 1); mbar_init(empty_bar(s), 1); }
        mbar_init(accum_bar, 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == PW) {
        tmem_alloc(smem_u32(tmem_slot), S::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < PW) {
        // ===== producers ==========================================================================
        const int prow = tid & 127;                                   // weight row within the tile
        const int part = tid >> 7;
        const int mat = GATED ? (part & 1) : 0;                        // which weight matrix this thread decodes
        const int half0 = S::kHalvesPerThread == 2 ? 0 : (GATED ? part >> 1 : part);  // first (or only) half-slice
        const int frow = min(f0 + prow, p.n - 1);
        const uint8_t* wrow = (mat ? p.w1 : p.w0) + ((size_t)expert * p.n + frow) * p.row_bytes;
        const uint32_t row_off = (uint32_t)(prow >> 3) * 1024u + (uint32_t)(prow & 7) * 128u + (uint32_t)mat * S::kABytes;
        const uint32_t sw = (uint32_t)(prow & 7);
        // Packed words of the next slices ride in registers while the current one is decoded.
        constexpr int kAhead = 1;
        constexpr int HPT = S::kHalvesPerThread;
        RawHalf<FMT> ring[kAhead + 1][HPT];
#pragma unroll
        for (int u = 0; u < kAhead; u++) {
            if (u < nkb) {
#pragma unroll
                for (int q = 0; q < HPT; q++) load_half<FMT>(wrow, u, half0 + q, p.K, ring[u][q]);
            }
        }
        for (int kb0 = 0; kb0 < nkb; kb0 += kAhead + 1) {
#pragma unroll
            for (int u = 0; u <= kAhead; u++) {
                const int kb = kb0 + u;
                if (kb < nkb) {
                    if (kb + kAhead < nkb) {
#pragma unroll
                        for (int q = 0; q < HPT; q++)
                            load_half<FMT>(wrow, kb + kAhead, half0 + q, p.K, ring[(u + kAhead) & kAhead][q]);
                    }
                    const int s = kb % S::kStages;
                    const uint32_t ph = (uint32_t)(kb / S::kStages) & 1u;
                    const uint32_t stage = base + (uint32_t)s * S::kStageBytes;
                    // One lane per warp waits and, below, arrives: hundreds of threads arriving on one
                    // barrier serialise on its shared-memory word and cost more than the decode.
                    if (lane == 0) mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, p.status);
                    __syncwarp();
                    if (tid == 0) {
                        mbar_arrive_expect_tx(full_bar(s), (uint32_t)S::kBBytes);
                        tma_load_2d(stage + S::kMats * S::kABytes, &tmap_b, kb * 64, (int)row0, full_bar(s));
                    }
#pragma unroll
                    for (int q = 0; q < HPT; q++)
                        produce_half<FMT>(ring[u][q], wrow, kb, half0 + q, p.K, stage + row_off, sw);
                    fence_proxy_async_smem();      // every lane: its stores, visible to the tensor core
                    __syncwarp();
                    if (lane == 0) mbar_arrive(full_bar(s));
                }
            }
        }
        // ===== epilogue ===========================================================================
        if (lane == 0) mbar_wait(accum_bar, 0u, abort_flag, p.status);
        __syncwarp();
        tc_fence_after();
        const int f = f0 + prow;
        const bool live = f < p.n;
        float bias0 = 0.f, bias1 = 0.f;
        if (live) {
            if (p.b0) bias0 = bf16_round(p.b0[((size_t)expert * p.n + f) * p.bias_stride]);
            if (EPI == kEpiSwigluF16) bias1 = bf16_round(__fadd_rn(p.b1[((size_t)expert * p.n + f) * p.bias_stride], 1.0f));
        }
        // Rows written for a later tile kernel keep the operand order within each block.
        const int fcol = EPI == kEpiDownBf16 ? f : operand_pos(FMT, f);
        // Each warp may touch the 32 tensor-memory lanes of its quarter (warp & 3); the kParts warps
        // that share a quarter split the tile's columns between them.
        const uint32_t taddr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
        const uint32_t c_begin = (uint32_t)part * (NT / S::kParts);
        const uint32_t c_end = min(nv, c_begin + NT / S::kParts);
        for (uint32_t c = c_begin; c < c_end; c += 16) {
            uint32_t ra[16], rb[16];
            tmem_ld16(taddr + c, ra);
            if (GATED) tmem_ld16(taddr + NT + c, rb);
            tmem_ld_wait();
            if (live) {
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    if (c + j < nv) {
                        float a = __fadd_rn(__uint_as_float(ra[j]), bias0);
                        float b = GATED ? __fadd_rn(__uint_as_float(rb[j]), bias1) : 0.f;
                        uint16_t h = epilogue_value<EPI>(a, b);
                        p.out[(size_t)out_rows[c + j] * p.n + fcol] = h;
                    }
                }
            }
        }
        tc_fence_before();
    } else if (lane == 0) {
        // ===== MMA issue ==========================================================================
        const uint32_t idesc = umma_idesc_f16(n_mma);
        for (int kb = 0; kb < nkb; kb++) {
            const int s = kb % S::kStages;
            const uint32_t ph = (uint32_t)(kb / S::kStages) & 1u;
            const uint32_t stage = base + (uint32_t)s * S::kStageBytes;
            mbar_wait(full_bar(s), ph, abort_flag, p.status);
            tc_fence_after();
            const uint64_t a0 = umma_desc(stage), a1 = umma_desc(stage + S::kABytes);
            const uint64_t b = umma_desc(stage + S::kMats * S::kABytes);
#pragma unroll
            for (int kk = 0; kk < 4; kk++) {
                const uint32_t acc = (kb | kk) != 0 ? 1u : 0u;
                umma_f16(tmem_base, a0 + 2u * kk, b + 2u * kk, idesc, acc);
                if (GATED) umma_f16(tmem_base + NT, a1 + 2u * kk, b + 2u * kk, idesc, acc);
            }
            umma_commit(empty_bar(s));
        }
        umma_commit(accum_bar);
        // The accumulator barrier also tells this thread that every MMA has retired.
        mbar_wait(accum_bar, 0u, abort_flag, p.status);
        tc_fence_before();
    }
    __syncthreads();
    if (*abort_flag) {
        // A wait gave up: leave time for copies still in flight to land before the CTA's shared
        // memory is handed to another CTA.
        for (int i = 0; i < 64; i++) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == PW) {
        tc_fence_after();
        tmem_dealloc(tmem_base, S::kTmemCols);
    }
}

// The same product on CUDA cores: one thread per output feature, eight routes at a time, fp32
// FMAs over half operands. Slow; kept as an independent second implementation for cross-checks.
template <int FMT, int EPI, int NT>
__global__ void __launch_bounds__(128) grouped_gemm_simt_kernel(const GemmParams p) {
    constexpr bool GATED = epi_gated(EPI);
    uint32_t expert, begin, count, row0;
    if (p.tiles) {
        if (blockIdx.y >= *p.tile_count) return;
        expert = p.tiles[2 * blockIdx.y];
        begin = p.tiles[2 * blockIdx.y + 1];
        row0 = p.offsets[expert] + begin;
        count = p.offsets[expert + 1] - p.offsets[expert];
    } else {
        expert = 0; begin = blockIdx.y * NT; row0 = begin; count = (uint32_t)p.dense_rows;
        if (begin >= count) return;
    }
    const uint32_t nv = min((uint32_t)NT, count - begin);
    const int f = blockIdx.x * 128 + threadIdx.x;
    const int frow = min(f, p.n - 1);
    const uint8_t* r0 = p.w0 + ((size_t)expert * p.n + frow) * p.row_bytes;
    const uint8_t* r1 = GATED ? p.w1 + ((size_t)expert * p.n + frow) * p.row_bytes : nullptr;
    const int nkb = (p.K + 63) / 64;
    float bias0 = 0.f, bias1 = 0.f;
    if (p.b0) bias0 = bf16_round(p.b0[((size_t)expert * p.n + frow) * p.bias_stride]);
    if (EPI == kEpiSwigluF16) bias1 = bf16_round(__fadd_rn(p.b1[((size_t)expert * p.n + frow) * p.bias_stride], 1.0f));
    for (uint32_t c = 0; c < nv; c += 8) {
        float acc0[8], acc1[8];
#pragma unroll
        for (int j = 0; j < 8; j++) { acc0[j] = 0.f; acc1[j] = 0.f; }
        for (int kb = 0; kb < nkb; kb++) {
            uint32_t v0[32], v1[32];
            decode_row_k64<FMT>(r0, kb, p.K, v0);
            if (GATED) decode_row_k64<FMT>(r1, kb, p.K, v1);
            int klen = min(64, p.K - kb * 64);
#pragma unroll
            for (int j = 0; j < 8; j++) {
                if (c + j >= nv) continue;
                const uint32_t* xr = reinterpret_cast<const uint32_t*>(p.xs + (size_t)(row0 + c + j) * p.K + kb * 64);
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    if (2 * i >= klen) break;
                    uint32_t xw = xr[i];
                    float2 xf = __half22float2(*reinterpret_cast<__half2*>(&xw));
                    float2 w0 = __half22float2(*reinterpret_cast<__half2*>(&v0[i]));
                    acc0[j] = __fmaf_rn(w0.x, xf.x, acc0[j]);
                    acc0[j] = __fmaf_rn(w0.y, xf.y, acc0[j]);
                    if (GATED) {
                        float2 w1 = __half22float2(*reinterpret_cast<__half2*>(&v1[i]));
                        acc1[j] = __fmaf_rn(w1.x, xf.x, acc1[j]);
                        acc1[j] = __fmaf_rn(w1.y, xf.y, acc1[j]);
                    }
                }
            }
        }
        if (f < p.n) {
#pragma unroll
            for (int j = 0; j < 8; j++) {
                if (c + j >= nv) continue;
                uint16_t h = epilogue_value<EPI>(__fadd_rn(acc0[j], bias0), __fadd_rn(acc1[j], bias1));
                uint32_t row = row0 + c + j;
                if (EPI == kEpiDownBf16 && p.route_of_row) row = p.route_of_row[row];
                p.out[(size_t)row * p.n + (EPI == kEpiDownBf16 ? f : operand_pos(FMT, f))] = h;
            }
        }
    }
}

// Block decoders exposed for bit-exact checks: n_elems weights of a packed tensor to f32 (as the
// single-token kernels use them) or to half (as the tiles use them).
template <int FMT>
__global__ void dequant_kernel(const uint8_t* __restrict__ w, size_t n_elems, float* out32, uint16_t* out16) {
    size_t chunk = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // one 64-element chunk per thread
    size_t k0 = chunk * 64;
    if (k0 >= n_elems) return;
    // treat the tensor as one long row
    uint32_t v[32];
    size_t kend = n_elems;
    int K = (int)min((size_t)0x7fffffc0, kend);
    if (out16) {
        decode_row_k64<FMT>(w, (int)chunk, K, v);
        for (int k = 0; k < 64; k++) {       // element k of the chunk sits at its operand position
            int pos = operand_pos(FMT, k);
            if (k0 + k < n_elems) out16[k0 + k] = (uint16_t)(pos & 1 ? v[pos >> 1] >> 16 : v[pos >> 1] & 0xffffu);
        }
    }
    if (out32) {
        for (int i = 0; i < 64; i++) {
            size_t k = k0 + i;
            if (k >= n_elems) break;
            float val;
            if (FMT == OCO_FMT_MXFP4) {
                const uint8_t* b = w + k / 32 * 17;
                uint32_t j = (uint32_t)(k % 32);
                uint32_t byte = b[1 + j % 16];
                uint32_t h2 = e2m1x2_to_half2(byte);
                float m = f16_bits_to_f32((uint16_t)(j < 16 ? (h2 & 0xffffu) : (h2 >> 16)));
                val = __fmul_rn(m, e8m0_scale(b[0]));
            } else if (FMT == OCO_FMT_Q4_0) {
                const uint8_t* b = w + k / 32 * 18;
                uint32_t j = (uint32_t)(k % 32);
                uint32_t q = (b[2 + j % 16] >> (j / 16 * 4)) & 15u;
                val = __fmul_rn(f16_bits_to_f32((uint16_t)(b[0] | ((uint16_t)b[1] << 8))), (float)((int)q - 8));
            } else {
                const uint8_t* b = w + k / 256 * 144;
                uint32_t j = (uint32_t)(k % 256), s = j / 32;
                const uint8_t* sc8 = b + 4;
                uint32_t sc = s < 4 ? (sc8[s] & 63u) : ((sc8[s + 4] & 15u) | ((uint32_t)(sc8[s - 4] >> 6) << 4));
                uint32_t mn = s < 4 ? (sc8[s + 4] & 63u) : ((uint32_t)(sc8[s + 4] >> 4) | ((uint32_t)(sc8[s] >> 6) << 4));
                uint32_t q = (b[16 + j / 64 * 32 + j % 32] >> (s % 2 * 4)) & 15u;
                float d = f16_bits_to_f32((uint16_t)(b[0] | ((uint16_t)b[1] << 8)));
                float dm = f16_bits_to_f32((uint16_t)(b[2] | ((uint16_t)b[3] << 8)));
                val = __fsub_rn(__fmul_rn(__fmul_rn(d, (float)sc), (float)q), __fmul_rn(dm, (float)mn));
            }
            out32[k] = val;
        }
    }
}

}  // namespace oco
