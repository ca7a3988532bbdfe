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
    uint32_t row_bytes;  // packed bytes of one weight row
    const uint32_t* tiles;       // (expert, first row within expert) pairs; null = dense
    const uint32_t* tile_count;
    const uint32_t* offsets;     // exclusive expert offsets into the sorted rows
    const uint32_t* route_of_row;  // null = identity
    const uint16_t* xs;  // B operand rows, half [rows, K] (used by the CUDA-core variant)
    uint16_t* out;       // half [rows, n] sorted, or bf16 [routes, n]
    uint32_t* status;
    int dense_rows;      // dense mode: number of rows (single expert 0)
    int tile_rows;       // NT
};

// ---- packed block -> 32 halves -------------------------------------------------------------------
// out[0..3]: elements 0-7, out[4..7]: 8-15, out[8..11]: 16-23, out[12..15]: 24-31 (half2 each).
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) { return __byte_perm(a, b, sel); }
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
    __half2 r = __hmul2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
}

// Raw words of one 64-element slice of a packed row, fetched ahead of use so the next slice's
// global loads overlap the current slice's decode.
//   MXFP4: 2 blocks x 5 aligned words;  Q4_0: 2 blocks x 6 aligned words;
//   Q4_K : 4 header words (d, dmin, 12 scale bytes) + 8 code words of one sub-block pair.
template <int FMT>
struct RawK64 {
    static constexpr int kWords = FMT == OCO_FMT_MXFP4 ? 10 : 12;
    uint32_t w[kWords];
};

template <int FMT>
__device__ __forceinline__ void load_raw_k64(const uint8_t* row, int kb64, int K, RawK64<FMT>& raw) {
    if (FMT == OCO_FMT_Q4_K) {
        // Super-blocks are 144 bytes; rows are whole super-blocks, so 4-byte alignment of the
        // tensor base carries to every word read here. Unaligned bases take the byte path.
        const uint8_t* b = row + (size_t)(kb64 >> 2) * 144;
        const uint8_t* codes = b + 16 + (kb64 & 3) * 32;
        if ((((uintptr_t)b) & 3u) == 0) {
            const uint32_t* hw = reinterpret_cast<const uint32_t*>(b);
            const uint32_t* cw = reinterpret_cast<const uint32_t*>(codes);
#pragma unroll
            for (int i = 0; i < 4; i++) raw.w[i] = __ldg(hw + i);
#pragma unroll
            for (int i = 0; i < 8; i++) raw.w[4 + i] = __ldg(cw + i);
        } else {
#pragma unroll
            for (int i = 0; i < 4; i++) raw.w[i] = ldg_u32_unaligned(b + 4 * i);
#pragma unroll
            for (int i = 0; i < 8; i++) raw.w[4 + i] = ldg_u32_unaligned(codes + 4 * i);
        }
    } else {
        constexpr int kBytes = FMT == OCO_FMT_MXFP4 ? 17 : 18;
        constexpr int kW = FMT == OCO_FMT_MXFP4 ? 5 : 6;
        const int nblk = K >> 5;
#pragma unroll
        for (int b = 0; b < 2; b++) {
            int blk = 2 * kb64 + b;
            if (blk < nblk) {
                uintptr_t a = (uintptr_t)(row + (size_t)blk * kBytes);
                const uint32_t* w = (const uint32_t*)(a & ~(uintptr_t)3);
#pragma unroll
                for (int i = 0; i < kW; i++) raw.w[b * kW + i] = __ldg(w + i);
            } else {
#pragma unroll
                for (int i = 0; i < kW; i++) raw.w[b * kW + i] = 0;
            }
        }
    }
}

// MXFP4 block (17 bytes starting `sh` bits into w[0]) -> 32 halves
// (reference decoder: shaders/matrix/weights.metal:40-46; half rounding: projections.metal:227).
// out[0..3]: elements 0-7, [4..7]: 8-15, [8..11]: 16-23, [12..15]: 24-31 (half2 each).
__device__ __forceinline__ void decode_mxfp4_block(const uint32_t* w, uint32_t sh, uint32_t* out) {
    uint32_t e = (w[0] >> sh) & 0xffu;
    uint32_t s1 = sh + 8u;
    uint32_t q[4] = {__funnelshift_rc(w[0], w[1], s1), __funnelshift_rc(w[1], w[2], s1),
                     __funnelshift_rc(w[2], w[3], s1), __funnelshift_rc(w[3], w[4], s1)};
    bool fast = (e - 103u) <= 39u;  // 2^-24 .. 2^15: the scale itself is a half
    uint32_t sc = 0;
    if (fast) {
        uint32_t hb = e >= 113u ? ((e - 112u) << 10) : (1u << (e - 103u));
        sc = hb | (hb << 16);
    }
    float fs = e8m0_scale(e);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        uint32_t A0 = e2m1x2_to_half2(q[i]), A1 = e2m1x2_to_half2(q[i] >> 8), A2 = e2m1x2_to_half2(q[i] >> 16),
                 A3 = e2m1x2_to_half2(q[i] >> 24);
        uint32_t r[4] = {prmt(A0, A1, 0x5410), prmt(A2, A3, 0x5410), prmt(A0, A1, 0x7632), prmt(A2, A3, 0x7632)};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            if (fast) {
                r[j] = hmul2_u32(r[j], sc);
            } else {
                __half2 h = *reinterpret_cast<__half2*>(&r[j]);
                __half2 o = __floats2half2_rn(__fmul_rn(__low2float(h), fs), __fmul_rn(__high2float(h), fs));
                r[j] = *reinterpret_cast<uint32_t*>(&o);
            }
        }
        out[2 * i] = r[0]; out[2 * i + 1] = r[1];
        out[8 + 2 * i] = r[2]; out[8 + 2 * i + 1] = r[3];
    }
}

// Q4_0 block (18 bytes starting `sh` bits into w[0]): half( d * (q - 8) ) (reference q4_decode,
// shaders/matrix/q4_tile.metal:24-37). d*(q-8) is exact in f32, so one half multiply rounds once.
__device__ __forceinline__ void decode_q4_0_block(const uint32_t* w, uint32_t sh, uint32_t* out) {
    uint32_t hd = __funnelshift_rc(w[0], w[1], sh) & 0xffffu;  // sh <= 24
    uint32_t d2 = hd | (hd << 16);
    uint32_t s2 = sh + 16u;  // 16..40
    uint32_t q[4];
    if (s2 <= 32u) {
        q[0] = __funnelshift_rc(w[0], w[1], s2); q[1] = __funnelshift_rc(w[1], w[2], s2);
        q[2] = __funnelshift_rc(w[2], w[3], s2); q[3] = __funnelshift_rc(w[3], w[4], s2);
    } else {
        uint32_t s3 = s2 - 32u;
        q[0] = __funnelshift_rc(w[1], w[2], s3); q[1] = __funnelshift_rc(w[2], w[3], s3);
        q[2] = __funnelshift_rc(w[3], w[4], s3); q[3] = __funnelshift_rc(w[4], w[5], s3);
    }
    const uint32_t magic = 0x64006400u, bias = 0x64086408u;  // 1024 and 1032 as halves
#pragma unroll
    for (int i = 0; i < 4; i++) {
        // bytes b0..b3 hold codes j..j+3 (low nibbles) and j+16..j+19 (high nibbles)
        uint32_t lo = q[i] & 0x0f0f0f0fu, hi = (q[i] >> 4) & 0x0f0f0f0fu;
        uint32_t r[4] = {prmt(lo, 0, 0x4140) | magic, prmt(lo, 0, 0x4342) | magic, prmt(hi, 0, 0x4140) | magic,
                         prmt(hi, 0, 0x4342) | magic};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            __half2 h = __hsub2(*reinterpret_cast<__half2*>(&r[j]), *reinterpret_cast<const __half2*>(&bias));
            __half2 o = __hmul2(h, *reinterpret_cast<__half2*>(&d2));
            r[j] = *reinterpret_cast<uint32_t*>(&o);
        }
        out[2 * i] = r[0]; out[2 * i + 1] = r[1];
        out[8 + 2 * i] = r[2]; out[8 + 2 * i + 1] = r[3];
    }
}

// Q4_K: sub-blocks 2c and 2c+1 of one super-block -> 64 halves: half( d*sc*q - dmin*m ) with one
// f32 rounding in the subtraction (weights.metal:67-77). hdr = the super-block's first 16 bytes,
// codes = the pair's 32 code bytes. out[0..15]: elements 0-31 (low nibbles), [16..31]: 32-63.
__device__ __forceinline__ void decode_q4_k_pair(const uint32_t* hdr, const uint32_t* codes, int c, uint32_t* out) {
    float d = f16_bits_to_f32((uint16_t)(hdr[0] & 0xffffu)), dm = f16_bits_to_f32((uint16_t)(hdr[0] >> 16));
    auto sbyte = [&](int i) -> uint32_t {  // scale byte i of 12 (hdr words 1..3)
        uint32_t word = i < 4 ? hdr[1] : (i < 8 ? hdr[2] : hdr[3]);
        return (word >> (8 * (i & 3))) & 0xffu;
    };
    float scale[2], minimum[2];
#pragma unroll
    for (int h = 0; h < 2; h++) {
        int s = 2 * c + h;
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
    for (int i = 0; i < 8; i++) {
        uint32_t word = codes[i];
#pragma unroll
        for (int j = 0; j < 2; j++) {
            uint32_t b0 = (word >> (16 * j)) & 0xffu, b1 = (word >> (16 * j + 8)) & 0xffu;
            __half2 lo = __floats2half2_rn(__fsub_rn(__fmul_rn(scale[0], (float)(b0 & 15u)), minimum[0]),
                                           __fsub_rn(__fmul_rn(scale[0], (float)(b1 & 15u)), minimum[0]));
            __half2 hi = __floats2half2_rn(__fsub_rn(__fmul_rn(scale[1], (float)(b0 >> 4)), minimum[1]),
                                           __fsub_rn(__fmul_rn(scale[1], (float)(b1 >> 4)), minimum[1]));
            out[2 * i + j] = *reinterpret_cast<uint32_t*>(&lo);
            out[16 + 2 * i + j] = *reinterpret_cast<uint32_t*>(&hi);
        }
    }
}

// Decodes a fetched slice into `out` (32 half2, ascending k); positions at or past K are zero.
template <int FMT>
__device__ __forceinline__ void decode_raw_k64(const RawK64<FMT>& raw, const uint8_t* row, int kb64, int K,
                                               uint32_t (&out)[32]) {
    if (FMT == OCO_FMT_Q4_K) {
        decode_q4_k_pair(raw.w, raw.w + 4, kb64 & 3, out);
    } else {
        constexpr int kBytes = FMT == OCO_FMT_MXFP4 ? 17 : 18;
        constexpr int kW = FMT == OCO_FMT_MXFP4 ? 5 : 6;
        const int nblk = K >> 5;
#pragma unroll
        for (int b = 0; b < 2; b++) {
            int blk = 2 * kb64 + b;
            if (blk < nblk) {
                uint32_t sh = ((uint32_t)(uintptr_t)(row + (size_t)blk * kBytes) & 3u) * 8u;
                if (FMT == OCO_FMT_MXFP4) decode_mxfp4_block(raw.w + b * kW, sh, out + 16 * b);
                else decode_q4_0_block(raw.w + b * kW, sh, out + 16 * b);
            } else {
#pragma unroll
                for (int i = 0; i < 16; i++) out[16 * b + i] = 0;
            }
        }
    }
}

// Decodes the 64 weights [64*kb64, 64*kb64 + 64) of one packed row (fetch + decode).
template <int FMT>
__device__ __forceinline__ void decode_row_k64(const uint8_t* row, int kb64, int K, uint32_t (&out)[32]) {
    RawK64<FMT> raw;
    load_raw_k64<FMT>(row, kb64, K, raw);
    decode_raw_k64<FMT>(raw, row, kb64, K, out);
}

// ---- epilogue arithmetic -------------------------------------------------------------------------
// a: accumulator of w0 (+ bias), b: accumulator of w1 (+ bias); returns the stored 16-bit pattern.
template <int EPI>
__device__ __forceinline__ uint16_t epilogue_value(float a, float b) {
    if (EPI == kEpiSwigluF16) return f32_to_f16_bits(swiglu_clipped(a, b));
    if (EPI == kEpiSiluF16) return f32_to_f16_bits(silu_gate_bf16(bf16_round(a), bf16_round(b)));
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

constexpr int kGemmThreads = 160;  // warps 0-3: producers then epilogue; warp 4: MMA issue + TMEM

template <int EPI, int NT>
struct GemmShape {
    static constexpr bool kGated = epi_gated(EPI);
    static constexpr int kABytes = 128 * 128;                 // 128 rows x 64 halves
    static constexpr int kBBytes = NT * 128;
    static constexpr int kStageBytes = (kGated ? 2 : 1) * kABytes + kBBytes;
    static constexpr int kBudget = 110 * 1024;                // two CTAs per SM
    static constexpr int kStagesRaw = kBudget / kStageBytes;
    static constexpr int kStages = kStagesRaw > 4 ? 4 : kStagesRaw;
    static constexpr int kTmemCols = (kGated ? 2 : 1) * NT;
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment*/ + 256 /*barriers*/;
};

template <int FMT, int EPI, int NT>
__global__ void __launch_bounds__(kGemmThreads, 2)
grouped_gemm_tc_kernel(const GemmParams p, const __grid_constant__ CUtensorMap tmap_b) {
    using S = GemmShape<EPI, NT>;
    constexpr bool GATED = S::kGated;
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

    if (tid == 0) {
        for (int s = 0; s < S::kStages; s++) { mbar_init(full_bar(s), 129); mbar_init(empty_bar(s), 1); }
        mbar_init(accum_bar, 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 4) {
        tmem_alloc(smem_u32(tmem_slot), S::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < 4) {
        // ===== producers ==========================================================================
        const int frow = min(f0 + tid, p.n - 1);
        const uint8_t* row0p = p.w0 + ((size_t)expert * p.n + frow) * p.row_bytes;
        const uint8_t* row1p = GATED ? p.w1 + ((size_t)expert * p.n + frow) * p.row_bytes : nullptr;
        const uint32_t row_off = (uint32_t)(tid >> 3) * 1024u + (uint32_t)(tid & 7) * 128u;
        const uint32_t sw = (uint32_t)(tid & 7);
        RawK64<FMT> cur0, cur1, nxt0, nxt1;
        load_raw_k64<FMT>(row0p, 0, p.K, cur0);
        if (GATED) load_raw_k64<FMT>(row1p, 0, p.K, cur1);
        for (int kb = 0; kb < nkb; kb++) {
            const int s = kb % S::kStages;
            const uint32_t ph = (uint32_t)(kb / S::kStages) & 1u;
            const uint32_t stage = base + (uint32_t)s * S::kStageBytes;
            if (kb + 1 < nkb) {  // next slice's loads fly while this one is decoded
                load_raw_k64<FMT>(row0p, kb + 1, p.K, nxt0);
                if (GATED) load_raw_k64<FMT>(row1p, kb + 1, p.K, nxt1);
            }
            mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, p.status);
            if (tid == 0) {
                mbar_arrive_expect_tx(full_bar(s), (uint32_t)S::kBBytes);
                tma_load_2d(stage + (GATED ? 2 : 1) * S::kABytes, &tmap_b, kb * 64, (int)row0, full_bar(s));
            }
            uint32_t v[32];
            decode_raw_k64<FMT>(cur0, row0p, kb, p.K, v);
#pragma unroll
            for (int c = 0; c < 8; c++) {
                uint32_t addr = stage + row_off + (((uint32_t)c ^ sw) << 4);
                asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v[4 * c]), "r"(v[4 * c + 1]),
                             "r"(v[4 * c + 2]), "r"(v[4 * c + 3]) : "memory");
            }
            if (GATED) {
                decode_raw_k64<FMT>(cur1, row1p, kb, p.K, v);
#pragma unroll
                for (int c = 0; c < 8; c++) {
                    uint32_t addr = stage + S::kABytes + row_off + (((uint32_t)c ^ sw) << 4);
                    asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v[4 * c]), "r"(v[4 * c + 1]),
                                 "r"(v[4 * c + 2]), "r"(v[4 * c + 3]) : "memory");
                }
            }
            fence_proxy_async_smem();
            mbar_arrive(full_bar(s));
            cur0 = nxt0;
            if (GATED) cur1 = nxt1;
        }
        // ===== epilogue ===========================================================================
        mbar_wait(accum_bar, 0u, abort_flag, p.status);
        tc_fence_after();
        const int f = f0 + tid;
        const bool live = f < p.n;
        float bias0 = 0.f, bias1 = 0.f;
        if (live) {
            if (p.b0) bias0 = bf16_round(p.b0[(size_t)expert * p.n + f]);
            if (EPI == kEpiSwigluF16) bias1 = bf16_round(__fadd_rn(p.b1[(size_t)expert * p.n + f], 1.0f));
        }
        const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16);
        for (uint32_t c = 0; c < nv; c += 16) {
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
                        uint32_t row = row0 + c + j;
                        if (EPI == kEpiDownBf16 && p.route_of_row) row = p.route_of_row[row];
                        p.out[(size_t)row * p.n + f] = h;
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
            const uint64_t b = umma_desc(stage + (GATED ? 2 : 1) * S::kABytes);
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
    if (warp == 4) {
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
    if (p.b0) bias0 = bf16_round(p.b0[(size_t)expert * p.n + frow]);
    if (EPI == kEpiSwigluF16) bias1 = bf16_round(__fadd_rn(p.b1[(size_t)expert * p.n + frow], 1.0f));
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
                p.out[(size_t)row * p.n + f] = h;
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
        for (int i = 0; i < 32; i++) {
            size_t k = k0 + 2 * i;
            if (k < n_elems) out16[k] = (uint16_t)(v[i] & 0xffffu);
            if (k + 1 < n_elems) out16[k + 1] = (uint16_t)(v[i] >> 16);
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
