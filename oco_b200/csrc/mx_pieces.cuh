// Activation vectors as the B operand of the block-scaled e2m1 MMA: a value is split into e2m1 pieces
// with per-block UE8M0 scales (see mx.cuh), and the pieces are laid out as operand rows of a K-major,
// 128-byte-swizzled shared-memory image.
#pragma once
#include "common.cuh"

namespace oco {

constexpr int kMxPieces = 8;                         // operand rows (columns of the product) per activation vector

// 2^(b - 127) for a UE8M0 byte b (0 is 2^-127, a subnormal float).
__device__ __forceinline__ float mx_pow2(int b) { return __uint_as_float(b <= 0 ? 0x00400000u : (uint32_t)b << 23); }
__device__ __forceinline__ float mx_e2m1_value(uint32_t code) {
    const uint32_t m = code & 7u;
    const float mag = m < 2u ? 0.5f * (float)m : __uint_as_float(((126u + (m >> 1)) << 23) | ((m & 1u) << 22));
    return (code & 8u) ? -mag : mag;
}

// Byte offset of contraction block `blk` of operand row n inside a K-major, 128-byte-swizzled B image
// with N rows per K group.
__device__ __forceinline__ uint32_t mx_b_offset(uint32_t N, uint32_t n, uint32_t blk) {
    const uint32_t g = blk >> 3, c = blk & 7u;
    return g * (N * 128u) + (n >> 3) * 1024u + (n & 7u) * 128u + ((c ^ (n & 7u)) << 4);
}
__host__ __device__ inline uint32_t mx_b_bytes(uint32_t N, uint32_t nkb) { return ((nkb + 7u) / 8u) * N * 128u; }
// Scales of the operand rows: one 512-byte tile per four blocks, [32 rows][16 bytes] with a row's four
// scale bytes first (the layout tcgen05.cp spreads over one scale-factor column of tensor memory; the
// block-scaled MMA takes scale addresses in steps of four columns).
__host__ __device__ inline uint32_t mx_sfb_bytes(uint32_t nkb) { return ((nkb + 7u) / 8u) * 1024u; }   // whole K groups of eight blocks

// Splits one block of 32 activations into kMxPieces e2m1 pieces (operand rows n0 .. n0 + 7 of the B
// image) and their UE8M0 scales. Called by a whole warp; lane l holds the value at contraction
// position l of the block (operand order). A non-finite value makes the block's first scale NaN.
__device__ __forceinline__ void mx_split_block(float v, int lane, unsigned char* b_img, unsigned char* sfb_img, uint32_t N,
                                               uint32_t n0, uint32_t blk) {
    const bool bad = __any_sync(0xffffffffu, nonfinite(v));
    float amax = fabsf(v);
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
    const uint32_t ab = __float_as_uint(amax);
    // smallest scale 2^e0 with 6 * 2^e0 >= amax, as a UE8M0 byte
    int s0 = (int)((ab >> 23) & 0xffu) - 2 + ((ab & 0x7fffffu) > 0x400000u ? 1 : 0);
    s0 = max(0, min(254, s0));
    float r = bad ? 0.0f : v;
    unsigned char* sf = sfb_img + (blk >> 2) * 512u + (blk & 3u);
#pragma unroll
    for (int p = 0; p < kMxPieces; p++) {
        const int sp = max(0, s0 - (p == 0 ? 0 : 3 * p - 1));
        const float inv = __uint_as_float(sp >= 254 ? 0x00400000u : (uint32_t)(254 - sp) << 23);   // 2^(127 - sp)
        const uint32_t code = (uint32_t)__nv_cvt_float_to_fp4(__fmul_rn(r, inv), __NV_E2M1, cudaRoundNearest) & 0xfu;
        r = __fsub_rn(r, __fmul_rn(mx_e2m1_value(code), mx_pow2(sp)));
        // lanes 2i, 2i + 1 -> byte i; four bytes -> one word held by lanes 0, 8, 16, 24
        uint32_t w = code | (__shfl_down_sync(0xffffffffu, code, 1) << 4);
        w |= __shfl_down_sync(0xffffffffu, w, 2) << 8;
        w |= __shfl_down_sync(0xffffffffu, w, 4) << 16;
        if ((lane & 7) == 0)
            *reinterpret_cast<uint32_t*>(b_img + mx_b_offset(N, n0 + p, blk) + (lane >> 3) * 4) = w;
        if (lane == 0) sf[(n0 + p) * 16u] = (unsigned char)((bad && p == 0) ? 255 : sp);
    }
}

}  // namespace oco
