// Single-token expert products: memory-bound streaming of the packed weight rows.
//
// The unit of work is 16 packed weight rows (8 gate + 8 up rows of one expert, or 16 consecutive
// rows) over a range of 32-element blocks. ONE WARP owns a unit from the first byte to the
// activation: it brings the rows' bytes into its own shared-memory ring with bulk asynchronous
// copies (one per row and stage, completion counted on an mbarrier; a stage holds 16 blocks of
// each of the 16 rows), and multiplies them with m16n8k16
// tensor-core MMAs: the A fragment is a block's e2m1 codes converted to half in registers (one cvt
// per code byte), the B fragment is the activation vector split into hi + lo half parts in two of
// the eight columns, so the product is exact to f32 rounding. The block scale multiplies the
// block's partial sum afterwards in f32, as the reference's single-token kernels do
// (shaders/experts/projections.metal:57-59). A byte holds elements j and j + 16 of its block; the
// contraction index is permuted accordingly on the activation side instead of shuffling weights.
// Warps never wait for one another inside the stream (no CTA barrier); when there are fewer units
// than warps, several warps split a unit's blocks and meet once at a named barrier.
//
// FP32 FMA pipes cannot keep up with 4.25-bit weights at HBM rate (one FMA plus decode per weight
// needs more issue slots than an SM has per byte delivered), which is why the dot products ride
// on the tensor pipe even though the kernel is bandwidth-bound.
#pragma once
#include "common.cuh"
#include "mx_pieces.cuh"
#include "router.cuh"

namespace oco {

#ifndef OCO_TOK_WARPS
#define OCO_TOK_WARPS 20
#endif
#ifndef OCO_CHUNK_BLOCKS
#define OCO_CHUNK_BLOCKS 16
#endif
constexpr int kTokWarps = OCO_TOK_WARPS;            // one CTA per SM
constexpr int kTokThreads = kTokWarps * 32;
constexpr int kChunkBlocks = OCO_CHUNK_BLOCKS;      // blocks of each row per pipeline stage
// Bytes per row in a stage: room for 15 bytes of misalignment and the blocks, a multiple of 16,
// and 12 or 20 words modulo 32 so that the eight rows of a fragment start in distinct banks.
constexpr int row_pitch(int blocks) {
    int p = (15 + blocks * 18 + 15) / 16 * 16;
    while ((p / 4) % 32 != 12 && (p / 4) % 32 != 20) p += 16;
    return p;
}
constexpr int kRowPitch = row_pitch(kChunkBlocks);  // 304 for 16 blocks
constexpr int kStageBytes = 16 * kRowPitch;
constexpr int kScalePitch = kChunkBlocks * 2 + 16;   // per-warp table of the stage's scales, 16 bits each, padded against bank conflicts
constexpr int kScaleBytes = 16 * kScalePitch;
constexpr int kMiscBytes = 2048;                    // split sums (64 B a warp) | mbarriers from 1280 | give-up flag at 1984
static_assert(kChunkBlocks % 16 == 0 && kTokWarps <= 20, "layout of the token kernels");
// Q4_K keeps two floats per sub-block in its table, so fewer warps fit.
constexpr int kKTablePitch = 144;                   // 16 sub-blocks x (scale, offset) + 16 bytes against bank conflicts
constexpr int kKTableBytes = 16 * kKTablePitch;
__host__ __device__ constexpr int tok_warps(int fmt) { return fmt == OCO_FMT_Q4_K ? 16 : kTokWarps; }
__host__ __device__ constexpr int scale_table_bytes(int fmt) { return fmt == OCO_FMT_Q4_K ? kKTableBytes : kScaleBytes; }
// B fragments of nkb blocks, followed for Q4_K by the per-block sums of the fragments' columns.
__host__ __device__ constexpr uint32_t frag_region_bytes(int fmt, int nkb) {
    return (uint32_t)(nkb * 128 + (fmt == OCO_FMT_Q4_K ? nkb * 8 : 0) + 15) & ~15u;
}
constexpr int kFragBlockBytes = 128;                // B fragments of one block: 2 columns x 4 lanes x 16 bytes

// D = A * B with a zero accumulator, then D += A * B (fp32 accumulate, half operands).
__device__ __forceinline__ void mma16816_first(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// Shared-memory accesses as plain loads and stores (base = the kernel's shared array), so that the
// compiler is free to schedule them; the waits and barriers around them are compiler barriers.
using SharedBase = const unsigned char*;
__device__ __forceinline__ uint32_t lds32(SharedBase base, uint32_t off) {
    return *reinterpret_cast<const uint32_t*>(base + off);
}
__device__ __forceinline__ uint32_t lds8(SharedBase base, uint32_t off) { return base[off]; }
__device__ __forceinline__ uint4 lds128(SharedBase base, uint32_t off) {
    return *reinterpret_cast<const uint4*>(base + off);
}
__device__ __forceinline__ void sts128(SharedBase base, uint32_t off, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(const_cast<unsigned char*>(base) + off) = make_float4(a, b, c, d);
}
// Bulk asynchronous copy global -> shared, counted on an mbarrier. Both addresses and the size are
// multiples of 16 bytes.
__device__ __forceinline__ void bulk_copy(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ uint32_t hmul2_bits(uint32_t a, uint32_t b) {
    __half2 r = __hmul2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
}
// Barrier among the `threads` threads that name the same id (1..15); id 0 is __syncthreads.
__device__ __forceinline__ void named_barrier(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// Block codecs for the 32-element formats whose code byte j holds elements j (low nibble) and
// j + 16 (high nibble): MXFP4 (17 bytes, E8M0 scale) and Q4_0 (18 bytes, f16 scale, code - 8).
// `block` is the byte offset of the block in shared memory; quads() turns a word of four code
// bytes into four half2 (element j, element j + 16). Blocks kClasses apart start at the same
// offset within a 32-bit word.
template <int FMT>
struct Block32;
template <>
struct Block32<OCO_FMT_MXFP4> {
    static constexpr int kBytes = 17, kHeader = 1, kClasses = 4;
    // the scale as 16 bits (bf16 holds every power of two, 2^-127 as a subnormal) and back to f32
    __device__ static __forceinline__ uint32_t scale16(SharedBase base, uint32_t block) {
        const uint32_t e = lds8(base, block);
        return e == 255u ? 0x7fc0u : (e == 0u ? 0x0040u : e << 7);
    }
    __device__ static __forceinline__ float scale_f32(uint32_t bits) { return __uint_as_float(bits << 16); }
    __device__ static __forceinline__ void quads(uint32_t w, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
        cvt_e2m1x2_x4(w, r0, r1, r2, r3);
    }
};
template <>
struct Block32<OCO_FMT_Q4_0> {
    static constexpr int kBytes = 18, kHeader = 2, kClasses = 2;
    __device__ static __forceinline__ uint32_t scale16(SharedBase base, uint32_t block) {
        return lds8(base, block) | (lds8(base, block + 1) << 8);
    }
    __device__ static __forceinline__ float scale_f32(uint32_t bits) { return f16_bits_to_f32((uint16_t)bits); }
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

// Q4_K (144-byte super-blocks of 256 elements: f16 d, f16 dmin, 12 bytes of 6-bit scales and
// minima, 128 code bytes; byte l of each 32-byte run holds elements l and l + 32 of a 64-element
// group) is streamed as sub-blocks of 32 elements, 18 bytes on average; a stage holds two
// super-blocks of each row. The codecs of the other formats do not apply.
template <>
struct Block32<OCO_FMT_Q4_K> {
    static constexpr int kBytes = 18, kHeader = 0, kClasses = 1;
};

// One warp's pass over blocks [kb0, kb0 + nb) of 16 packed rows: rows 0..7 of span A and rows
// 0..7 of span B (each span is 8 consecutive rows of `row_bytes` bytes in a GGUF tensor, at any
// byte alignment). begin() starts the copies; run() multiplies. After run(), lane (g, tig) holds
// in sum[0..1] the products of row g of span A with fragment columns 2*tig and 2*tig + 1, and in
// sum[2..3] the same for row g of span B.
// COLS: columns of the B fragments kept per block (2: one token as hi + lo; 8: up to eight routes).
template <int FMT, int STAGES, int COLS = 2>
struct RowStream {
    using B = Block32<FMT>;
    static constexpr uint32_t kChunkBytes = kChunkBlocks * B::kBytes;   // 272 or 288: whole 16-byte pieces
    static constexpr uint32_t kFragBlock = COLS * 64;                   // bytes of one block's B fragments
    // Several tokens follow the tile kernels' numerics: weights enter the MMA as half(code * scale), as the
    // reference's tiles hold them. E8M0 scales are powers of two, so only Q4_0 rounds there.
    static constexpr bool kPrescale = FMT == OCO_FMT_Q4_0 && COLS == 8;
    int ncols = 2;             // columns in use: only the lanes that feed them load B fragments

    SharedBase base;           // the kernel's shared array; ring and stab are byte offsets into it
    uint32_t base_addr;        // its address in the shared window (for the copy and mbarrier instructions)
    uint32_t ring, stab, bars;
    uint32_t seq;              // stages used so far by this warp (mbarrier phases run on across units)
    volatile uint32_t* abort_flag;
    uint32_t* status;
    // warp-uniform description of the unit
    const uint8_t* spanA;
    const uint8_t* spanB;      // both advanced to the first block of the range
    uint32_t row_bytes, total_bytes;
    int nchunks, nb, kb_first;
    // per lane
    uint32_t mK = 0;           // Q4_K: misalignment of row lane / 2 (the row whose scales this lane unpacks)
    uint32_t xsum = 0;         // Q4_K: byte offset in shared memory of the fragments' per-block sums
    uint32_t mA, mB;           // misalignment of row g of each span
    uint32_t alA[B::kClasses], alB[B::kClasses], shA[B::kClasses], shB[B::kClasses];
    int g, tig, lane;

    // Once per kernel: this warp's ring, scale table and mbarriers (STAGES of them, 8 bytes each).
    __device__ __forceinline__ void init(SharedBase smem_base, uint32_t ring_off, uint32_t stab_off, uint32_t bars_off,
                                         volatile uint32_t* abort_word, uint32_t* status_word, int lane_) {
        base = smem_base; base_addr = smem_u32(smem_base);
        ring = ring_off; stab = stab_off; bars = base_addr + bars_off; abort_flag = abort_word; status = status_word;
        lane = lane_; g = lane >> 2; tig = lane & 3; seq = 0;
        if (lane == 0) {
#pragma unroll
            for (int s = 0; s < STAGES; s++) mbar_init(bars + 8u * s, 1);
            fence_barrier_init();
        }
        __syncwarp();
    }

    // a, b, rb, kb0, nblocks: the same in every lane.
    __device__ __forceinline__ void begin(const uint8_t* a, const uint8_t* b, uint32_t rb, int kb0, int nblocks) {
        nb = nblocks; row_bytes = rb; kb_first = kb0;
        const size_t skip = (size_t)kb0 * B::kBytes;
        spanA = a + skip; spanB = b + skip;
        nchunks = (nb + kChunkBlocks - 1) / kChunkBlocks;
        total_bytes = (uint32_t)nb * B::kBytes;
        mA = (uint32_t)(uintptr_t)(spanA + (size_t)g * row_bytes) & 15u;
        mB = (uint32_t)(uintptr_t)(spanB + (size_t)g * row_bytes) & 15u;
        if (FMT == OCO_FMT_Q4_K) {
            const int rr = lane >> 1;
            mK = (uint32_t)(uintptr_t)((rr < 8 ? spanA : spanB) + (size_t)(rr & 7) * row_bytes) & 15u;
        }
#pragma unroll
        for (int c = 0; c < B::kClasses; c++) {
            const uint32_t qa = (uint32_t)g * kRowPitch + mA + (uint32_t)(c * B::kBytes + B::kHeader) + 4u * tig;
            const uint32_t qb = (uint32_t)(8 + g) * kRowPitch + mB + (uint32_t)(c * B::kBytes + B::kHeader) + 4u * tig;
            alA[c] = qa & ~3u; shA[c] = (qa & 3u) * 8u;
            alB[c] = qb & ~3u; shB[c] = (qb & 3u) * 8u;
        }
#pragma unroll
        for (int s = 0; s < STAGES - 1; s++) issue(s);
    }

    // Starts the copies of chunk c of the unit (nothing past the last chunk). The stage was read
    // for the last time before the __syncwarp that precedes this call.
    __device__ __forceinline__ void issue(int c) {
        if (c >= nchunks) return;
        const uint32_t off = (uint32_t)c * kChunkBytes;
        const uint32_t len = min(kChunkBytes, total_bytes - off);
        const uint32_t stage = (seq + (uint32_t)c) % STAGES;
        const uint32_t bar = bars + 8u * stage;
        const uint32_t dst = base_addr + ring + stage * kStageBytes;
        // lanes 0..15 copy one row each; the byte total of the stage is summed over them first
        const uint8_t* row = (lane < 8 ? spanA : spanB) + (size_t)(lane & 7) * row_bytes;
        const uint32_t m = (uint32_t)(uintptr_t)row & 15u;
        const uint32_t bytes = lane < 16 ? ((m + len + 15u) & ~15u) : 0u;
        uint32_t total = bytes;
#pragma unroll
        for (int d = 8; d >= 1; d >>= 1) total += __shfl_xor_sync(0xffffffffu, total, d);
        if (lane == 0) mbar_arrive_expect_tx(bar, total);
        __syncwarp();
        if (lane < 16) bulk_copy(dst + (uint32_t)lane * kRowPitch, row - m + off, bytes, bar);
    }

    // The blocks of one stage. FULL: all 16 blocks are present. xa: byte offset in shared memory of
    // this lane's B fragment of the stage's first block. Only the lanes that feed a column in use
    // (g < ncols) load; the other columns multiply zeros.
    // Q4_K: unpacks the scales of the stage: lane l takes row l / 2, super-block l & 1, and leaves
    // per sub-block (d * scale, 1024 * d * scale + dmin * minimum): the codes enter the MMA as
    // 1024 + q (a half built with two bit operations), and sum(x) of the sub-block takes both the
    // 1024 and the minimum out again.
    __device__ __forceinline__ void scales_k(uint32_t st, int nbc) {
        const int rr = lane >> 1, sb = lane & 1;
        if (sb * 8 < nbc) {
            const uint32_t at = st + (uint32_t)rr * kRowPitch + mK + (uint32_t)sb * 144u;
            const uint32_t a4 = at & ~3u, sh = (at & 3u) * 8u;
            const uint32_t r0 = lds32(base, a4), r1 = lds32(base, a4 + 4), r2 = lds32(base, a4 + 8), r3 = lds32(base, a4 + 12),
                           r4 = lds32(base, a4 + 16);
            const uint32_t w0 = __funnelshift_r(r0, r1, sh), w1 = __funnelshift_r(r1, r2, sh), w2 = __funnelshift_r(r2, r3, sh),
                           w3 = __funnelshift_r(r3, r4, sh);
            const float d = f16_bits_to_f32((uint16_t)(w0 & 0xffffu)), dmin = f16_bits_to_f32((uint16_t)(w0 >> 16));
            const uint32_t scl = w1 & 0x3f3f3f3fu, mnl = w2 & 0x3f3f3f3fu;
            const uint32_t sch = (w3 & 0x0f0f0f0fu) | ((w1 >> 2) & 0x30303030u);
            const uint32_t mnh = ((w3 >> 4) & 0x0f0f0f0fu) | ((w2 >> 2) & 0x30303030u);
            float2* tab = reinterpret_cast<float2*>(const_cast<unsigned char*>(base) + stab + (uint32_t)rr * kKTablePitch + (uint32_t)sb * 64u);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float s1 = __fmul_rn(d, (float)((scl >> (8 * j)) & 0xffu));
                tab[j] = make_float2(s1, __fmaf_rn(1024.0f, s1, __fmul_rn(dmin, (float)((mnl >> (8 * j)) & 0xffu))));
                const float t1 = __fmul_rn(d, (float)((sch >> (8 * j)) & 0xffu));
                tab[4 + j] = make_float2(t1, __fmaf_rn(1024.0f, t1, __fmul_rn(dmin, (float)((mnh >> (8 * j)) & 0xffu))));
            }
        }
    }

    // Q4_K: the sub-blocks of one stage (two super-blocks). xa: this lane's B fragment of the
    // stage's first sub-block; xs: byte offset of the stage's first (sum hi, sum lo) pair.
    template <bool FULL>
    __device__ __forceinline__ void chunk_k(uint32_t st, uint32_t xa, uint32_t xs, int nbc, float (&sum)[4]) {
        const uint32_t pA = st + (((uint32_t)g * kRowPitch + mA) & ~3u), sA = (mA & 3u) * 8u;
        const uint32_t pB = st + (((uint32_t)(8 + g) * kRowPitch + mB) & ~3u), sB = (mB & 3u) * 8u;
        auto nib = [](uint32_t w, int shift) { return ((w >> shift) & 0x000f000fu) | 0x64006400u; };   // two halves 1024 + q
#pragma unroll
        for (int sb = 0; sb < 2; sb++) {
            if (FULL || sb * 8 < nbc) {
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const uint32_t off = (uint32_t)(sb * 144 + 16 + 32 * j) + 8u * tig;
                    const uint32_t a0 = lds32(base, pA + off), a1 = lds32(base, pA + off + 4), a2 = lds32(base, pA + off + 8);
                    const uint32_t b0 = lds32(base, pB + off), b1 = lds32(base, pB + off + 4), b2 = lds32(base, pB + off + 8);
                    const uint32_t wa0 = __funnelshift_r(a0, a1, sA), wa1 = __funnelshift_r(a1, a2, sA);
                    const uint32_t wb0 = __funnelshift_r(b0, b1, sB), wb1 = __funnelshift_r(b1, b2, sB);
                    const int kb = sb * 8 + 2 * j;                 // low nibbles: sub-block kb, high nibbles: kb + 1
                    uint4 xl = make_uint4(0u, 0u, 0u, 0u), xh = make_uint4(0u, 0u, 0u, 0u);
                    if (g < ncols) {
                        xl = lds128(base, xa + (uint32_t)kb * kFragBlock);
                        xh = lds128(base, xa + (uint32_t)(kb + 1) * kFragBlock);
                    }
                    const float4 ta = *reinterpret_cast<const float4*>(base + stab + (uint32_t)g * kKTablePitch + kb * 8);
                    const float4 tb = *reinterpret_cast<const float4*>(base + stab + (uint32_t)(8 + g) * kKTablePitch + kb * 8);
                    const float4 xv = *reinterpret_cast<const float4*>(base + xs + kb * 8);   // (hi, lo) sums of kb and kb + 1
                    float lo[4], hi[4];
                    mma16816_first(lo, nib(wa0, 0), nib(wb0, 0), nib(wa0, 8), nib(wb0, 8), xl.x, xl.y);
                    mma16816(lo, nib(wa1, 0), nib(wb1, 0), nib(wa1, 8), nib(wb1, 8), xl.z, xl.w);
                    mma16816_first(hi, nib(wa0, 4), nib(wb0, 4), nib(wa0, 12), nib(wb0, 12), xh.x, xh.y);
                    mma16816(hi, nib(wa1, 4), nib(wb1, 4), nib(wa1, 12), nib(wb1, 12), xh.z, xh.w);
                    sum[0] = __fmaf_rn(lo[0], ta.x, __fmaf_rn(-ta.y, xv.x, sum[0]));
                    sum[1] = __fmaf_rn(lo[1], ta.x, __fmaf_rn(-ta.y, xv.y, sum[1]));
                    sum[2] = __fmaf_rn(lo[2], tb.x, __fmaf_rn(-tb.y, xv.x, sum[2]));
                    sum[3] = __fmaf_rn(lo[3], tb.x, __fmaf_rn(-tb.y, xv.y, sum[3]));
                    sum[0] = __fmaf_rn(hi[0], ta.z, __fmaf_rn(-ta.w, xv.z, sum[0]));
                    sum[1] = __fmaf_rn(hi[1], ta.z, __fmaf_rn(-ta.w, xv.w, sum[1]));
                    sum[2] = __fmaf_rn(hi[2], tb.z, __fmaf_rn(-tb.w, xv.z, sum[2]));
                    sum[3] = __fmaf_rn(hi[3], tb.z, __fmaf_rn(-tb.w, xv.w, sum[3]));
                }
            }
        }
    }

    template <bool FULL>
    __device__ __forceinline__ void chunk(uint32_t st, uint32_t xa, int nbc, float (&sum)[4]) {
#pragma unroll
        for (int q = 0; q < kChunkBlocks / 4; q++) {
            if (FULL || q * 4 < nbc) {
                const uint2 sa = *reinterpret_cast<const uint2*>(base + stab + (uint32_t)g * kScalePitch + q * 8);
                const uint2 sb = *reinterpret_cast<const uint2*>(base + stab + (uint32_t)(8 + g) * kScalePitch + q * 8);
                const float fa[4] = {B::scale_f32(sa.x & 0xffffu), B::scale_f32(sa.x >> 16), B::scale_f32(sa.y & 0xffffu),
                                     B::scale_f32(sa.y >> 16)};
                const float fb[4] = {B::scale_f32(sb.x & 0xffffu), B::scale_f32(sb.x >> 16), B::scale_f32(sb.y & 0xffffu),
                                     B::scale_f32(sb.y >> 16)};
#pragma unroll
                for (int t = 0; t < 4; t++) {
                    const int i = q * 4 + t;
                    if (FULL || i < nbc) {
                        constexpr int kC = B::kClasses;
                        const uint32_t pa = st + alA[i % kC] + (uint32_t)((i / kC) * kC * B::kBytes);
                        const uint32_t pb = st + alB[i % kC] + (uint32_t)((i / kC) * kC * B::kBytes);
                        const uint32_t wa = __funnelshift_r(lds32(base, pa), lds32(base, pa + 4), shA[i % kC]);
                        const uint32_t wb = __funnelshift_r(lds32(base, pb), lds32(base, pb + 4), shB[i % kC]);
                        uint4 xf = make_uint4(0u, 0u, 0u, 0u);
                        if (g < ncols) xf = lds128(base, xa + (uint32_t)i * kFragBlock);
                        uint32_t qa0, qa1, qa2, qa3, qb0, qb1, qb2, qb3;
                        B::quads(wa, qa0, qa1, qa2, qa3);
                        B::quads(wb, qb0, qb1, qb2, qb3);
                        float acc[4];
                        if (kPrescale) {
                            const uint32_t ha = (t < 2 ? sa.x : sa.y) >> (16 * (t & 1)) & 0xffffu;
                            const uint32_t hb = (t < 2 ? sb.x : sb.y) >> (16 * (t & 1)) & 0xffffu;
                            const uint32_t da = ha | (ha << 16), db = hb | (hb << 16);
                            qa0 = hmul2_bits(qa0, da); qa1 = hmul2_bits(qa1, da); qa2 = hmul2_bits(qa2, da); qa3 = hmul2_bits(qa3, da);
                            qb0 = hmul2_bits(qb0, db); qb1 = hmul2_bits(qb1, db); qb2 = hmul2_bits(qb2, db); qb3 = hmul2_bits(qb3, db);
                        }
                        mma16816_first(acc, qa0, qb0, qa1, qb1, xf.x, xf.y);
                        mma16816(acc, qa2, qb2, qa3, qb3, xf.z, xf.w);
                        if (kPrescale) {
                            sum[0] = __fadd_rn(sum[0], acc[0]); sum[1] = __fadd_rn(sum[1], acc[1]);
                            sum[2] = __fadd_rn(sum[2], acc[2]); sum[3] = __fadd_rn(sum[3], acc[3]);
                        } else {
                            sum[0] = __fmaf_rn(acc[0], fa[t], sum[0]);
                            sum[1] = __fmaf_rn(acc[1], fa[t], sum[1]);
                            sum[2] = __fmaf_rn(acc[2], fb[t], sum[2]);
                            sum[3] = __fmaf_rn(acc[3], fb[t], sum[3]);
                        }
                    }
                }
            }
        }
    }

    // xaddr: byte offset in shared memory of this lane's B fragment (uint4) for block kb0.
    __device__ __forceinline__ void run(uint32_t xaddr, float (&sum)[4]) {
        for (int c = 0; c < nchunks; c++) {
            issue(c + STAGES - 1);
            const uint32_t n = seq + (uint32_t)c, stage = n % STAGES;
            mbar_wait(bars + 8u * stage, (n / STAGES) & 1u, abort_flag, status);
            const uint32_t st = ring + stage * kStageBytes;
            const int nbc = min(kChunkBlocks, nb - c * kChunkBlocks);
            const uint32_t xa = xaddr + (uint32_t)(c * kChunkBlocks) * kFragBlock;
            if constexpr (FMT == OCO_FMT_Q4_K) {
                scales_k(st, nbc);
                __syncwarp();
                const uint32_t xs = xsum + (uint32_t)(kb_first + c * kChunkBlocks) * 8u;
                if (nbc == kChunkBlocks) chunk_k<true>(st, xa, xs, nbc, sum);
                else chunk_k<false>(st, xa, xs, nbc, sum);
            } else {
                {   // the stage's scales, 16 bits each: lane (g, tig) gathers a quarter of the blocks of its two rows
                    constexpr int kPer = kChunkBlocks / 4;
                    const uint32_t ra = st + (uint32_t)g * kRowPitch + mA + (uint32_t)(tig * kPer * B::kBytes);
                    const uint32_t rb = st + (uint32_t)(8 + g) * kRowPitch + mB + (uint32_t)(tig * kPer * B::kBytes);
                    unsigned char* tab = const_cast<unsigned char*>(base) + stab;
#pragma unroll
                    for (int b = 0; b < kPer; b += 4) {
                        uint32_t ha[4], hb[4];
#pragma unroll
                        for (int u = 0; u < 4; u++) {
                            ha[u] = B::scale16(base, ra + (b + u) * B::kBytes);
                            hb[u] = B::scale16(base, rb + (b + u) * B::kBytes);
                        }
                        *reinterpret_cast<uint2*>(tab + (uint32_t)g * kScalePitch + (tig * kPer + b) * 2) =
                            make_uint2(ha[0] | (ha[1] << 16), ha[2] | (ha[3] << 16));
                        *reinterpret_cast<uint2*>(tab + (uint32_t)(8 + g) * kScalePitch + (tig * kPer + b) * 2) =
                            make_uint2(hb[0] | (hb[1] << 16), hb[2] | (hb[3] << 16));
                    }
                }
                __syncwarp();
                if (nbc == kChunkBlocks) chunk<true>(st, xa, nbc, sum);
                else chunk<false>(st, xa, nbc, sum);
            }
            __syncwarp();
        }
        seq += (uint32_t)nchunks;
    }
};

// The B fragments of one token, route or route group (`bytes` of global memory) into shared
// memory at offset 0 with one bulk copy by warp 0; every warp then waits on `bar` (phase 0).
__device__ __forceinline__ void fetch_fragments(SharedBase smem, const void* frag, uint32_t bytes, uint32_t bar, int warp, int lane) {
    if (warp == 0) {
        if (lane == 0) {
            mbar_init(bar, 1);
            fence_barrier_init();
            mbar_arrive_expect_tx(bar, bytes);
            bulk_copy(smem_u32(smem), frag, bytes, bar);
        }
    }
}

// Q4_K: (sum of the hi column, sum of the lo column) of every block of the fragments in shared memory,
// written behind them; called by all threads of the CTA once the fragments have landed.
__device__ __forceinline__ void fragment_sums(unsigned char* smem, int nkb, int tid, int threads) {
    for (int kb = tid; kb < nkb; kb += threads) {
        float s[2] = {0.f, 0.f};
#pragma unroll
        for (int col = 0; col < 2; col++)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint4 v = *reinterpret_cast<const uint4*>(smem + ((size_t)(kb * 2 + col) * 4 + i) * 16);
                const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[q]));
                    s[col] = __fadd_rn(s[col], __fadd_rn(f.x, f.y));
                }
            }
        *reinterpret_cast<float2*>(smem + (size_t)nkb * kFragBlockBytes + (size_t)kb * 8) = make_float2(s[0], s[1]);
    }
}

// Shared memory of the token kernels: B fragments | 2 KB (split sums, mbarriers, give-up flag) |
// per-warp scale tables | rings.
__host__ __device__ inline size_t token_smem_bytes(int fmt, int nkb, int stages) {
    return (size_t)frag_region_bytes(fmt, nkb) + kMiscBytes + (size_t)tok_warps(fmt) * scale_table_bytes(fmt) +
           (size_t)tok_warps(fmt) * stages * kStageBytes + 16;
}

// Splits f32 values into hi + lo halves and scatters them into the B-fragment layout:
// frag[((kb * 2 + col) * 4 + tig) * 4 + slot] is a half2 (element 4*tig+slot, element 4*tig+slot+16)
// of block kb; hi goes to column 0, lo to column 1.
// Q4_K delivers elements 8*tig .. 8*tig+7 of a sub-block to lane tig: slots 0, 1 hold (e0, e2), (e1, e3),
// slots 2, 3 the same of e4..e7.
__device__ __forceinline__ void frag_store(__half* frag, int k, float v, int fmt) {
    __half hi = __float2half_rn(v);
    float rem = nonfinite(v) ? 0.0f : v - __half2float(hi);
    __half lo = __float2half_rn(rem);
    int kb = k >> 5, j = k & 31, jj = j & 15, sel = j >> 4, tig = jj >> 2, slot = jj & 3;
    if (fmt == OCO_FMT_Q4_K) {
        const int r = j & 7;
        tig = j >> 3; slot = (r >> 2) * 2 + (r & 1); sel = (r >> 1) & 1;
    }
    size_t at = ((((size_t)kb * 2) * 4 + tig) * 4 + slot) * 2 + sel;
    frag[at] = hi;
    frag[at + (size_t)16 * 2] = lo;  // next column: 4 tig * 4 slots * 2 halves further
}

// Sums the per-warp partial results of a unit split over `ksplit` adjacent warps. `part`: shared
// scratch, 16 floats per warp. Returns the totals in the first warp of the group (lanes tig == 0).
__device__ __forceinline__ void join_split(float* part, int warp, int group, int s, int ksplit, int g, int tig,
                                           float& r0, float& r1) {
    if (ksplit == 1) return;
    if (s > 0 && tig == 0) { part[warp * 16 + g] = r0; part[warp * 16 + 8 + g] = r1; }
    named_barrier(1 + group, 32 * ksplit);
    if (s == 0 && tig == 0)
        for (int q = 1; q < ksplit; q++) {
            r0 = __fadd_rn(r0, part[(warp + q) * 16 + g]);
            r1 = __fadd_rn(r1, part[(warp + q) * 16 + 8 + g]);
        }
    named_barrier(1 + group, 32 * ksplit);   // the scratch may be written again after this
}

struct DecodeExpandParams {
    const uint8_t* gate_w;   // null when not gated
    const uint8_t* up_w;
    const float* gate_b;
    const float* up_b;
    const __half* xfrag;     // the token as B fragments, [H/32] blocks of 128 bytes (written by the router kernel)
    const uint32_t* ids;     // [K] selected experts; null = expert 0 (a one-expert bank)
    float* act;              // out f32 [K, F] (for inspection)
    __half* actfrag;         // out: B fragments of the down projection, [K][F/32] blocks of 128 bytes
    int H, F, K;
    int ksplit;              // warps per unit: a divisor of the warps per CTA
    uint32_t row_bytes;      // bytes from one gate (or up) row to the next: the packed length of a row of H
                             // elements, or twice that when gate and up rows are interleaved in one tensor
    int bias_stride;         // floats from one feature's bias to the next (1, or 2 when interleaved)
    uint32_t* status;        // device status word: a copy that never arrives is reported here
};

// Up (and gate) products of the K selected experts for one token, with the activation fused
// (reference expert_expand, projections.metal:78-137; matvec_q4 + relu^2, vector.metal:155-228).
// GATED: unit = 8 gate rows + 8 up rows (columns c0..c0+7); otherwise 16 up rows.
template <int ARCH, int FMT, int STAGES>
__global__ void __launch_bounds__(tok_warps(FMT) * 32, 1) decode_expand_kernel(const DecodeExpandParams p) {
    constexpr bool GATED = ARCH != OCO_ARCH_NEMOTRON;
    constexpr int COLS = GATED ? 8 : 16;
    constexpr int WARPS = tok_warps(FMT);
    extern __shared__ __align__(16) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, g = lane >> 2, tig = lane & 3;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);   // known to the compiler as the same in all lanes
    const int nkb = p.H / 32;
    const uint32_t part_off = frag_region_bytes(FMT, nkb);
    float* part = reinterpret_cast<float*>(smem + part_off);
    volatile uint32_t* give_up = reinterpret_cast<volatile uint32_t*>(part) + 496;
    const uint32_t xbar = smem_u32(smem) + part_off + 1920u;
    const uint32_t stab = part_off + kMiscBytes + (uint32_t)warp * scale_table_bytes(FMT);
    const uint32_t ring = part_off + kMiscBytes + (uint32_t)WARPS * scale_table_bytes(FMT) + (uint32_t)warp * STAGES * kStageBytes;
    pdl_launch_dependents();
    if (tid == 0) *give_up = 0u;

    const int ksplit = p.ksplit, group = warp / ksplit, s = warp - group * ksplit;
    const int groups = WARPS / ksplit;
    const int col_blocks = p.F / COLS;
    const int units = p.K * col_blocks;
    const int nslots = gridDim.x * groups;
    int bps = (nkb + ksplit - 1) / ksplit;
    if (FMT == OCO_FMT_Q4_K) bps = (bps + 7) & ~7;          // whole super-blocks
    const int kb0 = s * bps, nb = max(0, min(bps, nkb - kb0));
    const uint32_t xlane = (uint32_t)kb0 * kFragBlockBytes + (uint32_t)(((g & 1) * 4 + tig) * 16);

    RowStream<FMT, STAGES> rs;
    rs.init(smem, ring, stab, part_off + 1280u + (uint32_t)warp * (STAGES * 8), give_up, p.status, lane);
    rs.xsum = (uint32_t)nkb * kFragBlockBytes;
    pdl_wait();               // the router kernel's ids and fragments are complete
    fetch_fragments(smem, p.xfrag, (uint32_t)nkb * kFragBlockBytes, xbar, warp, lane);
    __syncthreads();          // the mbarriers exist
    if (FMT == OCO_FMT_Q4_K) {
        mbar_wait(xbar, 0u, give_up, p.status);
        fragment_sums(smem, nkb, tid, WARPS * 32);
        __syncthreads();
    }
    bool fetched = false;
    for (int unit = blockIdx.x * groups + group; unit < units; unit += nslots) {
        const int r = unit / col_blocks, c0 = (unit - r * col_blocks) * COLS;
        const uint32_t e = __shfl_sync(0xffffffffu, p.ids ? __ldg(p.ids + r) : 0u, 0);
        const size_t off = ((size_t)e * p.F + c0) * p.row_bytes;
        if (GATED) rs.begin(p.gate_w + off, p.up_w + off, p.row_bytes, kb0, nb);
        else rs.begin(p.up_w + off, p.up_w + off + (size_t)8 * p.row_bytes, p.row_bytes, kb0, nb);
        float b0 = 0.f, b1 = 0.f;
        if (ARCH == OCO_ARCH_GPT_OSS && s == 0 && tig == 0) {   // biases travel while the rows stream
            b0 = __ldg(p.gate_b + ((size_t)e * p.F + c0 + g) * p.bias_stride);
            b1 = __ldg(p.up_b + ((size_t)e * p.F + c0 + g) * p.bias_stride);
        }
        float sum[4] = {0.f, 0.f, 0.f, 0.f};
        if (!fetched) { mbar_wait(xbar, 0u, give_up, p.status); fetched = true; }
        rs.run(xlane, sum);
        float r0 = __fadd_rn(sum[0], sum[1]), r1 = __fadd_rn(sum[2], sum[3]);   // hi + lo columns (lanes tig == 0)
        join_split(part, warp, group, s, ksplit, g, tig, r0, r1);
        if (s == 0 && tig == 0) {
            auto put = [&](int col, float v) {
                p.act[(size_t)r * p.F + col] = v;
                frag_store(p.actfrag + (size_t)r * (p.F / 32) * (kFragBlockBytes / 2), col, v, FMT);
            };
            if (ARCH == OCO_ARCH_GPT_OSS) {
                float gate = __fadd_rn(r0, bf16_round(b0));
                float up = __fadd_rn(r1, bf16_round(__fadd_rn(b1, 1.0f)));
                put(c0 + g, swiglu_clipped(gate, up));
            } else if (ARCH == OCO_ARCH_QWEN) {
                put(c0 + g, silu_gate_bf16(bf16_round(r0), bf16_round(r1)));
            } else {
                float a = bf16_round(r0), b = bf16_round(r1);
                float ua = fmaxf(a, 0.0f), ub = fmaxf(b, 0.0f);
                put(c0 + g, a != a ? qnan() : __fmul_rn(ua, ua));
                put(c0 + 8 + g, b != b ? qnan() : __fmul_rn(ub, ub));
            }
        }
    }
}

struct DecodeDownParams {
    const uint8_t* down_w;
    const float* down_b;      // null when the family has no bias
    const uint32_t* ids;      // [K]; null = expert 0
    const __half* actfrag;    // [K][F/32] blocks of 128 bytes
    uint16_t* y;              // out bf16 [K, H]
    int H, F, K;
    int ksplit;
    uint32_t row_bytes;       // bytes of one packed row of length F
    // Fused combine (null residual = off): the warp that completes the last route of a block of 16
    // output rows adds the weighted expert outputs to the residual
    // (reference moe_sum, routing.metal:154-168; moe_add, nemotron.metal:222-236).
    uint32_t* arrivals;       // one zeroed counter per block of 16 output rows; left at zero again
    const float* probs;       // [K]
    uint16_t* residual;       // bf16 [H], in place
    const uint16_t* shared;   // bf16 [H] shared-expert output joining the sum, or null
    int round_sum;            // 1: the expert sum is rounded to bf16 before the residual add
    uint32_t* status;         // device status word
};

// Down products for one token: unit = 16 output rows of one route
// (reference matvec_mxfp4, projections.metal:140-182; matvec_q4, vector.metal:155-228).
// CTA c serves route c % K, so a CTA needs one route's fragments only.
template <int FMT, int STAGES>
__global__ void __launch_bounds__(tok_warps(FMT) * 32, 1) decode_down_kernel(const DecodeDownParams p) {
    constexpr int WARPS = tok_warps(FMT);
    extern __shared__ __align__(16) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, g = lane >> 2, tig = lane & 3;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const int nkb = p.F / 32;
    const int route = blockIdx.x % p.K, idx = blockIdx.x / p.K, ctas = gridDim.x / p.K;
    if (idx >= ctas) return;
    const uint32_t part_off = frag_region_bytes(FMT, nkb);
    float* part = reinterpret_cast<float*>(smem + part_off);
    volatile uint32_t* give_up = reinterpret_cast<volatile uint32_t*>(part) + 496;
    const uint32_t xbar = smem_u32(smem) + part_off + 1920u;
    const uint32_t stab = part_off + kMiscBytes + (uint32_t)warp * scale_table_bytes(FMT);
    const uint32_t ring = part_off + kMiscBytes + (uint32_t)WARPS * scale_table_bytes(FMT) + (uint32_t)warp * STAGES * kStageBytes;
    pdl_launch_dependents();
    if (tid == 0) *give_up = 0u;

    const int ksplit = p.ksplit, group = warp / ksplit, s = warp - group * ksplit;
    const int groups = WARPS / ksplit;
    const int row_blocks = p.H / 16;
    const int nslots = ctas * groups;
    int bps = (nkb + ksplit - 1) / ksplit;
    if (FMT == OCO_FMT_Q4_K) bps = (bps + 7) & ~7;
    const int kb0 = s * bps, nb = max(0, min(bps, nkb - kb0));
    const uint32_t xlane = (uint32_t)kb0 * kFragBlockBytes + (uint32_t)(((g & 1) * 4 + tig) * 16);

    RowStream<FMT, STAGES> rs;
    rs.init(smem, ring, stab, part_off + 1280u + (uint32_t)warp * (STAGES * 8), give_up, p.status, lane);
    rs.xsum = (uint32_t)nkb * kFragBlockBytes;
    pdl_wait();               // the expand kernel's fragments are complete
    // the route's activation fragments (written by the expand kernel)
    fetch_fragments(smem, p.actfrag + (size_t)route * nkb * (kFragBlockBytes / 2), (uint32_t)nkb * kFragBlockBytes, xbar, warp, lane);
    const uint32_t e = __shfl_sync(0xffffffffu, p.ids ? __ldg(p.ids + route) : 0u, 0);
    __syncthreads();          // the mbarriers exist
    if (FMT == OCO_FMT_Q4_K) {
        mbar_wait(xbar, 0u, give_up, p.status);
        fragment_sums(smem, nkb, tid, WARPS * 32);
        __syncthreads();
    }
    bool fetched = false;
    for (int rb = idx * groups + group; rb < row_blocks; rb += nslots) {
        const int d0 = rb * 16;
        const uint8_t* span = p.down_w + ((size_t)e * p.H + d0) * p.row_bytes;
        rs.begin(span, span + (size_t)8 * p.row_bytes, p.row_bytes, kb0, nb);
        float b0 = 0.f, b1 = 0.f;
        if (p.down_b && s == 0 && tig == 0) {
            b0 = __ldg(p.down_b + (size_t)e * p.H + d0 + g);
            b1 = __ldg(p.down_b + (size_t)e * p.H + d0 + 8 + g);
        }
        float sum[4] = {0.f, 0.f, 0.f, 0.f};
        if (!fetched) { mbar_wait(xbar, 0u, give_up, p.status); fetched = true; }
        rs.run(xlane, sum);
        float r0 = __fadd_rn(sum[0], sum[1]), r1 = __fadd_rn(sum[2], sum[3]);
        join_split(part, warp, group, s, ksplit, g, tig, r0, r1);
        if (s != 0) continue;
        if (tig == 0) {
            if (p.down_b) { r0 = __fadd_rn(r0, bf16_round(b0)); r1 = __fadd_rn(r1, bf16_round(b1)); }
            p.y[(size_t)route * p.H + d0 + g] = f32_to_bf16_bits(r0);
            p.y[(size_t)route * p.H + d0 + 8 + g] = f32_to_bf16_bits(r1);
        }
        if (p.residual) {
            // Whoever finishes a row block last combines it. No warp waits for another.
            __threadfence();
            __syncwarp();
            uint32_t seen = 0;
            if (lane == 0) {
                seen = atomicAdd(p.arrivals + rb, 1u);
                if (seen == (uint32_t)(p.K - 1)) p.arrivals[rb] = 0;   // ready for the next call on this stream
            }
            seen = __shfl_sync(0xffffffffu, seen, 0);
            // (a step during which a bounded wait gave up leaves the residual as it was)
            if (seen == (uint32_t)(p.K - 1) && lane < 16 && *reinterpret_cast<volatile uint32_t*>(p.status) == 0u) {
                __threadfence();
                const int row = d0 + lane;
                float sres = p.shared ? bf16_bits_to_f32(p.shared[row]) : 0.0f;
                for (int r = 0; r < p.K; r++)
                    sres = __fmaf_rn(bf16_bits_to_f32(__ldcg(p.y + (size_t)r * p.H + row)), p.probs[r], sres);
                if (p.round_sum) sres = bf16_round(sres);
                p.residual[row] = f32_to_bf16_bits(__fadd_rn(bf16_bits_to_f32(p.residual[row]), sres));
            }
        }
    }
}

// One token as the B fragments the single-token kernels multiply with (the router kernel does this on the
// side for the MoE layer; the dense products have no router). grid ceil(H / 256), 256 threads.
__global__ void __launch_bounds__(256) token_fragments_kernel(const uint16_t* __restrict__ x, int H, __half* __restrict__ xfrag, int fmt) {
    pdl_launch_dependents();
    pdl_wait();
    const int k = blockIdx.x * 256 + threadIdx.x;
    if (k < H) frag_store(xfrag, k, bf16_bits_to_f32(x[k]), fmt);
}

// Router of one token: logits (one warp per expert, reference router_logits, routing.metal:131-146),
// then the CTA that finishes last selects the experts and their weights for the whole token
// (routing.metal:71-94; nemotron.metal:167-211). On the side, the CTAs turn the token into the B
// fragments the expert kernels multiply with (or, for the block-scaled kernels, into e2m1 pieces).
// grid ceil(E/8), 256 threads.
template <int ARCH>
__global__ void __launch_bounds__(256) router_token_kernel(const uint16_t* __restrict__ x, const float* __restrict__ w,
                                                           const float* __restrict__ bias, int H, int E, int K,
                                                           int normalize, float scale, float* __restrict__ logits,
                                                           uint32_t* __restrict__ ids, float* __restrict__ probs,
                                                           __half* __restrict__ xfrag, int fmt, uint32_t* __restrict__ arrival,
                                                           unsigned char* __restrict__ mx_b, unsigned char* __restrict__ mx_sfb) {
    __shared__ int is_last;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e = blockIdx.x * 8 + warp;
    pdl_launch_dependents();  // the expand kernel may set itself up beside this small grid
    pdl_wait();               // the previous step no longer reads what this kernel writes
    if (e < E) {
        float s = H <= 128 * 24 ? canonical_logit_prefetch<ARCH == OCO_ARCH_GPT_OSS, 24>(x, w + (size_t)e * H, H, lane)
                                : canonical_logit<ARCH == OCO_ARCH_GPT_OSS>(x, w + (size_t)e * H, H, lane);
        if (ARCH == OCO_ARCH_GPT_OSS) s = __fadd_rn(s, bf16_round(bias[e]));
        if (lane == 0) logits[e] = s;
    }
    if (mx_b) {
        // the token as e2m1 pieces for the block-scaled expert kernels: one warp per 32-element block,
        // zero blocks up to the end of the last K group
        const int nkb = H >> 5, nblk = ((nkb + 7) >> 3) << 3;
        for (int blk = blockIdx.x * 8 + warp; blk < nblk; blk += gridDim.x * 8) {
            const float v = blk < nkb ? bf16_bits_to_f32(x[blk * 32 + (lane >> 1) + 16 * (lane & 1)]) : 0.0f;
            mx_split_block(v, lane, mx_b, mx_sfb, 8u, 0u, (uint32_t)blk);
        }
    } else {
        for (int k = blockIdx.x * 256 + threadIdx.x; k < H; k += gridDim.x * 256) frag_store(xfrag, k, bf16_bits_to_f32(x[k]), fmt);
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t seen = atomicAdd(arrival, 1u);
        is_last = seen == gridDim.x - 1;
        if (is_last) *arrival = 0;
    }
    __syncthreads();
    if (!is_last || warp != 0) return;
    __threadfence();
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int q = lane + 32 * j;
        v[j] = q < E ? __ldcg(logits + q) : 0.0f;
    }
    uint32_t id[kMaxTopK];
    float pr[kMaxTopK];
    select_experts<ARCH>(v, E, K, ARCH == OCO_ARCH_NEMOTRON ? bias : nullptr, normalize, scale, lane, id, pr);
#pragma unroll
    for (int r = 0; r < kMaxTopK; r++)
        if (r < K && lane == r) { ids[r] = id[r]; probs[r] = pr[r]; }
}

}  // namespace oco
