// CPU oracle for the mixture-of-experts layer of xhjkl/oco.
//
// TEST INFRASTRUCTURE ONLY. This file restates, in plain C++, the arithmetic of the reference's
// Metal kernels for the MoE path so that the CUDA implementation can be checked against it. It is
// never linked into, imported by or called from the product library; only the test-suite, the
// smoke check and the benchmark's CPU-baseline leg may load it.
//
// Parity status: the reference (Rust + Metal, macOS only) cannot be compiled or run on Linux and
// stores no golden files, so this oracle is pinned against the *constructions* of the reference's
// own kernel tests (same inputs, same independent f64 expectation, same analytic bound):
//   src/weights/dispatch_tests/mxfp4.rs:18-235   MXFP4 decode, expand, down matvec, NaN header
//   src/weights/dispatch_tests/mxfp4.rs:26-35,309-482  route plan, up/gate tiles, down tiles
//   src/weights/dispatch_tests/nemotron.rs:279-384     sigmoid router
//   src/weights/dispatch_tests/matrix_precision.rs:19-107  Q4_0 / Q4_K block decode
// Parts the reference has no test for (gpt-oss router softmax, moe_sum, moe_add, route_plan_n,
// the composed layer, every Qwen-MoE composition) are "parity unpinned": the oracle follows the
// shader text alone.
//
// Every function cites the reference file:line it follows (paths relative to the reference root).
//
// Accumulation: dot products are accumulated in double over exactly-representable products and
// rounded once to float ("fp32-accumulated result" up to summation order); every other rounding
// point (bf16 / fp16 conversions, f32 epilogue arithmetic) is the reference's.

#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>
#include <algorithm>
#include <limits>

#ifdef _OPENMP
#include <omp.h>
#endif

extern "C" {

// ----------------------------------------------------------------------------------------------
// Scalar conversions (round-to-nearest-even, as `half` 2.7.1 and MSL `bfloat(x)` / `half(x)` do).
// ----------------------------------------------------------------------------------------------
static inline uint32_t f2u(float f) { uint32_t u; std::memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; std::memcpy(&f, &u, 4); return f; }

uint16_t orc_f32_to_bf16(float f) {
    uint32_t u = f2u(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);  // quiet NaN
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return (uint16_t)(u >> 16);
}
float orc_bf16_to_f32(uint16_t h) { return u2f((uint32_t)h << 16); }
static inline float bf16r(float f) { return orc_bf16_to_f32(orc_f32_to_bf16(f)); }

uint16_t orc_f32_to_f16(float f) {
    uint32_t u = f2u(f);
    uint32_t sign = (u >> 16) & 0x8000u;
    uint32_t a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);           // NaN
    if (a >= 0x47800000u) return (uint16_t)(sign | 0x7c00u);          // >= 65536 -> inf (also inf)
    if (a < 0x33000000u) return (uint16_t)sign;                        // < 2^-25 -> 0
    int exp = (int)(a >> 23) - 127;
    uint32_t mant = (a & 0x7fffffu) | 0x800000u;
    int shift;            // bits to drop from the 24-bit significand
    uint32_t base;
    if (exp < -14) {      // subnormal half
        shift = 13 + (-14 - exp);
        base = 0;
    } else {
        shift = 13;
        base = (uint32_t)(exp + 15) << 10;
        mant &= 0x7fffffu;
    }
    uint32_t q = mant >> shift;
    uint32_t rem = mant & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) q++;
    uint32_t h = base + q;  // mantissa carry rolls into the exponent (and to inf) correctly
    return (uint16_t)(sign | h);
}
float orc_f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1fu, m = h & 0x3ffu;
    if (e == 0x1f) return u2f(sign | 0x7f800000u | (m << 13));
    if (e == 0) {
        if (m == 0) return u2f(sign);
        float v = (float)m * 5.9604644775390625e-08f;  // m * 2^-24
        return sign ? -v : v;
    }
    return u2f(sign | ((e + 112u) << 23) | (m << 13));
}
static inline float f16r(float f) { return orc_f16_to_f32(orc_f32_to_f16(f)); }

static inline bool nonfinite(float v) { return (f2u(v) & 0x7f800000u) == 0x7f800000u; }
static inline float qnan() { return u2f(0x7fc00000u); }

// Deterministic exp built only from IEEE basic operations (fma, add, mul, rint) so that the CUDA
// kernels, which carry the same sequence, return bit-identical values. The reference calls the
// Metal `exp` / `fast::exp` (routing.metal:91-93, projections.metal:10, nemotron.metal:177), whose
// last bits are not defined; any exp within a few ulp satisfies its tests (1e-3 / 1e-4 bounds).
float orc_exp(float a) {
    if (a != a) return a;
    if (a > 88.72283f) return std::numeric_limits<float>::infinity();
    if (a < -104.0f) return 0.0f;
    float n = rintf(a * 1.44269504088896341f);
    float r = fmaf(n, -0.693145751953125f, a);
    r = fmaf(n, -1.42860682030941723212e-6f, r);
    float p = 1.0f / 720.0f;
    p = fmaf(p, r, 1.0f / 120.0f);
    p = fmaf(p, r, 1.0f / 24.0f);
    p = fmaf(p, r, 1.0f / 6.0f);
    p = fmaf(p, r, 0.5f);
    p = fmaf(p, r, 1.0f);
    p = fmaf(p, r, 1.0f);
    int ni = (int)n;
    int n1 = ni / 2, n2 = ni - n1;
    float s1 = u2f((uint32_t)(n1 + 127) << 23), s2 = u2f((uint32_t)(n2 + 127) << 23);
    return (p * s1) * s2;
}

// ----------------------------------------------------------------------------------------------
// Block layouts (src/tensor.rs:24-36): GGUF type code -> (elements, bytes) per block.
// ----------------------------------------------------------------------------------------------
enum { FMT_Q4_0 = 2, FMT_Q4_K = 12, FMT_MXFP4 = 39 };

int orc_block_layout(int fmt, int* elems, int* bytes) {
    switch (fmt) {
        case FMT_Q4_0: *elems = 32; *bytes = 18; return 0;
        case FMT_Q4_K: *elems = 256; *bytes = 144; return 0;
        case FMT_MXFP4: *elems = 32; *bytes = 17; return 0;
    }
    return -1;
}

// E8M0 block scale (shaders/experts/projections.metal:19-23): 255 is NaN, 0 is 2^-127.
static inline float e8m0(uint32_t e) {
    if (e == 255) return qnan();
    return e == 0 ? u2f(0x00400000u) : u2f(e << 23);
}

// One weight as f32, element i of a row-major packed tensor (shaders/matrix/weights.metal:40-77).
static inline float weight_f32(const uint8_t* w, size_t i, int fmt) {
    if (fmt == FMT_MXFP4) {
        const uint8_t* b = w + i / 32 * 17;
        uint32_t j = (uint32_t)(i % 32);
        uint32_t q = (b[1 + j % 16] >> (j / 16 * 4)) & 15u;
        static const float mag[8] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
        float m = mag[q & 7];
        return ((q & 8) ? -m : m) * e8m0(b[0]);
    }
    if (fmt == FMT_Q4_0) {
        const uint8_t* b = w + i / 32 * 18;
        uint32_t j = (uint32_t)(i % 32);
        uint32_t q = (b[2 + j % 16] >> (j / 16 * 4)) & 15u;
        uint16_t d; std::memcpy(&d, b, 2);
        return orc_f16_to_f32(d) * (float)((int)q - 8);
    }
    // Q4_K (weights.metal:67-77): 144-byte super-block of 256.
    const uint8_t* b = w + i / 256 * 144;
    uint32_t j = (uint32_t)(i % 256), s = j / 32;
    const uint8_t* sc8 = b + 4;
    uint32_t sc = s < 4 ? (sc8[s] & 63u) : ((sc8[s + 4] & 15u) | ((uint32_t)(sc8[s - 4] >> 6) << 4));
    uint32_t mn = s < 4 ? (sc8[s + 4] & 63u) : ((uint32_t)(sc8[s + 4] >> 4) | ((uint32_t)(sc8[s] >> 6) << 4));
    uint32_t q = (b[16 + j / 64 * 32 + j % 32] >> (s % 2 * 4)) & 15u;
    uint16_t d, dm; std::memcpy(&d, b, 2); std::memcpy(&dm, b + 2, 2);
    // d*sc*q and dmin*mn are exact in f32 (11+6+4 and 11+6 significant bits); one rounding in the
    // subtraction, so the value does not depend on fused/unfused evaluation.
    float a = orc_f16_to_f32(d) * (float)sc * (float)q;
    float c = orc_f16_to_f32(dm) * (float)mn;
    return a - c;
}

void orc_dequant(int fmt, const uint8_t* w, size_t n_elems, float* out) {
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < (long long)n_elems; i++) out[i] = weight_f32(w, (size_t)i, fmt);
}

// The prefill tiles' operand precision: decoded coefficient rounded to half
// (projections.metal:227,312; shaders/matrix/q4_tile.metal:24-37).
void orc_dequant_f16(int fmt, const uint8_t* w, size_t n_elems, uint16_t* out) {
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < (long long)n_elems; i++)
        out[i] = orc_f32_to_f16(weight_f32(w, (size_t)i, fmt));
}

// ----------------------------------------------------------------------------------------------
// Router logits in the canonical summation order.
// Lane l of 32 owns k = 4*l + 128*i; four FMA chains (one per vector component), combined as
// (x+y)+(z+w) (routing.metal:105-112, 136-143; nemotron.metal:156-162), then the 32 lane sums are
// reduced. The reference's `simd_sum` order is unspecified; the order fixed here (xor butterfly
// 16,8,4,2,1) is this build's definition and the CUDA kernel carries the same one.
// ----------------------------------------------------------------------------------------------
static float canonical_dot(const uint16_t* x_bf16, const float* w, int n, bool round_w) {
    float lane_sum[32];
    for (int lane = 0; lane < 32; lane++) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int k = lane * 4; k < n; k += 128)
            for (int c = 0; c < 4; c++) {
                float a = orc_bf16_to_f32(x_bf16[k + c]);
                float b = round_w ? bf16r(w[k + c]) : w[k + c];
                acc[c] = fmaf(a, b, acc[c]);
            }
        lane_sum[lane] = (acc[0] + acc[1]) + (acc[2] + acc[3]);
    }
    for (int off = 16; off >= 1; off >>= 1) {
        float next[32];
        for (int l = 0; l < 32; l++) next[l] = lane_sum[l] + lane_sum[l ^ off];
        std::memcpy(lane_sum, next, sizeof(next));
    }
    return lane_sum[0];
}

// gpt-oss router: logits over bf16-rounded weights and bias, top-4 with ties to the lowest index,
// softmax over the four bf16-rounded winners, probabilities rounded to bf16
// (routing.metal:71-94 select_expert_values, :96-128 router, :131-146 router_logits).
void orc_router_gptoss(const uint16_t* x, const float* W, const float* bias, int T, int H, int E,
                       int top_k, float* logits_out, uint32_t* ids, float* probs) {
#pragma omp parallel for schedule(static)
    for (int t = 0; t < T; t++) {
        std::vector<float> logit(E);
        for (int e = 0; e < E; e++)
            logit[e] = canonical_dot(x + (size_t)t * H, W + (size_t)e * H, H, true) + bf16r(bias[e]);
        if (logits_out) std::memcpy(logits_out + (size_t)t * E, logit.data(), sizeof(float) * E);
        bool invalid = false;
        std::vector<float> v(E);
        std::vector<char> avail(E, 1);
        for (int e = 0; e < E; e++) {
            bool fin = !nonfinite(logit[e]);
            invalid = invalid || !fin;
            v[e] = fin ? logit[e] : -std::numeric_limits<float>::infinity();
        }
        std::vector<float> chosen(top_k);
        for (int r = 0; r < top_k; r++) {
            float mx = -std::numeric_limits<float>::infinity();
            for (int e = 0; e < E; e++) if (avail[e]) mx = std::max(mx, v[e]);
            uint32_t id = 0xffffffffu;
            for (int e = 0; e < E; e++) if (avail[e] && v[e] == mx) { id = (uint32_t)e; break; }
            ids[(size_t)t * top_k + r] = id;
            chosen[r] = bf16r(mx);
            if (id < (uint32_t)E) avail[id] = 0;
        }
        for (int r = 0; r < top_k; r++) invalid = invalid || nonfinite(chosen[r]);
        if (invalid) {
            for (int r = 0; r < top_k; r++) probs[(size_t)t * top_k + r] = qnan();
            continue;
        }
        float sum = 0.f;
        for (int r = 0; r < top_k; r++) sum += orc_exp(chosen[r] - chosen[0]);
        for (int r = 0; r < top_k; r++)
            probs[(size_t)t * top_k + r] = bf16r(orc_exp(chosen[r] - chosen[0]) / sum);
    }
}

// Sigmoid router (shaders/nemotron.metal:140-212): unrounded f32 weights, no logit bias,
// score = 1/(1+exp(-l)); selection by score + bias, iterative top-`active`, ties to the lowest
// index; weights are the unbiased scores, optionally normalised (floor 2^-14) and scaled.
void orc_router_sigmoid(const uint16_t* x, const float* W, const float* sel_bias, int T, int H,
                        int E, int active, int normalize, float scale, float* logits_out,
                        uint32_t* ids, float* probs) {
#pragma omp parallel for schedule(static)
    for (int t = 0; t < T; t++) {
        std::vector<float> logit(E), sel(E);
        bool invalid = false;
        for (int e = 0; e < E; e++) {
            logit[e] = canonical_dot(x + (size_t)t * H, W + (size_t)e * H, H, false);
            invalid = invalid || nonfinite(logit[e]);
            float score = 1.0f / (1.0f + orc_exp(-logit[e]));
            sel[e] = score + sel_bias[e];
        }
        if (logits_out) std::memcpy(logits_out + (size_t)t * E, logit.data(), sizeof(float) * E);
        float total = 0.f;
        std::vector<float> wts(active);
        for (int r = 0; r < active; r++) {
            // max with NaN-ignoring semantics of a strict `>` scan seeded by the first entry per
            // lane followed by simd_max: NaN selections never win against finite ones.
            float peak = -std::numeric_limits<float>::infinity();
            for (int e = 0; e < E; e++) if (sel[e] > peak) peak = sel[e];
            uint32_t id = 0xffffffffu;
            for (int e = 0; e < E; e++) if (sel[e] == peak) { id = (uint32_t)e; break; }
            if (id == 0xffffffffu) id = 0;  // all NaN: keep a valid index (probs become NaN below)
            ids[(size_t)t * active + r] = id;
            sel[id] = -std::numeric_limits<float>::infinity();
            float w = 1.0f / (1.0f + orc_exp(-logit[id]));
            wts[r] = w;
            total += w;
        }
        float divisor = normalize ? std::max(total, 6.103515625e-5f) : 1.0f;
        for (int r = 0; r < active; r++)
            probs[(size_t)t * active + r] = invalid ? qnan() : wts[r] / divisor * scale;
    }
}

// Softmax-over-all then top-k renormalised (Qwen3-MoE shaped layer). The reference has no such
// router (src/weights/qwen.rs:11 is dense-FFN only); this follows the benchmark's description and
// the sigmoid router's conventions (unrounded f32 weights, canonical logits, ties to the lowest
// index). Softmax over all experts followed by renormalising the top-k equals a softmax over the
// k winning logits: p_r = exp(l_r - l_0) / sum_j exp(l_j - l_0). Parity unpinned.
void orc_router_softmax_topk(const uint16_t* x, const float* W, int T, int H, int E, int active,
                             float* logits_out, uint32_t* ids, float* probs) {
#pragma omp parallel for schedule(static)
    for (int t = 0; t < T; t++) {
        std::vector<float> logit(E), v(E);
        bool invalid = false;
        for (int e = 0; e < E; e++) {
            logit[e] = canonical_dot(x + (size_t)t * H, W + (size_t)e * H, H, false);
            bool fin = !nonfinite(logit[e]);
            invalid = invalid || !fin;
            v[e] = fin ? logit[e] : -std::numeric_limits<float>::infinity();
        }
        if (logits_out) std::memcpy(logits_out + (size_t)t * E, logit.data(), sizeof(float) * E);
        std::vector<char> avail(E, 1);
        std::vector<float> chosen(active);
        for (int r = 0; r < active; r++) {
            float mx = -std::numeric_limits<float>::infinity();
            for (int e = 0; e < E; e++) if (avail[e]) mx = std::max(mx, v[e]);
            uint32_t id = 0;
            for (int e = 0; e < E; e++) if (avail[e] && v[e] == mx) { id = (uint32_t)e; break; }
            ids[(size_t)t * active + r] = id;
            chosen[r] = mx;
            avail[id] = 0;
        }
        for (int r = 0; r < active; r++) invalid = invalid || nonfinite(chosen[r]);
        if (invalid) {
            for (int r = 0; r < active; r++) probs[(size_t)t * active + r] = qnan();
            continue;
        }
        float sum = 0.f;
        for (int r = 0; r < active; r++) sum += orc_exp(chosen[r] - chosen[0]);
        for (int r = 0; r < active; r++)
            probs[(size_t)t * active + r] = orc_exp(chosen[r] - chosen[0]) / sum;
    }
}

// ----------------------------------------------------------------------------------------------
// Route plans in the reference's word layout.
// ----------------------------------------------------------------------------------------------
// route_plan_tiled<TileRows> for 32 experts (routing.metal:4-39). `plan` must hold
// 6 + 2*(ceil(R/16)+32) + 32*(R+1) + 32 + R words (src/weights/gpt_oss.rs:67-73).
size_t orc_route_plan_tiled_words(uint32_t routes) {
    return 6 + 2 * ((size_t)(routes + 15) / 16 + 32) + 32 * ((size_t)routes + 1) + 32 + routes;
}
void orc_route_plan_tiled(const uint32_t* ids, uint32_t routes, uint32_t tile_rows,
                          uint32_t up_tiles, uint32_t down_tiles, uint32_t* plan) {
    uint32_t grouped = 6 + 2 * ((routes + 15) / 16 + 32);
    for (uint32_t expert = 0; expert < 32; expert++) {
        uint32_t base = grouped + expert * (routes + 1), count = 0;
        for (uint32_t i = 0; i < routes; i++)
            if (ids[i] == expert) plan[base + 1 + count++] = i;
        plan[base] = count;
    }
    uint32_t sorted = grouped + 32 * (routes + 1);
    uint32_t tiles = 0, offset = 0;
    for (uint32_t e = 0; e < 32; e++) {
        uint32_t routed = plan[grouped + e * (routes + 1)];
        plan[sorted + e] = offset;
        offset += routed;
        for (uint32_t begin = 0; begin < routed; begin += tile_rows) {
            plan[6 + tiles * 2] = e;
            plan[6 + tiles * 2 + 1] = begin;
            tiles++;
        }
    }
    plan[0] = up_tiles; plan[1] = tiles; plan[2] = 1;
    plan[3] = down_tiles; plan[4] = tiles; plan[5] = 1;
    for (uint32_t expert = 0; expert < 32; expert++) {
        uint32_t base = grouped + expert * (routes + 1), count = plan[base];
        uint32_t off = plan[sorted + expert];
        for (uint32_t i = 0; i < count; i++) plan[sorted + 32 + plan[base + 1 + i]] = off + i;
    }
}

// route_plan_n (nemotron.metal:238-273): up to 128 experts, tile_rows 8 or 32, no sorted-row map.
// Sized exactly here: 6 + 2*(ceil(R/tile_rows)+E) + E*(R+1) words. (The reference host sizes the
// buffer with ceil(R/16), src/weights/compute/nemotron.rs:56-58, which is short for tile_rows = 8;
// that is not reproduced.)
size_t orc_route_plan_n_words(uint32_t routes, uint32_t experts, uint32_t tile_rows) {
    return 6 + 2 * ((size_t)(routes + tile_rows - 1) / tile_rows + experts) +
           (size_t)experts * ((size_t)routes + 1);
}
void orc_route_plan_n(const uint32_t* ids, uint32_t routes, uint32_t experts, uint32_t tile_rows,
                      uint32_t up_tiles, uint32_t down_tiles, uint32_t* plan) {
    uint32_t lists = 6 + 2 * ((routes + tile_rows - 1) / tile_rows + experts);
    for (uint32_t expert = 0; expert < experts; expert++) {
        uint32_t base = lists + expert * (routes + 1), count = 0;
        for (uint32_t i = 0; i < routes; i++)
            if (ids[i] == expert) plan[base + 1 + count++] = i;
        plan[base] = count;
    }
    uint32_t tiles = 0;
    for (uint32_t e = 0; e < experts; e++)
        for (uint32_t begin = 0; begin < plan[lists + e * (routes + 1)]; begin += tile_rows) {
            plan[6 + tiles * 2] = e;
            plan[6 + tiles * 2 + 1] = begin;
            tiles++;
        }
    plan[0] = up_tiles; plan[1] = tiles; plan[2] = 1;
    plan[3] = down_tiles; plan[4] = tiles; plan[5] = 1;
}

// The permutation those plans encode, in flat form: exclusive offsets per expert, each route's
// expert-sorted row (a stable sort of route indices by expert id) and its inverse.
void orc_permutation(const uint32_t* ids, uint32_t routes, uint32_t experts, uint32_t* offsets,
                     uint32_t* row_of_route, uint32_t* route_of_row) {
    std::vector<uint32_t> count(experts, 0);
    for (uint32_t i = 0; i < routes; i++) count[ids[i]]++;
    uint32_t acc = 0;
    for (uint32_t e = 0; e < experts; e++) { offsets[e] = acc; acc += count[e]; }
    offsets[experts] = acc;
    std::vector<uint32_t> cursor(offsets, offsets + experts);
    for (uint32_t i = 0; i < routes; i++) {
        uint32_t row = cursor[ids[i]]++;
        row_of_route[i] = row;
        route_of_row[row] = i;
    }
}

// ----------------------------------------------------------------------------------------------
// Activations.
// ----------------------------------------------------------------------------------------------
// Clipped SwiGLU (projections.metal:4-13, routing.metal:52-63).
static inline float swiglu_clipped(float g, float u) {
    if (nonfinite(g) || nonfinite(u)) return qnan();
    g = std::min(g, 7.0f);
    u = std::min(std::max(u, -6.0f), 8.0f);
    float e = orc_exp(-std::fabs(g) * 1.702f);
    float sigmoid = (g < 0 ? e : 1.0f) / (1.0f + e);
    return sigmoid * g * u;
}
float orc_swiglu_clipped(float g, float u) { return swiglu_clipped(g, u); }

// SiLU gate of bf16 operands (shaders/elementwise.metal:67-87): bf16( f32(bf16(sigmoid(a)*a)) * b ).
static inline float silu_gate_bf16(float a, float b) {
    if (nonfinite(a) || nonfinite(b)) return qnan();
    float e = orc_exp(-std::fabs(a));
    float sigmoid = (a < 0 ? e : 1.0f) / (1.0f + e);
    float activated = sigmoid * a;
    return bf16r(bf16r(activated) * b);
}
float orc_silu_gate_bf16(float a, float b) { return silu_gate_bf16(a, b); }

// ----------------------------------------------------------------------------------------------
// The layer.
// ----------------------------------------------------------------------------------------------
enum { ARCH_GPT_OSS = 0, ARCH_NEMOTRON = 1, ARCH_QWEN = 2 };

struct OrcLayer {
    int32_t arch;
    int32_t hidden, ffn, experts, top_k, shared_ffn;
    int32_t fmt;
    int32_t normalize;
    float scale;
    int32_t reserved;
    const float* router_w;      // [E, H] f32
    const float* router_b;      // gpt-oss: logit bias [E]; nemotron: selection bias [E]; qwen: null
    const uint8_t* gate_w;      // [E][ffn][H] packed (gated archs)
    const uint8_t* up_w;        // [E][ffn][H] packed
    const uint8_t* down_w;      // [E][H][ffn] packed
    const float* gate_b;        // gpt-oss [E, ffn]
    const float* up_b;          // gpt-oss [E, ffn]
    const float* down_b;        // gpt-oss [E, H]
    const uint8_t* shared_up_w;    // nemotron [shared_ffn][H] packed
    const uint8_t* shared_down_w;  // nemotron [H][shared_ffn] packed
};

struct OrcTrace {          // optional intermediates; any pointer may be null
    float* logits;         // [T, E]
    uint32_t* ids;         // [T*k]
    float* probs;          // [T*k]
    float* act;            // [R, ffn] activated intermediate as f32 values, route order
    uint16_t* y;           // [R, H] bf16 expert outputs, route order
};

static size_t row_bytes(int fmt, int k) {
    int el, by; orc_block_layout(fmt, &el, &by);
    return (size_t)k / el * by;
}

static void decode_row(const uint8_t* w, int fmt, int k, bool half, float* out) {
    for (int i = 0; i < k; i++) {
        float v = weight_f32(w, (size_t)i, fmt);
        out[i] = half ? f16r(v) : v;
    }
}

static inline float dotd(const float* a, const float* b, int n) {
    double s0 = 0, s1 = 0, s2 = 0, s3 = 0;
    int i = 0;
    for (; i + 3 < n; i += 4) {
        s0 += (double)a[i] * b[i];
        s1 += (double)a[i + 1] * b[i + 1];
        s2 += (double)a[i + 2] * b[i + 2];
        s3 += (double)a[i + 3] * b[i + 3];
    }
    for (; i < n; i++) s0 += (double)a[i] * b[i];
    return (float)((s0 + s1) + (s2 + s3));
}
static inline float dotf(const float* a, const float* b, int n) {
    float s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    int i = 0;
    for (; i + 7 < n; i += 8)
        for (int j = 0; j < 8; j++) s[j] = fmaf(a[i + j], b[i + j], s[j]);
    for (; i < n; i++) s[0] = fmaf(a[i], b[i], s[0]);
    return ((s[0] + s[1]) + (s[2] + s[3])) + ((s[4] + s[5]) + (s[6] + s[7]));
}

// ----------------------------------------------------------------------------------------------
// Kernel-level primitives, one per reference kernel, used to pin the oracle against the
// reference's own kernel tests. orc_moe_forward below composes the same arithmetic.
// ----------------------------------------------------------------------------------------------
// expert_expand (projections.metal:78-137): single-token up and gate products with the fused
// clipped SwiGLU. uy = sum + bf16(ub + 1); gy = swiglu(sum_g + bf16(gb), uy). x is one bf16 row.
void orc_expert_expand(const uint8_t* uw, const uint8_t* gw, const uint16_t* x_bf16,
                       const float* ub, const float* gb, const uint32_t* ids, int routes, int k,
                       int n, int fmt, float* uy, float* gy) {
    std::vector<float> x(k), wrow(k);
    for (int i = 0; i < k; i++) x[i] = orc_bf16_to_f32(x_bf16[i]);
    const size_t rb = row_bytes(fmt, k);
    for (int r = 0; r < routes; r++) {
        size_t e = ids[r];
        for (int c = 0; c < n; c++) {
            decode_row(uw + (e * n + c) * rb, fmt, k, false, wrow.data());
            float up = dotd(wrow.data(), x.data(), k) + bf16r(ub[e * n + c] + 1.0f);
            decode_row(gw + (e * n + c) * rb, fmt, k, false, wrow.data());
            float gate = dotd(wrow.data(), x.data(), k) + bf16r(gb[e * n + c]);
            uy[(size_t)r * n + c] = up;
            gy[(size_t)r * n + c] = swiglu_clipped(gate, up);
        }
    }
}

// matvec_mxfp4 / gathered matvec (projections.metal:140-182, vector.metal:155-228): f32 inputs per
// route, bf16( sum + bf16(bias) ). relu2 != 0 squares the positive part of the input on load
// (vector.metal:185-190).
void orc_expert_down_vector(const uint8_t* w, const float* x, const float* bias,
                            const uint32_t* ids, int routes, int k, int n, int fmt, int relu2,
                            uint16_t* y) {
    std::vector<float> wrow(k), xin(k);
    const size_t rb = row_bytes(fmt, k);
    for (int r = 0; r < routes; r++) {
        size_t e = ids[r];
        for (int i = 0; i < k; i++) {
            float v = x[(size_t)r * k + i];
            if (relu2) { v = std::max(v, 0.0f); v = v * v; }
            xin[i] = v;
        }
        for (int c = 0; c < n; c++) {
            decode_row(w + (e * n + c) * rb, fmt, k, false, wrow.data());
            float v = dotd(wrow.data(), xin.data(), k) + (bias ? bf16r(bias[e * n + c]) : 0.0f);
            y[(size_t)r * n + c] = orc_f32_to_bf16(v);
        }
    }
}

// expert_up_tensor / expert_mxfp4_up (projections.metal:192-271): half operands (decoded weight
// and gathered bf16 input both converted to half), fp32 accumulation, + bf16(bias + shift), f32
// result in route order. Route r reads token r / per_token.
void orc_expert_up_tile(const uint8_t* w, const uint16_t* x_bf16, const float* bias, float shift,
                        const uint32_t* ids, int routes, int per_token, int k, int n, int fmt,
                        float* y) {
    std::vector<float> wrow(k), xin(k);
    const size_t rb = row_bytes(fmt, k);
    for (int r = 0; r < routes; r++) {
        size_t e = ids[r];
        for (int i = 0; i < k; i++) xin[i] = f16r(orc_bf16_to_f32(x_bf16[(size_t)(r / per_token) * k + i]));
        for (int c = 0; c < n; c++) {
            decode_row(w + (e * n + c) * rb, fmt, k, true, wrow.data());
            y[(size_t)r * n + c] =
                dotd(wrow.data(), xin.data(), k) + (bias ? bf16r(bias[e * n + c] + shift) : 0.0f);
        }
    }
}

// expert_down_tensor / expert_mxfp4_down (projections.metal:278-346): half activations (given here
// in route order as f16 bits), half weights, fp32 accumulation, bf16( sum + bf16(bias) ).
void orc_expert_down_tile(const uint8_t* w, const uint16_t* act_f16, const float* bias,
                          const uint32_t* ids, int routes, int k, int n, int fmt, uint16_t* y) {
    std::vector<float> wrow(k), xin(k);
    const size_t rb = row_bytes(fmt, k);
    for (int r = 0; r < routes; r++) {
        size_t e = ids[r];
        for (int i = 0; i < k; i++) xin[i] = orc_f16_to_f32(act_f16[(size_t)r * k + i]);
        for (int c = 0; c < n; c++) {
            decode_row(w + (e * n + c) * rb, fmt, k, true, wrow.data());
            float v = dotd(wrow.data(), xin.data(), k) + (bias ? bf16r(bias[e * n + c]) : 0.0f);
            y[(size_t)r * n + c] = orc_f32_to_bf16(v);
        }
    }
}

// moe_activate (routing.metal:44-64): clipped SwiGLU of f32 projections, rounded to half.
void orc_moe_activate(const float* g, const float* u, size_t count, uint16_t* out_f16) {
    for (size_t i = 0; i < count; i++) out_f16[i] = orc_f32_to_f16(swiglu_clipped(g[i], u[i]));
}

// moe_sum (routing.metal:154-168).
// Residual add + RMS normalisation (shaders/elementwise.metal:5-30 norm, :32-60 add_norm; call
// sites src/weights/compute.rs:86-117, src/weights/gpt_oss.rs:122). hidden += delta as a bf16 add
// (delta may be null: plain norm), out = hidden * rsqrt(mean(hidden^2) + eps) * w with the
// family's rounding (full_layer: scale in f32, round once; else round the normalised value and
// the weight to bf16 first). The reference's simd_sum order is unspecified; the order fixed here
// (256 strided partial sums with FMA, xor butterfly 16..1 inside each group of 32, then the same
// butterfly over the eight group sums padded with zeros) is this build's definition and the CUDA
// kernel carries the same one. rsqrt is taken as 1 / sqrt with IEEE division and square root.
void orc_add_norm(uint16_t* hidden, const uint16_t* delta, const float* w, int rows, int n, float eps,
                  int full_layer, uint16_t* out) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; r++) {
        uint16_t* row = hidden + (size_t)r * n;
        float part[256];
        for (int t = 0; t < 256; t++) {
            float s = 0.f;
            for (int i = t; i < n; i += 256) {
                float v = orc_bf16_to_f32(row[i]);
                if (delta) {
                    v = bf16r(v + orc_bf16_to_f32(delta[(size_t)r * n + i]));
                    row[i] = orc_f32_to_bf16(v);
                }
                s = fmaf(v, v, s);
            }
            part[t] = s;
        }
        float group[32];
        for (int g = 0; g < 32; g++) group[g] = 0.f;
        for (int g = 0; g < 8; g++) {
            float lane[32];
            for (int l = 0; l < 32; l++) lane[l] = part[g * 32 + l];
            for (int off = 16; off >= 1; off >>= 1) {
                float next[32];
                for (int l = 0; l < 32; l++) next[l] = lane[l] + lane[l ^ off];
                std::memcpy(lane, next, sizeof(next));
            }
            group[g] = lane[0];
        }
        for (int off = 16; off >= 1; off >>= 1) {
            float next[32];
            for (int l = 0; l < 32; l++) next[l] = group[l] + group[l ^ off];
            std::memcpy(group, next, sizeof(next));
        }
        const float inv = 1.0f / sqrtf(group[0] / (float)n + eps);
        for (int i = 0; i < n; i++) {
            const float normalized = orc_bf16_to_f32(row[i]) * inv;
            const float v = full_layer ? normalized * w[i] : bf16r(normalized) * bf16r(w[i]);
            out[(size_t)r * n + i] = orc_f32_to_bf16(v);
        }
    }
}

void orc_moe_sum(const uint16_t* routes_bf16, const float* weights, uint16_t* out_bf16, int hidden,
                 int batch, int k) {
    for (int t = 0; t < batch; t++)
        for (int d = 0; d < hidden; d++) {
            float s = 0.f;
            for (int r = 0; r < k; r++)
                s = fmaf(orc_bf16_to_f32(routes_bf16[((size_t)t * k + r) * hidden + d]),
                         weights[(size_t)t * k + r], s);
            size_t i = (size_t)t * hidden + d;
            out_bf16[i] = orc_f32_to_bf16(orc_bf16_to_f32(out_bf16[i]) + bf16r(s));
        }
}

// moe_add (nemotron.metal:222-236).
void orc_moe_add(const uint16_t* routes_bf16, const float* weights, uint16_t* out_bf16,
                 const uint16_t* shared_bf16, int hidden, int batch, int k) {
    for (int t = 0; t < batch; t++)
        for (int d = 0; d < hidden; d++) {
            size_t i = (size_t)t * hidden + d;
            float s = shared_bf16 ? orc_bf16_to_f32(shared_bf16[i]) : 0.0f;
            for (int r = 0; r < k; r++)
                s = fmaf(orc_bf16_to_f32(routes_bf16[((size_t)t * k + r) * hidden + d]),
                         weights[(size_t)t * k + r], s);
            out_bf16[i] = orc_f32_to_bf16(orc_bf16_to_f32(out_bf16[i]) + s);
        }
}

// mode: 0 = as the reference (rows == 1 -> single-token numerics, else tile numerics),
//       1 = single-token numerics for every row, 2 = tile numerics for every row.
// accumulate_f32: 0 = double accumulation (the checker), 1 = f32 FMA accumulation (the timed CPU
// baseline, closer to what the shaders execute).
//
// gpt-oss: Bindings::experts (src/weights/compute/feed_forward.rs:107-275) with the kernels of
//   shaders/experts/{routing,projections}.metal.
// nemotron: Bindings::relu_experts / relu_experts_single (src/weights/compute/nemotron.rs:286-545)
//   with shaders/nemotron.metal:140-488 and shaders/matrix/vector.metal:151-228 (matvec_q4).
// qwen: composition defined by this build (parity unpinned), from the same building blocks.
int orc_moe_forward(const OrcLayer* L, const uint16_t* x, uint16_t* residual, int rows, int mode,
                    int accumulate_f32, OrcTrace* trace) {
    const int H = L->hidden, F = L->ffn, E = L->experts, K = L->top_k, T = rows;
    const int R = T * K;
    const bool tile = mode == 2 || (mode == 0 && rows > 1);
    auto dot = accumulate_f32 ? dotf : dotd;

    std::vector<uint32_t> ids((size_t)R);
    std::vector<float> probs((size_t)R);
    float* logits = trace ? trace->logits : nullptr;
    if (L->arch == ARCH_GPT_OSS)
        orc_router_gptoss(x, L->router_w, L->router_b, T, H, E, K, logits, ids.data(), probs.data());
    else if (L->arch == ARCH_NEMOTRON)
        orc_router_sigmoid(x, L->router_w, L->router_b, T, H, E, K, L->normalize, L->scale, logits,
                           ids.data(), probs.data());
    else
        orc_router_softmax_topk(x, L->router_w, T, H, E, K, logits, ids.data(), probs.data());
    if (trace && trace->ids) std::memcpy(trace->ids, ids.data(), sizeof(uint32_t) * R);
    if (trace && trace->probs) std::memcpy(trace->probs, probs.data(), sizeof(float) * R);

    // Input rows as the kernels see them: exact bf16 for single-token kernels
    // (projections.metal:114-123), converted to half for the tiles (projections.metal:229-233,
    // nemotron.metal:327-335).
    std::vector<float> xin((size_t)T * H);
    for (size_t i = 0; i < (size_t)T * H; i++) {
        float v = orc_bf16_to_f32(x[i]);
        xin[i] = tile ? f16r(v) : v;
    }

    // Routes grouped by expert so each expert's rows are decoded once.
    std::vector<uint32_t> offsets(E + 1), row_of_route(R), route_of_row(R);
    orc_permutation(ids.data(), R, E, offsets.data(), row_of_route.data(), route_of_row.data());

    std::vector<float> act((size_t)R * F);       // input of the down projection, per route
    std::vector<uint16_t> y((size_t)R * H);      // bf16 expert outputs, per route
    const size_t up_row = row_bytes(L->fmt, H), down_row = row_bytes(L->fmt, F);
    const bool gated = L->arch != ARCH_NEMOTRON;

#pragma omp parallel
    {
        std::vector<float> wrow(std::max(H, std::max(F, (int)L->shared_ffn)));
        std::vector<float> wrow2(std::max(H, F));
        // ---- up (and gate) projections + activation ------------------------------------------
#pragma omp for schedule(dynamic, 8) collapse(2)
        for (int e = 0; e < E; e++)
            for (int c = 0; c < F; c++) {
                uint32_t b = offsets[e], n = offsets[e + 1] - b;
                if (n == 0) continue;
                decode_row(L->up_w + ((size_t)e * F + c) * up_row, L->fmt, H, tile, wrow.data());
                if (gated)
                    decode_row(L->gate_w + ((size_t)e * F + c) * up_row, L->fmt, H, tile, wrow2.data());
                for (uint32_t i = 0; i < n; i++) {
                    uint32_t route = route_of_row[b + i];
                    const float* xr = xin.data() + (size_t)(route / K) * H;
                    float up = dot(wrow.data(), xr, H);
                    float a;
                    if (L->arch == ARCH_GPT_OSS) {
                        // projections.metal:130-136 (single token), :266-268 + routing.metal:52-63.
                        up += bf16r(L->up_b[(size_t)e * F + c] + 1.0f);
                        float gate = dot(wrow2.data(), xr, H) + bf16r(L->gate_b[(size_t)e * F + c]);
                        a = swiglu_clipped(gate, up);
                        if (tile) a = f16r(a);                      // routing.metal:63
                    } else if (L->arch == ARCH_NEMOTRON) {
                        // vector.metal:219-227 / nemotron.metal:386,478: bf16 store, then relu^2 in
                        // f32 on load (vector.metal:185-190; nemotron.metal:328-333 -> half).
                        float v = std::max(bf16r(up), 0.0f);
                        a = v * v;
                        if (tile) a = f16r(a);
                    } else {
                        float gate = dot(wrow2.data(), xr, H);
                        a = silu_gate_bf16(bf16r(gate), bf16r(up));  // a bf16 value
                        if (tile) a = f16r(a);                       // the tiles' operand conversion
                    }
                    act[(size_t)route * F + c] = a;
                }
            }
        // ---- down projection ------------------------------------------------------------------
#pragma omp for schedule(dynamic, 8) collapse(2)
        for (int e = 0; e < E; e++)
            for (int d = 0; d < H; d++) {
                uint32_t b = offsets[e], n = offsets[e + 1] - b;
                if (n == 0) continue;
                decode_row(L->down_w + ((size_t)e * H + d) * down_row, L->fmt, F, tile, wrow.data());
                float bias = L->arch == ARCH_GPT_OSS ? bf16r(L->down_b[(size_t)e * H + d]) : 0.0f;
                for (uint32_t i = 0; i < n; i++) {
                    uint32_t route = route_of_row[b + i];
                    float v = dot(wrow.data(), act.data() + (size_t)route * F, F) + bias;
                    y[(size_t)route * H + d] = orc_f32_to_bf16(v);   // projections.metal:179,343
                }
            }
    }
    if (trace && trace->act) std::memcpy(trace->act, act.data(), sizeof(float) * act.size());
    if (trace && trace->y) std::memcpy(trace->y, y.data(), sizeof(uint16_t) * y.size());

    // ---- shared expert (nemotron) ---------------------------------------------------------------
    std::vector<uint16_t> shared;   // bf16 [T, H]
    if (L->arch == ARCH_NEMOTRON && L->shared_ffn > 0) {
        const int S = L->shared_ffn;
        const size_t su_row = row_bytes(L->fmt, H), sd_row = row_bytes(L->fmt, S);
        std::vector<float> mid((size_t)T * S);
        shared.resize((size_t)T * H);
#pragma omp parallel
        {
            std::vector<float> wrow(std::max(H, S));
#pragma omp for schedule(static)
            for (int c = 0; c < S; c++) {
                decode_row(L->shared_up_w + (size_t)c * su_row, L->fmt, H, tile, wrow.data());
                for (int t = 0; t < T; t++) {
                    // dense up stored as bf16 (weights.metal:28-33); relu^2 either on load in f32
                    // (single token, vector.metal:185-190) or in place as bf16 (nemotron.metal:214-220),
                    // then to half for the dense tiles.
                    float v = std::max(bf16r(dot(wrow.data(), xin.data() + (size_t)t * H, H)), 0.0f);
                    float a = v * v;
                    if (tile) a = f16r(bf16r(a));
                    mid[(size_t)t * S + c] = a;
                }
            }
#pragma omp for schedule(static)
            for (int d = 0; d < H; d++) {
                decode_row(L->shared_down_w + (size_t)d * sd_row, L->fmt, S, tile, wrow.data());
                for (int t = 0; t < T; t++)
                    shared[(size_t)t * H + d] =
                        orc_f32_to_bf16(dot(wrow.data(), mid.data() + (size_t)t * S, S));
            }
        }
    }

    // ---- combine ------------------------------------------------------------------------------
#pragma omp parallel for schedule(static)
    for (int t = 0; t < T; t++)
        for (int d = 0; d < H; d++) {
            size_t i = (size_t)t * H + d;
            float res = orc_bf16_to_f32(residual[i]);
            if (L->arch == ARCH_GPT_OSS) {
                // moe_sum (routing.metal:154-168): the expert sum is rounded to bf16 first.
                float s = 0.f;
                for (int r = 0; r < K; r++)
                    s = fmaf(orc_bf16_to_f32(y[((size_t)t * K + r) * H + d]), probs[(size_t)t * K + r], s);
                residual[i] = orc_f32_to_bf16(res + bf16r(s));
            } else {
                // moe_add (nemotron.metal:222-236); for rows > 1 the shared expert was added to the
                // residual beforehand as a bf16 add (compute/nemotron.rs:316, elementwise.metal:62-66).
                float s = 0.f;
                if (!shared.empty()) {
                    if (tile) res = bf16r(res + orc_bf16_to_f32(shared[i]));
                    else s = orc_bf16_to_f32(shared[i]);
                }
                for (int r = 0; r < K; r++)
                    s = fmaf(orc_bf16_to_f32(y[((size_t)t * K + r) * H + d]), probs[(size_t)t * K + r], s);
                residual[i] = orc_f32_to_bf16(res + s);
            }
        }
    return 0;
}

// The dense products either side of the MoE path (DenseMatrix::apply, src/weights/compute/matrix.rs:130-278),
// composed as the reference composes them:
//   kind 0  projection: out[t][c] = bf16(up_w[c] . x[t])                       (weights.metal:28-33 store)
//   kind 1  relu^2 FFN, Nemotron's always-on expert (compute/nemotron.rs:302-315 for rows > 1,
//           :460-509 for one token): up stored as bf16, relu^2 on load in f32 (one token,
//           vector.metal:185-190) or in place as bf16 then to half (tiles, nemotron.metal:214-220), down
//   kind 2  gated FFN (feed_forward.rs:97-104): gate and up stored as bf16, gate kernel
//           y = bf16(bf16(silu(g)) * u) (elementwise.metal:70-87), down
// `tile` selects the operand conversions of the tiled kernels (inputs and decoded weights as half) over
// the exact ones of the one-token kernels. out is bf16 [T][F] for kind 0, [T][H] otherwise.
void orc_dense_forward(int kind, int fmt, int H, int F, const uint8_t* up_w, const uint8_t* gate_w,
                       const uint8_t* down_w, const uint16_t* x, int T, int tile_mode, uint16_t* out) {
    const bool tile = tile_mode != 0;
    auto dot = dotd;
    std::vector<float> xin((size_t)T * H);
    for (size_t i = 0; i < (size_t)T * H; i++) {
        float v = orc_bf16_to_f32(x[i]);
        xin[i] = tile ? f16r(v) : v;
    }
    const size_t up_row = row_bytes(fmt, H), down_row = row_bytes(fmt, F);
    std::vector<float> mid(kind == 0 ? 0 : (size_t)T * F);
#pragma omp parallel
    {
        std::vector<float> wrow(std::max(H, F)), wrow2(std::max(H, F));
#pragma omp for schedule(static)
        for (int c = 0; c < F; c++) {
            decode_row(up_w + (size_t)c * up_row, fmt, H, tile, wrow.data());
            if (kind == 2) decode_row(gate_w + (size_t)c * up_row, fmt, H, tile, wrow2.data());
            for (int t = 0; t < T; t++) {
                const float* xr = xin.data() + (size_t)t * H;
                float up = dot(wrow.data(), xr, H);
                if (kind == 0) {
                    out[(size_t)t * F + c] = orc_f32_to_bf16(up);
                } else if (kind == 1) {
                    float v = std::max(bf16r(up), 0.0f);
                    float a = v * v;
                    if (bf16r(up) != bf16r(up)) a = bf16r(up);
                    if (tile) a = f16r(bf16r(a));
                    mid[(size_t)t * F + c] = a;
                } else {
                    float a = silu_gate_bf16(bf16r(dot(wrow2.data(), xr, H)), bf16r(up));
                    mid[(size_t)t * F + c] = tile ? f16r(a) : a;
                }
            }
        }
        if (kind != 0) {
#pragma omp for schedule(static)
            for (int d = 0; d < H; d++) {
                decode_row(down_w + (size_t)d * down_row, fmt, F, tile, wrow.data());
                for (int t = 0; t < T; t++)
                    out[(size_t)t * H + d] = orc_f32_to_bf16(dot(wrow.data(), mid.data() + (size_t)t * F, F));
            }
        }
    }
}

int orc_num_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
void orc_set_num_threads(int n) {
#ifdef _OPENMP
    omp_set_num_threads(n);
#else
    (void)n;
#endif
}

}  // extern "C"
