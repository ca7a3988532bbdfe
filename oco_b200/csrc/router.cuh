// Router: logits in the canonical summation order, top-k selection and combination weights.
//
// Canonical order (shared with the host checker so expert ids agree bit for bit): lane l of a
// warp owns k = 4*l + 128*i, keeps four FMA chains (one per vector component), combines them as
// (x+y)+(z+w), and the 32 lane sums are reduced by an xor butterfly 16,8,4,2,1. This is the lane
// mapping of the reference's router kernels (shaders/experts/routing.metal:105-112,136-143;
// shaders/nemotron.metal:156-162) with its unspecified `simd_sum` order fixed.
#pragma once
#include "common.cuh"

namespace oco {

__device__ __forceinline__ float warp_butterfly_sum(float s) {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, off));
    return s;
}
__device__ __forceinline__ float warp_max(float s) {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) s = fmaxf(s, __shfl_xor_sync(0xffffffffu, s, off));
    return s;
}
__device__ __forceinline__ uint32_t warp_min_u32(uint32_t s) {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) s = min(s, __shfl_xor_sync(0xffffffffu, s, off));
    return s;
}
__device__ __forceinline__ bool warp_any(bool p) { return __any_sync(0xffffffffu, p) != 0; }

// One logit by one warp. x: bf16 row (global or shared), w: f32 row (global or shared).
// RoundW rounds each weight to bf16 first (gpt-oss, routing.metal:108-109).
template <bool RoundW>
__device__ __forceinline__ float canonical_logit(const uint16_t* x, const float* w, int n, int lane) {
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
    for (int k = lane * 4; k < n; k += 128) {
        uint2 xv = *reinterpret_cast<const uint2*>(x + k);
        float4 wv = *reinterpret_cast<const float4*>(w + k);
        if (RoundW) {
            wv.x = bf16_round(wv.x); wv.y = bf16_round(wv.y); wv.z = bf16_round(wv.z); wv.w = bf16_round(wv.w);
        }
        a0 = __fmaf_rn(__uint_as_float(xv.x << 16), wv.x, a0);
        a1 = __fmaf_rn(__uint_as_float(xv.x & 0xffff0000u), wv.y, a1);
        a2 = __fmaf_rn(__uint_as_float(xv.y << 16), wv.z, a2);
        a3 = __fmaf_rn(__uint_as_float(xv.y & 0xffff0000u), wv.w, a3);
    }
    return warp_butterfly_sum(__fadd_rn(__fadd_rn(a0, a1), __fadd_rn(a2, a3)));
}

// The same logit with every load issued before the first FMA (n <= 128 * ITERS): a single token
// has no other work to hide the memory latency of a load-then-FMA loop behind.
template <bool RoundW, int ITERS>
__device__ __forceinline__ float canonical_logit_prefetch(const uint16_t* x, const float* w, int n, int lane) {
    uint2 xv[ITERS];
    float4 wv[ITERS];
#pragma unroll
    for (int i = 0; i < ITERS; i++) {
        const int k = lane * 4 + 128 * i;
        if (k < n) {
            xv[i] = *reinterpret_cast<const uint2*>(x + k);
            wv[i] = *reinterpret_cast<const float4*>(w + k);
        } else {
            xv[i] = make_uint2(0u, 0u);
            wv[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
    for (int i = 0; i < ITERS; i++) {
        const int k = lane * 4 + 128 * i;
        if (k < n) {
            float4 v = wv[i];
            if (RoundW) { v.x = bf16_round(v.x); v.y = bf16_round(v.y); v.z = bf16_round(v.z); v.w = bf16_round(v.w); }
            a0 = __fmaf_rn(__uint_as_float(xv[i].x << 16), v.x, a0);
            a1 = __fmaf_rn(__uint_as_float(xv[i].x & 0xffff0000u), v.y, a1);
            a2 = __fmaf_rn(__uint_as_float(xv[i].y << 16), v.z, a2);
            a3 = __fmaf_rn(__uint_as_float(xv[i].y & 0xffff0000u), v.w, a3);
        }
    }
    return warp_butterfly_sum(__fadd_rn(__fadd_rn(a0, a1), __fadd_rn(a2, a3)));
}

// Top-k selection by one warp over logits distributed as logit[j] = expert (lane + 32*j).
// Every lane returns the same ids / probs.
//   GPT_OSS  (routing.metal:71-94): ties to the lowest index; winners rounded to bf16; softmax over
//            the winners; probabilities rounded to bf16; any non-finite logit makes all probs NaN.
//   NEMOTRON (nemotron.metal:167-211): score = sigmoid(logit); selection on score + bias; weights
//            are the unbiased scores, optionally normalised (floor 2^-14) and scaled.
//   QWEN     top-k of the logits, softmax over the winners (= softmax over all, renormalised).
template <int ARCH>
__device__ __forceinline__ void select_experts(const float (&logit)[4], int E, int K, const float* sel_bias,
                                               int normalize, float scale, int lane,
                                               uint32_t (&ids)[kMaxTopK], float (&probs)[kMaxTopK]) {
    const float ninf = __uint_as_float(0xff800000u);
    float v[4], score[4];
    bool invalid = false;
    uint32_t avail = 0;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        int e = lane + 32 * j;
        bool valid = e < E;
        float l = valid ? logit[j] : 0.0f;
        bool fin = !nonfinite(l);
        invalid = invalid || (valid && !fin);
        if (valid) avail |= 1u << j;
        if (ARCH == OCO_ARCH_NEMOTRON) {
            score[j] = __fdiv_rn(1.0f, __fadd_rn(1.0f, exp_det(-l)));
            v[j] = valid ? __fadd_rn(score[j], sel_bias[e]) : ninf;
        } else {
            score[j] = 0.f;
            v[j] = (valid && fin) ? l : ninf;
        }
    }
    invalid = warp_any(invalid);
    float chosen[kMaxTopK];
    float total = 0.f;
#pragma unroll
    for (int r = 0; r < kMaxTopK; r++) {
        ids[r] = 0; probs[r] = 0.f; chosen[r] = 0.f;
        if (r >= K) continue;
        if (ARCH == OCO_ARCH_NEMOTRON) {
            float bv = ninf;
#pragma unroll
            for (int j = 0; j < 4; j++)
                if (v[j] > bv) bv = v[j];
            float peak = warp_max(bv);
            uint32_t cand = 0xffffffffu;
#pragma unroll
            for (int j = 3; j >= 0; j--)
                if (((avail >> j) & 1u) && v[j] == peak) cand = (uint32_t)(lane + 32 * j);
            uint32_t id = warp_min_u32(cand);
            if (id == 0xffffffffu) id = 0;
            ids[r] = id;
            float mine = 0.f;
#pragma unroll
            for (int j = 0; j < 4; j++)
                if ((int)(id >> 5) == j) { mine = score[j]; if ((int)(id & 31u) == lane) v[j] = ninf; }
            float w = __shfl_sync(0xffffffffu, mine, (int)(id & 31u));
            chosen[r] = w;
            total = __fadd_rn(total, w);
        } else {
            float bv = ninf;
#pragma unroll
            for (int j = 0; j < 4; j++)
                if (((avail >> j) & 1u) && v[j] > bv) bv = v[j];
            float peak = warp_max(bv);
            uint32_t cand = 0xffffffffu;
#pragma unroll
            for (int j = 3; j >= 0; j--)
                if (((avail >> j) & 1u) && v[j] == peak) cand = (uint32_t)(lane + 32 * j);
            uint32_t id = warp_min_u32(cand);
            if (id == 0xffffffffu) id = 0;
            ids[r] = id;
            chosen[r] = ARCH == OCO_ARCH_GPT_OSS ? bf16_round(peak) : peak;
            if ((int)(id & 31u) == lane) avail &= ~(1u << (id >> 5));
        }
    }
    if (ARCH == OCO_ARCH_NEMOTRON) {
        float divisor = normalize ? fmaxf(total, 6.103515625e-5f) : 1.0f;
#pragma unroll
        for (int r = 0; r < kMaxTopK; r++)
            if (r < K) probs[r] = invalid ? qnan() : __fmul_rn(__fdiv_rn(chosen[r], divisor), scale);
    } else {
#pragma unroll
        for (int r = 0; r < kMaxTopK; r++)
            if (r < K) invalid = invalid || nonfinite(chosen[r]);
        float sum = 0.f;
        float ex[kMaxTopK];
#pragma unroll
        for (int r = 0; r < kMaxTopK; r++) {
            ex[r] = 0.f;
            if (r < K && !invalid) {
                ex[r] = exp_det(__fadd_rn(chosen[r], -chosen[0]));
                sum = __fadd_rn(sum, ex[r]);
            }
        }
#pragma unroll
        for (int r = 0; r < kMaxTopK; r++)
            if (r < K) {
                float p = invalid ? qnan() : __fdiv_rn(ex[r], sum);
                probs[r] = (ARCH == OCO_ARCH_GPT_OSS && !invalid) ? bf16_round(p) : p;
            }
    }
}

// Reads the E logits of one token into the distributed form select_experts takes.
__device__ __forceinline__ void load_logits(const float* logits, int E, int lane, float (&v)[4]) {
#pragma unroll
    for (int j = 0; j < 4; j++) {
        int e = lane + 32 * j;
        v[j] = e < E ? logits[e] : 0.0f;
    }
}

// ---- kernels ------------------------------------------------------------------------------------

// A few tokens: one warp per (expert, token), operands straight from global memory
// (reference router_logits, routing.metal:131-146). grid (ceil(E/8), T), 256 threads.
template <int ARCH>
__global__ void __launch_bounds__(256) router_logits_small_kernel(const uint16_t* __restrict__ x,
                                                                  const float* __restrict__ w,
                                                                  const float* __restrict__ bias,
                                                                  float* __restrict__ logits, int H, int E) {
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int e = blockIdx.x * 8 + warp, t = blockIdx.y;
    if (e >= E) return;
    float s = H <= 128 * 24
                  ? canonical_logit_prefetch<ARCH == OCO_ARCH_GPT_OSS, 24>(x + (size_t)t * H, w + (size_t)e * H, H, lane)
                  : canonical_logit<ARCH == OCO_ARCH_GPT_OSS>(x + (size_t)t * H, w + (size_t)e * H, H, lane);
    if (ARCH == OCO_ARCH_GPT_OSS) s = __fadd_rn(s, bf16_round(bias[e]));
    if (lane == 0) logits[(size_t)t * E + e] = s;
}

// Selection for tokens whose logits are already in memory. grid T, 32 threads.
template <int ARCH>
__global__ void __launch_bounds__(32) router_select_kernel(const float* __restrict__ logits,
                                                           const float* __restrict__ sel_bias, int E, int K,
                                                           int normalize, float scale, uint32_t* __restrict__ ids,
                                                           float* __restrict__ probs) {
    pdl_launch_dependents();   // the next kernel of the step may be set up beside this one
    pdl_wait();                // the kernel before has completed and its writes are visible
    int t = blockIdx.x, lane = threadIdx.x;
    float v[4];
    load_logits(logits + (size_t)t * E, E, lane, v);
    uint32_t id[kMaxTopK];
    float p[kMaxTopK];
    select_experts<ARCH>(v, E, K, sel_bias, normalize, scale, lane, id, p);
#pragma unroll
    for (int r = 0; r < kMaxTopK; r++)
        if (r < K && lane == r) { ids[(size_t)t * K + r] = id[r]; probs[(size_t)t * K + r] = p[r]; }
}

// Many tokens: eight tokens per CTA (one per warp) share each router row through shared memory,
// then each warp selects for its token (reference router, routing.metal:96-128;
// router_sigmoid, nemotron.metal:140-212). Dynamic shared memory: 8*H bf16 + H f32.
template <int ARCH>
__global__ void __launch_bounds__(256) router_batched_kernel(const uint16_t* __restrict__ x,
                                                             const float* __restrict__ w,
                                                             const float* __restrict__ bias, int T, int H, int E,
                                                             int K, int normalize, float scale,
                                                             float* __restrict__ logits, uint32_t* __restrict__ ids,
                                                             float* __restrict__ probs) {
    pdl_launch_dependents();   // the next kernel of the step may be set up beside this one
    pdl_wait();                // the kernel before has completed and its writes are visible
    extern __shared__ __align__(16) unsigned char smem[];
    float* ws = reinterpret_cast<float*>(smem);                      // [H]
    uint16_t* xs = reinterpret_cast<uint16_t*>(smem + (size_t)H * 4);  // [8][H]
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int t0 = blockIdx.x * 8;
    int t = t0 + warp;
    // Stage the CTA's eight token rows (8-byte chunks; H is a multiple of 4).
    int rows = min(8, T - t0);
    for (int i = threadIdx.x; i < rows * (H / 4); i += 256) {
        int r = i / (H / 4), c = i % (H / 4);
        reinterpret_cast<uint2*>(xs + (size_t)r * H)[c] = reinterpret_cast<const uint2*>(x + (size_t)(t0 + r) * H)[c];
    }
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    for (int e = 0; e < E; e++) {
        __syncthreads();
        for (int i = threadIdx.x; i < H / 4; i += 256) {
            float4 wv = reinterpret_cast<const float4*>(w + (size_t)e * H)[i];
            if (ARCH == OCO_ARCH_GPT_OSS) {
                wv.x = bf16_round(wv.x); wv.y = bf16_round(wv.y); wv.z = bf16_round(wv.z); wv.w = bf16_round(wv.w);
            }
            reinterpret_cast<float4*>(ws)[i] = wv;
        }
        __syncthreads();
        if (t < T) {
            float s = canonical_logit<false>(xs + (size_t)warp * H, ws, H, lane);
            if (ARCH == OCO_ARCH_GPT_OSS) s = __fadd_rn(s, bf16_round(bias[e]));
#pragma unroll
            for (int j = 0; j < 4; j++)
                if ((e >> 5) == j && (e & 31) == lane) v[j] = s;
        }
    }
    if (t >= T) return;
    if (logits) {
#pragma unroll
        for (int j = 0; j < 4; j++)
            if (lane + 32 * j < E) logits[(size_t)t * E + lane + 32 * j] = v[j];
    }
    uint32_t id[kMaxTopK];
    float p[kMaxTopK];
    select_experts<ARCH>(v, E, K, ARCH == OCO_ARCH_NEMOTRON ? bias : nullptr, normalize, scale, lane, id, p);
#pragma unroll
    for (int r = 0; r < kMaxTopK; r++)
        if (r < K && lane == r) { ids[(size_t)t * K + r] = id[r]; probs[(size_t)t * K + r] = p[r]; }
}

// Many tokens, hidden <= 128 * ITERS: one token per warp with its row held in registers as f32;
// the router rows stream through a shared-memory ring filled with cp.async (three stages of two
// rows), one __syncthreads per pair of experts. `w` holds the weights as they enter the FMAs (already rounded for
// gpt-oss). Same canonical order as canonical_logit. Dynamic shared memory: 6 * H floats.
// grid (ceil(T / (8 * TOK)), splits): with one split a CTA goes through all experts and selects; with
// more (few tokens, so that the grid still fills the GPU) CTA y takes experts [y * E / splits,
// (y + 1) * E / splits), writes their logits and leaves the selection to router_select_kernel.
// TOK tokens per warp share every router-row load. Measured: two tokens per warp (250 registers, one
// CTA per SM) lose more to latency than they save in shared-memory bandwidth (gpt-oss-20b prefill
// 71 us against 49 us), so the launches use TOK = 1.
template <int ARCH, int ITERS, int TOK>
__global__ void __launch_bounds__(256, TOK == 1 ? 2 : 1) router_stream_kernel(const uint16_t* __restrict__ x,
                                                               const float* __restrict__ w,
                                                               const float* __restrict__ bias, int T, int H, int E, int K,
                                                               int normalize, float scale, float* __restrict__ logits,
                                                               uint32_t* __restrict__ ids, float* __restrict__ probs) {
    pdl_launch_dependents();   // the next kernel of the step may be set up beside this one
    pdl_wait();                // the kernel before has completed and its writes are visible
    extern __shared__ __align__(16) unsigned char smem[];
    float* ring = reinterpret_cast<float*>(smem);                  // [3][2][H]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t0 = (blockIdx.x * 8 + warp) * TOK;
    float xr[TOK][ITERS][4];
#pragma unroll
    for (int j = 0; j < TOK; j++)
#pragma unroll
        for (int i = 0; i < ITERS; i++) {
            const int k = lane * 4 + 128 * i;
            if (t0 + j < T && k < H) {
                uint2 xv = *reinterpret_cast<const uint2*>(x + (size_t)(t0 + j) * H + k);
                xr[j][i][0] = __uint_as_float(xv.x << 16); xr[j][i][1] = __uint_as_float(xv.x & 0xffff0000u);
                xr[j][i][2] = __uint_as_float(xv.y << 16); xr[j][i][3] = __uint_as_float(xv.y & 0xffff0000u);
            } else {
                xr[j][i][0] = xr[j][i][1] = xr[j][i][2] = xr[j][i][3] = 0.f;
            }
        }
    const int chunks = H / 4;                                       // 16-byte chunks per router row
    const int e_begin = (int)(((long long)blockIdx.y * E) / gridDim.y), e_end = (int)(((long long)(blockIdx.y + 1) * E) / gridDim.y);
    // Two router rows per step: a stage of the ring holds rows e, e + 1 (three stages), so that each
    // lane runs eight independent FMA chains per token between two barriers.
    auto issue = [&](int p) {                                       // pair p: rows e_begin + 2p, + 2p + 1
        const int e = e_begin + 2 * p;
        if (e < e_end) {
            const int nrows = min(2, e_end - e);
            const float* src = w + (size_t)e * H;
            const uint32_t dst = smem_u32(ring + (size_t)(p % 3) * 2 * H);
            for (int c = threadIdx.x; c < nrows * chunks; c += 256) cp_async16(dst + 16u * c, src + 4 * c);
        }
        cp_async_commit();
    };
    issue(0); issue(1);
    float v[TOK][4];
#pragma unroll
    for (int j = 0; j < TOK; j++) v[j][0] = v[j][1] = v[j][2] = v[j][3] = 0.f;
    const int pairs = (e_end - e_begin + 1) / 2;
    for (int p = 0; p < pairs; p++) {
        cp_async_wait<1>();
        __syncthreads();            // pair p has landed for everyone; pair p - 1 is no longer read
        issue(p + 2);               // into the stage pair p - 1 used
        const int e = e_begin + 2 * p;
        const bool two = e + 1 < e_end;
        const float* wr = ring + (size_t)(p % 3) * 2 * H;
        float a[TOK][4], c2[TOK][4];
#pragma unroll
        for (int j = 0; j < TOK; j++) {
            a[j][0] = a[j][1] = a[j][2] = a[j][3] = 0.f;
            c2[j][0] = c2[j][1] = c2[j][2] = c2[j][3] = 0.f;
        }
#pragma unroll
        for (int i = 0; i < ITERS; i++) {
            const int k = lane * 4 + 128 * i;
            if (k < H) {
                const float4 wv = *reinterpret_cast<const float4*>(wr + k);
                const float4 wu = *reinterpret_cast<const float4*>(wr + H + k);   // stale bytes when the pair is single: unused
#pragma unroll
                for (int j = 0; j < TOK; j++) {
                    a[j][0] = __fmaf_rn(xr[j][i][0], wv.x, a[j][0]);
                    a[j][1] = __fmaf_rn(xr[j][i][1], wv.y, a[j][1]);
                    a[j][2] = __fmaf_rn(xr[j][i][2], wv.z, a[j][2]);
                    a[j][3] = __fmaf_rn(xr[j][i][3], wv.w, a[j][3]);
                    c2[j][0] = __fmaf_rn(xr[j][i][0], wu.x, c2[j][0]);
                    c2[j][1] = __fmaf_rn(xr[j][i][1], wu.y, c2[j][1]);
                    c2[j][2] = __fmaf_rn(xr[j][i][2], wu.z, c2[j][2]);
                    c2[j][3] = __fmaf_rn(xr[j][i][3], wu.w, c2[j][3]);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < TOK; j++) {
            float s0 = warp_butterfly_sum(__fadd_rn(__fadd_rn(a[j][0], a[j][1]), __fadd_rn(a[j][2], a[j][3])));
            float s1 = warp_butterfly_sum(__fadd_rn(__fadd_rn(c2[j][0], c2[j][1]), __fadd_rn(c2[j][2], c2[j][3])));
            if (ARCH == OCO_ARCH_GPT_OSS) {
                s0 = __fadd_rn(s0, bf16_round(bias[e]));
                if (two) s1 = __fadd_rn(s1, bf16_round(bias[e + 1]));
            }
#pragma unroll
            for (int q = 0; q < 4; q++) {
                if ((e >> 5) == q && (e & 31) == lane) v[j][q] = s0;
                if (two && ((e + 1) >> 5) == q && ((e + 1) & 31) == lane) v[j][q] = s1;
            }
        }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int j = 0; j < TOK; j++) {
        const int t = t0 + j;
        if (t >= T) continue;
        if (logits) {
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const int e = lane + 32 * q;
                if (e >= e_begin && e < e_end) logits[(size_t)t * E + e] = v[j][q];
            }
        }
        if (gridDim.y > 1) continue;
        uint32_t id[kMaxTopK];
        float pr[kMaxTopK];
        select_experts<ARCH>(v[j], E, K, ARCH == OCO_ARCH_NEMOTRON ? bias : nullptr, normalize, scale, lane, id, pr);
#pragma unroll
        for (int r = 0; r < kMaxTopK; r++)
            if (r < K && lane == r) { ids[(size_t)t * K + r] = id[r]; probs[(size_t)t * K + r] = pr[r]; }
    }
}


// Many tokens, register-blocked: a warp takes FOUR tokens against FOUR experts at a time, so that
// every shared-memory load feeds four FMAs per lane instead of one (router_stream_kernel reads one
// router-row float4 per four FMAs and is bound by shared-memory bandwidth). The CTA's 32 token rows
// stay in shared memory as bf16 (2 * H bytes each); the router rows stream through a ring of three
// stages of 4 experts x 640 columns filled with cp.async. Lane l still owns columns 4 l + 128 i with
// its four FMA chains in ascending i, the chains are joined as (a0 + a1) + (a2 + a3) and the lanes by
// the same butterfly, so the logits are bit-identical to canonical_logit.
// grid (ceil(T / 32), splits) as router_stream_kernel; hidden <= 3072 and a multiple of 8.
// Dynamic shared memory: router_block_smem_bytes(H).
constexpr int kRouterBlockTokens = 32, kRouterBlockCols = 384, kRouterBlockStages = 3;
constexpr int kRouterBlockExperts = 8;                              // experts per ring stage: two warps share four tokens, four experts each
constexpr int kRouterBlockThreads = kRouterBlockTokens * 8 * (kRouterBlockExperts / 4);
__host__ __device__ inline size_t router_block_smem_bytes(int H) {
    return (size_t)kRouterBlockTokens * H * 2 + (size_t)kRouterBlockStages * kRouterBlockExperts * kRouterBlockCols * 4;
}

template <int ARCH>
__global__ void __launch_bounds__(kRouterBlockThreads, 1) router_block_kernel(const uint16_t* __restrict__ x, const float* __restrict__ w,
                                                              const float* __restrict__ bias, int T, int H, int E, int K,
                                                              int normalize, float scale, float* __restrict__ logits,
                                                              uint32_t* __restrict__ ids, float* __restrict__ probs) {
    pdl_launch_dependents();   // the next kernel of the step may be set up beside this one
    pdl_wait();                // the kernel before has completed and its writes are visible
    extern __shared__ __align__(16) unsigned char smem[];
    constexpr int KC = kRouterBlockCols, STEPS = KC / 128;
    uint16_t* xs = reinterpret_cast<uint16_t*>(smem);                                   // [32][H] bf16
    constexpr int EB = kRouterBlockExperts;
    float* ring = reinterpret_cast<float*>(smem + (size_t)kRouterBlockTokens * H * 2);  // [3][EB][KC]
    const int warp = (threadIdx.x >> 5) & 7, lane = threadIdx.x & 31;                   // token group of four
    const int esub = (threadIdx.x >> 8) * 4;                                            // this warp's four experts of a block
    const int t0 = blockIdx.x * kRouterBlockTokens;
    const int e_begin = (int)(((long long)blockIdx.y * E) / gridDim.y), e_end = (int)(((long long)(blockIdx.y + 1) * E) / gridDim.y);
    const int nblocks = (e_end - e_begin + EB - 1) / EB;    // expert blocks of this CTA
    const int nkc = (H + KC - 1) / KC;                      // column chunks of a router row
    const int steps = nblocks * nkc;

    // the token rows (rows past T are zero)
    {
        const int per_row = H / 8;                          // 16-byte pieces
        for (int c = threadIdx.x; c < kRouterBlockTokens * per_row; c += kRouterBlockThreads) {
            const int r = c / per_row, j = c - r * per_row;
            if (t0 + r < T) cp_async16(smem_u32(xs + (size_t)r * H + 8 * j), x + (size_t)(t0 + r) * H + 8 * j);
            else *reinterpret_cast<uint4*>(xs + (size_t)r * H + 8 * j) = make_uint4(0u, 0u, 0u, 0u);
        }
    }
    // copy role: a ring stage is EB rows of KC / 4 pieces; thread t takes pieces t and t + threads of that grid
    // (row = piece / (KC / 4), column piece % (KC / 4): fixed per thread, so no division in the loop)
    constexpr int kPiecesPerRow = KC / 4, kPiecesPerThread = (EB * kPiecesPerRow + kRouterBlockThreads - 1) / kRouterBlockThreads;
    int prow[kPiecesPerThread], pcol[kPiecesPerThread];
#pragma unroll
    for (int u = 0; u < kPiecesPerThread; u++) {
        const int c = threadIdx.x + u * kRouterBlockThreads;
        prow[u] = c / kPiecesPerRow;
        pcol[u] = c - prow[u] * kPiecesPerRow;
    }
    int is_eb = 0, is_kc = 0;                                  // the (expert block, column chunk) of the next step to issue
    auto issue = [&](int s) {                               // step s: expert block s / nkc, column chunk s % nkc
        if (s < steps) {
            const int e0 = e_begin + EB * is_eb, rows = min(EB, e_end - e0);
            const int cols = min(KC, H - is_kc * KC);
            const uint32_t dst = smem_u32(ring + (size_t)(s % kRouterBlockStages) * EB * KC);
            const float* src = w + (size_t)e0 * H + is_kc * KC;
#pragma unroll
            for (int u = 0; u < kPiecesPerThread; u++)
                if (prow[u] < rows && 4 * pcol[u] < cols)
                    cp_async16(dst + (uint32_t)(prow[u] * KC + 4 * pcol[u]) * 4u, src + (size_t)prow[u] * H + 4 * pcol[u]);
            if (++is_kc == nkc) { is_kc = 0; is_eb++; }
        }
        cp_async_commit();
    };
    issue(0); issue(1);                                     // the token rows travel in the first group
    float v[4][4];                                          // token j: logit of expert lane + 32 q
#pragma unroll
    for (int j = 0; j < 4; j++) v[j][0] = v[j][1] = v[j][2] = v[j][3] = 0.f;
    float acc[4][4][4];                                     // [token][expert][chain]
    const uint16_t* xw = xs + (size_t)(4 * warp) * H;
    int cur_eb = 0, cur_kc = 0;
    for (int s = 0; s < steps; s++) {
        cp_async_wait<1>();
        __syncthreads();                                    // step s has landed for everyone; step s - 1 is no longer read
        issue(s + 2);
        const int eb = cur_eb, kc = cur_kc;
        if (++cur_kc == nkc) { cur_kc = 0; cur_eb++; }
        const float* wr = ring + (size_t)(s % kRouterBlockStages) * EB * KC + (size_t)esub * KC;
        if (kc == 0) {
#pragma unroll
            for (int j = 0; j < 4; j++)
#pragma unroll
                for (int q = 0; q < 4; q++) acc[j][q][0] = acc[j][q][1] = acc[j][q][2] = acc[j][q][3] = 0.f;
        }
#pragma unroll
        for (int i = 0; i < STEPS; i++) {
            const int kl = lane * 4 + 128 * i, k = kc * KC + kl;
            if (k < H) {
                float xv[4][4];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const uint2 b = *reinterpret_cast<const uint2*>(xw + (size_t)j * H + k);
                    xv[j][0] = __uint_as_float(b.x << 16); xv[j][1] = __uint_as_float(b.x & 0xffff0000u);
                    xv[j][2] = __uint_as_float(b.y << 16); xv[j][3] = __uint_as_float(b.y & 0xffff0000u);
                }
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const float4 wv = *reinterpret_cast<const float4*>(wr + q * KC + kl);   // stale past the range's last expert: unused
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        acc[j][q][0] = __fmaf_rn(xv[j][0], wv.x, acc[j][q][0]);
                        acc[j][q][1] = __fmaf_rn(xv[j][1], wv.y, acc[j][q][1]);
                        acc[j][q][2] = __fmaf_rn(xv[j][2], wv.z, acc[j][q][2]);
                        acc[j][q][3] = __fmaf_rn(xv[j][3], wv.w, acc[j][q][3]);
                    }
                }
            }
        }
        if (kc == nkc - 1) {
            const int e0 = e_begin + EB * eb + esub;
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const int e = e0 + q;
                if (e < e_end) {                            // the same in every lane
                    const float be = ARCH == OCO_ARCH_GPT_OSS ? bf16_round(bias[e]) : 0.f;
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        float sum = warp_butterfly_sum(__fadd_rn(__fadd_rn(acc[j][q][0], acc[j][q][1]), __fadd_rn(acc[j][q][2], acc[j][q][3])));
                        if (ARCH == OCO_ARCH_GPT_OSS) sum = __fadd_rn(sum, be);
#pragma unroll
                        for (int u = 0; u < 4; u++)
                            if ((e >> 5) == u && (e & 31) == lane) v[j][u] = sum;
                    }
                }
            }
        }
    }
    cp_async_wait<0>();
    // each warp stores the logits of the experts it computed; router_select_kernel picks from the complete rows
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int t = t0 + 4 * warp + j;
        if (t >= T) continue;
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const int e = lane + 32 * q;
            if (e >= e_begin && e < e_end && (((e - e_begin) % EB) >> 2) * 4 == esub) logits[(size_t)t * E + e] = v[j][q];
        }
    }
}

}  // namespace oco
