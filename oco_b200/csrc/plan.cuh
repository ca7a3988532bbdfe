// Token-to-expert permutation, tile schedule, row gather and the weighted combine.
#pragma once
#include "common.cuh"

namespace oco {

// Stable counting sort of route indices by expert id, by one CTA of 1024 threads.
//
// Produces what the reference's route plan encodes (route_plan_tiled, shaders/experts/routing.metal:4-39;
// route_plan_n, shaders/nemotron.metal:238-273) in flat form:
//   offsets[e]       exclusive scan of per-expert route counts (offsets[E] = R)
//   row_of_route[i]  offsets[ids[i]] + number of earlier routes with the same expert
//   route_of_row[r]  the inverse: the concatenated per-expert ascending route lists
//   tiles            (expert, first row within the expert) per `tile_rows` rows, experts ascending
// The reference scans all routes serially in one thread per expert; here each pass ranks 1024
// routes with warp match/ballot and a per-expert scan over the 32 warp counts. No atomics, so the
// result does not depend on scheduling.
__global__ void __launch_bounds__(1024) route_plan_kernel(const uint32_t* __restrict__ ids, uint32_t R, uint32_t E,
                                                          uint32_t tile_rows, uint32_t* __restrict__ offsets,
                                                          uint32_t* __restrict__ row_of_route,
                                                          uint32_t* __restrict__ route_of_row,
                                                          uint32_t* __restrict__ tiles,
                                                          uint32_t* __restrict__ tile_count) {
    __shared__ uint32_t running[kMaxExperts];
    __shared__ uint32_t warp_cnt[32][kMaxExperts];
    __shared__ uint32_t soff[kMaxExperts + 1];
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid < kMaxExperts) running[tid] = 0;
    __syncthreads();
    for (uint32_t base = 0; base < R; base += 1024) {
        for (uint32_t j = lane; j < E; j += 32) warp_cnt[warp][j] = 0;
        __syncwarp();
        uint32_t i = base + tid;
        uint32_t e = i < R ? ids[i] : 0xffffffffu;
        uint32_t peers = __match_any_sync(0xffffffffu, e);
        uint32_t rank = __popc(peers & ((1u << lane) - 1u));
        if (i < R && e < E && rank == 0) warp_cnt[warp][e] = __popc(peers);
        __syncthreads();
        if (tid < E) {
            uint32_t acc = running[tid];
            for (uint32_t w = 0; w < 32; w++) {
                uint32_t c = warp_cnt[w][tid];
                warp_cnt[w][tid] = acc;
                acc += c;
            }
            running[tid] = acc;
        }
        __syncthreads();
        if (i < R && e < E) row_of_route[i] = warp_cnt[warp][e] + rank;  // position within the expert
        __syncthreads();
    }
    if (tid == 0) {
        uint32_t acc = 0, nt = 0;
        for (uint32_t e = 0; e < E; e++) {
            soff[e] = acc;
            uint32_t c = running[e];
            for (uint32_t b = 0; b < c; b += tile_rows) {
                tiles[2 * nt] = e;
                tiles[2 * nt + 1] = b;
                nt++;
            }
            acc += c;
        }
        soff[E] = acc;
        *tile_count = nt;
    }
    __syncthreads();
    if (tid <= E) offsets[tid] = soff[tid];
    for (uint32_t i = tid; i < R; i += 1024) {
        uint32_t e = ids[i];
        if (e < E) {
            uint32_t row = soff[e] + row_of_route[i];
            row_of_route[i] = row;
            route_of_row[row] = i;
        }
    }
}

// Gathers token rows into expert-sorted order, converting bf16 to the tiles' half operand and
// laying each block out in the tiles' operand order (see operand_pos in gemm.cuh): `half_span` is
// the distance between the two elements a code byte holds (16 for MXFP4 / Q4_0, 32 for Q4_K).
// The reference gathers inside its tiles (shaders/experts/projections.metal:208-233).
// One CTA per sorted row; each thread emits one half2 = (x[k], x[k + half_span]).
__global__ void __launch_bounds__(256) permute_rows_kernel(const uint16_t* __restrict__ x,
                                                           const uint32_t* __restrict__ route_of_row, int K,
                                                           int H, int half_span, uint16_t* __restrict__ xs) {
    uint32_t row = blockIdx.x;
    uint32_t token = route_of_row ? route_of_row[row] / (uint32_t)K : row;  // null: rows keep token order
    const uint16_t* src = x + (size_t)token * H;
    uint32_t* dst = reinterpret_cast<uint32_t*>(xs + (size_t)row * H);
    for (int i = threadIdx.x; i < H / 2; i += 256) {
        int blk = i / half_span, j = i % half_span;           // pair i of the row: block, byte index
        int k = blk * 2 * half_span + j;
        __half2 h = __floats2half2_rn(__uint_as_float((uint32_t)src[k] << 16),
                                      __uint_as_float((uint32_t)src[k + half_span] << 16));
        dst[i] = *reinterpret_cast<uint32_t*>(&h);
    }
}

// Residual add and RMS normalisation in one pass (reference add_norm and norm,
// shaders/elementwise.metal:5-30,32-60; call sites src/weights/compute.rs:86-117,
// src/weights/gpt_oss.rs:122): hidden += delta (bf16 add; delta null = plain norm), then
// out = hidden * rsqrt(mean(hidden^2) + eps) * w, rounded as the model family asks: full_layer
// scales the f32 value and rounds once (gpt-oss); otherwise the normalised value and the weight
// are rounded to bf16 before the product (Qwen). The reference leaves the order of its simd_sum
// open; the order fixed here (per thread i = tid, tid + 256, ... with FMA, xor butterfly inside
// the warp, then the same butterfly over the eight warp sums) is carried by the CPU checker too.
// One CTA of 256 threads per row.
__global__ void __launch_bounds__(256) add_norm_kernel(uint16_t* __restrict__ hidden, const uint16_t* __restrict__ delta,
                                                       const float* __restrict__ w, uint16_t* __restrict__ out, int n,
                                                       float eps, int full_layer) {
    __shared__ float warp_sum[8];
    __shared__ float inv_s;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint16_t* row = hidden + (size_t)blockIdx.x * n;
    const uint16_t* drow = delta ? delta + (size_t)blockIdx.x * n : nullptr;
    float s = 0.f;
    for (int i = tid; i < n; i += 256) {
        float v = bf16_bits_to_f32(row[i]);
        if (drow) {
            v = bf16_round(__fadd_rn(v, bf16_bits_to_f32(drow[i])));
            row[i] = f32_to_bf16_bits(v);
        }
        s = __fmaf_rn(v, v, s);
    }
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, d));
    if (lane == 0) warp_sum[warp] = s;
    __syncthreads();
    if (warp == 0) {
        float t = lane < 8 ? warp_sum[lane] : 0.f;
#pragma unroll
        for (int d = 16; d >= 1; d >>= 1) t = __fadd_rn(t, __shfl_xor_sync(0xffffffffu, t, d));
        if (lane == 0) inv_s = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(t, (float)n), eps)));
    }
    __syncthreads();
    const float inv = inv_s;
    uint16_t* orow = out + (size_t)blockIdx.x * n;
    for (int i = tid; i < n; i += 256) {
        const float normalized = __fmul_rn(bf16_bits_to_f32(row[i]), inv);
        const float v = full_layer ? __fmul_rn(normalized, w[i]) : __fmul_rn(bf16_round(normalized), bf16_round(w[i]));
        orow[i] = f32_to_bf16_bits(v);
    }
}

// gpt-oss rounds every router weight to bf16 when it is used (routing.metal:108-109). The rounded
// copy is made once per bound weight set so the per-token kernels read plain f32.
__global__ void __launch_bounds__(256) round_router_kernel(const float* __restrict__ w, float* __restrict__ out, size_t n) {
    size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (i < n) out[i] = bf16_round(w[i]);
}

// Weighted combine onto the residual.
//   round_sum = 1: moe_sum (routing.metal:154-168): s = sum_r y_r * p_r; out = bf16(res + bf16(s))
//   round_sum = 0: moe_add (nemotron.metal:222-236): s = [shared] + sum_r fma(y_r, p_r); out = bf16(res + s)
//   shared_mode 0: none; 1: shared joins the f32 sum (single token); 2: shared is added to the
//   residual first as a bf16 add (tiled path, elementwise.metal:62-66 via compute/nemotron.rs:316).
__global__ void __launch_bounds__(256) moe_combine_kernel(const uint16_t* __restrict__ y,
                                                          const float* __restrict__ probs,
                                                          uint16_t* __restrict__ out,
                                                          const uint16_t* __restrict__ shared, int H, int T, int K,
                                                          int round_sum, int shared_mode,
                                                          const uint32_t* __restrict__ status) {
    size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
    size_t pairs = (size_t)T * H / 2;
    if (i >= pairs) return;
    // a step during which a bounded wait gave up leaves the residual rows as they were
    if (status && *reinterpret_cast<const volatile uint32_t*>(status) != 0u) return;
    int t = (int)(i / (H / 2)), d = (int)(i % (H / 2)) * 2;
    float s0 = 0.f, s1 = 0.f;
    uint32_t resw = *reinterpret_cast<const uint32_t*>(out + (size_t)t * H + d);
    float r0 = __uint_as_float(resw << 16), r1 = __uint_as_float(resw & 0xffff0000u);
    if (shared_mode) {
        uint32_t sw = *reinterpret_cast<const uint32_t*>(shared + (size_t)t * H + d);
        float h0 = __uint_as_float(sw << 16), h1 = __uint_as_float(sw & 0xffff0000u);
        if (shared_mode == 1) { s0 = h0; s1 = h1; }
        else { r0 = bf16_round(__fadd_rn(r0, h0)); r1 = bf16_round(__fadd_rn(r1, h1)); }
    }
    for (int r = 0; r < K; r++) {
        uint32_t yw = *reinterpret_cast<const uint32_t*>(y + ((size_t)t * K + r) * H + d);
        float p = probs[(size_t)t * K + r];
        s0 = __fmaf_rn(__uint_as_float(yw << 16), p, s0);
        s1 = __fmaf_rn(__uint_as_float(yw & 0xffff0000u), p, s1);
    }
    if (round_sum) { s0 = bf16_round(s0); s1 = bf16_round(s1); }
    uint32_t o = (uint32_t)f32_to_bf16_bits(__fadd_rn(r0, s0)) | ((uint32_t)f32_to_bf16_bits(__fadd_rn(r1, s1)) << 16);
    *reinterpret_cast<uint32_t*>(out + (size_t)t * H + d) = o;
}

// The bounded wait, run on a barrier that nobody arrives at: one warp waits `limit` clock cycles, gives
// up, sets the status word and returns normally. Lets a host test see the whole give-up path
// (status word -> oco_moe_poll -> OCO_DEVICE_TIMEOUT) without any fault on the device.
__global__ void __launch_bounds__(32) wait_timeout_kernel(uint32_t* status, long long limit) {
    __shared__ __align__(8) unsigned long long bar_storage;
    __shared__ volatile uint32_t give_up;
    const uint32_t bar = smem_u32(&bar_storage);
    if (threadIdx.x == 0) {
        give_up = 0u;
        mbar_init(bar, 1);
        fence_barrier_init();
    }
    __syncwarp();
    if (threadIdx.x == 0) mbar_wait_for(bar, 0u, &give_up, status, limit);
    __syncwarp();
}

}  // namespace oco
