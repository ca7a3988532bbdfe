// Token-to-expert permutation, tile schedule, row gather and the weighted combine.
#pragma once
#include "common.cuh"

namespace oco {

__device__ __forceinline__ uint32_t route_label(uint32_t i, uint32_t seg_len, uint32_t seg_stride);

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
                                                          uint32_t* __restrict__ tile_count, uint32_t seg_len = 0,
                                                          uint32_t seg_stride = 0) {
    pdl_launch_dependents();   // the next kernel of the step may be set up beside this one
    pdl_wait();                // the kernel before has completed and its writes are visible
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
            route_of_row[row] = route_label(i, seg_len, seg_stride);
        }
    }
}

// The same plan made by many CTAs, for route counts where one CTA's serial passes would dominate the
// step: chunk c = routes [1024 c, 1024 c + 1024).
//   route_count_kernel    per chunk: each route's rank among the chunk's routes of its expert (into
//                         row_of_route) and the chunk's count per expert (chunk_cnt[c][e])
//   route_scan_kernel     one CTA: per expert an exclusive scan of the chunk counts (in place), the
//                         expert offsets and the tile list
//   route_scatter_kernel  per chunk: row = offsets[e] + chunk_cnt[c][e] + rank
// Ranks come from warp match/ballot and fixed-order scans, so the plan equals route_plan_kernel's bit
// for bit and does not depend on scheduling.
//
// `seg_len`, `seg_stride` (both 0 = off): the value stored for route i in route_of_row is
// (i / seg_len) * seg_stride + i % seg_len, the route's row in a buffer that holds each source's
// seg_len routes at a stride of seg_stride rows (the expert-parallel window).
__device__ __forceinline__ uint32_t route_label(uint32_t i, uint32_t seg_len, uint32_t seg_stride) {
    return seg_len ? (i / seg_len) * seg_stride + i % seg_len : i;
}

__global__ void __launch_bounds__(1024) route_count_kernel(const uint32_t* __restrict__ ids, uint32_t R, uint32_t E,
                                                           uint32_t* __restrict__ row_of_route,
                                                           uint32_t* __restrict__ chunk_cnt) {
    pdl_launch_dependents();   // the next kernel of the step may be set up beside this one
    pdl_wait();                // the kernel before has completed and its writes are visible
    __shared__ uint32_t warp_cnt[32][kMaxExperts];
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (uint32_t j = lane; j < E; j += 32) warp_cnt[warp][j] = 0;
    __syncwarp();
    const uint32_t i = blockIdx.x * 1024u + tid;
    const uint32_t e = i < R ? ids[i] : 0xffffffffu;
    const uint32_t peers = __match_any_sync(0xffffffffu, e);
    const uint32_t rank = __popc(peers & ((1u << lane) - 1u));
    if (e < E && rank == 0) warp_cnt[warp][e] = __popc(peers);
    __syncthreads();
    if (tid < E) {
        uint32_t acc = 0;
        for (uint32_t w = 0; w < 32; w++) {
            const uint32_t c = warp_cnt[w][tid];
            warp_cnt[w][tid] = acc;
            acc += c;
        }
        chunk_cnt[(size_t)blockIdx.x * E + tid] = acc;
    }
    __syncthreads();
    if (e < E) row_of_route[i] = warp_cnt[warp][e] + rank;
}

__global__ void __launch_bounds__(1024) route_scan_kernel(uint32_t chunks, uint32_t E, uint32_t tile_rows,
                                                          uint32_t* __restrict__ chunk_cnt, uint32_t* __restrict__ offsets,
                                                          uint32_t* __restrict__ tiles, uint32_t* __restrict__ tile_count) {
    pdl_launch_dependents();   // the next kernel of the step may be set up beside this one
    pdl_wait();                // the kernel before has completed and its writes are visible
    __shared__ uint32_t total[kMaxExperts];
    __shared__ uint32_t soff[kMaxExperts + 1];
    __shared__ uint32_t tile_off[kMaxExperts + 1];
    __shared__ uint32_t part[1024];
    const uint32_t tid = threadIdx.x;
    // expert e's chunks split into `lanes` contiguous spans, one per thread; span totals scanned serially
    const uint32_t lanes = 1024u / kMaxExperts;                       // 8 threads per expert
    const uint32_t e = tid / lanes, span = tid % lanes;
    const uint32_t per = (chunks + lanes - 1) / lanes;
    const uint32_t c0 = span * per, c1 = min(chunks, c0 + per);
    uint32_t sum = 0;
    if (e < E)
        for (uint32_t c = c0; c < c1; c++) sum += chunk_cnt[(size_t)c * E + e];
    part[tid] = sum;
    __syncthreads();
    if (e < E) {
        uint32_t acc = 0;
        for (uint32_t s = 0; s < span; s++) acc += part[e * lanes + s];
        for (uint32_t c = c0; c < c1; c++) {
            const uint32_t v = chunk_cnt[(size_t)c * E + e];
            chunk_cnt[(size_t)c * E + e] = acc;
            acc += v;
        }
        if (span == lanes - 1) total[e] = acc;
    }
    __syncthreads();
    if (tid == 0) {
        uint32_t acc = 0, nt = 0;
        for (uint32_t x = 0; x < E; x++) {
            soff[x] = acc;
            tile_off[x] = nt;
            acc += total[x];
            nt += (total[x] + tile_rows - 1) / tile_rows;
        }
        soff[E] = acc;
        tile_off[E] = nt;
        *tile_count = nt;
    }
    __syncthreads();
    if (tid <= E) offsets[tid] = soff[tid];
    if (tid < E) {
        uint32_t nt = tile_off[tid];
        for (uint32_t b = 0; b < total[tid]; b += tile_rows, nt++) {
            tiles[2 * nt] = tid;
            tiles[2 * nt + 1] = b;
        }
    }
}

__global__ void __launch_bounds__(1024) route_scatter_kernel(const uint32_t* __restrict__ ids, uint32_t R, uint32_t E,
                                                             const uint32_t* __restrict__ chunk_cnt,
                                                             const uint32_t* __restrict__ offsets, uint32_t seg_len,
                                                             uint32_t seg_stride, uint32_t* __restrict__ row_of_route,
                                                             uint32_t* __restrict__ route_of_row) {
    pdl_launch_dependents();   // the next kernel of the step may be set up beside this one
    pdl_wait();                // the kernel before has completed and its writes are visible
    const uint32_t i = blockIdx.x * 1024u + threadIdx.x;
    if (i >= R) return;
    const uint32_t e = ids[i];
    if (e >= E) return;
    const uint32_t row = offsets[e] + chunk_cnt[(size_t)blockIdx.x * E + e] + row_of_route[i];
    row_of_route[i] = row;
    route_of_row[row] = route_label(i, seg_len, seg_stride);
}

// Gathers token rows into expert-sorted order, converting bf16 to the tiles' half operand and
// laying each block out in the tiles' operand order (see operand_pos in gemm.cuh): `half_span` is
// the distance between the two elements a code byte holds (16 for MXFP4 / Q4_0, 32 for Q4_K).
// The reference gathers inside its tiles (shaders/experts/projections.metal:208-233).
// CTAs stride over the sorted rows (`rows`, or *live_rows when given: the plan's route total, which
// may be less than the launch was sized for). A thread takes eight pairs of one block: two 16-byte
// loads (elements 8q .. 8q + 7 of the block's two halves; the row may sit in another GPU's memory, where
// small loads would waste the link) and two 16-byte stores of half2 = (x[k], x[k + half_span]). Rows that
// are not 16-byte aligned take the element-wise form.
__global__ void __launch_bounds__(256) permute_rows_kernel(const uint16_t* __restrict__ x,
                                                           const uint32_t* __restrict__ route_of_row, int K,
                                                           int H, int half_span, uint16_t* __restrict__ xs,
                                                           uint32_t rows, const uint32_t* __restrict__ live_rows) {
    pdl_launch_dependents();   // the next kernel of the step may be set up beside this one
    pdl_wait();                // the kernel before has completed and its writes are visible
    const uint32_t n = live_rows ? *live_rows : rows;
    const bool wide = (((uintptr_t)x | (uintptr_t)xs) & 15u) == 0 && (H & 7) == 0;
    const int per_block = half_span >> 3;                        // threads per block of 2 * half_span elements
    const int chunks = (H / (2 * half_span)) * per_block;        // 16-byte pieces of pairs per row
    for (uint32_t row = blockIdx.x; row < n; row += gridDim.x) {
        uint32_t token = route_of_row ? route_of_row[row] / (uint32_t)K : row;  // null: rows keep token order
        const uint16_t* src = x + (size_t)token * H;
        if (wide) {
            uint4* dst = reinterpret_cast<uint4*>(xs + (size_t)row * H);
            for (int c = threadIdx.x; c < chunks; c += 256) {
                const int blk = c / per_block, q = c - blk * per_block;
                const uint16_t* at = src + (size_t)blk * 2 * half_span + 8 * q;
                const uint4 a = *reinterpret_cast<const uint4*>(at);
                const uint4 b = *reinterpret_cast<const uint4*>(at + half_span);
                const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
                uint32_t o[8];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    __half2 lo = __floats2half2_rn(__uint_as_float(aw[j] << 16), __uint_as_float(bw[j] << 16));
                    __half2 hi = __floats2half2_rn(__uint_as_float(aw[j] & 0xffff0000u), __uint_as_float(bw[j] & 0xffff0000u));
                    o[2 * j] = *reinterpret_cast<uint32_t*>(&lo);
                    o[2 * j + 1] = *reinterpret_cast<uint32_t*>(&hi);
                }
                // pairs 8q .. 8q + 7 of the block: two pieces of the block's 2 * half_span halves
                uint4* out = dst + ((size_t)blk * half_span + 8 * q) / 4;
                out[0] = make_uint4(o[0], o[1], o[2], o[3]);
                out[1] = make_uint4(o[4], o[5], o[6], o[7]);
            }
            continue;
        }
        uint32_t* dst = reinterpret_cast<uint32_t*>(xs + (size_t)row * H);
        for (int i = threadIdx.x; i < H / 2; i += 256) {
            int blk = i / half_span, j = i % half_span;           // pair i of the row: block, byte index
            int k = blk * 2 * half_span + j;
            __half2 h = __floats2half2_rn(__uint_as_float((uint32_t)src[k] << 16),
                                          __uint_as_float((uint32_t)src[k + half_span] << 16));
            dst[i] = *reinterpret_cast<uint32_t*>(&h);
        }
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
    pdl_launch_dependents();   // the next kernel of the step may be set up beside this one
    pdl_wait();                // the kernel before has completed and its writes are visible
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

// The same combine with eight elements per thread (16-byte loads of the expert outputs and the residual):
// identical arithmetic per element, for hidden sizes that are multiples of eight. KT: the number of routes
// per token when it is known at compile time (their loads then go out together), 0: taken from K.
template <int KT>
__global__ void __launch_bounds__(256) moe_combine8_kernel(const uint16_t* __restrict__ y, const float* __restrict__ probs,
                                                           uint16_t* __restrict__ out, const uint16_t* __restrict__ shared,
                                                           int H, int T, int K, int round_sum, int shared_mode,
                                                           const uint32_t* __restrict__ status) {
    pdl_launch_dependents();   // the next kernel of the step may be set up beside this one
    pdl_wait();                // the kernel before has completed and its writes are visible
    const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
    const size_t octets = (size_t)T * H / 8;
    if (i >= octets) return;
    if (status && *reinterpret_cast<const volatile uint32_t*>(status) != 0u) return;
    const int per_row = H / 8;
    const int t = (int)(i / per_row), d = (int)(i % per_row) * 8;
    uint4 rw = *reinterpret_cast<const uint4*>(out + (size_t)t * H + d);
    uint32_t res[4] = {rw.x, rw.y, rw.z, rw.w};
    float r[8], s[8];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        r[2 * j] = __uint_as_float(res[j] << 16);
        r[2 * j + 1] = __uint_as_float(res[j] & 0xffff0000u);
        s[2 * j] = s[2 * j + 1] = 0.f;
    }
    if (shared_mode) {
        const uint4 sw4 = *reinterpret_cast<const uint4*>(shared + (size_t)t * H + d);
        const uint32_t sw[4] = {sw4.x, sw4.y, sw4.z, sw4.w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float h0 = __uint_as_float(sw[j] << 16), h1 = __uint_as_float(sw[j] & 0xffff0000u);
            if (shared_mode == 1) { s[2 * j] = h0; s[2 * j + 1] = h1; }
            else { r[2 * j] = bf16_round(__fadd_rn(r[2 * j], h0)); r[2 * j + 1] = bf16_round(__fadd_rn(r[2 * j + 1], h1)); }
        }
    }
    if (KT > 0) {
        uint4 yw4[KT > 0 ? KT : 1];
        float p[KT > 0 ? KT : 1];
#pragma unroll
        for (int k = 0; k < KT; k++) {
            yw4[k] = *reinterpret_cast<const uint4*>(y + ((size_t)t * KT + k) * H + d);
            p[k] = probs[(size_t)t * KT + k];
        }
#pragma unroll
        for (int k = 0; k < KT; k++) {                     // the same order of additions as the loop below
            const uint32_t yw[4] = {yw4[k].x, yw4[k].y, yw4[k].z, yw4[k].w};
#pragma unroll
            for (int j = 0; j < 4; j++) {
                s[2 * j] = __fmaf_rn(__uint_as_float(yw[j] << 16), p[k], s[2 * j]);
                s[2 * j + 1] = __fmaf_rn(__uint_as_float(yw[j] & 0xffff0000u), p[k], s[2 * j + 1]);
            }
        }
    } else {
        for (int k = 0; k < K; k++) {
            const uint4 yw4 = *reinterpret_cast<const uint4*>(y + ((size_t)t * K + k) * H + d);
            const uint32_t yw[4] = {yw4.x, yw4.y, yw4.z, yw4.w};
            const float p = probs[(size_t)t * K + k];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                s[2 * j] = __fmaf_rn(__uint_as_float(yw[j] << 16), p, s[2 * j]);
                s[2 * j + 1] = __fmaf_rn(__uint_as_float(yw[j] & 0xffff0000u), p, s[2 * j + 1]);
            }
        }
    }
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        float a = s[2 * j], b = s[2 * j + 1];
        if (round_sum) { a = bf16_round(a); b = bf16_round(b); }
        o[j] = (uint32_t)f32_to_bf16_bits(__fadd_rn(r[2 * j], a)) | ((uint32_t)f32_to_bf16_bits(__fadd_rn(r[2 * j + 1], b)) << 16);
    }
    *reinterpret_cast<uint4*>(out + (size_t)t * H + d) = make_uint4(o[0], o[1], o[2], o[3]);
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
