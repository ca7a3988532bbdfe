// Shared device helpers: rounding conversions, the deterministic exp, activations, block-scale
// decoding, bounded mbarrier waits and the small PTX wrappers the kernels use.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp4.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/oco_moe.h"

namespace oco {

constexpr int kMaxExperts = 128;
constexpr int kMaxTopK = 8;

// Status word written by device code (workspace word 0). Non-zero = a bounded wait gave up.
enum DeviceStatus : uint32_t { kDevOk = 0, kDevBarrierTimeout = 1 };

__device__ __forceinline__ float bf16_bits_to_f32(uint16_t h) { return __uint_as_float((uint32_t)h << 16); }
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float f) {
    return __bfloat16_as_ushort(__float2bfloat16_rn(f));
}
__device__ __forceinline__ float bf16_round(float f) { return __bfloat162float(__float2bfloat16_rn(f)); }
__device__ __forceinline__ uint16_t f32_to_f16_bits(float f) { return __half_as_ushort(__float2half_rn(f)); }
__device__ __forceinline__ float f16_bits_to_f32(uint16_t h) { return __half2float(__ushort_as_half(h)); }
__device__ __forceinline__ bool nonfinite(float v) { return (__float_as_uint(v) & 0x7f800000u) == 0x7f800000u; }
__device__ __forceinline__ float qnan() { return __uint_as_float(0x7fc00000u); }

// exp from IEEE basic operations only, so the host checker that carries the same sequence agrees
// bit for bit. Accuracy about 1 ulp over the finite range.
__device__ __forceinline__ float exp_det(float a) {
    if (a != a) return a;
    if (a > 88.72283f) return __uint_as_float(0x7f800000u);
    if (a < -104.0f) return 0.0f;
    float n = rintf(__fmul_rn(a, 1.44269504088896341f));
    float r = __fmaf_rn(n, -0.693145751953125f, a);
    r = __fmaf_rn(n, -1.42860682030941723212e-6f, r);
    float p = 1.0f / 720.0f;
    p = __fmaf_rn(p, r, 1.0f / 120.0f);
    p = __fmaf_rn(p, r, 1.0f / 24.0f);
    p = __fmaf_rn(p, r, 1.0f / 6.0f);
    p = __fmaf_rn(p, r, 0.5f);
    p = __fmaf_rn(p, r, 1.0f);
    p = __fmaf_rn(p, r, 1.0f);
    int ni = (int)n;
    int n1 = ni / 2, n2 = ni - n1;
    float s1 = __uint_as_float((uint32_t)(n1 + 127) << 23), s2 = __uint_as_float((uint32_t)(n2 + 127) << 23);
    return __fmul_rn(__fmul_rn(p, s1), s2);
}

// Clipped SwiGLU (reference shaders/experts/projections.metal:4-13).
__device__ __forceinline__ float swiglu_clipped(float g, float u) {
    if (nonfinite(g) || nonfinite(u)) return qnan();
    g = fminf(g, 7.0f);
    u = fminf(fmaxf(u, -6.0f), 8.0f);
    float e = exp_det(__fmul_rn(-fabsf(g), 1.702f));
    float sigmoid = __fdiv_rn(g < 0 ? e : 1.0f, __fadd_rn(1.0f, e));
    return __fmul_rn(__fmul_rn(sigmoid, g), u);
}

// SiLU gate over bf16 operands (reference shaders/elementwise.metal:67-87); returns a bf16 value.
__device__ __forceinline__ float silu_gate_bf16(float a, float b) {
    if (nonfinite(a) || nonfinite(b)) return qnan();
    float e = exp_det(-fabsf(a));
    float sigmoid = __fdiv_rn(a < 0 ? e : 1.0f, __fadd_rn(1.0f, e));
    float activated = __fmul_rn(sigmoid, a);
    return bf16_round(__fmul_rn(bf16_round(activated), b));
}

// E8M0 block scale (reference projections.metal:19-23): 255 is NaN, 0 is 2^-127.
__device__ __forceinline__ float e8m0_scale(uint32_t e) {
    if (e == 255u) return qnan();
    return __uint_as_float(e == 0u ? 0x00400000u : (e << 23));
}

// Two e2m1 codes of one byte -> half2 (low nibble in .x, high nibble in .y), one cvt on sm_100a.
__device__ __forceinline__ uint32_t e2m1x2_to_half2(uint32_t byte) {
    __half2_raw r = __nv_cvt_fp4x2_to_halfraw2((__nv_fp4x2_storage_t)(byte & 0xffu), __NV_E2M1);
    return (uint32_t)r.x | ((uint32_t)r.y << 16);
}

// The four code bytes of a word -> four half2 (low nibble in .x, high nibble in .y).
__device__ __forceinline__ void cvt_e2m1x2_x4(uint32_t w, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
        "mov.b32 {b0, b1, b2, b3}, %4;\n\t"
        "cvt.rn.f16x2.e2m1x2 %0, b0;\n\t"
        "cvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
        "cvt.rn.f16x2.e2m1x2 %2, b2;\n\t"
        "cvt.rn.f16x2.e2m1x2 %3, b3;\n\t}"
        : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
        : "r"(w));
}
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---- unaligned byte access through aligned words -----------------------------------------------
// 4 bytes starting at an arbitrary byte address of global memory.
__device__ __forceinline__ uint32_t ldg_u32_unaligned(const uint8_t* p) {
    uintptr_t a = (uintptr_t)p;
    const uint32_t* w = (const uint32_t*)(a & ~(uintptr_t)3);
    uint32_t sh = ((uint32_t)a & 3u) * 8u;
    uint32_t lo = __ldg(w);
    if (sh == 0) return lo;
    return __funnelshift_r(lo, __ldg(w + 1), sh);
}

// ---- cp.async (16-byte, L2 only) ----------------------------------------------------------------
__device__ __forceinline__ void cp_async16(uint32_t smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_dst), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// ---- mbarrier with bounded waits ----------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Waits for the phase with the given parity. Gives up after `limit` clock cycles, or at once when
// another thread of the CTA has already given up (`*abort_flag` set): the caller carries on with
// whatever is in memory, the kernel runs to its normal end and the host sees the status word.
constexpr long long kWaitCycles = 400000000LL;  // about 0.2 s at B200 clocks
__device__ __forceinline__ void mbar_wait_for(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                              uint32_t* status_word, long long limit) {
    if (mbar_try_wait(bar, parity)) return;
    long long start = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (*abort_flag) return;
        if (clock64() - start > limit) {
            *abort_flag = 1u;
            atomicExch(status_word, (uint32_t)kDevBarrierTimeout);
            return;
        }
    }
}
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                          uint32_t* status_word) {
    mbar_wait_for(bar, parity, abort_flag, status_word, kWaitCycles);
}

// Programmatic dependent launch: a kernel launched with the programmatic-serialization attribute may
// start while its predecessor in the stream still runs; pdl_wait() returns when the predecessor has
// completed and its writes are visible. pdl_launch_dependents() lets the successor start launching.
// Both do nothing in a kernel launched the ordinary way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

}  // namespace oco
