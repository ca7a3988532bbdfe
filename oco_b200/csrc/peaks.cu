// Measured tensor-pipe ceilings of this GPU: back-to-back tcgen05.mma of one kind on one shared-memory
// tile (M = 128, N = 256, zero operands, fp32 accumulators in tensor memory), one issuing thread per
// SM. The benchmark divides its tensor-bound kernels' rates by these figures beside the cuBLAS bf16
// figure it is given; nothing on the layer's path calls this.
#include "gemm.cuh"
#include "mx.cuh"

using namespace oco;

namespace {

__device__ __forceinline__ void umma_f8f6f4(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void umma_mxf8f6f4(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t sfa, uint32_t sfb, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc), "r"(sfa), "r"(sfb) : "memory");
}
// kind::mxf8f6f4 with e4m3 operands, UE8M0 scales, scale id = the byte of the scale column
__device__ __forceinline__ uint32_t idesc_mxf8(uint32_t n, uint32_t sf_id) {
    return (sf_id << 4) | ((n >> 3) << 17) | (1u << 23) | ((128u >> 4) << 24) | (sf_id << 29);
}

// kind: 0 f16, 1 f8f6f4 (e4m3), 2 mxf8f6f4 (e4m3, block-scaled), 3 mxf4 (e2m1, block-scaled)
__global__ void __launch_bounds__(128, 1) tensor_peak_kernel(int kind, int iters, uint32_t* status) {
    extern __shared__ unsigned char smem_raw[];
    const int tid = threadIdx.x, warp = tid >> 5;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char* gen = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t a_base = base, b_base = base + 16384u, ctrl = b_base + 32768u;
    for (uint32_t i = tid * 16; i < 16384u + 32768u + 1024u; i += 128 * 16) *reinterpret_cast<uint4*>(gen + i) = make_uint4(0, 0, 0, 0);
    __syncthreads();
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen + (ctrl - base) + 64);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    const uint32_t bar = ctrl;
    if (tid == 0) { mbar_init(bar, 1); *abort_flag = 0; fence_barrier_init(); }
    fence_proxy_async_smem();
    if (warp == 0) { tmem_alloc(smem_u32(tmem_slot), 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (tid == 0) {
        const uint32_t t_sf = tmem_base + 256;
        if (kind >= 2)
            for (int i = 0; i < 3; i++) mx_cp_scales(t_sf + 4u * i, mx_sf_desc(ctrl + 512u));
        const uint64_t a = umma_desc(a_base), b = umma_desc(b_base);
        const uint32_t id16 = umma_idesc_f16(256);
        for (int it = 0; it < iters; it++) {
#pragma unroll
            for (int kk = 0; kk < 4; kk++) {
                const uint32_t acc = (it | kk) ? 1u : 0u;
                if (kind == 0) umma_f16(tmem_base, a + 2u * kk, b + 2u * kk, id16, acc);
                else if (kind == 1) umma_f8f6f4(tmem_base, a + 2u * kk, b + 2u * kk, id16, acc);
                else if (kind == 2) umma_mxf8f6f4(tmem_base, a + 2u * kk, b + 2u * kk, idesc_mxf8(256, kk), t_sf, t_sf + 4, acc);
                else umma_mxf4(tmem_base, a + 2u * kk, b + 2u * kk, mx_idesc(256, (kk & 1) * 2), t_sf, t_sf + 4, acc);
            }
        }
        umma_commit(bar);
        mbar_wait(bar, 0u, abort_flag, status);
    }
    __syncthreads();
    tc_fence_before();
    __syncthreads();
    if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

}  // namespace

extern "C" int oco_tensor_peak(int kind, int iters, float* tflops_out) {
    if (kind < 0 || kind > 3 || iters < 1 || iters > (1 << 20) || !tflops_out) return OCO_INVALID_ARGUMENT;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return OCO_CUDA_ERROR;
    if (cudaFuncSetAttribute(tensor_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024) != cudaSuccess) return OCO_CUDA_ERROR;
    uint32_t* status = nullptr;
    if (cudaMalloc(&status, 256) != cudaSuccess) return OCO_CUDA_ERROR;
    cudaMemset(status, 0, 256);
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0); cudaEventCreate(&e1);
    tensor_peak_kernel<<<sms, 128, 56 * 1024>>>(kind, 64, status);   // warm-up
    float best = 1e30f;
    for (int rep = 0; rep < 3; rep++) {
        cudaEventRecord(e0);
        tensor_peak_kernel<<<sms, 128, 56 * 1024>>>(kind, iters, status);
        cudaEventRecord(e1);
        if (cudaEventSynchronize(e1) != cudaSuccess) break;
        float ms = 0.f;
        cudaEventElapsedTime(&ms, e0, e1);
        if (ms > 0.f && ms < best) best = ms;
    }
    uint32_t word = 1;
    cudaMemcpy(&word, status, 4, cudaMemcpyDeviceToHost);
    cudaEventDestroy(e0); cudaEventDestroy(e1); cudaFree(status);
    if (cudaGetLastError() != cudaSuccess || best > 1e29f) return OCO_CUDA_ERROR;
    if (word != 0) return OCO_DEVICE_TIMEOUT;
    static const int kper[4] = {16, 32, 32, 64};
    *tflops_out = (float)((double)sms * iters * 4 * 2.0 * 128 * 256 * kper[kind] / (best * 1e-3) / 1e12);
    return OCO_OK;
}
