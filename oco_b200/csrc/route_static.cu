// Single-token routing without any device allocation.
//
// Who needs this: hosts that fix their device-memory budget once and must not allocate afterwards.
// The reference engine is such a host: it plans every buffer of a session up front, packs them
// into an arena and checks the total against the device's working-set limit
// (src/gpu/arena.rs:50-112), so nothing on its decode path may ask the driver for memory. The same
// holds for a plugin that runs beside a framework whose caching allocator already owns the GPU's
// free memory (a raw cudaMalloc there can fail although the framework still has room), and for
// latency-critical loops that cannot afford the device-wide synchronisation cudaMalloc/cudaFree
// imply. Such callers cannot bind a workspace for a quick "which experts does this token go to?"
// query; this entry point answers it with the scratch it needs held in a fixed device array that
// is part of the library image.
//
// The scratch (router logits of one token plus an arrival counter) lives in a file-scope
// `__device__` array of kScratchBytes = 1024 bytes. Every GPU that loads the library carries that
// array until the process exits. All calls on a device share it, and it keeps whatever the last
// call left there; the counter is cleared at the start of every call. Two calls that overlap on
// the same GPU (different streams, or different threads) race on the array and must not be issued.
//
// The first call on each device looks the array's device address up (cudaGetSymbolAddress) and
// caches it; make that first call before any stream capture begins.
#include <cstdio>

#include "common.cuh"
#include "router.cuh"

using namespace oco;

namespace {

constexpr int kStaticMaxExperts = 128;   // logits held in the static scratch
constexpr int kStaticMaxHidden = 16384;  // bound on the contraction length accepted here
constexpr size_t kScratchBytes = 1024;   // 128 logits (512 B) + arrival counter, padded
constexpr int kMaxDevices = 64;

// In host code this name is only a handle for the symbol; the device address is looked up with
// cudaGetSymbolAddress below. Device code may name the array directly.
static __device__ __align__(256) unsigned char g_route_scratch[kScratchBytes];

struct ScratchView {
    float* logits;           // [kStaticMaxExperts]
    unsigned int* arrivals;  // [1]
};
__host__ __device__ inline ScratchView view(unsigned char* base) {
    ScratchView v;
    v.logits = reinterpret_cast<float*>(base);
    v.arrivals = reinterpret_cast<unsigned int*>(base + kStaticMaxExperts * sizeof(float));
    return v;
}

// One warp per expert computes its logit into the scratch; the CTA that arrives last (counted in
// the scratch) selects the experts and writes ids and weights. No CTA waits for another.
template <int ARCH>
__global__ void __launch_bounds__(256) route_token_static_kernel(const uint16_t* __restrict__ x,
                                                                 const float* __restrict__ w,
                                                                 const float* __restrict__ bias, int H, int E, int K,
                                                                 int normalize, float scale, unsigned char* scratch,
                                                                 uint32_t* __restrict__ ids, float* __restrict__ probs) {
    __shared__ int is_last;
    ScratchView s = view(scratch);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e = blockIdx.x * 8 + warp;
    if (e < E) {
        float v = canonical_logit<ARCH == OCO_ARCH_GPT_OSS>(x, w + (size_t)e * H, H, lane);
        if (ARCH == OCO_ARCH_GPT_OSS) v = __fadd_rn(v, bf16_round(bias[e]));
        if (lane == 0) s.logits[e] = v;
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) is_last = atomicAdd(s.arrivals, 1u) == gridDim.x - 1;
    __syncthreads();
    if (!is_last || warp != 0) return;
    __threadfence();
    float lv[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        int idx = lane + 32 * j;
        lv[j] = idx < E ? __ldcg(s.logits + idx) : 0.0f;
    }
    uint32_t id[kMaxTopK];
    float p[kMaxTopK];
    select_experts<ARCH>(lv, E, K, ARCH == OCO_ARCH_NEMOTRON ? bias : nullptr, normalize, scale, lane, id, p);
#pragma unroll
    for (int r = 0; r < kMaxTopK; r++)
        if (r < K && lane == r) { ids[r] = id[r]; probs[r] = p[r]; }
}

unsigned char* g_scratch_ptr[kMaxDevices] = {nullptr};

int complain(char* err, size_t err_len, int code, const char* msg) {
    if (err && err_len) snprintf(err, err_len, "%s", msg);
    return code;
}

}  // namespace

extern "C" int oco_moe_route_token_static(int arch, const uint16_t* x_bf16, const float* router_w,
                                          const float* router_b, int hidden, int experts, int top_k, int normalize,
                                          float scale, uint32_t* ids_out, float* probs_out, void* cuda_stream,
                                          char* err, size_t err_len) {
    if (err && err_len) err[0] = 0;
    if (!x_bf16 || !router_w || !ids_out || !probs_out)
        return complain(err, err_len, OCO_INVALID_ARGUMENT, "x, router_w, ids_out and probs_out must not be null");
    if (arch < OCO_ARCH_GPT_OSS || arch > OCO_ARCH_QWEN) return complain(err, err_len, OCO_INVALID_ARGUMENT, "unknown arch");
    if (arch != OCO_ARCH_QWEN && !router_b)
        return complain(err, err_len, OCO_INVALID_ARGUMENT, "this family needs router_b (logit or selection bias)");
    if (experts < 1 || experts > kStaticMaxExperts)
        return complain(err, err_len, OCO_UNSUPPORTED_SHAPE,
                        "experts exceeds the 128 logits the static scratch holds (1024-byte device array)");
    if (top_k < 1 || top_k > kMaxTopK || top_k > experts)
        return complain(err, err_len, OCO_UNSUPPORTED_SHAPE, "top_k must be 1..8 and at most experts");
    if (hidden < 4 || hidden % 4 || hidden > kStaticMaxHidden)
        return complain(err, err_len, OCO_UNSUPPORTED_SHAPE, "hidden must be a multiple of 4 and at most 16384");
    if (((uintptr_t)x_bf16 & 7u) || ((uintptr_t)router_w & 15u))
        return complain(err, err_len, OCO_INVALID_ARGUMENT, "x must be 8-byte and router_w 16-byte aligned");

    // Set-up, once per device, with that device current: the device address of the scratch.
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
        return complain(err, err_len, OCO_CUDA_ERROR, "no current CUDA device");
    if (!g_scratch_ptr[dev]) {
        unsigned char* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_route_scratch);
        if (e != cudaSuccess || !ptr) return complain(err, err_len, OCO_CUDA_ERROR, cudaGetErrorString(e));
        g_scratch_ptr[dev] = ptr;
    }
    unsigned char* scratch = g_scratch_ptr[dev];
    cudaStream_t st = (cudaStream_t)cuda_stream;
    // The arrival counter must start at zero; the logits are overwritten before they are read.
    cudaError_t e = cudaMemsetAsync(view(scratch).arrivals, 0, sizeof(unsigned int), st);
    if (e != cudaSuccess) return complain(err, err_len, OCO_CUDA_ERROR, cudaGetErrorString(e));
    const int grid = (experts + 7) / 8;
    switch (arch) {
        case OCO_ARCH_GPT_OSS:
            route_token_static_kernel<OCO_ARCH_GPT_OSS><<<grid, 256, 0, st>>>(x_bf16, router_w, router_b, hidden, experts,
                                                                             top_k, normalize, scale, scratch, ids_out, probs_out);
            break;
        case OCO_ARCH_NEMOTRON:
            route_token_static_kernel<OCO_ARCH_NEMOTRON><<<grid, 256, 0, st>>>(x_bf16, router_w, router_b, hidden, experts,
                                                                              top_k, normalize, scale, scratch, ids_out, probs_out);
            break;
        default:
            route_token_static_kernel<OCO_ARCH_QWEN><<<grid, 256, 0, st>>>(x_bf16, router_w, router_b, hidden, experts,
                                                                          top_k, normalize, scale, scratch, ids_out, probs_out);
            break;
    }
    e = cudaGetLastError();
    if (e != cudaSuccess) return complain(err, err_len, OCO_CUDA_ERROR, cudaGetErrorString(e));
    return OCO_OK;
}
