// C ABI of the MoE layer: plan object, workspace carve-up, TMA descriptors and launch sequencing.
// The sequencing mirrors the reference operators it replaces:
//   Bindings::experts        src/weights/compute/feed_forward.rs:107-275
//   Bindings::relu_experts   src/weights/compute/nemotron.rs:286-545
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <cstdlib>
#include <new>

#include "common.cuh"
#include "decode.cuh"
#include "batch.cuh"
#include "gemm.cuh"
#include "gemm_wide.cuh"
#include "gemm_pair.cuh"
#include "mx.cuh"
#include "gemm_mx.cuh"
#include <cmath>
#include "plan.cuh"
#include "router.cuh"

using namespace oco;

namespace {

constexpr int kTileSizes[4] = {32, 64, 128, 256};
constexpr int kTileKinds = 4;
constexpr int kMaxMarks = 16;

struct Workspace {
    uint32_t* status = nullptr;
    float* logits = nullptr;
    float* router_rounded = nullptr;  // gpt-oss: router weights rounded to bf16, as f32
    uint32_t* ids = nullptr;
    float* probs = nullptr;
    uint32_t* offsets = nullptr;
    uint32_t* tile_count = nullptr;
    uint32_t* tiles = nullptr;
    uint32_t* row_of_route = nullptr;
    uint32_t* route_of_row = nullptr;
    uint32_t* chunk_cnt = nullptr;   // many-CTA route plan: per chunk of 1024 routes, the count per expert
    uint16_t* xs = nullptr;       // half [R, H] expert-sorted input rows
    uint16_t* act = nullptr;      // half [R, F] expert-sorted activated rows
    uint16_t* y = nullptr;        // bf16 [R, H] expert outputs, route order
    float* act1 = nullptr;        // f32 [K, F] single-token activations
    __half* actfrag = nullptr;    // single-token B fragments of the down projection
    __half* xfrag = nullptr;      // single-token B fragments of the token itself
    __half* bfrag_in = nullptr;   // few-token path: B fragments of each route group, input rows
    __half* bfrag_out = nullptr;  //                 and activations
    uint32_t* arrivals = nullptr; // single-token combine: one counter per output row (or row block), then the router's
    uint16_t* xh = nullptr;       // half [T, H] token-order input rows (shared expert)
    uint16_t* mid = nullptr;      // half [T, S] shared expert intermediate
    uint16_t* shared_out = nullptr;  // bf16 [T, H]
    float* sh_act1 = nullptr;
    __half* sh_actfrag = nullptr;
    uint32_t* sh_ids = nullptr;
    uint16_t* norm = nullptr;     // bf16 [T, H] normalised rows of oco_moe_add_norm_forward
    unsigned char* mx_xb = nullptr;   // block-scaled single-token path: the token as e2m1 pieces
    unsigned char* mx_xsfb = nullptr; //   and their scales
    unsigned char* mx_actb = nullptr; //   each route's activations as e2m1 pieces [top_k][..], their scales,
    unsigned char* mx_actsfb = nullptr;
    uint32_t* mx_blk_arrivals = nullptr;   // and one counter per route and block of 32 activations
    unsigned char* mxq_x = nullptr;   // numerics 2: expert-sorted input rows quantised to e2m1 [R][H / 2], their scale tiles,
    unsigned char* mxq_xsf = nullptr;
    unsigned char* mxq_act = nullptr; //   and the same for the activated rows [R][F / 2]
    unsigned char* mxq_actsf = nullptr;
    uint16_t* host_x[2] = {nullptr, nullptr};     // staging for the host-buffer entry points: two calls may be in flight
    uint16_t* host_res[2] = {nullptr, nullptr};
    size_t total = 0;
};

}  // namespace

struct oco_moe_plan {
    oco_moe_desc d{};
    oco_moe_weights w{};
    Workspace ws{};
    bool have_ws = false, have_w = false;
    bool have_experts = false;   // expert banks bound (enough for oco_moe_experts)
    bool router_ready = false;   // the rounded router copy matches the bound weights and workspace
    int max_rows = 0;
    int device = -1;             // the device that was current when the workspace was bound
    int sm_count = 148;
    int launches = 0;
    int last_tile_rows = 0;
    uint32_t up_row_bytes = 0, down_row_bytes = 0, shared_up_row_bytes = 0, shared_down_row_bytes = 0;
    // Resolved gate / up operands: two tensors, or the rows of one interleaved tensor (row 2c = gate c,
    // row 2c + 1 = up c), in which case consecutive rows of either matrix lie two packed rows apart.
    const uint8_t* gate_rows = nullptr;
    const uint8_t* up_rows = nullptr;
    const float* gate_bias = nullptr;
    const float* up_bias = nullptr;
    uint32_t up_row_stride = 0;  // bytes between consecutive gate (or up) rows
    int up_bias_stride = 1;      // floats between consecutive gate (or up) biases
    // block-scaled single-token path (mx.cuh): usable once prepare_mx has built the tensor maps
    bool mx_ready = false, mx_on = false;    // OCO_MOE_TOKEN_MX=1 selects them (measured slower than the mma.sync kernels so far)
    CUtensorMap map_xs[kTileKinds], map_act[kTileKinds], map_xh[kTileKinds], map_mid[kTileKinds];
    CUtensorMap map_mxq_x, map_mxq_act;   // numerics 2: the quantised rows as bytes
    // numerics 2 with repacked weights (oco_moe_bind_repacked): code planes and scale tiles of gate, up, down
    bool rp_ready = false;
    bool rp_token = false;       // single-token calls read the repacked form too
    bool rp_token_on = false;    // OCO_MOE_REPACKED_TOKEN=1 (measured slower than the default single-token kernels: off unless asked for)
    unsigned char* rp_codes[3] = {nullptr, nullptr, nullptr};
    unsigned char* rp_sf[3] = {nullptr, nullptr, nullptr};
    // Per-phase timestamps (the counterpart of the reference's OCO_PROFILE counter heap,
    // src/gpu/profile.rs:1-31, src/gpu/dispatch.rs:189-208): one event before each kernel.
    // oco_moe_forward_host_begin / _end: the rows travel on two streams of the plan's own (one per direction);
    // call c uses staging slot c % 2, whose events say when its x rows, its residual rows, its kernels and its
    // copy back are done
    cudaStream_t in_stream = nullptr, out_stream = nullptr;
    cudaEvent_t ev_x[2] = {}, ev_res[2] = {}, ev_done[2] = {}, ev_out[2] = {};
    uint64_t host_begun = 0, host_ended = 0;
    bool no_batch_path = false;  // OCO_MOE_NO_BATCH=1: few tokens take the tile kernels too
    int batch_max_avg = 8;       // routes per expert (on average) up to which the streamed few-token kernels run
                                 // (measured: they win up to 16-32 at the gpt-oss shapes; OCO_MOE_BATCH_MAX_AVG overrides)
    int route_plan_single_max = 2048;   // routes up to which one CTA makes the route plan (OCO_MOE_ROUTE_PLAN_SINGLE_MAX)
    int wide_min_avg = 1;        // OCO_MOE_WIDE_MIN_AVG: routes per expert from which layers take the 256-route tiles
    int router_block_min = 512;  // OCO_MOE_ROUTER_BLOCK_MIN: rows from which the register-blocked router kernel runs
    bool static_tiles = false;   // OCO_MOE_STATIC_TILES=1: the wide tile kernel's CTA c takes items c, c + grid, ... (no counter)
    bool pair_tiles = false;     // OCO_MOE_PAIR_TILES=1: 256-route tiles on SM pairs (grouped_gemm_pair_kernel)
    bool narrow_tiles = false;   // OCO_MOE_NARROW_TILES=1: keep the generic tile kernel for 256-route tiles too
    bool profiling = false;
    int n_marks = 0;
    cudaEvent_t marks[kMaxMarks] = {};
    const char* mark_names[kMaxMarks] = {};
    char err[256] = {0};
};

struct oco_moe_graph {
    cudaGraphExec_t exec = nullptr;
    oco_moe_plan* plan = nullptr;
};

namespace {

int fail(oco_moe_plan* p, int code, const char* fmt, ...) {
    if (p) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(p->err, sizeof(p->err), fmt, ap);
        va_end(ap);
    }
    return code;
}

#define CK(call)                                                                                     \
    do {                                                                                             \
        cudaError_t e_ = (call);                                                                     \
        if (e_ != cudaSuccess) return fail(plan, OCO_CUDA_ERROR, "%s: %s", #call, cudaGetErrorString(e_)); \
    } while (0)

// A kernel's opt-in to large dynamic shared memory is a per-device attribute: this remembers, per
// launch site, on which devices it has been set (bit d = device d). Two threads may both find the
// bit clear and set the attribute twice, which is harmless; a set bit is never lost.
struct DeviceOnce {
    std::atomic<uint64_t> done{0};
    bool need(int dev) const { return dev < 0 || dev >= 64 || !((done.load(std::memory_order_acquire) >> dev) & 1u); }
    void mark(int dev) { if (dev >= 0 && dev < 64) done.fetch_or(1ull << dev, std::memory_order_release); }
};
#define ALLOW_SMEM_ONCE(kernel)                                   \
    do {                                                          \
        static DeviceOnce once_;                                  \
        if (once_.need(plan->device)) {                           \
            CK(allow_smem(kernel));                               \
            once_.mark(plan->device);                             \
        }                                                         \
    } while (0)

// Stamps the stream ahead of the phase called `name`; "end" closes the last phase.
void mark(oco_moe_plan* plan, cudaStream_t st, const char* name) {
    if (!plan->profiling || plan->n_marks >= kMaxMarks) return;
    int i = plan->n_marks;
    if (!plan->marks[i] && cudaEventCreate(&plan->marks[i]) != cudaSuccess) return;
    if (cudaEventRecord(plan->marks[i], st) != cudaSuccess) return;
    plan->mark_names[i] = name;
    plan->n_marks = i + 1;
}

uint32_t packed_row_bytes(int fmt, int k) {
    switch (fmt) {
        case OCO_FMT_MXFP4: return (uint32_t)(k / 32 * 17);
        case OCO_FMT_Q4_0: return (uint32_t)(k / 32 * 18);
        case OCO_FMT_Q4_K: return (uint32_t)(k / 256 * 144);
    }
    return 0;
}
int block_elems(int fmt) { return fmt == OCO_FMT_Q4_K ? 256 : 32; }

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Lays the workspace out; with base == nullptr only the total is meaningful.
// Route groups (up to eight routes of one expert) that R routes over E experts can form.
size_t batch_max_groups(size_t R, size_t E) { return R / 8 + (E < R ? E : R); }

Workspace carve(const oco_moe_desc& d, int max_rows, unsigned char* base) {
    Workspace w;
    size_t off = 0;
    auto take = [&](size_t bytes) {
        unsigned char* p = base ? base + off : nullptr;
        off = align_up(off + bytes, 256);
        return p;
    };
    const size_t T = (size_t)max_rows, K = (size_t)d.top_k, R = T * K, E = (size_t)d.experts;
    const size_t H = (size_t)d.hidden, F = (size_t)d.ffn, S = (size_t)d.shared_ffn;
    const size_t P = (K + 1) / 2;
    w.status = (uint32_t*)take(256);
    w.logits = (float*)take(T * E * 4);
    w.router_rounded = (float*)take(d.arch == OCO_ARCH_GPT_OSS ? E * H * 4 : 4);
    w.ids = (uint32_t*)take(R * 4);
    w.probs = (float*)take(R * 4);
    w.offsets = (uint32_t*)take((E + 1) * 4);
    w.tile_count = (uint32_t*)take(4);
    w.tiles = (uint32_t*)take(2 * (R / 8 + E + 1) * 4);
    w.row_of_route = (uint32_t*)take(R * 4);
    w.route_of_row = (uint32_t*)take(R * 4);
    w.chunk_cnt = (uint32_t*)take(((R + 1023) / 1024) * E * 4);
    w.xs = (uint16_t*)take(R * H * 2);
    w.act = (uint16_t*)take(R * F * 2);
    w.y = (uint16_t*)take(R * H * 2);
    w.act1 = (float*)take(K * F * 4);
    w.actfrag = (__half*)take(P * (F / 32) * 128 * 2);
    w.xfrag = (__half*)take((H / 32) * 128);
    {
        const size_t groups = batch_max_groups(R < 64 * E ? R : 64 * E, E);
        w.bfrag_in = (__half*)take(groups * (H / 32) * kBatchFragBlock);
        w.bfrag_out = (__half*)take(groups * (F / 32) * kBatchFragBlock);
    }
    w.arrivals = (uint32_t*)take((H + 1) * 4);
    if (S) {
        w.xh = (uint16_t*)take(T * H * 2);
        w.mid = (uint16_t*)take(T * S * 2);
        w.shared_out = (uint16_t*)take(T * H * 2);
        w.sh_act1 = (float*)take(S * 4);
        w.sh_actfrag = (__half*)take((S / 32) * 128 * 2);
        w.sh_ids = (uint32_t*)take(256);
    }
    w.norm = (uint16_t*)take(T * H * 2);
    if (d.weight_format == OCO_FMT_MXFP4) {
        w.mx_xb = (unsigned char*)take(mx_b_bytes(8, (uint32_t)(H / 32)));
        w.mx_xsfb = (unsigned char*)take(mx_sfb_bytes((uint32_t)(H / 32)));
        w.mx_actb = (unsigned char*)take(K * mx_b_bytes(8, (uint32_t)(F / 32)));
        w.mx_actsfb = (unsigned char*)take(K * mx_sfb_bytes((uint32_t)(F / 32)));
        w.mx_blk_arrivals = (uint32_t*)take(K * (F / 32) * 4);
    }
    if (d.numerics == 2) {
        const size_t tiles128 = R / 112 + E + 1;      // tiles of 128 routes (weights as stored) or 112 (repacked weights)
        w.mxq_x = (unsigned char*)take(R * H / 2);
        w.mxq_xsf = (unsigned char*)take(tiles128 * ((H / 32 + 7) / 8) * 1024);
        w.mxq_act = (unsigned char*)take(R * F / 2);
        w.mxq_actsf = (unsigned char*)take(tiles128 * ((F / 32 + 7) / 8) * 1024);
    }
    for (int i = 0; i < 2; i++) {
        w.host_x[i] = (uint16_t*)take(T * H * 2);
        w.host_res[i] = (uint16_t*)take(T * H * 2);
    }
    w.total = off;
    return w;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int make_row_map(oco_moe_plan* plan, CUtensorMap* map, void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    // looked up once per process (initialisation of a function-local static is thread-safe)
    static const EncodeTiledFn encode = [] {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            fn = nullptr;
        return (EncodeTiledFn)fn;
    }();
    if (!encode) return fail(plan, OCO_CUDA_ERROR, "cuTensorMapEncodeTiled unavailable");
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * 2};
    cuuint32_t box[2] = {64, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, base, dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(plan, OCO_CUDA_ERROR, "cuTensorMapEncodeTiled failed (%d)", (int)r);
    return OCO_OK;
}

// The same over rows of bytes (e2m1 pairs): box 128 bytes x box_rows.
int make_byte_map(oco_moe_plan* plan, CUtensorMap* map, void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_rows) {
    static const EncodeTiledFn encode = [] {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            fn = nullptr;
        return (EncodeTiledFn)fn;
    }();
    if (!encode) return fail(plan, OCO_CUDA_ERROR, "cuTensorMapEncodeTiled unavailable");
    cuuint64_t dims[2] = {row_bytes, rows};
    cuuint64_t strides[1] = {row_bytes};
    cuuint32_t box[2] = {128, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(plan, OCO_CUDA_ERROR, "cuTensorMapEncodeTiled (byte rows) failed (%d)", (int)r);
    return OCO_OK;
}

// Route-tile height by the average number of routes per expert. Layers take the 256-route tiles of
// the wide kernel from `wide_min_avg` routes per expert on (its cost per tile hardly depends on the
// live routes, and it decodes weights several times faster than the generic kernel). The generic
// kernel (OCO_MOE_NARROW_TILES=1, and the CUDA-core cross-check) picks among its heights: taller
// tiles decode an expert's weights fewer times, shorter ones waste fewer MMA columns on small experts.
int pick_tile_index(int routes, int experts, int wide_min_avg) {
    int avg = routes / (experts > 0 ? experts : 1);
    if (avg >= wide_min_avg) return 3;
    return avg >= 192 ? 3 : (avg >= 96 ? 2 : (avg >= 40 ? 1 : 0));
}

// ---- launch helpers ---------------------------------------------------------------------------
// Opts a kernel into the full 227 KB of dynamic shared memory; each launch then asks for what it needs.
constexpr size_t kMaxDynamicSmem = 232448;
template <typename Kern>
cudaError_t allow_smem(Kern k) {
    cudaFuncAttributes attr;
    cudaError_t e = cudaFuncGetAttributes(&attr, k);
    if (e != cudaSuccess) return e;
    // static and dynamic shared memory share the 227 KB a CTA may opt into
    return cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                (int)(kMaxDynamicSmem - attr.sharedSizeBytes));
}

// Launches a kernel with programmatic stream serialization: it may be scheduled (and, where it does so
// before its griddepcontrol.wait, set up its shared memory and barriers) while its predecessor in the stream
// still runs, and waits for it inside. Every kernel launched this way calls pdl_wait() before it touches
// anything a predecessor wrote or still reads.
template <typename... KArgs, typename... Args>
cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// The same for a kernel that runs in clusters of two CTAs.
template <typename... KArgs, typename... Args>
cudaError_t launch_dependent_pairs(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 2; attr[1].val.clusterDim.y = 1; attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 2;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

template <int FMT, int EPI, int NT>
int launch_gemm(oco_moe_plan* plan, const GemmParams& gp, const CUtensorMap& map, int max_tiles, cudaStream_t st) {
    using S = GemmShape<EPI, NT>;
    dim3 grid((gp.n + 127) / 128, max_tiles);
    if (plan->d.gemm_impl == 1) {
        grouped_gemm_simt_kernel<FMT, EPI, NT><<<grid, 128, 0, st>>>(gp);
    } else {
        ALLOW_SMEM_ONCE((grouped_gemm_tc_kernel<FMT, EPI, NT>));
        grouped_gemm_tc_kernel<FMT, EPI, NT><<<grid, S::kThreads, S::kSmemBytes, st>>>(gp, map);
    }
    plan->launches++;
    CK(cudaGetLastError());
    return OCO_OK;
}

// 256-route tiles take the wide kernel (two A tiles per CTA, coalesced weight streaming); the
// CUDA-core cross-check keeps the generic one.
template <int FMT, int EPI>
int launch_gemm_wide(oco_moe_plan* plan, GemmParams gp, const CUtensorMap* maps, int max_tiles, int experts,
                     cudaStream_t st) {
    // last row of the matrix ends (rows * stride - (stride - packed length)) bytes past its first row
    const size_t bytes = (size_t)experts * gp.n * gp.row_bytes - (gp.row_bytes - packed_row_bytes(FMT, gp.K));
    gp.w0_end = (const uint8_t*)(((uintptr_t)gp.w0 + bytes + 15) & ~(uintptr_t)15);
    gp.w1_end = gp.w1 ? (const uint8_t*)(((uintptr_t)gp.w1 + bytes + 15) & ~(uintptr_t)15) : nullptr;
    if (gp.tile_rows > 256) {
        // SM pairs on route tiles of up to 512 routes: an even, persistent grid of two-CTA clusters
        ALLOW_SMEM_ONCE((grouped_gemm_pair_kernel<FMT, EPI>));
        const int per = epi_gated(EPI) ? 128 : 256;
        const int pairs = std::min(plan->sm_count / 2, ((gp.n + per - 1) / per) * max_tiles);
        CK(launch_dependent_pairs(grouped_gemm_pair_kernel<FMT, EPI>, dim3(2 * pairs), dim3(PairShapeT<FMT>::kThreads), PairShapeT<FMT>::kSmemBytes, st, gp,
                                  maps[0], maps[1], maps[2]));
        plan->launches++;
        CK(cudaGetLastError());
        return OCO_OK;
    }
    ALLOW_SMEM_ONCE((grouped_gemm_wide_kernel<FMT, EPI>));
    // persistent: one CTA per SM walks the (route tile, feature tile) items; never more CTAs than items can exist
    const int feats = (gp.n + (epi_gated(EPI) ? 127 : 255)) / (epi_gated(EPI) ? 128 : 256);
    const int grid = std::min(plan->sm_count, feats * max_tiles);
    // With many items per CTA they are handed out as CTAs become free (two words of the zeroed status block count
    // items and leavers); with few (measured: four per CTA) the fixed deal c, c + grid, ... is as even and cheaper.
    gp.sched = (plan->static_tiles || feats * max_tiles < 5 * grid) ? nullptr : plan->ws.status + 16;
    CK(launch_dependent(grouped_gemm_wide_kernel<FMT, EPI>, dim3(grid), dim3(WideShapeT<FMT>::kThreads), WideShapeT<FMT>::kSmemBytes, st, gp, maps[0], maps[1],
                        maps[2], maps[3]));
    plan->launches++;
    CK(cudaGetLastError());
    return OCO_OK;
}

template <int FMT, int EPI>
int launch_gemm_nt(oco_moe_plan* plan, const GemmParams& gp, const CUtensorMap* maps, int nt_index, int max_tiles,
                   cudaStream_t st) {
    if (nt_index == 3 && plan->d.gemm_impl == 0 && !plan->narrow_tiles)
        return launch_gemm_wide<FMT, EPI>(plan, gp, maps, max_tiles, gp.tiles ? plan->d.experts : 1, st);
    switch (nt_index) {
        case 0: return launch_gemm<FMT, EPI, 32>(plan, gp, maps[0], max_tiles, st);
        case 1: return launch_gemm<FMT, EPI, 64>(plan, gp, maps[1], max_tiles, st);
        case 2: return launch_gemm<FMT, EPI, 128>(plan, gp, maps[2], max_tiles, st);
        default: return launch_gemm<FMT, EPI, 256>(plan, gp, maps[3], max_tiles, st);
    }
}

// Warps per unit of the single-token kernels: as many as keep every warp of the grid busy.
int pick_ksplit(int units, int ctas, int warps_per_cta) {
    for (int k : {10, 8, 5, 4, 2})
        if (warps_per_cta % k == 0 && units * k <= ctas * warps_per_cta) return k;
    return 1;
}

// Ring depth of the single-token kernels by what fits in shared memory (0: nothing fits).

template <int ARCH, int FMT>
int launch_expand(oco_moe_plan* plan, DecodeExpandParams ep, cudaStream_t st) {
    const int grid = plan->sm_count;
    if (token_smem_bytes(FMT, ep.H / 32, 2) > kMaxDynamicSmem) return fail(plan, OCO_UNSUPPORTED_SHAPE, "hidden %d too large for the single-token kernels", ep.H);
    ep.ksplit = pick_ksplit(ep.K * (ep.F / (ARCH == OCO_ARCH_NEMOTRON ? 16 : 8)), grid, tok_warps(FMT));
    ALLOW_SMEM_ONCE((decode_expand_kernel<ARCH, FMT, 2>));
    CK(launch_dependent(decode_expand_kernel<ARCH, FMT, 2>, dim3(grid), dim3(tok_warps(FMT) * 32), token_smem_bytes(FMT, ep.H / 32, 2), st, ep));
    plan->launches++;
    CK(cudaGetLastError());
    return OCO_OK;
}

template <int FMT>
int launch_down(oco_moe_plan* plan, DecodeDownParams dp, cudaStream_t st) {
    const int grid = plan->sm_count;
    if (token_smem_bytes(FMT, dp.F / 32, 2) > kMaxDynamicSmem) return fail(plan, OCO_UNSUPPORTED_SHAPE, "expert width %d too large for the single-token kernels", dp.F);
    if (dp.K > grid) return fail(plan, OCO_UNSUPPORTED_SHAPE, "more routes than multiprocessors");
    dp.ksplit = pick_ksplit(dp.H / 16, grid / dp.K, tok_warps(FMT));
    ALLOW_SMEM_ONCE((decode_down_kernel<FMT, 2>));
    CK(launch_dependent(decode_down_kernel<FMT, 2>, dim3(grid), dim3(tok_warps(FMT) * 32), token_smem_bytes(FMT, dp.F / 32, 2), st, dp));
    plan->launches++;
    CK(cudaGetLastError());
    return OCO_OK;
}

// ---- block-scaled single-token path (mx.cuh) --------------------------------------------------------
// Shapes the path cannot take leave mx_ready false and the mma.sync token kernels run (GPT_OSS / MXFP4 only).
int prepare_mx(oco_moe_plan* plan) {
    plan->mx_ready = false;
    const oco_moe_desc& d = plan->d;
    if (!plan->mx_on || d.arch != OCO_ARCH_GPT_OSS || !plan->have_ws || !plan->have_w || !plan->ws.mx_xb) return OCO_OK;
    const int H = d.hidden, F = d.ffn;
    if (F % 32 || H % 8 || H > 12288 || F > 12288) return OCO_OK;   // 384 tensor-memory columns of operand scales
    // shared memory: the fixed part and the rings of at least one pair of producer warps per matrix
    const int per_cta_up = std::min(16, (d.top_k * (F / 8) + plan->sm_count - 1) / plan->sm_count);
    const int per_cta_dn = std::min(16, (d.top_k * (H / 8) + plan->sm_count - 1) / plan->sm_count);
    if (mx_fixed_smem(2, (uint32_t)(H / 32)) + 16 * mx_ring_bytes(per_cta_up) > kMaxDynamicSmem ||
        mx_fixed_smem(1, (uint32_t)(F / 32)) + 8 * mx_ring_bytes(per_cta_dn) > kMaxDynamicSmem)
        return OCO_OK;
    plan->mx_ready = true;
    return OCO_OK;
}

template <bool EXPAND>
int launch_mx(oco_moe_plan* plan, MxParams mp, cudaStream_t st) {
    const int n_mat = EXPAND ? 2 : 1;
    const int units_total = mp.routes * (mp.rows_per_route / 8);
    const int grid = std::min(plan->sm_count, units_total);
    const uint32_t fixed = mx_fixed_smem(n_mat, (uint32_t)(mp.K / 32));
    // units per pass: a CTA's whole share if it fits the 128 tile rows (16 units)
    mp.pass_units = std::min(16, (units_total + grid - 1) / grid);
    const size_t smem = fixed + (size_t)n_mat * 8 * mx_ring_bytes(mp.pass_units);
    if (smem > kMaxDynamicSmem) return fail(plan, OCO_UNSUPPORTED_SHAPE, "shape too large for the block-scaled token kernels");
    ALLOW_SMEM_ONCE((mx_rows_kernel<EXPAND>));
    CK(launch_dependent(mx_rows_kernel<EXPAND>, dim3(grid), dim3(kMxThreads), smem, st, mp));
    plan->launches++;
    CK(cudaGetLastError());
    return OCO_OK;
}

template <bool EXPAND>
int launch_mx_tma(oco_moe_plan* plan, const MxParams& mp, const MxTmaParams& tp, cudaStream_t st) {
    const int n_mat = EXPAND ? 2 : 1;
    const int tiles_total = mp.routes * tp.row_tiles;
    const int grid = std::min(plan->sm_count, tiles_total);
    const size_t smem = mx_tma_smem(n_mat, (uint32_t)(mp.K / 32));
    ALLOW_SMEM_ONCE((mx_rows_tma_kernel<EXPAND>));
    CK(launch_dependent(mx_rows_tma_kernel<EXPAND>, dim3(grid), dim3(mx_tma_warps(n_mat) * 32), smem, st, mp, tp));
    plan->launches++;
    CK(cudaGetLastError());
    return OCO_OK;
}

template <int ARCH>
struct Family;
template <>
struct Family<OCO_ARCH_GPT_OSS> {
    static constexpr int kFmt = OCO_FMT_MXFP4, kEpiUp = kEpiSwigluF16;
};
template <>
struct Family<OCO_ARCH_NEMOTRON> {
    static constexpr int kFmt = OCO_FMT_Q4_0, kEpiUp = kEpiRelu2F16;
};
template <>
struct Family<OCO_ARCH_QWEN> {
    static constexpr int kFmt = OCO_FMT_Q4_K, kEpiUp = kEpiSiluF16;
};

// ---- single-token path ------------------------------------------------------------------------
// rows == 1 of Bindings::experts (feed_forward.rs:125-163,241-257) and relu_experts_single
// (compute/nemotron.rs:410-545): logits -> (selection fused into) expand -> down -> combine.
template <int ARCH>
int forward_single(oco_moe_plan* plan, const uint16_t* x, uint16_t* residual, cudaStream_t st) {
    constexpr int FMT = Family<ARCH>::kFmt;
    const oco_moe_desc& d = plan->d;
    Workspace& ws = plan->ws;
    const int H = d.hidden, F = d.ffn, E = d.experts, K = d.top_k;
    // logits, then (in the CTA that finishes last) the token's experts and weights
    const bool mx_tma = ARCH == OCO_ARCH_GPT_OSS && plan->rp_token;
    const bool mx = mx_tma || (ARCH == OCO_ARCH_GPT_OSS && plan->mx_ready);
    mark(plan, st, "router_logits");
    CK(launch_dependent(router_token_kernel<ARCH>, dim3((E + 7) / 8), dim3(256), 0, st, x, plan->w.router_w, plan->w.router_b, H, E, K,
                        d.normalize, d.scale, ws.logits, ws.ids, ws.probs, ws.xfrag, (int)FMT, ws.arrivals + H,
                        mx ? ws.mx_xb : nullptr, mx ? ws.mx_xsfb : nullptr));
    plan->launches++;
    if (mx) {
        // MXFP4 rows straight into the block-scaled MMA (mx.cuh): expand with the activation fused, then
        // down with the weighted sum onto the residual by whoever finishes an output-row block last
        auto envelope_end = [](const uint8_t* w, size_t rows, uint32_t stride, uint32_t len) {
            return (const uint8_t*)(((uintptr_t)w + (rows - 1) * stride + len + 15) & ~(uintptr_t)15);
        };
        MxParams ex{};
        ex.w[0] = plan->gate_rows; ex.w[1] = plan->up_rows;
        ex.w_end[0] = envelope_end(plan->gate_rows, (size_t)E * F, plan->up_row_stride, plan->up_row_bytes);
        ex.w_end[1] = envelope_end(plan->up_rows, (size_t)E * F, plan->up_row_stride, plan->up_row_bytes);
        ex.row_stride = plan->up_row_stride; ex.K = H; ex.rows_per_route = F; ex.routes = K; ex.ids = ws.ids;
        ex.b_img = ws.mx_xb; ex.sfb_img = ws.mx_xsfb; ex.b0 = plan->gate_bias; ex.b1 = plan->up_bias; ex.bias_stride = plan->up_bias_stride;
        ex.act_out = ws.act1; ex.act_b = ws.mx_actb; ex.act_sfb = ws.mx_actsfb; ex.blk_arrivals = ws.mx_blk_arrivals;
        ex.act_b_route_bytes = mx_b_bytes(8, (uint32_t)(F / 32)); ex.act_sfb_route_bytes = mx_sfb_bytes((uint32_t)(F / 32));
        ex.status = ws.status;
        mark(plan, st, "expand");
        MxTmaParams tx{}, td{};
        tx.sf[0] = plan->rp_sf[0]; tx.sf[1] = plan->rp_sf[1]; tx.codes[0] = plan->rp_codes[0]; tx.codes[1] = plan->rp_codes[1];
        tx.row_tiles = (F + 127) / 128;
        td.sf[0] = plan->rp_sf[2]; td.codes[0] = plan->rp_codes[2]; td.row_tiles = (H + 127) / 128;
        int rc = mx_tma ? launch_mx_tma<true>(plan, ex, tx, st) : launch_mx<true>(plan, ex, st);
        if (rc) return rc;
        MxParams dn{};
        dn.w[0] = plan->w.down_w; dn.w_end[0] = envelope_end(plan->w.down_w, (size_t)E * H, plan->down_row_bytes, plan->down_row_bytes);
        dn.row_stride = plan->down_row_bytes; dn.K = F; dn.rows_per_route = H; dn.routes = K; dn.ids = ws.ids;
        dn.b_img = ws.mx_actb; dn.sfb_img = ws.mx_actsfb; dn.b_route_bytes = ex.act_b_route_bytes; dn.sfb_route_bytes = ex.act_sfb_route_bytes;
        dn.b0 = plan->w.down_b; dn.bias_stride = 1; dn.y = ws.y; dn.arrivals = ws.arrivals; dn.probs = ws.probs; dn.residual = residual;
        dn.round_sum = 1; dn.status = ws.status;
        mark(plan, st, "down_combine");
        rc = mx_tma ? launch_mx_tma<false>(plan, dn, td, st) : launch_mx<false>(plan, dn, st);
        if (rc) return rc;
        mark(plan, st, "end");
        return OCO_OK;
    }
    {
        auto expand = [&](const uint8_t* gate_w, const uint8_t* up_w, const uint32_t* ids, int k, int f, float* act1,
                          __half* actfrag, uint32_t row_bytes) -> int {
            DecodeExpandParams ep{};
            ep.gate_w = gate_w; ep.up_w = up_w; ep.gate_b = plan->gate_bias; ep.up_b = plan->up_bias;
            ep.bias_stride = plan->up_bias_stride;
            ep.xfrag = ws.xfrag; ep.ids = ids; ep.act = act1; ep.actfrag = actfrag;
            ep.H = H; ep.F = f; ep.K = k; ep.row_bytes = row_bytes; ep.status = ws.status;
            return launch_expand<ARCH, FMT>(plan, ep, st);
        };
        auto down = [&](const uint8_t* down_w, const float* bias, const uint32_t* ids, const __half* actfrag, int k,
                        int f, uint32_t row_bytes, uint16_t* y, bool combine, const uint16_t* shared) -> int {
            DecodeDownParams dp{};
            dp.down_w = down_w; dp.down_b = bias; dp.ids = ids; dp.actfrag = actfrag; dp.y = y;
            if (combine) {
                dp.arrivals = ws.arrivals; dp.probs = ws.probs; dp.residual = residual; dp.shared = shared;
                dp.round_sum = ARCH == OCO_ARCH_GPT_OSS ? 1 : 0;
            }
            dp.H = H; dp.F = f; dp.K = k; dp.row_bytes = row_bytes; dp.status = ws.status;
            return launch_down<FMT>(plan, dp, st);
        };
        mark(plan, st, "expand");
        int rc = expand(plan->gate_rows, plan->up_rows, ws.ids, K, F, ws.act1, ws.actfrag, plan->up_row_stride);
        if (rc) return rc;
        const uint16_t* shared = nullptr;
        if (ARCH == OCO_ARCH_NEMOTRON && d.shared_ffn) {
            // The always-on expert runs through the same kernels as a one-expert bank
            // (compute/nemotron.rs:460-509 runs it as dense matvecs beside the routed ones); its
            // output joins the routed sum in f32 (moe_add with shared = 1).
            mark(plan, st, "shared_expand");
            rc = expand(nullptr, plan->w.shared_up_w, nullptr, 1, d.shared_ffn, ws.sh_act1, ws.sh_actfrag,
                        plan->shared_up_row_bytes);
            if (rc) return rc;
            mark(plan, st, "shared_down");
            rc = down(plan->w.shared_down_w, nullptr, nullptr, ws.sh_actfrag, 1, d.shared_ffn,
                      plan->shared_down_row_bytes, ws.shared_out, false, nullptr);
            if (rc) return rc;
            shared = ws.shared_out;
        }
        // Routed down products; the last warp to finish each block of output rows combines them
        // onto the residual (moe_sum / moe_add), so no separate combine launch is needed.
        mark(plan, st, "down_combine");
        rc = down(plan->w.down_w, plan->w.down_b, ws.ids, ws.actfrag, K, F, plan->down_row_bytes, ws.y, true, shared);
        if (rc) return rc;
        mark(plan, st, "end");
        return OCO_OK;
    }
}

// ---- tiled path ---------------------------------------------------------------------------------
// rows > 1 of Bindings::experts (feed_forward.rs:164-240,258-274) and relu_experts
// (compute/nemotron.rs:294-406): router -> plan -> gather -> up tiles (+activation) -> down tiles
// -> combine. The three stages are also entry points of their own for expert parallelism, where
// an all-to-all sits between them.

// Stage 1: logits, expert ids and combination weights of `rows` tokens into the workspace.
template <int ARCH>
int stage_route(oco_moe_plan* plan, const uint16_t* x, int rows, cudaStream_t st) {
    const oco_moe_desc& d = plan->d;
    Workspace& ws = plan->ws;
    const int H = d.hidden, E = d.experts, K = d.top_k;
    mark(plan, st, "router");
    if (H <= 3072 && H % 4 == 0) {
        const float* rw = plan->w.router_w;
        if (ARCH == OCO_ARCH_GPT_OSS) rw = ws.router_rounded;   // made when the weights were bound (prepare_router)
        ALLOW_SMEM_ONCE((router_stream_kernel<ARCH, 24, 1>));
        if (rows >= plan->router_block_min && H % 8 == 0) {
            // many tokens: four tokens x four experts per warp (router_block_kernel)
            ALLOW_SMEM_ONCE((router_block_kernel<ARCH>));
            const int ctas = (rows + kRouterBlockTokens - 1) / kRouterBlockTokens;
            // one CTA per SM at a time: split the experts over 1, 2, 4 or 8 CTAs per token group so that the
            // last round of CTAs is nearly full (the fewest splits that waste under 5 % of it, else the best)
            int splits = 1;
            double best = 1e9;
            for (int sp = 1; sp <= 8 && E / sp >= kRouterBlockExperts && E % (kRouterBlockExperts * sp) == 0; sp *= 2) {
                const double rounds = (double)ctas * sp / plan->sm_count;
                const double waste = std::ceil(rounds) / rounds;
                if (waste < best - 1e-9) { best = waste; splits = sp; }
                if (waste < 1.05) break;
            }
            CK(launch_dependent(router_block_kernel<ARCH>, dim3(ctas, splits), dim3(kRouterBlockThreads), router_block_smem_bytes(H), st,
                                x, rw, plan->w.router_b, rows, H, E, K, d.normalize, d.scale, ws.logits, ws.ids, ws.probs));
            // the logits of a token are spread over the kernel's warps (and CTAs): the selection is a launch of its own
            CK(launch_dependent(router_select_kernel<ARCH>, dim3(rows), dim3(32), 0, st, ws.logits,
                                ARCH == OCO_ARCH_NEMOTRON ? plan->w.router_b : (const float*)nullptr, E, K, d.normalize, d.scale, ws.ids, ws.probs));
            plan->launches++;
        } else {
            // few tokens: split the experts over several CTAs per token group so that the grid fills the GPU
            const int ctas = (rows + 7) / 8;
            int splits = 1;
            while (splits * 2 * ctas <= plan->sm_count && E / (splits * 2) >= 4) splits *= 2;
            CK(launch_dependent(router_stream_kernel<ARCH, 24, 1>, dim3(ctas, splits), dim3(256), (size_t)6 * H * 4, st,
                                x, rw, plan->w.router_b, rows, H, E, K, d.normalize, d.scale, ws.logits, ws.ids, ws.probs));
            if (splits > 1) {
                CK(launch_dependent(router_select_kernel<ARCH>, dim3(rows), dim3(32), 0, st, ws.logits,
                                    ARCH == OCO_ARCH_NEMOTRON ? plan->w.router_b : (const float*)nullptr, E, K, d.normalize, d.scale, ws.ids, ws.probs));
                plan->launches++;
            }
        }
    } else {
        size_t rsmem = (size_t)H * 4 + (size_t)8 * H * 2;
        ALLOW_SMEM_ONCE((router_batched_kernel<ARCH>));
        router_batched_kernel<ARCH><<<(rows + 7) / 8, 256, rsmem, st>>>(x, plan->w.router_w, plan->w.router_b, rows, H,
                                                                      E, K, d.normalize, d.scale, ws.logits, ws.ids,
                                                                      ws.probs);
    }
    plan->launches++;
    CK(cudaGetLastError());
    return OCO_OK;
}

// How the routes handed to the expert stage are numbered outside it. Route i of the call is labelled
// (i / seg_len) * seg_stride + i % seg_len (seg_len 0: i): its input row is label / per_row, its output
// row is label. `expected` (0: all of them) says how many of the routes carry an expert of this plan,
// for the choice of kernels; the others (ids >= experts) get no row.
struct RouteSpace {
    uint32_t seg_len = 0, seg_stride = 0;
    int expected = 0;
};

// The route plan: one CTA for a few passes' worth of routes, else three many-CTA launches.
void launch_route_plan(oco_moe_plan* plan, const uint32_t* ids, int R, int E, int tile_rows, const RouteSpace& rs, cudaStream_t st) {
    Workspace& ws = plan->ws;
    mark(plan, st, "route_plan");
    if (R <= plan->route_plan_single_max) {
        (void)launch_dependent(route_plan_kernel, dim3(1), dim3(1024), 0, st, ids, (uint32_t)R, (uint32_t)E, (uint32_t)tile_rows, ws.offsets,
                               ws.row_of_route, ws.route_of_row, ws.tiles, ws.tile_count, rs.seg_len, rs.seg_stride);
        plan->launches++;
        return;
    }
    const uint32_t chunks = ((uint32_t)R + 1023u) / 1024u;
    (void)launch_dependent(route_count_kernel, dim3(chunks), dim3(1024), 0, st, ids, (uint32_t)R, (uint32_t)E, ws.row_of_route, ws.chunk_cnt);
    (void)launch_dependent(route_scan_kernel, dim3(1), dim3(1024), 0, st, chunks, (uint32_t)E, (uint32_t)tile_rows, ws.chunk_cnt, ws.offsets, ws.tiles,
                           ws.tile_count);
    (void)launch_dependent(route_scatter_kernel, dim3(chunks), dim3(1024), 0, st, ids, (uint32_t)R, (uint32_t)E, ws.chunk_cnt, ws.offsets, rs.seg_len,
                           rs.seg_stride, ws.row_of_route, ws.route_of_row);
    plan->launches += 3;
}

// Stage 2 in the opt-in block-scaled numerics (oco_moe_desc.numerics = 2): route plan with 128-route tiles,
// the input rows gathered and quantised to MXFP4, up tiles on kind::mxf4 with the activation fused (half rows
// out, as in the reference numerics), those rows quantised, down tiles on kind::mxf4.
int stage_experts_mx(oco_moe_plan* plan, const uint16_t* x, const uint32_t* ids, int R, int per_row, uint16_t* y, cudaStream_t st,
                     const RouteSpace& rs) {
    const oco_moe_desc& d = plan->d;
    Workspace& ws = plan->ws;
    const int H = d.hidden, F = d.ffn, E = d.experts;
    const int NT = plan->rp_ready ? MxrGemmShape::kNT : MxGemmShape::kNT;
    plan->last_tile_rows = NT;
    launch_route_plan(plan, ids, R, E, NT, rs, st);
    const int max_tiles = R / NT + (E < R ? E : R);
    mark(plan, st, "quantize_x");
    mx_quantize_kernel<true><<<4 * max_tiles, 256, 0, st>>>(x, ws.tiles, ws.tile_count, ws.offsets, ws.route_of_row, per_row, H, ws.mxq_x, ws.mxq_xsf, (uint32_t)NT);
    plan->launches += 1;
    CK(cudaGetLastError());
    ALLOW_SMEM_ONCE((grouped_gemm_mx_kernel<kEpiSwigluF16>));
    ALLOW_SMEM_ONCE((grouped_gemm_mx_kernel<kEpiDownBf16>));
    auto envelope_end = [](const uint8_t* w, size_t rows, uint32_t stride, uint32_t len) {
        return (const uint8_t*)(((uintptr_t)w + (rows - 1) * stride + len + 15) & ~(uintptr_t)15);
    };
    GemmParams up{};
    up.w0 = plan->gate_rows; up.w1 = plan->up_rows; up.b0 = plan->gate_bias; up.b1 = plan->up_bias;
    up.n = F; up.K = H; up.row_bytes = plan->up_row_stride; up.bias_stride = plan->up_bias_stride;
    up.tiles = ws.tiles; up.tile_count = ws.tile_count; up.offsets = ws.offsets; up.route_of_row = nullptr;
    up.out = ws.act; up.status = ws.status; up.tile_rows = NT; up.sfb = ws.mxq_xsf;
    up.w0_end = envelope_end(plan->gate_rows, (size_t)E * F, plan->up_row_stride, plan->up_row_bytes);
    up.w1_end = envelope_end(plan->up_rows, (size_t)E * F, plan->up_row_stride, plan->up_row_bytes);
    mark(plan, st, "up_tiles");
    {
        const int feats = (F + 127) / 128, grid = std::min(plan->sm_count, feats * max_tiles);
        if (plan->rp_ready) {
            ALLOW_SMEM_ONCE((grouped_gemm_mxr_kernel<kEpiSwigluF16>));
            up.sfa0 = plan->rp_sf[0]; up.sfa1 = plan->rp_sf[1]; up.sfa_tiles = (F + 127) / 128;
            up.w0 = plan->rp_codes[0]; up.w1 = plan->rp_codes[1];
            grouped_gemm_mxr_kernel<kEpiSwigluF16><<<grid, MxrGemmShape::kThreads, MxrGemmShape::kSmemBytes, st>>>(up, plan->map_mxq_x);
        } else {
            grouped_gemm_mx_kernel<kEpiSwigluF16><<<grid, MxGemmShape::kThreads, MxGemmShape::kSmemBytes, st>>>(up, plan->map_mxq_x);
        }
    }
    mark(plan, st, "quantize_act");
    mx_quantize_kernel<false><<<4 * max_tiles, 256, 0, st>>>(ws.act, ws.tiles, ws.tile_count, ws.offsets, nullptr, 1, F, ws.mxq_act, ws.mxq_actsf, (uint32_t)NT);
    GemmParams dn{};
    dn.w0 = plan->w.down_w; dn.b0 = plan->w.down_b; dn.n = H; dn.K = F; dn.row_bytes = plan->down_row_bytes; dn.bias_stride = 1;
    dn.tiles = ws.tiles; dn.tile_count = ws.tile_count; dn.offsets = ws.offsets; dn.route_of_row = ws.route_of_row;
    dn.out = y; dn.status = ws.status; dn.tile_rows = NT; dn.sfb = ws.mxq_actsf;
    dn.w0_end = envelope_end(plan->w.down_w, (size_t)E * H, plan->down_row_bytes, plan->down_row_bytes);
    mark(plan, st, "down_tiles");
    {
        const int feats = (H + 255) / 256, grid = std::min(plan->sm_count, feats * max_tiles);
        if (plan->rp_ready) {
            ALLOW_SMEM_ONCE((grouped_gemm_mxr_kernel<kEpiDownBf16>));
            dn.sfa0 = plan->rp_sf[2]; dn.sfa1 = plan->rp_sf[2]; dn.sfa_tiles = (H + 127) / 128;
            dn.w0 = plan->rp_codes[2]; dn.w1 = plan->rp_codes[2];
            grouped_gemm_mxr_kernel<kEpiDownBf16><<<grid, MxrGemmShape::kThreads, MxrGemmShape::kSmemBytes, st>>>(dn, plan->map_mxq_act);
        } else {
            grouped_gemm_mx_kernel<kEpiDownBf16><<<grid, MxGemmShape::kThreads, MxGemmShape::kSmemBytes, st>>>(dn, plan->map_mxq_act);
        }
    }
    plan->launches += 3;
    CK(cudaGetLastError());
    return OCO_OK;
}

// Stage 2: expert products of R routes. Route i reads input row i / per_row of x (bf16) and goes
// to expert ids[i]; its bf16 output lands in row i of y.
template <int ARCH>
int stage_experts(oco_moe_plan* plan, const uint16_t* x, const uint32_t* ids, int R, int per_row, uint16_t* y,
                  cudaStream_t st, const RouteSpace& rs = RouteSpace()) {
    constexpr int FMT = Family<ARCH>::kFmt;
    constexpr int EPI_UP = Family<ARCH>::kEpiUp;
    const oco_moe_desc& d = plan->d;
    Workspace& ws = plan->ws;
    const int H = d.hidden, F = d.ffn, E = d.experts;
    const int live = rs.expected > 0 && rs.expected < R ? rs.expected : R;   // routes expected to carry this plan's experts
    if (FMT != OCO_FMT_Q4_K && d.numerics == 0 && live <= plan->batch_max_avg * E && (rs.expected == 0 || R <= 64 * E) && !plan->no_batch_path &&
        batch_smem_bytes(H / 32) <= kMaxDynamicSmem && batch_smem_bytes(F / 32) <= kMaxDynamicSmem) {
        // A few routes per expert: memory-bound, streamed with up to eight routes per MMA (batch.cuh).
        // (Layers too wide for the fragments to sit in shared memory take the tiles.)
        if constexpr (FMT != OCO_FMT_Q4_K) {
            plan->last_tile_rows = kBatchCols;
            launch_route_plan(plan, ids, R, E, kBatchCols, rs, st);
            const int groups = (int)batch_max_groups((size_t)R, (size_t)E);
            mark(plan, st, "fragments");
            batch_fragments_kernel<<<groups, 256, 0, st>>>(x, ws.tiles, ws.tile_count, ws.offsets, ws.route_of_row, per_row,
                                                           H, reinterpret_cast<uint4*>(ws.bfrag_in));
            plan->launches += 1;
            const int parts = std::max(1, std::min(8, (4 * plan->sm_count + groups - 1) / groups));
            ALLOW_SMEM_ONCE((batch_rows_kernel<FMT, EPI_UP>));
            ALLOW_SMEM_ONCE((batch_rows_kernel<FMT, kEpiDownBf16>));
            BatchParams bp{};
            bp.tiles = ws.tiles; bp.tile_count = ws.tile_count; bp.offsets = ws.offsets; bp.route_of_row = ws.route_of_row;
            bp.parts = parts; bp.status = ws.status;
            bp.w0 = ARCH == OCO_ARCH_NEMOTRON ? plan->up_rows : plan->gate_rows;
            bp.w1 = ARCH == OCO_ARCH_NEMOTRON ? nullptr : plan->up_rows;
            bp.b0 = ARCH == OCO_ARCH_GPT_OSS ? plan->gate_bias : nullptr;
            bp.b1 = ARCH == OCO_ARCH_GPT_OSS ? plan->up_bias : nullptr;
            bp.frag_in = ws.bfrag_in; bp.frag_out = ws.bfrag_out; bp.out = ws.act;
            bp.n_in = H; bp.n_out = F; bp.row_bytes = plan->up_row_stride; bp.bias_stride = plan->up_bias_stride;
            mark(plan, st, "up_rows");
            batch_rows_kernel<FMT, EPI_UP><<<groups * parts, kBatchThreads, batch_smem_bytes(H / 32), st>>>(bp);
            bp.w0 = plan->w.down_w; bp.w1 = nullptr;
            bp.b0 = ARCH == OCO_ARCH_GPT_OSS ? plan->w.down_b : nullptr; bp.b1 = nullptr;
            bp.frag_in = ws.bfrag_out; bp.frag_out = nullptr; bp.out = y;
            bp.n_in = F; bp.n_out = H; bp.row_bytes = plan->down_row_bytes; bp.bias_stride = 1;
            mark(plan, st, "down_rows");
            batch_rows_kernel<FMT, kEpiDownBf16><<<groups * parts, kBatchThreads, batch_smem_bytes(F / 32), st>>>(bp);
            plan->launches += 2;
            CK(cudaGetLastError());
            return OCO_OK;
        }
    }
    if constexpr (ARCH == OCO_ARCH_GPT_OSS) {
        if (d.numerics == 2) return stage_experts_mx(plan, x, ids, R, per_row, y, st, rs);
    }
    const int nt_index = pick_tile_index(live, E, plan->narrow_tiles ? 192 : plan->wide_min_avg);
    // SM pairs (grouped_gemm_pair_kernel) take route tiles of up to 512 routes
    const bool pair = plan->pair_tiles && nt_index == 3 && plan->d.gemm_impl == 0 && !plan->narrow_tiles;
    const int NT = pair ? 512 : kTileSizes[nt_index];
    plan->last_tile_rows = NT;
    launch_route_plan(plan, ids, R, E, NT, rs, st);
    mark(plan, st, "permute");
    CK(launch_dependent(permute_rows_kernel, dim3(std::min(R, 16 * plan->sm_count)), dim3(256), 0, st, x, ws.route_of_row, per_row, H,
                        FMT == OCO_FMT_Q4_K ? 32 : 16, ws.xs, (uint32_t)R, ws.offsets + E));
    plan->launches++;
    CK(cudaGetLastError());
    const int max_tiles = R / NT + (E < R ? E : R);

    GemmParams up{};
    up.w0 = ARCH == OCO_ARCH_NEMOTRON ? plan->up_rows : plan->gate_rows;
    up.w1 = ARCH == OCO_ARCH_NEMOTRON ? nullptr : plan->up_rows;
    up.b0 = ARCH == OCO_ARCH_GPT_OSS ? plan->gate_bias : nullptr;
    up.b1 = ARCH == OCO_ARCH_GPT_OSS ? plan->up_bias : nullptr;
    up.n = F; up.K = H; up.row_bytes = plan->up_row_stride; up.bias_stride = plan->up_bias_stride;
    up.tiles = ws.tiles; up.tile_count = ws.tile_count; up.offsets = ws.offsets; up.route_of_row = nullptr;
    up.xs = ws.xs; up.out = ws.act; up.status = ws.status; up.dense_rows = 0; up.tile_rows = NT;
    mark(plan, st, "up_tiles");
    int rc = launch_gemm_nt<FMT, EPI_UP>(plan, up, plan->map_xs, nt_index, max_tiles, st);
    if (rc) return rc;

    GemmParams dn{};
    dn.w0 = plan->w.down_w; dn.w1 = nullptr;
    dn.b0 = ARCH == OCO_ARCH_GPT_OSS ? plan->w.down_b : nullptr; dn.b1 = nullptr;
    dn.n = H; dn.K = F; dn.row_bytes = plan->down_row_bytes; dn.bias_stride = 1;
    dn.tiles = ws.tiles; dn.tile_count = ws.tile_count; dn.offsets = ws.offsets; dn.route_of_row = ws.route_of_row;
    dn.xs = ws.act; dn.out = y; dn.status = ws.status; dn.dense_rows = 0; dn.tile_rows = NT;
    mark(plan, st, "down_tiles");
    return launch_gemm_nt<FMT, kEpiDownBf16>(plan, dn, plan->map_act, nt_index, max_tiles, st);
}

// Stage 3: weighted combine of route-ordered expert outputs onto the residual.
template <int ARCH>
int stage_combine(oco_moe_plan* plan, const uint16_t* y, const float* probs, uint16_t* residual, int rows,
                  int shared_mode, cudaStream_t st, const uint16_t* shared = nullptr) {
    const oco_moe_desc& d = plan->d;
    const size_t pairs = (size_t)rows * d.hidden / 2;
    mark(plan, st, "combine");
    const uint16_t* sh = shared ? shared : plan->ws.shared_out;
    const uint32_t* status = plan->have_ws ? plan->ws.status : nullptr;
    const int round_sum = ARCH == OCO_ARCH_GPT_OSS ? 1 : 0;
    if (d.hidden % 8 == 0 && (((uintptr_t)y | (uintptr_t)residual | (uintptr_t)sh) & 15u) == 0) {
        const size_t octets = pairs / 4;
        const dim3 grid((unsigned)((octets + 255) / 256));
        auto go = [&](auto kernel) {
            return launch_dependent(kernel, grid, dim3(256), 0, st, y, probs, residual, sh, d.hidden, rows, d.top_k, round_sum, shared_mode, status);
        };
        switch (d.top_k) {      // the families' route counts get their loads unrolled
            case 4: CK(go(moe_combine8_kernel<4>)); break;
            case 6: CK(go(moe_combine8_kernel<6>)); break;
            case 8: CK(go(moe_combine8_kernel<8>)); break;
            default: CK(go(moe_combine8_kernel<0>)); break;
        }
    } else {
        moe_combine_kernel<<<(unsigned)((pairs + 255) / 256), 256, 0, st>>>(y, probs, residual, sh, d.hidden, rows, d.top_k, round_sum,
                                                                            shared_mode, status);
    }
    plan->launches++;
    CK(cudaGetLastError());
    return OCO_OK;
}

// residual_ready: an event after which the residual rows may be read (null: they are ready).
template <int ARCH>
int forward_tiled(oco_moe_plan* plan, const uint16_t* x, uint16_t* residual, int rows, cudaStream_t st,
                  cudaEvent_t residual_ready = nullptr) {
    constexpr int FMT = Family<ARCH>::kFmt;
    const oco_moe_desc& d = plan->d;
    Workspace& ws = plan->ws;
    const int H = d.hidden, K = d.top_k;
    int rc = stage_route<ARCH>(plan, x, rows, st);
    if (rc) return rc;
    rc = stage_experts<ARCH>(plan, x, ws.ids, rows * K, K, ws.y, st);
    if (rc) return rc;
    int shared_mode = 0;
    if (ARCH == OCO_ARCH_NEMOTRON && d.shared_ffn) {
        // Shared expert as dense tiles over all rows: up -> relu^2 (bf16) -> down, joined to the
        // residual as a bf16 add ahead of the routed sum (compute/nemotron.rs:302-316).
        const int S = d.shared_ffn;
        mark(plan, st, "shared_expert");
        permute_rows_kernel<<<std::min(rows, 16 * plan->sm_count), 256, 0, st>>>(x, nullptr, 1, H, FMT == OCO_FMT_Q4_K ? 32 : 16, ws.xh,
                                                                              (uint32_t)rows, nullptr);  // identity gather
        plan->launches++;
        const int snt = pick_tile_index(rows, 1, plan->narrow_tiles ? 192 : plan->wide_min_avg);
        const int SNT = kTileSizes[snt];
        GemmParams su{};
        su.w0 = plan->w.shared_up_w; su.n = S; su.K = H; su.row_bytes = plan->shared_up_row_bytes; su.bias_stride = 1;
        su.xs = ws.xh; su.out = ws.mid; su.status = ws.status; su.dense_rows = rows; su.tile_rows = SNT;
        rc = launch_gemm_nt<FMT, kEpiRelu2Bf16F16>(plan, su, plan->map_xh, snt, (rows + SNT - 1) / SNT, st);
        if (rc) return rc;
        GemmParams sd{};
        sd.w0 = plan->w.shared_down_w; sd.n = H; sd.K = S; sd.row_bytes = plan->shared_down_row_bytes; sd.bias_stride = 1;
        sd.xs = ws.mid; sd.out = ws.shared_out; sd.status = ws.status; sd.dense_rows = rows; sd.tile_rows = SNT;
        rc = launch_gemm_nt<FMT, kEpiDownBf16>(plan, sd, plan->map_mid, snt, (rows + SNT - 1) / SNT, st);
        if (rc) return rc;
        shared_mode = 2;
    }
    if (residual_ready) CK(cudaStreamWaitEvent(st, residual_ready, 0));
    rc = stage_combine<ARCH>(plan, ws.y, ws.probs, residual, rows, shared_mode, st);
    if (rc) return rc;
    mark(plan, st, "end");
    return OCO_OK;
}

template <int ARCH>
int forward_family(oco_moe_plan* plan, const uint16_t* x, uint16_t* residual, int rows, cudaStream_t st,
                   cudaEvent_t residual_ready = nullptr) {
    constexpr int FMT = Family<ARCH>::kFmt;
    const oco_moe_desc& d = plan->d;
    // The single-token kernels keep the token's (and each route's) MMA fragments in shared memory beside
    // their rings; layers too wide for that take the tile kernels, which have no such limit.
    const int widest = std::max(d.hidden, std::max(d.ffn, d.shared_ffn));
    if (rows == 1 && token_smem_bytes(FMT, widest / 32, 2) <= kMaxDynamicSmem) {
        if (residual_ready) CK(cudaStreamWaitEvent(st, residual_ready, 0));
        return forward_single<ARCH>(plan, x, residual, st);
    }
    return forward_tiled<ARCH>(plan, x, residual, rows, st, residual_ready);
}

// The gpt-oss router multiplies with its weights rounded to bf16 (reference routing.metal:131-146 reads
// bf16 router rows). The rounded copy is made here, as soon as both the router weights and the
// workspace are bound, and waited for, so that no later call, captured or on whatever stream, can
// meet a half-made copy.
int prepare_router(oco_moe_plan* plan) {
    if (plan->router_ready || !plan->have_ws || !plan->w.router_w) return OCO_OK;
    if (plan->d.arch == OCO_ARCH_GPT_OSS && plan->d.hidden <= 3072 && plan->d.hidden % 4 == 0) {
        const size_t n = (size_t)plan->d.experts * plan->d.hidden;
        round_router_kernel<<<(unsigned)((n + 255) / 256), 256, 0, cudaStreamPerThread>>>(plan->w.router_w, plan->ws.router_rounded, n);
        CK(cudaGetLastError());
        CK(cudaStreamSynchronize(cudaStreamPerThread));
    }
    plan->router_ready = true;
    return OCO_OK;
}

// Calls must be made with the device current on which the workspace was bound.
int check_device(oco_moe_plan* plan) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev != plan->device)
        return fail(plan, OCO_INVALID_ARGUMENT, "the plan's workspace was bound on device %d, the current device is %d", plan->device, dev);
    return OCO_OK;
}

int forward_any(oco_moe_plan* plan, const uint16_t* x, uint16_t* residual, int rows, cudaStream_t st,
                cudaEvent_t residual_ready) {
    plan->launches = 0;
    plan->n_marks = 0;
    switch (plan->d.arch) {
        case OCO_ARCH_GPT_OSS: return forward_family<OCO_ARCH_GPT_OSS>(plan, x, residual, rows, st, residual_ready);
        case OCO_ARCH_NEMOTRON: return forward_family<OCO_ARCH_NEMOTRON>(plan, x, residual, rows, st, residual_ready);
        default: return forward_family<OCO_ARCH_QWEN>(plan, x, residual, rows, st, residual_ready);
    }
}

}  // namespace

// =================================================================================================
extern "C" {

const char* oco_moe_version(void) { return "oco-moe-b200 0.1 (sm_100a)"; }

int oco_moe_plan_create(const oco_moe_desc* desc, oco_moe_plan** out) {
    if (!desc || !out) return OCO_INVALID_ARGUMENT;
    *out = nullptr;
    oco_moe_plan* plan = new (std::nothrow) oco_moe_plan();
    if (!plan) return OCO_INVALID_ARGUMENT;
    plan->d = *desc;
    *out = plan;  // handed out even on failure so the caller can read the message, then destroy
    const oco_moe_desc& d = plan->d;
    if (d.arch < OCO_ARCH_GPT_OSS || d.arch > OCO_ARCH_QWEN) return fail(plan, OCO_INVALID_ARGUMENT, "unknown arch %d", d.arch);
    const int want = d.arch == OCO_ARCH_GPT_OSS ? OCO_FMT_MXFP4 : (d.arch == OCO_ARCH_NEMOTRON ? OCO_FMT_Q4_0 : OCO_FMT_Q4_K);
    if (d.weight_format != want)
        return fail(plan, OCO_UNSUPPORTED_SHAPE, "arch %d is built for weight format %d, got %d", d.arch, want, d.weight_format);
    if (d.experts < 1 || d.experts > kMaxExperts) return fail(plan, OCO_UNSUPPORTED_SHAPE, "experts must be 1..128");
    // (a plan over a shard of the experts may hold fewer experts than routes per token: it never routes)
    if (d.top_k < 1 || d.top_k > kMaxTopK) return fail(plan, OCO_UNSUPPORTED_SHAPE, "top_k must be 1..8");
    const int be = block_elems(d.weight_format);
    if (d.hidden <= 0 || d.ffn <= 0 || d.hidden % be || d.ffn % be || (d.shared_ffn % be))
        return fail(plan, OCO_UNSUPPORTED_SHAPE, "hidden, ffn and shared_ffn must be multiples of the %d-element block", be);
    if (d.hidden % 32 || d.ffn % 32) return fail(plan, OCO_UNSUPPORTED_SHAPE, "hidden and ffn must be multiples of 32");
    if (d.shared_ffn && d.arch != OCO_ARCH_NEMOTRON) return fail(plan, OCO_UNSUPPORTED_SHAPE, "shared expert only with NEMOTRON");
    if (d.gemm_impl != 0 && d.gemm_impl != 1) return fail(plan, OCO_INVALID_ARGUMENT, "gemm_impl must be 0 or 1");
    if (d.numerics != 0 && d.numerics != 2) return fail(plan, OCO_INVALID_ARGUMENT, "numerics must be 0 (reference) or 2 (MXFP4 activations)");
    if (d.numerics == 2 && (d.arch != OCO_ARCH_GPT_OSS || d.gemm_impl != 0 || d.hidden % 32 || d.ffn % 32))
        return fail(plan, OCO_UNSUPPORTED_SHAPE, "numerics 2 runs the MXFP4 family on the tensor-core tiles only");
    plan->up_row_bytes = packed_row_bytes(d.weight_format, d.hidden);
    plan->down_row_bytes = packed_row_bytes(d.weight_format, d.ffn);
    if (d.shared_ffn) {
        plan->shared_up_row_bytes = packed_row_bytes(d.weight_format, d.hidden);
        plan->shared_down_row_bytes = packed_row_bytes(d.weight_format, d.shared_ffn);
    }
    { const char* e = getenv("OCO_MOE_NARROW_TILES"); plan->narrow_tiles = e && e[0] == '1'; }
    { const char* e = getenv("OCO_MOE_WIDE_MIN_AVG"); if (e && atoi(e) > 0) plan->wide_min_avg = atoi(e); }
    { const char* e = getenv("OCO_MOE_STATIC_TILES"); if (e) plan->static_tiles = atoi(e) != 0; }
    { const char* e = getenv("OCO_MOE_PAIR_TILES"); if (e) plan->pair_tiles = atoi(e) != 0; }
    { const char* e = getenv("OCO_MOE_ROUTER_BLOCK_MIN"); if (e && atoi(e) > 0) plan->router_block_min = atoi(e); }
    { const char* e = getenv("OCO_MOE_NO_BATCH"); plan->no_batch_path = e && e[0] == '1'; }
    { const char* e = getenv("OCO_MOE_TOKEN_MX"); plan->mx_on = e && e[0] == '1'; }
    { const char* e = getenv("OCO_MOE_ROUTE_PLAN_SINGLE_MAX"); if (e && atoi(e) >= 0) plan->route_plan_single_max = atoi(e); }
    { const char* e = getenv("OCO_MOE_REPACKED_TOKEN"); plan->rp_token_on = e && e[0] == '1'; }
    { const char* e = getenv("OCO_MOE_BATCH_MAX_AVG"); if (e && atoi(e) > 0) plan->batch_max_avg = atoi(e) < 64 ? atoi(e) : 64; }
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) == cudaSuccess &&
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && sms > 0)
        plan->sm_count = sms;
    (void)cudaGetLastError();
    return OCO_OK;
}

void oco_moe_plan_destroy(oco_moe_plan* plan) {
    if (!plan) return;
    while (plan->host_begun != plan->host_ended)        // host calls still in flight: their rows come back first
        if (oco_moe_forward_host_end(plan) != OCO_OK) break;
    for (int i = 0; i < kMaxMarks; i++)
        if (plan->marks[i]) cudaEventDestroy(plan->marks[i]);
    for (int i = 0; i < 2; i++) {
        if (plan->ev_x[i]) cudaEventDestroy(plan->ev_x[i]);
        if (plan->ev_res[i]) cudaEventDestroy(plan->ev_res[i]);
        if (plan->ev_done[i]) cudaEventDestroy(plan->ev_done[i]);
        if (plan->ev_out[i]) cudaEventDestroy(plan->ev_out[i]);
    }
    if (plan->in_stream) cudaStreamDestroy(plan->in_stream);
    if (plan->out_stream) cudaStreamDestroy(plan->out_stream);
    delete plan;
}

int oco_moe_set_profiling(oco_moe_plan* plan, int enabled) {
    if (!plan) return OCO_INVALID_ARGUMENT;
    plan->profiling = enabled != 0;
    plan->n_marks = 0;
    return OCO_OK;
}

int oco_moe_phase_times(oco_moe_plan* plan, int capacity, float* ms, const char** names) {
    if (!plan || capacity < 0) return -1;
    int phases = plan->n_marks > 0 ? plan->n_marks - 1 : 0;
    for (int i = 0; i < phases && i < capacity; i++) {
        float t = 0.f;
        if (cudaEventElapsedTime(&t, plan->marks[i], plan->marks[i + 1]) != cudaSuccess) t = -1.f;
        if (ms) ms[i] = t;
        if (names) names[i] = plan->mark_names[i];
    }
    return phases;
}

size_t oco_moe_workspace_bytes(const oco_moe_plan* plan, int max_rows) {
    if (!plan || max_rows < 1) return 0;
    return carve(plan->d, max_rows, nullptr).total;
}

int oco_moe_bind_workspace(oco_moe_plan* plan, void* workspace, size_t bytes, int max_rows) {
    if (!plan || !workspace || max_rows < 1) return fail(plan, OCO_INVALID_ARGUMENT, "null workspace or max_rows < 1");
    if (((uintptr_t)workspace & 255u) != 0) return fail(plan, OCO_INVALID_ARGUMENT, "workspace must be 256-byte aligned");
    Workspace ws = carve(plan->d, max_rows, (unsigned char*)workspace);
    if (bytes < ws.total) return fail(plan, OCO_INVALID_ARGUMENT, "workspace too small: %zu < %zu", bytes, ws.total);
    const oco_moe_desc& d = plan->d;
    // Control words and the never-written columns of the single-token fragments start at zero.
    CK(cudaMemset(ws.status, 0, 256));
    CK(cudaMemset(ws.actfrag, 0, (size_t)((d.top_k + 1) / 2) * (d.ffn / 32) * 128 * 2));
    CK(cudaMemset(ws.arrivals, 0, (size_t)(d.hidden + 1) * 4));
    if (ws.mx_actb) {
        // blocks past the end of a row stay zero for good; the counters are left at zero by every call
        CK(cudaMemset(ws.mx_actb, 0, (size_t)d.top_k * mx_b_bytes(8, (uint32_t)(d.ffn / 32))));
        CK(cudaMemset(ws.mx_actsfb, 0, (size_t)d.top_k * mx_sfb_bytes((uint32_t)(d.ffn / 32))));
        CK(cudaMemset(ws.mx_blk_arrivals, 0, (size_t)d.top_k * (d.ffn / 32) * 4));
    }
    if (d.shared_ffn) {
        CK(cudaMemset(ws.sh_actfrag, 0, (size_t)(d.shared_ffn / 32) * 128 * 2));
        CK(cudaMemset(ws.sh_ids, 0, 256));
    }
    const uint64_t R = (uint64_t)max_rows * d.top_k;
    for (int i = 0; i < kTileKinds; i++) {
        int rc = make_row_map(plan, &plan->map_xs[i], ws.xs, R, d.hidden, kTileSizes[i]);
        if (rc) return rc;
        rc = make_row_map(plan, &plan->map_act[i], ws.act, R, d.ffn, kTileSizes[i]);
        if (rc) return rc;
        if (d.shared_ffn) {
            rc = make_row_map(plan, &plan->map_xh[i], ws.xh, max_rows, d.hidden, kTileSizes[i]);
            if (rc) return rc;
            rc = make_row_map(plan, &plan->map_mid[i], ws.mid, max_rows, d.shared_ffn, kTileSizes[i]);
            if (rc) return rc;
        }
    }
    if (d.numerics == 2) {
        int rc = make_byte_map(plan, &plan->map_mxq_x, ws.mxq_x, R, (uint64_t)d.hidden / 2, 128);
        if (rc) return rc;
        rc = make_byte_map(plan, &plan->map_mxq_act, ws.mxq_act, R, (uint64_t)d.ffn / 2, 128);
        if (rc) return rc;
    }
    CK(cudaDeviceSynchronize());
    int dev = 0, sms = 0;
    CK(cudaGetDevice(&dev));
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && sms > 0) plan->sm_count = sms;
    plan->device = dev;
    plan->ws = ws;
    plan->max_rows = max_rows;
    plan->have_ws = true;
    plan->router_ready = false;
    if (int rc_r = prepare_router(plan)) return rc_r;
    return prepare_mx(plan);
}

int oco_moe_bind_weights(oco_moe_plan* plan, const oco_moe_weights* w) {
    if (!plan || !w) return fail(plan, OCO_INVALID_ARGUMENT, "null weights");
    const oco_moe_desc& d = plan->d;
    // A plan may hold only a router (it then serves oco_moe_route), only experts (oco_moe_experts),
    // or both (oco_moe_forward needs both).
    plan->rp_ready = plan->rp_token = false;      // a repacked form belongs to the weights it was made from
    const bool has_router = w->router_w != nullptr;
    const bool interleaved = w->gate_up_w != nullptr;
    const bool has_experts = w->up_w != nullptr || w->down_w != nullptr || w->gate_w != nullptr || interleaved;
    if (!has_router && !has_experts) return fail(plan, OCO_INVALID_ARGUMENT, "no weights given");
    if (has_experts) {
        if (interleaved) {
            if (d.arch == OCO_ARCH_NEMOTRON) return fail(plan, OCO_INVALID_ARGUMENT, "gate_up_w given for a family without a gate");
            if (w->gate_w || w->up_w) return fail(plan, OCO_INVALID_ARGUMENT, "give gate_up_w or gate_w + up_w, not both");
            if (!w->down_w) return fail(plan, OCO_INVALID_ARGUMENT, "down_w is required");
            if (d.arch == OCO_ARCH_GPT_OSS && (!w->gate_up_b || !w->down_b))
                return fail(plan, OCO_INVALID_ARGUMENT, "GPT_OSS with gate_up_w needs gate_up_b and down_b");
        } else {
            if (!w->up_w || !w->down_w) return fail(plan, OCO_INVALID_ARGUMENT, "up_w and down_w are required");
            if (d.arch != OCO_ARCH_NEMOTRON && !w->gate_w) return fail(plan, OCO_INVALID_ARGUMENT, "gate_w is required for gated experts");
            if (d.arch == OCO_ARCH_GPT_OSS && (!w->gate_b || !w->up_b || !w->down_b))
                return fail(plan, OCO_INVALID_ARGUMENT, "GPT_OSS needs gate, up and down biases");
        }
        if (d.shared_ffn && (!w->shared_up_w || !w->shared_down_w)) return fail(plan, OCO_INVALID_ARGUMENT, "shared expert weights missing");
    }
    if (has_router) {
        if (d.top_k > d.experts) return fail(plan, OCO_UNSUPPORTED_SHAPE, "a router over %d experts cannot pick %d", d.experts, d.top_k);
        if (d.arch != OCO_ARCH_QWEN && !w->router_b) return fail(plan, OCO_INVALID_ARGUMENT, "this family needs router_b");
        if (((uintptr_t)w->router_w & 15u) != 0) return fail(plan, OCO_INVALID_ARGUMENT, "router_w must be 16-byte aligned");
    }
    plan->w = *w;
    if (interleaved) {
        // row 2c = gate row c, row 2c + 1 = up row c; the biases likewise
        plan->gate_rows = w->gate_up_w;
        plan->up_rows = w->gate_up_w + plan->up_row_bytes;
        plan->up_row_stride = 2 * plan->up_row_bytes;
        plan->gate_bias = w->gate_up_b;
        plan->up_bias = w->gate_up_b ? w->gate_up_b + 1 : nullptr;
        plan->up_bias_stride = 2;
    } else {
        plan->gate_rows = w->gate_w;
        plan->up_rows = w->up_w;
        plan->up_row_stride = plan->up_row_bytes;
        plan->gate_bias = w->gate_b;
        plan->up_bias = w->up_b;
        plan->up_bias_stride = 1;
    }
    plan->have_w = has_router && has_experts;
    plan->have_experts = has_experts;
    plan->router_ready = false;
    if (int rc_r = prepare_router(plan)) return rc_r;
    return prepare_mx(plan);
}

int oco_moe_forward(oco_moe_plan* plan, const uint16_t* x, uint16_t* residual, int rows, void* cuda_stream) {
    if (!plan) return OCO_INVALID_ARGUMENT;
    if (!plan->have_ws || !plan->have_w) return fail(plan, OCO_INVALID_ARGUMENT, "bind a workspace and weights first");
    if (int rc_dev = check_device(plan)) return rc_dev;
    if (!x || !residual) return fail(plan, OCO_INVALID_ARGUMENT, "null x or residual");
    if (rows < 1 || rows > plan->max_rows) return fail(plan, OCO_INVALID_ARGUMENT, "rows %d outside 1..%d", rows, plan->max_rows);
    if (((uintptr_t)x & 15u) || ((uintptr_t)residual & 15u)) return fail(plan, OCO_INVALID_ARGUMENT, "x and residual must be 16-byte aligned");
    cudaStream_t st = (cudaStream_t)cuda_stream;
    plan->launches = 0;
    plan->n_marks = 0;
    switch (plan->d.arch) {
        case OCO_ARCH_GPT_OSS: return forward_family<OCO_ARCH_GPT_OSS>(plan, x, residual, rows, st);
        case OCO_ARCH_NEMOTRON: return forward_family<OCO_ARCH_NEMOTRON>(plan, x, residual, rows, st);
        default: return forward_family<OCO_ARCH_QWEN>(plan, x, residual, rows, st);
    }
}

// ---- stages as entry points (expert parallelism puts an all-to-all between them) ---------------
int oco_moe_add_norm_forward(oco_moe_plan* plan, uint16_t* hidden, const uint16_t* projected, const float* norm_weight,
                             float epsilon, int full_layer, int rows, void* cuda_stream) {
    if (!plan) return OCO_INVALID_ARGUMENT;
    if (!plan->have_ws || !plan->have_w) return fail(plan, OCO_INVALID_ARGUMENT, "bind a workspace and weights first");
    if (int rc_dev = check_device(plan)) return rc_dev;
    if (!hidden || !norm_weight) return fail(plan, OCO_INVALID_ARGUMENT, "null hidden rows or norm weight");
    if (rows < 1 || rows > plan->max_rows) return fail(plan, OCO_INVALID_ARGUMENT, "rows %d outside 1..%d", rows, plan->max_rows);
    if (((uintptr_t)hidden & 15u) || ((uintptr_t)projected & 15u)) return fail(plan, OCO_INVALID_ARGUMENT, "rows must be 16-byte aligned");
    cudaStream_t st = (cudaStream_t)cuda_stream;
    plan->launches = 0;
    plan->n_marks = 0;
    mark(plan, st, "add_norm");
    add_norm_kernel<<<rows, 256, 0, st>>>(hidden, projected, norm_weight, plan->ws.norm, plan->d.hidden, epsilon, full_layer);
    CK(cudaGetLastError());
    int launches = 1;
    int rc;
    switch (plan->d.arch) {   // the layer itself; its own launch count is added to the norm's
        case OCO_ARCH_GPT_OSS: rc = forward_family<OCO_ARCH_GPT_OSS>(plan, plan->ws.norm, hidden, rows, st); break;
        case OCO_ARCH_NEMOTRON: rc = forward_family<OCO_ARCH_NEMOTRON>(plan, plan->ws.norm, hidden, rows, st); break;
        default: rc = forward_family<OCO_ARCH_QWEN>(plan, plan->ws.norm, hidden, rows, st); break;
    }
    plan->launches += launches;
    return rc;
}

int oco_moe_route(oco_moe_plan* plan, const uint16_t* x, int rows, void* cuda_stream) {
    if (!plan) return OCO_INVALID_ARGUMENT;
    if (!plan->have_ws || !plan->w.router_w) return fail(plan, OCO_INVALID_ARGUMENT, "bind a workspace and router weights first");
    if (int rc_dev = check_device(plan)) return rc_dev;
    if (!x || rows < 1 || rows > plan->max_rows) return fail(plan, OCO_INVALID_ARGUMENT, "bad x or rows");
    cudaStream_t st = (cudaStream_t)cuda_stream;
    plan->launches = 0;
    plan->n_marks = 0;
    int rc;
    switch (plan->d.arch) {
        case OCO_ARCH_GPT_OSS: rc = stage_route<OCO_ARCH_GPT_OSS>(plan, x, rows, st); break;
        case OCO_ARCH_NEMOTRON: rc = stage_route<OCO_ARCH_NEMOTRON>(plan, x, rows, st); break;
        default: rc = stage_route<OCO_ARCH_QWEN>(plan, x, rows, st); break;
    }
    mark(plan, st, "end");
    return rc;
}

int oco_moe_experts(oco_moe_plan* plan, const uint16_t* rows_bf16, const uint32_t* expert_ids, int routes,
                    uint16_t* y_bf16, void* cuda_stream) {
    if (!plan) return OCO_INVALID_ARGUMENT;
    if (!plan->have_ws || !plan->have_experts) return fail(plan, OCO_INVALID_ARGUMENT, "bind a workspace and expert weights first");
    if (int rc_dev = check_device(plan)) return rc_dev;
    if (routes == 0) return OCO_OK;
    if (!rows_bf16 || !expert_ids || !y_bf16 || routes < 0 || routes > plan->max_rows * plan->d.top_k)
        return fail(plan, OCO_INVALID_ARGUMENT, "bad buffers, or more routes than max_rows * top_k");
    cudaStream_t st = (cudaStream_t)cuda_stream;
    plan->launches = 0;
    plan->n_marks = 0;
    int rc;
    switch (plan->d.arch) {
        case OCO_ARCH_GPT_OSS: rc = stage_experts<OCO_ARCH_GPT_OSS>(plan, rows_bf16, expert_ids, routes, 1, y_bf16, st); break;
        case OCO_ARCH_NEMOTRON: rc = stage_experts<OCO_ARCH_NEMOTRON>(plan, rows_bf16, expert_ids, routes, 1, y_bf16, st); break;
        default: rc = stage_experts<OCO_ARCH_QWEN>(plan, rows_bf16, expert_ids, routes, 1, y_bf16, st); break;
    }
    mark(plan, st, "end");
    return rc;
}

int oco_moe_experts_window(oco_moe_plan* plan, const uint16_t* token_rows_bf16, const uint32_t* expert_ids, int routes,
                           int routes_per_row, int seg_routes, int seg_stride, int expected_routes, uint16_t* y_bf16,
                           void* cuda_stream) {
    if (!plan) return OCO_INVALID_ARGUMENT;
    if (!plan->have_ws || !plan->have_experts) return fail(plan, OCO_INVALID_ARGUMENT, "bind a workspace and expert weights first");
    if (int rc_dev = check_device(plan)) return rc_dev;
    if (routes == 0) return OCO_OK;
    if (!token_rows_bf16 || !expert_ids || !y_bf16 || routes < 0 || routes > plan->max_rows * plan->d.top_k)
        return fail(plan, OCO_INVALID_ARGUMENT, "bad buffers, or more routes than max_rows * top_k");
    if (routes_per_row < 1 || seg_routes < 0 || expected_routes < 0 || (seg_routes && seg_stride < seg_routes) ||
        (seg_routes && seg_stride % routes_per_row))
        return fail(plan, OCO_INVALID_ARGUMENT, "bad route numbering: the segment stride must hold a segment and whole token rows");
    if (seg_routes && ((uint64_t)((routes - 1) / seg_routes) * (uint64_t)seg_stride + (uint64_t)seg_routes) > 0xffffffffull)
        return fail(plan, OCO_UNSUPPORTED_SHAPE, "route labels exceed 32 bits");
    cudaStream_t st = (cudaStream_t)cuda_stream;
    plan->launches = 0;
    plan->n_marks = 0;
    RouteSpace rs;
    rs.seg_len = (uint32_t)seg_routes; rs.seg_stride = (uint32_t)seg_stride; rs.expected = expected_routes ? expected_routes : routes;
    int rc;
    switch (plan->d.arch) {
        case OCO_ARCH_GPT_OSS: rc = stage_experts<OCO_ARCH_GPT_OSS>(plan, token_rows_bf16, expert_ids, routes, routes_per_row, y_bf16, st, rs); break;
        case OCO_ARCH_NEMOTRON: rc = stage_experts<OCO_ARCH_NEMOTRON>(plan, token_rows_bf16, expert_ids, routes, routes_per_row, y_bf16, st, rs); break;
        default: rc = stage_experts<OCO_ARCH_QWEN>(plan, token_rows_bf16, expert_ids, routes, routes_per_row, y_bf16, st, rs); break;
    }
    mark(plan, st, "end");
    return rc;
}

int oco_moe_combine(oco_moe_plan* plan, const uint16_t* y_bf16, const float* probs, uint16_t* residual_bf16, int rows,
                    void* cuda_stream) {
    if (!plan) return OCO_INVALID_ARGUMENT;
    if (!y_bf16 || !probs || !residual_bf16 || rows < 1) return fail(plan, OCO_INVALID_ARGUMENT, "bad buffers or rows");
    cudaStream_t st = (cudaStream_t)cuda_stream;
    plan->launches = 0;
    plan->n_marks = 0;
    int rc;
    switch (plan->d.arch) {
        case OCO_ARCH_GPT_OSS: rc = stage_combine<OCO_ARCH_GPT_OSS>(plan, y_bf16, probs, residual_bf16, rows, 0, st); break;
        case OCO_ARCH_NEMOTRON: rc = stage_combine<OCO_ARCH_NEMOTRON>(plan, y_bf16, probs, residual_bf16, rows, 0, st); break;
        default: rc = stage_combine<OCO_ARCH_QWEN>(plan, y_bf16, probs, residual_bf16, rows, 0, st); break;
    }
    mark(plan, st, "end");
    return rc;
}

int oco_moe_combine_shared(oco_moe_plan* plan, const uint16_t* y_bf16, const float* probs, const uint16_t* shared_bf16,
                           uint16_t* residual_bf16, int rows, void* cuda_stream) {
    if (!plan) return OCO_INVALID_ARGUMENT;
    if (!y_bf16 || !probs || !shared_bf16 || !residual_bf16 || rows < 1) return fail(plan, OCO_INVALID_ARGUMENT, "bad buffers or rows");
    if (plan->d.arch != OCO_ARCH_NEMOTRON) return fail(plan, OCO_UNSUPPORTED_SHAPE, "only the NEMOTRON family has an always-on expert");
    cudaStream_t st = (cudaStream_t)cuda_stream;
    plan->launches = 0;
    plan->n_marks = 0;
    int rc = stage_combine<OCO_ARCH_NEMOTRON>(plan, y_bf16, probs, residual_bf16, rows, 2, st, shared_bf16);
    mark(plan, st, "end");
    return rc;
}

// Sizes of the repacked form of one tensor of `n` rows per expert and rows of K elements.
static size_t rp_codes_bytes(const oco_moe_desc& d, int n, int K) { return (size_t)d.experts * ((n + 127) / 128) * (((K >> 5) + 7) >> 3) * 16384; }
static size_t rp_sf_bytes(const oco_moe_desc& d, int n, int K) {
    return (size_t)d.experts * ((n + 127) / 128) * (((K >> 5) + 7) >> 3) * 1024;
}

size_t oco_moe_repack_bytes(const oco_moe_plan* plan) {
    if (!plan || plan->d.arch != OCO_ARCH_GPT_OSS) return 0;
    const oco_moe_desc& d = plan->d;
    return 2 * (rp_codes_bytes(d, d.ffn, d.hidden) + rp_sf_bytes(d, d.ffn, d.hidden)) + rp_codes_bytes(d, d.hidden, d.ffn) +
           rp_sf_bytes(d, d.hidden, d.ffn);
}

int oco_moe_bind_repacked(oco_moe_plan* plan, void* buffer, size_t bytes, void* cuda_stream) {
    if (!plan) return OCO_INVALID_ARGUMENT;
    const oco_moe_desc& d = plan->d;
    if (d.arch != OCO_ARCH_GPT_OSS) return fail(plan, OCO_UNSUPPORTED_SHAPE, "repacked weights serve the MXFP4 family only");
    if (!plan->have_experts) return fail(plan, OCO_INVALID_ARGUMENT, "bind the expert weights first");
    if (int rc_dev = check_device(plan)) return rc_dev;
    if (!buffer) { plan->rp_ready = plan->rp_token = false; return OCO_OK; }                      // back to the weights as stored
    if (((uintptr_t)buffer & 1023u) != 0) return fail(plan, OCO_INVALID_ARGUMENT, "the buffer must be 1024-byte aligned");
    if (bytes < oco_moe_repack_bytes(plan)) return fail(plan, OCO_INVALID_ARGUMENT, "buffer too small: %zu < %zu", bytes, oco_moe_repack_bytes(plan));
    cudaStream_t st = (cudaStream_t)cuda_stream;
    const int H = d.hidden, F = d.ffn, E = d.experts;
    unsigned char* at = (unsigned char*)buffer;
    const uint8_t* src[3] = {plan->gate_rows, plan->up_rows, plan->w.down_w};
    const size_t stride[3] = {plan->up_row_stride, plan->up_row_stride, plan->down_row_bytes};
    const int n[3] = {F, F, H}, K[3] = {H, H, F};
    for (int t = 0; t < 3; t++) {
        plan->rp_codes[t] = at; at += rp_codes_bytes(d, n[t], K[t]);
        plan->rp_sf[t] = at; at += rp_sf_bytes(d, n[t], K[t]);
        CK(cudaMemsetAsync(plan->rp_codes[t], 0, rp_codes_bytes(d, n[t], K[t]), st));
        CK(cudaMemsetAsync(plan->rp_sf[t], 0, rp_sf_bytes(d, n[t], K[t]), st));
        const size_t total = (size_t)E * n[t] * (K[t] >> 5);
        const unsigned blocks = (unsigned)std::min<size_t>((total + 255) / 256, (size_t)plan->sm_count * 32);
        mx_repack_kernel<<<blocks, 256, 0, st>>>(src[t], stride[t], n[t], E, K[t], plan->rp_codes[t], plan->rp_sf[t]);
        CK(cudaGetLastError());
    }
    CK(cudaStreamSynchronize(st));
    plan->rp_ready = true;
    // single-token calls take the block-scaled kernels over the repacked form when the shape fits them
    plan->rp_token = plan->have_ws && plan->ws.mx_xb && F % 32 == 0 && H % 32 == 0 && H <= 12288 && F <= 12288 &&
                     mx_tma_smem(2, (uint32_t)(H / 32)) <= kMaxDynamicSmem && mx_tma_smem(1, (uint32_t)(F / 32)) <= kMaxDynamicSmem && plan->rp_token_on;
    return OCO_OK;
}

// Records one forward call as an executable graph. host = true: x and the residual rows are host buffers;
// the graph then also holds their copies into staging slot 0 and the copy of the residual rows back.
static int capture_forward(oco_moe_plan* plan, const uint16_t* x, uint16_t* residual, int rows, bool host, oco_moe_graph** out) {
    if (!plan || !out) return OCO_INVALID_ARGUMENT;
    *out = nullptr;
    if (plan->profiling) return fail(plan, OCO_INVALID_ARGUMENT, "switch profiling off before recording a graph");
    if (int rc_dev = check_device(plan)) return rc_dev;
    if (host) {
        if (!plan->have_ws || !plan->have_w) return fail(plan, OCO_INVALID_ARGUMENT, "bind a workspace and weights first");
        if (!x || !residual || rows < 1 || rows > plan->max_rows) return fail(plan, OCO_INVALID_ARGUMENT, "bad host buffers or rows");
        if (plan->host_begun != plan->host_ended) return fail(plan, OCO_INVALID_ARGUMENT, "end the host calls in flight first");
    }
    cudaStream_t side = nullptr;
    CK(cudaStreamCreateWithFlags(&side, cudaStreamNonBlocking));
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    int rc = OCO_OK;
    if (cudaStreamBeginCapture(side, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
        cudaStreamDestroy(side);
        return fail(plan, OCO_CUDA_ERROR, "cudaStreamBeginCapture failed");
    }
    if (host) {
        const size_t bytes = (size_t)rows * plan->d.hidden * 2;
        cudaError_t e = cudaMemcpyAsync(plan->ws.host_x[0], x, bytes, cudaMemcpyHostToDevice, side);
        if (e == cudaSuccess) e = cudaMemcpyAsync(plan->ws.host_res[0], residual, bytes, cudaMemcpyHostToDevice, side);
        if (e != cudaSuccess) rc = fail(plan, OCO_CUDA_ERROR, "cudaMemcpyAsync in capture: %s", cudaGetErrorString(e));
        if (rc == OCO_OK) rc = oco_moe_forward(plan, plan->ws.host_x[0], plan->ws.host_res[0], rows, side);
        if (rc == OCO_OK && cudaMemcpyAsync(residual, plan->ws.host_res[0], bytes, cudaMemcpyDeviceToHost, side) != cudaSuccess)
            rc = fail(plan, OCO_CUDA_ERROR, "cudaMemcpyAsync in capture failed");
    } else {
        rc = oco_moe_forward(plan, x, residual, rows, side);
    }
    const cudaError_t end = cudaStreamEndCapture(side, &graph);      // always ends the capture, also after a refused call
    if (rc == OCO_OK && (end != cudaSuccess || !graph)) rc = fail(plan, OCO_CUDA_ERROR, "cudaStreamEndCapture: %s", cudaGetErrorString(end));
    if (rc == OCO_OK && cudaGraphInstantiate(&exec, graph, 0) != cudaSuccess) rc = fail(plan, OCO_CUDA_ERROR, "cudaGraphInstantiate failed");
    if (graph) cudaGraphDestroy(graph);
    cudaStreamDestroy(side);
    (void)cudaGetLastError();
    if (rc != OCO_OK) return rc;
    oco_moe_graph* g = new (std::nothrow) oco_moe_graph();
    if (!g) { cudaGraphExecDestroy(exec); return OCO_OUT_OF_MEMORY; }
    g->exec = exec;
    g->plan = plan;
    *out = g;
    return OCO_OK;
}

int oco_moe_graph_capture(oco_moe_plan* plan, const uint16_t* x_bf16, uint16_t* residual_bf16, int rows, oco_moe_graph** out) {
    return capture_forward(plan, x_bf16, residual_bf16, rows, false, out);
}

int oco_moe_graph_capture_host(oco_moe_plan* plan, const uint16_t* x_bf16_host, uint16_t* residual_bf16_host, int rows,
                               oco_moe_graph** out) {
    return capture_forward(plan, x_bf16_host, residual_bf16_host, rows, true, out);
}

int oco_moe_graph_launch(oco_moe_graph* graph, void* cuda_stream) {
    if (!graph || !graph->exec) return OCO_INVALID_ARGUMENT;
    if (int rc_dev = check_device(graph->plan)) return rc_dev;
    if (cudaGraphLaunch(graph->exec, (cudaStream_t)cuda_stream) != cudaSuccess) {
        (void)cudaGetLastError();
        return fail(graph->plan, OCO_CUDA_ERROR, "cudaGraphLaunch failed");
    }
    return OCO_OK;
}

void oco_moe_graph_destroy(oco_moe_graph* graph) {
    if (!graph) return;
    if (graph->exec) cudaGraphExecDestroy(graph->exec);
    delete graph;
}

// Host calls of up to this many bytes per buffer run on the caller's stream alone.
constexpr size_t kHostOneStreamBytes = 256 * 1024;

int oco_moe_forward_host_begin(oco_moe_plan* plan, const uint16_t* x_host, uint16_t* residual_host, int rows,
                               void* cuda_stream) {
    if (!plan) return OCO_INVALID_ARGUMENT;
    if (!plan->have_ws) return fail(plan, OCO_INVALID_ARGUMENT, "bind a workspace first");
    if (int rc_dev = check_device(plan)) return rc_dev;
    if (!x_host || !residual_host || rows < 1 || rows > plan->max_rows) return fail(plan, OCO_INVALID_ARGUMENT, "bad host buffers or rows");
    if (!plan->have_w) return fail(plan, OCO_INVALID_ARGUMENT, "bind weights first");
    if (plan->host_begun - plan->host_ended >= 2) return fail(plan, OCO_INVALID_ARGUMENT, "two host calls are in flight: end one first");
    cudaStream_t st = (cudaStream_t)cuda_stream;
    const size_t bytes = (size_t)rows * plan->d.hidden * 2;
    if (!plan->in_stream) {
        CK(cudaStreamCreateWithFlags(&plan->in_stream, cudaStreamNonBlocking));
        CK(cudaStreamCreateWithFlags(&plan->out_stream, cudaStreamNonBlocking));
        for (int i = 0; i < 2; i++) {
            CK(cudaEventCreateWithFlags(&plan->ev_x[i], cudaEventDisableTiming));
            CK(cudaEventCreateWithFlags(&plan->ev_res[i], cudaEventDisableTiming));
            CK(cudaEventCreateWithFlags(&plan->ev_done[i], cudaEventDisableTiming));
            CK(cudaEventCreateWithFlags(&plan->ev_out[i], cudaEventDisableTiming));
        }
    }
    const int s = (int)(plan->host_begun & 1);
    uint16_t* dx = plan->ws.host_x[s];
    uint16_t* dres = plan->ws.host_res[s];
    if (bytes <= kHostOneStreamBytes) {
        // Few rows: the copies take microseconds, a hand-over between streams costs more than it could hide.
        // Everything goes to the caller's stream, in order, behind the copy back of the slot's last user.
        if (plan->host_begun >= 2) CK(cudaStreamWaitEvent(st, plan->ev_out[s], 0));
        CK(cudaMemcpyAsync(dx, x_host, bytes, cudaMemcpyHostToDevice, st));
        CK(cudaMemcpyAsync(dres, residual_host, bytes, cudaMemcpyHostToDevice, st));
        int rc = forward_any(plan, dx, dres, rows, st, nullptr);
        if (rc) return rc;
        CK(cudaMemcpyAsync(residual_host, dres, bytes, cudaMemcpyDeviceToHost, st));
        CK(cudaEventRecord(plan->ev_out[s], st));
        plan->host_begun++;
        return OCO_OK;
    }
    // In: the slot is free once the call that used it last has copied its rows back (which follows its
    // kernels); x goes first, the residual rows, which only the last kernel needs, behind it.
    CK(cudaStreamWaitEvent(plan->in_stream, plan->ev_out[s], 0));
    CK(cudaMemcpyAsync(dx, x_host, bytes, cudaMemcpyHostToDevice, plan->in_stream));
    CK(cudaEventRecord(plan->ev_x[s], plan->in_stream));
    CK(cudaMemcpyAsync(dres, residual_host, bytes, cudaMemcpyHostToDevice, plan->in_stream));
    CK(cudaEventRecord(plan->ev_res[s], plan->in_stream));
    // The layer, on the caller's stream, behind whatever that stream already holds (the call before).
    CK(cudaStreamWaitEvent(st, plan->ev_x[s], 0));
    int rc = forward_any(plan, dx, dres, rows, st, plan->ev_res[s]);
    if (rc) return rc;
    CK(cudaEventRecord(plan->ev_done[s], st));
    // Out: the residual rows back, beside the kernels of the next call.
    CK(cudaStreamWaitEvent(plan->out_stream, plan->ev_done[s], 0));
    CK(cudaMemcpyAsync(residual_host, dres, bytes, cudaMemcpyDeviceToHost, plan->out_stream));
    CK(cudaEventRecord(plan->ev_out[s], plan->out_stream));
    plan->host_begun++;
    return OCO_OK;
}

int oco_moe_forward_host_end(oco_moe_plan* plan) {
    if (!plan) return OCO_INVALID_ARGUMENT;
    if (plan->host_begun == plan->host_ended) return fail(plan, OCO_INVALID_ARGUMENT, "no host call is in flight");
    if (int rc_dev = check_device(plan)) return rc_dev;
    const int s = (int)(plan->host_ended & 1);
    plan->host_ended++;
    CK(cudaEventSynchronize(plan->ev_out[s]));
    return OCO_OK;
}

int oco_moe_forward_host(oco_moe_plan* plan, const uint16_t* x_host, uint16_t* residual_host, int rows,
                         void* cuda_stream) {
    if (!plan) return OCO_INVALID_ARGUMENT;
    while (plan->host_begun != plan->host_ended)                 // calls begun earlier finish first
        if (int rc = oco_moe_forward_host_end(plan)) return rc;
    if (int rc = oco_moe_forward_host_begin(plan, x_host, residual_host, rows, cuda_stream)) return rc;
    return oco_moe_forward_host_end(plan);
}

int oco_moe_poll(oco_moe_plan* plan, void* cuda_stream) {
    if (!plan || !plan->have_ws) return OCO_INVALID_ARGUMENT;
    cudaStream_t st = (cudaStream_t)cuda_stream;
    uint32_t word = 0;
    CK(cudaMemcpyAsync(&word, plan->ws.status, 4, cudaMemcpyDeviceToHost, st));
    CK(cudaStreamSynchronize(st));
    if (word != 0) {
        CK(cudaMemsetAsync(plan->ws.status, 0, 4, st));
        CK(cudaStreamSynchronize(st));
        return fail(plan, OCO_DEVICE_TIMEOUT, "a bounded device wait gave up (status %u)", word);
    }
    return OCO_OK;
}

int oco_moe_routing(const oco_moe_plan* plan, oco_moe_routing_view* out) {
    if (!plan || !out || !plan->have_ws) return OCO_INVALID_ARGUMENT;
    const Workspace& ws = plan->ws;
    out->logits = ws.logits; out->ids = ws.ids; out->probs = ws.probs; out->offsets = ws.offsets;
    out->row_of_route = ws.row_of_route; out->route_of_row = ws.route_of_row; out->tiles = ws.tiles;
    out->tile_count = ws.tile_count; out->act = ws.act; out->y = ws.y; out->norm = ws.norm;
    return OCO_OK;
}

}  // extern "C"

// ---- dense products ------------------------------------------------------------------------------------
// A dense plan is a one-expert plan of the family whose kernels carry the kind's arithmetic: every row
// is a route to expert 0, the tiles run in their dense mode, the single-token kernels take a null id list.
struct oco_dense_plan {
    oco_moe_plan* inner = nullptr;
    oco_dense_desc d{};
};

namespace {

template <int ARCH>
int dense_rows(oco_dense_plan* dp, const uint16_t* x, uint16_t* y, int rows, cudaStream_t st) {
    constexpr int FMT = Family<ARCH>::kFmt;
    oco_moe_plan* plan = dp->inner;
    Workspace& ws = plan->ws;
    const int H = dp->d.hidden, F = dp->d.ffn, kind = dp->d.kind;
    if (rows == 1) {
        mark(plan, st, "fragments");
        CK(launch_dependent(token_fragments_kernel, dim3((H + 255) / 256), dim3(256), 0, st, x, H, ws.xfrag, (int)FMT));
        plan->launches++;
        DecodeDownParams dn{};
        dn.ids = nullptr; dn.K = 1; dn.status = ws.status;
        if (kind == OCO_DENSE_PROJECTION) {
            dn.down_w = plan->w.up_w; dn.actfrag = ws.xfrag; dn.y = y; dn.H = F; dn.F = H; dn.row_bytes = plan->up_row_bytes;
            mark(plan, st, "project");
            return launch_down<FMT>(plan, dn, st);
        }
        DecodeExpandParams ep{};
        ep.gate_w = plan->w.gate_w; ep.up_w = plan->w.up_w; ep.bias_stride = 1;
        ep.xfrag = ws.xfrag; ep.ids = nullptr; ep.act = ws.act1; ep.actfrag = ws.actfrag;
        ep.H = H; ep.F = F; ep.K = 1; ep.row_bytes = plan->up_row_bytes; ep.status = ws.status;
        mark(plan, st, "expand");
        if (int rc = launch_expand<ARCH, FMT>(plan, ep, st)) return rc;
        dn.down_w = plan->w.down_w; dn.actfrag = ws.actfrag; dn.y = y; dn.H = H; dn.F = F; dn.row_bytes = plan->down_row_bytes;
        mark(plan, st, "down");
        return launch_down<FMT>(plan, dn, st);
    }
    const int nt_index = pick_tile_index(rows, 1, plan->narrow_tiles ? 192 : plan->wide_min_avg);
    const int NT = kTileSizes[nt_index], tiles = (rows + NT - 1) / NT;
    mark(plan, st, "to_half");
    permute_rows_kernel<<<std::min(rows, 16 * plan->sm_count), 256, 0, st>>>(x, nullptr, 1, H, FMT == OCO_FMT_Q4_K ? 32 : 16, ws.xs,
                                                                          (uint32_t)rows, nullptr);
    plan->launches++;
    CK(cudaGetLastError());
    GemmParams g{};
    g.status = ws.status; g.dense_rows = rows; g.tile_rows = NT; g.bias_stride = 1;
    if (kind == OCO_DENSE_PROJECTION) {
        g.w0 = plan->w.up_w; g.n = F; g.K = H; g.row_bytes = plan->up_row_bytes; g.xs = ws.xs; g.out = y;
        mark(plan, st, "project_tiles");
        return launch_gemm_nt<FMT, kEpiDownBf16>(plan, g, plan->map_xs, nt_index, tiles, st);
    }
    constexpr int EPI = ARCH == OCO_ARCH_NEMOTRON ? kEpiRelu2Bf16F16 : kEpiSiluF16;
    g.w0 = ARCH == OCO_ARCH_NEMOTRON ? plan->w.up_w : plan->w.gate_w;
    g.w1 = ARCH == OCO_ARCH_NEMOTRON ? nullptr : plan->w.up_w;
    g.n = F; g.K = H; g.row_bytes = plan->up_row_bytes; g.xs = ws.xs; g.out = ws.act;
    mark(plan, st, "up_tiles");
    if constexpr (ARCH != OCO_ARCH_GPT_OSS) {
        if (int rc = launch_gemm_nt<FMT, EPI>(plan, g, plan->map_xs, nt_index, tiles, st)) return rc;
    }
    GemmParams dn{};
    dn.status = ws.status; dn.dense_rows = rows; dn.tile_rows = NT; dn.bias_stride = 1;
    dn.w0 = plan->w.down_w; dn.n = H; dn.K = F; dn.row_bytes = plan->down_row_bytes; dn.xs = ws.act; dn.out = y;
    mark(plan, st, "down_tiles");
    return launch_gemm_nt<FMT, kEpiDownBf16>(plan, dn, plan->map_act, nt_index, tiles, st);
}

}  // namespace

extern "C" {

int oco_dense_plan_create(const oco_dense_desc* desc, oco_dense_plan** out) {
    if (!desc || !out) return OCO_INVALID_ARGUMENT;
    oco_dense_plan* dp = new (std::nothrow) oco_dense_plan();
    if (!dp) return OCO_INVALID_ARGUMENT;
    dp->d = *desc;
    *out = dp;   // handed out even on failure so that the caller can read the message, then destroy
    oco_moe_desc md{};
    md.hidden = desc->hidden; md.ffn = desc->ffn; md.experts = 1; md.top_k = 1; md.weight_format = desc->weight_format;
    md.scale = 1.0f;
    if (desc->kind == OCO_DENSE_PROJECTION && desc->ffn > 0 && desc->ffn % 32 == 0) {
        // a projection's outputs are rows of the matrix, not a contraction length: any multiple of 32 (the inner
        // plan, which sizes buffers by block multiples, is told the next one)
        const int be = desc->weight_format == OCO_FMT_Q4_K ? 256 : 32;
        md.ffn = (desc->ffn + be - 1) / be * be;
    }
    switch (desc->weight_format) {
        case OCO_FMT_MXFP4: md.arch = OCO_ARCH_GPT_OSS; break;
        case OCO_FMT_Q4_0: md.arch = OCO_ARCH_NEMOTRON; break;
        default: md.arch = OCO_ARCH_QWEN; break;
    }
    int rc = oco_moe_plan_create(&md, &dp->inner);
    if (rc) return rc;
    if (desc->kind < OCO_DENSE_PROJECTION || desc->kind > OCO_DENSE_FFN_SILU_GATE) return fail(dp->inner, OCO_INVALID_ARGUMENT, "unknown dense kind %d", desc->kind);
    if (desc->kind == OCO_DENSE_FFN_RELU2 && desc->weight_format != OCO_FMT_Q4_0)
        return fail(dp->inner, OCO_UNSUPPORTED_SHAPE, "the relu^2 feed-forward is built for Q4_0 weights");
    if (desc->kind == OCO_DENSE_FFN_SILU_GATE && desc->weight_format != OCO_FMT_Q4_K)
        return fail(dp->inner, OCO_UNSUPPORTED_SHAPE, "the gated feed-forward is built for Q4_K weights");
    return OCO_OK;
}

void oco_dense_plan_destroy(oco_dense_plan* plan) {
    if (!plan) return;
    oco_moe_plan_destroy(plan->inner);
    delete plan;
}

size_t oco_dense_workspace_bytes(const oco_dense_plan* plan, int max_rows) {
    return plan && plan->inner ? oco_moe_workspace_bytes(plan->inner, max_rows) : 0;
}

int oco_dense_bind_workspace(oco_dense_plan* plan, void* workspace, size_t bytes, int max_rows) {
    if (!plan || !plan->inner) return OCO_INVALID_ARGUMENT;
    return oco_moe_bind_workspace(plan->inner, workspace, bytes, max_rows);
}

int oco_dense_bind_weights(oco_dense_plan* plan, const oco_dense_weights* w) {
    if (!plan || !plan->inner) return OCO_INVALID_ARGUMENT;
    oco_moe_plan* in = plan->inner;
    if (!w || !w->up_w) return fail(in, OCO_INVALID_ARGUMENT, "up_w is required");
    if (plan->d.kind != OCO_DENSE_PROJECTION && !w->down_w) return fail(in, OCO_INVALID_ARGUMENT, "down_w is required for a feed-forward");
    if (plan->d.kind == OCO_DENSE_FFN_SILU_GATE && !w->gate_w) return fail(in, OCO_INVALID_ARGUMENT, "gate_w is required for the gated feed-forward");
    in->w = oco_moe_weights{};
    in->w.up_w = w->up_w; in->w.gate_w = w->gate_w; in->w.down_w = w->down_w;
    in->gate_rows = (const uint8_t*)w->gate_w; in->up_rows = (const uint8_t*)w->up_w;
    in->gate_bias = in->up_bias = nullptr;
    in->up_row_stride = in->up_row_bytes; in->up_bias_stride = 1;
    in->have_w = in->have_experts = true;
    return OCO_OK;
}

int oco_dense_forward(oco_dense_plan* dp, const uint16_t* x_bf16, uint16_t* y_bf16, int rows, void* cuda_stream) {
    if (!dp || !dp->inner) return OCO_INVALID_ARGUMENT;
    oco_moe_plan* plan = dp->inner;
    if (!plan->have_ws || !plan->have_w) return fail(plan, OCO_INVALID_ARGUMENT, "bind a workspace and weights first");
    if (int rc_dev = check_device(plan)) return rc_dev;
    if (!x_bf16 || !y_bf16 || rows < 1 || rows > plan->max_rows) return fail(plan, OCO_INVALID_ARGUMENT, "bad buffers, or rows outside 1 .. max_rows");
    cudaStream_t st = (cudaStream_t)cuda_stream;
    plan->launches = 0;
    plan->n_marks = 0;
    int rc;
    switch (plan->d.arch) {
        case OCO_ARCH_GPT_OSS: rc = dense_rows<OCO_ARCH_GPT_OSS>(dp, x_bf16, y_bf16, rows, st); break;
        case OCO_ARCH_NEMOTRON: rc = dense_rows<OCO_ARCH_NEMOTRON>(dp, x_bf16, y_bf16, rows, st); break;
        default: rc = dense_rows<OCO_ARCH_QWEN>(dp, x_bf16, y_bf16, rows, st); break;
    }
    mark(plan, st, "end");
    return rc;
}

int oco_dense_poll(oco_dense_plan* plan, void* cuda_stream) { return plan && plan->inner ? oco_moe_poll(plan->inner, cuda_stream) : OCO_INVALID_ARGUMENT; }
int oco_dense_last_launch_count(const oco_dense_plan* plan) { return plan && plan->inner ? plan->inner->launches : 0; }
const char* oco_dense_last_error(const oco_dense_plan* plan) { return plan && plan->inner ? plan->inner->err : "null plan"; }

const char* oco_moe_last_error(const oco_moe_plan* plan) { return plan ? plan->err : "null plan"; }
int oco_moe_last_launch_count(const oco_moe_plan* plan) { return plan ? plan->launches : 0; }

static int dequant_any(int fmt, const uint8_t* w, size_t n, float* o32, uint16_t* o16, void* stream) {
    if (!w || (!o32 && !o16)) return OCO_INVALID_ARGUMENT;
    size_t chunks = (n + 63) / 64;
    unsigned blocks = (unsigned)((chunks + 127) / 128);
    cudaStream_t st = (cudaStream_t)stream;
    switch (fmt) {
        case OCO_FMT_MXFP4: dequant_kernel<OCO_FMT_MXFP4><<<blocks, 128, 0, st>>>(w, n, o32, o16); break;
        case OCO_FMT_Q4_0: dequant_kernel<OCO_FMT_Q4_0><<<blocks, 128, 0, st>>>(w, n, o32, o16); break;
        case OCO_FMT_Q4_K: dequant_kernel<OCO_FMT_Q4_K><<<blocks, 128, 0, st>>>(w, n, o32, o16); break;
        default: return OCO_UNSUPPORTED_SHAPE;
    }
    return cudaGetLastError() == cudaSuccess ? OCO_OK : OCO_CUDA_ERROR;
}
int oco_moe_dequant_f32(int fmt, const uint8_t* w, size_t n, float* out, void* stream) {
    return dequant_any(fmt, w, n, out, nullptr, stream);
}
int oco_moe_dequant_f16(int fmt, const uint8_t* w, size_t n, uint16_t* out, void* stream) {
    return dequant_any(fmt, w, n, nullptr, out, stream);
}

// ---- runtime seam -----------------------------------------------------------------------------
static int cu(cudaError_t e) { return e == cudaSuccess ? OCO_OK : OCO_CUDA_ERROR; }
int oco_cuda_device_open(int device) { return cu(cudaSetDevice(device)); }
int oco_cuda_malloc(void** out, size_t bytes) { return out ? cu(cudaMalloc(out, bytes)) : OCO_INVALID_ARGUMENT; }
int oco_cuda_free(void* ptr) { return cu(cudaFree(ptr)); }
int oco_cuda_upload(void* dst, const void* src, size_t bytes, void* stream) {
    return cu(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream));
}
int oco_cuda_download(void* dst, const void* src, size_t bytes, void* stream) {
    return cu(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
}
int oco_cuda_stream_create(void** out) {
    if (!out) return OCO_INVALID_ARGUMENT;
    cudaStream_t s;
    cudaError_t e = cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking);
    *out = (void*)s;
    return cu(e);
}
int oco_cuda_stream_destroy(void* stream) { return cu(cudaStreamDestroy((cudaStream_t)stream)); }
int oco_cuda_stream_sync(void* stream) { return cu(cudaStreamSynchronize((cudaStream_t)stream)); }
int oco_cuda_event_create(void** out) {
    if (!out) return OCO_INVALID_ARGUMENT;
    cudaEvent_t e;
    cudaError_t r = cudaEventCreate(&e);
    *out = (void*)e;
    return cu(r);
}
int oco_cuda_event_destroy(void* event) { return cu(cudaEventDestroy((cudaEvent_t)event)); }
int oco_cuda_event_record(void* event, void* stream) { return cu(cudaEventRecord((cudaEvent_t)event, (cudaStream_t)stream)); }
int oco_cuda_event_sync(void* event) { return cu(cudaEventSynchronize((cudaEvent_t)event)); }
int oco_cuda_event_elapsed_ms(void* start, void* end, float* ms) {
    if (!ms) return OCO_INVALID_ARGUMENT;
    return cu(cudaEventElapsedTime(ms, (cudaEvent_t)start, (cudaEvent_t)end));
}

int oco_moe_selftest_wait_timeout(oco_moe_plan* plan, long long wait_cycles, void* cuda_stream) {
    if (!plan || !plan->have_ws) return OCO_INVALID_ARGUMENT;
    if (wait_cycles < 1 || wait_cycles > kWaitCycles) return fail(plan, OCO_INVALID_ARGUMENT, "wait_cycles outside 1..%lld", kWaitCycles);
    if (int rc_dev = check_device(plan)) return rc_dev;
    wait_timeout_kernel<<<1, 32, 0, (cudaStream_t)cuda_stream>>>(plan->ws.status, wait_cycles);
    CK(cudaGetLastError());
    return OCO_OK;
}

}  // extern "C"

