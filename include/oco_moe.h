/*
 * oco_moe.h — C ABI of the B200 (sm_100a) mixture-of-experts layer.
 *
 * This is the boundary a CUDA backend of the reference's `src/gpu` would bind through a thin FFI
 * crate: plain pointers and sizes, no C++ or framework types. One call enqueues the whole MoE
 * layer (router -> top-k -> token-to-expert permutation -> quantised expert products ->
 * activation -> weighted combine onto the residual) on a CUDA stream and returns; stream order
 * replaces the reference's dispatch barriers (reference `src/gpu/dispatch.rs:303-311`).
 *
 * Ownership: the caller owns all device memory (weights, x, residual, workspace) and keeps it
 * valid until the stream reaches the end of the call; the library owns only the plan object.
 * Weight tensors are the GGUF byte spans staged into device memory unchanged (block layouts of
 * reference `src/tensor.rs:24-36`). They may start at any byte address; kernels read whole
 * 16-byte-aligned chunks, so the 16-byte-aligned envelope of every weight tensor must be
 * readable (true for anything carved out of a cudaMalloc allocation with 16 bytes of slack).
 * x, residual and the workspace must be 256-byte aligned.
 *
 * Errors: every entry point returns an `oco_status`; nothing aborts or throws across the ABI.
 * Numerical failure keeps the reference's convention (reference `shaders/experts/routing.metal:69-70`,
 * `src/weights/session.rs:254-257`): a reserved E8M0 scale (255) or a non-finite logit yields NaN
 * in the output while the expert ids stay valid, so the caller's final-logit check still fires.
 * Device-side waits are bounded; a wait that gives up sets a status word that `oco_moe_poll`
 * reports as OCO_DEVICE_TIMEOUT.
 *
 * Threading: a plan with its bound workspace serves one stream at a time. Weights are immutable
 * and may be shared by several plans.
 */
#ifndef OCO_MOE_H
#define OCO_MOE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    OCO_OK = 0,
    OCO_INVALID_ARGUMENT = 1,
    OCO_UNSUPPORTED_SHAPE = 2,
    OCO_CUDA_ERROR = 3,
    OCO_NCCL_ERROR = 4,
    OCO_DEVICE_TIMEOUT = 5,
    OCO_OUT_OF_MEMORY = 6
} oco_status;

/* Layer families. Each fixes the router, the activation and the combine rule:
 *  GPT_OSS   top-k of bf16-rounded-weight logits, softmax over the winners, clipped SwiGLU with
 *            biases, expert sum rounded to bf16 before the residual
 *            (reference `Bindings::experts`, src/weights/compute/feed_forward.rs:107-275)
 *  NEMOTRON  sigmoid router with selection bias, non-gated squared-ReLU experts, optional shared
 *            expert, single-rounding weighted add
 *            (reference `Bindings::relu_experts`, src/weights/compute/nemotron.rs:286-545)
 *  QWEN      softmax over all experts, top-k renormalised, SiLU-gated experts (no counterpart
 *            operator in the reference, which runs Qwen as a dense FFN; semantics are composed
 *            from its SiLU gate, shaders/elementwise.metal:67-87, and its Q4_K decoder). */
typedef enum { OCO_ARCH_GPT_OSS = 0, OCO_ARCH_NEMOTRON = 1, OCO_ARCH_QWEN = 2 } oco_arch;

/* GGUF tensor type codes (reference `src/tensor.rs:9-22`). */
typedef enum { OCO_FMT_Q4_0 = 2, OCO_FMT_Q4_K = 12, OCO_FMT_MXFP4 = 39 } oco_weight_format;

/* Geometry lowered once per model, as the reference's `ExpertPlan::new`
 * (feed_forward.rs:43-72) and `ReluExpertPlan::new` (compute/nemotron.rs:142-184). */
typedef struct {
    int32_t arch;           /* oco_arch */
    int32_t hidden;         /* model width (k of up/gate, n of down) */
    int32_t ffn;            /* expert width */
    int32_t experts;        /* <= 128 */
    int32_t top_k;          /* <= 8 */
    int32_t shared_ffn;     /* NEMOTRON: width of the always-on shared expert, 0 = none */
    int32_t weight_format;  /* oco_weight_format of every expert bank */
    int32_t normalize;      /* NEMOTRON: divide the weights by their sum */
    float scale;            /* NEMOTRON: routed scaling factor */
    int32_t gemm_impl;      /* 0 = tcgen05 tiles (the product path); 1 = plain CUDA-core tiles, a
                               slow second implementation kept for cross-checking */
    int32_t numerics;       /* 0 = the reference's arithmetic (half x half tiles, f32 single-token products; the default
                               and the only mode whose results are held to the reference). 2 = GPT_OSS, rows > 1: the
                               expert tiles run on the block-scaled FP4 tensor-core kind (tcgen05 kind::mxf4): MXFP4
                               weights as stored, ACTIVATIONS quantised to MXFP4 (e2m1, one UE8M0 scale per 32 elements).
                               Several times faster, and about 1e-1 relative L2 away from mode 0: an explicit trade the
                               caller opts into, not a drop-in for the reference path. No counterpart in the reference. */
} oco_moe_desc;

/* Device pointers of one layer (reference `Experts{gate,up,down,router}`, src/weights/gpt_oss.rs:33-38;
 * `ReluExperts`, src/weights/nemotron.rs:60-66). Unused members are NULL. */
typedef struct {
    const float* router_w;        /* f32 [experts, hidden] */
    const float* router_b;        /* f32 [experts]: GPT_OSS logit bias / NEMOTRON selection bias */
    const uint8_t* gate_w;        /* [experts][ffn][hidden packed] (gated families) */
    const uint8_t* up_w;          /* [experts][ffn][hidden packed] */
    const uint8_t* down_w;        /* [experts][hidden][ffn packed] */
    const float* gate_b;          /* GPT_OSS f32 [experts, ffn] */
    const float* up_b;            /* GPT_OSS f32 [experts, ffn] */
    const float* down_b;          /* GPT_OSS f32 [experts, hidden] */
    const uint8_t* shared_up_w;   /* NEMOTRON [shared_ffn][hidden packed] */
    const uint8_t* shared_down_w; /* NEMOTRON [hidden][shared_ffn packed] */
    /* Gate and up projections as ONE tensor with interleaved rows, [experts][2 * ffn][hidden packed]:
     * row 2c is gate row c, row 2c + 1 is up row c (the layout checkpoints of the gpt-oss family
     * ship as `gate_up_proj`; the reference reads the two-tensor GGUF form, src/weights/gpt_oss/load.rs:131-133).
     * Give either this member (with gate_w and up_w NULL) or gate_w + up_w. gate_up_b: f32
     * [experts, 2 * ffn] with the same interleave (GPT_OSS). Results are bit-identical to the
     * two-tensor layout. */
    const uint8_t* gate_up_w;
    const float* gate_up_b;
} oco_moe_weights;

/* Addresses of the routing side-outputs inside the bound workspace, valid after a forward call
 * has completed (reference `Routing{ids,plan,prob}`, src/weights/state.rs:112-117). The
 * permutation is kept in flat form: `offsets` is the exclusive scan of per-expert route counts,
 * `row_of_route` the expert-sorted row of each route (a stable sort of route indices by expert
 * id, as `route_plan_tiled` produces, shaders/experts/routing.metal:4-39), `route_of_row` its
 * inverse (the concatenated per-expert route lists). */
typedef struct {
    const float* logits;          /* f32 [rows, experts] */
    const uint32_t* ids;          /* u32 [rows * top_k] */
    const float* probs;           /* f32 [rows * top_k] */
    const uint32_t* offsets;      /* u32 [experts + 1]  (rows > 1 only) */
    const uint32_t* row_of_route; /* u32 [rows * top_k] (rows > 1 only) */
    const uint32_t* route_of_row; /* u32 [rows * top_k] (rows > 1 only) */
    const uint32_t* tiles;        /* u32 pairs (expert, first row in expert), rows > 1 only */
    const uint32_t* tile_count;   /* u32 [1] */
    const uint16_t* act;          /* f16 [routes, ffn] activated intermediate, expert-sorted rows (rows > 1).
                                     Columns are in the tiles' operand order: within each 32-element block
                                     (64 for Q4_K) element j sits at 2*(j mod h) + j div h, h = 16 (32 for Q4_K),
                                     the order in which the packed code bytes hold their two nibbles. */
    const uint16_t* y;            /* bf16 [routes, hidden] expert outputs in route order */
    const uint16_t* norm;         /* bf16 [rows, hidden] normalised rows of the last oco_moe_add_norm_forward */
} oco_moe_routing_view;

typedef struct oco_moe_plan oco_moe_plan;

/* ---- the operator ------------------------------------------------------------------------ */

/* Replaces ExpertPlan::new / ReluExpertPlan::new plus Builder::experts / Builder::nemotron
 * (src/weights/pipelines.rs:456-501): validates the geometry and fixes launch shapes. */
int oco_moe_plan_create(const oco_moe_desc* desc, oco_moe_plan** out);
void oco_moe_plan_destroy(oco_moe_plan* plan);

/* Replaces the workspace sizing of CommonScratch::plan / Memory::new
 * (src/weights/state.rs:148-177, src/weights/gpt_oss.rs:48-74). */
size_t oco_moe_workspace_bytes(const oco_moe_plan* plan, int max_rows);

/* Hands the plan a caller-owned device workspace of at least oco_moe_workspace_bytes(max_rows)
 * bytes. Must be called with the owning device current; builds the TMA descriptors over it. A set-up
 * call: it clears control words and waits for the device. The plan remembers the device; every
 * later call on the plan must be made with that device current (OCO_INVALID_ARGUMENT otherwise).
 * Kernel attributes are set per device, so plans on several GPUs may live in one process. */
int oco_moe_bind_workspace(oco_moe_plan* plan, void* workspace, size_t bytes, int max_rows);

/* Replaces binding `w: &Experts` / `w: &ReluExperts` at the call site. A set-up call: once both the
 * workspace and GPT_OSS router weights are bound it makes the bf16-rounded router copy and waits for
 * it, so the first forward call may already be inside a stream capture or on any stream. */
int oco_moe_bind_weights(oco_moe_plan* plan, const oco_moe_weights* weights);

/* Replaces Bindings::experts (feed_forward.rs:107-114) and Bindings::relu_experts
 * (compute/nemotron.rs:286-293): reads x bf16 [rows, hidden] (the reference's `scratch.norm`),
 * accumulates the layer's output into residual bf16 [rows, hidden] in place. rows == 1 takes the
 * single-token kernels, rows > 1 the tiled ones, as in the reference. Only enqueues. */
int oco_moe_forward(oco_moe_plan* plan, const uint16_t* x_bf16, uint16_t* residual_bf16, int rows,
                    void* cuda_stream);

/* The three stages of the layer as calls of their own, for expert parallelism (experts sharded
 * over GPUs, an all-to-all between the stages). The reference has no multi-GPU path; these follow
 * the stage boundaries of its tiled operator (feed_forward.rs:165-274): router, then route plan +
 * up/down tiles, then moe_sum / moe_add.
 *   oco_moe_route    ids and weights of `rows` tokens into the workspace (read them with
 *                    oco_moe_routing); the plan needs only router weights bound.
 *   oco_moe_experts  expert products of `routes` rows that are already routed: row i (bf16
 *                    [routes, hidden]) goes to expert expert_ids[i] of THIS plan (0 .. experts-1, the
 *                    local shard), its bf16 output lands in row i of y. routes <= max_rows * top_k.
 *   oco_moe_combine  residual[t] += sum_r y[t * top_k + r] * probs[t * top_k + r] with the family's
 *                    rounding rule. */
int oco_moe_route(oco_moe_plan* plan, const uint16_t* x_bf16, int rows, void* cuda_stream);
int oco_moe_experts(oco_moe_plan* plan, const uint16_t* rows_bf16, const uint32_t* expert_ids, int routes,
                    uint16_t* y_bf16, void* cuda_stream);
int oco_moe_combine(oco_moe_plan* plan, const uint16_t* y_bf16, const float* probs, uint16_t* residual_bf16,
                    int rows, void* cuda_stream);
/* oco_moe_combine for the family with an always-on expert (NEMOTRON), whose output shared_bf16 [rows, hidden]
 * (oco_dense_forward, OCO_DENSE_FFN_RELU2, computed where the tokens live) joins the residual as a bf16 add
 * ahead of the routed sum, as on the reference's tiled path (compute/nemotron.rs:316). */
int oco_moe_combine_shared(oco_moe_plan* plan, const uint16_t* y_bf16, const float* probs, const uint16_t* shared_bf16,
                           uint16_t* residual_bf16, int rows, void* cuda_stream);

/* The step either side of the layer, in one call (reference Bindings::add_norm followed by
 * Bindings::experts, src/weights/compute.rs:100-117 and src/weights/gpt_oss.rs:122-123; kernels
 * add_norm / norm, shaders/elementwise.metal:5-60):
 *     hidden += projected            bf16 rows [rows, hidden]; projected may be NULL (plain norm)
 *     x = rmsnorm(hidden) * norm_weight   f32 weight [hidden]; full_layer = 1 scales in f32 and rounds
 *                                    once (gpt-oss), 0 rounds the normalised value and the weight to bf16
 *                                    first (Qwen)
 *     hidden += MoE(x)
 * The normalised rows stay in the workspace (oco_moe_routing gives their address). */
int oco_moe_add_norm_forward(oco_moe_plan* plan, uint16_t* hidden_bf16, const uint16_t* projected_bf16,
                             const float* norm_weight, float epsilon, int full_layer, int rows, void* cuda_stream);

/* The same call for host buffers, submitted eagerly (reference Compute::submit,
 * src/weights/compute/submission.rs:17-24: work is submitted at once and completion is signalled later; the
 * caller gives up host access to the writable buffer until then). _begin queues, without waiting: the copy
 * of x and then of the residual rows to the device on a stream the plan owns (the residual rows are needed
 * by the last kernel only, so their copy runs beside the router and the expert products), the layer on
 * `cuda_stream`, and the copy of the residual rows back on a second stream of the plan. _end waits until the
 * oldest begun call has its rows back in `residual_bf16_host`. Up to two calls may be in flight (the third
 * _begin is refused with OCO_INVALID_ARGUMENT): the copies of call c + 1 then cross the bus beside the
 * kernels of call c (calls of up to 256 KB per buffer run on `cuda_stream` alone: their copies take
 * microseconds and a hand-over between streams would cost more). All calls of a plan go to one `cuda_stream`. Staging space (two slots) lies inside the
 * bound workspace; pinned host buffers make the copies asynchronous. */
int oco_moe_forward_host_begin(oco_moe_plan* plan, const uint16_t* x_bf16_host, uint16_t* residual_bf16_host,
                               int rows, void* cuda_stream);
int oco_moe_forward_host_end(oco_moe_plan* plan);

/* _begin followed by _end (calls begun earlier are ended first): one layer call on host buffers that
 * returns with the result in `residual_bf16_host`. */
int oco_moe_forward_host(oco_moe_plan* plan, const uint16_t* x_bf16_host, uint16_t* residual_bf16_host,
                         int rows, void* cuda_stream);

/* Waits for `cuda_stream`, then reports OCO_DEVICE_TIMEOUT if any bounded device wait gave up
 * since the last poll, OCO_CUDA_ERROR on a CUDA failure, else OCO_OK. Maps to the completion of
 * the reference's `submit` future (src/weights/compute/submission.rs:56-98). */
int oco_moe_poll(oco_moe_plan* plan, void* cuda_stream);

int oco_moe_routing(const oco_moe_plan* plan, oco_moe_routing_view* out);
const char* oco_moe_last_error(const oco_moe_plan* plan);

/* Number of kernels the last oco_moe_forward call launched. */
int oco_moe_last_launch_count(const oco_moe_plan* plan);

/* Per-kernel device timestamps, the counterpart of the reference's OCO_PROFILE counter heap
 * (src/gpu/profile.rs:1-31, src/gpu/dispatch.rs:189-208). When enabled, oco_moe_forward records
 * one CUDA event on the stream ahead of every kernel. After the stream has been waited for,
 * oco_moe_phase_times fills up to `capacity` durations in milliseconds and the phase names of
 * the last forward call and returns the number of phases (negative on a bad argument). */
int oco_moe_set_profiling(oco_moe_plan* plan, int enabled);
int oco_moe_phase_times(oco_moe_plan* plan, int capacity, float* ms, const char** names);

/* Expert ids and combination weights of ONE token, computed without any device allocation and
 * without a bound workspace. This call has no counterpart in the reference. It serves hosts that
 * may not allocate once a session is set up: an engine that plans its whole device budget up
 * front the way oco's arena does, a plugin living beside a framework allocator that already
 * owns the GPU's free memory, or a loop that cannot take the device-wide stall of cudaMalloc.
 * The scratch it needs (one token's router logits and an arrival counter) sits in a 1024-byte
 * device array inside the library image, held by every GPU that loads the library until exit.
 * Limits: experts <= 128 (what the array holds), top_k <= 8, hidden a multiple of 4 and <= 16384;
 * anything larger is refused with OCO_UNSUPPORTED_SHAPE and a message in `err` (if given).
 * x_bf16, router_w, router_b, ids_out [top_k] and probs_out [top_k] are device pointers.
 * All calls on a GPU share the array, which keeps the last call's contents; calls that overlap on
 * the same GPU race on it and must be serialised by the caller. The first call on each device
 * looks the array's address up and should come before any stream capture starts.
 * Results equal those of oco_moe_forward at rows == 1 (same logits order, same selection). */
int oco_moe_route_token_static(int arch, const uint16_t* x_bf16, const float* router_w, const float* router_b,
                               int hidden, int experts, int top_k, int normalize, float scale,
                               uint32_t* ids_out, float* probs_out, void* cuda_stream, char* err, size_t err_len);

/* ---- block decoders, exposed for bit-exact checks ------------------------------------------- */

/* Decodes n_elems weights of a packed tensor to f32 exactly as the single-token kernels see
 * them (reference `weight()`, shaders/matrix/weights.metal:48-77). */
int oco_moe_dequant_f32(int weight_format, const uint8_t* w, size_t n_elems, float* out,
                        void* cuda_stream);
/* The tile kernels' operand: the same value rounded to half (reference projections.metal:227). */
int oco_moe_dequant_f16(int weight_format, const uint8_t* w, size_t n_elems, uint16_t* out,
                        void* cuda_stream);

/* ---- runtime seam (replaces the Metal side of reference src/gpu.rs, src/gpu/buffer.rs) ------- */
int oco_cuda_device_open(int device);                       /* Gpu::new, src/gpu.rs:40-60 */
int oco_cuda_malloc(void** out, size_t bytes);              /* Gpu::new_buffer, src/gpu/buffer.rs */
int oco_cuda_free(void* ptr);
int oco_cuda_upload(void* dst_device, const void* src_host, size_t bytes, void* cuda_stream);   /* MappedRegions::new: GGUF spans byte for byte */
int oco_cuda_download(void* dst_host, const void* src_device, size_t bytes, void* cuda_stream);
int oco_cuda_stream_create(void** out);
int oco_cuda_stream_destroy(void* cuda_stream);
int oco_cuda_stream_sync(void* cuda_stream);
/* Device timestamps: what the reference's dispatch encoder samples into its counter heap around each
 * dispatch (src/gpu/dispatch.rs:189-208, src/gpu/profile.rs:1-31). */
int oco_cuda_event_create(void** out);
int oco_cuda_event_destroy(void* event);
int oco_cuda_event_record(void* event, void* cuda_stream);
int oco_cuda_event_sync(void* event);
int oco_cuda_event_elapsed_ms(void* start_event, void* end_event, float* ms);

/* Self-test of the bounded-wait path, safe to run anywhere: enqueues a one-warp kernel that waits
 * `wait_cycles` clock cycles (1 .. 400 000 000) on a barrier nobody arrives at, gives up, sets the
 * workspace status word and returns normally. Afterwards oco_moe_poll reports OCO_DEVICE_TIMEOUT once
 * and clears the word; forward calls enqueued while the word is set leave the residual rows
 * untouched. No counterpart in the reference (Metal has no device-side waits on this path). */
int oco_moe_selftest_wait_timeout(oco_moe_plan* plan, long long wait_cycles, void* cuda_stream);

/* Measured tensor-pipe ceiling of the current GPU for one tcgen05.mma kind (0 = f16, 1 = f8f6f4 e4m3,
 * 2 = mxf8f6f4 block-scaled e4m3, 3 = mxf4 block-scaled e2m1): `iters` x 4 back-to-back MMAs of shape
 * M128 N256 on zero operands per SM, dense TFLOP/s in *tflops. Measurement support for the benchmark's
 * roofline fractions; allocates 256 bytes for the call's duration. No counterpart in the reference. */
int oco_tensor_peak(int kind, int iters, float* tflops);

/* Optional second form of the MXFP4 expert tensors (GPT_OSS): the blocks' code bytes and scale bytes in two
 * planes per tensor, laid out so that TMA and tcgen05.cp can take them as they are. The tiled path of the
 * block-scaled numerics (numerics = 2) reads it. Single-token calls can read it too, in ANY numerics (the
 * activations ride as exact e2m1 pieces, so the results keep the reference's single-token arithmetic), but only
 * when OCO_MOE_REPACKED_TOKEN=1 is set: those kernels measured slower than the default ones and exist for
 * measurement. The staging step of the reference keeps the checkpoint's spans unchanged and repacks only what
 * its kernels cannot read in place (Buffer::from_bytes for repacked operands, src/gpu/buffer.rs:223); here the
 * repack is optional: without it the same numerics run from the GGUF spans, with producer warps moving bytes.
 *   oco_moe_repack_bytes   size of the caller's buffer (0: the plan's family has no use for it)
 *   oco_moe_bind_repacked  repacks the bound gate / up / down tensors into `buffer` (1024-byte aligned) and makes
 *                          the tiled path of this plan read them; buffer == NULL goes back to the spans.
 * Set-up call: synchronises the stream. Bind the weights first; bind again after re-binding weights. The
 * original tensors must stay bound (single-token calls and the router read them). */
size_t oco_moe_repack_bytes(const oco_moe_plan* plan);
int oco_moe_bind_repacked(oco_moe_plan* plan, void* buffer, size_t bytes, void* cuda_stream);

/* One forward call recorded as a CUDA graph and replayed with one launch: the counterpart of the
 * reference encoding a step's dispatches into one command buffer and committing it
 * (Compute::submit, src/weights/compute/submission.rs:21-107). A single-token step is three to five small
 * kernels and is bound by the host's launch rate when they are launched one by one.
 *   oco_moe_graph_capture  records oco_moe_forward(plan, x, residual, rows) (the same pointers on every
 *                          replay: the caller refreshes their contents). Set-up call: synchronises.
 *   oco_moe_graph_launch   enqueues one replay on the stream.
 * The plan, its workspace and its weights must outlive the graph and must not be re-bound while it lives. */
typedef struct oco_moe_graph oco_moe_graph;
int oco_moe_graph_capture(oco_moe_plan* plan, const uint16_t* x_bf16, uint16_t* residual_bf16, int rows, oco_moe_graph** out);
/* The same for pinned host buffers: the graph also holds the copies of x and the residual rows into the
 * workspace's first staging slot and the copy of the residual rows back, so one oco_moe_graph_launch (then a
 * wait on the stream) is a whole oco_moe_forward_host call: for single tokens the launches and copies of that
 * call cost the host about as much as the kernels take. The buffers must stay where they are while the graph
 * lives; no host call may be in flight while it is recorded or runs (they share the staging slot). */
int oco_moe_graph_capture_host(oco_moe_plan* plan, const uint16_t* x_bf16_host, uint16_t* residual_bf16_host, int rows,
                               oco_moe_graph** out);
int oco_moe_graph_launch(oco_moe_graph* graph, void* cuda_stream);
void oco_moe_graph_destroy(oco_moe_graph* graph);

/* The dense products either side of the MoE layer: the reference's DenseMatrix::apply
 * (src/weights/compute/matrix.rs:130-278) composed as its callers compose it.
 *   OCO_DENSE_PROJECTION     y[rows, ffn] = up_w . x, stored as bf16 (any of the three weight formats)
 *   OCO_DENSE_FFN_RELU2      Nemotron's always-on expert (compute/nemotron.rs:302-315 for rows > 1,
 *                            :460-509 for one token): up -> relu^2 -> down, Q4_0; y[rows, hidden]
 *   OCO_DENSE_FFN_SILU_GATE  the gated feed-forward of dense layers (Compute::feed_forward,
 *                            compute/feed_forward.rs:97-104; gate kernel shaders/elementwise.metal:70-87):
 *                            gate, up -> bf16(bf16(silu(g)) * u) -> down, Q4_K; y[rows, hidden]
 * Weights are packed rows as in the expert banks, one matrix each: up_w [ffn][hidden], gate_w the same
 * (gated kind only), down_w [hidden][ffn] (the two feed-forward kinds). The result is written, not added:
 * the reference leaves it in `projected` for the caller's add. rows == 1 runs the single-token kernels
 * with exact operands, rows > 1 the tiles with half operands, as the MoE layer does. Other pairs of kind
 * and format answer OCO_UNSUPPORTED_SHAPE. Plan, workspace and weights follow the rules of the oco_moe_
 * calls of the same names. */
typedef enum { OCO_DENSE_PROJECTION = 0, OCO_DENSE_FFN_RELU2 = 1, OCO_DENSE_FFN_SILU_GATE = 2 } oco_dense_kind;
typedef struct {
    int32_t kind;           /* oco_dense_kind */
    int32_t weight_format;  /* oco_weight_format */
    int32_t hidden;         /* input features */
    int32_t ffn;            /* projection: output features (a multiple of 32); feed-forward kinds: intermediate
                             * features (a multiple of the format's block, as hidden is) */
} oco_dense_desc;
typedef struct {
    const uint8_t* up_w;
    const uint8_t* gate_w;
    const uint8_t* down_w;
} oco_dense_weights;
typedef struct oco_dense_plan oco_dense_plan;
int oco_dense_plan_create(const oco_dense_desc* desc, oco_dense_plan** out);
void oco_dense_plan_destroy(oco_dense_plan* plan);
size_t oco_dense_workspace_bytes(const oco_dense_plan* plan, int max_rows);
int oco_dense_bind_workspace(oco_dense_plan* plan, void* workspace, size_t bytes, int max_rows);
int oco_dense_bind_weights(oco_dense_plan* plan, const oco_dense_weights* weights);
int oco_dense_forward(oco_dense_plan* plan, const uint16_t* x_bf16, uint16_t* y_bf16, int rows, void* cuda_stream);
int oco_dense_poll(oco_dense_plan* plan, void* cuda_stream);
int oco_dense_last_launch_count(const oco_dense_plan* plan);
const char* oco_dense_last_error(const oco_dense_plan* plan);

/* Expert parallelism without a collective on the rows' way. The reference is single-device; nothing
 * below has a counterpart in it.
 *
 * A window is one device address range of `world` slots, `slot_stride` bytes apart, slot g backed by
 * `backed_bytes` of GPU g's memory (the rest of a slot is unmapped and must not be touched). Every
 * rank creates its window with the same sizes, hands its descriptor (oco_ep_window_fd; a POSIX file
 * descriptor of this process, to be passed over a Unix socket with SCM_RIGHTS) to each peer, and
 * attaches the descriptors it receives. From then on base + g * slot_stride + offset addresses the
 * same bytes of GPU g's slot on every rank, through plain loads and stores over NVLink.
 * slot_stride must be a multiple of oco_ep_window_granularity. Set-up calls: they allocate and
 * synchronise. oco_ep_window_error returns the calling thread's last message. */
typedef struct oco_ep_window oco_ep_window;
int oco_ep_window_granularity(size_t* bytes);
int oco_ep_window_create(int rank, int world, size_t slot_stride, size_t backed_bytes, oco_ep_window** out);
int oco_ep_window_fd(const oco_ep_window* window);
int oco_ep_window_attach(oco_ep_window* window, int peer, int fd);
void* oco_ep_window_base(const oco_ep_window* window);
size_t oco_ep_window_stride(const oco_ep_window* window);
size_t oco_ep_window_backed(const oco_ep_window* window);
void oco_ep_window_destroy(oco_ep_window* window);
const char* oco_ep_window_error(void);

/* oco_moe_experts over routes numbered in a window. Route i of the call (0 <= i < routes) goes to
 * expert expert_ids[i] of this plan; an id outside 0 .. experts-1 marks a route that belongs to
 * another shard and is skipped. The route's label is (i / seg_routes) * seg_stride + i % seg_routes
 * (seg_routes 0: i itself): its input is row label / routes_per_row of token_rows_bf16, its output
 * lands in row label of y_bf16. With token rows in one window (slot stride seg_stride /
 * routes_per_row rows) and outputs in another (slot stride seg_stride rows), source rank g's
 * seg_routes routes are gathered from GPU g and answered into GPU g's memory by this one call.
 * routes <= max_rows * top_k; expected_routes (0: all) is how many of them this shard expects to
 * own, which picks the kernels. Ordering between ranks (inputs written before a peer reads them,
 * outputs complete before their owner combines them) is the caller's, by collectives or events on
 * the streams. */
int oco_moe_experts_window(oco_moe_plan* plan, const uint16_t* token_rows_bf16, const uint32_t* expert_ids, int routes,
                           int routes_per_row, int seg_routes, int seg_stride, int expected_routes, uint16_t* y_bf16,
                           void* cuda_stream);

const char* oco_moe_version(void);

#ifdef __cplusplus
}
#endif
#endif /* OCO_MOE_H */
