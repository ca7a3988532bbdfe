"""Host-side mirror of the reference's expert-layer operators over the C ABI.

Names and argument meaning follow the reference (Rust, `src/weights/compute/feed_forward.rs`,
`src/weights/compute/nemotron.rs`, `src/weights/state.rs`, `src/weights/gpt_oss.rs`,
`src/weights/nemotron.rs`):

    ExpertPlan.new(hidden, ffn_width)                      <- ExpertPlan::new
    ReluExpertPlan.new(hidden, expert_width, shared_width, experts, active, normalize, scale)
                                                          <- ReluExpertPlan::new
    Experts / ReluExperts                                  <- the weight structs (device buffers)
    Routing                                                <- Routing{ids, plan, prob}: side outputs
    Bindings(scratch).experts(w, plan, routing, residual, rows)
    Bindings(scratch).relu_experts(w, plan, routing, residual, rows)

The input rows are `scratch.norm` (bf16 [rows, hidden]) and the result is accumulated into the
bf16 residual rows in place, as in the reference. PyTorch is used only to own device memory and
streams; every computation happens inside liboco_moe.so.
"""
from __future__ import annotations

import ctypes as C
import warnings
from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from . import _lib, synth
from ._lib import OcoError

ACTIVE_EXPERTS = 4   # reference src/weights/gpt_oss.rs:15
EXPERT_COUNT = 32    # reference src/weights/gpt_oss.rs:14


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream_ptr():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _dev_bytes(a: Optional[np.ndarray], device, misalign: int = 0) -> Optional[torch.Tensor]:
    """Stages a host array on the device byte for byte (the GGUF spans stay unchanged).
    `misalign` places the first byte that many bytes past a 256-byte boundary, the way GGUF tensors
    sit at arbitrary offsets of a mapped file (reference test: src/weights/dispatch_tests/mxfp4.rs:16)."""
    if a is None:
        return None
    a = np.ascontiguousarray(a)
    with warnings.catch_warnings():
        # views of a read-only file map are only read here (copied to the device)
        warnings.simplefilter("ignore", UserWarning)
        flat = torch.from_numpy(a.view(np.uint8).reshape(-1))
    if not misalign:
        return flat.to(device)
    buf = torch.full((flat.numel() + misalign + 64,), 0xA5, dtype=torch.uint8, device=device)
    buf[misalign:misalign + flat.numel()] = flat.to(device)
    return buf[misalign:misalign + flat.numel()]


class StepGraph:
    """A recorded forward step (oco_moe_graph_*); keeps its plan and buffers alive."""

    def __init__(self, plan, handle, keep):
        self.plan, self.handle, self._keep = plan, handle, keep

    def replay(self):
        self.plan._check(_lib.lib().oco_moe_graph_launch(self.handle, _stream_ptr()))

    def __del__(self):
        try:
            if self.handle:
                _lib.lib().oco_moe_graph_destroy(self.handle)
                self.handle = C.c_void_p()
        except Exception:
            pass


class _Plan:
    """Owns the C plan object, its workspace and the bound weights."""

    def __init__(self, arch, hidden, ffn, experts, top_k, fmt, shared_ffn=0, normalize=False, scale=1.0,
                 gemm_impl=0, numerics=0):
        self.desc = _lib.Desc(arch=arch, hidden=hidden, ffn=ffn, experts=experts, top_k=top_k,
                              shared_ffn=shared_ffn, weight_format=fmt, normalize=int(bool(normalize)),
                              scale=float(scale), gemm_impl=gemm_impl, numerics=numerics)
        self.handle = C.c_void_p()
        rc = _lib.lib().oco_moe_plan_create(C.byref(self.desc), C.byref(self.handle))
        if rc != _lib.OK:
            msg = _lib.lib().oco_moe_last_error(self.handle).decode() if self.handle else "plan_create failed"
            if self.handle:
                _lib.lib().oco_moe_plan_destroy(self.handle)
                self.handle = C.c_void_p()
            raise OcoError(rc, msg)
        self.workspace = None
        self.max_rows = 0
        self._weights = None

    def _check(self, rc):
        if rc != _lib.OK:
            raise OcoError(rc, _lib.lib().oco_moe_last_error(self.handle).decode())

    def reserve(self, max_rows: int, device="cuda"):
        """Session-time workspace (reference `Memory::new`, src/weights/gpt_oss.rs:48-91)."""
        if self.workspace is not None and max_rows <= self.max_rows:
            return
        nbytes = _lib.lib().oco_moe_workspace_bytes(self.handle, max_rows)
        self.workspace = torch.empty(nbytes, dtype=torch.uint8, device=device)
        self._check(_lib.lib().oco_moe_bind_workspace(self.handle, _ptr(self.workspace), nbytes, max_rows))
        self.max_rows = max_rows

    def bind(self, w: "_Weights"):
        if self._weights is w:
            return
        cw = _lib.Weights(**{k: (getattr(w, k).data_ptr() if getattr(w, k) is not None else None)
                             for k, _ in _lib.Weights._fields_})
        self._check(_lib.lib().oco_moe_bind_weights(self.handle, C.byref(cw)))
        self._weights = w

    def forward(self, x: torch.Tensor, residual: torch.Tensor, rows: int):
        self._check(_lib.lib().oco_moe_forward(self.handle, _ptr(x), _ptr(residual), rows, _stream_ptr()))

    def add_norm_forward(self, hidden: torch.Tensor, projected: Optional[torch.Tensor], norm_weight: torch.Tensor,
                         epsilon: float, full_layer: bool, rows: int):
        """hidden += projected; x = rmsnorm(hidden) * norm_weight; hidden += MoE(x) (reference
        `Bindings::add_norm` + `Bindings::experts`, src/weights/compute.rs:100-117, gpt_oss.rs:122-123)."""
        self._check(_lib.lib().oco_moe_add_norm_forward(self.handle, _ptr(hidden), _ptr(projected) if projected is not None else None,
                                                        _ptr(norm_weight), C.c_float(epsilon), int(bool(full_layer)), rows,
                                                        _stream_ptr()))

    def forward_host(self, x: np.ndarray, residual: np.ndarray, rows: int):
        self._check(_lib.lib().oco_moe_forward_host(self.handle, x.ctypes.data_as(C.c_void_p),
                                                    residual.ctypes.data_as(C.c_void_p), rows, _stream_ptr()))

    def forward_host_begin(self, x: np.ndarray, residual: np.ndarray, rows: int):
        """Queue the layer on host buffers (up to two calls in flight); `residual` is the caller's again after
        the matching forward_host_end."""
        self._check(_lib.lib().oco_moe_forward_host_begin(self.handle, x.ctypes.data_as(C.c_void_p),
                                                          residual.ctypes.data_as(C.c_void_p), rows, _stream_ptr()))

    def forward_host_end(self):
        self._check(_lib.lib().oco_moe_forward_host_end(self.handle))

    def repack(self, device="cuda"):
        """The optional second form of the expert tensors for numerics 2 (oco_moe_bind_repacked)."""
        nbytes = _lib.lib().oco_moe_repack_bytes(self.handle)
        if nbytes == 0:
            raise OcoError(_lib.UNSUPPORTED_SHAPE, "this plan has no use for repacked weights")
        self._repacked = torch.empty(nbytes + 1024, dtype=torch.uint8, device=device)
        base = (self._repacked.data_ptr() + 1023) & ~1023
        self._check(_lib.lib().oco_moe_bind_repacked(self.handle, C.c_void_p(base), nbytes, _stream_ptr()))
        return base, nbytes

    def capture(self, x: torch.Tensor, residual: torch.Tensor, rows: int) -> "StepGraph":
        """The forward call on these buffers as a graph of the library (one launch per replay)."""
        g = C.c_void_p()
        self._check(_lib.lib().oco_moe_graph_capture(self.handle, _ptr(x), _ptr(residual), rows, C.byref(g)))
        return StepGraph(self, g, (x, residual))

    def capture_host(self, x: np.ndarray, residual: np.ndarray, rows: int) -> "StepGraph":
        """The forward call on these pinned host buffers, copies included, as a graph of the library."""
        g = C.c_void_p()
        self._check(_lib.lib().oco_moe_graph_capture_host(self.handle, x.ctypes.data_as(C.c_void_p),
                                                          residual.ctypes.data_as(C.c_void_p), rows, C.byref(g)))
        return StepGraph(self, g, (x, residual))

    def poll(self):
        self._check(_lib.lib().oco_moe_poll(self.handle, _stream_ptr()))

    def launch_count(self) -> int:
        return _lib.lib().oco_moe_last_launch_count(self.handle)

    def set_profiling(self, enabled: bool):
        """Per-kernel device timestamps (reference `OCO_PROFILE`, src/gpu/profile.rs)."""
        self._check(_lib.lib().oco_moe_set_profiling(self.handle, int(enabled)))

    def phase_times(self) -> dict:
        """Milliseconds per phase of the last forward call; the stream must have been waited for."""
        ms = (C.c_float * 16)()
        names = (C.c_char_p * 16)()
        n = _lib.lib().oco_moe_phase_times(self.handle, 16, ms, names)
        return {names[i].decode(): float(ms[i]) for i in range(max(n, 0))}

    def __del__(self):
        try:
            if self.handle:
                _lib.lib().oco_moe_plan_destroy(self.handle)
        except Exception:
            pass


class ExpertPlan(_Plan):
    """gpt-oss expert geometry (reference `ExpertPlan`, feed_forward.rs:34-77)."""

    @classmethod
    def new(cls, hidden: int, ffn_width: int, experts: int = EXPERT_COUNT, active: int = ACTIVE_EXPERTS,
            gemm_impl: int = 0, numerics: int = 0) -> "ExpertPlan":
        return cls(synth.ARCH_GPT_OSS, hidden, ffn_width, experts, active, synth.FMT_MXFP4, gemm_impl=gemm_impl, numerics=numerics)

    def width(self) -> int:
        return self.desc.ffn


class ReluExpertPlan(_Plan):
    """Routed relu^2 expert geometry (reference `ReluExpertPlan`, compute/nemotron.rs:131-198)."""

    @classmethod
    def new(cls, hidden, expert_width, shared_width, experts, active, normalize, scale, gemm_impl=0):
        return cls(synth.ARCH_NEMOTRON, hidden, expert_width, experts, active, synth.FMT_Q4_0,
                   shared_ffn=shared_width, normalize=normalize, scale=scale, gemm_impl=gemm_impl)

    def active(self) -> int:
        return self.desc.top_k

    def experts(self) -> int:
        return self.desc.experts

    def expert_width(self) -> int:
        return self.desc.ffn


class GatedExpertPlan(_Plan):
    """SiLU-gated Q4_K experts with softmax-all / top-k-renormalised routing (Qwen3-MoE shaped).
    The reference has no operator for this family; the plan follows the other two."""

    @classmethod
    def new(cls, hidden, expert_width, experts, active, gemm_impl=0):
        return cls(synth.ARCH_QWEN, hidden, expert_width, experts, active, synth.FMT_Q4_K, gemm_impl=gemm_impl)


@dataclass
class _Weights:
    router_w: Optional[torch.Tensor] = None
    router_b: Optional[torch.Tensor] = None
    gate_w: Optional[torch.Tensor] = None
    up_w: Optional[torch.Tensor] = None
    down_w: Optional[torch.Tensor] = None
    gate_b: Optional[torch.Tensor] = None
    up_b: Optional[torch.Tensor] = None
    down_b: Optional[torch.Tensor] = None
    shared_up_w: Optional[torch.Tensor] = None
    shared_down_w: Optional[torch.Tensor] = None
    gate_up_w: Optional[torch.Tensor] = None   # one tensor, rows interleaved: 2c = gate row c, 2c + 1 = up row c
    gate_up_b: Optional[torch.Tensor] = None

    @classmethod
    def from_layer(cls, layer: synth.Layer, device="cuda", misalign: int = 0, interleaved: bool = False):
        """Uploads a host layer unchanged (reference `import()` / `MappedRegions::new`,
        src/gpu/buffer.rs:151-194: the GGUF bytes are registered, never repacked). `misalign`
        applies to the packed expert banks only; f32 tensors keep their natural alignment.
        `interleaved` stages gate and up as one tensor with alternating rows (and biases)."""
        packed = ("gate_w", "up_w", "down_w", "shared_up_w", "shared_down_w")
        names = ["router_w", "router_b", "gate_w", "up_w", "down_w", "gate_b", "up_b", "down_b", "shared_up_w", "shared_down_w"]
        if interleaved and layer.gate_w is not None:
            E, F, rb = layer.gate_w.shape
            both = np.empty((E, 2 * F, rb), np.uint8)
            both[:, 0::2], both[:, 1::2] = layer.gate_w, layer.up_w
            out = cls(**{k: _dev_bytes(getattr(layer, k), device, misalign if k in packed else 0)
                         for k in names if k not in ("gate_w", "up_w", "gate_b", "up_b")})
            out.gate_up_w = _dev_bytes(both, device, misalign)
            if layer.gate_b is not None:
                bias = np.empty((E, 2 * F), np.float32)
                bias[:, 0::2], bias[:, 1::2] = layer.gate_b, layer.up_b
                out.gate_up_b = _dev_bytes(bias, device)
            return out
        return cls(**{k: _dev_bytes(getattr(layer, k), device, misalign if k in packed else 0) for k in names})


class Experts(_Weights):
    """reference `Experts{gate, up, down, router}` (src/weights/gpt_oss.rs:33-38)."""


class ReluExperts(_Weights):
    """reference `ReluExperts{router, up, down, shared_up, shared_down}` (src/weights/nemotron.rs:60-66)."""


def operand_order(fmt: int, n: int) -> np.ndarray:
    """Column of element k in rows kept in the tile kernels' operand order: a packed code byte holds
    elements j and j + h of its block (h = 16, or 32 for Q4_K), and the tiles keep the two adjacent."""
    k = np.arange(n)
    if fmt == synth.FMT_Q4_K:
        return (k & ~63) + (((k & 31) << 1) | ((k >> 5) & 1))
    return (k & ~31) + (((k & 15) << 1) | ((k >> 4) & 1))


class Routing:
    """Expert selections and combination weights of the last call (reference `Routing`,
    src/weights/state.rs:112-117), read back from the plan's workspace."""

    def __init__(self):
        self.plan: Optional[_Plan] = None
        self.rows = 0

    def _view(self):
        v = _lib.RoutingView()
        rc = _lib.lib().oco_moe_routing(self.plan.handle, C.byref(v))
        if rc != _lib.OK:
            raise OcoError(rc, "no routing available")
        return v

    def _read(self, ptr, count, dtype):
        out = np.empty(count, dtype)
        torch.cuda.current_stream().synchronize()
        rc = _lib.lib().oco_cuda_download(out.ctypes.data_as(C.c_void_p), C.c_void_p(ptr), out.nbytes, _stream_ptr())
        if rc != _lib.OK:
            raise OcoError(rc, "download failed")
        torch.cuda.current_stream().synchronize()
        return out

    def read(self) -> dict:
        d = self.plan.desc
        v = self._view()
        R = self.rows * d.top_k
        out = dict(ids=self._read(v.ids, R, np.uint32).reshape(self.rows, d.top_k),
                   prob=self._read(v.probs, R, np.float32).reshape(self.rows, d.top_k),
                   logits=self._read(v.logits, self.rows * d.experts, np.float32).reshape(self.rows, d.experts),
                   y=self._read(v.y, R * d.hidden, np.uint16).reshape(R, d.hidden),
                   norm=self._read(v.norm, self.rows * d.hidden, np.uint16).reshape(self.rows, d.hidden))
        if self.rows > 1:
            out["offsets"] = self._read(v.offsets, d.experts + 1, np.uint32)
            out["row_of_route"] = self._read(v.row_of_route, R, np.uint32)
            out["route_of_row"] = self._read(v.route_of_row, R, np.uint32)
            n = int(self._read(v.tile_count, 1, np.uint32)[0])
            out["tiles"] = self._read(v.tiles, 2 * n, np.uint32).reshape(n, 2)
            act = self._read(v.act, R * d.ffn, np.uint16).reshape(R, d.ffn)
            out["act"] = act[:, operand_order(d.weight_format, d.ffn)]   # back to element order
        return out


@dataclass
class Scratch:
    """The slice of the reference's `CommonScratch` this path reads (src/weights/state.rs:148-177)."""
    norm: torch.Tensor  # bf16 [rows, hidden]: the layer's input rows


class Bindings:
    """reference `Bindings{kernels, scratch, encoder}` (src/weights/compute.rs:58-62): the encoder
    is the current CUDA stream."""

    def __init__(self, scratch: Scratch):
        self.scratch = scratch

    def _run(self, w: _Weights, plan: _Plan, routing: Optional[Routing], residual: torch.Tensor, rows: int):
        if rows < 1:
            raise OcoError(_lib.INVALID_ARGUMENT, "rows must be at least 1")
        plan.reserve(max(rows, plan.max_rows), residual.device)
        plan.bind(w)
        plan.forward(self.scratch.norm, residual, rows)
        if routing is not None:
            routing.plan, routing.rows = plan, rows

    def experts(self, w: Experts, plan: ExpertPlan, routing: Optional[Routing], residual: torch.Tensor, rows: int):
        """Route each token to its experts and add their weighted contributions to its features
        (reference `Bindings::experts`, feed_forward.rs:106-114)."""
        self._run(w, plan, routing, residual, rows)

    def relu_experts(self, w: ReluExperts, plan: ReluExpertPlan, routing: Optional[Routing],
                     residual: torch.Tensor, rows: int):
        """Add the shared expert and the weighted routed experts to the residual rows
        (reference `Bindings::relu_experts`, compute/nemotron.rs:285-293)."""
        self._run(w, plan, routing, residual, rows)

    def gated_experts(self, w: _Weights, plan: GatedExpertPlan, routing: Optional[Routing],
                      residual: torch.Tensor, rows: int):
        self._run(w, plan, routing, residual, rows)


def plan_for(layer: synth.Layer, gemm_impl: int = 0, numerics: int = 0) -> _Plan:
    if layer.arch == synth.ARCH_GPT_OSS:
        return ExpertPlan.new(layer.hidden, layer.ffn, layer.experts, layer.top_k, gemm_impl, numerics)
    if layer.arch == synth.ARCH_NEMOTRON:
        return ReluExpertPlan.new(layer.hidden, layer.ffn, layer.shared_ffn, layer.experts, layer.top_k,
                                  layer.normalize, layer.scale, gemm_impl)
    return GatedExpertPlan.new(layer.hidden, layer.ffn, layer.experts, layer.top_k, gemm_impl)


def run_layer(layer: synth.Layer, x_bits: np.ndarray, residual_bits: np.ndarray, gemm_impl: int = 0,
              device="cuda", state: Optional[dict] = None, misalign: int = 0, interleaved: bool = False, numerics: int = 0,
              repacked: bool = False):
    """Convenience used by tests and the benchmark: uploads (or reuses) a layer, runs it on bf16
    bit patterns given as uint16 arrays and returns (residual bits, routing dict)."""
    state = state if state is not None else {}
    if "plan" not in state:
        state["plan"] = plan_for(layer, gemm_impl, numerics)
        state["weights"] = _Weights.from_layer(layer, device, misalign, interleaved)
    plan, w = state["plan"], state["weights"]
    if repacked and not state.get("repacked"):
        plan.reserve(x_bits.shape[0], device)
        plan.bind(w)
        plan.repack(device)
        state["repacked"] = True
    rows = x_bits.shape[0]
    x = torch.from_numpy(np.ascontiguousarray(x_bits).view(np.int16)).to(device)
    res = torch.from_numpy(np.ascontiguousarray(residual_bits).view(np.int16).copy()).to(device)
    routing = Routing()
    b = Bindings(Scratch(norm=x))
    b._run(w, plan, routing, res, rows)
    plan.poll()
    return res.cpu().numpy().view(np.uint16), routing.read()


def dequant(fmt: int, packed: np.ndarray, n_elems: int, half: bool = False, device="cuda") -> np.ndarray:
    w = _dev_bytes(packed, device)
    out = torch.empty(n_elems, dtype=torch.int16 if half else torch.float32, device=device)
    fn = _lib.lib().oco_moe_dequant_f16 if half else _lib.lib().oco_moe_dequant_f32
    rc = fn(fmt, _ptr(w), n_elems, _ptr(out), _stream_ptr())
    if rc != _lib.OK:
        raise OcoError(rc, "dequant failed")
    torch.cuda.synchronize()
    r = out.cpu().numpy()
    return r.view(np.uint16) if half else r
