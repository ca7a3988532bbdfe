"""Host-side mirror of the reference's dense products for the steps either side of the MoE layer:
`DenseMatrix::apply` (src/weights/compute/matrix.rs:130-278), `Compute::feed_forward`
(src/weights/compute/feed_forward.rs:97-104) and Nemotron's always-on expert
(src/weights/compute/nemotron.rs:302-315, 460-509), through the C ABI (oco_dense_*). The CUDA
library does all arithmetic; there is no CPU fallback."""
from __future__ import annotations

import ctypes as C
from typing import Optional

import numpy as np
import torch

from . import _lib
from .moe import OcoError, _dev_bytes, _ptr, _stream_ptr

PROJECTION, FFN_RELU2, FFN_SILU_GATE = 0, 1, 2


class DensePlan:
    """Owns the C plan, its workspace and the staged weights of one dense projection or feed-forward."""

    def __init__(self, kind: int, fmt: int, hidden: int, ffn: int):
        self.kind, self.fmt, self.hidden, self.ffn = kind, fmt, hidden, ffn
        self.desc = _lib.DenseDesc(kind=kind, weight_format=fmt, hidden=hidden, ffn=ffn)
        self.handle = C.c_void_p()
        rc = _lib.lib().oco_dense_plan_create(C.byref(self.desc), C.byref(self.handle))
        if rc != _lib.OK:
            msg = _lib.lib().oco_dense_last_error(self.handle).decode() if self.handle else "plan_create failed"
            if self.handle:
                _lib.lib().oco_dense_plan_destroy(self.handle)
                self.handle = C.c_void_p()
            raise OcoError(rc, msg)
        self.workspace = None
        self.max_rows = 0
        self._weights = None

    def _check(self, rc):
        if rc != _lib.OK:
            raise OcoError(rc, _lib.lib().oco_dense_last_error(self.handle).decode())

    def reserve(self, max_rows: int, device="cuda"):
        if self.workspace is not None and max_rows <= self.max_rows:
            return
        nbytes = _lib.lib().oco_dense_workspace_bytes(self.handle, max_rows)
        self.workspace = torch.empty(nbytes, dtype=torch.uint8, device=device)
        self._check(_lib.lib().oco_dense_bind_workspace(self.handle, _ptr(self.workspace), nbytes, max_rows))
        self.max_rows = max_rows

    def bind(self, up_w: np.ndarray, gate_w: Optional[np.ndarray] = None, down_w: Optional[np.ndarray] = None, device="cuda"):
        """Packed rows as they sit in the file: up_w [ffn][hidden], gate_w the same, down_w [hidden][ffn]."""
        staged = tuple(_dev_bytes(a, device) for a in (up_w, gate_w, down_w))
        cw = _lib.DenseWeights(*[C.cast(C.c_void_p(t.data_ptr()), C.POINTER(C.c_uint8)) if t is not None else None for t in staged])
        self._check(_lib.lib().oco_dense_bind_weights(self.handle, C.byref(cw)))
        self._weights = staged

    def forward(self, x: torch.Tensor, y: torch.Tensor, rows: int):
        """x: bf16 bit patterns [rows, hidden]; y receives [rows, ffn] (projection) or [rows, hidden]."""
        self._check(_lib.lib().oco_dense_forward(self.handle, _ptr(x), _ptr(y), rows, _stream_ptr()))

    def poll(self):
        self._check(_lib.lib().oco_dense_poll(self.handle, _stream_ptr()))

    def launch_count(self) -> int:
        return _lib.lib().oco_dense_last_launch_count(self.handle)

    def __del__(self):
        try:
            if self.handle:
                _lib.lib().oco_dense_plan_destroy(self.handle)
                self.handle = C.c_void_p()
        except Exception:
            pass


def apply(plan: DensePlan, x_bits: np.ndarray, device="cuda") -> np.ndarray:
    """One call with host arrays: bf16 bit patterns [rows, hidden] in, the result's bit patterns out."""
    rows = x_bits.shape[0]
    plan.reserve(rows, device)
    x = torch.from_numpy(np.ascontiguousarray(x_bits).view(np.int16)).to(device)
    y = torch.empty((rows, plan.ffn if plan.kind == PROJECTION else plan.hidden), dtype=torch.int16, device=device)
    plan.forward(x, y, rows)
    torch.cuda.synchronize()
    plan.poll()
    return y.cpu().numpy().view(np.uint16)
