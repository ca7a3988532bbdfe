"""ctypes binding of the CPU oracle (``moe_oracle.cpp``).

Test infrastructure only: the product package never imports this module. It is loaded by the
test-suite, by the smoke check and by the benchmark's CPU-baseline leg, always as the checker or
as the timed CPU arm, never as part of the GPU path.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass
from typing import Optional

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libmoe_oracle.so")

FMT_Q4_0, FMT_Q4_K, FMT_MXFP4 = 2, 12, 39
ARCH_GPT_OSS, ARCH_NEMOTRON, ARCH_QWEN = 0, 1, 2


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside it (g++ only, no external libraries)."""
    src = os.path.join(_HERE, "moe_oracle.cpp")
    newest = max(os.path.getmtime(src), os.path.getmtime(os.path.join(_HERE, "Makefile")))
    stale = (not os.path.exists(_LIB_PATH)) or os.path.getmtime(_LIB_PATH) < newest
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B", "libmoe_oracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


class _Layer(C.Structure):
    _fields_ = [
        ("arch", C.c_int32), ("hidden", C.c_int32), ("ffn", C.c_int32), ("experts", C.c_int32),
        ("top_k", C.c_int32), ("shared_ffn", C.c_int32), ("fmt", C.c_int32),
        ("normalize", C.c_int32), ("scale", C.c_float), ("reserved", C.c_int32),
        ("router_w", C.c_void_p), ("router_b", C.c_void_p),
        ("gate_w", C.c_void_p), ("up_w", C.c_void_p), ("down_w", C.c_void_p),
        ("gate_b", C.c_void_p), ("up_b", C.c_void_p), ("down_b", C.c_void_p),
        ("shared_up_w", C.c_void_p), ("shared_down_w", C.c_void_p),
    ]


class _Trace(C.Structure):
    _fields_ = [("logits", C.c_void_p), ("ids", C.c_void_p), ("probs", C.c_void_p),
                ("act", C.c_void_p), ("y", C.c_void_p)]


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        L.orc_f32_to_bf16.argtypes = [C.c_float]; L.orc_f32_to_bf16.restype = C.c_uint16
        L.orc_bf16_to_f32.argtypes = [C.c_uint16]; L.orc_bf16_to_f32.restype = C.c_float
        L.orc_f32_to_f16.argtypes = [C.c_float]; L.orc_f32_to_f16.restype = C.c_uint16
        L.orc_f16_to_f32.argtypes = [C.c_uint16]; L.orc_f16_to_f32.restype = C.c_float
        L.orc_exp.argtypes = [C.c_float]; L.orc_exp.restype = C.c_float
        L.orc_swiglu_clipped.argtypes = [C.c_float, C.c_float]; L.orc_swiglu_clipped.restype = C.c_float
        L.orc_silu_gate_bf16.argtypes = [C.c_float, C.c_float]; L.orc_silu_gate_bf16.restype = C.c_float
        L.orc_dequant.argtypes = [C.c_int, C.c_void_p, C.c_size_t, C.c_void_p]
        L.orc_dequant_f16.argtypes = [C.c_int, C.c_void_p, C.c_size_t, C.c_void_p]
        L.orc_router_gptoss.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                        C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
        L.orc_router_sigmoid.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                         C.c_int, C.c_int, C.c_float, C.c_void_p, C.c_void_p, C.c_void_p]
        L.orc_router_softmax_topk.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                              C.c_void_p, C.c_void_p, C.c_void_p]
        L.orc_route_plan_tiled_words.argtypes = [C.c_uint32]; L.orc_route_plan_tiled_words.restype = C.c_size_t
        L.orc_route_plan_tiled.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p]
        L.orc_route_plan_n_words.argtypes = [C.c_uint32, C.c_uint32, C.c_uint32]
        L.orc_route_plan_n_words.restype = C.c_size_t
        L.orc_route_plan_n.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,
                                       C.c_uint32, C.c_void_p]
        L.orc_permutation.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p]
        L.orc_moe_forward.argtypes = [C.POINTER(_Layer), C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                      C.POINTER(_Trace)]
        L.orc_moe_forward.restype = C.c_int
        L.orc_expert_expand.argtypes = [C.c_void_p] * 6 + [C.c_int] * 4 + [C.c_void_p] * 2
        L.orc_expert_down_vector.argtypes = [C.c_void_p] * 4 + [C.c_int] * 5 + [C.c_void_p]
        L.orc_expert_up_tile.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_void_p] + \
            [C.c_int] * 5 + [C.c_void_p]
        L.orc_expert_down_tile.argtypes = [C.c_void_p] * 4 + [C.c_int] * 4 + [C.c_void_p]
        L.orc_moe_activate.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
        L.orc_moe_sum.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]
        L.orc_moe_add.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]
        L.orc_dense_forward.argtypes = [C.c_int] * 4 + [C.c_void_p] * 4 + [C.c_int] * 2 + [C.c_void_p]
        L.orc_num_threads.restype = C.c_int
        L.orc_set_num_threads.argtypes = [C.c_int]
        _lib = L
    return _lib


def _p(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dtype):
    return np.ascontiguousarray(a, dtype=dtype)


# ---- scalar / array conversions -------------------------------------------------------------
def f32_to_bf16(a) -> np.ndarray:
    a = _c(a, np.float32)
    f = np.vectorize(lambda v: lib().orc_f32_to_bf16(float(v)), otypes=[np.uint16])
    return f(a) if a.size < 4096 else _bf16_fast(a)


def _bf16_fast(a: np.ndarray) -> np.ndarray:
    u = a.view(np.uint32).astype(np.uint64)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    r[nan] = ((u[nan] >> 16) | 0x40).astype(np.uint16)
    return r


def bf16_to_f32(a) -> np.ndarray:
    return (_c(a, np.uint16).astype(np.uint32) << 16).view(np.float32)


def dequant(fmt: int, packed: np.ndarray, n_elems: int) -> np.ndarray:
    packed = _c(packed, np.uint8)
    out = np.empty(n_elems, np.float32)
    lib().orc_dequant(fmt, _p(packed), n_elems, _p(out))
    return out


def dequant_f16(fmt: int, packed: np.ndarray, n_elems: int) -> np.ndarray:
    packed = _c(packed, np.uint8)
    out = np.empty(n_elems, np.uint16)
    lib().orc_dequant_f16(fmt, _p(packed), n_elems, _p(out))
    return out


# ---- routers ---------------------------------------------------------------------------------
def router_gptoss(x_bf16, W, bias, top_k=4):
    x_bf16 = _c(x_bf16, np.uint16); W = _c(W, np.float32); bias = _c(bias, np.float32)
    T, H = x_bf16.shape; E = W.shape[0]
    logits = np.empty((T, E), np.float32); ids = np.empty((T, top_k), np.uint32)
    probs = np.empty((T, top_k), np.float32)
    lib().orc_router_gptoss(_p(x_bf16), _p(W), _p(bias), T, H, E, top_k, _p(logits), _p(ids), _p(probs))
    return logits, ids, probs


def router_sigmoid(x_bf16, W, sel_bias, active, normalize, scale):
    x_bf16 = _c(x_bf16, np.uint16); W = _c(W, np.float32); sel_bias = _c(sel_bias, np.float32)
    T, H = x_bf16.shape; E = W.shape[0]
    logits = np.empty((T, E), np.float32); ids = np.empty((T, active), np.uint32)
    probs = np.empty((T, active), np.float32)
    lib().orc_router_sigmoid(_p(x_bf16), _p(W), _p(sel_bias), T, H, E, active, int(normalize),
                             float(scale), _p(logits), _p(ids), _p(probs))
    return logits, ids, probs


def router_softmax_topk(x_bf16, W, active):
    x_bf16 = _c(x_bf16, np.uint16); W = _c(W, np.float32)
    T, H = x_bf16.shape; E = W.shape[0]
    logits = np.empty((T, E), np.float32); ids = np.empty((T, active), np.uint32)
    probs = np.empty((T, active), np.float32)
    lib().orc_router_softmax_topk(_p(x_bf16), _p(W), T, H, E, active, _p(logits), _p(ids), _p(probs))
    return logits, ids, probs


# ---- plans -----------------------------------------------------------------------------------
def route_plan_tiled(ids, tile_rows, up_tiles, down_tiles):
    ids = _c(ids, np.uint32).ravel()
    R = ids.size
    plan = np.zeros(lib().orc_route_plan_tiled_words(R), np.uint32)
    lib().orc_route_plan_tiled(_p(ids), R, tile_rows, up_tiles, down_tiles, _p(plan))
    return plan


def route_plan_n(ids, experts, tile_rows, up_tiles, down_tiles):
    ids = _c(ids, np.uint32).ravel()
    R = ids.size
    plan = np.zeros(lib().orc_route_plan_n_words(R, experts, tile_rows), np.uint32)
    lib().orc_route_plan_n(_p(ids), R, experts, tile_rows, up_tiles, down_tiles, _p(plan))
    return plan


def permutation(ids, experts):
    ids = _c(ids, np.uint32).ravel()
    R = ids.size
    offsets = np.empty(experts + 1, np.uint32)
    row_of_route = np.empty(R, np.uint32); route_of_row = np.empty(R, np.uint32)
    lib().orc_permutation(_p(ids), R, experts, _p(offsets), _p(row_of_route), _p(route_of_row))
    return offsets, row_of_route, route_of_row


# ---- kernel-level primitives -----------------------------------------------------------------
def expert_expand(uw, gw, x_bf16, ub, gb, ids, k, n, fmt=FMT_MXFP4):
    uw = _c(uw, np.uint8); gw = _c(gw, np.uint8); x_bf16 = _c(x_bf16, np.uint16)
    ub = _c(ub, np.float32); gb = _c(gb, np.float32); ids = _c(ids, np.uint32)
    uy = np.empty((ids.size, n), np.float32); gy = np.empty((ids.size, n), np.float32)
    lib().orc_expert_expand(_p(uw), _p(gw), _p(x_bf16), _p(ub), _p(gb), _p(ids), ids.size, k, n, fmt,
                            _p(uy), _p(gy))
    return uy, gy


def expert_down_vector(w, x_f32, bias, ids, k, n, fmt=FMT_MXFP4, relu2=False):
    w = _c(w, np.uint8); x_f32 = _c(x_f32, np.float32); ids = _c(ids, np.uint32)
    bias = None if bias is None else _c(bias, np.float32)
    y = np.empty((ids.size, n), np.uint16)
    lib().orc_expert_down_vector(_p(w), _p(x_f32), _p(bias), _p(ids), ids.size, k, n, fmt, int(relu2), _p(y))
    return y


def expert_up_tile(w, x_bf16, bias, shift, ids, per_token, k, n, fmt=FMT_MXFP4):
    w = _c(w, np.uint8); x_bf16 = _c(x_bf16, np.uint16); ids = _c(ids, np.uint32)
    bias = None if bias is None else _c(bias, np.float32)
    y = np.empty((ids.size, n), np.float32)
    lib().orc_expert_up_tile(_p(w), _p(x_bf16), _p(bias), float(shift), _p(ids), ids.size, per_token, k, n,
                             fmt, _p(y))
    return y


def expert_down_tile(w, act_f16, bias, ids, k, n, fmt=FMT_MXFP4):
    w = _c(w, np.uint8); act_f16 = _c(act_f16, np.uint16); ids = _c(ids, np.uint32)
    bias = None if bias is None else _c(bias, np.float32)
    y = np.empty((ids.size, n), np.uint16)
    lib().orc_expert_down_tile(_p(w), _p(act_f16), _p(bias), _p(ids), ids.size, k, n, fmt, _p(y))
    return y


def moe_activate(g, u):
    g = _c(g, np.float32); u = _c(u, np.float32)
    out = np.empty(g.shape, np.uint16)
    lib().orc_moe_activate(_p(g), _p(u), g.size, _p(out))
    return out


def add_norm(hidden_bf16, delta_bf16, weight, eps, full_layer):
    """Returns (hidden after the add, normalised rows), both bf16 bit patterns [rows, n]."""
    hidden = _c(hidden_bf16, np.uint16).copy()
    delta = None if delta_bf16 is None else _c(delta_bf16, np.uint16)
    weight = _c(weight, np.float32)
    rows, n = hidden.shape
    out = np.empty_like(hidden)
    lib().orc_add_norm(_p(hidden), _p(delta), _p(weight), rows, n, C.c_float(eps), int(full_layer), _p(out))
    return hidden, out


def moe_sum(routes_bf16, weights, out_bf16, k):
    routes_bf16 = _c(routes_bf16, np.uint16); weights = _c(weights, np.float32)
    out = _c(out_bf16, np.uint16).copy()
    batch, hidden = out.shape
    lib().orc_moe_sum(_p(routes_bf16), _p(weights), _p(out), hidden, batch, k)
    return out


def moe_add(routes_bf16, weights, out_bf16, shared_bf16, k):
    routes_bf16 = _c(routes_bf16, np.uint16); weights = _c(weights, np.float32)
    out = _c(out_bf16, np.uint16).copy()
    shared = None if shared_bf16 is None else _c(shared_bf16, np.uint16)
    batch, hidden = out.shape
    lib().orc_moe_add(_p(routes_bf16), _p(weights), _p(out), _p(shared), hidden, batch, k)
    return out


# ---- the layer -------------------------------------------------------------------------------
@dataclass
class Result:
    out: np.ndarray        # bf16 bits [T, H]: residual after the layer
    logits: np.ndarray
    ids: np.ndarray
    probs: np.ndarray
    act: np.ndarray        # f32 [R, ffn]
    y: np.ndarray          # bf16 bits [R, H]


def dense_forward(kind: int, fmt: int, hidden: int, ffn: int, up_w, gate_w, down_w, x_bf16, tile: bool) -> np.ndarray:
    """Dense projection (kind 0: bf16 [T, ffn]) or feed-forward (1 relu^2, 2 SiLU gate: bf16 [T, hidden])."""
    x = _c(x_bf16, np.uint16).reshape(-1, hidden)
    out = np.empty((x.shape[0], ffn if kind == 0 else hidden), dtype=np.uint16)
    lib().orc_dense_forward(kind, fmt, hidden, ffn, _p(up_w), _p(gate_w), _p(down_w), _p(x), x.shape[0], int(tile), _p(out))
    return out


def moe_forward(layer, x_bf16, residual_bf16, mode: int = 0, accumulate_f32: bool = False,
                trace: bool = True) -> Result:
    """Run the oracle on a layer description (any object exposing the attributes of
    ``oco_b200.synth.Layer``). ``x_bf16`` / ``residual_bf16`` are uint16 arrays [T, H]."""
    x = _c(x_bf16, np.uint16)
    res = _c(residual_bf16, np.uint16).copy()
    T, H = x.shape
    keep = []

    def ptr(a, dtype):
        if a is None:
            return None
        a = _c(a, dtype); keep.append(a)
        return a.ctypes.data

    st = _Layer(
        arch=layer.arch, hidden=layer.hidden, ffn=layer.ffn, experts=layer.experts, top_k=layer.top_k,
        shared_ffn=layer.shared_ffn, fmt=layer.fmt, normalize=int(layer.normalize),
        scale=float(layer.scale), reserved=0,
        router_w=ptr(layer.router_w, np.float32), router_b=ptr(layer.router_b, np.float32),
        gate_w=ptr(layer.gate_w, np.uint8), up_w=ptr(layer.up_w, np.uint8), down_w=ptr(layer.down_w, np.uint8),
        gate_b=ptr(layer.gate_b, np.float32), up_b=ptr(layer.up_b, np.float32),
        down_b=ptr(layer.down_b, np.float32),
        shared_up_w=ptr(layer.shared_up_w, np.uint8), shared_down_w=ptr(layer.shared_down_w, np.uint8))
    R = T * layer.top_k
    logits = np.empty((T, layer.experts), np.float32)
    ids = np.empty((T, layer.top_k), np.uint32)
    probs = np.empty((T, layer.top_k), np.float32)
    act = np.empty((R, layer.ffn), np.float32) if trace else None
    y = np.empty((R, H), np.uint16) if trace else None
    tr = _Trace(logits=_p(logits), ids=_p(ids), probs=_p(probs), act=_p(act), y=_p(y))
    rc = lib().orc_moe_forward(C.byref(st), _p(x), _p(res), T, mode, int(accumulate_f32), C.byref(tr))
    if rc != 0:
        raise RuntimeError(f"oracle failed: {rc}")
    return Result(res, logits, ids, probs, act, y)


def num_threads() -> int:
    return lib().orc_num_threads()


def set_num_threads(n: int) -> None:
    lib().orc_set_num_threads(int(n))
