"""ctypes view of liboco_moe.so, the C-ABI library declared in include/oco_moe.h.

There is no fallback: if the library has not been built, importing a symbol raises.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "liboco_moe.so")

OK, INVALID_ARGUMENT, UNSUPPORTED_SHAPE, CUDA_ERROR, NCCL_ERROR, DEVICE_TIMEOUT, OUT_OF_MEMORY = range(7)
STATUS_NAMES = ["OK", "INVALID_ARGUMENT", "UNSUPPORTED_SHAPE", "CUDA_ERROR", "NCCL_ERROR", "DEVICE_TIMEOUT", "OUT_OF_MEMORY"]


class Desc(C.Structure):
    _fields_ = [("arch", C.c_int32), ("hidden", C.c_int32), ("ffn", C.c_int32), ("experts", C.c_int32),
                ("top_k", C.c_int32), ("shared_ffn", C.c_int32), ("weight_format", C.c_int32),
                ("normalize", C.c_int32), ("scale", C.c_float), ("gemm_impl", C.c_int32), ("numerics", C.c_int32)]


class Weights(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("router_w", "router_b", "gate_w", "up_w", "down_w", "gate_b", "up_b",
                                          "down_b", "shared_up_w", "shared_down_w", "gate_up_w", "gate_up_b")]


class RoutingView(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("logits", "ids", "probs", "offsets", "row_of_route", "route_of_row",
                                          "tiles", "tile_count", "act", "y", "norm")]


# Every symbol include/oco_moe.h declares, with its signature.
class DenseDesc(C.Structure):
    _fields_ = [("kind", C.c_int32), ("weight_format", C.c_int32), ("hidden", C.c_int32), ("ffn", C.c_int32)]


class DenseWeights(C.Structure):
    _fields_ = [("up_w", C.POINTER(C.c_uint8)), ("gate_w", C.POINTER(C.c_uint8)), ("down_w", C.POINTER(C.c_uint8))]


SIGNATURES = {
    "oco_moe_plan_create": (C.c_int, [C.POINTER(Desc), C.POINTER(C.c_void_p)]),
    "oco_moe_plan_destroy": (None, [C.c_void_p]),
    "oco_moe_workspace_bytes": (C.c_size_t, [C.c_void_p, C.c_int]),
    "oco_moe_bind_workspace": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int]),
    "oco_moe_bind_weights": (C.c_int, [C.c_void_p, C.POINTER(Weights)]),
    "oco_moe_forward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "oco_moe_add_norm_forward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_int, C.c_int, C.c_void_p]),
    "oco_moe_route": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "oco_moe_experts": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]),
    "oco_moe_combine": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "oco_moe_forward_host": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "oco_moe_forward_host_begin": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "oco_moe_forward_host_end": (C.c_int, [C.c_void_p]),
    "oco_moe_poll": (C.c_int, [C.c_void_p, C.c_void_p]),
    "oco_moe_routing": (C.c_int, [C.c_void_p, C.POINTER(RoutingView)]),
    "oco_moe_last_error": (C.c_char_p, [C.c_void_p]),
    "oco_moe_last_launch_count": (C.c_int, [C.c_void_p]),
    "oco_moe_set_profiling": (C.c_int, [C.c_void_p, C.c_int]),
    "oco_moe_phase_times": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_float), C.POINTER(C.c_char_p)]),
    "oco_moe_route_token_static": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                              C.c_int, C.c_float, C.c_void_p, C.c_void_p, C.c_void_p, C.c_char_p,
                                              C.c_size_t]),
    "oco_moe_dequant_f32": (C.c_int, [C.c_int, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p]),
    "oco_moe_dequant_f16": (C.c_int, [C.c_int, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p]),
    "oco_cuda_device_open": (C.c_int, [C.c_int]),
    "oco_cuda_malloc": (C.c_int, [C.POINTER(C.c_void_p), C.c_size_t]),
    "oco_cuda_free": (C.c_int, [C.c_void_p]),
    "oco_cuda_upload": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "oco_cuda_download": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "oco_cuda_stream_create": (C.c_int, [C.POINTER(C.c_void_p)]),
    "oco_cuda_stream_destroy": (C.c_int, [C.c_void_p]),
    "oco_cuda_stream_sync": (C.c_int, [C.c_void_p]),
    "oco_cuda_event_create": (C.c_int, [C.POINTER(C.c_void_p)]),
    "oco_cuda_event_destroy": (C.c_int, [C.c_void_p]),
    "oco_cuda_event_record": (C.c_int, [C.c_void_p, C.c_void_p]),
    "oco_cuda_event_sync": (C.c_int, [C.c_void_p]),
    "oco_cuda_event_elapsed_ms": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_float)]),
    "oco_moe_selftest_wait_timeout": (C.c_int, [C.c_void_p, C.c_longlong, C.c_void_p]),
    "oco_tensor_peak": (C.c_int, [C.c_int, C.c_int, C.POINTER(C.c_float)]),
    "oco_moe_combine_shared": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "oco_moe_repack_bytes": (C.c_size_t, [C.c_void_p]),
    "oco_moe_bind_repacked": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "oco_moe_graph_capture": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.POINTER(C.c_void_p)]),
    "oco_moe_graph_capture_host": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.POINTER(C.c_void_p)]),
    "oco_moe_graph_launch": (C.c_int, [C.c_void_p, C.c_void_p]),
    "oco_moe_graph_destroy": (None, [C.c_void_p]),
    "oco_dense_plan_create": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "oco_dense_plan_destroy": (None, [C.c_void_p]),
    "oco_dense_workspace_bytes": (C.c_size_t, [C.c_void_p, C.c_int]),
    "oco_dense_bind_workspace": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int]),
    "oco_dense_bind_weights": (C.c_int, [C.c_void_p, C.c_void_p]),
    "oco_dense_forward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "oco_dense_poll": (C.c_int, [C.c_void_p, C.c_void_p]),
    "oco_dense_last_launch_count": (C.c_int, [C.c_void_p]),
    "oco_dense_last_error": (C.c_char_p, [C.c_void_p]),
    "oco_ep_window_granularity": (C.c_int, [C.POINTER(C.c_size_t)]),
    "oco_ep_window_create": (C.c_int, [C.c_int, C.c_int, C.c_size_t, C.c_size_t, C.POINTER(C.c_void_p)]),
    "oco_ep_window_fd": (C.c_int, [C.c_void_p]),
    "oco_ep_window_attach": (C.c_int, [C.c_void_p, C.c_int, C.c_int]),
    "oco_ep_window_base": (C.c_void_p, [C.c_void_p]),
    "oco_ep_window_stride": (C.c_size_t, [C.c_void_p]),
    "oco_ep_window_backed": (C.c_size_t, [C.c_void_p]),
    "oco_ep_window_destroy": (None, [C.c_void_p]),
    "oco_ep_window_error": (C.c_char_p, []),
    "oco_moe_experts_window": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                         C.c_void_p, C.c_void_p]),
    "oco_moe_version": (C.c_char_p, []),
}

_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m oco_b200.build` (nvcc, sm_100a). "
                "There is no CPU or PyTorch fallback for this path.")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)      # raises AttributeError if the symbol is not exported
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


class OcoError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"{STATUS_NAMES[code] if 0 <= code < len(STATUS_NAMES) else code}: {message}")
        self.code = code
