"""The C-ABI library loads and exports every symbol include/oco_moe.h declares; argument checks
that need no GPU return status codes instead of aborting."""
import ctypes as C
import os
import re

import pytest

from oco_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _lib.lib()


def test_header_symbols_are_exported(lib):
    header = open(os.path.join(ROOT, "include", "oco_moe.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(oco_(?:moe|cuda|tensor|dense|ep)_\w+)\s*\(", header))
    assert len(declared) >= 20
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    for name in declared:
        assert hasattr(lib, name), name
    assert b"sm_100a" in lib.oco_moe_version()


def _create(lib, **kw):
    d = dict(arch=0, hidden=2880, ffn=2880, experts=32, top_k=4, shared_ffn=0, weight_format=39, normalize=0,
             scale=1.0, gemm_impl=0)
    d.update(kw)
    desc = _lib.Desc(**d)
    h = C.c_void_p()
    rc = lib.oco_moe_plan_create(C.byref(desc), C.byref(h))
    msg = lib.oco_moe_last_error(h).decode() if h else ""
    return rc, h, msg


def test_plan_validation_and_workspace_size(lib):
    rc, h, _ = _create(lib)
    assert rc == _lib.OK
    one = lib.oco_moe_workspace_bytes(h, 1)
    big = lib.oco_moe_workspace_bytes(h, 2048)
    # expert-sorted rows, activations and route outputs dominate: 3 * R * 2880 * 2 bytes
    assert big > 3 * 2048 * 4 * 2880 * 2 and big < 4 * 2048 * 4 * 2880 * 2 + (64 << 20)
    assert 0 < one < big
    assert lib.oco_moe_workspace_bytes(h, 0) == 0
    # calls that need bound buffers fail with a status, never abort
    assert lib.oco_moe_forward(h, None, None, 1, None) == _lib.INVALID_ARGUMENT
    assert b"bind" in lib.oco_moe_last_error(h)
    lib.oco_moe_plan_destroy(h)
    for kw, code in ((dict(weight_format=12), _lib.UNSUPPORTED_SHAPE), (dict(experts=129), _lib.UNSUPPORTED_SHAPE),
                     (dict(top_k=9), _lib.UNSUPPORTED_SHAPE), (dict(hidden=2881), _lib.UNSUPPORTED_SHAPE),
                     (dict(arch=7), _lib.INVALID_ARGUMENT), (dict(shared_ffn=64), _lib.UNSUPPORTED_SHAPE),
                     (dict(arch=2, weight_format=12, hidden=2880), _lib.UNSUPPORTED_SHAPE)):
        rc, h, msg = _create(lib, **kw)
        assert rc == code, (kw, rc, msg)
        assert msg
        lib.oco_moe_plan_destroy(h)
    assert lib.oco_moe_plan_create(None, None) == _lib.INVALID_ARGUMENT


def test_product_package_does_not_touch_the_oracle():
    pkg = os.path.join(ROOT, "oco_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "import oracle" not in text and "from oracle" not in text, f
                assert "moe_oracle" not in text, f


def test_dense_window_and_graph_calls_check_their_arguments(lib):
    """The entry points added beside the layer answer bad arguments with a status and a message on a machine
    without a GPU too: nothing is dereferenced, nothing aborts."""
    h = C.c_void_p()
    for kind, fmt, code in ((0, 39, _lib.OK), (1, 2, _lib.OK), (2, 12, _lib.OK), (1, 12, _lib.UNSUPPORTED_SHAPE),
                            (2, 2, _lib.UNSUPPORTED_SHAPE), (1, 39, _lib.UNSUPPORTED_SHAPE), (5, 2, _lib.INVALID_ARGUMENT)):
        desc = _lib.DenseDesc(kind=kind, weight_format=fmt, hidden=512, ffn=512)
        rc = lib.oco_dense_plan_create(C.byref(desc), C.byref(h))
        assert rc == code, (kind, fmt, rc, lib.oco_dense_last_error(h))
        if rc != _lib.OK:
            assert lib.oco_dense_last_error(h)
        else:
            assert lib.oco_dense_workspace_bytes(h, 16) > 16 * 512 * 2
            assert lib.oco_dense_forward(h, None, None, 1, None) == _lib.INVALID_ARGUMENT      # nothing bound
        lib.oco_dense_plan_destroy(h)
    desc = _lib.DenseDesc(kind=0, weight_format=12, hidden=512, ffn=48)        # a projection's width: multiples of 32
    assert lib.oco_dense_plan_create(C.byref(desc), C.byref(h)) == _lib.UNSUPPORTED_SHAPE
    lib.oco_dense_plan_destroy(h)
    assert lib.oco_dense_plan_create(None, None) == _lib.INVALID_ARGUMENT
    # host-buffer entry points: no plan, nothing in flight
    g = C.c_void_p()
    assert lib.oco_moe_forward_host_begin(None, None, None, 1, None) == _lib.INVALID_ARGUMENT
    assert lib.oco_moe_forward_host_end(None) == _lib.INVALID_ARGUMENT
    assert lib.oco_moe_forward_host(None, None, None, 1, None) == _lib.INVALID_ARGUMENT
    assert lib.oco_moe_graph_capture_host(None, None, None, 1, C.byref(g)) == _lib.INVALID_ARGUMENT
    # windows: rank outside the world, no backing, backing larger than the slot
    w = C.c_void_p()
    for rank, world, stride, backed in ((2, 2, 1 << 21, 1 << 20), (0, 0, 1 << 21, 1 << 20), (0, 2, 1 << 21, 0), (0, 2, 1 << 20, 1 << 21)):
        assert lib.oco_ep_window_create(rank, world, stride, backed, C.byref(w)) == _lib.INVALID_ARGUMENT
        assert lib.oco_ep_window_error()
    assert lib.oco_ep_window_fd(None) == -1 and lib.oco_ep_window_base(None) is None and lib.oco_ep_window_stride(None) == 0
    assert lib.oco_ep_window_attach(None, 0, 0) == _lib.INVALID_ARGUMENT
    lib.oco_ep_window_destroy(None)
    # graphs and the windowed expert stage on a plan without buffers
    rc, plan, _ = _create(lib)
    assert rc == _lib.OK
    g = C.c_void_p()
    assert lib.oco_moe_graph_capture(plan, None, None, 1, C.byref(g)) != _lib.OK and not g
    assert lib.oco_moe_graph_launch(None, None) == _lib.INVALID_ARGUMENT
    lib.oco_moe_graph_destroy(None)
    assert lib.oco_moe_experts_window(plan, None, None, 4, 1, 0, 0, 0, None, None) == _lib.INVALID_ARGUMENT
    assert lib.oco_moe_combine_shared(plan, None, None, None, None, 1, None) == _lib.INVALID_ARGUMENT
    lib.oco_moe_plan_destroy(plan)
