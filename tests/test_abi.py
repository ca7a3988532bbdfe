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
