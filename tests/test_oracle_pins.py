"""Pins the CPU oracle against the reference's own kernel tests.

The reference stores no golden files: each of its kernel tests builds operands from closed
formulas, computes an independent f64 expectation and accepts the kernel inside an analytic
bound. The same operands, expectations and bounds are applied here to the oracle's restatement of
each kernel (reference: src/weights/dispatch_tests/{mxfp4,nemotron,matrix_precision}.rs).
"""
import numpy as np
import pytest

from oco_b200 import synth
from tests import refcases as rc


def test_mxfp4_decode_matches_independent_coefficients(oracle):
    c = rc.mxfp4_decode_case()
    k, n = c["k"], c["n"]
    # Dequantised weights are bit-exact against the independently built coefficients.
    deq = oracle.dequant(oracle.FMT_MXFP4, c["packed"], 4 * n * k).reshape(4, n, k)
    assert np.array_equal(deq.astype(np.float64), c["coefficients"])

    x_bf16 = synth.f32_to_bf16_bits(c["input_f32"][0])
    xv = synth.bf16_bits_to_f32(x_bf16).astype(np.float64)
    ids = c["ids"]
    uy, gy = oracle.expert_expand(c["packed"], c["packed"], x_bf16, c["bias"], c["bias"], ids, k, n)
    for route, e in enumerate(ids):
        w = c["coefficients"][e]
        prod = w * xv
        ub = synth.bf16_bits_to_f32(synth.f32_to_bf16_bits(c["bias"][e] + np.float32(1.0))).astype(np.float64)
        gb = synth.bf16_bits_to_f32(synth.f32_to_bf16_bits(c["bias"][e])).astype(np.float64)
        up_ref = prod.sum(1) + ub
        up_mag = np.abs(prod).sum(1) + np.abs(ub)
        assert np.all(np.abs(uy[route] - up_ref) <= rc.gamma_bound(up_ref, up_mag, k, False))
        gate_ref = prod.sum(1) + gb
        g = np.minimum(gate_ref, 7.0)
        u = np.clip(up_ref, -6.0, 8.0)
        expected = g / (1.0 + np.exp(-1.702 * g)) * u
        assert np.all(np.abs(gy[route] - expected) <= 1e-3 * np.maximum(np.abs(expected), 1.0))

    # Down matvec over f32 inputs, bf16 result.
    y = oracle.expert_down_vector(c["packed"], c["input_f32"], c["bias"], ids, k, n)
    for route, e in enumerate(ids):
        prod = c["coefficients"][e] * c["input_f32"][route].astype(np.float64)
        b = synth.bf16_bits_to_f32(synth.f32_to_bf16_bits(c["bias"][e])).astype(np.float64)
        ref = prod.sum(1) + b
        mag = np.abs(prod).sum(1) + np.abs(b)
        got = synth.bf16_bits_to_f32(y[route]).astype(np.float64)
        assert np.all(np.abs(got - ref) <= rc.gamma_bound(ref, mag, k, True))

    # A reserved E8M0 header (255) must surface as a non-finite result (mxfp4.rs:205-233).
    bad = c["packed"].copy()
    bad[ids[0], 0, 0] = 255
    uy2, _ = oracle.expert_expand(bad, bad, x_bf16, c["bias"], c["bias"], ids, k, n)
    assert not np.isfinite(uy2[0, 0])
    assert np.isfinite(uy2[0, 1])


def _f16(a):
    return np.asarray(a, np.float32).astype(np.float16).astype(np.float64)


@pytest.mark.parametrize("batch", [17, 257])
def test_routed_experts_preserve_half_products_and_route_boundaries(oracle, batch):
    c = rc.routed_experts_case(batch)
    k, n, down_n = c["k"], c["n"], c["down_n"]
    routes = batch * 4
    ids = c["ids"].ravel()
    up_tiles, down_tiles = 2 * -(-n // 64), -(-down_n // 64)
    plan = oracle.route_plan_tiled(ids, 64, up_tiles, down_tiles)
    grouped = 6 + 2 * (-(-routes // 16) + 32)
    sorted_base = grouped + 32 * (routes + 1)
    # Lists: ascending route indices per expert; offsets: exclusive scan; rows: stable positions.
    offset = 0
    tiles = []
    for e in range(32):
        base = grouped + e * (routes + 1)
        count = int(plan[base])
        expect = np.nonzero(ids == e)[0]
        assert count == expect.size
        assert np.array_equal(plan[base + 1: base + 1 + count], expect)
        assert plan[sorted_base + e] == offset
        assert np.array_equal(plan[sorted_base + 32 + expect], offset + np.arange(count))
        tiles += [(e, b) for b in range(0, count, 64)]
        offset += count
    assert list(plan[:6]) == [up_tiles, len(tiles), 1, down_tiles, len(tiles), 1]
    assert np.array_equal(plan[6: 6 + 2 * len(tiles)].reshape(-1, 2), np.array(tiles, np.uint32))
    offsets, row_of_route, route_of_row = oracle.permutation(ids, 32)
    assert np.array_equal(offsets[:32], plan[sorted_base: sorted_base + 32])
    assert np.array_equal(row_of_route, plan[sorted_base + 32: sorted_base + 32 + routes])
    assert np.array_equal(route_of_row[row_of_route], np.arange(routes))
    if batch == 257:
        assert sum(1 for e, _ in tiles if e == 31) > 1   # an over-full expert spans several tiles

    xv = _f16(synth.bf16_bits_to_f32(c["x"]))
    up = oracle.expert_up_tile(c["up_p"], c["x"], c["ub"], 1.0, ids, 4, k, n)
    gate = oracle.expert_up_tile(c["gate_p"], c["x"], c["gb"], 0.0, ids, 4, k, n)
    for out, vals, bias, shift in ((up, c["up_v"], c["ub"], 1.0), (gate, c["gate_v"], c["gb"], 0.0)):
        w = _f16(vals)[ids]                                        # [routes, n, k]
        xin = xv[np.arange(routes) // 4][:, None, :]
        prod = w * xin
        b = synth.bf16_bits_to_f32(synth.f32_to_bf16_bits(bias + np.float32(shift))).astype(np.float64)[ids]
        ref = prod.sum(2) + b
        mag = np.abs(prod).sum(2) + np.abs(b)
        assert np.all(np.abs(out - ref) <= rc.gamma_bound(ref, mag, k, False))
    # Down tiles consume the up projections rounded to half (mxfp4.rs:400-410).
    act = up.astype(np.float16).view(np.uint16)
    y = oracle.expert_down_tile(c["down_p"], act, c["db"], ids, n, down_n)
    w = _f16(c["down_v"])[ids]
    prod = w * _f16(up)[:, None, :]
    b = synth.bf16_bits_to_f32(synth.f32_to_bf16_bits(c["db"])).astype(np.float64)[ids]
    ref = prod.sum(2) + b
    mag = np.abs(prod).sum(2) + np.abs(b)
    got = synth.bf16_bits_to_f32(y).astype(np.float64)
    assert np.all(np.abs(got - ref) <= rc.gamma_bound(ref, mag, n, True))


def test_sigmoid_router_selects_biased_and_weights_unbiased(oracle):
    c = rc.sigmoid_router_case()
    _, ids, probs = oracle.router_sigmoid(c["x"], c["w"], c["bias"], c["active"], True, c["scale"])
    assert np.array_equal(ids, c["ids"])
    assert np.all(np.abs(probs - c["probs"]) <= 1e-4 * np.maximum(np.abs(c["probs"]), 1.0))
    assert np.count_nonzero(ids[0] % 10 == 3) >= 3


@pytest.mark.parametrize("fmt", [synth.FMT_Q4_0, synth.FMT_Q4_K])
def test_dense_block_decode(oracle, fmt):
    packed, coeff = rc.dense_q4_case(fmt)
    n, k = coeff.shape
    deq = oracle.dequant(fmt, packed, n * k).reshape(n, k).astype(np.float64)
    if fmt == synth.FMT_Q4_0:
        assert np.array_equal(deq, coeff)                    # d * (q - 8) is exact in f32
    else:
        # one f32 rounding in d*sc*q - dmin*m
        assert np.all(np.abs(deq - coeff) <= 2.0 ** -24 * np.maximum(np.abs(coeff), 2.0 ** -20) * 2)


def test_rounding_helpers_match_numpy(oracle):
    rng = np.random.default_rng(1)
    v = np.concatenate([rng.normal(0, 1, 4000), rng.normal(0, 1e-6, 500), rng.normal(0, 3e4, 500),
                        [0.0, -0.0, 65504.0, 65520.0, 65519.9, 1e-8, 5.96e-8, 2.98e-8, 2.9802322e-8,
                         np.inf, -np.inf]]).astype(np.float32)
    L = oracle.lib()
    with np.errstate(over="ignore"):
        expect = v.astype(np.float16).view(np.uint16)
    got = np.array([L.orc_f32_to_f16(float(x)) for x in v], np.uint16)
    assert np.array_equal(got, expect)
    back = np.array([L.orc_f16_to_f32(int(h)) for h in got], np.float32)
    assert np.array_equal(back.view(np.uint32), expect.view(np.float16).astype(np.float32).view(np.uint32))
    bf = np.array([L.orc_f32_to_bf16(float(x)) for x in v], np.uint16)
    assert np.array_equal(bf, synth.f32_to_bf16_bits(v))
    # deterministic exp stays within 2 ulp of libm over the range the layer uses
    a = np.linspace(-90, 20, 20001).astype(np.float32)
    e = np.array([L.orc_exp(float(x)) for x in a], np.float64)
    ref = np.exp(a.astype(np.float64))
    ok = ref > 1e-37
    assert np.max(np.abs(e[ok] - ref[ok]) / ref[ok]) < 3e-7
