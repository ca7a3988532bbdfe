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


def _dense_f64(kind, fmt, H, F, up_w, gate_w, down_w, x_bits, tile, orc):
    """The dense kinds in float64 with the kernels' declared operand conversions and bf16 stores, as the
    reference's own dense test builds its expectation (product_reference, roundoff_bound:
    src/weights/dispatch_tests/matrix_precision.rs:119-143). Returns (value, magnitude) of the last product."""
    def half(a):
        return a.astype(np.float32).astype(np.float16).astype(np.float64) if tile else a
    def bf(a):
        return synth.bf16_bits_to_f32(synth.f32_to_bf16_bits(a.astype(np.float32))).astype(np.float64)
    x = half(synth.bf16_bits_to_f32(x_bits).astype(np.float64))
    up = half(orc.dequant(fmt, up_w, F * H).reshape(F, H).astype(np.float64))
    if kind == 0:
        return x @ up.T, np.abs(x) @ np.abs(up).T
    u = bf(x @ up.T)
    if kind == 1:
        a = np.maximum(u, 0.0) ** 2
        a = half(bf(a)) if tile else a.astype(np.float32).astype(np.float64)
    else:
        g = bf(x @ half(orc.dequant(fmt, gate_w, F * H).reshape(F, H).astype(np.float64)).T)
        a = half(bf(bf(g / (1.0 + np.exp(-g))) * u))
    down = half(orc.dequant(fmt, down_w, H * F).reshape(H, F).astype(np.float64))
    return a @ down.T, np.abs(a) @ np.abs(down).T


@pytest.mark.parametrize("kind,fmt", [(0, synth.FMT_Q4_0), (0, synth.FMT_Q4_K), (0, synth.FMT_MXFP4),
                                      (1, synth.FMT_Q4_0), (2, synth.FMT_Q4_K)])
@pytest.mark.parametrize("rows", [2, 21])
def test_dense_products_stay_within_the_reference_roundoff_bound(oracle, kind, fmt, rows):
    """The reference checks its dense kernels at K = 512, n = 33, m = 2 (exact operands) and m = 21 (half
    operands) against gamma_(2K+8) * sum|w||x| plus one bf16 storage rounding; the oracle's dense function
    must sit inside the same bound (intermediate bf16 stores of the feed-forward kinds are applied to the
    float64 expectation too, so only the last product is bounded)."""
    H, F = 512, 64 if kind == 0 else 256
    tile = rows > 2
    rng = np.random.default_rng(5 + kind)
    gen = synth._RANDOM[fmt]
    up_w, gate_w, down_w = gen(rng, F, H), gen(rng, F, H), gen(rng, H, F)
    x_bits, _ = synth.make_tokens(H, rows, 3, "zero")
    got = synth.bf16_bits_to_f32(oracle.dense_forward(kind, fmt, H, F, up_w, gate_w, down_w, x_bits, tile)).astype(np.float64)
    want, mag = _dense_f64(kind, fmt, H, F, up_w, gate_w, down_w, x_bits, tile, oracle)
    k = H if kind == 0 else F
    ops = 2 * k + 8
    gamma = ops * 2.0 ** -24 / (1 - ops * 2.0 ** -24)
    bound = (1 + 2.0 ** -8) * gamma * mag + 2.0 ** -8 * np.abs(want)
    if kind != 0:
        # an intermediate that sits on a bf16 rounding boundary may round the other way in f32: allow the few
        # outputs that such a flip moves, by their share of the magnitude
        bound = bound + 2.0 ** -8 * mag * 4.0 / k
    assert np.all(np.isfinite(got)) and np.all(np.abs(got - want) <= bound), float(np.max(np.abs(got - want) - bound))


@pytest.mark.parametrize("tile", [False, True])
def test_dense_relu2_equals_the_layer_shared_expert(oracle, tile):
    """With routed down weights decoding to zero and a zero residual, the Nemotron layer's output is its
    always-on expert alone: the dense function must reproduce it bit for bit in both operand modes."""
    H, F, S, E, K = 128, 96, 160, 8, 2
    layer = synth.make_layer(synth.ARCH_NEMOTRON, H, F, E, K, synth.FMT_Q4_0, seed=12, shared_ffn=S, normalize=True, scale=2.5)
    layer.down_w = np.zeros_like(layer.down_w)              # scale 0: every routed weight is zero
    rows = 5 if tile else 1
    x_bits, res = synth.make_tokens(H, rows, 8, "zero")
    ref = oracle.moe_forward(layer, x_bits, res, mode=2 if tile else 1)
    got = oracle.dense_forward(1, synth.FMT_Q4_0, H, S, layer.shared_up_w, None, layer.shared_down_w, x_bits, tile)
    a, b = synth.bf16_bits_to_f32(got), synth.bf16_bits_to_f32(ref.out)
    assert np.array_equal(a, b)                             # (+0 and -0 compare equal)
