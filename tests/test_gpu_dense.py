"""Parity of the dense products (oco_dense_*) against the CPU oracle, through the C ABI: projections in
the three weight formats, Nemotron's always-on expert at its real shape, a gated feed-forward at a Qwen
dense-layer shape; one row (exact operands) and several (half operands).

Bars: rel-L2 <= 1e-3 against the oracle's result for the same operand mode, and every output within the
bound the reference's own dense test allows (src/weights/dispatch_tests/matrix_precision.rs:135-143)
of the oracle's value.
"""
import numpy as np
import pytest

from oco_b200 import synth

pytestmark = pytest.mark.gpu

REL_L2 = 1e-3


@pytest.fixture(scope="module")
def dense():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from oco_b200 import build
    build.build()
    from oco_b200 import dense as d
    return d


def rel_l2(got_bits, ref_bits):
    g = synth.bf16_bits_to_f32(got_bits).astype(np.float64)
    r = synth.bf16_bits_to_f32(ref_bits).astype(np.float64)
    assert np.all(np.isfinite(g)) and np.all(np.isfinite(r))
    return np.linalg.norm(g - r) / max(np.linalg.norm(r), 1e-30)


def check(dense, oracle, kind, fmt, H, F, rows, seed, x_scale=1.0):
    rng = np.random.default_rng(seed)
    gen = synth._RANDOM[fmt]
    up_w = gen(rng, F, H)
    gate_w = gen(rng, F, H) if kind == dense.FFN_SILU_GATE else None
    down_w = gen(rng, H, F) if kind != dense.PROJECTION else None
    x_bits, _ = synth.make_tokens(H, rows, seed + 1, "zero")
    if x_scale != 1.0:
        x_bits = synth.f32_to_bf16_bits(synth.bf16_bits_to_f32(x_bits) * np.float32(x_scale))
    plan = dense.DensePlan(kind, fmt, H, F)
    plan.reserve(rows)
    plan.bind(up_w, gate_w, down_w)
    got = dense.apply(plan, x_bits)
    ref = oracle.dense_forward(kind, fmt, H, F, up_w, gate_w, down_w, x_bits, tile=rows > 1)
    assert got.shape == ref.shape
    err = rel_l2(got, ref)
    assert err <= REL_L2, f"kind {kind} fmt {fmt} {H}x{F} rows {rows}: rel-L2 {err}"
    assert plan.launch_count() >= 2
    return got, ref, (up_w, gate_w, down_w, x_bits)


@pytest.mark.parametrize("fmt", [synth.FMT_Q4_0, synth.FMT_Q4_K, synth.FMT_MXFP4])
@pytest.mark.parametrize("rows", [1, 2, 21, 300])
def test_projection_at_the_reference_test_shape(dense, oracle, fmt, rows):
    """K = 512 as in dense_products_match_declared_operand_precision, n = 64; each output within the
    reference's bound of a float64 product over the kernel's declared operands."""
    H, F = 512, 64
    got, ref, (up_w, _, _, x_bits) = check(dense, oracle, dense.PROJECTION, fmt, H, F, rows, 40 + rows)
    tile = rows > 1
    conv = (lambda a: a.astype(np.float32).astype(np.float16).astype(np.float64)) if tile else (lambda a: a)
    x = conv(synth.bf16_bits_to_f32(x_bits).astype(np.float64))
    w = conv(oracle.dequant(fmt, up_w, F * H).reshape(F, H).astype(np.float64))
    want, mag = x @ w.T, np.abs(x) @ np.abs(w).T
    ops = 2 * H + 8
    gamma = ops * 2.0 ** -24 / (1 - ops * 2.0 ** -24)
    bound = (1 + 2.0 ** -8) * gamma * mag + 2.0 ** -8 * np.abs(want)
    g = synth.bf16_bits_to_f32(got).astype(np.float64)
    assert np.all(np.abs(g - want) <= bound), float(np.max(np.abs(g - want) - bound))


@pytest.mark.parametrize("rows", [1, 5, 300])
def test_nemotron_shared_expert_shape(dense, oracle, rows):
    """2688 -> 3712 -> 2688, Q4_0, relu^2 (the always-on expert of Nemotron-3-Nano)."""
    check(dense, oracle, dense.FFN_RELU2, synth.FMT_Q4_0, 2688, 3712, rows, 7, x_scale=0.25)


@pytest.mark.parametrize("rows", [1, 5, 300])
def test_qwen_dense_ffn_shape(dense, oracle, rows):
    """2048 -> 6144 -> 2048, Q4_K, SiLU gate (a Qwen3 dense layer)."""
    check(dense, oracle, dense.FFN_SILU_GATE, synth.FMT_Q4_K, 2048, 6144, rows, 9, x_scale=0.25)


def test_mxfp4_projection_at_the_gpt_oss_width(dense, oracle):
    for rows in (1, 64):
        check(dense, oracle, dense.PROJECTION, synth.FMT_MXFP4, 2880, 2880, rows, 21)


def test_unsupported_pairs_and_bad_calls_are_refused(dense):
    from oco_b200 import _lib
    from oco_b200.moe import OcoError
    import torch
    for kind, fmt in ((dense.FFN_RELU2, synth.FMT_Q4_K), (dense.FFN_SILU_GATE, synth.FMT_Q4_0), (dense.FFN_RELU2, synth.FMT_MXFP4)):
        with pytest.raises(OcoError) as e:
            dense.DensePlan(kind, fmt, 512, 512)
        assert e.value.code == _lib.UNSUPPORTED_SHAPE
    with pytest.raises(OcoError):
        dense.DensePlan(7, synth.FMT_Q4_0, 512, 512)
    plan = dense.DensePlan(dense.FFN_RELU2, synth.FMT_Q4_0, 512, 512)
    plan.reserve(4)
    x = torch.zeros((4, 512), dtype=torch.int16, device="cuda")
    with pytest.raises(OcoError):              # no weights bound
        plan.forward(x, x.clone(), 4)
    rng = np.random.default_rng(0)
    with pytest.raises(OcoError):              # a feed-forward without its down matrix
        plan.bind(synth.random_q4_0(rng, 512, 512), None, None)
    plan.bind(synth.random_q4_0(rng, 512, 512), None, synth.random_q4_0(rng, 512, 512))
    with pytest.raises(OcoError):              # more rows than reserved
        plan.forward(torch.zeros((5, 512), dtype=torch.int16, device="cuda"), torch.zeros((5, 512), dtype=torch.int16, device="cuda"), 5)
