"""Host-side logic that needs no GPU: block packers against the oracle's decoders, the oracle's
layer against its own kernel-level primitives, multi-rank sharding arithmetic."""
import numpy as np
import pytest

from oco_b200 import synth


def test_packers_round_trip_through_the_decoders(oracle):
    rng = np.random.default_rng(0)
    mag = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0.0, -.5, -1, -1.5, -2, -3, -4, -6])
    codes = rng.integers(0, 16, size=(5, 256), dtype=np.uint8)
    exps = rng.integers(100, 140, size=(5, 8), dtype=np.uint8)
    w = oracle.dequant(synth.FMT_MXFP4, synth.pack_mxfp4(codes, exps), 5 * 256).reshape(5, 256)
    assert np.array_equal(w, (mag[codes] * np.repeat(2.0 ** (exps.astype(np.float64) - 127), 32, axis=1)).astype(np.float32))
    d = rng.uniform(1e-3, 1e-2, size=(5, 8)).astype(np.float16)
    w = oracle.dequant(synth.FMT_Q4_0, synth.pack_q4_0(codes, d.view(np.uint16)), 5 * 256).reshape(5, 256)
    assert np.array_equal(w, (np.repeat(d.astype(np.float32), 32, axis=1) * (codes.astype(np.float32) - 8)))
    dk = rng.uniform(1e-3, 1e-2, size=(5, 1)).astype(np.float16)
    dm = rng.uniform(1e-3, 1e-2, size=(5, 1)).astype(np.float16)
    sc = rng.integers(0, 64, size=(5, 1, 8), dtype=np.uint8)
    mn = rng.integers(0, 64, size=(5, 1, 8), dtype=np.uint8)
    w = oracle.dequant(synth.FMT_Q4_K, synth.pack_q4_k(codes, dk.view(np.uint16), dm.view(np.uint16), sc, mn), 5 * 256)
    sub = np.arange(256) // 32
    ref = (dk.astype(np.float32) * sc[:, 0, sub].astype(np.float32) * codes.astype(np.float32)
           - dm.astype(np.float32) * mn[:, 0, sub].astype(np.float32))
    assert np.array_equal(w.reshape(5, 256), ref.astype(np.float32))


def test_layer_equals_composition_of_kernel_primitives(oracle):
    """orc_moe_forward must be exactly the sequence of per-kernel restatements the reference's
    operator encodes (feed_forward.rs:125-274): router, expand / tiles, activation, down, sum."""
    layer = synth.make_layer(synth.ARCH_GPT_OSS, 128, 96, 32, 4, synth.FMT_MXFP4, seed=7)
    H, F = layer.hidden, layer.ffn
    # single token
    x, res = synth.make_tokens(H, 1, 1, "normal")
    full = oracle.moe_forward(layer, x, res)
    _, ids, probs = oracle.router_gptoss(x, layer.router_w, layer.router_b)
    uy, gy = oracle.expert_expand(layer.up_w, layer.gate_w, x[0], layer.up_b, layer.gate_b, ids[0], H, F)
    y = oracle.expert_down_vector(layer.down_w, gy, layer.down_b, ids[0], F, H)
    out = oracle.moe_sum(y, probs, res, 4)
    assert np.array_equal(ids, full.ids) and np.array_equal(probs, full.probs)
    assert np.array_equal(gy, full.act) and np.array_equal(y, full.y) and np.array_equal(out, full.out)
    # tiles
    x, res = synth.make_tokens(H, 19, 2, "normal")
    full = oracle.moe_forward(layer, x, res)
    _, ids, probs = oracle.router_gptoss(x, layer.router_w, layer.router_b)
    flat = ids.ravel()
    up = oracle.expert_up_tile(layer.up_w, x, layer.up_b, 1.0, flat, 4, H, F)
    gate = oracle.expert_up_tile(layer.gate_w, x, layer.gate_b, 0.0, flat, 4, H, F)
    act = oracle.moe_activate(gate, up)
    y = oracle.expert_down_tile(layer.down_w, act, layer.down_b, flat, F, H)
    out = oracle.moe_sum(y, probs, res, 4)
    assert np.array_equal(act.view(np.float16).astype(np.float32), full.act)
    assert np.array_equal(y, full.y) and np.array_equal(out, full.out)


def test_double_and_float_accumulation_agree_within_tolerance(oracle):
    layer = synth.make_layer(synth.ARCH_GPT_OSS, 256, 128, 32, 4, synth.FMT_MXFP4, seed=9)
    x, res = synth.make_tokens(256, 12, 3, "normal")
    a = oracle.moe_forward(layer, x, res)
    b = oracle.moe_forward(layer, x, res, accumulate_f32=True)
    fa = synth.bf16_bits_to_f32(a.out).astype(np.float64)
    fb = synth.bf16_bits_to_f32(b.out).astype(np.float64)
    assert np.array_equal(a.ids, b.ids)
    assert np.linalg.norm(fa - fb) <= 1e-3 * np.linalg.norm(fa)


def test_route_plan_n_lists_and_tiles(oracle):
    """route_plan_n (nemotron.metal:238-273): lists ascending, tiles of 8 or 32 rows, exact sizing."""
    rng = np.random.default_rng(4)
    for tile_rows in (8, 32):
        ids = rng.integers(0, 100, size=300, dtype=np.uint32)
        plan = oracle.route_plan_n(ids, 100, tile_rows, 29, 42)
        R = ids.size
        lists = 6 + 2 * (-(-R // tile_rows) + 100)
        tiles = []
        for e in range(100):
            base = lists + e * (R + 1)
            where = np.nonzero(ids == e)[0]
            assert plan[base] == where.size
            assert np.array_equal(plan[base + 1: base + 1 + where.size], where)
            tiles += [(e, b) for b in range(0, where.size, tile_rows)]
        assert list(plan[:6]) == [29, len(tiles), 1, 42, len(tiles), 1]
        assert np.array_equal(plan[6:6 + 2 * len(tiles)].reshape(-1, 2), np.array(tiles, np.uint32))


def test_algorithmic_byte_counts_match_the_benchmark_description():
    L = synth.Layer(arch=synth.ARCH_GPT_OSS, hidden=2880, ffn=2880, experts=32, top_k=4, fmt=synth.FMT_MXFP4)
    assert L.expert_bytes() == 13_219_200 + 34_560          # packed weights + f32 biases per expert
    assert synth.row_bytes(synth.FMT_MXFP4, 2880) == 1530
    with pytest.raises(ValueError):
        synth.row_bytes(synth.FMT_Q4_K, 2688)               # Q4_K cannot encode the Nemotron row lengths
    N = synth.Layer(arch=synth.ARCH_NEMOTRON, hidden=2688, ffn=1856, experts=128, top_k=6, fmt=synth.FMT_Q4_0,
                    shared_ffn=3712)
    assert N.expert_bytes() == 5_612_544 and N.shared_bytes() == 11_225_088


def test_add_norm_oracle_against_float64(oracle):
    """The checker's residual add + RMS norm against a float64 restatement of the shader
    (elementwise.metal:32-60), within the bf16 roundings the shader makes."""
    from oco_b200 import synth
    rng = np.random.default_rng(3)
    rows, n, eps = 5, 2880, 1e-5
    hidden, delta = synth.make_tokens(n, rows, 21, "normal")
    w = rng.normal(1.0, 0.3, size=n).astype(np.float32)
    for full_layer in (True, False):
        for d in (delta, None):
            summed, normed = oracle.add_norm(hidden, d, w, eps, full_layer)
            h = synth.bf16_bits_to_f32(hidden).astype(np.float64)
            if d is not None:
                h = synth.bf16_bits_to_f32(synth.f32_to_bf16_bits((h + synth.bf16_bits_to_f32(d)).astype(np.float32))).astype(np.float64)
                assert np.array_equal(synth.f32_to_bf16_bits(h.astype(np.float32)), summed)
            else:
                assert np.array_equal(summed, hidden)
            inv = 1.0 / np.sqrt((h * h).mean(axis=1, keepdims=True) + eps)
            want = h * inv * w
            got = synth.bf16_bits_to_f32(normed).astype(np.float64)
            # one bf16 rounding (2^-9) when the scale is applied in f32, three when both factors are rounded first
            bound = 2.0 ** -8 if full_layer else 2.0 ** -6
            assert np.all(np.abs(got - want) <= np.abs(want) * bound + 1e-30)


def test_window_geometry_and_labels():
    """Slots of both windows start on granularity multiples, hold whole rows and the capacity; labels
    are a route's row in the output window and top_k times its token's row in the token window."""
    from oco_b200 import ep
    for hidden, top_k, cap, gran in ((2880, 4, 4096, 2 << 20), (2880, 4, 100, 2 << 20), (2048, 8, 512, 2 << 20),
                                     (2688, 6, 1024, 2 << 20), (64, 2, 6, 4096)):
        st, sr = ep.window_geometry(hidden, top_k, cap, gran)
        assert st >= cap and sr == st * top_k
        assert (st * hidden * 2) % gran == 0 and (sr * hidden * 2) % gran == 0
        unit = gran // np.gcd(gran, hidden * 2)
        assert st - cap < unit                    # the smallest such slot
        world = 3
        lab = ep.window_labels(world, cap * top_k, sr)
        src, r = np.divmod(np.arange(world * cap * top_k), cap * top_k)
        assert np.array_equal(lab, src * sr + r)
        assert np.array_equal(lab // top_k, src * st + r // top_k)      # the token's row in the token window
        assert len(np.unique(lab)) == len(lab)
