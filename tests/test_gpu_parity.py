"""Parity of the CUDA path against the CPU oracle, through the C ABI.

Bars: expert ids, combination weights, the permutation and dequantised weights are bit-exact;
layer outputs are within rel-L2 1e-3 of the oracle's fp32-accumulated result.
"""
import numpy as np
import pytest

from oco_b200 import synth
from tests import refcases as rc

pytestmark = pytest.mark.gpu

REL_L2 = 1e-3   # the tolerance the benchmark definition states for outputs


@pytest.fixture(scope="module")
def moe():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from oco_b200 import build
    build.build()
    from oco_b200 import moe as m
    return m


def rel_l2(got_bits, ref_bits):
    g = synth.bf16_bits_to_f32(got_bits).astype(np.float64)
    r = synth.bf16_bits_to_f32(ref_bits).astype(np.float64)
    fin = np.isfinite(r)
    assert np.array_equal(np.isfinite(g), fin), "finite masks differ"
    d = np.linalg.norm((g - r)[fin])
    return d / max(np.linalg.norm(r[fin]), 1e-30)


def check_layer(moe, oracle, layer, tokens, seed, residual="normal", gemm_impl=0, mode=0, misalign=0, x_scale=1.0):
    x, res = synth.make_tokens(layer.hidden, tokens, seed, residual)
    if x_scale != 1.0:      # a power of two: keeps the half activations of wide synthetic layers finite
        x = synth.f32_to_bf16_bits(synth.bf16_bits_to_f32(x) * np.float32(x_scale))
    ref = oracle.moe_forward(layer, x, res, mode=mode)
    out, routing = moe.run_layer(layer, x, res, gemm_impl=gemm_impl, misalign=misalign)
    assert np.array_equal(routing["ids"], ref.ids), "expert ids differ"
    assert np.array_equal(routing["logits"].view(np.uint32), ref.logits.view(np.uint32)), "logits differ"
    assert np.array_equal(routing["prob"].view(np.uint32), ref.probs.view(np.uint32)), "weights differ"
    if "offsets" in routing:
        offsets, row_of_route, route_of_row = oracle.permutation(ref.ids, layer.experts)
        assert np.array_equal(routing["offsets"], offsets)
        assert np.array_equal(routing["row_of_route"], row_of_route)
        assert np.array_equal(routing["route_of_row"], route_of_row)
        # activated intermediates (half, expert-sorted rows) against the oracle's route-ordered values
        act = routing["act"].view(np.float16).astype(np.float64)[row_of_route]
        ra = ref.act.astype(np.float64)
        assert np.linalg.norm(act - ra) <= 2e-3 * max(np.linalg.norm(ra), 1e-30)
    err_y = rel_l2(routing["y"], ref.y)
    err = rel_l2(out, ref.out)
    assert err_y <= REL_L2, f"expert outputs rel-L2 {err_y}"
    assert err <= REL_L2, f"layer output rel-L2 {err}"
    return err


@pytest.mark.parametrize("fmt", [synth.FMT_MXFP4, synth.FMT_Q4_0, synth.FMT_Q4_K])
def test_dequantised_weights_are_bit_exact(moe, oracle, fmt):
    rng = np.random.default_rng(fmt)
    k = 1024
    gen = {synth.FMT_MXFP4: lambda: synth.random_mxfp4(rng, 40, k, -30, 20), synth.FMT_Q4_0: lambda: synth.random_q4_0(rng, 40, k),
           synth.FMT_Q4_K: lambda: synth.random_q4_k(rng, 40, k)}[fmt]
    packed = gen()
    if fmt == synth.FMT_MXFP4:   # special headers: zero, the NaN code, extreme powers
        packed[0, 0], packed[1, 17], packed[2, 34], packed[3, 0] = 0, 255, 254, 1
    n = 40 * k
    got = moe.dequant(fmt, packed, n)
    ref = oracle.dequant(fmt, packed, n)
    assert np.array_equal(got.view(np.uint32) & np.where(np.isnan(ref), 0, 0xFFFFFFFF).astype(np.uint32),
                          ref.view(np.uint32) & np.where(np.isnan(ref), 0, 0xFFFFFFFF).astype(np.uint32))
    assert np.array_equal(np.isnan(got), np.isnan(ref))
    got16 = moe.dequant(fmt, packed, n, half=True)
    ref16 = oracle.dequant_f16(fmt, packed, n)
    nan16 = (ref16 & 0x7FFF) > 0x7C00
    assert np.array_equal(((got16 & 0x7FFF) > 0x7C00), nan16)
    assert np.array_equal(got16[~nan16], ref16[~nan16])


def test_reference_decode_case_weights(moe, oracle):
    """The reference's own MXFP4 fixture (K = 2880, n = 33, mirrored rows, powers -5..3) decodes to
    its independently built coefficients on the GPU as well."""
    c = rc.mxfp4_decode_case()
    got = moe.dequant(synth.FMT_MXFP4, c["packed"], 4 * c["n"] * c["k"]).reshape(4, c["n"], c["k"])
    assert np.array_equal(got.astype(np.float64), c["coefficients"])


@pytest.mark.parametrize("tokens", [1, 2, 17, 257], ids=["t1", "t2", "t17", "t257"])
@pytest.mark.parametrize("impl", [0, 1], ids=["tc", "simt"])
def test_gpt_oss_small(moe, oracle, tokens, impl):
    # hidden = ffn = 96: the reference's tile-test shape (k = n = 96): partial 128-feature tile,
    # K not a multiple of 64; batches 17 and 257 are its sparse / over-full expert cases.
    layer = synth.make_layer(synth.ARCH_GPT_OSS, 96, 96, 32, 4, synth.FMT_MXFP4, seed=11)
    if tokens == 1 and impl == 1:
        pytest.skip("single-token path has one implementation")
    check_layer(moe, oracle, layer, tokens, seed=tokens, gemm_impl=impl)


@pytest.mark.parametrize("tokens", [1, 64, 300], ids=["t1", "t64", "t300"])
def test_gpt_oss_medium(moe, oracle, tokens):
    layer = synth.make_layer(synth.ARCH_GPT_OSS, 640, 384, 32, 4, synth.FMT_MXFP4, seed=5)
    check_layer(moe, oracle, layer, tokens, seed=100 + tokens)


@pytest.mark.parametrize("hidden,ffn,tokens", [(96, 96, 700), (640, 384, 520), (320, 288, 1100)],
                         ids=["k96", "k640", "k320"])
def test_gpt_oss_wide_tiles(moe, oracle, hidden, ffn, tokens):
    """Few large experts: more than 192 routes per expert on average selects the 256-route tiles
    (two weight tiles per CTA, coalesced weight streaming). Shapes cover a partial last K slice
    (96, 288), partial 128- and 256-row feature tiles and experts spanning several route tiles."""
    layer = synth.make_layer(synth.ARCH_GPT_OSS, hidden, ffn, 4, 2, synth.FMT_MXFP4, seed=31)
    check_layer(moe, oracle, layer, tokens, seed=tokens)


@pytest.mark.parametrize("tokens", [100, 250], ids=["nt64", "nt128"])
@pytest.mark.parametrize("narrow", [False, True], ids=["wide", "generic"])
def test_gpt_oss_mid_tiles(moe, oracle, tokens, narrow, monkeypatch):
    """50 and 125 routes per expert on average: partly filled 256-route tiles of the wide kernel (TMA
    boxes of 64 and 128 rows), and the 64- and 128-route tiles of the generic tile kernel (the ones
    Q4_K layers run) when the wide kernel is switched off."""
    if narrow:
        monkeypatch.setenv("OCO_MOE_NARROW_TILES", "1")
    layer = synth.make_layer(synth.ARCH_GPT_OSS, 320, 288, 4, 2, synth.FMT_MXFP4, seed=33)
    check_layer(moe, oracle, layer, tokens, seed=tokens)


@pytest.mark.parametrize("tokens", [40, 9], ids=["avg20", "avg9"])
def test_nemotron_sparse_wide_tiles(moe, oracle, tokens):
    """Just above the few-token limit of eight routes per expert: every expert is one thinly filled
    256-route tile (32-row TMA boxes), shared expert as one dense tile."""
    layer = synth.make_layer(synth.ARCH_NEMOTRON, 256, 160, 4, 2, synth.FMT_Q4_0, seed=34, shared_ffn=320,
                             normalize=True, scale=2.5)
    check_layer(moe, oracle, layer, tokens, seed=tokens)


def test_nemotron_wide_tiles(moe, oracle):
    layer = synth.make_layer(synth.ARCH_NEMOTRON, 256, 160, 4, 2, synth.FMT_Q4_0, seed=32, shared_ffn=320,
                             normalize=True, scale=2.5)
    check_layer(moe, oracle, layer, 450, seed=5)


def test_gpt_oss_forced_routes_reference_ids(moe, oracle):
    """Ids forced as in the reference's tile test: every token sends routes to experts 31 and 30,
    the rest stay sparse (mxfp4.rs:345-347), through a router whose bias alone decides."""
    layer = synth.make_layer(synth.ARCH_GPT_OSS, 96, 96, 32, 4, synth.FMT_MXFP4, seed=3)
    layer.router_w[:] = 0
    tokens = 257
    x, res = synth.make_tokens(96, tokens, 9)
    # one router for all tokens: bias picks 31, 30 plus two fixed others -> over-full experts
    layer.router_b[:] = -10
    for rank, e in enumerate([31, 7, 22, 30]):
        layer.router_b[e] = 4.0 - rank
    ref = oracle.moe_forward(layer, x, res)
    out, routing = moe.run_layer(layer, x, res)
    assert np.array_equal(routing["ids"], np.tile(np.array([31, 7, 22, 30], np.uint32), (tokens, 1)))
    tiles = routing["tiles"]
    nt = int(tiles[1, 1])                      # first expert's second tile starts one tile further
    assert nt in (32, 64, 128, 256)
    per = -(-tokens // nt)
    assert np.array_equal(tiles[:, 0], np.repeat([7, 22, 30, 31], per))
    assert np.array_equal(tiles[:, 1], np.tile(np.arange(per) * nt, 4))
    assert rel_l2(out, ref.out) <= REL_L2


def test_item_counter_and_fixed_deal_agree(moe, oracle, monkeypatch):
    """The wide tile kernel hands its work items out from a counter where a CTA gets five or more (here: 64
    experts x 36 feature tiles on at most 148 CTAs) and deals them c, c + grid, ... otherwise or with
    OCO_MOE_STATIC_TILES=1: the same items either way, so the same bits; three calls in a row on one plan also
    show that the last CTA to leave has put the counter back."""
    layer = synth.make_layer(synth.ARCH_GPT_OSS, 128, 4608, 64, 4, synth.FMT_MXFP4, seed=91)
    x, res = synth.make_tokens(128, 900, 17, "normal")
    plan = moe.plan_for(layer)
    plan.reserve(900)
    plan.bind(moe._Weights.from_layer(layer))
    outs = []
    for _ in range(3):
        got = res.copy()
        plan.forward_host(x, got, 900)
        outs.append(got)
    plan.poll()
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[0], outs[2])
    monkeypatch.setenv("OCO_MOE_STATIC_TILES", "1")
    fixed, routing = moe.run_layer(layer, x, res)
    assert np.array_equal(outs[0], fixed)
    assert rel_l2(fixed, oracle.moe_forward(layer, x, res).out) <= REL_L2


@pytest.mark.parametrize("arch", ["gpt_oss", "nemotron", "qwen"])
def test_pair_tiles(moe, oracle, arch, monkeypatch):
    """The tile kernel on SM pairs (opt-in, OCO_MOE_PAIR_TILES=1: route tiles of up to 512 routes, two CTAs per
    tile): same ids, same tolerance as the default kernels, on experts with 1..128, 129..256, 257..384 and
    385..512 routes and more than 512 (a second tile), and a feature count that is no multiple of 128."""
    monkeypatch.setenv("OCO_MOE_PAIR_TILES", "1")
    if arch == "gpt_oss":
        layer = synth.make_layer(synth.ARCH_GPT_OSS, 192, 160, 8, 2, synth.FMT_MXFP4, seed=81)
    elif arch == "nemotron":
        layer = synth.make_layer(synth.ARCH_NEMOTRON, 256, 192, 8, 2, synth.FMT_Q4_0, seed=82)
    else:
        layer = synth.make_layer(synth.ARCH_QWEN, 512, 256, 8, 2, synth.FMT_Q4_K, seed=83)
    # a skewed router: the bias spreads the expert loads from a few routes to more than 512
    skewed = layer.router_b is not None
    if skewed:
        layer.router_b[:] = np.linspace(-1.5, 2.5, 8).astype(np.float32)
    for tokens in (700, 1100):
        x, res = synth.make_tokens(layer.hidden, tokens, 900 + tokens, "normal")
        if arch == "qwen":
            x = synth.f32_to_bf16_bits(synth.bf16_bits_to_f32(x) * 0.125)
        out, routing = moe.run_layer(layer, x, res)
        ref = oracle.moe_forward(layer, x, res)
        assert np.array_equal(routing["ids"], ref.ids)
        counts = np.bincount(ref.ids.ravel(), minlength=8)
        if skewed:
            assert counts.max() > 512 and counts.min() < 257      # one-half, two-half and two-tile experts all occur
        tiles = routing["tiles"]
        assert len(tiles) == int(np.sum(-(-counts // 512)))       # tiles of 512 routes
        assert rel_l2(out, ref.out) <= REL_L2


def test_gpt_oss_unaligned_weights(moe, oracle):
    """Packed tensors placed 7 bytes off alignment, as the reference tests them (mxfp4.rs:16)."""
    layer = synth.make_layer(synth.ARCH_GPT_OSS, 256, 160, 32, 4, synth.FMT_MXFP4, seed=21)
    check_layer(moe, oracle, layer, 1, seed=1, misalign=7)
    check_layer(moe, oracle, layer, 70, seed=2, misalign=7)


def test_reserved_scale_propagates_nan(moe, oracle):
    """E8M0 = 255 must surface as NaN in the output while ids stay valid (mxfp4.rs:205-233)."""
    layer = synth.make_layer(synth.ARCH_GPT_OSS, 128, 128, 32, 4, synth.FMT_MXFP4, seed=8)
    for tokens in (1, 40):
        x, res = synth.make_tokens(128, tokens, 77)
        clean = oracle.moe_forward(layer, x, res)
        victim = int(clean.ids[0, 0])
        bad = synth.Layer(**{**layer.__dict__})
        bad.up_w = layer.up_w.copy()
        bad.up_w[victim, 5, 0] = 255
        ref = oracle.moe_forward(bad, x, res)
        out, routing = moe.run_layer(bad, x, res)
        assert np.array_equal(routing["ids"], ref.ids)
        g = synth.bf16_bits_to_f32(out)
        r = synth.bf16_bits_to_f32(ref.out)
        assert np.array_equal(np.isnan(g), np.isnan(r))
        assert np.isnan(g[0]).any()


def test_outputs_stay_inside_their_buffers(moe, oracle):
    """Guard rows around the residual stay untouched (the reference's guard-word discipline,
    dispatch_tests.rs:12-13)."""
    import torch
    layer = synth.make_layer(synth.ARCH_GPT_OSS, 96, 96, 32, 4, synth.FMT_MXFP4, seed=4)
    for tokens in (1, 33):
        x, res = synth.make_tokens(96, tokens, 5, "normal")
        guard = 4
        buf = torch.full((tokens + 2 * guard, 96), 0x7FC1, dtype=torch.int16, device="cuda")
        buf[guard:guard + tokens] = torch.from_numpy(res.view(np.int16)).cuda()
        plan = moe.plan_for(layer)
        w = moe._Weights.from_layer(layer)
        xd = torch.from_numpy(x.view(np.int16)).cuda()
        moe.Bindings(moe.Scratch(norm=xd)).experts(w, plan, None, buf[guard:guard + tokens], tokens)
        plan.poll()
        host = buf.cpu().numpy().view(np.uint16)
        assert np.all(host[:guard] == 0x7FC1) and np.all(host[guard + tokens:] == 0x7FC1)
        ref = oracle.moe_forward(layer, x, res)
        assert rel_l2(host[guard:guard + tokens], ref.out) <= REL_L2


@pytest.mark.parametrize("tokens", [1, 9, 130])
def test_nemotron_small(moe, oracle, tokens):
    layer = synth.make_layer(synth.ARCH_NEMOTRON, 256, 160, 128, 6, synth.FMT_Q4_0, seed=12, shared_ffn=320,
                             normalize=True, scale=2.5)
    check_layer(moe, oracle, layer, tokens, seed=tokens)


def test_sigmoid_router_reference_case(moe, oracle):
    """The reference's sigmoid-router fixture (nemotron.rs:279-384): ids exact, weights within 1e-4."""
    c = rc.sigmoid_router_case()
    E, H = c["experts"], c["n"]
    layer = synth.make_layer(synth.ARCH_NEMOTRON, H, 64, E, c["active"], synth.FMT_Q4_0, seed=2, normalize=True,
                             scale=c["scale"])
    layer.router_w, layer.router_b = c["w"].copy(), c["bias"].copy()
    res = np.zeros_like(c["x"])
    _, routing = moe.run_layer(layer, c["x"], res)
    assert np.array_equal(routing["ids"], c["ids"])
    assert np.all(np.abs(routing["prob"] - c["probs"]) <= 1e-4 * np.maximum(np.abs(c["probs"]), 1.0))


@pytest.mark.parametrize("tokens", [1, 24, 200])
@pytest.mark.parametrize("narrow", [False, True], ids=["wide", "generic"])
def test_qwen_small(moe, oracle, tokens, narrow, monkeypatch):
    if narrow:
        if tokens == 1:
            pytest.skip("single-token path has one implementation")
        monkeypatch.setenv("OCO_MOE_NARROW_TILES", "1")
    layer = synth.make_layer(synth.ARCH_QWEN, 512, 256, 128, 8, synth.FMT_Q4_K, seed=13)
    check_layer(moe, oracle, layer, tokens, seed=tokens)


@pytest.mark.parametrize("hidden,ffn,tokens", [(768, 512, 1300), (512, 768, 900), (256, 1280, 700)],
                         ids=["k768", "k512", "k256"])
def test_qwen_wide_tiles(moe, oracle, hidden, ffn, tokens):
    """Q4_K through the 256-route tiles: experts spanning several route tiles, one and several
    super-blocks per row, partial 128- and 256-row feature tiles."""
    layer = synth.make_layer(synth.ARCH_QWEN, hidden, ffn, 8, 2, synth.FMT_Q4_K, seed=52)
    check_layer(moe, oracle, layer, tokens, seed=tokens, x_scale=0.125)


@pytest.mark.parametrize("arch", ["gpt-oss", "nemotron", "qwen"])
def test_register_blocked_router(moe, oracle, arch, monkeypatch):
    """The many-token router kernel (four tokens x four experts per warp) from 33 rows on: ragged last
    token group, expert ranges split over CTAs, a partial last column chunk; ids, logits and weights
    stay bit-exact."""
    monkeypatch.setenv("OCO_MOE_ROUTER_BLOCK_MIN", "33")
    if arch == "gpt-oss":
        layer = synth.make_layer(synth.ARCH_GPT_OSS, 736, 384, 32, 4, synth.FMT_MXFP4, seed=61)
    elif arch == "nemotron":
        layer = synth.make_layer(synth.ARCH_NEMOTRON, 256, 160, 20, 3, synth.FMT_Q4_0, seed=62, shared_ffn=320,
                                 normalize=True, scale=2.5)
    else:
        layer = synth.make_layer(synth.ARCH_QWEN, 512, 256, 128, 8, synth.FMT_Q4_K, seed=63)
    for tokens in (45, 333):
        check_layer(moe, oracle, layer, tokens, seed=700 + tokens, x_scale=0.125 if arch == "qwen" else 1.0)


def test_host_buffer_entry_point(moe, oracle):
    layer = synth.make_layer(synth.ARCH_GPT_OSS, 128, 128, 32, 4, synth.FMT_MXFP4, seed=6)
    x, res = synth.make_tokens(128, 50, 3, "normal")
    plan = moe.plan_for(layer)
    plan.reserve(50)
    plan.bind(moe._Weights.from_layer(layer))
    got = res.copy()
    plan.forward_host(x, got, 50)
    plan.poll()
    assert plan.launch_count() >= 5
    ref = oracle.moe_forward(layer, x, res)
    assert rel_l2(got, ref.out) <= REL_L2
    with pytest.raises(moe.OcoError):
        plan.forward_host(x, got, 51)      # beyond the reserved rows: a status, not a crash


def test_host_graph(moe, oracle):
    """oco_moe_graph_capture_host: one replay copies the pinned rows in, runs the layer and copies the residual
    rows back; refreshed host contents give the result of oco_moe_forward_host on them, bit for bit."""
    import torch
    layer = synth.make_layer(synth.ARCH_GPT_OSS, 256, 192, 32, 4, synth.FMT_MXFP4, seed=17)
    plan = moe.plan_for(layer)
    plan.reserve(8)
    plan.bind(moe._Weights.from_layer(layer))
    for rows in (1, 8):
        x, res = synth.make_tokens(256, rows, 60 + rows, "normal")
        hx = torch.from_numpy(x.view(np.int16).copy()).pin_memory().numpy().view(np.uint16)
        hres = torch.from_numpy(res.view(np.int16).copy()).pin_memory().numpy().view(np.uint16)
        g = plan.capture_host(hx, hres, rows)
        for seed in (1, 2):
            x2, res2 = synth.make_tokens(256, rows, 70 + seed, "normal")
            hx[:] = x2
            hres[:] = res2
            g.replay()
            torch.cuda.current_stream().synchronize()
            one = res2.copy()
            plan.forward_host(x2, one, rows)
            assert np.array_equal(hres, one)
            assert rel_l2(hres, oracle.moe_forward(layer, x2, res2).out) <= REL_L2
        del g
    plan.poll()


def test_host_calls_in_flight(moe, oracle):
    """Two host calls in flight (oco_moe_forward_host_begin / _end): six calls on different rows, each ended
    only after the next one was begun, give what the one-call-at-a-time entry point gives, bit for bit, and
    that equals the oracle; a third call in flight and an end without a call are refused with a status."""
    import torch
    layer = synth.make_layer(synth.ARCH_GPT_OSS, 256, 192, 32, 4, synth.FMT_MXFP4, seed=16)
    rows = 760
    plan = moe.plan_for(layer)
    plan.reserve(rows)
    plan.bind(moe._Weights.from_layer(layer))
    with pytest.raises(moe.OcoError):
        plan.forward_host_end()
    calls = []
    for c in range(6):
        # ragged: every call has its own row count; calls 2 and 5 are small enough (under 256 KB per buffer) to run
        # on the caller's stream alone, the others use the plan's copy streams, and all share the two staging slots
        n = 90 + c if c in (2, 5) else rows - 37 * c
        x, res = synth.make_tokens(256, n, 40 + c, "normal")
        hx = torch.from_numpy(x.view(np.int16)).pin_memory().numpy().view(np.uint16)
        hres = torch.from_numpy(res.view(np.int16).copy()).pin_memory().numpy().view(np.uint16)
        calls.append((n, x, res, hx, hres))
    for c, (n, x, res, hx, hres) in enumerate(calls):
        plan.forward_host_begin(hx, hres, n)
        if c == 1:
            with pytest.raises(moe.OcoError):               # calls 0 and 1 are in flight
                plan.forward_host_begin(hx, hres, n)
        if c >= 1:
            plan.forward_host_end()                         # call c - 1
    plan.forward_host_end()
    plan.poll()
    for n, x, res, hx, hres in calls:
        one = res.copy()
        plan.forward_host(x, one, n)
        assert np.array_equal(hres, one)
    n, x, res, hx, hres = calls[0]
    assert rel_l2(hres, oracle.moe_forward(layer, x, res).out) <= REL_L2


def selection_margin(layer, x_bits, logits_f32, ids):
    """Smallest gap, over the tokens, between the last selected and the first rejected expert, measured on
    logits recomputed in float64 from the same rounded operands (bf16 x; bf16 router weights and bias for the
    gpt-oss family), and the largest distance of the float32 logits from them. A margin far above that
    distance means no legal summation order could have selected other experts."""
    x = synth.bf16_bits_to_f32(x_bits).astype(np.float64)
    w = layer.router_w.astype(np.float64)
    if layer.arch == synth.ARCH_GPT_OSS:
        w = synth.bf16_bits_to_f32(synth.f32_to_bf16_bits(layer.router_w)).astype(np.float64)
    z = x @ w.T
    if layer.arch == synth.ARCH_GPT_OSS:
        z = z + synth.bf16_bits_to_f32(synth.f32_to_bf16_bits(layer.router_b)).astype(np.float64)
    score = z
    if layer.arch == synth.ARCH_NEMOTRON:        # selection on sigmoid(z) + bias: monotone in z only without the bias
        score = 1.0 / (1.0 + np.exp(-z)) + layer.router_b.astype(np.float64)
    chosen = np.zeros(score.shape, bool)
    np.put_along_axis(chosen, ids.astype(np.int64), True, axis=1)
    lowest_in = np.where(chosen, score, np.inf).min(axis=1)
    highest_out = np.where(chosen, -np.inf, score).max(axis=1)
    return float((lowest_in - highest_out).min()), float(np.abs(logits_f32.astype(np.float64) - z).max())


def _sampled_full_size(moe, oracle, name, tokens, sample, seed, mode):
    """Full benchmark shape on the GPU; the oracle re-computes a sample of the tokens (tokens are
    independent in this layer) plus the router for all of them. The sample is spread over the batch and
    always holds tokens routed to the fullest and to the emptiest expert."""
    layer = synth.make_config(name, seed=seed)
    x, res = synth.make_tokens(layer.hidden, tokens, seed, "normal")
    out, routing = moe.run_layer(layer, x, res)
    if layer.arch == synth.ARCH_GPT_OSS:
        _, ids, probs = oracle.router_gptoss(x, layer.router_w, layer.router_b, layer.top_k)
    elif layer.arch == synth.ARCH_NEMOTRON:
        _, ids, probs = oracle.router_sigmoid(x, layer.router_w, layer.router_b, layer.top_k, layer.normalize, layer.scale)
    else:
        _, ids, probs = oracle.router_softmax_topk(x, layer.router_w, layer.top_k)
    assert np.array_equal(routing["ids"], ids)
    assert np.array_equal(routing["prob"].view(np.uint32), probs.view(np.uint32))
    margin, drift = selection_margin(layer, x, routing["logits"], ids)
    print(f"{name} x {tokens}: smallest selection margin {margin:.3e}, largest |f32 logit - f64 logit| {drift:.3e}")
    assert margin > 0, "the float64 logits select other experts"
    pick = set(np.linspace(0, tokens - 1, sample).astype(int).tolist())
    if tokens > 1:
        offsets, row_of_route, route_of_row = oracle.permutation(ids, layer.experts)
        assert np.array_equal(routing["offsets"], offsets)
        assert np.array_equal(routing["row_of_route"], row_of_route)
        assert np.array_equal(routing["route_of_row"], route_of_row)
        counts = np.diff(offsets.astype(np.int64))
        fullest, emptiest = int(counts.argmax()), int(np.where(counts > 0, counts, counts.max() + 1).argmin())
        for e in (fullest, emptiest):
            rows = np.nonzero((ids == e).any(axis=1))[0]
            pick.update(rows[:2].tolist())
    pick = np.array(sorted(pick))
    ref = oracle.moe_forward(layer, x[pick], res[pick], mode=mode, trace=False)
    assert np.array_equal(ref.ids, ids[pick])
    err = rel_l2(out[pick], ref.out)
    assert err <= REL_L2, f"{name} rel-L2 {err}"


@pytest.mark.parametrize("tokens", [2, 5, 12, 31], ids=["t2", "t5", "t12", "t31"])
def test_gpt_oss_few_tokens_streamed(moe, oracle, tokens):
    """At most four routes per expert on average: the streamed few-token kernels (up to eight routes
    of an expert in the columns of one MMA), K not a multiple of 16 blocks, partial last group."""
    layer = synth.make_layer(synth.ARCH_GPT_OSS, 640, 384, 32, 4, synth.FMT_MXFP4, seed=41)
    check_layer(moe, oracle, layer, tokens, seed=300 + tokens)


def test_few_tokens_crowded_expert(moe, oracle):
    """One expert gets a route from every token (13 routes: two groups, 8 + 5) while the average
    stays small; the other routes are spread by the router."""
    layer = synth.make_layer(synth.ARCH_GPT_OSS, 320, 288, 32, 4, synth.FMT_MXFP4, seed=43)
    layer.router_b[9] = 50.0
    check_layer(moe, oracle, layer, 13, seed=77, residual="normal")


@pytest.mark.parametrize("tokens", [2, 20])
def test_nemotron_few_tokens_streamed(moe, oracle, tokens):
    layer = synth.make_layer(synth.ARCH_NEMOTRON, 256, 192, 32, 6, synth.FMT_Q4_0, seed=44, shared_ffn=320,
                             normalize=True, scale=2.5)
    check_layer(moe, oracle, layer, tokens, seed=tokens)


@pytest.mark.parametrize("tokens", [1, 3])
def test_wide_layer_falls_back_to_tiles(moe, oracle, tokens):
    """hidden = 8192 is too wide for the token's fragments to share the SM with the streaming rings:
    single tokens and small batches then take the tile kernels (tile numerics, also for one token)."""
    layer = synth.make_layer(synth.ARCH_GPT_OSS, 8192, 128, 8, 2, synth.FMT_MXFP4, seed=61)
    check_layer(moe, oracle, layer, tokens, seed=tokens, mode=2)


def test_hidden_4096_single_token(moe, oracle):
    layer = synth.make_layer(synth.ARCH_GPT_OSS, 4096, 256, 8, 2, synth.FMT_MXFP4, seed=62)
    check_layer(moe, oracle, layer, 1, seed=4)
    check_layer(moe, oracle, layer, 5, seed=5)


@pytest.mark.parametrize("arch,full_layer", [(synth.ARCH_GPT_OSS, True), (synth.ARCH_QWEN, False)], ids=["gpt-oss", "qwen"])
@pytest.mark.parametrize("rows", [1, 40])
def test_add_norm_forward(moe, oracle, arch, full_layer, rows):
    """Residual add + RMS norm + layer in one call: the summed rows and the normalised rows are
    bit-exact against the checker, the layer output meets the usual bar."""
    import torch
    fmt = synth.FMT_MXFP4 if arch == synth.ARCH_GPT_OSS else synth.FMT_Q4_K
    H = 512
    layer = synth.make_layer(arch, H, 256, 16, 4, fmt, seed=71)
    rng = np.random.default_rng(rows)
    hidden, projected = synth.make_tokens(H, rows, 11, "normal")
    weight = rng.normal(1.0, 0.2, size=H).astype(np.float32)
    eps = 1e-5
    for delta in (projected, None):
        summed, normed = oracle.add_norm(hidden, delta, weight, eps, full_layer)
        ref = oracle.moe_forward(layer, normed, summed)
        plan = moe.plan_for(layer)
        w = moe._Weights.from_layer(layer)
        plan.reserve(rows); plan.bind(w)
        h = torch.from_numpy(hidden.view(np.int16).copy()).cuda()
        d = None if delta is None else torch.from_numpy(delta.view(np.int16).copy()).cuda()
        nw = torch.from_numpy(weight).cuda()
        plan.add_norm_forward(h, d, nw, eps, full_layer, rows)
        plan.poll()
        routing = moe.Routing(); routing.plan, routing.rows = plan, rows
        view = routing.read()
        assert np.array_equal(view["norm"], normed), "normalised rows differ"
        assert np.array_equal(view["ids"], ref.ids)
        out = h.cpu().numpy().view(np.uint16)
        assert rel_l2(out, ref.out) <= REL_L2


@pytest.mark.parametrize("narrow", [False, True], ids=["wide", "generic"])
def test_few_tokens_tile_kernels(moe, oracle, monkeypatch, narrow):
    """The same small batches through the tile kernels instead of the streamed ones."""
    monkeypatch.setenv("OCO_MOE_NO_BATCH", "1")
    if narrow:
        monkeypatch.setenv("OCO_MOE_NARROW_TILES", "1")
    layer = synth.make_layer(synth.ARCH_GPT_OSS, 640, 384, 32, 4, synth.FMT_MXFP4, seed=41)
    for tokens in (2, 12):
        check_layer(moe, oracle, layer, tokens, seed=300 + tokens)


def test_gpt_oss_120b_decode_batch_full_size(moe, oracle):
    _sampled_full_size(moe, oracle, "gpt-oss-120b", 64, 4, seed=0, mode=2)


def test_qwen3_30b_decode_full_size(moe, oracle):
    _sampled_full_size(moe, oracle, "qwen3-30b-a3b", 1, 1, seed=0, mode=1)


def test_nemotron_h_decode_full_size(moe, oracle):
    _sampled_full_size(moe, oracle, "nemotron-h", 1, 1, seed=0, mode=1)


@pytest.mark.parametrize("hidden,ffn", [(256, 256), (768, 512), (2048, 768)])
def test_qwen_single_token_shapes(moe, oracle, hidden, ffn):
    """Q4_K single-token kernels: one and several super-blocks per row, splits that end inside a row."""
    layer = synth.make_layer(synth.ARCH_QWEN, hidden, ffn, 16, 4, synth.FMT_Q4_K, seed=51)
    check_layer(moe, oracle, layer, 1, seed=hidden, residual="normal")
    check_layer(moe, oracle, layer, 1, seed=hidden + 1, misalign=3)


def test_gpt_oss_20b_decode_full_size(moe, oracle):
    _sampled_full_size(moe, oracle, "gpt-oss-20b", 1, 1, seed=0, mode=1)


def test_gpt_oss_20b_prefill_full_size(moe, oracle):
    _sampled_full_size(moe, oracle, "gpt-oss-20b", 2048, 32, seed=0, mode=2)


def test_qwen3_30b_prefill_full_size(moe, oracle):
    _sampled_full_size(moe, oracle, "qwen3-30b-a3b", 512, 12, seed=0, mode=2)


def test_nemotron_h_prefill_full_size(moe, oracle):
    _sampled_full_size(moe, oracle, "nemotron-h", 1024, 8, seed=0, mode=2)


def test_gpt_oss_120b_prefill_full_size(moe, oracle):
    _sampled_full_size(moe, oracle, "gpt-oss-120b", 8192, 12, seed=0, mode=2)


# ---- the block-scaled single-token kernels (opt-in) --------------------------------------------------
@pytest.mark.parametrize("hidden,ffn,experts,misalign", [(96, 96, 32, 0), (640, 384, 32, 0), (256, 160, 32, 7), (2880, 2880, 32, 0),
                                                          (4096, 256, 8, 3)],
                         ids=["k96", "k640", "unaligned", "20b", "k4096"])
def test_gpt_oss_single_token_block_scaled(moe, oracle, monkeypatch, hidden, ffn, experts, misalign):
    """MXFP4 rows fed to tcgen05 kind::mxf4 as they are, the token split into e2m1 pieces: odd and even row
    strides (run-time and constant shifts), partial last K groups, unaligned tensors, the benchmark shape."""
    monkeypatch.setenv("OCO_MOE_TOKEN_MX", "1")
    layer = synth.make_layer(synth.ARCH_GPT_OSS, hidden, ffn, experts, min(4, experts), synth.FMT_MXFP4, seed=91)
    err = check_layer(moe, oracle, layer, 1, seed=hidden, residual="normal", misalign=misalign, mode=1)
    assert err <= 2e-4, f"pieces should carry the activations nearly exactly, rel-L2 {err}"


def test_block_scaled_token_path_propagates_nan(moe, oracle, monkeypatch):
    monkeypatch.setenv("OCO_MOE_TOKEN_MX", "1")
    layer = synth.make_layer(synth.ARCH_GPT_OSS, 128, 128, 32, 4, synth.FMT_MXFP4, seed=8)
    x, res = synth.make_tokens(128, 1, 77)
    clean = oracle.moe_forward(layer, x, res)
    bad = synth.Layer(**{**layer.__dict__})
    bad.up_w = layer.up_w.copy()
    bad.up_w[int(clean.ids[0, 0]), 5, 0] = 255
    ref = oracle.moe_forward(bad, x, res)
    out, routing = moe.run_layer(bad, x, res)
    assert np.array_equal(routing["ids"], ref.ids)
    assert np.array_equal(np.isnan(synth.bf16_bits_to_f32(out)), np.isnan(synth.bf16_bits_to_f32(ref.out)))


# ---- one interleaved gate_up tensor instead of two ---------------------------------------------------
@pytest.mark.parametrize("tokens,env", [(1, {}), (1, {"OCO_MOE_TOKEN_MX": "1"}), (6, {}), (70, {}), (70, {"OCO_MOE_NARROW_TILES": "1"}),
                                        (300, {})], ids=["t1", "t1-mx", "t6", "t70", "t70-generic", "t300"])
def test_interleaved_gate_up_is_bit_identical(moe, oracle, monkeypatch, tokens, env):
    """Row 2c = gate row c, row 2c + 1 = up row c (and the biases likewise) must give the very bits the
    two-tensor layout gives, on every kernel family."""
    for k, v in env.items():
        monkeypatch.setenv(k, v)
    layer = synth.make_layer(synth.ARCH_GPT_OSS, 320, 288, 8, 2, synth.FMT_MXFP4, seed=17)
    x, res = synth.make_tokens(320, tokens, 5, "normal")
    split, r0 = moe.run_layer(layer, x, res, misalign=5)
    both, r1 = moe.run_layer(layer, x, res, misalign=5, interleaved=True)
    assert np.array_equal(split, both)
    assert np.array_equal(r0["ids"], r1["ids"]) and np.array_equal(r0["y"], r1["y"])
    ref = oracle.moe_forward(layer, x, res)
    assert rel_l2(both, ref.out) <= REL_L2


def test_interleaved_and_split_tensors_are_exclusive(moe):
    from oco_b200 import _lib
    layer = synth.make_layer(synth.ARCH_GPT_OSS, 96, 96, 4, 2, synth.FMT_MXFP4, seed=3)
    plan = moe.plan_for(layer)
    w = moe._Weights.from_layer(layer, interleaved=True)
    w.gate_w = w.gate_up_w
    with pytest.raises(moe.OcoError) as e:
        plan.bind(w)
    assert e.value.code == _lib.INVALID_ARGUMENT


# ---- bounded device waits --------------------------------------------------------------------------
def test_bounded_wait_gives_up_and_recovers(moe, oracle):
    """A wait on a barrier nobody arrives at runs out (a few microseconds here), the kernel returns
    normally, poll reports DEVICE_TIMEOUT once, a forward enqueued before the poll leaves the residual
    untouched, and the first forward after the poll is correct again."""
    import ctypes as C
    import torch
    from oco_b200 import _lib
    layer = synth.make_layer(synth.ARCH_GPT_OSS, 128, 128, 32, 4, synth.FMT_MXFP4, seed=6)
    for tokens in (1, 40):
        x, res = synth.make_tokens(128, tokens, 3, "normal")
        plan = moe.plan_for(layer)
        plan.reserve(tokens)
        plan.bind(moe._Weights.from_layer(layer))
        xd = torch.from_numpy(x.view(np.int16)).cuda()
        rd = torch.from_numpy(res.view(np.int16).copy()).cuda()
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        assert _lib.lib().oco_moe_selftest_wait_timeout(plan.handle, 20000, stream) == _lib.OK
        plan.forward(xd, rd, tokens)                       # enqueued while the status word is set
        with pytest.raises(moe.OcoError) as e:
            plan.poll()
        assert e.value.code == _lib.DEVICE_TIMEOUT
        assert np.array_equal(rd.cpu().numpy().view(np.uint16), res), "a poisoned step changed the residual"
        plan.poll()                                        # reported once, then clear
        plan.forward(xd, rd, tokens)
        plan.poll()
        ref = oracle.moe_forward(layer, x, res)
        assert rel_l2(rd.cpu().numpy().view(np.uint16), ref.out) <= REL_L2
    assert _lib.lib().oco_moe_selftest_wait_timeout(plan.handle, 0, stream) == _lib.INVALID_ARGUMENT


def test_event_seam_times_a_forward(moe):
    import ctypes as C
    import torch
    from oco_b200 import _lib
    L = _lib.lib()
    layer = synth.make_layer(synth.ARCH_GPT_OSS, 128, 128, 8, 2, synth.FMT_MXFP4, seed=2)
    x, res = synth.make_tokens(128, 64, 1)
    plan = moe.plan_for(layer)
    plan.reserve(64)
    plan.bind(moe._Weights.from_layer(layer))
    xd = torch.from_numpy(x.view(np.int16)).cuda()
    rd = torch.from_numpy(res.view(np.int16).copy()).cuda()
    a, b = C.c_void_p(), C.c_void_p()
    assert L.oco_cuda_event_create(C.byref(a)) == _lib.OK and L.oco_cuda_event_create(C.byref(b)) == _lib.OK
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert L.oco_cuda_event_record(a, stream) == _lib.OK
    plan.forward(xd, rd, 64)
    assert L.oco_cuda_event_record(b, stream) == _lib.OK
    assert L.oco_cuda_event_sync(b) == _lib.OK
    ms = C.c_float(-1.0)
    assert L.oco_cuda_event_elapsed_ms(a, b, C.byref(ms)) == _lib.OK and 0.0 < ms.value < 1000.0
    assert L.oco_cuda_event_destroy(a) == _lib.OK and L.oco_cuda_event_destroy(b) == _lib.OK


def test_plan_is_tied_to_its_device(moe):
    """Kernel attributes and the workspace belong to one device: a call with another device current is
    refused (needs two GPUs to show; with one, the same-device call must pass)."""
    import torch
    from oco_b200 import _lib
    layer = synth.make_layer(synth.ARCH_GPT_OSS, 128, 128, 8, 2, synth.FMT_MXFP4, seed=2)
    x, res = synth.make_tokens(128, 1, 1)
    plan = moe.plan_for(layer)
    plan.reserve(1)
    plan.bind(moe._Weights.from_layer(layer))
    xd = torch.from_numpy(x.view(np.int16)).cuda()
    rd = torch.from_numpy(res.view(np.int16).copy()).cuda()
    plan.forward(xd, rd, 1)
    plan.poll()
    if torch.cuda.device_count() > 1:
        with torch.cuda.device(1):
            with pytest.raises(moe.OcoError) as e:
                plan.forward(xd, rd, 1)
            assert e.value.code == _lib.INVALID_ARGUMENT



def test_expert_shard_with_fewer_experts_than_routes_per_token(moe, oracle):
    """A plan over a shard of the experts (expert parallelism) may hold fewer experts than the layer's
    top_k: it never routes, it only multiplies rows that arrive with their local expert id."""
    import ctypes as C
    import torch
    from oco_b200 import _lib
    E, K, H, F, R = 4, 6, 256, 192, 50
    layer = synth.make_layer(synth.ARCH_NEMOTRON, H, F, E, 2, synth.FMT_Q4_0, seed=23, normalize=True, scale=2.5)
    plan = moe._Plan(synth.ARCH_NEMOTRON, H, F, E, K, synth.FMT_Q4_0, normalize=True, scale=2.5)
    shard = synth.Layer(**{**layer.__dict__})
    shard.router_w = shard.router_b = None
    w = moe._Weights.from_layer(shard)
    plan.reserve(R)
    plan.bind(w)
    rng = np.random.default_rng(1)
    x, _ = synth.make_tokens(H, R, 3)
    ids = rng.integers(0, E, size=R).astype(np.uint32)
    xd = torch.from_numpy(x.view(np.int16)).cuda()
    idd = torch.from_numpy(ids.view(np.int32)).cuda()
    y = torch.zeros((R, H), dtype=torch.int16, device="cuda")
    rc = _lib.lib().oco_moe_experts(plan.handle, C.c_void_p(xd.data_ptr()), C.c_void_p(idd.data_ptr()), R, C.c_void_p(y.data_ptr()),
                                    C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == _lib.OK, _lib.lib().oco_moe_last_error(plan.handle)
    plan.poll()
    up = oracle.expert_up_tile(layer.up_w, x, None, 0.0, ids, 1, H, F, fmt=synth.FMT_Q4_0)
    up = synth.bf16_bits_to_f32(synth.f32_to_bf16_bits(up))          # the projection is rounded to bf16, then relu^2 in f32 -> half
    act = (np.maximum(up, 0.0) ** 2).astype(np.float16)
    ref = oracle.expert_down_tile(layer.down_w, act.view(np.uint16), None, ids, F, H, fmt=synth.FMT_Q4_0)
    assert rel_l2(y.cpu().numpy().view(np.uint16), ref) <= 2e-3
    # a router over four experts cannot pick six
    bad = moe._Plan(synth.ARCH_NEMOTRON, H, F, E, K, synth.FMT_Q4_0, normalize=True, scale=2.5)
    with pytest.raises(moe.OcoError):
        bad.bind(moe._Weights.from_layer(layer))



# ---- opt-in block-scaled numerics (numerics = 2): MXFP4 activations on tcgen05 kind::mxf4 ---------------
def _swiglu(gate, up):
    g = np.minimum(gate, 7.0)
    u = np.clip(up, -6.0, 8.0)
    return g / (1.0 + np.exp(-1.702 * g)) * u


@pytest.mark.parametrize("repacked", [False, True], ids=["spans", "repacked"])
@pytest.mark.parametrize("hidden,ffn,experts,top_k,tokens", [(256, 256, 4, 2, 300), (320, 288, 8, 2, 700), (96, 96, 4, 2, 200),
                                                              (640, 384, 32, 4, 40)], ids=["k256", "k320", "k96", "sparse"])
def test_block_scaled_numerics_match_their_own_arithmetic(moe, oracle, hidden, ffn, experts, top_k, tokens, repacked):
    """The opt-in mode multiplies MXFP4 weights with MXFP4-quantised activations. Its results are held to a
    checker that multiplies THE SAME quantised operands in float64 (both stages, each fed what the GPU fed
    it), and the distance to the reference arithmetic is printed beside it: the price of the mode."""
    from tests import mxq
    layer = synth.make_layer(synth.ARCH_GPT_OSS, hidden, ffn, experts, top_k, synth.FMT_MXFP4, seed=hidden + tokens)
    x, res = synth.make_tokens(hidden, tokens, 3, "normal")
    out, routing = moe.run_layer(layer, x, res, numerics=2, repacked=repacked)
    if repacked:
        # the weights as stored (producer warps move the bytes) and their repacked form (every operand by TMA) feed
        # the same MMAs with the same operands: the two must agree bit for bit
        out_spans, routing_spans = moe.run_layer(layer, x, res, numerics=2)
        assert np.array_equal(out, out_spans) and np.array_equal(routing["y"], routing_spans["y"]), "repacked weights change the result"
    ref = oracle.moe_forward(layer, x, res, mode=2)
    assert np.array_equal(routing["ids"], ref.ids) and np.array_equal(routing["prob"].view(np.uint32), ref.probs.view(np.uint32))
    offsets, row_of_route, route_of_row = oracle.permutation(ref.ids, experts)
    assert np.array_equal(routing["row_of_route"], row_of_route)
    ids = ref.ids.reshape(-1)
    E, F, H = experts, ffn, hidden
    deq = lambda w, rows, k: oracle.dequant(synth.FMT_MXFP4, w.reshape(rows, -1), rows * k).reshape(rows, k).astype(np.float64)
    gate_w, up_w, down_w = deq(layer.gate_w, E * F, H).reshape(E, F, H), deq(layer.up_w, E * F, H).reshape(E, F, H), deq(layer.down_w, E * H, F).reshape(E, H, F)
    bf = lambda a: synth.bf16_bits_to_f32(synth.f32_to_bf16_bits(np.asarray(a, np.float32))).astype(np.float64)
    xq = mxq.quantize_dequantize(synth.bf16_bits_to_f32(x))                     # [T, H]
    act_gpu = routing["act"].view(np.float16)[row_of_route]                      # route order, element order
    y_gpu = synth.bf16_bits_to_f32(routing["y"]).astype(np.float64)
    act_ref = np.empty((ids.size, F)); y_ref = np.empty((ids.size, H))
    actq_gpu = mxq.quantize_dequantize(act_gpu.astype(np.float32))              # what the GPU's down tiles multiplied
    for r, e in enumerate(ids):
        xr = xq[r // top_k]
        g = gate_w[e] @ xr + bf(layer.gate_b[e])
        u = up_w[e] @ xr + bf(layer.up_b[e] + np.float32(1.0))
        act_ref[r] = _swiglu(g, u)
        y_ref[r] = down_w[e] @ actq_gpu[r] + bf(layer.down_b[e])
    rel = lambda a, b: np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30)
    err_act, err_y = rel(act_gpu.astype(np.float64), act_ref.astype(np.float16).astype(np.float64)), rel(y_gpu, bf(y_ref))
    ref_out = synth.bf16_bits_to_f32(ref.out).astype(np.float64)
    away = rel(synth.bf16_bits_to_f32(out).astype(np.float64), ref_out)
    print(f"numerics 2, hidden {hidden}: act rel-L2 {err_act:.2e}, expert outputs {err_y:.2e} against the same quantised operands; "
          f"layer output {away:.2e} away from the reference arithmetic")
    assert err_act <= REL_L2 and err_y <= REL_L2   # both sides rounded to the stored type (half rows, bf16 rows)
    got = oracle.moe_sum(routing["y"], ref.probs, res, top_k)
    assert np.array_equal(got, out), "combine of the mode's expert outputs"
    assert away < 0.5


def test_block_scaled_numerics_are_refused_where_they_do_not_apply(moe):
    from oco_b200 import _lib
    with pytest.raises(moe.OcoError) as e:
        moe._Plan(synth.ARCH_QWEN, 512, 256, 16, 4, synth.FMT_Q4_K, numerics=2)
    assert e.value.code == _lib.UNSUPPORTED_SHAPE
    with pytest.raises(moe.OcoError):
        moe._Plan(synth.ARCH_GPT_OSS, 512, 256, 16, 4, synth.FMT_MXFP4, numerics=1)


def test_recorded_step_replays_the_forward_call(moe, oracle):
    """oco_moe_graph_capture / _launch: one token's step recorded once and replayed on fresh buffer contents
    gives what the direct call gives, bit for bit; a refused call leaves no capture open."""
    import torch
    from oco_b200 import _lib
    layer = synth.make_layer(synth.ARCH_GPT_OSS, 256, 192, 32, 4, synth.FMT_MXFP4, seed=71)
    plan = moe.plan_for(layer)
    plan.reserve(4)
    w = moe._Weights.from_layer(layer)
    plan.bind(w)
    x = torch.zeros((1, layer.hidden), dtype=torch.int16, device="cuda")
    res = torch.zeros((1, layer.hidden), dtype=torch.int16, device="cuda")
    g = plan.capture(x, res, 1)
    for seed in (3, 4):
        xb, rb = synth.make_tokens(layer.hidden, 1, seed, "normal")
        x.copy_(torch.from_numpy(xb.view(np.int16)))
        res.copy_(torch.from_numpy(rb.view(np.int16)))
        g.replay()
        torch.cuda.synchronize()
        got = res.cpu().numpy().view(np.uint16).copy()
        res.copy_(torch.from_numpy(rb.view(np.int16)))
        plan.forward(x, res, 1)
        torch.cuda.synchronize()
        assert np.array_equal(got, res.cpu().numpy().view(np.uint16))
        ref = oracle.moe_forward(layer, xb, rb)
        assert rel_l2(got, ref.out) <= REL_L2
    plan.poll()
    # more rows than reserved: refused, and the next direct call still works (the capture was closed)
    with pytest.raises(moe.OcoError) as e:
        plan.capture(x, res, 9)
    assert e.value.code == _lib.INVALID_ARGUMENT
    plan.forward(x, res, 1)
    torch.cuda.synchronize()
    plan.poll()


@pytest.mark.parametrize("tokens_per_source,single_max", [(40, "2048"), (700, "0"), (700, "2048")], ids=["few", "many_cta_plan", "one_cta_plan"])
def test_expert_stage_over_a_window_numbering(moe, oracle, tokens_per_source, single_max, monkeypatch):
    """oco_moe_experts_window on one GPU, three sources' rows and outputs in one buffer laid out as the
    expert-parallel windows are (slot strides wider than the slots' contents): routes of this shard are read
    at label / top_k and answered at label exactly as oco_moe_experts answers the same rows handed over
    compactly; routes of other shards and the padding leave their output rows untouched."""
    import ctypes as C
    import torch
    from oco_b200 import _lib, ep
    monkeypatch.setenv("OCO_MOE_ROUTE_PLAN_SINGLE_MAX", single_max)
    E, K, H, F = 16, 4, 320, 288
    sources, cap = 3, tokens_per_source
    layer = synth.make_layer(synth.ARCH_GPT_OSS, H, F, E, K, synth.FMT_MXFP4, seed=91)
    lo, epr = 4, 8                                            # this shard: experts 4 .. 11
    shard = synth.Layer(**{**layer.__dict__})
    shard.experts = epr
    for name in ("gate_w", "up_w", "down_w", "gate_b", "up_b", "down_b"):
        setattr(shard, name, getattr(layer, name)[lo:lo + epr])
    shard.router_w = shard.router_b = None
    plan = moe._Plan(synth.ARCH_GPT_OSS, H, F, epr, K, synth.FMT_MXFP4)
    plan.reserve(sources * cap)
    plan.bind(moe._Weights.from_layer(shard))
    slot_tokens, slot_routes = ep.window_geometry(H, K, cap, 4096)       # any granularity: one buffer stands for the windows
    assert slot_tokens > cap or tokens_per_source % 32 == 0
    cap_routes = cap * K
    x_bits, _ = synth.make_tokens(H, sources * cap, 5, "normal")
    _, ids, _ = oracle.router_gptoss(x_bits, layer.router_w, layer.router_b, K)
    live = [cap, cap - 7, 1]                                             # tokens each source brings; the rest is padding
    xw = np.zeros((sources * slot_tokens, H), np.uint16)
    ids_all = np.full((sources, cap_routes), 0xffffffff, np.uint32)
    for g in range(sources):
        xw[g * slot_tokens: g * slot_tokens + live[g]] = x_bits[g * cap: g * cap + live[g]]
        ids_all[g, : live[g] * K] = ids[g * cap: g * cap + live[g]].reshape(-1)
    local = (ids_all.reshape(-1) - np.uint32(lo)).astype(np.uint32)     # other shards' ids wrap out of 0 .. epr - 1
    labels = ep.window_labels(sources, cap_routes, slot_routes)
    mine = np.nonzero(local < epr)[0]
    xd = torch.from_numpy(xw.view(np.int16)).cuda()
    idd = torch.from_numpy(local.view(np.int32)).cuda()
    sentinel = np.int16(0x7fc1)          # the canary the reference's tests put around their outputs
    yw = torch.full((sources * slot_routes, H), int(sentinel), dtype=torch.int16, device="cuda")
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = _lib.lib().oco_moe_experts_window(plan.handle, C.c_void_p(xd.data_ptr()), C.c_void_p(idd.data_ptr()), sources * cap_routes, K,
                                           cap_routes, slot_routes, len(mine), C.c_void_p(yw.data_ptr()), st)
    assert rc == _lib.OK, _lib.lib().oco_moe_last_error(plan.handle)
    torch.cuda.synchronize(); plan.poll()
    got = yw.cpu().numpy()
    # the same routes handed over compactly, in the same order
    rows = torch.from_numpy(xw[labels[mine] // K].view(np.int16)).cuda()
    cid = torch.from_numpy(local[mine].view(np.int32)).cuda()
    yc = torch.zeros((len(mine), H), dtype=torch.int16, device="cuda")
    rc = _lib.lib().oco_moe_experts(plan.handle, C.c_void_p(rows.data_ptr()), C.c_void_p(cid.data_ptr()), len(mine), C.c_void_p(yc.data_ptr()), st)
    assert rc == _lib.OK, _lib.lib().oco_moe_last_error(plan.handle)
    torch.cuda.synchronize(); plan.poll()
    assert np.array_equal(got[labels[mine]], yc.cpu().numpy()), "window numbering changes the result"
    untouched = np.ones(len(got), bool)
    untouched[labels[mine]] = False
    assert np.all(got[untouched] == sentinel), "rows that belong to other shards, to padding or to slot gaps were written"
    # and against the oracle
    gids = local[mine] + np.uint32(lo)
    xr = xw[labels[mine] // K]
    up = oracle.expert_up_tile(layer.up_w, xr, layer.up_b, 1.0, gids, 1, H, F)
    gate = oracle.expert_up_tile(layer.gate_w, xr, layer.gate_b, 0.0, gids, 1, H, F)
    ref = oracle.expert_down_tile(layer.down_w, oracle.moe_activate(gate, up), layer.down_b, gids, F, H)
    assert rel_l2(got[labels[mine]].view(np.uint16), ref) <= REL_L2
    # refused numberings
    for bad in (dict(per=0), dict(seg=cap_routes, stride=cap_routes - 1), dict(seg=cap_routes, stride=cap_routes + 1)):
        rc = _lib.lib().oco_moe_experts_window(plan.handle, C.c_void_p(xd.data_ptr()), C.c_void_p(idd.data_ptr()), sources * cap_routes,
                                               bad.get("per", K), bad.get("seg", cap_routes), bad.get("stride", slot_routes), 0,
                                               C.c_void_p(yw.data_ptr()), st)
        assert rc == _lib.INVALID_ARGUMENT


@pytest.mark.parametrize("config,tokens,numerics", [("gpt-oss-20b", 2048, 0), ("gpt-oss-20b", 1, 0), ("gpt-oss-20b", 2048, 2), ("gpt-oss-20b", 2048, 3),
                                                    ("gpt-oss-120b", 64, 0), ("nemotron-h", 300, 0), ("qwen3-30b-a3b", 1, 0)],
                         ids=["prefill", "token", "prefill_block_scaled", "prefill_block_scaled_repacked", "few_token", "nemotron", "qwen_token"])
def test_repeated_steps_are_bit_identical(moe, config, tokens, numerics):
    """The same step enqueued back to back on one plan, with no host synchronisation between the steps (so
    that each step's kernels are launched while the step before still runs), gives the same bits every time:
    no result depends on scheduling, on leftovers in the workspace or on how the launches overlap."""
    import torch
    layer = synth.make_config(config, seed=3)
    repacked, numerics = numerics == 3, min(numerics, 2)         # 3: numerics 2 over the repacked weights
    plan = moe.plan_for(layer, numerics=numerics)
    plan.reserve(tokens)
    w = moe._Weights.from_layer(layer)
    plan.bind(w)
    if repacked:
        plan.repack()
    xb, rb = synth.make_tokens(layer.hidden, tokens, 17, "normal")
    x = torch.from_numpy(xb.view(np.int16)).cuda()
    r0 = torch.from_numpy(rb.view(np.int16)).cuda()
    reps = 6 if tokens > 1 else 24
    outs = [r0.clone() for _ in range(reps)]
    for o in outs:
        plan.forward(x, o, tokens)
    torch.cuda.synchronize()
    plan.poll()
    first = outs[0].cpu().numpy()
    assert not np.array_equal(first, rb.view(np.int16)), "the step did nothing"
    for i, o in enumerate(outs[1:], 1):
        assert np.array_equal(first, o.cpu().numpy()), f"step {i} differs from step 0"
    if repacked:
        # at the benchmark's size too, the repacked form and the spans give the same bits
        spans = moe.plan_for(layer, numerics=2)
        spans.reserve(tokens)
        spans.bind(w)
        o = r0.clone()
        spans.forward(x, o, tokens)
        torch.cuda.synchronize()
        spans.poll()
        assert np.array_equal(first, o.cpu().numpy()), "repacked weights change the result at full size"


def test_repacked_planes_hold_the_blocks_bytes(moe):
    """oco_moe_bind_repacked: every block's sixteen code bytes where the MMA reads them from shared memory (tile of 128
    rows and 8 blocks, K-major with the 128-byte swizzle), its scale byte in the tile
    tcgen05.cp reads (tile of 128 rows, K group of 8 blocks, 512-byte half, (row % 32) * 16 + (row / 32) * 4 +
    block % 4), zero where a feature tile runs past the expert's last row; plans that have no use for it refuse."""
    import torch
    from oco_b200 import _lib
    H, F, E, K = 320, 288, 4, 2
    layer = synth.make_layer(synth.ARCH_GPT_OSS, H, F, E, K, synth.FMT_MXFP4, seed=5)
    plan = moe.plan_for(layer, numerics=2)
    plan.reserve(64)
    plan.bind(moe._Weights.from_layer(layer))
    base, nbytes = plan.repack()
    torch.cuda.synchronize()
    off = base - plan._repacked.data_ptr()
    buf = plan._repacked[off: off + nbytes].cpu().numpy()
    at = 0
    for w, n, k in ((layer.gate_w, F, H), (layer.up_w, F, H), (layer.down_w, H, F)):
        nkb, nt = k // 32, (n + 127) // 128
        nkg = (nkb + 7) // 8
        blocks = np.ascontiguousarray(w).reshape(E, n, nkb, 17)
        codes = buf[at: at + E * nt * nkg * 16384].reshape(E, nt, nkg, 16384)
        want_c = np.zeros_like(codes)
        r = np.arange(n)
        for blk in range(nkb):
            off = ((r % 128) // 8) * 1024 + (r % 8) * 128 + (((blk % 8) ^ (r % 8)) * 16)
            for j in range(16):
                want_c[:, r // 128, blk // 8, off + j] = blocks[:, :, blk, 1 + j]
        assert np.array_equal(codes, want_c)
        at += E * nt * nkg * 16384
        sf = buf[at: at + E * nt * nkg * 1024].reshape(E, nt, nkg, 2, 32, 16)
        want = np.zeros_like(sf)
        for blk in range(nkb):
            want[:, r // 128, blk // 8, (blk // 4) % 2, r % 32, ((r % 128) // 32) * 4 + blk % 4] = blocks[:, :, blk, 0]
        assert np.array_equal(sf, want)
        at += E * nt * nkg * 1024
    assert at == nbytes
    other = moe._Plan(synth.ARCH_NEMOTRON, 256, 192, 8, 2, synth.FMT_Q4_0)
    assert _lib.lib().oco_moe_repack_bytes(other.handle) == 0
    with pytest.raises(moe.OcoError):
        other.repack()


@pytest.mark.parametrize("hidden,ffn,experts,misalign", [(96, 96, 32, 0), (640, 384, 32, 0), (256, 160, 32, 7), (2880, 2880, 32, 0),
                                                          (4096, 256, 8, 3)],
                         ids=["k96", "k640", "unaligned", "20b", "k4096"])
def test_gpt_oss_single_token_over_repacked_weights(moe, oracle, monkeypatch, hidden, ffn, experts, misalign):
    """One token with the repacked form of the expert tensors bound (reference numerics): every weight tile
    reaches the block-scaled MMA by TMA, the token and the activations ride as exact e2m1 pieces. Same bars as
    the default single-token kernels (ids and weights bit-exact, outputs rel-L2 <= 1e-3 against the oracle's
    single-token arithmetic), last row tiles past the expert's rows, partly filled K groups, two calls in a row."""
    import torch
    monkeypatch.setenv("OCO_MOE_REPACKED_TOKEN", "1")          # opt-in: the default single-token kernels are faster
    layer = synth.make_layer(synth.ARCH_GPT_OSS, hidden, ffn, experts, min(4, experts), synth.FMT_MXFP4, seed=91)
    plan = moe.plan_for(layer)
    plan.reserve(4)
    w = moe._Weights.from_layer(layer, misalign=misalign)
    plan.bind(w)
    plan.repack()
    for seed in (hidden, hidden + 1):
        xb, rb = synth.make_tokens(hidden, 1, seed, "normal")
        x = torch.from_numpy(xb.view(np.int16)).cuda()
        res = torch.from_numpy(rb.view(np.int16).copy()).cuda()
        plan.forward(x, res, 1)
        torch.cuda.synchronize()
        plan.poll()
        assert plan.launch_count() == 3
        ref = oracle.moe_forward(layer, xb, rb, mode=1)
        routing = moe.Routing()
        routing.plan, routing.rows = plan, 1
        r = routing.read()
        assert np.array_equal(r["ids"], ref.ids) and np.array_equal(r["prob"].view(np.uint32), ref.probs.view(np.uint32))
        assert rel_l2(r["y"], ref.y) <= REL_L2
        assert rel_l2(res.cpu().numpy().view(np.uint16), ref.out) <= REL_L2
