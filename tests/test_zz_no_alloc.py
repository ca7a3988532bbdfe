"""The no-allocation routing call, checked against the regular operator.

`oco_moe_route_token_static` exists for hosts that cannot allocate device memory once they are
running: an engine with a fixed, pre-planned memory budget (the way the reference's session arena
works), a plugin next to a framework allocator that already holds the GPU's free memory, or a
latency-critical loop that must not stall the device in cudaMalloc. It keeps its scratch in a fixed
device array inside the library. This test calls it twice in a row through the C ABI (the second
call finds the first call's leftovers in that array) and requires the same expert ids and weights,
bit for bit, as `oco_moe_forward` produces for one token. It is collected last so that a failure
here cannot hide any other test.
"""
import ctypes as C

import numpy as np
import pytest

from oco_b200 import synth

pytestmark = pytest.mark.gpu

LAYERS = {
    "gpt_oss": dict(arch=synth.ARCH_GPT_OSS, hidden=2880, ffn=64, experts=32, top_k=4, fmt=synth.FMT_MXFP4, seed=51),
    "nemotron": dict(arch=synth.ARCH_NEMOTRON, hidden=2688, ffn=64, experts=128, top_k=6, fmt=synth.FMT_Q4_0, seed=52,
                     normalize=True, scale=2.5),
    "qwen": dict(arch=synth.ARCH_QWEN, hidden=2048, ffn=256, experts=128, top_k=8, fmt=synth.FMT_Q4_K, seed=53),
}


@pytest.mark.parametrize("name", sorted(LAYERS))
def test_static_route_matches_forward_twice(name, oracle):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from oco_b200 import _lib, build, moe
    build.build()
    lib = _lib.lib()
    layer = synth.make_layer(**LAYERS[name])
    w = moe._Weights.from_layer(layer)
    ids = torch.zeros(8, dtype=torch.int32, device="cuda")
    probs = torch.zeros(8, dtype=torch.float32, device="cuda")
    err = C.create_string_buffer(256)
    for call in range(2):     # two calls in a row share the library's static scratch
        x, res = synth.make_tokens(layer.hidden, 1, 900 + call, "normal")
        _, routing = moe.run_layer(layer, x, res)          # the existing entry point (oco_moe_forward)
        xd = torch.from_numpy(x.view(np.int16)).cuda()
        ids.fill_(-1); probs.fill_(-1.0)
        rc = lib.oco_moe_route_token_static(
            layer.arch, C.c_void_p(xd.data_ptr()), C.c_void_p(w.router_w.data_ptr()),
            C.c_void_p(w.router_b.data_ptr()) if w.router_b is not None else None, layer.hidden, layer.experts,
            layer.top_k, int(layer.normalize), float(layer.scale), C.c_void_p(ids.data_ptr()),
            C.c_void_p(probs.data_ptr()), C.c_void_p(torch.cuda.current_stream().cuda_stream), err, 256)
        assert rc == _lib.OK, err.value
        torch.cuda.synchronize()
        got_ids = ids.cpu().numpy().view(np.uint32)[:layer.top_k]
        got_probs = probs.cpu().numpy()[:layer.top_k]
        # ids and weights are held to bit-exactness everywhere in this suite
        assert np.array_equal(got_ids, routing["ids"][0]), f"call {call}"
        assert np.array_equal(got_probs.view(np.uint32), routing["prob"][0].view(np.uint32)), f"call {call}"
        # and against the CPU checker directly, so that both CUDA paths cannot be wrong together
        if layer.arch == synth.ARCH_GPT_OSS:
            _, ref_ids, ref_probs = oracle.router_gptoss(x, layer.router_w, layer.router_b, layer.top_k)
        elif layer.arch == synth.ARCH_NEMOTRON:
            _, ref_ids, ref_probs = oracle.router_sigmoid(x, layer.router_w, layer.router_b, layer.top_k, layer.normalize, layer.scale)
        else:
            _, ref_ids, ref_probs = oracle.router_softmax_topk(x, layer.router_w, layer.top_k)
        assert np.array_equal(got_ids, ref_ids[0].astype(np.uint32)), f"call {call}: ids differ from the checker"
        assert np.array_equal(got_probs.view(np.uint32), ref_probs[0].view(np.uint32)), f"call {call}: weights differ from the checker"
    # sizes beyond what the static array holds are refused with a message, nothing is launched
    rc = lib.oco_moe_route_token_static(layer.arch, C.c_void_p(xd.data_ptr()), C.c_void_p(w.router_w.data_ptr()),
                                        C.c_void_p(w.router_b.data_ptr()) if w.router_b is not None else None, layer.hidden, 129, layer.top_k, 0, 1.0,
                                        C.c_void_p(ids.data_ptr()), C.c_void_p(probs.data_ptr()), None, err, 256)
    assert rc == _lib.UNSUPPORTED_SHAPE and b"128" in err.value
