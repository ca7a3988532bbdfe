"""GGUF staging: synthetic layers written as checkpoints come back through the reader as the same
bytes, at whatever alignment the file gives them, and bad files are refused as the reference refuses
them (src/gguf.rs, src/weights/gpt_oss/load.rs:20-41, src/weights/nemotron/load.rs:92-128)."""
import numpy as np
import pytest

from oco_b200 import gguf, synth


def _same(a, b):
    return (a is None and b is None) or np.array_equal(np.asarray(a), np.asarray(b))


@pytest.mark.parametrize("skew", [0, 2, 6])
def test_gpt_oss_layer_round_trip(tmp_path, oracle, skew):
    layer = synth.make_layer(synth.ARCH_GPT_OSS, 128, 96, 8, 2, synth.FMT_MXFP4, seed=5)
    path = str(tmp_path / "m.gguf")
    # f32 tensors need 4-byte alignment; MXFP4 spans may start anywhere
    tensors = gguf.layer_tensors(layer, 3)
    gguf.write(path, {"general.architecture": "gpt-oss"}, tensors, skew=skew * 2 if skew else 0)
    f = gguf.GgufFile(path)
    assert f.metadata["general.architecture"] == "gpt-oss"
    back = gguf.moe_layer(f, 3, synth.ARCH_GPT_OSS, top_k=2)
    for name in ("router_w", "router_b", "gate_w", "up_w", "down_w", "gate_b", "up_b", "down_b"):
        assert _same(getattr(back, name), getattr(layer, name)), name
    assert (back.hidden, back.ffn, back.experts) == (128, 96, 8)
    x, res = synth.make_tokens(128, 5, 1, "normal")
    a, b = oracle.moe_forward(layer, x, res), oracle.moe_forward(back, x, res)
    assert np.array_equal(a.out, b.out)
    f.close()


def test_nemotron_layer_round_trip(tmp_path, oracle):
    layer = synth.make_layer(synth.ARCH_NEMOTRON, 128, 96, 8, 3, synth.FMT_Q4_0, seed=6, shared_ffn=160, normalize=True, scale=2.5)
    path = str(tmp_path / "n.gguf")
    gguf.write(path, {"general.architecture": "nemotron_h"}, gguf.layer_tensors(layer, 0), skew=4)
    f = gguf.GgufFile(path)
    back = gguf.moe_layer(f, 0, synth.ARCH_NEMOTRON, top_k=3, normalize=True, scale=2.5)
    for name in ("router_w", "router_b", "up_w", "down_w", "shared_up_w", "shared_down_w"):
        assert _same(getattr(back, name), getattr(layer, name)), name
    assert back.shared_ffn == 160
    x, res = synth.make_tokens(128, 4, 2, "normal")
    assert np.array_equal(oracle.moe_forward(layer, x, res).out, oracle.moe_forward(back, x, res).out)
    f.close()


def test_bad_files_are_refused(tmp_path):
    layer = synth.make_layer(synth.ARCH_GPT_OSS, 128, 96, 8, 2, synth.FMT_MXFP4, seed=7)
    tensors = gguf.layer_tensors(layer, 0)
    path = str(tmp_path / "bad.gguf")
    # not a GGUF file
    open(path, "wb").write(b"GGML" + b"\0" * 64)
    with pytest.raises(gguf.CheckpointError):
        gguf.GgufFile(path)
    # a tensor is missing
    gguf.write(path, {}, [t for t in tensors if not t[0].endswith("ffn_up_exps.bias")])
    f = gguf.GgufFile(path)
    with pytest.raises(gguf.CheckpointError, match="missing tensor"):
        gguf.moe_layer(f, 0, synth.ARCH_GPT_OSS, top_k=2)
    f.close()
    # the wrong coefficient type
    wrong = [(n, synth.FMT_Q4_0 if n.endswith("ffn_down_exps.weight") else c, s, d) for n, c, s, d in tensors]
    gguf.write(path, {}, wrong)
    f = gguf.GgufFile(path)
    with pytest.raises(gguf.CheckpointError):
        gguf.moe_layer(f, 0, synth.ARCH_GPT_OSS, top_k=2)
    f.close()
    # f32 data off its scalar alignment
    gguf.write(path, {}, tensors, skew=1)
    f = gguf.GgufFile(path)
    with pytest.raises(gguf.CheckpointError, match="unaligned"):
        gguf.moe_layer(f, 0, synth.ARCH_GPT_OSS, top_k=2)
    f.close()
    # data running past the end of the file
    gguf.write(path, {}, tensors)
    data = open(path, "rb").read()
    open(path, "wb").write(data[:-100])
    f = gguf.GgufFile(path)
    with pytest.raises(gguf.CheckpointError, match="past the file"):
        gguf.moe_layer(f, 0, synth.ARCH_GPT_OSS, top_k=2)
    f.close()


@pytest.mark.gpu
def test_layer_from_gguf_on_the_gpu(tmp_path, oracle):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from oco_b200 import build, moe
    build.build()
    layer = synth.make_layer(synth.ARCH_GPT_OSS, 256, 192, 16, 4, synth.FMT_MXFP4, seed=8)
    path = str(tmp_path / "g.gguf")
    gguf.write(path, {}, gguf.layer_tensors(layer, 1), skew=4)     # MXFP4 spans start 4 bytes off the file alignment
    f = gguf.GgufFile(path)
    staged = gguf.moe_layer(f, 1, synth.ARCH_GPT_OSS, top_k=4)
    for tokens in (1, 50):
        x, res = synth.make_tokens(256, tokens, tokens, "normal")
        ref = oracle.moe_forward(layer, x, res)
        out, routing = moe.run_layer(staged, x, res)
        assert np.array_equal(routing["ids"], ref.ids)
        g = synth.bf16_bits_to_f32(out).astype(np.float64)
        r = synth.bf16_bits_to_f32(ref.out).astype(np.float64)
        assert np.linalg.norm(g - r) <= 1e-3 * np.linalg.norm(r)
    f.close()
