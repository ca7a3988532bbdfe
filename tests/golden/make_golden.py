"""Generates tests/golden/*.npz: small seeded layers with the CPU oracle's outputs.

The reference stores no golden vectors and cannot run on Linux (Rust + Metal), so these files are
made from the oracle after it has been pinned to the reference's own kernel tests
(tests/test_oracle_pins.py). They freeze that state: a later change of the oracle or of the CUDA
kernels that moves any id, weight or output bit shows up against them.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from oco_b200 import synth  # noqa: E402

CASES = {
    # name: (layer kwargs, tokens, oracle mode)
    "gpt_oss_decode": (dict(arch=synth.ARCH_GPT_OSS, hidden=128, ffn=96, experts=32, top_k=4, fmt=synth.FMT_MXFP4, seed=41), 1, 0),
    "gpt_oss_prefill": (dict(arch=synth.ARCH_GPT_OSS, hidden=128, ffn=96, experts=32, top_k=4, fmt=synth.FMT_MXFP4, seed=41), 37, 0),
    "nemotron_decode": (dict(arch=synth.ARCH_NEMOTRON, hidden=128, ffn=96, experts=128, top_k=6, fmt=synth.FMT_Q4_0, seed=42,
                             shared_ffn=160, normalize=True, scale=2.5), 1, 0),
    "nemotron_prefill": (dict(arch=synth.ARCH_NEMOTRON, hidden=128, ffn=96, experts=128, top_k=6, fmt=synth.FMT_Q4_0, seed=42,
                              shared_ffn=160, normalize=True, scale=2.5), 21, 0),
    "qwen_prefill": (dict(arch=synth.ARCH_QWEN, hidden=256, ffn=256, experts=128, top_k=8, fmt=synth.FMT_Q4_K, seed=43), 19, 2),
}


def make(name):
    kw, tokens, mode = CASES[name]
    layer = synth.make_layer(**kw)
    x, res = synth.make_tokens(layer.hidden, tokens, kw["seed"], "normal")
    r = oracle.moe_forward(layer, x, res, mode=mode)
    return dict(x=x, residual=res, out=r.out, ids=r.ids, probs=r.probs, logits=r.logits, y=r.y,
                act=r.act.astype(np.float32))


if __name__ == "__main__":
    here = os.path.dirname(os.path.abspath(__file__))
    for name in CASES:
        np.savez_compressed(os.path.join(here, name + ".npz"), **make(name))
        print("wrote", name)
