"""Seeded synthetic MoE layers in unmodified GGUF block layouts.

The benchmark configurations are defined on synthetic tensors (there are no checkpoints in this
environment): shapes, block formats and value distributions follow the benchmark description, one
seed per layer. Everything here is host-side numpy; the same bytes are uploaded to the GPU and
handed to the CPU checker.

Block layouts (reference `src/tensor.rs:24-36`, decoders `shaders/matrix/weights.metal:40-77`):
  MXFP4  32 elements / 17 bytes: E8M0 scale byte, then 16 code bytes (low nibble = element j,
         high nibble = element j + 16).
  Q4_0   32 elements / 18 bytes: f16 d, then 16 code bytes (same nibble order), w = d * (q - 8).
  Q4_K   256 elements / 144 bytes: f16 d, f16 dmin, 12 bytes of 6-bit sub-scales / minima,
         128 code bytes; w = d * sc * q - dmin * m.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import numpy as np

FMT_Q4_0, FMT_Q4_K, FMT_MXFP4 = 2, 12, 39
ARCH_GPT_OSS, ARCH_NEMOTRON, ARCH_QWEN = 0, 1, 2

BLOCK = {FMT_MXFP4: (32, 17), FMT_Q4_0: (32, 18), FMT_Q4_K: (256, 144)}


def row_bytes(fmt: int, k: int) -> int:
    el, by = BLOCK[fmt]
    if k % el:
        raise ValueError(f"row length {k} is not a multiple of the {el}-element block")
    return k // el * by


# ---- bf16 helpers (round to nearest even) -------------------------------------------------------
def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    r[nan] = ((u[nan] >> 16) | 0x40).astype(np.uint16)
    return r.reshape(a.shape)


def bf16_bits_to_f32(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, np.uint16)
    return (a.astype(np.uint32) << 16).view(np.float32).reshape(a.shape)


# ---- block packers ---------------------------------------------------------------------------
def pack_mxfp4(codes: np.ndarray, exponents: np.ndarray) -> np.ndarray:
    """codes: uint8 [rows, k] of 4-bit e2m1 codes; exponents: uint8 [rows, k/32] E8M0 bytes."""
    rows, k = codes.shape
    c = codes.reshape(rows, k // 32, 32).astype(np.uint8)
    out = np.empty((rows, k // 32, 17), np.uint8)
    out[:, :, 0] = exponents
    out[:, :, 1:] = (c[:, :, :16] & 15) | ((c[:, :, 16:] & 15) << 4)
    return out.reshape(rows, -1)


def pack_q4_0(codes: np.ndarray, d_f16_bits: np.ndarray) -> np.ndarray:
    rows, k = codes.shape
    c = codes.reshape(rows, k // 32, 32).astype(np.uint8)
    out = np.empty((rows, k // 32, 18), np.uint8)
    out[:, :, 0:2] = d_f16_bits.astype("<u2").reshape(rows, k // 32, 1).view(np.uint8)
    out[:, :, 2:] = (c[:, :, :16] & 15) | ((c[:, :, 16:] & 15) << 4)
    return out.reshape(rows, -1)


def pack_q4_k(codes: np.ndarray, d_bits: np.ndarray, dmin_bits: np.ndarray, scales: np.ndarray,
              minima: np.ndarray) -> np.ndarray:
    """codes [rows, k] 4-bit; d_bits/dmin_bits uint16 [rows, k/256]; scales/minima uint8 [rows, k/256, 8]
    (6-bit each)."""
    rows, k = codes.shape
    nb = k // 256
    out = np.zeros((rows, nb, 144), np.uint8)
    out[:, :, 0:2] = d_bits.astype("<u2").reshape(rows, nb, 1).view(np.uint8)
    out[:, :, 2:4] = dmin_bits.astype("<u2").reshape(rows, nb, 1).view(np.uint8)
    sc = scales.astype(np.uint8) & 63
    mn = minima.astype(np.uint8) & 63
    packed = np.zeros((rows, nb, 12), np.uint8)
    packed[:, :, 0:4] = sc[:, :, 0:4]
    packed[:, :, 4:8] = mn[:, :, 0:4]
    packed[:, :, 8:12] = (sc[:, :, 4:8] & 15) | ((mn[:, :, 4:8] & 15) << 4)
    packed[:, :, 0:4] |= (sc[:, :, 4:8] >> 4) << 6
    packed[:, :, 4:8] |= (mn[:, :, 4:8] >> 4) << 6
    out[:, :, 4:16] = packed
    c = codes.reshape(rows, nb, 4, 64).astype(np.uint8)
    out[:, :, 16:] = ((c[:, :, :, :32] & 15) | ((c[:, :, :, 32:] & 15) << 4)).reshape(rows, nb, 128)
    return out.reshape(rows, -1)


# ---- random tensors with the benchmark's distributions -----------------------------------------
def random_mxfp4(rng: np.random.Generator, rows: int, k: int, exp_lo: int = -8, exp_hi: int = -3) -> np.ndarray:
    nb = k // 32
    out = rng.integers(0, 256, size=(rows, nb, 17), dtype=np.uint8)
    out[:, :, 0] = (127 + rng.integers(exp_lo, exp_hi + 1, size=(rows, nb))).astype(np.uint8)
    return out.reshape(rows, -1)


def _f16_uniform(rng, shape, lo=1e-3, hi=1e-2) -> np.ndarray:
    return rng.uniform(lo, hi, size=shape).astype(np.float16).view(np.uint16)


def random_q4_0(rng: np.random.Generator, rows: int, k: int) -> np.ndarray:
    nb = k // 32
    out = rng.integers(0, 256, size=(rows, nb, 18), dtype=np.uint8)
    out[:, :, 0:2] = _f16_uniform(rng, (rows, nb, 1)).astype("<u2").view(np.uint8)
    return out.reshape(rows, -1)


def random_q4_k(rng: np.random.Generator, rows: int, k: int) -> np.ndarray:
    nb = k // 256
    out = rng.integers(0, 256, size=(rows, nb, 144), dtype=np.uint8)
    out[:, :, 0:2] = _f16_uniform(rng, (rows, nb, 1)).astype("<u2").view(np.uint8)
    out[:, :, 2:4] = _f16_uniform(rng, (rows, nb, 1)).astype("<u2").view(np.uint8)
    return out.reshape(rows, -1)


_RANDOM = {FMT_MXFP4: random_mxfp4, FMT_Q4_0: random_q4_0, FMT_Q4_K: random_q4_k}


@dataclass
class Layer:
    """One MoE layer on the host. Field names follow the reference's `Experts` / `ReluExperts`
    (`src/weights/gpt_oss.rs:33-38`, `src/weights/nemotron.rs:60-66`)."""
    arch: int
    hidden: int
    ffn: int
    experts: int
    top_k: int
    fmt: int
    shared_ffn: int = 0
    normalize: bool = False
    scale: float = 1.0
    router_w: Optional[np.ndarray] = None      # f32 [E, H]
    router_b: Optional[np.ndarray] = None      # f32 [E]: gpt-oss logit bias / nemotron selection bias
    gate_w: Optional[np.ndarray] = None        # uint8 [E, ffn, row_bytes(H)]
    up_w: Optional[np.ndarray] = None          # uint8 [E, ffn, row_bytes(H)]
    down_w: Optional[np.ndarray] = None        # uint8 [E, H, row_bytes(ffn)]
    gate_b: Optional[np.ndarray] = None        # f32 [E, ffn]
    up_b: Optional[np.ndarray] = None
    down_b: Optional[np.ndarray] = None        # f32 [E, H]
    shared_up_w: Optional[np.ndarray] = None   # uint8 [shared_ffn, row_bytes(H)]
    shared_down_w: Optional[np.ndarray] = None  # uint8 [H, row_bytes(shared_ffn)]
    name: str = ""
    meta: dict = field(default_factory=dict)

    def expert_bytes(self) -> int:
        """Quantised weight + bias bytes of one routed expert."""
        n_up = 2 if self.arch != ARCH_NEMOTRON else 1
        b = n_up * self.ffn * row_bytes(self.fmt, self.hidden) + self.hidden * row_bytes(self.fmt, self.ffn)
        if self.arch == ARCH_GPT_OSS:
            b += 4 * (2 * self.ffn + self.hidden)
        return b

    def shared_bytes(self) -> int:
        if not self.shared_ffn:
            return 0
        return self.shared_ffn * row_bytes(self.fmt, self.hidden) + self.hidden * row_bytes(self.fmt, self.shared_ffn)

    def router_bytes(self) -> int:
        return 4 * self.experts * self.hidden + (4 * self.experts if self.router_b is not None else 0)

    def flops(self, tokens: int) -> float:
        n_up = 2 if self.arch != ARCH_NEMOTRON else 1
        routed = 2.0 * tokens * self.top_k * (n_up * self.ffn * self.hidden + self.hidden * self.ffn)
        shared = 2.0 * tokens * 2 * self.shared_ffn * self.hidden
        router = 2.0 * tokens * self.experts * self.hidden
        return routed + shared + router


def make_layer(arch: int, hidden: int, ffn: int, experts: int, top_k: int, fmt: int, seed: int,
               shared_ffn: int = 0, normalize: bool = False, scale: float = 1.0, name: str = "") -> Layer:
    rng = np.random.default_rng(seed)
    gen = _RANDOM[fmt]
    L = Layer(arch=arch, hidden=hidden, ffn=ffn, experts=experts, top_k=top_k, fmt=fmt,
              shared_ffn=shared_ffn, normalize=normalize, scale=scale, name=name)
    L.router_w = rng.normal(0.0, 0.02, size=(experts, hidden)).astype(np.float32)
    if arch == ARCH_GPT_OSS:
        L.router_b = rng.normal(0.0, 0.01, size=experts).astype(np.float32)
    elif arch == ARCH_NEMOTRON:
        L.router_b = rng.normal(0.0, 0.1, size=experts).astype(np.float32)
    if arch != ARCH_NEMOTRON:
        L.gate_w = gen(rng, experts * ffn, hidden).reshape(experts, ffn, -1)
    L.up_w = gen(rng, experts * ffn, hidden).reshape(experts, ffn, -1)
    L.down_w = gen(rng, experts * hidden, ffn).reshape(experts, hidden, -1)
    if arch == ARCH_GPT_OSS:
        L.gate_b = rng.normal(0.0, 0.01, size=(experts, ffn)).astype(np.float32)
        L.up_b = rng.normal(0.0, 0.01, size=(experts, ffn)).astype(np.float32)
        L.down_b = rng.normal(0.0, 0.01, size=(experts, hidden)).astype(np.float32)
    if shared_ffn:
        L.shared_up_w = gen(rng, shared_ffn, hidden)
        L.shared_down_w = gen(rng, hidden, shared_ffn)
    return L


def make_tokens(hidden: int, tokens: int, seed: int, residual: str = "zero"):
    """x ~ N(0,1) rounded to bf16 at entry (the reference's MoE input is the bf16 post-norm row,
    `src/weights/compute/feed_forward.rs:132,169`); residual zero or N(0,1) bf16."""
    rng = np.random.default_rng(seed ^ 0x5EED)
    x = f32_to_bf16_bits(rng.normal(0.0, 1.0, size=(tokens, hidden)).astype(np.float32))
    if residual == "zero":
        res = np.zeros((tokens, hidden), np.uint16)
    else:
        res = f32_to_bf16_bits(rng.normal(0.0, 1.0, size=(tokens, hidden)).astype(np.float32))
    return x, res


# The benchmark's named configurations. `tokens` lists (single-token, tile) row counts.
CONFIGS = {
    "gpt-oss-20b": dict(arch=ARCH_GPT_OSS, hidden=2880, ffn=2880, experts=32, top_k=4, fmt=FMT_MXFP4),
    "qwen3-30b-a3b": dict(arch=ARCH_QWEN, hidden=2048, ffn=768, experts=128, top_k=8, fmt=FMT_Q4_K),
    # Q4_0, as the reference requires for these banks (`src/weights/nemotron/load.rs:104-112`): rows of
    # 2688 / 1856 / 3712 elements are not multiples of the 256-element Q4_K super-block.
    "nemotron-h": dict(arch=ARCH_NEMOTRON, hidden=2688, ffn=1856, experts=128, top_k=6, fmt=FMT_Q4_0,
                       shared_ffn=3712, normalize=True, scale=2.5),
    "gpt-oss-120b": dict(arch=ARCH_GPT_OSS, hidden=2880, ffn=2880, experts=128, top_k=4, fmt=FMT_MXFP4),
}


def make_config(name: str, seed: int = 0, **overrides) -> Layer:
    cfg = dict(CONFIGS[name])
    cfg.update(overrides)
    return make_layer(seed=seed, name=name, **cfg)
