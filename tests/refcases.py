"""Input constructions of the reference's own kernel tests, restated in numpy.

Each builder reproduces the *formulas* a reference test uses to make its operands and its
independent f64 expectation, so the same case can be put to the CPU oracle (to pin it) and to the
CUDA kernels (parity on the reference's edge cases: n = 33 tails, 17 / 257-token batches with
sparse and over-full experts, k = n = 96, down_n = 65).

Reference files: src/weights/dispatch_tests.rs:15-20 (noise), dispatch_tests/mxfp4.rs,
dispatch_tests/nemotron.rs:279-384, dispatch_tests/matrix_precision.rs:145-258.
"""
from __future__ import annotations

import numpy as np

from oco_b200 import synth

HALVES = np.array([0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12], np.float64)


def noise(index) -> np.ndarray:
    """The reference tests' integer hash (dispatch_tests.rs:15-20), vectorised."""
    v = np.asarray(index, dtype=np.uint64) & 0xFFFFFFFF
    v = ((v ^ (v >> 16)) * 0x7FEB352D) & 0xFFFFFFFF
    v = ((v ^ (v >> 15)) * 0x846CA68B) & 0xFFFFFFFF
    return (v ^ (v >> 16)).astype(np.uint32)


def gamma_bound(expected, magnitude, k, stored_bf16):
    """check_roundoff (mxfp4.rs:261-281) / roundoff_bound (matrix_precision.rs:136-142)."""
    ops = 2.0 * k + 8
    u = 2.0 ** -24
    gamma = ops * u / (1 - ops * u)
    s = 2.0 ** -8 if stored_bf16 else 0.0
    return (1 + s) * gamma * magnitude + s * np.abs(expected)


def mxfp4_decode_case(k=2880, n=33):
    """check_decode_reference (mxfp4.rs:46-111): 4 experts, powers in [-5,3], mirrored rows."""
    experts = 4
    e_i, r_i, b_i = np.meshgrid(np.arange(experts), np.arange(n), np.arange(k // 32), indexing="ij")
    power = (noise(e_i * n + r_i + b_i % (k // 64)) % 9).astype(np.int64) - 5           # [E,n,B]
    col = np.arange(k)
    e2, r2, c2 = np.meshgrid(np.arange(experts), np.arange(n), col, indexing="ij")
    mirrored = (r2 % 3 == 0)
    source = np.where(mirrored, c2 % (k // 2), c2)
    codes = (noise((e2 * n + r2) * k + source + 1327) % 16).astype(np.uint8)
    codes = np.where(mirrored & (c2 >= k // 2), codes ^ 8, codes).astype(np.uint8)
    scale = np.repeat(2.0 ** power.astype(np.float64), 32, axis=2)
    coefficients = HALVES[codes] * 0.5 * scale                                           # [E,n,k] f64
    packed = synth.pack_mxfp4(codes.reshape(experts * n, k), (127 + power).astype(np.uint8).reshape(experts * n, -1))
    i = np.arange(4 * k)
    index = i // k * k + i % (k // 2)
    inp = ((noise(index + 8719) % 10007).astype(np.int64) - 5003).astype(np.float32) / np.float32(4093.0)
    bias = ((noise(np.arange(4 * n) + 151) % 997).astype(np.int64) - 498).astype(np.float32) / np.float32(509.0)
    ids = np.array([3, 0, 2, 1], np.uint32)
    return dict(k=k, n=n, packed=packed.reshape(experts, n, -1), coefficients=coefficients,
                input_f32=inp.reshape(4, k), bias=bias.reshape(4, n), ids=ids)


def logits_selecting(ids, experts=32):
    """mxfp4.rs:38-44."""
    logits = np.full(experts, -10.0, np.float32)
    for rank, e in enumerate(ids):
        logits[int(e)] = 4.0 - rank
    return logits


def routed_weights(k, n, salt, experts=32):
    """weights() (mxfp4.rs:283-307): returns packed [E, n, bytes] and f32 values [E, n, k]."""
    e, r, b, c = np.meshgrid(np.arange(experts), np.arange(n), np.arange(k // 32), np.arange(32), indexing="ij")
    power = ((e + r + b + salt) % 5).astype(np.int64) - 3
    codes = ((c * 13 + c // 16 * 5 + e * 3 + r * 5 + b * 7 + salt) % 16).astype(np.uint8)
    values = (HALVES[codes] * 0.5 * 2.0 ** power).astype(np.float32)
    packed = synth.pack_mxfp4(codes.reshape(experts * n, k), (127 + power[..., 0]).astype(np.uint8).reshape(experts * n, -1))
    return packed.reshape(experts, n, -1), values.reshape(experts, n, k)


def routed_experts_case(batch, k=96, n=96, down_n=65):
    """check_experts (mxfp4.rs:309-364)."""
    up_p, up_v = routed_weights(k, n, 0)
    gate_p, gate_v = routed_weights(k, n, 3)
    down_p, down_v = routed_weights(n, down_n, 5)
    i = np.arange(batch * k)
    x = synth.f32_to_bf16_bits((((i // k * 3 + i % k * 5) % 17).astype(np.float32) / 16.0 - 0.5)).reshape(batch, k)
    ub = (((np.arange(32 * n) * 7 % 97).astype(np.float32) - 48.0) / 100.0).reshape(32, n)
    gb = (((np.arange(32 * n) * 3 % 97).astype(np.float32) - 48.0) / 100.0).reshape(32, n)
    db = (((np.arange(32 * down_n) * 5 % 97).astype(np.float32) - 48.0) / 100.0).reshape(32, down_n)
    t = np.arange(batch)
    ids = np.stack([np.full(batch, 31), t % 15, 15 + t % 8, np.full(batch, 30)], axis=1).astype(np.uint32)
    return dict(batch=batch, k=k, n=n, down_n=down_n, up_p=up_p, up_v=up_v, gate_p=gate_p, gate_v=gate_v,
                down_p=down_p, down_v=down_v, x=x, ub=ub, gb=gb, db=db, ids=ids)


def sigmoid_router_case():
    """sigmoid_router_selects_biased_and_weights_unbiased (nemotron.rs:279-330)."""
    n, experts, active, rows = 256, 100, 6, 3
    i = np.arange(rows * n)
    x = synth.f32_to_bf16_bits(((i * 7) % 19).astype(np.float32) / 8.0 - 1.0).reshape(rows, n)
    j = np.arange(experts * n)
    w = (((j * 13 + j // n) % 29).astype(np.float32) / 64.0 - np.float32(0.2)).reshape(experts, n)
    bias = np.where(np.arange(experts) % 10 == 3, 0.9, 0.0).astype(np.float32)
    scale = 2.5
    xf = synth.bf16_bits_to_f32(x).astype(np.float64)
    logits = xf @ w.astype(np.float64).T
    probs = 1.0 / (1.0 + np.exp(-logits))
    sel = probs + bias.astype(np.float64)
    exp_ids, exp_probs = [], []
    for t in range(rows):
        order = sorted(range(experts), key=lambda a: (-sel[t, a], a))[:active]
        total = max(sum(probs[t, e] for e in order), 6.103515625e-5)
        exp_ids.append(order)
        exp_probs.append([probs[t, e] / total * scale for e in order])
    return dict(n=n, experts=experts, active=active, rows=rows, x=x, w=w, bias=bias, scale=scale,
                ids=np.array(exp_ids, np.uint32), probs=np.array(exp_probs, np.float64))


def dense_q4_case(fmt, n=33, k=512):
    """dense_weights (matrix_precision.rs:145-258) for Q4_0 and Q4_K: packed rows + f64 coefficients."""
    block = 32 if fmt == synth.FMT_Q4_0 else 256
    rows = []
    coeff = np.zeros((n, k), np.float64)
    for row in range(n):
        chunks = []
        for start in range(0, k, block):
            seed = row * k + start
            scale = np.float16(np.float32(5 + int(noise(seed + 41)) % 43) * np.float32(0.00031))
            d = float(scale)
            codes = (noise(seed + np.arange(block) + 113) & 0xFF).astype(np.uint8) & 15
            if fmt == synth.FMT_Q4_0:
                coeff[row, start:start + block] = d * codes.astype(np.float64) - 8.0 * d
                chunks.append(synth.pack_q4_0(codes.reshape(1, block), np.array([[scale.view(np.uint16)]])).ravel())
            else:
                minimum = np.float16(d * 0.9375)
                scales = (1 + noise(seed + np.arange(8) + 223) % 63).astype(np.uint8)
                minima = (noise(seed + np.arange(8) + 317) % 64).astype(np.uint8)
                sub = np.arange(block) // 32
                coeff[row, start:start + block] = d * scales[sub].astype(np.float64) * codes - float(minimum) * minima[sub]
                chunks.append(synth.pack_q4_k(codes.reshape(1, block), np.array([[scale.view(np.uint16)]]),
                                              np.array([[minimum.view(np.uint16)]]), scales.reshape(1, 1, 8),
                                              minima.reshape(1, 1, 8)).ravel())
        rows.append(np.concatenate(chunks))
    return np.stack(rows), coeff
