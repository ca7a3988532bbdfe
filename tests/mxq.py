"""MXFP4 quantisation of activation rows as the block-scaled tile kernels do it (numpy restatement for the
parity tests of the opt-in numerics mode): per block of 32 values one power-of-two scale, the smallest
2^e with 6 * 2^e >= max |v|, and e2m1 codes rounded to nearest, ties to the even code."""
import numpy as np

GRID = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])


def _round_e2m1(u: np.ndarray) -> np.ndarray:
    """u >= 0, already divided by the scale; returns the e2m1 magnitude (saturating at 6)."""
    u = np.minimum(u, 6.0)
    hi = np.searchsorted(GRID, u, side="left").clip(1, 7)        # GRID[hi - 1] <= u <= GRID[hi]
    lo = hi - 1
    dl, dh = u - GRID[lo], GRID[hi] - u
    pick_hi = (dh < dl) | ((dh == dl) & (hi % 2 == 0))          # ties go to the even code
    return np.where(pick_hi, GRID[hi], GRID[lo])


def quantize_dequantize(v: np.ndarray) -> np.ndarray:
    """v: float32 [..., k] with k a multiple of 32. Returns the values the tensor core multiplies (float64)."""
    v = np.ascontiguousarray(v, np.float32)
    blocks = v.reshape(-1, 32)
    amax = np.abs(blocks).max(axis=1).astype(np.float32)
    bits = amax.view(np.uint32)
    s0 = ((bits >> 23) & 0xFF).astype(np.int64) - 2 + ((bits & 0x7FFFFF) > 0x400000)
    s0 = np.clip(s0, 0, 254)
    scale = np.ldexp(1.0, (s0 - 127).astype(np.int64))[:, None]
    mag = _round_e2m1(np.abs(blocks.astype(np.float64)) / scale)
    return (np.sign(blocks) * mag * scale).reshape(v.shape)
