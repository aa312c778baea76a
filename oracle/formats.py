"""Number formats of the block-scaled path, decoded and encoded on the CPU.

Follows src/cuda/tile/_bytecode/float.py:30-131 (e8m0 / e4m3 / e2m1 semantics) and the
nibble table and packing order of test/test_mma_scaled.py:149-160.
"""
from __future__ import annotations

import numpy as np
import torch

__all__ = ["E2M1_VALUES", "e2m1_decode_packed", "e2m1_encode_rne", "e2m1_pack", "e8m0_decode",
           "e8m0_encode_pow2", "e4m3_decode", "e4m3_encode_rne"]

# value of each e2m1 code 0..15: sign bit 3, exponent bits 2..1, mantissa bit 0
E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0,
                        -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0], dtype=np.float32)


def e2m1_decode_packed(packed: np.ndarray) -> np.ndarray:
    """(…, K/2) uint8 -> (…, K) float32; the low nibble is the even element."""
    packed = np.asarray(packed, dtype=np.uint8)
    lo = E2M1_VALUES[packed & 0xF]
    hi = E2M1_VALUES[packed >> 4]
    out = np.empty(packed.shape[:-1] + (packed.shape[-1] * 2,), dtype=np.float32)
    out[..., 0::2] = lo
    out[..., 1::2] = hi
    return out


def e2m1_encode_rne(x: np.ndarray) -> np.ndarray:
    """float32 -> e2m1 code (uint8 in 0..15): round to nearest, ties to the even code,
    saturating at +-6; NaN maps to +6 like the hardware's satfinite conversion."""
    x = np.asarray(x, dtype=np.float32)
    mag = np.abs(x).astype(np.float64)
    grid = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
    # midpoints between consecutive codes; a tie goes to the code with even index
    mids = (grid[:-1] + grid[1:]) / 2
    code = np.zeros(mag.shape, dtype=np.uint8)
    for i, mid in enumerate(mids):
        if (i + 1) % 2 == 0:      # upper neighbour is even: ties go up
            code = np.where(mag >= mid, i + 1, code)
        else:                     # lower neighbour is even: ties stay
            code = np.where(mag > mid, i + 1, code)
    code = np.where(np.isnan(x), 7, code).astype(np.uint8)
    sign = (np.signbit(x) & ~np.isnan(x)).astype(np.uint8) << 3
    return (code | sign).astype(np.uint8)


def e2m1_pack(codes: np.ndarray) -> np.ndarray:
    codes = np.asarray(codes, dtype=np.uint8)
    return (codes[..., 0::2] | (codes[..., 1::2] << 4)).astype(np.uint8)


def e8m0_decode(b: np.ndarray) -> np.ndarray:
    """ue8m0 byte -> float32: 2^(b - 127); 0xFF is NaN; there is no zero."""
    b = np.asarray(b, dtype=np.uint8)
    out = np.ldexp(np.float64(1.0), b.astype(np.int32) - 127).astype(np.float32)
    return np.where(b == 0xFF, np.float32(np.nan), out)


def e8m0_encode_pow2(exponent: np.ndarray) -> np.ndarray:
    return (np.asarray(exponent, dtype=np.int32) + 127).astype(np.uint8)


def e4m3_decode(b: np.ndarray) -> np.ndarray:
    return torch.from_numpy(np.ascontiguousarray(b, dtype=np.uint8)).view(torch.float8_e4m3fn).float().numpy()


def e4m3_encode_rne(x: np.ndarray) -> np.ndarray:
    """float32 -> e4m3fn byte, round to nearest even.  Inputs stay within +-448 on
    this path, where torch's cast and the saturating hardware conversion agree."""
    t = torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32))
    return t.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
