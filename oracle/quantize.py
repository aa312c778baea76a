"""Quantisers and scale relayout — CPU restatements.

block_quantize_ref   follows test/kernels/kernel_utils.py:38-80 with the input
                     up-cast to fp32 first (the samples feed fp32,
                     samples/BlockScaledMatMul.py:333-337)
swizzle_32_4_4_ref   follows test/kernels/kernel_utils.py:83-98 (and its inverse :101-112)
nvfp4_quantize_ref   no counterpart in the reference ("parity unpinned"); implements the
                     rule stated at b200k_nvfp4_quantize in include/b200k.h
"""
from __future__ import annotations

import numpy as np
import torch

from . import formats

__all__ = ["block_quantize_ref", "swizzle_32_4_4_ref", "unswizzle_32_4_4_ref",
           "mxfp8_dequantize_ref", "nvfp4_quantize_ref", "nvfp4_dequantize_ref"]


def block_quantize_ref(x: torch.Tensor, block_size: int = 32,
                       dtype: torch.dtype = torch.float8_e4m3fn):
    """Returns (x_q in `dtype`, scale as float8_e8m0fnu of shape (..., K/block))."""
    x = x.detach().cpu().float()
    if x.shape[-1] < block_size:
        raise ValueError("block larger than the innermost dimension")
    tail = x.shape[-1] % block_size
    if tail:
        x = torch.nn.functional.pad(x, (0, block_size - tail))
    blocks = x.unflatten(-1, (-1, block_size))
    amax = blocks.abs().amax(dim=-1, keepdim=True)
    s = (amax / torch.finfo(torch.float8_e4m3fn).max).clamp_min(1e-12)
    s = torch.exp2(torch.log2(s).ceil())
    q = (blocks / s).to(dtype).flatten(-2)
    return q, s.squeeze(-1).to(torch.float8_e8m0fnu)


def swizzle_32_4_4_ref(scale: torch.Tensor) -> torch.Tensor:
    """(M, Ks) -> (M/128, Ks/4, 32, 16): byte (r, c) of atom (i, j) is the scale of row
    128 i + 32 (c // 4) + r and block 4 j + c % 4."""
    m, ks = scale.shape
    if m % 128 or ks % 4:
        raise ValueError("rows must be a multiple of 128 and blocks a multiple of 4")
    u = scale.detach().cpu().view(torch.uint8).numpy()
    out = np.empty((m // 128, ks // 4, 32, 16), dtype=np.uint8)
    for c in range(16):
        rows = 32 * (c // 4) + np.arange(32)
        # one byte column of every atom: (tiles, 32 rows, katoms) -> (tiles, katoms, 32)
        sel = u.reshape(m // 128, 128, ks // 4, 4)[:, :, :, c % 4][:, rows, :]
        out[:, :, :, c] = sel.transpose(0, 2, 1)
    return torch.from_numpy(out).view(scale.dtype)


def unswizzle_32_4_4_ref(sw: torch.Tensor) -> torch.Tensor:
    tiles, katoms = sw.shape[:2]
    u = sw.detach().cpu().view(torch.uint8).numpy()
    out = np.empty((tiles * 128, katoms * 4), dtype=np.uint8)
    v = out.reshape(tiles, 128, katoms, 4)
    for c in range(16):
        rows = 32 * (c // 4) + np.arange(32)
        v[:, :, :, c % 4][:, rows, :] = u[:, :, :, c].transpose(0, 2, 1)
    return torch.from_numpy(out).view(sw.dtype)


def mxfp8_dequantize_ref(q: torch.Tensor, scale: torch.Tensor, block_size: int = 32) -> torch.Tensor:
    """fp32 value of an MXFP8 tensor with logical (…, K/block) ue8m0 scales
    (samples/BlockScaledMatMul.py:359-361)."""
    s = torch.from_numpy(formats.e8m0_decode(scale.detach().cpu().view(torch.uint8).numpy()))
    return q.detach().cpu().float() * s.repeat_interleave(block_size, dim=-1)[..., : q.shape[-1]]


def nvfp4_quantize_ref(x: torch.Tensor, tensor_scale=None):
    """Returns (packed e2m1 uint8 (rows, K/2), ue4m3 scale bytes (rows, K/16) uint8,
    tensor scale float32 scalar).  `tensor_scale` given: used instead of amax / (448 * 6);
    block scales and codes then saturate (448, +-6)."""
    x = x.detach().cpu().float().numpy()
    rows, k = x.shape
    pad = (-k) % 16
    xp = np.pad(x, ((0, 0), (0, pad))) if pad else x
    f32 = np.float32
    amax_t = f32(np.abs(x).max()) if x.size else f32(0)
    s_t = f32(amax_t / f32(2688.0)) if tensor_scale is None else f32(tensor_scale)
    six_st = f32(f32(6.0) * s_t)
    blocks = xp.reshape(rows, -1, 16)
    amax_b = np.abs(blocks).max(axis=-1).astype(f32)
    with np.errstate(divide="ignore", invalid="ignore"):
        r = np.where((amax_b > 0) & (six_st > 0), (amax_b / six_st).astype(f32), f32(0))
    sf = formats.e4m3_encode_rne(np.minimum(r, f32(448.0)))
    denom = (formats.e4m3_decode(sf).astype(f32) * s_t).astype(f32)
    # x / denom evaluated as x * (1 / denom), each step rounded to fp32 (one reciprocal per
    # block); a subnormal denom, whose reciprocal overflows, keeps the division
    normal = denom >= np.finfo(f32).tiny
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        inv = np.where(normal, (f32(1.0) / denom).astype(f32), f32(0))
        y = np.where(normal[..., None], (blocks * inv[..., None]).astype(f32),
                     np.where(denom[..., None] > 0, (blocks / denom[..., None]).astype(f32), f32(0)))
    codes = formats.e2m1_encode_rne(y).reshape(rows, -1)[:, :k]
    return formats.e2m1_pack(codes), sf, s_t


def nvfp4_dequantize_ref(packed, sf, s_t) -> torch.Tensor:
    vals = formats.e2m1_decode_packed(np.asarray(packed))
    s = np.repeat(formats.e4m3_decode(np.asarray(sf)), 16, axis=-1)[..., : vals.shape[-1]]
    return torch.from_numpy(vals * s * np.float32(s_t))
