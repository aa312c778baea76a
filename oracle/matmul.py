"""Ground truth for the GEMM entry points: fp32 matmul of the (de-quantised) operands on
the CPU, as the samples' correctness checks do (samples/MatMul.py:283,
samples/BlockScaledMatMul.py:359-361, test/test_mma_scaled.py:94-96)."""
from __future__ import annotations

import torch

from .quantize import mxfp8_dequantize_ref, nvfp4_dequantize_ref

__all__ = ["matmul_ref", "block_scaled_matmul_ref", "nvfp4_matmul_ref", "rel_frobenius"]


def matmul_ref(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return a.detach().cpu().float() @ b.detach().cpu().float()


def block_scaled_matmul_ref(a_q, a_scale, b_q_nk, b_scale_nk, block_size: int = 32) -> torch.Tensor:
    """a_q (M, K) with scales (M, K/32); b_q_nk (N, K) with scales (N, K/32)."""
    a = mxfp8_dequantize_ref(a_q, a_scale, block_size)
    b = mxfp8_dequantize_ref(b_q_nk, b_scale_nk, block_size)
    return a @ b.T


def nvfp4_matmul_ref(a_packed, a_sf, a_ts, b_packed, b_sf, b_ts) -> torch.Tensor:
    a = nvfp4_dequantize_ref(a_packed, a_sf, a_ts)
    b = nvfp4_dequantize_ref(b_packed, b_sf, b_ts)
    return a @ b.T


def rel_frobenius(x: torch.Tensor, ref: torch.Tensor) -> float:
    x = x.detach().cpu().double()
    ref = ref.detach().cpu().double()
    return float((x - ref).norm() / ref.norm().clamp_min(1e-30))
