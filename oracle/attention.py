"""Attention ground truth: fp32 softmax(scale * Q K^T + mask) V on the CPU, the
expression the reference's tests compare against (test/test_attention.py:50-57,
test/bench_attention.py:58-69): causal masking with the query positions offset by
`input_pos`, grouped-query heads mapped by integer division."""
from __future__ import annotations

import math

import torch

__all__ = ["fmha_ref"]


def fmha_ref(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, causal: bool = False,
             qk_scale: float | None = None, input_pos: int = 0,
             query_group_size: int = 1) -> torch.Tensor:
    """q (B, Hq, Sq, D), k/v (B, Hkv, Sk, D) -> fp32 (B, Hq, Sq, D), one head at a time."""
    q = q.detach().cpu().float()
    k = k.detach().cpu().float()
    v = v.detach().cpu().float()
    b, hq, sq, d = q.shape
    sk = k.shape[2]
    scale = 1.0 / math.sqrt(d) if qk_scale is None else qk_scale
    out = torch.empty((b, hq, sq, v.shape[3]), dtype=torch.float32)
    mask = None
    if causal:
        qpos = torch.arange(sq).unsqueeze(1) + input_pos
        mask = torch.arange(sk).unsqueeze(0) > qpos
    for bi in range(b):
        for h in range(hq):
            hk = h // query_group_size
            s = (q[bi, h] @ k[bi, hk].T) * scale
            if mask is not None:
                s = s.masked_fill(mask, float("-inf"))
            out[bi, h] = torch.softmax(s, dim=-1) @ v[bi, hk]
    return out
