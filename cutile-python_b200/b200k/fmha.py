"""Fused multi-head attention forward with the signature of the reference's sample.

cutile_fmha        samples/AttentionFMHA.py:138-210
cutile_fmha_into   test/bench_attention.py:96-113 (bench form: output passed in)
"""
from __future__ import annotations

import ctypes
import os
import math

import torch

from . import _lib


def _prep(t: torch.Tensor, d_pad: int) -> torch.Tensor:
    """Head dim padded with zeros to the kernel's width, unit stride on it, 16-byte strides."""
    d = t.shape[3]
    ok = (t.stride(3) == 1 and d == d_pad and t.data_ptr() % 16 == 0
          and all((t.stride(i) * t.element_size()) % 16 == 0 for i in range(3)))
    if ok:
        return t
    buf = torch.zeros(*t.shape[:3], d_pad, dtype=t.dtype, device=t.device)
    buf[..., :d].copy_(t)
    return buf


def cutile_fmha(Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor,
                qk_scale: float | None = None,
                input_pos: int = 0,
                tile_m: int = 128,
                tile_n: int = 128,
                query_group_size: int = 1,
                causal: bool = False,
                kernel=None,
                Out: torch.Tensor | None = None) -> torch.Tensor:
    """Out = softmax(qk_scale * Q K^T + causal mask) V, (Batch, Heads, SeqLen_Q, D_v).

    Q (Batch, Heads, SeqLen_Q, D_k), K (Batch, KV_Heads, SeqLen_KV, D_k),
    V (Batch, KV_Heads, SeqLen_KV, D_v); f16 or bf16.  ``tile_m``, ``tile_n`` and
    ``kernel`` are accepted for signature compatibility: the kernel's tiles are fixed
    at 128 x 128.  Head dims up to 128 are supported (smaller ones are zero-padded to
    64 or 128, which changes neither the scores nor the output columns kept).
    """
    if Q.ndim != 4 or K.ndim != 4 or V.ndim != 4:
        raise ValueError("Input tensors Q, K, V must be 4D (Batch, Heads, SeqLen, Dim).")
    if Q.shape[0] != K.shape[0] or Q.shape[0] != V.shape[0]:
        raise ValueError("Batch dimensions must match for Q, K, V.")
    if Q.shape[1] % query_group_size != 0:
        raise ValueError("Number of query heads must be divisible by query_group_size.")
    if K.shape[1] * query_group_size != Q.shape[1]:
        raise ValueError("K_Heads * query_group_size must equal Q_Heads.")
    if Q.shape[3] != K.shape[3]:
        raise ValueError("D_k (last dim of Q and K) must match.")
    if K.shape[2] != V.shape[2]:
        raise ValueError("SeqLen_KV (dim 2 of K and V) must match.")
    if Q.device != K.device or Q.device != V.device or not Q.is_cuda:
        raise ValueError("All input tensors must be on the same CUDA device.")
    if Q.dtype != K.dtype or Q.dtype != V.dtype:
        raise ValueError("All input tensors must have the same data type.")
    if Q.dtype not in (torch.float16, torch.bfloat16):
        raise TypeError("cutile_fmha supports float16 and bfloat16")

    batch, heads, seq_q, d_k = Q.shape
    _, kv_heads, seq_kv, d_v = V.shape
    if max(d_k, d_v) > 128:
        raise ValueError("head dimensions above 128 are not supported")
    if qk_scale is None:
        qk_scale = 1.0 / math.sqrt(d_k)
    d_pad = 64 if max(d_k, d_v) <= 64 else 128

    if Out is None:
        Out = torch.empty((batch, heads, seq_q, d_v), dtype=Q.dtype, device=Q.device)
    if batch == 0 or heads == 0 or seq_q == 0:
        return Out
    if seq_kv == 0:
        raise ValueError("SeqLen_KV must be positive")

    q, k, v = _prep(Q, d_pad), _prep(K, d_pad), _prep(V, d_pad)
    direct = (d_v == d_pad and Out.stride(3) == 1)
    o = Out if direct else torch.empty((batch, heads, seq_q, d_pad), dtype=Q.dtype, device=Q.device)

    a = _lib.FmhaArgs()
    a.q, a.k, a.v, a.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr()
    a.batch, a.heads_q, a.heads_kv, a.seq_q, a.seq_kv = batch, heads, kv_heads, seq_q, seq_kv
    a.q_stride_b, a.q_stride_h, a.q_stride_s = q.stride(0), q.stride(1), q.stride(2)
    a.k_stride_b, a.k_stride_h, a.k_stride_s = k.stride(0), k.stride(1), k.stride(2)
    a.v_stride_b, a.v_stride_h, a.v_stride_s = v.stride(0), v.stride(1), v.stride(2)
    a.o_stride_b, a.o_stride_h, a.o_stride_s = o.stride(0), o.stride(1), o.stride(2)
    a.input_pos = int(input_pos)
    a.head_dim = d_pad
    a.dtype = _lib.dtype_enum(Q.dtype)
    a.query_group_size = query_group_size
    a.causal = 1 if causal else 0
    a.qk_scale = float(qk_scale)
    with torch.cuda.device(Q.device):
        # a few query rows per KV head (decode): the split-KV kernels need scratch for the
        # partial softmax states (B200K_FMHA_NO_DECODE=1 keeps the tensor-core kernels)
        workspace = None
        if seq_q * query_group_size <= 8 and os.environ.get("B200K_FMHA_NO_DECODE") != "1":
            ws_bytes = _lib.lib().b200k_fmha_workspace_bytes(ctypes.byref(a))
            if ws_bytes > 0:
                workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=Q.device)
                a.workspace, a.workspace_bytes = workspace.data_ptr(), ws_bytes
        _lib.check(_lib.lib().b200k_fmha_fwd(ctypes.byref(a), _lib.stream_ptr(Q.device)))
    if not direct:
        Out.copy_(o[..., :d_v])
    return Out


def cutile_fmha_into(q, k, v, o, is_causal: bool, enable_gqa: bool = False):
    """Bench form: writes into ``o``; query positions are aligned to the end of the keys
    when the lengths differ (decode / chunked prefill), as the reference bench does."""
    q_len, k_len = q.shape[2], k.shape[2]
    group = q.shape[1] // k.shape[1]
    return cutile_fmha(q, k, v, qk_scale=1.0 / math.sqrt(q.shape[3]),
                       input_pos=0 if q_len == k_len else k_len - 1,
                       query_group_size=group, causal=is_causal, Out=o)
