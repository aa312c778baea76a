"""MoE routing / permutation and the MoE FFN — CPU restatements.

moe_align_ref  follows moe_align_tile_size_torch (test/kernels/fused_moe.py:113-173):
               stable sort of the flattened (token, k) replicas by expert, every expert's
               run padded to a multiple of tile_m with the sentinel num_tokens * topk, one
               expert id per tile_m block.
moe_ref        follows torch_moe (samples/MoE.py:292-334): per expert, gate/up
               projection, SiLU(gate) * up, down projection, scaled by the routing
               weight and summed per token.
"""
from __future__ import annotations

import numpy as np
import torch

__all__ = ["moe_align_ref", "moe_ref", "moe_route_ref", "moe_mxfp8_ref"]


def moe_align_ref(topk_ids: torch.Tensor, tile_m: int, num_experts: int):
    ids = topk_ids.detach().cpu().numpy().reshape(-1).astype(np.int64)
    total = ids.size
    order = np.argsort(ids, kind="stable")
    counts = np.bincount(ids, minlength=num_experts)
    blocks = -(-counts // tile_m)
    tokens = np.full(int(blocks.sum()) * tile_m, total, dtype=np.int32)
    experts = np.repeat(np.arange(num_experts, dtype=np.int32), blocks)
    src = 0
    dst = 0
    for e in range(num_experts):
        tokens[dst:dst + counts[e]] = order[src:src + counts[e]]
        src += counts[e]
        dst += blocks[e] * tile_m
    return torch.from_numpy(tokens), torch.from_numpy(experts)


def moe_ref(hidden: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, topk_weights: torch.Tensor,
            topk_ids: torch.Tensor) -> torch.Tensor:
    """fp32 result (num_tokens, hidden); w1 (E, 2I, H) gate rows then up rows, w2 (E, H, I)."""
    x = hidden.detach().cpu().float()
    w1 = w1.detach().cpu().float()
    w2 = w2.detach().cpu().float()
    tw = topk_weights.detach().cpu().float()
    ids = topk_ids.detach().cpu()
    inter = w2.shape[2]
    out = torch.zeros_like(x)
    for e in ids.unique().tolist():
        tok, slot = torch.where(ids == e)
        h = x[tok] @ w1[e].T
        act = torch.nn.functional.silu(h[:, :inter]) * h[:, inter:]
        out.index_add_(0, tok, (act @ w2[e].T) * tw[tok, slot].unsqueeze(-1))
    return out


def moe_route_ref(logits: torch.Tensor, topk: int):
    """top-k experts per token and softmax over the selected logits."""
    vals, ids = torch.topk(logits.detach().cpu().float(), topk, dim=-1)
    return torch.softmax(vals, dim=-1), ids


def moe_mxfp8_ref(hidden, w1_q, w1_scale, w2_q, w2_scale, topk_weights, topk_ids,
                  act_dtype=torch.bfloat16) -> torch.Tensor:
    """The FFN of moe_ref with MXFP8 quantisation points made explicit (no counterpart in the
    reference, which has only the bf16 form): expert weights given as (e4m3, ue8m0 / 32)
    pairs, activations quantised per 32 elements before each projection, the SiLU-and-
    multiply result rounded to `act_dtype` before it is re-quantised."""
    from .quantize import block_quantize_ref, mxfp8_dequantize_ref
    x = mxfp8_dequantize_ref(*block_quantize_ref(hidden))
    w1 = mxfp8_dequantize_ref(w1_q, w1_scale)
    w2 = mxfp8_dequantize_ref(w2_q, w2_scale)
    tw = topk_weights.detach().cpu().float()
    ids = topk_ids.detach().cpu()
    inter = w2.shape[2]
    out = torch.zeros(hidden.shape, dtype=torch.float32)
    for e in ids.unique().tolist():
        tok, slot = torch.where(ids == e)
        h = x[tok] @ w1[e].T
        act = (torch.nn.functional.silu(h[:, :inter]) * h[:, inter:]).to(act_dtype)
        act = mxfp8_dequantize_ref(*block_quantize_ref(act))
        y = ((act @ w2[e].T) * tw[tok, slot].unsqueeze(-1)).to(act_dtype).float()
        out.index_add_(0, tok, y)
    return out
