"""Expert-parallel MoE FFN: experts sharded over the ranks of one node, tokens sharded
over the same ranks, two exchange steps over NVLink (dispatch and combine).

The reference has no multi-GPU MoE (its only distributed code is the AllGather sample);
this composes the single-GPU pipeline of moe.py with an all-to-all:

  route     replicas (token, slot) sorted by global expert id on the device
  dispatch  rows, local expert ids and routing weights to the rank that owns the expert
            (torch.distributed.all_to_all_single over NCCL; split sizes from a bincount)
  experts   the local grouped-GEMM pipeline on the received rows (top-1 problem, routing
            weight applied in the down projection's epilogue)
  combine   results back to the source rank, un-permuted, summed over the top-k slots

`exchange()` and the split arithmetic are backend-agnostic torch, so the routing logic is
testable with gloo on CPU; only `local_experts()` needs the CUDA library.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def expert_owner_counts(counts_per_expert: torch.Tensor, world: int) -> list[int]:
    """Rows this rank sends to each rank, from its per-expert replica counts (experts are
    dealt to ranks in contiguous runs of E / world)."""
    e = counts_per_expert.numel()
    if e % world:
        raise ValueError(f"{e} experts do not split evenly over {world} ranks")
    return counts_per_expert.reshape(world, e // world).sum(dim=1).tolist()


def exchange(tensors, send_counts: list[int], group=None):
    """all_to_all_single of several row-aligned tensors with the same split sizes.
    Returns (received tensors, recv_counts)."""
    world = dist.get_world_size(group)
    if world == 1:   # everything stays here: no copy, no collective, no host round trip
        return list(tensors), list(send_counts)
    dev = tensors[0].device
    sc = torch.tensor(send_counts, dtype=torch.int64, device=dev)
    rc = torch.empty(world, dtype=torch.int64, device=dev)
    dist.all_to_all_single(rc, sc, group=group)
    recv_counts = rc.tolist()
    out = []
    for t in tensors:
        r = torch.empty((sum(recv_counts),) + tuple(t.shape[1:]), dtype=t.dtype, device=dev)
        dist.all_to_all_single(r, t.contiguous(), output_split_sizes=recv_counts,
                               input_split_sizes=send_counts, group=group)
        out.append(r)
    return out, recv_counts


def route(topk_ids: torch.Tensor, num_experts: int):
    """Replica order for dispatch: replica ids (token * topk + slot) sorted by expert id,
    stable, plus replicas per expert.  Plain torch (used by the CPU tests); the CUDA path
    gets the same order from the device-side alignment with tile 1."""
    flat = topk_ids.reshape(-1)
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=num_experts)
    return order, counts


class ExpertParallelMoE:
    """MoE FFN with this rank's slice of the experts.

    w1_local (E / world, 2I, H) and w2_local (E / world, H, I) hold experts
    [rank * E / world, (rank + 1) * E / world).  `forward` takes this rank's tokens with
    GLOBAL expert ids and returns their outputs."""

    def __init__(self, w1_local: torch.Tensor, w2_local: torch.Tensor, num_experts: int, group=None):
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if num_experts % self.world or w1_local.shape[0] != num_experts // self.world:
            raise ValueError("expert weights do not match num_experts / world")
        self.num_experts = num_experts
        self.local_experts_n = num_experts // self.world
        self.w1, self.w2 = w1_local, w2_local

    def local_experts(self, rows: torch.Tensor, local_ids: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
        """y[i] = weights[i] * FFN_{local_ids[i]}(rows[i]) through the grouped-GEMM pipeline."""
        from . import moe
        n = rows.shape[0]
        hidden = rows.shape[1]
        inter = self.w2.shape[2]
        # every received row is routed to exactly one local expert, so the scatter of the
        # down projection writes every row of y
        y = torch.empty((n, hidden), dtype=rows.dtype, device=rows.device)
        if n == 0:
            return y
        tile = moe._moe_tile()
        sorted_ids, expert_ids, num_blocks = moe.moe_align_device(local_ids.reshape(n, 1), tile,
                                                                  self.local_experts_n)
        cap = sorted_ids.numel()
        a_sorted = moe._gather_rows(rows, sorted_ids, 1, cap, num_blocks, tile)
        act = torch.empty((cap, inter), dtype=rows.dtype, device=rows.device)
        if inter % 128 == 0:
            moe._grouped_gemm(a_sorted, moe._check_weight(self.w1), act, expert_ids,
                              num_blocks=num_blocks, swiglu=True, tile=tile)
        else:
            gate_up = torch.empty((cap, 2 * inter), dtype=rows.dtype, device=rows.device)
            moe._grouped_gemm(a_sorted, moe._check_weight(self.w1), gate_up, expert_ids,
                              num_blocks=num_blocks, tile=tile)
            moe.invoke_silu_and_mul_kernel(gate_up, act)
        moe._grouped_gemm(act, moe._check_weight(self.w2), y, expert_ids, num_blocks=num_blocks,
                          row_map=sorted_ids, row_scale=weights.float().contiguous(), c_rows=n, tile=tile)
        return y

    def forward(self, hidden_states: torch.Tensor, topk_weights: torch.Tensor,
                topk_ids: torch.Tensor, expert_fn=None) -> torch.Tensor:
        tokens, hidden = hidden_states.shape
        topk = topk_ids.shape[1]
        cuda = hidden_states.is_cuda
        flat_ids = topk_ids.reshape(-1)
        if cuda:
            from . import moe
            order32, _, _ = moe.moe_align_device(topk_ids, 1, self.num_experts, want_expert_ids=False)
            order = order32.long()
            counts = torch.bincount(flat_ids, minlength=self.num_experts)
            x = hidden_states if hidden_states.stride(1) == 1 else hidden_states.contiguous()
            rows = moe._gather_rows(x, order32, topk, tokens * topk, None)
        else:
            order, counts = route(topk_ids, self.num_experts)
            rows = hidden_states[order // topk]
        send_counts = expert_owner_counts(counts, self.world)
        # local expert id and routing weight travel together as one (R, 2) fp32 tensor
        meta = torch.stack([(flat_ids[order] % self.local_experts_n).float(),
                            topk_weights.reshape(-1)[order].float()], dim=1)
        (rows_in, meta_in), recv_counts = exchange([rows, meta], send_counts, self.group)
        ids_in = meta_in[:, 0].to(torch.int32)
        wts_in = meta_in[:, 1].contiguous()
        fn = expert_fn if expert_fn is not None else self.local_experts
        y_in = fn(rows_in, ids_in, wts_in)
        (y_back,), _ = exchange_back(y_in, recv_counts, send_counts, self.group)
        # y_back is in dispatch order: replica order[i] sits in row i
        inverse = torch.empty_like(order)
        inverse[order] = torch.arange(order.numel(), device=order.device)
        if cuda and hidden % 8 == 0:
            from . import moe
            return moe._topk_sum(y_back, tokens, topk, hidden, index=inverse.to(torch.int32))
        return y_back[inverse].reshape(tokens, topk, hidden).float().sum(dim=1).to(hidden_states.dtype)


def exchange_back(t: torch.Tensor, send_counts: list[int], recv_counts: list[int], group=None):
    """The reverse all-to-all of `exchange` (split sizes already known on both sides)."""
    if dist.get_world_size(group) == 1:
        return (t,), recv_counts
    r = torch.empty((sum(recv_counts),) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
    dist.all_to_all_single(r, t.contiguous(), output_split_sizes=recv_counts,
                           input_split_sizes=send_counts, group=group)
    return (r,), recv_counts
