"""Expert-parallel MoE FFN: experts sharded over the ranks of one node, tokens sharded over
the same ranks, two exchange steps over NVLink (dispatch and combine).

The reference has no multi-GPU MoE (its only distributed code is the AllGather sample); the
single-GPU pipeline this must equal is cutile_moe / cutile_moe_mxfp8 (samples/MoE.py:197-288).
Per layer, on every rank, with nothing read back by the host:

  count     histogram of the rank's routing ids per global expert, stored into every rank's
            table (world x experts ints)
  barrier
  plan      from the table: where this rank's rows for each expert start in the owner's
            receive buffer, and the tile list of the grouped GEMM over the rows this rank
            will receive (csrc/moe_ep_plan.h)
  dispatch  every token replica's row - quantised once per token to e4m3 + a row of ue8m0
            scale bytes when the experts are MXFP8 - is stored by this rank's kernel into the
            owner's receive buffer at its final, tile-aligned position, with the replica's id
            and routing weight beside it (plain peer stores; no library collective, no
            multicast)
  barrier
  experts   the grouped-GEMM pipeline of moe.py on the received rows; the down projection's
            epilogue stores each result row straight into the y buffer of the rank the row
            came from (b200k_gemm c_peers): the combine transfer is part of the GEMM
  barrier
  combine   top-k sum of the rank's own y rows

The barriers are kernels of this library (b200k_peer_barrier: flags in peer memory, bounded
waits).  Buffers are symmetric-memory allocations sized for the worst case (every replica of
every rank routed to one rank), made on the first call for a problem size.

`emulate_ranks` runs the same phases for several ranks inside one process on one GPU (the
ranks' buffers are plain local tensors, the phases run in lock step, no barrier kernel is
launched): the multi-rank data path can be checked where only one GPU is at hand.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from . import _lib

TILE = 256   # row tile of the CTA-pair grouped GEMM


def _ptr_array(tensors):
    arr = (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])
    return arr, ctypes.cast(arr, ctypes.POINTER(ctypes.c_void_p))


class ExpertParallelMoE:
    """MoE FFN with this rank's slice of the experts.

    w1_local (E / world, 2I, H) and w2_local (E / world, H, I) hold experts
    [rank * E / world, (rank + 1) * E / world) as f16/bf16 tensors.  With ``mxfp8`` they are
    quantised once (e4m3 + ue8m0 per 32 along K) and activations travel and multiply as MXFP8.
    `forward` takes this rank's tokens with GLOBAL expert ids and returns their outputs; every
    rank must call it with the same number of tokens and the same top-k."""

    def __init__(self, w1_local: torch.Tensor, w2_local: torch.Tensor, num_experts: int, group=None, *,
                 mxfp8: bool = False, world: int | None = None, rank: int | None = None):
        if world is not None:                       # emulated ranks: see emulate_ranks
            if rank is None or not 0 <= rank < world:
                raise ValueError("an explicit world needs rank in [0, world)")
            self.world, self.rank, self.group, self.emulated = world, rank, None, True
        elif group is None and not (dist.is_available() and dist.is_initialized()):
            self.world, self.rank, self.group, self.emulated = 1, 0, None, False
        else:
            self.group = group if group is not None else dist.group.WORLD
            self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
            self.emulated = False
        if self.world > 16:
            raise ValueError("at most 16 ranks")
        if num_experts % self.world or w1_local.shape[0] != num_experts // self.world:
            raise ValueError("expert weights do not match num_experts / world")
        if w1_local.shape[1] != 2 * w2_local.shape[2] or w1_local.shape[2] != w2_local.shape[1]:
            raise ValueError("w1 must be (E / world, 2I, H) and w2 (E / world, H, I)")
        from . import moe
        self.num_experts = num_experts
        self.local_experts_n = num_experts // self.world
        self.hidden, self.inter = w2_local.shape[1], w2_local.shape[2]
        self.mxfp8 = mxfp8
        self.dtype = w1_local.dtype
        if mxfp8:
            if self.hidden % 512 or self.inter % 128:
                raise ValueError("MXFP8 experts need hidden a multiple of 512 and intermediate of 128")
            self.w1, self.w1_sf = moe.quantize_expert_weights(w1_local)
            self.w2, self.w2_sf = moe.quantize_expert_weights(w2_local)
        else:
            self.w1, self.w2 = moe._check_weight(w1_local), moe._check_weight(w2_local)
        self._sized_for = None
        self.own: dict[str, torch.Tensor] = {}
        self.peer: dict[str, list[torch.Tensor]] = {}

    # ---- buffers -----------------------------------------------------------------------------
    def _symmetric(self, shape, dtype, dev):
        """A zero-filled buffer every rank can store into: symmetric memory across processes, a
        plain tensor for one rank or emulated ranks."""
        if self.world == 1 or self.emulated:
            return torch.zeros(shape, dtype=dtype, device=dev)
        import torch.distributed._symmetric_memory as symm_mem
        return symm_mem.empty(shape, dtype=dtype, device=dev).zero_()

    def _ensure_buffers(self, tokens: int, topk: int, dtype: torch.dtype, dev) -> None:
        key = (tokens, topk, dtype, dev)
        if self._sized_for == key:
            return
        if dtype != self.dtype and not self.mxfp8:
            raise TypeError(f"activations are {dtype}, expert weights {self.dtype}")
        lib = _lib.lib()
        w, e, h = self.world, self.num_experts, self.hidden
        replicas = tokens * topk
        cap = lib.b200k_moe_ep_capacity_rows(replicas, w, e, TILE)
        self.replicas, self.capacity = replicas, cap
        row_bytes = h if self.mxfp8 else h * torch.empty(0, dtype=dtype).element_size()
        if row_bytes % 16:
            raise ValueError("rows must be multiples of 16 bytes")
        own = {
            "hist": self._symmetric((w, e), torch.int32, dev),
            "flags": self._symmetric((w,), torch.int32, dev),
            "rows": self._symmetric((cap, row_bytes), torch.uint8, dev),
            "meta": self._symmetric((cap,), torch.int32, dev),
            "weight": self._symmetric((cap,), torch.float32, dev),
            "y": self._symmetric((replicas, h), dtype, dev),
        }
        if self.mxfp8:
            own["aux"] = self._symmetric((cap, h // 32), torch.uint8, dev)
        self.own = own
        if self.world == 1:
            self.peer = {k: [t] for k, t in own.items()}
        elif not self.emulated:
            import torch.distributed._symmetric_memory as symm_mem
            self.peer = {}
            for k, t in own.items():
                handle = symm_mem.rendezvous(t, self.group.group_name)
                self.peer[k] = [handle.get_buffer(r, t.shape, t.dtype, 0) for r in range(w)]
        # rank-local state
        self.scratch = torch.zeros(e + 1, dtype=torch.int32, device=dev)
        self.first_row = torch.zeros(e, dtype=torch.int64, device=dev)
        self.cursor = torch.zeros(e, dtype=torch.int32, device=dev)
        self.tile_group = torch.zeros(cap // TILE, dtype=torch.int32, device=dev)
        self.num_row_tiles = torch.zeros(1, dtype=torch.int32, device=dev)
        self.epoch = torch.zeros(1, dtype=torch.int32, device=dev)
        from .block_scaled import swizzled_shape
        if self.mxfp8:
            self.a_sf = torch.zeros(swizzled_shape(cap, h // 32), dtype=torch.uint8, device=dev)
            self.act = torch.empty((cap, self.inter), dtype=torch.float8_e4m3fn, device=dev)
            self.act_sf = torch.zeros(swizzled_shape(cap, self.inter // 32), dtype=torch.uint8, device=dev)
        else:
            self.act = torch.empty((cap, self.inter), dtype=dtype, device=dev)
            self.gate_up = (torch.empty((cap, 2 * self.inter), dtype=dtype, device=dev)
                            if self.inter % 128 else None)
        self._sized_for = key
        if self.world > 1 and not self.emulated:
            dist.barrier(self.group)           # every rank's buffers exist and are zero

    # ---- phases ------------------------------------------------------------------------------
    def _ids(self, topk_ids):
        ids = topk_ids.contiguous()
        if ids.dtype not in (torch.int32, torch.int64):
            raise TypeError("topk_ids must be int32 or int64")
        return ids

    def _count(self, ids) -> None:
        a = _lib.MoeEpCountArgs()
        a.topk_ids, a.num_replicas = ids.data_ptr(), ids.numel()
        a.ids_are_int64 = 1 if ids.dtype == torch.int64 else 0
        a.num_experts, a.world, a.rank = self.num_experts, self.world, self.rank
        a.scratch = self.scratch.data_ptr()
        keep, a.hist_peers = _ptr_array(self.peer["hist"])
        dev = ids.device
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().b200k_moe_ep_count(ctypes.byref(a), _lib.stream_ptr(dev)))

    def _barrier(self) -> None:
        if self.world == 1 or self.emulated:
            return
        dev = self.epoch.device
        keep, flags = _ptr_array(self.peer["flags"])
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().b200k_peer_barrier(flags, self.world, self.rank, self.epoch.data_ptr(), 0,
                                                     _lib.stream_ptr(dev)))

    def _plan(self) -> None:
        a = _lib.MoeEpPlanArgs()
        a.hist = self.own["hist"].data_ptr()
        a.world, a.rank, a.num_experts, a.tile_rows = self.world, self.rank, self.num_experts, TILE
        a.capacity_rows = self.capacity
        a.first_row, a.cursor = self.first_row.data_ptr(), self.cursor.data_ptr()
        a.tile_group, a.num_row_tiles = self.tile_group.data_ptr(), self.num_row_tiles.data_ptr()
        a.meta = self.own["meta"].data_ptr()
        dev = self.epoch.device
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().b200k_moe_ep_plan(ctypes.byref(a), _lib.stream_ptr(dev)))

    def _dispatch(self, x, topk_weights, ids) -> None:
        from .block_scaled import block_quantize
        if self.mxfp8:
            src, aux = block_quantize(x, 32)             # once per token, not once per replica
            src, aux = src.view(torch.uint8), aux.view(torch.uint8)
        else:
            src, aux = x.view(torch.uint8), None
        weights = topk_weights.reshape(-1).float().contiguous()
        a = _lib.MoeEpDispatchArgs()
        a.topk_ids, a.weights, a.num_replicas = ids.data_ptr(), weights.data_ptr(), ids.numel()
        a.topk, a.ids_are_int64 = ids.shape[1], 1 if ids.dtype == torch.int64 else 0
        a.num_experts, a.world, a.rank = self.num_experts, self.world, self.rank
        a.src, a.src_stride_bytes, a.row_bytes = src.data_ptr(), src.stride(0), src.shape[1]
        if aux is not None:
            a.aux, a.aux_stride_bytes, a.aux_bytes = aux.data_ptr(), aux.stride(0), aux.shape[1]
        a.first_row, a.cursor, a.capacity_rows = self.first_row.data_ptr(), self.cursor.data_ptr(), self.capacity
        k1, a.row_peers = _ptr_array(self.peer["rows"])
        k2, a.meta_peers = _ptr_array(self.peer["meta"])
        k3, a.weight_peers = _ptr_array(self.peer["weight"])
        if aux is not None:
            k4, a.aux_peers = _ptr_array(self.peer["aux"])
        dev = x.device
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().b200k_moe_ep_dispatch(ctypes.byref(a), _lib.stream_ptr(dev)))

    def _experts(self) -> None:
        """Grouped GEMMs over the rows this rank received; results leave the second GEMM's
        epilogue for the y buffers of the ranks the rows came from."""
        from . import moe
        own = self.own
        peers = dict(row_map=own["meta"], row_scale=own["weight"], c_peers=self.peer["y"],
                     c_peer_rows=self.replicas, tile=TILE, num_blocks=self.num_row_tiles)
        if self.mxfp8:
            dev = own["rows"].device
            cap, kblocks = own["aux"].shape
            with torch.cuda.device(dev):
                _lib.check(_lib.lib().b200k_sf_swizzle(own["aux"].data_ptr(), cap, kblocks, kblocks,
                                                       self.a_sf.data_ptr(), self.a_sf.shape[1], 127,
                                                       self.num_row_tiles.data_ptr(), TILE,
                                                       _lib.stream_ptr(dev)))
            a_q = own["rows"].view(torch.float8_e4m3fn)
            moe._grouped_scaled_gemm(a_q, self.a_sf, self.w1, moe._as_u8(self.w1_sf), self.act, self.tile_group,
                                     num_blocks=self.num_row_tiles, swiglu=True, tile=TILE, c_sf=self.act_sf)
            moe._grouped_scaled_gemm(self.act, self.act_sf, self.w2, moe._as_u8(self.w2_sf), own["y"],
                                     self.tile_group, **peers)
        else:
            a = own["rows"].view(self.dtype)
            if self.gate_up is None:
                moe._grouped_gemm(a, self.w1, self.act, self.tile_group, num_blocks=self.num_row_tiles,
                                  swiglu=True, tile=TILE)
            else:
                moe._grouped_gemm(a, self.w1, self.gate_up, self.tile_group, num_blocks=self.num_row_tiles,
                                  tile=TILE)
                moe.invoke_silu_and_mul_kernel(self.gate_up, self.act)
            moe._grouped_gemm(self.act, self.w2, own["y"], self.tile_group, **peers)

    def _combine(self, tokens, topk, ids) -> torch.Tensor:
        from . import moe
        return moe._topk_sum(self.own["y"], tokens, topk, self.hidden, expert_ids=ids,
                             num_experts=self.num_experts)

    def _check(self, hidden_states, topk_weights, topk_ids):
        if hidden_states.dim() != 2 or hidden_states.shape[1] != self.hidden:
            raise ValueError("hidden size of the activations and the expert weights differ")
        if topk_ids.shape != topk_weights.shape or topk_ids.shape[0] != hidden_states.shape[0]:
            raise ValueError("topk_ids / topk_weights must be (num_tokens, topk)")
        if not hidden_states.is_cuda:
            raise ValueError("Input tensors must be on a CUDA device.")
        x = hidden_states if hidden_states.is_contiguous() else hidden_states.contiguous()
        ids = self._ids(topk_ids)
        self._ensure_buffers(x.shape[0], ids.shape[1], x.dtype, x.device)
        return x, ids

    def forward(self, hidden_states: torch.Tensor, topk_weights: torch.Tensor,
                topk_ids: torch.Tensor) -> torch.Tensor:
        if self.emulated:
            raise RuntimeError("emulated ranks run through emulate_ranks()")
        x, ids = self._check(hidden_states, topk_weights, topk_ids)
        tokens, topk = ids.shape
        if tokens == 0 and self.world == 1:
            return torch.empty_like(x)
        self._count(ids)
        self._barrier()
        self._plan()
        self._dispatch(x, topk_weights, ids)
        self._barrier()
        self._experts()
        self._barrier()
        return self._combine(tokens, topk, ids)


def emulate_ranks(moes: list[ExpertParallelMoE], xs, tws, idss) -> list[torch.Tensor]:
    """One layer for all ranks of an emulated world on one GPU: rank r is moes[r] (built with
    world=len(moes), rank=r) with inputs xs[r], tws[r], idss[r].  The phases run in lock step
    in one stream, which orders them the way the barriers do across processes."""
    world = len(moes)
    if any(m.world != world or m.rank != r or not m.emulated for r, m in enumerate(moes)):
        raise ValueError("moes[r] must be built with world=len(moes), rank=r")
    checked = [m._check(x, tw, ids) for m, x, tw, ids in zip(moes, xs, tws, idss)]
    for m in moes:                                   # every rank sees every rank's buffers
        m.peer = {k: [o.own[k] for o in moes] for k in m.own}
    for m, (x, ids) in zip(moes, checked):
        m._count(ids)
    for m in moes:
        m._plan()
    for m, (x, ids), tw in zip(moes, checked, tws):
        m._dispatch(x, tw, ids)
    for m in moes:
        m._experts()
    return [m._combine(ids.shape[0], ids.shape[1], ids) for m, (x, ids) in zip(moes, checked)]
