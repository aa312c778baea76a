"""AllGather + matmul with the entry point of the reference's sample.

cutile_gather_matmul   samples/AllGatherMatmul.py:85-120
    out[(p * M + m), :] = inp_p[m, :] @ w  for every rank p, on every rank.

Each rank pulls the other ranks' shards out of their symmetric-memory buffers into a local
staging buffer with one kernel (plain peer loads over NVLink, all peers at once) and runs
the tcgen05 GEMM on the staged A; the NVFP4 form multiplies its own rows while the gather
is in flight.  As in the sample, the caller makes the peers' inputs
visible first (a barrier) and keeps them unchanged until every rank has finished.

The kernels only need pointers this process can dereference, so every entry point also takes
the shards explicitly (``peers=[...]``, ``rank=``): the buffers of all ranks as this process
sees them.  With one process and plain local tensors that runs the whole multi-rank path on
one GPU (no kernel here waits on another, so emulated ranks may run one after the other).
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from . import _lib
from .block_scaled import _as_u8, _scaled_gemm
from .matmul import _gemm


def shard_rows(total_rows: int, world: int, rank: int) -> tuple[int, int]:
    """[begin, end) of the rows rank owns when `total_rows` are split evenly."""
    if total_rows % world:
        raise ValueError(f"{total_rows} rows do not split evenly over {world} ranks")
    per = total_rows // world
    return rank * per, (rank + 1) * per


def peer_buffers(t: torch.Tensor, group) -> list[torch.Tensor]:
    """The same symmetric-memory tensor as seen on every rank (index = rank)."""
    import torch.distributed._symmetric_memory as symm_mem
    handle = symm_mem.rendezvous(t, group.group_name)
    return [handle.get_buffer(r, t.shape, t.dtype, 0) for r in range(handle.world_size)]


def peer_gather(shards: list[torch.Tensor], rank: int, *, round_tf32: bool = False,
                out: torch.Tensor | None = None) -> torch.Tensor:
    """Concatenates `shards` (one (rows, cols) tensor per rank, peer-mapped) along dim 0 into
    a local tensor."""
    world = len(shards)
    mine = shards[rank]
    rows, cols = mine.shape
    if any(s.shape != mine.shape or s.dtype != mine.dtype or s.stride() != mine.stride() for s in shards):
        raise ValueError("all shards must have the same shape, dtype and strides")
    if mine.stride(1) != 1:
        raise ValueError("shards must have contiguous rows")
    if out is None:
        out = torch.empty((world * rows, cols), dtype=mine.dtype, device=mine.device)
    ptrs = (ctypes.c_void_p * world)(*[s.data_ptr() for s in shards])
    a = _lib.PeerGatherArgs()
    a.shards = ctypes.cast(ptrs, ctypes.POINTER(ctypes.c_void_p))
    a.dst = out.data_ptr()
    a.rows, a.row_bytes = rows, cols * mine.element_size()
    a.src_stride_bytes = mine.stride(0) * mine.element_size()
    a.dst_stride_bytes = out.stride(0) * out.element_size()
    a.world, a.rank = world, rank
    a.round_tf32 = 1 if (round_tf32 and mine.dtype == torch.float32) else 0
    with torch.cuda.device(mine.device):
        _lib.check(_lib.lib().b200k_peer_gather(ctypes.byref(a), _lib.stream_ptr(mine.device)))
    return out


_SIDE_STREAMS: dict = {}


def _side_stream(device) -> torch.cuda.Stream:
    """One side stream per device for the gather and the GEMM that follows it."""
    idx = torch.device(device).index
    if idx is None:
        idx = torch.cuda.current_device()
    if idx not in _SIDE_STREAMS:
        _SIDE_STREAMS[idx] = torch.cuda.Stream(torch.device("cuda", idx))
    return _SIDE_STREAMS[idx]


def _round_tf32(t: torch.Tensor) -> torch.Tensor:
    """fp32 -> nearest tf32 value (ties away from zero), still stored as fp32."""
    bits = t.contiguous().view(torch.int32)
    return ((bits + 0x1000) & ~0x1FFF).view(torch.float32)


def _world_and_rank(group, peers, rank):
    """(world, rank, group): from explicit peers, else from the process group, else a world of
    one (no process group initialised: the gather degenerates to the local shard)."""
    if peers is not None:
        if rank is None or not 0 <= rank < len(peers):
            raise ValueError("explicit peers need rank in [0, len(peers))")
        return len(peers), rank, None
    if group is None:
        if not (dist.is_available() and dist.is_initialized()):
            return 1, 0, None
        group = dist.group.WORLD
    return dist.get_world_size(group), dist.get_rank(group), group


def cutile_gather_matmul(inp: torch.Tensor, w: torch.Tensor, group=None, *,
                         transport: str = "p2p", peers: list[torch.Tensor] | None = None,
                         rank: int | None = None) -> torch.Tensor:
    """out (M * world, N) = concat over ranks of inp_p (M, K) @ w (K, N).

    ``inp`` must live in symmetric memory (``torch.distributed._symmetric_memory.empty``)
    for the default "p2p" transport; "nccl" gathers with ``all_gather_into_tensor``
    instead and accepts any tensor.  ``peers`` (every rank's ``inp`` as this process can
    address it) with ``rank`` replaces the symmetric-memory rendezvous.  fp32 operands are
    rounded to tf32 and multiplied on the tensor cores, as in the reference kernel
    (samples/AllGatherMatmul.py:57)."""
    if inp.dim() != 2 or w.dim() != 2:
        raise ValueError("inp and w must be 2-D")
    if inp.shape[1] != w.shape[0]:
        raise ValueError("reduction dimension mismatch")
    if not inp.is_cuda or inp.device != w.device:
        raise ValueError("Input tensors must be on the same CUDA device.")
    world, rank, group = _world_and_rank(group, peers, rank)
    m, k = inp.shape
    n = w.shape[1]
    fp32 = inp.dtype == torch.float32
    if transport == "p2p":
        if peers is None:
            peers = [inp] if world == 1 else peer_buffers(inp, group)
        if (world > 1 and not fp32 and m % 256 == 0 and m * n * k > 0 and inp.stride(1) == 1
                and (inp.stride(0) * inp.element_size()) % 16 == 0 and inp.data_ptr() % 16 == 0):
            # 16-bit shards of whole 256-row tiles: the own rows are multiplied straight out of
            # the rank's buffer while, on a side stream, the other shards arrive and are
            # multiplied in one launch whose raster leaves the own row tiles out
            out = torch.empty((world * m, n), dtype=inp.dtype, device=inp.device)
            staged = torch.empty((world * m, k), dtype=inp.dtype, device=inp.device)
            main = torch.cuda.current_stream(inp.device)
            side = _side_stream(inp.device)
            side.wait_stream(main)
            with torch.cuda.stream(side):
                peer_gather(peers, rank, out=staged)
                _gemm(staged, w, out, skip_rows=(rank * m, m))
            _gemm(inp, w, out[rank * m:(rank + 1) * m])
            main.wait_stream(side)
            staged.record_stream(side)
            return out
        staged = peer_gather(peers, rank, round_tf32=fp32)
    elif transport == "nccl":
        staged = torch.empty((world * m, k), dtype=inp.dtype, device=inp.device)
        if world == 1:
            staged.copy_(inp)
        else:
            dist.all_gather_into_tensor(staged, inp.contiguous(), group=group)
        if fp32:
            staged = _round_tf32(staged)
    else:
        raise ValueError("transport must be 'p2p' or 'nccl'")
    if fp32:
        w = _round_tf32(w.T).T      # (N, K) K-contiguous storage, viewed as (K, N)
    out = torch.empty((world * m, n), dtype=inp.dtype, device=inp.device)
    if world * m == 0 or n == 0:
        return out
    return _gemm(staged, w, out)


class Nvfp4GatherMatmul:
    """AllGather GEMM on NVFP4 operands with the peer mappings and staging buffers set up
    once: ``run()`` is then one gather kernel per operand part plus the GEMM, with no host
    synchronisation.  Each rank contributes the quantised rows it owns — a_q (M, K/2) packed
    e2m1, a_sf its swizzled ue4m3 scales (M/128, K/64, 32, 16), a_ts its fp32 tensor scale
    (1,) — all three whole symmetric-memory allocations; M a multiple of 128 so that scale
    atoms do not straddle ranks."""

    def __init__(self, a_q: torch.Tensor, a_sf: torch.Tensor, a_ts: torch.Tensor, group=None, *,
                 peers=None, rank: int | None = None):
        """``peers`` = (list of every rank's a_q, of a_sf, of a_ts) as this process can address
        them, with ``rank``, replaces the symmetric-memory rendezvous."""
        self.world, self.rank, group = _world_and_rank(group, None if peers is None else peers[0], rank)
        self.m = a_q.shape[0]
        if self.m % 128:
            raise ValueError("rows per rank must be a multiple of 128")
        self.sf_shape = tuple(a_sf.shape)
        if peers is not None:
            q_list, sf_list, ts_list = peers
        elif self.world == 1:
            q_list, sf_list, ts_list = [a_q], [a_sf], [a_ts]
        else:
            q_list = sf_list = ts_list = None
        if q_list is not None:
            self.q_peers = [_as_u8(t) for t in q_list]
            self.sf_peers = [_as_u8(t).reshape(t.shape[0], -1) for t in sf_list]
            self.ts_peers = [t.reshape(1, 1) for t in ts_list]
        else:
            self.q_peers = peer_buffers(_as_u8(a_q), group)
            self.sf_peers = peer_buffers(_as_u8(a_sf).reshape(a_sf.shape[0], -1), group)
            self.ts_peers = peer_buffers(a_ts.reshape(1, 1), group)
        dev = a_q.device
        self.q = torch.empty((self.world * self.m, a_q.shape[1]), dtype=torch.uint8, device=dev)
        self.sf = torch.empty((self.world * a_sf.shape[0], self.sf_peers[0].shape[1]),
                              dtype=torch.uint8, device=dev)
        self.ts = torch.empty((self.world, 1), dtype=torch.float32, device=dev)
        self.row_scale = torch.empty(self.world * self.m, dtype=torch.float32, device=dev)
        self.sf_own = _as_u8(a_sf)
        self.side = torch.cuda.Stream(dev)
        # whole 256-row tiles per rank: the other ranks' rows go through one GEMM launch
        self.one_remote_launch = self.m % 256 == 0
        self._batch = None

    def _batch_args(self):
        """Packed operand and scale atoms as one batch of two dense gathers, plus the pointer
        table of the tensor scales; built once, the buffers never move."""
        args = (_lib.PeerGatherArgs * 2)()
        keep = []
        for a, shards, out in ((args[0], self.q_peers, self.q), (args[1], self.sf_peers, self.sf)):
            mine = shards[self.rank]
            ptrs = (ctypes.c_void_p * self.world)(*[s.data_ptr() for s in shards])
            keep.append(ptrs)
            a.shards = ctypes.cast(ptrs, ctypes.POINTER(ctypes.c_void_p))
            a.dst = out.data_ptr()
            a.rows, a.row_bytes = mine.shape[0], mine.shape[1] * mine.element_size()
            a.src_stride_bytes = mine.stride(0) * mine.element_size()
            a.dst_stride_bytes = out.stride(0) * out.element_size()
            a.world, a.rank, a.round_tf32 = self.world, self.rank, 0
        ts = (ctypes.c_void_p * self.world)(*[t.data_ptr() for t in self.ts_peers])
        keep.append(ts)
        dense = all(a.src_stride_bytes == a.row_bytes == a.dst_stride_bytes for a in args)
        return args, ctypes.cast(ts, ctypes.POINTER(ctypes.c_void_p)), keep, dense

    def gather(self):
        """One launch for the packed operand, the scale atoms and the per-row expansion of the
        peers' tensor scales (three launches where a shard is not dense)."""
        if self._batch is None:
            self._batch = self._batch_args()
        args, ts, _, dense = self._batch
        dev = self.q.device
        with torch.cuda.device(dev):
            if dense:
                _lib.check(_lib.lib().b200k_peer_gather_batch(args, 2, ts, self.m, self.row_scale.data_ptr(),
                                                              _lib.stream_ptr(dev)))
                return
            peer_gather(self.q_peers, self.rank, out=self.q)
            peer_gather(self.sf_peers, self.rank, out=self.sf)
            _lib.check(_lib.lib().b200k_peer_scalar_expand(ts, self.world, self.m, self.row_scale.data_ptr(),
                                                           _lib.stream_ptr(dev)))

    def run(self, w_q, w_sf, w_ts, out: torch.Tensor | None = None,
            out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        """The gather and, behind it, the GEMM of the other ranks' rows run on a side stream
        while the rows this rank owns are multiplied straight out of its own buffers on the
        caller's stream: stream order is the only dependency (no kernel waits on another), and
        the CTAs of the second GEMM move in as those of the first leave, so the partly filled
        last round of the first costs nothing.  The caller's stream waits for the side stream
        before the call returns."""
        n = w_q.shape[0]
        dev = self.q.device
        m, world, rank = self.m, self.world, self.rank
        if out is None:
            out = torch.empty((world * m, n), dtype=out_dtype, device=dev)
        wq, wsf = _as_u8(w_q), _as_u8(w_sf)
        main = torch.cuda.current_stream(dev)
        if world > 1:
            self.side.wait_stream(main)    # operands are ready; the previous call is done with the staging
            with torch.cuda.stream(self.side):
                self.gather()
                tiles = self.sf_shape[0]       # 128-row scale tiles per rank
                sf = self.sf.reshape(world * tiles, *self.sf_shape[1:])
                if self.one_remote_launch:
                    # every other rank's rows in one launch over the gathered A: the row tiles of
                    # this rank's own shard are left out of the raster
                    _scaled_gemm(self.q, sf, wq, wsf, out, fp4=True, alpha_b=w_ts, row_scale=self.row_scale,
                                 skip_rows=(rank * m, m))
                else:
                    for lo, hi in ((0, rank), (rank + 1, world)):
                        if hi > lo:
                            _scaled_gemm(self.q[lo * m:hi * m], sf[lo * tiles:hi * tiles], wq, wsf,
                                         out[lo * m:hi * m], fp4=True, alpha_b=w_ts,
                                         row_scale=self.row_scale[lo * m:hi * m])
        _scaled_gemm(self.q_peers[rank], self.sf_own, wq, wsf, out[rank * m:(rank + 1) * m], fp4=True,
                     alpha_a=self.ts_peers[rank], alpha_b=w_ts)
        if world > 1:
            main.wait_stream(self.side)
        return out


def cutile_gather_matmul_nvfp4(a_q: torch.Tensor, a_sf: torch.Tensor, a_ts: torch.Tensor,
                               w_q: torch.Tensor, w_sf: torch.Tensor, w_ts: torch.Tensor,
                               group=None, *, out_dtype: torch.dtype = torch.bfloat16,
                               peers=None, rank: int | None = None) -> torch.Tensor:
    """One-shot form of Nvfp4GatherMatmul: returns (M * world, N)."""
    return Nvfp4GatherMatmul(a_q, a_sf, a_ts, group, peers=peers, rank=rank).run(
        w_q, w_sf, w_ts, out_dtype=out_dtype)
