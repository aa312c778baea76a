"""Mixture-of-experts FFN with the entry points of the reference's sample.

cutile_moe                   samples/MoE.py:197-288
moe_align_tile_size_torch    test/kernels/fused_moe.py:113-173
invoke_fused_moe_kernel      samples/MoE.py:338-375
invoke_silu_and_mul_kernel   samples/MoE.py:378-393
cutile_moe_mxfp8             the same FFN with MXFP8 expert weights and activations (the
                             reference has only the bf16 form)

Pipeline of cutile_moe (no host synchronisation anywhere): device-side alignment ->
row gather of the hidden states into expert order -> grouped GEMM with fused SiLU-and-
multiply epilogue -> grouped GEMM with routed-weight scaling and row scatter -> top-k sum.
The grouped GEMM runs on CTA pairs over 256-row tiles (each tile one expert), so the
alignment uses tile_m = 256 internally (128 with the one-CTA kernels, B200K_MOE_TILE=128);
`tile_m/tile_n/tile_k` are accepted for signature compatibility.
"""
from __future__ import annotations

import ctypes
import os

import torch

from . import _lib
from .block_scaled import _as_u8, swizzled_shape

ROW_TILE = 128          # row tile of the one-CTA grouped GEMM
ROW_TILES = (128, 256)  # 256: the CTA-pair grouped GEMM


def _moe_tile(replicas: int | None = None, experts: int | None = None) -> int:
    """Row tile the FFN entry points align with: 256 (the CTA-pair grouped GEMM), or 128 when
    the routing is so sparse that most of a tile would be padding (fewer than 64 token replicas
    per expert on average - the reference's 1408-expert bench shape has about one)."""
    if os.environ.get("B200K_SINGLE_CTA") == "1" or os.environ.get("B200K_MOE_TILE") == "128":
        return 128
    if os.environ.get("B200K_MOE_TILE") == "256":
        return 256
    if replicas is not None and experts and replicas < 64 * experts:
        return 128
    return 256


def _cdiv(a: int, b: int) -> int:
    return (a + b - 1) // b


def moe_align_device(topk_ids: torch.Tensor, tile_m: int, num_experts: int, *,
                     want_expert_ids: bool = True):
    """Device-side alignment.  Returns (sorted_token_ids [capacity] int32,
    sorted_expert_ids [capacity / tile_m] int32 (None when not wanted), num_blocks int32
    device scalar)."""
    if topk_ids.dim() != 2:
        raise ValueError("topk_ids must be (num_tokens, topk)")
    if not topk_ids.is_cuda:
        raise ValueError("Input tensors must be on a CUDA device.")
    if topk_ids.dtype not in (torch.int32, torch.int64):
        raise TypeError("topk_ids must be int32 or int64")
    ids = topk_ids.contiguous()
    total = ids.numel()
    blocks = _cdiv(total + num_experts * (tile_m - 1), tile_m)
    dev = ids.device
    sorted_ids = torch.empty(blocks * tile_m, dtype=torch.int32, device=dev)
    expert_ids = torch.empty(blocks, dtype=torch.int32, device=dev) if want_expert_ids else None
    num_blocks = torch.empty(1, dtype=torch.int32, device=dev)
    ws_bytes = _lib.lib().b200k_moe_align_workspace_bytes(total, num_experts)
    ws = torch.empty(max(ws_bytes, 4), dtype=torch.uint8, device=dev)
    a = _lib.MoeAlignArgs()
    a.topk_ids = ids.data_ptr()
    a.sorted_token_ids, a.sorted_expert_ids = sorted_ids.data_ptr(), _lib.ptr(expert_ids)
    a.num_blocks, a.workspace, a.workspace_bytes = num_blocks.data_ptr(), ws.data_ptr(), ws.numel()
    a.num_replicas, a.capacity, a.block_capacity = total, sorted_ids.numel(), blocks
    a.num_experts, a.tile_m = num_experts, tile_m
    a.ids_are_int64 = 1 if ids.dtype == torch.int64 else 0
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().b200k_moe_align(ctypes.byref(a), _lib.stream_ptr(dev)))
    return sorted_ids, expert_ids, num_blocks


def moe_align_tile_size_torch(topk_ids: torch.Tensor, tile_m: int, num_experts: int):
    """Same outputs as the reference function (exact lengths), computed on the device.
    Reading the block count back is the one host synchronisation; cutile_moe avoids it by
    using moe_align_device."""
    sorted_ids, expert_ids, num_blocks = moe_align_device(topk_ids, tile_m, num_experts)
    n = int(num_blocks.item())
    return sorted_ids[: n * tile_m], expert_ids[:n]


def _gather_rows(src: torch.Tensor, index: torch.Tensor, divisor: int, rows: int,
                 num_blocks: torch.Tensor | None, tile: int = ROW_TILE, *,
                 by_source: bool = False) -> torch.Tensor:
    """dst row i = src row index[i] // divisor (zero rows for sentinels).  ``by_source``: the
    valid entries of ``index`` are distinct replica ids (the alignment's output); every source
    row is then read once and stored to all its places."""
    if src.stride(1) != 1 or (src.stride(0) * src.element_size()) % 16 or src.data_ptr() % 16 \
            or (src.shape[1] * src.element_size()) % 16:
        raise ValueError("gather source rows must be contiguous multiples of 16 bytes")
    dst = torch.empty((rows, src.shape[1]), dtype=src.dtype, device=src.device)
    if by_source:
        scratch = torch.empty(max(src.shape[0] * divisor, 1), dtype=torch.int32, device=src.device)
        with torch.cuda.device(src.device):
            _lib.check(_lib.lib().b200k_gather_rows_by_source(
                src.data_ptr(), src.shape[0], src.shape[1] * src.element_size(),
                src.stride(0) * src.element_size(), index.data_ptr(), divisor,
                _lib.ptr(num_blocks), tile, rows, dst.data_ptr(),
                dst.stride(0) * dst.element_size(), scratch.data_ptr(), _lib.stream_ptr(src.device)))
        return dst
    with torch.cuda.device(src.device):
        _lib.check(_lib.lib().b200k_gather_rows(
            src.data_ptr(), src.shape[0], src.shape[1] * src.element_size(),
            src.stride(0) * src.element_size(), index.data_ptr(), divisor,
            _lib.ptr(num_blocks), tile, rows, dst.data_ptr(),
            dst.stride(0) * dst.element_size(), _lib.stream_ptr(src.device)))
    return dst


def _set_c_peers(args, c_peers, c_peer_rows):
    """Output rows scattered over several buffers (b200k_gemm_args.c_peers).  Returns the
    pointer array, which must stay alive until the call has returned."""
    if c_peers is None:
        return None
    arr = (ctypes.c_void_p * len(c_peers))(*[t.data_ptr() for t in c_peers])
    args.c_peers = ctypes.cast(arr, ctypes.POINTER(ctypes.c_void_p))
    args.num_c_peers, args.c_peer_rows = len(c_peers), c_peer_rows
    return arr


def _grouped_gemm(a_sorted, w, c, expert_ids, *, num_blocks=None, row_map=None, row_scale=None,
                  c_rows=0, swiglu=False, tile=ROW_TILE, c_peers=None, c_peer_rows=0):
    """a_sorted (Mp, K) x w (E, N, K)^T with the expert of each `tile`-row tile in expert_ids."""
    mp, k = a_sorted.shape
    e, n, _ = w.shape
    args = _lib.GemmArgs()
    args.a, args.b, args.c = a_sorted.data_ptr(), w.data_ptr(), c.data_ptr()
    args.m, args.n, args.k, args.batch = mp, n, k, e
    args.lda, args.ldb, args.ldc = a_sorted.stride(0), w.stride(1), c.stride(0)
    args.stride_a, args.stride_b, args.stride_c = 0, w.stride(0), 0
    args.ab_dtype = _lib.dtype_enum(a_sorted.dtype)
    args.c_dtype = _lib.dtype_enum(c.dtype)
    args.b_layout = _lib.B_NK
    args.epilogue = _lib.EPI_SWIGLU if swiglu else _lib.EPI_STORE
    args.alpha = 1.0
    args.tile_group = expert_ids.data_ptr()
    args.num_row_tiles = _lib.ptr(num_blocks)
    args.row_map = _lib.ptr(row_map)
    args.row_scale = _lib.ptr(row_scale)
    args.c_rows = c_rows
    args.tile_rows = tile
    keep = _set_c_peers(args, c_peers, c_peer_rows)
    with torch.cuda.device(c.device):
        _lib.check(_lib.lib().b200k_gemm(ctypes.byref(args), _lib.stream_ptr(c.device)))
    del keep
    return c


def _check_weight(w: torch.Tensor) -> torch.Tensor:
    if w.stride(2) != 1 or (w.stride(1) * w.element_size()) % 16 or (w.stride(0) * w.element_size()) % 16:
        w = w.contiguous()
    if (w.shape[2] * w.element_size()) % 16:
        raise ValueError("expert weight rows must be multiples of 16 bytes")
    return w


def invoke_fused_moe_kernel(A, B, C, topk_weights, sorted_token_ids, sorted_expert_ids,
                            mul_routed_weight: bool, num_token_replicas: int,
                            tile_m: int = ROW_TILE, tile_n: int = 128, tile_k: int = 64) -> None:
    """C.view(-1, N)[r] = (A[r // num_token_replicas] @ B[expert(r)].T) [* topk_weights[r]] for
    every replica id r in sorted_token_ids; sentinel ids are skipped."""
    if tile_m not in ROW_TILES:
        raise ValueError(f"this kernel's row tiles are {ROW_TILES}: align with one of them")
    if sorted_token_ids.numel() != sorted_expert_ids.numel() * tile_m:
        raise ValueError("sorted_token_ids / sorted_expert_ids lengths disagree")
    c2 = C.view(-1, C.shape[-1])
    rows = sorted_token_ids.numel()
    if rows == 0:
        return
    a_sorted = _gather_rows(A, sorted_token_ids, num_token_replicas, rows, None, tile_m)
    scale = topk_weights.reshape(-1).float().contiguous() if mul_routed_weight else None
    _grouped_gemm(a_sorted, _check_weight(B), c2, sorted_expert_ids, row_map=sorted_token_ids,
                  row_scale=scale, c_rows=c2.shape[0], tile=tile_m)


def invoke_silu_and_mul_kernel(AB: torch.Tensor, C: torch.Tensor) -> None:
    rows, two_n = AB.shape
    with torch.cuda.device(AB.device):
        _lib.check(_lib.lib().b200k_silu_and_mul(AB.data_ptr(), rows, two_n // 2, AB.stride(0),
                                                 C.data_ptr(), C.stride(0),
                                                 _lib.dtype_enum(AB.dtype),
                                                 _lib.stream_ptr(AB.device)))


def _topk_sum(x: torch.Tensor, tokens: int, topk: int, hidden: int,
              index: torch.Tensor | None = None, *, expert_ids: torch.Tensor | None = None,
              num_experts: int = 0) -> torch.Tensor:
    """out[t] = sum over the token's slots of its rows of x.  With `expert_ids` (the routing
    ids) entries routed outside [0, num_experts) count as zero: the alignment dropped them, so
    their rows were never written."""
    out = torch.empty((tokens, hidden), dtype=x.dtype, device=x.device)
    ids = None
    if expert_ids is not None:
        ids = expert_ids.contiguous()
        if ids.dtype not in (torch.int32, torch.int64):
            raise TypeError("topk_ids must be int32 or int64")
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().b200k_topk_sum(x.data_ptr(), _lib.ptr(index), tokens, topk, hidden, out.data_ptr(),
                                             _lib.dtype_enum(x.dtype), _lib.ptr(ids),
                                             1 if (ids is not None and ids.dtype == torch.int64) else 0,
                                             num_experts, _lib.stream_ptr(x.device)))
    return out


def _sparse_routing(replicas: int, experts: int, hidden: int, inter: int, elem_bytes: int) -> bool:
    """True where the routed experts hold about one token each (at most two replicas per expert
    on average): a 128-row tile per expert would then be almost all padding, and streaming the
    expert's weights once per replica is cheaper.  B200K_MOE_SPARSE=0 / 1 forces the choice."""
    forced = os.environ.get("B200K_MOE_SPARSE")
    fits = (replicas <= 65535 and hidden <= 12288 and inter <= 12288 and
            (hidden * elem_bytes) % 16 == 0 and (inter * elem_bytes) % 16 == 0)
    if forced in ("0", "1"):
        return forced == "1" and fits
    return fits and replicas <= 2 * experts


def _moe_sparse(x, w1, w2, topk_weights, topk_ids) -> torch.Tensor:
    """cutile_moe for sparse routing (b200k_moe_sparse): two kernels that stream each replica's
    expert once, then the top-k sum."""
    tokens, hidden = x.shape
    experts, _, inter = w2.shape
    topk = topk_ids.shape[1]
    ids = topk_ids.contiguous()
    if ids.dtype not in (torch.int32, torch.int64):
        raise TypeError("topk_ids must be int32 or int64")
    weights = topk_weights.reshape(-1).float().contiguous()
    act = torch.empty((tokens * topk, inter), dtype=x.dtype, device=x.device)
    per_replica = torch.empty((tokens * topk, hidden), dtype=x.dtype, device=x.device)
    a = _lib.MoeSparseArgs()
    a.hidden_states, a.w1, a.w2 = x.data_ptr(), w1.data_ptr(), w2.data_ptr()
    a.topk_ids, a.topk_weights = ids.data_ptr(), weights.data_ptr()
    a.act, a.per_replica = act.data_ptr(), per_replica.data_ptr()
    a.tokens, a.hidden, a.intermediate = tokens, hidden, inter
    a.hidden_stride = x.stride(0)
    a.w1_stride_e, a.w1_ld, a.w2_stride_e, a.w2_ld = w1.stride(0), w1.stride(1), w2.stride(0), w2.stride(1)
    a.topk, a.num_experts = topk, experts
    a.ids_are_int64 = 1 if ids.dtype == torch.int64 else 0
    a.dtype = _lib.dtype_enum(x.dtype)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().b200k_moe_sparse(ctypes.byref(a), _lib.stream_ptr(x.device)))
    return _topk_sum(per_replica, tokens, topk, hidden)


def _validate(hidden_states, w1, w2, topk_weights, topk_ids):
    if w1.shape[1] != w2.shape[2] * 2:
        raise ValueError("w1 must have 2 * intermediate_size rows (gate + up projection)")
    if hidden_states.shape[1] != w1.shape[2] or hidden_states.shape[1] != w2.shape[1]:
        raise ValueError("hidden size of the activations and the expert weights differ")
    if topk_ids.shape != topk_weights.shape or topk_ids.shape[0] != hidden_states.shape[0]:
        raise ValueError("topk_ids / topk_weights must be (num_tokens, topk)")
    if not hidden_states.is_cuda:
        raise ValueError("Input tensors must be on a CUDA device.")


def cutile_moe(hidden_states: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor,
               topk_weights: torch.Tensor, topk_ids: torch.Tensor,
               tile_m: int = 128, tile_n: int = 128, tile_k: int = 64) -> torch.Tensor:
    """MoE FFN forward: out[t] = sum_j w[t, j] * W2[e] (silu(W1g[e] x_t) * (W1u[e] x_t)),
    e = topk_ids[t, j].  hidden_states (T, H) f16/bf16; w1 (E, 2I, H); w2 (E, H, I)."""
    _validate(hidden_states, w1, w2, topk_weights, topk_ids)
    tokens, hidden = hidden_states.shape
    experts, _, inter = w2.shape
    topk = topk_ids.shape[1]
    dtype, dev = hidden_states.dtype, hidden_states.device
    if tokens == 0:
        return torch.empty_like(hidden_states)
    x = hidden_states if hidden_states.stride(1) == 1 else hidden_states.contiguous()
    w1c, w2c = _check_weight(w1), _check_weight(w2)
    if _sparse_routing(tokens * topk, experts, hidden, inter, x.element_size()):
        return _moe_sparse(x, w1c, w2c, topk_weights, topk_ids)

    tile = _moe_tile(tokens * topk, experts)
    sorted_ids, expert_ids, num_blocks = moe_align_device(topk_ids, tile, experts)
    cap = sorted_ids.numel()
    a_sorted = _gather_rows(x, sorted_ids, topk, cap, num_blocks, tile, by_source=topk > 1)
    act = torch.empty((cap, inter), dtype=dtype, device=dev)
    if inter % 128 == 0:
        _grouped_gemm(a_sorted, w1c, act, expert_ids, num_blocks=num_blocks, swiglu=True, tile=tile)
    else:
        gate_up = torch.empty((cap, 2 * inter), dtype=dtype, device=dev)
        _grouped_gemm(a_sorted, w1c, gate_up, expert_ids, num_blocks=num_blocks, tile=tile)
        invoke_silu_and_mul_kernel(gate_up, act)
    per_replica = torch.empty((tokens * topk, hidden), dtype=dtype, device=dev)
    _grouped_gemm(act, w2c, per_replica, expert_ids, num_blocks=num_blocks, row_map=sorted_ids,
                  row_scale=topk_weights.reshape(-1).float().contiguous(), c_rows=tokens * topk,
                  tile=tile)
    return _topk_sum(per_replica, tokens, topk, hidden, expert_ids=topk_ids, num_experts=experts)


# ---- MXFP8 experts -----------------------------------------------------------------
def quantize_expert_weights(w: torch.Tensor):
    """(E, N, K) f16/bf16/f32 -> (e4m3 (E, N, K), swizzled ue8m0 scales (E, N/128, K/128, 32, 16)).
    N must be a multiple of 128 and K of 128 so that no scale atom straddles two experts."""
    from .block_scaled import block_quantize
    e, n, k = w.shape
    if n % 128 or k % 128:
        raise ValueError("expert weight dims must be multiples of 128 for MXFP8")
    q, sf = block_quantize(w.reshape(e * n, k), 32, swizzled_scale=True)
    return q.reshape(e, n, k), sf.reshape(e, n // 128, k // 128, 32, 16)


def _quantize_rows(x, *, rows, gather=None, divisor=1, num_blocks=None, tile=ROW_TILE):
    """MXFP8 quantisation of (optionally gathered) rows with swizzled scales."""
    k = x.shape[1]
    q = torch.empty((rows, k), dtype=torch.uint8, device=x.device)
    shape = swizzled_shape(rows, k // 32)
    sf = torch.empty(shape, dtype=torch.uint8, device=x.device)
    a = _lib.QuantizeArgs()
    a.x, a.q, a.sf_swizzled = x.data_ptr(), q.data_ptr(), sf.data_ptr()
    a.rows, a.k, a.ldx, a.ldq, a.sf_k_atoms = rows, k, x.stride(0), k, shape[1]
    a.x_dtype, a.q_dtype = _lib.dtype_enum(x.dtype), _lib.E4M3
    a.gather_index = _lib.ptr(gather)
    a.gather_divisor, a.tile_m, a.src_rows = divisor, tile, x.shape[0]
    a.live_blocks = _lib.ptr(num_blocks)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().b200k_mxfp8_quantize(ctypes.byref(a), _lib.stream_ptr(x.device)))
    return q.view(torch.float8_e4m3fn), sf


def _grouped_scaled_gemm(a_q, a_sf, w_q, w_sf, c, expert_ids, *, num_blocks, row_map=None,
                         row_scale=None, c_rows=0, swiglu=False, tile=ROW_TILE, c_sf=None,
                         c_peers=None, c_peer_rows=0):
    """`c` of dtype float8_e4m3fn together with `c_sf` (swizzled scale bytes) asks for the
    quantise-in-epilogue form: the result leaves the GEMM as an MXFP8 operand."""
    mp, k = a_q.shape
    e, n, _ = w_q.shape
    args = _lib.BlockScaledGemmArgs()
    args.a, args.b, args.c = a_q.data_ptr(), w_q.data_ptr(), c.data_ptr()
    args.sfa, args.sfb = a_sf.data_ptr(), w_sf.data_ptr()
    args.m, args.n, args.k, args.batch = mp, n, k, e
    args.lda, args.ldb, args.ldc = a_q.stride(0), w_q.stride(1), c.stride(0)
    args.stride_a, args.stride_b, args.stride_c = 0, w_q.stride(0), 0
    args.sf_k_atoms = a_sf.shape[1]
    args.stride_sfa, args.stride_sfb = 0, w_sf.stride(0)
    args.ab_dtype, args.c_dtype = _lib.E4M3, _lib.dtype_enum(c.dtype)
    args.epilogue = _lib.EPI_SWIGLU if swiglu else _lib.EPI_STORE
    args.alpha = 1.0
    args.tile_group = expert_ids.data_ptr()
    args.num_row_tiles = _lib.ptr(num_blocks)
    args.row_map = _lib.ptr(row_map)
    args.row_scale = _lib.ptr(row_scale)
    args.c_rows = c_rows
    args.tile_rows = tile
    if c_sf is not None:
        args.c_sf, args.c_sf_k_atoms = c_sf.data_ptr(), c_sf.shape[1]
    keep = _set_c_peers(args, c_peers, c_peer_rows)
    with torch.cuda.device(c.device):
        _lib.check(_lib.lib().b200k_block_scaled_gemm(ctypes.byref(args), _lib.stream_ptr(c.device)))
    del keep
    return c


def cutile_moe_mxfp8(hidden_states: torch.Tensor, w1_q: torch.Tensor, w1_sf: torch.Tensor,
                     w2_q: torch.Tensor, w2_sf: torch.Tensor, topk_weights: torch.Tensor,
                     topk_ids: torch.Tensor) -> torch.Tensor:
    """The MoE FFN with MXFP8 expert weights (from quantize_expert_weights).  Activations are
    quantised to MXFP8 on the fly, fused with the permutation; the SiLU-and-multiply
    output is rounded to the activation dtype and re-quantised before the down projection."""
    _validate(hidden_states, w1_q, w2_q, topk_weights, topk_ids)
    tokens, hidden = hidden_states.shape
    experts, _, inter = w2_q.shape
    topk = topk_ids.shape[1]
    dtype, dev = hidden_states.dtype, hidden_states.device
    if hidden % 128 or inter % 128:
        raise ValueError("hidden and intermediate sizes must be multiples of 128 for MXFP8")
    if tokens == 0:
        return torch.empty_like(hidden_states)
    x = hidden_states if hidden_states.stride(1) == 1 else hidden_states.contiguous()
    tile = _moe_tile(tokens * topk, experts)
    sorted_ids, expert_ids, num_blocks = moe_align_device(topk_ids, tile, experts)
    cap = sorted_ids.numel()
    a_q, a_sf = _quantize_rows(x, rows=cap, gather=sorted_ids, divisor=topk, num_blocks=num_blocks,
                               tile=tile)
    if tile == 256 and dtype == torch.bfloat16 and os.environ.get("B200K_MOE_FUSED_QUANT") != "0":
        # the gate/up GEMM quantises its SiLU-and-multiply output in the epilogue: the
        # activation never exists as a 16-bit tensor in memory (same bytes as the two-step form)
        act_q = torch.empty((cap, inter), dtype=torch.float8_e4m3fn, device=dev)
        act_sf = torch.empty(swizzled_shape(cap, inter // 32), dtype=torch.uint8, device=dev)
        _grouped_scaled_gemm(a_q, a_sf, w1_q, _as_u8(w1_sf), act_q, expert_ids, num_blocks=num_blocks,
                             swiglu=True, tile=tile, c_sf=act_sf)
    else:
        act = torch.empty((cap, inter), dtype=dtype, device=dev)
        _grouped_scaled_gemm(a_q, a_sf, w1_q, _as_u8(w1_sf), act, expert_ids, num_blocks=num_blocks,
                             swiglu=True, tile=tile)
        act_q, act_sf = _quantize_rows(act, rows=cap, num_blocks=num_blocks, tile=tile)
    per_replica = torch.empty((tokens * topk, hidden), dtype=dtype, device=dev)
    _grouped_scaled_gemm(act_q, act_sf, w2_q, _as_u8(w2_sf), per_replica, expert_ids,
                         num_blocks=num_blocks, row_map=sorted_ids,
                         row_scale=topk_weights.reshape(-1).float().contiguous(),
                         c_rows=tokens * topk, tile=tile)
    return _topk_sum(per_replica, tokens, topk, hidden, expert_ids=topk_ids, num_experts=experts)
