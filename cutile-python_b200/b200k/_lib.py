"""ctypes binding of libb200k.so (the C ABI declared in include/b200k.h).

The shared library is the only compute path of this package: if it is missing or
fails to load, importing an operator raises — there is no fallback.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_void_p

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# B200K_LIB points at an alternative build of the library (e.g. one with tracing compiled in)
LIB_PATH = os.environ.get("B200K_LIB") or os.path.join(_HERE, "libb200k.so")

# enum b200k_dtype
F16, BF16, F32, E4M3, E5M2, E2M1X2 = range(6)
# enum b200k_b_layout
B_KN, B_NK = 0, 1
# enum b200k_epilogue
EPI_STORE, EPI_SWIGLU = 0, 1
# enum b200k_status
OK, INVALID_ARG, UNSUPPORTED, CUDA_ERROR, TIMEOUT = 0, -1, -2, -3, -4


class B200KError(RuntimeError):
    """A b200k entry point returned a negative status."""

    def __init__(self, code: int, message: str):
        super().__init__(f"b200k error {code}: {message}")
        self.code = code


class GemmConfig(Structure):
    _fields_ = [("kernel", c_int32), ("tile_n", c_int32), ("epilogue_store", c_int32),
                ("split_k", c_int32), ("wait_budget_us", c_int32), ("withhold_arrival", c_int32),
                ("programmatic_launch", c_int32), ("group_m", c_int32)]


class GemmArgs(Structure):
    _fields_ = [
        ("a", c_void_p), ("b", c_void_p), ("c", c_void_p),
        ("m", c_int64), ("n", c_int64), ("k", c_int64), ("batch", c_int64),
        ("lda", c_int64), ("ldb", c_int64), ("ldc", c_int64),
        ("stride_a", c_int64), ("stride_b", c_int64), ("stride_c", c_int64),
        ("ab_dtype", c_int32), ("c_dtype", c_int32), ("b_layout", c_int32), ("epilogue", c_int32),
        ("alpha", c_float), ("max_ctas", c_int32),
        ("tile_group", c_void_p), ("num_row_tiles", c_void_p),
        ("row_map", c_void_p), ("row_scale", c_void_p), ("c_rows", c_int64),
        ("tile_rows", c_int32),
        ("workspace", c_void_p), ("workspace_bytes", c_int64),
        ("config", POINTER(GemmConfig)),
        ("c_peers", POINTER(c_void_p)), ("num_c_peers", c_int32), ("c_peer_rows", c_int64),
        ("skip_rows_begin", c_int64), ("skip_rows_count", c_int64),
    ]


class GroupProblem(Structure):
    _fields_ = [("a", c_void_p), ("b", c_void_p), ("c", c_void_p),
                ("m", c_int64), ("n", c_int64), ("k", c_int64),
                ("lda", c_int64), ("ldb", c_int64), ("ldc", c_int64)]


class GroupGemmArgs(Structure):
    _fields_ = [("problems", POINTER(GroupProblem)), ("num_problems", c_int32),
                ("ab_dtype", c_int32), ("c_dtype", c_int32), ("b_layout", c_int32)]


class BlockScaledGemmArgs(Structure):
    _fields_ = [
        ("a", c_void_p), ("b", c_void_p), ("sfa", c_void_p), ("sfb", c_void_p), ("c", c_void_p),
        ("m", c_int64), ("n", c_int64), ("k", c_int64), ("batch", c_int64),
        ("lda", c_int64), ("ldb", c_int64), ("ldc", c_int64),
        ("stride_a", c_int64), ("stride_b", c_int64), ("stride_c", c_int64),
        ("sf_k_atoms", c_int64), ("stride_sfa", c_int64), ("stride_sfb", c_int64),
        ("ab_dtype", c_int32), ("c_dtype", c_int32), ("epilogue", c_int32), ("alpha", c_float),
        ("alpha_a", c_void_p), ("alpha_b", c_void_p),
        ("max_ctas", c_int32),
        ("tile_group", c_void_p), ("num_row_tiles", c_void_p),
        ("row_map", c_void_p), ("row_scale", c_void_p), ("c_rows", c_int64),
        ("tile_rows", c_int32),
        ("c_sf", c_void_p), ("c_sf_k_atoms", c_int64),
        ("config", POINTER(GemmConfig)),
        ("c_scale", c_void_p),
        ("c_peers", POINTER(c_void_p)), ("num_c_peers", c_int32), ("c_peer_rows", c_int64),
        ("skip_rows_begin", c_int64), ("skip_rows_count", c_int64),
    ]


class QuantizeArgs(Structure):
    _fields_ = [
        ("x", c_void_p), ("q", c_void_p), ("sf_logical", c_void_p), ("sf_swizzled", c_void_p),
        ("tensor_scale", c_void_p), ("scratch", c_void_p),
        ("rows", c_int64), ("k", c_int64), ("ldx", c_int64), ("ldq", c_int64),
        ("sf_k_atoms", c_int64),
        ("x_dtype", c_int32), ("q_dtype", c_int32),
        ("gather_index", c_void_p), ("gather_divisor", c_int32), ("tile_m", c_int32),
        ("src_rows", c_int64), ("live_blocks", c_void_p),
        ("tensor_scale_given", c_int32),
    ]


class MoeAlignArgs(Structure):
    _fields_ = [
        ("topk_ids", c_void_p), ("sorted_token_ids", c_void_p), ("sorted_expert_ids", c_void_p),
        ("num_blocks", c_void_p), ("workspace", c_void_p), ("workspace_bytes", c_int64),
        ("num_replicas", c_int64), ("capacity", c_int64), ("block_capacity", c_int64),
        ("num_experts", c_int32), ("tile_m", c_int32), ("ids_are_int64", c_int32),
    ]


class MoeSparseArgs(Structure):
    _fields_ = [
        ("hidden_states", c_void_p), ("w1", c_void_p), ("w2", c_void_p), ("topk_ids", c_void_p),
        ("topk_weights", c_void_p), ("act", c_void_p), ("per_replica", c_void_p),
        ("tokens", c_int64), ("hidden", c_int64), ("intermediate", c_int64),
        ("hidden_stride", c_int64), ("w1_stride_e", c_int64), ("w1_ld", c_int64),
        ("w2_stride_e", c_int64), ("w2_ld", c_int64),
        ("topk", c_int32), ("num_experts", c_int32), ("ids_are_int64", c_int32), ("dtype", c_int32),
    ]


class MoeEpCountArgs(Structure):
    _fields_ = [
        ("topk_ids", c_void_p), ("num_replicas", c_int64), ("ids_are_int64", c_int32),
        ("num_experts", c_int32), ("world", c_int32), ("rank", c_int32),
        ("scratch", c_void_p), ("hist_peers", POINTER(c_void_p)),
    ]


class MoeEpPlanArgs(Structure):
    _fields_ = [
        ("hist", c_void_p), ("world", c_int32), ("rank", c_int32), ("num_experts", c_int32),
        ("tile_rows", c_int32), ("capacity_rows", c_int64),
        ("first_row", c_void_p), ("cursor", c_void_p), ("tile_group", c_void_p),
        ("num_row_tiles", c_void_p), ("meta", c_void_p),
    ]


class MoeEpDispatchArgs(Structure):
    _fields_ = [
        ("topk_ids", c_void_p), ("weights", c_void_p), ("num_replicas", c_int64),
        ("topk", c_int32), ("ids_are_int64", c_int32), ("num_experts", c_int32),
        ("world", c_int32), ("rank", c_int32),
        ("src", c_void_p), ("src_stride_bytes", c_int64), ("row_bytes", c_int64),
        ("aux", c_void_p), ("aux_stride_bytes", c_int64), ("aux_bytes", c_int64),
        ("first_row", c_void_p), ("cursor", c_void_p), ("capacity_rows", c_int64),
        ("row_peers", POINTER(c_void_p)), ("aux_peers", POINTER(c_void_p)),
        ("meta_peers", POINTER(c_void_p)), ("weight_peers", POINTER(c_void_p)),
    ]


class FmhaArgs(Structure):
    _fields_ = [
        ("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("out", c_void_p),
        ("batch", c_int64), ("heads_q", c_int64), ("heads_kv", c_int64),
        ("seq_q", c_int64), ("seq_kv", c_int64),
        ("q_stride_b", c_int64), ("q_stride_h", c_int64), ("q_stride_s", c_int64),
        ("k_stride_b", c_int64), ("k_stride_h", c_int64), ("k_stride_s", c_int64),
        ("v_stride_b", c_int64), ("v_stride_h", c_int64), ("v_stride_s", c_int64),
        ("o_stride_b", c_int64), ("o_stride_h", c_int64), ("o_stride_s", c_int64),
        ("input_pos", c_int64),
        ("head_dim", c_int32), ("dtype", c_int32), ("query_group_size", c_int32),
        ("causal", c_int32), ("qk_scale", c_float),
        ("workspace", c_void_p), ("workspace_bytes", c_int64),
    ]


class PeerGatherArgs(Structure):
    _fields_ = [
        ("shards", POINTER(c_void_p)), ("dst", c_void_p),
        ("rows", c_int64), ("row_bytes", c_int64),
        ("src_stride_bytes", c_int64), ("dst_stride_bytes", c_int64),
        ("world", c_int32), ("rank", c_int32), ("round_tf32", c_int32),
    ]


# name -> (restype, argtypes); every symbol include/b200k.h declares
SIGNATURES = {
    "b200k_version": (c_char_p, []),
    "b200k_last_error": (c_char_p, []),
    "b200k_sm_count": (c_int, []),
    "b200k_device_status": (c_int, [POINTER(c_int), POINTER(c_int)]),
    "b200k_tensor_map_cache_stats": (c_int, [POINTER(ctypes.c_uint64), POINTER(ctypes.c_uint64),
                                             POINTER(ctypes.c_uint64)]),
    "b200k_gemm": (c_int, [POINTER(GemmArgs), c_void_p]),
    "b200k_gemm_workspace_bytes": (c_int64, [POINTER(GemmArgs)]),
    "b200k_group_gemm_max_problems": (c_int32, []),
    "b200k_group_gemm": (c_int, [POINTER(GroupGemmArgs), c_void_p]),
    "b200k_block_scaled_gemm": (c_int, [POINTER(BlockScaledGemmArgs), c_void_p]),
    "b200k_mxfp8_quantize": (c_int, [POINTER(QuantizeArgs), c_void_p]),
    "b200k_nvfp4_quantize": (c_int, [POINTER(QuantizeArgs), c_void_p]),
    "b200k_nvfp4_quantize_noalloc": (c_int, [POINTER(QuantizeArgs), c_void_p]),
    "b200k_moe_align_workspace_bytes": (c_int64, [c_int64, c_int32]),
    "b200k_moe_align": (c_int, [POINTER(MoeAlignArgs), c_void_p]),
    "b200k_gather_rows": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int32, c_void_p,
                                  c_int32, c_int64, c_void_p, c_int64, c_void_p]),
    "b200k_gather_rows_by_source": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int32, c_void_p,
                                            c_int32, c_int64, c_void_p, c_int64, c_void_p, c_void_p]),
    "b200k_silu_and_mul": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64, c_int32,
                                   c_void_p]),
    "b200k_topk_sum": (c_int, [c_void_p, c_void_p, c_int64, c_int32, c_int64, c_void_p, c_int32, c_void_p,
                               c_int32, c_int32, c_void_p]),
    "b200k_peer_gather": (c_int, [POINTER(PeerGatherArgs), c_void_p]),
    "b200k_peer_scalar_expand": (c_int, [POINTER(c_void_p), c_int32, c_int64, c_void_p, c_void_p]),
    "b200k_peer_gather_batch": (c_int, [POINTER(PeerGatherArgs), c_int32, POINTER(c_void_p), c_int64, c_void_p,
                                        c_void_p]),
    "b200k_moe_sparse": (c_int, [POINTER(MoeSparseArgs), c_void_p]),
    "b200k_moe_ep_capacity_rows": (c_int64, [c_int64, c_int32, c_int32, c_int32]),
    "b200k_moe_ep_count": (c_int, [POINTER(MoeEpCountArgs), c_void_p]),
    "b200k_moe_ep_plan": (c_int, [POINTER(MoeEpPlanArgs), c_void_p]),
    "b200k_moe_ep_dispatch": (c_int, [POINTER(MoeEpDispatchArgs), c_void_p]),
    "b200k_peer_barrier": (c_int, [POINTER(c_void_p), c_int32, c_int32, c_void_p, c_int32, c_void_p]),
    "b200k_fmha_fwd": (c_int, [POINTER(FmhaArgs), c_void_p]),
    "b200k_fmha_workspace_bytes": (c_int64, [POINTER(FmhaArgs)]),
    "b200k_sf_swizzle": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64, c_int32,
                                 c_void_p, c_int32, c_void_p]),
}

_lib = None


def lib() -> ctypes.CDLL:
    """Loads the shared library once; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python cutile-python_b200/build.py` "
                "(b200k has no fallback path)")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def check(code: int) -> None:
    if code < 0:
        raise B200KError(code, lib().b200k_last_error().decode("utf-8", "replace"))


def stream_ptr(device: torch.device) -> int:
    """Raw handle of torch's current stream on `device`."""
    return torch._C._cuda_getCurrentRawStream(device.index if device.index is not None
                                              else torch.cuda.current_device())


class LaunchCache:
    """Remembered launches of one entry point: argument struct and everything it points at,
    keyed by what the caller passed (pointers, shapes, strides, dtypes, scalars).  A call that
    repeats an earlier one - the steady state of any model or benchmark loop - then costs a
    dictionary lookup and the C call, not a re-derivation of layouts and a struct refill.  This
    is the wrapper-side half of what the reference keeps per kernel in its launch path (hash
    lookup + cuLaunchKernelEx, cext/tile_kernel.cpp:3816-3844); the library-side half is the
    tensor-map cache.  An entry is only a function of its key, so it cannot go stale."""

    def __init__(self, entry_name: str, limit: int = 4096):
        self.entry_name, self.limit = entry_name, limit
        self.plans: dict = {}
        self.fn = None

    def get(self, key):
        return self.plans.get(key)

    def put(self, key, args, keep=()):
        if len(self.plans) >= self.limit:
            self.plans.clear()
        plan = (ctypes.byref(args), args, keep)
        self.plans[key] = plan
        return plan

    def launch(self, plan, device: torch.device) -> None:
        if self.fn is None:
            self.fn = getattr(lib(), self.entry_name)
        index = device.index
        if index is None or torch.cuda.current_device() == index:
            code = self.fn(plan[0], torch._C._cuda_getCurrentRawStream(
                index if index is not None else torch.cuda.current_device()))
        else:
            with torch.cuda.device(device):
                code = self.fn(plan[0], torch._C._cuda_getCurrentRawStream(index))
        if code < 0:
            check(code)


def device_status() -> tuple[int, int]:
    """(code, info) of the current device's status word; synchronise the stream first."""
    code, info = c_int(0), c_int(0)
    check(lib().b200k_device_status(ctypes.byref(code), ctypes.byref(info)))
    return code.value, info.value


def tensor_map_cache_stats() -> tuple[int, int, int]:
    """(hits, misses, entries) of the library's tensor-map cache."""
    h, m, e = ctypes.c_uint64(0), ctypes.c_uint64(0), ctypes.c_uint64(0)
    check(lib().b200k_tensor_map_cache_stats(ctypes.byref(h), ctypes.byref(m), ctypes.byref(e)))
    return h.value, m.value, e.value


def raise_on_device_error() -> None:
    code, info = device_status()
    if code != 0:
        raise B200KError(code, f"device-side wait gave up (role {(info >> 8) & 0xff}, "
                               f"detail {(info >> 16) & 0xffff})")


_TORCH_TO_ENUM = {
    torch.float16: F16,
    torch.bfloat16: BF16,
    torch.float32: F32,
    torch.float8_e4m3fn: E4M3,
    torch.float8_e5m2: E5M2,
}


def dtype_enum(dt: torch.dtype) -> int:
    try:
        return _TORCH_TO_ENUM[dt]
    except KeyError:
        raise TypeError(f"unsupported dtype {dt}") from None


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()
