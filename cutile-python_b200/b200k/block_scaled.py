"""Block-scaled (MXFP8 / NVFP4) matmul, the quantisers and the scale relayout.

cutile_block_scaled_matmul     samples/BlockScaledMatMul.py:229-297
cutile_swizzled_scaled_matmul  test/bench_matmul.py:443-452 (bench form, C passed in)
block_quantize                 test/kernels/kernel_utils.py:38-80
swizzle_32_4_4                 test/kernels/kernel_utils.py:83-98
nvfp4_quantize / cutile_nvfp4_matmul: the e2m1 + ue4m3/16 + fp32 tensor-scale format
the reference exposes only as an operand combination of ct.mma_scaled
(src/cuda/tile/_datatype.py:482-489, test/test_mma_scaled.py:149-183).
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib, tune

_E8M0 = torch.float8_e8m0fnu
_E8M0_ONE = 127  # byte of 2^0
_FP4X2 = getattr(torch, "float4_e2m1fn_x2", None)


def _as_u8(t: torch.Tensor) -> torch.Tensor:
    return t if t.dtype == torch.uint8 else t.view(torch.uint8)


def _cdiv(a: int, b: int) -> int:
    return (a + b - 1) // b


def swizzled_shape(rows: int, kblocks: int) -> tuple[int, int, int, int]:
    return (_cdiv(rows, 128), _cdiv(kblocks, 4), 32, 16)


def swizzle_32_4_4(scale: torch.Tensor, fill: int | None = None) -> torch.Tensor:
    """(M, K_s) scale tensor -> (ceil(M/128), ceil(K_s/4), 32, 16) atoms, same dtype.

    For M % 128 == 0 and K_s % 4 == 0 this is the reference's permutation
    (reshape(m0,4,32,k0,4).permute(0,3,2,1,4)); other shapes, which the reference's
    reshape rejects, are padded with ``fill`` (default: the byte of scale 1.0 for ue8m0,
    0 otherwise).
    """
    if scale.dim() != 2:
        raise ValueError("swizzle_32_4_4 expects a 2-D (M, K_s) tensor")
    if scale.element_size() != 1:
        raise TypeError("scale tensors are one byte per element")
    if not scale.is_cuda:
        raise ValueError("Input tensors must be on a CUDA device.")
    if fill is None:
        fill = _E8M0_ONE if scale.dtype == _E8M0 else 0
    rows, kblocks = scale.shape
    src = _as_u8(scale)
    if src.stride(1) != 1:
        src = src.contiguous()
    shape = swizzled_shape(rows, kblocks)
    out = torch.empty(shape, dtype=torch.uint8, device=scale.device)
    if rows and kblocks:
        with torch.cuda.device(scale.device):
            _lib.check(_lib.lib().b200k_sf_swizzle(src.data_ptr(), rows, kblocks, src.stride(0),
                                                   out.data_ptr(), shape[1], fill, None, 0,
                                                   _lib.stream_ptr(scale.device)))
    return out.view(scale.dtype)


def block_quantize(x: torch.Tensor, block_size: int = 32,
                   dtype: torch.dtype = torch.float8_e4m3fn, *, swizzled_scale: bool = False):
    """MXFP8 block quantisation along the last axis: returns (x_q, scale).

    Arithmetic is the reference's, evaluated in fp32 whatever the input dtype (the
    reference computes in the input dtype and its samples feed fp32): per block of 32,
    scale = 2^ceil(log2(max(amax/448, 1e-12))), x_q = (x/scale) rounded to ``dtype``,
    scale returned as float8_e8m0fnu of shape (..., K/32).  A last axis that is not a
    multiple of 32 is zero-padded, as in the reference.  With ``swizzled_scale`` the
    scale comes back in the swizzle_32_4_4 layout instead (2-D inputs only).
    """
    if block_size != 32:
        raise ValueError("MXFP8 uses blocks of 32 elements")
    if dtype not in (torch.float8_e4m3fn, torch.float8_e5m2):
        raise TypeError(f"unsupported quantised dtype {dtype}")
    if x.shape[-1] < block_size:
        raise ValueError(f"The requested block size {block_size} is larger than the inner most "
                         f"dimension of the input tensor {x.shape[-1]}")
    if not x.is_cuda:
        raise ValueError("Input tensors must be on a CUDA device.")
    if x.shape[-1] % block_size != 0:
        pad = (-x.shape[-1]) % block_size
        x = torch.nn.functional.pad(x, (0, pad), value=0)
    lead = x.shape[:-1]
    k = x.shape[-1]
    x2 = x.reshape(-1, k)
    if x2.stride(1) != 1:
        x2 = x2.contiguous()
    rows = x2.shape[0]
    kblocks = k // 32
    q = torch.empty((rows, k), dtype=torch.uint8, device=x.device)
    args = _lib.QuantizeArgs()
    args.x, args.q = x2.data_ptr(), q.data_ptr()
    args.rows, args.k, args.ldx, args.ldq = rows, k, x2.stride(0), k
    args.x_dtype = _lib.dtype_enum(x2.dtype)
    args.q_dtype = _lib.dtype_enum(dtype)
    if swizzled_scale:
        if x.dim() != 2:
            raise ValueError("swizzled scales need a 2-D input")
        shape = swizzled_shape(rows, kblocks)
        padded = rows % 128 != 0 or kblocks % 4 != 0
        sf = (torch.full(shape, _E8M0_ONE, dtype=torch.uint8, device=x.device) if padded
              else torch.empty(shape, dtype=torch.uint8, device=x.device))
        args.sf_swizzled = sf.data_ptr()
        args.sf_k_atoms = shape[1]
    else:
        sf = torch.empty((rows, kblocks), dtype=torch.uint8, device=x.device)
        args.sf_logical = sf.data_ptr()
    if rows:
        with torch.cuda.device(x.device):
            _lib.check(_lib.lib().b200k_mxfp8_quantize(ctypes.byref(args), _lib.stream_ptr(x.device)))
    x_q = q.view(dtype).reshape(*lead, k)
    scale = sf.view(_E8M0)
    if not swizzled_scale:
        scale = scale.reshape(*lead, kblocks)
    return x_q, scale


def nvfp4_quantize(x: torch.Tensor, *, swizzled_scale: bool = True,
                   tensor_scale: torch.Tensor | None = None):
    """bf16/fp16/fp32 (rows, K) -> (packed e2m1 (rows, K/2) uint8, ue4m3 block scales,
    fp32 tensor scale (1,) on the device).  The rule is stated in include/b200k.h.
    ``tensor_scale`` (one fp32 value on the device) given: it is used as the per-tensor scale
    and returned as is; x is then read once instead of twice."""
    if x.dim() != 2:
        raise ValueError("nvfp4_quantize expects a 2-D tensor")
    if not x.is_cuda:
        raise ValueError("Input tensors must be on a CUDA device.")
    rows, k = x.shape
    if k % 2:
        raise ValueError("K must be even")
    if x.stride(1) != 1:
        x = x.contiguous()
    kblocks = _cdiv(k, 16)
    q = torch.empty((rows, k // 2), dtype=torch.uint8, device=x.device)
    args = _lib.QuantizeArgs()
    if tensor_scale is not None:
        if tensor_scale.dtype != torch.float32 or tensor_scale.numel() != 1 or tensor_scale.device != x.device:
            raise ValueError("tensor_scale must be one fp32 value on the device of x")
        args.tensor_scale_given = 1
        scratch = None
    else:
        tensor_scale = torch.empty((1,), dtype=torch.float32, device=x.device)
        scratch = torch.empty((1,), dtype=torch.int32, device=x.device)
    args.x, args.q = x.data_ptr(), q.data_ptr()
    args.tensor_scale, args.scratch = tensor_scale.data_ptr(), _lib.ptr(scratch)
    args.rows, args.k, args.ldx, args.ldq = rows, k, x.stride(0), k // 2
    args.x_dtype = _lib.dtype_enum(x.dtype)
    if swizzled_scale:
        shape = swizzled_shape(rows, kblocks)
        padded = rows % 128 != 0 or kblocks % 4 != 0
        sf = (torch.zeros(shape, dtype=torch.uint8, device=x.device) if padded
              else torch.empty(shape, dtype=torch.uint8, device=x.device))
        args.sf_swizzled = sf.data_ptr()
        args.sf_k_atoms = shape[1]
    else:
        sf = torch.empty((rows, kblocks), dtype=torch.uint8, device=x.device)
        args.sf_logical = sf.data_ptr()
    if rows and k:
        with torch.cuda.device(x.device):
            _lib.check(_lib.lib().b200k_nvfp4_quantize(ctypes.byref(args), _lib.stream_ptr(x.device)))
    return q, sf.view(torch.float8_e4m3fn), tensor_scale


_SCALED_LAUNCHES = _lib.LaunchCache("b200k_block_scaled_gemm")


def _scaled_gemm(a_km, sfa, b_nk, sfb, c, *, fp4: bool, alpha: float = 1.0, alpha_a=None,
                 alpha_b=None, max_ctas: int = 0, row_scale=None, c_sf=None, c_scale=None,
                 skip_rows: tuple[int, int] = (0, 0)):
    """a_km (M, Kp), b_nk (N, Kp) K-contiguous byte tensors (Kp = K or K/2 bytes);
    sfa/sfb swizzled 4-D byte tensors.  ``skip_rows`` = (first, count): rows of A / C left out
    of the product (whole 256-row tiles)."""
    key = None
    if not tune.in_use():
        ptr = _lib.ptr
        key = (a_km.data_ptr(), b_nk.data_ptr(), c.data_ptr(), sfa.data_ptr(), sfb.data_ptr(), a_km.shape,
               a_km.stride(), b_nk.shape, b_nk.stride(), c.stride(), sfa.shape, sfb.shape, a_km.dtype, c.dtype,
               fp4, alpha, ptr(alpha_a), ptr(alpha_b), max_ctas, ptr(row_scale), ptr(c_sf),
               None if c_sf is None else c_sf.shape, ptr(c_scale), skip_rows)
        plan = _SCALED_LAUNCHES.get(key)
        if plan is not None:
            _SCALED_LAUNCHES.launch(plan, c.device)
            return c
    m, kp = a_km.shape
    n = b_nk.shape[0]
    k = kp * 2 if fp4 else kp
    args = _lib.BlockScaledGemmArgs()
    args.a, args.b, args.c = a_km.data_ptr(), b_nk.data_ptr(), c.data_ptr()
    args.sfa, args.sfb = sfa.data_ptr(), sfb.data_ptr()
    args.m, args.n, args.k, args.batch = m, n, k, 1
    mul = 2 if fp4 else 1
    args.lda, args.ldb, args.ldc = a_km.stride(0) * mul, b_nk.stride(0) * mul, c.stride(0)
    if c_scale is not None:                      # packed e2m1 output: leading dimension in elements
        args.ldc = c.stride(0) * 2
    args.sf_k_atoms = sfa.shape[1]
    if sfb.shape[1] != sfa.shape[1]:
        raise ValueError("A and B scale tensors disagree on K")
    args.ab_dtype = _lib.E2M1X2 if fp4 else _lib.dtype_enum(a_km.dtype)
    args.c_dtype = _lib.E2M1X2 if c_scale is not None else _lib.dtype_enum(c.dtype)
    args.c_scale = _lib.ptr(c_scale)
    args.epilogue = _lib.EPI_STORE
    args.alpha = alpha
    args.alpha_a = _lib.ptr(alpha_a)
    args.alpha_b = _lib.ptr(alpha_b)
    args.max_ctas = max_ctas
    args.row_scale = _lib.ptr(row_scale)
    args.skip_rows_begin, args.skip_rows_count = skip_rows
    if c_sf is not None:
        args.c_sf, args.c_sf_k_atoms = c_sf.data_ptr(), c_sf.shape[1]
    cfg = tune.config_for("block_scaled_gemm", args.ab_dtype, args.c_dtype, _lib.B_NK, m, n, k, 1)
    if cfg is not None:
        c_cfg = cfg.to_c()                      # kept alive until the call has returned
        args.config = ctypes.pointer(c_cfg)
    with torch.cuda.device(c.device):
        _lib.check(_lib.lib().b200k_block_scaled_gemm(ctypes.byref(args), _lib.stream_ptr(c.device)))
    if key is not None:
        _SCALED_LAUNCHES.put(key, args)
    return c


def _k_major(t: torch.Tensor) -> torch.Tensor:
    """Returns a (rows, K) tensor with unit K stride and 16-byte-aligned rows."""
    if t.stride(1) != 1 or (t.stride(0) * t.element_size()) % 16 or t.data_ptr() % 16:
        k = t.shape[1]
        per = 16
        buf = torch.zeros((t.shape[0], _cdiv(k, per) * per), dtype=t.dtype, device=t.device)
        buf[:, :k].copy_(t)
        return buf[:, :k]
    return t


def cutile_block_scaled_matmul(A: torch.Tensor, A_scale: torch.Tensor, B: torch.Tensor,
                               B_scale: torch.Tensor, *, out_dtype: torch.dtype = torch.float32,
                               C: torch.Tensor | None = None,
                               out_scale: torch.Tensor | None = None) -> torch.Tensor:
    """C = (A (.) A_scale) @ (B (.) B_scale) for fp8 operands with ue8m0 scales per 32
    elements of K.  A is (M, K); B is (K, N) (normally the transposed view of an (N, K)
    tensor); scales are 2-D logical ((M, K/32) and (K/32, N)) or 4-D swizzle_32_4_4
    tensors (B's swizzled over (N, K/32)).  The reference returns fp32; ``out_dtype``
    selects bf16/fp16 instead, and ``torch.float8_e4m3fn`` returns the pair (C quantised to
    MXFP8 in the epilogue, its swizzled scales): bit for bit
    ``block_quantize(C_bf16, 32, swizzled_scale=True)`` of the bf16 result.
    ``torch.float4_e2m1fn_x2`` with ``out_scale`` (fp32 device scalar, the result's per-tensor
    scale) returns the NVFP4 pair (packed codes (M, N/2) uint8, swizzled ue4m3 scales).
    """
    if A.shape[1] != B.shape[0]:
        raise ValueError(f"Incompatible matrices: K dimension of A ({A.shape[1]}) "
                         f"must match K dimension of B ({B.shape[0]})")
    if A.device != B.device or A.device != A_scale.device or A.device != B_scale.device:
        raise ValueError("Input tensors must be on the same device.")
    if not A.is_cuda or not A_scale.is_cuda or not B.is_cuda or not B_scale.is_cuda:
        raise ValueError("Input tensors must be on a CUDA device.")
    if A.dtype != B.dtype or A.dtype not in (torch.float8_e4m3fn, torch.float8_e5m2):
        raise TypeError("operands must both be float8_e4m3fn or float8_e5m2")
    m, k = A.shape
    n = B.shape[1]
    kblocks = _cdiv(k, 32)
    if A_scale.dim() == 2:
        if tuple(A_scale.shape) != (m, kblocks):
            raise ValueError(f"A_scale must be ({m}, {kblocks}), got {tuple(A_scale.shape)}")
        A_scale = swizzle_32_4_4(A_scale)
    if B_scale.dim() == 2:
        if tuple(B_scale.shape) != (kblocks, n):
            raise ValueError(f"B_scale must be ({kblocks}, {n}), got {tuple(B_scale.shape)}")
        B_scale = swizzle_32_4_4(B_scale.T)
    if tuple(A_scale.shape) != swizzled_shape(m, kblocks):
        raise ValueError(f"swizzled A_scale must be {swizzled_shape(m, kblocks)}")
    if tuple(B_scale.shape) != swizzled_shape(n, kblocks):
        raise ValueError(f"swizzled B_scale must be {swizzled_shape(n, kblocks)}")
    a_km = _k_major(A)
    b_nk = _k_major(B.T)
    if out_dtype == torch.float8_e4m3fn and C is None:
        # quantise in the epilogue: the product comes back as an MXFP8 operand
        # (e4m3 (M, N), swizzled ue8m0 scales over (M, N / 32)) for a GEMM chained on N
        if n % 32 or m == 0 or n == 0 or k == 0:
            raise ValueError("quantised output needs non-empty operands and N a multiple of 32")
        C = torch.empty((m, n), device=A.device, dtype=torch.float8_e4m3fn)
        shape = swizzled_shape(m, n // 32)
        C_sf = (torch.zeros if (m % 128 or (n // 32) % 4) else torch.empty)(shape, dtype=torch.uint8,
                                                                           device=A.device)
        _scaled_gemm(a_km, _as_u8(A_scale).contiguous(), b_nk, _as_u8(B_scale).contiguous(), C,
                     fp4=False, c_sf=C_sf)
        return C, C_sf.view(torch.float8_e8m0fnu)
    if out_dtype == torch.float4_e2m1fn_x2 and C is None:
        # the same with an NVFP4 result (packed e2m1 (M, N / 2), swizzled ue4m3 scales over
        # (M, N / 16)) under the per-tensor scale the caller provides
        if k == 0:
            raise ValueError("quantised output needs non-empty operands")
        C, C_sf = _nvfp4_output(m, n, out_scale, A.device)
        _scaled_gemm(a_km, _as_u8(A_scale).contiguous(), b_nk, _as_u8(B_scale).contiguous(), C,
                     fp4=False, c_sf=C_sf, c_scale=out_scale)
        return C, C_sf.view(torch.float8_e4m3fn)
    if C is None:
        C = torch.empty((m, n), device=A.device, dtype=out_dtype)
    if m == 0 or n == 0:
        return C
    if k == 0:
        return C.zero_()
    return _scaled_gemm(a_km, _as_u8(A_scale).contiguous(), b_nk, _as_u8(B_scale).contiguous(), C,
                        fp4=False)


def _nvfp4_output(m: int, n: int, out_scale: torch.Tensor, device):
    """Buffers of an NVFP4 result quantised in the epilogue: packed codes (M, N / 2), swizzled
    ue4m3 scales over (M, N / 16)."""
    if n % 32 or m == 0 or n == 0:
        raise ValueError("NVFP4 output needs non-empty operands and N a multiple of 32")
    if out_scale is None or out_scale.dtype != torch.float32 or out_scale.numel() != 1 or not out_scale.is_cuda:
        raise ValueError("NVFP4 output needs out_scale: one fp32 value on the device")
    c = torch.empty((m, n // 2), device=device, dtype=torch.uint8)
    shape = swizzled_shape(m, n // 16)
    c_sf = (torch.zeros if (m % 128 or (n // 16) % 4) else torch.empty)(shape, dtype=torch.uint8, device=device)
    return c, c_sf


def cutile_swizzled_scaled_matmul(A, A_s_swizzled, B, B_s_swizzled, C):
    return cutile_block_scaled_matmul(A, A_s_swizzled, B, B_s_swizzled, C=C)


def cutile_nvfp4_matmul(A_q: torch.Tensor, A_sf: torch.Tensor, A_ts: torch.Tensor,
                        B_q: torch.Tensor, B_sf: torch.Tensor, B_ts: torch.Tensor, *,
                        out_dtype: torch.dtype = torch.bfloat16,
                        C: torch.Tensor | None = None,
                        out_scale: torch.Tensor | None = None) -> torch.Tensor:
    """C = (A_ts * B_ts) * (A_q (.) A_sf) @ (B_q (.) B_sf)^T for NVFP4 operands as
    produced by nvfp4_quantize: A_q (M, K/2) and B_q (N, K/2) packed e2m1 bytes, both
    K-contiguous; *_sf swizzled ue4m3 scales; *_ts fp32 device scalars.
    ``out_dtype=torch.float4_e2m1fn_x2`` with ``out_scale`` (fp32 device scalar) quantises the
    result in the epilogue and returns (packed codes (M, N/2), swizzled ue4m3 scales): the
    next NVFP4 GEMM's A operand, bit for bit what quantising the bf16 result with that
    tensor scale gives."""
    a_km = _k_major(_as_u8(A_q))
    b_nk = _k_major(_as_u8(B_q))
    m, n = a_km.shape[0], b_nk.shape[0]
    if a_km.shape[1] != b_nk.shape[1]:
        raise ValueError("Incompatible matrices: K dimensions differ")
    if out_dtype == torch.float4_e2m1fn_x2 and C is None:
        C, C_sf = _nvfp4_output(m, n, out_scale, A_q.device)
        _scaled_gemm(a_km, _as_u8(A_sf).contiguous(), b_nk, _as_u8(B_sf).contiguous(), C,
                     fp4=True, alpha_a=A_ts, alpha_b=B_ts, c_sf=C_sf, c_scale=out_scale)
        return C, C_sf.view(torch.float8_e4m3fn)
    if C is None:
        C = torch.empty((m, n), device=A_q.device, dtype=out_dtype)
    if m == 0 or n == 0:
        return C
    return _scaled_gemm(a_km, _as_u8(A_sf).contiguous(), b_nk, _as_u8(B_sf).contiguous(), C,
                        fp4=True, alpha_a=A_ts, alpha_b=B_ts)
