"""Dense matmul entry points with the signatures of the reference's samples.

cutile_matmul            samples/MatMul.py:179-251
bmm                      samples/BatchMatMul.py:53-92
cutile_persistent_matmul test/bench_matmul.py:396-410 (bench form, output passed in)
cutile_batch_matmul      test/bench_matmul.py:323-329 (bench form)
cutile_group_matmul      the list-of-problems form of test/kernels/group_gemm.py:10-38

All of them run the tcgen05 GEMM behind ``b200k_gemm``; tile sizes are fixed by the
kernel (128 x 256 x one 128-byte K atom), so the reference's tile-size choice by dtype
has no counterpart here.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib, tune


def _aligned(t: torch.Tensor, ld: int) -> bool:
    return (ld * t.element_size()) % 16 == 0 and t.data_ptr() % 16 == 0


def _pad_last(t: torch.Tensor) -> torch.Tensor:
    """Copies ``t`` (..., R, C) into a buffer whose rows start on 16-byte boundaries.
    TMA cannot address rows at other pitches; the logical shape is unchanged."""
    per = 16 // t.element_size()
    cols = t.shape[-1]
    padded = (cols + per - 1) // per * per
    buf = torch.zeros(*t.shape[:-1], padded, dtype=t.dtype, device=t.device)
    buf[..., :cols].copy_(t)
    return buf[..., :cols]


_GEMM_LAUNCHES = _lib.LaunchCache("b200k_gemm")


def _gemm(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, *, alpha: float = 1.0,
          max_ctas: int = 0, skip_rows: tuple[int, int] = (0, 0)) -> torch.Tensor:
    """a: (B, M, K) or (M, K); b: (B, K, N) or (K, N) as a view; c likewise (M, N).
    ``skip_rows`` = (first, count): rows of a / c left out of the product (whole 256-row tiles,
    plain 2-D problems)."""
    key = None
    if not tune.in_use():
        key = (a.data_ptr(), b.data_ptr(), c.data_ptr(), a.shape, a.stride(), b.shape, b.stride(),
               c.stride(), a.dtype, b.dtype, c.dtype, alpha, max_ctas, skip_rows)
        plan = _GEMM_LAUNCHES.get(key)
        if plan is not None:
            _GEMM_LAUNCHES.launch(plan, c.device)
            return c
    copied = False
    batched = a.dim() == 3
    if not batched:
        a3, b3, c3 = a.unsqueeze(0), b.unsqueeze(0), c.unsqueeze(0)
    else:
        a3, b3, c3 = a, b, c
    nb, m, k = a3.shape
    n = b3.shape[2]
    if a3.dtype != b3.dtype:
        raise TypeError(f"operand dtypes differ: {a3.dtype} vs {b3.dtype}")

    # A must be K-contiguous
    if a3.stride(2) != 1 or not _aligned(a3, a3.stride(1)) or (nb > 1 and (a3.stride(0) * a3.element_size()) % 16):
        a3, copied = _pad_last(a3), True
    # B: (K, N) N-contiguous, or a transposed view of an (N, K) K-contiguous tensor.
    def rows_ok(t):
        return (t.stride(2) == 1 and _aligned(t, t.stride(1))
                and (nb == 1 or (t.stride(0) * t.element_size()) % 16 == 0))

    is_kn, is_nk = b3.stride(2) == 1, b3.stride(1) == 1
    if is_nk and (not is_kn or n == 1):
        layout = _lib.B_NK
        bt = b3.transpose(1, 2)
        if not rows_ok(bt):
            bt, copied = _pad_last(bt), True
        b3, ldb = bt, bt.stride(1)
    else:
        layout = _lib.B_KN
        if not rows_ok(b3):
            b3, copied = _pad_last(b3), True
        ldb = b3.stride(1)
    if c3.stride(2) != 1:
        raise ValueError("output must be row-major")

    args = _lib.GemmArgs()
    args.a, args.b, args.c = a3.data_ptr(), b3.data_ptr(), c3.data_ptr()
    args.m, args.n, args.k, args.batch = m, n, k, nb
    args.lda, args.ldb, args.ldc = a3.stride(1), ldb, c3.stride(1)
    args.stride_a, args.stride_b, args.stride_c = a3.stride(0), b3.stride(0), c3.stride(0)
    args.ab_dtype = _lib.dtype_enum(a3.dtype)
    args.c_dtype = _lib.dtype_enum(c3.dtype)
    args.b_layout = layout
    args.epilogue = _lib.EPI_STORE
    args.alpha = alpha
    args.max_ctas = max_ctas
    args.skip_rows_begin, args.skip_rows_count = skip_rows
    cfg = tune.config_for("gemm", args.ab_dtype, args.c_dtype, layout, m, n, k, nb)
    # plain dense GEMMs launch programmatically: a chain of short ones on one stream then runs
    # without launch gaps (2048 cubed fp16: 20.2 -> 18.0 us per call, the CUDA-graph figure)
    c_cfg = cfg.to_c() if cfg is not None else _lib.GemmConfig()
    c_cfg.programmatic_launch = 1
    args.config = ctypes.pointer(c_cfg)         # kept alive with the remembered launch
    with torch.cuda.device(a.device):
        # a few output tiles with a long K: split-K over the idle SMs needs fp32 scratch
        workspace = None
        if skip_rows[1] == 0 and ((cfg is not None and cfg.split_k > 1) or (
                -(-m // 128) * -(-n // 256) * nb * 4 <= 256 and k * a3.element_size() >= 1024)):
            ws_bytes = _lib.lib().b200k_gemm_workspace_bytes(ctypes.byref(args))
            if ws_bytes > 0:
                workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=a.device)
                args.workspace, args.workspace_bytes = workspace.data_ptr(), ws_bytes
        _lib.check(_lib.lib().b200k_gemm(ctypes.byref(args), _lib.stream_ptr(a.device)))
    # remembered for the next identical call, unless this one needed a repacked operand (whose
    # contents are a copy) or scratch memory (which concurrent streams must not share)
    if key is not None and not copied and workspace is None:
        _GEMM_LAUNCHES.put(key, args, keep=(c_cfg,))
    return c


def _validate(A: torch.Tensor, B: torch.Tensor) -> None:
    # same checks and messages as samples/MatMul.py:201-207
    if A.shape[-1] != B.shape[-2]:
        raise ValueError(f"Incompatible matrices: K dimension of A ({A.shape[-1]}) "
                         f"must match K dimension of B ({B.shape[-2]})")
    if A.device != B.device:
        raise ValueError("Input tensors must be on the same device.")
    if not A.is_cuda or not B.is_cuda:
        raise ValueError("Input tensors must be on a CUDA device.")


def _round_tf32(t: torch.Tensor) -> torch.Tensor:
    """fp32 -> nearest tf32 value (ties away from zero), kept in fp32; same strides."""
    bits = t.view(torch.int32)
    return ((bits + 0x1000) & ~0x1FFF).view(torch.float32)


def cutile_matmul(A: torch.Tensor, B: torch.Tensor, persistent: bool = False,
                  C: torch.Tensor | None = None, *, round_tf32: bool = False) -> torch.Tensor:
    """C = A @ B with fp32 accumulation; C has A's dtype and shape (M, N).

    fp32 operands are multiplied as tf32, like the reference kernel
    (test/kernels/matmul.py:74).  The tensor core reads the fp32 words as they are and
    ignores the low 13 mantissa bits, i.e. it TRUNCATES to tf32, where the reference's
    ``astype(tf32)`` rounds to nearest: each operand value is then up to 2^-10 (instead of
    2^-11) off in relative terms, always toward zero, so same-sign data (the sample's
    uniform [0, 1) inputs) carries a one-sided relative bias of about 2^-11 per operand.
    ``round_tf32=True`` rounds both operands to the nearest tf32 value first (one extra pass
    over A and B), which is what ``cutile_gather_matmul`` always does.  ``persistent`` is
    accepted for signature compatibility; the kernel is always persistent (one CTA per SM).
    """
    _validate(A, B)
    if A.dim() != 2 or B.dim() != 2:
        raise ValueError("cutile_matmul expects 2-D operands")
    m, n = A.shape[0], B.shape[1]
    if C is None:
        if A.element_size() == 1:
            raise TypeError("fp8 operands need an explicit fp16/bf16/fp32 output: pass C=")
        C = torch.empty((m, n), device=A.device, dtype=A.dtype)
    if m == 0 or n == 0:
        return C
    if A.shape[1] == 0:
        return C.zero_()
    if round_tf32 and A.dtype == torch.float32:
        A, B = _round_tf32(A), _round_tf32(B)
    return _gemm(A, B, C)


def cutile_persistent_matmul(A: torch.Tensor, B: torch.Tensor, C: torch.Tensor) -> torch.Tensor:
    return cutile_matmul(A, B, persistent=True, C=C)


def bmm(a: torch.Tensor, b: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """Batched C[i] = a[i] @ b[i]; a (Batch, M, K), b (Batch, K, N).

    fp16/bf16 operands give an output of the same dtype; fp8 operands accumulate in
    fp32 and default to an fp32 output (samples/BatchMatMul.py:72-81).
    """
    if a.dim() != 3 or b.dim() != 3:
        raise ValueError("bmm expects 3-D operands")
    if a.shape[0] != b.shape[0]:
        raise ValueError(f"Batch dimensions differ: {a.shape[0]} vs {b.shape[0]}")
    _validate(a, b)
    if out_dtype is None:
        out_dtype = torch.float32 if a.element_size() == 1 else a.dtype
    nb, m, _ = a.shape
    n = b.shape[2]
    c = torch.empty((nb, m, n), device=a.device, dtype=out_dtype)
    if nb == 0 or m == 0 or n == 0:
        return c
    if a.shape[2] == 0:
        return c.zero_()
    return _gemm(a, b, c)


def cutile_batch_matmul(bs: int, A: torch.Tensor, B: torch.Tensor, C: torch.Tensor) -> torch.Tensor:
    if A.shape[0] != bs:
        raise ValueError("batch size does not match A")
    _validate(A, B)
    return _gemm(A, B, C)


def cutile_group_matmul(As, Bs, Cs=None):
    """Cs[g] = As[g] @ Bs[g] for a list of independent problems of any shapes, in ONE persistent
    launch that walks the tiles of all problems (grouped_matmul_kernel,
    test/kernels/group_gemm.py:10-38).  The problems of a list share dtypes; lists that mix the
    layout of B (row-major (K, N) and transposed views of (N, K) tensors), or hold more problems
    than one launch takes, become one launch per layout and chunk.  Operands whose rows do not
    start on 16-byte boundaries (TMA's rule) are repacked first."""
    if len(As) != len(Bs) or (Cs is not None and len(Cs) != len(As)):
        raise ValueError("As, Bs and Cs must list the same number of problems")
    if Cs is None:
        Cs = [torch.empty((a.shape[0], b.shape[1]), device=a.device, dtype=a.dtype) for a, b in zip(As, Bs)]
    if not As:
        return Cs
    dev, ab_dtype, c_dtype = As[0].device, As[0].dtype, Cs[0].dtype
    by_layout: dict[int, list] = {_lib.B_KN: [], _lib.B_NK: []}
    keep = []
    for a, b, c in zip(As, Bs, Cs):
        _validate(a, b)
        if a.dim() != 2 or b.dim() != 2:
            raise ValueError("cutile_group_matmul expects 2-D operands")
        if c.shape != (a.shape[0], b.shape[1]):
            raise ValueError("output shape does not match its problem")
        if a.dtype != ab_dtype or b.dtype != ab_dtype or c.dtype != c_dtype or a.device != dev:
            raise TypeError("all problems of a list share operand dtype, output dtype and device")
        if c.stride(1) != 1 and c.numel():
            raise ValueError("output must be row-major")
        m, k = a.shape
        n = b.shape[1]
        if m == 0 or n == 0:
            continue
        if k == 0:
            c.zero_()
            continue
        if a.stride(1) != 1 or not _aligned(a, a.stride(0)):
            a = _pad_last(a)
        if b.stride(0) == 1 and (b.stride(1) != 1 or n == 1):      # a transposed view of (N, K)
            layout, bt = _lib.B_NK, b.T
            if not _aligned(bt, bt.stride(0)):
                bt = _pad_last(bt)
            b, ldb = bt, bt.stride(0)
        else:
            layout = _lib.B_KN
            if b.stride(1) != 1 or not _aligned(b, b.stride(0)):
                b = _pad_last(b)
            ldb = b.stride(0)
        keep += [a, b]
        by_layout[layout].append(_lib.GroupProblem(a.data_ptr(), b.data_ptr(), c.data_ptr(), m, n, k,
                                                   a.stride(0), ldb, c.stride(0)))
    lib = _lib.lib()
    limit = lib.b200k_group_gemm_max_problems()
    with torch.cuda.device(dev):
        for layout, problems in by_layout.items():
            for lo in range(0, len(problems), limit):
                chunk = problems[lo:lo + limit]
                table = (_lib.GroupProblem * len(chunk))(*chunk)
                args = _lib.GroupGemmArgs(ctypes.cast(table, ctypes.POINTER(_lib.GroupProblem)), len(chunk),
                                          _lib.dtype_enum(ab_dtype), _lib.dtype_enum(c_dtype), layout)
                _lib.check(lib.b200k_group_gemm(ctypes.byref(args), _lib.stream_ptr(dev)))
    return Cs
