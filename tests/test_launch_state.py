"""Launch-path state of the library: the tensor-map cache and the bounded waits.

The reference keeps its per-kernel launch state (hoisted descriptors, a hash lookup per call)
in cext/tile_kernel.cpp:2884-2945, 3816-3844; here that state is a cache of encoded tensor
maps.  Device-side waits are bounded: a wait that runs out of its budget ends the kernel
normally and is reported through the status word, which this file shows with a budget of one
millisecond and an arrival that is deliberately never made (nothing faults or hangs).
"""
import ctypes

import pytest
import torch

import b200k
import oracle
from b200k import _lib

pytestmark = pytest.mark.gpu


def _dense_args(a, b_nk, c, cfg=None):
    args = _lib.GemmArgs()
    m, k = a.shape
    n = b_nk.shape[0]
    args.a, args.b, args.c = a.data_ptr(), b_nk.data_ptr(), c.data_ptr()
    args.m, args.n, args.k, args.batch = m, n, k, 1
    args.lda, args.ldb, args.ldc = a.stride(0), b_nk.stride(0), c.stride(0)
    args.ab_dtype, args.c_dtype = _lib.dtype_enum(a.dtype), _lib.dtype_enum(c.dtype)
    args.b_layout, args.epilogue, args.alpha = _lib.B_NK, _lib.EPI_STORE, 1.0
    if cfg is not None:
        args.config = ctypes.pointer(cfg)
    return args


def test_tensor_maps_are_encoded_once_per_operand(device_ok):
    g = torch.Generator().manual_seed(3)
    a = torch.randn(512, 256, generator=g).bfloat16().cuda()
    b = torch.randn(384, 256, generator=g).bfloat16().cuda()
    c = torch.empty(512, 384, dtype=torch.bfloat16, device="cuda")
    args = _dense_args(a, b, c)
    stream = _lib.stream_ptr(a.device)
    _lib.check(_lib.lib().b200k_gemm(ctypes.byref(args), stream))
    h0, m0, e0 = _lib.tensor_map_cache_stats()
    for _ in range(5):
        _lib.check(_lib.lib().b200k_gemm(ctypes.byref(args), stream))
    h1, m1, e1 = _lib.tensor_map_cache_stats()
    assert m1 == m0 and e1 == e0          # nothing new was encoded
    assert h1 - h0 >= 5 * 2               # A and B looked up on every call
    torch.testing.assert_close(c.float().cpu(), oracle.matmul_ref(a, b.T), atol=0.5, rtol=2e-2)
    # the same shapes at another address are another key, and still correct
    a2, b2 = a.clone(), b.clone() * 2
    c2 = torch.empty_like(c)
    _lib.check(_lib.lib().b200k_gemm(ctypes.byref(_dense_args(a2, b2, c2)), stream))
    assert _lib.tensor_map_cache_stats()[1] > m1
    torch.testing.assert_close(c2.float().cpu(), oracle.matmul_ref(a2, b2.T), atol=1.0, rtol=2e-2)


def test_a_wait_that_runs_out_returns_and_is_reported():
    # 256 x 256 x 256 bf16 on the CTA-pair kernel: one tile, four k-steps, both MMA issuers.
    g = torch.Generator().manual_seed(4)
    a = torch.randn(256, 256, generator=g).bfloat16().cuda()
    b = torch.randn(256, 256, generator=g).bfloat16().cuda()
    c = torch.zeros(256, 256, dtype=torch.bfloat16, device="cuda")
    stream = _lib.stream_ptr(a.device)
    torch.cuda.synchronize()
    assert b200k.device_status() == (0, 0)
    cfg = _lib.GemmConfig(kernel=2, tile_n=256, wait_budget_us=1000, withhold_arrival=1)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    rc = _lib.lib().b200k_gemm(ctypes.byref(_dense_args(a, b, c, cfg)), stream)
    stop.record()
    assert rc == _lib.OK                   # the launch itself is fine
    torch.cuda.synchronize()               # and the kernel comes back by itself
    # every role gives up within its own budget (waits are entered one after the other at most
    # a few deep), far from the two-second default
    assert start.elapsed_time(stop) < 100.0
    code, info = b200k.device_status()
    assert code == _lib.TIMEOUT
    role, detail = (info >> 8) & 0xff, (info >> 16) & 0xffff
    # whichever wait ran out first reports: the second MMA issuer waiting for the tile to be
    # opened (role 52, detail 300 + accumulator window) or an epilogue warp waiting for the
    # accumulator that therefore never completes (role 53, detail = window)
    assert (role, detail) in {(52, 300), (53, 0)}, (role, detail)
    assert b200k.device_status() == (0, 0)  # reading cleared it
    with pytest.raises(b200k.B200KError):
        # the helper the wrappers' callers use turns a set status word into an exception
        _lib.lib().b200k_gemm(ctypes.byref(_dense_args(a, b, c, cfg)), stream)
        torch.cuda.synchronize()
        b200k.raise_on_device_error()
    # the next ordinary call on the same context is correct
    c.zero_()
    _lib.check(_lib.lib().b200k_gemm(ctypes.byref(_dense_args(a, b, c)), stream))
    torch.cuda.synchronize()
    assert b200k.device_status() == (0, 0)
    torch.testing.assert_close(c.float().cpu(), oracle.matmul_ref(a, b.T), atol=0.5, rtol=2e-2)
    # a short budget alone changes nothing when every arrival is made
    c.zero_()
    ok_cfg = _lib.GemmConfig(kernel=2, tile_n=256, wait_budget_us=1000)
    _lib.check(_lib.lib().b200k_gemm(ctypes.byref(_dense_args(a, b, c, ok_cfg)), stream))
    torch.cuda.synchronize()
    assert b200k.device_status() == (0, 0)
    torch.testing.assert_close(c.float().cpu(), oracle.matmul_ref(a, b.T), atol=0.5, rtol=2e-2)
