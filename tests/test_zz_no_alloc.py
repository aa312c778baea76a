"""b200k_nvfp4_quantize_noalloc: the NVFP4 quantiser for callers that cannot allocate.

A host that embeds this library may be unable to call cudaMalloc at the point where it
quantises (it runs inside someone else's stream-ordered region, or the process's device
memory is fully handed out already).  For them the library keeps the quantiser's temporary
in a 64 KB array of its own image.  This test drives that entry point through the C ABI
with caller-owned inputs and outputs and requires bit-identical results to
b200k_nvfp4_quantize (the same tolerance the other quantiser tests use: exact bytes), on
two calls in a row with different data, so stale scratch contents would show.

Collected last on purpose (file name): a run that stops at the first failure has then
already run every other test.
"""
import ctypes

import pytest
import torch

from b200k import _lib

pytestmark = pytest.mark.gpu


def _run(entry_name, x, scratch, given_scale=None):
    rows, k = x.shape
    q = torch.full((rows, k // 2), 0xAA, dtype=torch.uint8, device=x.device)
    sf = torch.full((rows, k // 16), 0xAA, dtype=torch.uint8, device=x.device)
    ts = torch.full((1,), -1.0 if given_scale is None else given_scale, dtype=torch.float32,
                    device=x.device)
    a = _lib.QuantizeArgs()
    a.tensor_scale_given = 0 if given_scale is None else 1
    a.x, a.q, a.sf_logical, a.tensor_scale = x.data_ptr(), q.data_ptr(), sf.data_ptr(), ts.data_ptr()
    a.scratch = None if scratch is None else scratch.data_ptr()
    a.rows, a.k, a.ldx, a.ldq = rows, k, x.stride(0), k // 2
    a.x_dtype = _lib.dtype_enum(x.dtype)
    fn = getattr(_lib.lib(), entry_name)
    with torch.cuda.device(x.device):
        _lib.check(fn(ctypes.byref(a), _lib.stream_ptr(x.device)))
    torch.cuda.synchronize()
    return q, sf, ts


def test_noalloc_matches_allocating_entry_twice_in_a_row():
    g = torch.Generator().manual_seed(42)
    scratch = torch.empty(1, dtype=torch.int32, device="cuda")
    # the second tensor is 1000x smaller in magnitude and a different shape: a maximum left
    # over from the first call would change every scale of the second
    cases = [torch.randn(300, 1024, generator=g).bfloat16().cuda() * 8,
             (torch.randn(257, 96, generator=g) * 1e-3).cuda()]
    for x in cases:
        want = _run("b200k_nvfp4_quantize", x, scratch)
        got = _run("b200k_nvfp4_quantize_noalloc", x, None)
        for w, g_ in zip(want, got):
            assert torch.equal(w, g_)
        assert got[2].item() > 0


def test_noalloc_strided_rows_f16_and_slab_boundary_inside_a_row():
    g = torch.Generator().manual_seed(43)
    scratch = torch.empty(1, dtype=torch.int32, device="cuda")
    # 1000 x 96 fp32: the partial maxima are taken over 65536 elements each, so the first
    # boundary falls inside row 682; the largest value sits right behind it
    x32 = torch.randn(1000, 96, generator=g)
    x32[682, 70] = 37.5
    # rows of a wider allocation (row stride 1024 + 64 elements), fp16 and bf16
    wide16 = (torch.randn(300, 1088, generator=g) * 3).half().cuda()
    widebf = (torch.randn(130, 1088, generator=g) * 0.01).bfloat16().cuda()
    cases = [x32.cuda(), wide16[:, :1024], widebf[:, 32:1056]]
    assert cases[1].stride(0) == 1088 and not cases[2].is_contiguous()
    for x in cases:
        want = _run("b200k_nvfp4_quantize", x, scratch)
        got = _run("b200k_nvfp4_quantize_noalloc", x, None)
        for w, g_ in zip(want, got):
            assert torch.equal(w, g_)


def test_noalloc_keeps_a_scale_the_caller_gives():
    g = torch.Generator().manual_seed(44)
    x = torch.randn(200, 512, generator=g).bfloat16().cuda()
    scale = 0.00390625    # a calibrated scale, not amax / 2688: values beyond 10.5 saturate
    want = _run("b200k_nvfp4_quantize", x, None, given_scale=scale)
    got = _run("b200k_nvfp4_quantize_noalloc", x, None, given_scale=scale)
    for w, g_ in zip(want, got):
        assert torch.equal(w, g_)
    assert got[2].item() == scale       # read, never overwritten
    free = _run("b200k_nvfp4_quantize_noalloc", x, None)
    assert not torch.equal(free[1], got[1])   # the found scale differs, so do the block scales


def test_noalloc_rejects_tensors_beyond_its_scratch():
    a = _lib.QuantizeArgs()
    dummy = torch.empty(16, dtype=torch.uint8, device="cuda")
    a.x = a.q = dummy.data_ptr()
    a.rows, a.k = 1 << 20, (1 << 10) + 16          # just over 2^30 elements
    a.ldx, a.ldq = a.k, a.k // 2
    a.x_dtype = _lib.BF16
    rc = _lib.lib().b200k_nvfp4_quantize_noalloc(ctypes.byref(a), None)
    assert rc == _lib.UNSUPPORTED
    assert b"exceeds the built-in scratch" in _lib.lib().b200k_last_error()
