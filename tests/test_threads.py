"""Concurrent callers: the entry points are re-entrant (reference: launches are serialised
by the GIL or `g_launch_mutex`, cext/tile_kernel.cpp:4542-4544, and may come from any thread).
Several Python threads issue different problems on their own streams at the same time; every
result must match the oracle and no call may see another thread's error message."""
import threading

import pytest
import torch

import b200k
import oracle
from b200k import _lib

pytestmark = pytest.mark.gpu


def test_concurrent_threads_on_their_own_streams(device_ok):
    shapes = [(256, 384, 512), (512, 256, 1024), (128, 640, 256), (384, 384, 2048)]
    problems = []
    for i, (m, n, k) in enumerate(shapes):
        g = torch.Generator().manual_seed(20 + i)
        a = torch.randn(m, k, generator=g).half()
        b = torch.randn(k, n, generator=g).half()
        problems.append((a.cuda(), b.cuda(), oracle.matmul_ref(a, b)))
    torch.cuda.synchronize()
    errors = []

    def worker(idx):
        try:
            a, b, ref = problems[idx]
            stream = torch.cuda.Stream()
            with torch.cuda.stream(stream):
                for it in range(25):
                    c = b200k.cutile_matmul(a, b)
                    if it % 5 == 0:
                        # a failing call in this thread: its message is this thread's own
                        with pytest.raises(ValueError, match="Incompatible matrices"):
                            b200k.cutile_matmul(a, a)
                        args = _lib.GemmArgs()
                        args.m, args.n, args.k, args.batch = -(idx + 1), 1, 1, 1
                        assert _lib.lib().b200k_gemm(_lib.ctypes.byref(args), None) == _lib.INVALID_ARG
                        assert b"negative dimension" in _lib.lib().b200k_last_error()
                stream.synchronize()
            torch.testing.assert_close(c.float().cpu(), ref, atol=2e-2, rtol=2e-2)
        except BaseException as e:  # noqa: BLE001 - reported by the main thread
            errors.append((idx, repr(e)))

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(len(shapes))]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
