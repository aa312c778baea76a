"""Parity of the dense tcgen05 GEMM (through the C ABI) with the fp32 CPU oracle.

Shapes and tolerances follow the reference: samples/MatMul.py:268-330 (512x512x768 and the
ragged 1000x500x700), samples/BatchMatMul.py:128-163, test/test_mma.py:46-59 (per-dtype
tolerances), and the all-ones known answers of src/cuda/tile/_stub.py:2171-2193.
"""
import pytest
import torch

import b200k
import oracle

pytestmark = pytest.mark.gpu

# |err| <= atol + rtol * |ref|, fp32 accumulation over K <= 2048 of N(0,1) products
TOL = {
    torch.float16: dict(atol=2e-2, rtol=2e-2),
    torch.bfloat16: dict(atol=2e-2, rtol=2e-2),
    torch.float32: dict(atol=5e-2, rtol=1e-2),   # multiplied as tf32
}


def _rand(shape, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g).to(dtype)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("m,n,k", [(512, 512, 768), (1000, 500, 700), (128, 256, 64), (1, 1, 8),
                                   (130, 264, 72), (2048, 2048, 2048)])
def test_cutile_matmul_row_major_b(dtype, m, n, k, device_ok):
    a = _rand((m, k), dtype, 0)
    b = _rand((k, n), dtype, 1)
    c = b200k.cutile_matmul(a.cuda(), b.cuda())
    assert c.shape == (m, n) and c.dtype == dtype
    tol = dict(TOL[dtype])
    if dtype == torch.float32:
        # tf32 keeps 10 mantissa bits of each operand: the error of a K-term sum of N(0,1)
        # products grows like sqrt(K) * 2^-10
        tol["atol"] = max(tol["atol"], 6e-3 * k ** 0.5)
    torch.testing.assert_close(c.float().cpu(), oracle.matmul_ref(a, b), **tol)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_cutile_matmul_transposed_b_view(dtype, device_ok):
    a = _rand((300, 520), dtype, 2)
    b_nk = _rand((260, 520), dtype, 3)
    c = b200k.cutile_matmul(a.cuda(), b_nk.cuda().T, persistent=True)
    torch.testing.assert_close(c.float().cpu(), oracle.matmul_ref(a, b_nk.T), **TOL[dtype])


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("m,n,k,b_nk", [(256, 256, 4096, False),    # the reference's split-K bench shape
                                        (256, 256, 4096, True), (100, 300, 4104, False),
                                        (128, 512, 8192, True), (8, 8, 4096, False)])
def test_split_k_shapes(dtype, m, n, k, b_nk, device_ok):
    # few output tiles, long K: the library spreads K over the idle SMs (fp32 partials + a
    # reduction kernel); the result must not depend on that choice
    a = (_rand((m, k), dtype, 5) * 0.25).to(dtype)
    b = _rand((n, k), dtype, 6) if b_nk else _rand((k, n), dtype, 6)
    bd = b.cuda().T if b_nk else b.cuda()
    ref = oracle.matmul_ref(a, b.T if b_nk else b)
    c = b200k.cutile_matmul(a.cuda(), bd)
    tol = dict(TOL[dtype])
    tol["atol"] = max(tol["atol"], (2e-3 if dtype != torch.bfloat16 else 8e-3) * 0.25 * k ** 0.5)
    torch.testing.assert_close(c.float().cpu(), ref, **tol)
    import ctypes
    from b200k import _lib
    probe = _lib.GemmArgs()
    probe.m, probe.n, probe.k, probe.batch = m, n, k, 1
    probe.ab_dtype = _lib.dtype_enum(dtype)
    assert _lib.lib().b200k_gemm_workspace_bytes(ctypes.byref(probe)) > 0   # the split path ran
    # the same product on one CTA per tile, no workspace: same result within rounding
    c1 = torch.empty_like(c)
    args = _lib.GemmArgs()
    a_d = a.cuda()
    b_k = (b.cuda() if b_nk else b.cuda().T.contiguous())
    args.a, args.b, args.c = a_d.data_ptr(), b_k.data_ptr(), c1.data_ptr()
    args.m, args.n, args.k, args.batch = m, n, k, 1
    args.lda, args.ldb, args.ldc = k, k, n
    args.ab_dtype = args.c_dtype = _lib.dtype_enum(dtype)
    args.b_layout, args.epilogue, args.alpha = _lib.B_NK, _lib.EPI_STORE, 1.0
    if (k * a.element_size()) % 16 == 0:
        _lib.check(_lib.lib().b200k_gemm(ctypes.byref(args), _lib.stream_ptr(c.device)))
        torch.testing.assert_close(c1.float(), c.float(), **tol)


def test_split_k_batched(device_ok):
    a = _rand((3, 128, 4096), torch.float16, 8) * 0.25
    b = _rand((3, 4096, 256), torch.float16, 9)
    c = b200k.bmm(a.cuda(), b.cuda(), torch.float16)
    ref = torch.bmm(a.float(), b.float())
    torch.testing.assert_close(c.float().cpu(), ref, atol=5e-2, rtol=2e-2)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("bn", ["128", "256"])
@pytest.mark.parametrize("b_nk", [False, True])
@pytest.mark.parametrize("m,n,k", [(512, 640, 256), (1000, 500, 700), (2304, 1152, 192)])
@pytest.mark.parametrize("epilogue", ["coalesced", "direct"])
def test_pair_kernel_tile_widths_and_b_layouts(dtype, bn, b_nk, m, n, k, epilogue, device_ok, monkeypatch):
    # the CTA-pair kernel with 256 x 128 and 256 x 256 tiles, B stored (K, N) and (N, K), both
    # epilogue forms (stores straight from registers / through shared memory)
    monkeypatch.setenv("B200K_PAIR_BN", bn)
    monkeypatch.setenv("B200K_EPILOGUE", epilogue)
    a = _rand((m, k), dtype, 11)
    b = _rand((n, k), dtype, 12) if b_nk else _rand((k, n), dtype, 12)
    c = b200k.cutile_matmul(a.cuda(), b.cuda().T if b_nk else b.cuda())
    tol = dict(TOL[dtype])
    if dtype == torch.float32:
        tol["atol"] = max(tol["atol"], 6e-3 * k ** 0.5)
    torch.testing.assert_close(c.float().cpu(), oracle.matmul_ref(a, b.T if b_nk else b), **tol)


def test_pair_kernel_fp8_row_major_b(device_ok):
    g = torch.Generator().manual_seed(3)
    a = torch.randn(2, 384, 256, generator=g).to(torch.float8_e4m3fn)
    b = torch.randn(2, 256, 512, generator=g).to(torch.float8_e4m3fn)
    c = b200k.bmm(a.cuda(), b.cuda(), torch.float32)
    torch.testing.assert_close(c.cpu(), torch.bmm(a.float(), b.float()), atol=1e-3, rtol=1e-3)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("mnk", [[(4, 4, 8)], [(2, 4, 8), (8, 6, 8), (12, 16, 8)],
                                 [(300, 200, 64), (1024, 2048, 512), (8, 8, 4096), (64, 640, 72)]])
def test_group_matmul_list_of_problems(dtype, mnk, device_ok):
    # shapes of test/test_group_gemm.py (K raised to the 16-byte row pitch of fp16) and larger ones
    As = [_rand((m, k), dtype, 20 + i) for i, (m, n, k) in enumerate(mnk)]
    Bs = [_rand((k, n), dtype, 40 + i) for i, (m, n, k) in enumerate(mnk)]
    Cs = b200k.cutile_group_matmul([a.cuda() for a in As], [b.cuda() for b in Bs])
    for a, b, c, (m, n, k) in zip(As, Bs, Cs, mnk):
        tol = dict(TOL[dtype])
        if dtype == torch.float32:
            tol["atol"] = max(tol["atol"], 6e-3 * k ** 0.5)
        else:
            tol["atol"] = max(tol["atol"], 2e-3 * k ** 0.5)
        torch.testing.assert_close(c.float().cpu(), oracle.matmul_ref(a, b), **tol)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("mnk", [[(4, 4, 4)], [(2, 4, 4), (8, 6, 6), (12, 16, 8)]])
def test_group_matmul_reference_test_shapes(dtype, mnk, device_ok):
    # test/test_group_gemm.py:14-33 as they are: rows of 4 or 6 elements start off the 16-byte
    # boundaries TMA needs, so the wrapper repacks them; tolerances of that test
    As = [torch.rand(m, k, generator=torch.Generator().manual_seed(i)).to(dtype) for i, (m, n, k) in enumerate(mnk)]
    Bs = [torch.rand(k, n, generator=torch.Generator().manual_seed(9 + i)).to(dtype) for i, (m, n, k) in enumerate(mnk)]
    Cs = [torch.rand(m, n).to(dtype).cuda() for (m, n, k) in mnk]
    out = b200k.cutile_group_matmul([a.cuda() for a in As], [b.cuda() for b in Bs], Cs)
    tol = 5e-3 if dtype == torch.float32 else 1e-2      # fp32 operands multiply as (truncated) tf32 here
    for a, b, c, c_in in zip(As, Bs, out, Cs):
        assert c is c_in
        torch.testing.assert_close(c.float().cpu(), oracle.matmul_ref(a, b), atol=tol, rtol=tol)


def test_group_matmul_many_problems_mixed_layouts_and_empty_ones(device_ok):
    # more problems than one launch takes, B given both row-major and as transposed views, a
    # problem without rows and one without a reduction dimension
    g = torch.Generator().manual_seed(77)
    mnk = [(8 + 13 * i, 24 + 8 * (i % 7), 64 + 32 * (i % 5)) for i in range(60)] + [(0, 16, 32), (16, 24, 0)]
    As = [torch.randn(m, k, generator=g).bfloat16() for m, n, k in mnk]
    Bs = [torch.randn(k, n, generator=g).bfloat16() for m, n, k in mnk]
    dev_b = [b.cuda() if i % 3 else b.T.contiguous().cuda().T for i, b in enumerate(Bs)]
    Cs = b200k.cutile_group_matmul([a.cuda() for a in As], dev_b)
    for a, b, c, (m, n, k) in zip(As, Bs, Cs, mnk):
        assert c.shape == (m, n)
        if m and k:
            torch.testing.assert_close(c.float().cpu(), oracle.matmul_ref(a, b), atol=2e-3 * k ** 0.5 + 0.05, rtol=2e-2)
        elif m:
            assert float(c.abs().max()) == 0.0
    with pytest.raises(TypeError, match="share"):
        b200k.cutile_group_matmul([As[0].cuda(), As[1].cuda().half()], [Bs[0].cuda(), Bs[1].cuda().half()])


def test_all_ones_known_answer(device_ok):
    # mma of all-ones tiles: every output equals K
    a = torch.ones(128, 448, dtype=torch.float16, device="cuda")
    b = torch.ones(448, 256, dtype=torch.float16, device="cuda")
    assert torch.all(b200k.cutile_matmul(a, b) == 448.0)


def test_one_hot_rows_pick_columns(device_ok):
    # A one-hot in K selects rows of B exactly: catches any operand-layout mix-up
    k, n = 192, 320
    idx = torch.arange(256) % k
    a = torch.nn.functional.one_hot(idx, k).to(torch.float16)
    b = _rand((k, n), torch.float16, 4)
    c = b200k.cutile_matmul(a.cuda(), b.cuda())
    assert torch.equal(c.cpu(), b[idx])


def test_unaligned_leading_dimensions_are_repacked(device_ok):
    a = _rand((64, 100), torch.float16, 5)     # 200-byte rows
    b = _rand((100, 36), torch.float16, 6)     # 72-byte rows
    c = b200k.cutile_matmul(a.cuda(), b.cuda())
    torch.testing.assert_close(c.float().cpu(), oracle.matmul_ref(a, b), **TOL[torch.float16])


def test_empty_and_zero_k():
    a = torch.zeros(0, 64, dtype=torch.float16, device="cuda")
    b = torch.zeros(64, 32, dtype=torch.float16, device="cuda")
    assert b200k.cutile_matmul(a, b).shape == (0, 32)
    a = torch.zeros(16, 0, dtype=torch.float16, device="cuda")
    b = torch.zeros(0, 32, dtype=torch.float16, device="cuda")
    assert torch.all(b200k.cutile_matmul(a, b) == 0)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_bmm_half(dtype, device_ok):
    a = _rand((4, 512, 256), dtype, 7)
    b = _rand((4, 256, 1024), dtype, 8)
    c = b200k.bmm(a.cuda(), b.cuda(), dtype)
    assert c.shape == (4, 512, 1024)
    torch.testing.assert_close(c.float().cpu(), oracle.matmul_ref(a, b), **TOL[dtype])


@pytest.mark.parametrize("fp8", [torch.float8_e4m3fn, torch.float8_e5m2])
def test_bmm_fp8_fp32_out(fp8, device_ok):
    a = _rand((4, 512, 256), torch.float32, 9).to(fp8)
    b = _rand((4, 256, 1024), torch.float32, 10).to(fp8)
    c = b200k.bmm(a.cuda(), b.cuda(), torch.float32)
    # fp8 products are exact in fp32; only the summation order differs
    torch.testing.assert_close(c.cpu(), oracle.matmul_ref(a, b), atol=1e-3, rtol=1e-4)


def test_bench_forms_write_into_c(device_ok):
    a = _rand((256, 128), torch.bfloat16, 11).cuda()
    b = _rand((128, 256), torch.bfloat16, 12).cuda()
    c = torch.empty(256, 256, dtype=torch.bfloat16, device="cuda")
    assert b200k.cutile_persistent_matmul(a, b, c) is c
    torch.testing.assert_close(c.float().cpu(), oracle.matmul_ref(a, b), **TOL[torch.bfloat16])
    a3, b3 = a.unsqueeze(0).repeat(2, 1, 1), b.unsqueeze(0).repeat(2, 1, 1)
    c3 = torch.empty(2, 256, 256, dtype=torch.bfloat16, device="cuda")
    b200k.cutile_batch_matmul(2, a3, b3, c3)
    torch.testing.assert_close(c3[1].float().cpu(), oracle.matmul_ref(a, b), **TOL[torch.bfloat16])


def test_linearity_at_full_size(device_ok):
    # size-independent property at a bench-sized problem: (A1 + A2) B == A1 B + A2 B up to
    # one rounding of each output, and a sampled block against the oracle
    m = n = k = 4096
    g = torch.Generator(device="cuda").manual_seed(13)
    a1 = torch.randn(m, k, device="cuda", generator=g).half()
    a2 = torch.randn(m, k, device="cuda", generator=g).half()
    b = torch.randn(k, n, device="cuda", generator=g).half()
    c12 = b200k.cutile_matmul(a1 + a2, b).float()
    c1 = b200k.cutile_matmul(a1, b).float()
    c2 = b200k.cutile_matmul(a2, b).float()
    torch.testing.assert_close(c12, c1 + c2, atol=0.5, rtol=1e-2)
    rows = torch.tensor([0, 127, 128, 2049, 4095])
    ref = oracle.matmul_ref(a1[rows].cpu(), b.cpu())
    torch.testing.assert_close(c1[rows].cpu(), ref, **TOL[torch.float16])


def test_fp32_operands_truncate_to_tf32_unless_rounding_is_asked_for(device_ok):
    # same-sign data shows the difference: truncation biases every product low, rounding to
    # nearest does not; both stay within the tf32 error bound of the fp32 product
    g = torch.Generator().manual_seed(12)
    a = torch.rand(256, 1024, generator=g)
    b = torch.rand(1024, 384, generator=g)
    ref = oracle.matmul_ref(a, b)

    def tf32(t, nearest):
        bits = t.contiguous().view(torch.int32)
        return ((bits + 0x1000) & ~0x1FFF if nearest else bits & ~0x1FFF).view(torch.float32)

    plain = b200k.cutile_matmul(a.cuda(), b.cuda()).cpu()
    rounded = b200k.cutile_matmul(a.cuda(), b.cuda(), round_tf32=True).cpu()
    # each form equals the fp32 product of operands cut to tf32 its way, up to summation order
    torch.testing.assert_close(plain, oracle.matmul_ref(tf32(a, False), tf32(b, False)), rtol=2e-5, atol=0)
    torch.testing.assert_close(rounded, oracle.matmul_ref(tf32(a, True), tf32(b, True)), rtol=2e-5, atol=0)
    assert float(((plain - ref) / ref).mean()) < -2e-4           # one-sided
    assert abs(float(((rounded - ref) / ref).mean())) < 5e-5     # centred
    torch.testing.assert_close(plain, ref, rtol=2e-3, atol=0)
    # the gather form at a world of one rounds, like the reference's cast: same result as round_tf32
    gathered = b200k.cutile_gather_matmul(a.cuda(), b.cuda(), peers=[a.cuda()], rank=0).cpu()
    torch.testing.assert_close(gathered, rounded, rtol=2e-5, atol=0)
