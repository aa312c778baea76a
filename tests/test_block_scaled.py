"""Parity of the block-scaled GEMMs (MXFP8, NVFP4) with the de-quantised fp32 oracle.

Follows samples/BlockScaledMatMul.py:318-365 (512x512x768, logical and swizzled scales,
atol 1e-4 / rtol 1e-3 on fp32 output), test/test_mma_scaled.py:94-183 (reference
expression, fp4 nibble order, scale/block combinations), the docstring known answers of
src/cuda/tile/_stub.py:2248-2328 and the non-uniform-exponent case of
experimental/cuda-lang/test/examples/tk/test_mxfp8_b200_gemm.py:749-755.
"""
import numpy as np
import pytest
import torch

import b200k
import oracle

pytestmark = pytest.mark.gpu


def _quantised_pair(m, n, k, seed, pattern=None):
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(m, k, generator=g)
    b = torch.randn(n, k, generator=g)
    if pattern == "exponents":
        kb = -(-k // 32)
        ea = ((torch.arange(m)[:, None] + torch.arange(kb)[None, :]) % 5 - 2).float()
        eb = ((3 * torch.arange(n)[:, None] + torch.arange(kb)[None, :]) % 7 - 3).float()
        a = a * torch.exp2(ea).repeat_interleave(32, 1)[:, :k]
        b = b * torch.exp2(eb).repeat_interleave(32, 1)[:, :k]
    aq, sa = oracle.block_quantize_ref(a)
    bq, sb = oracle.block_quantize_ref(b)
    return aq, sa, bq, sb


@pytest.mark.parametrize("m,n,k", [(512, 512, 768), (128, 256, 128), (256, 512, 1024),
                                   (200, 300, 160), (1, 8, 32), (640, 1280, 4096)])
@pytest.mark.parametrize("pattern", [None, "exponents"])
def test_mxfp8_logical_scales(m, n, k, pattern, device_ok):
    aq, sa, bq, sb = _quantised_pair(m, n, k, 10 + m, pattern)
    ref = oracle.block_scaled_matmul_ref(aq, sa, bq, sb)
    c = b200k.cutile_block_scaled_matmul(aq.cuda(), sa.cuda(), bq.cuda().T, sb.cuda().T)
    assert c.dtype == torch.float32 and c.shape == (m, n)
    # products and scales are exact in fp32; only the summation order differs
    torch.testing.assert_close(c.cpu(), ref, atol=1e-4 * float(ref.abs().max()), rtol=1e-3)


def test_mxfp8_swizzled_scales_and_bench_form(device_ok):
    m = n = 512
    k = 768
    aq, sa, bq, sb = _quantised_pair(m, n, k, 3)
    ref = oracle.block_scaled_matmul_ref(aq, sa, bq, sb)
    sa_sw = oracle.swizzle_32_4_4_ref(sa).cuda()
    sb_sw = oracle.swizzle_32_4_4_ref(sb).cuda()
    c = b200k.cutile_block_scaled_matmul(aq.cuda(), sa_sw, bq.cuda().T, sb_sw)
    torch.testing.assert_close(c.cpu(), ref, atol=1e-4, rtol=1e-3)
    out = torch.empty(m, n, dtype=torch.float32, device="cuda")
    assert b200k.cutile_swizzled_scaled_matmul(aq.cuda(), sa_sw, bq.cuda().T, sb_sw, out) is out
    torch.testing.assert_close(out.cpu(), ref, atol=1e-4, rtol=1e-3)


def test_mxfp8_known_answers(device_ok):
    # ones with every scale = 2: each 32-block contributes 2 * 2 * 32 = 128
    for k, want in ((64, 256.0), (128, 512.0)):
        a = torch.ones(128, k, device="cuda").to(torch.float8_e4m3fn)
        s = torch.full((128, k // 32), 128, dtype=torch.uint8, device="cuda").view(torch.float8_e8m0fnu)
        c = b200k.cutile_block_scaled_matmul(a, s, a.T, s.T)
        assert torch.all(c == want)


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float16])
def test_mxfp8_half_outputs(out_dtype, device_ok):
    aq, sa, bq, sb = _quantised_pair(384, 512, 512, 5)
    ref = oracle.block_scaled_matmul_ref(aq, sa, bq, sb)
    c = b200k.cutile_block_scaled_matmul(aq.cuda(), sa.cuda(), bq.cuda().T, sb.cuda().T,
                                         out_dtype=out_dtype)
    torch.testing.assert_close(c.float().cpu(), ref, atol=2e-2, rtol=2e-2)


def test_mxfp8_e5m2(device_ok):
    g = torch.Generator().manual_seed(8)
    a = torch.randn(256, 256, generator=g)
    b = torch.randn(256, 256, generator=g)
    aq, sa = oracle.block_quantize_ref(a, 32, torch.float8_e5m2)
    bq, sb = oracle.block_quantize_ref(b, 32, torch.float8_e5m2)
    ref = oracle.block_scaled_matmul_ref(aq, sa, bq, sb)
    c = b200k.cutile_block_scaled_matmul(aq.cuda(), sa.cuda(), bq.cuda().T, sb.cuda().T)
    torch.testing.assert_close(c.cpu(), ref, atol=1e-3, rtol=1e-3)


def test_mxfp8_validation():
    a = torch.zeros(128, 64, device="cuda").to(torch.float8_e4m3fn)
    s = torch.zeros(128, 2, dtype=torch.uint8, device="cuda").view(torch.float8_e8m0fnu)
    with pytest.raises(ValueError, match="Incompatible matrices"):
        b200k.cutile_block_scaled_matmul(a, s, torch.zeros(32, 8, device="cuda").to(torch.float8_e4m3fn), s.T)
    with pytest.raises(ValueError, match="CUDA device"):
        b200k.cutile_block_scaled_matmul(a.cpu(), s.cpu(), a.T.cpu(), s.T.cpu())


def _t(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


@pytest.mark.parametrize("m,n,k", [(128, 256, 256), (512, 512, 768), (200, 300, 320), (256, 256, 64),
                                   (384, 1024, 2048)])
def test_nvfp4_matmul(m, n, k, device_ok):
    g = torch.Generator().manual_seed(m + k)
    a = torch.randn(m, k, generator=g)
    b = 0.02 * torch.randn(n, k, generator=g)
    aq, asf, ats = oracle.nvfp4_quantize_ref(a)
    bq, bsf, bts = oracle.nvfp4_quantize_ref(b)
    ref = oracle.nvfp4_matmul_ref(aq, asf, ats, bq, bsf, bts)
    asw = b200k.swizzle_32_4_4(_t(asf).view(torch.float8_e4m3fn))
    bsw = b200k.swizzle_32_4_4(_t(bsf).view(torch.float8_e4m3fn))
    c = b200k.cutile_nvfp4_matmul(_t(aq), asw, torch.tensor([float(ats)], device="cuda"),
                                  _t(bq), bsw, torch.tensor([float(bts)], device="cuda"),
                                  out_dtype=torch.float32)
    # against the de-quantised operands the kernel is exact up to fp32 summation order
    torch.testing.assert_close(c.cpu(), ref, atol=1e-4 * float(ref.abs().max()), rtol=1e-3)
    # against the unquantised product: the 5e-2 Frobenius bound applies to bf16 outputs of the
    # quantised pipeline; fp4 quantisation noise itself is ~13 % per operand pair
    assert oracle.rel_frobenius(c, a @ b.T) < 0.2


def test_nvfp4_end_to_end_bf16(device_ok):
    g = torch.Generator().manual_seed(2)
    a = torch.randn(256, 1024, generator=g).bfloat16()
    b = (0.02 * torch.randn(512, 1024, generator=g)).bfloat16()
    aq, asf, ats = b200k.nvfp4_quantize(a.cuda())
    bq, bsf, bts = b200k.nvfp4_quantize(b.cuda())
    c = b200k.cutile_nvfp4_matmul(aq, asf, ats, bq, bsf, bts)
    assert c.dtype == torch.bfloat16
    qa = oracle.nvfp4_quantize_ref(a)
    qb = oracle.nvfp4_quantize_ref(b)
    ref = oracle.nvfp4_matmul_ref(*qa, *qb)
    assert oracle.rel_frobenius(c, ref) < 5e-2
    torch.testing.assert_close(c.float().cpu(), ref, atol=2e-2 * float(ref.abs().max()), rtol=2e-2)


@pytest.mark.parametrize("operands", ["nvfp4", "mxfp8"])
@pytest.mark.parametrize("m,n,k", [(256, 256, 256), (384, 640, 512), (1000, 96, 192)])
def test_nvfp4_quantise_in_epilogue_equals_two_steps(operands, m, n, k, device_ok):
    # packed e2m1 + swizzled ue4m3 scales straight from the GEMM epilogue == quantising the bf16
    # result (oracle rule) with the same per-tensor scale
    g = torch.Generator().manual_seed(m + n + 1)
    a = torch.randn(m, k, generator=g).bfloat16().cuda()
    b = (0.05 * torch.randn(n, k, generator=g)).bfloat16().cuda()
    if operands == "nvfp4":
        aq, asf, ats = b200k.nvfp4_quantize(a)
        bq, bsf, bts = b200k.nvfp4_quantize(b)
        run = lambda **kw: b200k.cutile_nvfp4_matmul(aq, asf, ats, bq, bsf, bts, **kw)
    else:
        aq, asf = b200k.block_quantize(a, 32, swizzled_scale=True)
        bq, bsf = b200k.block_quantize(b, 32, swizzled_scale=True)
        run = lambda **kw: b200k.cutile_block_scaled_matmul(aq, asf, bq.T, bsf, **kw)
    c_bf16 = run(out_dtype=torch.bfloat16)
    q_ref, sf_ref, st_ref = oracle.nvfp4_quantize_ref(c_bf16.cpu())
    out_scale = torch.tensor([float(st_ref)], device="cuda")
    q, sf = run(out_dtype=torch.float4_e2m1fn_x2, out_scale=out_scale)
    assert q.shape == (m, n // 2) and q.dtype == torch.uint8
    assert np.array_equal(q.cpu().numpy(), q_ref)
    lo = oracle.unswizzle_32_4_4_ref(sf.cpu().view(torch.uint8))[:m, : n // 16]
    assert np.array_equal(lo.numpy(), sf_ref)
    # and the library's own two-step path gives the same bytes
    q2, sf2, st2 = b200k.nvfp4_quantize(c_bf16)
    assert float(st2) == float(st_ref) and torch.equal(q2, q)


def test_nvfp4_output_chains_into_the_next_gemm(device_ok):
    # up projection quantised in the epilogue feeds the down projection without a bf16 tensor
    g = torch.Generator().manual_seed(9)
    x = torch.randn(256, 512, generator=g).bfloat16().cuda()
    w1 = (0.05 * torch.randn(768, 512, generator=g)).bfloat16().cuda()
    w2 = (0.05 * torch.randn(384, 768, generator=g)).bfloat16().cuda()
    xq, xsf, xts = b200k.nvfp4_quantize(x)
    w1q, w1sf, w1ts = b200k.nvfp4_quantize(w1)
    w2q, w2sf, w2ts = b200k.nvfp4_quantize(w2)
    h_bf16 = b200k.cutile_nvfp4_matmul(xq, xsf, xts, w1q, w1sf, w1ts)
    hq_ref, hsf_ref, hts = b200k.nvfp4_quantize(h_bf16)
    y_ref = b200k.cutile_nvfp4_matmul(hq_ref, hsf_ref, hts, w2q, w2sf, w2ts, out_dtype=torch.float32)
    hq, hsf = b200k.cutile_nvfp4_matmul(xq, xsf, xts, w1q, w1sf, w1ts, out_dtype=torch.float4_e2m1fn_x2,
                                        out_scale=hts)
    y = b200k.cutile_nvfp4_matmul(hq, hsf, hts, w2q, w2sf, w2ts, out_dtype=torch.float32)
    torch.testing.assert_close(y, y_ref, atol=1e-5 * float(y_ref.abs().max()), rtol=1e-4)


def test_nvfp4_output_validation(device_ok):
    a = torch.randn(128, 64).bfloat16().cuda()
    aq, asf, ats = b200k.nvfp4_quantize(a)
    with pytest.raises(ValueError, match="out_scale"):
        b200k.cutile_nvfp4_matmul(aq, asf, ats, aq, asf, ats, out_dtype=torch.float4_e2m1fn_x2)
    aq48, asf48, ats48 = b200k.nvfp4_quantize(a[:48])
    with pytest.raises(ValueError, match="multiple of 32"):
        b200k.cutile_nvfp4_matmul(aq, asf, ats, aq48, asf48, ats48, out_dtype=torch.float4_e2m1fn_x2,
                                  out_scale=ats)


def test_mxfp8_sampled_rows_at_full_size(device_ok):
    # the headline configuration (8192^3, bf16 out): sampled rows against the oracle and a
    # row-sum identity over the whole output
    n = 8192
    g = torch.Generator(device="cuda").manual_seed(1)
    a = torch.randn(n, n, device="cuda", generator=g).bfloat16()
    b = torch.randn(n, n, device="cuda", generator=g).bfloat16()
    aq, sa = b200k.block_quantize(a, 32)
    bq, sb = b200k.block_quantize(b, 32)
    c = b200k.cutile_block_scaled_matmul(aq, sa, bq.T, sb.T, out_dtype=torch.bfloat16)
    rows = torch.tensor([0, 1, 127, 128, 4097, 8191])
    ref = oracle.block_scaled_matmul_ref(aq[rows].cpu(), sa[rows].cpu(), bq.cpu(), sb.cpu())
    torch.testing.assert_close(c[rows].float().cpu(), ref, atol=2e-2 * float(ref.abs().max()), rtol=2e-2)
    # sum_j C[i, j] == A_deq[i, :] . (sum_j B_deq[j, :])
    bsum = (bq.float() * torch.exp2(sb.view(torch.uint8).float() - 127).repeat_interleave(32, 1)).sum(0)
    adeq = aq.float() * torch.exp2(sa.view(torch.uint8).float() - 127).repeat_interleave(32, 1)
    want = adeq @ bsum
    got = c.float().sum(1)
    torch.testing.assert_close(got, want, atol=0.02 * float(want.abs().max()), rtol=2e-2)


@pytest.mark.parametrize("m,n,k", [(256, 256, 256), (384, 640, 512), (1000, 96, 160)])
def test_quantise_in_epilogue_equals_two_steps(m, n, k, device_ok):
    # e4m3 output + swizzled scales straight from the GEMM epilogue == quantising the bf16 result
    g = torch.Generator().manual_seed(m + n)
    a = torch.randn(m, k, generator=g).bfloat16().cuda()
    b = torch.randn(n, k, generator=g).bfloat16().cuda()
    aq, sa = b200k.block_quantize(a, 32, swizzled_scale=True)
    bq, sb = b200k.block_quantize(b, 32, swizzled_scale=True)
    c_bf16 = b200k.cutile_block_scaled_matmul(aq, sa, bq.T, sb, out_dtype=torch.bfloat16)
    # the oracle's quantiser over the bf16 result is the reference of this step
    q_ref, s_ref = oracle.block_quantize_ref(c_bf16.cpu())
    q, s = b200k.cutile_block_scaled_matmul(aq, sa, bq.T, sb, out_dtype=torch.float8_e4m3fn)
    assert q.shape == (m, n) and q.dtype == torch.float8_e4m3fn
    assert torch.equal(q.cpu().view(torch.uint8), q_ref.view(torch.uint8))
    # scale atoms: compare the bytes that belong to real rows / blocks
    lo = oracle.unswizzle_32_4_4_ref(s.cpu().view(torch.uint8))[:m, : n // 32]
    assert torch.equal(lo, s_ref.view(torch.uint8))
    # and the library's own two-step path gives the same bytes
    q2, s2 = b200k.block_quantize(c_bf16, 32)
    assert torch.equal(q2.view(torch.uint8), q.view(torch.uint8))
    assert torch.equal(s2.cpu().view(torch.uint8), s_ref.view(torch.uint8))


@pytest.mark.parametrize("fp4", [False, True])
@pytest.mark.parametrize("skip", [(0, 256), (256, 512), (768, 256)])
def test_skip_rows_leaves_whole_tiles_out(fp4, skip, device_ok):
    """skip_rows of b200k_block_scaled_gemm_args (the AllGather GEMM multiplies a rank's own
    rows separately): the skipped rows of C keep their contents, every other row is bit for
    bit the row of the full product."""
    from b200k.block_scaled import _as_u8, _scaled_gemm
    g = torch.Generator().manual_seed(31 + skip[0] + fp4)
    m, n, k = 1024, 768, 512
    a = torch.randn(m, k, generator=g).bfloat16().cuda()
    w = (0.05 * torch.randn(n, k, generator=g)).bfloat16().cuda()
    if fp4:
        aq, asf, ats = b200k.nvfp4_quantize(a)
        wq, wsf, wts = b200k.nvfp4_quantize(w)
        kw = dict(fp4=True, alpha_a=ats, alpha_b=wts)
    else:
        aq, asf = b200k.block_quantize(a, swizzled_scale=True)
        wq, wsf = b200k.block_quantize(w, swizzled_scale=True)
        kw = dict(fp4=False)
    ops = (_as_u8(aq) if fp4 else aq, _as_u8(asf), _as_u8(wq) if fp4 else wq, _as_u8(wsf))
    full = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    _scaled_gemm(*ops, full, **kw)
    part = torch.full((m, n), 7.0, dtype=torch.bfloat16, device="cuda")
    _scaled_gemm(*ops, part, skip_rows=skip, **kw)
    lo, cnt = skip
    assert torch.all(part[lo:lo + cnt] == 7.0)
    keep = torch.ones(m, dtype=torch.bool, device="cuda")
    keep[lo:lo + cnt] = False
    assert torch.equal(part[keep], full[keep])
    assert b200k.device_status() == (0, 0)


def test_skip_rows_validation(device_ok):
    from b200k.block_scaled import _as_u8, _scaled_gemm
    a = torch.randn(512, 256, device="cuda").bfloat16()
    w = torch.randn(256, 256, device="cuda").bfloat16()
    aq, asf = b200k.block_quantize(a, swizzled_scale=True)
    wq, wsf = b200k.block_quantize(w, swizzled_scale=True)
    c = torch.empty(512, 256, dtype=torch.bfloat16, device="cuda")
    for bad in [(128, 256), (0, 100), (256, 512), (-256, 256)]:
        with pytest.raises(b200k.B200KError):
            _scaled_gemm(aq, _as_u8(asf), wq, _as_u8(wsf), c, fp4=False, skip_rows=bad)
