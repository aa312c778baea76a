"""Bit-exact parity of the quantisers and the scale relayout with the oracle and with the
golden vectors produced by the reference's block_quantize / swizzle_32_4_4
(test/kernels/kernel_utils.py:38-98)."""
import os

import numpy as np
import pytest
import torch

import b200k
import oracle

pytestmark = pytest.mark.gpu


def _u8(t):
    return t.cpu().view(torch.uint8).numpy()


def test_block_quantize_golden(golden_dir, device_ok):
    g = np.load(os.path.join(golden_dir, "block_quantize.npz"))
    q, s = b200k.block_quantize(torch.from_numpy(g["x"]).cuda(), 32)
    assert q.dtype == torch.float8_e4m3fn and s.dtype == torch.float8_e8m0fnu
    assert np.array_equal(_u8(q), g["q"])
    assert np.array_equal(_u8(s), g["scale"])
    qb, sb = b200k.block_quantize(torch.from_numpy(g["xb"]).bfloat16().cuda(), 32)
    assert np.array_equal(_u8(qb), g["qb"])
    assert np.array_equal(_u8(sb), g["scaleb"])
    sw = b200k.swizzle_32_4_4(s)
    assert sw.shape == (1, 2, 32, 16)
    assert np.array_equal(_u8(sw), g["swizzled"])
    _, sw2 = b200k.block_quantize(torch.from_numpy(g["x"]).cuda(), 32, swizzled_scale=True)
    assert np.array_equal(_u8(sw2), g["swizzled"])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,k", [(256, 512), (100, 96), (1, 32), (384, 4096), (7, 70)])
def test_block_quantize_vs_oracle(dtype, rows, k, device_ok):
    g = torch.Generator().manual_seed(rows * 131 + k)
    # per-row magnitudes spread over the exponent range the dtype can hold without inf
    span = 12 if dtype == torch.float16 else 20
    x = (torch.randn(rows, k, generator=g) * torch.exp2(torch.randint(-span, span, (rows, 1), generator=g).float())).to(dtype)
    x[0, :32] = 0
    q, s = b200k.block_quantize(x.cuda(), 32)
    qr, sr = oracle.block_quantize_ref(x)
    assert q.shape == qr.shape and s.shape == sr.shape
    assert np.array_equal(_u8(q), _u8(qr))
    assert np.array_equal(_u8(s), _u8(sr))


def test_block_quantize_power_of_two_boundaries(device_ok):
    # amax at, one bf16 ulp below and one bf16 ulp above 448 * 2^e for every exponent the
    # format can carry
    es = torch.arange(-60, 60)
    base = 448.0 * torch.exp2(es.float())
    rows = []
    for f in (1.0, 1 - 2.0 ** -8, 1 + 2.0 ** -7):
        blk = torch.zeros(len(es), 32)
        blk[:, 5] = base * f
        rows.append(blk)
    x = torch.cat(rows, 0)
    q, s = b200k.block_quantize(x.cuda(), 32)
    qr, sr = oracle.block_quantize_ref(x)
    assert np.array_equal(_u8(s), _u8(sr))
    assert np.array_equal(_u8(q), _u8(qr))


def test_block_quantize_e5m2_and_nd(device_ok):
    g = torch.Generator().manual_seed(3)
    x = torch.randn(2, 3, 64, generator=g)
    q, s = b200k.block_quantize(x.cuda(), 32, torch.float8_e5m2)
    qr, sr = oracle.block_quantize_ref(x, 32, torch.float8_e5m2)
    assert q.shape == (2, 3, 64) and s.shape == (2, 3, 2)
    assert np.array_equal(_u8(q), _u8(qr)) and np.array_equal(_u8(s), _u8(sr))


@pytest.mark.parametrize("rows,ks", [(128, 4), (256, 8), (1024, 64), (100, 3), (129, 5)])
def test_swizzle_vs_oracle(rows, ks, device_ok):
    g = torch.Generator().manual_seed(rows + ks)
    s = torch.randint(0, 255, (rows, ks), generator=g, dtype=torch.uint8)
    sw = b200k.swizzle_32_4_4(s.cuda().view(torch.float8_e8m0fnu))
    rp, kp = -(-rows // 128) * 128, -(-ks // 4) * 4
    padded = torch.full((rp, kp), 127, dtype=torch.uint8)
    padded[:rows, :ks] = s
    assert np.array_equal(_u8(sw), _u8(oracle.swizzle_32_4_4_ref(padded)))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,k", [(256, 512), (128, 1024), (33, 48), (5, 16)])
def test_nvfp4_quantize_vs_oracle(dtype, rows, k, device_ok):
    g = torch.Generator().manual_seed(rows * 7 + k)
    x = torch.randn(rows, k, generator=g).to(dtype)
    x[0, :16] = 0
    q, sf, ts = b200k.nvfp4_quantize(x.cuda(), swizzled_scale=False)
    qr, sfr, tsr = oracle.nvfp4_quantize_ref(x)
    assert ts.item() == float(tsr)
    assert np.array_equal(_u8(sf), sfr)
    assert np.array_equal(q.cpu().numpy(), qr)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("factor", [1.0, 0.25, 3.0])
def test_nvfp4_quantize_with_given_tensor_scale(dtype, factor, device_ok):
    # one pass under a caller-given per-tensor scale: the scale the two-pass form would find
    # (same bytes), a quarter of it (block scales and codes saturate), three times it
    g = torch.Generator().manual_seed(11)
    x = torch.randn(200, 96, generator=g).to(dtype)
    _, _, own = oracle.nvfp4_quantize_ref(x)
    given = np.float32(own) * np.float32(factor)
    scale = torch.tensor([float(given)], dtype=torch.float32, device="cuda")
    q, sf, ts = b200k.nvfp4_quantize(x.cuda(), swizzled_scale=False, tensor_scale=scale)
    qr, sfr, tsr = oracle.nvfp4_quantize_ref(x, tensor_scale=given)
    assert ts is scale and ts.item() == float(tsr)
    assert np.array_equal(_u8(sf), sfr)
    assert np.array_equal(q.cpu().numpy(), qr)
    if factor == 1.0:
        q2, sf2, _ = b200k.nvfp4_quantize(x.cuda(), swizzled_scale=False)
        assert torch.equal(q, q2) and torch.equal(_as(sf), _as(sf2))


def _as(t):
    return t.view(torch.uint8)


def test_nvfp4_quantize_all_zero_tensor(device_ok):
    x = torch.zeros(128, 64, dtype=torch.bfloat16, device="cuda")
    q, sf, ts = b200k.nvfp4_quantize(x, swizzled_scale=False)
    assert ts.item() == 0 and not q.any() and not _u8(sf).any()


def test_quantize_fixed_point_at_full_size(device_ok):
    # size-independent properties at the bench size: the de-quantised tensor is a fixed
    # point of quantise -> de-quantise, and the scale bytes obey the exact integer rule
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(8192, 8192, device="cuda", generator=g).bfloat16()

    def dequant(q, s):
        return q.float() * torch.exp2(s.view(torch.uint8).float() - 127.0).repeat_interleave(32, 1)

    q, s = b200k.block_quantize(x, 32)
    deq = dequant(q, s)
    q2, s2 = b200k.block_quantize(deq, 32)
    assert torch.equal(dequant(q2, s2), deq)
    amax = x.float().reshape(8192, -1, 32).abs().amax(-1)
    mant, exp = torch.frexp(amax / 448.0)        # amax/448 = mant * 2^exp, mant in [0.5, 1)
    e = torch.where(mant == 0.5, exp - 1, exp)
    assert torch.equal(s.view(torch.uint8).int(), (e + 127).int())
