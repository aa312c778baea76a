"""Parity at the sizes the benchmark runs: the NVFP4 FFN up-projection (8192 x 28672 x 8192),
causal attention B4 H32 S8192 D128 and the MoE FFN with 16384 tokens, 64 experts, top-8.

The oracle cannot evaluate these problems whole in seconds, so each test compares sampled
rows (query rows, tokens) of the full-size GPU result with the oracle evaluated for those
rows only, picked where the kernels' tiling has its seams (first / last row of a 128-row
tile, of a 256-row CTA-pair tile, of the last wave of tiles), and adds a size-independent
identity over the whole output where the operator has one.  The reference's benches check
their full-size outputs the same way before timing (test/bench_matmul.py:34-36,111-112,
test/bench_attention.py:58-69, test/bench_moe.py:58-68); tolerances are those of the
small-shape tests.  Inputs are drawn on the CPU from a seeded torch.Generator and copied over.
"""
import numpy as np
import pytest
import torch

import b200k
import oracle

pytestmark = pytest.mark.gpu


def _nvfp4_dequant_gpu(q, sf_logical, ts):
    """fp32 value of packed e2m1 codes with logical ue4m3 scales, on the device (torch ops
    only: used for whole-tensor identities, never as the reference of a parity check)."""
    lut = torch.tensor([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6],
                       dtype=torch.float32, device=q.device)
    lo = lut[(q & 0xF).long()]
    hi = lut[(q >> 4).long()]
    vals = torch.stack([lo, hi], dim=-1).reshape(q.shape[0], -1)
    s = sf_logical.view(torch.float8_e4m3fn).float().repeat_interleave(16, dim=1)
    return vals * s * ts


def test_nvfp4_ffn_up_projection_sampled_rows(device_ok):
    m, n, k = 8192, 28672, 8192
    g = torch.Generator().manual_seed(2)
    a = torch.randn(m, k, generator=g).bfloat16()
    b = (0.02 * torch.randn(n, k, generator=g)).bfloat16()
    aq, asf, ats = b200k.nvfp4_quantize(a.cuda(), swizzled_scale=False)
    bq, bsf, bts = b200k.nvfp4_quantize(b.cuda(), swizzled_scale=False)
    c = b200k.cutile_nvfp4_matmul(aq, b200k.swizzle_32_4_4(asf), ats, bq, b200k.swizzle_32_4_4(bsf), bts)
    assert c.shape == (m, n) and c.dtype == torch.bfloat16
    # 32 x 112 tiles of 256 x 256 on 74 CTA pairs: rows at the seams of a 128-row half tile, of
    # a 256-row tile, and in the tiles of the last (partial) wave
    rows = torch.tensor([0, 127, 128, 255, 256, 6144, 8064, 8191])
    # the quantiser's bytes for those rows equal the oracle's under the same tensor scale
    a_ref = oracle.nvfp4_quantize_ref(a[rows], tensor_scale=float(ats))
    assert float(ats) == float(np.float32(np.float32(a.float().abs().max()) / np.float32(2688.0)))
    assert np.array_equal(aq[rows.cuda()].cpu().numpy(), a_ref[0])
    assert np.array_equal(asf[rows.cuda()].cpu().view(torch.uint8).numpy(), a_ref[1])
    got = c[rows.cuda()].float().cpu()
    bq_h, bsf_h = bq.cpu().numpy(), bsf.cpu().view(torch.uint8).numpy()
    worst = 0.0
    for lo in range(0, n, 4096):       # B de-quantised 4096 rows at a time (bounded host memory)
        ref = oracle.nvfp4_matmul_ref(a_ref[0], a_ref[1], a_ref[2], bq_h[lo:lo + 4096],
                                      bsf_h[lo:lo + 4096], float(bts))
        part = got[:, lo:lo + 4096]
        torch.testing.assert_close(part, ref, atol=2e-2 * float(ref.abs().max()), rtol=2e-2)
        worst = max(worst, oracle.rel_frobenius(part, ref))
    assert worst < 5e-2
    # sum_j C[i, j] == A_deq[i, :] . sum_j B_deq[j, :] over all 28672 columns, every row
    bsum = torch.zeros(k, dtype=torch.float32, device="cuda")
    for lo in range(0, n, 4096):
        bsum += _nvfp4_dequant_gpu(bq[lo:lo + 4096], bsf[lo:lo + 4096], bts).sum(0)
    want = torch.cat([_nvfp4_dequant_gpu(aq[lo:lo + 1024], asf[lo:lo + 1024], ats) @ bsum
                      for lo in range(0, m, 1024)])
    have = c.float().sum(1)
    torch.testing.assert_close(have, want, atol=2e-2 * float(want.abs().max()), rtol=2e-2)


def test_causal_attention_b4_h32_s8192_sampled_rows(device_ok):
    bsz, heads, seq, d = 4, 32, 8192, 128
    g = torch.Generator().manual_seed(3)
    q, k, v = (torch.randn(bsz, heads, seq, d, generator=g).bfloat16() for _ in range(3))
    out = b200k.cutile_fmha(q.cuda(), k.cuda(), v.cuda(), causal=True)
    assert out.shape == q.shape and out.dtype == torch.bfloat16
    # query blocks: the first tile, one that straddles a 256-row CTA tile, the last tile
    blocks = [(0, 128), (4032, 4160), (8064, 8192)]
    for b_i, h_i in [(0, 0), (1, 17), (2, 5), (3, 31)]:
        for lo, hi in blocks:
            ref = oracle.fmha_ref(q[b_i:b_i + 1, h_i:h_i + 1, lo:hi], k[b_i:b_i + 1, h_i:h_i + 1, :hi],
                                  v[b_i:b_i + 1, h_i:h_i + 1, :hi], causal=True, input_pos=lo)
            torch.testing.assert_close(out[b_i:b_i + 1, h_i:h_i + 1, lo:hi].float().cpu(), ref,
                                       atol=1e-2, rtol=5e-2)
    # row 0 of every (batch, head) attends to key 0 only: its output is V[0]
    torch.testing.assert_close(out[:, :, 0].float().cpu(), v[:, :, 0].float(), atol=1e-2, rtol=1e-2)


@pytest.fixture(scope="module")
def moe_config5():
    tokens, hidden, experts, inter, topk = 16384, 4096, 64, 1536, 8
    g = torch.Generator().manual_seed(4)
    tw, ids = oracle.moe_route_ref(torch.randn(tokens, experts, generator=g), topk)
    x = torch.randn(tokens, hidden, generator=g).bfloat16()
    w1 = (0.02 * torch.randn(experts, 2 * inter, hidden, generator=g)).bfloat16()
    w2 = (0.02 * torch.randn(experts, hidden, inter, generator=g)).bfloat16()
    return x, w1, w2, tw.bfloat16(), ids


def _sampled_tokens(ids, count):
    g = torch.Generator().manual_seed(5)
    pick = torch.randperm(ids.shape[0], generator=g)[:count - 2]
    return torch.cat([torch.tensor([0, ids.shape[0] - 1]), pick]).sort().values


def test_moe_config5_bf16_sampled_tokens(moe_config5, device_ok):
    x, w1, w2, tw, ids = moe_config5
    experts = w1.shape[0]
    idc = ids.cuda()
    out = b200k.cutile_moe(x.cuda(), w1.cuda(), w2.cuda(), tw.cuda(), idc)
    assert out.shape == x.shape and out.dtype == torch.bfloat16
    # routing / permutation indices of the whole problem, both row tiles: bit-exact
    for tile in (128, 256):
        st, se = b200k.moe_align_tile_size_torch(idc, tile, experts)
        st_ref, se_ref = oracle.moe_align_ref(ids, tile, experts)
        assert torch.equal(st.cpu(), st_ref) and torch.equal(se.cpu(), se_ref)
    tok = _sampled_tokens(ids, 16)
    ref = oracle.moe_ref(x[tok], w1, w2, tw[tok], ids[tok])
    got = out[tok.cuda()].float().cpu()
    torch.testing.assert_close(got, ref, rtol=1e-1, atol=1e-1)    # test/bench_moe.py:60-66
    assert oracle.rel_frobenius(got, ref) < 2e-2
    # nothing but real rows contributes: every output row is finite
    assert bool(torch.isfinite(out).all())


def test_moe_config5_mxfp8_sampled_tokens(moe_config5, device_ok):
    x, w1, w2, tw, ids = moe_config5
    e, n1, hidden = w1.shape
    inter = w2.shape[2]
    w1c, w2c = w1.cuda(), w2.cuda()
    w1q, w1s = b200k.quantize_expert_weights(w1c)
    w2q, w2s = b200k.quantize_expert_weights(w2c)
    out = b200k.cutile_moe_mxfp8(x.cuda(), w1q, w1s, w2q, w2s, tw.cuda(), ids.cuda())
    assert out.shape == x.shape and out.dtype == torch.bfloat16
    # logical scales of the same quantisation for the oracle (the quantiser's bytes are held
    # bit-exact to oracle.block_quantize_ref by the quantiser tests; spot-check one expert here)
    _, w1l = b200k.block_quantize(w1c.reshape(e * n1, hidden), 32)
    _, w2l = b200k.block_quantize(w2c.reshape(e * hidden, inter), 32)
    q_ref, s_ref = oracle.block_quantize_ref(w1[7])
    assert torch.equal(w1q[7].cpu().view(torch.uint8), q_ref.view(torch.uint8))
    assert torch.equal(w1l.reshape(e, n1, -1)[7].cpu().view(torch.uint8), s_ref.view(torch.uint8))
    tok = _sampled_tokens(ids, 16)
    ref = oracle.moe_mxfp8_ref(x[tok], w1q.cpu(), w1l.reshape(e, n1, -1).cpu(), w2q.cpu(),
                               w2l.reshape(e, hidden, -1).cpu(), tw[tok], ids[tok])
    got = out[tok.cuda()].float().cpu()
    assert oracle.rel_frobenius(got, ref) < 2e-2
    torch.testing.assert_close(got, ref, rtol=1e-1, atol=1e-1)
    # and the quantised pipeline stays close to the unquantised FFN
    assert oracle.rel_frobenius(got, oracle.moe_ref(x[tok], w1, w2, tw[tok], ids[tok])) < 1e-1
