"""MoE: bit-exact routing alignment against the oracle and the reference's golden vectors,
and the FFN against torch_moe's restatement.

Follows test/kernels/fused_moe.py:113-173 (alignment), samples/MoE.py:292-334 and :405-468
(sample problem: 48 tokens, hidden 512, 64 experts, intermediate 1024, top-8, bf16,
rtol = atol = 1e-1) and test/bench_moe.py:58-68.
"""
import os

import numpy as np
import pytest
import torch

import b200k
import oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("case", list("abcde"))
def test_moe_align_golden(golden_dir, case, device_ok):
    g = np.load(os.path.join(golden_dir, "moe_align.npz"))
    tokens, topk, experts, tile_m = g[f"{case}_cfg"].tolist()
    ids = torch.from_numpy(g[f"{case}_ids"]).cuda()
    st, se = b200k.moe_align_tile_size_torch(ids, tile_m, experts)
    assert st.dtype == torch.int32 and se.dtype == torch.int32
    assert np.array_equal(st.cpu().numpy(), g[f"{case}_sorted_token_ids"])
    assert np.array_equal(se.cpu().numpy(), g[f"{case}_sorted_expert_ids"])


@pytest.mark.parametrize("tokens,topk,experts,tile_m,dtype", [
    (16384, 8, 64, 128, torch.int64), (1000, 2, 7, 16, torch.int32), (3, 1, 300, 128, torch.int64),
    (4096, 8, 256, 128, torch.int64), (513, 4, 5, 1, torch.int32)])
def test_moe_align_vs_oracle(tokens, topk, experts, tile_m, dtype, device_ok):
    g = torch.Generator().manual_seed(tokens + experts)
    ids = torch.topk(torch.randn(tokens, experts, generator=g), topk, dim=-1).indices.to(dtype)
    st, se, nb = b200k.moe_align_device(ids.cuda(), tile_m, experts)
    rt, re = oracle.moe_align_ref(ids, tile_m, experts)
    n = int(nb.item())
    assert n == re.numel()
    assert torch.equal(st[: n * tile_m].cpu(), rt)
    assert torch.equal(se[:n].cpu(), re)
    # worst-case-sized tails: sentinel ids and -1 block owners
    assert torch.all(st[n * tile_m:] == tokens * topk)
    assert torch.all(se[n:] == -1)
    # every replica id appears exactly once
    live = st[st < tokens * topk]
    assert torch.equal(torch.sort(live).values.cpu(), torch.arange(tokens * topk, dtype=torch.int32))


def test_moe_align_skewed_routing(device_ok):
    ids = torch.zeros(700, 4, dtype=torch.int64)        # everything to expert 0
    ids[:, 1] = 5
    st, se = b200k.moe_align_tile_size_torch(ids.cuda(), 128, 8)
    rt, re = oracle.moe_align_ref(ids, 128, 8)
    assert torch.equal(st.cpu(), rt) and torch.equal(se.cpu(), re)


def test_silu_and_mul(device_ok):
    g = torch.Generator().manual_seed(1)
    ab = torch.randn(77, 2 * 96, generator=g).bfloat16()
    c = torch.empty(77, 96, dtype=torch.bfloat16, device="cuda")
    b200k.invoke_silu_and_mul_kernel(ab.cuda(), c)
    ref = torch.nn.functional.silu(ab[:, :96].float()) * ab[:, 96:].float()
    torch.testing.assert_close(c.float().cpu(), ref, atol=1e-2, rtol=1e-2)


def _problem(tokens, hidden, experts, inter, topk, seed, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    x = (0.5 * torch.randn(tokens, hidden, generator=g)).to(dtype)
    w1 = (0.1 * torch.randn(experts, 2 * inter, hidden, generator=g)).to(dtype)
    w2 = (0.1 * torch.randn(experts, hidden, inter, generator=g)).to(dtype)
    tw, ids = oracle.moe_route_ref(torch.randn(tokens, experts, generator=g), topk)
    return x, w1, w2, tw.to(dtype), ids


@pytest.mark.parametrize("tokens,hidden,experts,inter,topk", [
    (48, 512, 64, 1024, 8),      # the sample's problem
    (24, 64, 4, 32, 2),          # intermediate not a multiple of 128: unfused SiLU path
    (300, 256, 8, 128, 2), (1, 128, 4, 128, 1),
    (1500, 512, 6, 384, 3)])     # several row tiles per expert, three column tiles
@pytest.mark.parametrize("row_tile", ["128", "256"])   # one-CTA and CTA-pair grouped GEMM
def test_cutile_moe_bf16(tokens, hidden, experts, inter, topk, row_tile, device_ok, monkeypatch):
    monkeypatch.setenv("B200K_MOE_TILE", row_tile)
    x, w1, w2, tw, ids = _problem(tokens, hidden, experts, inter, topk, tokens)
    out = b200k.cutile_moe(x.cuda(), w1.cuda(), w2.cuda(), tw.cuda(), ids.cuda(), 128, 128, 64)
    assert out.shape == x.shape and out.dtype == x.dtype
    ref = oracle.moe_ref(x, w1, w2, tw, ids)
    torch.testing.assert_close(out.float().cpu(), ref, rtol=1e-1, atol=1e-1)
    assert oracle.rel_frobenius(out, ref) < 2e-2


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("tokens,hidden,experts,inter,topk", [
    (110, 1024, 16, 512, 4),      # the reference's bench shapes (test/bench_moe.py:16-19) ...
    (256, 2048, 1408, 32, 6)])    # ... about one token per expert: the automatic row tile is 128
def test_cutile_moe_reference_bench_shapes(tokens, hidden, experts, inter, topk, dtype, device_ok):
    x, w1, w2, tw, ids = _problem(tokens, hidden, experts, inter, topk, 3 * tokens, dtype)
    out = b200k.cutile_moe(x.cuda(), w1.cuda(), w2.cuda(), tw.cuda(), ids.cuda())
    assert out.shape == x.shape and out.dtype == dtype
    ref = oracle.moe_ref(x, w1, w2, tw, ids)
    # the reference bench's own tolerances (test/bench_moe.py:60-66); fp32 operands are
    # multiplied as tf32 here
    tol = {torch.float16: 5e-2, torch.bfloat16: 1e-1, torch.float32: 1e-2}[dtype]
    torch.testing.assert_close(out.float().cpu(), ref, rtol=tol, atol=tol)


@pytest.mark.parametrize("tile_m", [128, 256])
def test_invoke_fused_moe_kernel_matches_manual_pipeline(tile_m, device_ok):
    # the sample's three-launch pipeline driven through the reference-named helpers
    x, w1, w2, tw, ids = _problem(40, 256, 8, 128, 2, 7)
    xc, w1c, w2c, twc, idc = (t.cuda() for t in (x, w1, w2, tw, ids))
    st, se = b200k.moe_align_tile_size_torch(idc, tile_m, 8)
    c1 = torch.zeros(40, 2, 256, dtype=torch.bfloat16, device="cuda")
    b200k.invoke_fused_moe_kernel(xc, w1c, c1, twc, st, se, False, 2, tile_m, 128, 64)
    c2 = torch.zeros(80, 128, dtype=torch.bfloat16, device="cuda")
    b200k.invoke_silu_and_mul_kernel(c1.view(-1, 256), c2)
    c3 = torch.zeros(40, 2, 256, dtype=torch.bfloat16, device="cuda")
    b200k.invoke_fused_moe_kernel(c2, w2c, c3, twc, st, se, True, 1, tile_m, 128, 64)
    out = torch.sum(c3, dim=1)
    torch.testing.assert_close(out.float().cpu(), oracle.moe_ref(x, w1, w2, tw, ids), rtol=1e-1, atol=1e-1)
    with pytest.raises(ValueError, match="row tile"):
        b200k.invoke_fused_moe_kernel(xc, w1c, c1, twc, st, se, False, 2, 64, 128, 64)


def test_torch_moe_golden_problem(golden_dir, device_ok):
    g = np.load(os.path.join(golden_dir, "torch_moe.npz"))
    x, w1, w2, tw, ids = (torch.from_numpy(g[k]) for k in ("hidden", "w1", "w2", "topk_weights", "topk_ids"))
    out = b200k.cutile_moe(x.bfloat16().cuda(), w1.bfloat16().cuda(), w2.bfloat16().cuda(),
                           tw.bfloat16().cuda(), ids.cuda())
    torch.testing.assert_close(out.float().cpu(), torch.from_numpy(g["out"]), rtol=1e-1, atol=1e-1)


@pytest.mark.parametrize("tokens,hidden,experts,inter,topk", [(64, 256, 8, 128, 2), (500, 512, 16, 256, 4),
                                                             (1500, 512, 6, 384, 3)])
@pytest.mark.parametrize("row_tile", ["128", "256"])
def test_cutile_moe_mxfp8(tokens, hidden, experts, inter, topk, row_tile, device_ok, monkeypatch):
    monkeypatch.setenv("B200K_MOE_TILE", row_tile)
    x, w1, w2, tw, ids = _problem(tokens, hidden, experts, inter, topk, 11)
    w1q, w1s = b200k.quantize_expert_weights(w1.cuda())
    w2q, w2s = b200k.quantize_expert_weights(w2.cuda())
    # quantised weights are bit-exact to the oracle's
    q_ref, s_ref = oracle.block_quantize_ref(w1)
    assert torch.equal(w1q.cpu().view(torch.uint8), q_ref.view(torch.uint8))
    out = b200k.cutile_moe_mxfp8(x.cuda(), w1q, w1s, w2q, w2s, tw.cuda(), ids.cuda())
    q2_ref, s2_ref = oracle.block_quantize_ref(w2)
    ref = oracle.moe_mxfp8_ref(x, q_ref, s_ref, q2_ref, s2_ref, tw, ids)
    assert oracle.rel_frobenius(out, ref) < 2e-2
    # and the quantised pipeline stays close to the unquantised FFN
    assert oracle.rel_frobenius(out, oracle.moe_ref(x, w1, w2, tw, ids)) < 1e-1


@pytest.mark.parametrize("mxfp8", [False, True])
def test_routing_entries_outside_the_expert_range_contribute_zero(mxfp8):
    # a sentinel-padded or corrupt topk_ids: the alignment drops the entry and records it in the
    # status word; the token's output is the sum over its remaining slots (never stale memory)
    x, w1, w2, tw, ids = _problem(200, 256, 8, 128, 2, 21)
    bad = ids.clone()
    bad[3, 0], bad[77, 1], bad[199, 0], bad[199, 1] = -1, 8, 1000, -5
    tw_eff = tw.clone()
    tw_eff[(bad < 0) | (bad >= 8)] = 0
    poison = torch.full((4096, 256), float("nan"), dtype=torch.bfloat16, device="cuda")
    del poison                                     # the caching allocator hands these pages out next
    if mxfp8:
        w1q, w1s = b200k.quantize_expert_weights(w1.cuda())
        w2q, w2s = b200k.quantize_expert_weights(w2.cuda())
        out = b200k.cutile_moe_mxfp8(x.cuda(), w1q, w1s, w2q, w2s, tw.cuda(), bad.cuda())
    else:
        out = b200k.cutile_moe(x.cuda(), w1.cuda(), w2.cuda(), tw.cuda(), bad.cuda())
    torch.cuda.synchronize()
    code, info = b200k.device_status()
    assert code != 0 and (info >> 8) & 0xff == 40      # reported, and cleared by the read
    assert b200k.device_status()[0] == 0
    ref = oracle.moe_ref(x, w1, w2, tw_eff, bad.clamp(0, 7))
    assert bool(torch.isfinite(out).all())
    assert float(out[199].abs().max()) == 0.0          # both slots dropped
    assert oracle.rel_frobenius(out, ref) < (1e-1 if mxfp8 else 2e-2)   # mxfp8: against the unquantised FFN


def test_cutile_moe_hidden_not_a_multiple_of_eight_elements(device_ok):
    # fp32 rows of 20 elements are 16-byte multiples for the gather and the GEMMs, but not a
    # multiple of 8 elements: the top-k sum takes its one-element-per-thread form
    x, w1, w2, tw, ids = _problem(64, 20, 4, 12, 2, 5, torch.float32)
    out = b200k.cutile_moe(x.cuda(), w1.cuda(), w2.cuda(), tw.cuda(), ids.cuda())
    torch.testing.assert_close(out.cpu(), oracle.moe_ref(x, w1, w2, tw, ids), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("tokens,hidden,experts,inter,topk", [
    (256, 2048, 1408, 32, 6),      # the reference's sparse bench shape (test/bench_moe.py:16-19)
    (8, 512, 64, 384, 8),          # a decode-sized batch over many experts
    (5, 264, 40, 24, 3)])          # row lengths that are not powers of two
def test_sparse_routing_path_matches_the_oracle_and_the_grouped_path(tokens, hidden, experts, inter, topk, dtype,
                                                                    device_ok, monkeypatch):
    x, w1, w2, tw, ids = _problem(tokens, hidden, experts, inter, topk, 17 + tokens, dtype)
    dev = [t.cuda() for t in (x, w1, w2, tw, ids)]
    monkeypatch.setenv("B200K_MOE_SPARSE", "1")
    out = b200k.cutile_moe(*dev)
    assert out.shape == x.shape and out.dtype == dtype
    ref = oracle.moe_ref(x, w1, w2, tw, ids)
    tol = {torch.float16: 5e-2, torch.bfloat16: 1e-1, torch.float32: 1e-2}[dtype]   # test/bench_moe.py:60-66
    torch.testing.assert_close(out.float().cpu(), ref, rtol=tol, atol=tol)
    assert oracle.rel_frobenius(out, ref) < (1e-3 if dtype == torch.float32 else 2e-2)
    # the automatic choice takes this path exactly where routing is sparse
    from b200k import moe
    monkeypatch.delenv("B200K_MOE_SPARSE")
    assert moe._sparse_routing(256 * 6, 1408, 2048, 32, 2) and not moe._sparse_routing(110 * 4, 16, 1024, 512, 2)
    if inter % 8 == 0 and hidden % 8 == 0:
        monkeypatch.setenv("B200K_MOE_SPARSE", "0")
        dense = b200k.cutile_moe(*dev)
        torch.testing.assert_close(out.float(), dense.float(), rtol=tol, atol=tol)


def test_sparse_routing_path_drops_entries_outside_the_expert_range(monkeypatch):
    monkeypatch.setenv("B200K_MOE_SPARSE", "1")
    x, w1, w2, tw, ids = _problem(40, 256, 64, 64, 2, 3)
    bad = ids.clone()
    bad[0, 0], bad[39, 1] = -3, 64
    tw_eff = tw.clone()
    tw_eff[(bad < 0) | (bad >= 64)] = 0
    out = b200k.cutile_moe(x.cuda(), w1.cuda(), w2.cuda(), tw.cuda(), bad.cuda())
    torch.cuda.synchronize()
    code, info = b200k.device_status()
    assert code != 0 and (info >> 8) & 0xff == 40
    ref = oracle.moe_ref(x, w1, w2, tw_eff, bad.clamp(0, 63))
    assert oracle.rel_frobenius(out, ref) < 2e-2


@pytest.mark.parametrize("tokens,hidden,experts,topk", [(300, 512, 8, 2), (64, 4096, 16, 8), (17, 264, 5, 3)])
def test_gather_rows_by_source_equals_gather_rows(tokens, hidden, experts, topk, device_ok):
    """b200k_gather_rows_by_source (every token row read once, stored to all its places) fills the
    destination exactly as b200k_gather_rows does (one read per destination row), padding rows
    and entries routed outside the experts included."""
    from b200k import moe
    g = torch.Generator().manual_seed(tokens + hidden)
    x = torch.randn(tokens, hidden, generator=g).bfloat16().cuda()
    ids = torch.stack([torch.randperm(experts, generator=g)[:topk] for _ in range(tokens)]).int()
    ids[0, 0] = experts + 3                      # dropped entries: not in the sorted order
    ids[tokens - 1, topk - 1] = -1
    sorted_ids, _, num_blocks = moe.moe_align_device(ids.cuda(), 128, experts)
    cap = sorted_ids.numel()
    a = moe._gather_rows(x, sorted_ids, topk, cap, num_blocks, 128)
    b = moe._gather_rows(x, sorted_ids, topk, cap, num_blocks, 128, by_source=True)
    live = int(num_blocks.item()) * 128
    assert torch.equal(a[:live], b[:live])
    # without the live-row bound every row of the capacity is produced
    a = moe._gather_rows(x, sorted_ids[:live], topk, live, None, 128)
    b = moe._gather_rows(x, sorted_ids[:live], topk, live, None, 128, by_source=True)
    assert torch.equal(a, b)
    torch.cuda.synchronize()
    code, info = b200k.device_status()           # the alignment records the dropped entries; reading clears
    assert code != 0 and (info >> 8) & 0xff == 40
