"""Parity of the attention forward kernel with the fp32 CPU oracle.

Shapes follow test/test_attention.py:13-64 (batch {1,4}, q heads {8,16} over 8 kv heads,
ragged q/k lengths, causal with input_pos) scaled to this kernel's head dims, plus
slices of the benchmark-sized problem; tolerances are the reference's for 16-bit inputs
(atol 1e-2, rtol 5e-2, test/test_attention.py:62-63).
"""
import math

import pytest
import torch

import b200k
import oracle

pytestmark = pytest.mark.gpu

TOL = dict(atol=1e-2, rtol=5e-2)


def _qkv(b, hq, hkv, sq, sk, d, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(b, hq, sq, d, generator=g).to(dtype)
    k = torch.randn(b, hkv, sk, d, generator=g).to(dtype)
    v = torch.randn(b, hkv, sk, d, generator=g).to(dtype)
    return q, k, v


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("sq,sk", [(128, 128), (256, 384), (100, 100), (129, 300), (512, 512)])
@pytest.mark.parametrize("d", [64, 128])
def test_fmha_matches_oracle(dtype, causal, sq, sk, d, device_ok):
    q, k, v = _qkv(2, 4, 4, sq, sk, d, dtype, sq + sk + d)
    input_pos = sk - sq if (causal and sk > sq) else 0
    out = b200k.cutile_fmha(q.cuda(), k.cuda(), v.cuda(), causal=causal, input_pos=input_pos)
    assert out.shape == (2, 4, sq, d) and out.dtype == dtype
    ref = oracle.fmha_ref(q, k, v, causal=causal, input_pos=input_pos)
    torch.testing.assert_close(out.float().cpu(), ref, **TOL)


@pytest.mark.parametrize("batch", [1, 4])
@pytest.mark.parametrize("q_heads", [8, 16])
@pytest.mark.parametrize("q_len,k_len", [(1, 32), (15, 63), (32, 32)])
@pytest.mark.parametrize("causal", [False, True])
def test_fmha_reference_test_shapes_gqa(batch, q_heads, q_len, k_len, causal, device_ok):
    # D = 32 as in the reference test: zero-padded to the kernel's 64 by the wrapper
    q, k, v = _qkv(batch, q_heads, 8, q_len, k_len, 32, torch.bfloat16, q_heads + q_len)
    group = q_heads // 8
    input_pos = k_len - q_len if causal else 0
    out = b200k.cutile_fmha(q.cuda(), k.cuda(), v.cuda(), query_group_size=group, causal=causal,
                            input_pos=input_pos)
    ref = oracle.fmha_ref(q, k, v, causal=causal, input_pos=input_pos, query_group_size=group)
    torch.testing.assert_close(out.float().cpu(), ref, **TOL)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("b,hq,hkv,sq,sk,causal", [
    (1, 32, 32, 1, 1024, True),     # the reference's decode bench shape
    (2, 32, 8, 1, 1000, True),      # grouped-query decode: 4 rows share a KV head, ragged keys
    (1, 16, 4, 2, 4100, True),      # two new tokens, 8 rows per KV head, many splits
    (2, 8, 8, 3, 70, True),         # keys shorter than one chunk
    (1, 8, 2, 1, 300, False),
    (3, 4, 4, 5, 129, False),
    (5, 32, 8, 2, 600, True),       # enough KV heads for the one-kernel (cluster) path, 8 rows each
    (20, 8, 8, 3, 200, False),      # cluster path, 3 rows
    (4, 8, 8, 1, 20, True)])        # cluster path with most CTAs of a cluster idle
def test_fmha_decode_split_kv(dtype, d, b, hq, hkv, sq, sk, causal, device_ok, monkeypatch):
    q, k, v = _qkv(b, hq, hkv, sq, sk, d, dtype, b + hq + sk)
    group = hq // hkv
    input_pos = sk - sq if causal else 0
    args = dict(query_group_size=group, causal=causal, input_pos=input_pos)
    out = b200k.cutile_fmha(q.cuda(), k.cuda(), v.cuda(), **args)
    ref = oracle.fmha_ref(q, k, v, **args)
    torch.testing.assert_close(out.float().cpu(), ref, **TOL)
    # the tensor-core kernels on the same inputs agree with the split-KV path
    monkeypatch.setenv("B200K_FMHA_NO_DECODE", "1")
    out_tc = b200k.cutile_fmha(q.cuda(), k.cuda(), v.cuda(), **args)
    torch.testing.assert_close(out.float(), out_tc.float(), **TOL)


@pytest.mark.parametrize("plan", ["1", "2", "4", "8", "s", "3", "16"])   # 3 and 16 are ignored
@pytest.mark.parametrize("b,hq,hkv,sq,sk,causal", [
    (2, 8, 8, 1, 777, True),        # one row, ragged last batch, masked tail CTAs for large clusters
    (1, 16, 4, 2, 1300, True),      # eight rows (sixteen lanes per key), two query positions under the mask
    (3, 12, 4, 1, 96, False)])      # three rows of a four-row kernel (row predicates), short keys
def test_fmha_decode_every_plan(plan, b, hq, hkv, sq, sk, causal, device_ok, monkeypatch):
    # every cluster size of the one-kernel path and the two-kernel path give the oracle's result
    monkeypatch.setenv("B200K_DECODE_PLAN", plan)
    q, k, v = _qkv(b, hq, hkv, sq, sk, 128, torch.bfloat16, 3 * b + sk)
    args = dict(query_group_size=hq // hkv, causal=causal, input_pos=sk - sq if causal else 0)
    out = b200k.cutile_fmha(q.cuda(), k.cuda(), v.cuda(), **args)
    torch.testing.assert_close(out.float().cpu(), oracle.fmha_ref(q, k, v, **args), **TOL)


def test_fmha_decode_mid_sequence_position(device_ok):
    # input_pos in the middle of a longer cache: keys beyond the position are never read
    q, k, v = _qkv(1, 8, 8, 1, 2048, 128, torch.bfloat16, 77)
    out = b200k.cutile_fmha(q.cuda(), k.cuda(), v.cuda(), causal=True, input_pos=700)
    ref = oracle.fmha_ref(q, k[:, :, :701], v[:, :, :701], causal=False)
    torch.testing.assert_close(out.float().cpu(), ref, **TOL)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("sq,sk", [(257, 257), (640, 640), (300, 1000), (1024, 2048 + 17), (384, 64)])
def test_fmha_long_rows_head_dim_128(dtype, causal, sq, sk, device_ok):
    # several key steps per query tile, ragged tails in both directions, grouped-query heads
    q, k, v = _qkv(2, 4, 2, sq, sk, 128, dtype, sq * 3 + sk)
    input_pos = sk - sq if (causal and sk > sq) else 0
    out = b200k.cutile_fmha(q.cuda(), k.cuda(), v.cuda(), causal=causal, input_pos=input_pos,
                            query_group_size=2)
    ref = oracle.fmha_ref(q, k, v, causal=causal, input_pos=input_pos, query_group_size=2)
    torch.testing.assert_close(out.float().cpu(), ref, **TOL)


def test_fmha_bshd_storage_and_scale(device_ok):
    # (B, S, H, D) storage viewed as (B, H, S, D), explicit scale
    g = torch.Generator().manual_seed(5)
    q = torch.randn(2, 200, 4, 128, generator=g).bfloat16().transpose(1, 2)
    k = torch.randn(2, 200, 4, 128, generator=g).bfloat16().transpose(1, 2)
    v = torch.randn(2, 200, 4, 128, generator=g).bfloat16().transpose(1, 2)
    out = b200k.cutile_fmha(q.cuda(), k.cuda(), v.cuda(), qk_scale=0.05, causal=True)
    ref = oracle.fmha_ref(q, k, v, causal=True, qk_scale=0.05)
    torch.testing.assert_close(out.float().cpu(), ref, **TOL)


def test_fmha_large_score_range_exercises_rescale(device_ok):
    # growing score magnitudes along the keys force the running maximum up by far more
    # than the deferred-rescale threshold
    g = torch.Generator().manual_seed(6)
    q = torch.randn(1, 2, 256, 128, generator=g)
    k = torch.randn(1, 2, 1024, 128, generator=g) * torch.linspace(0.2, 6.0, 1024)[None, None, :, None]
    v = torch.randn(1, 2, 1024, 128, generator=g)
    q, k, v = q.bfloat16(), k.bfloat16(), v.bfloat16()
    out = b200k.cutile_fmha(q.cuda(), k.cuda(), v.cuda(), qk_scale=1.0 / math.sqrt(128))
    ref = oracle.fmha_ref(q, k, v)
    torch.testing.assert_close(out.float().cpu(), ref, atol=2e-2, rtol=5e-2)


def test_fmha_uniform_values_known_answer(device_ok):
    # identical keys -> uniform attention -> output = mean of the visible values
    q = torch.ones(1, 1, 128, 64, dtype=torch.float16)
    k = torch.ones(1, 1, 256, 64, dtype=torch.float16)
    v = torch.arange(256, dtype=torch.float32).remainder(16).reshape(1, 1, 256, 1).expand(1, 1, 256, 64).half()
    out = b200k.cutile_fmha(q.cuda(), k.cuda(), v.cuda().contiguous())
    torch.testing.assert_close(out.float().cpu(), torch.full((1, 1, 128, 64), 7.5), atol=1e-2, rtol=1e-2)


def test_fmha_bench_form_and_validation(device_ok):
    q, k, v = _qkv(1, 4, 2, 1, 256, 128, torch.float16, 9)     # decode with GQA
    o = torch.empty(1, 4, 1, 128, dtype=torch.float16, device="cuda")
    b200k.cutile_fmha_into(q.cuda(), k.cuda(), v.cuda(), o, True, True)
    ref = oracle.fmha_ref(q, k, v, causal=True, input_pos=255, query_group_size=2)
    torch.testing.assert_close(o.float().cpu(), ref, **TOL)
    with pytest.raises(ValueError, match="must be 4D"):
        b200k.cutile_fmha(q[0].cuda(), k.cuda(), v.cuda())
    with pytest.raises(ValueError, match="query_group_size must equal"):
        b200k.cutile_fmha(q.cuda(), k.cuda(), v.cuda())


def test_fmha_baseline_shape_slice(device_ok):
    # the benchmark-sized problem is (4, 32, 8192, 128) causal; one batch and 2 heads of it at full
    # sequence length against the oracle on sampled query rows, plus the row-sum property
    # that attention over a constant V returns that constant
    g = torch.Generator().manual_seed(3)
    q = torch.randn(1, 2, 8192, 128, generator=g).bfloat16()
    k = torch.randn(1, 2, 8192, 128, generator=g).bfloat16()
    v = torch.randn(1, 2, 8192, 128, generator=g).bfloat16()
    out = b200k.cutile_fmha(q.cuda(), k.cuda(), v.cuda(), causal=True).float().cpu()
    rows = torch.tensor([0, 1, 127, 128, 4095, 4096, 8191])
    for r in rows.tolist():
        ref = oracle.fmha_ref(q[:, :, r:r + 1], k[:, :, :r + 1], v[:, :, :r + 1])
        torch.testing.assert_close(out[:, :, r:r + 1], ref, **TOL)
    ones = torch.ones_like(v)
    const = b200k.cutile_fmha(q.cuda(), k.cuda(), ones.cuda(), causal=True).float().cpu()
    torch.testing.assert_close(const, torch.ones_like(const), atol=1e-2, rtol=1e-2)
