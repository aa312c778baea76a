"""Pins the CPU oracle to the reference: golden vectors produced by the reference's own
functions (tests/golden/make_golden.py) and the known-answer cases in its docstrings."""
import os

import numpy as np
import pytest
import torch

import oracle


def _u8(t):
    return t.view(torch.uint8).numpy()


def test_block_quantize_matches_reference_golden(golden_dir):
    g = np.load(os.path.join(golden_dir, "block_quantize.npz"))
    q, s = oracle.block_quantize_ref(torch.from_numpy(g["x"]))
    assert np.array_equal(_u8(q), g["q"])
    assert np.array_equal(_u8(s), g["scale"])
    qb, sb = oracle.block_quantize_ref(torch.from_numpy(g["xb"]))
    assert np.array_equal(_u8(qb), g["qb"])
    assert np.array_equal(_u8(sb), g["scaleb"])


def test_block_quantize_edge_rows(golden_dir):
    g = np.load(os.path.join(golden_dir, "block_quantize.npz"))
    s = g["scale"]
    assert s[0, 0] == 88          # all-zero block: clamp 1e-12 -> 2^-39
    assert s[1, 0] == 127         # amax 448 -> scale 1
    assert s[2, 0] == 122         # amax 448 * 2^-5
    assert s[4, 0] == 88          # below the clamp


def test_block_quantize_is_exact_rule_on_bf16_data():
    # smallest e with 448 * 2^e >= amax, for bf16-representable inputs
    gen = torch.Generator().manual_seed(5)
    x = (torch.randn(64, 512, generator=gen) * 10).bfloat16().float()
    _, s = oracle.block_quantize_ref(x)
    amax = x.reshape(64, -1, 32).abs().amax(-1).double().numpy()
    e = np.ceil(np.log2(np.maximum(amax / 448.0, 1e-300)))
    assert np.array_equal(_u8(s).astype(np.int64) - 127, e.astype(np.int64))


def test_swizzle_matches_reference_golden(golden_dir):
    g = np.load(os.path.join(golden_dir, "block_quantize.npz"))
    s = torch.from_numpy(g["scale"]).view(torch.float8_e8m0fnu)
    sw = oracle.swizzle_32_4_4_ref(s)
    assert np.array_equal(_u8(sw), g["swizzled"])
    assert np.array_equal(_u8(oracle.unswizzle_32_4_4_ref(sw)), g["scale"])


def test_swizzle_byte_rule():
    rows, ks = 256, 8
    s = torch.arange(rows * ks, dtype=torch.int64).remainder(251).to(torch.uint8).reshape(rows, ks)
    sw = _u8(oracle.swizzle_32_4_4_ref(s))
    for (r, k) in [(0, 0), (33, 5), (127, 3), (200, 7), (255, 4)]:
        assert sw[r // 128, k // 4, r % 32, ((r // 32) % 4) * 4 + k % 4] == s[r, k]


@pytest.mark.parametrize("case", list("abcde"))
def test_moe_align_matches_reference_golden(golden_dir, case):
    g = np.load(os.path.join(golden_dir, "moe_align.npz"))
    tokens, topk, experts, tile_m = g[f"{case}_cfg"].tolist()
    st, se = oracle.moe_align_ref(torch.from_numpy(g[f"{case}_ids"]), tile_m, experts)
    assert st.dtype == torch.int32 and se.dtype == torch.int32
    assert np.array_equal(st.numpy(), g[f"{case}_sorted_token_ids"])
    assert np.array_equal(se.numpy(), g[f"{case}_sorted_expert_ids"])


def test_moe_matches_reference_golden(golden_dir):
    g = np.load(os.path.join(golden_dir, "torch_moe.npz"))
    out = oracle.moe_ref(*(torch.from_numpy(g[k]) for k in
                           ("hidden", "w1", "w2", "topk_weights", "topk_ids")))
    np.testing.assert_allclose(out.numpy(), g["out"], rtol=1e-5, atol=1e-5)


def test_e2m1_table_and_packing():
    # value table and nibble order of test/test_mma_scaled.py:149-160
    assert oracle.E2M1_VALUES[:8].tolist() == [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    assert oracle.E2M1_VALUES[8:].tolist() == [-0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0]
    packed = np.array([[0x21, 0xF7]], dtype=np.uint8)
    assert oracle.e2m1_decode_packed(packed).tolist() == [[0.5, 1.0, 6.0, -6.0]]
    codes = np.array([[1, 2, 7, 15]], dtype=np.uint8)
    assert np.array_equal(oracle.e2m1_pack(codes), packed)


def test_e2m1_round_to_nearest_even():
    x = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0, -0.25, 0.2, 0.3, 100.0], dtype=np.float32)
    got = oracle.E2M1_VALUES[oracle.e2m1_encode_rne(x)]
    # ties go to the code with an even mantissa bit: 0.25->0, 0.75->1, 1.25->1, 1.75->2,
    # 2.5->2, 3.5->4, 5->4
    assert got.tolist() == [0.0, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0, 6.0, -0.0, 0.0, 0.5, 6.0]


def test_e8m0_decode():
    assert oracle.e8m0_decode(np.array([127, 128, 120], dtype=np.uint8)).tolist() == [1.0, 2.0, 2.0 ** -7]
    assert np.isnan(oracle.e8m0_decode(np.array([255], dtype=np.uint8))[0])


def test_mma_scaled_docstring_known_answers():
    # ones (16 x 32) . ones (32 x 16) with all scales 2 -> 2 * 2 * 32 = 128 per block pair;
    # the docstring case uses K = 64 (two blocks): 256 (src/cuda/tile/_stub.py:2248-2270)
    a = torch.ones(16, 64).to(torch.float8_e4m3fn)
    sa = torch.full((16, 2), 128, dtype=torch.uint8).view(torch.float8_e8m0fnu)
    ref = oracle.block_scaled_matmul_ref(a, sa, a, sa)
    assert torch.all(ref == 256.0)


def test_nvfp4_quantize_roundtrip_properties():
    gen = torch.Generator().manual_seed(9)
    x = torch.randn(64, 256, generator=gen)
    x[2, :16] = 0
    q, sf, st = oracle.nvfp4_quantize_ref(x)
    assert q.shape == (64, 128) and sf.shape == (64, 16)
    assert sf[2, 0] == 0 and not q[2, :8].any()
    d = oracle.nvfp4_dequantize_ref(q, sf, st)
    assert oracle.rel_frobenius(d, x) < 0.15
    # the largest element of the tensor maps to +-6 with block scale 448
    i = x.abs().argmax()
    r, c = divmod(int(i), 256)
    assert sf[r, c // 16] == 0x7E  # e4m3 448
    code = (q[r, c // 2] >> (4 * (c % 2))) & 7
    assert code == 7


def test_fmha_ref_matches_sdpa():
    gen = torch.Generator().manual_seed(3)
    q = torch.randn(1, 4, 15, 32, generator=gen)
    k = torch.randn(1, 2, 63, 32, generator=gen)
    v = torch.randn(1, 2, 63, 32, generator=gen)
    out = oracle.fmha_ref(q, k, v, causal=True, input_pos=48, query_group_size=2)
    mask = torch.arange(63)[None, :] <= (torch.arange(15)[:, None] + 48)
    ref = torch.nn.functional.scaled_dot_product_attention(
        q, k.repeat_interleave(2, 1), v.repeat_interleave(2, 1), attn_mask=mask)
    torch.testing.assert_close(out, ref, rtol=1e-5, atol=1e-5)
