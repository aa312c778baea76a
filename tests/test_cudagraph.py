"""Every operator is capturable in a CUDA graph and replays on new input contents.

The reference states this for its launch path (test/test_cudagraph.py:17-57: a launch inside
`torch.cuda.graph`, replayed N times, acts N times on the captured buffers).  Here each case
runs the operator once eagerly (first-use set-up such as kernel attributes and the status word
happens outside the capture, as torch asks of any captured code), captures one call, then
replays it after the inputs were overwritten in place and compares with an eager call on the
same contents.  Nothing in a wrapper may synchronise or read device data on the host, or the
capture itself fails.
"""
import pytest
import torch

import b200k

pytestmark = pytest.mark.gpu


def _capture_and_replay(make_inputs, run, refresh):
    """`make_inputs()` -> list of static input tensors; `run(*inputs)` -> output tensor(s);
    `refresh(inputs)` overwrites the inputs in place."""
    inputs = make_inputs()
    run(*inputs)                                   # eager warm-up, outside the capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = run(*inputs)
    outs = out if isinstance(out, (tuple, list)) else (out,)
    for _ in range(2):
        refresh(inputs)
        graph.replay()
        torch.cuda.synchronize()
        got = [o.clone() for o in outs]
        want = run(*inputs)
        want = want if isinstance(want, (tuple, list)) else (want,)
        for g, w in zip(got, want):
            if g.dtype.itemsize == 1:
                # quantised bytes and scales are deterministic
                assert torch.equal(g.view(torch.uint8), w.view(torch.uint8))
            else:
                # sums over K: the two MMA issuers interleave differently from run to run, so
                # the fp32 summation order (and the last bit of the result) may differ
                torch.testing.assert_close(g.float(), w.float(), rtol=1e-2,
                                           atol=1e-2 * float(w.float().abs().max()))
    code, info = b200k.device_status()
    assert code == 0, f"device status {code}, info {info:#x}"


def _randn_(t):
    if t.dtype.is_floating_point and t.dtype.itemsize >= 2:
        t.normal_()


def _refresh_all(inputs):
    for t in inputs:
        _randn_(t)


@pytest.mark.parametrize("m,n,k", [(512, 768, 1024), (256, 256, 4096)])   # pair kernel; split-K + reduce
def test_matmul_replays(m, n, k):
    _capture_and_replay(
        lambda: [torch.randn(m, k, device="cuda").half(), torch.randn(k, n, device="cuda").half()],
        lambda a, b: b200k.cutile_matmul(a, b), _refresh_all)


def test_replays_accumulate_like_repeated_launches():
    # N replays == N launches: a captured C = A @ C chain advances once per replay
    a = torch.eye(256, device="cuda").half() * 2
    c = torch.ones(256, 256, device="cuda").half()
    tmp = torch.empty_like(c)
    b200k.cutile_matmul(a, c, C=tmp)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        b200k.cutile_matmul(a, c, C=tmp)
        c.copy_(tmp)
    for _ in range(4):
        graph.replay()
    torch.cuda.synchronize()
    assert torch.all(c == 16)


def test_batch_matmul_fp8_replays():
    def make():
        return [torch.randn(2, 256, 400, device="cuda").to(torch.float8_e4m3fn),
                torch.randn(2, 400, 512, device="cuda").to(torch.float8_e4m3fn),
                torch.empty(2, 256, 512, device="cuda")]

    def refresh(inp):
        inp[0].copy_(torch.randn(2, 256, 400, device="cuda").to(torch.float8_e4m3fn))

    _capture_and_replay(make, lambda a, b, c: b200k.cutile_batch_matmul(2, a, b, c), refresh)


def test_group_matmul_replays():
    # a list of problems (the reference's launch refuses list arguments under capture:
    # test/test_cudagraph.py:60-75): one launch, its problem table carried in the kernel parameters
    shapes = [(128, 256, 512), (300, 200, 256), (64, 64, 64), (1024, 1024, 256)]

    def make():
        return ([torch.randn(m, k, device="cuda").half() for m, n, k in shapes] +
                [torch.randn(k, n, device="cuda").half() for m, n, k in shapes])

    def run(*ts):
        return b200k.cutile_group_matmul(list(ts[:4]), list(ts[4:]))

    _capture_and_replay(make, run, _refresh_all)


def test_quantisers_and_block_scaled_matmul_replay():
    def make():
        return [torch.randn(384, 512, device="cuda").bfloat16(), torch.randn(640, 512, device="cuda").bfloat16()]

    def run_mx(a, b):
        aq, sa = b200k.block_quantize(a, 32, swizzled_scale=True)
        bq, sb = b200k.block_quantize(b, 32, swizzled_scale=True)
        return (b200k.cutile_block_scaled_matmul(aq, sa, bq.T, sb, out_dtype=torch.bfloat16), aq, sa)

    def run_nv(a, b):
        aq, asf, ats = b200k.nvfp4_quantize(a)
        bq, bsf, bts = b200k.nvfp4_quantize(b)
        return (b200k.cutile_nvfp4_matmul(aq, asf, ats, bq, bsf, bts), aq, asf, ats)

    _capture_and_replay(make, run_mx, _refresh_all)
    _capture_and_replay(make, run_nv, _refresh_all)


@pytest.mark.parametrize("seq_q,seq_k,heads_kv", [(512, 512, 8), (1, 1024, 8), (1, 1024, 2)])
def test_fmha_replays(seq_q, seq_k, heads_kv):
    heads = 8

    def make():
        return [torch.randn(2, heads, seq_q, 128, device="cuda").bfloat16(),
                torch.randn(2, heads_kv, seq_k, 128, device="cuda").bfloat16(),
                torch.randn(2, heads_kv, seq_k, 128, device="cuda").bfloat16()]

    def run(q, k, v):
        return b200k.cutile_fmha(q, k, v, causal=True, input_pos=seq_k - seq_q,
                                 query_group_size=heads // heads_kv)

    _capture_and_replay(make, run, _refresh_all)


@pytest.mark.parametrize("mxfp8", [False, True])
def test_moe_replays(mxfp8):
    tokens, hidden, inter, experts, topk = 300, 512, 256, 8, 2

    def make():
        logits = torch.randn(tokens, experts, device="cuda")
        w, ids = torch.topk(torch.softmax(logits, -1), topk)
        return [torch.randn(tokens, hidden, device="cuda").bfloat16(),
                (0.05 * torch.randn(experts, 2 * inter, hidden, device="cuda")).bfloat16(),
                (0.05 * torch.randn(experts, hidden, inter, device="cuda")).bfloat16(),
                w.bfloat16(), ids]

    def refresh(inp):
        inp[0].normal_()
        logits = torch.randn(tokens, experts, device="cuda")       # new routing: other tile counts
        w, ids = torch.topk(torch.softmax(logits, -1), topk)
        inp[3].copy_(w)
        inp[4].copy_(ids)

    if mxfp8:
        def run(x, w1, w2, tw, ids):
            q = run.q
            return b200k.cutile_moe_mxfp8(x, q[0], q[1], q[2], q[3], tw, ids)
        probe = make()
        run.q = b200k.quantize_expert_weights(probe[1]) + b200k.quantize_expert_weights(probe[2])
    else:
        def run(x, w1, w2, tw, ids):
            return b200k.cutile_moe(x, w1, w2, tw, ids)

    _capture_and_replay(make, run, refresh)
