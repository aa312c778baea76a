"""AllGather GEMM: out[(p * M + m), :] = inp_p[m, :] @ w on every rank
(samples/AllGatherMatmul.py:85-175: 256 x 1024 fp32 per rank, w 1024 x 512, checked against
all_gather_into_tensor + matmul with atol = rtol = 1e-3).

CPU part: layout helpers and a world-size-2 gloo run of the gather semantics.
GPU part (needs >= 2 GPUs, one process per GPU over NCCL): the p2p and nccl transports
against the fp32 CPU oracle, for fp32 (tf32), bf16 and NVFP4 operands.
"""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_shard_rows():
    from b200k import shard_rows
    assert shard_rows(8192, 8, 0) == (0, 1024)
    assert shard_rows(8192, 8, 7) == (7168, 8192)
    with pytest.raises(ValueError):
        shard_rows(100, 8, 0)


def _gloo_worker(rank, world, port, q):
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    torch.manual_seed(52 + rank)
    inp = torch.rand(64, 96)
    g = torch.Generator().manual_seed(7)
    w = torch.rand(96, 32, generator=g)
    parts = [torch.empty_like(inp) for _ in range(world)]
    dist.all_gather(parts, inp)
    # rank p's shard lands in rows [p * M, (p + 1) * M): the layout peer_gather produces
    from b200k import shard_rows
    full = torch.cat(parts)
    lo, hi = shard_rows(full.shape[0], world, rank)
    ok = torch.equal(full[lo:hi], inp)
    out = oracle.matmul_ref(full, w)
    sums = out.sum().reshape(1).clone()
    dist.all_reduce(sums)                       # every rank holds the same full product
    ok = ok and abs(sums.item() - world * out.sum().item()) < 1e-2
    q.put((rank, ok))
    dist.destroy_process_group()


def test_gather_layout_gloo_world2():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_gloo_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(60)
    assert sorted(results) == [(0, True), (1, True)]


# ---------------------------------------------------------------------------------------
def _nccl_worker(rank, world, port, q):
    try:
        import torch.distributed._symmetric_memory as symm_mem
        import b200k
        device = torch.device("cuda", rank)
        torch.cuda.set_device(device)
        dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank,
                                world_size=world, device_id=device)
        group = dist.group.WORLD
        failures = []

        def check(name, got, want, **tol):
            try:
                torch.testing.assert_close(got.float().cpu(), want, **tol)
            except AssertionError as e:
                failures.append(f"{name}: {str(e)[:300]}")

        def gather_cpu(t):
            parts = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(parts, t)
            return torch.cat(parts).cpu()

        # the sample's problem: fp32 (tf32 on the tensor cores), uniform [0, 1) inputs
        torch.manual_seed(52 + rank)
        ref_inp = torch.rand(256, 1024, device=device)
        inp = symm_mem.empty(256, 1024, device=device).copy_(ref_inp)
        torch.manual_seed(7)
        w = torch.rand(1024, 512, device=device)
        dist.barrier()
        want = oracle.matmul_ref(gather_cpu(ref_inp), w.cpu())
        out = b200k.cutile_gather_matmul(inp, w, group)
        assert out.shape == (256 * world, 512)
        check("fp32 p2p", out, want, atol=1e-3, rtol=1e-3)
        check("fp32 nccl", b200k.cutile_gather_matmul(ref_inp, w, group, transport="nccl"), want,
              atol=1e-3, rtol=1e-3)
        dist.barrier()

        # bf16, N(0,1)
        torch.manual_seed(100 + rank)
        ref_b = torch.randn(384, 512, device=device).bfloat16()
        inp_b = symm_mem.empty(384, 512, device=device, dtype=torch.bfloat16).copy_(ref_b)
        torch.manual_seed(8)
        wb = torch.randn(512, 768, device=device).bfloat16()
        dist.barrier()
        want = oracle.matmul_ref(gather_cpu(ref_b), wb.cpu())
        check("bf16 p2p", b200k.cutile_gather_matmul(inp_b, wb, group), want, atol=2e-1, rtol=2e-2)
        dist.barrier()

        # NVFP4: each rank quantises its own rows; weights identical on every rank
        torch.manual_seed(200 + rank)
        a = torch.randn(256, 1024, device=device).bfloat16()
        torch.manual_seed(9)
        wn = (0.02 * torch.randn(512, 1024, device=device)).bfloat16()
        aq, asf, ats = b200k.nvfp4_quantize(a)
        wq, wsf, wts = b200k.nvfp4_quantize(wn)
        s_q = symm_mem.empty(aq.shape, device=device, dtype=torch.uint8).copy_(aq)
        s_sf = symm_mem.empty(asf.shape, device=device, dtype=torch.uint8).copy_(asf.view(torch.uint8))
        s_ts = symm_mem.empty(1, device=device, dtype=torch.float32).copy_(ats)
        dist.barrier()
        out = b200k.cutile_gather_matmul_nvfp4(s_q, s_sf, s_ts, wq, wsf, wts, group, out_dtype=torch.float32)
        a_all = gather_cpu(a)
        rows = []
        for p in range(world):
            qa = oracle.nvfp4_quantize_ref(a_all[p * 256:(p + 1) * 256])
            rows.append(oracle.nvfp4_matmul_ref(*qa, *oracle.nvfp4_quantize_ref(wn.cpu())))
        want = torch.cat(rows)
        check("nvfp4 p2p", out, want, atol=1e-4 * float(want.abs().max()), rtol=1e-3)
        dist.barrier()

        torch.cuda.synchronize()
        code, info = b200k.device_status()
        if code:
            failures.append(f"device status {code} {info:#x}")
        q.put((rank, failures))
        dist.destroy_process_group()
    except Exception as e:  # report instead of hanging the parent
        import traceback
        q.put((rank, [traceback.format_exc()[-1500:]]))


@pytest.mark.gpu
def test_gather_matmul_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    env = {"NCCL_NVLS_ENABLE": "0"}
    os.environ.update(env)
    procs = [ctx.Process(target=_nccl_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=600) for _ in procs]
    for p in procs:
        p.join(120)
    for rank, failures in results:
        assert not failures, f"rank {rank}: {failures}"
