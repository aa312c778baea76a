"""Expert-parallel MoE: experts and tokens sharded over ranks, rows pushed to the expert's owner
and results pushed back (no counterpart in the reference; the result must equal the
single-process oracle, oracle.moe_ref, which follows torch_moe, samples/MoE.py:292-334).

CPU: the placement arithmetic of the dispatch (csrc/moe_ep_plan.h, the header the planning
kernel includes, compiled with g++) on random routing tables, and a world-size-2 gloo run that
moves real rows to the positions that arithmetic gives and computes the FFN there.
GPU: the CUDA path for several ranks emulated on one GPU (bf16 and MXFP8 experts), a world of
one against the single-GPU operator, a barrier whose peer never arrives, and the two-process
NCCL run on two GPUs.
"""
import ctypes
import os
import shutil
import socket
import subprocess

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _problem(world, tokens_per_rank, hidden, experts, inter, topk, dtype, seed=4):
    g = torch.Generator().manual_seed(seed)
    t = world * tokens_per_rank
    x = (0.5 * torch.randn(t, hidden, generator=g)).to(dtype)
    w1 = (0.1 * torch.randn(experts, 2 * inter, hidden, generator=g)).to(dtype)
    w2 = (0.1 * torch.randn(experts, hidden, inter, generator=g)).to(dtype)
    tw, ids = oracle.moe_route_ref(torch.randn(t, experts, generator=g), topk)
    return x, w1, w2, tw.to(dtype), ids


# ---- placement arithmetic on the host ---------------------------------------------------------
_HARNESS = r"""
#include <stdint.h>
#include "moe_ep_plan.h"
using namespace b200k;
// The planning kernel's per-expert work, in the kernel's own terms, for one rank.
extern "C" void host_ep_plan(const int32_t* hist, int world, int rank, int experts, int tile,
                             int64_t* first_row, int32_t* tile_group, int32_t* num_row_tiles,
                             int64_t* total, int64_t* tile_start) {
  const int local = experts / world;
  for (int e = 0; e < experts; ++e) {
    first_row[e] = ep_first_row(hist, world, experts, local, tile, rank, e);
    total[e] = ep_total(hist, world, experts, e);
    tile_start[e] = ep_tile_start(hist, world, experts, local, tile, e);
    if (ep_owner(e, local) != rank) continue;
    const int64_t tiles = ep_tiles(total[e], tile);
    for (int64_t t = 0; t < tiles; ++t) tile_group[tile_start[e] + t] = e - rank * local;
    if (e == (rank + 1) * local - 1) *num_row_tiles = (int32_t)(tile_start[e] + tiles);
  }
}
extern "C" int64_t host_ep_capacity(int64_t replicas, int world, int local, int tile) {
  return ep_capacity_rows(replicas, world, local, tile);
}
"""


def _build_plan_harness(directory):
    cxx = shutil.which("g++") or shutil.which("c++")
    if cxx is None:
        return None
    src = os.path.join(directory, "ep_plan_harness.cpp")
    lib = os.path.join(directory, "ep_plan_harness.so")
    with open(src, "w") as f:
        f.write(_HARNESS)
    subprocess.run([cxx, "-O1", "-shared", "-fPIC", "-I", os.path.join(ROOT, "cutile-python_b200", "csrc"),
                    src, "-o", lib], check=True)
    return lib


def _host_plan(lib_path, hist, rank, tile):
    """(first_row, tile_group, num_row_tiles, total, tile_start) for `rank` from the (world,
    experts) table."""
    h = ctypes.CDLL(lib_path)
    h.host_ep_capacity.restype = ctypes.c_int64
    world, experts = hist.shape
    hist = hist.to(torch.int32).contiguous()
    cap = h.host_ep_capacity(ctypes.c_int64(int(hist.sum())), 1, experts // world, tile)
    first = torch.zeros(experts, dtype=torch.int64)
    total = torch.zeros(experts, dtype=torch.int64)
    start = torch.zeros(experts, dtype=torch.int64)
    group = torch.full((cap // tile,), -7, dtype=torch.int32)
    n = torch.zeros(1, dtype=torch.int32)
    h.host_ep_plan(ctypes.c_void_p(hist.data_ptr()), world, rank, experts, tile,
                   ctypes.c_void_p(first.data_ptr()), ctypes.c_void_p(group.data_ptr()),
                   ctypes.c_void_p(n.data_ptr()), ctypes.c_void_p(total.data_ptr()),
                   ctypes.c_void_p(start.data_ptr()))
    return first, group, int(n), total, start


@pytest.fixture(scope="module")
def plan_lib(tmp_path_factory):
    lib = _build_plan_harness(str(tmp_path_factory.mktemp("ep_plan")))
    if lib is None:
        pytest.skip("no C++ compiler")
    return lib


@pytest.mark.parametrize("world,experts,tile", [(1, 8, 256), (2, 8, 4), (4, 64, 256), (8, 64, 256), (8, 8, 128)])
def test_dispatch_placement_on_random_routing_tables(plan_lib, world, experts, tile):
    g = torch.Generator().manual_seed(world * 100 + experts)
    local = experts // world
    for trial in range(4):
        hist = torch.randint(0, 3 * tile if trial else 2, (world, experts), generator=g, dtype=torch.int32)
        if trial == 2:
            hist[:, ::3] = 0                          # experts nobody routes to
        plans = [_host_plan(plan_lib, hist, r, tile) for r in range(world)]
        total = hist.sum(0).long()
        for d in range(world):                        # one owner's receive buffer at a time
            first_d, group, n_tiles, tot, start = plans[d]
            assert torch.equal(tot, total)
            taken = torch.zeros(max(1, n_tiles) * tile, dtype=torch.int32)
            for e in range(d * local, (d + 1) * local):
                lo = int(start[e]) * tile
                tiles = -(-int(total[e]) // tile)
                assert group[int(start[e]):int(start[e]) + tiles].tolist() == [e - d * local] * tiles
                run = 0
                for s in range(world):                # source s writes hist[s][e] rows from its first_row
                    f = int(plans[s][0][e])
                    assert f == lo + run              # ranks in order inside the expert's run
                    taken[f:f + int(hist[s, e])] += 1
                    run += int(hist[s, e])
                assert run == int(total[e]) and lo + run <= (int(start[e]) + tiles) * tile
            assert int(taken.max()) <= 1              # no two rows share a slot
            assert int(taken.sum()) == int(total[d * local:(d + 1) * local].sum())
            assert n_tiles == sum(-(-int(total[e]) // tile) for e in range(d * local, (d + 1) * local))
            # the worst-case capacity covers it
            h = ctypes.CDLL(plan_lib)
            h.host_ep_capacity.restype = ctypes.c_int64
            replicas = int(hist.sum(1).max())
            assert n_tiles * tile <= h.host_ep_capacity(ctypes.c_int64(replicas), world, local, tile)


def _ffn_rows(rows, expert_of_row, weights, w1, w2):
    inter = w2.shape[2]
    y = torch.zeros_like(rows, dtype=torch.float32)
    for e in expert_of_row.unique().tolist():
        if e < 0:
            continue
        sel = (expert_of_row == e).nonzero().squeeze(1)
        h = rows[sel].float() @ w1[e].float().T
        act = torch.nn.functional.silu(h[:, :inter]) * h[:, inter:]
        y[sel] = (act @ w2[e].float().T) * weights[sel].unsqueeze(1)
    return y


def _exchange(parts):
    """parts[d] (n_d, width) goes to rank d; returns what every rank sent here, concatenated."""
    world, width = len(parts), parts[0].shape[1]
    sc = torch.tensor([p.shape[0] for p in parts], dtype=torch.int64)
    rc = torch.empty(world, dtype=torch.int64)
    dist.all_to_all_single(rc, sc)
    out = torch.empty(int(rc.sum()), width)
    dist.all_to_all_single(out, torch.cat(parts), output_split_sizes=rc.tolist(), input_split_sizes=sc.tolist())
    return out


def _gloo_worker(rank, world, port, q, lib_path):
    try:
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
        experts, topk, tile, tpr, hidden = 8, 2, 4, 20, 32
        x, w1, w2, tw, ids = _problem(world, tpr, hidden, experts, 16, topk, torch.float32)
        local = experts // world
        lo, hi = rank * tpr, (rank + 1) * tpr
        xl, twl, idl = x[lo:hi], tw[lo:hi], ids[lo:hi]
        replicas = tpr * topk
        # count -> exchange of the table (the kernels push it; here all_gather)
        mine = torch.bincount(idl.reshape(-1), minlength=experts).to(torch.int32)
        table = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(table, mine)
        hist = torch.stack(table)
        first, group, n_tiles, total, start = _host_plan(lib_path, hist, rank, tile)
        # dispatch: every replica gets row first_row[e] + running count, on its expert's owner
        cursor = torch.zeros(experts, dtype=torch.int64)
        packets = [[] for _ in range(world)]
        for i, e in enumerate(idl.reshape(-1).tolist()):
            r = int(first[e] + cursor[e])
            cursor[e] += 1
            packets[e // local].append(torch.cat([torch.tensor([float(r), float(rank * replicas + i),
                                                                float(twl.reshape(-1)[i])]), xl[i // topk]]))
        recv = [_exchange([torch.stack(p) if p else torch.empty(0, 3 + hidden) for p in packets])]
        cap = group.numel() * tile
        rows = torch.zeros(cap, hidden)
        meta = torch.full((cap,), -1, dtype=torch.int64)
        weight = torch.zeros(cap)
        seen = torch.zeros(cap, dtype=torch.int32)
        for part in recv:
            r = part[:, 0].long()
            rows[r], meta[r], weight[r] = part[:, 3:], part[:, 1].long(), part[:, 2]
            seen[r] += 1
        ok = int(seen.max()) <= 1
        # experts: every live tile belongs to one local expert, padding rows carry no replica
        expert_of_row = group[:n_tiles].repeat_interleave(tile).long()
        expert_of_row = torch.where(meta[:n_tiles * tile] >= 0, expert_of_row, torch.full_like(expert_of_row, -1))
        w1l, w2l = w1[rank * local:(rank + 1) * local], w2[rank * local:(rank + 1) * local]
        y = _ffn_rows(rows[:n_tiles * tile], expert_of_row, weight[:n_tiles * tile], w1l, w2l)
        # combine: every result row goes back to the rank and replica slot its meta names
        live = (meta[:n_tiles * tile] >= 0).nonzero().squeeze(1)
        back = [[] for _ in range(world)]
        for r in live.tolist():
            back[int(meta[r]) // replicas].append(torch.cat([torch.tensor([float(int(meta[r]) % replicas)]), y[r]]))
        recv = [_exchange([torch.stack(p) if p else torch.empty(0, 1 + hidden) for p in back])]
        y_back = torch.zeros(replicas, hidden)
        for part in recv:
            y_back[part[:, 0].long()] = part[:, 1:]
        out = y_back.reshape(tpr, topk, hidden).sum(1)
        ref = oracle.moe_ref(x, w1, w2, tw, ids)[lo:hi]
        q.put((rank, ok and bool(torch.allclose(out, ref, atol=1e-4, rtol=1e-4))))
        dist.destroy_process_group()
    except Exception:
        import traceback
        q.put((rank, traceback.format_exc()[-2500:]))


def test_expert_parallel_dispatch_and_combine_gloo_world2(plan_lib):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_gloo_worker, args=(r, 2, port, q, plan_lib)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=180) for _ in procs)
    for p in procs:
        p.join(60)
    assert results == [(0, True), (1, True)], results


# ---- CUDA path ----------------------------------------------------------------------------------
def _reference(x, w1, w2, tw, ids, mxfp8):
    if not mxfp8:
        return oracle.moe_ref(x, w1, w2, tw, ids)
    q1, s1 = oracle.block_quantize_ref(w1)
    q2, s2 = oracle.block_quantize_ref(w2)
    return oracle.moe_mxfp8_ref(x, q1, s1, q2, s2, tw, ids)


@pytest.mark.gpu
@pytest.mark.parametrize("mxfp8", [False, True])
@pytest.mark.parametrize("world,tpr,hidden,experts,inter,topk", [
    (2, 64, 512, 8, 128, 2), (4, 300, 512, 16, 256, 4), (8, 33, 1024, 64, 128, 8),
    (2, 100, 512, 6, 96, 3)])       # intermediate not a multiple of 128: unfused SiLU (bf16 only)
def test_expert_parallel_moe_emulated_ranks_one_gpu(world, tpr, hidden, experts, inter, topk, mxfp8, device_ok):
    import b200k
    if mxfp8 and inter % 128:
        pytest.skip("MXFP8 experts need an intermediate size that is a multiple of 128")
    x, w1, w2, tw, ids = _problem(world, tpr, hidden, experts, inter, topk, torch.bfloat16, seed=world + tpr)
    per = experts // world
    moes = [b200k.ExpertParallelMoE(w1[r * per:(r + 1) * per].cuda(), w2[r * per:(r + 1) * per].cuda(), experts,
                                    mxfp8=mxfp8, world=world, rank=r) for r in range(world)]
    cut = lambda t: [t[r * tpr:(r + 1) * tpr].cuda() for r in range(world)]
    ref = _reference(x, w1, w2, tw, ids, mxfp8)
    for attempt in range(2):        # a second layer over the same buffers: stale contents must not matter
        outs = b200k.emulate_ranks(moes, cut(x), cut(tw), cut(ids))
        out = torch.cat(outs)
        assert out.shape == x.shape and out.dtype == torch.bfloat16
        assert oracle.rel_frobenius(out, ref) < 2e-2
        torch.testing.assert_close(out.float().cpu(), ref, rtol=1e-1, atol=1e-1)
    # what each rank received: exactly the replicas routed to its experts, once each
    replicas = tpr * topk
    flat = ids.reshape(-1)
    for r, m in enumerate(moes):
        n_tiles = int(m.num_row_tiles)
        meta = m.own["meta"][: n_tiles * 256].cpu()
        got = sorted(meta[meta >= 0].tolist())
        want = sorted(i for i in range(world * replicas) if int(flat[i]) // per == r)
        assert got == want
        owner_expert = m.tile_group[:n_tiles].cpu().repeat_interleave(256)
        live = meta >= 0
        assert torch.equal(owner_expert[live].long() + r * per, flat[meta[live].long()])


@pytest.mark.gpu
@pytest.mark.parametrize("mxfp8", [False, True])
def test_expert_parallel_moe_world_of_one_equals_the_single_gpu_operator(mxfp8, device_ok):
    import b200k
    x, w1, w2, tw, ids = _problem(1, 500, 512, 16, 256, 4, torch.bfloat16, seed=9)
    ids[7, 1] = 99                                       # one routing entry outside the expert range
    ep = b200k.ExpertParallelMoE(w1.cuda(), w2.cuda(), 16, mxfp8=mxfp8)
    out = ep.forward(x.cuda(), tw.cuda(), ids.cuda())
    torch.cuda.synchronize()
    code, info = b200k.device_status()
    assert code != 0 and (info >> 8) & 0xff == 40        # reported; the entry contributes nothing
    if mxfp8:
        w1q, w1s = b200k.quantize_expert_weights(w1.cuda())
        w2q, w2s = b200k.quantize_expert_weights(w2.cuda())
        single = b200k.cutile_moe_mxfp8(x.cuda(), w1q, w1s, w2q, w2s, tw.cuda(), ids.cuda())
    else:
        single = b200k.cutile_moe(x.cuda(), w1.cuda(), w2.cuda(), tw.cuda(), ids.cuda())
    torch.cuda.synchronize()
    b200k.device_status()
    # same arithmetic, rows in a different order inside the tiles: equal up to fp32 summation order
    torch.testing.assert_close(out.float(), single.float(), rtol=2e-2, atol=2e-2)
    tw_eff = tw.clone()
    tw_eff[7, 1] = 0
    ref = _reference(x, w1, w2, tw_eff, ids.clamp(0, 15), mxfp8)
    assert oracle.rel_frobenius(out, ref) < 2e-2


@pytest.mark.gpu
def test_a_barrier_whose_peer_never_arrives_returns_and_is_reported():
    # two "ranks" whose flag arrays are local buffers nobody else writes: rank 0's wait for rank 1
    # runs out of its one-millisecond budget; the kernel returns and the status word names the wait
    import b200k
    from b200k import _lib
    flags = [torch.zeros(2, dtype=torch.int32, device="cuda") for _ in range(2)]
    epoch = torch.zeros(1, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    assert b200k.device_status() == (0, 0)
    arr = (ctypes.c_void_p * 2)(*[f.data_ptr() for f in flags])
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    _lib.check(_lib.lib().b200k_peer_barrier(ctypes.cast(arr, ctypes.POINTER(ctypes.c_void_p)), 2, 0,
                                             epoch.data_ptr(), 1000, _lib.stream_ptr(epoch.device)))
    stop.record()
    torch.cuda.synchronize()
    assert start.elapsed_time(stop) < 100.0
    code, info = b200k.device_status()
    assert code == _lib.TIMEOUT and (info >> 8) & 0xff == 60 and (info >> 16) == 1    # waited for rank 1
    assert int(epoch) == 1 and flags[0].tolist() == [1, 0] and flags[1].tolist() == [1, 0]
    # once the peer's flag is there the same barrier passes at once
    flags[0][1] = 2
    _lib.check(_lib.lib().b200k_peer_barrier(ctypes.cast(arr, ctypes.POINTER(ctypes.c_void_p)), 2, 0,
                                             epoch.data_ptr(), 1000, _lib.stream_ptr(epoch.device)))
    torch.cuda.synchronize()
    assert b200k.device_status() == (0, 0) and int(epoch) == 2


def _nccl_worker(rank, world, port, q):
    try:
        import b200k
        device = torch.device("cuda", rank)
        torch.cuda.set_device(device)
        dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank,
                                world_size=world, device_id=device)
        failures = []
        for mxfp8 in (False, True):
            for (tpr, hidden, experts, inter, topk) in [(64, 512, 8, 128, 2), (300, 512, 16, 256, 4)]:
                x, w1, w2, tw, ids = _problem(world, tpr, hidden, experts, inter, topk, torch.bfloat16)
                per = experts // world
                lo, hi = rank * tpr, (rank + 1) * tpr
                ep = b200k.ExpertParallelMoE(w1[rank * per:(rank + 1) * per].cuda(),
                                             w2[rank * per:(rank + 1) * per].cuda(), experts, mxfp8=mxfp8)
                ref = _reference(x, w1, w2, tw, ids, mxfp8)[lo:hi]
                for layer in range(3):      # back-to-back layers reuse the buffers across ranks
                    out = ep.forward(x[lo:hi].cuda(), tw[lo:hi].cuda(), ids[lo:hi].cuda())
                err = oracle.rel_frobenius(out, ref)
                if not (err < 2e-2):
                    failures.append(f"mxfp8={mxfp8} tokens/rank {tpr}: relative error {err}")
                try:
                    torch.testing.assert_close(out.float().cpu(), ref, rtol=1e-1, atol=1e-1)
                except AssertionError as e:
                    failures.append(str(e)[:300])
        torch.cuda.synchronize()
        code, info = b200k.device_status()
        if code:
            failures.append(f"device status {code} {info:#x}")
        q.put((rank, failures))
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        import traceback
        q.put((rank, [traceback.format_exc()[-1500:]]))


@pytest.mark.gpu
def test_expert_parallel_moe_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_nccl_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=600) for _ in procs]
    for p in procs:
        p.join(120)
    for rank, failures in results:
        assert not failures, f"rank {rank}: {failures}"
