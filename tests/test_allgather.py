"""AllGather GEMM: out[(p * M + m), :] = inp_p[m, :] @ w on every rank
(samples/AllGatherMatmul.py:85-175: 256 x 1024 fp32 per rank, w 1024 x 512, checked against
all_gather_into_tensor + matmul with atol = rtol = 1e-3).

CPU part: layout helpers, the peer-gather kernel's index arithmetic run on the host over
fake shards (the header the kernel includes, compiled with g++), and a world-size-2 gloo run
of the gather semantics.
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


_HARNESS = r"""
#include <stdint.h>
#include <string.h>
#include "peer_gather_index.h"
// The kernel's loop nest on the host: `threads` grid-stride workers walk the items exactly as
// the CUDA threads do and move 16 bytes per valid item.  hits[] counts writes per destination
// vector, first_peer[] records the peer of each worker's first valid item.
extern "C" void host_peer_gather(const uint8_t* const* shards, int world, int rank, int64_t rows,
                                 int64_t row_vecs, int64_t src_stride, uint8_t* dst,
                                 int64_t dst_stride, int64_t threads, int32_t* hits,
                                 int32_t* first_peer) {
  const int64_t items = b200k::peer_gather_items(world, rows, row_vecs);
  for (int64_t t = 0; t < threads; ++t) {
    first_peer[t] = -1;
    for (int64_t i = t; i < items; i += threads) {
      const b200k::PeerGatherItem it = b200k::peer_gather_item(i, world, rank, rows, row_vecs);
      if (!it.valid) continue;
      if (first_peer[t] < 0) first_peer[t] = it.peer;
      memcpy(dst + (int64_t(it.peer) * rows + it.row) * dst_stride + it.col * 16,
             shards[it.peer] + it.row * src_stride + it.col * 16, 16);
      hits[(int64_t(it.peer) * rows + it.row) * row_vecs + it.col] += 1;
    }
  }
}

// The bulk-copy kernel's loop nest on the host for a batch of dense gathers: blocks dealt over
// the jobs by peer_gather_batch_blocks, block b of a job walking its runs b, b + blocks, ...
// Returns the grid size, or -1 when a job got no block or the grid exceeds `sms` (+ jobs).
extern "C" int host_bulk_batch(const uint8_t* const* const* shards, uint8_t* const* dst,
                               const int64_t* shard_bytes, int jobs, int world, int rank, int sms,
                               int32_t* const* hits) {
  int64_t runs[b200k::kPeerGatherMaxBatch];
  int first[b200k::kPeerGatherMaxBatch + 1];
  for (int j = 0; j < jobs; ++j) runs[j] = b200k::peer_gather_runs(world, shard_bytes[j] / 16, 1);
  const int grid = b200k::peer_gather_batch_blocks(runs, jobs, sms, first);
  first[jobs] = grid;
  if (grid > (sms > jobs ? sms : jobs)) return -1;
  for (int j = 0; j < jobs; ++j) {
    const int blocks = first[j + 1] - first[j];
    if (blocks < 1) return -1;
    for (int block = 0; block < blocks; ++block) {
      for (int64_t run = block; run < runs[j]; run += blocks) {
        const b200k::PeerGatherRun r = b200k::peer_gather_run(run, world, rank);
        const int64_t off = r.first_vec * 16;
        if (off >= shard_bytes[j]) return -2;          // every run holds at least one vector
        const int64_t left = shard_bytes[j] - off;
        const int64_t bytes = left < 4096 ? left : 4096;
        memcpy(dst[j] + int64_t(r.peer) * shard_bytes[j] + off, shards[j][r.peer] + off, bytes);
        for (int64_t v = 0; v < bytes / 16; ++v) hits[j][(int64_t(r.peer) * shard_bytes[j] + off) / 16 + v] += 1;
      }
    }
  }
  return grid;
}
"""


@pytest.fixture(scope="module")
def host_gather(tmp_path_factory):
    """The index arithmetic of peer_gather_kernel (csrc/peer_gather_index.h, the header the
    kernel itself includes) compiled for the host."""
    import ctypes
    import shutil
    import subprocess
    cxx = shutil.which("g++") or shutil.which("c++")
    if cxx is None:
        pytest.skip("no C++ compiler")
    d = tmp_path_factory.mktemp("peer_gather")
    src = d / "harness.cpp"
    src.write_text(_HARNESS)
    lib = d / "harness.so"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    subprocess.run([cxx, "-O1", "-shared", "-fPIC", "-I", os.path.join(root, "cutile-python_b200", "csrc"),
                    str(src), "-o", str(lib)], check=True)
    handle = ctypes.CDLL(str(lib))
    fn = handle.host_peer_gather
    fn.restype = None

    def run(shards, rank, threads, dst_cols=None):
        world = len(shards)
        rows, cols = shards[0].shape
        row_vecs = cols * shards[0].element_size() // 16
        dst_cols = dst_cols or cols
        dst = torch.full((world * rows, dst_cols), -1, dtype=shards[0].dtype)
        hits = torch.zeros(world * rows * row_vecs, dtype=torch.int32)
        first = torch.zeros(threads, dtype=torch.int32)
        ptrs = (ctypes.c_void_p * world)(*[t.data_ptr() for t in shards])
        fn(ptrs, ctypes.c_int(world), ctypes.c_int(rank), ctypes.c_int64(rows), ctypes.c_int64(row_vecs),
           ctypes.c_int64(shards[0].stride(0) * shards[0].element_size()), ctypes.c_void_p(dst.data_ptr()),
           ctypes.c_int64(dst.stride(0) * dst.element_size()), ctypes.c_int64(threads),
           ctypes.c_void_p(hits.data_ptr()), ctypes.c_void_p(first.data_ptr()))
        return dst, hits, first

    run.batch = handle.host_bulk_batch
    run.batch.restype = ctypes.c_int
    return run


@pytest.mark.parametrize("world", [1, 2, 3, 8])
@pytest.mark.parametrize("rows,cols", [(8, 64), (5, 36), (96, 260), (1, 4)])   # fp32 columns
def test_peer_gather_index_math_on_fake_shards(host_gather, world, rows, cols):
    # shards with a row pitch wider than the payload, as a view into a larger allocation
    g = torch.Generator().manual_seed(world * 1000 + rows)
    backing = [torch.randn(rows, cols + 8, generator=g) for _ in range(world)]
    shards = [b[:, :cols] for b in backing]
    want = torch.cat(shards)
    for rank in range(world):
        for threads in (1, 7, 256 * 3):
            dst, hits, first = host_gather(shards, rank, threads, dst_cols=cols + 4)
            assert torch.equal(dst[:, :cols], want)                 # shard p -> rows [p * rows, ...)
            assert bool((dst[:, cols:] == -1).all())                # nothing outside the payload
            assert bool((hits == 1).all())                          # every vector moved exactly once
        # runs of 256 vectors are dealt round-robin over the peers, remote shards first
        _, _, first = host_gather(shards, rank, 256 * world)
        vecs = rows * cols * 4 // 16
        for slot in range(world):
            if vecs > 0:
                assert int(first[256 * slot]) == (rank + 1 + slot) % world
        if world > 1:
            assert int(first[0]) != rank and int(first[256 * (world - 1)]) == rank


@pytest.mark.parametrize("world", [1, 2, 5, 8])
@pytest.mark.parametrize("sizes,sms", [((4096 * 50, 4096 * 3), 148), ((4096 * 1024, 4096 * 128 + 48), 148),
                                       ((16, 16, 16, 16), 148), ((4096 * 9 + 160, 4096 * 200), 16),
                                       ((4096 * 3,), 2), ((4096 * 7, 32, 4096 * 40 + 16), 3)])
def test_bulk_batch_covers_every_vector_once(host_gather, world, sizes, sms):
    """The block distribution and run walk of the bulk-copy gather (one launch for several
    tensors): every 16-byte vector of every shard of every job is copied exactly once, every
    job owns at least one block, and the grid never exceeds one block per SM."""
    import ctypes
    g = torch.Generator().manual_seed(world + len(sizes) + sms)
    jobs = len(sizes)
    shards = [[torch.randint(0, 256, (nbytes,), generator=g, dtype=torch.uint8) for _ in range(world)] for nbytes in sizes]
    dst = [torch.zeros(world * nbytes, dtype=torch.uint8) for nbytes in sizes]
    hits = [torch.zeros(world * nbytes // 16, dtype=torch.int32) for nbytes in sizes]
    per_job = [(ctypes.c_void_p * world)(*[t.data_ptr() for t in job]) for job in shards]
    shard_tab = (ctypes.c_void_p * jobs)(*[ctypes.addressof(p) for p in per_job])
    dst_tab = (ctypes.c_void_p * jobs)(*[t.data_ptr() for t in dst])
    hit_tab = (ctypes.c_void_p * jobs)(*[t.data_ptr() for t in hits])
    size_tab = (ctypes.c_int64 * jobs)(*sizes)
    for rank in (0, world - 1):
        for t in dst + hits:
            t.zero_()
        grid = host_gather.batch(shard_tab, dst_tab, size_tab, ctypes.c_int(jobs), ctypes.c_int(world),
                                 ctypes.c_int(rank), ctypes.c_int(sms), hit_tab)
        assert 1 <= grid <= max(sms, jobs)
        for j in range(jobs):
            assert torch.equal(dst[j], torch.cat(shards[j]))
            assert bool((hits[j] == 1).all())


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


# ---------------------------------------------------------------------------------------
# The same path on ONE GPU: the shards of all ranks are local buffers handed over as explicit
# peers, and the ranks run one after the other (no kernel of this path waits on another).
@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 3, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gather_matmul_emulated_ranks_one_gpu(world, dtype, device_ok):
    import b200k
    g = torch.Generator().manual_seed(52 + world)
    m, k, n = (256, 1024, 512) if dtype == torch.float32 else (384, 512, 768)
    if dtype == torch.bfloat16 and world == 3:
        m = 512      # whole 256-row tiles per rank: own rows and the other ranks' rows as two overlapped GEMMs
    draw = torch.rand if dtype == torch.float32 else torch.randn    # the sample feeds uniform fp32
    shards = [draw(m, k, generator=g).to(dtype) for _ in range(world)]
    w = draw(k, n, generator=g).to(dtype)
    want = oracle.matmul_ref(torch.cat(shards), w)
    dev_shards = [s.cuda() for s in shards]
    tol = dict(atol=1e-3, rtol=1e-3) if dtype == torch.float32 else dict(atol=2e-1, rtol=2e-2)
    if dtype == torch.float32:      # tf32 products: the sample's tolerance holds for its [0, 1) data
        tol = dict(atol=1e-3 * float(want.abs().max()), rtol=1e-3)
    for rank in range(world):
        out = b200k.cutile_gather_matmul(dev_shards[rank], w.cuda(), peers=dev_shards, rank=rank)
        assert out.shape == (m * world, n) and out.dtype == dtype
        torch.testing.assert_close(out.float().cpu(), want, **tol)
    # the staging gather alone is a byte-exact concatenation, whatever the rank
    for rank in (0, world - 1):
        staged = b200k.peer_gather(dev_shards, rank)
        assert torch.equal(staged.cpu(), torch.cat(shards))


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 8])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_gather_matmul_whole_tile_shards_overlap(world, dtype, device_ok):
    """Shards of whole 256-row tiles: own rows and the other ranks' rows are two GEMMs on two
    streams (the second skips the own row tiles).  Against one GEMM over the concatenation
    (which may split K for so small a problem: another summation order) to a rounding step of
    the 16-bit output, and against the oracle."""
    import b200k
    g = torch.Generator().manual_seed(77 + world)
    m, k, n = 256, 384, 640
    shards = [torch.randn(m, k, generator=g).to(dtype).cuda() for _ in range(world)]
    w = torch.randn(k, n, generator=g).to(dtype).cuda()
    whole = b200k.cutile_matmul(torch.cat(shards), w)
    want = oracle.matmul_ref(torch.cat(shards).cpu(), w.cpu())
    for rank in range(world):
        out = b200k.cutile_gather_matmul(shards[rank], w, peers=shards, rank=rank)
        assert out.shape == (m * world, n) and out.dtype == dtype
        torch.testing.assert_close(out.float(), whole.float(), atol=2e-2 * float(want.abs().max()), rtol=1e-2)
        torch.testing.assert_close(out.float().cpu(), want, atol=2e-1, rtol=2e-2)
    assert b200k.device_status() == (0, 0)


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 5, 8])
@pytest.mark.parametrize("rows,cols", [(256, 4096), (100, 48), (7, 16), (1024, 512)])
def test_peer_gather_kernel_forms(world, rows, cols, device_ok, monkeypatch):
    """The bulk-copy form (dense shards), the load / store form (forced, and taken by itself
    for strided shards) and the batch entry give the byte-exact concatenation; shard sizes
    that end inside a 4 KB run included."""
    import ctypes
    import b200k
    from b200k import _lib
    g = torch.Generator().manual_seed(rows + cols + world)
    shards = [torch.randint(0, 256, (rows, cols), generator=g, dtype=torch.uint8).cuda() for _ in range(world)]
    want = torch.cat(shards)
    for rank in (0, world - 1):
        assert torch.equal(b200k.peer_gather(shards, rank), want)
        monkeypatch.setenv("B200K_GATHER", "ldst")
        assert torch.equal(b200k.peer_gather(shards, rank), want)
        monkeypatch.delenv("B200K_GATHER")
    # strided shards: views into wider buffers
    wide = [torch.zeros(rows, cols + 32, dtype=torch.uint8, device="cuda") for _ in range(world)]
    for w, sh in zip(wide, shards):
        w[:, :cols].copy_(sh)
    assert torch.equal(b200k.peer_gather([w[:, :cols] for w in wide], 1), want)
    # the batch entry: two gathers and a scalar expansion in one launch
    other = [torch.randint(0, 256, (rows, 32), generator=g, dtype=torch.uint8).cuda() for _ in range(world)]
    scal = [torch.full((1,), 1.5 + p, device="cuda") for p in range(world)]
    out_a, out_b = torch.zeros_like(want), torch.zeros(world * rows, 32, dtype=torch.uint8, device="cuda")
    out_s = torch.zeros(world * rows, device="cuda")
    args = (_lib.PeerGatherArgs * 2)()
    keep = []
    for a, sh, out in ((args[0], shards, out_a), (args[1], other, out_b)):
        ptrs = (ctypes.c_void_p * world)(*[t.data_ptr() for t in sh])
        keep.append(ptrs)
        a.shards = ctypes.cast(ptrs, ctypes.POINTER(ctypes.c_void_p))
        a.dst, a.rows, a.row_bytes = out.data_ptr(), rows, sh[0].shape[1]
        a.src_stride_bytes = a.dst_stride_bytes = a.row_bytes
        a.world, a.rank = world, world - 1
    sp = (ctypes.c_void_p * world)(*[t.data_ptr() for t in scal])
    _lib.check(_lib.lib().b200k_peer_gather_batch(args, 2, ctypes.cast(sp, ctypes.POINTER(ctypes.c_void_p)), rows,
                                                  out_s.data_ptr(), _lib.stream_ptr(want.device)))
    torch.cuda.synchronize()
    assert torch.equal(out_a, want) and torch.equal(out_b, torch.cat(other))
    assert torch.equal(out_s, torch.cat([s.expand(rows) for s in scal]))
    # a strided member is refused before anything is enqueued
    args[1].dst_stride_bytes = 64
    with pytest.raises(b200k.B200KError):
        _lib.check(_lib.lib().b200k_peer_gather_batch(args, 2, None, 0, None, _lib.stream_ptr(want.device)))
    assert b200k.device_status() == (0, 0)


@pytest.mark.gpu
@pytest.mark.parametrize("m", [128, 256, 512])   # 128: two remote GEMMs; 256, 512: one that skips the own rows
@pytest.mark.parametrize("world", [2, 4])
def test_gather_matmul_nvfp4_emulated_ranks_one_gpu(world, m, device_ok):
    import b200k
    g = torch.Generator().manual_seed(200 + world + m)
    k, n = 1024, 512
    shards = [(torch.randn(m, k, generator=g) * (1 + p)).bfloat16() for p in range(world)]
    wn = (0.02 * torch.randn(n, k, generator=g)).bfloat16()
    quant = [b200k.nvfp4_quantize(s.cuda()) for s in shards]     # each rank quantises its own rows
    wq, wsf, wts = b200k.nvfp4_quantize(wn.cuda())
    w_ref = oracle.nvfp4_quantize_ref(wn)
    want = torch.cat([oracle.nvfp4_matmul_ref(*oracle.nvfp4_quantize_ref(s), *w_ref) for s in shards])
    peers = ([q[0] for q in quant], [q[1] for q in quant], [q[2] for q in quant])
    for rank in range(world):
        out = b200k.cutile_gather_matmul_nvfp4(*quant[rank], wq, wsf, wts, out_dtype=torch.float32,
                                               peers=peers, rank=rank)
        assert out.shape == (m * world, n)
        torch.testing.assert_close(out.cpu(), want, atol=1e-4 * float(want.abs().max()), rtol=1e-3)
    # a plan kept across calls gives the same result again (staging buffers are reused)
    plan = b200k.Nvfp4GatherMatmul(*quant[1], peers=peers, rank=1)
    first = plan.run(wq, wsf, wts).clone()
    assert torch.equal(first, plan.run(wq, wsf, wts))
    torch.testing.assert_close(first.float().cpu(), want, atol=2e-2 * float(want.abs().max()), rtol=2e-2)
