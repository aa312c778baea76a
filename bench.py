"""Benchmark of the hot path on B200: TFLOPS of the block-scaled / dense contraction kernels.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload ag_nvfp4_gemm|mxfp8_gemm|nvfp4_gemm|dense_f16|fmha_causal|fmha_decode|
                                moe_bf16|moe_mxfp8|moe_sparse|moe_ep_bf16|moe_ep_mxfp8|mxfp8_quantize|nvfp4_quantize|
                                ref_shapes]

One step = one pass of the workload's kernels over one batch of seeded synthetic input.  Inputs
are drawn on the CPU from torch.Generator().manual_seed(seed) and copied to the device, so the
GPU arm, its parity check and the CPU arm see the same numbers.

The default workload is the path that shards: the NVFP4 FFN up-projection (M = 8192 tokens,
N = 28672, K = 8192, e2m1 operands with ue4m3 scales per 16 elements of K and one fp32 scale
per tensor, bf16 output) run as the AllGather GEMM.  A is row-sharded M / N_gpus per rank and
gathered over NVLink out of the peers' symmetric-memory buffers while the rank's own rows are
already being multiplied; every rank computes the full (M, N) product against its own
weights, so the work per rank is fixed (weak scaling) and at one GPU the workload is the plain
8192 x 28672 x 8192 NVFP4 GEMM.  The same JSON line carries the MXFP8 8192-cubed GEMM as a
secondary record (`also`).

Before anything is timed, one step's output is compared with the CPU oracle on sampled rows
(`parity_checked`, `max_err`), as the reference's benches do (test/bench_matmul.py:34-36,
111-112, test/bench_attention.py:58-69, test/bench_moe.py:58-68); a mismatch aborts the run.

`--impl reference` times the reference's CPU ground truth for the same workload (the
de-quantised fp32 matmul of samples/BlockScaledMatMul.py:359-361 and its siblings, restated in
oracle/) on the host cores, on a bounded block of the same inputs.

Prints ONE JSON line (rank 0).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "cutile-python_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

import torch  # noqa: E402

L2_BYTES = 126 * 1024 * 1024
NVLINK_PEER_COPY_GBS = 770.0    # measured peer copy per direction on this pool (nominal 900)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"bf16_tflops": float(d["bf16_tflops"]), "hbm_gbs": float(d["hbm_gbs"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


def bind_near_gpu(device) -> str:
    """Runs this process on the cores of the NUMA node the GPU hangs off, so that the pinned
    host buffers of the end-to-end leg are allocated there (first touch) and the ranks of one
    box do not all stream through one socket.  Best effort: returns what it did."""
    try:
        props = torch.cuda.get_device_properties(device)
        bdf = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bdf}/numa_node") as f:
            node = int(f.read().strip())
        if node < 0:
            return "no NUMA information"
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            cpus = set()
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if not allowed:
            return f"node {node}: none of its cores are available to this process"
        os.sched_setaffinity(0, allowed)
        return f"node {node}, {len(allowed)} cores"
    except Exception as e:  # pragma: no cover - depends on the box
        return f"unavailable ({type(e).__name__})"


def randn_rows(gen, rows: int, cols: int, take: int | None = None) -> torch.Tensor:
    """The first `take` rows of torch.randn(rows, cols, generator=gen).  For column counts that
    are multiples of 16 the CPU generator fills a tensor front to back in blocks of 16, so the
    leading rows of a large draw equal a smaller draw from the same state; a partial draw leaves
    the generator short of the full one, so only the LAST tensor of a sequence may be cut."""
    assert cols % 16 == 0
    return torch.randn(rows if take is None else min(take, rows), cols, generator=gen)


def close_or_die(name: str, got: torch.Tensor, ref: torch.Tensor, rtol: float, atol_rel: float) -> float:
    """Asserts |got - ref| <= atol_rel * max|ref| + rtol * |ref| elementwise; returns the
    largest error relative to max|ref|."""
    got, ref = got.detach().float().cpu(), ref.detach().float().cpu()
    scale = float(ref.abs().max()) or 1.0
    err = (got - ref).abs()
    bad = err > (atol_rel * scale + rtol * ref.abs())
    if bool(bad.any()) or not bool(torch.isfinite(got).all()):
        raise SystemExit(f"bench.py: parity check failed for {name}: {int(bad.sum())} of {bad.numel()} sampled "
                         f"values differ from the oracle (max error {float(err.max()):.4g}, scale {scale:.4g})")
    return float(err.max()) / scale


# --------------------------------------------------------------------------------------
# Workloads
# --------------------------------------------------------------------------------------
class Workload:
    name = ""
    dtype = ""
    tensor_rate_vs_bf16 = 1.0   # tensor-core rate of the operand format relative to bf16
    distributed = False         # needs a process group even on one GPU
    world, rank = 1, 0

    def config(self):
        raise NotImplementedError

    def parity(self) -> dict:
        raise NotImplementedError

    def launches(self) -> int:
        return getattr(self, "launches_per_step", 1)

    # ---- end-to-end leg as a two-slot software pipeline ---------------------------------
    # Every step still copies its inputs from pinned host memory and its result back to
    # pinned host memory; the H2D copy, the kernel and the D2H copy of consecutive steps run
    # on three streams, so the two directions of the host link and the GPU overlap.
    e2e_pipelined = False

    def pipe_setup(self, device, host_in, out_like):
        self.p_host_in = host_in
        self.p_dev_in = [[torch.empty_like(t, device=device) for t in host_in] for _ in range(2)]
        self.p_dev_out = [torch.empty_like(out_like) for _ in range(2)]
        self.p_host_out = [torch.empty_like(out_like, device="cpu").pin_memory() for _ in range(2)]
        self.p_streams = [torch.cuda.Stream(device) for _ in range(3)]
        self.p_ev = {k: [torch.cuda.Event() for _ in range(2)] for k in ("in", "comp", "out")}
        self.p_i = 0
        self.e2e_pipelined = True
        self.h2d = sum(t.numel() * t.element_size() for t in host_in)
        self.d2h = out_like.numel() * out_like.element_size()

    def pipe_step(self, compute):
        i, slot = self.p_i, self.p_i & 1
        self.p_i += 1
        s_in, s_comp, s_out = self.p_streams
        with torch.cuda.stream(s_in):
            if i >= 2:   # the kernel of step i - 2 has consumed this slot's device inputs
                s_in.wait_event(self.p_ev["comp"][slot])
            for d, h in zip(self.p_dev_in[slot], self.p_host_in):
                d.copy_(h, non_blocking=True)
            self.p_ev["in"][slot].record(s_in)
        with torch.cuda.stream(s_comp):
            s_comp.wait_event(self.p_ev["in"][slot])
            if i >= 2:   # the D2H copy of step i - 2 has drained this slot's device output
                s_comp.wait_event(self.p_ev["out"][slot])
            compute(self.p_dev_in[slot], self.p_dev_out[slot])
            self.p_ev["comp"][slot].record(s_comp)
        with torch.cuda.stream(s_out):
            s_out.wait_event(self.p_ev["comp"][slot])
            self.p_host_out[slot].copy_(self.p_dev_out[slot], non_blocking=True)
            self.p_ev["out"][slot].record(s_out)

    def e2e_begin(self):
        if self.e2e_pipelined:
            self.p_i = 0
            for st in self.p_streams:
                st.wait_stream(torch.cuda.current_stream())

    def e2e_end(self):
        if self.e2e_pipelined:
            for st in self.p_streams:
                torch.cuda.current_stream().wait_stream(st)


def _sample(n: int, fixed, count: int, seed: int) -> torch.Tensor:
    """Sorted sample of `count` indices below n that always contains `fixed` (tile seams)."""
    g = torch.Generator().manual_seed(seed)
    pick = torch.randperm(n, generator=g)[:count].tolist()
    return torch.tensor(sorted(set(i for i in fixed if 0 <= i < n) | set(pick)))


class Mxfp8Gemm(Workload):
    """BASELINE config 2: MXFP8 GEMM 8192 cubed, bf16 output."""
    name = "mxfp8_gemm_8192x8192x8192_bf16out"
    dtype = "e4m3 x e4m3 (ue8m0 scale / 32) -> fp32 accumulate -> bf16"
    tensor_rate_vs_bf16 = 2.0
    M = N = K = 8192
    seed = 1
    sets = 2   # rotating operand/output sets, so that no step finds its inputs in L2
    cpu_block_limit = 8192
    b_std = 1.0
    launches_per_step = 1

    def flops(self):
        return 2.0 * self.M * self.N * self.K

    def algorithmic_bytes(self):
        ks = self.K // 32
        return self.M * self.K + self.N * self.K + (self.M + self.N) * ks + 2 * self.M * self.N

    def draw(self, gen, take_a=None, take_b=None):
        """A (M, K) activations and B (N, K) weights as bf16 CPU tensors, A first."""
        a = randn_rows(gen, self.M, self.K)                      # always whole: B follows it
        b = randn_rows(gen, self.N, self.K, take_b)
        if self.b_std != 1.0:
            b = self.b_std * b
        return (a if take_a is None else a[:take_a]).bfloat16(), b.bfloat16()

    def setup(self, device):
        import b200k
        g = torch.Generator().manual_seed(self.seed)
        self.inputs = []
        for i in range(self.sets):
            a, b = self.draw(g)
            if i == 0:
                self.a_cpu, self.b_cpu = a, b
            aq, sa = b200k.block_quantize(a.to(device), 32, swizzled_scale=True)
            bq, sb = b200k.block_quantize(b.to(device), 32, swizzled_scale=True)
            c = torch.empty(self.M, self.N, device=device, dtype=torch.bfloat16)
            self.inputs.append((aq, sa, bq, sb, c))
        self.b200k = b200k
        self.i = 0

    def step(self):
        aq, sa, bq, sb, c = self.inputs[self.i % self.sets]
        self.i += 1
        self.b200k.cutile_block_scaled_matmul(aq, sa, bq.T, sb, C=c)
        return c

    def parity(self):
        import oracle
        self.i = 0
        c = self.step()
        rows = _sample(self.M, (0, 127, 128, 255, 256, self.M - 1), 10, 11)
        cols = _sample(self.N, (0, 255, 256, self.N - 1), 256, 12)
        aq, sa = oracle.block_quantize_ref(self.a_cpu[rows])
        bq, sb = oracle.block_quantize_ref(self.b_cpu[cols])
        got_q = self.inputs[0][0][rows.to(c.device)].cpu().view(torch.uint8)
        if not torch.equal(got_q, aq.view(torch.uint8)):
            raise SystemExit("bench.py: parity check failed: quantised bytes differ from the oracle's")
        ref = oracle.block_scaled_matmul_ref(aq, sa, bq, sb)
        got = c[rows.to(c.device)][:, cols.to(c.device)]
        self.i = 0
        return {"max_err": close_or_die(self.name, got, ref, 2e-2, 2e-2), "tol": "rtol 2e-2, atol 2e-2 of max|ref|",
                "what": f"{len(rows)} rows x {len(cols)} columns of one step's output against the de-quantised "
                        "fp32 product of the oracle-quantised operands; quantised bytes of those rows bit-exact"}

    # ---- end-to-end: host buffers in, host buffer out, through the public call
    def setup_e2e(self, device):
        aq, sa, bq, sb, c = self.inputs[0]
        self.pipe_setup(device, [t.cpu().pin_memory() for t in (aq, sa, bq, sb)], c)

    def step_e2e(self):
        def compute(dev_in, dev_out):
            aq, sa, bq, sb = dev_in
            self.b200k.cutile_block_scaled_matmul(aq, sa, bq.T, sb, C=dev_out)
        self.pipe_step(compute)

    # ---- CPU ground truth on an S x S block of the output, same numbers as the GPU arm
    def cpu_setup(self):
        import oracle
        g = torch.Generator().manual_seed(self.seed)
        s = self.cpu_block_limit
        a, b = self.draw(g, take_a=s, take_b=s)
        self.cpu_ops = oracle.block_quantize_ref(a) + oracle.block_quantize_ref(b)
        self.oracle = oracle

    def cpu_step(self, s):
        aq, sa, bq, sb = self.cpu_ops
        return self.oracle.block_scaled_matmul_ref(aq[:s], sa[:s], bq[:s], sb[:s])

    def cpu_flops(self, s):
        return 2.0 * s * s * self.K

    def cpu_sample_desc(self, s):
        return (f"{s}x{s} block of the {self.M}x{self.N} output, K={self.K}: de-quantise both "
                f"operand blocks to fp32 and matmul (torch CPU)")

    def config(self):
        return {"workload": self.name, "M": self.M, "N": self.N, "K": self.K,
                "scale_block": 32, "out": "bf16", "seed": self.seed,
                "inputs": "torch.Generator().manual_seed(seed) on the CPU, copied to the device",
                "l2": f"{self.sets} rotating operand/output sets of "
                      f"{self.algorithmic_bytes() / 2**20:.0f} MiB each (> 126 MiB L2)"}


class Nvfp4Gemm(Mxfp8Gemm):
    """BASELINE config 3 on one GPU: the NVFP4 FFN up-projection 8192 x 28672 x 8192."""
    name = "nvfp4_gemm_8192x28672x8192_bf16out"
    dtype = "e2m1 x e2m1 (ue4m3 scale / 16, fp32 tensor scale) -> fp32 accumulate -> bf16"
    tensor_rate_vs_bf16 = 4.0
    M, N, K = 8192, 28672, 8192
    seed = 2
    sets = 1
    b_std = 0.02
    cpu_block_limit = 2048

    def algorithmic_bytes(self):
        return (self.M + self.N) * (self.K // 2 + self.K // 16) + 2 * self.M * self.N

    def setup(self, device):
        import b200k
        g = torch.Generator().manual_seed(self.seed)
        self.a_cpu, self.b_cpu = self.draw(g)
        self.qa = b200k.nvfp4_quantize(self.a_cpu.to(device))
        self.qb = b200k.nvfp4_quantize(self.b_cpu.to(device))
        self.c = torch.empty(self.M, self.N, device=device, dtype=torch.bfloat16)
        self.b200k = b200k

    def step(self):
        self.b200k.cutile_nvfp4_matmul(*self.qa, *self.qb, C=self.c)
        return self.c

    def _nvfp4_parity(self, c, shard_rows, shard_scales, w_scale):
        """Sampled rows x columns of c against the oracle: the rows' operands quantised by the
        oracle under their shard's tensor scale (amax / 2688 of the shard, checked against the
        scale the device found), the de-quantised fp32 product as the reference."""
        import numpy as np
        import oracle
        m = self.M
        seams = (0, 127, 128, 255, 256, shard_rows - 1, shard_rows, m - shard_rows, m - 256, m - 1)
        rows = _sample(m, seams, 6, 21)
        cols = _sample(self.N, (0, 255, 256, self.N - 1), 256, 22)
        f32 = np.float32
        ts_b = f32(f32(self.b_cpu.float().abs().max()) / f32(2688.0))
        if float(w_scale) != float(ts_b):
            raise SystemExit("bench.py: parity check failed: tensor scale of the weights differs from amax / 2688")
        bq = oracle.nvfp4_quantize_ref(self.b_cpu[cols], tensor_scale=ts_b)
        worst = 0.0
        for p in sorted(set((rows // shard_rows).tolist())):
            mine = rows[(rows // shard_rows) == p]
            shard = self.a_cpu[p * shard_rows:(p + 1) * shard_rows]
            ts_a = f32(f32(shard.float().abs().max()) / f32(2688.0))
            if float(shard_scales[p]) != float(ts_a):
                raise SystemExit(f"bench.py: parity check failed: tensor scale of shard {p} differs from amax / 2688")
            aq = oracle.nvfp4_quantize_ref(self.a_cpu[mine], tensor_scale=ts_a)
            ref = oracle.nvfp4_matmul_ref(*aq, *bq)
            got = c[mine.to(c.device)][:, cols.to(c.device)]
            worst = max(worst, close_or_die(self.name, got, ref, 2e-2, 2e-2))
        return {"max_err": worst, "tol": "rtol 2e-2, atol 2e-2 of max|ref|",
                "what": f"{len(rows)} rows (tile and shard seams) x {len(cols)} columns of one step's output "
                        "against the de-quantised fp32 product of the oracle-quantised operands"}

    def parity(self):
        c = self.step()
        return self._nvfp4_parity(c, self.M, [float(self.qa[2])], float(self.qb[2]))

    def setup_e2e(self, device):
        flat = list(self.qa) + list(self.qb)
        self.pipe_setup(device, [t.cpu().pin_memory() for t in flat], self.c)

    def step_e2e(self):
        self.pipe_step(lambda dev_in, dev_out: self.b200k.cutile_nvfp4_matmul(*dev_in, C=dev_out))

    def cpu_setup(self):
        import oracle
        g = torch.Generator().manual_seed(self.seed)
        s = self.cpu_block_limit
        a, b = self.draw(g, take_a=s, take_b=s)
        self.cpu_ops = (oracle.nvfp4_quantize_ref(a), oracle.nvfp4_quantize_ref(b))
        self.oracle = oracle

    def cpu_step(self, s):
        (aq, asf, ats), (bq, bsf, bts) = self.cpu_ops
        return self.oracle.nvfp4_matmul_ref(aq[:s], asf[:s], ats, bq[:s], bsf[:s], bts)

    def config(self):
        c = super().config()
        c["scale_block"] = 16
        c["l2"] = "operands and output of one step are 610 MiB (> 126 MiB L2)"
        return c


class AgNvfp4Gemm(Nvfp4Gemm):
    """BASELINE config 3 as it is stated: the NVFP4 FFN up-projection as the AllGather GEMM.  A is
    row-sharded M / world per rank (every rank quantises its own rows), gathered over NVLink from
    the peers' symmetric-memory buffers, every rank computing the full (M, N) product against
    its own weights (fixed work per rank: weak scaling).  One GPU: the plain GEMM."""
    name = "allgather_nvfp4_gemm_8192x28672x8192_bf16out"

    def launches(self):
        if self.world == 1:
            return 1
        if (self.M // self.world) % 256 == 0:
            return 3        # one gather launch, the GEMM of the own rows, one GEMM of every other row
        return 3 + 1 + (1 if self.rank in (0, self.world - 1) else 2)   # gathers, local GEMM, remote GEMMs

    def gathered_bytes(self):
        return (self.world - 1) * (self.M // self.world) * (self.K // 2 + self.K // 16)

    def setup(self, device):
        import b200k
        world, rank = self.world, self.rank
        if self.M % (128 * world):
            raise SystemExit(f"{self.M} rows do not split into 128-row scale tiles over {world} ranks")
        rows = self.M // world
        g = torch.Generator().manual_seed(self.seed)
        self.a_cpu, self.b_cpu = self.draw(g)           # the whole problem, the same on every rank
        mine = self.a_cpu[rank * rows:(rank + 1) * rows].to(device)
        aq, asf, ats = b200k.nvfp4_quantize(mine)       # each rank quantises its own rows
        self.qb = b200k.nvfp4_quantize(self.b_cpu.to(device))
        del mine
        if world > 1:
            import torch.distributed as dist
            import torch.distributed._symmetric_memory as symm_mem
            self.s_q = symm_mem.empty(aq.shape, device=device, dtype=torch.uint8).copy_(aq)
            self.s_sf = symm_mem.empty(asf.shape, device=device, dtype=torch.uint8).copy_(asf.view(torch.uint8))
            self.s_ts = symm_mem.empty(1, device=device, dtype=torch.float32).copy_(ats)
        else:
            self.s_q, self.s_sf, self.s_ts = aq, asf.view(torch.uint8), ats
        self.plan = b200k.Nvfp4GatherMatmul(self.s_q, self.s_sf, self.s_ts)
        self.c = torch.empty(self.M, self.N, device=device, dtype=torch.bfloat16)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        self.b200k = b200k

    def step(self):
        return self.plan.run(*self.qb, out=self.c)

    def parity(self):
        c = self.step()
        torch.cuda.synchronize()
        rows = self.M // self.world
        if self.world > 1:   # the gathered per-row scale vector holds every shard's own scale
            scales = self.plan.row_scale[::rows].cpu().tolist()
        else:
            scales = [float(self.s_ts)]
        return self._nvfp4_parity(c, self.M // self.world, scales, float(self.qb[2]))

    def gather_only_us(self, reps=10):
        """Device time of the peer gather alone (the bytes that cross NVLink per step)."""
        if self.world == 1:
            return None
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(2):
            self.plan.gather()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            self.plan.gather()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / reps

    def setup_e2e(self, device):
        host = [t.cpu().pin_memory() for t in (self.s_q, self.s_sf, self.s_ts)]
        self.pipe_setup(device, host, self.c)

    def step_e2e(self):
        def compute(dev_in, dev_out):
            # this rank's freshly uploaded shard goes into the buffers the peers read
            for dst, src in zip((self.s_q, self.s_sf, self.s_ts), dev_in):
                dst.copy_(src, non_blocking=True)
            self.plan.run(*self.qb, out=dev_out)
        self.pipe_step(compute)

    def config(self):
        c = super().config()
        c["sharding"] = ("A rows M / n_gpus per rank, each rank's shard quantised by its owner and "
                         "gathered by peer loads over NVLink; B replicated; every rank computes (M, N)")
        return c


def _expert_weights(seed, e, inter, hidden):
    """w1[e] (2I, H) and w2[e] (H, I) of one expert, N(0, 0.02), from their own generator: any
    rank (and the CPU arm) can rebuild any expert without drawing the others."""
    g = torch.Generator().manual_seed(seed * 1000 + 1 + e)
    w1 = (0.02 * torch.randn(2 * inter, hidden, generator=g)).bfloat16()
    w2 = (0.02 * torch.randn(hidden, inter, generator=g)).bfloat16()
    return w1, w2


class MoeBf16(Workload):
    """BASELINE config 5 on one GPU, bf16 weights: the MoE FFN (16384 tokens, hidden 4096, 64
    experts, intermediate 1536, top-8): align -> gather -> grouped GEMM + SwiGLU -> grouped GEMM
    + scatter -> sum."""
    name = "moe_ffn_16384tok_h4096_e64_i1536_top8_bf16"
    dtype = "bf16 x bf16 -> fp32 accumulate -> bf16"
    tensor_rate_vs_bf16 = 1.0
    T, H, E, I, K = 16384, 4096, 64, 1536, 8
    seed = 4
    mxfp8 = False
    launches_per_step = 8

    def flops(self):
        return 6.0 * self.T * self.K * self.H * self.I / self.world   # per rank

    def algorithmic_bytes(self):
        return 2 * (self.E * 3 * self.I * self.H + 2 * self.T * self.H) // self.world

    def draw_tokens(self):
        """Router outcome and hidden states of the whole problem (CPU)."""
        import oracle
        g = torch.Generator().manual_seed(self.seed)
        tw, ids = oracle.moe_route_ref(torch.randn(self.T, self.E, generator=g), self.K)
        x = torch.randn(self.T, self.H, generator=g).bfloat16()
        return x, tw.bfloat16(), ids

    def expert_range(self):
        per = self.E // self.world
        return range(self.rank * per, (self.rank + 1) * per)

    def load_weights(self, device):
        w = [_expert_weights(self.seed, e, self.I, self.H) for e in self.expert_range()]
        w1 = torch.stack([a for a, _ in w]).to(device)
        w2 = torch.stack([b for _, b in w]).to(device)
        return w1, w2

    def setup(self, device):
        import b200k
        self.x_cpu, self.tw_cpu, self.ids_cpu = self.draw_tokens()
        self.x, self.tw, self.ids = (t.to(device) for t in (self.x_cpu, self.tw_cpu, self.ids_cpu))
        w1, w2 = self.load_weights(device)
        if self.mxfp8:
            self.w = b200k.quantize_expert_weights(w1) + b200k.quantize_expert_weights(w2)
        else:
            self.w = (w1, w2)
        self.b200k = b200k

    def step(self):
        if self.mxfp8:
            return self.b200k.cutile_moe_mxfp8(self.x, *self.w, self.tw, self.ids)
        return self.b200k.cutile_moe(self.x, *self.w, self.tw, self.ids)

    def _moe_parity(self, out, x_cpu, tw_cpu, ids_cpu):
        """Sampled tokens against the oracle's FFN evaluated for those tokens only, with the
        experts they use rebuilt from their seeds."""
        import oracle
        tok = _sample(x_cpu.shape[0], (0, x_cpu.shape[0] - 1), 2, 31)
        used = sorted(set(ids_cpu[tok].reshape(-1).tolist()))
        remap = {e: i for i, e in enumerate(used)}
        ids = torch.tensor([[remap[int(e)] for e in row] for row in ids_cpu[tok]])
        w = [_expert_weights(self.seed, e, self.I, self.H) for e in used]
        w1, w2 = torch.stack([a for a, _ in w]), torch.stack([b for _, b in w])
        if self.mxfp8:
            q1, s1 = oracle.block_quantize_ref(w1)
            q2, s2 = oracle.block_quantize_ref(w2)
            ref = oracle.moe_mxfp8_ref(x_cpu[tok], q1, s1, q2, s2, tw_cpu[tok], ids)
        else:
            ref = oracle.moe_ref(x_cpu[tok], w1, w2, tw_cpu[tok], ids)
        got = out[tok.to(out.device)]
        err = oracle.rel_frobenius(got, ref)
        if not err < 2e-2:
            raise SystemExit(f"bench.py: parity check failed for {self.name}: relative Frobenius error {err:.4g}")
        close_or_die(self.name, got, ref, 1e-1, 1e-1 / max(float(ref.abs().max()), 1e-30))
        return {"max_err": err, "tol": "relative Frobenius error < 2e-2; rtol 1e-1, atol 1e-1 elementwise",
                "what": f"{len(tok)} tokens ({len(used)} experts) of one step's output against the oracle's FFN "
                        "for those tokens"}

    def parity(self):
        return self._moe_parity(self.step(), self.x_cpu, self.tw_cpu, self.ids_cpu)

    def setup_e2e(self, device):
        self.host_in = [t.cpu().pin_memory() for t in (self.x, self.tw, self.ids)]
        self.dev_in = [self.x, self.tw, self.ids]
        self.host_out = torch.empty_like(self.x, device="cpu").pin_memory()
        self.h2d = sum(t.numel() * t.element_size() for t in self.host_in)
        self.d2h = self.host_out.numel() * self.host_out.element_size()

    def step_e2e(self):
        for d, h in zip(self.dev_in, self.host_in):
            d.copy_(h, non_blocking=True)
        self.host_out.copy_(self.step(), non_blocking=True)

    # CPU arm: the same tokens, routed among the first 8 experts, top-2 (a bounded slice)
    def cpu_setup(self):
        import oracle
        t, e = 512, 8
        x, _, _ = self.draw_tokens()
        g = torch.Generator().manual_seed(self.seed + 77)
        w = [_expert_weights(self.seed, i, self.I, self.H) for i in range(e)]
        self.cpu_ops = (x[:t].float(), torch.stack([a for a, _ in w]).float(), torch.stack([b for _, b in w]).float())
        self.cpu_route = oracle.moe_route_ref(torch.randn(t, e, generator=g), 2)
        self.oracle = oracle

    def cpu_step(self, s):
        x, w1, w2 = self.cpu_ops
        tw, ids = self.cpu_route
        return self.oracle.moe_ref(x[:s], w1, w2, tw[:s], ids[:s])

    def cpu_flops(self, s):
        return 6.0 * s * 2 * self.H * self.I

    def cpu_sample_desc(self, s):
        return f"the first {s} tokens through 8 of the experts, top-2, same FFN in fp32 (torch CPU)"

    def config(self):
        return {"workload": self.name, "tokens": self.T, "hidden": self.H, "experts": self.E,
                "intermediate": self.I, "topk": self.K, "seed": self.seed,
                "inputs": "torch.Generator().manual_seed(seed) on the CPU (one generator per expert)",
                "l2": "expert weights alone are 2.4 GB (> 126 MiB L2)"}


class MoeMxfp8(MoeBf16):
    name = "moe_ffn_16384tok_h4096_e64_i1536_top8_mxfp8"
    dtype = "e4m3 x e4m3 (ue8m0 scale / 32) -> fp32 accumulate -> bf16"
    tensor_rate_vs_bf16 = 2.0
    mxfp8 = True
    launches_per_step = 9


class MoeSparse(MoeBf16):
    """The reference's sparse MoE bench shape (test/bench_moe.py:16-19): 256 tokens, 1408 experts,
    top-6, hidden 2048, intermediate 32 - about one token per expert.  Every replica streams
    its expert's weights once on the CUDA cores: HBM-bound, the algorithmic bytes are the
    routed experts' weights."""
    name = "moe_ffn_sparse_256tok_h2048_e1408_i32_top6_bf16"
    dtype = "bf16 x bf16 -> fp32 accumulate -> bf16 (CUDA cores)"
    bound = "hbm"
    T, H, E, I, K = 256, 2048, 1408, 32, 6
    seed = 6
    launches_per_step = 3
    cuda_graph = True

    def flops(self):
        return float(self.algorithmic_bytes())

    def algorithmic_bytes(self):
        # per replica the expert's W1 and W2 once, its token in, its row out and back in for the sum
        return self.T * self.K * (3 * self.I * self.H * 2 + 3 * self.H * 2) + self.T * self.H * 2

    def cpu_setup(self):
        import oracle
        x, tw, ids = self.draw_tokens()
        t = 64
        used = sorted(set(ids[:t].reshape(-1).tolist()))
        remap = {e: i for i, e in enumerate(used)}
        w = [_expert_weights(self.seed, e, self.I, self.H) for e in used]
        self.cpu_ops = (x[:t].float(), torch.stack([a for a, _ in w]).float(), torch.stack([b for _, b in w]).float())
        self.cpu_route = (tw[:t].float(), torch.tensor([[remap[int(e)] for e in row] for row in ids[:t]]))
        self.oracle = oracle

    def cpu_flops(self, s):
        return float(s * self.K * 3 * self.I * self.H * 2)

    def cpu_sample_desc(self, s):
        return f"the first {s} tokens of the same problem through torch_moe's restatement in fp32 (torch CPU)"

    cpu_limit = 64

    def config(self):
        c = super().config()
        c["l2"] = "the routed experts' weights are 0.6 GB per step (> 126 MiB L2)"
        return c


class MoeEpBf16(MoeBf16):
    """BASELINE config 5 expert-parallel: experts E / world and tokens T / world per rank, an
    NVLink exchange for dispatch and one for combine.  The whole problem is fixed, so this
    scales strongly."""
    name = "moe_ffn_ep_16384tok_h4096_e64_i1536_top8_bf16"
    distributed = True
    scaling = "strong"
    launches_per_step = 10

    def setup(self, device):
        import b200k
        x, tw, ids = self.draw_tokens()
        tl = self.T // self.world
        sl = slice(self.rank * tl, (self.rank + 1) * tl)
        self.x_cpu, self.tw_cpu, self.ids_cpu = x[sl], tw[sl], ids[sl]
        self.x, self.tw, self.ids = (t.to(device) for t in (self.x_cpu, self.tw_cpu, self.ids_cpu))
        w1, w2 = self.load_weights(device)
        self.ep = b200k.ExpertParallelMoE(w1, w2, self.E, mxfp8=self.mxfp8)
        self.b200k = b200k

    def step(self):
        return self.ep.forward(self.x, self.tw, self.ids)

    def config(self):
        c = super().config()
        c["sharding"] = "experts E / n_gpus and tokens T / n_gpus per rank; dispatch and combine over NVLink"
        return c


class MoeEpMxfp8(MoeEpBf16):
    name = "moe_ffn_ep_16384tok_h4096_e64_i1536_top8_mxfp8"
    dtype = MoeMxfp8.dtype
    tensor_rate_vs_bf16 = 2.0
    mxfp8 = True


class FmhaCausal(Workload):
    """BASELINE config 4: causal attention forward, bf16, batch 4, 32 heads, sequence 8192, head dim 128."""
    name = "fmha_causal_bf16_b4_h32_s8192_d128"
    dtype = "bf16 x bf16 -> fp32 softmax / accumulate -> bf16"
    tensor_rate_vs_bf16 = 1.0
    B, H, S, D = 4, 32, 8192, 128
    seed = 3
    cpu_limit = 4096
    launches_per_step = 1

    def flops(self):
        return 4.0 * self.B * self.H * self.S * self.S * self.D * 0.5

    def algorithmic_bytes(self):
        return 4 * self.B * self.H * self.S * self.D * 2

    def draw(self, gen, batch=None):
        shape = (self.B if batch is None else batch, self.H, self.S, self.D)
        return tuple(torch.randn(shape, generator=gen).bfloat16() for _ in range(3))

    def setup(self, device):
        import b200k
        g = torch.Generator().manual_seed(self.seed)
        self.cpu_qkv = self.draw(g)
        self.q, self.k, self.v = (t.to(device) for t in self.cpu_qkv)
        self.o = torch.empty_like(self.q)
        self.b200k = b200k

    def step(self):
        return self.b200k.cutile_fmha(self.q, self.k, self.v, causal=True, Out=self.o)

    def parity(self):
        import oracle
        out = self.step()
        q, k, v = self.cpu_qkv
        worst = 0.0
        for (b, h), (lo, hi) in zip([(0, 0), (self.B - 1, self.H - 1)], [(4032, 4160), (self.S - 128, self.S)]):
            ref = oracle.fmha_ref(q[b:b + 1, h:h + 1, lo:hi], k[b:b + 1, h:h + 1, :hi], v[b:b + 1, h:h + 1, :hi],
                                  causal=True, input_pos=lo)
            got = out[b:b + 1, h:h + 1, lo:hi]
            worst = max(worst, close_or_die(self.name, got, ref, 5e-2, 1e-2 / max(float(ref.abs().max()), 1e-30)))
        return {"max_err": worst, "tol": "rtol 5e-2, atol 1e-2",
                "what": "two 128-row query blocks (one across a 256-row tile seam, the last one) in the first "
                        "and the last (batch, head) against fp32 softmax(QK^T + mask)V"}

    def setup_e2e(self, device):
        self.pipe_setup(device, [t.pin_memory() for t in self.cpu_qkv], self.o)

    def step_e2e(self):
        self.pipe_step(lambda dev_in, dev_out: self.b200k.cutile_fmha(*dev_in, causal=True, Out=dev_out))

    def cpu_setup(self):
        import oracle
        g = torch.Generator().manual_seed(self.seed)
        # head (0, 0) of the same draw: only the first batch entry is needed
        q = torch.randn(self.B, self.H, self.S, self.D, generator=g)[0:1, 0:1].bfloat16()
        k = torch.randn(self.B, self.H, self.S, self.D, generator=g)[0:1, 0:1].bfloat16()
        v = torch.randn(self.B, self.H, self.S, self.D, generator=g)[0:1, 0:1].bfloat16()
        self.cpu_ops = (q, k, v)
        self.oracle = oracle

    def cpu_step(self, s):
        q, k, v = self.cpu_ops
        return self.oracle.fmha_ref(q[:, :, :s], k[:, :, :s], v[:, :, :s], causal=True)

    def cpu_flops(self, s):
        return 4.0 * s * s * self.D * 0.5

    def cpu_sample_desc(self, s):
        return f"head (0, 0), first {s} positions: fp32 softmax(QK^T + causal mask)V (torch CPU)"

    def config(self):
        return {"workload": self.name, "batch": self.B, "heads": self.H, "seq": self.S,
                "head_dim": self.D, "causal": True, "seed": self.seed,
                "inputs": "torch.Generator().manual_seed(seed) on the CPU, copied to the device",
                "l2": "Q, K, V and O are 268 MB each (> 126 MiB L2)"}


class Mxfp8Quantize(Workload):
    """The quantiser that feeds the MXFP8 GEMM: bf16 8192 x 8192 -> e4m3 + swizzled ue8m0
    scales.  One pass over the data: HBM-bound."""
    name = "mxfp8_quantize_bf16_8192x8192"
    dtype = "bf16 -> e4m3 + ue8m0 / 32"
    bound = "hbm"
    M = K = 8192
    seed = 1
    sets = 3
    launches_per_step = 1
    cuda_graph = True

    def flops(self):
        return float(self.algorithmic_bytes())   # "work" of an HBM-bound kernel = its bytes

    def algorithmic_bytes(self):
        return self.M * self.K * 2 + self.M * self.K + self.M * self.K // 32

    def setup(self, device):
        import b200k
        g = torch.Generator().manual_seed(self.seed)
        self.x_cpu = [torch.randn(self.M, self.K, generator=g).bfloat16() for _ in range(self.sets)]
        self.xs = [x.to(device) for x in self.x_cpu]
        self.b200k = b200k
        self.i = 0

    def step(self):
        x = self.xs[self.i % self.sets]
        self.i += 1
        return self.b200k.block_quantize(x, 32, swizzled_scale=True)

    def parity(self):
        import oracle
        q, s = self.b200k.block_quantize(self.xs[0], 32)
        rows = _sample(self.M, (0, 127, 128, self.M - 1), 28, 41)
        q_ref, s_ref = oracle.block_quantize_ref(self.x_cpu[0][rows])
        same = (torch.equal(q[rows.to(q.device)].cpu().view(torch.uint8), q_ref.view(torch.uint8)) and
                torch.equal(s[rows.to(q.device)].cpu().view(torch.uint8), s_ref.view(torch.uint8)))
        if not same:
            raise SystemExit(f"bench.py: parity check failed for {self.name}: bytes differ from the oracle's")
        return {"max_err": 0.0, "tol": "bit-exact",
                "what": f"codes and scale bytes of {len(rows)} rows against the oracle's block_quantize"}

    def setup_e2e(self, device):
        self.host_in = [self.xs[0].cpu().pin_memory()]
        q, s = self.step()
        self.host_out = [torch.empty_like(q.view(torch.uint8), device="cpu").pin_memory(),
                         torch.empty_like(s.view(torch.uint8), device="cpu").pin_memory()]
        self.h2d = self.host_in[0].numel() * 2
        self.d2h = sum(t.numel() for t in self.host_out)

    def step_e2e(self):
        self.xs[0].copy_(self.host_in[0], non_blocking=True)
        q, s = self.b200k.block_quantize(self.xs[0], 32, swizzled_scale=True)
        self.host_out[0].copy_(q.view(torch.uint8), non_blocking=True)
        self.host_out[1].copy_(s.view(torch.uint8), non_blocking=True)

    def cpu_setup(self):
        import oracle
        g = torch.Generator().manual_seed(self.seed)
        self.cpu_ops = (torch.randn(self.M, self.K, generator=g)[:4096].bfloat16(),)
        self.oracle = oracle

    def cpu_step(self, s):
        return self.oracle.block_quantize_ref(self.cpu_ops[0][:s])

    def cpu_flops(self, s):
        return float(s * self.K * 3 + s * self.K // 32)

    def cpu_sample_desc(self, s):
        return f"{s} rows of {self.K} bf16 values through block_quantize's restatement (torch CPU)"

    def config(self):
        return {"workload": self.name, "rows": self.M, "K": self.K, "seed": self.seed,
                "inputs": "torch.Generator().manual_seed(seed) on the CPU, copied to the device",
                "l2": f"{self.sets} rotating inputs of 128 MiB each (> 126 MiB L2)"}


class Nvfp4Quantize(Mxfp8Quantize):
    """bf16 8192 x 8192 -> packed e2m1 + swizzled ue4m3 scales + fp32 tensor scale.  Two kernels
    (tensor maximum, then the quantiser), so the input is read twice: HBM-bound."""
    name = "nvfp4_quantize_bf16_8192x8192"
    dtype = "bf16 -> e2m1 + ue4m3 / 16 + fp32 tensor scale"
    launches_per_step = 3   # memset of the maximum, absmax, quantise

    def algorithmic_bytes(self):
        # the input twice (maximum, then values), codes, scales
        return 2 * self.M * self.K * 2 + self.M * self.K // 2 + self.M * self.K // 16

    def step(self):
        x = self.xs[self.i % self.sets]
        self.i += 1
        return self.b200k.nvfp4_quantize(x)

    def parity(self):
        import numpy as np
        import oracle
        q, s, ts = self.b200k.nvfp4_quantize(self.xs[0], swizzled_scale=False)
        rows = _sample(self.M, (0, 127, 128, self.M - 1), 28, 42)
        want_ts = np.float32(np.float32(self.x_cpu[0].float().abs().max()) / np.float32(2688.0))
        q_ref, s_ref, _ = oracle.nvfp4_quantize_ref(self.x_cpu[0][rows], tensor_scale=want_ts)
        same = (float(ts) == float(want_ts) and
                np.array_equal(q[rows.to(q.device)].cpu().numpy(), q_ref) and
                np.array_equal(s[rows.to(q.device)].cpu().view(torch.uint8).numpy(), s_ref))
        if not same:
            raise SystemExit(f"bench.py: parity check failed for {self.name}: bytes differ from the oracle's")
        return {"max_err": 0.0, "tol": "bit-exact",
                "what": f"tensor scale, codes and scale bytes of {len(rows)} rows against the oracle's quantiser"}

    def setup_e2e(self, device):
        self.host_in = [self.xs[0].cpu().pin_memory()]
        q, s, t = self.step()
        self.host_out = [torch.empty_like(q.view(torch.uint8), device="cpu").pin_memory(),
                         torch.empty_like(s.view(torch.uint8), device="cpu").pin_memory()]
        self.h2d = self.host_in[0].numel() * 2
        self.d2h = sum(t.numel() for t in self.host_out)

    def step_e2e(self):
        self.xs[0].copy_(self.host_in[0], non_blocking=True)
        q, s, _ = self.b200k.nvfp4_quantize(self.xs[0])
        self.host_out[0].copy_(q.view(torch.uint8), non_blocking=True)
        self.host_out[1].copy_(s.view(torch.uint8), non_blocking=True)

    def cpu_step(self, s):
        return self.oracle.nvfp4_quantize_ref(self.cpu_ops[0][:s])

    def cpu_flops(self, s):
        return float(s * self.K * 4 + s * self.K // 2 + s * self.K // 16)

    def cpu_sample_desc(self, s):
        return f"{s} rows of {self.K} bf16 values through the NVFP4 quantiser's restatement (numpy CPU)"


class FmhaDecode(Workload):
    """One decode step of grouped-query attention over a long KV cache: the reference's decode
    bench shapes (test/bench_attention.py:33-44: one query per sequence, 32 query heads on 8 KV
    heads) at a serving-size batch.  K and V are read once: HBM-bound."""
    name = "fmha_decode_bf16_b32_hq32_hkv8_s2048_d128"
    dtype = "bf16, fp32 softmax"
    bound = "hbm"
    B, HQ, HKV, S, D = 32, 32, 8, 2048, 128
    seed = 5
    sets = 2
    launches_per_step = 1
    cuda_graph = True

    def flops(self):
        return float(self.algorithmic_bytes())

    def algorithmic_bytes(self):
        return 2 * self.B * self.HKV * self.S * self.D * 2 + 2 * self.B * self.HQ * self.D * 2

    def draw(self, gen):
        mk = lambda *sh: torch.randn(*sh, generator=gen).bfloat16()
        return (mk(self.B, self.HQ, 1, self.D), mk(self.B, self.HKV, self.S, self.D),
                mk(self.B, self.HKV, self.S, self.D))

    def setup(self, device):
        import b200k
        g = torch.Generator().manual_seed(self.seed)
        self.x_cpu = [self.draw(g) for _ in range(self.sets)]
        self.xs = [tuple(t.to(device) for t in qkv) for qkv in self.x_cpu]
        self.out = torch.empty(self.B, self.HQ, 1, self.D, device=device, dtype=torch.bfloat16)
        self.b200k = b200k
        self.i = 0

    def _run(self, q, k, v):
        return self.b200k.cutile_fmha(q, k, v, causal=True, input_pos=self.S - 1,
                                      query_group_size=self.HQ // self.HKV, Out=self.out)

    def step(self):
        q, k, v = self.xs[self.i % self.sets]
        self.i += 1
        return self._run(q, k, v)

    def parity(self):
        import oracle
        out = self._run(*self.xs[0])
        q, k, v = self.x_cpu[0]
        sel = [0, self.B - 1]
        ref = oracle.fmha_ref(q[sel], k[sel], v[sel], causal=True, input_pos=self.S - 1,
                              query_group_size=self.HQ // self.HKV)
        err = close_or_die(self.name, out[sel], ref, 5e-2, 1e-2 / max(float(ref.abs().max()), 1e-30))
        return {"max_err": err, "tol": "rtol 5e-2, atol 1e-2",
                "what": "the first and the last sequence of the batch against fp32 softmax(q k^T) v"}

    def setup_e2e(self, device):
        # a decode step's KV cache lives on the device; the step's own traffic is the new query
        # in and the attention output back
        self.host_in = [self.xs[0][0].cpu().pin_memory()]
        self.host_out = [torch.empty_like(self.out, device="cpu").pin_memory()]
        self.h2d = self.host_in[0].numel() * 2
        self.d2h = self.host_out[0].numel() * 2

    def step_e2e(self):
        q, k, v = self.xs[0]
        q.copy_(self.host_in[0], non_blocking=True)
        self.host_out[0].copy_(self._run(q, k, v), non_blocking=True)

    def cpu_setup(self):
        import oracle
        g = torch.Generator().manual_seed(self.seed)
        self.cpu_ops = self.draw(g)
        self.oracle = oracle

    def cpu_step(self, s):
        q, k, v = self.cpu_ops
        s = min(s, self.B)
        return self.oracle.fmha_ref(q[:s], k[:s], v[:s], causal=True, input_pos=self.S - 1,
                                    query_group_size=self.HQ // self.HKV)

    def cpu_flops(self, s):
        return float(self.algorithmic_bytes()) * min(s, self.B) / self.B

    def cpu_sample_desc(self, s):
        return f"{min(s, self.B)} of {self.B} sequences through fp32 softmax(q k^T) v (torch CPU)"

    cpu_limit = 32

    def config(self):
        return {"workload": self.name, "batch": self.B, "heads_q": self.HQ, "heads_kv": self.HKV,
                "keys": self.S, "head_dim": self.D, "seed": self.seed,
                "inputs": "torch.Generator().manual_seed(seed) on the CPU, copied to the device",
                "l2": f"{self.sets} rotating K/V sets of 268 MB each (> 126 MiB L2)"}


class DenseF16(Workload):
    """BASELINE config 1: the sample-sized dense fp16 matmul (2048 cubed), B row-major (K, N)."""
    name = "dense_f16_gemm_2048x2048x2048"
    dtype = "f16 x f16 -> fp32 accumulate -> f16"
    tensor_rate_vs_bf16 = 1.0
    M = N = K = 2048
    seed = 0
    sets = 12   # 12 x 24 MiB > L2
    launches_per_step = 1

    def flops(self):
        return 2.0 * self.M * self.N * self.K

    def algorithmic_bytes(self):
        return 2 * (self.M * self.K + self.K * self.N + self.M * self.N)

    def setup(self, device):
        import b200k
        g = torch.Generator().manual_seed(self.seed)
        self.inputs = []
        for i in range(self.sets):
            a = torch.randn(self.M, self.K, generator=g).half()
            b = torch.randn(self.K, self.N, generator=g).half()
            if i == 0:
                self.a_cpu, self.b_cpu = a, b
            self.inputs.append((a.to(device), b.to(device),
                                torch.empty(self.M, self.N, device=device, dtype=torch.float16)))
        self.b200k = b200k
        self.i = 0

    def step(self):
        a, b, c = self.inputs[self.i % self.sets]
        self.i += 1
        return self.b200k.cutile_matmul(a, b, C=c)

    def parity(self):
        import oracle
        self.i = 0
        c = self.step()
        self.i = 0
        rows = _sample(self.M, (0, 127, 128, 255, 256, self.M - 1), 26, 51)
        ref = oracle.matmul_ref(self.a_cpu[rows], self.b_cpu)
        return {"max_err": close_or_die(self.name, c[rows.to(c.device)], ref, 2e-2, 2e-2),
                "tol": "rtol 2e-2, atol 2e-2 of max|ref|",
                "what": f"{len(rows)} whole rows of one step's output against A.float() @ B.float()"}

    def setup_e2e(self, device):
        a, b, c = self.inputs[0]
        self.pipe_setup(device, [t.cpu().pin_memory() for t in (a, b)], c)

    def step_e2e(self):
        self.pipe_step(lambda dev_in, dev_out: self.b200k.cutile_matmul(dev_in[0], dev_in[1], C=dev_out))

    def cpu_setup(self):
        import oracle
        g = torch.Generator().manual_seed(self.seed)
        self.cpu_ops = (torch.randn(self.M, self.K, generator=g).half(),
                        torch.randn(self.K, self.N, generator=g).half())
        self.oracle = oracle

    def cpu_step(self, s):
        a, b = self.cpu_ops
        return self.oracle.matmul_ref(a[:s], b[:, :s])

    def cpu_flops(self, s):
        return 2.0 * s * s * self.K

    def cpu_sample_desc(self, s):
        return f"{s}x{s} block of the output, K={self.K}: A.float() @ B.float() (torch CPU)"

    def config(self):
        return {"workload": self.name, "M": self.M, "N": self.N, "K": self.K, "out": "f16", "seed": self.seed,
                "inputs": "torch.Generator().manual_seed(seed) on the CPU, copied to the device",
                "l2": f"{self.sets} rotating operand/output sets of 24 MiB each (> 126 MiB L2)"}


WORKLOADS = {"ag_nvfp4_gemm": AgNvfp4Gemm, "mxfp8_gemm": Mxfp8Gemm, "nvfp4_gemm": Nvfp4Gemm,
             "dense_f16": DenseF16, "fmha_causal": FmhaCausal, "fmha_decode": FmhaDecode,
             "moe_bf16": MoeBf16, "moe_mxfp8": MoeMxfp8, "moe_sparse": MoeSparse, "moe_ep_bf16": MoeEpBf16,
             "moe_ep_mxfp8": MoeEpMxfp8, "mxfp8_quantize": Mxfp8Quantize, "nvfp4_quantize": Nvfp4Quantize}
DEFAULT_WORKLOAD = "ag_nvfp4_gemm"


# --------------------------------------------------------------------------------------
# Clock sampling (read-only NVML queries during the timed region)
# --------------------------------------------------------------------------------------
class ClockSampler:
    REASONS = {
        0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap",
        0x8: "hw_slowdown", 0x10: "sync_boost", 0x20: "sw_thermal_slowdown",
        0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting",
    }

    def __init__(self, device, period_s=0.005):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self.period_s = period_s
        self._stop = threading.Event()
        self._thread = None
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(device).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception as e:  # pragma: no cover - depends on the box
            self.err = repr(e)

    def _run(self):
        while not self._stop.is_set():
            self.sample()
            time.sleep(self.period_s)

    def sample(self):
        if not self.ok:
            return
        try:
            self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
            mask = self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
            for bit, name in self.REASONS.items():
                if mask & bit and name != "gpu_idle":
                    self.reasons.add(name)
        except Exception:
            pass

    def start(self):
        self.samples, self.reasons = [], set()
        self._stop.clear()
        if self.ok:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        self.sample()
        self._stop.set()
        if self._thread:
            self._thread.join()
            self._thread = None

    def summary(self):
        if not self.ok or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_min_mhz": s[0], "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


# --------------------------------------------------------------------------------------
def time_cpu(w, steps, warmup, budget_s=120.0):
    """Times the CPU ground truth on an S x S output block sized so the run fits the budget."""
    torch.set_num_threads(os.cpu_count() or 1)
    w.cpu_setup()
    probe = 256
    t0 = time.perf_counter()
    w.cpu_step(probe)
    t_probe = time.perf_counter() - t0
    t0 = time.perf_counter()
    w.cpu_step(probe)
    t_probe = min(t_probe, time.perf_counter() - t0)
    limit = getattr(w, "cpu_limit", None)
    if limit is None:
        limit = len(w.cpu_ops[0][0]) if isinstance(w.cpu_ops[0], tuple) else w.cpu_ops[0].shape[0]
    per_step = budget_s / max(1, steps + warmup)
    # cost grows about quadratically with the block edge
    s = int(probe * max(1.0, (per_step / max(t_probe, 1e-4)) ** 0.5))
    s = max(256, min(limit, s // 128 * 128))
    for _ in range(warmup):
        w.cpu_step(s)
    t0 = time.perf_counter()
    for _ in range(steps):
        w.cpu_step(s)
    dt = (time.perf_counter() - t0) / steps
    return dt, s


def run_reference(args, w):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    dt, s = time_cpu(w, args.steps, args.warmup)
    hbm = getattr(w, "bound", "tensor") == "hbm"
    unit = "GB/s" if hbm else "TFLOP/s"
    rate = w.cpu_flops(s) / dt / (1e9 if hbm else 1e12)
    line = {
        "impl": "reference", "metric": "hbm_gbs" if hbm else "tflops", "value": rate, "unit": unit,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": getattr(w, "scaling", "weak"),
        "vs_baseline": None, "dtype": "f32 (torch CPU)", "data": "synthetic",
        "config": w.config(),
        "cpu_baseline": {"value": rate, "unit": unit, "cores": torch.get_num_threads(),
                         "kind": "port", "sample": w.cpu_sample_desc(s)},
        "e2e": {"value": rate, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def timed_steps(w, steps, barrier, graph=False):
    """Device time in ms per step of `steps` back-to-back steps, events on the launching stream."""
    ev0 = torch.cuda.Event(enable_timing=True)
    ev1 = torch.cuda.Event(enable_timing=True)
    if graph:
        # launch-bound workloads (kernels of a few tens of microseconds): the steps are
        # captured once and replayed as one graph, so the device never waits for the host
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(steps):
                w.step()
        g.replay()
        barrier()
        ev0.record()
        g.replay()
        ev1.record()
    else:
        barrier()
        ev0.record()
        for _ in range(steps):
            w.step()
        ev1.record()
    barrier()
    return ev0.elapsed_time(ev1) / steps


def run_ours(args, w):
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    affinity = os.sched_getaffinity(0)
    numa = bind_near_gpu(device)
    distributed = world > 1 or getattr(w, "distributed", False)
    if distributed:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29531")
        os.environ.setdefault("RANK", "0")
        os.environ.setdefault("WORLD_SIZE", "1")
        # NCCL only carries barriers and the max over ranks here; without NVLink multicast objects a
        # rank that dies cannot fault its peers' GPUs
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=device)
    w.world, w.rank = world, rank

    def barrier():
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(values):
        if world == 1:
            return values
        t = torch.tensor(values, device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    import b200k

    def check_device(phase):
        """A device-side wait that gave up (status word) ends the run, naming the phase."""
        torch.cuda.synchronize()
        code, info = b200k.device_status()
        if code != 0:
            raise SystemExit(f"bench.py: rank {rank}: device-side wait gave up during '{phase}' "
                             f"(role {(info >> 8) & 0xff}, detail {(info >> 16) & 0xffff})")

    warmup = max(3, args.warmup)
    w.setup(device)
    for _ in range(warmup):
        w.step()
    barrier()
    check_device("warm-up")
    # the output is checked before it is timed
    parity = w.parity()
    barrier()
    check_device("parity check")

    use_graph = (args.launch == "graph" or (args.launch == "auto" and bool(getattr(w, "cuda_graph", False)))) \
        and not distributed
    sampler = ClockSampler(device)
    sampler.start()
    ms = timed_steps(w, args.steps, barrier, use_graph)
    sampler.stop()
    clocks = sampler.summary()
    check_device("timed steps")

    # the same loop for at least a second: the burst above runs at boost clocks, this one at
    # what the power cap sustains
    sustained = None
    if not args.kernel_only and args.sustain_s > 0:
        # every rank must run the same number of steps (the expert-parallel layers meet in
        # barriers): size the loop from the slowest rank's burst time
        ms_all = max_over_ranks([ms])[0]
        n = int(min(2000 if use_graph else 20000, max(args.steps, args.sustain_s * 1e3 / max(ms_all, 1e-3))))
        sampler.start()
        ms_s = timed_steps(w, n, barrier, use_graph)
        sampler.stop()
        sustained = {"steps": n, "ms_per_step": ms_s, "clocks": sampler.summary()}
        check_device("sustained loop")

    gather_us = w.gather_only_us() if hasattr(w, "gather_only_us") else None

    # end to end: pinned host buffers -> device -> kernel -> pinned host buffer
    e2e_steps = max(3, min(args.steps, 20))
    if args.kernel_only:
        ms_e2e, w.h2d, w.d2h = float("nan"), 0, 0
    else:
        ev0 = torch.cuda.Event(enable_timing=True)
        ev1 = torch.cuda.Event(enable_timing=True)
        w.setup_e2e(device)
        w.e2e_begin()
        for _ in range(2):
            w.step_e2e()
        w.e2e_end()
        barrier()
        ev0.record()
        w.e2e_begin()
        for _ in range(e2e_steps):
            w.step_e2e()
        w.e2e_end()
        ev1.record()
        barrier()
        ms_e2e = ev0.elapsed_time(ev1) / e2e_steps
        check_device("end-to-end steps")

    # secondary record of the default workload: BASELINE config 2 (MXFP8 8192 cubed) on this GPU
    also = None
    if args.workload == DEFAULT_WORKLOAD and not args.kernel_only and not args.no_also:
        w2 = Mxfp8Gemm()
        w2.setup(device)
        for _ in range(warmup):
            w2.step()
        p2 = w2.parity()
        ms2 = timed_steps(w2, args.steps, barrier)
        also = (w2, p2, ms2)
        check_device("secondary MXFP8 record")

    vals = [ms, ms_e2e, sustained["ms_per_step"] if sustained else 0.0, also[2] if also else 0.0,
            gather_us or 0.0]
    ms, ms_e2e, ms_sus, ms_also, gather_us_max = max_over_ranks(vals)

    if rank == 0:
        peaks = load_peaks()
        flops = w.flops()
        hbm = getattr(w, "bound", "tensor") == "hbm"
        unit = "GB/s" if hbm else "TFLOP/s"
        scale = 1e9 if hbm else 1e12
        value = world * flops / (ms * 1e-3) / scale
        per_gpu = flops / (ms * 1e-3) / scale
        if hbm:
            peak = peaks["hbm_gbs"]
            peak_source = f"{peaks['source']} copy bandwidth"
        else:
            peak = peaks["bf16_tflops"] * w.tensor_rate_vs_bf16
            peak_source = (f"{peaks['source']} cuBLAS bf16 burst x {w.tensor_rate_vs_bf16:g} "
                           f"(tensor-core rate of the operand format relative to bf16)")
        line = {
            "metric": "hbm_gbs" if hbm else "tflops", "value": value, "unit": unit, "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": getattr(w, "scaling", "weak"), "vs_baseline": None,
            "dtype": w.dtype, "data": "synthetic",
            "config": w.config(),
            "launch": "cuda_graph" if use_graph else "stream",
            "parity_checked": True, "max_err": parity["max_err"], "parity": parity,
            "e2e": {"value": world * flops / (ms_e2e * 1e-3) / scale, "unit": unit,
                    "h2d_bytes_per_step": w.h2d, "d2h_bytes_per_step": w.d2h,
                    "ms_per_step": ms_e2e, "steps": e2e_steps, "host_numa": numa,
                    "overlap": "H2D, kernel and D2H of consecutive steps on three streams"
                               if w.e2e_pipelined else "none (one stream)"},
            "gpu_launches": args.steps * w.launches(),
            "clocks": clocks,
            "roofline": {"bound": "hbm" if hbm else "tensor", "achieved": per_gpu, "peak": peak,
                         "unit": unit, "frac": per_gpu / peak, "peak_source": peak_source,
                         "traffic": TRAFFIC_BYTES.get(w.name),
                         "algorithmic_bytes": w.algorithmic_bytes()},
        }
        if sustained:
            sus_rate = flops / (ms_sus * 1e-3) / scale
            sus_peak = peak if hbm else peaks["bf16_tflops_sustained"] * w.tensor_rate_vs_bf16
            line["sustained"] = {"value": world * sus_rate, "unit": unit, "ms_per_step": ms_sus,
                                 "steps": sustained["steps"], "clocks": sustained["clocks"],
                                 "frac_of_sustained_peak": sus_rate / sus_peak,
                                 "note": "the same steps back to back for at least a second (power-capped clocks)"}
        if gather_us:
            gb = w.gathered_bytes()
            line["nvlink"] = {"gathered_bytes_per_step": gb, "gather_us": gather_us_max,
                              "achieved_gbs": gb / (gather_us_max * 1e-6) / 1e9,
                              "peak_gbs": NVLINK_PEER_COPY_GBS,
                              "note": "peer_gather kernels alone (inbound bytes per rank); in a step they run "
                                      "under the GEMM of the rank's own rows"}
        if also:
            w2, p2, _ = also
            r2 = w2.flops() / (ms_also * 1e-3) / 1e12
            line["also"] = {w2.name: {"value": world * r2, "unit": "TFLOP/s", "ms_per_step": ms_also,
                                      "frac": r2 / (peaks["bf16_tflops"] * 2.0), "parity_checked": True,
                                      "max_err": p2["max_err"], "traffic": TRAFFIC_BYTES.get(w2.name),
                                      "note": "independent replica per GPU, device-resident operands"}}
        if args.kernel_only:
            line["e2e"] = None
        if world == 1 and not args.no_cpu_baseline and not args.kernel_only:
            os.sched_setaffinity(0, affinity)      # the CPU baseline may use every core again
            dt, s = time_cpu(w, 1, 1, budget_s=30.0)
            line["cpu_baseline"] = {"value": w.cpu_flops(s) / dt / scale, "unit": unit,
                                    "cores": torch.get_num_threads(), "kind": "port",
                                    "sample": w.cpu_sample_desc(s)}
        print(json.dumps(line), flush=True)
    if distributed:
        dist.barrier()
        dist.destroy_process_group()


# --------------------------------------------------------------------------------------
# The reference's own tuned bench shapes (the only timings it publishes, for a B200:
# test/benchmark_tuning.json), timed its way: one call captured in a CUDA graph, an
# L2-sized zero fill before every sample (test/util.py:156-193), uniform [0, 1) inputs
# (test/bench_matmul.py:28-29).
# --------------------------------------------------------------------------------------
def run_ref_shapes(args):
    import b200k
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    reps = max(5, args.steps)

    def timeit(fn):
        for _ in range(max(3, args.warmup)):
            fn()
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                  for _ in range(reps)]
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                fn()
            for e0, e1 in events:
                flush.zero_()
                e0.record(side)
                graph.replay()
                e1.record(side)
        torch.cuda.synchronize()
        ts = sorted(e0.elapsed_time(e1) * 1e3 for e0, e1 in events)
        return ts[len(ts) // 2]

    g = torch.Generator(device=dev).manual_seed(0)
    rand = lambda *shape: torch.rand(*shape, device=dev, generator=g)
    shapes = []

    def add(name, fn, flops, published_us, source):
        us = timeit(fn)
        shapes.append({"name": name, "us": round(us, 2), "tflops": round(flops / us / 1e6, 1),
                       "published_us": published_us, "speedup": round(published_us / us, 3),
                       "source": source})

    a, b = rand(4096, 4096).half(), rand(4096, 4096).half()
    c = torch.empty(4096, 4096, device=dev, dtype=torch.float16)
    add("fp16 matmul 4096^3", lambda: b200k.cutile_matmul(a, b, C=c), 2 * 4096 ** 3, 96.27,
        "test/benchmark_tuning.json:46-59")
    aq, sa = b200k.block_quantize(rand(4096, 4096), 32, swizzled_scale=True)
    bq, sb = b200k.block_quantize(rand(4096, 4096), 32, swizzled_scale=True)
    c32 = torch.empty(4096, 4096, device=dev, dtype=torch.float32)
    add("MXFP8 4096^3, swizzled scales, fp32 out",
        lambda: b200k.cutile_swizzled_scaled_matmul(aq, sa, bq.T, sb, c32), 2 * 4096 ** 3, 71.38,
        "test/benchmark_tuning.json:549-562")
    a8 = rand(4, 8192, 2000).to(torch.float8_e4m3fn)
    b8 = rand(4, 2000, 8192).to(torch.float8_e4m3fn)
    c8 = torch.empty(4, 8192, 8192, device=dev, dtype=torch.float32)
    add("fp8 e4m3 batch matmul 4 x 8192 x 8192 x 2000, fp32 out",
        lambda: b200k.cutile_batch_matmul(4, a8, b8, c8), 2 * 4 * 8192 * 8192 * 2000, 600.73,
        "test/benchmark_tuning.json:4-17")
    del a8, b8, c8
    q, k, v = (torch.randn(1, 32, 8192, 128, device=dev, generator=g).half() for _ in range(3))
    o = torch.empty_like(q)
    add("FMHA causal fp16 B1 H32 S8192 D128", lambda: b200k.cutile_fmha(q, k, v, causal=True, Out=o),
        4 * 32 * 8192 * 8192 * 128 / 2, 587.55, "test/benchmark_tuning.json:32-44")
    qd = torch.randn(1, 32, 1, 128, device=dev, generator=g).half()
    kd, vd = (torch.randn(1, 32, 1024, 128, device=dev, generator=g).half() for _ in range(2))
    od = torch.empty_like(qd)
    add("FMHA decode q (1,32,1,128) x kv (1,32,1024,128)",
        lambda: b200k.cutile_fmha(qd, kd, vd, input_pos=1023, causal=True, Out=od),
        4 * 32 * 1024 * 128, 16.17, "test/benchmark_tuning.json:19-31")
    ak, bk = rand(256, 4096).half(), rand(4096, 256).half()
    ck = torch.empty(256, 256, device=dev, dtype=torch.float16)
    add("fp16 split-K matmul 256 x 256 x 4096", lambda: b200k.cutile_matmul(ak, bk, C=ck),
        2 * 256 * 256 * 4096, 23.11, "test/benchmark_tuning.json:60-73")
    b200k.raise_on_device_error()
    geo = 1.0
    for sh in shapes:
        geo *= sh["speedup"]
    geo **= 1.0 / len(shapes)
    line = {"metric": "geomean speed-up over the reference's published B200 timings", "value": geo,
            "unit": "x", "n_gpus": 1, "steps": reps, "warmup": max(3, args.warmup),
            "ms_per_step": sum(sh["us"] for sh in shapes) * 1e-3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": geo, "dtype": "per shape", "data": "synthetic",
            "config": {"workload": "ref_shapes", "protocol": "one call per CUDA graph, 256 MiB zero "
                       "fill before every sample, median of the samples", "shapes": shapes},
            "gpu_launches": reps * len(shapes)}
    print(json.dumps(line), flush=True)


# dram__bytes_read.sum + dram__bytes_write.sum per launch of the workload's dominant kernel,
# from one ncu capture of that kernel (None until captured).  The two AllGather / plain NVFP4
# entries are the same kernel on the same problem.
TRAFFIC_BYTES: dict[str, float | None] = {
    "mxfp8_gemm_8192x8192x8192_bf16out": 377.0e6,
    "nvfp4_gemm_8192x28672x8192_bf16out": 726.0e6,
    "allgather_nvfp4_gemm_8192x28672x8192_bf16out": 726.0e6,
    "fmha_causal_bf16_b4_h32_s8192_d128": 1066.0e6,
    "mxfp8_quantize_bf16_8192x8192": 173.0e6,
    "dense_f16_gemm_2048x2048x2048": 16.8e6,
    "fmha_decode_bf16_b32_hq32_hkv8_s2048_d128": 272.0e6,
    "nvfp4_quantize_bf16_8192x8192": 293.0e6,    # both kernels
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS) + ["ref_shapes"], default=DEFAULT_WORKLOAD)
    ap.add_argument("--launch", choices=["auto", "stream", "graph"], default="auto",
                    help="graph = the K steps replayed as one CUDA graph; auto = graph for the "
                         "workloads whose kernels are shorter than their launch path")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-also", action="store_true", help="skip the secondary MXFP8 record")
    ap.add_argument("--sustain-s", type=float, default=1.0,
                    help="seconds of the back-to-back loop reported under `sustained` (0 = skip)")
    ap.add_argument("--kernel-only", action="store_true",
                    help="skip the end-to-end, sustained and CPU legs (for profiler runs)")
    args = ap.parse_args()
    if args.workload == "ref_shapes":
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
        return run_ref_shapes(args)
    w = WORKLOADS[args.workload]()
    if args.impl == "reference":
        run_reference(args, w)
    else:
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
        run_ours(args, w)


if __name__ == "__main__":
    main()
