"""Benchmark of the hot path on B200: TFLOPS of the block-scaled / dense contraction kernels.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload mxfp8_gemm|nvfp4_gemm|dense_f16|ag_nvfp4_gemm|moe_ep_bf16|ref_shapes|fmha_decode|
                                fmha_causal|moe_bf16|moe_mxfp8|mxfp8_quantize|nvfp4_quantize]

One step = one pass of the workload's kernel over one batch of seeded synthetic input.
The default workload is the headline configuration: MXFP8 GEMM, M = N = K = 8192, e4m3 operands
with ue8m0 scales per 32 elements of K, fp32 accumulation, bf16 output.  With N > 1 every
rank runs the same problem on its own GPU (the GEMM does not shard: replicas only) and the
value is the sum over ranks divided by the slowest rank's time.

`--impl reference` times the reference's CPU ground truth for the same workload (the
de-quantised fp32 matmul of samples/BlockScaledMatMul.py:359-361, restated in oracle/) on
the host cores, on a bounded block of the output.

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


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"bf16_tflops": float(d["bf16_tflops"]), "hbm_gbs": float(d["hbm_gbs"]),
                "source": "measured"}
    return {"bf16_tflops": 1590.0, "hbm_gbs": 6650.0, "source": "fallback"}


# --------------------------------------------------------------------------------------
# Workloads
# --------------------------------------------------------------------------------------
class Workload:
    name = ""
    dtype = ""
    tensor_rate_vs_bf16 = 1.0   # tensor-core rate of the operand format relative to bf16
    distributed = False         # needs a process group even on one GPU

    def config(self):
        raise NotImplementedError

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


class Mxfp8Gemm(Workload):
    """The headline MXFP8 configuration (8192 cubed, bf16 output)."""
    name = "mxfp8_gemm_8192x8192x8192_bf16out"
    dtype = "e4m3 x e4m3 (ue8m0 scale / 32) -> fp32 accumulate -> bf16"
    tensor_rate_vs_bf16 = 2.0
    M = N = K = 8192
    seed = 1
    sets = 2   # rotating operand/output sets, so that no step finds its inputs in L2
    cpu_block_limit = 8192

    def flops(self):
        return 2.0 * self.M * self.N * self.K

    def algorithmic_bytes(self):
        ks = self.K // 32
        return self.M * self.K + self.N * self.K + (self.M + self.N) * ks + 2 * self.M * self.N

    def setup(self, device):
        import b200k
        g = torch.Generator(device=device).manual_seed(self.seed)
        self.inputs = []
        for i in range(self.sets):
            a = torch.randn(self.M, self.K, device=device, generator=g).bfloat16()
            b = torch.randn(self.N, self.K, device=device, generator=g).bfloat16()
            aq, sa = b200k.block_quantize(a, 32, swizzled_scale=True)
            bq, sb = b200k.block_quantize(b, 32, swizzled_scale=True)
            c = torch.empty(self.M, self.N, device=device, dtype=torch.bfloat16)
            self.inputs.append((aq, sa, bq, sb, c))
            del a, b
        self.b200k = b200k
        self.i = 0

    def step(self):
        aq, sa, bq, sb, c = self.inputs[self.i % self.sets]
        self.i += 1
        self.b200k.cutile_block_scaled_matmul(aq, sa, bq.T, sb, C=c)
        return c

    launches_per_step = 1

    # ---- end-to-end: host buffers in, host buffer out, through the public call
    def setup_e2e(self, device):
        aq, sa, bq, sb, c = self.inputs[0]
        self.pipe_setup(device, [t.cpu().pin_memory() for t in (aq, sa, bq, sb)], c)

    def step_e2e(self):
        def compute(dev_in, dev_out):
            aq, sa, bq, sb = dev_in
            self.b200k.cutile_block_scaled_matmul(aq, sa, bq.T, sb, C=dev_out)
        self.pipe_step(compute)

    # ---- CPU ground truth on an S x S block of the output
    def cpu_setup(self):
        import oracle
        g = torch.Generator().manual_seed(self.seed)
        s = self.cpu_block_limit
        a = torch.randn(s, self.K, generator=g).bfloat16()
        b = torch.randn(s, self.K, generator=g).bfloat16()
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
                "l2": f"{self.sets} rotating operand/output sets of "
                      f"{self.algorithmic_bytes() / 2**20:.0f} MiB each (> 126 MiB L2)"}


class Nvfp4Gemm(Mxfp8Gemm):
    """The NVFP4 FFN up-projection (8192 x 28672 x 8192) on one GPU: the per-rank problem of
    the AllGather GEMM."""
    name = "nvfp4_gemm_8192x28672x8192_bf16out"
    dtype = "e2m1 x e2m1 (ue4m3 scale / 16, fp32 tensor scale) -> fp32 accumulate -> bf16"
    tensor_rate_vs_bf16 = 4.0
    M, N, K = 8192, 28672, 8192
    seed = 2

    def algorithmic_bytes(self):
        return (self.M + self.N) * (self.K // 2 + self.K // 16) + 2 * self.M * self.N

    def setup(self, device):
        import b200k
        g = torch.Generator(device=device).manual_seed(self.seed)
        self.inputs = []
        for i in range(self.sets):
            a = torch.randn(self.M, self.K, device=device, generator=g).bfloat16()
            b = (0.02 * torch.randn(self.N, self.K, device=device, generator=g)).bfloat16()
            qa = b200k.nvfp4_quantize(a)
            qb = b200k.nvfp4_quantize(b)
            c = torch.empty(self.M, self.N, device=device, dtype=torch.bfloat16)
            self.inputs.append((qa, qb, c))
            del a, b
        self.b200k = b200k
        self.i = 0

    def step(self):
        qa, qb, c = self.inputs[self.i % self.sets]
        self.i += 1
        self.b200k.cutile_nvfp4_matmul(*qa, *qb, C=c)
        return c

    def setup_e2e(self, device):
        qa, qb, c = self.inputs[0]
        flat = list(qa) + list(qb)
        self.pipe_setup(device, [t.cpu().pin_memory() for t in flat], c)

    def step_e2e(self):
        self.pipe_step(lambda dev_in, dev_out: self.b200k.cutile_nvfp4_matmul(*dev_in, C=dev_out))

    def cpu_setup(self):
        import oracle
        g = torch.Generator().manual_seed(self.seed)
        s = 2048
        a = torch.randn(s, self.K, generator=g).bfloat16()
        b = (0.02 * torch.randn(s, self.K, generator=g)).bfloat16()
        self.cpu_ops = (oracle.nvfp4_quantize_ref(a), oracle.nvfp4_quantize_ref(b))
        self.oracle = oracle

    def cpu_step(self, s):
        (aq, asf, ats), (bq, bsf, bts) = self.cpu_ops
        return self.oracle.nvfp4_matmul_ref(aq[:s], asf[:s], ats, bq[:s], bsf[:s], bts)

    def config(self):
        c = super().config()
        c["scale_block"] = 16
        return c


class AgNvfp4Gemm(Nvfp4Gemm):
    """The NVFP4 FFN up-projection as the AllGather GEMM: A row-sharded M / world per rank, gathered
    over NVLink from the peers' symmetric-memory buffers, every rank computing the full
    (M, N) product against its own weights (fixed work per rank: weak scaling)."""
    name = "allgather_nvfp4_gemm_8192x28672x8192_bf16out"
    distributed = True
    sets = 1
    launches_per_step = 3   # two gather kernels + the GEMM

    def setup(self, device):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        import b200k
        world, rank = dist.get_world_size(), dist.get_rank()
        rows = self.M // world
        g = torch.Generator(device=device).manual_seed(self.seed + 1000 * rank)
        a = torch.randn(rows, self.K, device=device, generator=g).bfloat16()
        gw = torch.Generator(device=device).manual_seed(self.seed)
        b = (0.02 * torch.randn(self.N, self.K, device=device, generator=gw)).bfloat16()
        aq, asf, ats = b200k.nvfp4_quantize(a)
        self.wq = b200k.nvfp4_quantize(b)
        del a, b
        self.s_q = symm_mem.empty(aq.shape, device=device, dtype=torch.uint8).copy_(aq)
        self.s_sf = symm_mem.empty(asf.shape, device=device, dtype=torch.uint8).copy_(asf.view(torch.uint8))
        self.s_ts = symm_mem.empty(1, device=device, dtype=torch.float32).copy_(ats)
        self.plan = b200k.Nvfp4GatherMatmul(self.s_q, self.s_sf, self.s_ts)
        self.c = torch.empty(self.M, self.N, device=device, dtype=torch.bfloat16)
        self.flush = torch.empty(L2_BYTES * 2, dtype=torch.uint8, device=device)
        dist.barrier()
        torch.cuda.synchronize()
        self.b200k = b200k

    def step(self):
        return self.plan.run(*self.wq, out=self.c)

    def setup_e2e(self, device):
        self.host_in = [t.cpu().pin_memory() for t in (self.s_q, self.s_sf, self.s_ts)]
        self.host_out = torch.empty_like(self.c, device="cpu").pin_memory()
        self.h2d = sum(t.numel() * t.element_size() for t in self.host_in)
        self.d2h = self.host_out.numel() * self.host_out.element_size()

    def step_e2e(self):
        for d, h in zip((self.s_q, self.s_sf, self.s_ts), self.host_in):
            d.copy_(h, non_blocking=True)
        self.plan.run(*self.wq, out=self.c)
        self.host_out.copy_(self.c, non_blocking=True)

    def config(self):
        c = super().config()
        c["l2"] = "operands and output of one step are 610 MiB (> 126 MiB L2)"
        c["sharding"] = "A rows M/world per rank, gathered by peer loads; B replicated"
        return c


class MoeEpBf16(Workload):
    """The MoE FFN configuration (16384 tokens, hidden 4096, 64 experts, intermediate 1536,
    top-8) with experts and tokens sharded over the ranks and an NVLink all-to-all for
    dispatch and combine.  The whole problem is fixed, so this scales strongly."""
    name = "moe_ffn_ep_16384tok_h4096_e64_i1536_top8_bf16"
    dtype = "bf16 x bf16 -> fp32 accumulate -> bf16"
    tensor_rate_vs_bf16 = 1.0
    distributed = True
    scaling = "strong"
    T, H, E, I, K = 16384, 4096, 64, 1536, 8
    seed = 4
    launches_per_step = 8

    def flops(self):
        return 6.0 * self.T * self.K * self.H * self.I / self.world   # per rank

    def algorithmic_bytes(self):
        return 2 * (self.E * 3 * self.I * self.H + 2 * self.T * self.H) // self.world

    def setup(self, device):
        import torch.distributed as dist
        import b200k
        self.world, rank = dist.get_world_size(), dist.get_rank()
        tl, el = self.T // self.world, self.E // self.world
        g = torch.Generator(device=device).manual_seed(self.seed + 1000 * rank)
        self.x = torch.randn(tl, self.H, device=device, generator=g).bfloat16()
        w1 = (0.02 * torch.randn(el, 2 * self.I, self.H, device=device, generator=g)).bfloat16()
        w2 = (0.02 * torch.randn(el, self.H, self.I, device=device, generator=g)).bfloat16()
        logits = torch.randn(tl, self.E, device=device, generator=g)
        vals, self.ids = torch.topk(logits, self.K, dim=-1)
        self.tw = torch.softmax(vals, dim=-1).bfloat16()
        self.ep = b200k.ExpertParallelMoE(w1, w2, self.E)
        self.b200k = b200k

    def step(self):
        return self.ep.forward(self.x, self.tw, self.ids)

    def setup_e2e(self, device):
        self.host_in = [t.cpu().pin_memory() for t in (self.x, self.tw, self.ids)]
        self.dev_in = [torch.empty_like(t) for t in (self.x, self.tw, self.ids)]
        self.host_out = torch.empty_like(self.x, device="cpu").pin_memory()
        self.h2d = sum(t.numel() * t.element_size() for t in self.host_in)
        self.d2h = self.host_out.numel() * self.host_out.element_size()

    def step_e2e(self):
        for d, h in zip(self.dev_in, self.host_in):
            d.copy_(h, non_blocking=True)
        out = self.ep.forward(*self.dev_in)
        self.host_out.copy_(out, non_blocking=True)

    def cpu_setup(self):
        import oracle
        g = torch.Generator().manual_seed(self.seed)
        t, e = 512, 8
        self.cpu_ops = ((0.5 * torch.randn(t, self.H, generator=g)),
                        0.02 * torch.randn(e, 2 * self.I, self.H, generator=g),
                        0.02 * torch.randn(e, self.H, self.I, generator=g))
        self.cpu_route = oracle.moe_route_ref(torch.randn(t, e, generator=g), 2)
        self.oracle = oracle

    def cpu_step(self, s):
        x, w1, w2 = self.cpu_ops
        tw, ids = self.cpu_route
        return self.oracle.moe_ref(x[:s], w1, w2, tw[:s], ids[:s])

    def cpu_flops(self, s):
        return 6.0 * s * 2 * self.H * self.I

    def cpu_sample_desc(self, s):
        return f"{s} tokens, 8 experts, top-2 of the same FFN in fp32 (torch CPU)"

    def config(self):
        return {"workload": self.name, "tokens": self.T, "hidden": self.H, "experts": self.E,
                "intermediate": self.I, "topk": self.K, "seed": self.seed,
                "sharding": "experts E/world and tokens T/world per rank; all_to_all dispatch + combine",
                "l2": "expert weights alone are 2.4 GB / world per rank (> 126 MiB L2)"}


class FmhaCausal(Workload):
    """Causal attention forward, bf16, batch 4, 32 heads, sequence 8192, head dim 128."""
    name = "fmha_causal_bf16_b4_h32_s8192_d128"
    dtype = "bf16 x bf16 -> fp32 softmax / accumulate -> bf16"
    tensor_rate_vs_bf16 = 1.0
    B, H, S, D = 4, 32, 8192, 128
    seed = 3
    sets = 1
    cpu_limit = 4096
    launches_per_step = 1

    def flops(self):
        return 4.0 * self.B * self.H * self.S * self.S * self.D * 0.5

    def algorithmic_bytes(self):
        return 4 * self.B * self.H * self.S * self.D * 2

    def setup(self, device):
        import b200k
        g = torch.Generator(device=device).manual_seed(self.seed)
        shape = (self.B, self.H, self.S, self.D)
        self.q, self.k, self.v = (torch.randn(shape, device=device, generator=g).bfloat16() for _ in range(3))
        self.o = torch.empty_like(self.q)
        self.b200k = b200k

    def step(self):
        return self.b200k.cutile_fmha(self.q, self.k, self.v, causal=True, Out=self.o)

    def setup_e2e(self, device):
        self.pipe_setup(device, [t.cpu().pin_memory() for t in (self.q, self.k, self.v)], self.o)

    def step_e2e(self):
        self.pipe_step(lambda dev_in, dev_out: self.b200k.cutile_fmha(*dev_in, causal=True, Out=dev_out))

    def cpu_setup(self):
        import oracle
        g = torch.Generator().manual_seed(self.seed)
        self.cpu_ops = tuple(torch.randn(1, 1, 4096, self.D, generator=g).bfloat16() for _ in range(3))
        self.oracle = oracle

    def cpu_step(self, s):
        q, k, v = self.cpu_ops
        return self.oracle.fmha_ref(q[:, :, :s], k[:, :, :s], v[:, :, :s], causal=True)

    def cpu_flops(self, s):
        return 4.0 * s * s * self.D * 0.5

    def cpu_sample_desc(self, s):
        return f"one head, sequence {s}: fp32 softmax(QK^T + causal mask)V (torch CPU)"

    def config(self):
        return {"workload": self.name, "batch": self.B, "heads": self.H, "seq": self.S,
                "head_dim": self.D, "causal": True, "seed": self.seed,
                "l2": "Q, K, V and O are 268 MB each (> 126 MiB L2)"}


class MoeBf16(Workload):
    """The MoE FFN (16384 tokens, hidden 4096, 64 experts, intermediate 1536, top-8) on one GPU,
    bf16 weights: align -> gather -> grouped GEMM + SwiGLU -> grouped GEMM + scatter -> sum."""
    name = "moe_ffn_16384tok_h4096_e64_i1536_top8_bf16"
    dtype = "bf16 x bf16 -> fp32 accumulate -> bf16"
    tensor_rate_vs_bf16 = 1.0
    T, H, E, I, K = 16384, 4096, 64, 1536, 8
    seed = 4
    mxfp8 = False
    launches_per_step = 8

    def flops(self):
        return 6.0 * self.T * self.K * self.H * self.I

    def algorithmic_bytes(self):
        return 2 * (self.E * 3 * self.I * self.H + 2 * self.T * self.H)

    def setup(self, device):
        import b200k
        g = torch.Generator(device=device).manual_seed(self.seed)
        self.x = torch.randn(self.T, self.H, device=device, generator=g).bfloat16()
        w1 = (0.02 * torch.randn(self.E, 2 * self.I, self.H, device=device, generator=g)).bfloat16()
        w2 = (0.02 * torch.randn(self.E, self.H, self.I, device=device, generator=g)).bfloat16()
        vals, self.ids = torch.topk(torch.randn(self.T, self.E, device=device, generator=g), self.K, dim=-1)
        self.tw = torch.softmax(vals, dim=-1).bfloat16()
        if self.mxfp8:
            self.w = b200k.quantize_expert_weights(w1) + b200k.quantize_expert_weights(w2)
        else:
            self.w = (w1, w2)
        self.b200k = b200k

    def step(self):
        if self.mxfp8:
            return self.b200k.cutile_moe_mxfp8(self.x, *self.w, self.tw, self.ids)
        return self.b200k.cutile_moe(self.x, *self.w, self.tw, self.ids)

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

    cpu_setup = MoeEpBf16.cpu_setup
    cpu_step = MoeEpBf16.cpu_step
    cpu_flops = MoeEpBf16.cpu_flops
    cpu_sample_desc = MoeEpBf16.cpu_sample_desc

    def config(self):
        return {"workload": self.name, "tokens": self.T, "hidden": self.H, "experts": self.E,
                "intermediate": self.I, "topk": self.K, "seed": self.seed,
                "l2": "expert weights alone are 2.4 GB (> 126 MiB L2)"}


class MoeMxfp8(MoeBf16):
    name = "moe_ffn_16384tok_h4096_e64_i1536_top8_mxfp8"
    dtype = "e4m3 x e4m3 (ue8m0 scale / 32) -> fp32 accumulate -> bf16"
    tensor_rate_vs_bf16 = 2.0
    mxfp8 = True
    launches_per_step = 9


class Mxfp8Quantize(Workload):
    """The quantiser that feeds the headline GEMM: bf16 8192 x 8192 -> e4m3 + swizzled ue8m0
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
        g = torch.Generator(device=device).manual_seed(self.seed)
        self.xs = [torch.randn(self.M, self.K, device=device, generator=g).bfloat16() for _ in range(self.sets)]
        self.b200k = b200k
        self.i = 0

    def step(self):
        x = self.xs[self.i % self.sets]
        self.i += 1
        return self.b200k.block_quantize(x, 32, swizzled_scale=True)

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
        self.cpu_ops = (torch.randn(4096, self.K, generator=g).bfloat16(),)
        self.oracle = oracle

    def cpu_step(self, s):
        return self.oracle.block_quantize_ref(self.cpu_ops[0][:s])

    def cpu_flops(self, s):
        return float(s * self.K * 3 + s * self.K // 32)

    def cpu_sample_desc(self, s):
        return f"{s} rows of {self.K} bf16 values through block_quantize's restatement (torch CPU)"

    def config(self):
        return {"workload": self.name, "rows": self.M, "K": self.K, "seed": self.seed,
                "l2": f"{self.sets} rotating inputs of 128 MiB each (> 126 MiB L2)"}


class FmhaDecode(Mxfp8Quantize):
    """One decode step of grouped-query attention over a long KV cache: the reference's decode
    bench shapes (test/bench_attention.py:33-44: one query per sequence, 32 query heads on 8 KV
    heads) at a serving-size batch.  K and V are read once: HBM-bound."""
    name = "fmha_decode_bf16_b32_hq32_hkv8_s2048_d128"
    dtype = "bf16, fp32 softmax"
    B, HQ, HKV, S, D = 32, 32, 8, 2048, 128
    seed = 5
    sets = 2
    launches_per_step = 1

    def algorithmic_bytes(self):
        return 2 * self.B * self.HKV * self.S * self.D * 2 + 2 * self.B * self.HQ * self.D * 2

    def setup(self, device):
        import b200k
        g = torch.Generator(device=device).manual_seed(self.seed)
        mk = lambda *sh: torch.randn(*sh, device=device, generator=g).bfloat16()
        self.xs = [(mk(self.B, self.HQ, 1, self.D), mk(self.B, self.HKV, self.S, self.D),
                    mk(self.B, self.HKV, self.S, self.D)) for _ in range(self.sets)]
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
        mk = lambda *sh: torch.randn(*sh, generator=g).bfloat16()
        self.cpu_ops = (mk(self.B, self.HQ, 1, self.D), mk(self.B, self.HKV, self.S, self.D),
                        mk(self.B, self.HKV, self.S, self.D))
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

    def config(self):
        return {"workload": self.name, "batch": self.B, "heads_q": self.HQ, "heads_kv": self.HKV,
                "keys": self.S, "head_dim": self.D, "seed": self.seed,
                "l2": f"{self.sets} rotating K/V sets of 268 MB each (> 126 MiB L2)"}


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


class DenseF16(Mxfp8Gemm):
    """The sample-sized dense fp16 matmul (2048 cubed)."""
    name = "dense_f16_gemm_2048x2048x2048"
    dtype = "f16 x f16 -> fp32 accumulate -> f16"
    tensor_rate_vs_bf16 = 1.0
    M = N = K = 2048
    seed = 0
    sets = 12   # 12 x 24 MiB > L2
    cuda_graph = True

    def algorithmic_bytes(self):
        return 2 * (self.M * self.K + self.K * self.N + self.M * self.N)

    def setup(self, device):
        import b200k
        g = torch.Generator(device=device).manual_seed(self.seed)
        self.inputs = []
        for i in range(self.sets):
            a = torch.randn(self.M, self.K, device=device, generator=g).half()
            b = torch.randn(self.K, self.N, device=device, generator=g).half()
            self.inputs.append((a, b, torch.empty(self.M, self.N, device=device, dtype=torch.float16)))
        self.b200k = b200k
        self.i = 0

    def step(self):
        a, b, c = self.inputs[self.i % self.sets]
        self.i += 1
        return self.b200k.cutile_matmul(a, b, C=c)

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

    def cpu_sample_desc(self, s):
        return f"{s}x{s} block of the output, K={self.K}: A.float() @ B.float() (torch CPU)"

    def config(self):
        c = super().config()
        c.pop("scale_block")
        c["out"] = "f16"
        return c


WORKLOADS = {"mxfp8_gemm": Mxfp8Gemm, "nvfp4_gemm": Nvfp4Gemm, "dense_f16": DenseF16,
             "ag_nvfp4_gemm": AgNvfp4Gemm, "moe_ep_bf16": MoeEpBf16, "fmha_causal": FmhaCausal,
             "moe_bf16": MoeBf16, "moe_mxfp8": MoeMxfp8, "mxfp8_quantize": Mxfp8Quantize,
             "nvfp4_quantize": Nvfp4Quantize, "fmha_decode": FmhaDecode}


# --------------------------------------------------------------------------------------
# Clock sampling (read-only NVML queries during the timed region)
# --------------------------------------------------------------------------------------
class ClockSampler:
    REASONS = {
        0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap",
        0x8: "hw_slowdown", 0x10: "sync_boost", 0x20: "sw_thermal_slowdown",
        0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting",
    }

    def __init__(self, device):
        self.samples, self.reasons, self.max_mhz = [], set(), None
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
            time.sleep(0.02)

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
        if self.ok:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread:
            self._thread.join()

    def summary(self):
        if not self.ok or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz,
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


def run_ours(args, w):
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    distributed = world > 1 or getattr(w, "distributed", False)
    if distributed:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29531")
        os.environ.setdefault("RANK", "0")
        os.environ.setdefault("WORLD_SIZE", "1")
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    import b200k
    w.setup(device)
    for _ in range(max(3, args.warmup)):
        w.step()
    barrier()
    sampler = ClockSampler(device)
    sampler.start()
    ev0 = torch.cuda.Event(enable_timing=True)
    ev1 = torch.cuda.Event(enable_timing=True)
    use_graph = bool(getattr(w, "cuda_graph", False)) and not distributed
    if use_graph:
        # launch-bound workloads (kernels of a few tens of microseconds): the K steps are
        # captured once and replayed as one graph, so the device never waits for the host
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(args.steps):
                w.step()
        graph.replay()
        barrier()
        ev0.record()
        graph.replay()
        ev1.record()
    else:
        ev0.record()
        for _ in range(args.steps):
            w.step()
        ev1.record()
    barrier()
    sampler.sample()
    sampler.stop()
    ms = ev0.elapsed_time(ev1) / args.steps
    b200k.raise_on_device_error()

    # end to end: pinned host buffers -> device -> kernel -> pinned host buffer
    e2e_steps = max(3, min(args.steps, 20))
    if args.kernel_only:
        ms_e2e, w.h2d, w.d2h = float("nan"), 0, 0
    else:
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

    if world > 1:
        t = torch.tensor([ms, ms_e2e], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e = t.tolist()

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
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms,
            "higher_is_better": True, "scaling": getattr(w, "scaling", "weak"), "vs_baseline": None,
            "dtype": w.dtype, "data": "synthetic",
            "config": dict(w.config(), launch="cuda_graph" if use_graph else "stream"),
            "e2e": {"value": world * flops / (ms_e2e * 1e-3) / scale, "unit": unit,
                    "h2d_bytes_per_step": w.h2d, "d2h_bytes_per_step": w.d2h,
                    "ms_per_step": ms_e2e, "steps": e2e_steps,
                    "overlap": "H2D, kernel and D2H of consecutive steps on three streams"
                               if w.e2e_pipelined else "none (one stream)"},
            "gpu_launches": args.steps * w.launches_per_step,
            "clocks": sampler.summary(),
            "roofline": {"bound": "hbm" if hbm else "tensor", "achieved": per_gpu, "peak": peak,
                         "unit": unit, "frac": per_gpu / peak, "peak_source": peak_source,
                         "traffic": TRAFFIC_BYTES.get(w.name),
                         "algorithmic_bytes": w.algorithmic_bytes()},
        }
        if args.kernel_only:
            line["e2e"] = None
        if world == 1 and not args.no_cpu_baseline and not args.kernel_only:
            dt, s = time_cpu(w, 1, 1, budget_s=30.0)
            line["cpu_baseline"] = {"value": w.cpu_flops(s) / dt / scale, "unit": unit,
                                    "cores": torch.get_num_threads(), "kind": "port",
                                    "sample": w.cpu_sample_desc(s)}
        print(json.dumps(line), flush=True)
    if distributed:
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


# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the
# ncu captures summarised under profiles/ (None until captured)
TRAFFIC_BYTES: dict[str, float | None] = {
    "mxfp8_gemm_8192x8192x8192_bf16out": 477.0e6,          # profiles/gemm_pair_mxfp8_8192.md
    "nvfp4_gemm_8192x28672x8192_bf16out": 1007.0e6,        # profiles/gemm_pair_nvfp4_8192x28672x8192.md
    "fmha_causal_bf16_b4_h32_s8192_d128": 1066.0e6,        # profiles/fmha_fwd_pair_causal_b4_h32_s8192_d128.md
    "mxfp8_quantize_bf16_8192x8192": 173.0e6,              # profiles/mxfp8_quantize_bf16_8192x8192.md
    "dense_f16_gemm_2048x2048x2048": 16.8e6,               # profiles/gemm_dense_f16_2048.md
    "fmha_decode_bf16_b32_hq32_hkv8_s2048_d128": 272.0e6,  # profiles/fmha_decode_bf16_b32_hq32_hkv8_s2048_d128.md
    "nvfp4_quantize_bf16_8192x8192": 293.0e6,              # profiles/nvfp4_quantize_bf16_8192x8192.md (both kernels)
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS) + ["ref_shapes"], default="mxfp8_gemm")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--kernel-only", action="store_true",
                    help="skip the end-to-end and CPU legs (for profiler runs)")
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
