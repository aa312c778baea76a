"""Generates tests/golden/*.npz by running the REFERENCE's own torch helpers on the CPU.

Run where the reference checkout is available:
    REFERENCE_PATH=/path/to/cutile-python python tests/golden/make_golden.py
(the checkout's `test/` and `samples/` directories are imported; nothing is copied).
The fixtures hold small seeded inputs together with the outputs of
  block_quantize, swizzle_32_4_4       test/kernels/kernel_utils.py:38-98
  moe_align_tile_size_torch            test/kernels/fused_moe.py:113-173
  torch_moe                            samples/MoE.py:292-334
so the oracle can be pinned to them on machines without the reference.
"""
import os
import sys

import numpy as np
import torch

REF = os.environ.get("REFERENCE_PATH", os.path.expanduser("~/reference"))
sys.path.insert(0, os.path.join(REF, "test"))
sys.path.insert(0, os.path.join(REF, "samples"))
HERE = os.path.dirname(os.path.abspath(__file__))


def u8(t):
    return t.view(torch.uint8).numpy()


def main():
    from kernels.kernel_utils import block_quantize, swizzle_32_4_4
    from kernels.fused_moe import moe_align_tile_size_torch
    import MoE as moe_sample

    g = torch.Generator().manual_seed(1234)
    # --- block_quantize: random fp32, bf16-representable data, and edge rows
    x = torch.randn(128, 256, generator=g)
    x[0, :32] = 0.0                                   # all-zero block -> clamp path
    x[1, :32] = 0.0; x[1, 3] = 448.0                  # amax exactly 448 * 2^0
    x[2, :32] = 0.0; x[2, 7] = -448.0 * 2.0 ** -5     # exact power-of-two boundary
    x[3, :32] = 0.0; x[3, 9] = 448.0 * 2.0 ** 4 * (1 + 2.0 ** -7)   # one bf16 ulp above
    x[4, :32] = 1e-20                                 # below the 1e-12 clamp
    x[5, :32] = torch.linspace(-500, 500, 32)         # large values
    x[6, 32:64] = 2.0 ** -30
    xb = (torch.randn(128, 256, generator=g) * 3.0).bfloat16().float()
    q, s = block_quantize(x, 32)
    qb, sb = block_quantize(xb, 32)
    sw = swizzle_32_4_4(s)
    np.savez_compressed(os.path.join(HERE, "block_quantize.npz"),
                        x=x.numpy(), q=u8(q), scale=u8(s), swizzled=u8(sw),
                        xb=xb.numpy(), qb=u8(qb), scaleb=u8(sb))

    # --- moe_align_tile_size_torch
    cases = {}
    for name, (tokens, topk, experts, tile_m, seed) in {
        "a": (37, 3, 8, 16, 1), "b": (64, 8, 64, 128, 2), "c": (5, 2, 4, 4, 3),
        "d": (256, 4, 16, 32, 4), "e": (1, 1, 8, 16, 5),
    }.items():
        gg = torch.Generator().manual_seed(seed)
        logits = torch.randn(tokens, experts, generator=gg)
        ids = torch.topk(logits, topk, dim=-1).indices
        if name == "c":
            ids[:] = ids[0]                            # every token to the same experts
        st, se = moe_align_tile_size_torch(ids, tile_m, experts)
        cases[f"{name}_ids"] = ids.numpy()
        cases[f"{name}_cfg"] = np.array([tokens, topk, experts, tile_m])
        cases[f"{name}_sorted_token_ids"] = st.numpy()
        cases[f"{name}_sorted_expert_ids"] = se.numpy()
    np.savez_compressed(os.path.join(HERE, "moe_align.npz"), **cases)

    # --- torch_moe on a small fp32 problem
    gg = torch.Generator().manual_seed(77)
    T, H, I, E, K = 24, 64, 32, 4, 2
    hidden = torch.randn(T, H, generator=gg)
    w1 = 0.1 * torch.randn(E, 2 * I, H, generator=gg)
    w2 = 0.1 * torch.randn(E, H, I, generator=gg)
    logits = torch.randn(T, E, generator=gg)
    vals, ids = torch.topk(logits, K, dim=-1)
    tw = torch.softmax(vals, dim=-1)
    out = moe_sample.torch_moe(hidden, w1, w2, tw, ids)
    np.savez_compressed(os.path.join(HERE, "torch_moe.npz"), hidden=hidden.numpy(), w1=w1.numpy(),
                        w2=w2.numpy(), topk_weights=tw.numpy(), topk_ids=ids.numpy(),
                        out=out.numpy())
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
