"""Host-side checks of bench.py: every workload describes itself without a GPU, the traffic
figures it reports belong to workloads that exist and have a committed profile summary, and the
GPU and CPU arms describe and draw the same problem."""
import importlib.util
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_every_workload_describes_itself():
    bench = _bench()
    names = set()
    for key, cls in bench.WORKLOADS.items():
        w = cls()
        if getattr(w, "distributed", False):
            w.world, w.rank = 1, 0                     # set by setup() from the process group
        cfg = w.config()
        assert cfg["workload"] == w.name and w.name not in names, key
        names.add(w.name)
        assert "model" not in cfg                      # a workload, not a model
        assert w.flops() > 0 and w.algorithmic_bytes() > 0, key
        assert isinstance(w.dtype, str) and w.dtype, key
        assert getattr(w, "bound", "tensor") in ("tensor", "hbm"), key


def test_traffic_figures_belong_to_workloads_with_a_committed_profile():
    bench = _bench()
    names = {cls().name for cls in bench.WORKLOADS.values()}
    profiles = " ".join(open(os.path.join(ROOT, "profiles", f)).read()
                        for f in os.listdir(os.path.join(ROOT, "profiles")))
    for name, value in bench.TRAFFIC_BYTES.items():
        assert name in names, f"{name}: no such workload"
        assert value is None or value > 0
        key = [k for k, cls in bench.WORKLOADS.items() if cls().name == name][0]
        # a summary of the capture the figure comes from names the workload's bench command
        plain = {"ag_nvfp4_gemm": "nvfp4_gemm"}.get(key, key)
        assert f"--workload {plain}" in profiles or f"--workload {key}" in profiles or \
            (key == "mxfp8_gemm" and "bench.py" in profiles), key


def test_both_arms_describe_the_same_config_and_draw_the_same_numbers():
    bench = _bench()
    for key, cls in bench.WORKLOADS.items():
        a, b = cls(), cls()
        b.world, b.rank = 8, 3                 # the config names the problem, not the launch
        assert a.config() == b.config(), key
        assert "launch" not in a.config()
    # the leading rows of a large CPU draw equal a smaller draw from the same state
    import torch
    g1, g2 = torch.Generator().manual_seed(2), torch.Generator().manual_seed(2)
    full = bench.randn_rows(g1, 512, 64)
    part = bench.randn_rows(g2, 512, 64, take=96)
    assert torch.equal(full[:96], part)
    # and the GEMM workloads' CPU arm reuses the GPU arm's draw
    w = bench.Mxfp8Gemm()
    w.M = w.N = 256
    w.K = 128
    a_full, b_full = w.draw(torch.Generator().manual_seed(w.seed))
    a_cut, b_cut = w.draw(torch.Generator().manual_seed(w.seed), take_a=64, take_b=32)
    assert torch.equal(a_full[:64], a_cut) and torch.equal(b_full[:32], b_cut)


def test_profile_summaries_are_text_and_name_their_command():
    pdir = os.path.join(ROOT, "profiles")
    files = sorted(os.listdir(pdir))
    assert files
    for f in files:
        assert f.endswith((".md", ".txt")), f
        body = open(os.path.join(pdir, f)).read()
        assert "--clock-control none" in body, f"{f}: every ncu command carries --clock-control none"
        assert "bench.py" in body or "pytest tests/" in body, f"{f}: the command runs committed files"
        assert os.path.getsize(os.path.join(pdir, f)) < 16 << 10, f
