"""Host-side checks of bench.py: every workload describes itself without a GPU, the traffic
figures it reports belong to workloads that exist and to profile summaries that are committed."""
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


def test_traffic_figures_point_at_committed_profiles():
    bench = _bench()
    names = {cls().name for cls in bench.WORKLOADS.values()}
    text = open(os.path.join(ROOT, "bench.py")).read()
    block = text[text.index("TRAFFIC_BYTES"):]
    block = block[:block.index("}")]
    for name, value in bench.TRAFFIC_BYTES.items():
        assert name in names, f"{name}: no such workload"
        assert value is None or value > 0
    for path in re.findall(r"profiles/[\w.\-]+\.md", block):
        assert os.path.exists(os.path.join(ROOT, path)), path


def test_profile_summaries_are_text_and_name_their_command():
    pdir = os.path.join(ROOT, "profiles")
    files = sorted(os.listdir(pdir))
    assert files
    for f in files:
        assert f.endswith((".md", ".txt")), f
        body = open(os.path.join(pdir, f)).read()
        assert "--clock-control none" in body, f"{f}: every ncu command carries --clock-control none"
        assert "bench.py" in body, f"{f}: the command runs committed files"
        assert os.path.getsize(os.path.join(pdir, f)) < 16 << 10, f
