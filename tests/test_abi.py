"""The C-ABI library loads without a GPU and exports every symbol include/b200k.h
declares; host-side argument validation answers before any CUDA work is enqueued."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200k.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200k_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_entry_points():
    names = _declared_symbols()
    for must in ("b200k_gemm", "b200k_block_scaled_gemm", "b200k_mxfp8_quantize",
                 "b200k_nvfp4_quantize", "b200k_sf_swizzle", "b200k_last_error"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from b200k import _lib
    handle = _lib.lib()
    for name in _declared_symbols():
        assert hasattr(handle, name), f"{name} declared in b200k.h but not exported"
    assert set(_lib.SIGNATURES) == set(_declared_symbols())


def test_version_and_error_strings():
    from b200k import _lib
    assert b"sm_100a" in _lib.lib().b200k_version()
    assert isinstance(_lib.lib().b200k_last_error(), bytes)


def test_null_args_rejected_without_gpu():
    from b200k import _lib
    h = _lib.lib()
    assert h.b200k_gemm(None, None) == _lib.INVALID_ARG
    assert b"null" in h.b200k_last_error()
    assert h.b200k_block_scaled_gemm(None, None) == _lib.INVALID_ARG
    assert h.b200k_mxfp8_quantize(None, None) == _lib.INVALID_ARG
    args = _lib.GemmArgs()
    args.m, args.n, args.k, args.batch = -1, 4, 4, 1
    assert h.b200k_gemm(ctypes.byref(args), None) == _lib.INVALID_ARG
    # empty problems are accepted and do nothing
    args.m = 0
    assert h.b200k_gemm(ctypes.byref(args), None) == _lib.OK


def test_wrappers_validate_like_the_samples():
    import torch
    import b200k
    a = torch.zeros(4, 8)
    b = torch.zeros(9, 4)
    with pytest.raises(ValueError, match="Incompatible matrices"):
        b200k.cutile_matmul(a, b)
    with pytest.raises(ValueError, match="CUDA device"):
        b200k.cutile_matmul(a, torch.zeros(8, 4))
    with pytest.raises(ValueError, match="larger than the inner most"):
        b200k.block_quantize(torch.zeros(4, 16), 32)


def test_ctypes_mirrors_match_the_header_layout(tmp_path):
    """Every ctypes.Structure in b200k/_lib.py has the size and field offsets a C compiler
    gives the struct of the same role in include/b200k.h."""
    import shutil
    import subprocess
    from b200k import _lib
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        pytest.skip("no C compiler")
    pairs = {"b200k_gemm_args": _lib.GemmArgs, "b200k_block_scaled_gemm_args": _lib.BlockScaledGemmArgs,
             "b200k_quantize_args": _lib.QuantizeArgs, "b200k_moe_align_args": _lib.MoeAlignArgs,
             "b200k_fmha_args": _lib.FmhaArgs, "b200k_peer_gather_args": _lib.PeerGatherArgs,
             "b200k_gemm_config": _lib.GemmConfig, "b200k_group_problem": _lib.GroupProblem,
             "b200k_group_gemm_args": _lib.GroupGemmArgs, "b200k_moe_sparse_args": _lib.MoeSparseArgs, "b200k_moe_ep_count_args": _lib.MoeEpCountArgs,
             "b200k_moe_ep_plan_args": _lib.MoeEpPlanArgs, "b200k_moe_ep_dispatch_args": _lib.MoeEpDispatchArgs}
    lines = ["#include <stdio.h>", "#include <stddef.h>", '#include "b200k.h"', "int main(void) {"]
    for cname, mirror in pairs.items():
        lines.append(f'  printf("{cname} size %zu\\n", sizeof({cname}));')
        for field, _ in mirror._fields_:
            lines.append(f'  printf("{cname} {field} %zu\\n", offsetof({cname}, {field}));')
    lines += ["  return 0;", "}"]
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run([cc, "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout
    seen = 0
    for line in out.splitlines():
        cname, what, value = line.split()
        mirror = pairs[cname]
        if what == "size":
            assert ctypes.sizeof(mirror) == int(value), cname
        else:
            assert getattr(mirror, what).offset == int(value), f"{cname}.{what}"
        seen += 1
    assert seen == sum(len(m._fields_) + 1 for m in pairs.values())
