"""CPU tests of the drop-in boundary: the C-ABI library loads, exports every symbol the
public header declares, agrees with the header on struct layout, and rejects bad
arguments before touching a device."""
import ctypes
import os
import re
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "fused_moe_c.h")


@pytest.fixture(scope="module")
def lib():
    sys.path.insert(0, ROOT)
    from therock_b200 import build, api
    build.build()
    return api.lib()


def declared_symbols():
    text = open(HEADER).read()
    return sorted(set(re.findall(r"FMOE_API\s+[\w\s\*]+?\b(fmoe_\w+)\s*\(", text)))


def test_header_declares_expected_entry_points():
    syms = declared_symbols()
    for s in ("fmoe_version", "fmoe_last_error", "fmoe_sort", "fmoe_get_workspace_size", "fmoe_run",
              "fmoe_sort_capacity", "fmoe_get_workspace_layout", "fmoe_check_status"):
        assert s in syms


def test_library_exports_every_declared_symbol(lib):
    for s in declared_symbols():
        assert hasattr(lib, s), f"{s} declared in the header but not exported"
    assert lib.fmoe_version() >= 100


def test_struct_layout_matches_header(tmp_path):
    from therock_b200 import api
    src = tmp_path / "layout.c"
    src.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "fused_moe_c.h"\n'
                   'int main(void){printf("%zu %zu %zu %zu %zu %zu\\n", sizeof(fmoe_traits_c), sizeof(fmoe_args_c),'
                   ' sizeof(fmoe_ws_layout_c), offsetof(fmoe_args_c, workspace_bytes), offsetof(fmoe_args_c, T),'
                   ' offsetof(fmoe_ws_layout_c, slots));return 0;}\n')
    exe = tmp_path / "layout"
    env = {k: v for k, v in os.environ.items() if k not in ("CC", "CXX")}
    subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)], check=True, env=env)
    got = [int(v) for v in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()]
    want = [ctypes.sizeof(api._Traits), ctypes.sizeof(api._Args), ctypes.sizeof(api._Layout),
            api._Args.workspace_bytes.offset, api._Args.T.offset, api._Layout.slots.offset]
    assert got == want


def test_cpp_host_header_compiles(tmp_path):
    src = tmp_path / "use.cpp"
    src.write_text('#include "fused_moe.hpp"\nint main(){fused_moe_traits t; fused_moe_args a; stream_config s;'
                   ' t.prec_w = "fp8"; t.quant = "token_channel"; (void)a; (void)s;'
                   ' fmoe_traits_c c; return fmoe_detail::to_c(t, &c) == FMOE_OK && c.weight_dtype == FMOE_FP8_E4M3 ? 0 : 1;}\n')
    env = {k: v for k, v in os.environ.items() if k not in ("CC", "CXX")}
    exe = tmp_path / "use"
    subprocess.run(["g++", "-std=c++17", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe),
                    "-Wl,--unresolved-symbols=ignore-all"], check=True, env=env)
    assert subprocess.run([str(exe)]).returncode == 0


def test_sort_capacity(lib):
    from therock_b200 import api
    assert api.sort_capacity(128, 2, 8, 128) == 1280
    assert api.sort_capacity(4096, 2, 8, 128) == 9216
    assert api.sort_capacity(8192, 8, 256, 128) == 98048
    assert api.sort_capacity(0, 2, 4, 128) == 512


def test_argument_errors_are_reported_before_any_launch(lib):
    from therock_b200 import api
    t = api._Traits(); a = api._Args(); n = ctypes.c_uint64(0)
    t.quant, t.weight_dtype, t.block_m = 0, 0, 128
    a.T, a.H, a.I, a.E, a.K = 128, 512, 1024, 8, 2
    assert lib.fmoe_get_workspace_size(ctypes.byref(t), ctypes.byref(a), ctypes.byref(n)) == 0
    assert n.value > 128 * 2 * 512 * 4
    # null pointers -> invalid argument, with a message
    assert lib.fmoe_run(ctypes.byref(t), ctypes.byref(a), None, None) == -1
    assert b"required" in lib.fmoe_last_error()
    # dtype / quant mismatch
    t.weight_dtype = 1
    assert lib.fmoe_get_workspace_size(ctypes.byref(t), ctypes.byref(a), ctypes.byref(n)) == -1
    t.weight_dtype = 0
    # unsupported block size and shapes
    t.block_m = 64
    assert lib.fmoe_get_workspace_size(ctypes.byref(t), ctypes.byref(a), ctypes.byref(n)) == -2
    t.block_m = 128
    a.H = 500
    assert lib.fmoe_get_workspace_size(ctypes.byref(t), ctypes.byref(a), ctypes.byref(n)) == -2
    a.H = 512; a.K = 9
    # more experts per token than experts is legal: the receiving side of a de-duplicated
    # expert-parallel dispatch passes K-wide id lists (-1 = elsewhere) to a rank owning fewer experts
    assert lib.fmoe_get_workspace_size(ctypes.byref(t), ctypes.byref(a), ctypes.byref(n)) == 0
    a.K = 0
    assert lib.fmoe_get_workspace_size(ctypes.byref(t), ctypes.byref(a), ctypes.byref(n)) == -1
    assert lib.fmoe_get_workspace_size(None, ctypes.byref(a), ctypes.byref(n)) == -1
    # gate-only: intermediate size must tile by 256, and block128 scales are not built for it
    a.K = 2
    t.gate_only = 1
    assert lib.fmoe_get_workspace_size(ctypes.byref(t), ctypes.byref(a), ctypes.byref(n)) == 0
    a.I = 384
    assert lib.fmoe_get_workspace_size(ctypes.byref(t), ctypes.byref(a), ctypes.byref(n)) == -2
    a.I = 1024
    t.quant, t.weight_dtype = 2, 1
    assert lib.fmoe_get_workspace_size(ctypes.byref(t), ctypes.byref(a), ctypes.byref(n)) == -2
    t.quant, t.weight_dtype, t.gate_only = 0, 0, 0
    t.weight_layout = 7
    assert lib.fmoe_get_workspace_size(ctypes.byref(t), ctypes.byref(a), ctypes.byref(n)) == -1
    t.weight_layout = 0
    t.partial_dtype = 5
    assert lib.fmoe_get_workspace_size(ctypes.byref(t), ctypes.byref(a), ctypes.byref(n)) == -1
    t.partial_dtype = 0
    # entry points outside the operator proper report through the same error text
    assert lib.fmoe_route(None, 1, 1, 1, 0, None, None, None) == -1
    assert b"fmoe_route" in lib.fmoe_last_error()
    assert lib.fmoe_ep_plan(None, 1, 1, 1, 1, None, None, None, None, None) == -1
    assert b"fmoe_ep_plan" in lib.fmoe_last_error()
    assert lib.fmoe_sort(None, None, 1, 1, 1, 128, None, None, None, None, None) == -1


def test_python_mirror_rejects_cpu_tensors(lib):
    import torch
    from therock_b200 import FusedMoeArgs, FusedMoeTraits, FmoeError, fused_moe
    args = FusedMoeArgs(a=torch.zeros(4, 256, dtype=torch.bfloat16), g=torch.zeros(2, 256, 256, dtype=torch.bfloat16),
                        d=torch.zeros(2, 256, 128, dtype=torch.bfloat16), topk_ids=torch.zeros(4, 1, dtype=torch.int32),
                        topk_weight=torch.ones(4, 1))
    with pytest.raises(FmoeError):
        fused_moe(FusedMoeTraits(), args)      # no CPU fallback exists


def test_product_does_not_import_the_oracle():
    for dirpath, _, files in os.walk(os.path.join(ROOT, "therock_b200")):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower(), f"{f} mentions the oracle"
