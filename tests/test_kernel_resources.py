"""What ptxas reports for the hot kernels (registers, spills), read from the build's own logs.

The block-scaled promotion loop runs at the edge of its register budget (232 per epilogue
thread): a change that lets the compiler overlap the loop's phases shows up as spill stores in
the loop and costs a quarter of the second GEMM's time.  The plain kernels must not spill at all."""
import os
import re
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def _ptxas_log(tmp_path):
    from therock_b200 import build as B
    B.build()
    log = os.path.join(ROOT, "therock_b200", "build", "gemm.o.log")
    if os.path.exists(log) and "Compiling entry function" in open(log).read():
        return open(log).read()
    # objects built before the logs were kept: compile the one file again
    cmd = [B._nvcc(), *B.NVCC_FLAGS, "-Xptxas", "-v", "-c", os.path.join(ROOT, "therock_b200", "csrc", "gemm.cu"),
           "-o", str(tmp_path / "gemm.o")]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert r.returncode == 0, r.stdout[-2000:]
    return r.stdout


def _kernels(text):
    """{mangled name: (spill store bytes, spill load bytes, registers)}"""
    out = {}
    for m in re.finditer(r"Compiling entry function '(\S+)' for 'sm_100a'(.*?)Used (\d+) registers", text, re.S):
        sp = re.search(r"(\d+) bytes spill stores, (\d+) bytes spill loads", m.group(2))
        out[m.group(1)] = (int(sp.group(1)), int(sp.group(2)), int(m.group(3)))
    return out


def test_hot_kernels_do_not_spill_in_their_loops(tmp_path):
    ks = _kernels(_ptxas_log(tmp_path))
    assert ks, "no kernels found in the ptxas output"
    plain = {n: v for n, v in ks.items() if "fmoe_grouped_gemm_kernel" in n or "fmoe_grouped_gemm_pair_kernel" in n}
    assert len(plain) >= 6
    for name, (st, ld, regs) in plain.items():
        assert st == 0 and ld == 0, (name, st, ld)
    # promotion kernel (f32 block scales): template arguments <epilogue, false, 256>
    promo = {n: v for n, v in ks.items() if "fmoe_grouped_gemm_block_kernelILi" in n and "ELb0E" in n}
    assert len(promo) == 2
    for name, (st, ld, regs) in promo.items():
        assert st <= 64, f"{name}: {st} bytes of spill stores (the K loop's phases are overlapping again)"
    # every kernel that redistributes registers is compiled for exactly the launch-time budget
    for name, (st, ld, regs) in ks.items():
        if "block_kernel" in name or "tokn_kernel" in name:
            assert regs == 168, (name, regs)
