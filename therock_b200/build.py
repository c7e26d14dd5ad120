"""Builds libfmoe_b200.so (sm_100a only) in-tree with nvcc."""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ_DIR = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libfmoe_b200.so")
SOURCES = ["sorting.cu", "rows.cu", "gemm.cu", "api.cu", "ep.cu", "router.cu"]
HEADERS = ["ptx.cuh", "gemm.cuh", "gemm_block.cuh", "scales.cuh", "plan.hpp", "internal.h", os.path.join("..", "..", "include", "fused_moe_c.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    return "nvcc"


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False, checked: bool = False, timing_switches: bool = False) -> str:
    """Builds the product library, or with checked=True libfmoe_b200_checked.so (the same
    sources with -DFMOE_BOUNDS_CHECKS), or with timing_switches=True libfmoe_b200_timing.so
    (-DFMOE_TIMING_SWITCHES: FMOE_DEBUG_FLAGS / FMOE_GEMM_MODE are honoured; results are invalid
    while they are set).  The variants never replace the product library."""
    if checked or timing_switches:
        return _build_variant("checked" if checked else "timing",
                              ["-DFMOE_BOUNDS_CHECKS"] if checked else ["-DFMOE_TIMING_SWITCHES"], force, verbose)
    return _build_variant("", [], force, verbose)


def _build_variant(suffix: str, defines: list, force: bool, verbose: bool) -> str:
    OBJ_DIR = os.path.join(HERE, "build" + ("_" + suffix if suffix else ""))
    LIB = os.path.join(HERE, "libfmoe_b200" + ("_" + suffix if suffix else "") + ".so")
    NVCC_FLAGS = globals()["NVCC_FLAGS"] + defines
    os.makedirs(OBJ_DIR, exist_ok=True)
    hdrs = [os.path.join(CSRC, h) for h in HEADERS]
    jobs = []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ_DIR, src.replace(".cu", ".o"))
        if force or _stale(o, [s] + hdrs):
            jobs.append([_nvcc(), *NVCC_FLAGS, "-Xptxas", "-v", "-c", s, "-o", o])
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)

    def run(cmd):
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
        return cmd, r.returncode, r.stdout

    with ThreadPoolExecutor(max_workers=4) as ex:
        for cmd, rc, out in ex.map(run, jobs):
            # ptxas -v output (registers, spills, shared memory per kernel) is kept beside the object
            with open(cmd[-1] + ".log", "w") as f:
                f.write(out)
            if verbose or rc != 0:
                print(" ".join(cmd))
                print(out)
            if rc != 0:
                raise RuntimeError(f"nvcc failed for {cmd[-3]}")
    objs = [os.path.join(OBJ_DIR, s.replace(".cu", ".o")) for s in SOURCES]
    if force or jobs or _stale(LIB, objs):
        cmd = [_nvcc(), "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
        if r.returncode != 0:
            print(r.stdout)
            raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True, checked="--checked" in sys.argv,
                timing_switches="--timing-switches" in sys.argv))
