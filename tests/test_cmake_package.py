"""The library as a CMake package: install it, then let a tiny consumer project find it with
find_package(fmoe_b200) and link fmoe::fmoe_b200 -- what the reference super-project gets from
the `composable_kernel` package (math-libs/CMakeLists.txt:606)."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _env():
    return {k: v for k, v in os.environ.items() if k not in ("CC", "CXX", "CUDACXX")}


@pytest.mark.skipif(shutil.which("cmake") is None, reason="cmake not installed")
def test_consumer_finds_the_installed_package(tmp_path):
    from therock_b200 import build
    lib = build.build()
    bdir, prefix, cdir = tmp_path / "build", tmp_path / "prefix", tmp_path / "consumer"
    run = lambda *cmd: subprocess.run(cmd, check=True, env=_env(), capture_output=True, text=True)
    # package the library built by `python -m therock_b200.build` (compiling the kernels through
    # CMake takes minutes; the source path of CMakeLists.txt is configured in the next test)
    run("cmake", "-S", ROOT, "-B", str(bdir), f"-DFMOE_PREBUILT_LIBRARY={lib}", f"-DCMAKE_INSTALL_PREFIX={prefix}")
    run("cmake", "--install", str(bdir))
    assert (prefix / "lib" / "libfmoe_b200.so").exists() or (prefix / "lib64" / "libfmoe_b200.so").exists()
    assert (prefix / "include" / "fused_moe_c.h").exists() and (prefix / "include" / "fused_moe.hpp").exists()
    run("cmake", "-S", os.path.join(ROOT, "tests", "cmake_consumer"), "-B", str(cdir), f"-DCMAKE_PREFIX_PATH={prefix}")
    run("cmake", "--build", str(cdir))
    r = subprocess.run([str(cdir / "fmoe_consumer")], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "capacity 1280" in r.stdout


@pytest.mark.skipif(shutil.which("cmake") is None or shutil.which("nvcc") is None, reason="cmake / nvcc not installed")
def test_source_build_configures_for_sm_100a(tmp_path):
    """Configure (not build) the from-source path: CUDA language, sm_100a, the six sources."""
    r = subprocess.run(["cmake", "-S", ROOT, "-B", str(tmp_path / "b"), "-DFMOE_BOUNDS_CHECKS=ON"], env=_env(),
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    cache = open(tmp_path / "b" / "CMakeCache.txt").read()
    assert "FMOE_BOUNDS_CHECKS:BOOL=ON" in cache
