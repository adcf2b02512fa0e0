"""Builds tests/abi_driver.cpp against include/yuuka_cuda.h and the in-tree library with the host C++
compiler and runs it: the ABI as a compiled caller sees it (no ctypes, no Python types in between)."""
import os
import shutil
import subprocess

import pytest

from yuuka_b200 import build

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


@pytest.fixture(scope="module")
def driver(tmp_path_factory):
    cxx = shutil.which("g++")
    if cxx is None:
        pytest.skip("no host C++ compiler")
    build.build_all(force=False, verbose=False)
    exe = str(tmp_path_factory.mktemp("abi") / "abi_driver")
    libdir = os.path.dirname(build.CUDA_LIB)
    cmd = [cxx, "-std=c++17", "-O1", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), os.path.join(HERE, "abi_driver.cpp"),
           "-o", exe, "-L", libdir, "-lyuuka_cuda", f"-Wl,-rpath,{libdir}", "-lpthread"]
    done = subprocess.run(cmd, capture_output=True, text=True)
    assert done.returncode == 0, done.stderr
    return exe


def run(exe, mode):
    done = subprocess.run([exe, mode], capture_output=True, text=True, timeout=300)
    assert done.returncode == 0, done.stdout + done.stderr
    assert f"checks passed ({mode})" in done.stdout and "FAIL" not in done.stdout, done.stdout
    return done.stdout


def test_compiled_caller_host_side(driver):
    out = run(driver, "host")
    for line in ("ok abi version", "ok thread-local errors", "ok allocator and table", "ok prompt lookup", "ok gguf open failure"):
        assert line in out, out


@pytest.mark.gpu
def test_compiled_caller_on_the_device(driver):
    out = run(driver, "gpu")
    for line in ("ok device", "ok buffers and copies", "ok gemm_quant", "ok refusals"):
        assert line in out, out
