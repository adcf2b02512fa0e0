"""Builds tests/dependency_cost.cu with nvcc and runs it: the cost of a dependency point between two phases of a
step as a dependent launch inside a CUDA graph and as a grid-wide barrier inside a cooperative kernel. The figures
are printed (run with -s to see them); the test holds that both forms complete, that no bounded wait runs out and
that the figures are sane."""
import os
import re
import shutil
import subprocess

import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def test_dependent_launch_and_grid_barrier(tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("no nvcc on this machine")
    exe = str(tmp_path / "dependency_cost")
    done = subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-o", exe, os.path.join(HERE, "dependency_cost.cu")],
                          capture_output=True, text=True)
    assert done.returncode == 0, done.stderr
    run = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert run.returncode == 0, run.stdout + run.stderr
    print(run.stdout)
    launches = [float(x) for x in re.findall(r"([0-9.]+) us per launch", run.stdout)]
    barriers = [float(x) for x in re.findall(r"([0-9.]+) us per barrier", run.stdout)]
    assert len(launches) == 3 and len(barriers) == 3
    assert "(expired 1)" not in run.stdout
    assert 0.1 < min(launches) < 50.0 and 0.1 < min(barriers) < 50.0
