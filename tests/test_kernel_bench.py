"""The C++ micro-benchmark (counterpart of the reference's Sources/DFlashKernelBench/main.swift)."""
import os
import re
import subprocess

import pytest

from swiftlm_b200 import build

BIN = os.path.join(os.path.dirname(build.__file__), "bin", "dflash_kernel_bench")


def test_bench_binary_is_built():
    build.build()
    assert os.access(BIN, os.X_OK)


@pytest.mark.gpu
def test_bench_runs_every_section():
    build.build()
    r = subprocess.run([BIN, "--iterations", "5", "--warmup", "2", "--kernels", "tape,gdelta,sdpa"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    lines = [l for l in r.stdout.splitlines() if " med " in l]
    # 4 replay variants + 4 forward variants + 3 context lengths (main.swift:127-137, 172-186, 204)
    assert len(lines) == 11, r.stdout
    for l in lines:
        m = re.search(r"med\s+([\d.]+) us\s+min\s+([\d.]+) us\s+max\s+([\d.]+) us\s+([\d.]+) GB/s", l)
        assert m, l
        med, mn, mx = float(m.group(1)), float(m.group(2)), float(m.group(3))
        assert 0 < mn <= med <= mx
    assert r.stdout.rstrip().endswith("Done.")


@pytest.mark.gpu
def test_bench_cold_cache_mode():
    """--cold rotates the large inputs among copies that exceed the L2 cache; same sections, same line format."""
    build.build()
    r = subprocess.run([BIN, "--iterations", "6", "--warmup", "2", "--kernels", "tape,sdpa", "--cold"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert re.search(r"L2:\s+cold", r.stdout), r.stdout
    assert len([l for l in r.stdout.splitlines() if " med " in l]) == 7, r.stdout
    assert r.stdout.rstrip().endswith("Done.")


SELFTEST = os.path.join(os.path.dirname(build.__file__), "bin", "dflash_host_selftest")


def test_host_selftest_binary_is_built():
    build.build()
    assert os.access(SELFTEST, os.X_OK)


@pytest.mark.gpu
def test_cpp_host_layer_selftest():
    """The C++ mirror of DFlashKernels / RecurrentRollbackCache (swiftlm_b200/host/dflash_host.hpp) on the GPU."""
    build.build()
    r = subprocess.run([SELFTEST], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "all checks passed" in r.stdout and "FAIL" not in r.stdout
