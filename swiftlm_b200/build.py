"""Builds swiftlm_b200/lib/libdflash_cuda.so from swiftlm_b200/csrc/*.cu with nvcc for sm_100a.

    python -m swiftlm_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU.  Objects are rebuilt only when a source or header is newer.
"""
from __future__ import annotations

import concurrent.futures as cf
import glob
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIBDIR = os.path.join(PKG, "lib")
OBJDIR = os.path.join(PKG, "build")
LIB = os.path.join(LIBDIR, "libdflash_cuda.so")

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _newer(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(LIBDIR, exist_ok=True)
    os.makedirs(OBJDIR, exist_ok=True)
    nvcc = _nvcc()
    # the SwiftPM C target carries a copy of the header: keep it in step with include/
    hdr = os.path.join(os.path.dirname(PKG), "include", "dflash_cuda.h")
    hdr_copy = os.path.join(PKG, "swift", "Sources", "CDFlashCUDA", "include", "dflash_cuda.h")
    if os.path.isdir(os.path.dirname(hdr_copy)) and (not os.path.exists(hdr_copy) or open(hdr).read() != open(hdr_copy).read()):
        shutil.copyfile(hdr, hdr_copy)
    sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    headers = sorted(glob.glob(os.path.join(CSRC, "*.cuh"))) + \
        [os.path.join(os.path.dirname(PKG), "include", "dflash_cuda.h"), os.path.abspath(__file__)]
    jobs = []
    for src in sources:
        obj = os.path.join(OBJDIR, os.path.basename(src)[:-3] + ".o")
        if force or _newer(obj, [src] + headers):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        cmd = [nvcc] + NVCC_FLAGS + ["-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        return src, r

    with cf.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for src, r in ex.map(compile_one, jobs):
            log = os.path.join(OBJDIR, os.path.basename(src)[:-3] + ".ptxas.log")
            with open(log, "w") as f:
                f.write(r.stderr)
            if verbose or r.returncode != 0:
                sys.stderr.write(r.stdout + r.stderr)
            if r.returncode != 0:
                raise RuntimeError("nvcc failed on " + src)
    objs = [os.path.join(OBJDIR, os.path.basename(s)[:-3] + ".o") for s in sources]
    if force or jobs or _newer(LIB, objs):
        cmd = [nvcc, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    # host program: the kernel micro-benchmark (counterpart of the reference's DFlashKernelBench)
    bench_src = os.path.join(PKG, "host", "dflash_kernel_bench.cu")
    bench_bin = os.path.join(PKG, "bin", "dflash_kernel_bench")
    os.makedirs(os.path.dirname(bench_bin), exist_ok=True)
    if force or _newer(bench_bin, [bench_src, LIB] + headers):
        cmd = [nvcc, "-std=c++17", "-O2", "-gencode", "arch=compute_100a,code=sm_100a", bench_src, "-o", bench_bin,
               "-L" + LIBDIR, "-ldflash_cuda", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../lib"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("building dflash_kernel_bench failed")
    # host program: self-test of the C++ host layer (dflash_host.hpp)
    st_src = os.path.join(PKG, "host", "dflash_host_selftest.cu")
    st_hdr = os.path.join(PKG, "host", "dflash_host.hpp")
    st_bin = os.path.join(PKG, "bin", "dflash_host_selftest")
    if force or _newer(st_bin, [st_src, st_hdr, LIB] + headers):
        cmd = [nvcc, "-std=c++17", "-O2", "-gencode", "arch=compute_100a,code=sm_100a", st_src, "-o", st_bin,
               "-L" + LIBDIR, "-ldflash_cuda", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../lib"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("building dflash_host_selftest failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
