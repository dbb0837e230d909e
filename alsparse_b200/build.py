"""Builds the native pieces in-tree.

    python -m alsparse_b200.build            # library + generators + CPU checkers

* ``alsparse_b200/libalphasparse_b200.so`` -- the product: CUDA kernels and the C ABI,
  compiled by nvcc for sm_100a only (cross-compiles without a GPU).
* ``alsparse_b200/synth/libsynth.so`` -- seeded input generators (host C).
* ``libbench_gather_probe.so`` (repository root) -- the gather-rate probe of ``bench.py``.
* ``oracle/liboracle.so`` and, when the reference tree is present, ``oracle/_ref/libalpha_ref.so``
  -- the CPU checkers used by tests and by the CPU legs of the benchmark (``make -C oracle``).
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libalphasparse_b200.so")
SYNTH_SRC = os.path.join(HERE, "synth", "synth.c")
SYNTH_LIB = os.path.join(HERE, "synth", "libsynth.so")
CUDA_SOURCES = ["core.cu", "spmv.cu", "spmv_band.cu", "spmv_bins.cu", "spmm.cu", "exchange.cu", "coo2csr.cu", "host_util.cu", "host_args.cu"]


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _run(cmd, **kw):
    print("+", " ".join(cmd), flush=True)
    subprocess.check_call(cmd, **kw)


def nvcc_path():
    return shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"


def build_library(force=False, verbose_ptxas=False):
    srcs = [os.path.join(CSRC, s) for s in CUDA_SOURCES]
    deps = srcs + [os.path.join(CSRC, "internal.h")] + [
        os.path.join(ROOT, "include", "alphasparse", h)
        for h in os.listdir(os.path.join(ROOT, "include", "alphasparse"))
    ]
    if not force and not _newer(LIB, deps):
        return LIB
    cmd = [
        nvcc_path(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3",
        "-std=c++17", "-shared", "-Xcompiler", "-fPIC,-fopenmp,-O2,-Wall",
        "-I", os.path.join(ROOT, "include"), "-I", CSRC, "-ccbin", "/usr/bin/g++",
        "-cudart", "static", "-o", LIB,
    ]
    if verbose_ptxas:
        cmd += ["-Xptxas", "-v"]
    _run(cmd + srcs + ["-lgomp"])
    return LIB


def build_synth(force=False):
    if force or _newer(SYNTH_LIB, [SYNTH_SRC]):
        _run(["/usr/bin/gcc", "-O2", "-std=gnu11", "-fPIC", "-shared", "-fopenmp", "-o", SYNTH_LIB,
              SYNTH_SRC, "-lm"])
    return SYNTH_LIB


PROBE_SRC = os.path.join(ROOT, "bench_gather_probe.cu")
PROBE_LIB = os.path.join(ROOT, "libbench_gather_probe.so")


def build_bench_probe(force=False):
    """The gather-rate probe bench.py reports beside its kernel times (a helper of the benchmark, not of the library)."""
    if os.path.exists(PROBE_SRC) and (force or _newer(PROBE_LIB, [PROBE_SRC])):
        _run([nvcc_path(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-shared",
              "-Xcompiler", "-fPIC", "-ccbin", "/usr/bin/g++", "-cudart", "static", "-o", PROBE_LIB, PROBE_SRC])
    return PROBE_LIB


def build_oracle():
    """C restatement always; the reference's own objects only where its tree is mounted."""
    _run(["make", "-s", "-C", os.path.join(ROOT, "oracle"), "all"])


def build_all(force=False):
    build_library(force)
    build_synth(force)
    build_bench_probe(force)
    build_oracle()


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
