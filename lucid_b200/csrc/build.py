"""Build ``liblucid_b200.so`` in-tree with nvcc for sm_100a.

    python -m lucid_b200.csrc.build [--force] [--verbose]

nvcc cross-compiles without a GPU.  The library links the CUDA runtime only;
the one driver entry point it needs (tensor-map encoding for TMA) is resolved
at run time through the runtime's driver-entry-point query.
"""

from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
SOURCES = ["capi.cu", "stream_kernels.cu", "histogram.cu", "embedding.cu", "exchange.cu", "lstm.cu", "groupwise.cu",
           "gemm_s8.cu"]
# the test-only library: the GEMM with its wait-expiry hook compiled in (-DLQ_TESTING)
TEST_SOURCES = ["capi.cu", "gemm_s8.cu"]
HEADERS = ["common.cuh", os.path.join(ROOT, "include", "lucid_b200.h")]
LIB = os.path.join(HERE, "liblucid_b200.so")
TEST_LIB = os.path.join(HERE, "liblucid_b200_testing.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    # exact arithmetic: no FMA contraction, IEEE divide / sqrt, no flush-to-zero
    "-fmad=false", "-prec-div=true", "-prec-sqrt=true", "-ftz=false",
    "-Xcompiler", "-fPIC",
    "-I", os.path.join(ROOT, "include"),
]


def _stale(lib: str, sources) -> bool:
    if not os.path.exists(lib):
        return True
    t = os.path.getmtime(lib)
    deps = [os.path.join(HERE, s) for s in sources] + \
        [h if os.path.isabs(h) else os.path.join(HERE, h) for h in HEADERS] + [__file__]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the product library and the test-only library (all files in parallel)."""
    todo = []
    if force or _stale(LIB, SOURCES):
        todo.append((LIB, SOURCES, [], ""))
    if force or _stale(TEST_LIB, TEST_SOURCES):
        todo.append((TEST_LIB, TEST_SOURCES, ["-DLQ_TESTING"], ".testing"))
    if not todo:
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    procs = []
    for lib, sources, defs, tag in todo:
        for s in sources:
            obj = os.path.join(HERE, s.replace(".cu", tag + ".o"))
            cmd = [nvcc, *NVCC_FLAGS, *defs, "-c", os.path.join(HERE, s), "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            procs.append((lib, s, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)))
    for lib, s, obj, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            sys.stderr.write(out.decode())
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {s}")
    for lib, sources, defs, tag in todo:
        objs = [obj for l, s, obj, p in procs if l == lib]
        # link beside the target and rename, so a reader never sees a half-written library
        tmp = lib + ".tmp"
        subprocess.check_call([nvcc, "-arch=sm_100a", "-shared", "-o", tmp, *objs, "-lcudart"])
        os.replace(tmp, lib)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
