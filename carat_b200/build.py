"""Builds carat_b200/libcarat_b200.so in-tree with nvcc for sm_100a.

The library is plain CUDA C++ behind a C ABI (include/carat_b200.h); it does not link torch.
Run `python -m carat_b200.build` (or call build()) after changing anything under csrc/.
"""
from __future__ import annotations

import os
import subprocess
import sys

PACKAGE = os.path.dirname(os.path.abspath(__file__))
SOURCES = ["fp8_linear.cu", "fp8_linear_static.cu", "int4_linear.cu", "row_ops.cu", "qkv_post.cu", "attention_simt.cu", "attention_tc.cu",
    "attention_fused.cu", "attention_stream.cu", "accept.cu",
           "context.cu", "selftest.cu", "weights.cu", "placement.cu", "runner.cu", "capi_linear.cu", "capi_ops.cu"]
LIBRARY = os.path.join(PACKAGE, "libcarat_b200.so")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC,-fvisibility=hidden", "-Xptxas", "-v"]


def _stale() -> bool:
    if not os.path.exists(LIBRARY):
        return True
    built = os.path.getmtime(LIBRARY)
    folder = os.path.join(PACKAGE, "csrc")
    inputs = [os.path.join(folder, name) for name in os.listdir(folder)]
    inputs.append(os.path.join(os.path.dirname(PACKAGE), "include", "carat_b200.h"))
    return any(os.path.getmtime(path) > built for path in inputs)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compiles every CUDA source into one shared library; returns its path."""
    if not force and not _stale():
        return LIBRARY
    folder = os.path.join(PACKAGE, "csrc")
    objects = []
    jobs = []
    for source in SOURCES:
        target = os.path.join(folder, source[:-3] + ".o")
        objects.append(target)
        command = ["nvcc", *FLAGS, "-c", os.path.join(folder, source), "-o", target]
        jobs.append((source, subprocess.Popen(command, stdout=subprocess.PIPE,
                                              stderr=subprocess.STDOUT, text=True)))
    for source, job in jobs:
        output, _ = job.communicate()
        if verbose or job.returncode != 0:
            sys.stderr.write(output)
        if job.returncode != 0:
            raise RuntimeError(f"nvcc failed on {source}")
    link = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", LIBRARY, *objects]
    subprocess.run(link, check=True)
    return LIBRARY


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
