"""Builds the in-tree CUDA library with nvcc for sm_100a only.

    python -m lightron_b200.csrc.build [--verbose] [--force]

The result, ``liblightron_b200.so``, sits beside the sources (git-ignored) and is loaded through
ctypes by ``lightron_b200.ops.native``.  No torch headers are involved, so a full build takes
seconds and cross-compiles on a machine without a GPU.
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "liblightron_b200.so")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def sources():
    return sorted(glob.glob(os.path.join(HERE, "*.cu")))


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = sources() + glob.glob(os.path.join(HERE, "*.cuh")) + glob.glob(os.path.join(HERE, "*.h"))
    return any(os.path.getmtime(s) > t for s in deps)


def build(verbose: bool = False, force: bool = False) -> str:
    if not force and not needs_build():
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    objs, procs = [], []
    for src in sources():                      # one nvcc per source, all at once
        obj = src[:-3] + ".o"
        cmd = [nvcc, *ARCH, "-O3", "-lineinfo", "-std=c++17", "--use_fast_math", "-Xcompiler", "-fPIC", "-c", src, "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)))
        objs.append(obj)
    failed = []
    for src, pr in procs:
        out, err = pr.communicate()
        if verbose or pr.returncode:
            sys.stderr.write(out + err)
        if pr.returncode:
            failed.append(os.path.basename(src))
    if failed:
        raise RuntimeError(f"nvcc failed on {', '.join(failed)}")
    cmd = [nvcc, *ARCH, "-shared", "-o", LIB + ".tmp", *objs, "-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("link failed")
    os.replace(LIB + ".tmp", LIB)
    return LIB


if __name__ == "__main__":
    print(build(verbose="--verbose" in sys.argv, force="--force" in sys.argv))
