"""Builds the in-tree CUDA library with nvcc for sm_100a only.

    python -m lightron_b200.csrc.build [--verbose] [--force] [--sanitize]

The result, ``liblightron_b200.so``, sits beside the sources (git-ignored) and is loaded through
ctypes by ``lightron_b200.ops.native``.  No torch headers are involved, so a full build takes
seconds and cross-compiles on a machine without a GPU.

``--sanitize`` builds ``liblightron_b200_asan.so`` instead: the same sources with the HOST code under
AddressSanitizer + UndefinedBehaviorSanitizer (device code is unchanged).  Load it with
``LD_PRELOAD=$(gcc -print-file-name=libasan.so)``, ``ASAN_OPTIONS=detect_leaks=0:protect_shadow_gap=0`` and
``LIGHTRON_B200_LIB=<that file>``; ``tests/test_grouped_cpu.py`` runs the host-only entry points that way.
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


ASAN_LIB = os.path.join(HERE, "liblightron_b200_asan.so")
_SAN = ["-Xcompiler", "-fsanitize=address", "-Xcompiler", "-fsanitize=undefined", "-Xcompiler", "-fno-omit-frame-pointer"]


def build_sanitized(out: str = ASAN_LIB) -> str:
    """Host code under ASan + UBSan (objects go to a temporary directory; the normal build is untouched)."""
    import tempfile
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    with tempfile.TemporaryDirectory() as tmp:
        procs, objs = [], []
        for src in sources():
            obj = os.path.join(tmp, os.path.basename(src)[:-3] + ".o")
            cmd = [nvcc, *ARCH, "-O1", "-g", "-std=c++17", "--use_fast_math", "-Xcompiler", "-fPIC", *_SAN, "-c", src, "-o", obj]
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)))
            objs.append(obj)
        for src, pr in procs:
            so, se = pr.communicate()
            if pr.returncode:
                sys.stderr.write(so + se)
                raise RuntimeError(f"nvcc (sanitized) failed on {os.path.basename(src)}")
        r = subprocess.run([nvcc, *ARCH, "-shared", *_SAN, "-o", out, *objs, "-lcudart"], capture_output=True, text=True)
        if r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link (sanitized) failed")
    return out


if __name__ == "__main__":
    if "--sanitize" in sys.argv:
        print(build_sanitized())
    else:
        print(build(verbose="--verbose" in sys.argv, force="--force" in sys.argv))
