"""Compile the CUDA sources under csrc/ into one shared library for sm_100a, in-tree.

    python -m selective_attention_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU.  The library sits beside this file so that it ships with the
source tree; nothing is installed into site-packages and nothing is JIT-cached elsewhere.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(os.path.dirname(HERE), "csrc")
LIB_NAME = "libselective_attention_b200.so"
LIB_PATH = os.path.join(HERE, LIB_NAME)
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _inputs():
    root = os.path.dirname(os.path.dirname(HERE))
    extra = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    extra.append(os.path.join(root, "include", "selective_attention_b200.h"))
    return sources() + extra


def up_to_date() -> bool:
    if not os.path.exists(LIB_PATH):
        return False
    built = os.path.getmtime(LIB_PATH)
    return all(os.path.getmtime(f) <= built for f in _inputs())


def nvcc_path() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found; the CUDA library cannot be built")
    return found


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and up_to_date():
        return LIB_PATH
    objs = []
    obj_dir = os.path.join(os.path.dirname(HERE), "build")
    os.makedirs(obj_dir, exist_ok=True)
    common = [nvcc_path(), *ARCH, "-O3", "-lineinfo", "-std=c++17", "--use_fast_math" if False else "-DNDEBUG",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v" if verbose else "-O3"]
    procs = []
    for src in sources():
        obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        newest_dep = max(os.path.getmtime(f) for f in _inputs() if not f.endswith(".cu") or f == src)
        if not force and os.path.exists(obj) and os.path.getmtime(obj) >= newest_dep:
            continue
        procs.append((src, subprocess.Popen(common + ["-c", src, "-o", obj], stdout=subprocess.PIPE,
                                            stderr=subprocess.STDOUT, text=True)))
    for src, proc in procs:
        out, _ = proc.communicate()
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{out}")
        if verbose:
            print(out)
    link = [nvcc_path(), *ARCH, "-shared", "--cudart", "shared", "-o", LIB_PATH, *objs,
            "-Xlinker", "-rpath,/usr/local/cuda/lib64"]
    res = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}")
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
