"""In-tree build of ``libiex_b200.so`` (the C-ABI CUDA library) for sm_100a with nvcc.

``python intrasm_engine_b200/build.py`` (run as a script, so that it works before the
library exists) compiles every ``csrc/*.cu`` to an object file
under ``build/`` (one nvcc process per file, in parallel) and links them into
``intrasm_engine_b200/libiex_b200.so``.  The CUDA runtime is linked statically, so the
library has no load-time dependency besides libc/libstdc++ and the driver.
``CMakeLists.txt`` beside this file describes the same build for CMake users.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
REPO_DIR = os.path.dirname(PKG_DIR)
CSRC = os.path.join(PKG_DIR, "csrc")
OBJ_DIR = os.path.join(REPO_DIR, "build", "iex_b200")
LIB_PATH = os.path.join(PKG_DIR, "libiex_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "-DIEX_TARGET_SM=100",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or add it to PATH")


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _deps_mtime() -> float:
    newest = 0.0
    for root in (CSRC, os.path.join(REPO_DIR, "include")):
        for f in os.listdir(root):
            if f.endswith((".cuh", ".h")):
                newest = max(newest, os.path.getmtime(os.path.join(root, f)))
    return newest


def _compile(src: str, verbose: bool) -> str:
    obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
    newest_dep = max(os.path.getmtime(src), _deps_mtime(), os.path.getmtime(__file__))
    if os.path.exists(obj) and os.path.getmtime(obj) >= newest_dep:
        return obj
    cmd = [_nvcc(), *NVCC_FLAGS, "-c", src, "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        sys.stderr.write(res.stderr)
    return obj


def build(verbose: bool = False, force: bool = False) -> str:
    """Compile and link the library; returns its path.  Up-to-date objects are reused."""
    os.makedirs(OBJ_DIR, exist_ok=True)
    if force:
        for f in os.listdir(OBJ_DIR):
            if f.endswith(".o"):
                os.remove(os.path.join(OBJ_DIR, f))
    srcs = sources()
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        objs = list(pool.map(lambda s: _compile(s, verbose), srcs))
    if (not os.path.exists(LIB_PATH)) or any(
            os.path.getmtime(o) > os.path.getmtime(LIB_PATH) for o in objs):
        cmd = [_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a",
               "-Xcompiler", "-fPIC", "-o", LIB_PATH, *objs]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="--force" in sys.argv))
