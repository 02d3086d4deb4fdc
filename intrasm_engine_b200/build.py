"""In-tree build of ``libiex_b200.so`` (the C-ABI CUDA library) for sm_100a with nvcc.

``python intrasm_engine_b200/build.py`` (run as a script, so that it works before the
library exists) compiles every ``csrc/*.cu`` to an object file
under ``build/`` (one nvcc process per file, in parallel) and links them into
``intrasm_engine_b200/libiex_b200.so``.  The CUDA runtime is linked statically, so the
library has no load-time dependency besides libc/libstdc++ and the driver.
It then compiles ``torch_ext/iex_torch_ext.cpp`` with g++ against the installed torch
headers into ``intrasm_engine_b200/libiex_torch_ext.so``, the extension that registers
``torch.ops.iex_ops`` and calls the C ABI (it finds ``libiex_b200.so`` beside itself through
an ``$ORIGIN`` run path).  ``CMakeLists.txt`` beside this file describes the C-ABI build for
CMake users.
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
EXT_SRC = os.path.join(PKG_DIR, "torch_ext", "iex_torch_ext.cpp")
EXT_PATH = os.path.join(PKG_DIR, "libiex_torch_ext.so")

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


def _cuda_include() -> str:
    return os.path.join(os.path.dirname(os.path.dirname(_nvcc())), "include")


def build_torch_ext(force: bool = False) -> str:
    """Compile the torch extension that registers ``torch.ops.iex_ops``; returns its path."""
    newest = max(os.path.getmtime(EXT_SRC), os.path.getmtime(LIB_PATH), os.path.getmtime(__file__),
                 os.path.getmtime(os.path.join(REPO_DIR, "include", "iex_b200.h")))
    if not force and os.path.exists(EXT_PATH) and os.path.getmtime(EXT_PATH) >= newest:
        return EXT_PATH
    import torch
    torch_dir = os.path.dirname(torch.__file__)
    torch_lib = os.path.join(torch_dir, "lib")
    torch_inc = os.path.join(torch_dir, "include")
    # The system g++ on PATH, not $CXX: the extension must share the process's libstdc++.so with
    # torch.  A toolchain that links its own static C++ runtime into the extension gives the
    # process two exception runtimes, and an error raised by TORCH_CHECK then crashes while
    # unwinding through the extension's frames.  IEX_CXX overrides.
    cxx = os.environ.get("IEX_CXX") or shutil.which("g++") or "g++"
    cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch.compiled_with_cxx11_abi())}",
           "-I", os.path.join(REPO_DIR, "include"),
           "-I", torch_inc, "-I", os.path.join(torch_inc, "torch", "csrc", "api", "include"),
           "-I", _cuda_include(),
           EXT_SRC, "-o", EXT_PATH,
           "-L", PKG_DIR, "-liex_b200",
           "-L", torch_lib, "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch",
           "-Wl,-rpath,$ORIGIN"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"torch extension build failed:\n{res.stdout}\n{res.stderr}")
    return EXT_PATH


def build(verbose: bool = False, force: bool = False) -> str:
    """Compile and link the library and the torch extension; returns the library's path.
    Up-to-date objects are reused."""
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
    build_torch_ext(force)
    return LIB_PATH


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="--force" in sys.argv))
