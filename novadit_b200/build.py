"""In-tree build of the native code.

    python -m novadit_b200.build            # C-ABI library + torch extension
    python -m novadit_b200.build --no-torch-ext

Produces, inside the package directory:

* ``libnovadit_b200.so`` - the C-ABI library (``include/novadit_b200.h``): every CUDA kernel,
  compiled by nvcc for sm_100a only (``-gencode arch=compute_100a,code=sm_100a``). No torch
  dependency.
* ``novadit_cuda.<abi>.so`` - the thin PyTorch C++ extension (pybind11 module ``novadit_cuda``,
  same 15 functions as the reference's ``csrc/bindings.cpp``) that validates tensors, allocates
  outputs and calls the C ABI on torch's current stream.

nvcc cross-compiles without a GPU. Objects are cached in ``build/`` by source hash.
"""
from __future__ import annotations

import argparse
import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG_DIR)
CSRC = os.path.join(PKG_DIR, "csrc")
BUILD_DIR = os.path.join(ROOT, "build")
LIB_PATH = os.path.join(PKG_DIR, "libnovadit_b200.so")
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
NVCC = os.path.join(CUDA_HOME, "bin", "nvcc")

CU_SOURCES = [
    "runtime.cu",
    "norm_api.cu",
    "norm_f16.cu",
    "norm_bf16.cu",
    "norm_f32.cu",
    "gate_act.cu",
    "rowops.cu",
    "quant.cu",
    "fc1.cu",
    "noalloc.cu",
]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
]


def ext_path() -> str:
    return os.path.join(PKG_DIR, "novadit_cuda" + sysconfig.get_config_var("EXT_SUFFIX"))


def _hash_inputs(paths: list[str], extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        with open(p, "rb") as f:
            h.update(p.encode())
            h.update(f.read())
    return h.hexdigest()[:16]


def _headers() -> list[str]:
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hs.append(os.path.join(ROOT, "include", "novadit_b200.h"))
    hs.append(os.path.join(ROOT, "include", "novadit_b200_tuning.h"))
    return hs


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)


def _compile_cu(src: str) -> str:
    path = os.path.join(CSRC, src)
    tag = _hash_inputs([path] + _headers(), " ".join(NVCC_FLAGS))
    obj = os.path.join(BUILD_DIR, f"{os.path.splitext(src)[0]}.{tag}.o")
    if not os.path.exists(obj):
        _run([NVCC, *NVCC_FLAGS, "-c", path, "-o", obj])
    return obj


def build_library(verbose: bool = True) -> str:
    """Compile every .cu for sm_100a and link libnovadit_b200.so."""
    if not os.path.exists(NVCC):
        raise RuntimeError(f"nvcc not found at {NVCC}")
    os.makedirs(BUILD_DIR, exist_ok=True)
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objs = list(pool.map(_compile_cu, CU_SOURCES))
    tag = _hash_inputs(objs, "link")
    stamp = os.path.join(BUILD_DIR, "lib.stamp")
    if not (os.path.exists(LIB_PATH) and os.path.exists(stamp) and open(stamp).read() == tag):
        _run([NVCC, "-shared", "-o", LIB_PATH, *objs, "-gencode", "arch=compute_100a,code=sm_100a"])
        with open(stamp, "w") as f:
            f.write(tag)
    if verbose:
        print("built", LIB_PATH)
    return LIB_PATH


def build_torch_ext(verbose: bool = True) -> str:
    """Compile csrc/torch_ext.cpp into the pybind11 module novadit_cuda (links libnovadit_b200.so)."""
    import torch
    from torch.utils import cpp_extension

    src = os.path.join(CSRC, "torch_ext.cpp")
    out = ext_path()
    os.makedirs(BUILD_DIR, exist_ok=True)
    tag = _hash_inputs([src, os.path.join(ROOT, "include", "novadit_b200.h")], torch.__version__)
    stamp = os.path.join(BUILD_DIR, "ext.stamp")
    if os.path.exists(out) and os.path.exists(stamp) and open(stamp).read() == tag:
        return out
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    includes = cpp_extension.include_paths() + [os.path.join(CUDA_HOME, "include"), sysconfig.get_paths()["include"]]
    cmd = [
        os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden",
        "-DTORCH_EXTENSION_NAME=novadit_cuda", "-DTORCH_API_INCLUDE_EXTENSION_H",
        f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
        *[f"-I{p}" for p in includes], f"-I{os.path.join(ROOT, 'include')}",
        src, "-o", out,
        f"-L{PKG_DIR}", "-lnovadit_b200", f"-L{torch_lib}",
        "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch", "-ltorch_python",
        "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}",
    ]
    _run(cmd)
    with open(stamp, "w") as f:
        f.write(tag)
    if verbose:
        print("built", out)
    return out


def build_all(torch_ext: bool = True, verbose: bool = True) -> None:
    build_library(verbose)
    if torch_ext:
        build_torch_ext(verbose)


def clean() -> None:
    shutil.rmtree(BUILD_DIR, ignore_errors=True)
    for p in (LIB_PATH, ext_path()):
        if os.path.exists(p):
            os.remove(p)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--no-torch-ext", action="store_true")
    ap.add_argument("--clean", action="store_true")
    ns = ap.parse_args()
    if ns.clean:
        clean()
        sys.exit(0)
    build_all(torch_ext=not ns.no_torch_ext)
