"""Builds the REFERENCE's own CUDA extension (its seven native sources, where they lie in a checkout of the
reference) for sm_100 into oracle/_ref/novadit_cuda_ref*.so - test infrastructure, never the product.

    python oracle/build_ref_cuda.py /path/to/reference

The recipe restates the reference's `setup.py:20-88` (same sources, `-O3 --use_fast_math`, the half/bfloat16
operator switches, `NOVADIT_HAS_CUTLASS`) as plain nvcc / g++ commands; it does not run the reference's build
system and copies no source. The reference's kernels use `cutlass::AlignedArray`; its CUTLASS submodule
(`third_party/cutlass`) is not part of the checkout, so the header tree comes from `NOVADIT_CUTLASS_PATH`
(the variable the reference's setup.py reads) or, failing that, from the CUTLASS headers that the installed
`flashinfer` package carries. Without either the build raises. The module is named `novadit_cuda_ref` so that it can be imported next to this
repository's `novadit_cuda`. Used by tests/test_gpu_reference_cuda.py (parity of this library against the
reference's kernels on the same GPU).
"""
from __future__ import annotations

import concurrent.futures
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
SOURCES = [
    "csrc/bindings.cpp",
    "csrc/ops/adaln_kernel.cu",
    "csrc/ops/adarmsnorm_kernel.cu",
    "csrc/ops/qkv_pack_kernel.cu",
    "csrc/ops/residual_kernel.cu",
    "csrc/ops/gate_act_kernel.cu",
    "csrc/ops/fc1_bias_act_kernel.cu",
]
NAME = "novadit_cuda_ref"


def out_path() -> str:
    return os.path.join(OUT_DIR, NAME + sysconfig.get_config_var("EXT_SUFFIX"))


def cutlass_root() -> str:
    env = os.environ.get("NOVADIT_CUTLASS_PATH")
    if env and os.path.isdir(os.path.join(env, "include", "cutlass")):
        return env
    try:
        import flashinfer

        root = os.path.join(os.path.dirname(flashinfer.__file__), "data", "cutlass")
        if os.path.isdir(os.path.join(root, "include", "cutlass")):
            return root
    except Exception:
        pass
    raise RuntimeError("no CUTLASS header tree: set NOVADIT_CUTLASS_PATH")


def build(ref_root: str, verbose: bool = True) -> str:
    import torch
    from torch.utils import cpp_extension

    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    nvcc = os.path.join(cuda_home, "bin", "nvcc")
    os.makedirs(OUT_DIR, exist_ok=True)
    incs = [os.path.join(ref_root, "csrc"), sysconfig.get_paths()["include"], os.path.join(cuda_home, "include")]
    incs.append(os.path.join(cutlass_root(), "include"))
    incs += cpp_extension.include_paths()
    inc_flags = [f"-I{p}" for p in incs]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    defs = ["-DNOVADIT_HAS_CUTLASS=1", "-DCUTE_USE_PACKED_TUPLE=1", f"-DTORCH_EXTENSION_NAME={NAME}", "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={abi}"]
    nvcc_flags = ["-O3", "--use_fast_math", "-lineinfo", "--expt-relaxed-constexpr", "--expt-extended-lambda",
                  "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
                  "-U__CUDA_NO_BFLOAT16_OPERATORS__", "-U__CUDA_NO_BFLOAT16_CONVERSIONS__",
                  "-gencode", "arch=compute_100,code=sm_100", "-std=c++17", "-Xcompiler", "-fPIC"]

    def compile_one(src: str) -> str:
        path = os.path.join(ref_root, src)
        obj = os.path.join(OUT_DIR, os.path.basename(src) + ".o")
        if src.endswith(".cu"):
            cmd = [nvcc, *nvcc_flags, *defs, *inc_flags, "-c", path, "-o", obj]
        else:
            cmd = ["g++", "-O3", "-std=c++17", "-fPIC", *defs, *inc_flags, "-c", path, "-o", obj]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError("reference source failed to compile: " + src + "\n" + proc.stderr[-4000:])
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(7, os.cpu_count() or 1)) as pool:
        objs = list(pool.map(compile_one, SOURCES))
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    out = out_path()
    link = ["g++", "-shared", "-o", out, *objs, f"-L{torch_lib}", f"-L{os.path.join(cuda_home, 'lib64')}",
            "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart",
            f"-Wl,-rpath,{torch_lib}"]
    proc = subprocess.run(link, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("link failed\n" + proc.stderr[-4000:])
    for o in objs:
        os.remove(o)
    if verbose:
        print("built", out)
    return out


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    build(sys.argv[1])
