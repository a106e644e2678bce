"""In-tree build of the native libraries (no JIT cache: the built files travel with the tree).

``python gaudirt_b200/build.py`` compiles

* ``lib/libgaudirt_b200.so``  -- the C ABI (``include/gaudirt_b200.h``): CUDA kernels for sm_100a
  plus the host-side metadata/plan code; depends on nothing but the CUDA runtime;
* ``lib/libgaudirt_ops.so``   -- the PyTorch operator layer (``torch.ops.gaudirt.*`` and the
  ``PagedMetadata`` class) that calls the C ABI.
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "lib")
ABI_SO = os.path.join(LIB, "libgaudirt_b200.so")
OPS_SO = os.path.join(LIB, "libgaudirt_ops.so")

NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA 12.9 toolkit is required to build gaudirt_b200")
    return exe


def _stale(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    built = os.path.getmtime(target)
    return any(os.path.getmtime(s) > built for s in sources)


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise RuntimeError("build failed:\n" + " ".join(cmd) + "\n" + proc.stdout)


def abi_sources() -> list[str]:
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")) + [os.path.join(CSRC, "host_plan.cpp")])


def build_abi(force: bool = False, verbose: bool = False) -> str:
    sources = abi_sources()
    deps = sources + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(ROOT, "include", "*.h"))
    if force or _stale(ABI_SO, deps):
        os.makedirs(LIB, exist_ok=True)
        # built beside the target and moved into place, so that a reader never sees a half-written library
        fresh = ABI_SO + ".new"
        cmd = [_nvcc(), *NVCC_ARCH, "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC,-fvisibility=hidden",
               "-shared", "-o", fresh, *sources]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        _run(cmd)
        os.replace(fresh, ABI_SO)
    return ABI_SO


def build_ops(force: bool = False) -> str:
    import torch
    from torch.utils import cpp_extension

    sources = sorted(glob.glob(os.path.join(CSRC, "torch", "*.cpp")))
    deps = sources + glob.glob(os.path.join(CSRC, "torch", "*.h")) + glob.glob(os.path.join(ROOT, "include", "*.h"))
    build_abi(force)
    if not sources:
        raise RuntimeError("operator-layer sources are missing")
    if force or _stale(OPS_SO, deps):
        inc = [f"-I{p}" for p in cpp_extension.include_paths(device_type="cuda")]
        torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
        abi_flag = f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"
        objs = []
        for src in sources:
            obj = os.path.join(LIB, os.path.basename(src) + ".o")
            if force or _stale(obj, deps):
                _run(["g++", "-O2", "-std=c++17", "-fPIC", abi_flag, "-DTORCH_API_INCLUDE_EXTENSION_H", *inc,
                      f"-I{os.path.join(ROOT, 'include')}", "-c", src, "-o", obj])
            objs.append(obj)
        fresh = OPS_SO + ".new"
        _run(["g++", "-shared", "-o", fresh, *objs, f"-L{LIB}", "-lgaudirt_b200", f"-L{torch_lib}",
              "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda",
              "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}"])
        os.replace(fresh, OPS_SO)
    return OPS_SO


def build_all(force: bool = False) -> None:
    build_abi(force)
    if glob.glob(os.path.join(CSRC, "torch", "*.cpp")):
        build_ops(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
    print("built", ABI_SO, OPS_SO if os.path.exists(OPS_SO) else "")
