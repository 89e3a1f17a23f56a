"""Builds the native libraries of this package in-tree with nvcc for sm_100a.

``librecsdk_b200.so``        the C ABI (include/recsdk_b200.h): CUDA kernels + host drivers.
``librecsdk_b200_torch.so``  torch custom-op registrations over that C ABI (optional, see build_torch_ops).

Objects are compiled in parallel and only when a source or header is newer.
"""
from __future__ import annotations

import concurrent.futures as cf
import glob
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "build")
LIB = os.path.join(PKG, "librecsdk_b200.so")
TORCH_LIB = os.path.join(PKG, "librecsdk_b200_torch.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17", "-fmad=false",
    f"-I{os.path.join(ROOT, 'include')}", "-Xcompiler", "-fPIC,-fvisibility=hidden",
]


def _nvcc() -> str:
    for c in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if c and (os.path.isabs(c) and os.path.exists(c) or not os.path.isabs(c)):
            return c
    return "nvcc"


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(verbose: bool = False, ptxas_info: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    headers = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(ROOT, "include", "*.h"))
    sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    jobs = []
    objs = []
    for src in sources:
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        if _stale(obj, [src] + headers) or ptxas_info:
            # RECSDK_NVCC_EXTRA: extra flags, e.g. "-DRECSDK_SELFCHECK" for the bounds-checking debug build
            cmd = [_nvcc(), *NVCC_FLAGS, *os.environ.get("RECSDK_NVCC_EXTRA", "").split(), "-c", src, "-o", obj]
            if ptxas_info:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for cmd, r in ex.map(run, jobs):
                if verbose or r.returncode != 0 or ptxas_info:
                    print(" ".join(cmd))
                    print(r.stdout + r.stderr)
                if r.returncode != 0:
                    raise RuntimeError("nvcc failed for " + cmd[-3])
    if jobs or _stale(LIB, objs):
        subprocess.check_call([_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", LIB, *objs])
    return LIB


def build_torch_ops(verbose: bool = False) -> str:
    """Compiles csrc_torch/torch_ops.cpp (torch custom-op registration over the C ABI) against the installed
    libtorch and links it to librecsdk_b200.so (found at run time next to it through $ORIGIN)."""
    import torch

    src = os.path.join(PKG, "csrc_torch", "torch_ops.cpp")
    hdr = os.path.join(ROOT, "include", "recsdk_b200.h")
    if not _stale(TORCH_LIB, [src, hdr]) and os.path.exists(LIB):
        return TORCH_LIB
    build()
    tdir = os.path.dirname(torch.__file__)
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cuda_inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
           f"-I{os.path.join(ROOT, 'include')}", f"-I{tdir}/include", f"-I{tdir}/include/torch/csrc/api/include",
           f"-I{cuda_inc}", src, "-o", TORCH_LIB, f"-L{PKG}", "-lrecsdk_b200", f"-L{tdir}/lib", "-ltorch", "-ltorch_cpu",
           "-ltorch_cuda", "-lc10", "-lc10_cuda", "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{tdir}/lib"]
    if verbose:
        print(" ".join(cmd))
    subprocess.check_call(cmd)
    return TORCH_LIB


if __name__ == "__main__":
    if "--torch" in sys.argv:
        print(build_torch_ops(verbose=True))
        sys.exit(0)
    print(build(verbose="-v" in sys.argv, ptxas_info="--ptxas" in sys.argv))
    if "--native-only" not in sys.argv and "--ptxas" not in sys.argv:
        print(build_torch_ops(verbose="-v" in sys.argv))  # shares the header's structs: keep the two in step
