"""In-tree build of the native code: ``libb200moe.so`` (CUDA kernels + C ABI, nvcc, sm_100a) and
the ``cinfer_ascendc`` torch extension (g++, thin binding over the C ABI).

    python ascend_kernel_b200/build.py            # build what is stale
    python ascend_kernel_b200/build.py --force

nvcc cross-compiles without a GPU.  Objects go to ``ascend_kernel_b200/build/``; the two shared
objects land next to this file so they travel with the source tree.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libb200moe.so")
EXT = os.path.join(HERE, "cinfer_ascendc" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))

CU_SOURCES = ["host_util.cu", "fp4_dequant.cu", "grouped_gemv.cu", "grouped_gemm.cu", "grouped_gemm_packed.cu", "moe_aux.cu",
              "ep_exchange.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build step failed:\n  " + " ".join(cmd) + "\n" + r.stdout + r.stderr)


def build_lib(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(os.path.dirname(HERE), "include", "b200moe.h"))
    sources = [s for s in CU_SOURCES if os.path.exists(os.path.join(CSRC, s))]
    jobs = []
    for src in sources:
        obj = os.path.join(OBJ, src.replace(".cu", ".o"))
        if force or _stale(obj, [os.path.join(CSRC, src)] + headers):
            cmd = [_nvcc()] + NVCC_FLAGS + ["-c", os.path.join(CSRC, src), "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(_run, jobs))
    objs = [os.path.join(OBJ, s.replace(".cu", ".o")) for s in sources]
    if force or jobs or _stale(LIB, objs):
        _run([_nvcc(), "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static"])
    return LIB


def build_ext(force: bool = False) -> str:
    """The drop-in python module: same name and keyword arguments as the reference's extension."""
    src = os.path.join(CSRC, "ext", "cinfer_ascendc.cpp")
    if not (force or _stale(EXT, [src, LIB, os.path.join(os.path.dirname(HERE), "include", "b200moe.h")])):
        return EXT
    import torch
    from torch.utils import cpp_extension as ce

    inc = []
    for p in ce.include_paths() + [sysconfig.get_paths()["include"], "/usr/local/cuda/include"]:
        inc += ["-I", p]
    libdirs = ce.library_paths()
    cmd = ["g++", "-O2", "-fPIC", "-shared", "-std=c++17", "-DTORCH_EXTENSION_NAME=cinfer_ascendc",
           "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           src, "-o", EXT] + inc
    for d in libdirs:
        cmd += ["-L", d, f"-Wl,-rpath,{d}"]
    cmd += ["-L", HERE, "-Wl,-rpath,$ORIGIN", "-lb200moe", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda",
            "-ltorch", "-ltorch_python"]
    _run(cmd)
    return EXT


def build_all(force: bool = False) -> None:
    build_lib(force)
    build_ext(force)


if __name__ == "__main__":
    build_all("--force" in sys.argv)
    print(LIB)
    print(EXT)
