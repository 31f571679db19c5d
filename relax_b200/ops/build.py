"""In-tree build of the sm_100a extension.

Kernels live in ``csrc/*.cu`` and do not include PyTorch headers (nvcc compiles
each in seconds); ``csrc/bindings*.cpp`` adapt tensors to the C launchers.  The
result is ``relax_b200/_C.so`` beside the Python sources, so it travels with the
tree to a GPU machine and is the file the ops import.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
CSRC = os.path.join(ROOT, "csrc")
OBJ = os.path.join(ROOT, "build", "obj")
SO_PATH = os.path.join(ROOT, "relax_b200", "_C.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v",
]


def _nvcc() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def _stale(out: str, deps: list) -> bool:
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    return any(os.path.getmtime(d) > t for d in deps)


def _run(cmd: list, log_path: str | None = None):
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if log_path:
        with open(log_path, "w") as f:
            f.write(" ".join(cmd) + "\n" + p.stdout)
    if p.returncode != 0:
        raise RuntimeError(f"command failed: {' '.join(cmd)}\n{p.stdout[-6000:]}")
    return p.stdout


def build_extension(verbose: bool = False, force: bool = False) -> str:
    import torch
    from torch.utils import cpp_extension as ce

    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    cus = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    cpps = sorted(f for f in os.listdir(CSRC) if f.endswith(".cpp"))
    jobs = []
    objs = []
    for f in cus:
        src, out = os.path.join(CSRC, f), os.path.join(OBJ, f + ".o")
        objs.append(out)
        if force or _stale(out, [src] + headers):
            jobs.append(([_nvcc()] + NVCC_FLAGS + ["-I", CSRC, "-c", src, "-o", out], out + ".log"))
    abi = int(getattr(torch._C, "_GLIBCXX_USE_CXX11_ABI", True))
    inc = []
    for p in ce.include_paths("cuda") if "device_type" in ce.include_paths.__code__.co_varnames else ce.include_paths(True):
        inc += ["-isystem", p]
    inc += ["-isystem", sysconfig.get_paths()["include"], "-I", CSRC]
    cxx = os.environ.get("CXX", "g++")
    for f in cpps:
        src, out = os.path.join(CSRC, f), os.path.join(OBJ, f + ".o")
        objs.append(out)
        if force or _stale(out, [src] + headers):
            jobs.append(([cxx, "-O2", "-std=c++17", "-fPIC", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
                          "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H", "-w"] + inc +
                         ["-c", src, "-o", out], out + ".log"))
    if jobs:
        if verbose:
            print(f"[relax_b200.build] compiling {len(jobs)} translation unit(s) for sm_100a", flush=True)
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(lambda j: _run(*j), jobs))
    if jobs or force or _stale(SO_PATH, objs):
        tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
        cuda_lib = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "lib64")
        cmd = [cxx, "-shared", "-o", SO_PATH] + objs + [
            f"-L{tlib}", "-lc10", "-ltorch", "-ltorch_cpu", "-ltorch_python", "-lc10_cuda", "-ltorch_cuda",
            f"-L{cuda_lib}", "-lcudart", f"-Wl,-rpath,{tlib}", f"-Wl,-rpath,{cuda_lib}",
        ]
        _run(cmd)
        if verbose:
            print(f"[relax_b200.build] linked {SO_PATH}", flush=True)
    return SO_PATH


def ptxas_report() -> str:
    """Concatenated ``-Xptxas -v`` output of the last build (registers, spills, shared memory)."""
    out = []
    for f in sorted(os.listdir(OBJ)) if os.path.isdir(OBJ) else []:
        if f.endswith(".cu.o.log"):
            out.append(open(os.path.join(OBJ, f)).read())
    return "\n".join(out)


if __name__ == "__main__":
    build_extension(verbose=True, force="--force" in sys.argv)
