"""In-tree build of the sm_100a extension ``picotron_b200/_C*.so``.

``python -m picotron_b200.build`` (or ``python setup.py build_ext --inplace``) compiles every ``.cu`` under
``csrc/`` with ``nvcc -gencode arch=compute_100a,code=sm_100a`` (device code only, no PyTorch headers, so
a file takes seconds), compiles ``bindings.cpp`` against the PyTorch headers with the host compiler and
links everything into one shared object next to the package sources. Objects are rebuilt only when
their sources (or ``common.cuh``) are newer. nvcc cross-compiles, so no GPU is needed to build.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "csrc", "_obj")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--use_fast_math", "-Xcompiler", "-fPIC", "-Xptxas", "-v"]


def ext_path() -> str:
    return os.path.join(PKG, "_C" + sysconfig.get_config_var("EXT_SUFFIX"))


def _newer(src_list, target) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in src_list)


def _run(cmd, log_name=None):
    res = subprocess.run(cmd, capture_output=True, text=True)
    if log_name:
        with open(os.path.join(OBJ, log_name), "w") as f:
            f.write(" ".join(cmd) + "\n" + res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"build step failed: {' '.join(cmd)}\n{res.stdout}\n{res.stderr}")


def build(verbose: bool = True) -> str:
    import torch
    from torch.utils import cpp_extension as ce
    os.makedirs(OBJ, exist_ok=True)
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    cu_files = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    objs, jobs = [], []
    for f in cu_files:
        src, obj = os.path.join(CSRC, f), os.path.join(OBJ, f[:-3] + ".o")
        objs.append(obj)
        if _newer([src] + headers, obj):
            jobs.append(([nvcc] + NVCC_FLAGS + ["-I", CSRC, "-c", src, "-o", obj], f[:-3] + ".nvcc.log"))
    bsrc, bobj = os.path.join(CSRC, "bindings.cpp"), os.path.join(OBJ, "bindings.o")
    objs.append(bobj)
    if _newer([bsrc], bobj):
        inc = []
        for p in ce.include_paths("cuda") if "device_type" in ce.include_paths.__code__.co_varnames else ce.include_paths(cuda=True):
            inc += ["-I", p]
        inc += ["-I", sysconfig.get_paths()["include"]]
        abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
        jobs.append((["g++", "-O2", "-std=c++17", "-fPIC", "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H",
                      f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-Wno-deprecated-declarations"] + inc +
                     ["-c", bsrc, "-o", bobj], "bindings.gxx.log"))
    if jobs:
        if verbose:
            print(f"[picotron_b200.build] compiling {len(jobs)} file(s) for sm_100a", flush=True)
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(lambda j: _run(*j), jobs))
    target = ext_path()
    if jobs or _newer(objs, target):
        libs = []
        for p in ce.library_paths("cuda") if "device_type" in ce.library_paths.__code__.co_varnames else ce.library_paths(cuda=True):
            libs += ["-L", p, f"-Wl,-rpath,{p}"]
        _run(["g++", "-shared", "-o", target] + objs + libs +
             ["-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python", "-lc10_cuda", "-ltorch_cuda", "-lcudart"], "link.log")
        if verbose:
            print(f"[picotron_b200.build] linked {target}", flush=True)
    return target


def ptxas_report() -> str:
    """Concatenated ``-Xptxas -v`` output of the last build (registers, spills, shared memory per kernel)."""
    out = []
    for f in sorted(os.listdir(OBJ)) if os.path.isdir(OBJ) else []:
        if f.endswith(".nvcc.log"):
            with open(os.path.join(OBJ, f)) as fh:
                out.append(fh.read())
    return "\n".join(out)


if __name__ == "__main__":
    build()
    sys.exit(0)
