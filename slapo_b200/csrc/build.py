"""Build the in-tree ``slapo_b200/_C.so`` for sm_100a.

``python -m slapo_b200.csrc.build`` compiles every ``.cu`` file with::

    nvcc -gencode arch=compute_100a,code=sm_100a -lineinfo -O3

(the kernel sources include no torch header, so each takes seconds), the
``.cpp`` binding files with the host compiler against the installed torch,
and links them into one shared object next to the package, which is what
``slapo_b200.ops.native`` loads.  Objects are rebuilt only when their source
or a header changed.  No GPU is needed.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
OUT = os.path.join(PKG, "_C.so")
OBJ_DIR = os.path.join(HERE, "build")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--use_fast_math", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
              "-Xptxas", "-v"]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-D_GLIBCXX_USE_CXX11_ABI=1",
             "-DTORCH_API_INCLUDE_EXTENSION_H", "-Wno-deprecated-declarations"]


def _cuda_home():
    return os.environ.get("CUDA_HOME", "/usr/local/cuda")


def _torch_paths():
    import torch
    from torch.utils import cpp_extension

    inc = cpp_extension.include_paths("cuda") if "device_type" in \
        cpp_extension.include_paths.__code__.co_varnames else cpp_extension.include_paths(True)
    lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    return inc, lib, abi


def _newer(src_list, target):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in src_list)


def _run(cmd, log):
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    log.append((" ".join(cmd), res.stdout))
    if res.returncode != 0:
        raise RuntimeError(f"build step failed:\n{' '.join(cmd)}\n{res.stdout}")
    return res.stdout


def build(verbose: bool = False, force: bool = False) -> str:
    os.makedirs(OBJ_DIR, exist_ok=True)
    inc, torch_lib, abi = _torch_paths()
    headers = [os.path.join(HERE, f) for f in os.listdir(HERE) if f.endswith((".h", ".cuh"))]
    cu_srcs = sorted(f for f in os.listdir(HERE) if f.endswith(".cu"))
    cpp_srcs = sorted(f for f in os.listdir(HERE) if f.endswith(".cpp"))
    nvcc = os.path.join(_cuda_home(), "bin", "nvcc")
    # SLAPO_B200_DEBUG=1 at build time: index / alignment checks inside the fused kernels that
    # report through the device status word (code 7) instead of touching a bad peer address
    debug = ["-DSLAPO_B200_DEBUG"] if os.environ.get("SLAPO_B200_DEBUG", "0") == "1" else []
    cxx = os.environ.get("CXX", "g++")
    log, jobs, objs = [], [], []
    for src in cu_srcs:
        obj = os.path.join(OBJ_DIR, src + ".o")
        objs.append(obj)
        if force or _newer([os.path.join(HERE, src)] + headers, obj):
            jobs.append([nvcc] + NVCC_FLAGS + debug + ["-I", HERE, "-c", os.path.join(HERE, src),
                                                       "-o", obj])
    cxx_flags = [f.replace("ABI=1", f"ABI={abi}") for f in CXX_FLAGS]
    for src in cpp_srcs:
        obj = os.path.join(OBJ_DIR, src + ".o")
        objs.append(obj)
        if force or _newer([os.path.join(HERE, src)] + headers, obj):
            cmd = [cxx] + cxx_flags + ["-I", HERE, "-I", os.path.join(_cuda_home(), "include")]
            for path in inc:
                cmd += ["-isystem", path]
            jobs.append(cmd + ["-c", os.path.join(HERE, src), "-o", obj])
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            outs = list(pool.map(lambda c: _run(c, log), jobs))
        if verbose:
            for (cmd, out) in log:
                print(cmd)
                print(out)
        ptxas = os.path.join(OBJ_DIR, "ptxas.log")
        # append, but start over once the log has grown past a few MB
        mode = "a" if os.path.exists(ptxas) and os.path.getsize(ptxas) < 4 * 2**20 else "w"
        with open(ptxas, mode) as fh:
            for cmd, out in log:
                fh.write(cmd + "\n" + out + "\n")
    if jobs or force or _newer(objs, OUT):
        # link beside the target and rename: a reader never sees a half-written library
        tmp = OUT + ".tmp"
        link = [cxx, "-shared", "-o", tmp] + objs + [
            "-L", torch_lib, "-L", os.path.join(_cuda_home(), "lib64"),
            "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda", "-lcudart",
            f"-Wl,-rpath,{torch_lib}"]
        _run(link, log)
        os.replace(tmp, OUT)
    return OUT


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv, force="-f" in sys.argv)
    print(path)
