"""In-tree build of the two native artefacts:

* ``libattn_b200.so``  -- CUDA kernels + C ABI (``include/attn_b200.h``), built with
  ``nvcc -gencode arch=compute_100a,code=sm_100a``; no PyTorch dependency.
* ``attention_cuda*.so`` -- the PyTorch extension module with the reference's
  ``v7_forward / v7_backward / v7_double_backward`` surface, linked against the
  library above (found through ``$ORIGIN`` at run time).

Both land next to this file so that they travel with the source tree.
``python -m`` style use:  ``python 610sample_b200/_build.py [--force]``.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(ROOT, "include")
BUILD = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libattn_b200.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-I" + INCLUDE, "-I" + CSRC]
CU_SOURCES = ["attn_capi.cu", "attn_prep.cu", "attn_simt.cu", "attn_tc.cu", "attn_tc_fb.cu", "attn_tc_fwd.cu", "attn_tc_hvp_row.cu", "attn_tc_hvp_col.cu"]
HEADERS = ["attn_common.cuh", "attn_launch.h", "tc_primitives.cuh", "tc_common.cuh", os.path.join(INCLUDE, "attn_b200.h")]


def _nvcc() -> str:
    for c in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if c and (os.path.isabs(c) and os.path.exists(c) or not os.path.isabs(c)):
            return c
    return "nvcc"


def _digest(paths) -> str:
    h = hashlib.sha256()
    for p in paths:
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def _stale(target: str, stamp_name: str, digest: str) -> bool:
    stamp = os.path.join(BUILD, stamp_name)
    if not os.path.exists(target) or not os.path.exists(stamp):
        return True
    with open(stamp) as f:
        return f.read().strip() != digest


def _write_stamp(stamp_name: str, digest: str) -> None:
    with open(os.path.join(BUILD, stamp_name), "w") as f:
        f.write(digest)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)


def ext_path() -> str:
    return os.path.join(HERE, "attention_cuda" + sysconfig.get_config_var("EXT_SUFFIX"))


def build_library(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(BUILD, exist_ok=True)
    hdrs = [h if os.path.isabs(h) else os.path.join(CSRC, h) for h in HEADERS]
    srcs = [os.path.join(CSRC, s) for s in CU_SOURCES]
    digest = _digest(srcs + hdrs + [__file__])
    if not force and not _stale(LIB, "lib.stamp", digest):
        return LIB
    procs, objs = [], []
    for s in srcs:
        o = os.path.join(BUILD, os.path.basename(s)[:-3] + ".o")
        objs.append(o)
        cmd = [_nvcc()] + NVCC_FLAGS + ["-c", s, "-o", o]
        if verbose:
            print(" ".join(cmd), flush=True)
        procs.append(subprocess.Popen(cmd))
    for p in procs:
        if p.wait() != 0:
            raise RuntimeError("nvcc failed")
    _run([_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", LIB] + objs, verbose)
    _write_stamp("lib.stamp", digest)
    return LIB


def build_extension(force: bool = False, verbose: bool = False) -> str:
    import torch
    from torch.utils import cpp_extension as ce

    build_library(force, verbose)
    target = ext_path()
    src = os.path.join(CSRC, "attention_ext.cpp")
    digest = _digest([src, os.path.join(INCLUDE, "attn_b200.h"), __file__]) + torch.__version__
    if not force and not _stale(target, "ext.stamp", digest):
        return target
    inc = []
    for p in ce.include_paths("cuda") if "device_type" in ce.include_paths.__code__.co_varnames else ce.include_paths(True):
        inc += ["-isystem", p]
    inc += ["-isystem", sysconfig.get_paths()["include"], "-I" + INCLUDE]
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cuda_home = ce.CUDA_HOME or "/usr/local/cuda"
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-DTORCH_EXTENSION_NAME=attention_cuda",
           "-DTORCH_API_INCLUDE_EXTENSION_H", "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI),
           src, "-o", target] + inc + [
           "-L" + torch_lib, "-L" + HERE, "-L" + os.path.join(cuda_home, "lib64"),
           "-lattn_b200", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
           "-lcudart", "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + torch_lib]
    _run(cmd, verbose)
    _write_stamp("ext.stamp", digest)
    return target


def build_all(force: bool = False, verbose: bool = False):
    return build_library(force, verbose), build_extension(force, verbose)


if __name__ == "__main__":
    print(build_all(force="--force" in sys.argv, verbose=True))
