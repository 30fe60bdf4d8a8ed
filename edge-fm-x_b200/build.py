"""Build recipe: nvcc for the sm_100a backend library, g++ for the host engine and the pybind
module.  No CMake, no network; every output lands in-tree under lib/ and python/.

    python edge-fm-x_b200/build.py            # build what is out of date
    python edge-fm-x_b200/build.py --force    # rebuild everything
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
LIB_DIR = os.path.join(HERE, "lib")
PY_DIR = os.path.join(HERE, "python")
OBJ_DIR = os.path.join(HERE, "build")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
CUDA_INC = "/usr/local/cuda/include"
CUDA_LIB = "/usr/local/cuda/lib64"

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr", "-Xptxas", "-v"]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-Wextra", "-Wno-unused-parameter"]

BACKEND_CU = ["src/backends/b200/efm_b200.cu", "src/layers/qwen_text.cu", "src/backends/b200/vit_b200.cu", "src/backends/b200/vla_b200.cu",
              "src/backends/b200/nccl_glue.cpp"]
ENGINE_CPP = sorted(glob.glob(os.path.join(HERE, "src", "engine", "*.cpp"))) + \
    [os.path.join(HERE, "src", "edge-fm.cpp"), os.path.join(HERE, "src", "tensor.cpp")]


def _newer(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def _all_sources():
    out = []
    for pat in ("src/**/*.cu", "src/**/*.cuh", "src/**/*.h", "src/**/*.cpp", "include/**/*.h"):
        out += glob.glob(os.path.join(HERE, pat), recursive=True)
    out += glob.glob(os.path.join(ROOT, "include", "*.h"))
    return out


def _run(cmd, log=None):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if log is not None:
        with open(log, "w") as f:
            f.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError("build step failed: " + cmd[0])
    return r


def dlpack_include() -> str:
    """dlpack/dlpack.h is taken from a package already in the image (never vendored)."""
    import importlib.util
    for mod, rel in (("tvm_ffi", "include"), ("xgrammar", "include")):
        spec = importlib.util.find_spec(mod)
        if spec and spec.submodule_search_locations:
            p = os.path.join(list(spec.submodule_search_locations)[0], rel)
            if os.path.exists(os.path.join(p, "dlpack", "dlpack.h")):
                return p
    raise RuntimeError("dlpack/dlpack.h not found in the image")


def build_backend(force=False) -> str:
    os.makedirs(LIB_DIR, exist_ok=True)
    os.makedirs(OBJ_DIR, exist_ok=True)
    out = os.path.join(LIB_DIR, "libefm_b200.so")
    deps = _all_sources()
    if not force and not _newer(out, deps):
        return out
    objs = []

    def compile_one(rel):
        obj = os.path.join(OBJ_DIR, os.path.basename(rel) + ".o")
        _run([NVCC, *NVCC_FLAGS, "-I", os.path.join(ROOT, "include"), "-c", os.path.join(HERE, rel), "-o", obj],
             log=obj + ".log")
        return obj
    with ThreadPoolExecutor(max_workers=4) as ex:
        objs = list(ex.map(compile_one, BACKEND_CU))
    _run([NVCC, "-shared", "-o", out, *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-lcudart", "-ldl"])
    return out


def build_engine(force=False):
    """Host engine (libedge_fm.so) + pybind11 module edge_fm; both call the backend through its C ABI."""
    import pybind11
    os.makedirs(PY_DIR, exist_ok=True)
    backend = build_backend(force)
    inc = ["-I", os.path.join(HERE, "include"), "-I", os.path.join(ROOT, "include"), "-I", dlpack_include(),
           "-I", CUDA_INC]
    lib = os.path.join(LIB_DIR, "libedge_fm.so")
    deps = _all_sources()
    if force or _newer(lib, deps):
        _run(["g++", *CXX_FLAGS, "-shared", "-o", lib, *ENGINE_CPP, *inc, "-L", LIB_DIR, "-lefm_b200",
              "-L", CUDA_LIB, "-lcudart", "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + CUDA_LIB])
    mod = os.path.join(PY_DIR, "edge_fm" + sysconfig.get_config_var("EXT_SUFFIX"))
    if force or _newer(mod, deps + [lib]):
        _run(["g++", *CXX_FLAGS, "-shared", "-fvisibility=hidden", "-o", mod,
              os.path.join(HERE, "src", "python", "pybind.cpp"), *inc, "-I", pybind11.get_include(),
              "-I", sysconfig.get_paths()["include"], "-L", LIB_DIR, "-ledge_fm", "-lefm_b200",
              "-Wl,-rpath,$ORIGIN/../lib", "-Wl,-rpath," + CUDA_LIB])
    return backend, lib, mod


def ptxas_report() -> str:
    out = []
    for f in sorted(glob.glob(os.path.join(OBJ_DIR, "*.log"))):
        out.append(open(f).read())
    return "\n".join(out)


if __name__ == "__main__":
    force = "--force" in sys.argv
    if "--backend-only" in sys.argv:
        print(build_backend(force))
    else:
        print(build_engine(force))
