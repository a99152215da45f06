"""In-tree build of the CUDA library (sm_100a) with nvcc.

``python -m deepscalemd_b200.build`` compiles ``csrc/*.cu`` into ``libdsmd_b200.so`` beside this file. The built
library is loaded by :mod:`deepscalemd_b200.capi` through ctypes; there is no other compute path.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SOURCES = ["csrc/dsmd_core.cu", "csrc/dsmd_edges.cu", "csrc/dsmd_domain.cu", "csrc/dsmd_noalloc.cu"]
LIBRARY = os.path.join(HERE, "libdsmd_b200.so")
# host-side input layer (run description, coordinate / topology / restart files): plain C++, no CUDA
HOST_SOURCES = ["csrc/host/run_config.cpp", "csrc/host/system_input.cpp", "csrc/host/restart_file.cpp",
                "csrc/host/dynamics.cpp", "csrc/host/dsmd_input_capi.cpp"]
HOST_LIBRARY = os.path.join(HERE, "libdsmd_input.so")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17", "--use_fast_math=false",
         "-Xcompiler", "-fPIC", "-shared"]


def nvcc_path() -> str:
    path = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(path):
        raise RuntimeError("nvcc not found: the CUDA toolkit is required to build libdsmd_b200.so")
    return path


def sources() -> list[str]:
    return [os.path.join(HERE, s) for s in SOURCES if os.path.exists(os.path.join(HERE, s))]


def is_stale() -> bool:
    if not os.path.exists(LIBRARY):
        return True
    built = os.path.getmtime(LIBRARY)
    deps = sources() + [os.path.join(HERE, "csrc", f) for f in os.listdir(os.path.join(HERE, "csrc"))]
    deps.append(os.path.join(HERE, "..", "include", "dsmd_b200.h"))
    return any(os.path.getmtime(d) > built for d in deps if os.path.exists(d))


def build_host(force: bool = False) -> str:
    srcs = [os.path.join(HERE, s) for s in HOST_SOURCES]
    deps = srcs + [os.path.join(HERE, "csrc", "host", f) for f in os.listdir(os.path.join(HERE, "csrc", "host"))]
    deps.append(os.path.join(HERE, "..", "include", "dsmd_input.h"))
    if not force and os.path.exists(HOST_LIBRARY) and all(os.path.getmtime(d) <= os.path.getmtime(HOST_LIBRARY) for d in deps):
        return HOST_LIBRARY
    cmd = ["/usr/bin/g++", "-std=c++17", "-O2", "-Wall", "-fPIC", "-shared", "-I", os.path.join(HERE, "..", "include"),
           "-o", HOST_LIBRARY, *srcs]
    subprocess.run(cmd, check=True, cwd=HERE)
    return HOST_LIBRARY


DRIVER = os.path.join(HERE, "bin", "dsmd_b200_run")


def build_driver(force: bool = False) -> str:
    """The MD driver executable (host C++ over the C ABI; linked against libdsmd_b200.so beside it)."""
    srcs = [os.path.join(HERE, "csrc", "host", "dsmd_run.cpp")] + [os.path.join(HERE, s) for s in HOST_SOURCES[:-1]]
    deps = srcs + [LIBRARY, os.path.join(HERE, "..", "include", "dsmd_b200.h")]
    deps += [os.path.join(HERE, "csrc", "host", f) for f in os.listdir(os.path.join(HERE, "csrc", "host"))]
    if not force and os.path.exists(DRIVER) and all(os.path.getmtime(d) <= os.path.getmtime(DRIVER) for d in deps):
        return DRIVER
    os.makedirs(os.path.dirname(DRIVER), exist_ok=True)
    cuda_lib = os.path.join(os.path.dirname(os.path.dirname(nvcc_path())), "lib64")
    cmd = ["/usr/bin/g++", "-std=c++17", "-O2", "-Wall", "-I", os.path.join(HERE, "..", "include"), "-I",
           os.path.join(HERE, "csrc", "host"), "-o", DRIVER, *srcs, "-L", HERE, "-l:libdsmd_b200.so",
           "-Wl,-rpath,$ORIGIN/..", f"-Wl,-rpath,{cuda_lib}"]
    subprocess.run(cmd, check=True, cwd=HERE)
    return DRIVER


def build(force: bool = False, verbose: bool = False) -> str:
    build_host(force)
    library = _build_cuda(force, verbose)
    build_driver(force)
    return library


def _build_cuda(force: bool = False, verbose: bool = False) -> str:
    if not force and not is_stale():
        return LIBRARY
    flags = [f for f in FLAGS if f != "--use_fast_math=false"]
    cmd = [nvcc_path(), *flags, "-ccbin", "/usr/bin/g++", "-o", LIBRARY, *sources(), "-ldl"]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
        print(" ".join(cmd))
    subprocess.run(cmd, check=True, cwd=HERE)
    return LIBRARY


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(LIBRARY)
