"""Build ``libqutai_moe.so`` with nvcc for sm_100a (cross-compiles on a machine without a GPU).

``python -m qutai_b200.build`` builds in-tree; ``ensure_built()`` builds only when a source is newer
than the library.  The upstream package compiles its kernels at run time through NVRTC
(src/qutai/backends/cuda_runtime.py:274-297); this library is built ahead of time instead.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PACKAGE_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PACKAGE_DIR, "csrc")
INCLUDE = os.path.join(os.path.dirname(PACKAGE_DIR), "include")
LIBRARY = os.path.join(PACKAGE_DIR, "libqutai_moe.so")
SOURCES = ("runtime.cu", "routing.cu", "permute.cu", "gemm_simt.cu", "gemm_tcgen05.cu", "router.cu", "layer.cu", "ep.cu", "optim.cu", "norm.cu", "head.cu", "attention.cu", "lm_ops.cu")
ARCH_FLAGS = ("-gencode", "arch=compute_100a,code=sm_100a")


def nvcc_path():
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and os.path.isfile(candidate):
            return candidate
    raise RuntimeError("nvcc not found: set NVCC or put the CUDA toolkit on PATH")


def _inputs():
    files = [os.path.join(CSRC, name) for name in os.listdir(CSRC) if name.endswith((".cu", ".cuh"))]
    files.append(os.path.join(INCLUDE, "qutai_moe.h"))
    return files


def is_stale():
    if not os.path.isfile(LIBRARY):
        return True
    built = os.path.getmtime(LIBRARY)
    return any(os.path.getmtime(path) > built for path in _inputs())


def build(verbose=False, ptxas_info=False):
    """Compile every source to an object and link the shared library.  Returns its path."""
    nvcc = nvcc_path()
    objdir = os.path.join(PACKAGE_DIR, "build")
    os.makedirs(objdir, exist_ok=True)
    common = [nvcc, *ARCH_FLAGS, "-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC",
              "-I", INCLUDE, "--expt-relaxed-constexpr"]
    if ptxas_info:
        common += ["-Xptxas", "-v"]
    procs, objects = [], []
    for name in SOURCES:
        obj = os.path.join(objdir, name.replace(".cu", ".o"))
        objects.append(obj)
        cmd = common + ["-c", os.path.join(CSRC, name), "-o", obj]
        if verbose:
            print(" ".join(cmd), flush=True)
        procs.append((name, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = []
    for name, proc in procs:
        out, _ = proc.communicate()
        if proc.returncode:
            failed.append(f"--- {name} ---\n{out}")
        elif (verbose or ptxas_info) and out.strip():
            print(f"--- {name} ---\n{out}", flush=True)
    if failed:
        raise RuntimeError("nvcc failed:\n" + "\n".join(failed))
    link = [nvcc, *ARCH_FLAGS, "-shared", "-o", LIBRARY + ".tmp", *objects, "-ldl"]
    done = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if done.returncode:
        raise RuntimeError("link failed:\n" + done.stdout)
    os.replace(LIBRARY + ".tmp", LIBRARY)
    return LIBRARY


def ensure_built():
    """Path of the library, building it first when it is missing or older than its sources."""
    if is_stale():
        try:
            nvcc_path()
        except RuntimeError:
            if os.path.isfile(LIBRARY):
                return LIBRARY  # no compiler on this machine: use the library that was shipped
            raise
        build()
    return LIBRARY


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, ptxas_info="--ptxas" in sys.argv))
