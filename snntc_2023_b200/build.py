"""Builds the CUDA libraries (sm_100a only) in-tree with nvcc.

    python -m snntc_2023_b200.build [--force] [-v]

Two shared libraries come out of the same sources:
    libsnntc_b200.so          the product: the C ABI declared in include/snntc_b200.h
    libsnntc_b200_measure.so  the same compiled with -DSNNTC_MEASURE: it adds the entry points that take the
                              kernel choice of a call explicitly (bench.py times the kernels of an operator
                              apart with them, the tests check kernel variants against each other)
Both are plain CUDA runtime code behind a C ABI and link the CUDA runtime statically, so the only requirement
at load time is an NVIDIA driver.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libsnntc_b200.so")
LIB_MEASURE = os.path.join(HERE, "libsnntc_b200_measure.so")
SOURCES = ["snntc_forward.cu", "snntc_lists.cu", "snntc_backward.cu", "snntc_dw_skip.cu", "snntc_dw_tma.cu", "snntc_dx_sparse.cu", "snntc_pool.cu",
           "snntc_noalloc.cu", "snntc_train.cu", "snntc_api.cu"]
API_SOURCE = "snntc_api.cu"   # the only file that reads SNNTC_MEASURE
HEADERS = [os.path.join(CSRC, "snntc_common.cuh"), os.path.join(CSRC, "snntc_merge.cuh"),
           os.path.join(HERE, "..", "include", "snntc_b200.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


def _nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; libsnntc_b200.so cannot be built")


def sources():
    return [os.path.join(CSRC, s) for s in SOURCES]


def up_to_date():
    if not (os.path.exists(LIB) and os.path.exists(LIB_MEASURE)):
        return False
    t = min(os.path.getmtime(LIB), os.path.getmtime(LIB_MEASURE))
    return all(os.path.getmtime(p) <= t for p in sources() + HEADERS)


def build(force=False, verbose=False):
    if not force and up_to_date():
        return LIB
    nvcc = _nvcc()
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    objs = []
    procs = []
    extra = ["-Xptxas", "-v"] if verbose else []
    for src in sources():
        obj = os.path.join(objdir, os.path.basename(src)[:-3] + ".o")
        cmd = [nvcc] + NVCC_FLAGS + extra + ["-c", src, "-o", obj]
        procs.append((cmd, subprocess.Popen(cmd)))
        objs.append(obj)
    api_measure = os.path.join(objdir, "snntc_api_measure.o")
    cmd = [nvcc] + NVCC_FLAGS + ["-DSNNTC_MEASURE", "-c", os.path.join(CSRC, API_SOURCE), "-o", api_measure]
    procs.append((cmd, subprocess.Popen(cmd)))
    for cmd, p in procs:
        if p.wait() != 0:
            raise RuntimeError("nvcc failed: " + " ".join(cmd))
    subprocess.check_call([nvcc, "-shared", "-o", LIB] + objs)
    api_obj = os.path.join(objdir, API_SOURCE[:-3] + ".o")
    subprocess.check_call([nvcc, "-shared", "-o", LIB_MEASURE] + [api_measure if o == api_obj else o for o in objs])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
