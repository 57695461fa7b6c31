"""Build recipe for the test oracle (TEST INFRASTRUCTURE ONLY).

Two artefacts, both git-ignored:
  oracle/liboracle.so                 -- the plain-C restatement in snntc_oracle.c (always buildable)
  oracle/_ref/libsnntc_ref_cpu.so     -- the reference's own four CPU operator files, compiled
                                         unmodified from the reference checkout against the stand-in
                                         op_kernel.h in ref_shim/ (only where that checkout exists)
  oracle/_ref/libsnntc_ref_gpu.so     -- the reference's own four GPU operator files (*.cu.cc), compiled
                                         unmodified for sm_100a against the stand-in in ref_shim_gpu/;
                                         used to time the reference's GPU kernels on a B200 and as a
                                         second parity check

Run:  python oracle/build.py [--reference-root DIR]   (default: $SNNTC_REFERENCE_ROOT, else ../reference)
"""
import argparse
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "liboracle.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_SO = os.path.join(REF_DIR, "libsnntc_ref_cpu.so")
REF_SOURCES = ["snnfc_kernels.cc", "snnfcgrad_kernels.cc", "snncv_kernels.cc", "snncvgrad_kernels.cc"]
REF_GPU_SO = os.path.join(REF_DIR, "libsnntc_ref_gpu.so")
REF_GPU_SOURCES = ["snnfc_kernels.cu.cc", "snnfcgrad_kernels.cu.cc", "snncv_kernels.cu.cc", "snncvgrad_kernels.cu.cc"]


def default_reference_root():
    """Where the reference checkout is looked for: $SNNTC_REFERENCE_ROOT, else a directory named `reference`
    beside this repository."""
    env = os.environ.get("SNNTC_REFERENCE_ROOT")
    if env:
        return env
    return os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def _newer(target, deps):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def build_oracle(force=False):
    src = [os.path.join(HERE, "snntc_oracle.c"), os.path.join(HERE, "snntc_oracle_impl.h")]
    if not force and _newer(ORACLE_SO, src):
        return ORACLE_SO
    cmd = ["gcc", "-O2", "-std=c11", "-fPIC", "-shared", "-ffp-contract=off", "-Wall", "-Wextra",
           "-o", ORACLE_SO, src[0], "-lm"]
    subprocess.check_call(cmd)
    return ORACLE_SO


def build_ref(reference_root=None, force=False):
    """Compile the reference CPU operators where they lie. Returns the .so path or None."""
    src_dir = os.path.join(reference_root or default_reference_root(), "snntc")
    srcs = [os.path.join(src_dir, s) for s in REF_SOURCES]
    if not all(os.path.exists(s) for s in srcs):
        return REF_SO if os.path.exists(REF_SO) else None
    shim = os.path.join(HERE, "ref_shim")
    deps = srcs + [os.path.join(shim, "ref_capi.cc"),
                   os.path.join(shim, "tensorflow/core/framework/op_kernel.h")]
    if not force and _newer(REF_SO, deps):
        return REF_SO
    os.makedirs(REF_DIR, exist_ok=True)
    cmd = ["g++", "-std=c++17", "-O3", "-fPIC", "-shared", "-w", "-pthread", "-I", shim, "-I", src_dir,
           os.path.join(shim, "ref_capi.cc")] + srcs + ["-o", REF_SO]
    subprocess.check_call(cmd)
    return REF_SO


def build_ref_gpu(reference_root=None, force=False):
    """Compile the reference GPU operators where they lie (nvcc, sm_100a). Returns the .so path or None."""
    import shutil
    src_dir = os.path.join(reference_root or default_reference_root(), "snntc")
    srcs = [os.path.join(src_dir, s) for s in REF_GPU_SOURCES]
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not all(os.path.exists(s) for s in srcs) or not os.path.exists(nvcc):
        return REF_GPU_SO if os.path.exists(REF_GPU_SO) else None
    shim = os.path.join(HERE, "ref_shim_gpu")
    capi = os.path.join(shim, "ref_gpu_capi.cu")
    deps = srcs + [capi, os.path.join(shim, "tensorflow/core/framework/op_kernel.h")]
    if not force and _newer(REF_GPU_SO, deps):
        return REF_GPU_SO
    os.makedirs(REF_DIR, exist_ok=True)
    flags = ["-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-DGOOGLE_CUDA=1",
             "--expt-relaxed-constexpr", "-w", "-Xcompiler", "-fPIC", "-I", shim, "-I", src_dir]
    objs = []
    for src in srcs:
        obj = os.path.join(REF_DIR, os.path.basename(src).replace(".cu.cc", "_gpu.o"))
        subprocess.check_call([nvcc] + flags + ["-x", "cu", "-c", src, "-o", obj])
        objs.append(obj)
    obj = os.path.join(REF_DIR, "ref_gpu_capi.o")
    subprocess.check_call([nvcc] + flags + ["-c", capi, "-o", obj])
    subprocess.check_call([nvcc, "-shared", "-o", REF_GPU_SO] + objs + [obj])
    return REF_GPU_SO


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference-root", default=None, help="default: $SNNTC_REFERENCE_ROOT or ../reference")
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    print(build_oracle(a.force))
    print(build_ref(a.reference_root, a.force) or "reference checkout not present: _ref not built", file=sys.stdout)
    print(build_ref_gpu(a.reference_root, a.force) or "reference checkout or nvcc not present: GPU _ref not built")
