"""In-tree build of the native libraries (no JIT cache: the built .so files travel with the source tree).

  libspark_kernels.so : every .cu under csrc/kernels, compiled for sm_100a only
  _runtime*.so        : C++ host runtime (KV pool, scheduler core, prefix-cache I/O, ...) as a pybind11 module

Usage: `python -m spark_engine_b200.build [--force]`.
"""
from __future__ import annotations

import concurrent.futures as cf
import glob
import os
import subprocess
import sys
import sysconfig

ROOT = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(ROOT, "csrc")
LIBDIR = os.path.join(ROOT, "_lib")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-I", os.path.join(CSRC, "common")]


def _newer(src_list, out):
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    return any(os.path.getmtime(s) > t for s in src_list)


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build failed: " + " ".join(cmd) + "\n" + r.stdout + r.stderr)
    return r.stdout + r.stderr


def build_kernels(force=False, verbose=False) -> str:
    os.makedirs(LIBDIR, exist_ok=True)
    out = os.path.join(LIBDIR, "libspark_kernels.so")
    cus = sorted(glob.glob(os.path.join(CSRC, "kernels", "*.cu")))
    headers = glob.glob(os.path.join(CSRC, "**", "*.cuh"), recursive=True) + glob.glob(os.path.join(CSRC, "**", "*.h"), recursive=True)
    objs, jobs = [], []
    for cu in cus:
        obj = os.path.join(LIBDIR, os.path.basename(cu)[:-3] + ".o")
        objs.append(obj)
        if force or _newer([cu] + headers, obj):
            jobs.append([NVCC] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", cu, "-o", obj])
    with cf.ThreadPoolExecutor(max_workers=8) as ex:
        for log in ex.map(_run, jobs):
            if verbose and log:
                print(log)
    if jobs or not os.path.exists(out):
        _run([NVCC, "-shared", "-o", out] + objs + ["-lcudart"])
    return out


def build_runtime(force=False) -> str:
    import pybind11
    os.makedirs(LIBDIR, exist_ok=True)
    ext = sysconfig.get_config_var("EXT_SUFFIX")
    out = os.path.join(LIBDIR, "_runtime" + ext)
    srcs = sorted(glob.glob(os.path.join(CSRC, "runtime", "*.cpp")))
    hdrs = glob.glob(os.path.join(CSRC, "runtime", "*.h"))
    if not srcs:
        return ""
    if force or _newer(srcs + hdrs, out):
        _run(["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-pthread", "-I", pybind11.get_include(),
              "-I", sysconfig.get_paths()["include"]] + srcs + ["-o", out, "-lrt", "-ldl"])
    return out


def build_race_stress(sanitizer: str = "thread", force=False) -> str:
    """The host runtime's concurrency stress driver (csrc/runtime/stress/race_stress.cpp) linked against the runtime
    sources with -fsanitize=<sanitizer> ("thread", or "address,undefined"); returns the executable's path.  It needs
    no GPU: device memory is the fake driver's host memory."""
    os.makedirs(LIBDIR, exist_ok=True)
    out = os.path.join(LIBDIR, "race_stress_" + sanitizer.replace(",", "_"))
    rt = os.path.join(CSRC, "runtime")
    srcs = [os.path.join(rt, "stress", "race_stress.cpp")] + [os.path.join(rt, f) for f in
                                                              ("pcache.cpp", "oplog.cpp", "memguard.cpp", "devmem.cpp")]
    if force or _newer(srcs + glob.glob(os.path.join(rt, "*.h")), out):
        _run(["g++", "-O1", "-g", "-std=c++17", "-pthread", "-fsanitize=" + sanitizer] + srcs + ["-o", out, "-lrt", "-ldl"])
    return out


def build_all(force=False, verbose=False):
    return build_kernels(force, verbose), build_runtime(force)


if __name__ == "__main__":
    k, r = build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print("built", k, r)
