"""Build the native libraries in-tree.

``lib/liblmoe.so``       CUDA kernels for sm_100a (every ``csrc/*.cu``), plain C ABI, loaded with ctypes
``lib/liblmoe_host.so``  host-side C++ helpers (``csrc/host/*.cpp``)

``nvcc`` cross-compiles without a GPU.  Objects are rebuilt only when a source or header is newer.
Run ``python -m linear_moe_b200.build`` or call :func:`build_all`.
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

ROOT = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(ROOT, "csrc")
LIB = os.path.join(ROOT, "lib")
OBJ = os.path.join(ROOT, "build")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found")
    return cand


def _newer(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(cmd) + "\n" + r.stdout + r.stderr)
    return r.stdout + r.stderr


def build_cuda(verbose: bool = False, extra_flags=()) -> str:
    os.makedirs(LIB, exist_ok=True)
    os.makedirs(OBJ, exist_ok=True)
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    hdrs = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h"))
    nvcc = _nvcc()
    objs, jobs = [], []
    for s in srcs:
        o = os.path.join(OBJ, os.path.basename(s)[:-3] + ".o")
        objs.append(o)
        if _newer(o, [s] + hdrs):
            jobs.append([nvcc, *NVCC_FLAGS, *extra_flags, "-I", CSRC, "-c", s, "-o", o])
    with ThreadPoolExecutor(max_workers=min(8, max(len(jobs), 1))) as ex:
        for out in ex.map(_run, jobs):
            if verbose and out.strip():
                print(out)
    so = os.path.join(LIB, "liblmoe.so")
    if jobs or _newer(so, objs):
        _run([nvcc, "-shared", "-o", so, *objs, "-lcudart"])
    return so


def build_host(verbose: bool = False, sanitize: bool = False, out_dir: str = None) -> str:
    """``sanitize``: an AddressSanitizer + UndefinedBehaviorSanitizer build (``liblmoe_host_asan.so``) for the tests that
    run the host helpers under the sanitizers; it is loaded into a process that preloads the ASan runtime."""
    out_dir = out_dir or LIB
    os.makedirs(out_dir, exist_ok=True)
    srcs = sorted(glob.glob(os.path.join(CSRC, "host", "*.cpp")))
    so = os.path.join(out_dir, "liblmoe_host_asan.so" if sanitize else "liblmoe_host.so")
    if srcs and _newer(so, srcs):
        flags = ["-O1", "-g", "-fsanitize=address,undefined", "-fno-sanitize-recover=all", "-fno-omit-frame-pointer"] \
            if sanitize else ["-O3"]
        _run(["g++", *flags, "-std=c++17", "-fPIC", "-shared", "-pthread", "-o", so, *srcs])
    return so


def build_all(verbose: bool = False):
    return build_cuda(verbose), build_host(verbose)


if __name__ == "__main__":
    print(build_all(verbose="-v" in sys.argv))
