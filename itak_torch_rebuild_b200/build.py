"""Builds the sm_100a shared library (and a static archive) from csrc/*.cu with nvcc.

The products land in ``itak_torch_rebuild_b200/lib/`` so they travel with the tree:
``libitak_cuda_compute.so`` (what the Python harness loads through ctypes) and
``libitak_cuda_compute.a`` (what a ``crates/cuda-compute`` build script links).
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
SO_PATH = os.path.join(LIB_DIR, "libitak_cuda_compute.so")
A_PATH = os.path.join(LIB_DIR, "libitak_cuda_compute.a")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-cudart", "static",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA toolkit is required to build the kernels")


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _stale(target: str) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    deps = sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.hpp")) + glob.glob(os.path.join(HERE, "..", "include", "*.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every kernel for sm_100a; returns the path of the shared library."""
    if not force and not _stale(SO_PATH) and not _stale(A_PATH):
        return SO_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    nvcc = _nvcc()
    objs = []
    extra = ["-Xptxas", "-v"] if verbose else []
    for src in sources():
        obj = os.path.join(LIB_DIR, os.path.basename(src)[:-3] + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-c", src, "-o", obj]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}")
        objs.append(obj)
    res = subprocess.run([nvcc, *NVCC_FLAGS, "-shared", *objs, "-o", SO_PATH], capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed to link the shared library")
    if os.path.exists(A_PATH):
        os.remove(A_PATH)
    subprocess.run(["ar", "rcs", A_PATH, *objs], check=True)
    return SO_PATH


ASAN_PATH = os.path.join(LIB_DIR, "libitak_host_asan.so")
HOST_ONLY_SOURCES = ["prefix_store.cu"]  # no kernel, no CUDA call: compiles as plain C++


def sanitizer_compiler():
    """The first C++ compiler among the system g++, the one on PATH and $CXX that can link the sanitizer runtimes
    (a toolchain without libasan fails at link time), or None."""
    import tempfile

    seen = []
    for cand in ("/usr/bin/g++", shutil.which("g++"), os.environ.get("CXX")):
        if not cand or cand in seen or not os.path.exists(cand):
            continue
        seen.append(cand)
        with tempfile.TemporaryDirectory() as tmp:
            src = os.path.join(tmp, "probe.cpp")
            with open(src, "w") as f:
                f.write("int main() { return 0; }\n")
            res = subprocess.run([cand, "-fsanitize=address,undefined", src, "-o", os.path.join(tmp, "probe")],
                                 capture_output=True, text=True)
            if res.returncode == 0:
                return cand
    return None


def build_sanitized(force: bool = False) -> str:
    """The host-only part of the library (the prefix store and the ITKV decoder, which parse untrusted bytes) built
    with g++ under AddressSanitizer and UndefinedBehaviorSanitizer, for the CPU tests that feed it forged input."""
    srcs = [os.path.join(CSRC, f) for f in HOST_ONLY_SOURCES]
    deps = srcs + glob.glob(os.path.join(CSRC, "*.hpp")) + glob.glob(os.path.join(HERE, "..", "include", "*.h"))
    if not force and os.path.exists(ASAN_PATH) and all(os.path.getmtime(d) <= os.path.getmtime(ASAN_PATH) for d in deps):
        return ASAN_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    cxx = sanitizer_compiler()
    if cxx is None:
        raise RuntimeError("no C++ compiler here links -fsanitize=address,undefined")
    cmd = [cxx, "-std=c++17", "-O1", "-g", "-fPIC", "-shared", "-fsanitize=address,undefined",
           "-fno-sanitize-recover=undefined", "-fno-omit-frame-pointer"]
    for src in srcs:
        cmd += ["-x", "c++", src]
    cmd += ["-x", "none", "-o", ASAN_PATH]  # "-x c++" must not reach the sanitizer runtimes the driver appends
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("sanitized host build failed")
    return ASAN_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
