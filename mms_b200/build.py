"""Builds libmms_sim.so (CUDA kernels + C ABI) in-tree with nvcc for sm_100a.

Run as `python -m mms_b200.build`.  nvcc cross-compiles without a GPU.
"""
import os
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
REPO_DIR = os.path.dirname(PKG_DIR)
LIB_PATH = os.path.join(PKG_DIR, "libmms_sim.so")
SOURCES = [os.path.join(PKG_DIR, "csrc", "mms_sim.cu"),
           os.path.join(PKG_DIR, "csrc", "latency_stats.cu")]
HEADERS = [os.path.join(REPO_DIR, "include", "mms_sim.h"),
           os.path.join(PKG_DIR, "csrc", "sim_core.cuh"),
           os.path.join(PKG_DIR, "csrc", "sim_chunk.cuh"),
           os.path.join(PKG_DIR, "csrc", "sim_batching.cuh"),
           os.path.join(PKG_DIR, "csrc", "mms_abi.inl")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    # time arithmetic must keep the reference's operation order
    "-fmad=false", "-prec-div=true", "-prec-sqrt=true",
    "-Xcompiler", "-fPIC", "-shared",
]


HOST_LIB_PATH = os.path.join(PKG_DIR, "libmms_host.so")
HOST_SOURCE = os.path.join(PKG_DIR, "csrc", "encode_host.c")


def build_host(force=False):
    """Compile the host-side helper (gcc, CPython headers): flattens placement
    lists for the encoder.  Optional: without it the encoder walks the lists
    in Python."""
    import sysconfig
    if (not force and os.path.exists(HOST_LIB_PATH)
            and os.path.getmtime(HOST_LIB_PATH) >= os.path.getmtime(HOST_SOURCE)):
        return HOST_LIB_PATH
    include = sysconfig.get_paths()["include"]
    if not os.path.exists(os.path.join(include, "Python.h")):
        return None
    cmd = [os.environ.get("CC", "gcc"), "-O2", "-pthread", "-shared", "-fPIC", "-I", include,
           "-o", HOST_LIB_PATH, HOST_SOURCE]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout)
        raise RuntimeError("gcc failed building libmms_host.so")
    return HOST_LIB_PATH


def _nvcc():
    cand = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    return cand if os.path.exists(cand) else "nvcc"


def is_stale():
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(p) > built for p in SOURCES + HEADERS)


def build(force=False, verbose=False):
    """Compile the extension if it is missing or older than its sources."""
    build_host(force)
    if not force and not is_stale():
        return LIB_PATH
    cmd = [_nvcc()] + NVCC_FLAGS + ["-I", os.path.join(REPO_DIR, "include")]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", LIB_PATH] + SOURCES
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libmms_sim.so")
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
