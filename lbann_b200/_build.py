"""In-tree native build: every ``csrc/*.cu`` / ``csrc/*.cpp`` -> ``_native/liblbann_b200.so``.

The kernels are plain CUDA C++ with ``extern "C"`` launchers (no torch headers), so a
file compiles in seconds and the library can be loaded with ``ctypes`` by any host
program.  nvcc cross-compiles for sm_100a without a GPU present.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT_DIR = os.path.join(HERE, "_native")
LIB_NAME = "liblbann_b200.so"
HOST_LIB_NAME = "liblbann_b200_host.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-pthread"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC")


def _digest(path: str, extra: str) -> str:
    h = hashlib.sha1(extra.encode())
    with open(path, "rb") as f:
        h.update(f.read())
    for hdr in sorted(os.listdir(CSRC)):
        if hdr.endswith((".cuh", ".h", ".hpp")):
            with open(os.path.join(CSRC, hdr), "rb") as f:
                h.update(f.read())
    return h.hexdigest()


def _compile_one(cmd, src, obj, stamp, digest, verbose):
    if verbose:
        print("[lbann_b200 build]", os.path.basename(src), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"compile failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    with open(stamp, "w") as f:
        f.write(digest)


def build_native(verbose: bool = False, force: bool = False) -> dict:
    """Compile (incrementally) and link both native libraries; returns their paths."""
    os.makedirs(OUT_DIR, exist_ok=True)
    obj_dir = os.path.join(OUT_DIR, "obj")
    os.makedirs(obj_dir, exist_ok=True)
    nvcc = _nvcc()
    cu_srcs = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    cpp_srcs = sorted(f for f in os.listdir(CSRC) if f.endswith(".cpp"))
    jobs = []
    cu_objs, cpp_objs = [], []
    relink_cu = relink_cpp = force
    for name in cu_srcs + cpp_srcs:
        src = os.path.join(CSRC, name)
        obj = os.path.join(obj_dir, name + ".o")
        stamp = obj + ".sha1"
        is_cu = name.endswith(".cu")
        if is_cu:
            cmd = [nvcc] + NVCC_FLAGS + ["-I", CSRC, "-c", src, "-o", obj]
            cu_objs.append(obj)
        else:
            cmd = ["g++"] + CXX_FLAGS + ["-I", CSRC, "-c", src, "-o", obj]
            cpp_objs.append(obj)
        digest = _digest(src, " ".join(cmd))
        old = open(stamp).read() if os.path.exists(stamp) else ""
        if force or old != digest or not os.path.exists(obj):
            jobs.append((cmd, src, obj, stamp, digest, verbose))
            if is_cu:
                relink_cu = True
            else:
                relink_cpp = True
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
            list(ex.map(lambda j: _compile_one(*j), jobs))
    lib = os.path.join(OUT_DIR, LIB_NAME)
    host_lib = os.path.join(OUT_DIR, HOST_LIB_NAME)
    if cu_objs and (relink_cu or not os.path.exists(lib)):
        # cudart is linked statically (nvcc's default): the library then carries its own
        # runtime and shares streams / memory with the host program through the driver.
        cmd = [nvcc, "-shared", "-o", lib] + cu_objs
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    if cpp_objs and (relink_cpp or not os.path.exists(host_lib)):
        cmd = ["g++", "-shared", "-pthread", "-o", host_lib] + cpp_objs
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return {"cuda": lib if cu_objs else None, "host": host_lib if cpp_objs else None}


if __name__ == "__main__":
    out = build_native(verbose=True, force="--force" in sys.argv)
    print(out)
