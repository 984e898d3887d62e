"""Builds the CUDA library in-tree: paraselect_b200/libpsb.so (sm_100a only).

Usable as `python -m paraselect_b200.build`; `ensure_built()` rebuilds only when a source is newer than
the library.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
OBJ = os.path.join(HERE, "_obj")
LIB = os.path.join(HERE, "libpsb.so")
NVCC = os.environ.get("PSB_NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC,-O3", "-ccbin", "g++", "--expt-relaxed-constexpr"]


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _deps():
    out = sources() + [os.path.join(INCLUDE, "psb.h")]
    out += [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    return out


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build_library(verbose: bool = False, ptxas_info: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    deps = _deps()
    headers = [d for d in deps if not d.endswith(".cu")]
    jobs = []
    for src in sources():
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        if _stale(obj, [src] + headers):
            cmd = [NVCC] + FLAGS + (["-Xptxas", "-v"] if ptxas_info else []) + ["-I", INCLUDE, "-c", src, "-o", obj]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed: %s\n%s\n%s" % (" ".join(cmd), r.stdout, r.stderr))
        if verbose or ptxas_info:
            sys.stderr.write(r.stdout + r.stderr)

    with ThreadPoolExecutor(max_workers=8) as ex:
        list(ex.map(run, jobs))
    objs = [os.path.join(OBJ, os.path.basename(s)[:-3] + ".o") for s in sources()]
    if jobs or _stale(LIB, objs):
        run([NVCC, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-ccbin", "g++"])
    return LIB


def build_nvtx_variant() -> str:
    """libpsb_nvtx.so: the same library with NVTX ranges around the stages (-DPSB_USE_NVTX=1).  Only the session layer holds
    ranges, so only that file is compiled again; load it with api.load(path)."""
    build_library()
    obj_dir = os.path.join(HERE, "_obj_nvtx")
    os.makedirs(obj_dir, exist_ok=True)
    src = os.path.join(CSRC, "session.cu")
    obj = os.path.join(obj_dir, "session.o")
    out = os.path.join(HERE, "libpsb_nvtx.so")
    headers = [d for d in _deps() if not d.endswith(".cu")]
    if _stale(obj, [src] + headers):
        r = subprocess.run([NVCC] + FLAGS + ["-DPSB_USE_NVTX=1", "-I", INCLUDE, "-c", src, "-o", obj], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed (nvtx variant):\n%s\n%s" % (r.stdout, r.stderr))
    objs = [obj if os.path.basename(s_) == "session.cu" else os.path.join(OBJ, os.path.basename(s_)[:-3] + ".o") for s_ in sources()]
    if _stale(out, objs):
        r = subprocess.run([NVCC, "-shared", "-o", out] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-ccbin", "g++", "-ldl"],
                           capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed (nvtx variant):\n%s\n%s" % (r.stdout, r.stderr))
    return out


def ensure_built() -> str:
    if _stale(LIB, _deps()):
        build_library()
    return LIB


if __name__ == "__main__":
    print(build_library(verbose=True, ptxas_info="--ptxas" in sys.argv))
    if "--nvtx" in sys.argv:
        print(build_nvtx_variant())
