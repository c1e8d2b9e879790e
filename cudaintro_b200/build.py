"""Builds ``libb200gemm.so`` in-tree with nvcc for sm_100a.

    python -m cudaintro_b200.build            # build if sources are newer than the library
    python -m cudaintro_b200.build --force
    python -m cudaintro_b200.build --stamps   # measurement build: libb200gemm_stamps.so, whose skinny kernel
                                              # records a per-k-block timeline and whose large tensor-core
                                              # kernel accounts for its waits (see cudaintro_b200/timeline.py)

The library is a plain C-ABI shared object (see ``include/b200gemm.h``); nothing in it links
against Python or torch.  Objects are compiled in parallel, one nvcc per source file.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
ROOT = os.path.dirname(PKG)
LIB = os.path.join(PKG, "libb200gemm.so")
OBJ_DIR = os.path.join(PKG, "build")

SOURCES = ["api.cu", "gemm_umma.cu", "gemm_skinny.cu", "gemm_f32.cu", "simt_misc.cu", "legacy_suite.cu"]
HEADERS = ["internal.h", "ptx_sm100.cuh", os.path.join(ROOT, "include", "b200gemm.h"),
           os.path.join(ROOT, "include", "gemm_common.h")]

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC",
    "-I", os.path.join(ROOT, "include"),
]


def _nvcc() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def _mtime(path: str) -> float:
    return os.path.getmtime(path) if os.path.exists(path) else 0.0


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    newest = max(_mtime(os.path.join(CSRC, s)) for s in SOURCES)
    newest = max([newest] + [_mtime(h if os.path.isabs(h) else os.path.join(CSRC, h)) for h in HEADERS])
    return newest > _mtime(LIB)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if needed and return its path."""
    if not force and not needs_build():
        return LIB
    os.makedirs(OBJ_DIR, exist_ok=True)
    hdr_time = max(_mtime(h if os.path.isabs(h) else os.path.join(CSRC, h)) for h in HEADERS)

    def compile_one(src: str) -> str:
        obj = os.path.join(OBJ_DIR, src.replace(".cu", ".o"))
        spath = os.path.join(CSRC, src)
        if not force and _mtime(obj) > max(_mtime(spath), hdr_time):
            return obj
        cmd = [_nvcc(), *NVCC_FLAGS, "-c", spath, "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{res.stdout}\n{res.stderr}")
        if verbose:
            sys.stderr.write(res.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(SOURCES))) as pool:
        objs = list(pool.map(compile_one, SOURCES))
    link = [_nvcc(), "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a",
            "-cudart", "shared"]
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB


STAMPS_LIB = os.path.join(PKG, "libb200gemm_stamps.so")


def build_stamps() -> str:
    """The same sources with -DB200_SKINNY_STAMPS, into a library of its own (never loaded by the package)."""
    obj_dir = os.path.join(PKG, "build", "stamps")
    os.makedirs(obj_dir, exist_ok=True)

    def compile_one(src: str) -> str:
        obj = os.path.join(obj_dir, src.replace(".cu", ".o"))
        cmd = [_nvcc(), *NVCC_FLAGS, "-DB200_SKINNY_STAMPS", "-c", os.path.join(CSRC, src), "-o", obj]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{res.stdout}\n{res.stderr}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(SOURCES))) as pool:
        objs = list(pool.map(compile_one, SOURCES))
    res = subprocess.run([_nvcc(), "-shared", "-o", STAMPS_LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a",
                          "-cudart", "shared"], capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return STAMPS_LIB


if __name__ == "__main__":
    if "--stamps" in sys.argv:
        print(build_stamps())
    else:
        print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
