"""Builds libfa_sm100.so in-tree with nvcc for sm_100a.

Run as ``python -m triton_flashattn_b200.build`` (add ``--force`` to rebuild
everything, ``--verbose`` for ptxas register/shared-memory statistics).  Objects
are rebuilt only when a source or header is newer than them.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
BUILD_DIR = os.path.join(PKG_DIR, "build")
LIB_PATH = os.path.join(PKG_DIR, "libfa_sm100.so")
INCLUDE_DIR = os.path.join(os.path.dirname(PKG_DIR), "include")

SOURCES = [
    "fa_api.cu",
    "fa_selftest.cu",
    "fa_fwd.cu",
    "fa_bwd_pre.cu",
    "fa_bwd_dkdv.cu",
    "fa_bwd_dq.cu",
    "fa_bwd_dkdv256.cu",
    "fa_bwd_static.cu",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; libfa_sm100.so cannot be built")
    return exe


def _headers() -> list[str]:
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hs += [os.path.join(INCLUDE_DIR, f) for f in os.listdir(INCLUDE_DIR) if f.endswith(".h")]
    return hs


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every translation unit and link the shared library; returns its path."""
    os.makedirs(BUILD_DIR, exist_ok=True)
    nvcc = _nvcc()
    headers = _headers()
    srcs = [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    flags = [
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-std=c++17", "-O3", "-lineinfo",
        "-Xcompiler", "-fPIC",
        "--expt-relaxed-constexpr",
        "-I", INCLUDE_DIR,
    ]
    if verbose:
        flags += ["-Xptxas", "-v"]

    def compile_one(src: str) -> tuple[str, bool, str]:
        obj = os.path.join(BUILD_DIR, src.replace(".cu", ".o"))
        path = os.path.join(CSRC, src)
        if not force and not _stale(obj, [path] + headers):
            return obj, False, ""
        cmd = [nvcc, *flags, "-c", path, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        return obj, True, r.stderr

    with ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 4)) as ex:
        results = list(ex.map(compile_one, srcs))
    objs = [o for o, _, _ in results]
    if verbose:
        for _, _, log in results:
            if log:
                print(log)
    if force or any(c for _, c, _ in results) or _stale(LIB_PATH, objs):
        cmd = [nvcc, "-shared", "-o", LIB_PATH, *objs, "-gencode", "arch=compute_100a,code=sm_100a",
               "-Xcompiler", "-fPIC"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB_PATH


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose))


if __name__ == "__main__":
    sys.exit(main())
