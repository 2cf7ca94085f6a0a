"""Builds libgpx.so (sm_100a) in-tree with nvcc.

    python -m gpreempt_b200.build [--force] [--verbose]

The library links the CUDA runtime statically and resolves the few driver entry points it
needs at run time, so it loads (and exports every symbol of include/gpx.h) on a machine
without a GPU or driver; compute entry points then fail with a clear error.
"""
from __future__ import annotations

import argparse
import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
OBJDIR = os.path.join(HERE, "lib", "obj")
LIB = os.path.join(LIBDIR, "libgpx.so")

NVCC_FLAGS = [
    "-std=c++17",
    "-O3",
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-Xcompiler",
    "-fPIC,-Wall,-Wno-unused-function,-fvisibility=default",
    "--expt-relaxed-constexpr",
    "-cudart",
    "static",
]


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; libgpx cannot be built")
    return exe


def sources() -> list[str]:
    return sorted(
        os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu")
    )


def _digest() -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    inc = os.path.join(HERE, "..", "include")
    files = [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC))]
    files += [os.path.join(inc, f) for f in sorted(os.listdir(inc))]
    for f in files:
        if os.path.isfile(f):
            h.update(f.encode())
            with open(f, "rb") as fp:
                h.update(fp.read())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False, defines: list[str] | None = None,
          out_dir: str | None = None) -> str:
    """Builds the library.  `defines` adds -D macros (development variants such as
    GPX_CGEMM_TIMING) and `out_dir` places that variant elsewhere; GPX_LIB selects it at load time."""
    libdir = os.path.abspath(out_dir) if out_dir else LIBDIR
    objdir = os.path.join(libdir, "obj")
    lib = os.path.join(libdir, "libgpx.so")
    dflags = [f"-D{d}" for d in (defines or [])]
    os.makedirs(objdir, exist_ok=True)
    stamp = os.path.join(libdir, "libgpx.digest")
    digest = _digest() + "|" + " ".join(dflags)
    if not force and os.path.exists(lib) and os.path.exists(stamp):
        with open(stamp) as fp:
            if fp.read().strip() == digest:
                return lib
    exe = nvcc()

    def compile_one(src: str) -> str:
        obj = os.path.join(objdir, os.path.basename(src)[:-3] + ".o")
        cmd = [exe, *NVCC_FLAGS, *dflags, "-c", src, "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
        if verbose:
            sys.stderr.write(res.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objs = list(pool.map(compile_one, sources()))
    cmd = [exe, "-shared", "-o", lib, *objs, "-cudart", "static",
           "-gencode", "arch=compute_100a,code=sm_100a", "-lpthread", "-ldl", "-lrt"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    with open(stamp, "w") as fp:
        fp.write(digest)
    return lib


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--define", action="append", default=[], help="extra -D macro (repeatable)")
    ap.add_argument("--out", default=None, help="directory for this variant (default: the package's lib/)")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose, defines=a.define, out_dir=a.out))
