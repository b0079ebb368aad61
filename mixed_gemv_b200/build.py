"""Builds libmixed_gemv_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python -m mixed_gemv_b200.build [--force] [--verbose] [--out PATH] [-DNAME[=VALUE] ...]

--out and -D build another copy of the library elsewhere (a tuning build with -DMGV_TUNING reads
MGV_* environment variables; the library the package loads never does).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG_DIR)
CSRC = os.path.join(PKG_DIR, "csrc")
INCLUDE = os.path.join(ROOT, "include")
LIB_PATH = os.path.join(PKG_DIR, "libmixed_gemv_b200.so")
SOURCES = ["mgv_abi.cu", "mgv_preprocess.cu", "mgv_gemv.cu", "mgv_gemv_fast.cu", "mgv_gemv_tile.cu", "mgv_gemv_batch.cu", "mgv_exchange.cu"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC")


def sources():
    return [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = sources() + [os.path.join(CSRC, "mgv_common.cuh"), os.path.join(CSRC, "mgv_gemv_parts.cuh"),
                        os.path.join(INCLUDE, "mixed_gemv_b200.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, out: str | None = None, defines=()) -> str:
    custom = out is not None or bool(defines)
    out = out or LIB_PATH
    if not custom and not force and not is_stale():
        return LIB_PATH
    objs = []
    obj_dir = os.path.join(PKG_DIR, "build") if not custom else os.path.splitext(out)[0] + "_obj"
    os.makedirs(obj_dir, exist_ok=True)
    common = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-I", INCLUDE, "-I", CSRC] + list(defines)
    if verbose:
        common += ["-Xptxas", "-v"]
    procs = []
    for src in sources():
        obj = os.path.join(obj_dir, os.path.basename(src) + ".o")
        objs.append(obj)
        procs.append((src, subprocess.Popen(common + ["-c", src, "-o", obj], stdout=subprocess.PIPE,
                                            stderr=subprocess.STDOUT, text=True)))
    for src, p in procs:
        log, _ = p.communicate()
        if verbose or p.returncode:
            sys.stderr.write(log)
        if p.returncode:
            raise RuntimeError(f"nvcc failed on {src}")
    subprocess.run([_nvcc(), "-shared", "-o", out] + objs, check=True)
    return out


if __name__ == "__main__":
    _out = sys.argv[sys.argv.index("--out") + 1] if "--out" in sys.argv else None
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, out=_out,
                defines=[a for a in sys.argv[1:] if a.startswith("-D")]))
