"""Builds tests/cpp/adaptor_driver.cpp (the reference-style driver over the C++ face of the library)."""
import os
import shutil
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "adaptor_driver.cpp")


def cuda_home() -> str:
    for cand in (os.environ.get("CUDA_HOME"), "/usr/local/cuda"):
        if cand and os.path.exists(os.path.join(cand, "include", "cuda_runtime.h")):
            return cand
    return ""


def build_driver(out_dir: str) -> str:
    """g++ the driver against the in-tree library and the CUDA runtime; returns the binary's path."""
    from mixed_gemv_b200 import build
    lib = build.build()
    cxx, cuda = shutil.which("g++"), cuda_home()
    if not cxx or not cuda:
        raise RuntimeError("needs g++ and the CUDA toolkit headers")
    exe = os.path.join(out_dir, "adaptor_driver")
    lib_dir = os.path.dirname(lib)
    cmd = [cxx, "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(cuda, "include"), SRC, "-o", exe,
           "-L", lib_dir, "-lmixed_gemv_b200", "-L", os.path.join(cuda, "lib64"), "-lcudart",
           f"-Wl,-rpath,{lib_dir}", f"-Wl,-rpath,{os.path.join(cuda, 'lib64')}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode:
        raise RuntimeError("driver build failed:\n" + r.stderr[-3000:])
    return exe
