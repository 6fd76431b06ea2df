"""Build liba2a.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python gpu-mode-kernels_b200/build.py [--verbose]

nvcc cross-compiles without a GPU.  The library links the CUDA runtime
statically, so it depends on nothing but the driver at run time.
"""
import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG_DIR)
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "liba2a.so")
SOURCES = [os.path.join(CSRC, "a2a.cu"), os.path.join(CSRC, "a2a_noalloc.cu"), os.path.join(CSRC, "histogram.cu")]
HEADERS = [os.path.join(CSRC, "a2a_kernels.cuh"), os.path.join(CSRC, "a2a_pipe.cuh"), os.path.join(CSRC, "a2a_device.cuh"),
           os.path.join(ROOT, "include", "a2a.h")]


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found (set NVCC=/path/to/nvcc)")


def needs_build() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(f) > t for f in SOURCES + HEADERS + [os.path.abspath(__file__)])


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if it is missing or older than its sources; return its path."""
    if not force and not needs_build():
        return LIB_PATH
    cmd = [
        nvcc_path(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
        "-shared", "-Xcompiler", "-fPIC", "-cudart", "static",
        "-I", os.path.join(ROOT, "include"), "-I", CSRC,
        "-o", LIB_PATH, *SOURCES,
    ]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + res.stdout + res.stderr)
    if verbose:
        print(res.stdout + res.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force=True, verbose="--verbose" in sys.argv))
