"""Build the CUDA library in-tree:  python -m culsh_b200.build

Compiles culsh_b200/csrc/culsh_b200.cu for sm_100a into culsh_b200/libculsh_b200.so
(nvcc cross-compiles without a GPU).  The library exposes only the C ABI declared in
include/culsh_b200.h and links cudart + curand + the CUDA driver stub (for the tensor-map
encoder used by the TMA loads).
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "csrc", "culsh_b200.cu")
OUT = os.path.join(HERE, "libculsh_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",
]


def _sources():
    d = os.path.join(HERE, "csrc")
    inc = os.path.join(os.path.dirname(HERE), "include")
    out = [os.path.join(d, f) for f in sorted(os.listdir(d))]
    out += [os.path.join(inc, f) for f in sorted(os.listdir(inc))]
    return out


def is_stale() -> bool:
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    return any(os.path.getmtime(s) > t for s in _sources())


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not is_stale():
        return OUT
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: cannot build libculsh_b200.so")
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + [SRC, "-o", OUT, "-lcurand"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    if verbose:
        print(res.stderr)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
