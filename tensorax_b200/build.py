"""In-tree build of the CUDA library: ``python -m tensorax_b200.build``.

nvcc cross-compiles for sm_100a without a GPU.  The output,
``tensorax_b200/csrc/libtensorax_b200.so``, is what ``tensorax_b200._lib`` loads.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(CSRC, "libtensorax_b200.so")
SOURCES = ["sdpa_api.cu"]
HEADERS = ["ptx.cuh", "sdpa_simt.cuh", "sdpa_tc.cuh", "sdpa_tc_pair.cuh", "sdpa_tc_x3.cuh", "bounded_wait.h", "sdpa_bwd.cuh", "linear_simt.cuh", "linear_tc.cuh", os.path.join("..", "..", "include", "tensorax_b200.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--compiler-options", "-fPIC,-fvisibility=hidden", "-shared",
]


def _nvcc() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.isfile(cand) else (shutil.which("nvcc") or "nvcc")


def up_to_date() -> bool:
    if not os.path.isfile(OUT):
        return False
    t = os.path.getmtime(OUT)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS]
    return all(os.path.getmtime(d) <= t for d in deps if os.path.isfile(d))


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and up_to_date():
        return OUT
    cmd = [_nvcc(), *NVCC_FLAGS]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", OUT, *[os.path.join(CSRC, s) for s in SOURCES]]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose:
        sys.stderr.write(proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + proc.stderr[-4000:])
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
