"""Build libq3mk.so (the C-ABI library) for sm_100a with nvcc.  No GPU is needed to build.

    python qwen3-megakernel_b200/build.py [--force] [--verbose]

The library lands next to the Python package (qwen3mk/libq3mk.so) so that it travels with the tree.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OUT = HERE / "qwen3mk" / "libq3mk.so"
STAMP = HERE / "qwen3mk" / ".libq3mk.stamp"
SOURCES = ["q3_api.cu", "q3_layered.cu", "q3_persist.cu", "q3_static.cu", "q3_gemm_tc.cu", "q3_prefill_attn_tc.cu", "q3_sample.cu", "q3_layer_tc.cu", "q3_attn_mma.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
              "-Xcompiler", "-fPIC", "-shared", "--fmad=true"]


def nvcc() -> str:
    for c in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if c and (os.path.sep not in c or os.path.exists(c)):
            return c
    raise RuntimeError("nvcc not found")


def source_digest() -> str:
    h = hashlib.sha256()
    for f in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) +
                    [HERE.parent / "include" / "q3mk.h", Path(__file__)]):
        h.update(f.name.encode())
        h.update(f.read_bytes())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False) -> Path:
    dig = source_digest()
    if not force and OUT.exists() and STAMP.exists() and STAMP.read_text() == dig:
        return OUT
    cmd = [nvcc(), *NVCC_FLAGS, "-I", str(HERE.parent / "include"), "-o", str(OUT)] + [str(CSRC / s) for s in SOURCES]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
        print(" ".join(cmd))
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed:\n{r.stdout}\n{r.stderr}")
    if verbose:
        print(r.stderr)
    STAMP.write_text(dig)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
