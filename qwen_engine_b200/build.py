"""Builds libw4a16_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python -m qwen_engine_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libw4a16_b200.so"
SOURCES = ["c_abi.cu", "q8_1_quantize.cu", "gemv_decode.cu", "gemm_prefill.cu", "gemm_tc.cu", "decode_sweep.cu", "sweep_persistent.cu",
           "gemv_static_scratch.cu", "sampling.cu", "embed_lookup.cu", "qwenbin.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++20", "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "-shared",
]


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found: the CUDA library cannot be built")
    return exe


def _inputs():
    files = [CSRC / s for s in SOURCES]
    files += sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.hpp"))
    files += [PKG.parent / "include" / "w4a16_b200.h"]
    return files


def up_to_date() -> bool:
    if not LIB.exists():
        return False
    t = LIB.stat().st_mtime
    return all(f.stat().st_mtime <= t for f in _inputs())


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and up_to_date():
        return LIB
    cmd = [nvcc(), *NVCC_FLAGS]
    if os.environ.get("W4A16_TC_PROFILE"):
        cmd += ["-DW4A16_TC_PROFILE"]
    if os.environ.get("W4A16_GEMV_PROFILE"):
        cmd += ["-DW4A16_GEMV_PROFILE"]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", str(LIB), *[str(CSRC / s) for s in SOURCES]]
    res = subprocess.run(cmd, cwd=str(CSRC), capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libw4a16_b200.so")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
