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
    """One nvcc -c per source file, in parallel, then one link step."""
    if not force and up_to_date():
        return LIB
    from concurrent.futures import ThreadPoolExecutor
    objdir = PKG / "build"
    objdir.mkdir(exist_ok=True)
    flags = [f for f in NVCC_FLAGS if f != "-shared"]
    if verbose:
        flags += ["-Xptxas", "-v"]

    def compile_one(src: str):
        obj = objdir / (Path(src).stem + ".o")
        res = subprocess.run([nvcc(), *flags, "-c", str(CSRC / src), "-o", str(obj)], cwd=str(CSRC),
                             capture_output=True, text=True)
        return src, obj, res

    with ThreadPoolExecutor(max_workers=min(len(SOURCES), os.cpu_count() or 4)) as pool:
        results = list(pool.map(compile_one, SOURCES))
    failed = False
    for src, _, res in results:
        if verbose or res.returncode != 0:
            sys.stderr.write(f"---- {src}\n" + res.stdout + res.stderr)
        failed = failed or res.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed building libw4a16_b200.so")
    link = subprocess.run([nvcc(), *NVCC_FLAGS, "-o", str(LIB), *[str(o) for _, o, _ in results]],
                          capture_output=True, text=True)
    if link.returncode != 0:
        sys.stderr.write(link.stdout + link.stderr)
        raise RuntimeError("linking libw4a16_b200.so failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
