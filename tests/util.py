"""Shared helpers of the test-suite: upload/download, error metrics, the reference-kernel
loader.  The oracle (oracle/) and the rebuilt reference kernels (oracle/_ref/) are used
here as checkers only."""
from __future__ import annotations

import ctypes
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
REF_DIR = ROOT / "oracle" / "_ref"


def cuda_available() -> bool:
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def to_dev(a: np.ndarray):
    """numpy -> CUDA tensor with the same bits (uint32 travels as int32, as torch lacks full uint32 support)."""
    import torch
    if a.dtype == np.uint32:
        return torch.from_numpy(a.view(np.int32).copy()).cuda()
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16).copy()).cuda()
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def to_np(t, dtype=None) -> np.ndarray:
    a = t.detach().cpu().numpy()
    return a.view(dtype) if dtype is not None else a


def fp16_ulp(ref: np.ndarray) -> np.ndarray:
    """Spacing of fp16 at |ref| (normal range; subnormal spacing below 2^-14)."""
    a = np.abs(np.asarray(ref, dtype=np.float64))
    e = np.floor(np.log2(np.maximum(a, 2.0 ** -14)))
    return 2.0 ** (e - 10)


def error_report(y: np.ndarray, ref64: np.ndarray, magnitude: np.ndarray | None = None) -> dict:
    """y: fp16 result, ref64: exact value in double.  magnitude (optional): size of the operands the
    result was rounded at -- for an epilogue that rounds the accumulator to fp16 BEFORE adding the
    residual (the prefill GEMM), errors are judged at max(|ref|, |accumulator|), not at a sum that
    may have cancelled.
    rel: |y - ref| / max(|ref|, 1e-2 * rms(ref))  -- relative error with a floor, so outputs that
    cancel to ~0 are judged against the vector's scale;  ulp: error in fp16 ulps at ref."""
    y64 = np.asarray(y, dtype=np.float64).reshape(-1)
    r = np.asarray(ref64, dtype=np.float64).reshape(-1)
    rms = float(np.sqrt(np.mean(r * r))) or 1.0
    err = np.abs(y64 - r)
    size = np.abs(r)
    if magnitude is not None:
        size = np.maximum(size, np.abs(np.asarray(magnitude, dtype=np.float64).reshape(-1)))
    rel = err / np.maximum(size, 1e-2 * rms)
    # ulp measured at max(|ref|, 1e-3 rms): fp32 accumulation noise is absolute, so outputs that
    # cancel to nearly zero are not held to the spacing of fp16 at their own tiny magnitude
    ulp = err / fp16_ulp(np.maximum(size, 1e-3 * rms))
    return {"max_rel": float(rel.max()), "median_ulp": float(np.median(ulp)), "max_ulp": float(ulp.max()),
            "max_abs": float(err.max()), "finite": bool(np.isfinite(y64).all())}


def assert_fp16_close(y, ref64, max_rel=1e-2, median_ulp=2.0, what="", magnitude=None):
    """The stated tolerance of the path: max relative error <= 1e-2, median <= 2 fp16 ulp."""
    rep = error_report(y, ref64, magnitude)
    assert rep["finite"], f"{what}: non-finite output"
    assert rep["max_rel"] <= max_rel, f"{what}: {rep}"
    assert rep["median_ulp"] <= median_ulp, f"{what}: {rep}"
    return rep


from oracle import RefKernels  # noqa: E402,F401  (the loader of the rebuilt reference kernels lives with the checkers)


def stream_ptr() -> ctypes.c_void_p:
    import torch
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
