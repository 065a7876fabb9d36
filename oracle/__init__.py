"""ctypes front end of the CPU oracle (oracle/w4a16_oracle.c).  TEST INFRASTRUCTURE ONLY.

Only the tests, the smoke check and the benchmark's cpu_baseline / reference arm import
this module; the product package never does.  fp16 arrays are numpy float16 and cross
into C as their raw bits.

The shared object is built per host ISA (the file name carries it), so a library built
on one machine is never loaded on a CPU that lacks its instructions; a missing one is
compiled on first use with gcc.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
GROUP = 128

ROUND_HALF_EVEN = 0  # device __float2int_rn; canonical
ROUND_HALF_AWAY = 1  # std::round, the reference test's CPU flavour


def _host_isa() -> str:
    try:
        flags = set()
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    flags = set(line.split(":", 1)[1].split())
                    break
        if {"avx2", "fma", "f16c"} <= flags:
            return "x86-64-v3"
    except OSError:
        pass
    return "generic"


def lib_path() -> Path:
    return _HERE / "_build" / f"libw4a16_oracle.{_host_isa()}.so"


def build(force: bool = False) -> Path:
    """Compile the C oracle for this host (gcc), unless an up-to-date build exists."""
    out = lib_path()
    src = _HERE / "w4a16_oracle.c"
    if force or not out.exists() or out.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE), f"ISA={_host_isa()}"], check=True,
                       stdout=subprocess.DEVNULL)
    return out


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(str(build()))
        _lib.orc_rmsnorm.restype = ctypes.c_float
        _lib.orc_sample.restype = ctypes.c_int32
        _lib.orc_philox_first.restype = ctypes.c_uint32
    return _lib


def default_threads() -> int:
    return max(1, len(os.sched_getaffinity(0)))


def _p(a: np.ndarray | None):
    if a is None:
        return ctypes.c_void_p(0)
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be contiguous"
    return ctypes.c_void_p(a.ctypes.data)


def _i64(v):
    return ctypes.c_int64(int(v))


def pack_nibbles(q: np.ndarray) -> np.ndarray:
    """q uint8 [N][K] in 0..15 -> packed uint32 [N][K/8] (reference nibble order)."""
    q = np.ascontiguousarray(q, dtype=np.uint8)
    N, K = q.shape
    out = np.empty((N, K // 8), dtype=np.uint32)
    lib().orc_pack_nibbles(_p(q), _p(out), _i64(N), ctypes.c_int(K))
    return out


def unpack_nibbles(packed: np.ndarray) -> np.ndarray:
    packed = np.ascontiguousarray(packed, dtype=np.uint32)
    N, W = packed.shape
    out = np.empty((N, W * 8), dtype=np.uint8)
    lib().orc_unpack_nibbles(_p(packed), _p(out), _i64(N), ctypes.c_int(W * 8))
    return out


def quantize_weights(w: np.ndarray):
    """fp32 [N][K] -> (packed uint32 [N][K/8], scales float16 [N][K/128])."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    N, K = w.shape
    packed = np.empty((N, K // 8), dtype=np.uint32)
    scales = np.empty((N, K // GROUP), dtype=np.float16)
    lib().orc_quantize_weights(_p(w), _i64(N), ctypes.c_int(K), _p(packed), _p(scales))
    return packed, scales


def quantize_q8_1(x: np.ndarray, round_mode: int = ROUND_HALF_EVEN):
    """float16 [n] -> (q8 int8 [n], scale float32 [n/128], sum8 int32 [n/8])."""
    x = np.ascontiguousarray(x, dtype=np.float16).reshape(-1)
    n = x.size
    assert n % GROUP == 0
    q8 = np.empty(n, dtype=np.int8)
    scale = np.empty(n // GROUP, dtype=np.float32)
    sum8 = np.empty(n // 8, dtype=np.int32)
    lib().orc_quantize_q8_1(_p(x), _i64(n), _p(q8), _p(scale), _p(sum8), ctypes.c_int(round_mode))
    return q8, scale, sum8


def quantize_heads_f32(acc: np.ndarray):
    """acc: fp32 [heads][head_dim] -> (fp16 attn_out, q8, scale[heads], sum8), the flash-decode epilogue's Q8_1."""
    acc = np.ascontiguousarray(acc, dtype=np.float32)
    heads, hd = acc.shape
    out16 = np.empty((heads, hd), dtype=np.float16)
    q8 = np.empty(heads * hd, dtype=np.int8)
    scale = np.empty(heads, dtype=np.float32)
    sum8 = np.empty(heads * hd // 8, dtype=np.int32)
    lib().orc_quantize_heads_f32(_p(acc), heads, hd, _p(out16), _p(q8), _p(scale), _p(sum8))
    return out16, q8, scale, sum8


def group_dots(packed: np.ndarray, q8: np.ndarray, threads: int | None = None) -> np.ndarray:
    """int32 [N][K/128]: the per-group integer dots of (q-8) with the Q8_1 bytes."""
    packed = np.ascontiguousarray(packed, dtype=np.uint32)
    q8 = np.ascontiguousarray(q8, dtype=np.int8)
    N, W = packed.shape
    K = W * 8
    assert q8.size == K
    D = np.empty((N, K // GROUP), dtype=np.int32)
    lib().orc_group_dots(_p(packed), _p(q8), _i64(N), ctypes.c_int(K), _p(D),
                         ctypes.c_int(threads or default_threads()))
    return D


def _gemv_common(fn, packed, scales, xarg, xscale, residual, swiglu, threads, want64=True):
    packed = np.ascontiguousarray(packed, dtype=np.uint32)
    scales = np.ascontiguousarray(scales, dtype=np.float16)
    N, W = packed.shape
    K = W * 8
    n_out = N // 2 if swiglu else N
    y64 = np.empty(n_out, dtype=np.float64) if want64 else None
    y16 = np.empty(n_out, dtype=np.float16)
    if residual is not None:
        residual = np.ascontiguousarray(residual, dtype=np.float16)
    args = [_p(packed), _p(scales)] + xarg + [_p(residual), _i64(N), ctypes.c_int(K),
                                              ctypes.c_int(1 if swiglu else 0), _p(y64), _p(y16),
                                              ctypes.c_int(threads or default_threads())]
    fn(*args)
    return y64, y16


def gemv_q8(packed, scales, q8, xscale, residual=None, swiglu=False, threads=None, want64=True):
    """W4A8 golden on Q8_1 activations: (double [n_out], float16 [n_out])."""
    q8 = np.ascontiguousarray(q8, dtype=np.int8)
    xscale = np.ascontiguousarray(xscale, dtype=np.float32)
    return _gemv_common(lib().orc_gemv_q8, packed, scales, [_p(q8), _p(xscale)], None, residual,
                        swiglu, threads, want64)


def gemv_dequant(packed, scales, x_f32, residual=None, swiglu=False, threads=None):
    """fp32 dequantise-then-matmul golden on fp32 activations."""
    x_f32 = np.ascontiguousarray(x_f32, dtype=np.float32)
    return _gemv_common(lib().orc_gemv_dequant, packed, scales, [_p(x_f32)], None, residual,
                        swiglu, threads)


def gemm_prefill(packed, scales, x, m_idx, n_idx, residual=None, swiglu=False, threads=None):
    """Prefill golden on the listed token rows / output columns: (double, float16) [nm][nn]."""
    packed = np.ascontiguousarray(packed, dtype=np.uint32)
    scales = np.ascontiguousarray(scales, dtype=np.float16)
    x = np.ascontiguousarray(x, dtype=np.float16)
    m_idx = np.ascontiguousarray(m_idx, dtype=np.int32)
    n_idx = np.ascontiguousarray(n_idx, dtype=np.int32)
    K = packed.shape[1] * 8
    assert x.shape[1] == K
    ldr = 0
    if residual is not None:
        residual = np.ascontiguousarray(residual, dtype=np.float16)
        ldr = residual.shape[1]
    out64 = np.empty((m_idx.size, n_idx.size), dtype=np.float64)
    out16 = np.empty((m_idx.size, n_idx.size), dtype=np.float16)
    lib().orc_gemm_prefill(_p(packed), _p(scales), _p(x), _p(residual), _i64(ldr), ctypes.c_int(K),
                           ctypes.c_int(1 if swiglu else 0), _p(m_idx), ctypes.c_int(m_idx.size),
                           _p(n_idx), ctypes.c_int(n_idx.size), _p(out64), _p(out16),
                           ctypes.c_int(threads or default_threads()))
    return out64, out16


def rmsnorm(x, gamma, eps=1e-6, inv_rms_override=0.0):
    """RMSNorm with the reference's fp16 roundings: (float16 [n], inv_rms float)."""
    x = np.ascontiguousarray(x, dtype=np.float16).reshape(-1)
    gamma = np.ascontiguousarray(gamma, dtype=np.float16).reshape(-1)
    y = np.empty_like(x)
    inv = lib().orc_rmsnorm(_p(x), _p(gamma), ctypes.c_int(x.size), ctypes.c_float(eps),
                            ctypes.c_float(inv_rms_override), _p(y))
    return y, float(inv)


def philox_first(seed, c0, c1):
    """First output word of Philox-4x32-10 for counter (c0, c1, 0, 0) and the 64-bit key `seed`."""
    return int(lib().orc_philox_first(ctypes.c_uint64(seed), ctypes.c_uint32(c0), ctypes.c_uint32(c1)))


def sample(logits, temperature=0.0, seed=0, seq_pos=0, index_offset=0):
    """Greedy / Gumbel-max token selection over fp16 logits: (token, best score, scores float32 [n])."""
    logits = np.ascontiguousarray(logits, dtype=np.float16).reshape(-1)
    scores = np.empty(logits.size, dtype=np.float32)
    best = ctypes.c_float(0.0)
    tok = lib().orc_sample(_p(logits), ctypes.c_int(logits.size), ctypes.c_float(temperature),
                           ctypes.c_uint64(seed), ctypes.c_uint32(seq_pos), ctypes.c_int32(index_offset),
                           ctypes.byref(best), _p(scores))
    return int(tok), float(best.value), scores


def decode_sweep(layers, h0, threads=None, collect=False):
    """CPU restatement of the decode projection sweep (the chain the library's DecodeSweep runs;
    reference order of launches: src/engine.cu:361-451 with the attention output replaced by the
    q projection).  layers: list of dicts of numpy arrays -- 'input_norm', 'post_norm' fp16 gamma,
    'q','k','v','o','gate_up','down' -> (packed, scales).  Returns the final hidden state fp16
    (and, with collect=True, every intermediate per layer)."""
    h = np.ascontiguousarray(h0, dtype=np.float16).copy()
    trace = []
    for L in layers:
        xn, _ = rmsnorm(h, L["input_norm"])
        q8, xs, _ = quantize_q8_1(xn)
        q = gemv_q8(*L["q"], q8, xs, threads=threads, want64=False)[1]
        k = gemv_q8(*L["k"], q8, xs, threads=threads, want64=False)[1]
        v = gemv_q8(*L["v"], q8, xs, threads=threads, want64=False)[1]
        a8, as_, _ = quantize_q8_1(q)
        h_attn = gemv_q8(*L["o"], a8, as_, residual=h, threads=threads, want64=False)[1]
        xn2, _ = rmsnorm(h_attn, L["post_norm"])
        p8, ps, _ = quantize_q8_1(xn2)
        mlp = gemv_q8(*L["gate_up"], p8, ps, swiglu=True, threads=threads, want64=False)[1]
        m8, ms, _ = quantize_q8_1(mlp)
        h_new = gemv_q8(*L["down"], m8, ms, residual=h_attn, threads=threads, want64=False)[1]
        if collect:
            trace.append({"h_in": h, "q": q, "k": k, "v": v, "h_attn": h_attn, "mlp": mlp, "h_out": h_new})
        h = h_new
    return (h, trace) if collect else h


class RefKernels:
    """The reference's CUDA kernels rebuilt for sm_100a (oracle/Makefile `ref`), if present."""

    class QKVPod(ctypes.Structure):
        _fields_ = [(n, ctypes.c_void_p) for n in ("q_weight", "q_scale", "d_q", "k_weight", "k_scale", "d_k",
                                                   "v_weight", "v_scale", "d_v")]

    def __init__(self, flavour: str):
        path = _HERE / "_ref" / f"libqwen_ref_{flavour}.so"
        self.lib = ctypes.CDLL(str(path))
        self.flavour = flavour

    @staticmethod
    def available(flavour: str = "ieee") -> bool:
        return (_HERE / "_ref" / f"libqwen_ref_{flavour}.so").exists()

    def call(self, name: str, *args):
        fn = getattr(self.lib, name)
        fn.restype = ctypes.c_int
        conv = []
        for a in args:
            if a is None:
                conv.append(ctypes.c_void_p(0))
            elif isinstance(a, ctypes.c_void_p):
                conv.append(a)
            elif isinstance(a, int):
                conv.append(ctypes.c_int(a))
            elif isinstance(a, ctypes.Structure):
                conv.append(ctypes.byref(a))
            else:  # torch tensor
                conv.append(ctypes.c_void_p(a.data_ptr()))
        st = fn(*conv)
        assert st == 0, f"{name} ({self.flavour}) failed with {st}"
