"""Loads libw4a16_b200.so and declares its C ABI (include/w4a16_b200.h) for ctypes.

There is no fallback: if the shared library is missing or cannot be loaded, importing the
operators raises.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_int, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libw4a16_b200.so"


class QKVView(ctypes.Structure):
    """Mirror of w4a16_qkv_view / the reference's QKVProjectionView (include/kernels.cuh:23-27)."""
    _fields_ = [(n, c_void_p) for n in ("q_weight", "q_scale", "d_q", "k_weight", "k_scale", "d_k",
                                        "v_weight", "v_scale", "d_v")]


class LayerWeights(ctypes.Structure):
    """Mirror of w4a16_layer_weights."""
    _fields_ = [(n, c_void_p) for n in (
        "input_norm_gamma", "q_weight", "q_scale", "k_weight", "k_scale", "v_weight", "v_scale",
        "o_weight", "o_scale", "post_norm_gamma", "gate_up_weight", "gate_up_scale", "down_weight", "down_scale")]


class QwenBinHeader(ctypes.Structure):
    """Mirror of w4a16_qwenbin_header."""
    _fields_ = [(n, ctypes.c_uint32) for n in (
        "version", "hidden_size", "intermediate_size", "num_layers", "num_q_heads", "num_kv_heads", "head_dim",
        "vocab_size", "max_seq_len", "quant_type", "tie_word_embeddings")] + [
        ("rms_norm_eps", ctypes.c_float), ("rope_theta", ctypes.c_float), ("file_bytes", ctypes.c_uint64)]


class QwenBinGlobals(ctypes.Structure):
    """Mirror of w4a16_qwenbin_globals."""
    _fields_ = [(n, c_void_p) for n in ("embed_weight", "embed_scale", "final_norm_gamma", "lm_head_weight",
                                        "lm_head_scale")]


class QwenBinBiases(ctypes.Structure):
    """Mirror of w4a16_qwenbin_biases."""
    _fields_ = [(n, c_void_p) for n in ("q_bias", "k_bias", "v_bias")]


class SweepDesc(ctypes.Structure):
    """Mirror of w4a16_sweep_desc."""
    _fields_ = [("num_layers", c_int), ("hidden_size", c_int), ("intermediate_size", c_int),
                ("num_q_heads", c_int), ("num_kv_heads", c_int), ("head_dim", c_int),
                ("layers", POINTER(LayerWeights)), ("workspace", c_void_p), ("flags", c_int)]


# name -> argtypes; every function returns int except those in RESTYPES
SIGNATURES = {
    "w4a16_version": [],
    "w4a16_init": [],
    "w4a16_set_option": [c_int, c_int],
    "w4a16_get_option": [c_int],
    "w4a16_quantize_fp16_to_q8_1": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    "w4a16_rmsnorm_q8_1": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int],
    "w4a16_gemv_w4a16": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "w4a16_quantize_attn_heads_f32_to_q8_1": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "w4a16_gemv_attn_heads_f32_w4a16": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "w4a16_gemv_w4a16_static_scratch": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "w4a16_gemv_w4a8": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                        c_void_p],
    "w4a16_gemv_w4a8_peers": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, POINTER(c_void_p), c_int,
                              c_int, c_int, c_void_p],
    "w4a16_gemv_w4a8_peers_signal": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, POINTER(c_void_p),
                                     POINTER(c_void_p), c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "w4a16_gather_after_signals": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    "w4a16_qwenbin_parse": [c_void_p, ctypes.c_uint64, POINTER(QwenBinHeader)],
    "w4a16_qwenbin_tensors": [c_void_p, ctypes.c_uint64, c_void_p, POINTER(LayerWeights), c_int, POINTER(QwenBinGlobals),
                              POINTER(QwenBinBiases)],
    "w4a16_embed_lookup_w4a16": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int],
    "w4a16_sample_and_advance": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int],
    "w4a16_sample_slots": [c_int],
    "w4a16_gemv_w4a8_sample_candidates": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                          c_void_p, c_int, c_int, c_int, c_void_p],
    "w4a16_gemv_w4a8_sample_candidates_peers": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                POINTER(c_void_p), POINTER(c_void_p), c_int, c_void_p, c_int, c_int,
                                                c_int, c_void_p],
    "w4a16_gemv_w4a8_sample_candidates_signal": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                 POINTER(c_void_p), POINTER(c_void_p), POINTER(c_void_p), c_int, c_void_p,
                                                 c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p],
    "w4a16_sample_finish_after_signals": [c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                          c_void_p, c_void_p],
    "w4a16_gemv_w4a8_sample_one_launch": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                          c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "w4a16_sample_finish": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p],
    "w4a16_gemv_w4a8_sample_and_advance": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                           c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "w4a16_gemv_qkv_w4a8": [POINTER(QKVView), c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int],
    "w4a16_gemv_dual_gate_up_swiglu_w4a16": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "w4a16_gemv_dual_gate_up_swiglu_w4a8": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                            c_int, c_void_p],
    "w4a16_gemv_rmsnorm_w4a16": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "w4a16_gemv_qkv_rmsnorm_w4a16": [POINTER(QKVView), c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int],
    "w4a16_gemv_dual_gate_up_swiglu_rmsnorm_w4a16": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                                     c_void_p],
    "w4a16_gemv_dual_gate_up_swiglu_rmsnorm_w4a16_q8_1": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                          c_void_p, c_void_p, c_int, c_int, c_void_p],
    "w4a16_gemm_prefill_w4a16": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p,
                                 c_int],
    "w4a16_gemm_prefill_w4a16_block": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, POINTER(c_void_p), c_int,
                                       c_int, c_int, c_int, c_void_p],
    "w4a16_gemm_prefill_qkv_w4a16": [POINTER(QKVView), c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                                     c_int],
    "w4a16_gemm_prefill_dual_gate_up_swiglu_w4a16": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                                     c_int, c_int],
    "w4a16_gemv_group_dots": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "w4a16_debug_counter": [c_int, POINTER(ctypes.c_uint)],
    "w4a16_sweep_workspace_bytes": [c_int, c_int, c_int, c_int, c_int],
    "w4a16_sweep_create": [POINTER(SweepDesc), c_void_p, POINTER(c_void_p)],
    "w4a16_sweep_destroy": [c_void_p],
    "w4a16_sweep_launches": [c_void_p],
    "w4a16_sweep_run_device": [c_void_p, c_void_p, c_void_p, c_void_p],
    "w4a16_sweep_run_host": [c_void_p, c_void_p, c_void_p, c_void_p],
    "w4a16_sweep_buffer": [c_void_p, c_int],
    "w4a16_sweep_status": [c_void_p, POINTER(c_int)],
}
RESTYPES = {"w4a16_sweep_workspace_bytes": ctypes.c_int64, "w4a16_sweep_buffer": c_void_p}

_lib = None


def load() -> ctypes.CDLL:
    """Returns the loaded library; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m qwen_engine_b200.build` "
            "(there is no non-CUDA fallback)")
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, argtypes in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.argtypes = argtypes
        fn.restype = RESTYPES.get(name, c_int)
    lib.w4a16_status_string.argtypes = [c_int]
    lib.w4a16_status_string.restype = c_char_p
    _lib = lib
    return lib


class W4A16Error(RuntimeError):
    """A launcher returned a nonzero status (the reference throws std::runtime_error there)."""

    def __init__(self, fn: str, status: int):
        msg = load().w4a16_status_string(status).decode()
        super().__init__(f"{fn}: status {status}: {msg}")
        self.status = status


def check(fn: str, status: int) -> None:
    if status != 0:
        raise W4A16Error(fn, status)
