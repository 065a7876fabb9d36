"""Python mirror of the reference's `qwen::launch_*` functions for the W4 projection path
(reference include/kernels.cuh), calling the C ABI of libw4a16_b200.so.

Names, argument order and meaning follow the reference; tensors are torch CUDA tensors
(torch is used for device memory and streams only).  Every call goes to the CUDA library;
there is no other implementation behind these functions, and a nonzero status raises
`W4A16Error` where the reference throws std::runtime_error.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from ._lib import LayerWeights, QKVView, SweepDesc, W4A16Error, check, load  # noqa: F401

__all__ = [
    "QKVProjectionView", "W4A16Error", "init", "set_pdl", "load", "set_option", "get_option", "OPT_PDL",
    "OPT_SIGNAL_WAIT_SPINS", "OPT_GEMV_FORM", "OPT_GEMM_MIN_TOKENS_TENSOR_CORE", "OPT_GEMM_FORM", "OPT_GEMM_MMA_MAX_TOKENS", "GEMV_FORM_AUTO",
    "GEMV_FORM_REGISTERS", "GEMV_FORM_BULK", "quantize_attn_heads_f32_to_q8_1", "gemv_attn_heads_f32_w4a16",
    "launch_quantize_fp16_to_q8_1", "launch_rmsnorm_q8_1",
    "launch_gemv_w4a16", "launch_gemv_w4a8", "launch_gemv_qkv_w4a8",
    "launch_gemv_dual_gate_up_swiglu_w4a16", "launch_gemv_dual_gate_up_swiglu_w4a8",
    "launch_gemm_prefill_w4a16", "launch_gemm_prefill_qkv_w4a16",
    "launch_gemm_prefill_dual_gate_up_swiglu_w4a16", "gemv_group_dots", "DecodeSweep",
    "launch_gemv_rmsnorm_w4a16", "launch_gemv_qkv_rmsnorm_w4a16", "launch_gemv_dual_gate_up_swiglu_rmsnorm_w4a16", "launch_gemv_dual_gate_up_swiglu_rmsnorm_w4a16_q8_1",
    "gemv_w4a8_peers", "gemm_prefill_w4a16_block", "make_sample_control", "launch_embed_lookup_w4a16", "read_sample_control", "launch_sample_and_advance", "sample_slots", "launch_gemv_w4a8_sample_candidates", "launch_sample_finish", "launch_gemv_w4a8_sample_one_launch", "gemv_w4a8_sample_candidates_peers", "gemv_w4a8_sample_candidates_signal", "sample_finish_after_signals", "gemv_w4a8_peers_signal", "gather_after_signals", "launch_gemv_w4a8_sample_and_advance", "SWEEP_SEPARATE", "SWEEP_FUSE_ALL", "SWEEP_PERSISTENT", "SWEEP_QUANT_IN_GATE_UP", "SWEEP_PUBLISH_SUMSQ", "SWEEP_PUBLISH_AMAX", "SWEEP_DEFAULT", "gemv_w4a16_static_scratch", "debug_counter",
]

# Qwen2.5-1.5B defaults of the reference's launchers (include/config.cuh:10-22)
HIDDEN_SIZE, INTERMEDIATE_SIZE = 1536, 8960
NUM_Q_HEADS, NUM_KV_HEADS, HEAD_DIM = 12, 2, 128


def _ptr(t: torch.Tensor | None) -> int | None:
    if t is None:
        return None
    if not t.is_cuda:
        raise ValueError("device pointer expected: tensor is not on a CUDA device")
    return t.data_ptr()


def _stream(stream) -> int:
    if stream is None:
        stream = torch.cuda.current_stream()
    return stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream)


@dataclass
class QKVProjectionView:
    """reference include/kernels.cuh:23-27"""
    q_weight: torch.Tensor
    q_scale: torch.Tensor
    d_q: torch.Tensor
    k_weight: torch.Tensor
    k_scale: torch.Tensor
    d_k: torch.Tensor
    v_weight: torch.Tensor
    v_scale: torch.Tensor
    d_v: torch.Tensor

    def pod(self) -> QKVView:
        return QKVView(*[_ptr(getattr(self, n)) for n, _ in QKVView._fields_])


def debug_counter(which: int = 0) -> int:
    """Device-side debug counters (0: bounded waits of the tensor-core kernel that ran out)."""
    v = ctypes.c_uint(0)
    check("w4a16_debug_counter", load().w4a16_debug_counter(which, ctypes.byref(v)))
    return v.value


def init() -> None:
    check("w4a16_init", load().w4a16_init())


# run-time options of the library (include/w4a16_b200.h, W4A16_OPT_*)
OPT_PDL, OPT_SIGNAL_WAIT_SPINS, OPT_GEMV_FORM, OPT_GEMM_MIN_TOKENS_TENSOR_CORE, OPT_GEMM_FORM = 1, 2, 3, 4, 5
OPT_GEMM_MMA_MAX_TOKENS = 6
GEMV_FORM_AUTO, GEMV_FORM_REGISTERS, GEMV_FORM_BULK = 0, 1, 2


def set_option(which: int, value: int) -> None:
    check("w4a16_set_option", load().w4a16_set_option(which, int(value)))


def get_option(which: int) -> int:
    return int(load().w4a16_get_option(which))


def set_pdl(enabled: bool) -> None:
    """Programmatic dependent launch on (default) or off for all launchers."""
    set_option(OPT_PDL, int(bool(enabled)))


def launch_quantize_fp16_to_q8_1(input_x, out_q8, out_scale, out_sum8, num_elements, stream=None):
    check("w4a16_quantize_fp16_to_q8_1", load().w4a16_quantize_fp16_to_q8_1(
        _ptr(input_x), _ptr(out_q8), _ptr(out_scale), _ptr(out_sum8), num_elements, _stream(stream)))


def launch_rmsnorm_q8_1(input, gamma, output_fp16_opt, out_q8, out_scale, out_sum8, stream=None,
                        hidden_size=HIDDEN_SIZE):
    check("w4a16_rmsnorm_q8_1", load().w4a16_rmsnorm_q8_1(
        _ptr(input), _ptr(gamma), _ptr(output_fp16_opt), _ptr(out_q8), _ptr(out_scale), _ptr(out_sum8),
        _stream(stream), hidden_size))


def quantize_attn_heads_f32_to_q8_1(attn_acc, attn_out_fp16_opt, out_q8, out_scale, out_sum8, num_heads, head_dim=128,
                                    stream=None):
    """Q8_1 of attention heads from their fp32 accumulators, with the rule of the reference's flash-decode
    combine step (src/kernels/attention_gqa.cu:258-310): per head, q = rn(acc / d)."""
    check("w4a16_quantize_attn_heads_f32_to_q8_1", load().w4a16_quantize_attn_heads_f32_to_q8_1(
        _ptr(attn_acc), _ptr(attn_out_fp16_opt), _ptr(out_q8), _ptr(out_scale), _ptr(out_sum8), num_heads, head_dim,
        _stream(stream)))


def gemv_attn_heads_f32_w4a16(qweight, scales, attn_acc, residual, output_y, out_features, in_features, stream=None):
    """O projection straight from the fp32 attention accumulators (quantised per head in the GEMV's prologue)."""
    check("w4a16_gemv_attn_heads_f32_w4a16", load().w4a16_gemv_attn_heads_f32_w4a16(
        _ptr(qweight), _ptr(scales), _ptr(attn_acc), _ptr(residual), _ptr(output_y), out_features, in_features,
        _stream(stream)))


def launch_gemv_w4a16(qweight, scales, input_x, residual, output_y, out_features, in_features, stream=None):
    check("w4a16_gemv_w4a16", load().w4a16_gemv_w4a16(
        _ptr(qweight), _ptr(scales), _ptr(input_x), _ptr(residual), _ptr(output_y), out_features, in_features,
        _stream(stream)))


def gemv_w4a16_static_scratch(qweight, scales, input_x, residual, output_y, out_features, in_features,
                              stream=None):
    """launch_gemv_w4a16 for callers that can neither pass nor allocate scratch: the Q8_1 form of
    the activation goes into a fixed array inside the library (in_features <= 32768; calls that
    overlap on the GPU race on that array)."""
    check("w4a16_gemv_w4a16_static_scratch", load().w4a16_gemv_w4a16_static_scratch(
        _ptr(qweight), _ptr(scales), _ptr(input_x), _ptr(residual), _ptr(output_y), out_features, in_features,
        _stream(stream)))


def launch_gemv_w4a8(qweight, scales, input_q8, input_scale, input_sum8, residual, output_y, out_features,
                     in_features, stream=None):
    check("w4a16_gemv_w4a8", load().w4a16_gemv_w4a8(
        _ptr(qweight), _ptr(scales), _ptr(input_q8), _ptr(input_scale), _ptr(input_sum8), _ptr(residual),
        _ptr(output_y), out_features, in_features, _stream(stream)))


def gemv_w4a8_peers(qweight, scales, input_q8, input_scale, input_sum8, output_y, peer_ptrs, out_features,
                    in_features, stream=None):
    """launch_gemv_w4a8 that also stores its output slice at the device addresses `peer_ptrs` (the slice's
    place in each peer GPU's gathered buffer, mapped into this process)."""
    arr = (ctypes.c_void_p * max(1, len(peer_ptrs)))(*peer_ptrs)
    check("w4a16_gemv_w4a8_peers", load().w4a16_gemv_w4a8_peers(
        _ptr(qweight), _ptr(scales), _ptr(input_q8), _ptr(input_scale), _ptr(input_sum8), _ptr(output_y), arr,
        len(peer_ptrs), out_features, in_features, _stream(stream)))


# ---- token selection after lm_head ------------------------------------------------------------

VOCAB_SIZE = 151936


def make_sample_control(temperature=0.0, rng_seed=0, seq_pos=0, token_id=0) -> "torch.Tensor":
    """A device copy of the control block {int32 token_id, int32 seq_pos, float temperature, uint32 reserved,
    uint64 rng_seed} (the reference's DeviceControlBlock, include/tensor.cuh:28-34) as an int32 tensor [6]."""
    import struct
    raw = struct.pack("<iifIQ", token_id, seq_pos, temperature, 0, rng_seed & 0xFFFFFFFFFFFFFFFF)
    return torch.frombuffer(bytearray(raw), dtype=torch.int32).cuda()


def read_sample_control(control) -> dict:
    import struct
    token_id, seq_pos, temperature, _, rng_seed = struct.unpack("<iifIQ", control.cpu().numpy().tobytes())
    return {"token_id": token_id, "seq_pos": seq_pos, "temperature": temperature, "rng_seed": rng_seed}


def launch_embed_lookup_w4a16(embed_qweight, embed_scales, d_token_ids, out_hidden, d_control, num_tokens, stream=None,
                              hidden_size=HIDDEN_SIZE, vocab_size=VOCAB_SIZE):
    """Mirror of launch_embed_lookup_w4a16 (reference include/kernels.cuh); vocab_size bounds the token ids."""
    check("w4a16_embed_lookup_w4a16", load().w4a16_embed_lookup_w4a16(
        _ptr(embed_qweight), _ptr(embed_scales), _ptr(d_token_ids), _ptr(out_hidden), _ptr(d_control), num_tokens,
        _stream(stream), hidden_size, vocab_size))


def launch_sample_and_advance(logits, sample_scratch_val, sample_scratch_idx, d_control, d_token_out, stream=None,
                              vocab_size=VOCAB_SIZE):
    """Mirror of launch_sample_and_advance (reference include/kernels.cuh:210-219)."""
    check("w4a16_sample_and_advance", load().w4a16_sample_and_advance(
        _ptr(logits), _ptr(sample_scratch_val), _ptr(sample_scratch_idx), _ptr(d_control), _ptr(d_token_out),
        _stream(stream), vocab_size))


def sample_slots(out_features: int) -> int:
    n = load().w4a16_sample_slots(out_features)
    if n < 0:
        check("w4a16_sample_slots", n)
    return n


def launch_gemv_w4a8_sample_candidates(qweight, scales, input_q8, input_scale, input_sum8, output_logits, candidate_val,
                                       candidate_idx, d_control, index_offset, out_features, in_features, stream=None):
    """lm_head GEMV that leaves one (score, index) candidate per CTA; output_logits may be None."""
    check("w4a16_gemv_w4a8_sample_candidates", load().w4a16_gemv_w4a8_sample_candidates(
        _ptr(qweight), _ptr(scales), _ptr(input_q8), _ptr(input_scale), _ptr(input_sum8), _ptr(output_logits),
        _ptr(candidate_val), _ptr(candidate_idx), _ptr(d_control), index_offset, out_features, in_features,
        _stream(stream)))


def gemv_w4a8_sample_candidates_peers(qweight, scales, input_q8, input_scale, input_sum8, candidate_val, candidate_idx,
                                      peer_val_ptrs, peer_idx_ptrs, d_control, index_offset, out_features,
                                      in_features, stream=None):
    """The candidates launch, which also stores its candidates at the device addresses given per peer GPU."""
    n = len(peer_val_ptrs)
    assert n == len(peer_idx_ptrs)
    pv = (ctypes.c_void_p * max(1, n))(*peer_val_ptrs)
    pi = (ctypes.c_void_p * max(1, n))(*peer_idx_ptrs)
    check("w4a16_gemv_w4a8_sample_candidates_peers", load().w4a16_gemv_w4a8_sample_candidates_peers(
        _ptr(qweight), _ptr(scales), _ptr(input_q8), _ptr(input_scale), _ptr(input_sum8), _ptr(candidate_val),
        _ptr(candidate_idx), pv, pi, n, _ptr(d_control), index_offset, out_features, in_features, _stream(stream)))


def gemv_w4a8_sample_candidates_signal(qweight, scales, input_q8, input_scale, input_sum8, candidate_val_ptr,
                                       candidate_idx_ptr, peer_val_ptrs, peer_idx_ptrs, peer_flag_ptrs, local_flag_ptr,
                                       done_counter, step_word, half_stride, d_control, index_offset, out_features,
                                       in_features, stream=None):
    """Candidates launch with peer stores and the completion signal (addresses as integers where they point
    into symmetric memory)."""
    n = len(peer_val_ptrs)
    pv = (ctypes.c_void_p * max(1, n))(*peer_val_ptrs)
    pi = (ctypes.c_void_p * max(1, n))(*peer_idx_ptrs)
    pf = (ctypes.c_void_p * max(1, n))(*peer_flag_ptrs)
    check("w4a16_gemv_w4a8_sample_candidates_signal", load().w4a16_gemv_w4a8_sample_candidates_signal(
        _ptr(qweight), _ptr(scales), _ptr(input_q8), _ptr(input_scale), _ptr(input_sum8), candidate_val_ptr,
        candidate_idx_ptr, pv, pi, pf, n, local_flag_ptr, _ptr(done_counter), _ptr(step_word), half_stride,
        _ptr(d_control), index_offset, out_features, in_features, _stream(stream)))


def gemv_w4a8_peers_signal(qweight, scales, input_q8, input_scale, input_sum8, gathered_slice_ptr, peer_slice_ptrs,
                           peer_flag_ptrs, local_flag_ptr, done_counter, step_word, half_stride, out_features, in_features,
                           stream=None):
    """Row-split GEMV whose epilogue stores the slice into every GPU's gathered vector and signals completion
    (addresses as integers where they point into symmetric memory)."""
    n = len(peer_slice_ptrs)
    ps = (ctypes.c_void_p * max(1, n))(*peer_slice_ptrs)
    pf = (ctypes.c_void_p * max(1, n))(*peer_flag_ptrs)
    check("w4a16_gemv_w4a8_peers_signal", load().w4a16_gemv_w4a8_peers_signal(
        _ptr(qweight), _ptr(scales), _ptr(input_q8), _ptr(input_scale), _ptr(input_sum8), gathered_slice_ptr, ps, pf, n,
        local_flag_ptr, _ptr(done_counter), _ptr(step_word), half_stride, out_features, in_features, _stream(stream)))


def gather_after_signals(gathered_ptr, half_stride, flags_ptr, num_flags, step_word, d_status, output, num_elements,
                         stream=None):
    check("w4a16_gather_after_signals", load().w4a16_gather_after_signals(
        gathered_ptr, half_stride, flags_ptr, num_flags, _ptr(step_word), _ptr(d_status), _ptr(output), num_elements,
        _stream(stream)))


def sample_finish_after_signals(candidate_val_ptr, candidate_idx_ptr, count, half_stride, flags_ptr, num_flags, step_word,
                                d_status, d_control, d_token_out, stream=None):
    check("w4a16_sample_finish_after_signals", load().w4a16_sample_finish_after_signals(
        candidate_val_ptr, candidate_idx_ptr, count, half_stride, flags_ptr, num_flags, _ptr(step_word), _ptr(d_status),
        _ptr(d_control), _ptr(d_token_out), _stream(stream)))


def launch_gemv_w4a8_sample_one_launch(qweight, scales, input_q8, input_scale, input_sum8, output_logits, sample_scratch_val,
                                       sample_scratch_idx, d_counter, d_control, d_token_out, out_features, in_features,
                                       stream=None):
    """lm_head + token selection + control-block advance in one launch (d_counter: zero-initialised int32 [1])."""
    check("w4a16_gemv_w4a8_sample_one_launch", load().w4a16_gemv_w4a8_sample_one_launch(
        _ptr(qweight), _ptr(scales), _ptr(input_q8), _ptr(input_scale), _ptr(input_sum8), _ptr(output_logits),
        _ptr(sample_scratch_val), _ptr(sample_scratch_idx), _ptr(d_counter), _ptr(d_control), _ptr(d_token_out),
        out_features, in_features, _stream(stream)))


def launch_sample_finish(candidate_val, candidate_idx, count, d_control, d_token_out, stream=None):
    check("w4a16_sample_finish", load().w4a16_sample_finish(
        _ptr(candidate_val), _ptr(candidate_idx), count, _ptr(d_control), _ptr(d_token_out), _stream(stream)))


def launch_gemv_w4a8_sample_and_advance(qweight, scales, input_q8, input_scale, input_sum8, output_logits,
                                        sample_scratch_val, sample_scratch_idx, d_control, d_token_out, out_features,
                                        in_features, stream=None):
    """launch_gemv_w4a8 (lm_head) + launch_sample_and_advance in one pass over the weights."""
    check("w4a16_gemv_w4a8_sample_and_advance", load().w4a16_gemv_w4a8_sample_and_advance(
        _ptr(qweight), _ptr(scales), _ptr(input_q8), _ptr(input_scale), _ptr(input_sum8), _ptr(output_logits),
        _ptr(sample_scratch_val), _ptr(sample_scratch_idx), _ptr(d_control), _ptr(d_token_out), out_features,
        in_features, _stream(stream)))


def launch_gemv_qkv_w4a8(view: QKVProjectionView, input_q8, input_scale, input_sum8, stream=None,
                         in_features=HIDDEN_SIZE, num_q_heads=NUM_Q_HEADS, num_kv_heads=NUM_KV_HEADS,
                         head_dim=HEAD_DIM):
    pod = view.pod()
    check("w4a16_gemv_qkv_w4a8", load().w4a16_gemv_qkv_w4a8(
        ctypes.byref(pod), _ptr(input_q8), _ptr(input_scale), _ptr(input_sum8), _stream(stream), in_features,
        num_q_heads, num_kv_heads, head_dim))


def launch_gemv_dual_gate_up_swiglu_w4a16(gate_up_qweight, gate_up_scales, input_x, output_mlp, hidden_size,
                                          intermediate_size, stream=None):
    check("w4a16_gemv_dual_gate_up_swiglu_w4a16", load().w4a16_gemv_dual_gate_up_swiglu_w4a16(
        _ptr(gate_up_qweight), _ptr(gate_up_scales), _ptr(input_x), _ptr(output_mlp), hidden_size,
        intermediate_size, _stream(stream)))


def launch_gemv_dual_gate_up_swiglu_w4a8(gate_up_qweight, gate_up_scales, input_q8, input_scale, input_sum8,
                                         output_mlp, hidden_size, intermediate_size, stream=None):
    check("w4a16_gemv_dual_gate_up_swiglu_w4a8", load().w4a16_gemv_dual_gate_up_swiglu_w4a8(
        _ptr(gate_up_qweight), _ptr(gate_up_scales), _ptr(input_q8), _ptr(input_scale), _ptr(input_sum8),
        _ptr(output_mlp), hidden_size, intermediate_size, _stream(stream)))


def launch_gemv_rmsnorm_w4a16(qweight, scales, input_x, gamma, residual, output_y, out_features, in_features,
                              stream=None):
    """launch_rmsnorm_q8_1 + launch_gemv_w4a8 in one launch (gamma None: quantise only)."""
    check("w4a16_gemv_rmsnorm_w4a16", load().w4a16_gemv_rmsnorm_w4a16(
        _ptr(qweight), _ptr(scales), _ptr(input_x), _ptr(gamma), _ptr(residual), _ptr(output_y), out_features,
        in_features, _stream(stream)))


def launch_gemv_qkv_rmsnorm_w4a16(view: QKVProjectionView, input_x, gamma, stream=None, in_features=HIDDEN_SIZE,
                                  num_q_heads=NUM_Q_HEADS, num_kv_heads=NUM_KV_HEADS, head_dim=HEAD_DIM):
    """launch_rmsnorm_q8_1 + launch_gemv_qkv_w4a8 in one launch."""
    pod = view.pod()
    check("w4a16_gemv_qkv_rmsnorm_w4a16", load().w4a16_gemv_qkv_rmsnorm_w4a16(
        ctypes.byref(pod), _ptr(input_x), _ptr(gamma), _stream(stream), in_features, num_q_heads, num_kv_heads,
        head_dim))


def launch_gemv_dual_gate_up_swiglu_rmsnorm_w4a16(gate_up_qweight, gate_up_scales, input_x, gamma, output_mlp,
                                                  hidden_size, intermediate_size, stream=None):
    """launch_rmsnorm_q8_1 + launch_gemv_dual_gate_up_swiglu_w4a8 in one launch."""
    check("w4a16_gemv_dual_gate_up_swiglu_rmsnorm_w4a16", load().w4a16_gemv_dual_gate_up_swiglu_rmsnorm_w4a16(
        _ptr(gate_up_qweight), _ptr(gate_up_scales), _ptr(input_x), _ptr(gamma), _ptr(output_mlp), hidden_size,
        intermediate_size, _stream(stream)))


def launch_gemv_dual_gate_up_swiglu_rmsnorm_w4a16_q8_1(gate_up_qweight, gate_up_scales, input_x, gamma, output_mlp,
                                                       output_q8, output_scale, output_sum8, hidden_size,
                                                       intermediate_size, stream=None):
    """The launch above, which also leaves the Q8_1 form of output_mlp (the down projection's input)."""
    check("w4a16_gemv_dual_gate_up_swiglu_rmsnorm_w4a16_q8_1",
          load().w4a16_gemv_dual_gate_up_swiglu_rmsnorm_w4a16_q8_1(
              _ptr(gate_up_qweight), _ptr(gate_up_scales), _ptr(input_x), _ptr(gamma), _ptr(output_mlp),
              _ptr(output_q8), _ptr(output_scale), _ptr(output_sum8), hidden_size, intermediate_size,
              _stream(stream)))


def gemm_prefill_w4a16_block(qweight, scales, input_x, residual_ptr, output_ptr, ldc, peer_ptrs, M, N, K, stream=None):
    """launch_gemm_prefill_w4a16 into a column block of an [M][ldc] matrix (addresses as integers), also stored
    at `peer_ptrs` (the block's place in peer GPUs' matrices)."""
    arr = (ctypes.c_void_p * max(1, len(peer_ptrs)))(*peer_ptrs)
    check("w4a16_gemm_prefill_w4a16_block", load().w4a16_gemm_prefill_w4a16_block(
        _ptr(qweight), _ptr(scales), _ptr(input_x), residual_ptr, output_ptr, ldc, arr, len(peer_ptrs), M, N, K,
        _stream(stream)))


def launch_gemm_prefill_w4a16(qweight, scales, input_x, residual, output_y, M, N, K, stream=None, sm_count=0):
    check("w4a16_gemm_prefill_w4a16", load().w4a16_gemm_prefill_w4a16(
        _ptr(qweight), _ptr(scales), _ptr(input_x), _ptr(residual), _ptr(output_y), M, N, K, _stream(stream),
        sm_count))


def launch_gemm_prefill_qkv_w4a16(view: QKVProjectionView, input_x, M, stream=None, in_features=HIDDEN_SIZE,
                                  num_q_heads=NUM_Q_HEADS, num_kv_heads=NUM_KV_HEADS, head_dim=HEAD_DIM,
                                  sm_count=0):
    pod = view.pod()
    check("w4a16_gemm_prefill_qkv_w4a16", load().w4a16_gemm_prefill_qkv_w4a16(
        ctypes.byref(pod), _ptr(input_x), M, _stream(stream), in_features, num_q_heads, num_kv_heads, head_dim,
        sm_count))


def launch_gemm_prefill_dual_gate_up_swiglu_w4a16(gate_up_qweight, gate_up_scales, input_x, output_mlp, M,
                                                  stream=None, hidden_size=HIDDEN_SIZE,
                                                  intermediate_size=INTERMEDIATE_SIZE):
    check("w4a16_gemm_prefill_dual_gate_up_swiglu_w4a16", load().w4a16_gemm_prefill_dual_gate_up_swiglu_w4a16(
        _ptr(gate_up_qweight), _ptr(gate_up_scales), _ptr(input_x), _ptr(output_mlp), M, _stream(stream),
        hidden_size, intermediate_size))


def gemv_group_dots(qweight, input_q8, input_sum8, out_dots, out_features, in_features, stream=None):
    """Diagnostic: int32 per-group partial sums of the decode GEMV (no reference launcher)."""
    check("w4a16_gemv_group_dots", load().w4a16_gemv_group_dots(
        _ptr(qweight), _ptr(input_q8), _ptr(input_sum8), _ptr(out_dots), out_features, in_features,
        _stream(stream)))


SWEEP_SEPARATE, SWEEP_FUSE_NORM, SWEEP_FUSE_QUANT_O, SWEEP_FUSE_QUANT_DOWN, SWEEP_FUSE_ALL = 0, 1, 2, 4, 7
SWEEP_PERSISTENT = 8
SWEEP_QUANT_IN_GATE_UP = 16
SWEEP_PUBLISH_SUMSQ = 32
SWEEP_PUBLISH_AMAX = 64
# the fastest measured form on B200: RMSNorm inside QKV / gate_up, Q8_1 inside O, a separate quantiser before down
SWEEP_DEFAULT = SWEEP_FUSE_NORM | SWEEP_FUSE_QUANT_O | SWEEP_PUBLISH_SUMSQ


class DecodeSweep:
    """The W4 projections of one batch-1 decode pass as one CUDA graph (C ABI w4a16_sweep_*).

    layers: list of dicts with keys input_norm, q, k, v, o, post_norm, gate_up, down; the norm
    entries are fp16 gamma tensors, the others (qweight, scales) tensor pairs -- or a ready ctypes array of
    LayerWeights (e.g. QwenBin.layer_table over an uploaded `.qwenbin` file; the caller keeps that memory alive).  The object keeps
    the tensors alive; the native sweep owns only its graph.
    """

    def __init__(self, layers, hidden=HIDDEN_SIZE, inter=INTERMEDIATE_SIZE, num_q_heads=NUM_Q_HEADS,
                 num_kv_heads=NUM_KV_HEADS, head_dim=HEAD_DIM, stream=None, flags=SWEEP_DEFAULT):
        lib = load()
        self._layers = layers
        self.hidden = hidden
        nbytes = lib.w4a16_sweep_workspace_bytes(hidden, inter, num_q_heads, num_kv_heads, head_dim)
        if nbytes < 0:
            check("w4a16_sweep_workspace_bytes", int(nbytes))
        self._ws = torch.zeros(nbytes + 256, dtype=torch.uint8, device="cuda")
        ws_ptr = (self._ws.data_ptr() + 255) // 256 * 256
        arr = layers if isinstance(layers, ctypes.Array) else (LayerWeights * len(layers))()
        for i, L in enumerate([] if isinstance(layers, ctypes.Array) else layers):
            arr[i] = LayerWeights(
                _ptr(L["input_norm"]), _ptr(L["q"][0]), _ptr(L["q"][1]), _ptr(L["k"][0]), _ptr(L["k"][1]),
                _ptr(L["v"][0]), _ptr(L["v"][1]), _ptr(L["o"][0]), _ptr(L["o"][1]), _ptr(L["post_norm"]),
                _ptr(L["gate_up"][0]), _ptr(L["gate_up"][1]), _ptr(L["down"][0]), _ptr(L["down"][1]))
        desc = SweepDesc(len(layers), hidden, inter, num_q_heads, num_kv_heads, head_dim, arr, ws_ptr, flags)
        handle = ctypes.c_void_p()
        check("w4a16_sweep_create", lib.w4a16_sweep_create(ctypes.byref(desc), _stream(stream), ctypes.byref(handle)))
        self._h = handle
        self.launches = lib.w4a16_sweep_launches(handle)

    def run_device(self, h_in: torch.Tensor, h_out: torch.Tensor, stream=None):
        check("w4a16_sweep_run_device", load().w4a16_sweep_run_device(self._h, _ptr(h_in), _ptr(h_out),
                                                                      _stream(stream)))

    def run_host(self, h_in: torch.Tensor, h_out: torch.Tensor, stream=None):
        """h_in / h_out: pinned host fp16 tensors; asynchronous on the stream."""
        assert not h_in.is_cuda and not h_out.is_cuda
        check("w4a16_sweep_run_host", load().w4a16_sweep_run_host(self._h, h_in.data_ptr(), h_out.data_ptr(),
                                                                  _stream(stream)))

    def status(self) -> int:
        """0 after clean passes; nonzero if a bounded wait of the persistent kernel ran out."""
        v = ctypes.c_int(0)
        check("w4a16_sweep_status", load().w4a16_sweep_status(self._h, ctypes.byref(v)))
        return v.value

    def buffer_ptr(self, which: int) -> int:
        return load().w4a16_sweep_buffer(self._h, which)

    def close(self):
        if self._h is not None:
            load().w4a16_sweep_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
