// Header-only C++ shim: the reference engine's `qwen::launch_*` functions for the W4
// projection path (reference include/kernels.cuh:23-27, 39-153), implemented on top of the
// C ABI of libw4a16_b200.so.
//
// A translation unit of the reference (src/engine.cu, tests/test_kernels.cu) that is
// compiled against this header instead of linking the reference's gemv_w4a16.cu /
// gemm_prefill.cu (and the two quantiser launchers of rmsnorm_rope.cu) gets the same
// names, parameter lists, default arguments and error behaviour: a failed launch throws
// std::runtime_error, as CUDA_KERNEL_CHECK does there (reference include/tensor.cuh:11-23).
//
// The default arguments are the Qwen2.5-1.5B dimensions of reference include/config.cuh:10-22;
// when that header is present its constants are used (define W4A16_COMPAT_USE_REFERENCE_CONFIG
// and include it first), otherwise the literals below.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <stdexcept>
#include <string>

#include "w4a16_b200.h"

namespace qwen {

// Two ways to use it:
//   * header mode (default): inline functions with the reference's default arguments, for a build whose
//     kernels.cuh no longer declares these functions;
//   * link mode (define W4A16_COMPAT_OUT_OF_LINE and include the reference's kernels.cuh FIRST): the same
//     functions as ordinary external definitions, without default arguments, matching the declarations
//     already in scope.  One translation unit built this way plus libw4a16_b200.so replaces
//     src/kernels/gemv_w4a16.cu and src/kernels/gemm_prefill.cu at link time with no edit to the reference.
#ifdef W4A16_COMPAT_OUT_OF_LINE
#define W4A16_COMPAT_NO_QKV_VIEW
#define W4A16_INLINE
#define W4A16_DEFAULT(value)
#else
#define W4A16_INLINE inline
#define W4A16_DEFAULT(value) = value
#endif

#if !defined(W4A16_COMPAT_USE_REFERENCE_CONFIG) && !defined(W4A16_COMPAT_OUT_OF_LINE)
namespace w4a16_compat_defaults {
constexpr int HIDDEN_SIZE = 1536;
constexpr int INTERMEDIATE_SIZE = 8960;
constexpr int NUM_Q_HEADS = 12;
constexpr int NUM_KV_HEADS = 2;
constexpr int HEAD_DIM = 128;
}  // namespace w4a16_compat_defaults
#define W4A16_DFLT(name) w4a16_compat_defaults::name
#else
#define W4A16_DFLT(name) name
#endif

namespace w4a16_detail {
inline void check(int status, const char* what) {
    if (status == 0) return;
    std::fprintf(stderr, "w4a16 error in %s: %s (status %d)\n", what, w4a16_status_string(status), status);
    std::fflush(stderr);
    throw std::runtime_error(std::string("CUDA error: ") + w4a16_status_string(status));
}
}  // namespace w4a16_detail

#ifndef W4A16_COMPAT_NO_QKV_VIEW
// reference include/kernels.cuh:23-27
struct QKVProjectionView {
    const void* q_weight; const half* q_scale; half* d_q;
    const void* k_weight; const half* k_scale; half* d_k;
    const void* v_weight; const half* v_scale; half* d_v;
};
#endif

namespace w4a16_detail {
inline w4a16_qkv_view to_pod(const QKVProjectionView& v) {
    return w4a16_qkv_view{v.q_weight, v.q_scale, v.d_q, v.k_weight, v.k_scale, v.d_k, v.v_weight, v.v_scale, v.d_v};
}
}  // namespace w4a16_detail

// reference include/kernels.cuh:39-48
W4A16_INLINE void launch_rmsnorm_q8_1(const half* input, const half* gamma, half* output_fp16_opt, int8_t* out_q8,
                                float* out_scale, int32_t* out_sum8, cudaStream_t stream,
                                int hidden_size W4A16_DEFAULT(W4A16_DFLT(HIDDEN_SIZE))) {
    w4a16_detail::check(w4a16_rmsnorm_q8_1(input, gamma, output_fp16_opt, out_q8, out_scale, out_sum8, stream,
                                           hidden_size),
                        "launch_rmsnorm_q8_1");
}

// reference include/kernels.cuh:50-57
W4A16_INLINE void launch_quantize_fp16_to_q8_1(const half* input_x, int8_t* out_q8, float* out_scale, int32_t* out_sum8,
                                         int num_elements, cudaStream_t stream) {
    w4a16_detail::check(w4a16_quantize_fp16_to_q8_1(input_x, out_q8, out_scale, out_sum8, num_elements, stream),
                        "launch_quantize_fp16_to_q8_1");
}

// reference include/kernels.cuh:60-69
W4A16_INLINE void launch_gemv_w4a16(const uint32_t* qweight, const half* scales, const half* input_x, const half* residual,
                              half* output_y, int out_features, int in_features, cudaStream_t stream) {
    w4a16_detail::check(
        w4a16_gemv_w4a16(qweight, scales, input_x, residual, output_y, out_features, in_features, stream),
        "launch_gemv_w4a16");
}

// reference include/kernels.cuh:71-82
W4A16_INLINE void launch_gemv_w4a8(const uint32_t* qweight, const half* scales, const int8_t* input_q8,
                             const float* input_scale, const int32_t* input_sum8, const half* residual,
                             half* output_y, int out_features, int in_features, cudaStream_t stream) {
    w4a16_detail::check(w4a16_gemv_w4a8(qweight, scales, input_q8, input_scale, input_sum8, residual, output_y,
                                        out_features, in_features, stream),
                        "launch_gemv_w4a8");
}

// reference include/kernels.cuh:84-94
W4A16_INLINE void launch_gemv_qkv_w4a8(const QKVProjectionView& view, const int8_t* input_q8, const float* input_scale,
                                 const int32_t* input_sum8, cudaStream_t stream,
                                 int in_features W4A16_DEFAULT(W4A16_DFLT(HIDDEN_SIZE)), int num_q_heads W4A16_DEFAULT(W4A16_DFLT(NUM_Q_HEADS)),
                                 int num_kv_heads W4A16_DEFAULT(W4A16_DFLT(NUM_KV_HEADS)), int head_dim W4A16_DEFAULT(W4A16_DFLT(HEAD_DIM))) {
    const w4a16_qkv_view pod = w4a16_detail::to_pod(view);
    w4a16_detail::check(w4a16_gemv_qkv_w4a8(&pod, input_q8, input_scale, input_sum8, stream, in_features,
                                            num_q_heads, num_kv_heads, head_dim),
                        "launch_gemv_qkv_w4a8");
}

// reference include/kernels.cuh:96-104
W4A16_INLINE void launch_gemv_dual_gate_up_swiglu_w4a16(const uint32_t* gate_up_qweight, const half* gate_up_scales,
                                                  const half* input_x, half* output_mlp, int hidden_size,
                                                  int intermediate_size, cudaStream_t stream) {
    w4a16_detail::check(w4a16_gemv_dual_gate_up_swiglu_w4a16(gate_up_qweight, gate_up_scales, input_x, output_mlp,
                                                             hidden_size, intermediate_size, stream),
                        "launch_gemv_dual_gate_up_swiglu_w4a16");
}

// reference include/kernels.cuh:106-116
W4A16_INLINE void launch_gemv_dual_gate_up_swiglu_w4a8(const uint32_t* gate_up_qweight, const half* gate_up_scales,
                                                 const int8_t* input_q8, const float* input_scale,
                                                 const int32_t* input_sum8, half* output_mlp, int hidden_size,
                                                 int intermediate_size, cudaStream_t stream) {
    w4a16_detail::check(
        w4a16_gemv_dual_gate_up_swiglu_w4a8(gate_up_qweight, gate_up_scales, input_q8, input_scale, input_sum8,
                                            output_mlp, hidden_size, intermediate_size, stream),
        "launch_gemv_dual_gate_up_swiglu_w4a8");
}

// reference include/kernels.cuh:119-130
W4A16_INLINE void launch_gemm_prefill_w4a16(const uint32_t* qweight, const half* scales, const half* input_x,
                                      const half* residual, half* output_y, int M, int N, int K, cudaStream_t stream,
                                      int sm_count W4A16_DEFAULT(0)) {
    w4a16_detail::check(w4a16_gemm_prefill_w4a16(qweight, scales, input_x, residual, output_y, M, N, K, stream,
                                                 sm_count),
                        "launch_gemm_prefill_w4a16");
}

// reference include/kernels.cuh:132-142
W4A16_INLINE void launch_gemm_prefill_qkv_w4a16(const QKVProjectionView& view, const half* input_x, int M,
                                          cudaStream_t stream, int in_features W4A16_DEFAULT(W4A16_DFLT(HIDDEN_SIZE)),
                                          int num_q_heads W4A16_DEFAULT(W4A16_DFLT(NUM_Q_HEADS)),
                                          int num_kv_heads W4A16_DEFAULT(W4A16_DFLT(NUM_KV_HEADS)),
                                          int head_dim W4A16_DEFAULT(W4A16_DFLT(HEAD_DIM)), int sm_count W4A16_DEFAULT(0)) {
    const w4a16_qkv_view pod = w4a16_detail::to_pod(view);
    w4a16_detail::check(w4a16_gemm_prefill_qkv_w4a16(&pod, input_x, M, stream, in_features, num_q_heads,
                                                     num_kv_heads, head_dim, sm_count),
                        "launch_gemm_prefill_qkv_w4a16");
}

// reference include/kernels.cuh:144-153
W4A16_INLINE void launch_gemm_prefill_dual_gate_up_swiglu_w4a16(const uint32_t* gate_up_qweight,
                                                          const half* gate_up_scales, const half* input_x,
                                                          half* output_mlp, int M, cudaStream_t stream,
                                                          int hidden_size W4A16_DEFAULT(W4A16_DFLT(HIDDEN_SIZE)),
                                                          int intermediate_size W4A16_DEFAULT(W4A16_DFLT(INTERMEDIATE_SIZE))) {
    w4a16_detail::check(w4a16_gemm_prefill_dual_gate_up_swiglu_w4a16(gate_up_qweight, gate_up_scales, input_x,
                                                                     output_mlp, M, stream, hidden_size,
                                                                     intermediate_size),
                        "launch_gemm_prefill_dual_gate_up_swiglu_w4a16");
}

// ---- the callers either side of the projections (optional: define W4A16_COMPAT_WITH_CONTROL_BLOCK in a
// translation unit that has the reference's DeviceControlBlock, include/tensor.cuh:28-34, in scope) ----
#ifdef W4A16_COMPAT_WITH_CONTROL_BLOCK
static_assert(sizeof(DeviceControlBlock) >= sizeof(w4a16_sample_control), "control block layout");

// reference include/kernels.cuh:11-20 (src/kernels/rmsnorm_rope.cu:15-69)
#ifdef W4A16_COMPAT_OUT_OF_LINE
// the reference's declaration has no vocabulary parameter: its kernel bounds the ids by the constant VOCAB_SIZE
void launch_embed_lookup_w4a16(const uint32_t* embed_qweight, const half* embed_scales, const int32_t* d_token_ids,
                               half* out_hidden, const DeviceControlBlock* d_control, int num_tokens,
                               cudaStream_t stream, int hidden_size) {
    const int vocab_size = VOCAB_SIZE;
#else
inline void launch_embed_lookup_w4a16(const uint32_t* embed_qweight, const half* embed_scales,
                                      const int32_t* d_token_ids, half* out_hidden,
                                      const DeviceControlBlock* d_control, int num_tokens, cudaStream_t stream,
                                      int hidden_size = W4A16_DFLT(HIDDEN_SIZE), int vocab_size = 151936) {
#endif
    w4a16_detail::check(w4a16_embed_lookup_w4a16(embed_qweight, embed_scales, d_token_ids, out_hidden, d_control,
                                                 num_tokens, stream, hidden_size, vocab_size),
                        "launch_embed_lookup_w4a16");
}

// reference include/kernels.cuh:210-219 (src/kernels/sampling.cu:206-230)
W4A16_INLINE void launch_sample_and_advance(const half* logits, float* sample_scratch_val, int32_t* sample_scratch_idx,
                                      DeviceControlBlock* d_control, int32_t* d_mapped_pinned_token,
                                      cudaStream_t stream, int vocab_size W4A16_DEFAULT(151936)) {
    w4a16_detail::check(w4a16_sample_and_advance(logits, sample_scratch_val, sample_scratch_idx, d_control,
                                                 d_mapped_pinned_token, stream, vocab_size),
                        "launch_sample_and_advance");
}
#endif

#undef W4A16_DFLT
#undef W4A16_DEFAULT
#undef W4A16_INLINE

}  // namespace qwen
