// extern "C" boundary of the library: argument checks, then the kernel launchers.
// Declarations and the reference functions they replace: include/w4a16_b200.h.
#include <atomic>
#include <cstdlib>
#include <mutex>

#include "w4a16_internal.hpp"

namespace w4 {
namespace {

constexpr int kMaxDevices = 64;
DeviceInfo g_dev[kMaxDevices];
std::mutex g_dev_mutex;
std::atomic<bool> g_dev_ready[kMaxDevices];
// run-time options (w4a16_set_option): plain process-wide integers, read at launch time
std::atomic<int> g_options[W4A16_OPT_COUNT_];
const int kOptionDefaults[W4A16_OPT_COUNT_] = {0, /*PDL*/ 1, /*SIGNAL_WAIT_SPINS*/ 1 << 22, /*GEMV_FORM*/ 0,
                                                /*GEMM_MIN_TOKENS_TENSOR_CORE*/ 0, /*GEMM_FORM*/ 0, /*GEMM_MMA_MAX_TOKENS*/ 0};
std::once_flag g_options_once;
void init_options() {
    std::call_once(g_options_once, [] {
        for (int i = 0; i < W4A16_OPT_COUNT_; ++i) g_options[i].store(kOptionDefaults[i], std::memory_order_relaxed);
    });
}

}  // namespace

int option(int which) {
    init_options();
    return (which > 0 && which < W4A16_OPT_COUNT_) ? g_options[which].load(std::memory_order_relaxed) : 0;
}
bool pdl_enabled() { return option(W4A16_OPT_PDL) != 0; }

int ensure_device_ready(const DeviceInfo** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (dev < 0 || dev >= kMaxDevices) return W4A16_ERR_NO_DEVICE;
    if (!g_dev_ready[dev].load(std::memory_order_acquire)) {
        std::lock_guard<std::mutex> lock(g_dev_mutex);
        if (!g_dev_ready[dev].load(std::memory_order_relaxed)) {
            DeviceInfo info;
            if ((e = cudaDeviceGetAttribute(&info.sm_count, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess)
                return static_cast<int>(e);
            if ((e = cudaDeviceGetAttribute(&info.cc_major, cudaDevAttrComputeCapabilityMajor, dev)) != cudaSuccess)
                return static_cast<int>(e);
            if (info.cc_major != 10) return W4A16_ERR_NO_DEVICE;  // the kernels are sm_100a only
            if (int st = quantize_set_attributes()) return st;
            if (int st = gemv_set_attributes()) return st;
            if (int st = gemm_set_attributes()) return st;
            info.ready = true;
            g_dev[dev] = info;
            g_dev_ready[dev].store(true, std::memory_order_release);
        }
    }
    if (out) *out = &g_dev[dev];
    return 0;
}

}  // namespace w4

namespace {

using namespace w4;

inline const __half* H(const void* p) { return static_cast<const __half*>(p); }
inline __half* H(void* p) { return static_cast<__half*>(p); }
inline cudaStream_t S(w4a16_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }
inline bool misaligned(const void* p, size_t a) { return reinterpret_cast<uintptr_t>(p) % a != 0; }

int check_k(int K) { return (K > 0 && K % 256 == 0) ? 0 : W4A16_ERR_SHAPE; }

}  // namespace

extern "C" {

int w4a16_version(void) { return 100; }

const char* w4a16_status_string(int status) {
    switch (status) {
        case W4A16_OK: return "ok";
        case W4A16_ERR_INVALID_ARG: return "invalid argument (null pointer or non-positive size)";
        case W4A16_ERR_SHAPE: return "unsupported shape (in_features must be a positive multiple of 256)";
        case W4A16_ERR_ALIGNMENT: return "pointer below the minimum alignment of its element type";
        case W4A16_ERR_NO_DEVICE: return "current device is not an sm_100 GPU";
        case W4A16_ERR_TOO_LARGE: return "size beyond the supported maximum";
        default: break;
    }
    if (status > 0) return cudaGetErrorString(static_cast<cudaError_t>(status));
    return "unknown status";
}

int w4a16_init(void) { return ensure_device_ready(nullptr); }

int w4a16_set_option(int which, int value) {
    if (which <= 0 || which >= W4A16_OPT_COUNT_) return W4A16_ERR_INVALID_ARG;
    switch (which) {
        case W4A16_OPT_PDL: value = value != 0; break;
        case W4A16_OPT_SIGNAL_WAIT_SPINS: if (value < 1) return W4A16_ERR_INVALID_ARG; break;
        case W4A16_OPT_GEMV_FORM: if (value < 0 || value > 2) return W4A16_ERR_INVALID_ARG; break;
        case W4A16_OPT_GEMM_MIN_TOKENS_TENSOR_CORE: if (value < 0) return W4A16_ERR_INVALID_ARG; break;
        case W4A16_OPT_GEMM_FORM: if (value < 0 || value > 2) return W4A16_ERR_INVALID_ARG; break;
        case W4A16_OPT_GEMM_MMA_MAX_TOKENS: if (value < 0) return W4A16_ERR_INVALID_ARG; break;
        default: break;
    }
    init_options();
    g_options[which].store(value, std::memory_order_relaxed);
    return 0;
}
int w4a16_get_option(int which) {
    if (which <= 0 || which >= W4A16_OPT_COUNT_) return W4A16_ERR_INVALID_ARG;
    return option(which);
}

int w4a16_quantize_fp16_to_q8_1(const void* input_x, int8_t* out_q8, float* out_scale, int32_t* out_sum8,
                                int num_elements, w4a16_stream_t stream) {
    if (!input_x || !out_q8 || !out_scale || !out_sum8 || num_elements <= 0) return W4A16_ERR_INVALID_ARG;
    if (num_elements % 128 != 0) return W4A16_ERR_SHAPE;
    if (misaligned(input_x, 8) || misaligned(out_q8, 4) || misaligned(out_scale, 4) || misaligned(out_sum8, 4))
        return W4A16_ERR_ALIGNMENT;
    if (int st = ensure_device_ready(nullptr)) return st;
    return quantize_fp16_to_q8_1(H(input_x), out_q8, out_scale, out_sum8, num_elements, S(stream));
}

int w4a16_rmsnorm_q8_1(const void* input, const void* gamma, void* output_fp16_opt, int8_t* out_q8, float* out_scale,
                       int32_t* out_sum8, w4a16_stream_t stream, int hidden_size) {
    if (!input || !gamma || !out_q8 || !out_scale || !out_sum8 || hidden_size <= 0) return W4A16_ERR_INVALID_ARG;
    if (hidden_size % 128 != 0) return W4A16_ERR_SHAPE;
    if (hidden_size > 100 * 1024) return W4A16_ERR_TOO_LARGE;
    if (misaligned(input, 8) || misaligned(gamma, 4) || misaligned(output_fp16_opt, 4) || misaligned(out_q8, 4) ||
        misaligned(out_scale, 4) || misaligned(out_sum8, 4))
        return W4A16_ERR_ALIGNMENT;
    if (int st = ensure_device_ready(nullptr)) return st;
    return rmsnorm_q8_1(H(input), H(gamma), H(output_fp16_opt), out_q8, out_scale, out_sum8, hidden_size, S(stream));
}

static int gemv_plain(const uint32_t* qweight, const void* scales, const void* x_fp16, const int8_t* q8,
                      const float* xscale, const int32_t* sum8, const void* residual, void* y, int N, int K,
                      w4a16_stream_t stream, const void* gamma = nullptr, void* const* peers = nullptr,
                      int num_peers = 0, const float* x_f32 = nullptr) {
    if (!qweight || !scales || !y || N <= 0) return W4A16_ERR_INVALID_ARG;
    if (misaligned(x_f32, 16)) return W4A16_ERR_ALIGNMENT;
    if (int st = check_k(K)) return st;
    if (misaligned(qweight, 4) || misaligned(scales, 2) || misaligned(y, 2) || misaligned(residual, 2) ||
        misaligned(x_fp16, 8) || misaligned(xscale, 4) || misaligned(sum8, 4))
        return W4A16_ERR_ALIGNMENT;
    GemvArgs a = {};
    a.qweight[0] = qweight; a.scales[0] = H(scales); a.out[0] = H(y); a.rows[0] = N;
    a.q8 = q8; a.xscale = xscale; a.sum8 = sum8; a.x_fp16 = H(x_fp16); a.gamma = H(gamma);
    a.x_f32 = x_f32;
    a.residual = H(residual);
    a.K = K; a.units = N;
    if (misaligned(gamma, 8)) return W4A16_ERR_ALIGNMENT;
    if (num_peers < 0 || num_peers > 7 || (num_peers > 0 && !peers)) return W4A16_ERR_INVALID_ARG;
    for (int p = 0; p < num_peers; ++p) {
        if (!peers[p]) return W4A16_ERR_INVALID_ARG;
        if (misaligned(peers[p], 2)) return W4A16_ERR_ALIGNMENT;
        a.peer_out[p] = H(peers[p]);
    }
    a.num_peers = num_peers;
    return gemv_launch(kPlain, a, S(stream));
}

int w4a16_embed_lookup_w4a16(const uint32_t* embed_qweight, const void* embed_scales, const int32_t* d_token_ids,
                             void* out_hidden, const void* d_control, int num_tokens, w4a16_stream_t stream,
                             int hidden_size, int vocab_size) {
    if (!embed_qweight || !embed_scales || !out_hidden || num_tokens <= 0 || vocab_size <= 0) return W4A16_ERR_INVALID_ARG;
    if (!d_token_ids && !d_control) return W4A16_ERR_INVALID_ARG;
    if (hidden_size <= 0 || hidden_size % 128) return W4A16_ERR_SHAPE;
    if (misaligned(embed_qweight, 4) || misaligned(embed_scales, 2) || misaligned(out_hidden, 16) ||
        misaligned(d_token_ids, 4) || misaligned(d_control, 8))
        return W4A16_ERR_ALIGNMENT;
    if (int st = ensure_device_ready(nullptr)) return st;
    return embed_lookup(embed_qweight, H(embed_scales), d_token_ids, H(out_hidden), d_control, num_tokens, hidden_size,
                        vocab_size, S(stream));
}

// ---- token selection ----
int w4a16_sample_and_advance(const void* logits, float* sample_scratch_val, int32_t* sample_scratch_idx,
                             void* d_control, int32_t* d_token_out, w4a16_stream_t stream, int vocab_size) {
    if (!logits || !sample_scratch_val || !sample_scratch_idx || vocab_size <= 0) return W4A16_ERR_INVALID_ARG;
    if (misaligned(logits, 2) || misaligned(sample_scratch_val, 4) || misaligned(sample_scratch_idx, 4) ||
        misaligned(d_control, 8) || misaligned(d_token_out, 4))
        return W4A16_ERR_ALIGNMENT;
    if (int st = ensure_device_ready(nullptr)) return st;
    if (int st = sample_stage1(H(logits), sample_scratch_val, sample_scratch_idx, d_control, vocab_size, 0, S(stream)))
        return st;
    return sample_stage2(sample_scratch_val, sample_scratch_idx, sample_stage1_blocks(), d_control, d_token_out, S(stream));
}

int w4a16_sample_slots(int out_features) {
    if (out_features <= 0) return W4A16_ERR_INVALID_ARG;
    return gemv_sample_slots(out_features);
}

static int sample_candidates(const uint32_t* qweight, const void* scales, const int8_t* input_q8,
                             const float* input_scale, const int32_t* input_sum8, void* output_logits,
                             float* candidate_val, int32_t* candidate_idx, float* const* peer_val,
                             int32_t* const* peer_idx, int num_peers, const void* d_control, int index_offset,
                             int out_features, int in_features, w4a16_stream_t stream,
                             uint32_t* const* peer_flags = nullptr, uint32_t* local_flag = nullptr,
                             uint32_t* done_counter = nullptr, uint32_t* step_word = nullptr, int half_stride = 0) {
    if (!qweight || !scales || !input_q8 || !input_scale || !input_sum8 || !candidate_val || !candidate_idx ||
        out_features <= 0 || index_offset < 0)
        return W4A16_ERR_INVALID_ARG;
    if (num_peers < 0 || num_peers > 7 || (num_peers > 0 && (!peer_val || !peer_idx))) return W4A16_ERR_INVALID_ARG;
    if (int st = check_k(in_features)) return st;
    if (misaligned(qweight, 16) || misaligned(scales, 2) || misaligned(output_logits, 2) || misaligned(input_scale, 4) ||
        misaligned(input_sum8, 4) || misaligned(candidate_val, 4) || misaligned(candidate_idx, 4) ||
        misaligned(d_control, 8))
        return W4A16_ERR_ALIGNMENT;
    GemvArgs a = {};
    a.qweight[0] = qweight; a.scales[0] = H(scales); a.out[0] = H(output_logits); a.rows[0] = out_features;
    a.q8 = input_q8; a.xscale = input_scale; a.sum8 = input_sum8;
    a.K = in_features; a.units = out_features;
    a.sample_val = candidate_val; a.sample_idx = candidate_idx; a.sample_control = d_control;
    a.sample_index_offset = index_offset;
    for (int p = 0; p < num_peers; ++p) {
        if (!peer_val[p] || !peer_idx[p]) return W4A16_ERR_INVALID_ARG;
        if (misaligned(peer_val[p], 4) || misaligned(peer_idx[p], 4)) return W4A16_ERR_ALIGNMENT;
        a.sample_peer_val[p] = peer_val[p];
        a.sample_peer_idx[p] = peer_idx[p];
    }
    a.sample_num_peers = num_peers;
    if (local_flag != nullptr) {
        if (!done_counter || !step_word || half_stride < 0 || (num_peers > 0 && !peer_flags)) return W4A16_ERR_INVALID_ARG;
        if (misaligned(local_flag, 4) || misaligned(done_counter, 4) || misaligned(step_word, 4)) return W4A16_ERR_ALIGNMENT;
        a.sample_flag_local = local_flag;
        a.sample_done_counter = done_counter;
        a.sample_step_word = step_word;
        a.sample_half_stride = half_stride;
        for (int p = 0; p < num_peers; ++p) {
            if (!peer_flags[p]) return W4A16_ERR_INVALID_ARG;
            if (misaligned(peer_flags[p], 4)) return W4A16_ERR_ALIGNMENT;
            a.sample_peer_flag[p] = peer_flags[p];
        }
    }
    return gemv_launch(kPlain, a, S(stream));
}

int w4a16_gemv_w4a8_sample_one_launch(const uint32_t* qweight, const void* scales, const int8_t* input_q8,
                                      const float* input_scale, const int32_t* input_sum8, void* output_logits,
                                      float* sample_scratch_val, int32_t* sample_scratch_idx, uint32_t* d_counter,
                                      void* d_control, int32_t* d_token_out, int out_features, int in_features,
                                      w4a16_stream_t stream) {
    if (!qweight || !scales || !input_q8 || !input_scale || !input_sum8 || !sample_scratch_val || !sample_scratch_idx ||
        !d_counter || out_features <= 0)
        return W4A16_ERR_INVALID_ARG;
    if (int st = check_k(in_features)) return st;
    if (misaligned(qweight, 16) || misaligned(scales, 2) || misaligned(output_logits, 2) || misaligned(input_scale, 4) ||
        misaligned(input_sum8, 4) || misaligned(sample_scratch_val, 4) || misaligned(sample_scratch_idx, 4) ||
        misaligned(d_counter, 4) || misaligned(d_control, 8) || misaligned(d_token_out, 4))
        return W4A16_ERR_ALIGNMENT;
    GemvArgs a = {};
    a.qweight[0] = qweight; a.scales[0] = H(scales); a.out[0] = H(output_logits); a.rows[0] = out_features;
    a.q8 = input_q8; a.xscale = input_scale; a.sum8 = input_sum8;
    a.K = in_features; a.units = out_features;
    a.sample_val = sample_scratch_val; a.sample_idx = sample_scratch_idx; a.sample_control = d_control;
    a.sample_done_counter = d_counter;
    a.sample_finish_inline = 1; a.sample_control_rw = d_control; a.sample_token_out = d_token_out;
    return gemv_launch(kPlain, a, S(stream));
}

int w4a16_gemv_w4a8_sample_candidates(const uint32_t* qweight, const void* scales, const int8_t* input_q8,
                                      const float* input_scale, const int32_t* input_sum8, void* output_logits,
                                      float* candidate_val, int32_t* candidate_idx, const void* d_control,
                                      int index_offset, int out_features, int in_features, w4a16_stream_t stream) {
    return sample_candidates(qweight, scales, input_q8, input_scale, input_sum8, output_logits, candidate_val,
                             candidate_idx, nullptr, nullptr, 0, d_control, index_offset, out_features, in_features,
                             stream);
}

int w4a16_gemv_w4a8_sample_candidates_peers(const uint32_t* qweight, const void* scales, const int8_t* input_q8,
                                            const float* input_scale, const int32_t* input_sum8,
                                            float* candidate_val, int32_t* candidate_idx,
                                            float* const* peer_candidate_val, int32_t* const* peer_candidate_idx,
                                            int num_peers, const void* d_control, int index_offset, int out_features,
                                            int in_features, w4a16_stream_t stream) {
    return sample_candidates(qweight, scales, input_q8, input_scale, input_sum8, nullptr, candidate_val, candidate_idx,
                             peer_candidate_val, peer_candidate_idx, num_peers, d_control, index_offset, out_features,
                             in_features, stream);
}

int w4a16_gemv_w4a8_sample_candidates_signal(const uint32_t* qweight, const void* scales, const int8_t* input_q8,
                                             const float* input_scale, const int32_t* input_sum8,
                                             float* candidate_val, int32_t* candidate_idx,
                                             float* const* peer_candidate_val, int32_t* const* peer_candidate_idx,
                                             uint32_t* const* peer_flags, int num_peers, uint32_t* local_flag,
                                             uint32_t* done_counter, uint32_t* step_word, int half_stride,
                                             const void* d_control, int index_offset, int out_features,
                                             int in_features, w4a16_stream_t stream) {
    if (!local_flag) return W4A16_ERR_INVALID_ARG;
    return sample_candidates(qweight, scales, input_q8, input_scale, input_sum8, nullptr, candidate_val, candidate_idx,
                             peer_candidate_val, peer_candidate_idx, num_peers, d_control, index_offset, out_features,
                             in_features, stream, peer_flags, local_flag, done_counter, step_word, half_stride);
}

int w4a16_sample_finish_after_signals(const float* candidate_val, const int32_t* candidate_idx, int count,
                                      int half_stride, const uint32_t* flags, int num_flags,
                                      const uint32_t* step_word, int* d_status, void* d_control,
                                      int32_t* d_token_out, w4a16_stream_t stream) {
    if (!candidate_val || !candidate_idx || count <= 0 || half_stride < 0 || !flags || num_flags <= 0 || num_flags > 256 ||
        !step_word)
        return W4A16_ERR_INVALID_ARG;
    if (misaligned(candidate_val, 4) || misaligned(candidate_idx, 4) || misaligned(flags, 4) || misaligned(d_status, 4) ||
        misaligned(step_word, 4) ||
        misaligned(d_control, 8) || misaligned(d_token_out, 4))
        return W4A16_ERR_ALIGNMENT;
    if (int st = ensure_device_ready(nullptr)) return st;
    return sample_stage2_after_flags(candidate_val, candidate_idx, count, half_stride, flags, num_flags, step_word,
                                     d_status, d_control, d_token_out, S(stream));
}

int w4a16_sample_finish(const float* candidate_val, const int32_t* candidate_idx, int count, void* d_control,
                        int32_t* d_token_out, w4a16_stream_t stream) {
    if (!candidate_val || !candidate_idx || count <= 0) return W4A16_ERR_INVALID_ARG;
    if (misaligned(candidate_val, 4) || misaligned(candidate_idx, 4) || misaligned(d_control, 8) || misaligned(d_token_out, 4))
        return W4A16_ERR_ALIGNMENT;
    if (int st = ensure_device_ready(nullptr)) return st;
    return sample_stage2(candidate_val, candidate_idx, count, d_control, d_token_out, S(stream));
}

int w4a16_gemv_w4a8_sample_and_advance(const uint32_t* qweight, const void* scales, const int8_t* input_q8,
                                       const float* input_scale, const int32_t* input_sum8, void* output_logits,
                                       float* sample_scratch_val, int32_t* sample_scratch_idx, void* d_control,
                                       int32_t* d_token_out, int out_features, int in_features,
                                       w4a16_stream_t stream) {
    if (int st = w4a16_gemv_w4a8_sample_candidates(qweight, scales, input_q8, input_scale, input_sum8, output_logits,
                                                   sample_scratch_val, sample_scratch_idx, d_control, 0, out_features,
                                                   in_features, stream))
        return st;
    const int slots = gemv_sample_slots(out_features);
    if (slots < 0) return slots;
    return sample_stage2(sample_scratch_val, sample_scratch_idx, slots, d_control, d_token_out, S(stream));
}

int w4a16_gemv_w4a16(const uint32_t* qweight, const void* scales, const void* input_x, const void* residual,
                     void* output_y, int out_features, int in_features, w4a16_stream_t stream) {
    if (!input_x) return W4A16_ERR_INVALID_ARG;
    return gemv_plain(qweight, scales, input_x, nullptr, nullptr, nullptr, residual, output_y, out_features,
                      in_features, stream);
}

int w4a16_quantize_attn_heads_f32_to_q8_1(const float* attn_acc, void* attn_out_fp16_opt, int8_t* out_q8,
                                          float* out_scale, int32_t* out_sum8, int num_heads, int head_dim,
                                          w4a16_stream_t stream) {
    if (!attn_acc || !out_q8 || !out_scale || !out_sum8 || num_heads <= 0) return W4A16_ERR_INVALID_ARG;
    if (head_dim != 128) return W4A16_ERR_SHAPE;   // one head = one quantisation group of the W4 path
    if (misaligned(attn_acc, 16) || misaligned(attn_out_fp16_opt, 16) || misaligned(out_q8, 8) ||
        misaligned(out_scale, 4) || misaligned(out_sum8, 4))
        return W4A16_ERR_ALIGNMENT;
    if (int st = ensure_device_ready(nullptr)) return st;
    return quantize_heads_f32_to_q8_1(attn_acc, H(attn_out_fp16_opt), out_q8, out_scale, out_sum8, num_heads, S(stream));
}

int w4a16_gemv_attn_heads_f32_w4a16(const uint32_t* qweight, const void* scales, const float* attn_acc,
                                    const void* residual, void* output_y, int out_features, int in_features,
                                    w4a16_stream_t stream) {
    if (!attn_acc) return W4A16_ERR_INVALID_ARG;
    return gemv_plain(qweight, scales, nullptr, nullptr, nullptr, nullptr, residual, output_y, out_features,
                      in_features, stream, nullptr, nullptr, 0, attn_acc);
}

int w4a16_gemv_w4a8(const uint32_t* qweight, const void* scales, const int8_t* input_q8, const float* input_scale,
                    const int32_t* input_sum8, const void* residual, void* output_y, int out_features,
                    int in_features, w4a16_stream_t stream) {
    if (!input_q8 || !input_scale || !input_sum8) return W4A16_ERR_INVALID_ARG;
    return gemv_plain(qweight, scales, nullptr, input_q8, input_scale, input_sum8, residual, output_y, out_features,
                      in_features, stream);
}

int w4a16_gemv_w4a8_peers_signal(const uint32_t* qweight, const void* scales, const int8_t* input_q8,
                                 const float* input_scale, const int32_t* input_sum8, void* gathered_slice,
                                 void* const* peer_slices, uint32_t* const* peer_flags, int num_peers,
                                 uint32_t* local_flag, uint32_t* done_counter, uint32_t* step_word, int half_stride,
                                 int out_features, int in_features, w4a16_stream_t stream) {
    if (!qweight || !scales || !input_q8 || !input_scale || !input_sum8 || !gathered_slice || !local_flag ||
        !done_counter || !step_word || out_features <= 0 || half_stride < out_features)
        return W4A16_ERR_INVALID_ARG;
    if (int st = check_k(in_features)) return st;
    if (num_peers < 0 || num_peers > 7 || (num_peers > 0 && (!peer_slices || !peer_flags))) return W4A16_ERR_INVALID_ARG;
    if (misaligned(qweight, 16) || misaligned(scales, 2) || misaligned(gathered_slice, 2) || misaligned(input_scale, 4) ||
        misaligned(input_sum8, 4) || misaligned(local_flag, 4) || misaligned(done_counter, 4) || misaligned(step_word, 4))
        return W4A16_ERR_ALIGNMENT;
    GemvArgs a = {};
    a.qweight[0] = qweight; a.scales[0] = H(scales); a.out[0] = H(gathered_slice); a.rows[0] = out_features;
    a.q8 = input_q8; a.xscale = input_scale; a.sum8 = input_sum8;
    a.K = in_features; a.units = out_features;
    for (int p = 0; p < num_peers; ++p) {
        if (!peer_slices[p] || !peer_flags[p]) return W4A16_ERR_INVALID_ARG;
        if (misaligned(peer_slices[p], 2) || misaligned(peer_flags[p], 4)) return W4A16_ERR_ALIGNMENT;
        a.peer_out[p] = H(peer_slices[p]);
        a.sample_peer_flag[p] = peer_flags[p];
    }
    a.num_peers = num_peers;
    a.sample_flag_local = local_flag;
    a.sample_done_counter = done_counter;
    a.sample_step_word = step_word;
    a.sample_half_stride = half_stride;
    return gemv_launch(kPlain, a, S(stream));
}

int w4a16_gather_after_signals(const void* gathered, int half_stride, const uint32_t* flags, int num_flags,
                               const uint32_t* step_word, int* d_status, void* output, int num_elements,
                               w4a16_stream_t stream) {
    if (!gathered || !flags || !step_word || !output || num_flags <= 0 || num_flags > 256 || num_elements <= 0 ||
        half_stride < num_elements)
        return W4A16_ERR_INVALID_ARG;
    if (misaligned(gathered, 2) || misaligned(output, 2) || misaligned(flags, 4) || misaligned(step_word, 4) ||
        misaligned(d_status, 4))
        return W4A16_ERR_ALIGNMENT;
    if (int st = ensure_device_ready(nullptr)) return st;
    return gather_after_flags(H(gathered), half_stride, flags, num_flags, step_word, d_status, H(output), num_elements,
                              S(stream));
}

int w4a16_gemv_w4a8_peers(const uint32_t* qweight, const void* scales, const int8_t* input_q8,
                          const float* input_scale, const int32_t* input_sum8, void* output_y,
                          void* const* peer_outputs, int num_peers, int out_features, int in_features,
                          w4a16_stream_t stream) {
    if (!input_q8 || !input_scale || !input_sum8) return W4A16_ERR_INVALID_ARG;
    return gemv_plain(qweight, scales, nullptr, input_q8, input_scale, input_sum8, nullptr, output_y, out_features,
                      in_features, stream, nullptr, peer_outputs, num_peers);
}

static int fill_qkv(const w4a16_qkv_view* v, int nq, int nkv, int hd, const uint32_t* qw[3], const __half* sc[3],
                    __half* out[3], int rows[3]) {
    if (!v || !v->q_weight || !v->q_scale || !v->d_q || !v->k_weight || !v->k_scale || !v->d_k || !v->v_weight ||
        !v->v_scale || !v->d_v || nq <= 0 || nkv <= 0 || hd <= 0)
        return W4A16_ERR_INVALID_ARG;
    const void* ws[3] = {v->q_weight, v->k_weight, v->v_weight};
    const void* ss[3] = {v->q_scale, v->k_scale, v->v_scale};
    void* os[3] = {v->d_q, v->d_k, v->d_v};
    for (int t = 0; t < 3; ++t) {
        if (misaligned(ws[t], 4) || misaligned(ss[t], 2) || misaligned(os[t], 2)) return W4A16_ERR_ALIGNMENT;
        qw[t] = static_cast<const uint32_t*>(ws[t]);
        sc[t] = H(ss[t]);
        out[t] = H(os[t]);
    }
    rows[0] = nq * hd;
    rows[1] = nkv * hd;
    rows[2] = nkv * hd;
    return 0;
}

int w4a16_gemv_qkv_w4a8(const w4a16_qkv_view* view, const int8_t* input_q8, const float* input_scale,
                        const int32_t* input_sum8, w4a16_stream_t stream, int in_features, int num_q_heads,
                        int num_kv_heads, int head_dim) {
    if (!input_q8 || !input_scale || !input_sum8) return W4A16_ERR_INVALID_ARG;
    if (int st = check_k(in_features)) return st;
    if (misaligned(input_scale, 4) || misaligned(input_sum8, 4)) return W4A16_ERR_ALIGNMENT;
    GemvArgs a = {};
    if (int st = fill_qkv(view, num_q_heads, num_kv_heads, head_dim, a.qweight, a.scales, a.out, a.rows)) return st;
    a.q8 = input_q8; a.xscale = input_scale; a.sum8 = input_sum8;
    a.K = in_features;
    a.units = a.rows[0] + a.rows[1] + a.rows[2];
    return gemv_launch(kQkv, a, S(stream));
}

static int gemv_swiglu(const uint32_t* qweight, const void* scales, const void* x_fp16, const int8_t* q8,
                       const float* xscale, const int32_t* sum8, void* out, int hidden, int inter,
                       w4a16_stream_t stream, const void* gamma = nullptr, int8_t* q8_out = nullptr,
                       float* xscale_out = nullptr, int32_t* sum8_out = nullptr) {
    if (!qweight || !scales || !out || inter <= 0) return W4A16_ERR_INVALID_ARG;
    if (int st = check_k(hidden)) return st;
    if (misaligned(qweight, 4) || misaligned(scales, 2) || misaligned(out, 2) || misaligned(x_fp16, 8) ||
        misaligned(xscale, 4) || misaligned(sum8, 4))
        return W4A16_ERR_ALIGNMENT;
    GemvArgs a = {};
    a.qweight[0] = qweight; a.scales[0] = H(scales); a.out[0] = H(out); a.rows[0] = 2 * inter;
    a.q8 = q8; a.xscale = xscale; a.sum8 = sum8; a.x_fp16 = H(x_fp16); a.gamma = H(gamma);
    a.K = hidden; a.units = inter;
    a.q8_out = q8_out; a.xscale_out = xscale_out; a.sum8_out = sum8_out;
    if (misaligned(gamma, 8) || misaligned(xscale_out, 4) || misaligned(sum8_out, 4)) return W4A16_ERR_ALIGNMENT;
    return gemv_launch(kSwiglu, a, S(stream));
}

int w4a16_gemv_dual_gate_up_swiglu_w4a16(const uint32_t* gate_up_qweight, const void* gate_up_scales,
                                         const void* input_x, void* output_mlp, int hidden_size,
                                         int intermediate_size, w4a16_stream_t stream) {
    if (!input_x) return W4A16_ERR_INVALID_ARG;
    return gemv_swiglu(gate_up_qweight, gate_up_scales, input_x, nullptr, nullptr, nullptr, output_mlp, hidden_size,
                       intermediate_size, stream);
}

int w4a16_gemv_dual_gate_up_swiglu_w4a8(const uint32_t* gate_up_qweight, const void* gate_up_scales,
                                        const int8_t* input_q8, const float* input_scale, const int32_t* input_sum8,
                                        void* output_mlp, int hidden_size, int intermediate_size,
                                        w4a16_stream_t stream) {
    if (!input_q8 || !input_scale || !input_sum8) return W4A16_ERR_INVALID_ARG;
    return gemv_swiglu(gate_up_qweight, gate_up_scales, nullptr, input_q8, input_scale, input_sum8, output_mlp,
                       hidden_size, intermediate_size, stream);
}

int w4a16_gemv_rmsnorm_w4a16(const uint32_t* qweight, const void* scales, const void* input_x, const void* gamma,
                             const void* residual, void* output_y, int out_features, int in_features,
                             w4a16_stream_t stream) {
    if (!input_x) return W4A16_ERR_INVALID_ARG;
    return gemv_plain(qweight, scales, input_x, nullptr, nullptr, nullptr, residual, output_y, out_features,
                      in_features, stream, gamma);
}

int w4a16_gemv_qkv_rmsnorm_w4a16(const w4a16_qkv_view* view, const void* input_x, const void* gamma,
                                 w4a16_stream_t stream, int in_features, int num_q_heads, int num_kv_heads,
                                 int head_dim) {
    if (!input_x) return W4A16_ERR_INVALID_ARG;
    if (int st = check_k(in_features)) return st;
    if (misaligned(input_x, 8) || misaligned(gamma, 8)) return W4A16_ERR_ALIGNMENT;
    GemvArgs a = {};
    if (int st = fill_qkv(view, num_q_heads, num_kv_heads, head_dim, a.qweight, a.scales, a.out, a.rows)) return st;
    a.x_fp16 = H(input_x); a.gamma = H(gamma);
    a.K = in_features;
    a.units = a.rows[0] + a.rows[1] + a.rows[2];
    return gemv_launch(kQkv, a, S(stream));
}

int w4a16_gemv_dual_gate_up_swiglu_rmsnorm_w4a16(const uint32_t* gate_up_qweight, const void* gate_up_scales,
                                                 const void* input_x, const void* gamma, void* output_mlp,
                                                 int hidden_size, int intermediate_size, w4a16_stream_t stream) {
    if (!input_x) return W4A16_ERR_INVALID_ARG;
    return gemv_swiglu(gate_up_qweight, gate_up_scales, input_x, nullptr, nullptr, nullptr, output_mlp, hidden_size,
                       intermediate_size, stream, gamma);
}

int w4a16_gemv_dual_gate_up_swiglu_rmsnorm_w4a16_q8_1(const uint32_t* gate_up_qweight, const void* gate_up_scales,
                                                      const void* input_x, const void* gamma, void* output_mlp,
                                                      int8_t* output_q8, float* output_scale, int32_t* output_sum8,
                                                      int hidden_size, int intermediate_size, w4a16_stream_t stream) {
    if (!input_x || !output_q8 || !output_scale || !output_sum8) return W4A16_ERR_INVALID_ARG;
    return gemv_swiglu(gate_up_qweight, gate_up_scales, input_x, nullptr, nullptr, nullptr, output_mlp, hidden_size,
                       intermediate_size, stream, gamma, output_q8, output_scale, output_sum8);
}

int w4a16_gemm_prefill_w4a16(const uint32_t* qweight, const void* scales, const void* input_x, const void* residual,
                             void* output_y, int M, int N, int K, w4a16_stream_t stream, int sm_count) {
    (void)sm_count;
    if (!qweight || !scales || !input_x || !output_y || M <= 0 || N <= 0) return W4A16_ERR_INVALID_ARG;
    if (int st = check_k(K)) return st;
    if (misaligned(qweight, 4) || misaligned(scales, 2) || misaligned(input_x, 16) || misaligned(output_y, 2) ||
        misaligned(residual, 2))
        return W4A16_ERR_ALIGNMENT;
    GemmArgs g = {};
    g.qweight[0] = qweight; g.scales[0] = H(scales); g.out[0] = H(output_y); g.rows[0] = N;
    g.x = H(input_x); g.residual = H(residual);
    g.M = M; g.K = K; g.mode = kPlain;
    return gemm_launch(g, S(stream));
}

int w4a16_gemm_prefill_w4a16_block(const uint32_t* qweight, const void* scales, const void* input_x,
                                   const void* residual, void* output_y, int ldc, void* const* peer_outputs,
                                   int num_peers, int M, int N, int K, w4a16_stream_t stream) {
    if (!qweight || !scales || !input_x || !output_y || M <= 0 || N <= 0 || ldc < N) return W4A16_ERR_INVALID_ARG;
    if (num_peers < 0 || num_peers > 7 || (num_peers > 0 && !peer_outputs)) return W4A16_ERR_INVALID_ARG;
    if (int st = check_k(K)) return st;
    if (misaligned(qweight, 4) || misaligned(scales, 2) || misaligned(input_x, 16) || misaligned(output_y, 2) ||
        misaligned(residual, 2))
        return W4A16_ERR_ALIGNMENT;
    GemmArgs g = {};
    g.qweight[0] = qweight; g.scales[0] = H(scales); g.out[0] = H(output_y); g.rows[0] = N;
    g.x = H(input_x); g.residual = H(residual);
    g.M = M; g.K = K; g.mode = kPlain; g.ldc = ldc;
    for (int p = 0; p < num_peers; ++p) {
        if (!peer_outputs[p]) return W4A16_ERR_INVALID_ARG;
        if (misaligned(peer_outputs[p], 2)) return W4A16_ERR_ALIGNMENT;
        g.peer_out[p] = H(peer_outputs[p]);
    }
    g.num_peers = num_peers;
    return gemm_launch(g, S(stream));
}

int w4a16_gemm_prefill_qkv_w4a16(const w4a16_qkv_view* view, const void* input_x, int M, w4a16_stream_t stream,
                                 int in_features, int num_q_heads, int num_kv_heads, int head_dim, int sm_count) {
    (void)sm_count;
    if (!input_x || M <= 0) return W4A16_ERR_INVALID_ARG;
    if (int st = check_k(in_features)) return st;
    if (misaligned(input_x, 16)) return W4A16_ERR_ALIGNMENT;
    GemmArgs g = {};
    if (int st = fill_qkv(view, num_q_heads, num_kv_heads, head_dim, g.qweight, g.scales, g.out, g.rows)) return st;
    g.x = H(input_x);
    g.M = M; g.K = in_features; g.mode = kQkv;
    return gemm_launch(g, S(stream));
}

int w4a16_gemm_prefill_dual_gate_up_swiglu_w4a16(const uint32_t* gate_up_qweight, const void* gate_up_scales,
                                                 const void* input_x, void* output_mlp, int M,
                                                 w4a16_stream_t stream, int hidden_size, int intermediate_size) {
    if (!gate_up_qweight || !gate_up_scales || !input_x || !output_mlp || M <= 0 || intermediate_size <= 0)
        return W4A16_ERR_INVALID_ARG;
    if (int st = check_k(hidden_size)) return st;
    if (misaligned(gate_up_qweight, 4) || misaligned(gate_up_scales, 2) || misaligned(input_x, 16) ||
        misaligned(output_mlp, 2))
        return W4A16_ERR_ALIGNMENT;
    GemmArgs g = {};
    g.qweight[0] = gate_up_qweight; g.scales[0] = H(gate_up_scales); g.out[0] = H(output_mlp);
    g.rows[0] = 2 * intermediate_size;
    g.x = H(input_x);
    g.M = M; g.K = hidden_size; g.mode = kSwiglu;
    return gemm_launch(g, S(stream));
}

int w4a16_gemv_group_dots(const uint32_t* qweight, const int8_t* input_q8, const int32_t* input_sum8,
                          int32_t* out_dots, int out_features, int in_features, w4a16_stream_t stream) {
    if (!qweight || !input_q8 || !input_sum8 || !out_dots || out_features <= 0) return W4A16_ERR_INVALID_ARG;
    if (int st = check_k(in_features)) return st;
    if (misaligned(qweight, 4) || misaligned(input_sum8, 4) || misaligned(out_dots, 4)) return W4A16_ERR_ALIGNMENT;
    return gemv_group_dots(qweight, input_q8, input_sum8, out_dots, out_features, in_features, S(stream));
}

int w4a16_debug_counter(int which, unsigned int* out) {
    if (!out) return W4A16_ERR_INVALID_ARG;
    if (int st = ensure_device_ready(nullptr)) return st;
    if (which == 0) return gemm_tc_timeouts(out);
    if (which == 1) return gemv_copy_timeouts(out);
    return W4A16_ERR_INVALID_ARG;
}

}  // extern "C"
