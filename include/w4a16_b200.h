/*
 * w4a16_b200 -- C ABI of the B200 (sm_100a) W4A16 group-128 contraction kernels.
 *
 * One entry point per launch function of the reference engine's include/kernels.cuh
 * that lies on the W4 projection path, with the same parameter order and meaning.
 * Differences from the reference functions, all forced by the C boundary:
 *   - `half*` is `void*` (fp16 storage), `cudaStream_t` is `w4a16_stream_t`;
 *   - QKVProjectionView is passed by pointer to an identical 9-pointer struct;
 *   - instead of throwing std::runtime_error (reference include/tensor.cuh:11-23) every
 *     function returns a status: 0 = ok, >0 = the cudaError_t of the failed CUDA call,
 *     <0 = one of the W4A16_ERR_* argument errors below.  Nothing is launched when an
 *     argument error is returned.
 *
 * Contract shared by all launchers (as the reference's): the caller owns every buffer,
 * all pointers are device pointers valid on the current device, launchers allocate
 * nothing, keep no per-call state, do not synchronise, and may be stream-captured into
 * a CUDA graph after one eager call on the device (that first call sets kernel
 * attributes).  `residual` may alias `output_y` (the engine calls it in place).
 *
 * Data layout (reference include/quant_primitives.cuh:20-26, tools/export_qwen25.py:42-78):
 *   qweight  uint32 [N][K/8], row-major, linear in K; word w of a row holds elements
 *            8w..8w+7 as nibbles q0 | q4<<4 | q1<<8 | q5<<12 | q2<<16 | q6<<20 | q3<<24 | q7<<28,
 *            weight = (q - 8) * scale;
 *   scales   fp16 [N][K/128];
 *   Q8_1 x   int8 q8[K], fp32 scale[K/128], int32 sum8[K/8] (= -8 * sum of each octet).
 * K must be a multiple of 256 (the exporter asserts it).
 */
#ifndef W4A16_B200_H
#define W4A16_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define W4A16_API __attribute__((visibility("default")))
#else
#define W4A16_API
#endif

typedef struct CUstream_st* w4a16_stream_t; /* == cudaStream_t */

enum {
    W4A16_OK = 0,
    W4A16_ERR_INVALID_ARG = -1, /* null pointer, non-positive size */
    W4A16_ERR_SHAPE = -2,       /* K not a multiple of 256, dims the kernels cannot tile */
    W4A16_ERR_ALIGNMENT = -3,   /* a pointer below the minimum alignment of its type */
    W4A16_ERR_NO_DEVICE = -4,   /* no sm_100 device current */
    W4A16_ERR_TOO_LARGE = -5    /* a size beyond a stated maximum */
};

/* Mirror of reference include/kernels.cuh:23-27 (QKVProjectionView). */
typedef struct w4a16_qkv_view {
    const void* q_weight; const void* q_scale; void* d_q;
    const void* k_weight; const void* k_scale; void* d_k;
    const void* v_weight; const void* v_scale; void* d_v;
} w4a16_qkv_view;

/* Library version (major*10000 + minor*100 + patch). */
W4A16_API int w4a16_version(void);

/* Text for a status returned by any function here. Never NULL. */
W4A16_API const char* w4a16_status_string(int status);

/*
 * Optional one-time set-up for the current device: queries the SM count and raises the
 * dynamic shared-memory limit of every kernel.  The launchers do the same lazily on
 * their first call per device; call this (or make one eager call) before stream capture.
 */
W4A16_API int w4a16_init(void);

/*
 * Run-time options: process-wide integers read when a launcher is called (so a launch captured into a CUDA
 * graph keeps the values of capture time).  With the defaults every launch configuration is a function of
 * the call's arguments and the device alone.  w4a16_set_option returns W4A16_ERR_INVALID_ARG for an unknown
 * option or a value outside its range.
 */
enum {
    W4A16_OPT_PDL = 1,               /* 1 (default): programmatic dependent launch, so that the next kernel's weight
                                        prefetch overlaps this kernel's tail; 0: plain stream-ordered launches */
    W4A16_OPT_SIGNAL_WAIT_SPINS = 2, /* polls (about 0.2 us apart) that w4a16_sample_finish_after_signals and
                                        w4a16_gather_after_signals spend on a peer's flag, and a CTA of the persistent
                                        sweep on another CTA's counter or tagged word, before giving up and reporting
                                        it (*d_status, w4a16_sweep_status); default 1 << 22, about a second */
    W4A16_OPT_GEMV_FORM = 3,         /* how the batch-1 GEMV brings its weights on chip: 0 (default) the measured
                                        best, which is 1; 1 register-held 16-byte streaming loads issued before the
                                        wait for the previous kernel, 2 bulk copies (cp.async.bulk) into shared
                                        memory (K slices of long plain projections on the CTAs of a cluster).
                                        Same output bits in every form. */
    W4A16_OPT_GEMM_MIN_TOKENS_TENSOR_CORE = 4, /* token count from which the M-token contraction runs on the
                                        tensor cores; 0 (default): the measured crossover (4 or 5 tokens) */
    W4A16_OPT_GEMM_FORM = 5,         /* tensor-core form of the M-token contraction: 0 (default) chosen by token
                                        count, 1 one CTA per tile, 2 CTA pairs (cta_group::2) */
    W4A16_OPT_GEMM_MMA_MAX_TOKENS = 6, /* largest token count that takes the weight-streaming mma.sync kernel instead of
                                        the tcgen05 kernels: 0 (default) the measured crossover, 1 never, n up to n */
    W4A16_OPT_COUNT_ = 7
};
W4A16_API int w4a16_set_option(int option, int value);
W4A16_API int w4a16_get_option(int option);

/* ---- Q8_1 activation quantisers ------------------------------------------------ */

/* reference include/kernels.cuh:50-57 launch_quantize_fp16_to_q8_1
 * (src/kernels/rmsnorm_rope.cu:273-314).  num_elements: multiple of 128. */
W4A16_API int w4a16_quantize_fp16_to_q8_1(const void* input_x, int8_t* out_q8, float* out_scale,
                                          int32_t* out_sum8, int num_elements, w4a16_stream_t stream);

/* reference include/kernels.cuh:39-48 launch_rmsnorm_q8_1
 * (src/kernels/rmsnorm_rope.cu:156-267).  output_fp16_opt may be NULL. */
W4A16_API int w4a16_rmsnorm_q8_1(const void* input, const void* gamma, void* output_fp16_opt,
                                 int8_t* out_q8, float* out_scale, int32_t* out_sum8,
                                 w4a16_stream_t stream, int hidden_size);

/*
 * Q8_1 of the attention output as the reference's flash-decode combine step produces it for the O projection
 * (src/kernels/attention_gqa.cu:258-310, the out_q8 / out_scale / out_sum8 arguments of
 * launch_attention_gqa_flash_decode, include/kernels.cuh:177-193), as an operator of its own so that an
 * attention kernel which is not part of this library can hand its result to the W4 path with the reference's
 * bits: one quantisation group per head, taken from the fp32 accumulator before it is rounded to fp16,
 * d = max(max|acc| / 127, 1e-8), q = clamp(rn(acc / d), -127, 127) -- a division per element, so the bytes can
 * differ from w4a16_quantize_fp16_to_q8_1 applied to fp16(acc).  attn_acc: fp32 [num_heads][head_dim],
 * 16-byte aligned; attn_out_fp16_opt (may be NULL): fp16(acc), the reference's attn_out.  head_dim must be
 * 128 (W4A16_ERR_SHAPE otherwise): a head is a quantisation group.
 */
W4A16_API int w4a16_quantize_attn_heads_f32_to_q8_1(const float* attn_acc, void* attn_out_fp16_opt, int8_t* out_q8,
                                                    float* out_scale, int32_t* out_sum8, int num_heads,
                                                    int head_dim, w4a16_stream_t stream);

/* ---- batch-1 decode GEMV ------------------------------------------------------- */

/*
 * The O projection straight from the attention accumulators: the same quantisation as
 * w4a16_quantize_attn_heads_f32_to_q8_1, done by every CTA of the GEMV in its prologue (in_features / 128
 * heads of 128), then w4a16_gemv_w4a8 -- same output bits as that pair of calls, one launch less
 * (src/engine.cu:389-402 issues the attention kernel with the Q8_1 outputs and then launch_gemv_w4a8).
 * attn_acc: fp32 [in_features], 16-byte aligned.
 */
W4A16_API int w4a16_gemv_attn_heads_f32_w4a16(const uint32_t* qweight, const void* scales, const float* attn_acc,
                                              const void* residual, void* output_y, int out_features,
                                              int in_features, w4a16_stream_t stream);

/* reference include/kernels.cuh:60-69 launch_gemv_w4a16 (src/kernels/gemv_w4a16.cu:636-746,
 * 960-979): fp16 activations, quantised to Q8_1 inside the kernel.  residual may be NULL. */
W4A16_API int w4a16_gemv_w4a16(const uint32_t* qweight, const void* scales, const void* input_x,
                               const void* residual, void* output_y, int out_features,
                               int in_features, w4a16_stream_t stream);

/* reference include/kernels.cuh:71-82 launch_gemv_w4a8 (src/kernels/gemv_w4a16.cu:74-121,
 * 264-381, 864-891): pre-quantised Q8_1 activations.  residual may be NULL. */
W4A16_API int w4a16_gemv_w4a8(const uint32_t* qweight, const void* scales, const int8_t* input_q8,
                              const float* input_scale, const int32_t* input_sum8,
                              const void* residual, void* output_y, int out_features,
                              int in_features, w4a16_stream_t stream);

/*
 * w4a16_gemv_w4a8 whose epilogue also stores the output slice into up to 7 more buffers -- the same
 * slice position in the gathered output of every PEER GPU, whose memory is mapped into this process
 * (CUDA IPC / symmetric memory); the stores are plain stores that travel over NVLink.  With the rows of
 * a large projection (lm_head) split over the GPUs of a node, this replaces the all-gather that would
 * follow the GEMV; the caller orders the ranks afterwards (a barrier on the stream) before reading.
 * No counterpart in the reference, which is single-GPU.  peer_outputs[i] points at element 0 of THIS
 * rank's slice inside peer i's buffer.
 */
W4A16_API int w4a16_gemv_w4a8_peers(const uint32_t* qweight, const void* scales, const int8_t* input_q8,
                                    const float* input_scale, const int32_t* input_sum8, void* output_y,
                                    void* const* peer_outputs, int num_peers, int out_features,
                                    int in_features, w4a16_stream_t stream);

/*
 * The row-split GEMV without a barrier between the ranks (no reference counterpart).  Every rank's launch stores
 * its slice -- with 16-byte stores -- into half (step & 1) of ITS OWN gathered vector and of every peer's
 * (gathered_slice / peer_slices[i] point at this rank's first element inside half 0 of each buffer; the halves are
 * half_stride elements apart), and when its last CTA is through it writes the step number to *step_word, to
 * *local_flag and, behind one system-scope fence, to peer_flags[i] -- this rank's slot in GPU i's flag array.
 * step = *step_word + 1; *step_word and *done_counter are device words, zero at first, that only this sequence of
 * launches touches: nothing about a step comes from the host, so the pair of calls replays as a CUDA graph.
 * Two halves are used in turn because a fast rank's next slice must not land in the vector a slow rank's readers
 * still use; a rank reaches step s + 2 only after w4a16_gather_after_signals of step s + 1 has seen every
 * rank's flag, i.e. after every rank has finished reading step s.
 * w4a16_gather_after_signals waits until flags[0 .. num_flags) all show this rank's step (bounded by
 * W4A16_OPT_SIGNAL_WAIT_SPINS; on expiry *d_status = 1 + the rank it missed and the copy runs on what is there)
 * and copies num_elements of half (step & 1) of the gathered vector into `output`.
 * Needs 16-byte aligned weights and in_features <= 2048.  Ranks on DIFFERENT GPUs only: launches that wait for
 * one another must not share a GPU.
 */
W4A16_API int w4a16_gemv_w4a8_peers_signal(const uint32_t* qweight, const void* scales, const int8_t* input_q8,
                                           const float* input_scale, const int32_t* input_sum8, void* gathered_slice,
                                           void* const* peer_slices, uint32_t* const* peer_flags, int num_peers,
                                           uint32_t* local_flag, uint32_t* done_counter, uint32_t* step_word,
                                           int half_stride, int out_features, int in_features, w4a16_stream_t stream);
W4A16_API int w4a16_gather_after_signals(const void* gathered, int half_stride, const uint32_t* flags, int num_flags,
                                         const uint32_t* step_word, int* d_status, void* output, int num_elements,
                                         w4a16_stream_t stream);

/* ---- embedding lookup on the W4 table ---------------------------------------------------- */
/*
 * reference include/kernels.cuh launch_embed_lookup_w4a16 (src/kernels/rmsnorm_rope.cu:15-69): row `token` of
 * the packed table (the tied lm_head matrix) dequantised to fp16, (q - 8) * scale with one fp16 rounding
 * (include/quant_primitives.cuh:92-115).  Token i is d_token_ids[i] if d_token_ids is given, else the
 * control block's token_id; ids outside [0, vocab_size) read row 0, as in the reference.  out_hidden:
 * fp16 [num_tokens][hidden_size], 16-byte aligned; hidden_size a multiple of 128.
 */
W4A16_API int w4a16_embed_lookup_w4a16(const uint32_t* embed_qweight, const void* embed_scales,
                                       const int32_t* d_token_ids, void* out_hidden, const void* d_control,
                                       int num_tokens, w4a16_stream_t stream, int hidden_size, int vocab_size);

/* ---- token selection after lm_head ------------------------------------------------------ */
/* Same layout as the reference's DeviceControlBlock (include/tensor.cuh:28-34); lives in device memory. */
typedef struct w4a16_sample_control {
    int32_t token_id;      /* written by the samplers */
    int32_t seq_pos;       /* Philox counter word 1; incremented by the samplers */
    float temperature;     /* <= 1e-5: greedy argmax; else Gumbel-max on logit / temperature */
    uint32_t reserved;
    uint64_t rng_seed;     /* Philox key; advanced by 0x9E3779B97F4A7C15 per token */
} w4a16_sample_control;

/*
 * reference include/kernels.cuh:210-219 launch_sample_and_advance (src/kernels/sampling.cu:60-232): token =
 * index of the largest score, lowest index among equals; score = logit, or logit / temperature + Gumbel noise
 * from Philox-4x32-10 keyed by (rng_seed; vocabulary index, seq_pos); writes the token into the control
 * block and *d_token_out (either may be NULL) and advances seq_pos and rng_seed.  The two scratch arrays hold
 * 256 entries, as in the reference.  Arithmetic is IEEE fp32 with the accurate logf (the reference's
 * fast-math build uses approximations, so at temperature > 0 the two can pick different tokens when two scores
 * agree to the last bits; greedy selection is identical).
 */
W4A16_API int w4a16_sample_and_advance(const void* logits, float* sample_scratch_val, int32_t* sample_scratch_idx,
                                       void* d_control, int32_t* d_token_out, w4a16_stream_t stream,
                                       int vocab_size);

/*
 * lm_head and token selection in one pass over the weights (no reference counterpart; replaces the pair
 * launch_gemv_w4a8 + launch_sample_and_advance at src/engine.cu:440-450): every CTA of the GEMV scores the
 * rows it produced and leaves ONE (score, index) candidate; w4a16_sample_finish reduces the candidates,
 * writes the token and advances the control block.  The fp16 logits are stored only if output_logits is not
 * NULL.  The token equals w4a16_sample_and_advance on the logits w4a16_gemv_w4a8 would write.
 * candidate_val / candidate_idx: w4a16_sample_slots(out_features) entries.  index_offset is the vocabulary
 * index of row 0 -- with the rows of lm_head split over GPUs every rank passes its slab's first row, the
 * ranks exchange their candidates (8 bytes per slot instead of the logits) and one w4a16_sample_finish over
 * all of them gives the token.  Needs 16-byte aligned weights and in_features <= 2048 (W4A16_ERR_SHAPE).
 */
W4A16_API int w4a16_sample_slots(int out_features);
W4A16_API int w4a16_gemv_w4a8_sample_candidates(const uint32_t* qweight, const void* scales, const int8_t* input_q8,
                                                const float* input_scale, const int32_t* input_sum8,
                                                void* output_logits, float* candidate_val, int32_t* candidate_idx,
                                                const void* d_control, int index_offset, int out_features,
                                                int in_features, w4a16_stream_t stream);
/* The same, with the candidates also stored at the given addresses: this rank's place in the gathered candidate
 * arrays of up to 7 PEER GPUs (memory mapped into this process; plain stores over NVLink).  With every rank
 * doing so, a barrier over the ranks replaces the exchange and w4a16_sample_finish runs on the gathered arrays. */
W4A16_API int w4a16_gemv_w4a8_sample_candidates_peers(const uint32_t* qweight, const void* scales,
                                                      const int8_t* input_q8, const float* input_scale,
                                                      const int32_t* input_sum8, float* candidate_val,
                                                      int32_t* candidate_idx, float* const* peer_candidate_val,
                                                      int32_t* const* peer_candidate_idx, int num_peers,
                                                      const void* d_control, int index_offset, int out_features,
                                                      int in_features, w4a16_stream_t stream);
/*
 * Peer stores plus a completion signal, so that no barrier kernel is needed between the ranks' GEMVs and the
 * reduction, and nothing about a step comes from the host (the pair can sit in a replayed CUDA graph):
 * *step_word (device, zero at first) counts this rank's finished launches.  A launch calls its step number
 * *step_word + 1, stores its candidates into half (step & 1) of every candidate array (each array is
 * 2 * half_stride entries: a fast rank's next stores must not land in the half a slow rank is still
 * reducing), and when its last CTA is through writes the step number to *step_word, to *local_flag and --
 * behind one system-scope fence -- to peer_flags[i], this rank's slot in GPU i's flag array.  *done_counter is a device
 * word, zero at first, that only this sequence of launches touches.
 * w4a16_sample_finish_after_signals reads this rank's *step_word, waits until flags[0 .. num_flags) all show that
 * step (bounded: about a second, then *d_status = 1 + the rank it missed and the reduction runs on what is
 * there), and reduces half (step & 1) of the gathered arrays like w4a16_sample_finish; `count` entries per half.
 * All ranks must take part in every step.  Ranks on DIFFERENT GPUs only: launches that wait for one another
 * must not share a GPU.
 */
W4A16_API int w4a16_gemv_w4a8_sample_candidates_signal(const uint32_t* qweight, const void* scales,
                                                       const int8_t* input_q8, const float* input_scale,
                                                       const int32_t* input_sum8, float* candidate_val,
                                                       int32_t* candidate_idx, float* const* peer_candidate_val,
                                                       int32_t* const* peer_candidate_idx,
                                                       uint32_t* const* peer_flags, int num_peers,
                                                       uint32_t* local_flag, uint32_t* done_counter,
                                                       uint32_t* step_word, int half_stride, const void* d_control,
                                                       int index_offset, int out_features, int in_features,
                                                       w4a16_stream_t stream);
W4A16_API int w4a16_sample_finish_after_signals(const float* candidate_val, const int32_t* candidate_idx, int count,
                                                int half_stride, const uint32_t* flags, int num_flags,
                                                const uint32_t* step_word, int* d_status, void* d_control,
                                                int32_t* d_token_out, w4a16_stream_t stream);
W4A16_API int w4a16_sample_finish(const float* candidate_val, const int32_t* candidate_idx, int count,
                                  void* d_control, int32_t* d_token_out, w4a16_stream_t stream);
/* Both steps on one GPU; the scratch arrays hold w4a16_sample_slots(out_features) entries. */
W4A16_API int w4a16_gemv_w4a8_sample_and_advance(const uint32_t* qweight, const void* scales, const int8_t* input_q8,
                                                 const float* input_scale, const int32_t* input_sum8,
                                                 void* output_logits, float* sample_scratch_val,
                                                 int32_t* sample_scratch_idx, void* d_control, int32_t* d_token_out,
                                                 int out_features, int in_features, w4a16_stream_t stream);

/* The same in ONE launch: the GEMV's CTA that finishes last reduces all candidates, writes the token and advances
 * the control block.  *d_counter is a device word, zero before the first call, that only this sequence of
 * launches touches (it wraps back to zero in every launch). */
W4A16_API int w4a16_gemv_w4a8_sample_one_launch(const uint32_t* qweight, const void* scales, const int8_t* input_q8,
                                                const float* input_scale, const int32_t* input_sum8,
                                                void* output_logits, float* sample_scratch_val,
                                                int32_t* sample_scratch_idx, uint32_t* d_counter, void* d_control,
                                                int32_t* d_token_out, int out_features, int in_features,
                                                w4a16_stream_t stream);

/* reference include/kernels.cuh:84-94 launch_gemv_qkv_w4a8 (src/kernels/gemv_w4a16.cu:123-194,
 * 387-513, 893-926): q, k and v projections in one launch. */
W4A16_API int w4a16_gemv_qkv_w4a8(const w4a16_qkv_view* view, const int8_t* input_q8,
                                  const float* input_scale, const int32_t* input_sum8,
                                  w4a16_stream_t stream, int in_features, int num_q_heads,
                                  int num_kv_heads, int head_dim);

/* reference include/kernels.cuh:96-104 launch_gemv_dual_gate_up_swiglu_w4a16
 * (src/kernels/gemv_w4a16.cu:752-858, 981-999): rows 2i / 2i+1 = gate_i / up_i,
 * output_mlp[i] = silu(gate_i . x) * (up_i . x). */
W4A16_API int w4a16_gemv_dual_gate_up_swiglu_w4a16(const uint32_t* gate_up_qweight,
                                                   const void* gate_up_scales, const void* input_x,
                                                   void* output_mlp, int hidden_size,
                                                   int intermediate_size, w4a16_stream_t stream);

/* reference include/kernels.cuh:106-116 launch_gemv_dual_gate_up_swiglu_w4a8
 * (src/kernels/gemv_w4a16.cu:196-258, 519-630, 928-958). */
W4A16_API int w4a16_gemv_dual_gate_up_swiglu_w4a8(const uint32_t* gate_up_qweight,
                                                  const void* gate_up_scales, const int8_t* input_q8,
                                                  const float* input_scale, const int32_t* input_sum8,
                                                  void* output_mlp, int hidden_size,
                                                  int intermediate_size, w4a16_stream_t stream);

/*
 * fp16-input GEMV that brings its own scratch.  No counterpart in the reference.
 * Same arguments and same output bits as w4a16_gemv_w4a16, but the activation is quantised
 * to Q8_1 once, into a fixed array inside the library's device image (50 176 bytes per GPU,
 * held until the process exits), and the GEMV reads it from there.  It is meant for callers
 * that have no spare device buffer to pass and are not allowed to allocate one -- an engine
 * whose memory all went into one start-up arena, a plugin host that bans allocation calls on
 * the inference path.  The function itself allocates nothing, on the host or the device.
 *   - in_features above 32768 is refused with W4A16_ERR_TOO_LARGE (nothing is launched).
 *   - The first call on each device looks up the array's device address; make that first
 *     call before any stream capture.
 *   - All calls share the one array: two calls that may run at the same time on the GPU
 *     (different streams, no ordering between them) race on it.  Calls on one stream, or
 *     otherwise ordered, are safe; leftovers of an earlier call are never read.
 */
W4A16_API int w4a16_gemv_w4a16_static_scratch(const uint32_t* qweight, const void* scales,
                                              const void* input_x, const void* residual,
                                              void* output_y, int out_features, int in_features,
                                              w4a16_stream_t stream);

/* ---- fused forms: RMSNorm + Q8_1 inside the GEMV -------------------------------------- */
/*
 * Each of these gives the same output bits as the pair of calls it replaces -- the reference's
 * launch_rmsnorm_q8_1 (include/kernels.cuh:39-48, src/engine.cu:367-371, 414-418, 434-438) followed
 * by the W4A8 GEMV -- with one launch less: every CTA normalises and quantises the fp16 vector
 * for itself.  gamma == NULL skips the normalisation (plain quantisation, as w4a16_gemv_w4a16).
 */
W4A16_API int w4a16_gemv_rmsnorm_w4a16(const uint32_t* qweight, const void* scales, const void* input_x,
                                       const void* gamma, const void* residual, void* output_y,
                                       int out_features, int in_features, w4a16_stream_t stream);
W4A16_API int w4a16_gemv_qkv_rmsnorm_w4a16(const w4a16_qkv_view* view, const void* input_x, const void* gamma,
                                           w4a16_stream_t stream, int in_features, int num_q_heads,
                                           int num_kv_heads, int head_dim);
W4A16_API int w4a16_gemv_dual_gate_up_swiglu_rmsnorm_w4a16(const uint32_t* gate_up_qweight,
                                                           const void* gate_up_scales, const void* input_x,
                                                           const void* gamma, void* output_mlp, int hidden_size,
                                                           int intermediate_size, w4a16_stream_t stream);

/*
 * The same launch, which in addition leaves the Q8_1 form of output_mlp in output_q8 [intermediate],
 * output_scale [intermediate/128] and output_sum8 [intermediate/8] -- what launch_quantize_fp16_to_q8_1
 * (include/kernels.cuh:50-57, src/engine.cu:441-444) would compute from output_mlp, bit for bit -- so the
 * down projection can start from w4a16_gemv_w4a8 without a quantiser launch in between.  The CTAs of one
 * group of 128 outputs form a thread-block cluster and agree on the group's scale through distributed
 * shared memory.  intermediate_size must be a multiple of 128 (W4A16_ERR_SHAPE otherwise).
 * No reference counterpart.
 */
W4A16_API int w4a16_gemv_dual_gate_up_swiglu_rmsnorm_w4a16_q8_1(const uint32_t* gate_up_qweight,
                                                                const void* gate_up_scales, const void* input_x,
                                                                const void* gamma, void* output_mlp,
                                                                int8_t* output_q8, float* output_scale,
                                                                int32_t* output_sum8, int hidden_size,
                                                                int intermediate_size, w4a16_stream_t stream);

/* ---- M-token contraction (small-M decode batches and prefill) ------------------- */

/* reference include/kernels.cuh:119-130 launch_gemm_prefill_w4a16
 * (src/kernels/gemm_prefill.cu:319-386, 616-640): Y[M][N] = X[M][K] . dequant(W)^T (+ residual),
 * fp16 in, fp32 accumulate, fp16 out.  sm_count is accepted for signature parity and ignored. */
W4A16_API int w4a16_gemm_prefill_w4a16(const uint32_t* qweight, const void* scales, const void* input_x,
                                       const void* residual, void* output_y, int M, int N, int K,
                                       w4a16_stream_t stream, int sm_count);

/*
 * w4a16_gemm_prefill_w4a16 writing a COLUMN BLOCK of a wider matrix: output_y (and residual) point at the
 * block's first element inside an [M][ldc] matrix, ldc >= N.  With the weight rows of a large projection
 * split over the GPUs of a node every rank produces one such block of the full [M][N_total] output; the
 * block is also stored at up to 7 peer addresses -- its place in every other GPU's matrix, mapped into this
 * process -- so that the all-gather of the blocks is done by the epilogue's stores over NVLink while other
 * tiles are still being computed; the caller orders the ranks afterwards.  Peer stores need the tensor-core
 * form (16-byte aligned weights and activations; W4A16_ERR_SHAPE otherwise).  No reference counterpart.
 */
W4A16_API int w4a16_gemm_prefill_w4a16_block(const uint32_t* qweight, const void* scales, const void* input_x,
                                             const void* residual, void* output_y, int ldc,
                                             void* const* peer_outputs, int num_peers, int M, int N, int K,
                                             w4a16_stream_t stream);

/* reference include/kernels.cuh:132-142 launch_gemm_prefill_qkv_w4a16
 * (src/kernels/gemm_prefill.cu:392-489, 642-666). */
W4A16_API int w4a16_gemm_prefill_qkv_w4a16(const w4a16_qkv_view* view, const void* input_x, int M,
                                           w4a16_stream_t stream, int in_features, int num_q_heads,
                                           int num_kv_heads, int head_dim, int sm_count);

/* reference include/kernels.cuh:144-153 launch_gemm_prefill_dual_gate_up_swiglu_w4a16
 * (src/kernels/gemm_prefill.cu:495-610, 668-684). */
W4A16_API int w4a16_gemm_prefill_dual_gate_up_swiglu_w4a16(const uint32_t* gate_up_qweight,
                                                           const void* gate_up_scales,
                                                           const void* input_x, void* output_mlp, int M,
                                                           w4a16_stream_t stream, int hidden_size,
                                                           int intermediate_size);

/* ---- decode projection sweep -------------------------------------------------------- */

/*
 * The W4 projections of one batch-1 decode pass, in the order the reference engine issues
 * them (reference src/engine.cu:361-451, execute_gqa_decode_layer / execute_decode_pass),
 * captured once into a CUDA graph as the engine does (src/engine.cu:453-470).  Per layer:
 *   rmsnorm_q8_1(h) -> QKV GEMV -> [attention stand-in: Q8_1 of the q output]
 *   -> O GEMV (+h, in place) -> rmsnorm_q8_1(h) -> gate_up GEMV + SwiGLU
 *   -> Q8_1 of the MLP activation -> down GEMV (+h, in place).
 * Attention, RoPE and the KV cache are not part of this library; the attention output is
 * replaced by the q projection so that every GEMV keeps a true data dependency.
 * All pointers are device pointers owned by the caller and must stay valid while the
 * sweep object lives.  The object owns one CUDA graph and no device memory.
 */
typedef struct w4a16_layer_weights {
    const void* input_norm_gamma;          /* fp16 [hidden] */
    const void* q_weight;  const void* q_scale;
    const void* k_weight;  const void* k_scale;
    const void* v_weight;  const void* v_scale;
    const void* o_weight;  const void* o_scale;
    const void* post_norm_gamma;           /* fp16 [hidden] */
    const void* gate_up_weight; const void* gate_up_scale;
    const void* down_weight;    const void* down_scale;
} w4a16_layer_weights;

typedef struct w4a16_sweep_desc {
    int num_layers, hidden_size, intermediate_size, num_q_heads, num_kv_heads, head_dim;
    const w4a16_layer_weights* layers;     /* host array [num_layers], copied */
    void* workspace;                       /* device, >= w4a16_sweep_workspace_bytes(), 256-byte aligned */
    int flags;                             /* W4A16_SWEEP_* */
} w4a16_sweep_desc;

enum {
    W4A16_SWEEP_SEPARATE = 0,    /* the reference's launch sequence: 8 launches per layer */
    W4A16_SWEEP_FUSE_NORM = 1,   /* RMSNorm + Q8_1 inside the QKV and gate_up GEMVs */
    W4A16_SWEEP_FUSE_QUANT_O = 2,    /* Q8_1 of the attention output inside the O GEMV */
    W4A16_SWEEP_FUSE_QUANT_DOWN = 4, /* Q8_1 of the MLP activation inside the down GEMV */
    W4A16_SWEEP_FUSE_ALL = 7,    /* 4 launches per layer, same output bits */
    W4A16_SWEEP_QUANT_IN_GATE_UP = 16, /* the gate_up launch writes the Q8_1 form of its own output (clusters
                                    of four CTAs share one group of 128): no quantiser launch and no
                                    re-quantisation in front of down; needs intermediate % 128 == 0; takes
                                    precedence over FUSE_QUANT_DOWN; same output bits */
    W4A16_SWEEP_PUBLISH_SUMSQ = 32, /* FUSE_NORM | FUSE_QUANT_O, and the O and down GEMVs add the squares of their
                                    outputs into partial sums that the next RMSNorm prologue reads instead of
                                    reducing; same output bits */
    W4A16_SWEEP_PUBLISH_AMAX = 64,  /* FUSE_NORM | FUSE_QUANT_O, and the gate_up GEMV leaves the |max| of every group of
                                    128 outputs (atomicMax) so that the down GEMV quantises its fp16 input element by
                                    element, without a reduction and without a quantiser launch (4 launches per
                                    layer); same output bits */
    W4A16_SWEEP_PERSISTENT = 8   /* the whole pass as ONE persistent kernel (one CTA per SM): weights of all
                                    layers stream through a shared-memory ring while the CTAs exchange the
                                    small activation vectors through tagged 8-byte words; needs
                                    hidden <= 4096, intermediate and q width <= 9216, 16-byte aligned weights */
};

typedef struct w4a16_sweep w4a16_sweep;

/* Bytes of device workspace the sweep needs (hidden state, q/k/v, MLP activation, Q8_1 scratch). */
W4A16_API int64_t w4a16_sweep_workspace_bytes(int hidden_size, int intermediate_size, int num_q_heads,
                                              int num_kv_heads, int head_dim);

/* Builds the sweep: one eager pass on `stream`, then graph capture.  Synchronises `stream`. */
W4A16_API int w4a16_sweep_create(const w4a16_sweep_desc* desc, w4a16_stream_t stream, w4a16_sweep** out);
W4A16_API int w4a16_sweep_destroy(w4a16_sweep* sweep);

/* Kernels launched per w4a16_sweep_run_* call. */
W4A16_API int w4a16_sweep_launches(const w4a16_sweep* sweep);

/* One sweep with the hidden state in device memory: h_in fp16 [hidden] -> h_out fp16 [hidden]
 * (two small device copies around the graph launch).  Asynchronous on `stream`. */
W4A16_API int w4a16_sweep_run_device(w4a16_sweep* sweep, const void* d_h_in, void* d_h_out,
                                     w4a16_stream_t stream);

/* Same with HOST buffers (pinned for true asynchrony): copies h_in to the device, runs the
 * sweep, copies the result back.  Asynchronous on `stream`; synchronise before reading. */
W4A16_API int w4a16_sweep_run_host(w4a16_sweep* sweep, const void* h_h_in, void* h_h_out,
                                   w4a16_stream_t stream);

/* 0 after a clean pass; nonzero if a bounded wait of the persistent kernel ran out (1 ring, 2 exchange):
 * the pass's output is then invalid, and this call re-bases the exchange (device idle, tags, counters and the
 * status word cleared, launch count and tags restarted) so that the next pass starts clean -- call it after
 * every pass whose result matters.  Synchronises the device.  Always 0 for graph-mode sweeps. */
W4A16_API int w4a16_sweep_status(w4a16_sweep* sweep, int* out);

/* Device pointer of a workspace region, for tests: 0 hidden, 1 q, 2 k, 3 v, 4 mlp. */
W4A16_API void* w4a16_sweep_buffer(const w4a16_sweep* sweep, int which);

/* ---- the reference's `.qwenbin` weight container --------------------------------------- */
/*
 * Host-side reader of the file format the reference engine loads (include/config.cuh:75-170,
 * docs/SPECIFICATION.md, written by tools/export_qwen25.py): versions 1 and 2, W4A16 group 128.  The file's
 * bytes stay the caller's (mmap or a read buffer); nothing is allocated or copied.  Every offset is checked
 * against the file size and the 256-byte tensor alignment before an address is formed.
 */
typedef struct w4a16_qwenbin_header {
    uint32_t version, hidden_size, intermediate_size, num_layers, num_q_heads, num_kv_heads, head_dim, vocab_size,
        max_seq_len, quant_type, tie_word_embeddings;
    float rms_norm_eps, rope_theta;
    uint64_t file_bytes;
} w4a16_qwenbin_header;
typedef struct w4a16_qwenbin_globals {
    const void* embed_weight;  const void* embed_scale;      /* [vocab][hidden] packed, fp16 [vocab][hidden/128] */
    const void* final_norm_gamma;                            /* fp16 [hidden] */
    const void* lm_head_weight; const void* lm_head_scale;   /* the embedding tensors when tied */
} w4a16_qwenbin_globals;
typedef struct w4a16_qwenbin_biases { const void* q_bias; const void* k_bias; const void* v_bias; } w4a16_qwenbin_biases;

W4A16_API int w4a16_qwenbin_parse(const void* file_bytes, uint64_t nbytes, w4a16_qwenbin_header* header);
/*
 * Fills layers[0 .. num_layers) (the table w4a16_sweep_create takes), `globals` and `biases[num_layers]` (either
 * may be NULL) with base + offset, `base` being where the caller put a copy of the whole file, e.g. in device
 * memory as the reference does (src/engine.cu:85-348); base must be 256-byte aligned.  W4A16_ERR_INVALID_ARG
 * for a bad magic / version / offset, W4A16_ERR_SHAPE for dimensions or a quantisation the path does not take.
 */
W4A16_API int w4a16_qwenbin_tensors(const void* file_bytes, uint64_t nbytes, const void* base,
                                    w4a16_layer_weights* layers, int max_layers, w4a16_qwenbin_globals* globals,
                                    w4a16_qwenbin_biases* biases);

/* ---- diagnostics ----------------------------------------------------------------- */

/*
 * Per-group integer partial sums of the decode GEMV, D[n][g] = sum over the 128 elements
 * of group g of (q[n][k] - 8) * q8[k], computed with the same dp4a routine the GEMV
 * kernels use (the quantity reference include/quant_primitives.cuh:28-32 accumulates).
 * No counterpart launcher in the reference; it exists so the integer intermediates can
 * be compared bit for bit.  out_dots: int32 [N][K/128].
 */
W4A16_API int w4a16_gemv_group_dots(const uint32_t* qweight, const int8_t* input_q8,
                                    const int32_t* input_sum8, int32_t* out_dots, int out_features,
                                    int in_features, w4a16_stream_t stream);

/*
 * Counters of bounded device-side waits that ran out, kept on the current device; each count means that a
 * launch gave up waiting and its output is invalid (0 in normal operation).  which = 0: barrier waits of the
 * tensor-core kernels; 1: waits of the batch-1 GEMV for its bulk copies.  Synchronises the device.
 */
W4A16_API int w4a16_debug_counter(int which, unsigned int* out);

#ifdef __cplusplus
}
#endif
#endif /* W4A16_B200_H */
