// Internal C++ interface between the C-ABI translation unit and the kernel files.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <utility>

#include <cstdint>

#include "../../include/w4a16_b200.h"

namespace w4 {

// Per-process switches and per-device facts.
struct DeviceInfo {
    int sm_count = 0;
    int cc_major = 0;
    bool ready = false;
};
int ensure_device_ready(const DeviceInfo** out);  // lazy per-device set-up; returns a status
bool pdl_enabled();
int option(int which);                             // current value of a W4A16_OPT_* run-time option

// One launch with (optionally) the programmatic-serialisation attribute and thread-block cluster dimensions.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                         cudaStream_t stream, bool pdl, dim3 cluster, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (pdl) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster.x * cluster.y * cluster.z > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = cluster.x;
        attr[n].val.clusterDim.y = cluster.y;
        attr[n].val.clusterDim.z = cluster.z;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 bool pdl, Args&&... args) {
    return launch_kernel_cluster(kernel, grid, block, smem, stream, pdl, dim3(1, 1, 1), std::forward<Args>(args)...);
}

// ---- Q8_1 quantisers (q8_1_quantize.cu) ----
int quantize_fp16_to_q8_1(const __half* x, int8_t* q8, float* scale, int32_t* sum8, int n, cudaStream_t stream);
int rmsnorm_q8_1(const __half* in, const __half* gamma, __half* out_opt, int8_t* q8, float* scale, int32_t* sum8,
                 int hidden, cudaStream_t stream);
int quantize_heads_f32_to_q8_1(const float* acc, __half* out_fp16_opt, int8_t* q8, float* scale, int32_t* sum8,
                               int heads, cudaStream_t stream);
int quantize_set_attributes();

// ---- decode GEMV (gemv_decode.cu) ----
enum GemvMode { kPlain = 0, kQkv = 1, kSwiglu = 2 };

constexpr int kSumsqSlots = 8;   // partial sums a producer spreads its double atomics over

struct GemvArgs {
    // PLAIN / SWIGLU use index 0 only; QKV uses q, k, v in 0, 1, 2.
    const uint32_t* qweight[3];
    const __half* scales[3];
    __half* out[3];
    int rows[3];  // weight rows of each tensor
    // activation: either pre-quantised Q8_1 or fp16 (quantised in the kernel's prologue)
    const int8_t* q8;
    const float* xscale;
    const int32_t* sum8;
    const __half* x_fp16;
    const __half* gamma;     // with x_fp16: RMSNorm gain applied before the quantiser (null = no norm)
    const float* x_f32;      // PLAIN only: fp32 attention accumulators, one group of 128 per head, quantised in the
                             // prologue as the reference's flash-decode epilogue does (division by the scale)
    const __half* residual;  // PLAIN only, may be null, may alias out[0]
    // PLAIN only: the same output slice is also stored into these buffers (peer GPUs' memory mapped into
    // this process: plain stores travel over NVLink)
    __half* peer_out[7];
    int num_peers;
    // SWIGLU only, all three or none: the Q8_1 form of the output vector, written by the same launch
    // (clusters of four CTAs = one group of 128 outputs; needs units % 128 == 0)
    int8_t* q8_out;
    float* xscale_out;
    int32_t* sum8_out;
    // PLAIN only, streaming form: token selection in the epilogue.  Every CTA leaves its best (score, index)
    // candidate in sample_val / sample_idx [gemv_sample_slots()]; out[0] may then be null (logits not stored).
    float* sample_val;
    int32_t* sample_idx;
    const void* sample_control;   // SampleControl (temperature, seed, position) in device memory, may be null
    int sample_index_offset;      // added to the row number: vocabulary index of row 0 (row-split lm_head)
    // the same candidates are also stored at these addresses (the rank's place in every peer GPU's gathered
    // candidate arrays, mapped into this process)
    float* sample_peer_val[7];
    int32_t* sample_peer_idx[7];
    int sample_num_peers;
    // optional completion signal, safe under CUDA-graph replay (nothing about it comes from the host per step):
    // *sample_step_word counts this rank's finished launches.  A launch reads it, calls its own step
    // number word + 1, stores its candidates into half (step & 1) of every array (arrays are
    // 2 * sample_half_stride long), and when its last CTA is through writes the step number to the step word,
    // to sample_flag_local and (behind one system-scope fence) to every sample_peer_flag -- this rank's slot in the flag
    // array of each GPU.  sample_done_counter is a zero-initialised device word that wraps back to zero.
    uint32_t* sample_step_word;
    uint32_t* sample_flag_local;
    uint32_t* sample_peer_flag[7];
    uint32_t* sample_done_counter;
    int sample_half_stride;
    // optional, single GPU: the launch's last CTA (counted in sample_done_counter, no step word) reduces all
    // candidates itself, writes the token here / into the control block and advances the block -- no second launch
    int32_t* sample_token_out;
    void* sample_control_rw;
    int sample_finish_inline;
    // Hand-offs between the launches of a decode pass (all optional): a producer publishes the reductions its
    // consumer would otherwise redo in every CTA, on the critical path between two dependent launches.
    //   amax_out   SWIGLU: max |output| (the fp16 value, as float bits) of every group of 128 outputs, by atomicMax;
    //              the words must be zero when the launch starts
    //   amax_in    PLAIN, x_fp16 without gamma: those maxima for x; the prologue quantises without reducing
    //   sumsq_out  PLAIN: squares of the fp16 outputs added (double) into kSumsqSlots partial sums, slot = CTA % slots;
    //              zero when the launch starts
    //   sumsq_in   x_fp16 with gamma: the partial sums of x's squares; the prologue skips its own reduction
    //   clear_words / clear_count  words CTA 0 zeroes after its wait for the prior grid (the scratch of a LATER launch)
    uint32_t* amax_out;
    const uint32_t* amax_in;
    double* sumsq_out;
    const double* sumsq_in;
    uint32_t* clear_words;
    int clear_count;
    int K;
    int units;  // outputs produced: rows (PLAIN, QKV total) or row pairs (SWIGLU)
    // filled in by the planner
    int units_per_cta;
    int ksplit;
    int steps_per_split;
    int vec_ok;
};
int gemv_launch(GemvMode mode, GemvArgs args, cudaStream_t stream);
int gemv_group_dots(const uint32_t* qweight, const int8_t* q8, const int32_t* sum8, int32_t* out, int N, int K,
                    cudaStream_t stream);
int gemv_set_attributes();
int gemv_copy_timeouts(unsigned int* out);   // bounded waits of the bulk-copy GEMV that ran out, on the current device
int gemv_sample_slots(int out_features);   // candidates the sampling epilogue writes for a matrix of that height

// ---- embedding lookup (embed_lookup.cu) ----
int embed_lookup(const uint32_t* qweight, const __half* scales, const int32_t* token_ids, __half* out,
                 const void* control, int num_tokens, int hidden, int vocab, cudaStream_t stream);

// ---- token selection (sampling.cu) ----
int sample_stage1_blocks();
int sample_stage1(const __half* logits, float* part_val, int32_t* part_idx, const void* control, int vocab,
                  int index_offset, cudaStream_t stream);
int sample_stage2(const float* part_val, const int32_t* part_idx, int count, void* control, int32_t* token_out,
                  cudaStream_t stream);
int sample_stage2_after_flags(const float* part_val, const int32_t* part_idx, int count, int half_stride,
                              const uint32_t* flags, int num_flags, const uint32_t* step_word, int* status,
                              void* control, int32_t* token_out, cudaStream_t stream);

int gather_after_flags(const __half* gathered, int half_stride, const uint32_t* flags, int num_flags,
                       const uint32_t* step_word, int* status, __half* out, int n, cudaStream_t stream);

// ---- M-token contraction (gemm_prefill.cu) ----
struct GemmArgs {
    const uint32_t* qweight[3];
    const __half* scales[3];
    __half* out[3];
    int rows[3];
    const __half* x;         // [M][K]
    const __half* residual;  // [M][N] or null; may alias out[0]
    int M;
    int K;
    int mode;  // GemvMode values
    // PLAIN only: row stride of out[0] / residual in elements (0 = rows[0]): a column block of a wider [M][ldc]
    // matrix, e.g. one rank's slice of an output split by weight rows over several GPUs
    int ldc;
    // PLAIN only, tensor-core form: the same block is also stored at these addresses (its place in every peer
    // GPU's [M][ldc] matrix, mapped into this process; plain stores over NVLink)
    __half* peer_out[7];
    int num_peers;
};
int gemm_launch(GemmArgs args, cudaStream_t stream);
int gemm_set_attributes();
// tensor-core (tcgen05) form of the same contraction (gemm_tc.cu)
bool gemm_tc_supported(const GemmArgs& g);
int gemm_tc_launch(const GemmArgs& g, int sm_count, cudaStream_t stream);
int gemm_tc_set_attributes();
int gemm_tc_timeouts(unsigned int* out);

// ---- persistent one-kernel decode sweep (sweep_persistent.cu) ----
struct PSweepArgs {
    const void* layers;   // device array of the kernel's per-layer pointer table
    int num_layers, H, I, qdim, kvdim;
    const __half* h_in;   // plain fp16 [H]
    __half* h_out;        // plain fp16 [H] (may alias h_in)
    uint2* ll_h_attn;     // [H/2]     tagged words published by the O projection
    uint2* ll_h_down;     // [H/2]     ... by the down projection
    uint2* ll_q;          // [qdim/2]
    uint2* ll_mlp;        // [I/2]
    __half* k_out;        // plain [kvdim]
    __half* v_out;        // plain [kvdim]
    uint32_t epoch;       // tags of this launch are epoch + stage + 1
    uint32_t* counters;   // [4 * num_layers] at 32-byte spacing: CTAs that have published each stage, ever
    uint32_t counter_target;   // value a stage counter reaches when all CTAs of THIS launch have published
    int* status;          // 0 ok; 1 ring wait ran out; 2 tag poll ran out
    unsigned poll_limit;  // polls a CTA spends on another CTA's counter or tagged word before it gives up
};
size_t psweep_layer_bytes();
bool psweep_supported(int H, int I, int qdim, int kvdim);
int psweep_set_attributes();
void psweep_fill_layer(void* dst, const w4a16_layer_weights& L);
int psweep_launch(const PSweepArgs& args, int sm_count, cudaStream_t stream);

}  // namespace w4
