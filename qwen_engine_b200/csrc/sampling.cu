// Token selection after the lm_head projection: the stand-alone two-stage sampler (replaces the
// reference's launch_sample_and_advance, src/kernels/sampling.cu:60-232) and the second stage that also
// finishes the fused form, where the lm_head GEMV leaves one (score, index) candidate per CTA
// (gemv_decode.cu) and the fp16 logits never have to be read back.
#include "sampling.cuh"
#include "w4a16_common.cuh"
#include "w4a16_internal.hpp"

namespace w4 {
namespace {

constexpr int kStage1Blocks = 256, kStage1Threads = 256;   // the reference's launch shape (sampling.cu:215-216)

__global__ void __launch_bounds__(kStage1Threads) sample_stage1_kernel(const __half* __restrict__ logits,
                                                                        float* __restrict__ part_val,
                                                                        int32_t* __restrict__ part_idx,
                                                                        const SampleControl* __restrict__ control,
                                                                        int vocab, int index_offset) {
    __shared__ float s_v[32];
    __shared__ int32_t s_i[32];
    pdl_release_dependents();
    pdl_wait_prior_grids();
    float temperature = 0.0f;
    uint64_t seed = 0;
    uint32_t seq_pos = 0;
    if (control != nullptr) {
        temperature = control->temperature;
        seed = control->rng_seed;
        seq_pos = static_cast<uint32_t>(control->seq_pos);
    }
    float best = kSampleFloor;
    int32_t best_idx = 0;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < vocab; i += gridDim.x * blockDim.x) {
        const float v = sample_score(__half2float(logits[i]), static_cast<uint32_t>(i + index_offset), temperature, seed, seq_pos);
        sample_take(best, best_idx, v, i + index_offset);
    }
    sample_block_reduce(best, best_idx, s_v, s_i);
    if (threadIdx.x == 0) {
        part_val[blockIdx.x] = best;
        part_idx[blockIdx.x] = best_idx;
    }
}

// One CTA over all candidates; writes the token and advances the control block like the reference
// (sampling.cu:190-202): token_id, seq_pos + 1, rng_seed + 0x9E3779B97F4A7C15.
__global__ void __launch_bounds__(256) sample_stage2_kernel(const float* __restrict__ part_val,
                                                            const int32_t* __restrict__ part_idx, int count,
                                                            SampleControl* __restrict__ control,
                                                            int32_t* __restrict__ token_out) {
    __shared__ float s_v[32];
    __shared__ int32_t s_i[32];
    pdl_release_dependents();
    pdl_wait_prior_grids();
    float best = kSampleFloor;
    int32_t best_idx = 0x7FFFFFFF;
    for (int i = threadIdx.x; i < count; i += blockDim.x) sample_take(best, best_idx, part_val[i], part_idx[i]);
    sample_block_reduce(best, best_idx, s_v, s_i);
    if (threadIdx.x == 0) {
        if (best_idx == 0x7FFFFFFF) best_idx = 0;   // no candidate at all
        if (control != nullptr) {
            control->token_id = best_idx;
            control->seq_pos += 1;
            control->rng_seed += 0x9E3779B97F4A7C15ull;
        }
        if (token_out != nullptr) *token_out = best_idx;
    }
}

}  // namespace

int sample_stage1_blocks() { return kStage1Blocks; }

int sample_stage1(const __half* logits, float* part_val, int32_t* part_idx, const void* control, int vocab,
                  int index_offset, cudaStream_t stream) {
    return static_cast<int>(launch_kernel(sample_stage1_kernel, dim3(kStage1Blocks), dim3(kStage1Threads), 0, stream,
                                          pdl_enabled(), logits, part_val, part_idx,
                                          static_cast<const SampleControl*>(control), vocab, index_offset));
}

int sample_stage2(const float* part_val, const int32_t* part_idx, int count, void* control, int32_t* token_out,
                  cudaStream_t stream) {
    return static_cast<int>(launch_kernel(sample_stage2_kernel, dim3(1), dim3(256), 0, stream, pdl_enabled(), part_val,
                                          part_idx, count, static_cast<SampleControl*>(control), token_out));
}

}  // namespace w4
