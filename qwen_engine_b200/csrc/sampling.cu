// Token selection after the lm_head projection: the stand-alone two-stage sampler (replaces the
// reference's launch_sample_and_advance, src/kernels/sampling.cu:60-232) and the second stage that also
// finishes the fused form, where the lm_head GEMV leaves one (score, index) candidate per CTA
// (gemv_decode.cu) and the fp16 logits never have to be read back.
#include <algorithm>

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

// The same reduction for candidates that other GPUs store into this GPU's memory: first wait (bounded) until
// every rank's flag shows this rank's own step number (all ranks produce one token per step, in lockstep) --
// that rank's lm_head launch has stored all its candidates (gemv_decode.cu) --
// so no separate barrier kernel is needed between the GEMV and the reduction.  A wait that runs out sets
// *status to 1 + the rank it waited for and the reduction goes ahead on whatever is there.
__global__ void __launch_bounds__(256) sample_stage2_after_flags_kernel(const float* __restrict__ part_val,
                                                                        const int32_t* __restrict__ part_idx, int count,
                                                                        int half_stride, const uint32_t* flags, int num_flags,
                                                                        const uint32_t* step_word, int* status,
                                                                        SampleControl* __restrict__ control,
                                                                        int32_t* __restrict__ token_out, uint32_t spin_limit) {
    __shared__ float s_v[32];
    __shared__ int32_t s_i[32];
    pdl_release_dependents();
    pdl_wait_prior_grids();
    // the step this rank's own lm_head launch (earlier on the stream) has just finished
    const uint32_t step = *reinterpret_cast<const volatile uint32_t*>(step_word);
    part_val += static_cast<size_t>(step & 1u) * half_stride;
    part_idx += static_cast<size_t>(step & 1u) * half_stride;
    if (static_cast<int>(threadIdx.x) < num_flags) {
        const uint32_t* f = flags + threadIdx.x;
        bool seen = false;
        for (uint32_t spin = 0; spin < spin_limit; ++spin) {     // W4A16_OPT_SIGNAL_WAIT_SPINS: about a second by default
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
            if (static_cast<int32_t>(v - step) >= 0) { seen = true; break; }   // step numbers only grow (wrap-safe)
            __nanosleep(spin < 64 ? 20 : 200);
        }
        if (!seen && status != nullptr) atomicExch(status, 1 + static_cast<int>(threadIdx.x));
    }
    __syncthreads();
    float best = kSampleFloor;
    int32_t best_idx = 0x7FFFFFFF;
    for (int i = threadIdx.x; i < count; i += blockDim.x) {
        // written by other GPUs: read past the (non-coherent) L1
        const float v = __ldcg(part_val + i);
        const int32_t ix = __ldcg(part_idx + i);
        sample_take(best, best_idx, v, ix);
    }
    sample_block_reduce(best, best_idx, s_v, s_i);
    if (threadIdx.x == 0) {
        if (best_idx == 0x7FFFFFFF) best_idx = 0;
        if (control != nullptr) {
            control->token_id = best_idx;
            control->seq_pos += 1;
            control->rng_seed += 0x9E3779B97F4A7C15ull;
        }
        if (token_out != nullptr) *token_out = best_idx;
    }
}

// The consumer side of the signalled row split for whole vectors (logits): waits (bounded) until every rank's flag
// shows this rank's own step number, then copies half (step & 1) of the gathered vector -- written by all GPUs'
// GEMV epilogues -- into a plain output vector.  Every CTA polls the flags itself (a handful of words), then
// copies its share with 16-byte loads that bypass the non-coherent L1.
__global__ void __launch_bounds__(256) gather_after_flags_kernel(const __half* __restrict__ gathered, int half_stride,
                                                                 const uint32_t* flags, int num_flags,
                                                                 const uint32_t* step_word, int* status,
                                                                 __half* __restrict__ out, int n, uint32_t spin_limit) {
    pdl_release_dependents();
    pdl_wait_prior_grids();
    const uint32_t step = *reinterpret_cast<const volatile uint32_t*>(step_word);
    if (static_cast<int>(threadIdx.x) < num_flags) {
        const uint32_t* f = flags + threadIdx.x;
        bool seen = false;
        for (uint32_t spin = 0; spin < spin_limit; ++spin) {
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
            if (static_cast<int32_t>(v - step) >= 0) { seen = true; break; }
            __nanosleep(spin < 64 ? 20 : 200);
        }
        if (!seen && status != nullptr) atomicExch(status, 1 + static_cast<int>(threadIdx.x));
    }
    __syncthreads();
    const __half* src = gathered + static_cast<size_t>(step & 1u) * half_stride;
    const bool vec = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0;
    const int stride = gridDim.x * blockDim.x * 8;
    for (int i = (blockIdx.x * blockDim.x + threadIdx.x) * 8; i < n; i += stride) {
        if (vec && i + 8 <= n) {
            *reinterpret_cast<uint4*>(out + i) = __ldcg(reinterpret_cast<const uint4*>(src + i));
        } else {
            for (int j = i; j < min(i + 8, n); ++j)
                out[j] = __ushort_as_half(__ldcg(reinterpret_cast<const unsigned short*>(src + j)));
        }
    }
}

}  // namespace

int gather_after_flags(const __half* gathered, int half_stride, const uint32_t* flags, int num_flags,
                       const uint32_t* step_word, int* status, __half* out, int n, cudaStream_t stream) {
    const int grid = std::max(1, std::min(64, (n + 2047) / 2048));
    return static_cast<int>(launch_kernel(gather_after_flags_kernel, dim3(grid), dim3(256), 0, stream, pdl_enabled(), gathered,
                                          half_stride, flags, num_flags, step_word, status, out, n,
                                          static_cast<uint32_t>(option(W4A16_OPT_SIGNAL_WAIT_SPINS))));
}

int sample_stage2_after_flags(const float* part_val, const int32_t* part_idx, int count, int half_stride,
                              const uint32_t* flags, int num_flags, const uint32_t* step_word, int* status,
                              void* control, int32_t* token_out, cudaStream_t stream) {
    return static_cast<int>(launch_kernel(sample_stage2_after_flags_kernel, dim3(1), dim3(256), 0, stream, pdl_enabled(),
                                          part_val, part_idx, count, half_stride, flags, num_flags, step_word, status,
                                          static_cast<SampleControl*>(control), token_out,
                                          static_cast<uint32_t>(option(W4A16_OPT_SIGNAL_WAIT_SPINS))));
}

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
