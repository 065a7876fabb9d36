// Device-side pieces of greedy / Gumbel-max token selection, shared by the stand-alone sampler and the
// lm_head GEMV that samples in its epilogue.
//
// Semantics of the reference (src/kernels/sampling.cu:60-204): the token is the index of the largest
// score, the lowest index among equals; score = logit for temperature <= 1e-5, else
// logit / temperature - log(-log(u)) with u a uniform number drawn from Philox-4x32-10 keyed by the
// control block's seed, counter = (vocabulary index, sequence position, 0, 0).  Any reduction tree
// gives the same token because "larger score, then smaller index" is a total order.
#pragma once

#include <cstdint>
#include <cuda_runtime.h>

namespace w4 {

// Same layout as the reference's DeviceControlBlock (include/tensor.cuh:28-34).
struct SampleControl {
    int32_t token_id;
    int32_t seq_pos;
    float temperature;
    uint32_t reserved;
    uint64_t rng_seed;
};

constexpr float kSampleFloor = -1e30f;       // initial best score (reference: sampling.cu:78)
constexpr float kGreedyTemperature = 1e-5f;  // at or below: plain argmax (sampling.cu:88)

// Philox-4x32 with 10 rounds (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3",
// SC'11): counter (c0, c1, 0, 0), key = the two halves of the seed; returns the first output word.
__device__ __forceinline__ uint32_t philox4x32_10_first(uint64_t seed, uint32_t c0, uint32_t c1) {
    uint32_t c2 = 0, c3 = 0;
    uint32_t k0 = static_cast<uint32_t>(seed), k1 = static_cast<uint32_t>(seed >> 32);
#pragma unroll
    for (int round = 0; round < 10; ++round) {
        const uint64_t p0 = static_cast<uint64_t>(0xD2511F53u) * c0;
        const uint64_t p1 = static_cast<uint64_t>(0xCD9E8D57u) * c2;
        const uint32_t n0 = static_cast<uint32_t>(p1 >> 32) ^ c1 ^ k0;
        const uint32_t n1 = static_cast<uint32_t>(p1);
        const uint32_t n2 = static_cast<uint32_t>(p0 >> 32) ^ c3 ^ k1;
        const uint32_t n3 = static_cast<uint32_t>(p0);
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    return c0;
}

// Score of one vocabulary entry.  IEEE fp32 throughout (the division and the conversion are written with
// the _rn intrinsics so that compiler flags cannot change them); logf is the accurate one.
__device__ __forceinline__ float sample_score(float logit, uint32_t vocab_index, float temperature, uint64_t seed,
                                              uint32_t seq_pos) {
    if (!(temperature > kGreedyTemperature)) return logit;
    const uint32_t r = philox4x32_10_first(seed, vocab_index, seq_pos);
    float u = __fdiv_rn(__fadd_rn(__uint2float_rn(r), 1.0f), 4294967296.0f);   // the reference's 4294967298.0f is 2^32 in fp32
    u = fminf(fmaxf(u, 1e-7f), 1.0f - 1e-7f);
    const float gumbel = -logf(-logf(u));
    return __fadd_rn(__fdiv_rn(logit, temperature), gumbel);
}

// (score, index) candidates: larger score wins, equal scores go to the smaller index.
__device__ __forceinline__ void sample_take(float& best, int32_t& best_idx, float v, int32_t i) {
    if (v > best || (v == best && i < best_idx)) { best = v; best_idx = i; }
}
__device__ __forceinline__ void sample_warp_reduce(float& best, int32_t& best_idx) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) {
        const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, m);
        const int32_t oi = __shfl_xor_sync(0xFFFFFFFFu, best_idx, m);
        sample_take(best, best_idx, ov, oi);
    }
}
// Whole-CTA reduction (at most 32 warps); the result is valid in thread 0.  s_v / s_i: 32 entries each.
__device__ __forceinline__ void sample_block_reduce(float& best, int32_t& best_idx, float* s_v, int32_t* s_i) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    sample_warp_reduce(best, best_idx);
    if (lane == 0) { s_v[warp] = best; s_i[warp] = best_idx; }
    __syncthreads();
    if (warp == 0) {
        best = lane < nwarps ? s_v[lane] : kSampleFloor;
        best_idx = lane < nwarps ? s_i[lane] : 0x7FFFFFFF;
        sample_warp_reduce(best, best_idx);
    }
}

}  // namespace w4
