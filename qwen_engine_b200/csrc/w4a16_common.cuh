// Device-side building blocks shared by the W4A16 kernels (sm_100a only).
//
// Layout facts used here (reference include/quant_primitives.cuh:10-32):
//   packed word = q0 | q4<<4 | q1<<8 | q5<<12 | q2<<16 | q6<<20 | q3<<24 | q7<<28, so
//   (w & 0x0F0F0F0F) holds elements 0..3 as bytes and ((w >> 4) & 0x0F0F0F0F) elements 4..7;
//   weight = (q - 8) * scale;  Q8_1 activation = int8 q8[K], fp32 scale[K/128],
//   int32 sum8[K/8] = -8 * (sum of the octet's q8).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace w4 {

constexpr int kGroup = 128;       // elements per quantisation group
constexpr int kChunk = 32;        // elements covered by one 16-byte weight load
constexpr int kSubwarp = 8;       // lanes that share one weight row (8 x 16 B = 256 elements per step)
constexpr int kStepElems = 256;   // elements of a row consumed per sub-warp step

// ---- loads -------------------------------------------------------------------

// 16-byte streaming load of weights: read-only path, no L1 allocation.  volatile keeps
// the issue order the code states (weight loads go out before the activation staging).
__device__ __forceinline__ uint4 ld_weights_16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
// Same 16 bytes through four 4-byte loads, for weight tensors that are only 4-byte aligned.
__device__ __forceinline__ uint4 ld_weights_4x4(const void* p) {
    const uint32_t* q = static_cast<const uint32_t*>(p);
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v.x) : "l"(q));
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v.y) : "l"(q + 1));
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v.z) : "l"(q + 2));
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v.w) : "l"(q + 3));
    return v;
}
template <bool ALIGNED16>
__device__ __forceinline__ uint4 ld_weights(const void* p) {
    if constexpr (ALIGNED16) return ld_weights_16(p);
    else return ld_weights_4x4(p);
}
__device__ __forceinline__ uint16_t ld_scale_bits(const __half* p) {
    uint16_t v;
    asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}

// ---- programmatic dependent launch ---------------------------------------------
// Both are no-ops for a kernel launched without the programmatic-serialisation attribute.
__device__ __forceinline__ void pdl_wait_prior_grids() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_release_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }

// ---- integer core -----------------------------------------------------------------

// Sum over 8 elements of (q_j - 8) * x_j added to `seed`, when seed already carries the
// -8 * sum(x) term; without it, this is the plain sum of q_j * x_j.
__device__ __forceinline__ int32_t octet_dot(uint32_t packed, int32_t x_lo, int32_t x_hi, int32_t seed) {
    const int32_t w_lo = static_cast<int32_t>(packed & 0x0F0F0F0Fu);
    const int32_t w_hi = static_cast<int32_t>((packed >> 4) & 0x0F0F0F0Fu);
    return __dp4a(w_hi, x_hi, __dp4a(w_lo, x_lo, seed));
}

// dp4a with unsigned bytes on the weight side and signed bytes on the activation side.
__device__ __forceinline__ int32_t dp4a_u8s8(uint32_t a, int32_t b, int32_t c) {
    int32_t d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// One 16-byte weight chunk (32 elements) against its 32 activation bytes.
// chunk_seed = -8 * (sum of the 32 activation bytes), i.e. the four sum8 entries added up.
// The high nibbles are not shifted down: masked in place they are the unsigned bytes 16*q, their
// dot product is exactly 16 times the wanted one, and the factor leaves with one arithmetic shift
// at the end (the sum is a multiple of 16 and far from overflow: |.| <= 16*15*127*16).  That is four
// instructions per weight word instead of five and two independent dp4a chains instead of one; the
// integer result is the same as octet_dot's.
__device__ __forceinline__ int32_t chunk_dot(const uint4& w, const uint4& xa, const uint4& xb, int32_t chunk_seed) {
    constexpr uint32_t kLo = 0x0F0F0F0Fu, kHi = 0xF0F0F0F0u;
    int32_t lo = chunk_seed, hi = 0;
    lo = dp4a_u8s8(w.x & kLo, static_cast<int32_t>(xa.x), lo);
    hi = dp4a_u8s8(w.x & kHi, static_cast<int32_t>(xa.y), hi);
    lo = dp4a_u8s8(w.y & kLo, static_cast<int32_t>(xa.z), lo);
    hi = dp4a_u8s8(w.y & kHi, static_cast<int32_t>(xa.w), hi);
    lo = dp4a_u8s8(w.z & kLo, static_cast<int32_t>(xb.x), lo);
    hi = dp4a_u8s8(w.z & kHi, static_cast<int32_t>(xb.y), hi);
    lo = dp4a_u8s8(w.w & kLo, static_cast<int32_t>(xb.z), lo);
    hi = dp4a_u8s8(w.w & kHi, static_cast<int32_t>(xb.w), hi);
    return lo + (hi >> 4);
}

// ---- Q8_1 quantiser ------------------------------------------------------------------
// One warp quantises one group of 128: lane l owns elements 4l..4l+3.
// d = max(max|x| / 127, 1e-8), inv_d = 1 / d, q = clamp(rn(x * inv_d), -127, 127), all in
// IEEE fp32 (explicit _rn intrinsics: the result does not depend on compiler flags).
// Returns the four int8 packed little-endian; *d_out is the group scale (same in all lanes).
__device__ __forceinline__ uint32_t quantize_group128_lane(const float v[4], float* d_out) {
    float m = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
    for (int mask = 16; mask > 0; mask >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, mask));
    const float d = fmaxf(__fdiv_rn(m, 127.0f), 1e-8f);
    const float inv_d = __fdiv_rn(1.0f, d);
    uint32_t packed = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        int q = __float2int_rn(__fmul_rn(v[j], inv_d));
        q = max(-127, min(127, q));
        packed |= (static_cast<uint32_t>(q) & 0xFFu) << (8 * j);
    }
    *d_out = d;
    return packed;
}
// Sum of the four signed bytes of a packed word.
__device__ __forceinline__ int32_t byte_sum(uint32_t packed) {
    return __dp4a(static_cast<int32_t>(packed), 0x01010101, 0);
}

__device__ __forceinline__ void load_half4_as_float(const __half* p, float v[4]) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const __half2 a = *reinterpret_cast<const __half2*>(&raw.x);
    const __half2 b = *reinterpret_cast<const __half2*>(&raw.y);
    const float2 fa = __half22float2(a), fb = __half22float2(b);
    v[0] = fa.x; v[1] = fa.y; v[2] = fb.x; v[3] = fb.y;
}

// Layout of the staged activation in shared memory (all 16-byte aligned):
//   q8[K] int8 (chunk-interleaved, see q8_slot) | chunk_seed[K/32] int32 | scale[K/128] fp32
struct StagedX {
    const int8_t* q8;
    const int32_t* seed;
    const float* scale;
};
__host__ __device__ inline size_t staged_x_bytes(int K) {
    return static_cast<size_t>(K) + static_cast<size_t>(K / kChunk) * 4 + static_cast<size_t>(K / kGroup) * 4;
}

// Where the staged int8 activation keeps its bytes.  A lane of the GEMV reads the 32 bytes of one chunk as two
// 16-byte halves, and the 8 lanes of a sub-warp read 8 consecutive chunks: in natural order that is a 32-byte
// stride, two lanes per bank.  So chunks are interleaved in blocks of eight: the first halves of the eight chunks
// (128 contiguous bytes), then their second halves.  K is a multiple of 256, i.e. of eight chunks.
//   q8_slot(c, h): uint4 index of half h of chunk c;  q8_byte(e): byte offset of element e.
__host__ __device__ __forceinline__ int q8_slot(int c, int h) { return ((c >> 3) << 4) + (h << 3) + (c & 7); }
__host__ __device__ __forceinline__ int q8_byte(int e) { return q8_slot(e >> 5, (e >> 4) & 1) * 16 + (e & 15); }

// RMSNorm scale from the sum of squares.  The sum is taken in double (squares of fp16 values are exact there
// and their sum is off by parts in 2^50 at most, so the order of the additions does not reach the fp32 mean
// and every kernel of this library gets the same value); everything after it is IEEE fp32
// as in the reference (src/kernels/rmsnorm_rope.cu:214-233): mean, + eps, square root, reciprocal.
__device__ __forceinline__ float inv_rms_from_sumsq(double sumsq, int n, float eps) {
    const float mean = __fdiv_rn(__double2float_rn(sumsq), static_cast<float>(n));
    return __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
}

// Copies a pre-quantised Q8_1 activation from global into shared memory, folding the four
// per-octet sum8 of each chunk into one seed.  vec_ok: q8 and sum8 are 16-byte aligned.
__device__ __forceinline__ void stage_x_from_q8_1(const int8_t* __restrict__ g_q8, const float* __restrict__ g_scale,
                                                  const int32_t* __restrict__ g_sum8, int K, bool vec_ok,
                                                  int8_t* s_q8, int32_t* s_seed, float* s_scale) {
    const int tid = threadIdx.x, nthr = blockDim.x;
    if (vec_ok) {
        const uint4* src = reinterpret_cast<const uint4*>(g_q8);
        uint4* dst = reinterpret_cast<uint4*>(s_q8);
        for (int i = tid; i < K / 16; i += nthr) dst[q8_slot(i >> 1, i & 1)] = src[i];
        const int4* s8 = reinterpret_cast<const int4*>(g_sum8);
        for (int c = tid; c < K / kChunk; c += nthr) {
            const int4 v = s8[c];
            s_seed[c] = v.x + v.y + v.z + v.w;
        }
    } else {
        for (int i = tid; i < K; i += nthr) s_q8[q8_byte(i)] = g_q8[i];
        for (int c = tid; c < K / kChunk; c += nthr)
            s_seed[c] = g_sum8[4 * c] + g_sum8[4 * c + 1] + g_sum8[4 * c + 2] + g_sum8[4 * c + 3];
    }
    for (int g = tid; g < K / kGroup; g += nthr) s_scale[g] = g_scale[g];
}

// Quantises an fp16 activation into the same shared-memory layout (every CTA does it for
// itself; the result is identical to what the stand-alone quantiser writes to global).
// x must be 8-byte aligned.
__device__ __forceinline__ void stage_x_from_fp16(const __half* __restrict__ g_x, int K, int8_t* s_q8,
                                                  int32_t* s_seed, float* s_scale) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int g = warp; g < K / kGroup; g += nwarps) {
        float v[4];
        load_half4_as_float(g_x + g * kGroup + lane * 4, v);
        float d;
        const uint32_t packed = quantize_group128_lane(v, &d);
        *reinterpret_cast<uint32_t*>(s_q8 + q8_byte(g * kGroup + lane * 4)) = packed;
        int32_t s = byte_sum(packed);
        s += __shfl_xor_sync(0xFFFFFFFFu, s, 1);
        s += __shfl_xor_sync(0xFFFFFFFFu, s, 2);
        s += __shfl_xor_sync(0xFFFFFFFFu, s, 4);
        if ((lane & 7) == 0) s_seed[g * 4 + (lane >> 3)] = -8 * s;
        if (lane == 0) s_scale[g] = d;
    }
}

// RMSNorm fused in front of the quantiser, per CTA: y = fp16(fp16(x * inv_rms) * gamma) with
// inv_rms = 1 / sqrt(mean(x^2) + eps) rounded to fp16 -- the arithmetic of the stand-alone
// rmsnorm_q8_1 kernel (mean of squares in double), so both give the same Q8_1 arrays.
// Needs blockDim.x to be a multiple of 32 and at most 256.
__device__ __forceinline__ void stage_x_from_fp16_rmsnorm(const __half* __restrict__ g_x,
                                                          const __half* __restrict__ g_gamma, int K, float eps,
                                                          int8_t* s_q8, int32_t* s_seed, float* s_scale) {
    __shared__ double s_red[8];
    __shared__ float s_inv;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    double ss = 0.0;
    for (int g = warp; g < K / kGroup; g += nwarps) {
        float v[4];
        load_half4_as_float(g_x + g * kGroup + lane * 4, v);
#pragma unroll
        for (int j = 0; j < 4; ++j) ss += static_cast<double>(v[j]) * static_cast<double>(v[j]);
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, m);
    if (lane == 0) s_red[warp] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int w = 0; w < nwarps; ++w) t += s_red[w];
        s_inv = inv_rms_from_sumsq(t, K, eps);
    }
    __syncthreads();
    const __half2 inv2 = __float2half2_rn(s_inv);
    for (int g = warp; g < K / kGroup; g += nwarps) {
        const uint2 xr = *reinterpret_cast<const uint2*>(g_x + g * kGroup + lane * 4);
        const uint2 gr = *reinterpret_cast<const uint2*>(g_gamma + g * kGroup + lane * 4);
        const __half2 y0 = __hmul2(__hmul2(*reinterpret_cast<const __half2*>(&xr.x), inv2),
                                   *reinterpret_cast<const __half2*>(&gr.x));
        const __half2 y1 = __hmul2(__hmul2(*reinterpret_cast<const __half2*>(&xr.y), inv2),
                                   *reinterpret_cast<const __half2*>(&gr.y));
        const float2 f0 = __half22float2(y0), f1 = __half22float2(y1);
        const float v[4] = {f0.x, f0.y, f1.x, f1.y};
        float d;
        const uint32_t packed = quantize_group128_lane(v, &d);
        *reinterpret_cast<uint32_t*>(s_q8 + q8_byte(g * kGroup + lane * 4)) = packed;
        int32_t s = byte_sum(packed);
        s += __shfl_xor_sync(0xFFFFFFFFu, s, 1);
        s += __shfl_xor_sync(0xFFFFFFFFu, s, 2);
        s += __shfl_xor_sync(0xFFFFFFFFu, s, 4);
        if ((lane & 7) == 0) s_seed[g * 4 + (lane >> 3)] = -8 * s;
        if (lane == 0) s_scale[g] = d;
    }
}

// ---- low-latency staging (the forms the decode GEMV uses when the shape allows) ---------------
// Between two dependent GEMVs every global round trip in the prologue is on the critical path
// (about 0.4 us each on B200), so these forms issue ALL of a thread's global loads back to back
// before the first use, take the RMSNorm gain before the wait for the prior grid, and give each
// group of 128 to a half-warp (lane = 8 consecutive elements = one 16-byte load = one sum8 octet)
// so that K = 1536 is one round for a 192-thread CTA.  Same arithmetic, same bits as the loops above.
constexpr int kStageRounds = 1;   // groups per half-warp held in registers (K <= 128 * blockDim / 16)

// Half-warp quantiser: 16 lanes per group, lane hl owns elements 8*hl .. 8*hl+7.  Both halves of a
// warp must call it together (shuffles); `on` = this half-warp has a real group.
__device__ __forceinline__ void quantize_group_halfwarp_to_smem(const float v[8], int g, int hl, bool on, int8_t* s_q8,
                                                                int32_t* s_seed, float* s_scale) {
    float m = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) m = fmaxf(m, fabsf(v[j]));
#pragma unroll
    for (int mask = 8; mask > 0; mask >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, mask));
    const float d = fmaxf(__fdiv_rn(m, 127.0f), 1e-8f);
    const float inv_d = __fdiv_rn(1.0f, d);
    uint32_t packed[2] = {0, 0};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        int q = __float2int_rn(__fmul_rn(v[j], inv_d));
        q = max(-127, min(127, q));
        packed[j >> 2] |= (static_cast<uint32_t>(q) & 0xFFu) << (8 * (j & 3));
    }
    int32_t sum = byte_sum(packed[0]) + byte_sum(packed[1]);   // one octet; four lanes make a chunk
    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
    if (on) {
        *reinterpret_cast<uint2*>(s_q8 + q8_byte(g * kGroup + hl * 8)) = make_uint2(packed[0], packed[1]);
        if ((hl & 3) == 0) s_seed[g * 4 + (hl >> 2)] = -8 * sum;
        if (hl == 0) s_scale[g] = d;
    }
}

// Q8_1 of one group of 128 taken straight from fp32 values, as the reference's flash-decode combine step
// quantises an attention head for the O projection (src/kernels/attention_gqa.cu:263-310):
//   d = max(max|v| / 127, 1e-8),  q = clamp(rn(v / d), -127, 127)  -- one division per element, where the
// fp16 quantiser above multiplies by 1 / d; the bytes can therefore differ from quantising fp16(v).
// Half-warp form: lane hl owns elements 8 hl .. 8 hl + 7, i.e. exactly one sum8 octet.  Both halves of a
// warp call it together.  Returns the eight bytes; *octet_sum = their plain sum, *d_out the group scale.
__device__ __forceinline__ uint2 quantize_group_f32_div_halfwarp(const float v[8], int32_t* octet_sum, float* d_out) {
    float m = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) m = fmaxf(m, fabsf(v[j]));
#pragma unroll
    for (int mask = 8; mask > 0; mask >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, mask));
    const float d = fmaxf(__fdiv_rn(m, 127.0f), 1e-8f);
    uint32_t packed[2] = {0, 0};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        int q = __float2int_rn(__fdiv_rn(v[j], d));
        q = max(-127, min(127, q));
        packed[j >> 2] |= (static_cast<uint32_t>(q) & 0xFFu) << (8 * (j & 3));
    }
    *octet_sum = byte_sum(packed[0]) + byte_sum(packed[1]);
    *d_out = d;
    return make_uint2(packed[0], packed[1]);
}

// fp32 vector of whole groups (attention heads of 128) -> staged Q8_1 in shared memory, every CTA for itself.
// x must be 16-byte aligned; blockDim.x a multiple of 32.
__device__ __forceinline__ void stage_x_from_f32_heads(const float* __restrict__ g_x, int K, int8_t* s_q8,
                                                       int32_t* s_seed, float* s_scale) {
    const int hw = threadIdx.x >> 4, hl = threadIdx.x & 15, nhw = blockDim.x >> 4;
    const int groups = K / kGroup;
    for (int g0 = 0; g0 < groups; g0 += nhw) {   // uniform trip count: both halves of a warp shuffle together
        const int g = g0 + hw;
        const bool on = g < groups;
        float v[8];
        if (on) {
            const float4 a = reinterpret_cast<const float4*>(g_x + g * kGroup + hl * 8)[0];
            const float4 b = reinterpret_cast<const float4*>(g_x + g * kGroup + hl * 8)[1];
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = 0.0f;
        }
        int32_t sum;
        float d;
        const uint2 packed = quantize_group_f32_div_halfwarp(v, &sum, &d);
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);   // four lanes = one 32-element chunk
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
        if (on) {
            *reinterpret_cast<uint2*>(s_q8 + q8_byte(g * kGroup + hl * 8)) = packed;
            if ((hl & 3) == 0) s_seed[g * 4 + (hl >> 2)] = -8 * sum;
            if (hl == 0) s_scale[g] = d;
        }
    }
}

// True when the register form applies: few enough groups for kStageRounds rounds and 16-byte aligned vectors.
__device__ __forceinline__ bool stage_regs_ok(const void* x, const void* gamma, int K) {
    const int nhw = blockDim.x >> 4;
    return (K / kGroup) <= kStageRounds * nhw &&
           ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(gamma)) & 15u) == 0;
}

// The RMSNorm gain words this thread will need; a weight, so it may be read before the prior grid is done.
__device__ __forceinline__ void prefetch_gamma(const __half* __restrict__ g_gamma, int K, uint4 (&gam)[kStageRounds]) {
    const int hw = threadIdx.x >> 4, hl = threadIdx.x & 15, nhw = blockDim.x >> 4;
#pragma unroll
    for (int r = 0; r < kStageRounds; ++r) {
        const int g = hw + r * nhw;
        gam[r] = g < K / kGroup ? __ldg(reinterpret_cast<const uint4*>(g_gamma + g * kGroup + hl * 8)) : make_uint4(0, 0, 0, 0);
    }
}

// fp16 activation (optionally RMSNorm'ed with the prefetched gain) -> staged Q8_1.  One global round trip.
// sumsq_in (NORM only, may be null): the sum of x's squares as the producing launch published it, in 8 partial
// sums; the CTA then skips its own reduction (conversions to double, two shuffle trees, one barrier).  The value
// is the same sum of the same exact squares, so the rounded mean does not change.
template <bool NORM>
__device__ __forceinline__ void stage_x_fp16_regs(const __half* g_x, const uint4 (&gam)[kStageRounds], int K, float eps,
                                                  int8_t* s_q8, int32_t* s_seed, float* s_scale,
                                                  const double* sumsq_in = nullptr) {
    __shared__ double s_red[8];
    const int hw = threadIdx.x >> 4, hl = threadIdx.x & 15, nhw = blockDim.x >> 4;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int groups = K / kGroup;
    uint4 xr[kStageRounds];
#pragma unroll
    for (int r = 0; r < kStageRounds; ++r) {
        const int g = hw + r * nhw;
        xr[r] = g < groups ? *reinterpret_cast<const uint4*>(g_x + g * kGroup + hl * 8) : make_uint4(0, 0, 0, 0);
    }
    __half2 inv2 = __float2half2_rn(1.0f);
    if (NORM && sumsq_in != nullptr) {
        // One warp fetches the 8 partial sums (one 64-byte request per CTA: every CTA of the grid reads the same
        // line, and a request per thread makes that line a hot spot) in the same round trip as the loads above.
        if (warp == 0) {
            double s = lane < 8 ? __ldcg(sumsq_in + lane) : 0.0;
            s += __shfl_xor_sync(0xFFFFFFFFu, s, 4);
            s += __shfl_xor_sync(0xFFFFFFFFu, s, 2);
            s += __shfl_xor_sync(0xFFFFFFFFu, s, 1);
            if (lane == 0) s_red[0] = s;
        }
        __syncthreads();
        inv2 = __float2half2_rn(inv_rms_from_sumsq(s_red[0], K, eps));
    } else if constexpr (NORM) {
        double ss = 0.0;
#pragma unroll
        for (int r = 0; r < kStageRounds; ++r) {
            const uint32_t* xw = reinterpret_cast<const uint32_t*>(&xr[r]);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&xw[k]));
                ss += static_cast<double>(f.x) * static_cast<double>(f.x);
                ss += static_cast<double>(f.y) * static_cast<double>(f.y);
            }
        }
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, m);
        if (lane == 0) s_red[warp] = ss;
        __syncthreads();
        double t = 0.0;
        for (int w = 0; w < nwarps; ++w) t += s_red[w];   // every thread, same order: no second barrier
        inv2 = __float2half2_rn(inv_rms_from_sumsq(t, K, eps));
    }
    const int rounds = (groups + nhw - 1) / nhw;
#pragma unroll
    for (int r = 0; r < kStageRounds; ++r) {
        if (r < rounds) {   // uniform over the CTA: both halves of a warp shuffle together
            const int g = hw + r * nhw;
            const uint32_t* xw = reinterpret_cast<const uint32_t*>(&xr[r]);
            const uint32_t* gw = reinterpret_cast<const uint32_t*>(&gam[r]);
            float v[8];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                __half2 y = *reinterpret_cast<const __half2*>(&xw[k]);
                if constexpr (NORM) y = __hmul2(__hmul2(y, inv2), *reinterpret_cast<const __half2*>(&gw[k]));
                const float2 f = __half22float2(y);
                v[2 * k] = f.x;
                v[2 * k + 1] = f.y;
            }
            quantize_group_halfwarp_to_smem(v, g, hl, g < groups, s_q8, s_seed, s_scale);
        }
    }
}

// fp16 activation whose per-group |max| the producing launch has published (float bits, one word per group of
// 128): every CTA quantises it element by element, no reduction.  The raw vector goes through shared memory
// (cp.async, no registers held), the scales are derived while it is in flight.  Same arithmetic as
// quantize_group128_lane given the same maximum, so the staged arrays equal the stand-alone quantiser's.
// s_raw: K halves, 16-byte aligned; s_inv: K / 128 floats.  Needs x 16-byte aligned; all threads call it.
__device__ __forceinline__ void stage_x_fp16_amax(const __half* g_x, const uint32_t* g_amax, int K, int8_t* s_q8,
                                                  int32_t* s_seed, float* s_scale, __half* s_raw, float* s_inv) {
    const int tid = threadIdx.x, nthr = blockDim.x;
    const int octets = K / 8;
    for (int i = tid; i < octets; i += nthr) {
        const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(s_raw + i * 8));
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(g_x + i * 8) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    for (int g = tid; g < K / kGroup; g += nthr) {
        const float m = __uint_as_float(__ldcg(g_amax + g));
        const float d = fmaxf(__fdiv_rn(m, 127.0f), 1e-8f);
        s_scale[g] = d;
        s_inv[g] = __fdiv_rn(1.0f, d);
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    const int rounds = (octets + nthr - 1) / nthr;
    for (int r = 0; r < rounds; ++r) {   // uniform trip count: the four lanes of a chunk shuffle together
        const int i = tid + r * nthr;
        const bool on = i < octets;
        uint4 xr = make_uint4(0, 0, 0, 0);
        float inv_d = 0.0f;
        if (on) {
            xr = *reinterpret_cast<const uint4*>(s_raw + i * 8);
            inv_d = s_inv[i >> 4];
        }
        const uint32_t* xw = reinterpret_cast<const uint32_t*>(&xr);
        uint32_t packed[2] = {0, 0};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&xw[k]));
            int q0 = __float2int_rn(__fmul_rn(f.x, inv_d)), q1 = __float2int_rn(__fmul_rn(f.y, inv_d));
            q0 = max(-127, min(127, q0));
            q1 = max(-127, min(127, q1));
            packed[k >> 1] |= ((static_cast<uint32_t>(q0) & 0xFFu) | ((static_cast<uint32_t>(q1) & 0xFFu) << 8)) << (16 * (k & 1));
        }
        int32_t sum = byte_sum(packed[0]) + byte_sum(packed[1]);
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
        if (on) {
            *reinterpret_cast<uint2*>(s_q8 + q8_byte(i * 8)) = make_uint2(packed[0], packed[1]);
            if ((i & 3) == 0) s_seed[i >> 2] = -8 * sum;
        }
    }
}

// Pre-quantised Q8_1 -> shared memory with every global load of the thread in flight at once.
// Returns false (nothing done) when the vector is too long for the register budget or not 16-byte aligned.
// LEAN: two round trips (bytes, then sums and scales) for callers that are short of registers.
template <bool LEAN>
__device__ __forceinline__ bool stage_x_from_q8_1_regs(const int8_t* g_q8, const float* g_scale, const int32_t* g_sum8,
                                                       int K, bool vec_ok, int8_t* s_q8, int32_t* s_seed, float* s_scale) {
    constexpr int MAXQ = 4, MAXS = 2;
    const int tid = threadIdx.x, nthr = blockDim.x;
    if (!vec_ok || K / 16 > MAXQ * nthr || K / kChunk > MAXS * nthr || K / kGroup > nthr) return false;
    uint4 q[MAXQ];
    int4 sv[MAXS];
    float sc = 0.0f;
#pragma unroll
    for (int i = 0; i < MAXQ; ++i) {
        const int idx = tid + i * nthr;
        if (idx < K / 16) q[i] = reinterpret_cast<const uint4*>(g_q8)[idx];
    }
    if constexpr (LEAN) {
#pragma unroll
        for (int i = 0; i < MAXQ; ++i) {
            const int idx = tid + i * nthr;
            if (idx < K / 16) reinterpret_cast<uint4*>(s_q8)[q8_slot(idx >> 1, idx & 1)] = q[i];
        }
    }
#pragma unroll
    for (int i = 0; i < MAXS; ++i) {
        const int idx = tid + i * nthr;
        if (idx < K / kChunk) sv[i] = reinterpret_cast<const int4*>(g_sum8)[idx];
    }
    if (tid < K / kGroup) sc = g_scale[tid];
    if constexpr (!LEAN) {
#pragma unroll
        for (int i = 0; i < MAXQ; ++i) {
            const int idx = tid + i * nthr;
            if (idx < K / 16) reinterpret_cast<uint4*>(s_q8)[q8_slot(idx >> 1, idx & 1)] = q[i];
        }
    }
#pragma unroll
    for (int i = 0; i < MAXS; ++i) {
        const int idx = tid + i * nthr;
        if (idx < K / kChunk) s_seed[idx] = sv[i].x + sv[i].y + sv[i].z + sv[i].w;
    }
    if (tid < K / kGroup) s_scale[tid] = sc;
    return true;
}

}  // namespace w4
