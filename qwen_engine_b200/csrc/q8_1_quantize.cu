// Q8_1 activation quantisers: fp16 -> (int8 q8, fp32 group scale, int32 per-octet sum8).
//
// Same outputs, bit for bit, as the reference's quantize_group128_fp16_to_q8_1
// (include/quant_primitives.cuh:37-89) evaluated in IEEE fp32; the thread mapping is this
// library's own (one warp per group of 128, four elements per lane).
#include "w4a16_common.cuh"
#include "w4a16_internal.hpp"

namespace w4 {
namespace {

constexpr int kQuantThreads = 128;  // 4 warps = 4 groups per CTA

// Writes one quantised group to global memory.  lane l owns elements 4l..4l+3.
__device__ __forceinline__ void store_group_q8_1(const float v[4], int g, int lane, int8_t* __restrict__ q8,
                                                 float* __restrict__ scale, int32_t* __restrict__ sum8) {
    float d;
    const uint32_t packed = quantize_group128_lane(v, &d);
    reinterpret_cast<uint32_t*>(q8)[g * (kGroup / 4) + lane] = packed;
    int32_t s = byte_sum(packed);
    s += __shfl_xor_sync(0xFFFFFFFFu, s, 1);  // two lanes = one octet
    if ((lane & 1) == 0) sum8[g * 16 + (lane >> 1)] = -8 * s;
    if (lane == 0) scale[g] = d;
}

// reference: quantize_fp16_to_q8_1_kernel, src/kernels/rmsnorm_rope.cu:273-299
__global__ void __launch_bounds__(kQuantThreads) quantize_q8_1_kernel(const __half* __restrict__ x,
                                                                       int8_t* __restrict__ q8,
                                                                       float* __restrict__ scale,
                                                                       int32_t* __restrict__ sum8, int groups) {
    pdl_release_dependents();
    pdl_wait_prior_grids();
    const int lane = threadIdx.x & 31;
    const int g = blockIdx.x * (kQuantThreads / 32) + (threadIdx.x >> 5);
    if (g >= groups) return;
    float v[4];
    load_half4_as_float(x + g * kGroup + lane * 4, v);
    store_group_q8_1(v, g, lane, q8, scale, sum8);
}

// RMSNorm fused with the quantiser: one CTA, the vector is staged in shared memory.
// reference: rmsnorm_q8_1_kernel, src/kernels/rmsnorm_rope.cu:156-250.
//   inv_rms = 1 / sqrt(mean(x^2) + eps), rounded to fp16;  y = fp16(fp16(x * inv_rms) * gamma).
// The mean of squares is taken in double (squares of fp16 values are exact there), so the
// result does not depend on the reduction order; the reference sums in fp32 in thread order.
constexpr int kNormThreads = 256;
__global__ void __launch_bounds__(kNormThreads) rmsnorm_q8_1_kernel(const __half* __restrict__ in,
                                                                    const __half* __restrict__ gamma,
                                                                    __half* __restrict__ out_opt,
                                                                    int8_t* __restrict__ q8, float* __restrict__ scale,
                                                                    int32_t* __restrict__ sum8, int hidden, float eps) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    __half* s_y = reinterpret_cast<__half*>(smem_raw);
    __shared__ double s_warp[kNormThreads / 32];
    __shared__ float s_inv;

    pdl_release_dependents();
    pdl_wait_prior_grids();

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    double ss = 0.0;
    for (int i = tid; i < hidden / 4; i += kNormThreads) {
        float v[4];
        load_half4_as_float(in + i * 4, v);
#pragma unroll
        for (int j = 0; j < 4; ++j) ss += static_cast<double>(v[j]) * static_cast<double>(v[j]);
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, m);
    if (lane == 0) s_warp[warp] = ss;
    __syncthreads();
    if (tid == 0) {
        double t = 0.0;
        for (int w = 0; w < kNormThreads / 32; ++w) t += s_warp[w];
        s_inv = inv_rms_from_sumsq(t, hidden, eps);
    }
    __syncthreads();
    const __half2 inv2 = __float2half2_rn(s_inv);
    for (int i = tid; i < hidden / 2; i += kNormThreads) {
        const __half2 v = reinterpret_cast<const __half2*>(in)[i];
        const __half2 g = reinterpret_cast<const __half2*>(gamma)[i];
        const __half2 y = __hmul2(__hmul2(v, inv2), g);
        reinterpret_cast<__half2*>(s_y)[i] = y;
        if (out_opt != nullptr) reinterpret_cast<__half2*>(out_opt)[i] = y;
    }
    __syncthreads();
    for (int g = warp; g < hidden / kGroup; g += kNormThreads / 32) {
        float v[4];
        load_half4_as_float(s_y + g * kGroup + lane * 4, v);
        store_group_q8_1(v, g, lane, q8, scale, sum8);
    }
}

// Q8_1 of attention heads from their fp32 accumulators (the epilogue of the reference's flash-decode combine
// kernel, src/kernels/attention_gqa.cu:258-310, as a kernel of its own): one half-warp per head of 128.
// Also writes fp16(acc) -- the reference's attn_out -- when out_fp16_opt is given.
__global__ void __launch_bounds__(kQuantThreads) quantize_heads_f32_q8_1_kernel(const float* __restrict__ acc,
                                                                                 __half* __restrict__ out_fp16_opt,
                                                                                 int8_t* __restrict__ q8,
                                                                                 float* __restrict__ scale,
                                                                                 int32_t* __restrict__ sum8, int heads) {
    pdl_release_dependents();
    pdl_wait_prior_grids();
    const int hl = threadIdx.x & 15;
    const int h = blockIdx.x * (kQuantThreads / 16) + (threadIdx.x >> 4);
    const bool on = h < heads;
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = 0.0f;
    if (on) {
        const float4 a = reinterpret_cast<const float4*>(acc + h * kGroup + hl * 8)[0];
        const float4 b = reinterpret_cast<const float4*>(acc + h * kGroup + hl * 8)[1];
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
    int32_t sum;
    float d;
    const uint2 packed = quantize_group_f32_div_halfwarp(v, &sum, &d);   // whole warps call it (shuffles)
    if (!on) return;
    reinterpret_cast<uint2*>(q8)[h * (kGroup / 8) + hl] = packed;
    sum8[h * (kGroup / 8) + hl] = -8 * sum;
    if (hl == 0) scale[h] = d;
    if (out_fp16_opt != nullptr) {
        __half2 o[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) o[k] = __floats2half2_rn(v[2 * k], v[2 * k + 1]);
        reinterpret_cast<uint4*>(out_fp16_opt + h * kGroup + hl * 8)[0] = *reinterpret_cast<const uint4*>(o);
    }
}

}  // namespace

int quantize_heads_f32_to_q8_1(const float* acc, __half* out_fp16_opt, int8_t* q8, float* scale, int32_t* sum8,
                               int heads, cudaStream_t stream) {
    const int per_cta = kQuantThreads / 16;
    cudaError_t e = launch_kernel(quantize_heads_f32_q8_1_kernel, dim3((heads + per_cta - 1) / per_cta),
                                  dim3(kQuantThreads), 0, stream, pdl_enabled(), acc, out_fp16_opt, q8, scale, sum8, heads);
    return static_cast<int>(e);
}

int quantize_set_attributes() {
    cudaError_t e = cudaFuncSetAttribute(rmsnorm_q8_1_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    return static_cast<int>(e);
}

int quantize_fp16_to_q8_1(const __half* x, int8_t* q8, float* scale, int32_t* sum8, int n, cudaStream_t stream) {
    const int groups = n / kGroup;
    const int grid = (groups + kQuantThreads / 32 - 1) / (kQuantThreads / 32);
    cudaError_t e = launch_kernel(quantize_q8_1_kernel, dim3(grid), dim3(kQuantThreads), 0, stream, pdl_enabled(), x,
                                  q8, scale, sum8, groups);
    return static_cast<int>(e);
}

int rmsnorm_q8_1(const __half* in, const __half* gamma, __half* out_opt, int8_t* q8, float* scale, int32_t* sum8,
                 int hidden, cudaStream_t stream) {
    constexpr float kEps = 1e-6f;  // reference include/config.cuh:20 RMS_NORM_EPS
    const size_t smem = static_cast<size_t>(hidden) * sizeof(__half);
    cudaError_t e = launch_kernel(rmsnorm_q8_1_kernel, dim3(1), dim3(kNormThreads), smem, stream, pdl_enabled(), in,
                                  gamma, out_opt, q8, scale, sum8, hidden, kEps);
    return static_cast<int>(e);
}

}  // namespace w4
