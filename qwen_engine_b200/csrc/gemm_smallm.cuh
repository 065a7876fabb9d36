// M-token W4A16 contraction on CUDA cores, for token counts below the tensor-core tile
// (weight-streaming: each CTA owns output rows and walks K once per pass of MT tokens).
//
// Arithmetic follows the reference's prefill GEMM (src/kernels/gemm_prefill.cu:100-150,
// include/quant_primitives.cuh:92-115): weights are dequantised to fp16 as (q - 8) * scale
// with one fp16 rounding, multiplied with fp16 activations exactly, accumulated in fp32.
// Epilogue (gemm_prefill.cu:257-275, 572-605): fp16(acc), then an fp16 add of the residual;
// SwiGLU on the fp32 accumulators of rows 2i / 2i+1.
#pragma once

#include "w4a16_common.cuh"
#include "w4a16_internal.hpp"

namespace w4 {

// Eight nibbles of one packed word -> eight fp16 weights in K order, (q - 8) * scale.
// 0x6400 is fp16 1024: OR-ing a nibble into its mantissa gives 1024 + q exactly, and
// subtracting 1032 leaves q - 8 exactly; the multiply by the scale rounds once.
__device__ __forceinline__ void dequant_word_fp16(uint32_t packed, __half2 scale2, __half2 out[4]) {
    const uint32_t lo = packed & 0x0F0F0F0Fu;         // elements 0..3, one per byte
    const uint32_t hi = (packed >> 4) & 0x0F0F0F0Fu;  // elements 4..7
    const uint32_t magic = 0x64646464u;
    uint32_t h01 = __byte_perm(lo, magic, 0x4140);
    uint32_t h23 = __byte_perm(lo, magic, 0x4342);
    uint32_t h45 = __byte_perm(hi, magic, 0x4140);
    uint32_t h67 = __byte_perm(hi, magic, 0x4342);
    const __half2 bias = __half2half2(__ushort_as_half(static_cast<unsigned short>(0x6408)));  // 1032
    out[0] = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&h01), bias), scale2);
    out[1] = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&h23), bias), scale2);
    out[2] = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&h45), bias), scale2);
    out[3] = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&h67), bias), scale2);
}

struct SmallMArgs {
    GemmArgs g;
    int units;          // output rows (PLAIN/QKV) or pairs (SWIGLU)
    int units_per_cta;
    int out_ld[3];      // row stride of each output tensor in elements
};

template <int MODE, int MT>
__global__ void __launch_bounds__(256) gemm_smallm_kernel(const SmallMArgs a) {
    constexpr int R = (MODE == kSwiglu) ? 2 : 1;
    const int K = a.g.K, M = a.g.M;
    const int sub = threadIdx.x >> 3, l = threadIdx.x & 7;
    const int unit = blockIdx.x * a.units_per_cta + sub;
    const bool active = sub < a.units_per_cta && unit < a.units;  // a rounded-up block has idle sub-warps
    const int words = K / 8, groups = K / kGroup;

    const uint32_t* wrow[R] = {};
    const __half* srow[R] = {};
    __half* out_col = nullptr;
    int out_ld = 0;
    if (active) {
        if constexpr (MODE == kQkv) {
            int t = 0, local = unit;
            if (local >= a.g.rows[0]) { local -= a.g.rows[0]; t = 1; }
            if (t == 1 && local >= a.g.rows[1]) { local -= a.g.rows[1]; t = 2; }
            wrow[0] = a.g.qweight[t] + static_cast<size_t>(local) * words;
            srow[0] = a.g.scales[t] + static_cast<size_t>(local) * groups;
            out_col = a.g.out[t] + local;
            out_ld = a.out_ld[t];
        } else {
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const size_t row = static_cast<size_t>(unit) * R + r;
                wrow[r] = a.g.qweight[0] + row * words;
                srow[r] = a.g.scales[0] + row * groups;
            }
            out_col = a.g.out[0] + unit;
            out_ld = a.out_ld[0];
        }
    }

    pdl_release_dependents();
    pdl_wait_prior_grids();

    for (int m0 = 0; m0 < M; m0 += MT) {
        float acc[R][MT];
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int m = 0; m < MT; ++m) acc[r][m] = 0.0f;

        if (active) {
            for (int s = 0; s < K / kStepElems; ++s) {
                const int c = s * kSubwarp + l;
                float wf[R][32];
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const uint4 w = ld_weights_4x4(wrow[r] + c * 4);
                    const __half sc = __ushort_as_half(ld_scale_bits(srow[r] + (c >> 2)));
                    const __half2 sc2 = __half2half2(sc);
                    const uint32_t wv[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        __half2 h[4];
                        dequant_word_fp16(wv[j], sc2, h);
#pragma unroll
                        for (int p = 0; p < 4; ++p) {
                            const float2 f = __half22float2(h[p]);
                            wf[r][j * 8 + p * 2] = f.x;
                            wf[r][j * 8 + p * 2 + 1] = f.y;
                        }
                    }
                }
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    if (m0 + m < M) {
                        const uint4* xp =
                            reinterpret_cast<const uint4*>(a.g.x + static_cast<size_t>(m0 + m) * K + c * kChunk);
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const uint4 xv = __ldg(xp + q);
                            const __half2* xh = reinterpret_cast<const __half2*>(&xv);
#pragma unroll
                            for (int p = 0; p < 4; ++p) {
                                const float2 xf = __half22float2(xh[p]);
#pragma unroll
                                for (int r = 0; r < R; ++r) {
                                    acc[r][m] = fmaf(wf[r][q * 8 + p * 2], xf.x, acc[r][m]);
                                    acc[r][m] = fmaf(wf[r][q * 8 + p * 2 + 1], xf.y, acc[r][m]);
                                }
                            }
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                acc[r][m] += __shfl_xor_sync(0xFFFFFFFFu, acc[r][m], 4);
                acc[r][m] += __shfl_xor_sync(0xFFFFFFFFu, acc[r][m], 2);
                acc[r][m] += __shfl_xor_sync(0xFFFFFFFFu, acc[r][m], 1);
            }
        if (active && l == 0) {
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                if (m0 + m < M) {
                    __half y;
                    if constexpr (MODE == kSwiglu) {
                        const float gate = acc[0][m];
                        y = __float2half_rn((gate / (1.0f + expf(-gate))) * acc[R - 1][m]);
                    } else {
                        y = __float2half_rn(acc[0][m]);
                        if constexpr (MODE == kPlain) {
                            if (a.g.residual != nullptr)
                                y = __hadd(y, a.g.residual[static_cast<size_t>(m0 + m) * out_ld + unit]);
                        }
                    }
                    out_col[static_cast<size_t>(m0 + m) * out_ld] = y;
                }
            }
        }
    }
}


// ---- few-token form with the decode GEMV's memory behaviour -----------------------------------
// Same arithmetic as the kernel above, organised like the batch-1 GEMV: eight lanes share a weight row, the
// CTA holds units_per_cta x ksplit sub-warps (rows x slices of K), and every lane has ALL its 16-byte weight
// loads in flight before it waits for the prior grid, so the matrix streams at the memory system's pace
// instead of one dependent load per step.  The tokens are staged MT at a time in shared memory as fp32
// (each 32-element chunk padded by four floats: the eight lanes of a sub-warp read different chunks and
// would otherwise collide on the same banks); the weights stay in registers across the token passes.
// Needs 16-byte aligned weights and at most U steps per K slice.
// Two fp32 fused multiply-adds in one instruction (sm_100 packed fp32): acc.{x,y} += a.{x,y} * b.{x,y}.
__device__ __forceinline__ void ffma2(float2& acc, float2 a, float2 b) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;"
        : "=l"(d)
        : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)),
          "l"(*reinterpret_cast<unsigned long long*>(&acc)));
    acc = *reinterpret_cast<float2*>(&d);
}

struct SmallMPlan {
    int units_per_cta, ksplit, steps_per_split;
};
__host__ __device__ inline int smallm_x_stride(int K) { return K + K / kChunk * 4; }

template <int MODE, int U, int MT>
__global__ void __launch_bounds__(256, 2) gemm_smallm_v2_kernel(const SmallMArgs a, const SmallMPlan p) {
    constexpr int R = (MODE == kSwiglu) ? 2 : 1;
    extern __shared__ __align__(16) float s_x[];     // [MT][stride] then the K-slice partials
    const int K = a.g.K, M = a.g.M;
    const int xs = smallm_x_stride(K);
    float* s_part = s_x + MT * xs;
    const int tid = threadIdx.x;
    const int sub = tid >> 3, l = tid & 7;
    const int u_local = sub % p.units_per_cta, ks = sub / p.units_per_cta;
    const int unit = blockIdx.x * p.units_per_cta + u_local;
    const bool active = ks < p.ksplit && unit < a.units;
    const int words = K / 8, groups = K / kGroup;

    const uint32_t* wrow[R] = {};
    const __half* srow[R] = {};
    __half* out_col = nullptr;
    int out_ld = 0;
    if (active) {
        if constexpr (MODE == kQkv) {
            int t = 0, local = unit;
            if (local >= a.g.rows[0]) { local -= a.g.rows[0]; t = 1; }
            if (t == 1 && local >= a.g.rows[1]) { local -= a.g.rows[1]; t = 2; }
            wrow[0] = a.g.qweight[t] + static_cast<size_t>(local) * words;
            srow[0] = a.g.scales[t] + static_cast<size_t>(local) * groups;
            out_col = a.g.out[t] + local;
            out_ld = a.out_ld[t];
        } else {
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const size_t row = static_cast<size_t>(unit) * R + r;
                wrow[r] = a.g.qweight[0] + row * words;
                srow[r] = a.g.scales[0] + row * groups;
            }
            out_col = a.g.out[0] + unit;
            out_ld = a.out_ld[0];
        }
    }
    const int total_steps = K / kStepElems;
    const int s_begin = ks * p.steps_per_split;
    const int s_end = active ? min(s_begin + p.steps_per_split, total_steps) : s_begin;

    uint4 w[R][U];
    uint16_t sb[R][U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int s = s_begin + u;
        if (s < s_end) {
#pragma unroll
            for (int r = 0; r < R; ++r) {
                w[r][u] = ld_weights_16(wrow[r] + (s * kSubwarp + l) * 4);
                sb[r][u] = ld_scale_bits(srow[r] + 2 * s + (l >> 2));
            }
        }
    }
    pdl_release_dependents();
    pdl_wait_prior_grids();

    for (int m0 = 0; m0 < M; m0 += MT) {
        if (m0 > 0) __syncthreads();   // the previous pass has finished reading the staged tokens
        // stage MT tokens as fp32, eight elements per thread and turn
        for (int idx = tid; idx < MT * (K / 8); idx += blockDim.x) {
            const int m = idx / (K / 8), e = (idx - m * (K / 8)) * 8;
            uint4 xv = make_uint4(0, 0, 0, 0);
            if (m0 + m < M) xv = *reinterpret_cast<const uint4*>(a.g.x + static_cast<size_t>(m0 + m) * K + e);
            const __half2* xh = reinterpret_cast<const __half2*>(&xv);
            const float2 f0 = __half22float2(xh[0]), f1 = __half22float2(xh[1]);
            const float2 f2 = __half22float2(xh[2]), f3 = __half22float2(xh[3]);
            float4* dst = reinterpret_cast<float4*>(s_x + m * xs + e + (e / kChunk) * 4);
            dst[0] = make_float4(f0.x, f0.y, f1.x, f1.y);
            dst[1] = make_float4(f2.x, f2.y, f3.x, f3.y);
        }
        __syncthreads();

        float2 acc2[R][MT];   // even / odd elements of K, added at the end
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int m = 0; m < MT; ++m) acc2[r][m] = make_float2(0.0f, 0.0f);

#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int s = s_begin + u;
            if (s < s_end) {
                const int c = s * kSubwarp + l;               // 32-element chunk along K
                const float* xc = s_x + c * (kChunk + 4);
                __half2 sc2[R];
#pragma unroll
                for (int r = 0; r < R; ++r) sc2[r] = __half2half2(__ushort_as_half(sb[r][u]));
#pragma unroll
                for (int j = 0; j < 4; ++j) {                  // one packed word = 8 elements
                    float2 wf[R][4];
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        uint32_t word = j == 0 ? w[r][u].x : j == 1 ? w[r][u].y : j == 2 ? w[r][u].z : w[r][u].w;
                        asm volatile("" : "+r"(word));   // dequantise here, in every token pass: hoisted out of the
                                                         // pass loop the fp32 weights would not fit the registers
                        __half2 h[4];
                        dequant_word_fp16(word, sc2[r], h);
#pragma unroll
                        for (int q = 0; q < 4; ++q) wf[r][q] = __half22float2(h[q]);
                    }
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        const float4 xa = *reinterpret_cast<const float4*>(xc + m * xs + j * 8);
                        const float4 xb = *reinterpret_cast<const float4*>(xc + m * xs + j * 8 + 4);
#pragma unroll
                        for (int r = 0; r < R; ++r) {
                            ffma2(acc2[r][m], wf[r][0], make_float2(xa.x, xa.y));
                            ffma2(acc2[r][m], wf[r][1], make_float2(xa.z, xa.w));
                            ffma2(acc2[r][m], wf[r][2], make_float2(xb.x, xb.y));
                            ffma2(acc2[r][m], wf[r][3], make_float2(xb.z, xb.w));
                        }
                    }
                    asm volatile("" ::: "memory");   // keep the next word's shared-memory loads behind this word's
                                                     // arithmetic: the weights already fill the register file
                }
            }
        }
        float acc[R][MT];
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int m = 0; m < MT; ++m) acc[r][m] = acc2[r][m].x + acc2[r][m].y;
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                acc[r][m] += __shfl_xor_sync(0xFFFFFFFFu, acc[r][m], 4);
                acc[r][m] += __shfl_xor_sync(0xFFFFFFFFu, acc[r][m], 2);
                acc[r][m] += __shfl_xor_sync(0xFFFFFFFFu, acc[r][m], 1);
            }
        if (p.ksplit > 1) {
            if (l == 0 && ks < p.ksplit) {
#pragma unroll
                for (int r = 0; r < R; ++r)
#pragma unroll
                    for (int m = 0; m < MT; ++m) s_part[((ks * p.units_per_cta + u_local) * R + r) * MT + m] = acc[r][m];
            }
            __syncthreads();
            if (ks == 0 && l == 0) {
#pragma unroll
                for (int r = 0; r < R; ++r)
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        float t = 0.0f;
                        for (int k = 0; k < p.ksplit; ++k) t += s_part[((k * p.units_per_cta + u_local) * R + r) * MT + m];
                        acc[r][m] = t;
                    }
            }
        }
        if (active && ks == 0 && l == 0) {
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                if (m0 + m < M) {
                    __half y;
                    if constexpr (MODE == kSwiglu) {
                        const float gate = acc[0][m];
                        y = __float2half_rn((gate / (1.0f + expf(-gate))) * acc[R - 1][m]);
                    } else {
                        y = __float2half_rn(acc[0][m]);
                        if constexpr (MODE == kPlain) {
                            if (a.g.residual != nullptr)
                                y = __hadd(y, a.g.residual[static_cast<size_t>(m0 + m) * out_ld + unit]);
                        }
                    }
                    out_col[static_cast<size_t>(m0 + m) * out_ld] = y;
                }
            }
        }
    }
}

}  // namespace w4
