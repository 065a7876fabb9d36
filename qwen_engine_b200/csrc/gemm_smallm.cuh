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

}  // namespace w4
