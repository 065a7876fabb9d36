// Few-token W4A16 contraction (decode batches of about 4 to 32 tokens) as a weight-streaming kernel whose
// inner product runs on the warp-level tensor-core instruction mma.sync.m16n8k16 (fp16 x fp16 -> fp32).
//
// Why not the tcgen05 kernel here: below a few dozen tokens the contraction is bound by streaming the packed
// weights, and a tcgen05 launch carries fixed costs (tensor-memory allocation, TMA round trip, commit, the K-split
// exchange over a cluster) of 7-13 us whatever the token count.  This kernel keeps the decode GEMV's memory
// behaviour -- every 16-byte weight load of a lane issued before the wait for the previous kernel, whole grid
// resident, K slices inside the CTA -- and feeds the dequantised weights straight from registers into the
// A fragment of the MMA; the tokens are staged once per CTA in shared memory in B-fragment order.
//
// Arithmetic: the reference's prefill GEMM (src/kernels/gemm_prefill.cu:100-150): fp16 weights (q - 8) * scale with
// one rounding (dequant_word_fp16), fp16 activations, fp32 accumulation; epilogue as gemm_prefill.cu:257-275, 572-605.
//
// Mapping.  A warp owns 16 MMA rows: lane (g = lane / 4, t = lane % 4) loads, per 128-element step along K, the
// 16 bytes [32 t, 32 t + 32) of rows g and g + 8.  PLAIN / QKV: MMA row r is output row base + r.  SWIGLU: MMA row g
// is the gate row of pair base + g and row g + 8 its up row, so a lane ends with gate and up of the same output.
// The k index inside an MMA is free as long as A and B agree: MMA j (0..7) of a step takes, from each lane's piece,
// elements 4 j .. 4 j + 3 (k slots 2t, 2t+1 <- 4j, 4j+1; slots 2t+8, 2t+9 <- 4j+2, 4j+3), which are 8 contiguous
// bytes of the fp16 activation: one 8-byte shared-memory load per MMA and token tile.
#pragma once

#include "gemm_smallm.cuh"

namespace w4 {

struct SmallMmaPlan {
    int groups_per_cta;     // row groups (16 MMA rows each) of a CTA
    int ksplit;             // K slices (one warp per group and slice)
    int steps_per_split;    // 128-element steps per slice (<= U)
    int passes_tokens;      // tokens staged per pass (8 * NT)
};

// Shared-memory cell (8 bytes = 4 fp16) of the staged activation: elements k = 128 step + 32 t + 4 j + {0..3} of
// token `tok`; TOK tokens per pass.  The 32 lanes of an MMA's B load read 32 consecutive cells.
__host__ __device__ __forceinline__ int mma_x_cell(int step, int j, int tok, int t, int TOK) {
    return ((step * 8 + j) * TOK + tok) * 4 + t;
}

__device__ __forceinline__ void mma_m16n8k16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                             uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int MODE, int U, int NT>
__global__ void __launch_bounds__(512) gemm_smallm_mma_kernel(const SmallMArgs a, const SmallMmaPlan p) {
    constexpr int TOK = 8 * NT;
    constexpr int UW = (MODE == kSwiglu) ? 8 : 16;   // outputs per warp
    extern __shared__ __align__(16) uint8_t s_raw[];
    const int K = a.g.K, M = a.g.M;
    uint2* s_x = reinterpret_cast<uint2*>(s_raw);                                       // [K / 4][TOK] cells
    float* s_part = reinterpret_cast<float*>(s_raw + static_cast<size_t>(K / 4) * TOK * 8);   // K-slice partials
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int ug = warp % p.groups_per_cta, ks = warp / p.groups_per_cta;
    const int unit0 = (blockIdx.x * p.groups_per_cta + ug) * UW;    // first output of this warp
    const bool active = ks < p.ksplit && unit0 < a.units;
    const int words = K / 8, groups = K / kGroup;

    // the two weight rows of this lane (MMA rows g and g + 8) and where their outputs go
    const uint32_t* wrow[2] = {nullptr, nullptr};
    const __half* srow[2] = {nullptr, nullptr};
    __half* out_col[2] = {nullptr, nullptr};
    int out_ld = 0;
    int out_unit[2] = {0, 0};
    if (active) {
        if constexpr (MODE == kSwiglu) {
            const size_t pair = static_cast<size_t>(unit0 + g);
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                wrow[r] = a.g.qweight[0] + (2 * pair + r) * words;
                srow[r] = a.g.scales[0] + (2 * pair + r) * groups;
            }
            out_col[0] = a.g.out[0] + pair;
            out_ld = a.out_ld[0];
            out_unit[0] = static_cast<int>(pair);
        } else {
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                int tns = 0, local = unit0 + g + 8 * r;
                if constexpr (MODE == kQkv) {
                    if (local >= a.g.rows[0]) { local -= a.g.rows[0]; tns = 1; }
                    if (tns == 1 && local >= a.g.rows[1]) { local -= a.g.rows[1]; tns = 2; }
                }
                wrow[r] = a.g.qweight[tns] + static_cast<size_t>(local) * words;
                srow[r] = a.g.scales[tns] + static_cast<size_t>(local) * groups;
                out_col[r] = a.g.out[tns] + local;
                out_unit[r] = local;
                out_ld = a.out_ld[tns];     // the 16 rows of a warp come from one tensor (host check)
            }
        }
    }
    const int total_steps = K / kGroup;
    const int s_begin = ks * p.steps_per_split;
    const int s_end = active ? min(s_begin + p.steps_per_split, total_steps) : s_begin;

    // Half of a lane's weight loads go out before the wait for the previous kernel, the other half right behind the
    // first token loads: the tokens, which everything waits for, then do not queue behind the whole weight stream,
    // and the MMAs of the early steps run while the late steps' weights arrive.
    constexpr int kEarlyU = U == 8 ? U : U / 2;   // (the 8-step form has no registers to spare for the token batch)
    uint4 w[2][U];
    uint16_t sb[2][U];
#pragma unroll
    for (int u = 0; u < kEarlyU; ++u) {
        const int s = s_begin + u;
        if (s < s_end) {
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                w[r][u] = ld_weights_16(wrow[r] + s * 16 + t * 4);
                sb[r][u] = ld_scale_bits(srow[r] + s);
            }
        }
    }
    pdl_release_dependents();
    pdl_wait_prior_grids();

    for (int m0 = 0; m0 < M; m0 += TOK) {
        if (m0 > 0) __syncthreads();   // the previous pass has finished reading the staged tokens
        // stage TOK tokens in B-fragment order: 16 bytes of a token = two cells (j, j + 1) of the same (step, t)
        // (every global round trip here is on the critical path: several loads of a thread are in flight at once)
        constexpr int kBatch = U == 8 ? 4 : 8;   // what the registers beside the weights allow
        const int pieces = TOK * (K / 8);
        auto load_batch = [&](int base, uint4 (&xv)[kBatch]) {
#pragma unroll
            for (int b = 0; b < kBatch; ++b) {
                const int idx = base + b * blockDim.x + tid;
                const int tok = idx / (K / 8), e = (idx - tok * (K / 8)) * 8;
                xv[b] = make_uint4(0, 0, 0, 0);
                if (idx < pieces && m0 + tok < M)
                    xv[b] = *reinterpret_cast<const uint4*>(a.g.x + static_cast<size_t>(m0 + tok) * K + e);
            }
        };
        auto store_batch = [&](int base, const uint4 (&xv)[kBatch]) {
#pragma unroll
            for (int b = 0; b < kBatch; ++b) {
                const int idx = base + b * blockDim.x + tid;
                if (idx < pieces) {
                    const int tok = idx / (K / 8), e = (idx - tok * (K / 8)) * 8;
                    const int step = e >> 7, tt = (e >> 5) & 3, j0 = (e & 31) >> 2;
                    s_x[mma_x_cell(step, j0, tok, tt, TOK)] = make_uint2(xv[b].x, xv[b].y);
                    s_x[mma_x_cell(step, j0 + 1, tok, tt, TOK)] = make_uint2(xv[b].z, xv[b].w);
                }
            }
        };
        {
            uint4 xv[kBatch];
            load_batch(0, xv);
            if (m0 == 0) {     // the rest of the weights, right behind the first token loads
#pragma unroll
                for (int u = kEarlyU; u < U; ++u) {
                    const int s = s_begin + u;
                    if (s < s_end) {
#pragma unroll
                        for (int r = 0; r < 2; ++r) {
                            w[r][u] = ld_weights_16(wrow[r] + s * 16 + t * 4);
                            sb[r][u] = ld_scale_bits(srow[r] + s);
                        }
                    }
                }
            }
            store_batch(0, xv);
        }
        for (int base = kBatch * blockDim.x; base < pieces; base += kBatch * blockDim.x) {
            uint4 xv[kBatch];
            load_batch(base, xv);
            store_batch(base, xv);
        }
        __syncthreads();

        // two accumulators per token tile (even / odd MMA of a word): consecutive MMAs of a warp do not wait for each other
        constexpr int ACC = NT <= 2 ? 2 : 1;
        float d2[NT][ACC][4];
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int c = 0; c < ACC; ++c)
#pragma unroll
                for (int i = 0; i < 4; ++i) d2[n][c][i] = 0.0f;

#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int s = s_begin + u;
            if (s < s_end) {
                const __half2 sc0 = __half2half2(__ushort_as_half(sb[0][u]));
                const __half2 sc1 = __half2half2(__ushort_as_half(sb[1][u]));
#pragma unroll
                for (int m = 0; m < 4; ++m) {                 // one packed word of each row = two MMAs
                    uint32_t word0 = m == 0 ? w[0][u].x : m == 1 ? w[0][u].y : m == 2 ? w[0][u].z : w[0][u].w;
                    uint32_t word1 = m == 0 ? w[1][u].x : m == 1 ? w[1][u].y : m == 2 ? w[1][u].z : w[1][u].w;
                    asm volatile("" : "+r"(word0), "+r"(word1));   // dequantise in every token pass: the fp16 weights
                                                                   // of all steps would not fit the registers
                    __half2 h0[4], h1[4];
                    dequant_word_fp16(word0, sc0, h0);
                    dequant_word_fp16(word1, sc1, h1);
#pragma unroll
                    for (int jj = 0; jj < 2; ++jj) {
                        const int j = 2 * m + jj;
                        const uint32_t a0 = *reinterpret_cast<const uint32_t*>(&h0[2 * jj]);
                        const uint32_t a1 = *reinterpret_cast<const uint32_t*>(&h1[2 * jj]);
                        const uint32_t a2 = *reinterpret_cast<const uint32_t*>(&h0[2 * jj + 1]);
                        const uint32_t a3 = *reinterpret_cast<const uint32_t*>(&h1[2 * jj + 1]);
#pragma unroll
                        for (int n = 0; n < NT; ++n) {
                            const uint2 b = s_x[mma_x_cell(s, j, n * 8 + g, t, TOK)];
                            mma_m16n8k16(d2[n][jj % ACC], a0, a1, a2, a3, b.x, b.y);
                        }
                    }
                }
            }
        }

        float d[NT][4];
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) d[n][i] = ACC == 2 ? d2[n][0][i] + d2[n][ACC - 1][i] : d2[n][0][i];
        // K slices: the warps of a row group add their accumulators through shared memory, in slice order
        if (p.ksplit > 1) {
            if (ks < p.ksplit) {
#pragma unroll
                for (int n = 0; n < NT; ++n)
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        s_part[(((ks * p.groups_per_cta + ug) * NT + n) * 4 + i) * 32 + lane] = d[n][i];
            }
            __syncthreads();
            if (ks == 0) {
#pragma unroll
                for (int n = 0; n < NT; ++n)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        float sum = 0.0f;
                        for (int k = 0; k < p.ksplit; ++k)
                            sum += s_part[(((k * p.groups_per_cta + ug) * NT + n) * 4 + i) * 32 + lane];
                        d[n][i] = sum;
                    }
            }
        }
        if (active && ks == 0) {
#pragma unroll
            for (int n = 0; n < NT; ++n) {
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int tok = m0 + n * 8 + 2 * t + i;      // accumulators 0/1: row g, 2/3: row g + 8
                    if (tok < M) {
                        if constexpr (MODE == kSwiglu) {
                            const float gate = d[n][i], up = d[n][2 + i];
                            out_col[0][static_cast<size_t>(tok) * out_ld] = __float2half_rn((gate / (1.0f + expf(-gate))) * up);
                        } else {
#pragma unroll
                            for (int r = 0; r < 2; ++r) {
                                __half y = __float2half_rn(d[n][2 * r + i]);
                                if constexpr (MODE == kPlain) {
                                    if (a.g.residual != nullptr)
                                        y = __hadd(y, a.g.residual[static_cast<size_t>(tok) * out_ld + out_unit[r]]);
                                }
                                out_col[r][static_cast<size_t>(tok) * out_ld] = y;
                            }
                        }
                    }
                }
            }
        }
    }
}

}  // namespace w4
