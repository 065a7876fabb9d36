// Batch-1 decode GEMV on W4 group-128 weights and Q8_1 activations (sm_100a).
//
// Replaces the reference's gemv_w4a8_u4_kernel / gemv_qkv_w4a8_u4_kernel /
// gemv_dual_gate_up_swiglu_w4a8_u4_kernel, their 32-bit fall-backs and the two fp16-input
// "standalone" kernels (src/kernels/gemv_w4a16.cu:74-858) with one kernel template.
//
// Work split.  Eight lanes share a weight row; each lane reads 16 bytes (32 weights) per
// step, so a sub-warp consumes 256 elements of K per step.  A CTA holds
// units_per_cta x ksplit sub-warps: `units_per_cta` output rows (row pairs for SwiGLU) and
// `ksplit` slices of K, chosen on the host so that even a 1536 x 1536 projection gives
// every SM a CTA and every lane only a handful of loads -- the whole matrix is then in
// flight at once, which is what bounds these latency-limited shapes.
//
// Order inside a CTA: (1) issue the first batch of weight and scale loads into registers --
// they do not depend on the previous kernel; (2) release dependents / wait for the prior
// grid (programmatic dependent launch), then stage the activation in shared memory
// (copy of the Q8_1 arrays, or quantise fp16 on the fly); (3) dp4a over the chunks,
// fp32 accumulate per lane; (4) 3-step shuffle reduce over the sub-warp, shared-memory
// reduce over the K slices; (5) epilogue (residual / QKV scatter / SwiGLU), fp16 store.
#include <algorithm>

#include "sampling.cuh"
#include "w4a16_common.cuh"
#include "w4a16_internal.hpp"

namespace w4 {
namespace {

constexpr int kMaxThreads = 256;
constexpr int kMaxSubwarps = kMaxThreads / kSubwarp;  // 32
constexpr float kRmsEps = 1e-6f;                      // reference include/config.cuh:20 RMS_NORM_EPS

// XIN: where the activation comes from.
enum XIn { kXQ8 = 0,        // pre-quantised Q8_1 arrays in global memory
           kXFp16 = 1,      // fp16 vector, quantised in the prologue
           kXFp16Norm = 2,  // fp16 vector, RMSNorm then quantised in the prologue
           kXF32Heads = 3,  // fp32 attention accumulators, quantised per head with the flash-decode epilogue's rule
           kXFp16Amax = 4 };  // fp16 vector whose per-group |max| the producing launch published: quantised without a reduction

// Shared memory behind the staged activation and the K-split partial sums, kXFp16Amax only: 1/scale per group,
// then the raw fp16 vector (16-byte aligned).
__host__ __device__ inline size_t amax_stage_offset(int K, int part_floats) {
    return (staged_x_bytes(K) + static_cast<size_t>(part_floats) * 4 + 15) / 16 * 16;
}
__host__ __device__ inline size_t amax_stage_bytes(int K) { return (static_cast<size_t>(K / kGroup) * 4 + 15) / 16 * 16 + static_cast<size_t>(K) * 2; }

// Register caps.  What matters in a chain of dependent launches is that the CTAs of the NEXT launch become
// resident, and issue their weight loads, while this one still runs: 88 registers for the single-row forms with
// 8 loads per lane (down: three 192-thread CTAs per SM leave room for CTAs of the next QKV launch; measured
// 1 % of the 28-layer pass against a cap of 96, no spills), 128 for the rest (the SwiGLU row pairs spill below
// 120; capping the 4-load forms at 64 costs them 0.2 us per launch).
constexpr int gemv_reg_cap(int mode, int u) { return (mode != kSwiglu && u == 8) ? 88 : 128; }

template <int MODE, int U, int XIN, bool ALIGNED16>
__global__ void __maxnreg__(gemv_reg_cap(MODE, U)) gemv_w4_kernel(const GemvArgs a) {
    constexpr int R = (MODE == kSwiglu) ? 2 : 1;  // weight rows per sub-warp
    extern __shared__ __align__(16) uint8_t smem[];
    const int K = a.K;
    int8_t* s_q8 = reinterpret_cast<int8_t*>(smem);
    int32_t* s_seed = reinterpret_cast<int32_t*>(smem + K);
    float* s_scale = reinterpret_cast<float*>(smem + K + (K / kChunk) * 4);
    float* s_part = reinterpret_cast<float*>(smem + staged_x_bytes(K));

    const int tid = threadIdx.x;
    const int sub = tid >> 3, l = tid & 7;
    const int u_local = sub % a.units_per_cta;
    const int ks = sub / a.units_per_cta;
    const int unit = blockIdx.x * a.units_per_cta + u_local;
    const bool active = unit < a.units;

    // Resolve the weight rows this sub-warp reads and where its output goes.
    const uint32_t* wrow[R];
    const __half* srow[R];
    __half* out_ptr = nullptr;
    const int words = K / 8, groups = K / kGroup;
    if (active) {
        if constexpr (MODE == kQkv) {
            int t = 0, local = unit;
            if (local >= a.rows[0]) { local -= a.rows[0]; t = 1; }
            if (t == 1 && local >= a.rows[1]) { local -= a.rows[1]; t = 2; }
            wrow[0] = a.qweight[t] + static_cast<size_t>(local) * words;
            srow[0] = a.scales[t] + static_cast<size_t>(local) * groups;
            out_ptr = a.out[t] + local;
        } else {
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const size_t row = static_cast<size_t>(unit) * R + r;
                wrow[r] = a.qweight[0] + row * words;
                srow[r] = a.scales[0] + row * groups;
            }
            out_ptr = a.out[0] + unit;
        }
    } else {
#pragma unroll
        for (int r = 0; r < R; ++r) { wrow[r] = nullptr; srow[r] = nullptr; }
    }

    const int total_steps = K / kStepElems;
    const int s_begin = ks * a.steps_per_split;
    const int s_end = active ? min(s_begin + a.steps_per_split, total_steps) : s_begin;

    uint4 w[R][U];
    uint16_t sb[R][U];
    auto issue = [&](int s0) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int s = s0 + u;
            if (s < s_end) {
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    w[r][u] = ld_weights<ALIGNED16>(wrow[r] + (s * kSubwarp + l) * 4);
                    sb[r][u] = ld_scale_bits(srow[r] + 2 * s + (l >> 2));
                }
            }
        }
    };

    issue(s_begin);
    if constexpr (MODE == kSwiglu) {
        // Q8_1 epilogue: its remote shared-memory stores need every CTA of the cluster to have started; each CTA
        // says so here (the wait sits just before the stores, so it overlaps everything in between).
        if (a.q8_out != nullptr) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
    }
    // Everything that does not depend on the prior grid goes before the wait: the weights above and the
    // RMSNorm gain.  After it, every global round trip is on the critical path between two GEMVs, so the
    // residual element is requested first and the activation is staged with one round trip.
    [[maybe_unused]] uint4 gam[kStageRounds];
    [[maybe_unused]] bool regs_form = false;
    if constexpr (XIN == kXFp16 || XIN == kXFp16Norm) {
        regs_form = stage_regs_ok(a.x_fp16, XIN == kXFp16Norm ? static_cast<const void*>(a.gamma) : nullptr, K);
        if constexpr (XIN == kXFp16Norm) {
            if (regs_form) prefetch_gamma(a.gamma, K, gam);
        }
    }
    pdl_release_dependents();
    pdl_wait_prior_grids();

    [[maybe_unused]] __half res_pre = __ushort_as_half(0);
    if constexpr (MODE == kPlain) {
        if (active && ks == 0 && l == 0 && a.residual != nullptr) res_pre = a.residual[unit];
    }
    if (blockIdx.x == 0)   // scratch of a later launch
        for (int i = tid; i < a.clear_count; i += blockDim.x) a.clear_words[i] = 0u;
    if constexpr (XIN == kXFp16Norm) {
        if (regs_form) stage_x_fp16_regs<true>(a.x_fp16, gam, K, kRmsEps, s_q8, s_seed, s_scale, a.sumsq_in);
        else stage_x_from_fp16_rmsnorm(a.x_fp16, a.gamma, K, kRmsEps, s_q8, s_seed, s_scale);
    } else if constexpr (XIN == kXFp16Amax) {
        uint8_t* extra = smem + amax_stage_offset(K, a.ksplit * a.units_per_cta * R);
        float* s_inv = reinterpret_cast<float*>(extra);
        __half* s_raw = reinterpret_cast<__half*>(extra + (static_cast<size_t>(K / kGroup) * 4 + 15) / 16 * 16);
        stage_x_fp16_amax(a.x_fp16, a.amax_in, K, s_q8, s_seed, s_scale, s_raw, s_inv);
    } else if constexpr (XIN == kXFp16) {
        if (regs_form) stage_x_fp16_regs<false>(a.x_fp16, gam, K, kRmsEps, s_q8, s_seed, s_scale);
        else stage_x_from_fp16(a.x_fp16, K, s_q8, s_seed, s_scale);
    } else if constexpr (XIN == kXF32Heads) {
        stage_x_from_f32_heads(a.x_f32, K, s_q8, s_seed, s_scale);
    } else {
        if (!stage_x_from_q8_1_regs<(R * U >= 16)>(a.q8, a.xscale, a.sum8, K, a.vec_ok != 0, s_q8, s_seed, s_scale))
            stage_x_from_q8_1(a.q8, a.xscale, a.sum8, K, a.vec_ok != 0, s_q8, s_seed, s_scale);
    }
    __syncthreads();

    float acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = 0.0f;

    for (int s0 = s_begin; s0 < s_end; s0 += U) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int s = s0 + u;
            if (s < s_end) {
                const int c = s * kSubwarp + l;  // 32-element chunk index along K
                const uint4 xa = reinterpret_cast<const uint4*>(s_q8)[q8_slot(c, 0)];
                const uint4 xb = reinterpret_cast<const uint4*>(s_q8)[q8_slot(c, 1)];
                const int32_t seed = s_seed[c];
                const float xs = s_scale[c >> 2];
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const int32_t d = chunk_dot(w[r][u], xa, xb, seed);
                    const float ws = __half2float(__ushort_as_half(sb[r][u]));
                    acc[r] = fmaf(static_cast<float>(d), ws * xs, acc[r]);
                }
            }
        }
        if (s0 + U < s_end) issue(s0 + U);
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        acc[r] += __shfl_xor_sync(0xFFFFFFFFu, acc[r], 4);
        acc[r] += __shfl_xor_sync(0xFFFFFFFFu, acc[r], 2);
        acc[r] += __shfl_xor_sync(0xFFFFFFFFu, acc[r], 1);
    }

    if (a.ksplit > 1) {
        if (l == 0 && ks < a.ksplit) {  // padding threads of a rounded-up block have ks >= ksplit
#pragma unroll
            for (int r = 0; r < R; ++r) s_part[(ks * a.units_per_cta + u_local) * R + r] = acc[r];
        }
        __syncthreads();
        if (ks == 0 && l == 0) {
#pragma unroll
            for (int r = 0; r < R; ++r) {
                float t = 0.0f;
                for (int k = 0; k < a.ksplit; ++k) t += s_part[(k * a.units_per_cta + u_local) * R + r];
                acc[r] = t;
            }
        }
    }

    [[maybe_unused]] float y_rounded = 0.0f;   // SWIGLU: the fp16 output as a float, for the Q8_1 epilogue
    if (active && ks == 0 && l == 0) {
        float y;
        if constexpr (MODE == kSwiglu) {
            const float gate = acc[0];
            y = (gate / (1.0f + expf(-gate))) * acc[R - 1];
        } else {
            y = acc[0];
            if constexpr (MODE == kPlain) {
                if (a.residual != nullptr) y += __half2float(res_pre);
            }
        }
        const __half yh = __float2half_rn(y);
        *out_ptr = yh;
        y_rounded = __half2float(yh);
        if constexpr (MODE == kPlain) {
            for (int p = 0; p < a.num_peers; ++p) a.peer_out[p][unit] = yh;   // slice into every peer's buffer
        }
    }
    if constexpr (MODE == kPlain) {
        // Squares of this launch's fp16 outputs for the next RMSNorm: the output threads of a warp are its lanes
        // 0, 8, 16, 24; one double atomic per warp that has any.
        if (a.sumsq_out != nullptr && (tid >> 5) * 4 < a.units_per_cta) {
            double sq = static_cast<double>(y_rounded) * static_cast<double>(y_rounded);   // 0 in lanes without an output
            sq += __shfl_xor_sync(0xFFFFFFFFu, sq, 8);
            sq += __shfl_xor_sync(0xFFFFFFFFu, sq, 16);
            if ((tid & 31) == 0) atomicAdd(a.sumsq_out + (blockIdx.x % kSumsqSlots), sq);
        }
    }
    if constexpr (MODE == kSwiglu) {
        // |max| of every group of 128 outputs for the launch that quantises them: a warp's four outputs are
        // consecutive and start at a multiple of four, hence in one group.
        if (a.amax_out != nullptr && ks == 0) {
            const uint32_t m = __reduce_max_sync(0xFFFFFFFFu, __float_as_uint(fabsf(y_rounded)));
            if ((tid & 31) == 0 && m != 0u) atomicMax(a.amax_out + (blockIdx.x * a.units_per_cta + u_local) / kGroup, m);
        }
    }

    if constexpr (MODE == kSwiglu) {
        // Q8_1 of the output vector in the same launch.  The launch guarantees 32 outputs per CTA, no K
        // split and clusters of four CTAs, i.e. one quantisation group of 128 per cluster: the CTAs swap
        // their |max| through distributed shared memory, one cluster barrier, then each quantises its own
        // 32 outputs (one chunk: 32 bytes, four sum8 entries) with the group's scale.  Same arithmetic as
        // quantize_group128_lane, so the arrays equal the stand-alone quantiser's bit for bit.
        if (a.q8_out != nullptr) {
            __shared__ float s_y[kMaxSubwarps];
            __shared__ float s_cluster_max[4];
            if (l == 0) s_y[sub] = y_rounded;
            __syncthreads();
            uint32_t rank;
            asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
            asm volatile("barrier.cluster.wait.aligned;" ::: "memory");   // pairs with the arrive at kernel entry
            float v = 0.0f;
            if (tid < 32) {
                v = s_y[tid];
                float m = fabsf(v);
#pragma unroll
                for (int mask = 16; mask > 0; mask >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, mask));
                if (tid < 4) {   // lane t puts this CTA's maximum into slot `rank` of CTA t
                    const uint32_t local = static_cast<uint32_t>(__cvta_generic_to_shared(&s_cluster_max[rank]));
                    uint32_t remote;
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(static_cast<uint32_t>(tid)));
                    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(m) : "memory");
                }
            }
            asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
            asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
            if (tid < 32) {
                const float m = fmaxf(fmaxf(s_cluster_max[0], s_cluster_max[1]), fmaxf(s_cluster_max[2], s_cluster_max[3]));
                const float d = fmaxf(__fdiv_rn(m, 127.0f), 1e-8f);
                const float inv_d = __fdiv_rn(1.0f, d);
                int q = __float2int_rn(__fmul_rn(v, inv_d));
                q = max(-127, min(127, q));
                const int first = blockIdx.x * kMaxSubwarps;
                a.q8_out[first + tid] = static_cast<int8_t>(q);
                int sum = q;
                sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
                sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
                sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 4);
                if ((tid & 7) == 0) a.sum8_out[(first + tid) >> 3] = -8 * sum;
                if (rank == 0 && tid == 0) a.xscale_out[first / kGroup] = d;
            }
        }
    }
}


// ---- bulk-copy form -----------------------------------------------------------------------------
// The same GEMV with the CTA's weight rows brought into SHARED MEMORY by the copy engine (cp.async.bulk,
// completion on an mbarrier) instead of into registers.  A CTA's rows are adjacent in the row-major matrix,
// so its whole share of the weights is one contiguous range: one elected thread asks for it before the wait
// for the previous kernel and the bytes arrive without holding a register.  The kernel then needs about 60
// registers per thread instead of 96-128, which is what lets the CTAs of the NEXT projection become
// resident, and start their own copies, while this one still computes: on-chip staging for weights is the
// shared memory of all SMs (33 MB) in addition to the register file.
// Work split, arithmetic and summation order are those of gemv_w4_kernel (same plan, same chunk_dot, the K
// slices added in the same order), so both forms give the same bits.
//
// CLUSTERK (PLAIN only): the K slices of a row block are spread over the CTAs of a thread-block cluster
// instead of over the sub-warps of one CTA.  Each CTA then stages -- and, for an fp16 input, quantises --
// only ITS slice of the activation (a vector of 8960 costs every CTA six quantiser rounds otherwise), copies
// 32 rows x its slice of the weights, and the partial sums meet in the leading CTA through distributed shared
// memory: the others store their fp32 partial into the leader's array, one cluster barrier, the leader adds
// them in slice order.  This is what lets the down projection take the fp16 MLP activation directly, without
// a quantiser launch in front of it.
constexpr unsigned kBulkPollLimit = 1u << 20;     // polls of the copy barrier before a CTA gives up (tens of ms)
__device__ unsigned int g_gemv_copy_timeouts = 0; // bounded waits that ran out (0 in normal operation)

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

struct BulkLayout {            // byte offsets inside the CTA's dynamic shared memory
    int part, weights, bar, total;
};
__host__ __device__ inline BulkLayout bulk_layout(int klen, int part_floats, int weight_bytes) {
    BulkLayout L;
    L.part = static_cast<int>((staged_x_bytes(klen) + 15) & ~size_t(15));
    L.weights = (L.part + part_floats * 4 + 127) & ~127;
    L.bar = L.weights + ((weight_bytes + 15) & ~15);
    L.total = L.bar + 16;
    return L;
}

template <int MODE, int XIN, bool CLUSTERK>
__global__ void __maxnreg__(64) gemv_w4_bulk_kernel(const GemvArgs a) {
    static_assert(!CLUSTERK || (MODE == kPlain && (XIN == kXQ8 || XIN == kXFp16)), "cluster K split: plain rows, no norm");
    constexpr int R = (MODE == kSwiglu) ? 2 : 1;
    constexpr int U = 8;       // scale words a lane keeps per batch of steps
    extern __shared__ __align__(16) uint8_t smem[];
    const int K = a.K;
    const int tid = threadIdx.x;
    const int sub = tid >> 3, l = tid & 7;

    // Which rows and which part of K this CTA covers.
    uint32_t krank = 0;
    int row_block = blockIdx.x;
    if constexpr (CLUSTERK) {
        asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(krank));
        row_block = blockIdx.x / a.ksplit;
        asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");   // "this CTA has started", see below
    }
    const int total_steps = K / kStepElems;
    const int k_step0 = CLUSTERK ? static_cast<int>(krank) * a.steps_per_split : 0;    // first 256-element step of the CTA
    const int cta_steps = CLUSTERK ? max(0, min(a.steps_per_split, total_steps - k_step0)) : total_steps;
    const int klen = cta_steps * kStepElems;
    const int u_local = CLUSTERK ? sub : sub % a.units_per_cta;
    const int ks = CLUSTERK ? 0 : sub / a.units_per_cta;
    const int unit0 = row_block * a.units_per_cta;
    const int unit = unit0 + u_local;
    const bool active = unit < a.units && (CLUSTERK ? sub < a.units_per_cta : ks < a.ksplit);
    const int cta_units = min(a.units_per_cta, a.units - unit0);

    // offsets are taken from the longest K range of any CTA of the cluster, so that they agree in all of them
    // (the partial sums are addressed in the leader's shared memory by the offset they have here)
    const int klen_max = CLUSTERK ? a.steps_per_split * kStepElems : K;
    const BulkLayout L = bulk_layout(klen_max, a.ksplit * a.units_per_cta * R, a.units_per_cta * R * (klen_max / 2));
    int8_t* s_q8 = reinterpret_cast<int8_t*>(smem);
    int32_t* s_seed = reinterpret_cast<int32_t*>(smem + klen_max);
    float* s_scale = reinterpret_cast<float*>(smem + klen_max + (klen_max / kChunk) * 4);
    float* s_part = reinterpret_cast<float*>(smem + L.part);
    const uint32_t s_w = smem_addr(smem + L.weights);
    const uint32_t bar = smem_addr(smem + L.bar);

    // the CTA's weight rows, scales and outputs
    const int words = K / 8, groups = K / kGroup;
    const uint32_t* wbase = a.qweight[0];
    const __half* sbase = a.scales[0];
    __half* obase = a.out[0];
    int first = unit0;                       // first unit of the CTA inside its tensor
    if constexpr (MODE == kQkv) {            // a CTA's rows come from one tensor (the planner sees to it)
        int t = 0;
        if (first >= a.rows[0]) { first -= a.rows[0]; t = 1; }
        if (t == 1 && first >= a.rows[1]) { first -= a.rows[1]; t = 2; }
        wbase = a.qweight[t]; sbase = a.scales[t]; obase = a.out[t];
    }
    const size_t row0 = static_cast<size_t>(first) * R;          // first weight row of the CTA
    const int row_bytes = klen / 2;                             // bytes of one row inside the CTA's K range

    // (1) one thread starts the copies: a contiguous range when the CTA takes whole rows, else one piece per row
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        const uint32_t bytes = static_cast<uint32_t>(cta_units * R) * static_cast<uint32_t>(row_bytes);
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
        const uint8_t* src = reinterpret_cast<const uint8_t*>(wbase + row0 * words) + static_cast<size_t>(k_step0) * (kStepElems / 2);
        if constexpr (!CLUSTERK) {
            constexpr uint32_t kPiece = 16384;   // several requests in flight rather than one long one
            for (uint32_t off = 0; off < bytes; off += kPiece)
                bulk_copy_g2s(s_w + off, src + off, min(kPiece, bytes - off), bar);
        }
    }
    if constexpr (CLUSTERK) {
        // one piece per row (the rows' slices are not adjacent in memory), issued by the lanes of warp 0 side by side
        if (tid < 32) {
            __syncwarp();      // after lane 0 has set up the barrier
            const uint8_t* src = reinterpret_cast<const uint8_t*>(wbase + row0 * words) + static_cast<size_t>(k_step0) * (kStepElems / 2);
            for (int r = tid; r < cta_units; r += 32)
                bulk_copy_g2s(s_w + r * row_bytes, src + static_cast<size_t>(r) * (K / 2), row_bytes, bar);
        }
    }

    // (2) the lane's scale words (2 bytes each, not alignable for a bulk copy) and the RMSNorm gain: weights of
    // the model, so they too are requested before the wait
    const int s_begin = CLUSTERK ? 0 : ks * a.steps_per_split;
    const int s_end = active ? (CLUSTERK ? cta_steps : min(s_begin + a.steps_per_split, total_steps)) : s_begin;
    uint16_t sb[R][U];
    auto load_scales = [&](int s0) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int s = s0 + u;
            if (s < s_end) {
#pragma unroll
                for (int r = 0; r < R; ++r)
                    sb[r][u] = ld_scale_bits(sbase + (row0 + static_cast<size_t>(u_local) * R + r) * groups + 2 * (k_step0 + s) + (l >> 2));
            }
        }
    };
    load_scales(s_begin);
    [[maybe_unused]] uint4 gam[kStageRounds];
    [[maybe_unused]] bool regs_form = false;
    const __half* x16 = a.x_fp16 != nullptr ? a.x_fp16 + static_cast<size_t>(k_step0) * kStepElems : nullptr;
    if constexpr (XIN == kXFp16 || XIN == kXFp16Norm) {
        regs_form = stage_regs_ok(x16, XIN == kXFp16Norm ? static_cast<const void*>(a.gamma) : nullptr, klen);
        if constexpr (XIN == kXFp16Norm) {
            if (regs_form) prefetch_gamma(a.gamma, klen, gam);
        }
    }
    pdl_release_dependents();
    pdl_wait_prior_grids();

    // (3) the activation: everything after the wait is on the critical path between two projections
    [[maybe_unused]] __half res_pre = __ushort_as_half(0);
    if constexpr (MODE == kPlain) {
        if (active && ks == 0 && krank == 0 && l == 0 && a.residual != nullptr) res_pre = a.residual[unit];
    }
    if constexpr (XIN == kXFp16Norm) {
        if (regs_form) stage_x_fp16_regs<true>(x16, gam, klen, kRmsEps, s_q8, s_seed, s_scale);
        else stage_x_from_fp16_rmsnorm(x16, a.gamma, klen, kRmsEps, s_q8, s_seed, s_scale);
    } else if constexpr (XIN == kXFp16) {
        if (regs_form) stage_x_fp16_regs<false>(x16, gam, klen, kRmsEps, s_q8, s_seed, s_scale);
        else stage_x_from_fp16(x16, klen, s_q8, s_seed, s_scale);
    } else if constexpr (XIN == kXF32Heads) {
        stage_x_from_f32_heads(a.x_f32, klen, s_q8, s_seed, s_scale);
    } else {
        const int8_t* q8 = a.q8 + static_cast<size_t>(k_step0) * kStepElems;
        const float* xsc = a.xscale + k_step0 * (kStepElems / kGroup);
        const int32_t* s8 = a.sum8 + k_step0 * (kStepElems / 8);
        if (!stage_x_from_q8_1_regs<false>(q8, xsc, s8, klen, a.vec_ok != 0, s_q8, s_seed, s_scale))
            stage_x_from_q8_1(q8, xsc, s8, klen, a.vec_ok != 0, s_q8, s_seed, s_scale);
    }
    __syncthreads();

    // (4) the weights must have landed (bounded wait; phase 0 of a barrier used once)
    {
        bool landed = false;
        for (unsigned it = 0; it < kBulkPollLimit; ++it) {
            uint32_t ok;
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                         : "=r"(ok) : "r"(bar), "r"(0u) : "memory");
            if (ok) { landed = true; break; }
            if (it > 64) __nanosleep(32);
        }
        if (!landed && tid == 0) atomicAdd(&g_gemv_copy_timeouts, 1u);   // the output of this launch is invalid
    }

    float acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = 0.0f;
    const uint32_t w_lane = s_w + static_cast<uint32_t>(u_local * R) * row_bytes + l * 16;
    for (int s0 = s_begin; s0 < s_end; s0 += U) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int s = s0 + u;
            if (s < s_end) {
                const int c = s * kSubwarp + l;   // 32-element chunk index inside the CTA's K range
                const uint4 xa = reinterpret_cast<const uint4*>(s_q8)[q8_slot(c, 0)];
                const uint4 xb = reinterpret_cast<const uint4*>(s_q8)[q8_slot(c, 1)];
                const int32_t seed = s_seed[c];
                const float xs = s_scale[c >> 2];
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const uint4 w = lds128(w_lane + r * row_bytes + s * (kSubwarp * 16));
                    const int32_t d = chunk_dot(w, xa, xb, seed);
                    const float ws = __half2float(__ushort_as_half(sb[r][u]));
                    acc[r] = fmaf(static_cast<float>(d), ws * xs, acc[r]);
                }
            }
        }
        if (s0 + U < s_end) load_scales(s0 + U);
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        acc[r] += __shfl_xor_sync(0xFFFFFFFFu, acc[r], 4);
        acc[r] += __shfl_xor_sync(0xFFFFFFFFu, acc[r], 2);
        acc[r] += __shfl_xor_sync(0xFFFFFFFFu, acc[r], 1);
    }

    bool finisher = active && ks == 0 && l == 0;
    if constexpr (CLUSTERK) {
        // Every CTA of the cluster has started (the arrive at entry) before anyone writes into the leader's
        // shared memory; the second barrier orders those stores before the leader's reads.
        asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
        if (active && l == 0) {
            if (krank == 0) {
                s_part[sub] = acc[0];
            } else {
                uint32_t remote;
                asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_addr(&s_part[krank * a.units_per_cta + sub])), "r"(0u));
                asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(acc[0]) : "memory");
            }
        }
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        finisher = finisher && krank == 0;
        if (finisher) {
            float t = 0.0f;
            for (int k = 0; k < a.ksplit; ++k) t += s_part[k * a.units_per_cta + sub];
            acc[0] = t;
        }
    } else if (a.ksplit > 1) {
        if (l == 0 && ks < a.ksplit) {
#pragma unroll
            for (int r = 0; r < R; ++r) s_part[(ks * a.units_per_cta + u_local) * R + r] = acc[r];
        }
        __syncthreads();
        if (ks == 0 && l == 0) {
#pragma unroll
            for (int r = 0; r < R; ++r) {
                float t = 0.0f;
                for (int k = 0; k < a.ksplit; ++k) t += s_part[(k * a.units_per_cta + u_local) * R + r];
                acc[r] = t;
            }
        }
    }

    if (finisher) {
        float y;
        if constexpr (MODE == kSwiglu) {
            const float gate = acc[0];
            y = (gate / (1.0f + expf(-gate))) * acc[R - 1];
        } else {
            y = acc[0];
            if constexpr (MODE == kPlain) {
                if (a.residual != nullptr) y += __half2float(res_pre);
            }
        }
        const __half yh = __float2half_rn(y);
        obase[first + u_local] = yh;
        if constexpr (MODE == kPlain) {
            for (int p = 0; p < a.num_peers; ++p) a.peer_out[p][unit] = yh;
        }
    }
}

}  // namespace

namespace {

// Streaming form for very tall matrices (lm_head): a persistent grid, each CTA walks row blocks of 32 with
// the weights of the NEXT block already in flight while the current one is reduced, and the lane's share
// of the quantised activation lives in registers for the whole launch (a lane always meets the same
// 16-byte chunks l, l+8, ... of every row).  PLAIN mode, 16-byte aligned weights, K <= 256 * STEPS.
// EPI: 0 plain epilogue; 1 token selection (SAMPLE); 2 signalled row-split output (SIGNAL): the slice goes into
// half (step & 1) of this GPU's and every peer's gathered vector with 16-byte stores, and the launch's last
// CTA publishes the step number to every GPU's flag array, so that no barrier kernel has to follow.
template <int XIN, int STEPS, bool SWIGLU, int EPI = 0>
__global__ void __launch_bounds__(kMaxThreads, 2) gemv_w4_stream_kernel(const GemvArgs a, const int num_blocks) {
    constexpr bool SAMPLE = EPI == 1, SIGNAL = EPI == 2;
    static_assert(!(SWIGLU && EPI != 0), "token selection and signalled outputs follow a plain projection");
    extern __shared__ __align__(16) uint8_t smem[];
    const int K = a.K;
    int8_t* s_q8 = reinterpret_cast<int8_t*>(smem);
    int32_t* s_seed = reinterpret_cast<int32_t*>(smem + K);
    float* s_scale = reinterpret_cast<float*>(smem + K + (K / kChunk) * 4);

    const int tid = threadIdx.x, sub = tid >> 3, l = tid & 7;
    const int words = K / 8, groups = K / kGroup, steps = K / kStepElems;
    const int N = SWIGLU ? 2 * a.units : a.units;   // weight rows (SwiGLU: gate/up pairs = adjacent sub-warps)

    uint4 w0[STEPS], w1[STEPS];
    uint16_t sb0[STEPS], sb1[STEPS];
    auto issue = [&](uint4 (&w)[STEPS], uint16_t (&sb)[STEPS], int blk) {
        const int row = blk * kMaxSubwarps + sub;
        const bool on_row = row < N;
        const uint32_t* wrow = a.qweight[0] + static_cast<size_t>(on_row ? row : 0) * words;
        const __half* srow = a.scales[0] + static_cast<size_t>(on_row ? row : 0) * groups;
#pragma unroll
        for (int i = 0; i < STEPS; ++i) {
            if (on_row && i < steps) {
                w[i] = ld_weights_16(wrow + (i * kSubwarp + l) * 4);
                sb[i] = ld_scale_bits(srow + 2 * i + (l >> 2));
            } else {
                w[i] = make_uint4(0, 0, 0, 0);
                sb[i] = 0;
            }
        }
    };

    int blk = blockIdx.x;
    if (blk < num_blocks) issue(w0, sb0, blk);
    pdl_release_dependents();
    pdl_wait_prior_grids();

    // Token selection in the epilogue (PLAIN only): the fp16-rounded outputs of eight row blocks are parked in
    // shared memory and then scored by all 256 threads at once (the Gumbel draw costs ~150 instructions per
    // row; left to the one lane per row that holds the sum it would double the kernel's instruction count).
    constexpr bool sampling = SAMPLE;
    __shared__ float s_scores[SAMPLE ? 2 : 1][SAMPLE ? kMaxThreads : 1];
    [[maybe_unused]] float temperature = 0.0f, best = kSampleFloor;
    [[maybe_unused]] uint64_t rng_seed = 0;
    [[maybe_unused]] uint32_t seq_pos = 0;
    [[maybe_unused]] int32_t best_idx = 0;
    [[maybe_unused]] int it = 0, buf = 0;
    [[maybe_unused]] uint32_t sample_step = 0;
    [[maybe_unused]] __shared__ __align__(16) __half s_blk[SIGNAL ? 2 : 1][kMaxSubwarps];
    if constexpr (SIGNAL) sample_step = *reinterpret_cast<volatile uint32_t*>(a.sample_step_word) + 1u;
    if constexpr (SAMPLE) {
        if (a.sample_step_word != nullptr) sample_step = *reinterpret_cast<volatile uint32_t*>(a.sample_step_word) + 1u;
        if (a.sample_control != nullptr) {
            const SampleControl* c = static_cast<const SampleControl*>(a.sample_control);
            temperature = c->temperature;
            rng_seed = c->rng_seed;
            seq_pos = static_cast<uint32_t>(c->seq_pos);
        }
    }
    if constexpr (XIN == kXFp16Norm) stage_x_from_fp16_rmsnorm(a.x_fp16, a.gamma, K, kRmsEps, s_q8, s_seed, s_scale);
    else if constexpr (XIN == kXFp16) stage_x_from_fp16(a.x_fp16, K, s_q8, s_seed, s_scale);
    else stage_x_from_q8_1(a.q8, a.xscale, a.sum8, K, a.vec_ok != 0, s_q8, s_seed, s_scale);
    __syncthreads();

    uint4 xa[STEPS], xb[STEPS];
    int32_t seed[STEPS];
    float xs[STEPS];
#pragma unroll
    for (int i = 0; i < STEPS; ++i) {
        const int c = (i < steps ? i : 0) * kSubwarp + l;
        xa[i] = reinterpret_cast<const uint4*>(s_q8)[q8_slot(c, 0)];
        xb[i] = reinterpret_cast<const uint4*>(s_q8)[q8_slot(c, 1)];
        seed[i] = s_seed[c];
        xs[i] = i < steps ? s_scale[c >> 2] : 0.0f;     // a zero factor switches an unused slot off
    }

    for (; blk < num_blocks; blk += gridDim.x) {
        const int nxt = blk + gridDim.x;
        if (nxt < num_blocks) issue(w1, sb1, nxt);
        float acc = 0.0f;
#pragma unroll
        for (int i = 0; i < STEPS; ++i) {
            const int32_t d = chunk_dot(w0[i], xa[i], xb[i], seed[i]);
            acc = fmaf(static_cast<float>(d), __half2float(__ushort_as_half(sb0[i])) * xs[i], acc);
        }
        acc += __shfl_xor_sync(0xFFFFFFFFu, acc, 4);
        acc += __shfl_xor_sync(0xFFFFFFFFu, acc, 2);
        acc += __shfl_xor_sync(0xFFFFFFFFu, acc, 1);
        const int row = blk * kMaxSubwarps + sub;
        if constexpr (SWIGLU) {
            const float up = __shfl_xor_sync(0xFFFFFFFFu, acc, 8);   // the odd row's sum sits 8 lanes over
            if (l == 0 && (sub & 1) == 0 && row < N)
                a.out[0][row >> 1] = __float2half_rn((acc / (1.0f + expf(-acc))) * up);
        } else {
            if constexpr (SIGNAL) {
                // the block's 32 outputs are collected in shared memory and leave as 16-byte stores: lane = (destination,
                // segment of 8 rows); one barrier per block, the two buffers used in turn
                if (l == 0) s_blk[it & 1][sub] = __float2half_rn(acc);
                __syncthreads();
                if (tid < 4 * (1 + a.num_peers)) {
                    const int d = tid >> 2, seg = tid & 3;
                    __half* dst = (d == 0 ? a.out[0] : a.peer_out[d - 1]) +
                                  static_cast<size_t>(sample_step & 1u) * a.sample_half_stride + blk * kMaxSubwarps + seg * 8;
                    const int r0 = blk * kMaxSubwarps + seg * 8;
                    if (r0 + 8 <= N && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
                        *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(&s_blk[it & 1][seg * 8]);
                    } else {
                        for (int j = 0; j < 8 && r0 + j < N; ++j) dst[j] = s_blk[it & 1][seg * 8 + j];
                    }
                }
                ++it;
            } else if (l == 0 && row < N) {
                float y = acc;
                if (a.residual != nullptr) y += __half2float(a.residual[row]);
                const __half yh = __float2half_rn(y);
                if (a.out[0] != nullptr) a.out[0][row] = yh;
                for (int p = 0; p < a.num_peers; ++p) a.peer_out[p][row] = yh;
                if constexpr (sampling) s_scores[buf][(it & 7) * kMaxSubwarps + sub] = __half2float(yh);
            }
            if constexpr (sampling) {
                if ((it & 7) == 7 || nxt >= num_blocks) {      // uniform over the CTA
                    __syncthreads();
                    const int it_j = (it & ~7) + (tid >> 5);   // thread = (iteration of the group, row of the block)
                    const int row_j = (static_cast<int>(blockIdx.x) + it_j * static_cast<int>(gridDim.x)) * kMaxSubwarps + (tid & 31);
                    if (it_j <= it && row_j < N) {
                        const int32_t index = row_j + a.sample_index_offset;
                        sample_take(best, best_idx,
                                    sample_score(s_scores[buf][tid], static_cast<uint32_t>(index), temperature, rng_seed, seq_pos),
                                    index);
                    }
                    buf ^= 1;   // the next eight blocks park in the other half: one barrier per group is enough
                }
                ++it;
            }
        }
#pragma unroll
        for (int i = 0; i < STEPS; ++i) { w0[i] = w1[i]; sb0[i] = sb1[i]; }
    }
    if constexpr (SIGNAL) {
        // "last block" pattern: the storing lanes fence, the CTA counts itself; the CTA that completes the count
        // fences at system scope (cumulative over what it observed through the counter) and publishes the step
        // number with independent relaxed stores, which the gathering kernel of every GPU takes with acquire loads
        if (tid < 32) __threadfence();
        __syncthreads();
        if (tid == 0 && atomicInc(a.sample_done_counter, gridDim.x - 1u) == gridDim.x - 1u) {
            __threadfence_system();
            *reinterpret_cast<volatile uint32_t*>(a.sample_step_word) = sample_step;
            asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(a.sample_flag_local), "r"(sample_step) : "memory");
            for (int p = 0; p < a.num_peers; ++p)
                asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(a.sample_peer_flag[p]), "r"(sample_step) : "memory");
        }
    }
    if constexpr (SAMPLE) {
        __shared__ float s_v[32];
        __shared__ int32_t s_i[32];
        sample_block_reduce(best, best_idx, s_v, s_i);
        if (tid == 0) {
            const size_t slot = static_cast<size_t>(sample_step & 1u) * a.sample_half_stride + blockIdx.x;
            a.sample_val[slot] = best;
            a.sample_idx[slot] = best_idx;
            for (int p = 0; p < a.sample_num_peers; ++p) {   // plain stores over NVLink
                a.sample_peer_val[p][slot] = best;
                a.sample_peer_idx[p][slot] = best_idx;
            }
            if (a.sample_step_word != nullptr) {
                // "last block" pattern: stores, fence, count; the CTA that completes the count fences at system
                // scope (cumulative over what it observed through the counter) and publishes the step number,
                // which a reader on another GPU then takes with an acquire load
                __threadfence();
                if (atomicInc(a.sample_done_counter, gridDim.x - 1u) == gridDim.x - 1u) {
                    __threadfence_system();   // ONE system-scope fence, then independent flag stores: a release
                                              // store per peer would wait for the previous peer's round trip
                    *reinterpret_cast<volatile uint32_t*>(a.sample_step_word) = sample_step;
                    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(a.sample_flag_local), "r"(sample_step) : "memory");
                    for (int p = 0; p < a.sample_num_peers; ++p)
                        asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(a.sample_peer_flag[p]), "r"(sample_step) : "memory");
                }
            }
        }
        if (a.sample_finish_inline) {
            // Single launch: the CTA that arrives last (stores, fence, wrapping counter) reduces the candidates of
            // all CTAs -- every other CTA is through by then, so the control block may be advanced here too.
            __shared__ int s_last;
            if (tid == 0) {
                __threadfence();
                s_last = atomicInc(a.sample_done_counter, gridDim.x - 1u) == gridDim.x - 1u ? 1 : 0;
                __threadfence();
            }
            __syncthreads();
            if (s_last) {
                best = kSampleFloor;
                best_idx = 0x7FFFFFFF;
                for (int i = tid; i < static_cast<int>(gridDim.x); i += blockDim.x)
                    sample_take(best, best_idx, __ldcg(a.sample_val + i), __ldcg(a.sample_idx + i));
                __syncthreads();   // s_v / s_i are reused
                sample_block_reduce(best, best_idx, s_v, s_i);
                if (tid == 0) {
                    if (best_idx == 0x7FFFFFFF) best_idx = 0;
                    SampleControl* c = static_cast<SampleControl*>(a.sample_control_rw);
                    if (c != nullptr) {
                        c->token_id = best_idx;
                        c->seq_pos += 1;
                        c->rng_seed += 0x9E3779B97F4A7C15ull;
                    }
                    if (a.sample_token_out != nullptr) *a.sample_token_out = best_idx;
                }
            }
        }
    }
}

// Streaming form for tall matrices with a LONG K (more than 2048 elements): the same persistent walk over row
// blocks of 32, but a row's K range is taken in slices of 2048 (8 steps of 256), the next slice's -- or the next
// row block's -- weight words already in flight while the current slice is multiplied, and the quantised
// activation read from shared memory (a lane's share of an 8192-element vector would not fit registers).
// A row's chunks are accumulated in K order by the same lane as in gemv_w4_kernel without a K split, so the
// two agree bit for bit.  PLAIN mode, 16-byte aligned weights.
template <int XIN, bool FULL>     // FULL: K is a multiple of 2048, every slice has all 8 steps (no guards in the loops)
__global__ void __launch_bounds__(kMaxThreads, 2) gemv_w4_stream_longk_kernel(const GemvArgs a, const int num_blocks) {
    constexpr int STEPS = 8;
    extern __shared__ __align__(16) uint8_t smem[];
    const int K = a.K;
    int8_t* s_q8 = reinterpret_cast<int8_t*>(smem);
    int32_t* s_seed = reinterpret_cast<int32_t*>(smem + K);
    float* s_scale = reinterpret_cast<float*>(smem + K + (K / kChunk) * 4);
    const int tid = threadIdx.x, sub = tid >> 3, l = tid & 7;
    const int words = K / 8, groups = K / kGroup, steps = K / kStepElems;
    const int nslices = (steps + STEPS - 1) / STEPS;
    const int N = a.units;

    // the unit after (blk, sl) in this CTA's walk: the row block's next slice, else the CTA's next row block
    auto next_unit = [&](int& blk, int& sl) {
        if (++sl == nslices) { sl = 0; blk += gridDim.x; }
    };
    auto issue = [&](uint4 (&w)[STEPS], uint16_t (&sb)[STEPS], int blk, int sl) {
        const int row = min(blk * kMaxSubwarps + sub, N - 1);      // rows past the end re-read the last row; never stored
        const uint32_t* wp = a.qweight[0] + static_cast<size_t>(row) * words + (sl * STEPS * kSubwarp + l) * 4;
        const __half* sp = a.scales[0] + static_cast<size_t>(row) * groups + 2 * sl * STEPS + (l >> 2);
#pragma unroll
        for (int i = 0; i < STEPS; ++i) {
            if (FULL || sl * STEPS + i < steps) {
                w[i] = ld_weights_16(wp + i * (kSubwarp * 4));
                sb[i] = ld_scale_bits(sp + 2 * i);
            } else {
                w[i] = make_uint4(0, 0, 0, 0);
                sb[i] = 0;       // a zero scale switches an unused slot off
            }
        }
    };
    float acc = 0.0f;
    // one unit: 8 chunks of this lane against the staged activation; at a row's last slice reduce and store
    auto consume = [&](const uint4 (&w)[STEPS], const uint16_t (&sb)[STEPS], int blk, int sl) {
        const uint4* xq = reinterpret_cast<const uint4*>(s_q8) + q8_slot(sl * STEPS * kSubwarp + l, 0);   // chunk-interleaved
        const int32_t* xseed = s_seed + sl * STEPS * kSubwarp + l;
        const float* xscale = s_scale + 2 * sl * STEPS + (l >> 2);
#pragma unroll
        for (int i = 0; i < STEPS; ++i) {
            if (FULL || sl * STEPS + i < steps) {
                const uint4 xa = xq[16 * i];        // chunk + 8 i: the next block of eight chunks
                const uint4 xb = xq[16 * i + 8];
                const int32_t d = chunk_dot(w[i], xa, xb, xseed[i * kSubwarp]);
                acc = fmaf(static_cast<float>(d), __half2float(__ushort_as_half(sb[i])) * xscale[2 * i], acc);
            }
        }
        if (sl == nslices - 1) {
            acc += __shfl_xor_sync(0xFFFFFFFFu, acc, 4);
            acc += __shfl_xor_sync(0xFFFFFFFFu, acc, 2);
            acc += __shfl_xor_sync(0xFFFFFFFFu, acc, 1);
            const int row = blk * kMaxSubwarps + sub;
            if (l == 0 && row < N) {
                float y = acc;
                if (a.residual != nullptr) y += __half2float(a.residual[row]);
                const __half yh = __float2half_rn(y);
                a.out[0][row] = yh;
                for (int p = 0; p < a.num_peers; ++p) a.peer_out[p][row] = yh;
            }
            acc = 0.0f;
        }
    };

    uint4 w0[STEPS], w1[STEPS];
    uint16_t sb0[STEPS], sb1[STEPS];
    int blk = blockIdx.x, sl = 0;
    if (blk < num_blocks) issue(w0, sb0, blk, 0);
    pdl_release_dependents();
    pdl_wait_prior_grids();
    if constexpr (XIN == kXFp16Norm) stage_x_from_fp16_rmsnorm(a.x_fp16, a.gamma, K, kRmsEps, s_q8, s_seed, s_scale);
    else if constexpr (XIN == kXFp16) stage_x_from_fp16(a.x_fp16, K, s_q8, s_seed, s_scale);
    else stage_x_from_q8_1(a.q8, a.xscale, a.sum8, K, a.vec_ok != 0, s_q8, s_seed, s_scale);
    __syncthreads();
    // two register sets used in turn: the next unit's words are in flight while this one is multiplied
    while (blk < num_blocks) {
        int nblk = blk, nsl = sl;
        next_unit(nblk, nsl);
        if (nblk < num_blocks) issue(w1, sb1, nblk, nsl);
        consume(w0, sb0, blk, sl);
        if (nblk >= num_blocks) break;
        blk = nblk; sl = nsl;
        next_unit(nblk, nsl);
        if (nblk < num_blocks) issue(w0, sb0, nblk, nsl);
        consume(w1, sb1, blk, sl);
        blk = nblk; sl = nsl;
    }
}

// Diagnostic: the per-group int32 dots, through the same staging and chunk_dot as above.
__global__ void __launch_bounds__(kMaxThreads) gemv_group_dots_kernel(const uint32_t* __restrict__ qweight,
                                                                       const int8_t* __restrict__ q8,
                                                                       const int32_t* __restrict__ sum8,
                                                                       int32_t* __restrict__ out, int N, int K,
                                                                       int vec_ok, int aligned16) {
    extern __shared__ __align__(16) uint8_t smem[];
    int8_t* s_q8 = reinterpret_cast<int8_t*>(smem);
    int32_t* s_seed = reinterpret_cast<int32_t*>(smem + K);
    // only the integer part is needed: q8 bytes and the per-chunk seeds
    {
        const int tid = threadIdx.x, nthr = blockDim.x;
        if (vec_ok) {
            for (int i = tid; i < K / 16; i += nthr)
                reinterpret_cast<uint4*>(s_q8)[q8_slot(i >> 1, i & 1)] = reinterpret_cast<const uint4*>(q8)[i];
            for (int c = tid; c < K / kChunk; c += nthr) {
                const int4 v = reinterpret_cast<const int4*>(sum8)[c];
                s_seed[c] = v.x + v.y + v.z + v.w;
            }
        } else {
            for (int i = tid; i < K; i += nthr) s_q8[q8_byte(i)] = q8[i];
            for (int c = tid; c < K / kChunk; c += nthr)
                s_seed[c] = sum8[4 * c] + sum8[4 * c + 1] + sum8[4 * c + 2] + sum8[4 * c + 3];
        }
    }
    __syncthreads();
    const int sub = threadIdx.x >> 3, l = threadIdx.x & 7;
    const int row = blockIdx.x * kMaxSubwarps + sub;
    const bool active = row < N;
    const uint32_t* wrow = qweight + static_cast<size_t>(active ? row : 0) * (K / 8);
    const int groups = K / kGroup;
    for (int s = 0; s < K / kStepElems; ++s) {
        const int c = s * kSubwarp + l;
        int32_t d = 0;
        if (active) {
            const uint4 w = aligned16 ? ld_weights_16(wrow + c * 4) : ld_weights_4x4(wrow + c * 4);
            const uint4 xa = reinterpret_cast<const uint4*>(s_q8)[q8_slot(c, 0)];
            const uint4 xb = reinterpret_cast<const uint4*>(s_q8)[q8_slot(c, 1)];
            d = chunk_dot(w, xa, xb, s_seed[c]);
        }
        d += __shfl_xor_sync(0xFFFFFFFFu, d, 1);
        d += __shfl_xor_sync(0xFFFFFFFFu, d, 2);
        if (active && (l & 3) == 0) out[static_cast<size_t>(row) * groups + 2 * s + (l >> 2)] = d;
    }
}

// ---- host side -------------------------------------------------------------------

struct Plan {
    int units_per_cta, ksplit, steps_per_split, U;
};

// Warps of one kernel variant that fit an SM at once.  Registers are handed out per scheduler partition
// (16384 each, whole warps), so a variant capped at 96 registers holds 5 warps per partition, one at 128
// holds 4, and the 4-load forms (<= 80 registers) hold 6.
int resident_warps_per_sm(GemvMode mode, int U) {
    if (mode == kSwiglu) return 16;
    return U == 8 ? 20 : 24;
}

// Picks the CTA shape.  units: output rows (or pairs).  Goals, in order: about 1.25 CTAs per SM when the matrix
// allows it, and no more (see below); all 32 sub-warps of a CTA busy; at most 8 loads per lane per batch so one
// batch covers a lane's whole K slice for the model's shapes; and the whole grid resident at once (a second wave
// of CTAs would start its weight loads only after the wait).
Plan make_plan(GemvMode mode, int units, int K, int sm_count) {
    const int steps = K / kStepElems;
    // Fewest CTAs that still give every SM work (1.25 per SM; 1.3 where the K slices would otherwise not fit one batch
    // of 8 loads per lane):
    // what a grid leaves free on an SM is where the NEXT launch's CTAs become resident and fetch their weights
    // while this one still runs (O projection 1536 x 1536: 192 CTAs instead of 384 let 53 % instead of 24 % of the
    // following gate_up launch's CTAs start early, 5 % of the whole 28-layer pass).
    auto depth_for = [&](int u) {
        const int c = std::min(std::max(1, kMaxSubwarps / u), steps);
        return (steps + c - 1) / c;
    };
    auto upc_for = [&](int target_ctas) {
        int u = 32;
        while (u > 4 && (units + u - 1) / u < target_ctas) u /= 2;
        return u;
    };
    int upc = upc_for((sm_count * 5) / 4);
    if (depth_for(upc) > 8) upc = upc_for((sm_count * 13 + 9) / 10);
    int cap = std::max(1, kMaxSubwarps / upc);   // most K slices the CTA can hold
    cap = std::min(cap, steps);
    int per = (steps + cap - 1) / cap;           // steps per slice if all slices were used
    int ksplit = (steps + per - 1) / per;        // fewest slices that reach that depth
    auto pick_u = [&](int depth) { return depth <= 4 ? 4 : 8; };
    const int grid = (units + upc - 1) / upc;
    while (ksplit > 1) {
        const int warps = (upc * ksplit * kSubwarp + 31) / 32;
        const int ctas_per_sm = resident_warps_per_sm(mode, pick_u(per)) / warps;
        if (grid <= ctas_per_sm * sm_count || per >= 8) break;
        per = (steps + (ksplit - 1) - 1) / (ksplit - 1);   // one slice fewer, deeper slices
        ksplit = (steps + per - 1) / per;
    }
    Plan p;
    p.units_per_cta = upc;
    p.ksplit = ksplit;
    p.steps_per_split = per;
    p.U = pick_u(per);
    return p;
}

template <int MODE, int U, int XIN>
cudaError_t launch_aligned(const GemvArgs& a, bool aligned16, dim3 grid, dim3 block, size_t smem,
                           cudaStream_t stream) {
    const dim3 cluster_x(a.q8_out != nullptr ? 4 : 1, 1, 1);   // Q8_1 epilogue: four CTAs = one group of 128 outputs
    if (aligned16)
        return launch_kernel_cluster(gemv_w4_kernel<MODE, U, XIN, true>, grid, block, smem, stream, pdl_enabled(),
                                     cluster_x, a);
    return launch_kernel_cluster(gemv_w4_kernel<MODE, U, XIN, false>, grid, block, smem, stream, pdl_enabled(),
                                 cluster_x, a);
}
template <int MODE, int U>
cudaError_t launch_input(const GemvArgs& a, bool aligned16, dim3 grid, dim3 block, size_t smem, cudaStream_t stream) {
    if constexpr (MODE == kPlain) {
        if (a.x_f32 != nullptr) return launch_aligned<MODE, U, kXF32Heads>(a, aligned16, grid, block, smem, stream);
    }
    if (a.x_fp16 != nullptr) {
        if (a.gamma != nullptr) return launch_aligned<MODE, U, kXFp16Norm>(a, aligned16, grid, block, smem, stream);
        if constexpr (MODE == kPlain) {
            if (a.amax_in != nullptr && reinterpret_cast<uintptr_t>(a.x_fp16) % 16 == 0) {
                const size_t smem_amax = amax_stage_offset(a.K, a.ksplit * a.units_per_cta) + amax_stage_bytes(a.K);
                if (smem_amax <= 200 * 1024)
                    return launch_aligned<MODE, U, kXFp16Amax>(a, aligned16, grid, block, smem_amax, stream);
            }
        }
        return launch_aligned<MODE, U, kXFp16>(a, aligned16, grid, block, smem, stream);
    }
    return launch_aligned<MODE, U, kXQ8>(a, aligned16, grid, block, smem, stream);
}
template <int MODE>
cudaError_t launch_mode(const GemvArgs& a, int U, bool aligned16, dim3 grid, dim3 block, size_t smem,
                        cudaStream_t stream) {
    if (U == 4) return launch_input<MODE, 4>(a, aligned16, grid, block, smem, stream);
    return launch_input<MODE, 8>(a, aligned16, grid, block, smem, stream);
}

// ---- bulk-copy form: instantiations, attributes, launch ----
template <typename F>
cudaError_t prepare_bulk(F* f) {
    cudaError_t e = cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    // the largest shared-memory carve-out, the same for every kernel of a decode pass: CTAs of two kernels
    // share an SM only if they agree on it
    if (e == cudaSuccess) e = cudaFuncSetAttribute(f, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    return e;
}
template <int MODE>
cudaError_t prepare_bulk_mode() {
    cudaError_t e = prepare_bulk(gemv_w4_bulk_kernel<MODE, kXQ8, false>);
    if (e == cudaSuccess) e = prepare_bulk(gemv_w4_bulk_kernel<MODE, kXFp16, false>);
    if (e == cudaSuccess) e = prepare_bulk(gemv_w4_bulk_kernel<MODE, kXFp16Norm, false>);
    if constexpr (MODE == kPlain) {
        if (e == cudaSuccess) e = prepare_bulk(gemv_w4_bulk_kernel<kPlain, kXF32Heads, false>);
        if (e == cudaSuccess) e = prepare_bulk(gemv_w4_bulk_kernel<kPlain, kXQ8, true>);
        if (e == cudaSuccess) e = prepare_bulk(gemv_w4_bulk_kernel<kPlain, kXFp16, true>);
    }
    return e;
}
template <int MODE>
cudaError_t launch_bulk(const GemvArgs& a, bool cluster_k, dim3 grid, dim3 block, size_t smem, cudaStream_t stream) {
    const bool pdl = pdl_enabled();
    if constexpr (MODE == kPlain) {
        if (cluster_k) {
            const dim3 cl(static_cast<unsigned>(a.ksplit), 1, 1);
            if (a.x_fp16 != nullptr)
                return launch_kernel_cluster(gemv_w4_bulk_kernel<kPlain, kXFp16, true>, grid, block, smem, stream, pdl, cl, a);
            return launch_kernel_cluster(gemv_w4_bulk_kernel<kPlain, kXQ8, true>, grid, block, smem, stream, pdl, cl, a);
        }
        if (a.x_f32 != nullptr) return launch_kernel(gemv_w4_bulk_kernel<kPlain, kXF32Heads, false>, grid, block, smem, stream, pdl, a);
    }
    if (a.x_fp16 != nullptr) {
        if (a.gamma != nullptr) return launch_kernel(gemv_w4_bulk_kernel<MODE, kXFp16Norm, false>, grid, block, smem, stream, pdl, a);
        return launch_kernel(gemv_w4_bulk_kernel<MODE, kXFp16, false>, grid, block, smem, stream, pdl, a);
    }
    return launch_kernel(gemv_w4_bulk_kernel<MODE, kXQ8, false>, grid, block, smem, stream, pdl, a);
}

template <typename F>
cudaError_t raise_smem(F* f) {
    return cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
}
template <int MODE, int U>
cudaError_t raise_smem_mode() {
    cudaError_t e = raise_smem(gemv_w4_kernel<MODE, U, kXQ8, true>);
    if (e == cudaSuccess) e = raise_smem(gemv_w4_kernel<MODE, U, kXQ8, false>);
    if (e == cudaSuccess) e = raise_smem(gemv_w4_kernel<MODE, U, kXFp16, true>);
    if (e == cudaSuccess) e = raise_smem(gemv_w4_kernel<MODE, U, kXFp16, false>);
    if (e == cudaSuccess) e = raise_smem(gemv_w4_kernel<MODE, U, kXFp16Norm, true>);
    if (e == cudaSuccess) e = raise_smem(gemv_w4_kernel<MODE, U, kXFp16Norm, false>);
    if constexpr (MODE == kPlain) {
        if (e == cudaSuccess) e = raise_smem(gemv_w4_kernel<MODE, U, kXF32Heads, true>);
        if (e == cudaSuccess) e = raise_smem(gemv_w4_kernel<MODE, U, kXF32Heads, false>);
        if (e == cudaSuccess) e = raise_smem(gemv_w4_kernel<MODE, U, kXFp16Amax, true>);
        if (e == cudaSuccess) e = raise_smem(gemv_w4_kernel<MODE, U, kXFp16Amax, false>);
    }
    return e;
}

}  // namespace

int gemv_set_attributes() {
    cudaError_t e = raise_smem_mode<kPlain, 4>();
    if (e == cudaSuccess) e = raise_smem_mode<kPlain, 8>();
    if (e == cudaSuccess) e = raise_smem_mode<kQkv, 4>();
    if (e == cudaSuccess) e = raise_smem_mode<kQkv, 8>();
    if (e == cudaSuccess) e = raise_smem_mode<kSwiglu, 4>();
    if (e == cudaSuccess) e = raise_smem_mode<kSwiglu, 8>();
    if (e == cudaSuccess) e = raise_smem(gemv_group_dots_kernel);
    if (e == cudaSuccess) e = raise_smem(gemv_w4_stream_longk_kernel<kXQ8, true>);
    if (e == cudaSuccess) e = raise_smem(gemv_w4_stream_longk_kernel<kXQ8, false>);
    if (e == cudaSuccess) e = raise_smem(gemv_w4_stream_longk_kernel<kXFp16, true>);
    if (e == cudaSuccess) e = raise_smem(gemv_w4_stream_longk_kernel<kXFp16, false>);
    if (e == cudaSuccess) e = raise_smem(gemv_w4_stream_longk_kernel<kXFp16Norm, true>);
    if (e == cudaSuccess) e = raise_smem(gemv_w4_stream_longk_kernel<kXFp16Norm, false>);
    if (e == cudaSuccess) e = prepare_bulk_mode<kPlain>();
    if (e == cudaSuccess) e = prepare_bulk_mode<kQkv>();
    if (e == cudaSuccess) e = prepare_bulk_mode<kSwiglu>();
    return static_cast<int>(e);
}

int gemv_copy_timeouts(unsigned int* out) {
    return static_cast<int>(cudaMemcpyFromSymbol(out, g_gemv_copy_timeouts, sizeof(unsigned int)));
}

int gemv_sample_slots(int out_features) {
    const DeviceInfo* dev = nullptr;
    if (int st = ensure_device_ready(&dev)) return st;
    const int num_blocks = (out_features + kMaxSubwarps - 1) / kMaxSubwarps;
    return std::min(num_blocks, 2 * dev->sm_count);   // the streaming form's grid
}

int gemv_launch(GemvMode mode, GemvArgs a, cudaStream_t stream) {
    const DeviceInfo* dev = nullptr;
    if (int st = ensure_device_ready(&dev)) return st;

    Plan p = make_plan(mode, a.units, a.K, dev->sm_count);
    const bool q8_epilogue = a.q8_out != nullptr || a.xscale_out != nullptr || a.sum8_out != nullptr;
    if (q8_epilogue) {
        if (mode != kSwiglu || !a.q8_out || !a.xscale_out || !a.sum8_out) return W4A16_ERR_INVALID_ARG;
        if (a.units % kGroup != 0) return W4A16_ERR_SHAPE;
        // the epilogue's layout: 32 outputs per CTA, the whole of K in each sub-warp
        p.units_per_cta = kMaxSubwarps;
        p.ksplit = 1;
        p.steps_per_split = a.K / kStepElems;
        p.U = 8;
    }
    // Hand-offs of a decode pass exist in the register form only (the other forms ignore amax_in / sumsq_in, which
    // merely save work, but would drop what a later launch relies on).
    const bool handoff = a.sumsq_out != nullptr || a.amax_out != nullptr || a.clear_count > 0;
    if (a.clear_count < 0 || a.clear_count > 128 || (a.clear_count > 0 && !a.clear_words)) return W4A16_ERR_INVALID_ARG;
    if ((a.amax_out && (mode != kSwiglu || p.units_per_cta % 4)) || (a.sumsq_out && mode != kPlain)) return W4A16_ERR_SHAPE;
    if (mode == kQkv) {
        // a CTA's rows must come from one tensor
        while (p.units_per_cta > 1 && (a.rows[0] % p.units_per_cta || a.rows[1] % p.units_per_cta)) p.units_per_cta /= 2;
    }
    a.units_per_cta = p.units_per_cta;
    a.ksplit = p.ksplit;
    a.steps_per_split = p.steps_per_split;

    bool aligned16 = true;
    const int ntens = (mode == kQkv) ? 3 : 1;
    for (int t = 0; t < ntens; ++t) aligned16 = aligned16 && (reinterpret_cast<uintptr_t>(a.qweight[t]) % 16 == 0);
    a.vec_ok = (a.x_fp16 == nullptr) && (a.x_f32 == nullptr) && (reinterpret_cast<uintptr_t>(a.q8) % 16 == 0) &&
               (reinterpret_cast<uintptr_t>(a.sum8) % 16 == 0);

    const int R = (mode == kSwiglu) ? 2 : 1;
    const int threads = a.units_per_cta * a.ksplit * kSubwarp;
    const int grid = (a.units + a.units_per_cta - 1) / a.units_per_cta;
    const size_t smem = staged_x_bytes(a.K) + static_cast<size_t>(a.ksplit) * a.units_per_cta * R * sizeof(float);
    if (smem > 200 * 1024) return W4A16_ERR_TOO_LARGE;
    // fp16 staging quantises with whole warps
    const int block = (threads + 31) / 32 * 32;

    cudaError_t e;
    // very tall PLAIN matrices: persistent streaming kernel (two CTAs per SM, >= 8 row blocks each)
    const int steps = a.K / kStepElems;
    const int weight_rows = mode == kSwiglu ? 2 * a.units : a.units;
    const int num_blocks = (weight_rows + kMaxSubwarps - 1) / kMaxSubwarps;
    constexpr int kStreamMinBlocksPerSm = 16;   // row blocks per SM from which the persistent streaming form pays
    const bool tall = num_blocks >= kStreamMinBlocksPerSm * dev->sm_count;
    const bool sampling = a.sample_val != nullptr || a.sample_idx != nullptr;
    // signalled row-split output (no sampling): step word + flags given, the streaming kernel whatever the height
    const bool signalled = !sampling && a.sample_step_word != nullptr;
    if (signalled && (mode != kPlain || !aligned16 || steps > 8 || a.residual != nullptr || !a.sample_done_counter ||
                      !a.sample_flag_local || !a.out[0]))
        return W4A16_ERR_SHAPE;
    if (sampling && (mode != kPlain || !a.sample_val || !a.sample_idx || !aligned16 || steps > 8)) return W4A16_ERR_SHAPE;
    // tall plain matrices with a long K: the streaming form that takes K in slices of 2048
    if (mode == kPlain && !q8_epilogue && !sampling && !handoff && aligned16 && steps > 8 && a.x_f32 == nullptr &&
        static_cast<long long>(num_blocks) * ((steps + 7) / 8) >= 8LL * 2 * dev->sm_count &&
        staged_x_bytes(a.K) <= 160 * 1024 && option(W4A16_OPT_GEMV_FORM) != 2) {
        const dim3 sgrid(std::min(num_blocks, 2 * dev->sm_count)), sblock(kMaxThreads);
        const size_t ssmem = staged_x_bytes(a.K);
        const bool pdl = pdl_enabled();
#define W4_LONGK(XINV) (steps % 8 == 0 ? launch_kernel(gemv_w4_stream_longk_kernel<XINV, true>, sgrid, sblock, ssmem, stream, pdl, a, num_blocks) \
                                       : launch_kernel(gemv_w4_stream_longk_kernel<XINV, false>, sgrid, sblock, ssmem, stream, pdl, a, num_blocks))
        if (a.x_fp16 != nullptr) e = a.gamma != nullptr ? W4_LONGK(kXFp16Norm) : W4_LONGK(kXFp16);
        else e = W4_LONGK(kXQ8);
#undef W4_LONGK
        return static_cast<int>(e);
    }
    if (!q8_epilogue && !handoff && aligned16 && steps <= 8 && a.x_f32 == nullptr &&
        ((mode == kPlain && (tall || sampling || signalled)) || (mode == kSwiglu && tall))) {
        const dim3 sgrid(std::min(num_blocks, 2 * dev->sm_count)), sblock(kMaxThreads);
        const size_t ssmem = staged_x_bytes(a.K);
        const bool pdl = pdl_enabled();
#define W4_STREAM3(XINV, SW, SA)                                                                                                \
    (steps <= 4 ? launch_kernel(gemv_w4_stream_kernel<XINV, 4, SW, SA>, sgrid, sblock, ssmem, stream, pdl, a, num_blocks)     \
     : steps <= 6 ? launch_kernel(gemv_w4_stream_kernel<XINV, 6, SW, SA>, sgrid, sblock, ssmem, stream, pdl, a, num_blocks)  \
                  : launch_kernel(gemv_w4_stream_kernel<XINV, 8, SW, SA>, sgrid, sblock, ssmem, stream, pdl, a, num_blocks))
#define W4_STREAM(XINV) (mode == kSwiglu ? W4_STREAM3(XINV, true, 0) : sampling ? W4_STREAM3(XINV, false, 1) : signalled ? W4_STREAM3(XINV, false, 2) : W4_STREAM3(XINV, false, 0))
        if (a.x_fp16 != nullptr) e = a.gamma != nullptr ? W4_STREAM(kXFp16Norm) : W4_STREAM(kXFp16);
        else e = W4_STREAM(kXQ8);
#undef W4_STREAM
#undef W4_STREAM3
        return static_cast<int>(e);
    }
    // Bulk-copy form (weights through shared memory): needs 16-byte aligned weights and a CTA share that leaves
    // room for a second CTA on the SM.
    // Forms.  Measured on B200, per shape and in the 28-layer chain, register-held weight loads beat bulk copies
    // into shared memory for every shape of the model (the copies complete as a whole, so no dot product
    // overlaps their arrival, and the weights cross shared memory once more), and spreading the K slices of the
    // down projection over a cluster costs more in cluster scheduling than the smaller activation staging saves.
    // The bulk-copy form therefore runs only on request (W4A16_OPT_GEMV_FORM = 2); it splits K over a cluster
    // where one CTA would otherwise stage or quantise more than 16 groups.
    const int form = option(W4A16_OPT_GEMV_FORM);
    if (form == 2 && aligned16 && !q8_epilogue && !handoff) {
        const bool cluster_k = mode == kPlain && a.gamma == nullptr && a.x_f32 == nullptr && a.ksplit >= 2 &&
                               a.ksplit <= 8 && a.K / kGroup > 16;
        GemvArgs b = a;
        size_t bsmem;
        dim3 bgrid, bblock;
        if (cluster_k) {
            b.units_per_cta = kMaxSubwarps;
            const int klen = b.steps_per_split * kStepElems;
            bsmem = bulk_layout(klen, b.ksplit * b.units_per_cta, b.units_per_cta * (klen / 2)).total;
            bgrid = dim3(static_cast<unsigned>((b.units + b.units_per_cta - 1) / b.units_per_cta) * b.ksplit);
            bblock = dim3(kMaxThreads);
            b.vec_ok = (b.x_fp16 == nullptr) && (reinterpret_cast<uintptr_t>(b.q8) % 16 == 0) &&
                       (reinterpret_cast<uintptr_t>(b.sum8) % 16 == 0);
        } else {
            bsmem = bulk_layout(b.K, b.ksplit * b.units_per_cta * R, b.units_per_cta * R * (b.K / 2)).total;
            bgrid = dim3(grid);
            bblock = dim3(block);
        }
        if (bsmem <= 110 * 1024) {
            switch (mode) {
                case kPlain: e = launch_bulk<kPlain>(b, cluster_k, bgrid, bblock, bsmem, stream); break;
                case kQkv: e = launch_bulk<kQkv>(b, false, bgrid, bblock, bsmem, stream); break;
                default: e = launch_bulk<kSwiglu>(b, false, bgrid, bblock, bsmem, stream); break;
            }
            return static_cast<int>(e);
        }
    }
    switch (mode) {
        case kPlain: e = launch_mode<kPlain>(a, p.U, aligned16, dim3(grid), dim3(block), smem, stream); break;
        case kQkv: e = launch_mode<kQkv>(a, p.U, aligned16, dim3(grid), dim3(block), smem, stream); break;
        default: e = launch_mode<kSwiglu>(a, p.U, aligned16, dim3(grid), dim3(block), smem, stream); break;
    }
    return static_cast<int>(e);
}

int gemv_group_dots(const uint32_t* qweight, const int8_t* q8, const int32_t* sum8, int32_t* out, int N, int K,
                    cudaStream_t stream) {
    const DeviceInfo* dev = nullptr;
    if (int st = ensure_device_ready(&dev)) return st;
    const int vec_ok = (reinterpret_cast<uintptr_t>(q8) % 16 == 0) && (reinterpret_cast<uintptr_t>(sum8) % 16 == 0);
    const int aligned16 = reinterpret_cast<uintptr_t>(qweight) % 16 == 0;
    const size_t smem = staged_x_bytes(K);
    if (smem > 200 * 1024) return W4A16_ERR_TOO_LARGE;
    const int grid = (N + kMaxSubwarps - 1) / kMaxSubwarps;
    gemv_group_dots_kernel<<<grid, kMaxThreads, smem, stream>>>(qweight, q8, sum8, out, N, K, vec_ok, aligned16);
    return static_cast<int>(cudaGetLastError());
}

}  // namespace w4
