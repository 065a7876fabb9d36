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
#include <cstdlib>

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
           kXFp16Norm = 2 };  // fp16 vector, RMSNorm then quantised in the prologue

// Optional timeline of the decode GEMV (-DW4A16_GEMV_PROFILE): thread 0 of CTA 0 of every launch appends one
// record {globaltimer at entry, after the wait for the prior grid, at the end; latest end time of any CTA
// of the launches before it; cycles spent waiting, staging x, in the dot loop, in the reduction + epilogue}.  Read with w4a16_debug_counter.
#ifdef W4A16_GEMV_PROFILE
constexpr int kProfRecords = 1024;
__device__ unsigned int g_gemv_prof[kProfRecords * 8];
__device__ unsigned int g_gemv_prof_n;
__device__ unsigned int g_gemv_last_end;   // latest end time of any CTA of any GEMV so far
__device__ __forceinline__ unsigned int gtimer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return static_cast<unsigned int>(t);
}
#define GP_DECL() const bool gp_on = blockIdx.x == 0 && threadIdx.x == 0; unsigned int gp[8]; long long gp_c = 0; \
    if (gp_on) { gp[0] = gtimer(); gp_c = clock64(); }
#define GP_MARK(i) if (gp_on) { const long long c_ = clock64(); gp[i] = static_cast<unsigned int>(c_ - gp_c); gp_c = c_; }
#define GP_GT(i) if (gp_on) { gp[i] = gtimer(); }
#define GP_PREV_END(i) if (gp_on) { gp[i] = *reinterpret_cast<volatile unsigned int*>(&g_gemv_last_end); }
#define GP_END() if (threadIdx.x == 0) { atomicMax(&g_gemv_last_end, gtimer()); }
#define GP_FLUSH() if (gp_on) { const unsigned int n_ = atomicAdd(&g_gemv_prof_n, 1u); if (n_ < kProfRecords) { \
    for (int i_ = 0; i_ < 8; ++i_) g_gemv_prof[n_ * 8 + i_] = gp[i_]; } }
#else
#define GP_DECL()
#define GP_MARK(i)
#define GP_GT(i)
#define GP_PREV_END(i)
#define GP_END()
#define GP_FLUSH()
#endif

// Register caps: two 256-thread CTAs per SM need <= 128; the single-row forms with 8 loads per lane run as
// 224-thread CTAs (down projection) of which three must fit an SM for the whole grid to be resident at once.
constexpr int gemv_reg_cap(int mode, int u) { return (mode != kSwiglu && u == 8) ? 96 : 128; }

template <int MODE, int U, int XIN, bool ALIGNED16>
__global__ void __maxnreg__(gemv_reg_cap(MODE, U)) gemv_w4_kernel(const GemvArgs a) {
    GP_DECL();
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
    // Everything that does not depend on the prior grid goes before the wait: the weights above and the
    // RMSNorm gain.  After it, every global round trip is on the critical path between two GEMVs, so the
    // residual element is requested first and the activation is staged with one round trip.
    [[maybe_unused]] uint4 gam[kStageRounds];
    [[maybe_unused]] bool regs_form = false;
    if constexpr (XIN != kXQ8) {
        regs_form = stage_regs_ok(a.x_fp16, XIN == kXFp16Norm ? static_cast<const void*>(a.gamma) : nullptr, K);
        if constexpr (XIN == kXFp16Norm) {
            if (regs_form) prefetch_gamma(a.gamma, K, gam);
        }
    }
    pdl_release_dependents();
    GP_MARK(4);
    pdl_wait_prior_grids();
    GP_MARK(4);
    GP_GT(1);
    GP_PREV_END(3);

    [[maybe_unused]] __half res_pre = __ushort_as_half(0);
    if constexpr (MODE == kPlain) {
        if (active && ks == 0 && l == 0 && a.residual != nullptr) res_pre = a.residual[unit];
    }
    if constexpr (XIN == kXFp16Norm) {
#ifdef W4A16_GEMV_PROFILE
        if (regs_form) stage_x_fp16_regs<true>(a.x_fp16, gam, K, kRmsEps, s_q8, s_seed, s_scale,
                                               gp_on ? &g_gemv_prof[8000 + 8 * MODE] : nullptr);
#else
        if (regs_form) stage_x_fp16_regs<true>(a.x_fp16, gam, K, kRmsEps, s_q8, s_seed, s_scale);
#endif
        else stage_x_from_fp16_rmsnorm(a.x_fp16, a.gamma, K, kRmsEps, s_q8, s_seed, s_scale);
    } else if constexpr (XIN == kXFp16) {
#ifdef W4A16_GEMV_PROFILE
        if (regs_form) stage_x_fp16_regs<false>(a.x_fp16, gam, K, kRmsEps, s_q8, s_seed, s_scale,
                                                gp_on ? &g_gemv_prof[8000 + 8 * 3] : nullptr);
#else
        if (regs_form) stage_x_fp16_regs<false>(a.x_fp16, gam, K, kRmsEps, s_q8, s_seed, s_scale);
#endif
        else stage_x_from_fp16(a.x_fp16, K, s_q8, s_seed, s_scale);
    } else {
        if (!stage_x_from_q8_1_regs<(R * U >= 16)>(a.q8, a.xscale, a.sum8, K, a.vec_ok != 0, s_q8, s_seed, s_scale))
            stage_x_from_q8_1(a.q8, a.xscale, a.sum8, K, a.vec_ok != 0, s_q8, s_seed, s_scale);
    }
    __syncthreads();
    GP_MARK(5);

    float acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = 0.0f;

    for (int s0 = s_begin; s0 < s_end; s0 += U) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int s = s0 + u;
            if (s < s_end) {
                const int c = s * kSubwarp + l;  // 32-element chunk index along K
                const uint4 xa = reinterpret_cast<const uint4*>(s_q8)[2 * c];
                const uint4 xb = reinterpret_cast<const uint4*>(s_q8)[2 * c + 1];
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

    GP_MARK(6);
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

    if constexpr (MODE == kSwiglu) {
        // Q8_1 of the output vector in the same launch.  The launch guarantees 32 outputs per CTA, no K
        // split and clusters of four CTAs, i.e. one quantisation group of 128 per cluster: the CTAs swap
        // their |max| through distributed shared memory, one cluster barrier, then each quantises its own
        // 32 outputs (one chunk: 32 bytes, four sum8 entries) with the group's scale.  Same arithmetic as
        // quantize_group128_lane, so the arrays equal the stand-alone quantiser's bit for bit.
        if (a.q8_out != nullptr) {
            __shared__ float s_y[kMaxSubwarps];
            __shared__ float s_cluster_max[4];
#ifdef W4A16_GEMV_PROFILE
            long long qt = clock64();
#define GP_Q(i) if (gp_on) { const long long c_ = clock64(); g_gemv_prof[8100 + (i)] = static_cast<unsigned int>(c_ - qt); qt = c_; }
#else
#define GP_Q(i)
#endif
            if (l == 0) s_y[sub] = y_rounded;
            __syncthreads();
            GP_Q(0);
            uint32_t rank;
            asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
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
            GP_Q(1);
            asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
            asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
            GP_Q(2);
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
            GP_Q(3);
        }
    }
    GP_MARK(7);
    GP_GT(2);
    GP_FLUSH();
    GP_END();
}

}  // namespace

// Timeline records of the decode GEMV (zeros unless built with -DW4A16_GEMV_PROFILE).  which: -1 resets the
// record count, -2 returns it, otherwise word `which` of the record table.
int gemv_prof(int which, unsigned int* out) {
#ifdef W4A16_GEMV_PROFILE
    if (which == -1) { const unsigned int z = 0; *out = 0; return static_cast<int>(cudaMemcpyToSymbol(g_gemv_prof_n, &z, sizeof(z))); }
    if (which == -2) return static_cast<int>(cudaMemcpyFromSymbol(out, g_gemv_prof_n, sizeof(unsigned int)));
    if (which >= kProfRecords * 8) return W4A16_ERR_INVALID_ARG;
    return static_cast<int>(cudaMemcpyFromSymbol(out, g_gemv_prof, sizeof(unsigned int), sizeof(unsigned int) * which));
#else
    (void)which; *out = 0; return 0;
#endif
}

namespace {

// Streaming form for very tall matrices (lm_head): a persistent grid, each CTA walks row blocks of 32 with
// the weights of the NEXT block already in flight while the current one is reduced, and the lane's share
// of the quantised activation lives in registers for the whole launch (a lane always meets the same
// 16-byte chunks l, l+8, ... of every row).  PLAIN mode, 16-byte aligned weights, K <= 256 * STEPS.
template <int XIN, int STEPS, bool SWIGLU, bool SAMPLE = false>
__global__ void __launch_bounds__(kMaxThreads, 2) gemv_w4_stream_kernel(const GemvArgs a, const int num_blocks) {
    static_assert(!(SWIGLU && SAMPLE), "token selection follows a plain projection");
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
        xa[i] = reinterpret_cast<const uint4*>(s_q8)[2 * c];
        xb[i] = reinterpret_cast<const uint4*>(s_q8)[2 * c + 1];
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
            if (l == 0 && row < N) {
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
                reinterpret_cast<uint4*>(s_q8)[i] = reinterpret_cast<const uint4*>(q8)[i];
            for (int c = tid; c < K / kChunk; c += nthr) {
                const int4 v = reinterpret_cast<const int4*>(sum8)[c];
                s_seed[c] = v.x + v.y + v.z + v.w;
            }
        } else {
            for (int i = tid; i < K; i += nthr) s_q8[i] = q8[i];
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
            const uint4 xa = reinterpret_cast<const uint4*>(s_q8)[2 * c];
            const uint4 xb = reinterpret_cast<const uint4*>(s_q8)[2 * c + 1];
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

// Picks the CTA shape.  units: output rows (or pairs).  Goals, in order: at least ~1.3 CTAs
// per SM when the matrix allows it; all 32 sub-warps of a CTA busy; at most 8 loads per lane
// per batch so one batch covers a lane's whole K slice for the model's shapes; and the whole grid
// resident at once (a second wave of CTAs would start its weight loads only after the wait).
Plan make_plan(GemvMode mode, int units, int K, int sm_count) {
    static const int force_units = env_int("W4A16_GEMV_UNITS", 0);
    static const int force_ksplit = env_int("W4A16_GEMV_KSPLIT", 0);
    static const int force_u = env_int("W4A16_GEMV_U", 0);
    const int steps = K / kStepElems;
    const int target_ctas = (sm_count * 13 + 9) / 10;
    int upc = 32;
    while (upc > 4 && (units + upc - 1) / upc < target_ctas) upc /= 2;
    if (force_units > 0) upc = std::min(32, std::max(1, force_units));
    int cap = std::max(1, kMaxSubwarps / upc);   // most K slices the CTA can hold
    cap = std::min(cap, steps);
    int per = (steps + cap - 1) / cap;           // steps per slice if all slices were used
    int ksplit = (steps + per - 1) / per;        // fewest slices that reach that depth
    auto pick_u = [&](int depth) { return force_u == 4 || force_u == 8 ? force_u : (depth <= 4 ? 4 : 8); };
    if (force_ksplit > 0) {
        ksplit = std::min(std::min(force_ksplit, steps), kMaxSubwarps / upc);
        ksplit = std::max(1, ksplit);
        per = (steps + ksplit - 1) / ksplit;
    } else {
        const int grid = (units + upc - 1) / upc;
        while (ksplit > 1) {
            const int warps = (upc * ksplit * kSubwarp + 31) / 32;
            const int ctas_per_sm = resident_warps_per_sm(mode, pick_u(per)) / warps;
            if (grid <= ctas_per_sm * sm_count || per >= 8) break;
            per = (steps + (ksplit - 1) - 1) / (ksplit - 1);   // one slice fewer, deeper slices
            ksplit = (steps + per - 1) / per;
        }
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
    if (a.x_fp16 != nullptr) {
        if (a.gamma != nullptr) return launch_aligned<MODE, U, kXFp16Norm>(a, aligned16, grid, block, smem, stream);
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
    return static_cast<int>(e);
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
    a.vec_ok = (a.x_fp16 == nullptr) && (reinterpret_cast<uintptr_t>(a.q8) % 16 == 0) &&
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
    static const int stream_on = env_int("W4A16_GEMV_STREAM", 1);
    const int steps = a.K / kStepElems;
    const int weight_rows = mode == kSwiglu ? 2 * a.units : a.units;
    const int num_blocks = (weight_rows + kMaxSubwarps - 1) / kMaxSubwarps;
    static const int stream_min_blocks = env_int("W4A16_GEMV_STREAM_MIN", 16);   // row blocks per SM from which it pays
    static const int stream_swiglu = env_int("W4A16_GEMV_STREAM_SWIGLU", 0);
    const bool tall = num_blocks >= stream_min_blocks * dev->sm_count;
    const bool sampling = a.sample_val != nullptr || a.sample_idx != nullptr;
    if (sampling && (mode != kPlain || !a.sample_val || !a.sample_idx || !aligned16 || steps > 8)) return W4A16_ERR_SHAPE;
    if ((sampling || stream_on) && !q8_epilogue && aligned16 && steps <= 8 &&
        ((mode == kPlain && (tall || sampling)) || (mode == kSwiglu && (tall || (stream_swiglu && num_blocks >= 3 * dev->sm_count))))) {
        const dim3 sgrid(std::min(num_blocks, 2 * dev->sm_count)), sblock(kMaxThreads);
        const size_t ssmem = staged_x_bytes(a.K);
        const bool pdl = pdl_enabled();
#define W4_STREAM3(XINV, SW, SA)                                                                                                \
    (steps <= 4 ? launch_kernel(gemv_w4_stream_kernel<XINV, 4, SW, SA>, sgrid, sblock, ssmem, stream, pdl, a, num_blocks)     \
     : steps <= 6 ? launch_kernel(gemv_w4_stream_kernel<XINV, 6, SW, SA>, sgrid, sblock, ssmem, stream, pdl, a, num_blocks)  \
                  : launch_kernel(gemv_w4_stream_kernel<XINV, 8, SW, SA>, sgrid, sblock, ssmem, stream, pdl, a, num_blocks))
#define W4_STREAM(XINV) (mode == kSwiglu ? W4_STREAM3(XINV, true, false) : sampling ? W4_STREAM3(XINV, false, true) : W4_STREAM3(XINV, false, false))
        if (a.x_fp16 != nullptr) e = a.gamma != nullptr ? W4_STREAM(kXFp16Norm) : W4_STREAM(kXFp16);
        else e = W4_STREAM(kXQ8);
#undef W4_STREAM
#undef W4_STREAM3
        return static_cast<int>(e);
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
