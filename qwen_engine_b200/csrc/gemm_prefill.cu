// Host dispatch of the M-token W4A16 contraction (small-M decode batches and prefill).
#include <algorithm>

#include "gemm_smallm.cuh"
#include "gemm_smallm_mma.cuh"
#include "w4a16_internal.hpp"

namespace w4 {
namespace {

template <int MODE>
cudaError_t launch_smallm(const SmallMArgs& a, int mt, dim3 grid, dim3 block, cudaStream_t stream) {
    const bool pdl = pdl_enabled();
    switch (mt) {
        case 1: return launch_kernel(gemm_smallm_kernel<MODE, 1>, grid, block, 0, stream, pdl, a);
        case 2: return launch_kernel(gemm_smallm_kernel<MODE, 2>, grid, block, 0, stream, pdl, a);
        default: return launch_kernel(gemm_smallm_kernel<MODE, 4>, grid, block, 0, stream, pdl, a);
    }
}

// ---- few-token form (gemm_smallm_v2_kernel) ----
template <int MODE, int U, int MT>
cudaError_t launch_v2_one(const SmallMArgs& a, const SmallMPlan& p, dim3 grid, dim3 block, size_t smem, cudaStream_t stream) {
    return launch_kernel(gemm_smallm_v2_kernel<MODE, U, MT>, grid, block, smem, stream, pdl_enabled(), a, p);
}
template <int MODE>
cudaError_t launch_v2(const SmallMArgs& a, const SmallMPlan& p, int U, int mt, dim3 grid, dim3 block, size_t smem,
                      cudaStream_t stream) {
    if (U == 4) {
        if (mt == 1) return launch_v2_one<MODE, 4, 1>(a, p, grid, block, smem, stream);
        if (mt == 2) return launch_v2_one<MODE, 4, 2>(a, p, grid, block, smem, stream);
        return launch_v2_one<MODE, 4, 4>(a, p, grid, block, smem, stream);
    }
    if (mt == 1) return launch_v2_one<MODE, 8, 1>(a, p, grid, block, smem, stream);
    if (mt == 2) return launch_v2_one<MODE, 8, 2>(a, p, grid, block, smem, stream);
    return launch_v2_one<MODE, 8, 4>(a, p, grid, block, smem, stream);
}
template <int MODE, int U, int MT>
cudaError_t raise_v2() {
    return cudaFuncSetAttribute(gemm_smallm_v2_kernel<MODE, U, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
}
template <int MODE>
cudaError_t raise_v2_mode() {
    cudaError_t e = raise_v2<MODE, 4, 1>();
    if (e == cudaSuccess) e = raise_v2<MODE, 4, 2>();
    if (e == cudaSuccess) e = raise_v2<MODE, 4, 4>();
    if (e == cudaSuccess) e = raise_v2<MODE, 8, 1>();
    if (e == cudaSuccess) e = raise_v2<MODE, 8, 2>();
    if (e == cudaSuccess) e = raise_v2<MODE, 8, 4>();
    return e;
}

// CTA shape of the few-token form: as the decode GEMV's -- enough CTAs for every SM, all sub-warps busy,
// the K range of a sub-warp at most 8 steps deep, and the whole grid resident (16 warps per SM at the
// kernel's 128 registers).  Returns false when a K slice would be deeper than 8 steps.
bool plan_v2(const GemmArgs& g, int units, int sm_count, SmallMPlan* out, int* U) {
    const int steps = g.K / kStepElems;
    const int target = (sm_count * 13 + 9) / 10;
    int upc = 32;
    while (upc > 4 && (units + upc - 1) / upc < target) upc /= 2;
    if (g.mode == kQkv)
        while (upc > 1 && (g.rows[0] % upc || g.rows[1] % upc)) upc /= 2;
    int cap = std::min(std::max(1, 32 / upc), steps);
    int per = (steps + cap - 1) / cap;
    int ksplit = (steps + per - 1) / per;
    const int grid = (units + upc - 1) / upc;
    while (ksplit > 1 && per < 8) {
        const int warps = (upc * ksplit * kSubwarp + 31) / 32;
        if (grid <= (16 / warps) * sm_count) break;
        per = (steps + (ksplit - 1) - 1) / (ksplit - 1);
        ksplit = (steps + per - 1) / per;
    }
    if (per > 8) return false;
    out->units_per_cta = upc;
    out->ksplit = ksplit;
    out->steps_per_split = per;
    *U = per <= 4 ? 4 : 8;
    return true;
}

// ---- few-token mma.sync form (gemm_smallm_mma_kernel) ----
template <int MODE, int U>
cudaError_t launch_mma_nt(const SmallMArgs& a, const SmallMmaPlan& p, int NT, dim3 grid, dim3 block, size_t smem, cudaStream_t stream) {
    const bool pdl = pdl_enabled();
    if (NT == 1) return launch_kernel(gemm_smallm_mma_kernel<MODE, U, 1>, grid, block, smem, stream, pdl, a, p);
    if (NT == 2) return launch_kernel(gemm_smallm_mma_kernel<MODE, U, 2>, grid, block, smem, stream, pdl, a, p);
    return launch_kernel(gemm_smallm_mma_kernel<MODE, U, 4>, grid, block, smem, stream, pdl, a, p);
}
template <int MODE>
cudaError_t launch_mma(const SmallMArgs& a, const SmallMmaPlan& p, int U, int NT, dim3 grid, dim3 block, size_t smem, cudaStream_t stream) {
    if (U == 4) return launch_mma_nt<MODE, 4>(a, p, NT, grid, block, smem, stream);
    return launch_mma_nt<MODE, 8>(a, p, NT, grid, block, smem, stream);
}
template <int MODE, int U, int NT>
cudaError_t raise_mma() {
    return cudaFuncSetAttribute(gemm_smallm_mma_kernel<MODE, U, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
}
template <int MODE>
cudaError_t raise_mma_mode() {
    cudaError_t e = raise_mma<MODE, 4, 1>();
    if (e == cudaSuccess) e = raise_mma<MODE, 4, 2>();
    if (e == cudaSuccess) e = raise_mma<MODE, 4, 4>();
    if (e == cudaSuccess) e = raise_mma<MODE, 8, 1>();
    if (e == cudaSuccess) e = raise_mma<MODE, 8, 2>();
    if (e == cudaSuccess) e = raise_mma<MODE, 8, 4>();
    return e;
}

// CTA shape of the mma.sync form.  A warp = 16 MMA rows x one K slice of at most 8 steps of 128; enough slices that
// about 8 warps per SM exist where the matrix is short, row groups per CTA so that a CTA has up to 8-16 warps while
// the grid still covers the SMs.  False when the shape does not fit (rows not in whole groups, shared memory).
bool plan_mma(const GemmArgs& g, int units, int sm_count, SmallMmaPlan* out, int* U, int* NT, size_t* smem) {
    const int uw = g.mode == kSwiglu ? 8 : 16;
    if (units % uw) return false;
    if (g.mode == kQkv && (g.rows[0] % 16 || g.rows[1] % 16 || g.rows[2] % 16)) return false;
    const int steps = g.K / kGroup;
    const int groups_total = units / uw;
    // slices of at most 4 steps where 16 warps allow it (the 4-step form has registers to spare for the token loads)
    int ksplit = std::max((steps + 3) / 4, (8 * sm_count + groups_total - 1) / groups_total);
    ksplit = std::min(ksplit, std::min(steps, 16));
    int per = (steps + ksplit - 1) / ksplit;
    ksplit = (steps + per - 1) / per;
    // the whole grid must be resident (16 warps per SM at 128 registers): deeper slices where it would not be
    while (static_cast<long long>(groups_total) * ksplit > 16LL * sm_count && per < 8) {
        ++per;
        ksplit = (steps + per - 1) / per;
    }
    if (per > 8 || static_cast<long long>(groups_total) * ksplit > 16LL * sm_count) return false;
    // every CTA stages all the tokens, so fewer and larger CTAs mean less traffic for them: up to 16 warps per CTA
    // as long as about one CTA per SM remains
    int gpc = std::max(1, std::min(8, 16 / ksplit));
    while (gpc > 1 && groups_total / gpc < (sm_count * 9) / 10) gpc /= 2;
    int nt = g.M <= 8 ? 1 : (g.M <= 16 ? 2 : 4);
    auto bytes = [&](int n) {
        return static_cast<size_t>(g.K / 4) * (8 * n) * 8 + static_cast<size_t>(ksplit) * gpc * n * 4 * 32 * sizeof(float);
    };
    while (nt > 1 && bytes(nt) > 100 * 1024) nt /= 2;
    if (bytes(nt) > 200 * 1024) return false;
    out->groups_per_cta = gpc;
    out->ksplit = ksplit;
    out->steps_per_split = per;
    out->passes_tokens = 8 * nt;
    *U = per <= 4 ? 4 : 8;
    *NT = nt;
    *smem = bytes(nt);
    return true;
}

}  // namespace

int gemm_set_attributes() {
    cudaError_t e = raise_v2_mode<kPlain>();
    if (e == cudaSuccess) e = raise_v2_mode<kQkv>();
    if (e == cudaSuccess) e = raise_v2_mode<kSwiglu>();
    if (e == cudaSuccess) e = raise_mma_mode<kPlain>();
    if (e == cudaSuccess) e = raise_mma_mode<kQkv>();
    if (e == cudaSuccess) e = raise_mma_mode<kSwiglu>();
    if (e != cudaSuccess) return static_cast<int>(e);
    return gemm_tc_set_attributes();
}

int gemm_launch(GemmArgs g, cudaStream_t stream) {
    const DeviceInfo* dev = nullptr;
    if (int st = ensure_device_ready(&dev)) return st;

    // The tcgen05 kernel pads the token count to its smallest tile (16), so below a handful of tokens the CUDA-core
    // few-token form (the decode GEMV's memory behaviour with fp16 arithmetic) is the faster one.  Measured
    // crossovers on B200: 3 tokens where K > 4096 (down: the few-token form stages only two tokens per pass there),
    // 4 on matrices tall enough to give every SM a CTA of their own (gate_up), 7 on the narrow K <= 4096 shapes
    // (QKV, O).  The CUDA-core forms also take what TMA cannot address.
    const int tc_min_m_opt = option(W4A16_OPT_GEMM_MIN_TOKENS_TENSOR_CORE);
    const int rows_all = g.rows[0] + (g.mode == kQkv ? g.rows[1] + g.rows[2] : 0);
    const int tc_min_m = tc_min_m_opt > 0 ? tc_min_m_opt : (g.K > 4096 ? 3 : (rows_all >= 64 * dev->sm_count ? 4 : 7));
    SmallMArgs a;
    a.g = g;
    const int total_rows = g.rows[0] + (g.mode == kQkv ? g.rows[1] + g.rows[2] : 0);
    a.units = (g.mode == kSwiglu) ? total_rows / 2 : total_rows;
    if (g.mode == kQkv) {
        a.out_ld[0] = g.rows[0]; a.out_ld[1] = g.rows[1]; a.out_ld[2] = g.rows[2];
    } else {
        a.out_ld[0] = (g.mode == kPlain && g.ldc > 0) ? g.ldc : a.units; a.out_ld[1] = a.out_ld[2] = 0;
    }
    bool aligned = reinterpret_cast<uintptr_t>(g.x) % 16 == 0;
    for (int t = 0; t < (g.mode == kQkv ? 3 : 1); ++t) aligned = aligned && reinterpret_cast<uintptr_t>(g.qweight[t]) % 16 == 0;

    // Two to sixteen tokens: the weight-streaming kernel with the warp-level MMA (no fixed tcgen05 costs).  Measured on
    // B200 against the other two forms: faster from 2 tokens on every Qwen shape (QKV: equal to the CUDA-core form up
    // to 4), and up to 16 tokens as long as they are staged in one pass (K = 8960 holds 8 tokens per pass: from 9 the
    // tcgen05 kernel wins there).
    const int mma_max_opt = option(W4A16_OPT_GEMM_MMA_MAX_TOKENS);
    const int mma_max_m = mma_max_opt > 0 ? mma_max_opt : 16;
    if (aligned && g.num_peers == 0 && g.M >= std::max(2, tc_min_m_opt) && g.M <= mma_max_m) {
        SmallMmaPlan mp;
        int mU = 8, mNT = 1;
        size_t msmem = 0;
        if (plan_mma(g, a.units, dev->sm_count, &mp, &mU, &mNT, &msmem) && (mma_max_opt > 0 || g.M <= mp.passes_tokens)) {
            const dim3 mgrid((a.units / (g.mode == kSwiglu ? 8 : 16) + mp.groups_per_cta - 1) / mp.groups_per_cta);
            const dim3 mblock(32 * mp.groups_per_cta * mp.ksplit);
            cudaError_t me;
            switch (g.mode) {
                case kPlain: me = launch_mma<kPlain>(a, mp, mU, mNT, mgrid, mblock, msmem, stream); break;
                case kQkv: me = launch_mma<kQkv>(a, mp, mU, mNT, mgrid, mblock, msmem, stream); break;
                default: me = launch_mma<kSwiglu>(a, mp, mU, mNT, mgrid, mblock, msmem, stream); break;
            }
            return static_cast<int>(me);
        }
    }
    if ((g.M >= tc_min_m || g.num_peers > 0) && gemm_tc_supported(g)) return gemm_tc_launch(g, dev->sm_count, stream);
    if (g.num_peers > 0) return W4A16_ERR_SHAPE;   // peer stores exist in the tensor-core form only

    // few tokens, 16-byte aligned tensors: the form that streams like the decode GEMV
    SmallMPlan plan;
    int U = 8;
    if (aligned && plan_v2(g, a.units, dev->sm_count, &plan, &U)) {
        const int R = g.mode == kSwiglu ? 2 : 1;
        // tokens per pass: as many as the shared-memory budget of a CTA (about a third of an SM) allows
        int mt = g.M >= 4 ? 4 : (g.M >= 2 ? 2 : 1);
        auto smem_for = [&](int t) {
            return (static_cast<size_t>(t) * smallm_x_stride(g.K) + static_cast<size_t>(plan.ksplit) * plan.units_per_cta * R * t) * sizeof(float);
        };
        if (g.mode == kSwiglu && U == 8) mt = std::min(mt, 2);   // row pairs with 8 loads each: the registers are full
        while (mt > 1 && smem_for(mt) > 72 * 1024) mt /= 2;
        if (smem_for(mt) <= 160 * 1024) {
            const int threads = plan.units_per_cta * plan.ksplit * kSubwarp;
            const dim3 grid2((a.units + plan.units_per_cta - 1) / plan.units_per_cta), block2((threads + 31) / 32 * 32);
            cudaError_t e2;
            switch (g.mode) {
                case kPlain: e2 = launch_v2<kPlain>(a, plan, U, mt, grid2, block2, smem_for(mt), stream); break;
                case kQkv: e2 = launch_v2<kQkv>(a, plan, U, mt, grid2, block2, smem_for(mt), stream); break;
                default: e2 = launch_v2<kSwiglu>(a, plan, U, mt, grid2, block2, smem_for(mt), stream); break;
            }
            return static_cast<int>(e2);
        }
    }
    int upc = 32;
    const int target = (dev->sm_count * 13 + 9) / 10;
    while (upc > 4 && (a.units + upc - 1) / upc < target) upc /= 2;
    if (g.mode == kQkv)
        while (upc > 1 && (g.rows[0] % upc || g.rows[1] % upc)) upc /= 2;
    a.units_per_cta = upc;
    const int mt = g.M >= 4 ? 4 : (g.M >= 2 ? 2 : 1);
    const dim3 grid((a.units + upc - 1) / upc), block(std::max(32, upc * kSubwarp));
    cudaError_t e;
    switch (g.mode) {
        case kPlain: e = launch_smallm<kPlain>(a, mt, grid, block, stream); break;
        case kQkv: e = launch_smallm<kQkv>(a, mt, grid, block, stream); break;
        default: e = launch_smallm<kSwiglu>(a, mt, grid, block, stream); break;
    }
    return static_cast<int>(e);
}

}  // namespace w4
