// Host dispatch of the M-token W4A16 contraction (small-M decode batches and prefill).
#include <algorithm>

#include "gemm_smallm.cuh"
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

}  // namespace

int gemm_set_attributes() { return gemm_tc_set_attributes(); }

int gemm_launch(GemmArgs g, cudaStream_t stream) {
    const DeviceInfo* dev = nullptr;
    if (int st = ensure_device_ready(&dev)) return st;

    // The tcgen05 kernel pads the token count to its smallest tile (16) and is already faster than the
    // CUDA-core weight-streaming kernel from a handful of tokens (measured crossover on B200: 3-5 tokens
    // depending on the shape); the CUDA-core kernel serves 1-3 tokens and pointers or shapes TMA cannot address.
    static const int tc_min_m = env_int("W4A16_TC_MIN_M", 4);
    if (g.M >= tc_min_m && gemm_tc_supported(g)) return gemm_tc_launch(g, dev->sm_count, stream);

    SmallMArgs a;
    a.g = g;
    const int total_rows = g.rows[0] + (g.mode == kQkv ? g.rows[1] + g.rows[2] : 0);
    a.units = (g.mode == kSwiglu) ? total_rows / 2 : total_rows;
    if (g.mode == kQkv) {
        a.out_ld[0] = g.rows[0]; a.out_ld[1] = g.rows[1]; a.out_ld[2] = g.rows[2];
    } else {
        a.out_ld[0] = a.units; a.out_ld[1] = a.out_ld[2] = 0;
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
