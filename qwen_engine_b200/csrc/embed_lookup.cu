// Embedding lookup on the W4 group-128 table (the tied lm_head matrix read the other way round):
// one row of packed nibbles and its group scales -> fp16, (q - 8) * scale with one fp16 rounding.
// Replaces the reference's launch_embed_lookup_w4a16 (include/kernels.cuh, src/kernels/rmsnorm_rope.cu:15-69);
// same token source rule: d_token_ids if given, else the control block's token, invalid ids read row 0.
#include "gemm_smallm.cuh"
#include "sampling.cuh"
#include "w4a16_common.cuh"
#include "w4a16_internal.hpp"

namespace w4 {
namespace {

__global__ void __launch_bounds__(256) embed_lookup_kernel(const uint32_t* __restrict__ qweight,
                                                           const __half* __restrict__ scales,
                                                           const int32_t* __restrict__ token_ids, __half* __restrict__ out,
                                                           const SampleControl* __restrict__ control, int hidden,
                                                           int vocab) {
    pdl_release_dependents();
    pdl_wait_prior_grids();
    int32_t token = 0;
    if (token_ids != nullptr) token = token_ids[blockIdx.x];
    else if (control != nullptr) token = control->token_id;
    if (token < 0 || token >= vocab) token = 0;
    const int words = hidden / 8, groups = hidden / kGroup;
    const uint32_t* wrow = qweight + static_cast<size_t>(token) * words;
    const __half* srow = scales + static_cast<size_t>(token) * groups;
    __half* dst = out + static_cast<size_t>(blockIdx.x) * hidden;
    for (int i = threadIdx.x; i < words; i += blockDim.x) {
        __half2 h[4];
        dequant_word_fp16(wrow[i], __half2half2(srow[i / (kGroup / 8)]), h);
        *reinterpret_cast<uint4*>(dst + i * 8) = *reinterpret_cast<const uint4*>(h);
    }
}

}  // namespace

int embed_lookup(const uint32_t* qweight, const __half* scales, const int32_t* token_ids, __half* out,
                 const void* control, int num_tokens, int hidden, int vocab, cudaStream_t stream) {
    const int threads = std::min(256, std::max(32, (hidden / 8 + 31) / 32 * 32));
    return static_cast<int>(launch_kernel(embed_lookup_kernel, dim3(num_tokens), dim3(threads), 0, stream, pdl_enabled(),
                                          qweight, scales, token_ids, out, static_cast<const SampleControl*>(control),
                                          hidden, vocab));
}

}  // namespace w4
