// extern "C" wrapper around the reference's flash-decode COMBINE kernel
// (attention_gqa_flash_decode_stage2_kernel, src/kernels/attention_gqa.cu:200-310), whose epilogue produces
// the Q8_1 input of the O projection.  The reference exposes it only behind launch_attention_gqa_flash_decode,
// which runs the attention itself first; to drive the combine step with chosen accumulators this translation
// unit compiles the reference's file in place (an #include of the file where it lies, nothing copied) and
// launches the kernel directly.  TEST INFRASTRUCTURE ONLY.
#include "src/kernels/attention_gqa.cu"

#include <cstdint>

#define REF_API extern "C" __attribute__((visibility("default")))

// partial_out: fp32 [heads][FLASH_DECODE_SPLITS][head_dim]; partial_lse: fp32 [heads][FLASH_DECODE_SPLITS][2]
// (running maximum, denominator) as stage 1 leaves them.
REF_API int ref_flash_decode_combine(const float* partial_out, const float* partial_lse, void* attn_out,
                                     int8_t* out_q8, float* out_scale, int32_t* out_sum8, int heads, int head_dim,
                                     void* stream) {
    qwen::attention_gqa_flash_decode_stage2_kernel<<<dim3(heads, 1), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        partial_out, partial_lse, static_cast<half*>(attn_out), out_q8, out_scale, out_sum8, head_dim);
    return static_cast<int>(cudaGetLastError());
}

REF_API int ref_flash_decode_splits() { return qwen::FLASH_DECODE_SPLITS; }
