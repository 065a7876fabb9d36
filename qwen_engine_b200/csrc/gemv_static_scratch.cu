// fp16-input decode GEMV for callers that cannot hand the library any scratch memory and
// cannot allocate it either: the Q8_1 form of the activation lives in a fixed array that is
// part of the library's device image.
//
// Why it exists.  w4a16_gemv_w4a16 quantises the activation inside every CTA, which costs
// nothing for short vectors but is repeated work for long ones (the down projection,
// K = 8960, runs faster when the vector is quantised once and the GEMV reads the result).
// Quantising once needs somewhere to put the int8 / scale / sum arrays.  An engine that
// gave its whole device-memory budget to one arena at start-up, or a plugin host that
// forbids allocation calls on its inference path, has no buffer to pass and may not call
// cudaMalloc; this entry point brings its own.
//
// The array is `static __device__`, so every GPU that loads the library holds those
// 50 176 bytes until the process exits.  Its name is only a host-side handle here: the
// device address is looked up once per device with cudaGetSymbolAddress (below) and that
// pointer is what the kernels receive.
#include <mutex>

#include "w4a16_internal.hpp"

namespace {

constexpr int kMaxK = 32768;                                   // largest in_features accepted
constexpr size_t kQ8Bytes = kMaxK;                             // int8  q8[K]
constexpr size_t kScaleBytes = (kMaxK / 128) * sizeof(float);  // fp32  scale[K/128]
constexpr size_t kSum8Bytes = (kMaxK / 8) * sizeof(int32_t);   // int32 sum8[K/8]
constexpr size_t kScratchBytes = kQ8Bytes + kScaleBytes + kSum8Bytes;

static __device__ __align__(256) unsigned char g_q8_1_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
unsigned char* g_scratch_ptr[kMaxDevices] = {};
std::mutex g_scratch_mutex;

// Device address of the array on the current device (looked up on the first call per device).
int scratch_for_current_device(unsigned char** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (dev < 0 || dev >= kMaxDevices) return W4A16_ERR_NO_DEVICE;
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (g_scratch_ptr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_q8_1_scratch);  // with `dev` current: this device's copy
        if (e != cudaSuccess) return static_cast<int>(e);
        g_scratch_ptr[dev] = static_cast<unsigned char*>(p);
    }
    *out = g_scratch_ptr[dev];
    return 0;
}

}  // namespace

extern "C" int w4a16_gemv_w4a16_static_scratch(const uint32_t* qweight, const void* scales, const void* input_x,
                                               const void* residual, void* output_y, int out_features,
                                               int in_features, w4a16_stream_t stream_) {
    using namespace w4;
    if (!qweight || !scales || !input_x || !output_y || out_features <= 0) return W4A16_ERR_INVALID_ARG;
    if (in_features <= 0 || in_features % 256 != 0) return W4A16_ERR_SHAPE;
    if (in_features > kMaxK) return W4A16_ERR_TOO_LARGE;  // the fixed array holds at most kMaxK elements
    auto mis = [](const void* p, size_t a) { return reinterpret_cast<uintptr_t>(p) % a != 0; };
    if (mis(qweight, 4) || mis(scales, 2) || mis(input_x, 8) || mis(output_y, 2) || mis(residual, 2))
        return W4A16_ERR_ALIGNMENT;
    if (int st = ensure_device_ready(nullptr)) return st;
    unsigned char* base = nullptr;
    if (int st = scratch_for_current_device(&base)) return st;

    int8_t* q8 = reinterpret_cast<int8_t*>(base);
    float* xscale = reinterpret_cast<float*>(base + kQ8Bytes);
    int32_t* sum8 = reinterpret_cast<int32_t*>(base + kQ8Bytes + kScaleBytes);
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);

    // Nothing in the array has to start at zero: the quantiser overwrites every byte the GEMV
    // reads for this in_features, so what an earlier call left behind is never seen.
    if (int st = quantize_fp16_to_q8_1(static_cast<const __half*>(input_x), q8, xscale, sum8, in_features, stream))
        return st;
    GemvArgs a = {};
    a.qweight[0] = qweight;
    a.scales[0] = static_cast<const __half*>(scales);
    a.out[0] = static_cast<__half*>(output_y);
    a.rows[0] = out_features;
    a.q8 = q8;
    a.xscale = xscale;
    a.sum8 = sum8;
    a.residual = static_cast<const __half*>(residual);
    a.K = in_features;
    a.units = out_features;
    return gemv_launch(kPlain, a, stream);
}
