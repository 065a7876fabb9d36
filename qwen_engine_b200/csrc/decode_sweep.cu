// Host driver of the decode projection sweep: the W4 launches of one batch-1 decode pass in
// the reference engine's order (reference src/engine.cu:361-451), captured once into a CUDA
// graph like the engine's decode graph (src/engine.cu:453-470).  Host C++ only; the kernels
// are the library's ordinary launchers.
#include <memory>
#include <new>
#include <vector>

#include "w4a16_internal.hpp"

struct w4a16_sweep {
    w4a16_sweep_desc desc{};
    std::vector<w4a16_layer_weights> layers;
    // workspace carve-up (device)
    __half* h = nullptr;      // hidden state [hidden]
    __half* q = nullptr;      // [nq*hd]
    __half* k = nullptr;      // [nkv*hd]
    __half* v = nullptr;      // [nkv*hd]
    __half* mlp = nullptr;    // [inter]
    int8_t* act_q8 = nullptr; // [max(hidden, inter)]
    float* act_scale = nullptr;
    int32_t* act_sum8 = nullptr;
    int8_t* mlp_q8 = nullptr; // Q8_1 of the MLP activation when the gate_up launch writes it itself
    float* mlp_scale = nullptr;
    int32_t* mlp_sum8 = nullptr;
    // reductions published from launch to launch (W4A16_SWEEP_PUBLISH_*): [sumsq_attn: 8 doubles][amax: inter / 128 words]
    // contiguous (one clear range), then [sumsq_down: 8 doubles]
    double* sumsq_attn = nullptr;
    uint32_t* mlp_amax = nullptr;
    double* sumsq_down = nullptr;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    int launches = 0;
    // persistent form
    bool persistent = false;
    w4::PSweepArgs pargs{};
    uint32_t epoch = 0;
    uint32_t launch_count = 0;
    int sm_count = 0;
    uint8_t* exchange_begin = nullptr;   // tagged exchange buffers, status word and arrival counters: one range
    size_t exchange_bytes = 0;
};

namespace {

using namespace w4;

constexpr size_t kAlign = 256;
constexpr size_t kMaxPersistentLayers = 256;   // capacity of the persistent kernel's layer table in the workspace
size_t align_up(size_t v) { return (v + kAlign - 1) / kAlign * kAlign; }

struct Carve {
    size_t h, q, k, v, mlp, q8, scale, sum8, total;
    // persistent form: exchange buffers (8-byte tagged words), device copy of the layer table, status word
    size_t ll_h_attn, ll_h_down, ll_q, ll_mlp, layer_table, status, counters;
    size_t mlp_q8, mlp_scale, mlp_sum8;
    size_t pub_attn, pub_down;
};
Carve carve(int hidden, int inter, int nq, int nkv, int hd) {
    const size_t kmax = static_cast<size_t>(hidden > inter ? hidden : inter);
    const size_t qdim = static_cast<size_t>(nq) * hd, kvdim = static_cast<size_t>(nkv) * hd;
    Carve c{};
    size_t off = 0;
    c.h = off; off += align_up(hidden * sizeof(__half));
    c.q = off; off += align_up((qdim > static_cast<size_t>(hidden) ? qdim : hidden) * sizeof(__half));
    c.k = off; off += align_up(kvdim * sizeof(__half));
    c.v = off; off += align_up(kvdim * sizeof(__half));
    c.mlp = off; off += align_up(inter * sizeof(__half));
    c.q8 = off; off += align_up(kmax);
    c.scale = off; off += align_up(kmax / 128 * sizeof(float));
    c.sum8 = off; off += align_up(kmax / 8 * sizeof(int32_t));
    c.ll_h_attn = off; off += align_up(hidden / 2 * 8);
    c.ll_h_down = off; off += align_up(hidden / 2 * 8);
    c.ll_q = off; off += align_up(qdim / 2 * 8);
    c.ll_mlp = off; off += align_up(inter / 2 * 8);
    c.status = off; off += align_up(sizeof(int));
    c.counters = off; off += align_up(4 * kMaxPersistentLayers * 32);   // one 32-byte cell per projection
    c.layer_table = off; off += align_up(kMaxPersistentLayers * w4::psweep_layer_bytes());
    c.mlp_q8 = off; off += align_up(inter);
    c.mlp_scale = off; off += align_up(inter / 128 * sizeof(float));
    c.mlp_sum8 = off; off += align_up(inter / 8 * sizeof(int32_t));
    c.pub_attn = off; off += align_up(w4::kSumsqSlots * sizeof(double) + (inter / 128 + 1) * sizeof(uint32_t));
    c.pub_down = off; off += align_up(w4::kSumsqSlots * sizeof(double));
    c.total = off;
    return c;
}

// Issues the launches of one pass on `stream`; returns the first nonzero status.
int issue_pass(w4a16_sweep* s, cudaStream_t stream, int* launches) {
    const auto& d = s->desc;
    const int H = d.hidden_size, I = d.intermediate_size;
    const int qdim = d.num_q_heads * d.head_dim, kvdim = d.num_kv_heads * d.head_dim;
    int n = 0;
    const int flags = d.flags;
    const bool pub_sums = (flags & W4A16_SWEEP_PUBLISH_SUMSQ) != 0, pub_amax = (flags & W4A16_SWEEP_PUBLISH_AMAX) != 0;
    const bool publish = pub_sums || pub_amax;
    bool first = true;
    for (const auto& L : s->layers) {
        GemvArgs a = {};
        a.qweight[0] = static_cast<const uint32_t*>(L.q_weight); a.scales[0] = static_cast<const __half*>(L.q_scale);
        a.qweight[1] = static_cast<const uint32_t*>(L.k_weight); a.scales[1] = static_cast<const __half*>(L.k_scale);
        a.qweight[2] = static_cast<const uint32_t*>(L.v_weight); a.scales[2] = static_cast<const __half*>(L.v_scale);
        a.out[0] = s->q; a.out[1] = s->k; a.out[2] = s->v;
        a.rows[0] = qdim; a.rows[1] = kvdim; a.rows[2] = kvdim;
        a.K = H; a.units = qdim + 2 * kvdim;
        if (publish) {
            // takes the sum of squares the previous layer's down launch left (the first layer reduces itself);
            // clears what the O and gate_up launches of this layer will add to
            a.x_fp16 = s->h; a.gamma = static_cast<const __half*>(L.input_norm_gamma);
            a.sumsq_in = (first || !pub_sums) ? nullptr : s->sumsq_down;
            a.clear_words = reinterpret_cast<uint32_t*>(s->sumsq_attn);
            a.clear_count = 2 * kSumsqSlots + I / 128;
        } else if (flags & W4A16_SWEEP_FUSE_NORM) {
            a.x_fp16 = s->h; a.gamma = static_cast<const __half*>(L.input_norm_gamma);
        } else {
            if (int st = rmsnorm_q8_1(s->h, static_cast<const __half*>(L.input_norm_gamma), nullptr, s->act_q8,
                                      s->act_scale, s->act_sum8, H, stream))
                return st;
            ++n;
            a.q8 = s->act_q8; a.xscale = s->act_scale; a.sum8 = s->act_sum8;
        }
        if (int st = gemv_launch(kQkv, a, stream)) return st;
        ++n;
        // attention stand-in: the q projection plays the attention output
        GemvArgs o = {};
        o.qweight[0] = static_cast<const uint32_t*>(L.o_weight); o.scales[0] = static_cast<const __half*>(L.o_scale);
        o.out[0] = s->h; o.rows[0] = H; o.residual = s->h;
        o.K = qdim; o.units = H;
        if (pub_sums) o.sumsq_out = s->sumsq_attn;
        if (publish || (flags & W4A16_SWEEP_FUSE_QUANT_O)) {
            o.x_fp16 = s->q;
        } else {
            if (int st = quantize_fp16_to_q8_1(s->q, s->act_q8, s->act_scale, s->act_sum8, qdim, stream)) return st;
            ++n;
            o.q8 = s->act_q8; o.xscale = s->act_scale; o.sum8 = s->act_sum8;
        }
        if (int st = gemv_launch(kPlain, o, stream)) return st;
        ++n;
        GemvArgs g = {};
        g.qweight[0] = static_cast<const uint32_t*>(L.gate_up_weight);
        g.scales[0] = static_cast<const __half*>(L.gate_up_scale);
        g.out[0] = s->mlp; g.rows[0] = 2 * I;
        g.K = H; g.units = I;
        if (publish) {
            g.x_fp16 = s->h; g.gamma = static_cast<const __half*>(L.post_norm_gamma);
            if (pub_sums) g.sumsq_in = s->sumsq_attn;
            if (pub_amax) g.amax_out = s->mlp_amax;
            g.clear_words = reinterpret_cast<uint32_t*>(s->sumsq_down);
            g.clear_count = 2 * kSumsqSlots;
        } else if (flags & W4A16_SWEEP_FUSE_NORM) {
            g.x_fp16 = s->h; g.gamma = static_cast<const __half*>(L.post_norm_gamma);
        } else {
            if (int st = rmsnorm_q8_1(s->h, static_cast<const __half*>(L.post_norm_gamma), nullptr, s->act_q8,
                                      s->act_scale, s->act_sum8, H, stream))
                return st;
            ++n;
            g.q8 = s->act_q8; g.xscale = s->act_scale; g.sum8 = s->act_sum8;
        }
        const bool quant_in_gate_up = !publish && (flags & W4A16_SWEEP_QUANT_IN_GATE_UP) != 0;
        if (quant_in_gate_up) { g.q8_out = s->mlp_q8; g.xscale_out = s->mlp_scale; g.sum8_out = s->mlp_sum8; }
        if (int st = gemv_launch(kSwiglu, g, stream)) return st;
        ++n;
        GemvArgs dn = {};
        dn.qweight[0] = static_cast<const uint32_t*>(L.down_weight);
        dn.scales[0] = static_cast<const __half*>(L.down_scale);
        dn.out[0] = s->h; dn.rows[0] = H; dn.residual = s->h;
        dn.K = I; dn.units = H;
        if (pub_sums) dn.sumsq_out = s->sumsq_down;
        if (pub_amax) {
            dn.x_fp16 = s->mlp; dn.amax_in = s->mlp_amax;
        } else if (quant_in_gate_up) {
            dn.q8 = s->mlp_q8; dn.xscale = s->mlp_scale; dn.sum8 = s->mlp_sum8;
        } else if (flags & W4A16_SWEEP_FUSE_QUANT_DOWN) {
            dn.x_fp16 = s->mlp;
        } else {
            if (int st = quantize_fp16_to_q8_1(s->mlp, s->act_q8, s->act_scale, s->act_sum8, I, stream)) return st;
            ++n;
            dn.q8 = s->act_q8; dn.xscale = s->act_scale; dn.sum8 = s->act_sum8;
        }
        if (int st = gemv_launch(kPlain, dn, stream)) return st;
        ++n;
        first = false;
    }
    if (launches) *launches = n;
    return 0;
}

// One pass over the resident hidden state: graph replay, or the persistent kernel with fresh tags.
int run_pass(w4a16_sweep* s, cudaStream_t stream) {
    if (!s->persistent) return static_cast<int>(cudaGraphLaunch(s->exec, stream));
    s->pargs.epoch = s->epoch;
    s->pargs.counter_target = ++s->launch_count * static_cast<uint32_t>(s->sm_count);
    s->epoch += 4u * static_cast<uint32_t>(s->desc.num_layers);
    return w4::psweep_launch(s->pargs, s->sm_count, stream);
}

}  // namespace

extern "C" {

int64_t w4a16_sweep_workspace_bytes(int hidden_size, int intermediate_size, int num_q_heads, int num_kv_heads,
                                    int head_dim) {
    if (hidden_size <= 0 || intermediate_size <= 0 || num_q_heads <= 0 || num_kv_heads <= 0 || head_dim <= 0)
        return W4A16_ERR_INVALID_ARG;
    return static_cast<int64_t>(carve(hidden_size, intermediate_size, num_q_heads, num_kv_heads, head_dim).total);
}

int w4a16_sweep_create(const w4a16_sweep_desc* desc, w4a16_stream_t stream_, w4a16_sweep** out) {
    if (!desc || !out || !desc->layers || !desc->workspace || desc->num_layers <= 0) return W4A16_ERR_INVALID_ARG;
    const int H = desc->hidden_size, I = desc->intermediate_size;
    const int qdim = desc->num_q_heads * desc->head_dim;
    if (H <= 0 || I <= 0 || qdim <= 0 || desc->num_kv_heads <= 0) return W4A16_ERR_INVALID_ARG;
    if (H % 256 || I % 256 || qdim % 256) return W4A16_ERR_SHAPE;
    if (reinterpret_cast<uintptr_t>(desc->workspace) % kAlign) return W4A16_ERR_ALIGNMENT;
    for (int l = 0; l < desc->num_layers; ++l) {
        const w4a16_layer_weights& L = desc->layers[l];
        const void* ptrs[] = {L.input_norm_gamma, L.q_weight, L.q_scale, L.k_weight, L.k_scale, L.v_weight, L.v_scale,
                              L.o_weight, L.o_scale, L.post_norm_gamma, L.gate_up_weight, L.gate_up_scale,
                              L.down_weight, L.down_scale};
        for (const void* p : ptrs)
            if (!p) return W4A16_ERR_INVALID_ARG;
    }
    if (int st = w4::ensure_device_ready(nullptr)) return st;

    std::unique_ptr<w4a16_sweep> s(new (std::nothrow) w4a16_sweep);
    if (!s) return static_cast<int>(cudaErrorMemoryAllocation);
    s->desc = *desc;
    s->layers.assign(desc->layers, desc->layers + desc->num_layers);
    s->desc.layers = s->layers.data();
    const Carve c = carve(H, I, desc->num_q_heads, desc->num_kv_heads, desc->head_dim);
    uint8_t* base = static_cast<uint8_t*>(desc->workspace);
    s->h = reinterpret_cast<__half*>(base + c.h);
    s->q = reinterpret_cast<__half*>(base + c.q);
    s->k = reinterpret_cast<__half*>(base + c.k);
    s->v = reinterpret_cast<__half*>(base + c.v);
    s->mlp = reinterpret_cast<__half*>(base + c.mlp);
    s->act_q8 = reinterpret_cast<int8_t*>(base + c.q8);
    s->act_scale = reinterpret_cast<float*>(base + c.scale);
    s->act_sum8 = reinterpret_cast<int32_t*>(base + c.sum8);
    s->mlp_q8 = reinterpret_cast<int8_t*>(base + c.mlp_q8);
    s->mlp_scale = reinterpret_cast<float*>(base + c.mlp_scale);
    s->mlp_sum8 = reinterpret_cast<int32_t*>(base + c.mlp_sum8);
    s->sumsq_attn = reinterpret_cast<double*>(base + c.pub_attn);
    s->mlp_amax = reinterpret_cast<uint32_t*>(base + c.pub_attn + w4::kSumsqSlots * sizeof(double));
    s->sumsq_down = reinterpret_cast<double*>(base + c.pub_down);
    if ((desc->flags & (W4A16_SWEEP_PUBLISH_SUMSQ | W4A16_SWEEP_PUBLISH_AMAX)) && (I % 128 || 2 * w4::kSumsqSlots + I / 128 > 128)) return W4A16_ERR_SHAPE;
    if ((desc->flags & W4A16_SWEEP_QUANT_IN_GATE_UP) && I % 128) return W4A16_ERR_SHAPE;

    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    cudaError_t e = cudaMemsetAsync(s->h, 0, H * sizeof(__half), stream);
    if (e != cudaSuccess) return static_cast<int>(e);

    if (desc->flags & W4A16_SWEEP_PERSISTENT) {
        const int kvdim = desc->num_kv_heads * desc->head_dim;
        if (!w4::psweep_supported(H, I, qdim, kvdim) || static_cast<size_t>(desc->num_layers) > kMaxPersistentLayers)
            return W4A16_ERR_SHAPE;
        for (const auto& L : s->layers) {
            const void* w16[] = {L.q_weight, L.k_weight, L.v_weight, L.o_weight, L.gate_up_weight, L.down_weight};
            const void* s4[] = {L.q_scale, L.k_scale, L.v_scale, L.o_scale, L.gate_up_scale, L.down_scale};
            for (const void* p : w16)
                if (reinterpret_cast<uintptr_t>(p) % 16) return W4A16_ERR_ALIGNMENT;   // bulk copies
            for (const void* p : s4)
                if (reinterpret_cast<uintptr_t>(p) % 4) return W4A16_ERR_ALIGNMENT;    // 4-byte async copies
            if (reinterpret_cast<uintptr_t>(L.input_norm_gamma) % 16 || reinterpret_cast<uintptr_t>(L.post_norm_gamma) % 16)
                return W4A16_ERR_ALIGNMENT;
        }
        const w4::DeviceInfo* dev = nullptr;
        if (int st = w4::ensure_device_ready(&dev)) return st;
        if (int st = w4::psweep_set_attributes()) return st;
        std::vector<uint8_t> table(s->layers.size() * w4::psweep_layer_bytes());
        for (size_t l = 0; l < s->layers.size(); ++l)
            w4::psweep_fill_layer(table.data() + l * w4::psweep_layer_bytes(), s->layers[l]);
        uint8_t* d_table = base + c.layer_table;
        if ((e = cudaMemcpyAsync(d_table, table.data(), table.size(), cudaMemcpyHostToDevice, stream)) != cudaSuccess)
            return static_cast<int>(e);
        // tags start above zero, so zeroed exchange buffers never look published
        s->exchange_begin = base + c.ll_h_attn;
        s->exchange_bytes = c.layer_table - c.ll_h_attn;
        if ((e = cudaMemsetAsync(s->exchange_begin, 0, s->exchange_bytes, stream)) != cudaSuccess)
            return static_cast<int>(e);
        if ((e = cudaStreamSynchronize(stream)) != cudaSuccess) return static_cast<int>(e);   // `table` is a local
        s->persistent = true;
        s->sm_count = dev->sm_count;
        w4::PSweepArgs& a = s->pargs;
        a.layers = d_table;
        a.num_layers = desc->num_layers; a.H = H; a.I = I; a.qdim = qdim; a.kvdim = kvdim;
        a.h_in = s->h; a.h_out = s->h;
        a.ll_h_attn = reinterpret_cast<uint2*>(base + c.ll_h_attn);
        a.ll_h_down = reinterpret_cast<uint2*>(base + c.ll_h_down);
        a.ll_q = reinterpret_cast<uint2*>(base + c.ll_q);
        a.ll_mlp = reinterpret_cast<uint2*>(base + c.ll_mlp);
        a.k_out = s->k; a.v_out = s->v;
        a.status = reinterpret_cast<int*>(base + c.status);
        a.counters = reinterpret_cast<uint32_t*>(base + c.counters);
        s->launches = 1;
        // one eager pass: validates the launch
        a.epoch = s->epoch;
        a.counter_target = ++s->launch_count * static_cast<uint32_t>(s->sm_count);
        if (int st = w4::psweep_launch(a, s->sm_count, stream)) return st;
        s->epoch += 4u * static_cast<uint32_t>(desc->num_layers);
        if ((e = cudaStreamSynchronize(stream)) != cudaSuccess) return static_cast<int>(e);
        *out = s.release();
        return 0;
    }
    // one eager pass (sets kernel attributes, validates the launches), then capture
    if (int st = issue_pass(s.get(), stream, &s->launches)) return st;
    if ((e = cudaStreamSynchronize(stream)) != cudaSuccess) return static_cast<int>(e);
    // capture on a stream of our own: the caller's may be the legacy default stream, which cannot capture
    cudaStream_t cap = nullptr;
    if ((e = cudaStreamCreateWithFlags(&cap, cudaStreamNonBlocking)) != cudaSuccess) return static_cast<int>(e);
    if ((e = cudaStreamBeginCapture(cap, cudaStreamCaptureModeThreadLocal)) != cudaSuccess) {
        cudaStreamDestroy(cap);
        return static_cast<int>(e);
    }
    const int st = issue_pass(s.get(), cap, nullptr);
    e = cudaStreamEndCapture(cap, &s->graph);
    cudaStreamDestroy(cap);
    if (st) {
        if (s->graph) cudaGraphDestroy(s->graph);
        return st;
    }
    if (e != cudaSuccess) return static_cast<int>(e);
    if ((e = cudaGraphInstantiate(&s->exec, s->graph, 0)) != cudaSuccess) {
        cudaGraphDestroy(s->graph);
        return static_cast<int>(e);
    }
    *out = s.release();
    return 0;
}

int w4a16_sweep_destroy(w4a16_sweep* s) {
    if (!s) return 0;
    if (s->exec) cudaGraphExecDestroy(s->exec);
    if (s->graph) cudaGraphDestroy(s->graph);
    delete s;
    return 0;
}

int w4a16_sweep_launches(const w4a16_sweep* s) { return s ? s->launches : W4A16_ERR_INVALID_ARG; }

int w4a16_sweep_run_device(w4a16_sweep* s, const void* d_h_in, void* d_h_out, w4a16_stream_t stream_) {
    if (!s || !d_h_in || !d_h_out) return W4A16_ERR_INVALID_ARG;
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    const size_t bytes = s->desc.hidden_size * sizeof(__half);
    cudaError_t e = cudaMemcpyAsync(s->h, d_h_in, bytes, cudaMemcpyDeviceToDevice, stream);
    if (e == cudaSuccess) e = static_cast<cudaError_t>(run_pass(s, stream));
    if (e == cudaSuccess) e = cudaMemcpyAsync(d_h_out, s->h, bytes, cudaMemcpyDeviceToDevice, stream);
    return static_cast<int>(e);
}

int w4a16_sweep_run_host(w4a16_sweep* s, const void* h_h_in, void* h_h_out, w4a16_stream_t stream_) {
    if (!s || !h_h_in || !h_h_out) return W4A16_ERR_INVALID_ARG;
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    const size_t bytes = s->desc.hidden_size * sizeof(__half);
    cudaError_t e = cudaMemcpyAsync(s->h, h_h_in, bytes, cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess) e = static_cast<cudaError_t>(run_pass(s, stream));
    if (e == cudaSuccess) e = cudaMemcpyAsync(h_h_out, s->h, bytes, cudaMemcpyDeviceToHost, stream);
    return static_cast<int>(e);
}

int w4a16_sweep_status(w4a16_sweep* s, int* out) {
    if (!s || !out) return W4A16_ERR_INVALID_ARG;
    *out = 0;
    if (!s->persistent) return 0;
    cudaError_t e = cudaMemcpy(out, s->pargs.status, sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess || *out == 0) return static_cast<int>(e);
    // A bounded wait ran out: the CTAs left early, so the arrival counters are short for ever and every later
    // launch would run into its own bounds.  Start over: nothing of the pass is in flight once the device is
    // idle; clear tags, counters and status and count launches and tags from zero again.
    if ((e = cudaDeviceSynchronize()) != cudaSuccess) return static_cast<int>(e);
    if ((e = cudaMemset(s->exchange_begin, 0, s->exchange_bytes)) != cudaSuccess) return static_cast<int>(e);
    s->launch_count = 0;
    s->epoch = 0;
    return 0;
}

void* w4a16_sweep_buffer(const w4a16_sweep* s, int which) {
    if (!s) return nullptr;
    switch (which) {
        case 0: return s->h;
        case 1: return s->q;
        case 2: return s->k;
        case 3: return s->v;
        case 4: return s->mlp;
        default: return nullptr;
    }
}

}  // extern "C"
