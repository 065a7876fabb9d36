// Reader of the reference's `.qwenbin` weight container (host code only): header and layer table are checked
// and turned into the tensor addresses the projection path needs -- the layer table of the decode sweep, the
// embedding / lm_head matrix and the final norm -- relative to wherever the caller placed the file's bytes
// (the reference uploads the file as it is into its arena and adds offsets, src/engine.cu:85-348).
//
// Formats (reference include/config.cuh:75-97 and :107-170, docs/SPECIFICATION.md, tools/export_qwen25.py):
//   v1  QWQwenHeader: 12 x uint32 {magic, 1, quant_mode, vocab, hidden, inter, layers, q heads, kv heads,
//       head_dim, group size, 0}, 3 x uint64 {embed weight, embed scale, final norm}, then per layer 17 x uint64
//       in the order of LayerTensorIdx (norm1, q w/s/b, k w/s/b, v w/s/b, o w/s, norm2, gate_up w/s, down w/s).
//   v2  QwenBinHeaderV2: 12 x uint32 {magic, 2, hidden, inter, layers, q heads, kv heads, head_dim, vocab,
//       max_seq_len, quant_type, tie}, 2 x float {eps, rope theta}, 2 x uint32, 11 x uint64 {layer table, embed,
//       final norm, lm_head, weights, embed scales, lm_head scales, 4 reserved}; layer table = per layer
//       2 x uint32 + 26 x uint64 (slots named below).
// All little-endian; every tensor starts on a 256-byte boundary.
#include <cstring>

#include "w4a16_internal.hpp"

namespace {

constexpr uint32_t kMagic = 0x5157454Eu;   // "QWEN"

struct Reader {
    const uint8_t* p;
    uint64_t n;
    bool ok = true;
    uint32_t u32(uint64_t off) {
        uint32_t v = 0;
        if (off + 4 > n) { ok = false; return 0; }
        std::memcpy(&v, p + off, 4);
        return v;
    }
    uint64_t u64(uint64_t off) {
        uint64_t v = 0;
        if (off + 8 > n) { ok = false; return 0; }
        std::memcpy(&v, p + off, 8);
        return v;
    }
    float f32(uint64_t off) {
        float v = 0;
        if (off + 4 > n) { ok = false; return 0; }
        std::memcpy(&v, p + off, 4);
        return v;
    }
};

struct Parsed {
    w4a16_qwenbin_header h{};
    uint64_t embed_w = 0, embed_s = 0, final_norm = 0, lm_head_w = 0, lm_head_s = 0;
    uint64_t layer_table = 0;   // v2: descriptors; v1: the offset array inside the header
};

// One tensor of `bytes` bytes at `off`: inside the file, 256-byte aligned, not overlapping the header.
bool tensor_ok(uint64_t off, uint64_t bytes, uint64_t n) { return off >= 4096 && off % 256 == 0 && off <= n && bytes <= n - off; }

int parse(const void* file_bytes, uint64_t nbytes, Parsed* out) {
    if (!file_bytes || nbytes < 4096) return W4A16_ERR_INVALID_ARG;
    Reader r{static_cast<const uint8_t*>(file_bytes), nbytes};
    if (r.u32(0) != kMagic) return W4A16_ERR_INVALID_ARG;
    const uint32_t version = r.u32(4);
    w4a16_qwenbin_header& h = out->h;
    h.version = version;
    if (version == 1) {
        h.quant_type = r.u32(8); h.vocab_size = r.u32(12); h.hidden_size = r.u32(16); h.intermediate_size = r.u32(20);
        h.num_layers = r.u32(24); h.num_q_heads = r.u32(28); h.num_kv_heads = r.u32(32); h.head_dim = r.u32(36);
        if (r.u32(40) != 128) return W4A16_ERR_SHAPE;   // quantisation group size
        h.max_seq_len = 0; h.tie_word_embeddings = 1; h.rms_norm_eps = 1e-6f; h.rope_theta = 1000000.0f;
        out->embed_w = r.u64(48); out->embed_s = r.u64(56); out->final_norm = r.u64(64);
        out->lm_head_w = out->embed_w; out->lm_head_s = out->embed_s;
        out->layer_table = 72;
        if (72 + static_cast<uint64_t>(h.num_layers) * 17 * 8 > 4096) return W4A16_ERR_SHAPE;   // the table lives in the header
    } else if (version == 2) {
        h.hidden_size = r.u32(8); h.intermediate_size = r.u32(12); h.num_layers = r.u32(16); h.num_q_heads = r.u32(20);
        h.num_kv_heads = r.u32(24); h.head_dim = r.u32(28); h.vocab_size = r.u32(32); h.max_seq_len = r.u32(36);
        h.quant_type = r.u32(40); h.tie_word_embeddings = r.u32(44); h.rms_norm_eps = r.f32(48); h.rope_theta = r.f32(52);
        out->layer_table = r.u64(64); out->embed_w = r.u64(72); out->final_norm = r.u64(80);
        out->lm_head_w = r.u64(88); out->embed_s = r.u64(104); out->lm_head_s = r.u64(112);
        if (h.tie_word_embeddings || out->lm_head_w == 0 || out->lm_head_w == out->embed_w) {
            out->lm_head_w = out->embed_w; out->lm_head_s = out->embed_s;
        } else if (out->lm_head_s == 0) {
            return W4A16_ERR_INVALID_ARG;   // an untied lm_head needs its own scales
        }
        if (out->layer_table % 8 || out->layer_table > nbytes ||
            static_cast<uint64_t>(h.num_layers) * 216 > nbytes - out->layer_table)
            return W4A16_ERR_INVALID_ARG;
    } else {
        return W4A16_ERR_INVALID_ARG;
    }
    if (!r.ok) return W4A16_ERR_INVALID_ARG;
    if (h.quant_type != 1) return W4A16_ERR_SHAPE;   // W4A16 group 128 only
    if (h.num_layers == 0 || h.num_layers > 4096 || h.hidden_size == 0 || h.hidden_size % 256 || h.intermediate_size == 0 ||
        h.intermediate_size % 256 || h.num_q_heads == 0 || h.num_kv_heads == 0 || h.head_dim == 0 || h.vocab_size == 0 ||
        (static_cast<uint64_t>(h.num_q_heads) * h.head_dim) % 256)
        return W4A16_ERR_SHAPE;
    h.file_bytes = nbytes;
    return 0;
}

uint64_t wbytes(uint64_t rows, uint64_t k) { return rows * k / 2; }
uint64_t sbytes(uint64_t rows, uint64_t k) { return rows * (k / 128) * 2; }

}  // namespace

extern "C" {

int w4a16_qwenbin_parse(const void* file_bytes, uint64_t nbytes, w4a16_qwenbin_header* header) {
    if (!header) return W4A16_ERR_INVALID_ARG;
    Parsed p;
    if (int st = parse(file_bytes, nbytes, &p)) return st;
    *header = p.h;
    return 0;
}

int w4a16_qwenbin_tensors(const void* file_bytes, uint64_t nbytes, const void* base, w4a16_layer_weights* layers,
                          int max_layers, w4a16_qwenbin_globals* globals, w4a16_qwenbin_biases* biases) {
    Parsed p;
    if (int st = parse(file_bytes, nbytes, &p)) return st;
    const w4a16_qwenbin_header& h = p.h;
    if (!base || !layers || max_layers < static_cast<int>(h.num_layers)) return W4A16_ERR_INVALID_ARG;
    if (reinterpret_cast<uintptr_t>(base) % 256) return W4A16_ERR_ALIGNMENT;   // keeps the tensors' 256-byte alignment
    const uint64_t H = h.hidden_size, I = h.intermediate_size, V = h.vocab_size;
    const uint64_t qdim = static_cast<uint64_t>(h.num_q_heads) * h.head_dim, kvdim = static_cast<uint64_t>(h.num_kv_heads) * h.head_dim;
    const uint8_t* b = static_cast<const uint8_t*>(base);
    bool ok = true;
    auto at = [&](uint64_t off, uint64_t bytes) -> const void* {
        if (!tensor_ok(off, bytes, nbytes)) { ok = false; return nullptr; }
        return b + off;
    };
    Reader r{static_cast<const uint8_t*>(file_bytes), nbytes};
    for (uint32_t l = 0; l < h.num_layers; ++l) {
        uint64_t norm1, norm2, qw, qs, qb, kw, ks, kb, vw, vs, vb, ow, os, guw, gus, dw, ds;
        if (h.version == 1) {
            const uint64_t t = p.layer_table + static_cast<uint64_t>(l) * 17 * 8;
            norm1 = r.u64(t); qw = r.u64(t + 8); qs = r.u64(t + 16); qb = r.u64(t + 24); kw = r.u64(t + 32); ks = r.u64(t + 40);
            kb = r.u64(t + 48); vw = r.u64(t + 56); vs = r.u64(t + 64); vb = r.u64(t + 72); ow = r.u64(t + 80); os = r.u64(t + 88);
            norm2 = r.u64(t + 96); guw = r.u64(t + 104); gus = r.u64(t + 112); dw = r.u64(t + 120); ds = r.u64(t + 128);
        } else {
            const uint64_t t = p.layer_table + static_cast<uint64_t>(l) * 216;
            if (r.u32(t) != 0) return W4A16_ERR_SHAPE;   // LAYER_GQA only
            auto slot = [&](int i) { return r.u64(t + 8 + 8ull * i); };   // 26 slots after the two uint32
            norm1 = slot(0); norm2 = slot(1); qw = slot(2); qb = slot(3); kb = slot(4); vb = slot(5); ow = slot(6);
            guw = slot(12); dw = slot(14); kw = slot(17); vw = slot(18); qs = slot(19); ks = slot(20); vs = slot(21);
            os = slot(22); gus = slot(23); ds = slot(25);
            if (slot(13) != guw || slot(24) != gus) return W4A16_ERR_SHAPE;   // gate and up are one interleaved matrix
        }
        w4a16_layer_weights& L = layers[l];
        L.input_norm_gamma = at(norm1, H * 2);
        L.q_weight = at(qw, wbytes(qdim, H)); L.q_scale = at(qs, sbytes(qdim, H));
        L.k_weight = at(kw, wbytes(kvdim, H)); L.k_scale = at(ks, sbytes(kvdim, H));
        L.v_weight = at(vw, wbytes(kvdim, H)); L.v_scale = at(vs, sbytes(kvdim, H));
        L.o_weight = at(ow, wbytes(H, qdim)); L.o_scale = at(os, sbytes(H, qdim));
        L.post_norm_gamma = at(norm2, H * 2);
        L.gate_up_weight = at(guw, wbytes(2 * I, H)); L.gate_up_scale = at(gus, sbytes(2 * I, H));
        L.down_weight = at(dw, wbytes(H, I)); L.down_scale = at(ds, sbytes(H, I));
        if (biases) {
            biases[l].q_bias = at(qb, qdim * 2);
            biases[l].k_bias = at(kb, kvdim * 2);
            biases[l].v_bias = at(vb, kvdim * 2);
        }
        if (!r.ok || !ok) return W4A16_ERR_INVALID_ARG;
    }
    if (globals) {
        globals->embed_weight = at(p.embed_w, wbytes(V, H));
        globals->embed_scale = at(p.embed_s, sbytes(V, H));
        globals->final_norm_gamma = at(p.final_norm, H * 2);
        globals->lm_head_weight = at(p.lm_head_w, wbytes(V, H));
        globals->lm_head_scale = at(p.lm_head_s, sbytes(V, H));
        if (!ok) return W4A16_ERR_INVALID_ARG;
    }
    return 0;
}

}  // extern "C"
