// The decode projection sweep as ONE persistent kernel (one CTA per SM, all resident).
//
// Why.  A chain of per-projection kernels is bound by what happens between two dependent launches:
// on B200 even an empty kernel costs ~1 us in a CUDA graph, and each projection adds the DRAM
// latency of its first weight bytes, while the data it waits for is a 3 KB vector.  Weights do not
// depend on activations, so here a producer warp per CTA streams the CTA's share of EVERY
// projection of EVERY layer into a shared-memory ring with bulk copies, as fast as the ring
// drains, and the 8 consumer warps only ever wait for the small activation vector of the next
// projection.
//
// Exchange between CTAs.  The output of a projection is needed in full by every CTA for the next
// one.  Outputs are published as 8-byte words {two fp16 values, 32-bit tag}; an aligned 8-byte
// store / load is single-copy atomic, so a reader can tell for every word on its own whether it is
// the value of this projection: no fence is needed between the data and any flag.  To keep 38 000
// threads from hammering the same few cache lines while they wait, only ONE thread per CTA polls a
// per-projection arrival counter (a relaxed add by each publishing CTA); when it shows all CTAs,
// every thread reads its words once and re-reads the rare word whose tag is still old.  Tags and
// counters only ever grow, across launches too (their bases are kernel arguments), so nothing is
// ever cleared.  A buffer written
// by projection t is read by all CTAs in projection t+1 and rewritten in projection t+4; a CTA can
// reach t+4 only after every CTA has published t+3, i.e. has finished reading t.
//
// Arithmetic is that of the per-projection kernels (same quantiser, same dp4a core, fp32 tail);
// the reference order of launches is src/engine.cu:361-451, with the q projection standing in
// for the attention output.
//
// Every wait (ring barriers, tag polls) is bounded; on expiry the CTA records a status code,
// leaves, and the remaining CTAs run into their own bounds.
#include <algorithm>

#include "w4a16_common.cuh"
#include "w4a16_internal.hpp"

namespace w4 {
namespace {

constexpr int kConsumerWarps = 15;   // + 1 producer warp = 512 threads, which leaves 128 registers per thread
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kBlockThreads = kConsumerThreads + 32;    // + one producer warp
constexpr int kSlotBytes = 18432;      // weights of one ring slot: 24 rows at K=1536, 4 rows at K=8960
constexpr int kSlotScaleBytes = 640;   // their scales (<= kSlotBytes / 32 = 576)
constexpr int kSlotStride = kSlotBytes + kSlotScaleBytes;
constexpr int kSlots = 10;
constexpr int kMaxK = 9216;            // longest activation vector (in_features) the staging holds
constexpr int kMaxHidden = 4096;       // longest residual-stream vector
constexpr int kMaxRowWarps = 4;          // a weight row is spread over at most 4 warps (128 lanes)
constexpr unsigned kPollLimit = 1u << 22;
constexpr int kPartFloats = 64 * kMaxRowWarps;   // up to 64 rows per chunk
constexpr float kEps = 1e-6f;          // reference include/config.cuh:20

// Pointers of one layer, device copy.  Tensor order: q, k, v, o, gate_up, down.
struct LayerDev {
    const uint8_t* w[6];
    const __half* sc[6];
    const __half* gamma_in;
    const __half* gamma_post;
};

}  // namespace

namespace {

// ---- PTX helpers ----------------------------------------------------------------------------
__device__ __forceinline__ uint32_t s32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void bar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void bar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void bar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool bar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool bar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool bar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    if (bar_test_wait(bar, parity)) return true;   // the common case (data already there) without parking the thread
    for (unsigned it = 0; it < kPollLimit; ++it) {
        if (bar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (it > 1024) __nanosleep(64);
    }
    *abort_flag = 1;
    return false;
}
// 1-D bulk copy global -> shared, completion counted in bytes on an mbarrier.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async_4(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
// Arrive on the mbarrier once all cp.async issued so far by this thread have landed.
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint2 ld_ll(const uint2* p) {
    uint2 v;
    asm volatile("ld.relaxed.gpu.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_ll(uint2* p, uint32_t data, uint32_t tag) {
    asm volatile("st.relaxed.gpu.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(data), "r"(tag) : "memory");
}
__device__ __forceinline__ uint32_t ld_counter(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void add_counter(uint32_t* p) {
    asm volatile("red.relaxed.gpu.global.add.u32 [%0], 1;" ::"l"(p) : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory"); }

// ---- the static schedule, shared by producer and consumers --------------------------------------
// A stage is one projection of one layer.  Outputs are handed out in PAIRS (an 8-byte word of the
// exchange format); a pair costs 2 weight rows (4 for gate_up: two gate/up row pairs).
struct StagePlan {
    int kind;            // 0 QKV, 1 O, 2 GATE_UP, 3 DOWN
    int K;               // in_features
    int row_bytes;       // K / 2
    int groups;          // K / 128
    int rows_per_pair;   // weight rows per output pair
    int first_row;       // first (virtual) weight row of this CTA
    int num_rows;        // weight rows of this CTA
    int first_pair;      // first output pair of this CTA
    int num_pairs;
    int chunk_rows;      // weight rows per ring slot
};

__device__ __forceinline__ StagePlan make_plan(const PSweepArgs& a, int stage, int cta, int nctas) {
    StagePlan p;
    p.kind = stage & 3;
    int pairs;
    switch (p.kind) {
        case 0: p.K = a.H; pairs = (a.qdim + 2 * a.kvdim) / 2; p.rows_per_pair = 2; break;
        case 1: p.K = a.qdim; pairs = a.H / 2; p.rows_per_pair = 2; break;
        case 2: p.K = a.H; pairs = a.I / 2; p.rows_per_pair = 4; break;
        default: p.K = a.I; pairs = a.H / 2; p.rows_per_pair = 2; break;
    }
    p.row_bytes = p.K / 2;
    p.groups = p.K / kGroup;
    const int base = pairs / nctas, rem = pairs - base * nctas;
    p.first_pair = cta * base + min(cta, rem);
    p.num_pairs = base + (cta < rem ? 1 : 0);
    p.first_row = p.first_pair * p.rows_per_pair;
    p.num_rows = p.num_pairs * p.rows_per_pair;
    p.chunk_rows = (kSlotBytes / p.row_bytes) & ~3;
    return p;
}

// Tensor (index into LayerDev) and local row of a virtual row of the stage.
__device__ __forceinline__ void locate_row(const PSweepArgs& a, int kind, int vrow, int* tensor, int* local,
                                           int* rows_left_in_tensor) {
    if (kind == 0) {
        if (vrow < a.qdim) { *tensor = 0; *local = vrow; *rows_left_in_tensor = a.qdim - vrow; }
        else if (vrow < a.qdim + a.kvdim) { *tensor = 1; *local = vrow - a.qdim; *rows_left_in_tensor = a.kvdim - *local; }
        else { *tensor = 2; *local = vrow - a.qdim - a.kvdim; *rows_left_in_tensor = a.kvdim - *local; }
    } else {
        *tensor = kind + 2;   // 1 -> o (3), 2 -> gate_up (4), 3 -> down (5)
        *local = vrow;
        *rows_left_in_tensor = 1 << 30;
    }
}

// ---- producer warp ------------------------------------------------------------------------------
__device__ void producer_loop(const PSweepArgs& a, uint8_t* ring, uint32_t full0, uint32_t empty0,
                              volatile int* s_abort, int lane) {
    const int cta = blockIdx.x, nctas = gridDim.x;
    int slot = 0, issued = 0;
    uint32_t phase = 0;
    const int num_stages = a.num_layers * 4;
    for (int st = 0; st < num_stages; ++st) {
        const StagePlan p = make_plan(a, st, cta, nctas);
        const LayerDev& L = static_cast<const LayerDev*>(a.layers)[st >> 2];
        for (int r = 0; r < p.num_rows; r += p.chunk_rows) {
            const int rows = min(p.chunk_rows, p.num_rows - r);
            int ok = 1;
            if (lane == 0) ok = bar_wait(empty0 + 8u * slot, phase ^ 1, s_abort) ? 1 : 0;
            ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
            if (!ok) {
                // Leaving early: a CTA must not exit while bulk copies into its shared memory are in flight.  The
                // latest fill of every slot (at most kSlots of them) is waited for, each wait bounded.
                asm volatile("cp.async.wait_all;" ::: "memory");
                if (lane == 0) {
                    for (int k = 0; k < min(issued, kSlots); ++k) {
                        const int j = (slot - 1 - k + 2 * kSlots) % kSlots;
                        const uint32_t ph = j < slot ? phase : phase ^ 1u;
                        for (unsigned it = 0; it < kPollLimit; ++it)
                            if (bar_try_wait(full0 + 8u * j, ph)) break;
                    }
                }
                __syncwarp();
                return;
            }
            const uint32_t full = full0 + 8u * slot;
            uint8_t* dst_w = ring + slot * kSlotStride;
            uint8_t* dst_s = dst_w + kSlotBytes;
            if (lane == 0) bar_arrive_expect_tx(full, static_cast<uint32_t>(rows * p.row_bytes));
            // the rows may cross from q into k into v: one bulk copy per tensor segment
            int done = 0;
            while (done < rows) {
                int t, local, left;
                locate_row(a, p.kind, p.first_row + r + done, &t, &local, &left);
                const int seg = min(rows - done, left);
                if (lane == 0)
                    bulk_g2s(s32(dst_w + done * p.row_bytes), L.w[t] + static_cast<size_t>(local) * p.row_bytes,
                             static_cast<uint32_t>(seg * p.row_bytes), full);
                // scales of the segment: seg * groups halves, contiguous, 4-byte aligned
                const uint32_t* src_s = reinterpret_cast<const uint32_t*>(L.sc[t] + static_cast<size_t>(local) * p.groups);
                const int words = seg * p.groups / 2;
                const uint32_t dst_s32 = s32(dst_s + done * p.groups * 2);
                for (int i = lane; i < words; i += 32) cp_async_4(dst_s32 + 4u * i, src_s + i);
                done += seg;
            }
            cp_async_arrive_noinc(full);   // every lane: its scale copies count towards this slot
            ++issued;
            if (++slot == kSlots) { slot = 0; phase ^= 1; }
        }
    }
}

// ---- consumer side --------------------------------------------------------------------------------

// Reads `count` tagged words (word i of this thread sits at index idx(i)) until all carry `tag`;
// data[i] receives their payloads.  The arrival counter has normally been seen before, so the first
// read succeeds; a word whose store is still in flight is read again.  False on time-out / abort.
template <int MAXW, typename IdxFn>
__device__ __forceinline__ bool poll_words(const uint2* base, IdxFn idx, int count, uint32_t tag, uint32_t (&data)[MAXW],
                                           volatile int* s_abort, int* status, unsigned limit) {
    uint32_t tags[MAXW];
#pragma unroll
    for (int i = 0; i < MAXW; ++i) {
        if (i < count) {
            const uint2 v = ld_ll(base + idx(i));
            data[i] = v.x;
            tags[i] = v.y;
        } else {
            data[i] = 0;
            tags[i] = tag;
        }
    }
    for (unsigned it = 0; it < limit; ++it) {
        bool all = true;
#pragma unroll
        for (int i = 0; i < MAXW; ++i) {
            if (tags[i] != tag) {
                const uint2 v = ld_ll(base + idx(i));
                data[i] = v.x;
                tags[i] = v.y;
                all = all && (v.y == tag);
            }
        }
        if (all) return true;
        if (*s_abort) return false;
        if (it > 4096) __nanosleep(100);
    }
    *s_abort = 1;
    atomicExch(status, 2);
    return false;
}

struct ConsumerSmem {
    int8_t* q8;        // [kMaxK]
    int32_t* seed;     // [kMaxK / 32]
    float* xscale;     // [kMaxK / 128]
    __half* h;         // residual stream [kMaxHidden]
    __half* out;       // outputs of this CTA for the current stage [512]
    float* part;       // [2][kPartFloats] per-warp partial sums of rows, double-buffered by chunk parity
    double* red;       // [kConsumerWarps]
    float* inv;        // [1]
};

// Half-warp form of the group quantiser: 16 lanes per group of 128, lane owns 8 consecutive elements, so the
// two halves of a warp quantise two groups at once.  Same arithmetic (and bits) as quantize_group128_lane.
// hl = lane & 15.  Inactive half-warps pass on = false and still take part in the shuffles.
__device__ __forceinline__ void quantize_group_halfwarp(const float v[8], int g, int hl, bool on, const ConsumerSmem& s) {
    float m = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) m = fmaxf(m, fabsf(v[j]));
#pragma unroll
    for (int mask = 8; mask > 0; mask >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, mask));
    const float d = fmaxf(__fdiv_rn(m, 127.0f), 1e-8f);
    const float inv_d = __fdiv_rn(1.0f, d);
    uint32_t packed[2] = {0, 0};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        int q = __float2int_rn(__fmul_rn(v[j], inv_d));
        q = max(-127, min(127, q));
        packed[j >> 2] |= (static_cast<uint32_t>(q) & 0xFFu) << (8 * (j & 3));
    }
    int32_t sum = byte_sum(packed[0]) + byte_sum(packed[1]);     // 8 of the 32 elements of a chunk
    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
    if (on) {
        reinterpret_cast<uint2*>(s.q8)[g * (kGroup / 8) + hl] = make_uint2(packed[0], packed[1]);
        if ((hl & 3) == 0) s.seed[g * 4 + (hl >> 2)] = -8 * sum;
        if (hl == 0) s.xscale[g] = d;
    }
}

// Input of a stage WITH RMSNorm (QKV, gate_up): the residual stream, H elements.  Fetches it into
// s.h (the later residual add reads it there), then normalises + quantises from there.
__device__ bool stage_input_norm(const PSweepArgs& a, const uint2* ll, const __half* plain, uint32_t tag,
                                 const uint4* gamma_regs, int ngam, const ConsumerSmem& s, volatile int* s_abort,
                                 int tid) {
    const int H = a.H, words = H / 2;
    const int lane = tid & 31, warp = tid >> 5;
    double ss = 0.0;
    constexpr int MAXW = (kMaxHidden / 2 + kConsumerThreads - 1) / kConsumerThreads;   // words per thread at most
    uint32_t data[MAXW];
    auto idx = [tid](int i) { return tid + i * kConsumerThreads; };
    int count = 0;
#pragma unroll
    for (int i = 0; i < MAXW; ++i)
        if (idx(i) < words) count = i + 1;
    if (plain != nullptr) {
#pragma unroll
        for (int i = 0; i < MAXW; ++i)
            if (i < count) data[i] = reinterpret_cast<const uint32_t*>(plain)[idx(i)];
    } else {
        if (!poll_words<MAXW>(ll, idx, count, tag, data, s_abort, a.status, a.poll_limit)) return false;
    }
#pragma unroll
    for (int i = 0; i < MAXW; ++i) {
        if (i < count) {
            reinterpret_cast<uint32_t*>(s.h)[idx(i)] = data[i];
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&data[i]));
            ss += static_cast<double>(f.x) * f.x + static_cast<double>(f.y) * f.y;
        }
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, m);
    if (lane == 0) s.red[warp] = ss;
    consumer_sync();
    // every warp adds the per-warp sums itself (same order everywhere): no second barrier, no serial thread
    double t = lane < kConsumerWarps ? s.red[lane] : 0.0;
#pragma unroll
    for (int m = 8; m > 0; m >>= 1) t += __shfl_xor_sync(0xFFFFFFFFu, t, m);
    t = __shfl_sync(0xFFFFFFFFu, t, 0);
    const float inv = inv_rms_from_sumsq(t, H, kEps);
    const __half2 inv2 = __float2half2_rn(inv);
    // quantise: half-warp per group, the gain was fetched before the wait (gamma_regs[i] = group 2*(warp + i*W) + half)
    const int hl = lane & 15, half = lane >> 4;
    const int groups = H / kGroup;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        if (i < ngam) {
            const int g = 2 * (warp + i * kConsumerWarps) + half;
            const bool on = g < groups;
            const uint4 xr = *reinterpret_cast<const uint4*>(s.h + (on ? g : 0) * kGroup + hl * 8);
            const uint4 gr = gamma_regs[i];
            const uint32_t xw[4] = {xr.x, xr.y, xr.z, xr.w}, gw[4] = {gr.x, gr.y, gr.z, gr.w};
            float v[8];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const __half2 y = __hmul2(__hmul2(*reinterpret_cast<const __half2*>(&xw[k]), inv2),
                                          *reinterpret_cast<const __half2*>(&gw[k]));
                const float2 f = __half22float2(y);
                v[2 * k] = f.x;
                v[2 * k + 1] = f.y;
            }
            quantize_group_halfwarp(v, g, hl, on, s);
        }
    }
    return true;
}

// Input of a stage WITHOUT norm (O, down): n elements, quantised straight from the polled words
// (a warp owns whole groups: lane l needs words 2l and 2l+1 of the group).
__device__ bool stage_input_plain(const PSweepArgs& a, const uint2* ll, int n, uint32_t tag, const ConsumerSmem& s,
                                  volatile int* s_abort, int tid) {
    const int lane = tid & 31, warp = tid >> 5;
    const int hl = lane & 15, half = lane >> 4;
    const int groups = n / kGroup;
    // half-warp per group: group of round i = 2 * (warp + i * warps) + half; lane owns elements 8*hl .. 8*hl+7
    constexpr int MAXR = (kMaxK / kGroup + 2 * kConsumerWarps - 1) / (2 * kConsumerWarps);   // rounds per warp
    uint32_t data[4 * MAXR];
    auto grp = [warp, half](int i) { return 2 * (warp + i * kConsumerWarps) + half; };
    auto idx = [grp, hl](int w) { return grp(w >> 2) * (kGroup / 2) + 4 * hl + (w & 3); };
    int count = 0;
#pragma unroll
    for (int i = 0; i < MAXR; ++i)
        if (grp(i) < groups) count = 4 * i + 4;
    if (!poll_words<4 * MAXR>(ll, idx, count, tag, data, s_abort, a.status, a.poll_limit)) return false;
    const int rounds = (groups + 2 * kConsumerWarps - 1) / (2 * kConsumerWarps);
#pragma unroll
    for (int i = 0; i < MAXR; ++i) {
        if (i < rounds) {       // uniform across the warp: both halves shuffle together
            float v[8];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&data[4 * i + k]));
                v[2 * k] = f.x;
                v[2 * k + 1] = f.y;
            }
            quantize_group_halfwarp(v, grp(i), hl, grp(i) < groups, s);
        }
    }
    return true;
}

// One lane's share of a weight row held in a ring slot: the 16-byte chunks j, j + lpr, j + 2 lpr ...
// (CPL of them at most, `cpr` chunks per row).  All shared-memory loads are issued before the first
// dp4a so that their latencies overlap.
template <int CPL>
__device__ __forceinline__ float row_dot(const uint8_t* wrow, const __half* srow, const ConsumerSmem& s, int j, int lpr,
                                         int cpr, bool busy) {
    uint4 w[CPL], xa[CPL], xb[CPL];
    int32_t seed[CPL];
    float f[CPL];
#pragma unroll
    for (int i = 0; i < CPL; ++i) {
        const int c = j + i * lpr;
        const bool on = busy && c < cpr;
        const int cc = on ? c : 0;
        w[i] = *reinterpret_cast<const uint4*>(wrow + cc * 16);
        xa[i] = reinterpret_cast<const uint4*>(s.q8)[2 * cc];
        xb[i] = reinterpret_cast<const uint4*>(s.q8)[2 * cc + 1];
        seed[i] = s.seed[cc];
        f[i] = on ? __half2float(srow[cc >> 2]) * s.xscale[cc >> 2] : 0.0f;   // f = 0 switches a slot off
    }
    float acc = 0.0f;
#pragma unroll
    for (int i = 0; i < CPL; ++i) acc = fmaf(static_cast<float>(chunk_dot(w[i], xa[i], xb[i], seed[i])), f[i], acc);
    return acc;
}

__device__ void consumer_loop(const PSweepArgs& a, uint8_t* ring, uint32_t full0, uint32_t empty0,
                              const ConsumerSmem& s, volatile int* s_abort, int tid) {
    const int cta = blockIdx.x, nctas = gridDim.x;
    const int lane = tid & 31;
    int slot = 0;
    uint32_t phase = 0;
    int chunk_parity = 0;
    const int num_stages = a.num_layers * 4;
    for (int st = 0; st < num_stages; ++st) {
        const StagePlan p = make_plan(a, st, cta, nctas);
        const LayerDev& L = static_cast<const LayerDev*>(a.layers)[st >> 2];
        const uint32_t in_tag = a.epoch + static_cast<uint32_t>(st);        // tag of the previous stage
        const uint32_t out_tag = a.epoch + static_cast<uint32_t>(st) + 1;
        // ---- 1. the activation vector of this projection ----
        // RMSNorm gains of this thread's groups: constant data, fetched before the wait
        uint4 gamma_regs[2] = {};
        int ngam = 0;
        if (p.kind == 0 || p.kind == 2) {
            const __half* gamma = p.kind == 0 ? L.gamma_in : L.gamma_post;
            const int groups = a.H / kGroup;
            ngam = (groups + 2 * kConsumerWarps - 1) / (2 * kConsumerWarps);   // <= 2 for H <= 4096... checked on the host
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int g = 2 * ((tid >> 5) + i * kConsumerWarps) + ((tid & 31) >> 4);
                if (i < ngam && g < groups)
                    gamma_regs[i] = *reinterpret_cast<const uint4*>(gamma + g * kGroup + (tid & 15) * 8);
            }
        }
        if (st > 0) {
            // one thread waits until every CTA has published the previous projection
            if (tid == 0) {
                const uint32_t* ctr = a.counters + 8 * (st - 1);
                bool seen = false;
                for (unsigned it = 0; it < a.poll_limit; ++it) {
                    // counters may have wrapped past the target of a later launch: compare as a distance
                    if (static_cast<int32_t>(ld_counter(ctr) - a.counter_target) >= 0) { seen = true; break; }
                    if (*s_abort) break;
                    __nanosleep(20);
                }
                if (!seen) { *s_abort = 1; atomicExch(a.status, 2); }
            }
            consumer_sync();
            if (*s_abort) return;
        }
        bool ok;
        switch (p.kind) {
            case 0: ok = stage_input_norm(a, a.ll_h_down, st == 0 ? a.h_in : nullptr, in_tag, gamma_regs, ngam, s, s_abort, tid); break;
            case 1: ok = stage_input_plain(a, a.ll_q, a.qdim, in_tag, s, s_abort, tid); break;
            case 2: ok = stage_input_norm(a, a.ll_h_attn, nullptr, in_tag, gamma_regs, ngam, s, s_abort, tid); break;
            default: ok = stage_input_plain(a, a.ll_mlp, a.I, in_tag, s, s_abort, tid); break;
        }
        if (!ok) return;
        consumer_sync();
        // ---- 2. this CTA's rows, one ring slot at a time ----
        const int cpr = p.row_bytes / 16;          // 16-byte chunks per weight row
        // Fast path: a row is spread over `flpr` lanes, at most 3 chunks per lane, and the lane's share of
        // the quantised activation stays in registers for the whole projection (48 chunks -> 16 lanes,
        // 280 chunks -> 128 lanes).  Other shapes take the shared-memory path below.
        // lanes per row: 8, 16, 32, then whole warps (64, 96, 128)
        int flpr = 8;
        while (3 * flpr < cpr && flpr < 32) flpr *= 2;
        while (3 * flpr < cpr && flpr < 32 * kMaxRowWarps) flpr += 32;
        const bool fast = 3 * flpr >= cpr;
        const int fj = tid % flpr, fslot = tid / flpr, rows_per_pass = kConsumerThreads / flpr;
        uint4 xa[3], xb[3];
        int32_t xseed[3];
        float xs[3];
        if (fast) {
#pragma unroll
            for (int i = 0; i < 3; ++i) {
                const int c = fj + i * flpr;
                const bool on = c < cpr;
                const int cc = on ? c : 0;
                xa[i] = reinterpret_cast<const uint4*>(s.q8)[2 * cc];
                xb[i] = reinterpret_cast<const uint4*>(s.q8)[2 * cc + 1];
                xseed[i] = s.seed[cc];
                xs[i] = on ? s.xscale[cc >> 2] : 0.0f;     // a zero factor switches the slot off
            }
        }
        for (int r = 0; r < p.num_rows; r += p.chunk_rows) {
            const int rows = min(p.chunk_rows, p.num_rows - r);
            int wait_ok = 1;
            if (lane == 0) wait_ok = bar_wait(full0 + 8u * slot, phase, s_abort) ? 1 : 0;
            wait_ok = __shfl_sync(0xFFFFFFFFu, wait_ok, 0);
            if (!wait_ok) {
                if (tid == 0) atomicExch(a.status, 1);
                return;
            }
            const uint8_t* w_base = ring + slot * kSlotStride;
            const __half* sc_base = reinterpret_cast<const __half*>(w_base + kSlotBytes);
            float* part = s.part + chunk_parity * kPartFloats;
            const bool in_warp = fast && (p.kind == 2 ? 2 * flpr <= 32 : flpr <= 32);   // row (pair) inside one warp
            int lpr = flpr;
            if (fast) {
                for (int r0 = 0; r0 < rows; r0 += rows_per_pass) {
                    const int row = r0 + fslot;
                    const bool busy = row < rows;
                    const uint8_t* wrow = w_base + (busy ? row : 0) * p.row_bytes;
                    const __half* srow = sc_base + (busy ? row : 0) * p.groups;
                    uint4 w[3];
                    float f[3];
#pragma unroll
                    for (int i = 0; i < 3; ++i) {
                        const int c = fj + i * flpr;
                        const int cc = c < cpr ? c : 0;
                        w[i] = *reinterpret_cast<const uint4*>(wrow + cc * 16);
                        f[i] = __half2float(srow[cc >> 2]) * xs[i];
                    }
                    float acc = 0.0f;
#pragma unroll
                    for (int i = 0; i < 3; ++i)
                        acc = fmaf(static_cast<float>(chunk_dot(w[i], xa[i], xb[i], xseed[i])), f[i], acc);
                    const int wl = min(flpr, 32);
                    for (int m = wl >> 1; m > 0; m >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, m);
                    if (in_warp) {
                        // every lane of the row holds its sum: finish the row right here
                        if (p.kind == 2) {
                            const float other = __shfl_xor_sync(0xFFFFFFFFu, acc, flpr);   // the up row's sum
                            if (busy && fj == 0 && (row & 1) == 0)
                                s.out[(r + row) >> 1] = __float2half_rn((acc / (1.0f + expf(-acc))) * other);
                        } else if (busy && fj == 0) {
                            float v = acc;
                            if (p.kind != 0) v += __half2float(s.h[p.first_row + r + row]);
                            s.out[r + row] = __float2half_rn(v);
                        }
                    } else if (busy && (tid % wl) == 0) {
                        part[row * kMaxRowWarps + (fj >> 5)] = acc;
                    }
                }
            } else {
                // lanes per row: the largest power of two that lets all rows of the slot run side by side
                lpr = 8;
                while (lpr * 2 * rows <= kConsumerThreads && lpr < 32 * kMaxRowWarps && lpr < cpr) lpr *= 2;
                const int cpl = (cpr + lpr - 1) / lpr;     // chunks per lane
                const int row = tid / lpr, j = tid % lpr;
                const bool busy = row < rows;
                const uint8_t* wrow = w_base + (busy ? row : 0) * p.row_bytes;
                const __half* srow = sc_base + (busy ? row : 0) * p.groups;
                float acc = 0.0f;
                for (int c0 = 0; c0 < cpl; c0 += 2) acc += row_dot<2>(wrow, srow, s, j + c0 * lpr, lpr, cpr, busy);
                const int wl = min(lpr, 32);
                for (int m = wl >> 1; m > 0; m >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, m);
                if (busy && (tid % wl) == 0) part[row * kMaxRowWarps + (j >> 5)] = acc;
            }
            if (in_warp) {
                __syncwarp();
                if (lane == 0) bar_arrive(empty0 + 8u * slot);   // this warp has read its rows of the slot
            } else {
                consumer_sync();                        // partial sums visible; the slot has been read
                if (lane == 0) bar_arrive(empty0 + 8u * slot);   // one arrival per consumer warp
                // final value of each row (fixed summation order), epilogue into s.out
                const int nw = (lpr + 31) >> 5;         // warps that share a row
                if (p.kind == 2) {
                    if (tid < rows / 2) {
                        float g = 0.0f, u = 0.0f;
                        for (int k = 0; k < nw; ++k) { g += part[(2 * tid) * kMaxRowWarps + k]; u += part[(2 * tid + 1) * kMaxRowWarps + k]; }
                        s.out[(r >> 1) + tid] = __float2half_rn((g / (1.0f + expf(-g))) * u);
                    }
                } else if (tid < rows) {
                    float v = 0.0f;
                    for (int k = 0; k < nw; ++k) v += part[tid * kMaxRowWarps + k];
                    if (p.kind != 0) v += __half2float(s.h[p.first_row + r + tid]);   // residual add (O, down)
                    s.out[r + tid] = __float2half_rn(v);
                }
            }
            chunk_parity ^= 1;
            if (++slot == kSlots) { slot = 0; phase ^= 1; }
        }
        consumer_sync();   // s.out complete
        // ---- 3. publish this CTA's output pairs ----
        if (tid < p.num_pairs) {
            const uint32_t data = reinterpret_cast<const uint32_t*>(s.out)[tid];
            const int pair = p.first_pair + tid;
            switch (p.kind) {
                case 0: {
                    const int e = 2 * pair;   // virtual output index
                    if (e < a.qdim) st_ll(a.ll_q + pair, data, out_tag);
                    else if (e < a.qdim + a.kvdim) reinterpret_cast<uint32_t*>(a.k_out)[(e - a.qdim) >> 1] = data;
                    else reinterpret_cast<uint32_t*>(a.v_out)[(e - a.qdim - a.kvdim) >> 1] = data;
                    break;
                }
                case 1: st_ll(a.ll_h_attn + pair, data, out_tag); break;
                case 2: st_ll(a.ll_mlp + pair, data, out_tag); break;
                default:
                    st_ll(a.ll_h_down + pair, data, out_tag);
                    if (st == num_stages - 1) reinterpret_cast<uint32_t*>(a.h_out)[pair] = data;
                    break;
            }
        }
        // announce: issued after this thread's own stores; the words carry their own tags, so the count
        // may overtake stores of other threads without harm
        if (tid == 0) add_counter(a.counters + 8 * st);
        // s.out and the staged activation are rewritten only after the next stage's first
        // consumer_sync, which every thread reaches after this point.
    }
}

__global__ void __launch_bounds__(kBlockThreads, 1) decode_sweep_persistent_kernel(const PSweepArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* ring = smem;
    uint8_t* p = smem + kSlots * kSlotStride;
    ConsumerSmem s;
    s.q8 = reinterpret_cast<int8_t*>(p); p += kMaxK;
    s.seed = reinterpret_cast<int32_t*>(p); p += kMaxK / kChunk * 4;
    s.xscale = reinterpret_cast<float*>(p); p += kMaxK / kGroup * 4;
    s.h = reinterpret_cast<__half*>(p); p += kMaxHidden * 2;
    s.out = reinterpret_cast<__half*>(p); p += 512 * 2;
    s.part = reinterpret_cast<float*>(p); p += 2 * kPartFloats * 4;
    s.red = reinterpret_cast<double*>(p); p += kConsumerWarps * 8;
    s.inv = reinterpret_cast<float*>(p); p += 16;
    uint64_t* bars = reinterpret_cast<uint64_t*>(p); p += 2 * kSlots * 8;
    volatile int* s_abort = reinterpret_cast<volatile int*>(p);
    const uint32_t full0 = s32(bars), empty0 = s32(bars + kSlots);

    const int tid = threadIdx.x;
    if (tid == 0) {
        for (int i = 0; i < kSlots; ++i) {
            bar_init(full0 + 8u * i, 1 + 32);             // expect_tx arrival + 32 lanes' scale copies
            bar_init(empty0 + 8u * i, kConsumerWarps);
        }
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (tid >= kConsumerThreads) {
        producer_loop(a, ring, full0, empty0, s_abort, tid & 31);
        if (*s_abort && (tid & 31) == 0) atomicCAS(a.status, 0, 1);
    } else {
        consumer_loop(a, ring, full0, empty0, s, s_abort, tid);
    }
}

constexpr size_t kSmemBytes = static_cast<size_t>(kSlots) * kSlotStride + kMaxK + kMaxK / kChunk * 4 + kMaxK / kGroup * 4 +
                              kMaxHidden * 2 + 512 * 2 + 2 * kPartFloats * 4 + kConsumerWarps * 8 + 16 + 2 * kSlots * 8 + 16;

}  // namespace

// ---- host interface (used by decode_sweep.cu) -------------------------------------------------------

size_t psweep_layer_bytes() { return sizeof(LayerDev); }

// Can the persistent kernel run this model?  (vector lengths the staging holds, slot geometry, alignment)
bool psweep_supported(int H, int I, int qdim, int kvdim) {
    if (H > kMaxHidden || I > kMaxK || qdim > kMaxK || H % 256 || I % 256 || qdim % 256 || kvdim % 2) return false;
    const int ks[3] = {H, I, qdim};
    for (int K : ks)
        if (((kSlotBytes / (K / 2)) & ~3) < 4) return false;
    // a CTA publishes at most 512 outputs per stage from its staging buffer (ample for >= 64 CTAs)
    return true;
}

int psweep_set_attributes() {
    return static_cast<int>(cudaFuncSetAttribute(decode_sweep_persistent_kernel,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 static_cast<int>(kSmemBytes)));
}

// Fills one LayerDev in host memory (the caller copies the array to the device).
void psweep_fill_layer(void* dst, const w4a16_layer_weights& L) {
    LayerDev d;
    const void* w[6] = {L.q_weight, L.k_weight, L.v_weight, L.o_weight, L.gate_up_weight, L.down_weight};
    const void* s[6] = {L.q_scale, L.k_scale, L.v_scale, L.o_scale, L.gate_up_scale, L.down_scale};
    for (int i = 0; i < 6; ++i) {
        d.w[i] = static_cast<const uint8_t*>(w[i]);
        d.sc[i] = static_cast<const __half*>(s[i]);
    }
    d.gamma_in = static_cast<const __half*>(L.input_norm_gamma);
    d.gamma_post = static_cast<const __half*>(L.post_norm_gamma);
    *static_cast<LayerDev*>(dst) = d;
}

int psweep_launch(const PSweepArgs& args, int sm_count, cudaStream_t stream) {
    PSweepArgs a = args;
    const int spins = option(W4A16_OPT_SIGNAL_WAIT_SPINS);
    a.poll_limit = spins > 0 ? static_cast<unsigned>(spins) : kPollLimit;
    void* params[] = {&a};
    const int max_pairs = std::max(std::max(a.H, a.I), a.qdim + 2 * a.kvdim) / 2;
    int grid = sm_count;
    if ((max_pairs + grid - 1) / grid > 256) return W4A16_ERR_TOO_LARGE;   // s.out holds 512 outputs
    // cooperative launch: all CTAs must be resident, they wait for each other's outputs
    return static_cast<int>(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(decode_sweep_persistent_kernel),
                                                        dim3(grid), dim3(kBlockThreads), params, kSmemBytes, stream));
}

}  // namespace w4
