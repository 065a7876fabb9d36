// M-token W4A16 contraction on the 5th-generation tensor cores (tcgen05 / TMEM), sm_100a.
//
// Replaces the reference's wmma prefill GEMMs (src/kernels/gemm_prefill.cu:319-610).
// Arithmetic is the reference's: weights dequantised to fp16 as (q - 8) * scale with one fp16
// rounding (include/quant_primitives.cuh:92-115), fp16 x fp16 products exact, fp32 accumulation,
// epilogue fp16(acc) [+ fp16 residual add] / SwiGLU on the fp32 accumulators
// (gemm_prefill.cu:257-275, 572-605).
//
// Formulation: D[n][m] = sum_k W[n][k] * X[m][k] with the WEIGHT rows on the 128-wide M side of
// the MMA and the tokens on its N side (16..256), so a decode batch of 16 tokens fills the
// tensor core as well as a prefill chunk does, and weights stream through each CTA exactly once.
//
//   warps 0..4*NG-1 : NG groups of 4 warps dequantise raw nibbles -> fp16 A tile [128 x 64] in the
//                 K-major 128B-swizzled layout the UMMA shared-memory descriptor expects; inside a
//                 group a thread owns a weight row, and group g takes k-blocks g, g+NG, ... so the
//                 fixed cost of a k-block (barrier waits, proxy fence, arrive) is paid by 4 warps
//                 while the other groups work on the next k-blocks; later all of them run the epilogue
//   next warp   : allocates TMEM, issues tcgen05.mma (one thread), commits to mbarriers
//   next warp   : TMA producer of the token tile B [T x 64] fp16 (128B swizzle)
//   last warp   : TMA producer of raw packed weights, 128 rows x 128 B (= 256 k) per stage,
//                 128B-swizzled so that row-per-thread reads are bank-conflict free
//   epilogue    : tcgen05.ld 32x32b (thread = weight row, registers = tokens), fp16 stores
//
// One destination per copy, no cluster.  Every mbarrier wait is bounded: on expiry the kernel raises an
// abort flag, all roles leave their loops, TMEM is freed and the kernel returns; the host can
// read the count of such events with w4a16_debug_counter(0).
#include <cuda.h>

#include <algorithm>
#include <mutex>
#include <utility>
#include <vector>

#include "gemm_smallm.cuh"
#include "w4a16_common.cuh"
#include "w4a16_internal.hpp"

namespace w4 {

__device__ unsigned int g_tc_wait_timeouts = 0;

namespace {

constexpr int kTileRows = 128;          // weight rows per CTA (UMMA M)
constexpr int kBK = 64;                 // fp16 elements per k-block: one 128-byte swizzle row
constexpr int kRawStages = 3;
constexpr int kRawBytes = kTileRows * 128;   // 128 rows x 128 bytes of packed nibbles = 256 k
constexpr int kABytes = kTileRows * 128;     // 128 rows x 64 fp16
constexpr int kMaxStages = 8;
constexpr int kMaxIssuers = 2;          // warps that may issue tensor-core instructions (k-blocks dealt round robin;
                                        // measured: a third and fourth bring nothing)
constexpr unsigned kWaitLimit = 1u << 22;

struct TcArgs {
    CUtensorMap tmap_w[3];
    CUtensorMap tmap_x;
    const __half* scales[3];
    __half* out[3];
    int rows[3];
    int out_ld[3];
    int tiles[3];            // 128-row tiles per weight tensor
    const __half* residual;
    int M, K, T, stages, tmem_cols;
    int ksplit;              // CTAs (one cluster along grid z) that share the K range of one output tile
    int issuers;             // 1 or 2 warps issuing the tensor-core instructions (even / odd k-blocks, own accumulators)
    __half* peer_out[7];     // PLAIN: the output block's place in other GPUs' matrices
    int num_peers;
    int panel;               // CTA-pair kernel: token tiles per panel of the tile order
};

// ---- PTX wrappers ------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Non-blocking test of a phase (try_wait may park the thread for a while when the phase is still open).
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false if the barrier did not flip within the limit or another role gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_test_wait(bar, parity)) return true;   // already complete: no need to park the thread
    for (unsigned it = 0; it < kWaitLimit; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (it > 2048) __nanosleep(64);
    }
    *abort_flag = 1;
    atomicAdd(&g_tc_wait_timeouts, 1u);
    return false;
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]^T, fp16 inputs, fp32 accumulate.
__device__ __forceinline__ void tc_mma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                           uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
// Cluster-wide barrier (all threads of all CTAs of the cluster) and stores into another CTA's shared memory.
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_map_shared(uint32_t local_addr, uint32_t cta_rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(cta_rank));
    return remote;
}
__device__ __forceinline__ void st_shared_cluster_u32(uint32_t addr, uint32_t v) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// v += the 16 columns at taddr (another issuing warp's accumulator).
__device__ __forceinline__ void add_second_accumulator(uint32_t taddr, uint32_t (&v)[16]) {
    uint32_t u[16];
    tmem_ld16(taddr, u);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(u[j]));
}

// Shared-memory matrix descriptor: K-major tile, 128-byte swizzle, rows 128 B apart, 8-row groups
// 1024 B apart (stride byte offset), descriptor version 1 (sm_100).  `addr` may be advanced by
// 32 B per 16-element K slice inside the 128-byte swizzle row.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr & 0x3FFFFu) >> 4);   // start address, 16-byte units
    d |= static_cast<uint64_t>(1) << 16;                  // leading byte offset (unused with swizzle)
    d |= static_cast<uint64_t>(1024 >> 4) << 32;          // stride byte offset
    d |= static_cast<uint64_t>(1) << 46;                  // version
    d |= static_cast<uint64_t>(2) << 61;                  // SWIZZLE_128B
    return d;
}
// Instruction descriptor: D fp32, A/B fp16, both K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t make_idesc(int n) {
    return (1u << 4) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(kTileRows >> 4) << 24);
}

// One lane polls the barrier for its warp (512 threads polling would keep the mbarrier unit busy and
// delay the single MMA-issuing thread); __syncwarp then orders the other lanes' reads after it.
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int lane) {
    int ok = 1;
    if (lane == 0) ok = mbar_wait(bar, parity, abort_flag) ? 1 : 0;
    __syncwarp();
    return __shfl_sync(0xFFFFFFFFu, ok, 0) != 0;
}

// EXTRAS = false is the plain form (one issuing warp, no K split, no peer stores): those options cost the
// prefill shapes 5-18 % when they are runtime branches in the epilogue, so they are compiled out there.
template <int MODE, int NG, bool EXTRAS>
__global__ void __launch_bounds__((4 * NG + kMaxIssuers + 2) * 32, 1) gemm_w4a16_tc_kernel(const __grid_constant__ TcArgs a) {
    constexpr int kDqWarps = 4 * NG;             // dequantising warps: NG groups of 4
    constexpr int kDqThreads = kDqWarps * 32;
    constexpr int kIssuerWarps = EXTRAS ? kMaxIssuers : 1;   // then one warp for the token TMA, one for the weight TMA
    extern __shared__ uint8_t smem_raw_base[];
    // 1024-byte alignment for the swizzled tiles
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw_base) + 1023) & ~uintptr_t(1023));
    const int T = a.T, S = a.stages, K = a.K;
    const int G = K / kGroup;
    const int b_bytes = T * 128;
    uint8_t* s_raw = smem;                                  // kRawStages x 16 KB
    uint8_t* s_a = s_raw + kRawStages * kRawBytes;          // S x 16 KB
    uint8_t* s_b = s_a + S * kABytes;                       // S x T*128
    __half* s_scale = reinterpret_cast<__half*>(s_b + S * b_bytes);   // [G][128]
    uint64_t* s_bar = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(s_scale) + ((G * kTileRows * 2 + 15) & ~15));
    // barrier slots: raw_full[3] raw_empty[3] full[S] (A dequantised AND B landed) ab_empty[S] accum_full
    const uint32_t bar0 = smem_u32(s_bar);
    auto raw_full = [&](int i) { return bar0 + 8u * i; };
    auto raw_empty = [&](int i) { return bar0 + 8u * (kRawStages + i); };
    auto full = [&](int i) { return bar0 + 8u * (2 * kRawStages + i); };
    auto ab_empty = [&](int i) { return bar0 + 8u * (2 * kRawStages + 2 * kMaxStages + i); };
    const uint32_t accum_full = bar0 + 8u * (2 * kRawStages + 3 * kMaxStages);
    uint32_t* s_tmem = reinterpret_cast<uint32_t*>(s_bar + (2 * kRawStages + 3 * kMaxStages + 1));
    volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // which weight tensor / which rows
    int t = 0, tile = blockIdx.x;
    if constexpr (MODE == kQkv) {
        if (tile >= a.tiles[0]) { tile -= a.tiles[0]; t = 1; }
        if (t == 1 && tile >= a.tiles[1]) { tile -= a.tiles[1]; t = 2; }
    }
    const int n0 = tile * kTileRows;         // first weight row of this CTA inside tensor t
    const int m0 = blockIdx.y * T;           // first token
    const int rows_t = a.rows[t];
    // K range of this CTA: whole 256-element super-blocks, spread over the cluster as evenly as they go
    const int ksplit = EXTRAS ? a.ksplit : 1, krank = EXTRAS ? static_cast<int>(blockIdx.z) : 0;
    const int issuers = EXTRAS ? a.issuers : 1, num_peers = EXTRAS ? a.num_peers : 0;
    const int total_sb = K / 256;
    const int sb_begin = krank * (total_sb / ksplit) + min(krank, total_sb % ksplit);
    const int num_sb = total_sb / ksplit + (krank < total_sb % ksplit ? 1 : 0);
    const int num_kb = num_sb * (256 / kBK), kb_begin = sb_begin * (256 / kBK);

    if (tid == 0) {
        for (int i = 0; i < kRawStages; ++i) { mbar_init(raw_full(i), 1); mbar_init(raw_empty(i), kDqWarps); }
        for (int i = 0; i < S; ++i) { mbar_init(full(i), 4 + 1); mbar_init(ab_empty(i), 1); }   // 4 warps + the TMA thread
        mbar_init(accum_full, issuers);   // every issuing warp commits once at its end (a K range holds >= 4 k-blocks)
        *s_abort = 0;
        fence_barrier_init();
        tma_prefetch_desc(&a.tmap_x);
        tma_prefetch_desc(&a.tmap_w[t]);
    }
    if (warp == kDqWarps) {
        tmem_alloc(smem_u32(s_tmem), static_cast<uint32_t>(a.tmem_cols));
        tmem_relinquish();
    }
    pdl_release_dependents();
    pdl_wait_prior_grids();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem;

    if (warp < kDqWarps) {
        // ---------------- dequantise: group = warp / 4, thread = weight row inside the group ----------------
        const int r = (warp & 3) * 32 + lane;    // weight row inside the tile == TMEM lane of the epilogue
        const int part = warp >> 2;              // group index; also the epilogue's column share
        // scales of the 128 rows, transposed to [group][row]
        {
            const __half* sc = a.scales[t];
            const int g_local = 2 * num_sb, g_begin = 2 * sb_begin;    // this CTA's groups of 128 only
            for (int idx = tid; idx < kTileRows * g_local; idx += kDqThreads) {
                const int rr = idx / g_local, g = idx - rr * g_local;
                const int row = n0 + rr;
                s_scale[g * kTileRows + rr] =
                    row < rows_t ? sc[static_cast<size_t>(row) * G + g_begin + g] : __float2half(0.0f);
            }
            asm volatile("bar.sync 1, %0;" ::"n"(kDqThreads) : "memory");
        }
        const int sw = r & 7;
        bool ok = true;
        int rs = 0;
        uint32_t rph = 0;
        // ring position of this group's first k-block (k-block index == part), then += NG per visit
        int s = part;
        uint32_t ph = 0;
        while (s >= S) { s -= S; ph ^= 1; }
        for (int sb = 0; sb < num_sb && ok; ++sb) {
            ok = warp_wait(raw_full(rs), rph, s_abort, lane);
            if (!ok) break;
            const uint8_t* raw_row = s_raw + rs * kRawBytes + r * 128;
            const __half2 sc0 = __half2half2(s_scale[(2 * sb) * kTileRows + r]);
            const __half2 sc1 = __half2half2(s_scale[(2 * sb + 1) * kTileRows + r]);
#pragma unroll
            for (int j = part; j < 4; j += NG) {     // this group's k-blocks of the 256-element super-block
                ok = warp_wait(ab_empty(s), ph ^ 1, s_abort, lane);
                if (!ok) break;
                const uint4 w0 = *reinterpret_cast<const uint4*>(raw_row + (((2 * j) ^ sw) << 4));
                const uint4 w1 = *reinterpret_cast<const uint4*>(raw_row + (((2 * j + 1) ^ sw) << 4));
                const uint32_t words[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
                const __half2 sc2 = (j < 2) ? sc0 : sc1;
                uint8_t* a_row = s_a + s * kABytes + r * 128;
#pragma unroll
                for (int w = 0; w < 8; ++w) {
                    __half2 h[4];
                    dequant_word_fp16(words[w], sc2, h);
                    *reinterpret_cast<uint4*>(a_row + ((w ^ sw) << 4)) = *reinterpret_cast<const uint4*>(h);
                }
                fence_proxy_async_smem();   // generic-proxy writes -> visible to the tensor core's async proxy
                __syncwarp();
                if (lane == 0) mbar_arrive(full(s));
                s += NG;
                while (s >= S) { s -= S; ph ^= 1; }
            }
            __syncwarp();
            if (lane == 0 && ok) mbar_arrive(raw_empty(rs));
            if (++rs == kRawStages) { rs = 0; rph ^= 1; }
        }
        // ---------------- epilogue: thread = weight row, registers = tokens ----------------
        if (ok) ok = warp_wait(accum_full, 0, s_abort, lane);
        tc_fence_after();
        // Split K: the CTAs of the cluster hold partial sums of the same output tile.  After a first cluster
        // barrier (everyone's main loop is over, so the leader's pipeline buffers are free) the others store
        // their fp32 partials into the leader's shared memory, [rank-1][token][row] (conflict-free for row-per-thread); after a second barrier the
        // leader adds them in rank order and finishes alone.  Every thread of every CTA passes both barriers,
        // also when a bounded wait gave up.
        float* s_part = reinterpret_cast<float*>(smem);
        if (ksplit > 1) {
            cluster_sync_all();
            if (krank != 0 && ok) {
                const uint32_t remote0 = cluster_map_shared(smem_u32(s_part), 0);
                for (int c0 = part * 16; c0 < T; c0 += 16 * NG) {
                    uint32_t v[16];
                    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
                    tmem_ld16(lane_base + static_cast<uint32_t>(c0), v);
                    tmem_ld_wait();
                    for (int w = 1; w < issuers; ++w) add_second_accumulator(lane_base + static_cast<uint32_t>(w * T + c0), v);
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        st_shared_cluster_u32(remote0 + 4u * static_cast<uint32_t>(((krank - 1) * T + c0 + j) * kTileRows + r), v[j]);
                }
            }
            cluster_sync_all();
        }
        if (ok && krank == 0) {
            const int n = n0 + r;
            const bool row_ok = n < rows_t;
            __half* out = a.out[t];
            const int ld = a.out_ld[t];
            // the NG warps that share a TMEM lane quarter take the 16-column chunks in turn
            for (int c0 = part * 16; c0 < T; c0 += 16 * NG) {
                uint32_t v[16];
                const uint32_t lane_base = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
                tmem_ld16(lane_base + static_cast<uint32_t>(c0), v);
                tmem_ld_wait();
                for (int w = 1; w < issuers; ++w) add_second_accumulator(lane_base + static_cast<uint32_t>(w * T + c0), v);

                // the other CTAs' partial sums, slice after slice (16 independent loads in flight each)
                for (int k = 1; k < ksplit; ++k) {
                    float p[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) p[j] = s_part[((k - 1) * T + c0 + j) * kTileRows + r];
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) + p[j]);
                }
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int m = m0 + c0 + j;
                    const float acc = __uint_as_float(v[j]);
                    if constexpr (MODE == kSwiglu) {
                        const float up = __shfl_xor_sync(0xFFFFFFFFu, acc, 1);
                        if ((lane & 1) == 0 && row_ok && m < a.M) {
                            const float y = (acc / (1.0f + expf(-acc))) * up;
                            out[static_cast<size_t>(m) * ld + (n >> 1)] = __float2half_rn(y);
                        }
                    } else {
                        if (row_ok && m < a.M) {
                            __half y = __float2half_rn(acc);
                            if constexpr (MODE == kPlain) {
                                if (a.residual != nullptr) y = __hadd(y, a.residual[static_cast<size_t>(m) * ld + n]);
                            }
                            out[static_cast<size_t>(m) * ld + n] = y;
                            if constexpr (MODE == kPlain) {
                                for (int p = 0; p < num_peers; ++p) a.peer_out[p][static_cast<size_t>(m) * ld + n] = y;
                            }
                        }
                    }
                }
            }
        }
    } else if (warp >= kDqWarps && warp < kDqWarps + kIssuerWarps) {
        // ---------------- MMA issue ----------------
        // Issuing a tensor-core instruction costs its thread a fixed time however small the instruction, and
        // with few tokens that time, not the tensor pipe, bounds a k-block.  Two warps can therefore
        // issue: warp w takes the k-blocks w, w + n, ..., each into its OWN accumulator (TMEM columns
        // [w T, (w + 1) T)) so that no order between the instruction streams is needed; the epilogue adds them.  The whole warp walks the loop with warp-uniform values; one lane issues.  The barrier
        // of the warp's NEXT k-block is tested before this k-block's MMAs are issued so that the test's
        // latency overlaps the issue.
        const int w = warp - kDqWarps, nw = issuers;
        if constexpr (!EXTRAS) {
            // one issuing warp, the whole K range: ring positions by compare-and-reset, descriptors by plain adds
        {
            const uint32_t idesc = make_idesc(T);
            const uint64_t a_desc0 = make_smem_desc(smem_u32(s_a));
            const uint64_t b_desc0 = make_smem_desc(smem_u32(s_b));
            const uint32_t a_step = kABytes >> 4, b_step = static_cast<uint32_t>(b_bytes) >> 4;
            uint64_t a_desc = a_desc0, b_desc = b_desc0;
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            bool ready = mbar_test_wait(full(0), 0);
            for (int kb = 0; kb < num_kb; ++kb) {
                if (!ready) ok = warp_wait(full(s), ph, s_abort, lane);
                if (!ok) break;
                // position of the next k-block, and an early look at its barrier
                int sn = s + 1;
                uint32_t phn = ph;
                if (sn == S) { sn = 0; phn ^= 1; }
                if (lane == 0) {
#pragma unroll
                    for (int ks = 0; ks < kBK / 16; ++ks)
                        tc_mma_f16(tmem_base, a_desc + 2 * ks, b_desc + 2 * ks, idesc, (kb | ks) != 0 ? 1u : 0u);
                    tc_commit(ab_empty(s));    // frees the stage when these MMAs have read it
                }
                ready = (kb + 1 < num_kb) ? mbar_test_wait(full(sn), phn) : true;
                ready = __all_sync(0xFFFFFFFFu, ready);
                a_desc += a_step;
                b_desc += b_step;
                if (sn == 0) { a_desc = a_desc0; b_desc = b_desc0; }
                s = sn;
                ph = phn;
            }
            if (ok && lane == 0) tc_commit(accum_full);
        }
        } else if (w < nw) {
            const uint32_t idesc = make_idesc(T);
            const uint64_t a_desc0 = make_smem_desc(smem_u32(s_a));
            const uint64_t b_desc0 = make_smem_desc(smem_u32(s_b));
            const uint32_t a_step = kABytes >> 4, b_step = static_cast<uint32_t>(b_bytes) >> 4;
            const uint32_t tmem_acc = tmem_base + static_cast<uint32_t>(w * T);
            int s = w % S;
            uint32_t ph = static_cast<uint32_t>(w / S) & 1u;
            bool ok = true;
            bool ready = __all_sync(0xFFFFFFFFu, mbar_test_wait(full(s), ph));
            uint64_t a_desc = a_desc0 + static_cast<uint32_t>(s) * a_step, b_desc = b_desc0 + static_cast<uint32_t>(s) * b_step;
            for (int kb = w; kb < num_kb; kb += nw) {
                if (!ready) ok = warp_wait(full(s), ph, s_abort, lane);
                if (!ok) break;
                // position of this warp's next k-block, and an early look at its barrier
                int sn = s + nw;
                uint32_t phn = ph;
                while (sn >= S) { sn -= S; phn ^= 1; }
                if (lane == 0) {
#pragma unroll
                    for (int ks = 0; ks < kBK / 16; ++ks)
                        tc_mma_f16(tmem_acc, a_desc + 2 * ks, b_desc + 2 * ks, idesc, (kb >= nw || ks != 0) ? 1u : 0u);
                    tc_commit(ab_empty(s));    // frees the stage when these MMAs have read it
                }
                ready = (kb + nw < num_kb) ? mbar_test_wait(full(sn), phn) : true;
                ready = __all_sync(0xFFFFFFFFu, ready);
                // descriptors by plain adds on their low word (the start-address field counts 16-byte units and
                // cannot carry out of its 14 bits for shared-memory addresses), recomputed when the ring wraps
                if (sn > s) { a_desc += static_cast<uint32_t>(nw) * a_step; b_desc += static_cast<uint32_t>(nw) * b_step; }
                else { a_desc = a_desc0 + static_cast<uint32_t>(sn) * a_step; b_desc = b_desc0 + static_cast<uint32_t>(sn) * b_step; }
                s = sn;
                ph = phn;
            }
            if (ok && lane == 0) tc_commit(accum_full);
        }
        __syncwarp();
        if (ksplit > 1) { cluster_sync_all(); cluster_sync_all(); }
    } else if (warp == kDqWarps + kIssuerWarps) {
        // ---------------- TMA: token tiles ----------------
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            for (int kb = 0; kb < num_kb; ++kb) {
                const bool okx = mbar_wait(ab_empty(s), ph ^ 1, s_abort);
                if (!okx) break;
                mbar_arrive_expect_tx(full(s), static_cast<uint32_t>(b_bytes));
                tma_load_2d(smem_u32(s_b + s * b_bytes), &a.tmap_x, (kb_begin + kb) * kBK, m0, full(s));
                if (++s == S) { s = 0; ph ^= 1; }
            }
        }
        __syncwarp();
        if (ksplit > 1) { cluster_sync_all(); cluster_sync_all(); }
    } else {
        // ---------------- TMA: raw packed weights ----------------
        if (lane == 0) {
            int rs = 0;
            uint32_t rph = 0;
            for (int sb = 0; sb < num_sb; ++sb) {
                if (!mbar_wait(raw_empty(rs), rph ^ 1, s_abort)) break;
                mbar_arrive_expect_tx(raw_full(rs), kRawBytes);
                tma_load_2d(smem_u32(s_raw + rs * kRawBytes), &a.tmap_w[t], (sb_begin + sb) * 128, n0, raw_full(rs));
                if (++rs == kRawStages) { rs = 0; rph ^= 1; }
            }
        }
        __syncwarp();
        if (ksplit > 1) { cluster_sync_all(); cluster_sync_all(); }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == kDqWarps) tmem_dealloc(tmem_base, static_cast<uint32_t>(a.tmem_cols));
}


// ---- CTA pairs (cta_group::2) ---------------------------------------------------------------------------------
// Prefill-sized token tiles on the single-CTA kernel above are bound by shared memory: one 128 x 256 x 16
// instruction reads 12 KB of operands per 128 tensor-core cycles and every CTA fetches the whole 256-token
// tile from L2 (measured: 0.57 of the bf16 peak, 0.74 even with dequantisation and token loads switched off).
// Here two CTAs of a cluster -- two SMs -- share one 256-row x 256-token output tile: each dequantises ITS 128
// weight rows (the A operand, M = 256 split over the pair) and loads ITS 128 tokens (half of the B operand,
// N = 256 split over the pair); one thread of the leading CTA issues tcgen05.mma.cta_group::2, which reads
// both CTAs' shared memory and accumulates into both CTAs' tensor memory.  Per CTA and k-block that is 16 KB of
// tokens from L2 instead of 32 KB and 8 KB of operand reads per instruction instead of 12 KB.  The dequantised
// weights do not pass through shared memory at all: a dequantising thread owns a weight row, which is a lane of
// tensor memory, and writes its 64 fp16 values of a k-block there with tcgen05.st; the MMA takes A from tensor
// memory (columns 256.. next to the 256 accumulator columns, eight k-block stages) and only B from shared
// memory.  That removes the A tile's shared-memory writes and reads -- the kernel is bound by shared-memory
// bandwidth otherwise -- and leaves room for eight token stages.
//
// Synchronisation.  Every stage has ONE "full" barrier, in the leader: the dequantising warps of both CTAs
// arrive on it (the peer's through the cluster shared-memory window, after a proxy fence and with release at
// cluster scope) and both CTAs' token loads complete their bytes on it (each CTA loads its own half with the
// cta_group::2 form of the tensor copy; every load has one destination).  The leader's tcgen05.commit.cta_group::2
// arrives on the "empty" barrier of the stage in BOTH CTAs (a CTA mask of 3), and at the end on both
// "accumulator ready" barriers.  Raw weight rings are private to each CTA.
// All mbarrier waits are bounded as above; both cluster barriers are reached by every thread of both CTAs
// whatever happened before, and tensor memory is allocated and freed by the same warp of each CTA.
__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void mbar_arrive_remote_release(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t leader_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(leader_bar)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// arrives on the barrier at this shared-memory offset in both CTAs of the pair once the MMAs issued so far are done
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(static_cast<uint16_t>(3)) : "memory");
}
// Instruction descriptor of the pair: D fp32, A/B fp16, both K-major, M = 256 (128 rows per CTA), N = n.
__device__ __forceinline__ uint32_t make_idesc_pair(int n) {
    return (1u << 4) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(256 >> 4) << 24);
}

constexpr int kPairGroups = 4;
constexpr int kPairDqWarps = 4 * kPairGroups;
constexpr int kPairThreads = (kPairDqWarps + 3) * 32;   // + MMA warp, token TMA warp, weight TMA warp

// 16 consecutive 32-bit columns of this thread's tensor-memory lane, from registers.
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// D[tmem] (+)= A[tmem] * B[smem]^T over the CTA pair: A (this pair's 256 weight rows, 128 per CTA, 16 k as 8 packed
// columns) comes from tensor memory, B from both CTAs' shared memory.
__device__ __forceinline__ void tc_mma_f16_pair_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                                   uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
constexpr int kPairAccumCols = 256;          // accumulator: 256 tokens
constexpr int kPairACols = kBK / 2;          // one k-block of dequantised weights: 64 fp16 = 32 packed columns

constexpr int kPairTokens = 256;             // tokens of a pair's tile (128 loaded by each CTA)
constexpr int kPairStageTokens = kPairTokens;   // the staging buffer holds the whole tile's outputs of this CTA
constexpr int kPairStagePitch = kTileRows * 2;         // bytes per token row of the staging buffer
constexpr int kPairRawStages = 2;            // raw weight ring: 2 x 256 k ahead is ample; the room goes to token stages
constexpr int kPairStageBytes = kPairStageTokens * kPairStagePitch;

// Which 128-row tile of which tensor, and which tokens, a pair tile index stands for (this CTA's half).
struct PairTile {
    int t, n0, m0;
};
__device__ __forceinline__ PairTile pair_tile(const TcArgs& a, int pt, int n_pairs, int rank, bool qkv, int tokens) {
    PairTile r;
    // Tile order: panels of a.panel token tiles; inside a panel the token tile runs fastest.  With a panel of 4 the
    // tiles in flight at one time (one per CTA pair) cover 4 token tiles x about 18 row-tile pairs, and both the
    // token slabs and the packed weight rows are re-used out of L2; a panel of 1 (row tiles fastest) shares one
    // token slab among all tiles in flight but streams the whole weight matrix once per token tile, which is
    // right only while the matrix stays in L2 (the host picks).
    const int m_tiles = (a.M + tokens - 1) / tokens;
    const int per_panel = a.panel * n_pairs;
    const int panel = pt / per_panel;
    const int q = pt - panel * per_panel;
    const int w = min(a.panel, m_tiles - panel * a.panel);
    const int m_idx = panel * a.panel + q % w;
    int tile = 2 * (q / w) + rank;      // consecutive 128-row tiles form a pair
    r.t = 0;
    if (qkv) {
        if (tile >= a.tiles[0]) { tile -= a.tiles[0]; r.t = 1; }
        if (r.t == 1 && tile >= a.tiles[1]) { tile -= a.tiles[1]; r.t = 2; }
    }
    r.n0 = tile * kTileRows;
    r.m0 = m_idx * tokens;
    return r;
}

// Persistent: every pair walks the pair tiles p, p + P, ... (neighbouring indices share their tokens, so the token
// slab stays in L2 while the weights stream).  The rings of raw weights, dequantised weights (tensor memory)
// and tokens run on across tile boundaries, so the loaders fill them for the next tile while this tile's
// accumulators are drained.  The group scales are not staged: a dequantising thread reads the two scales of
// its row per 256-element super-block straight from global memory, one super-block ahead.
// Epilogue: fp32 accumulators -> fp16 -> a [token][row] staging tile in shared memory -> 16-byte row-contiguous
// stores (a warp writes 256 consecutive bytes of two token rows), residual added from 16-byte loads.
// T: tokens of a pair's tile, 256 or 128 (the host takes 128 where there are fewer 256-token tiles than CTA pairs).
template <int MODE, int T>
__global__ void __launch_bounds__(kPairThreads, 1) gemm_w4a16_tc_pair_kernel(const __grid_constant__ TcArgs a) {
    static_assert(T == 256 || T == 128, "token tile of the CTA-pair kernel");
    constexpr int NG = kPairGroups;
    constexpr int kDqWarps = kPairDqWarps;
    constexpr int kDqThreads = kDqWarps * 32;
    constexpr int Th = T / 2;
    constexpr int kPartTokens = T / 4;       // tokens each of the four warp groups drains
    constexpr int QN = kPartTokens / 16;     // 16-column tensor-memory loads per warp and tile
    constexpr int b_bytes = Th * 128;
    extern __shared__ uint8_t smem_raw_base[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw_base) + 1023) & ~uintptr_t(1023));
    const int S = a.stages, K = a.K;
    const int G = K / kGroup;
    uint8_t* s_raw = smem;
    uint8_t* s_b = s_raw + kPairRawStages * kRawBytes;
    uint8_t* s_stage = s_b + S * b_bytes;
    uint64_t* s_bar = reinterpret_cast<uint64_t*>(s_stage + kPairStageBytes);
    const uint32_t bar0 = smem_u32(s_bar);
    auto raw_full = [&](int i) { return bar0 + 8u * i; };
    auto raw_empty = [&](int i) { return bar0 + 8u * (kPairRawStages + i); };
    auto full = [&](int i) { return bar0 + 8u * (2 * kPairRawStages + i); };
    auto ab_empty = [&](int i) { return bar0 + 8u * (2 * kPairRawStages + 2 * kMaxStages + i); };
    const uint32_t accum_full = bar0 + 8u * (2 * kPairRawStages + 3 * kMaxStages);
    const uint32_t accum_empty = accum_full + 8u;
    uint32_t* s_tmem = reinterpret_cast<uint32_t*>(s_bar + (2 * kPairRawStages + 3 * kMaxStages + 2));
    volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int rank = static_cast<int>(cluster_cta_rank());
    const bool leader = rank == 0;
    const int pair_id = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const int n_pairs = (a.tiles[0] + a.tiles[1] + a.tiles[2]) / 2;
    const int total_pt = n_pairs * ((a.M + T - 1) / T);
    const int num_sb = K / 256, num_kb = K / kBK;

    if (tid == 0) {
        for (int i = 0; i < kPairRawStages; ++i) { mbar_init(raw_full(i), 1); mbar_init(raw_empty(i), kDqWarps); }
        // full: 4 warps of each CTA's dequantising group + the leader's expect_tx arrival
        for (int i = 0; i < S; ++i) { mbar_init(full(i), 2 * 4 + 1); mbar_init(ab_empty(i), 1); }
        mbar_init(accum_full, 1);
        mbar_init(accum_empty, 2 * kDqWarps);     // every draining warp of both CTAs
        *s_abort = 0;
        fence_barrier_init();
        tma_prefetch_desc(&a.tmap_x);
        tma_prefetch_desc(&a.tmap_w[0]);
    }
    if (warp == kDqWarps) {          // the same warp in both CTAs, the same shared-memory offset for the result
        tmem_alloc_pair(smem_u32(s_tmem), static_cast<uint32_t>(a.tmem_cols));
        tmem_relinquish_pair();
    }
    pdl_release_dependents();
    pdl_wait_prior_grids();
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();              // the peer's barriers exist before anything arrives on them from here
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem;

    if (warp < kDqWarps) {
        // ================= dequantise (thread = weight row = tensor-memory lane), then drain =================
        const int r = (warp & 3) * 32 + lane;
        const int part = warp >> 2;              // this group's k-block of every super-block, its token share when draining
        const int sw = r & 7;
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
        bool ok = true;
        int rs = 0;
        uint32_t rph = 0;
        int s = part;                            // ring position of this group's next k-block
        uint32_t ph = 0;
        while (s >= S) { s -= S; ph ^= 1; }
        uint32_t acc_ph = 0;
        const int my_tiles = pair_id < total_pt ? (total_pt - pair_id + num_pairs - 1) / num_pairs : 0;
        auto load_scales = [&](const PairTile& pt, int sb) -> uint32_t {
            const int row = pt.n0 + r;
            if (row >= a.rows[pt.t]) return 0u;   // rows past the tensor dequantise to zero
            return __ldg(reinterpret_cast<const uint32_t*>(a.scales[pt.t] + static_cast<size_t>(row) * G + 2 * sb));
        };
        // The dequantising cursor: (tile iteration, super-block) of the next k-block this group produces.  It runs
        // ahead of the draining below by one super-block, so that the tensor core has work while a tile's outputs
        // are still on their way to global memory.
        int cur_it = 0, cur_sb = 0;
        PairTile cur_pt = my_tiles > 0 ? pair_tile(a, pair_id, n_pairs, rank, MODE == kQkv, T) : PairTile{0, 0, 0};
        uint32_t sc_next = my_tiles > 0 ? load_scales(cur_pt, 0) : 0u;
        auto advance = [&]() {      // dequantises the cursor's k-block; false when a bounded wait ran out
            const uint32_t sc_pair = sc_next;
            const int sb = cur_sb;
            // move the cursor and fetch its scales one step ahead
            if (++cur_sb == num_sb) {
                cur_sb = 0;
                ++cur_it;
                if (cur_it < my_tiles) cur_pt = pair_tile(a, pair_id + cur_it * num_pairs, n_pairs, rank, MODE == kQkv, T);
            }
            if (cur_it < my_tiles) sc_next = load_scales(cur_pt, cur_sb);
            (void)sb;
            if (!warp_wait(raw_full(rs), rph, s_abort, lane)) return false;
            const uint8_t* raw_row = s_raw + rs * kRawBytes + r * 128;
            const int j = part;              // NG == 4: one k-block of the super-block per group
            if (!warp_wait(ab_empty(s), ph ^ 1, s_abort, lane)) return false;
            tc_fence_after();
            const uint4 w0 = *reinterpret_cast<const uint4*>(raw_row + (((2 * j) ^ sw) << 4));
            const uint4 w1 = *reinterpret_cast<const uint4*>(raw_row + (((2 * j + 1) ^ sw) << 4));
            const uint32_t words[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
            const uint16_t sbits = static_cast<uint16_t>(j < 2 ? (sc_pair & 0xFFFFu) : (sc_pair >> 16));
            const __half2 sc2 = __half2half2(__ushort_as_half(sbits));
            const uint32_t a_lane = lane_base + static_cast<uint32_t>(kPairAccumCols + s * kPairACols);
#pragma unroll
            for (int hw = 0; hw < 2; ++hw) {
                uint32_t cols[16];
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    __half2 h[4];
                    dequant_word_fp16(words[4 * hw + w], sc2, h);
#pragma unroll
                    for (int q = 0; q < 4; ++q) cols[4 * w + q] = *reinterpret_cast<const uint32_t*>(&h[q]);
                }
                tmem_st16(a_lane + 16u * hw, cols);
            }
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (leader) mbar_arrive(full(s));
                else mbar_arrive_remote_release(cluster_map_shared(full(s), 0));
                mbar_arrive(raw_empty(rs));
            }
            s += NG;
            while (s >= S) { s -= S; ph ^= 1; }
            if (++rs == kPairRawStages) { rs = 0; rph ^= 1; }
            return true;
        };
        // Every one of the 16 warps reaches every bar.sync of this loop, whatever its waits returned: a warp
        // whose bounded wait ran out has raised the abort flag, and all warps leave together right after the
        // first barrier of the tile.
        for (int it = 0; it < my_tiles; ++it) {
            const PairTile pt = pair_tile(a, pair_id + it * num_pairs, n_pairs, rank, MODE == kQkv, T);
            const int rows_t = a.rows[pt.t];
            while (ok && cur_it == it) ok = advance();          // the rest of this tile's k-blocks
            // Look-ahead: while the tensor core works off the tail of this tile, fill the ring with the first
            // k-blocks of the next one (S / NG per group, i.e. every stage once: those stages are freed by MMAs of
            // THIS tile, so the wait cannot depend on the draining below), so that the next tile starts the
            // moment its accumulators are free and keeps running while the outputs go to global memory.
            for (int la = 0; la < S / NG && ok && cur_it == it + 1 && cur_it < my_tiles; ++la) ok = advance();
            // ---- drain this tile: 128 weight rows of this CTA x T tokens ----
            if (ok) ok = warp_wait(accum_full, acc_ph, s_abort, lane);
            acc_ph ^= 1;
            asm volatile("bar.sync 1, %0;" ::"n"(kDqThreads) : "memory");
            if (*s_abort) break;             // the same answer in all 16 warps
            tc_fence_after();
            __half* out = a.out[pt.t];
            const int ld = a.out_ld[pt.t];
            constexpr int kOutPerRow = MODE == kSwiglu ? kTileRows / 2 : kTileRows;    // outputs of a token row in the tile
            const int n_out0 = MODE == kSwiglu ? pt.n0 / 2 : pt.n0;
            const int n_valid = MODE == kSwiglu ? max(0, min(kOutPerRow, (rows_t - pt.n0) / 2)) : max(0, min(kOutPerRow, rows_t - pt.n0));
            bool vec_ok = (ld % 8 == 0) && (reinterpret_cast<uintptr_t>(out) % 16 == 0) && (n_valid % 8 == 0) &&
                          (MODE != kPlain || a.residual == nullptr || reinterpret_cast<uintptr_t>(a.residual) % 16 == 0);
            if constexpr (MODE == kPlain) {
                for (int p = 0; p < a.num_peers; ++p) vec_ok = vec_ok && reinterpret_cast<uintptr_t>(a.peer_out[p]) % 16 == 0;
            }
            // (1) this warp's 32 rows x T / 4 tokens of the accumulators into registers; with that the tensor memory is
            // free, and the next tile's first MMA may overwrite it while the values are still being stored
            uint32_t v[QN][16];
#pragma unroll
            for (int q = 0; q < QN; ++q) tmem_ld16(lane_base + static_cast<uint32_t>(part * kPartTokens + q * 16), v[q]);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (leader) mbar_arrive(accum_empty);
                else mbar_arrive_remote_release(cluster_map_shared(accum_empty, 0));
            }
            // (2) fp32 -> fp16 -> staging tile [token][row]
#pragma unroll
            for (int q = 0; q < QN; ++q) {
                const int tok0 = part * kPartTokens + q * 16;
#pragma unroll
                for (int jj = 0; jj < 16; ++jj) {
                    const float acc = __uint_as_float(v[q][jj]);
                    uint8_t* row_ptr = s_stage + (tok0 + jj) * kPairStagePitch;
                    if constexpr (MODE == kSwiglu) {
                        const float up = __shfl_xor_sync(0xFFFFFFFFu, acc, 1);
                        if ((lane & 1) == 0)
                            reinterpret_cast<__half*>(row_ptr)[r >> 1] = __float2half_rn((acc / (1.0f + expf(-acc))) * up);
                    } else {
                        reinterpret_cast<__half*>(row_ptr)[r] = __float2half_rn(acc);
                    }
                }
            }
            asm volatile("bar.sync 1, %0;" ::"n"(kDqThreads) : "memory");       // the staging tile is complete
            // (3) staging -> global, row-contiguous
            constexpr int kSegs = kOutPerRow / 8;            // 16-byte segments per token row
            if (vec_ok) {
                for (int idx = tid; idx < T * kSegs; idx += kDqThreads) {
                    const int tok = idx / kSegs, seg = idx - tok * kSegs;
                    const int m = pt.m0 + tok;
                    if (m < a.M && seg * 8 < n_valid) {
                        uint4 val = *reinterpret_cast<const uint4*>(s_stage + tok * kPairStagePitch + seg * 16);
                        const size_t off = static_cast<size_t>(m) * ld + n_out0 + seg * 8;
                        if constexpr (MODE == kPlain) {
                            if (a.residual != nullptr) {
                                const uint4 res = *reinterpret_cast<const uint4*>(a.residual + off);
                                __half2* vh = reinterpret_cast<__half2*>(&val);
                                const __half2* rh = reinterpret_cast<const __half2*>(&res);
#pragma unroll
                                for (int e = 0; e < 4; ++e) vh[e] = __hadd2(vh[e], rh[e]);
                            }
                        }
                        *reinterpret_cast<uint4*>(out + off) = val;
                        if constexpr (MODE == kPlain) {     // the block's place in the other GPUs' matrices: 16-byte stores over NVLink
                            for (int p = 0; p < a.num_peers; ++p) *reinterpret_cast<uint4*>(a.peer_out[p] + off) = val;
                        }
                    }
                }
            } else {
                for (int idx = tid; idx < T * kOutPerRow; idx += kDqThreads) {
                    const int tok = idx / kOutPerRow, c = idx - tok * kOutPerRow;
                    const int m = pt.m0 + tok;
                    if (m < a.M && c < n_valid) {
                        __half y = reinterpret_cast<const __half*>(s_stage + tok * kPairStagePitch)[c];
                        const size_t off = static_cast<size_t>(m) * ld + n_out0 + c;
                        if constexpr (MODE == kPlain) {
                            if (a.residual != nullptr) y = __hadd(y, a.residual[off]);
                        }
                        out[off] = y;
                        if constexpr (MODE == kPlain) {
                            for (int p = 0; p < a.num_peers; ++p) a.peer_out[p][off] = y;
                        }
                    }
                }
            }
            asm volatile("bar.sync 1, %0;" ::"n"(kDqThreads) : "memory");   // the staging tile is free again
        }
    } else if (warp == kDqWarps) {
        // ================= MMA issue: the leading CTA only =================
        if (leader) {
            const uint32_t idesc = make_idesc_pair(T);
            const uint64_t b_desc0 = make_smem_desc(smem_u32(s_b));
            constexpr uint32_t b_step = static_cast<uint32_t>(b_bytes) >> 4;
            const uint32_t a_tmem0 = tmem_base + kPairAccumCols;
            uint64_t b_desc = b_desc0;
            uint32_t a_tmem = a_tmem0;
            int s = 0;
            uint32_t ph = 0, empty_ph = 0;
            bool ok = true;
            for (int pt_i = pair_id, it = 0; pt_i < total_pt && ok; pt_i += num_pairs, ++it) {
                if (it > 0) {            // both CTAs have drained the previous tile's accumulators
                    ok = warp_wait(accum_empty, empty_ph, s_abort, lane);
                    empty_ph ^= 1;
                    if (!ok) break;
                }
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_test_wait(full(s), ph)) ok = warp_wait(full(s), ph, s_abort, lane);
                    if (!ok) break;
                    tc_fence_after();
                    if (lane == 0) {
#pragma unroll
                        for (int ks = 0; ks < kBK / 16; ++ks)
                            tc_mma_f16_pair_ts(tmem_base, a_tmem + 8u * ks, b_desc + 2 * ks, idesc, (kb | ks) != 0 ? 1u : 0u);
                        tc_commit_pair(ab_empty(s));
                    }
                    __syncwarp();
                    a_tmem += kPairACols;
                    b_desc += b_step;
                    if (++s == S) { s = 0; ph ^= 1; a_tmem = a_tmem0; b_desc = b_desc0; }
                }
                if (ok && lane == 0) tc_commit_pair(accum_full);
                __syncwarp();
            }
        }
        __syncwarp();
    } else if (warp == kDqWarps + 1) {
        // ================= TMA: this CTA's half of the token tile; bytes counted on the LEADER's barrier =================
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int pt_i = pair_id; pt_i < total_pt && ok; pt_i += num_pairs) {
                const PairTile pt = pair_tile(a, pt_i, n_pairs, rank, MODE == kQkv, T);
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(ab_empty(s), ph ^ 1, s_abort)) { ok = false; break; }
                    if (leader) mbar_arrive_expect_tx(full(s), static_cast<uint32_t>(2 * b_bytes));
                    tma_load_2d_pair(smem_u32(s_b + s * b_bytes), &a.tmap_x, kb * kBK, pt.m0 + rank * Th,
                                     cluster_map_shared(full(s), 0));
                    if (++s == S) { s = 0; ph ^= 1; }
                }
            }
        }
        __syncwarp();
    } else {
        // ================= TMA: raw packed weights of this CTA's 128 rows (private ring) =================
        if (lane == 0) {
            int rs = 0;
            uint32_t rph = 0;
            bool ok = true;
            for (int pt_i = pair_id; pt_i < total_pt && ok; pt_i += num_pairs) {
                const PairTile pt = pair_tile(a, pt_i, n_pairs, rank, MODE == kQkv, T);
                for (int sb = 0; sb < num_sb; ++sb) {
                    if (!mbar_wait(raw_empty(rs), rph ^ 1, s_abort)) { ok = false; break; }
                    mbar_arrive_expect_tx(raw_full(rs), kRawBytes);
                    tma_load_2d(smem_u32(s_raw + rs * kRawBytes), &a.tmap_w[pt.t], sb * 128, pt.n0, raw_full(rs));
                    if (++rs == kPairRawStages) { rs = 0; rph ^= 1; }
                }
            }
        }
        __syncwarp();
    }

    // Neither CTA may leave (or free its tensor memory) while the other's instructions can still touch its
    // shared memory, barriers or accumulators.
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == kDqWarps) tmem_dealloc_pair(tmem_base, static_cast<uint32_t>(a.tmem_cols));
}

// ---- host side ----------------------------------------------------------------------------

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// Encoded maps are kept per (pointer, shape, box): a model's weight matrices and an engine's activation buffers
// come back launch after launch, and an encode costs the host a microsecond or two.  A map holds nothing but the
// address and the geometry, so an entry stays valid even if the memory behind it was freed and handed out again.
struct MapKey {
    const void* base;
    uint64_t inner, outer, row_bytes;
    uint32_t box_inner, box_outer;
    int dt;
    bool operator==(const MapKey& o) const {
        return base == o.base && inner == o.inner && outer == o.outer && row_bytes == o.row_bytes &&
               box_inner == o.box_inner && box_outer == o.box_outer && dt == o.dt;
    }
};
constexpr size_t kMapCacheEntries = 256;

bool encode_2d(CUtensorMap* map, CUtensorMapDataType dt, const void* base, uint64_t inner, uint64_t outer,
               uint64_t row_bytes, uint32_t box_inner, uint32_t box_outer) {
    static std::mutex mu;
    static std::vector<std::pair<MapKey, CUtensorMap>> cache;
    static size_t next = 0;
    const MapKey key{base, inner, outer, row_bytes, box_inner, box_outer, static_cast<int>(dt)};
    {
        std::lock_guard<std::mutex> lock(mu);
        for (const auto& kv : cache)
            if (kv.first == key) { *map = kv.second; return true; }
    }
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {inner, outer};
    const cuuint64_t strides[1] = {row_bytes};
    const cuuint32_t box[2] = {box_inner, box_outer};
    const cuuint32_t estr[2] = {1, 1};
    if (fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    std::lock_guard<std::mutex> lock(mu);
    if (cache.size() < kMapCacheEntries) cache.emplace_back(key, *map);
    else { cache[next] = {key, *map}; next = (next + 1) % kMapCacheEntries; }
    return true;
}

size_t tc_smem_bytes(int T, int S, int K) {
    const size_t G = K / kGroup;
    return 1024 + static_cast<size_t>(kRawStages) * kRawBytes + static_cast<size_t>(S) * (kABytes + T * 128) +
           ((G * kTileRows * 2 + 15) & ~size_t(15)) + (2 * kRawStages + 3 * kMaxStages + 1) * 8 + 16;
}

size_t tc_pair_smem_bytes(int S) {     // per CTA: raw weight ring, token halves, epilogue staging, barriers
    return 1024 + static_cast<size_t>(kPairRawStages) * kRawBytes + static_cast<size_t>(S) * ((kPairTokens / 2) * 128) +
           kPairStageBytes + (2 * kPairRawStages + 3 * kMaxStages + 2) * 8 + 16;
}

}  // namespace

namespace {
template <int MODE, int NG>
cudaError_t raise_tc_smem() {
    cudaError_t e = cudaFuncSetAttribute(gemm_w4a16_tc_kernel<MODE, NG, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(gemm_w4a16_tc_kernel<MODE, NG, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    return e;
}
template <int NG>
cudaError_t raise_tc_smem_modes() {
    cudaError_t e = raise_tc_smem<kPlain, NG>();
    if (e == cudaSuccess) e = raise_tc_smem<kQkv, NG>();
    if (e == cudaSuccess) e = raise_tc_smem<kSwiglu, NG>();
    return e;
}
template <int NG>
cudaError_t launch_tc(int mode, dim3 grid, size_t smem, cudaStream_t stream, const TcArgs& a) {
    const dim3 cluster(1, 1, static_cast<unsigned>(a.ksplit));   // the K slices of one output tile
    const bool extras = a.ksplit > 1 || a.issuers > 1 || a.num_peers > 0;
    const dim3 block((4 * NG + (extras ? kMaxIssuers : 1) + 2) * 32);
    const bool pdl = pdl_enabled();
#define W4_TC_LAUNCH(M_, X_) launch_kernel_cluster(gemm_w4a16_tc_kernel<M_, NG, X_>, grid, block, smem, stream, pdl, cluster, a)
    switch (mode) {
        case kPlain: return extras ? W4_TC_LAUNCH(kPlain, true) : W4_TC_LAUNCH(kPlain, false);
        case kQkv: return extras ? W4_TC_LAUNCH(kQkv, true) : W4_TC_LAUNCH(kQkv, false);
        default: return extras ? W4_TC_LAUNCH(kSwiglu, true) : W4_TC_LAUNCH(kSwiglu, false);
    }
#undef W4_TC_LAUNCH
}
}  // namespace


int groups_for(int S) { return S >= 4 ? 4 : 2; }

// Clusters of `ksplit` CTAs of the K-split kernel that can be resident at once on the current device (cached).
int max_active_clusters(int mode, int groups, int ksplit, size_t smem) {
    static std::mutex mu;
    static std::vector<std::pair<uint64_t, int>> cache;
    int dev = 0;
    cudaGetDevice(&dev);
    const uint64_t key = (static_cast<uint64_t>(dev) << 48) ^ (static_cast<uint64_t>(mode) << 40) ^ (static_cast<uint64_t>(groups) << 36) ^
                         (static_cast<uint64_t>(ksplit) << 32) ^ static_cast<uint64_t>(smem);
    {
        std::lock_guard<std::mutex> lock(mu);
        for (const auto& kv : cache)
            if (kv.first == key) return kv.second;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1, 1, static_cast<unsigned>(ksplit));
    cfg.blockDim = dim3((4 * groups + kMaxIssuers + 2) * 32);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = static_cast<unsigned>(ksplit);
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    cudaError_t e;
#define W4_OCC(M_, G_) cudaOccupancyMaxActiveClusters(&n, gemm_w4a16_tc_kernel<M_, G_, true>, &cfg)
    if (groups == 2) e = mode == kPlain ? W4_OCC(kPlain, 2) : mode == kQkv ? W4_OCC(kQkv, 2) : W4_OCC(kSwiglu, 2);
    else e = mode == kPlain ? W4_OCC(kPlain, 4) : mode == kQkv ? W4_OCC(kQkv, 4) : W4_OCC(kSwiglu, 4);
#undef W4_OCC
    if (e != cudaSuccess) { cudaGetLastError(); n = 1 << 20; }   // unknown: do not restrict
    std::lock_guard<std::mutex> lock(mu);
    cache.emplace_back(key, n);
    return n;
}

int gemm_tc_set_attributes() {
    cudaError_t e = cudaSuccess;
    auto raise_pair = [&e](auto* kernel) {
        if (e == cudaSuccess) e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    };
    raise_pair(gemm_w4a16_tc_pair_kernel<kPlain, 256>);
    raise_pair(gemm_w4a16_tc_pair_kernel<kQkv, 256>);
    raise_pair(gemm_w4a16_tc_pair_kernel<kSwiglu, 256>);
    raise_pair(gemm_w4a16_tc_pair_kernel<kPlain, 128>);
    raise_pair(gemm_w4a16_tc_pair_kernel<kQkv, 128>);
    raise_pair(gemm_w4a16_tc_pair_kernel<kSwiglu, 128>);
    if (e == cudaSuccess) e = raise_tc_smem_modes<2>();
    if (e == cudaSuccess) e = raise_tc_smem_modes<4>();
    return static_cast<int>(e);
}

// Can the tensor-core kernel take this problem?  (alignment for TMA, tile-aligned QKV tensors)
bool gemm_tc_supported(const GemmArgs& g) {
    if (encode_tiled_fn() == nullptr) return false;
    const int nt = g.mode == kQkv ? 3 : 1;
    for (int t = 0; t < nt; ++t) {
        if (reinterpret_cast<uintptr_t>(g.qweight[t]) % 16) return false;
        if (g.mode == kQkv && g.rows[t] % kTileRows) return false;
    }
    if (reinterpret_cast<uintptr_t>(g.x) % 16) return false;
    // scales tile must fit next to at least two pipeline stages
    return tc_smem_bytes(16, 2, g.K) <= 227 * 1024;
}

int gemm_tc_launch(const GemmArgs& g, int sm_count, cudaStream_t stream) {
    TcArgs a;
    a.panel = 1;
    const int nt = g.mode == kQkv ? 3 : 1;
    int total_tiles = 0;
    for (int t = 0; t < 3; ++t) {
        a.scales[t] = g.scales[t];
        a.out[t] = g.out[t];
        a.rows[t] = t < nt ? g.rows[t] : 0;
        a.tiles[t] = (a.rows[t] + kTileRows - 1) / kTileRows;
        total_tiles += a.tiles[t];
        a.out_ld[t] = g.mode == kSwiglu ? g.rows[0] / 2 : a.rows[t];
        if (g.mode == kPlain && t == 0 && g.ldc > 0) a.out_ld[0] = g.ldc;
    }
    a.residual = g.residual;
    a.M = g.M;
    a.K = g.K;
    a.num_peers = g.mode == kPlain ? g.num_peers : 0;
    for (int p = 0; p < 7; ++p) a.peer_out[p] = p < a.num_peers ? g.peer_out[p] : nullptr;
    // CTA pairs (cta_group::2) from 256 tokens on: 256-token tiles, no K split, an even number of
    // 128-row tiles in every weight tensor (a pair never straddles two tensors) and 4-byte aligned scales (read
    // in pairs).  Measured faster than the single-CTA form from about 20 pair tiles on (a quarter of the GPU's 74
    // pairs busy); with fewer, narrower token tiles on more CTAs win.  W4A16_OPT_GEMM_FORM = 2 forces pairs.
    const int pair_tiles_256 = (total_tiles / 2) * ((g.M + 255) / 256);
    bool pairs = option(W4A16_OPT_GEMM_FORM) != 1 && g.M >= 256 &&
                 (pair_tiles_256 >= 20 || option(W4A16_OPT_GEMM_FORM) == 2);
    for (int t = 0; t < nt; ++t)
        pairs = pairs && a.tiles[t] % 2 == 0 && reinterpret_cast<uintptr_t>(g.scales[t]) % 4 == 0;
    // tokens per tile: the smallest power of two >= M (16..256); halve it while the grid is thin
    int T = 16;
    while (T < g.M && T < 256) T *= 2;
    while (!pairs && T > 64 && total_tiles * ((g.M + T - 1) / T) < sm_count) T /= 2;
    int S = kMaxStages;
    while (S > 2 && tc_smem_bytes(T, S, g.K) > 227 * 1024) --S;
    if (tc_smem_bytes(T, S, g.K) > 227 * 1024) return W4A16_ERR_TOO_LARGE;
    a.T = T;
    a.stages = S;
    // two issuing warps for token tiles of at most 128 (measured: gate_up at 16 tokens 18.3 -> 14.3 us, down at 128
    // tokens 39.0 -> 30.5 us; at 256 tokens the tensor pipe, not the issue, paces the loop and one warp is as fast);
    // each has its own accumulator, so the column count doubles
    a.issuers = T <= 128 ? 2 : 1;
    while (a.issuers > 1 && a.issuers * T > 512) --a.issuers;
    int cols = 32;
    while (cols < a.issuers * T) cols *= 2;
    a.tmem_cols = cols;
    // Split K over a cluster when the output tiles alone leave most SMs idle (decode batches on the per-layer
    // shapes): each tensor-core instruction costs its issuing thread a fixed time however few tokens it
    // carries, so a thin grid is bound by K / 16 instructions in a row per CTA.  Up to 8 CTAs (the portable
    // cluster size) share a tile; their fp32 partials must fit the leader's pipeline buffers.
    const int ctas = total_tiles * ((g.M + T - 1) / T);
    int ksplit = 1;
    if (!pairs && ctas * 2 <= sm_count) ksplit = std::min(8, sm_count / ctas);
    ksplit = std::min(ksplit, g.K / 256);
    const size_t ring_bytes = static_cast<size_t>(kRawStages) * kRawBytes + static_cast<size_t>(S) * (kABytes + T * 128);
    while (ksplit > 1 && static_cast<size_t>(ksplit - 1) * T * kTileRows * sizeof(float) > ring_bytes) --ksplit;
    a.ksplit = std::max(1, ksplit);
    // All clusters of a K-split launch should be resident at once (a second wave doubles the time).  How many fit
    // depends on how the SMs are spread over the GPCs, so the runtime is asked; fewer slices until they do.
    while (a.ksplit > 1 && max_active_clusters(g.mode, groups_for(S), a.ksplit, tc_smem_bytes(T, S, g.K)) < ctas) --a.ksplit;


    for (int t = 0; t < nt; ++t) {
        if (!encode_2d(&a.tmap_w[t], CU_TENSOR_MAP_DATA_TYPE_UINT8, g.qweight[t], static_cast<uint64_t>(g.K / 2),
                       static_cast<uint64_t>(g.rows[t]), static_cast<uint64_t>(g.K / 2), 128, kTileRows))
            return W4A16_ERR_INVALID_ARG;
    }
    for (int t = nt; t < 3; ++t) a.tmap_w[t] = a.tmap_w[0];

    if (pairs) {
        int SP = kMaxStages;
        while (SP > 2 && tc_pair_smem_bytes(SP) > 227 * 1024) --SP;
        a.stages = SP;
        a.issuers = 1;
        a.tmem_cols = 512;      // 256 accumulator columns + up to 8 stages x 32 columns of dequantised weights
        // weight matrices that do not stay in L2 next to the tokens and outputs: panels of 4 token tiles (measured on
        // 28672 x 8192 at 4096 tokens: 1.62 -> 1.56 ms, DRAM reads 1.77 -> under 1 GB); smaller ones: row tiles fastest
        const size_t weight_bytes = static_cast<size_t>(total_tiles) * kTileRows * (g.K / 2);
        a.panel = weight_bytes > (48u << 20) ? 4 : 1;
        // Token tile: 256, or 128 where the 256-token tiles are fewer than the CTA pairs (QKV, O, down at 1024 tokens:
        // 24-32 tiles on 74 pairs; half-size tiles keep twice as many pairs busy: 19.7 -> 18.1, 19.5 -> 17.7 us).  With
        // more tiles than pairs the half-size tile loses: a tile's dequantisation costs the same for half the MMA
        // work (O and down at 4096 tokens: 34 -> 43 and 148 -> 205 us).
        const int pairs_avail = std::max(1, sm_count / 2);
        const int tiles256 = (total_tiles / 2) * ((g.M + 255) / 256);
        T = tiles256 < pairs_avail ? 128 : 256;
        a.T = T;
        if (!encode_2d(&a.tmap_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, g.x, static_cast<uint64_t>(g.K),
                       static_cast<uint64_t>(g.M), static_cast<uint64_t>(g.K) * 2, kBK, static_cast<uint32_t>(T / 2)))
            return W4A16_ERR_INVALID_ARG;
        // persistent: one pair per two SMs, each walking the pair tiles p, p + P, ...
        const int pair_tiles = (total_tiles / 2) * ((g.M + T - 1) / T);
        const int num_pairs = std::max(1, std::min(sm_count / 2, pair_tiles));
        const dim3 pgrid(2 * num_pairs, 1, 1), pblock(kPairThreads), pcluster(2, 1, 1);
        const size_t psmem = tc_pair_smem_bytes(SP);
        const bool pdl = pdl_enabled();
        cudaError_t pe;
#define W4_PAIR_LAUNCH(M_) (T == 128 ? launch_kernel_cluster(gemm_w4a16_tc_pair_kernel<M_, 128>, pgrid, pblock, psmem, stream, pdl, pcluster, a) \
                                      : launch_kernel_cluster(gemm_w4a16_tc_pair_kernel<M_, 256>, pgrid, pblock, psmem, stream, pdl, pcluster, a))
        switch (g.mode) {
            case kPlain: pe = W4_PAIR_LAUNCH(kPlain); break;
            case kQkv: pe = W4_PAIR_LAUNCH(kQkv); break;
            default: pe = W4_PAIR_LAUNCH(kSwiglu); break;
        }
#undef W4_PAIR_LAUNCH
        return static_cast<int>(pe);
    }
    if (!encode_2d(&a.tmap_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, g.x, static_cast<uint64_t>(g.K),
                   static_cast<uint64_t>(g.M), static_cast<uint64_t>(g.K) * 2, kBK, static_cast<uint32_t>(T)))
        return W4A16_ERR_INVALID_ARG;

    const dim3 grid(total_tiles, (g.M + T - 1) / T, a.ksplit);
    const size_t smem = tc_smem_bytes(T, S, g.K);
    // A dequantising group revisits a ring slot every NG k-blocks and waits on a parity: it must never
    // be two uses of a slot ahead of the tensor core, which holds exactly when NG <= stages.
    const int groups = groups_for(S);
    const cudaError_t e = groups == 2 ? launch_tc<2>(g.mode, grid, smem, stream, a) : launch_tc<4>(g.mode, grid, smem, stream, a);
    return static_cast<int>(e);
}

int gemm_tc_timeouts(unsigned int* out) {
    return static_cast<int>(cudaMemcpyFromSymbol(out, g_tc_wait_timeouts, sizeof(unsigned int)));
}

}  // namespace w4
