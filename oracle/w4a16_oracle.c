/*
 * CPU oracle for the W4A16 group-128 contraction path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is a plain-C restatement of the arithmetic that the reference engine
 * (Areen-09/qwen-engine) performs on the GPU for its W4 projections.  It exists to
 * check the CUDA kernels of this repository and to be timed as the CPU baseline.
 * Nothing in the product path links, imports or calls it: only the tests, the smoke
 * check and the cpu_baseline / reference arm of the benchmark do.
 *
 * Every function names the reference lines it follows (paths relative to the
 * reference project root).  Where the reference has three behaviours for the same
 * expression (device code built with fast-math, device code as written, and the CPU
 * check in its test), the canonical one here is "IEEE fp32 as written, round half to
 * even", and the test's CPU flavour (round half away) is available as round_mode 1.
 *
 * Parity pin: nibble packing and weight quantisation are checked against vectors made
 * by the reference's own Python packer; Q8_1, per-group integer dots and fp16 outputs
 * are checked against vectors made by the reference's CUDA kernels rebuilt for sm_100a
 * (tests/golden/).
 *
 * fp16 values cross this interface as raw uint16_t bit patterns.
 * Build: gcc -O3 -fno-fast-math -ffp-contract=off -shared -fPIC -pthread (see Makefile).
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))
#define GROUP 128

/* ------------------------------------------------------------------------- */
/* fp16 helpers: _Float16 conversions are IEEE round-to-nearest-even.         */
/* ------------------------------------------------------------------------- */
static inline float h2f(uint16_t b) {
    _Float16 h;
    memcpy(&h, &b, 2);
    return (float)h;
}
static inline uint16_t f2h(float f) {
    _Float16 h = (_Float16)f;
    uint16_t b;
    memcpy(&b, &h, 2);
    return b;
}
/* one rounding, straight from double (used where the exact value is known in double) */
static inline uint16_t d2h(double d) {
    _Float16 h = (_Float16)d;
    uint16_t b;
    memcpy(&b, &h, 2);
    return b;
}

/* ------------------------------------------------------------------------- */
/* small parallel-for over a row range                                        */
/* ------------------------------------------------------------------------- */
typedef void (*row_fn)(int64_t r0, int64_t r1, void* ctx);
typedef struct {
    row_fn fn;
    void* ctx;
    int64_t r0, r1;
} job_t;
static void* job_main(void* p) {
    job_t* j = (job_t*)p;
    j->fn(j->r0, j->r1, j->ctx);
    return NULL;
}
static void parallel_rows(int64_t n, int nthreads, row_fn fn, void* ctx) {
    if (nthreads <= 1 || n < 2) {
        fn(0, n, ctx);
        return;
    }
    if (nthreads > 256) nthreads = 256;
    if ((int64_t)nthreads > n) nthreads = (int)n;
    pthread_t th[256];
    job_t jobs[256];
    int64_t per = (n + nthreads - 1) / nthreads;
    int started = 0;
    for (int t = 0; t < nthreads; ++t) {
        int64_t a = t * per, b = a + per;
        if (a >= n) break;
        if (b > n) b = n;
        jobs[t].fn = fn;
        jobs[t].ctx = ctx;
        jobs[t].r0 = a;
        jobs[t].r1 = b;
        if (pthread_create(&th[t], NULL, job_main, &jobs[t]) != 0) {
            fn(a, b, ctx); /* no thread: do it here */
            th[t] = 0;
            jobs[t].fn = NULL;
        }
        started = t + 1;
    }
    for (int t = 0; t < started; ++t)
        if (jobs[t].fn) pthread_join(th[t], NULL);
}

/* ------------------------------------------------------------------------- */
/* Nibble order of one packed word.                                           */
/* include/quant_primitives.cuh:20-26, tools/export_qwen25.py:62-72:          */
/*   word = q0 | q4<<4 | q1<<8 | q5<<12 | q2<<16 | q6<<20 | q3<<24 | q7<<28   */
/* so element j of the octet sits at bit 8*(j&3) + 4*(j>>2).                  */
/* ------------------------------------------------------------------------- */
static inline int nibble_shift(int j) { return 8 * (j & 3) + 4 * (j >> 2); }

/* q: [N][K] values 0..15  ->  packed: [N][K/8], linear in K. */
ORC_API void orc_pack_nibbles(const uint8_t* q, uint32_t* packed, int64_t N, int K) {
    int words = K / 8;
    for (int64_t n = 0; n < N; ++n)
        for (int w = 0; w < words; ++w) {
            uint32_t v = 0;
            for (int j = 0; j < 8; ++j)
                v |= (uint32_t)(q[n * K + w * 8 + j] & 0xF) << nibble_shift(j);
            packed[n * words + w] = v;
        }
}

ORC_API void orc_unpack_nibbles(const uint32_t* packed, uint8_t* q, int64_t N, int K) {
    int words = K / 8;
    for (int64_t n = 0; n < N; ++n)
        for (int w = 0; w < words; ++w) {
            uint32_t v = packed[n * words + w];
            for (int j = 0; j < 8; ++j) q[n * K + w * 8 + j] = (v >> nibble_shift(j)) & 0xF;
        }
}

/*
 * Weight quantiser + packer.  tools/export_qwen25.py:42-78 (same code in
 * tools/convert_gguf_to_qwenbin.py:64-97):
 *   scale = fp16(max|w| / 7); a zero scale is replaced by fp16(1e-5) for the division
 *   only (the stored scale stays 0); q = clip(round_half_even(w / scale) + 8, 0, 15).
 * The exporter's final reshape is an identity, so the packed row is linear in K.
 */
ORC_API void orc_quantize_weights(const float* w, int64_t N, int K, uint32_t* packed, uint16_t* scales) {
    int groups = K / GROUP, words = K / 8;
    const float tiny = h2f(f2h(1e-5f));
    for (int64_t n = 0; n < N; ++n) {
        for (int g = 0; g < groups; ++g) {
            const float* src = w + n * K + g * GROUP;
            float max_abs = 0.0f;
            for (int j = 0; j < GROUP; ++j) {
                float a = fabsf(src[j]);
                if (a > max_abs) max_abs = a;
            }
            uint16_t sb = f2h(max_abs / 7.0f);
            scales[n * groups + g] = sb;
            float s = h2f(sb);
            if (s == 0.0f) s = tiny;
            for (int wd = 0; wd < 16; ++wd) {
                uint32_t v = 0;
                for (int j = 0; j < 8; ++j) {
                    float r = nearbyintf(src[wd * 8 + j] / s) + 8.0f;
                    if (r < 0.0f) r = 0.0f;
                    if (r > 15.0f) r = 15.0f;
                    v |= (uint32_t)r << nibble_shift(j);
                }
                packed[n * words + g * 16 + wd] = v;
            }
        }
    }
}

/*
 * Q8_1 of the attention output, as the flash-decode combine step produces it for the O projection.
 * src/kernels/attention_gqa.cu:263-310: one group per head (head_dim elements, 128 in the model), taken
 * from the fp32 accumulator BEFORE it is rounded to fp16:
 *   d = max(max|acc| / 127, 1e-8);  q = clamp(rn(acc / d), -127, 127)   -- a division per element, where
 * the stand-alone quantiser above multiplies by 1/d, so the bytes can differ from quantising fp16(acc);
 * sum8 per octet as above; attn_out = fp16(acc) (attention_gqa.cu:260).
 * acc: [heads][head_dim] fp32.  out_fp16 / scale / sum8 may be NULL.  Round half to even.
 */
ORC_API void orc_quantize_heads_f32(const float* acc, int heads, int head_dim, uint16_t* out_fp16, int8_t* q8,
                                    float* scale, int32_t* sum8) {
    for (int h = 0; h < heads; ++h) {
        const float* a = acc + (int64_t)h * head_dim;
        float max_abs = 0.0f;
        for (int j = 0; j < head_dim; ++j) max_abs = fmaxf(max_abs, fabsf(a[j]));
        const float d = fmaxf(max_abs / 127.0f, 1e-8f);
        if (scale) scale[h] = d;
        for (int o = 0; o < head_dim / 8; ++o) {
            int32_t s = 0;
            for (int j = 0; j < 8; ++j) {
                const float v = a[o * 8 + j];
                int q = (int)nearbyintf(v / d);
                if (q < -127) q = -127;
                if (q > 127) q = 127;
                q8[(int64_t)h * head_dim + o * 8 + j] = (int8_t)q;
                s += q;
                if (out_fp16) out_fp16[(int64_t)h * head_dim + o * 8 + j] = f2h(v);
            }
            if (sum8) sum8[(int64_t)h * (head_dim / 8) + o] = -8 * s;
        }
    }
}

/*
 * Q8_1 activation quantiser, the reference's own flavour: int8 q8[n], fp32
 * scale[n/128], int32 sum8[n/8] with sum8[i] = -8 * sum of the octet's q8.
 * include/quant_primitives.cuh:37-89 (sum8: :13-17):
 *   d = max(max|x| / 127, 1e-8);  inv_d = 1 / d;  q = clamp(rn(x * inv_d), -127, 127).
 * round_mode 0: round half to even (the device's __float2int_rn; canonical).
 * round_mode 1: round half away from zero (std::round in tests/test_kernels.cu:317-323).
 * The outputs scale/sum8 may be NULL.
 */
ORC_API void orc_quantize_q8_1(const uint16_t* x, int64_t n, int8_t* q8, float* scale, int32_t* sum8,
                               int round_mode) {
    int64_t groups = n / GROUP;
    for (int64_t g = 0; g < groups; ++g) {
        float v[GROUP];
        float max_abs = 0.0f;
        for (int j = 0; j < GROUP; ++j) {
            v[j] = h2f(x[g * GROUP + j]);
            max_abs = fmaxf(max_abs, fabsf(v[j]));
        }
        float d = fmaxf(max_abs / 127.0f, 1e-8f);
        float inv_d = 1.0f / d;
        if (scale) scale[g] = d;
        for (int o = 0; o < 16; ++o) {
            int32_t s = 0;
            for (int j = 0; j < 8; ++j) {
                float t = v[o * 8 + j] * inv_d;
                int q = (int)(round_mode == 1 ? roundf(t) : nearbyintf(t));
                if (q < -127) q = -127;
                if (q > 127) q = 127;
                q8[g * GROUP + o * 8 + j] = (int8_t)q;
                s += q;
            }
            if (sum8) sum8[g * 16 + o] = -8 * s;
        }
    }
}

/* unpack one packed row into signed (q - 8) bytes, linear in K */
static inline void unpack_row_centered(const uint32_t* row, int K, int8_t* out) {
    for (int w = 0; w < K / 8; ++w) {
        uint32_t v = row[w];
        out[w * 8 + 0] = (int8_t)((v >> 0) & 0xF) - 8;
        out[w * 8 + 1] = (int8_t)((v >> 8) & 0xF) - 8;
        out[w * 8 + 2] = (int8_t)((v >> 16) & 0xF) - 8;
        out[w * 8 + 3] = (int8_t)((v >> 24) & 0xF) - 8;
        out[w * 8 + 4] = (int8_t)((v >> 4) & 0xF) - 8;
        out[w * 8 + 5] = (int8_t)((v >> 12) & 0xF) - 8;
        out[w * 8 + 6] = (int8_t)((v >> 20) & 0xF) - 8;
        out[w * 8 + 7] = (int8_t)((v >> 28) & 0xF) - 8;
    }
}

static inline int32_t dot_i8(const int8_t* a, const int8_t* b, int n) {
    int32_t s = 0;
    for (int i = 0; i < n; ++i) s += (int32_t)a[i] * (int32_t)b[i];
    return s;
}

/* ------------------------------------------------------------------------- */
/* Per-group integer dots D[n][g] = sum_{k in g} (q[n][k] - 8) * x_q8[k].      */
/* The quantity dp4a_w4_q8_oct accumulates (include/quant_primitives.cuh:28-32)*/
/* summed over the 16 octets of a group; tests/test_kernels.cu:337-353.       */
/* ------------------------------------------------------------------------- */
typedef struct {
    const uint32_t* packed;
    const int8_t* q8;
    int K;
    int32_t* D;
} gd_ctx;
static void gd_rows(int64_t r0, int64_t r1, void* p) {
    gd_ctx* c = (gd_ctx*)p;
    int K = c->K, groups = K / GROUP;
    int8_t* wrow = (int8_t*)malloc((size_t)K);
    for (int64_t n = r0; n < r1; ++n) {
        unpack_row_centered(c->packed + n * (K / 8), K, wrow);
        for (int g = 0; g < groups; ++g)
            c->D[n * groups + g] = dot_i8(wrow + g * GROUP, c->q8 + g * GROUP, GROUP);
    }
    free(wrow);
}
ORC_API void orc_group_dots(const uint32_t* packed, const int8_t* q8, int64_t N, int K, int32_t* D,
                            int nthreads) {
    gd_ctx c = {packed, q8, K, D};
    parallel_rows(N, nthreads, gd_rows, &c);
}

/* ------------------------------------------------------------------------- */
/* W4A8 GEMV golden on Q8_1 activations.                                      */
/* tests/test_kernels.cu:330-357: per group, int32 dot times                  */
/* (float(w_scale) * x_scale) [an fp32 product], accumulated in double.       */
/* Epilogue as the kernels do it (src/kernels/gemv_w4a16.cu:116-120):         */
/* + float(residual), one rounding to fp16.                                   */
/* y64 (optional) receives the double value before the fp16 rounding.         */
/* mode 0: y[n] for n < N.   mode 1 (SwiGLU, :252-257, test :359-362): rows   */
/* 2i / 2i+1 are gate / up, y[i] = silu(gate) * up for i < N/2.               */
/* ------------------------------------------------------------------------- */
typedef struct {
    const uint32_t* packed;
    const uint16_t* scales;
    const int8_t* q8;
    const float* xscale;
    const uint16_t* residual;
    int K;
    int mode;
    double* y64;
    uint16_t* y16;
} gv_ctx;
static double gv_row(const gv_ctx* c, int64_t n, int8_t* wrow) {
    int K = c->K, groups = K / GROUP;
    unpack_row_centered(c->packed + n * (K / 8), K, wrow);
    double acc = 0.0;
    for (int g = 0; g < groups; ++g) {
        int32_t d = dot_i8(wrow + g * GROUP, c->q8 + g * GROUP, GROUP);
        float factor = h2f(c->scales[n * groups + g]) * c->xscale[g];
        acc += (double)d * (double)factor;
    }
    return acc;
}
static void gv_rows(int64_t r0, int64_t r1, void* p) {
    gv_ctx* c = (gv_ctx*)p;
    int8_t* wrow = (int8_t*)malloc((size_t)c->K);
    for (int64_t i = r0; i < r1; ++i) {
        double y;
        if (c->mode == 1) {
            double gate = gv_row(c, 2 * i, wrow);
            double up = gv_row(c, 2 * i + 1, wrow);
            y = gate / (1.0 + exp(-gate)) * up;
        } else {
            y = gv_row(c, i, wrow);
            if (c->residual) y += (double)h2f(c->residual[i]);
        }
        if (c->y64) c->y64[i] = y;
        if (c->y16) c->y16[i] = f2h((float)y);
    }
    free(wrow);
}
ORC_API void orc_gemv_q8(const uint32_t* packed, const uint16_t* scales, const int8_t* q8,
                         const float* xscale, const uint16_t* residual, int64_t N, int K, int mode,
                         double* y64, uint16_t* y16, int nthreads) {
    gv_ctx c = {packed, scales, q8, xscale, residual, K, mode, y64, y16};
    parallel_rows(mode == 1 ? N / 2 : N, nthreads, gv_rows, &c);
}

/* ------------------------------------------------------------------------- */
/* fp32 dequantise-then-matmul golden: w = (q - 8) * float(scale) (an exact    */
/* fp32 value), activations given as fp32, products accumulated in double.    */
/* The reference has no host function for this; it is the check the           */
/* benchmark's tolerance is stated against.  mode as in orc_gemv_q8.          */
/* ------------------------------------------------------------------------- */
typedef struct {
    const uint32_t* packed;
    const uint16_t* scales;
    const float* x;
    const uint16_t* residual;
    int K;
    int mode;
    double* y64;
    uint16_t* y16;
} dq_ctx;
static double dq_row(const dq_ctx* c, int64_t n, int8_t* wrow) {
    int K = c->K, groups = K / GROUP;
    unpack_row_centered(c->packed + n * (K / 8), K, wrow);
    double acc = 0.0;
    for (int g = 0; g < groups; ++g) {
        float s = h2f(c->scales[n * groups + g]);
        double part = 0.0;
        for (int j = 0; j < GROUP; ++j) {
            float w = (float)wrow[g * GROUP + j] * s;
            part += (double)w * (double)c->x[g * GROUP + j];
        }
        acc += part;
    }
    return acc;
}
static void dq_rows(int64_t r0, int64_t r1, void* p) {
    dq_ctx* c = (dq_ctx*)p;
    int8_t* wrow = (int8_t*)malloc((size_t)c->K);
    for (int64_t i = r0; i < r1; ++i) {
        double y;
        if (c->mode == 1) {
            double gate = dq_row(c, 2 * i, wrow);
            double up = dq_row(c, 2 * i + 1, wrow);
            y = gate / (1.0 + exp(-gate)) * up;
        } else {
            y = dq_row(c, i, wrow);
            if (c->residual) y += (double)h2f(c->residual[i]);
        }
        if (c->y64) c->y64[i] = y;
        if (c->y16) c->y16[i] = f2h((float)y);
    }
    free(wrow);
}
ORC_API void orc_gemv_dequant(const uint32_t* packed, const uint16_t* scales, const float* x,
                              const uint16_t* residual, int64_t N, int K, int mode, double* y64,
                              uint16_t* y16, int nthreads) {
    dq_ctx c = {packed, scales, x, residual, K, mode, y64, y16};
    parallel_rows(mode == 1 ? N / 2 : N, nthreads, dq_rows, &c);
}

/* ------------------------------------------------------------------------- */
/* Prefill (M tokens) golden.                                                 */
/* Weights are dequantised to fp16 exactly as unpack_w4_to_half2_quad does    */
/* (include/quant_primitives.cuh:92-115): (q - 8) is exact in fp16, times the */
/* fp16 scale with ONE rounding to fp16.  The tensor cores multiply fp16 by   */
/* fp16 exactly and add in fp32; the golden adds the exact products in double.*/
/* Epilogue, src/kernels/gemm_prefill.cu:257-275: fp16(acc), then an fp16 add */
/* with the residual (vector path, the one the engine's shapes take).         */
/* SwiGLU epilogue (:572-605): silu(gate) * up on the accumulators, one fp16  */
/* rounding.                                                                  */
/* Only the listed token rows m_idx[nm] and output columns n_idx[nn] are      */
/* evaluated (for mode 1, n_idx holds SwiGLU output indices i).               */
/* out64 / out16: [nm][nn].  residual / x are full [M][N] / [M][K] arrays;    */
/* ldr is the residual row stride in elements.                                */
/* ------------------------------------------------------------------------- */
typedef struct {
    const uint32_t* packed;
    const uint16_t* scales;
    const uint16_t* x;
    const uint16_t* residual;
    int64_t ldr;
    int K;
    int mode;
    const int32_t* m_idx;
    int nm;
    const int32_t* n_idx;
    int nn;
    double* out64;
    uint16_t* out16;
} pf_ctx;
static void pf_dequant_row(const pf_ctx* c, int64_t n, int8_t* tmp, float* wf) {
    int K = c->K, groups = K / GROUP;
    unpack_row_centered(c->packed + n * (K / 8), K, tmp);
    for (int g = 0; g < groups; ++g) {
        float s = h2f(c->scales[n * groups + g]);
        for (int j = 0; j < GROUP; ++j) wf[g * GROUP + j] = h2f(f2h((float)tmp[g * GROUP + j] * s));
    }
}
static double pf_dot(const float* wf, const uint16_t* xrow, int K) {
    double acc = 0.0;
    for (int k = 0; k < K; ++k) acc += (double)wf[k] * (double)h2f(xrow[k]);
    return acc;
}
static void pf_cols(int64_t c0, int64_t c1, void* p) {
    pf_ctx* c = (pf_ctx*)p;
    int K = c->K;
    int8_t* tmp = (int8_t*)malloc((size_t)K);
    float* w0 = (float*)malloc(sizeof(float) * (size_t)K);
    float* w1 = (float*)malloc(sizeof(float) * (size_t)K);
    for (int64_t j = c0; j < c1; ++j) {
        int64_t n = c->n_idx[j];
        if (c->mode == 1) {
            pf_dequant_row(c, 2 * n, tmp, w0);
            pf_dequant_row(c, 2 * n + 1, tmp, w1);
        } else {
            pf_dequant_row(c, n, tmp, w0);
        }
        for (int i = 0; i < c->nm; ++i) {
            int64_t m = c->m_idx[i];
            const uint16_t* xrow = c->x + m * K;
            double y;
            uint16_t yh;
            if (c->mode == 1) {
                double gate = pf_dot(w0, xrow, K), up = pf_dot(w1, xrow, K);
                y = gate / (1.0 + exp(-gate)) * up;
                yh = f2h((float)y);
            } else {
                y = pf_dot(w0, xrow, K);
                yh = f2h((float)y);
                if (c->residual) {
                    double r = (double)h2f(c->residual[m * c->ldr + n]);
                    yh = d2h((double)h2f(yh) + r);
                    y += r;
                }
            }
            if (c->out64) c->out64[(int64_t)i * c->nn + j] = y;
            if (c->out16) c->out16[(int64_t)i * c->nn + j] = yh;
        }
    }
    free(tmp);
    free(w0);
    free(w1);
}
ORC_API void orc_gemm_prefill(const uint32_t* packed, const uint16_t* scales, const uint16_t* x,
                              const uint16_t* residual, int64_t ldr, int K, int mode,
                              const int32_t* m_idx, int nm, const int32_t* n_idx, int nn,
                              double* out64, uint16_t* out16, int nthreads) {
    pf_ctx c = {packed, scales, x, residual, ldr, K, mode, m_idx, nm, n_idx, nn, out64, out16};
    parallel_rows(nn, nthreads, pf_cols, &c);
}

/* ------------------------------------------------------------------------- */
/* RMSNorm in front of the Q8_1 quantiser.                                    */
/* src/kernels/rmsnorm_rope.cu:214-233 (CPU twin tests/test_kernels.cu:81-96):*/
/*   inv_rms = rsqrt(mean(x^2) + eps) in fp32, rounded to fp16;               */
/*   y = fp16(fp16(x * inv_rms_h) * gamma)   (two fp16 multiplies).           */
/* The sum of squares is taken in double (squares of fp16 values are exact     */
/* there and the sum is off by parts in 2^50 at most, so the summation order   */
/* does not reach the fp32 mean); the mean,                                    */
/* + eps, square root and reciprocal are IEEE fp32 as in the reference, whose */
/* kernels add in fp32 in an order of their own, so its inv_rms_h can differ  */
/* by one fp16 ulp in rare cases.  The caller passes inv_rms_override > 0 to  */
/* pin it to a device's value.                                                */
/* ------------------------------------------------------------------------- */
ORC_API float orc_rmsnorm(const uint16_t* x, const uint16_t* gamma, int n, float eps,
                          float inv_rms_override, uint16_t* y) {
    double ss = 0.0;
    for (int i = 0; i < n; ++i) {
        double v = (double)h2f(x[i]);
        ss += v * v;
    }
    float mean = (float)ss / (float)n;
    float inv_rms = 1.0f / sqrtf(mean + eps);
    if (inv_rms_override > 0.0f) inv_rms = inv_rms_override;
    float ih = h2f(f2h(inv_rms));
    for (int i = 0; i < n; ++i) {
        float t = h2f(f2h(h2f(x[i]) * ih));
        y[i] = f2h(t * h2f(gamma[i]));
    }
    return inv_rms;
}

/* ------------------------------------------------------------------------- */
/* Token selection after lm_head.  src/kernels/sampling.cu:13-57 (uniform     */
/* number from Philox-4x32-10: counter = (vocabulary index, sequence          */
/* position, 0, 0), key = the seed's two halves, first output word;           */
/* u = (word + 1) / 2^32 clamped to [1e-7, 1 - 1e-7]), :86-100 (score = logit */
/* for temperature <= 1e-5, else logit / temperature - log(-log(u)); a larger */
/* score wins, scanning in index order so that the lowest index wins among    */
/* equals; the running best starts at -1e30 with index 0).                    */
/* Philox as published: Salmon, Moraes, Dror, Shaw, SC'11.  fp32 arithmetic   */
/* with libm's logf; scores_out (optional, n floats) receives every score.    */
/* ------------------------------------------------------------------------- */
static uint32_t philox4x32_10_first(uint64_t seed, uint32_t c0, uint32_t c1) {
    uint32_t c2 = 0, c3 = 0;
    uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
    for (int round = 0; round < 10; ++round) {
        uint64_t p0 = (uint64_t)0xD2511F53u * c0;
        uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
        uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0;
        uint32_t n1 = (uint32_t)p1;
        uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1;
        uint32_t n3 = (uint32_t)p0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    return c0;
}
ORC_API uint32_t orc_philox_first(uint64_t seed, uint32_t c0, uint32_t c1) { return philox4x32_10_first(seed, c0, c1); }
ORC_API int32_t orc_sample(const uint16_t* logits, int n, float temperature, uint64_t seed, uint32_t seq_pos,
                           int32_t index_offset, float* best_out, float* scores_out) {
    float best = -1e30f;
    int32_t best_idx = 0;
    for (int i = 0; i < n; ++i) {
        float v = h2f(logits[i]);
        if (temperature > 1e-5f) {
            uint32_t r = philox4x32_10_first(seed, (uint32_t)(i + index_offset), seq_pos);
            float u = ((float)r + 1.0f) / 4294967296.0f;
            if (u < 1e-7f) u = 1e-7f;
            if (u > 1.0f - 1e-7f) u = 1.0f - 1e-7f;
            float gumbel = -logf(-logf(u));
            v = (v / temperature) + gumbel;
        }
        if (scores_out) scores_out[i] = v;
        if (v > best) { best = v; best_idx = i + index_offset; }
    }
    if (best_out) *best_out = best;
    return best_idx;
}

ORC_API int orc_version(void) { return 2; }
