/* TEST INFRASTRUCTURE - not part of the product.
 *
 * A CPU restatement of the reference's llama / qwen2 decoder, used only as the checker in tests, in the smoke test and as the timed CPU baseline of the
 * benchmark. The library never links or calls it.
 *
 * What it follows (paths inside the reference project):
 *   - the block formulas Q4_0 / Q5_0 / Q8_0 / Q4_K / Q6_K ::elem and scale_min_k4, src/backend/metal/llama_kernels.h:1012-1154;
 *   - the double-precision `Reference` class of the reference's own decoder test, tests/unit/test_metal_llama_decoder.cpp:110-192 (RMSNorm, qkv + bias,
 *     rotary pairs, keys and values rounded to f16 into the cache, grouped-query softmax attention, SwiGLU, residuals, final norm, lm_head);
 *   - the first-index argmax of llama_kernels.h:949-975 / src/core/argmax.h:15-53 (NaN never wins).
 *
 * Pinning: the reference checks in no golden files for this path (its tests compute the expectation live), so the checker is held to the reference's own
 * code and to independent implementations instead:
 *   - the decoder math against the reference's `Reference` class itself, compiled from the reference's test file (oracle/Makefile target `ref`,
 *     oracle/ref_decoder_shim.cpp): logits position by position to 1e-12 and the greedy tokens, on the reference test's f16 shapes and on quantized
 *     models whose values are exact in f16 (tests/test_oracle.py);
 *   - the dequantization bit for bit against gguf-py's dequantize (the file format's own Python package), against byte patterns worked out by hand from
 *     the formulas, and against committed vectors (tests/golden);
 *   - the argmax and the block tables against the reference's own functions compiled from its sources (oracle/_ref/libref_gguf.so).
 * At the boundary to llama.cpp, which the reference links but does not vendor, parity stays unpinned.
 *
 * Build: see oracle/Makefile (gcc, -ffp-contract=off so that the f32 block formulas round exactly as written).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef __AVX2__
#include <immintrin.h>
#endif
#ifdef _OPENMP
#include <omp.h>
#endif

#include "dooms_cuda.h"

#define ORACLE_API __attribute__((visibility("default")))

static float half_to_float(uint16_t h) { _Float16 v; memcpy(&v, &h, 2); return (float)v; }
static float ld_half(const uint8_t * p) { uint16_t h; memcpy(&h, p, 2); return half_to_float(h); }
static float round_to_half(float v) { return (float)(_Float16)v; }

ORACLE_API float oracle_round_to_half(float v) { return round_to_half(v); }

static int64_t block_elems(int dt) { return dt == DOOMS_Q4_K || dt == DOOMS_Q6_K ? 256 : (dt == DOOMS_Q4_0 || dt == DOOMS_Q5_0 || dt == DOOMS_Q8_0) ? 32 : 1; }
static int64_t block_bytes(int dt) {
    switch (dt) {
        case DOOMS_F32: case DOOMS_I32: return 4;
        case DOOMS_F16: case DOOMS_BF16: return 2;
        case DOOMS_Q4_0: return 18;
        case DOOMS_Q5_0: return 22;
        case DOOMS_Q8_0: return 34;
        case DOOMS_Q4_K: return 144;
        case DOOMS_Q6_K: return 210;
    }
    return 0;
}
static int64_t row_bytes(int dt, int64_t cols) { return cols / block_elems(dt) * block_bytes(dt); }

/* scale_min_k4, llama_kernels.h:1099-1102 */
static void scale_min_k4(unsigned j, const uint8_t * q, float * d, float * m) {
    if (j < 4) { *d = (float)(q[j] & 63u); *m = (float)(q[j + 4] & 63u); }
    else { *d = (float)((q[j + 4] & 15u) | ((q[j - 4] >> 6) << 4)); *m = (float)((q[j + 4] >> 4) | ((q[j] >> 6) << 4)); }
}

/* Element i of a row in each format: the elem() functions of llama_kernels.h:1014-1018, 1046-1050, 1076-1079, 1108-1115, 1147-1154. f32 arithmetic,
 * every product and difference rounded separately (the file is compiled without contraction). */
static float elem(int dt, const uint8_t * row, int64_t i) {
    switch (dt) {
        case DOOMS_F32: { float v; memcpy(&v, row + 4 * i, 4); return v; }
        case DOOMS_F16: return ld_half(row + 2 * i);
        case DOOMS_BF16: { uint32_t u = (uint32_t)(row[2 * i] | (row[2 * i + 1] << 8)) << 16; float v; memcpy(&v, &u, 4); return v; }
        case DOOMS_Q4_0: {
            const uint8_t * b = row + (i / 32) * 18;
            const unsigned j = (unsigned)(i % 32), q = b[2 + (j & 15)];
            return ld_half(b) * ((float)(j < 16 ? (q & 15u) : (q >> 4)) - 8.f);
        }
        case DOOMS_Q5_0: {
            const uint8_t * b = row + (i / 32) * 22;
            const unsigned j = (unsigned)(i % 32), q = b[6 + (j & 15)], low = j < 16 ? (q & 15u) : (q >> 4);
            uint32_t qh; memcpy(&qh, b + 2, 4);
            return ld_half(b) * ((float)(low | (((qh >> j) & 1u) << 4)) - 16.f);
        }
        case DOOMS_Q8_0: {
            const uint8_t * b = row + (i / 32) * 34;
            return ld_half(b) * (float)((const int8_t *)b)[2 + i % 32];
        }
        case DOOMS_Q4_K: {
            const uint8_t * b = row + (i / 256) * 144;
            const unsigned j = (unsigned)(i % 256), c = j / 32, l = j % 32;
            float sc, m;
            scale_min_k4(c, b + 4, &sc, &m);
            const unsigned q = b[16 + 32 * (c / 2) + l];
            const float a = ld_half(b) * sc;
            const float v = a * (float)((c & 1u) ? (q >> 4) : (q & 15u));
            const float o = ld_half(b + 2) * m;
            return v - o;
        }
        case DOOMS_Q6_K: {
            const uint8_t * b = row + (i / 256) * 210;
            const unsigned j = (unsigned)(i % 256), h = j / 128, k = (j % 128) / 32, l = j % 32;
            const unsigned qlb = b[64 * h + (k & 1u) * 32 + l], low = k < 2 ? (qlb & 15u) : (qlb >> 4);
            const unsigned hb = (b[128 + 32 * h + l] >> (2 * k)) & 3u;
            const float sc = (float)((const int8_t *)(b + 192))[8 * h + l / 16 + 2 * k];
            const float a = ld_half(b + 208) * sc;
            return a * (float)((int)(low | (hb << 4)) - 32);
        }
    }
    return 0.f;
}

/* n elements of one row (n a multiple of the block size). */
ORACLE_API void oracle_dequantize(int32_t dtype, const void * blocks, int64_t n, float * out) {
    #pragma omp parallel for schedule(static) if (n >= (1 << 16))
    for (int64_t i = 0; i < n; i++) out[i] = elem(dtype, (const uint8_t *)blocks, i);
}

/* argmax with the first index on ties; NaN is never chosen over a number, an all-NaN input gives 0 (src/core/argmax.h:15-16, 47-51). */
ORACLE_API int32_t oracle_argmax_f32(const float * v, int64_t n) {
    int64_t best = 0;
    float bv = v[0];
    for (int64_t i = 1; i < n; i++) if (v[i] > bv || (bv != bv && v[i] == v[i])) { bv = v[i]; best = i; }
    return (int32_t)best;
}
ORACLE_API int32_t oracle_argmax_f64(const double * v, int64_t n) {
    int64_t best = 0;
    double bv = v[0];
    for (int64_t i = 1; i < n; i++) if (v[i] > bv || (bv != bv && v[i] == v[i])) { bv = v[i]; best = i; }
    return (int32_t)best;
}

/* ---- The decoder ---- */

typedef struct { const uint8_t * data; int dtype; int64_t rows, cols; } mat_t;

typedef struct {
    float * attn_norm, * ffn_norm, * qkv_bias;   /* qkv_bias NULL: none */
    mat_t q, k, v, qkv;                           /* qkv.data set: fused */
    mat_t wo, gate, up, down;
} layer_t;

typedef struct oracle_decoder {
    dooms_llama_config cfg;
    mat_t embd, output;
    float * output_norm;
    layer_t * layers;
    float * kc, * vc;          /* [n_layer][n_ctx][KV], values rounded to f16 */
    int32_t pos;
    int fast;                  /* 1: f32 accumulation (the timed CPU baseline); 0: double (the checker) */
    int round_operands;        /* 1: multi-token calls round the projections' operands to f16 like the reference's prefill tiles (llama_kernels.h:186-199);
                                * 2: every call does, single positions and the output projection included: the arithmetic of a decode step that runs
                                * several sequences as the rows of one chunk through the same tiles */
} oracle_decoder;

static mat_t mat_of(const dooms_weight_ref * r) { mat_t m = {(const uint8_t *)r->data, r->dtype, r->rows, r->cols}; return m; }

static float * vec_of(const dooms_weight_ref * r) {
    float * v = (float *)malloc(sizeof(float) * (size_t)r->cols);
    for (int64_t i = 0; i < r->cols; i++) v[i] = elem(r->dtype, (const uint8_t *)r->data, i);
    return v;
}

/* The weights are referenced, not copied: they must outlive the decoder. Shapes are taken as given (the product validates them; the checker trusts). */
ORACLE_API oracle_decoder * oracle_create(const dooms_llama_config * cfg, const dooms_llama_weights * w) {
    oracle_decoder * d = (oracle_decoder *)calloc(1, sizeof *d);
    d->cfg = *cfg;
    const int64_t Q = (int64_t)cfg->n_head * cfg->head_dim, KV = (int64_t)cfg->n_head_kv * cfg->head_dim;
    d->embd = mat_of(&w->token_embd);
    d->output = mat_of(&w->output);
    d->output_norm = vec_of(&w->output_norm);
    d->layers = (layer_t *)calloc((size_t)cfg->n_layer, sizeof(layer_t));
    for (int l = 0; l < cfg->n_layer; l++) {
        const dooms_llama_layer_weights * s = &w->layers[l];
        layer_t * L = &d->layers[l];
        L->attn_norm = vec_of(&s->attn_norm);
        L->ffn_norm = vec_of(&s->ffn_norm);
        if (s->attn_qkv.data) L->qkv = mat_of(&s->attn_qkv);
        else { L->q = mat_of(&s->attn_q); L->k = mat_of(&s->attn_k); L->v = mat_of(&s->attn_v); }
        if (s->attn_qkv_bias.data) L->qkv_bias = vec_of(&s->attn_qkv_bias);
        else if (s->attn_q_bias.data) {
            L->qkv_bias = (float *)malloc(sizeof(float) * (size_t)(Q + 2 * KV));
            float * a = vec_of(&s->attn_q_bias), * b = vec_of(&s->attn_k_bias), * c = vec_of(&s->attn_v_bias);
            memcpy(L->qkv_bias, a, sizeof(float) * (size_t)Q);
            memcpy(L->qkv_bias + Q, b, sizeof(float) * (size_t)KV);
            memcpy(L->qkv_bias + Q + KV, c, sizeof(float) * (size_t)KV);
            free(a); free(b); free(c);
        }
        L->wo = mat_of(&s->attn_output);
        L->gate = mat_of(&s->ffn_gate);
        L->up = mat_of(&s->ffn_up);
        L->down = mat_of(&s->ffn_down);
    }
    const size_t cache = (size_t)cfg->n_layer * (size_t)cfg->n_ctx * (size_t)KV;
    d->kc = (float *)calloc(cache, sizeof(float));
    d->vc = (float *)calloc(cache, sizeof(float));
    return d;
}

ORACLE_API void oracle_destroy(oracle_decoder * d) {
    if (!d) return;
    for (int l = 0; l < d->cfg.n_layer; l++) { free(d->layers[l].attn_norm); free(d->layers[l].ffn_norm); free(d->layers[l].qkv_bias); }
    free(d->layers); free(d->output_norm); free(d->kc); free(d->vc); free(d);
}
ORACLE_API void oracle_reset(oracle_decoder * d) { d->pos = 0; }
ORACLE_API int32_t oracle_position(const oracle_decoder * d) { return d->pos; }
ORACLE_API void oracle_set_fast(oracle_decoder * d, int32_t fast) { d->fast = fast; }
/* Threads of the parallel loops from here on (a launcher may have exported OMP_NUM_THREADS=1 for its workers); returns the count in effect. */
ORACLE_API int32_t oracle_set_threads(int32_t n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
    return (int32_t)omp_get_max_threads();
#else
    (void)n;
    return 1;
#endif
}
ORACLE_API void oracle_set_round_operands(oracle_decoder * d, int32_t on) { d->round_operands = on; }

/* ---- The timed CPU baseline's one-token projection: f32 quantized dot products, the folding of the reference's Q::dot functions
 * (llama_kernels.h:1036-1040, 1065-1069, 1090-1094, 1132-1140, 1175-1183): the integer quants are multiplied with the input as they are, a block's scale is
 * applied once per block (sub-block), and the offsets (q4_0: -8, q5_0: -16, q6_K: -32, q4_K: -dmin m) come in through the sums of the input's 32- (16-)
 * element groups, computed once per call. Eight-wide f32 FMAs when the compiler targets AVX2. ---- */
#ifdef __AVX2__
typedef __m256 vec8;
static inline vec8 v8_zero(void) { return _mm256_setzero_ps(); }
static inline vec8 v8_u8(const uint8_t * q) { return _mm256_cvtepi32_ps(_mm256_cvtepu8_epi32(_mm_loadl_epi64((const __m128i *)q))); }
static inline vec8 v8_i8(const int8_t * q) { return _mm256_cvtepi32_ps(_mm256_cvtepi8_epi32(_mm_loadl_epi64((const __m128i *)q))); }
static inline vec8 v8_fma_x(vec8 q, const float * x, vec8 acc) { return _mm256_fmadd_ps(q, _mm256_loadu_ps(x), acc); }
static inline vec8 v8_fma_s(float s, vec8 v, vec8 acc) { return _mm256_fmadd_ps(_mm256_set1_ps(s), v, acc); }
static inline float v8_sum(vec8 v) {
    __m128 a = _mm_add_ps(_mm256_castps256_ps128(v), _mm256_extractf128_ps(v, 1));
    a = _mm_add_ps(a, _mm_movehl_ps(a, a));
    a = _mm_add_ss(a, _mm_shuffle_ps(a, a, 1));
    return _mm_cvtss_f32(a);
}
#else
typedef struct { float v[8]; } vec8;
static inline vec8 v8_zero(void) { vec8 r; for (int i = 0; i < 8; i++) r.v[i] = 0.f; return r; }
static inline vec8 v8_u8(const uint8_t * q) { vec8 r; for (int i = 0; i < 8; i++) r.v[i] = (float)q[i]; return r; }
static inline vec8 v8_i8(const int8_t * q) { vec8 r; for (int i = 0; i < 8; i++) r.v[i] = (float)q[i]; return r; }
static inline vec8 v8_fma_x(vec8 q, const float * x, vec8 acc) { for (int i = 0; i < 8; i++) acc.v[i] += q.v[i] * x[i]; return acc; }
static inline vec8 v8_fma_s(float s, vec8 v, vec8 acc) { for (int i = 0; i < 8; i++) acc.v[i] += s * v.v[i]; return acc; }
static inline float v8_sum(vec8 v) { float s = 0.f; for (int i = 0; i < 8; i++) s += v.v[i]; return s; }
#endif

/* sum of q[0..n) * x[0..n), n a multiple of 8, quants as unsigned / signed bytes */
static inline vec8 dot_u8(const uint8_t * q, const float * x, int n, vec8 acc) { for (int i = 0; i < n; i += 8) acc = v8_fma_x(v8_u8(q + i), x + i, acc); return acc; }
static inline vec8 dot_i8(const int8_t * q, const float * x, int n, vec8 acc) { for (int i = 0; i < n; i += 8) acc = v8_fma_x(v8_i8(q + i), x + i, acc); return acc; }

/* The 16 quant bytes of a q4_0 / q5_0 block as 32 values 0..15: low nibbles are elements 0..15, high nibbles 16..31. */
static inline void nibbles32(const uint8_t * qs, uint8_t * q) {
#ifdef __AVX2__
    const __m128i v = _mm_loadu_si128((const __m128i *)qs), m = _mm_set1_epi8(15);
    _mm_storeu_si128((__m128i *)q, _mm_and_si128(v, m));
    _mm_storeu_si128((__m128i *)(q + 16), _mm_and_si128(_mm_srli_epi16(v, 4), m));
#else
    for (int j = 0; j < 16; j++) { q[j] = qs[j] & 15u; q[16 + j] = qs[j] >> 4; }
#endif
}
/* bit i of b as 16 or 0 in byte i */
static inline uint64_t spread_bits_16(uint8_t b) {
    uint64_t x = ((uint64_t)b * 0x0101010101010101ULL) & 0x8040201008040201ULL;
    x = ((x + 0x7F7F7F7F7F7F7F7FULL) >> 7) & 0x0101010101010101ULL;
    return x << 4;
}

/* One row times x. xs16: the sums of x over groups of 16 elements. */
static float row_dot_fast(int dt, const uint8_t * row, const float * x, const float * xs16, int64_t K) {
    vec8 acc = v8_zero();
    float off = 0.f;
    switch (dt) {
        case DOOMS_Q4_0:
            for (int64_t b = 0; b < K / 32; b++) {
                const uint8_t * p = row + b * 18;
                uint8_t q[32];
                nibbles32(p + 2, q);
                const float d = ld_half(p);
                acc = v8_fma_s(d, dot_u8(q, x + 32 * b, 32, v8_zero()), acc);
                off += d * (xs16[2 * b] + xs16[2 * b + 1]);
            }
            return v8_sum(acc) - 8.f * off;
        case DOOMS_Q5_0:
            for (int64_t b = 0; b < K / 32; b++) {
                const uint8_t * p = row + b * 22;
                uint8_t q[32];
                nibbles32(p + 6, q);
                for (int j = 0; j < 4; j++) {          /* the fifth bits: byte j of qh covers elements 8j .. 8j+7 */
                    uint64_t lo, hb = spread_bits_16(p[2 + j]);
                    memcpy(&lo, q + 8 * j, 8);
                    lo |= hb;
                    memcpy(q + 8 * j, &lo, 8);
                }
                const float d = ld_half(p);
                acc = v8_fma_s(d, dot_u8(q, x + 32 * b, 32, v8_zero()), acc);
                off += d * (xs16[2 * b] + xs16[2 * b + 1]);
            }
            return v8_sum(acc) - 16.f * off;
        case DOOMS_Q8_0:
            for (int64_t b = 0; b < K / 32; b++) {
                const uint8_t * p = row + b * 34;
                acc = v8_fma_s(ld_half(p), dot_i8((const int8_t *)p + 2, x + 32 * b, 32, v8_zero()), acc);
            }
            return v8_sum(acc);
        case DOOMS_Q4_K:
            for (int64_t b = 0; b < K / 256; b++) {
                const uint8_t * p = row + b * 144;
                const float d = ld_half(p), dmin = ld_half(p + 2);
                for (unsigned c = 0; c < 8; c++) {
                    float sc, m;
                    scale_min_k4(c, p + 4, &sc, &m);
                    uint8_t q[32];
                    const uint8_t * qs = p + 16 + 32 * (c / 2);
                    if (c & 1u) for (int j = 0; j < 32; j++) q[j] = qs[j] >> 4;
                    else for (int j = 0; j < 32; j++) q[j] = qs[j] & 15u;
                    acc = v8_fma_s(d * sc, dot_u8(q, x + 256 * b + 32 * c, 32, v8_zero()), acc);
                    off += dmin * m * (xs16[16 * b + 2 * c] + xs16[16 * b + 2 * c + 1]);
                }
            }
            return v8_sum(acc) - off;
        case DOOMS_Q6_K:
            for (int64_t b = 0; b < K / 256; b++) {
                const uint8_t * p = row + b * 210;
                const float d = ld_half(p + 208);
                const int8_t * scales = (const int8_t *)(p + 192);
                for (unsigned h = 0; h < 2; h++) {
                    for (unsigned k = 0; k < 4; k++) {
                        uint8_t q[32];
                        const uint8_t * ql = p + 64 * h + (k & 1u) * 32, * qh = p + 128 + 32 * h;
                        for (int l = 0; l < 32; l++) q[l] = (uint8_t)((k < 2 ? (ql[l] & 15u) : (ql[l] >> 4)) | (((qh[l] >> (2 * k)) & 3u) << 4));
                        const float * xb = x + 256 * b + 128 * h + 32 * k;
                        const int64_t g16 = 16 * b + 8 * h + 2 * k;
                        for (unsigned s = 0; s < 2; s++) {
                            const float a = d * (float)scales[8 * h + s + 2 * k];
                            acc = v8_fma_s(a, dot_u8(q + 16 * s, xb + 16 * s, 16, v8_zero()), acc);
                            off += a * xs16[g16 + s];
                        }
                    }
                }
            }
            return v8_sum(acc) - 32.f * off;
        default: {
            float a = 0.f;
            for (int64_t k = 0; k < K; k++) a += elem(dt, row, k) * x[k];
            return a;
        }
    }
}

/* y[row0 + r] (+)= W[r] . x for one input row, on all threads. */
static void matvec_fast(const mat_t * W, const double * X, double * Y, int64_t row0, int accumulate) {
    const int64_t K = W->cols, RB = row_bytes(W->dtype, K);
    float * x = (float *)malloc(sizeof(float) * (size_t)(K + K / 16 + 1));
    float * xs16 = x + K;
    for (int64_t k = 0; k < K; k++) x[k] = (float)X[k];
    for (int64_t g = 0; g < K / 16; g++) { float s = 0.f; for (int j = 0; j < 16; j++) s += x[16 * g + j]; xs16[g] = s; }
    #pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < W->rows; r++) {
        const double acc = (double)row_dot_fast(W->dtype, W->data + r * RB, x, xs16, K);
        double * y = Y + row0 + r;
        *y = accumulate ? *y + acc : acc;
    }
    free(x);
}

/* Y[m][row0 + r] (+)= W[r] . X[m]   for M rows of X (stride xs) -> Y (stride ys). Reference::matvec (test_metal_llama_decoder.cpp:177-181), one weight
 * row dequantized at a time. */
static void matmul(const oracle_decoder * d, const mat_t * W, const double * X, int64_t xs, double * Y, int64_t ys, int64_t row0, int64_t M, int accumulate,
                   int round_ops) {
    const int64_t K = W->cols, RB = row_bytes(W->dtype, K);
    const int fast = d->fast;
    if (fast && M == 1 && !round_ops && K % 32 == 0) { matvec_fast(W, X, Y, row0, accumulate); return; }
    #pragma omp parallel
    {
        float * w = (float *)malloc(sizeof(float) * (size_t)K);
        #pragma omp for schedule(static)
        for (int64_t r = 0; r < W->rows; r++) {
            const uint8_t * row = W->data + r * RB;
            for (int64_t k = 0; k < K; k++) w[k] = elem(W->dtype, row, k);
            if (round_ops) for (int64_t k = 0; k < K; k++) w[k] = round_to_half(w[k]);
            for (int64_t m = 0; m < M; m++) {
                const double * x = X + m * xs;
                double acc;
                if (fast) {
                    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
                    for (int64_t k = 0; k + 3 < K; k += 4) {
                        a0 += w[k] * (float)x[k]; a1 += w[k + 1] * (float)x[k + 1]; a2 += w[k + 2] * (float)x[k + 2]; a3 += w[k + 3] * (float)x[k + 3];
                    }
                    acc = (double)((a0 + a1) + (a2 + a3));
                } else {
                    double a0 = 0, a1 = 0, a2 = 0, a3 = 0;
                    for (int64_t k = 0; k + 3 < K; k += 4) {
                        a0 += (double)w[k] * x[k]; a1 += (double)w[k + 1] * x[k + 1]; a2 += (double)w[k + 2] * x[k + 2]; a3 += (double)w[k + 3] * x[k + 3];
                    }
                    acc = (a0 + a1) + (a2 + a3);
                }
                double * y = Y + m * ys + row0 + r;
                *y = accumulate ? *y + acc : acc;
            }
        }
        free(w);
    }
}

/* Reference::rms (test_metal_llama_decoder.cpp:169-176). With round_ops the result is rounded to f16, the prefill tiles' A operand
 * (llama_kernels.h:186-199: half(x * gamma * scale)). */
static void rms_rows(const oracle_decoder * d, const double * X, const float * g, double * Y, int64_t M, int64_t E, int round_ops) {
    #pragma omp parallel for schedule(static)
    for (int64_t m = 0; m < M; m++) {
        const double * x = X + m * E;
        double ss = 0;
        for (int64_t i = 0; i < E; i++) ss += x[i] * x[i];
        const double inv = 1.0 / sqrt(ss / (double)E + (double)d->cfg.rms_eps);
        for (int64_t i = 0; i < E; i++) {
            const double v = x[i] * inv * (double)g[i];
            Y[m * E + i] = round_ops ? (double)round_to_half((float)v) : v;
        }
    }
}

/* Reference::rope (test_metal_llama_decoder.cpp:182-191). */
static void rope(const oracle_decoder * d, double * v, int pos) {
    const int hd = d->cfg.head_dim;
    for (int i = 0; i < hd / 2; i++) {
        const double th = pos * pow((double)d->cfg.rope_base, -2.0 * i / hd);
        const int i0 = d->cfg.rope_neox ? i : 2 * i, i1 = d->cfg.rope_neox ? i + hd / 2 : 2 * i + 1;
        const double a = v[i0], b = v[i1];
        v[i0] = a * cos(th) - b * sin(th);
        v[i1] = a * sin(th) + b * cos(th);
    }
}

/* Appends n positions given as embeddings (n x n_embd floats); logits (n_vocab doubles) of the last one. Layer by layer over all n positions, which is
 * Reference::step (test_metal_llama_decoder.cpp:114-161) applied to each position in turn: position t attends to cache positions 0..pos+t only.
 * Returns 0, or 1 when the context would overflow. */
ORACLE_API int32_t oracle_eval_embeddings(oracle_decoder * d, const float * emb, int32_t n, double * logits) {
    const dooms_llama_config * c = &d->cfg;
    const int64_t E = c->n_embd, F = c->n_ff, hd = c->head_dim, nh = c->n_head, nkv = c->n_head_kv, Q = nh * hd, KV = nkv * hd, W3 = Q + 2 * KV, M = n;
    if (n < 1 || (int64_t)d->pos + n > c->n_ctx) return 1;
    const int round_all = d->round_operands == 2;
    const int round_ops = round_all || (d->round_operands && M > 1);
    double * x = (double *)malloc(sizeof(double) * (size_t)(M * E));
    double * xn = (double *)malloc(sizeof(double) * (size_t)(M * (E > F ? E : F)));
    double * qkv = (double *)malloc(sizeof(double) * (size_t)(M * W3));
    double * att = (double *)malloc(sizeof(double) * (size_t)(M * Q));
    double * g = (double *)malloc(sizeof(double) * (size_t)(M * F));
    double * u = (double *)malloc(sizeof(double) * (size_t)(M * F));
    for (int64_t i = 0; i < M * E; i++) x[i] = (double)emb[i];
    const int p0 = d->pos;
    for (int l = 0; l < c->n_layer; l++) {
        const layer_t * L = &d->layers[l];
        float * kc = d->kc + (size_t)l * (size_t)c->n_ctx * (size_t)KV, * vc = d->vc + (size_t)l * (size_t)c->n_ctx * (size_t)KV;
        rms_rows(d, x, L->attn_norm, xn, M, E, round_ops);
        if (L->qkv.data) matmul(d, &L->qkv, xn, E, qkv, W3, 0, M, 0, round_ops);
        else {
            matmul(d, &L->q, xn, E, qkv, W3, 0, M, 0, round_ops);
            matmul(d, &L->k, xn, E, qkv, W3, Q, M, 0, round_ops);
            matmul(d, &L->v, xn, E, qkv, W3, Q + KV, M, 0, round_ops);
        }
        #pragma omp parallel for schedule(static)
        for (int64_t m = 0; m < M; m++) {
            double * row = qkv + m * W3;
            if (L->qkv_bias) for (int64_t i = 0; i < W3; i++) row[i] += (double)L->qkv_bias[i];
            for (int64_t s = 0; s < nh + nkv; s++) rope(d, row + s * hd, p0 + (int)m);
            for (int64_t i = 0; i < KV; i++) {
                kc[(size_t)(p0 + m) * (size_t)KV + (size_t)i] = round_to_half((float)row[Q + i]);
                vc[(size_t)(p0 + m) * (size_t)KV + (size_t)i] = round_to_half((float)row[Q + KV + i]);
            }
        }
        #pragma omp parallel for schedule(dynamic) collapse(2)
        for (int64_t m = 0; m < M; m++) {
            for (int64_t h = 0; h < nh; h++) {
                const int64_t kvh = h / (nh / nkv), np = p0 + m + 1;
                const double * q0 = qkv + m * W3 + h * hd;
                double q[512];
                /* the prefill tiles hold the rotated query as f16 and the probabilities as f16 relative to the running maximum, while the normalizing sum
                 * adds the unrounded exponentials (attention_prefill, llama_kernels.h:660, 708-713) */
                for (int64_t e = 0; e < hd; e++) q[e] = round_ops ? (double)round_to_half((float)q0[e]) : q0[e];
                double * sc = (double *)malloc(sizeof(double) * (size_t)np);
                double mx = -1e300;
                for (int64_t j = 0; j < np; j++) {
                    double s = 0;
                    const float * k = kc + (size_t)j * (size_t)KV + (size_t)(kvh * hd);
                    for (int64_t e = 0; e < hd; e++) s += q[e] * (double)k[e];
                    sc[j] = s / sqrt((double)hd);
                    if (sc[j] > mx) mx = sc[j];
                }
                double sum = 0;
                for (int64_t j = 0; j < np; j++) { sc[j] = exp(sc[j] - mx); sum += sc[j]; if (round_ops) sc[j] = (double)round_to_half((float)sc[j]); }
                for (int64_t e = 0; e < hd; e++) {
                    double a = 0;
                    for (int64_t j = 0; j < np; j++) a += sc[j] * (double)vc[(size_t)j * (size_t)KV + (size_t)(kvh * hd + e)];
                    const double o = a / sum;
                    att[m * Q + h * hd + e] = round_ops ? (double)round_to_half((float)o) : o;
                }
                free(sc);
            }
        }
        matmul(d, &L->wo, att, Q, x, E, 0, M, 1, round_ops);
        rms_rows(d, x, L->ffn_norm, xn, M, E, round_ops);
        matmul(d, &L->gate, xn, E, g, F, 0, M, 0, round_ops);
        matmul(d, &L->up, xn, E, u, F, 0, M, 0, round_ops);
        #pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < M * F; i++) {
            const double a = g[i], hv = a / (1 + exp(-a)) * u[i];
            g[i] = round_ops ? (double)round_to_half((float)hv) : hv;
        }
        matmul(d, &L->down, g, F, x, E, 0, M, 1, round_ops);
    }
    /* the logits of the last position only: never operand-rounded (the reference runs its one-token kernel there, metal_llama_decoder.mm:375) */
    rms_rows(d, x + (M - 1) * E, d->output_norm, xn, 1, E, round_all);
    matmul(d, &d->output, xn, E, logits, c->n_vocab, 0, 1, 0, round_all);
    d->pos += n;
    free(x); free(xn); free(qkv); free(att); free(g); free(u);
    return 0;
}

/* Row `token` of the embedding table as floats (Reference::embedding, test_metal_llama_decoder.cpp:163-167; embedq<Q>, llama_kernels.h:1289-1296). */
ORACLE_API void oracle_embedding(const oracle_decoder * d, int32_t token, float * out) {
    const int64_t E = d->cfg.n_embd;
    const uint8_t * row = d->embd.data + (int64_t)token * row_bytes(d->embd.dtype, E);
    for (int64_t i = 0; i < E; i++) out[i] = elem(d->embd.dtype, row, i);
}

/* Appends tokens; logits of the last. Returns 0, 1 on context overflow, 2 on a token outside the vocabulary. */
ORACLE_API int32_t oracle_eval_tokens(oracle_decoder * d, const int32_t * tokens, int32_t n, double * logits) {
    const int64_t E = d->cfg.n_embd;
    if (n < 1) return 1;
    for (int32_t i = 0; i < n; i++) if (tokens[i] < 0 || tokens[i] >= d->cfg.n_vocab) return 2;
    float * emb = (float *)malloc(sizeof(float) * (size_t)((int64_t)n * E));
    for (int32_t i = 0; i < n; i++) oracle_embedding(d, tokens[i], emb + (int64_t)i * E);
    const int32_t rc = oracle_eval_embeddings(d, emb, n, logits);
    free(emb);
    return rc;
}
