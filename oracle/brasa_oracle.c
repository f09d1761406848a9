/*
 * CPU restatement of the reference's arithmetic for the Qwen3 token loop.
 *
 * TEST INFRASTRUCTURE ONLY. Nothing in the product may link or call this file; it is the
 * checker that the CUDA path is compared against, and the timed CPU baseline of the bench.
 *
 * Parity pin: every function here is checked (tests/test_oracle_*.py) against
 *   - the known-answer vectors of the reference's own unit tests
 *     (crates/quant/src/qtype.rs:186-303, crates/quant/src/convert.rs:361-390,
 *      crates/runtime/src/sampler.rs:177-267), and
 *   - golden files produced by importing the reference's Python tools
 *     (tools/convert_brasa.py, tools/brasa_file.py, tools/qwen3_ref.py) — see
 *     tests/golden/make_golden.py.
 *
 * Each function names the reference code it follows. Accumulations are in double, like
 * crates/kernels/src/reference.rs, so the oracle is more precise than any f32 kernel and the
 * test tolerance measures the kernel's distance to this value.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define BO_BLOCK 32
#define BO_KV_DIM 128
#define BO_KV_ROW 136

enum { BO_Q4_0 = 0, BO_Q8_0 = 1, BO_Q6_0 = 2, BO_F32 = 3 };
enum { BO_KV_F32 = 0, BO_KV_F16 = 1, BO_KV_Q8 = 2 };

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* ---- binary16 <-> binary32 (crates/quant/src/qtype.rs:33-78) ------------------------------ */

float bo_f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    int e = (h >> 10) & 31;
    uint32_t m = h & 0x3ffu;
    if (e == 31) return u2f(sign | 0x7f800000u | (m << 13));
    if (e != 0) return u2f(sign | ((uint32_t)(e + 112) << 23) | (m << 13));
    if (m == 0) return u2f(sign);
    /* subnormal: m * 2^-24, exact in float */
    float v = (float)m * 5.9604644775390625e-8f;
    return u2f(f2u(v) | sign);
}

/* Round to nearest, ties to even; overflow to inf; NaN stays NaN. */
uint16_t bo_f32_to_f16(float f) {
    uint32_t x = f2u(f);
    uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    uint32_t a = x & 0x7fffffffu;
    if (a > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);
    if (a >= 0x47800000u) return (uint16_t)(sign | 0x7c00u); /* >= 65536 or inf */
    int e = (int)(a >> 23) - 127;
    uint32_t m = a & 0x7fffffu;
    uint32_t h, rem, half;
    if (e >= -14) {
        h = ((uint32_t)(e + 15) << 10) | (m >> 13);
        rem = m & 0x1fffu;
        half = 0x1000u;
    } else if (e >= -25) {
        uint32_t mant = m | 0x800000u;
        int shift = -1 - e; /* 14..24 */
        h = mant >> shift;
        rem = mant & ((1u << shift) - 1u);
        half = 1u << (shift - 1);
    } else {
        return sign;
    }
    if (rem > half || (rem == half && (h & 1u))) h += 1; /* carry may reach the exponent / inf */
    return (uint16_t)(sign | h);
}

float bo_round_f16(float v) { return bo_f16_to_f32(bo_f32_to_f16(v)); }
void bo_f32_to_f16_array(const float *x, size_t n, uint16_t *out) {
    for (size_t i = 0; i < n; ++i) out[i] = bo_f32_to_f16(x[i]);
}

static inline uint16_t rd16(const uint8_t *p) { return (uint16_t)(p[0] | (p[1] << 8)); }
static inline void wr16(uint8_t *p, uint16_t v) { p[0] = (uint8_t)v; p[1] = (uint8_t)(v >> 8); }

/* ---- block formats (crates/quant/src/qtype.rs:5-29,133-180) -------------------------------- */

size_t bo_nbytes(int q, size_t n) {
    switch (q) {
    case BO_Q4_0: return n / BO_BLOCK * 18;
    case BO_Q8_0: return n / BO_BLOCK * 34;
    case BO_Q6_0: return n / BO_BLOCK * 26;
    default: return n * 4;
    }
}

static inline int q6_code(const uint8_t *b, int i) {
    int ql = b[2 + (i & 15)];
    int lo = i < 16 ? (ql & 15) : (ql >> 4);
    int hi = (b[18 + (i & 7)] >> (2 * (i >> 3))) & 3;
    return lo | (hi << 4);
}

void bo_dequantize(int q, const uint8_t *data, size_t n, float *out) {
    size_t nb = n / BO_BLOCK;
    if (q == BO_F32) { memcpy(out, data, n * 4); return; }
    for (size_t b = 0; b < nb; ++b) {
        float *o = out + b * BO_BLOCK;
        if (q == BO_Q4_0) {
            const uint8_t *p = data + b * 18;
            float d = bo_f16_to_f32(rd16(p));
            for (int j = 0; j < 16; ++j) {
                o[j] = d * (float)((int)(p[2 + j] & 15) - 8);
                o[j + 16] = d * (float)((int)(p[2 + j] >> 4) - 8);
            }
        } else if (q == BO_Q6_0) {
            const uint8_t *p = data + b * 26;
            float d = bo_f16_to_f32(rd16(p));
            for (int j = 0; j < 32; ++j) o[j] = d * (float)(q6_code(p, j) - 32);
        } else {
            const uint8_t *p = data + b * 34;
            float d = bo_f16_to_f32(rd16(p));
            for (int j = 0; j < 32; ++j) o[j] = d * (float)(int8_t)p[2 + j];
        }
    }
}

/* ---- quantisers (crates/quant/src/convert.rs:70-151, tools/convert_brasa.py:49-89) -------- */

static inline float clampf(float v, float lo, float hi) { return v < lo ? lo : (v > hi ? hi : v); }

/* signed element of largest magnitude, first one on ties */
static float block_extreme(const float *v) {
    int idx = 0;
    float best = fabsf(v[0]);
    for (int i = 1; i < BO_BLOCK; ++i) {
        float a = fabsf(v[i]);
        if (a > best) { best = a; idx = i; }
    }
    return v[idx];
}

void bo_quant_q4_0(const float *w, size_t n, uint8_t *out) {
    for (size_t b = 0; b < n / BO_BLOCK; ++b) {
        const float *v = w + b * BO_BLOCK;
        uint8_t *p = out + b * 18;
        uint16_t d16 = bo_f32_to_f16(block_extreme(v) / -8.0f);
        float d = bo_f16_to_f32(d16);
        uint8_t q[BO_BLOCK];
        for (int j = 0; j < BO_BLOCK; ++j)
            q[j] = d != 0.0f ? (uint8_t)clampf(rintf(v[j] / d) + 8.0f, 0.0f, 15.0f) : 8;
        wr16(p, d16);
        for (int j = 0; j < 16; ++j) p[2 + j] = (uint8_t)(q[j] | (q[j + 16] << 4));
    }
}

void bo_quant_q6_0(const float *w, size_t n, uint8_t *out) {
    for (size_t b = 0; b < n / BO_BLOCK; ++b) {
        const float *v = w + b * BO_BLOCK;
        uint8_t *p = out + b * 26;
        uint16_t d16 = bo_f32_to_f16(block_extreme(v) / -32.0f);
        float d = bo_f16_to_f32(d16);
        uint8_t q[BO_BLOCK];
        for (int j = 0; j < BO_BLOCK; ++j)
            q[j] = d != 0.0f ? (uint8_t)clampf(rintf(v[j] / d) + 32.0f, 0.0f, 63.0f) : 32;
        wr16(p, d16);
        for (int j = 0; j < 16; ++j) p[2 + j] = (uint8_t)((q[j] & 15) | ((q[j + 16] & 15) << 4));
        for (int j = 0; j < 8; ++j)
            p[18 + j] = (uint8_t)((q[j] >> 4) | ((q[j + 8] >> 4) << 2) | ((q[j + 16] >> 4) << 4) |
                                  ((q[j + 24] >> 4) << 6));
    }
}

static void q8_block(const float *v, uint8_t *codes, uint16_t *d16_out) {
    float amax = 0.0f;
    for (int j = 0; j < BO_BLOCK; ++j) amax = fmaxf(amax, fabsf(v[j]));
    uint16_t d16 = bo_f32_to_f16(amax / 127.0f);
    float d = bo_f16_to_f32(d16);
    for (int j = 0; j < BO_BLOCK; ++j) {
        float q = d == 0.0f ? 0.0f : clampf(rintf(v[j] / d), -127.0f, 127.0f);
        codes[j] = (uint8_t)(int8_t)q;
    }
    *d16_out = d16;
}

void bo_quant_q8_0(const float *w, size_t n, uint8_t *out) {
    for (size_t b = 0; b < n / BO_BLOCK; ++b) {
        uint16_t d16;
        q8_block(w + b * BO_BLOCK, out + b * 34 + 2, &d16);
        wr16(out + b * 34, d16);
    }
}

/* ---- KV-cache Q8 rows (crates/quant/src/qtype.rs:89-130) ----------------------------------- */

void bo_quantize_kv_q8(const float *x, size_t n, uint8_t *out) {
    for (size_t r = 0; r < n / BO_KV_DIM; ++r) {
        uint8_t *o = out + r * BO_KV_ROW;
        for (int b = 0; b < 4; ++b) {
            uint16_t d16;
            q8_block(x + r * BO_KV_DIM + b * BO_BLOCK, o + b * BO_BLOCK, &d16);
            wr16(o + BO_KV_DIM + 2 * b, d16);
        }
    }
}

void bo_dequantize_kv_q8(const uint8_t *data, size_t n, float *out) {
    for (size_t r = 0; r < n / BO_KV_DIM; ++r) {
        const uint8_t *p = data + r * BO_KV_ROW;
        for (int i = 0; i < BO_KV_DIM; ++i) {
            float d = bo_f16_to_f32(rd16(p + BO_KV_DIM + 2 * (i / BO_BLOCK)));
            out[r * BO_KV_DIM + i] = d * (float)(int8_t)p[i];
        }
    }
}

/* values as they read back from a cache of type kv (tools/qwen3_ref.py:72-82,117-123) */
void bo_round_kv(int kv, const float *x, size_t n, float *out) {
    if (kv == BO_KV_F32) { memmove(out, x, n * 4); return; }
    if (kv == BO_KV_F16) { for (size_t i = 0; i < n; ++i) out[i] = bo_round_f16(x[i]); return; }
    uint8_t row[BO_KV_ROW];
    for (size_t r = 0; r < n / BO_KV_DIM; ++r) {
        bo_quantize_kv_q8(x + r * BO_KV_DIM, BO_KV_DIM, row);
        bo_dequantize_kv_q8(row, BO_KV_DIM, out + r * BO_KV_DIM);
    }
}

/* ---- per-kernel references (crates/kernels/src/reference.rs) ------------------------------- */

void bo_add(const float *a, const float *b, size_t n, float *out) {
    for (size_t i = 0; i < n; ++i) out[i] = a[i] + b[i];
}

void bo_swiglu(const float *gate, const float *up, size_t n, float *out) {
    for (size_t i = 0; i < n; ++i) {
        double g = gate[i];
        out[i] = (float)(g / (1.0 + exp(-g)) * (double)up[i]);
    }
}

void bo_rms_norm(const float *x, const float *w, size_t rows, size_t n, float eps, float *out) {
    for (size_t r = 0; r < rows; ++r) {
        const float *xr = x + r * n;
        double ss = 0.0;
        for (size_t i = 0; i < n; ++i) ss += (double)xr[i] * (double)xr[i];
        double scale = 1.0 / sqrt(ss / (double)n + (double)eps);
        for (size_t i = 0; i < n; ++i) out[r * n + i] = (float)((double)xr[i] * scale * (double)w[i]);
    }
}

void bo_softmax(const float *x, size_t rows, size_t n, float *out) {
    for (size_t r = 0; r < rows; ++r) {
        const float *xr = x + r * n;
        double m = -INFINITY, s = 0.0;
        for (size_t i = 0; i < n; ++i) m = fmax(m, (double)xr[i]);
        for (size_t i = 0; i < n; ++i) s += exp((double)xr[i] - m);
        for (size_t i = 0; i < n; ++i) out[r * n + i] = (float)(exp((double)xr[i] - m) / s);
    }
}

/* cos/sin(p * theta^(-2i/dim)) in double, stored as float (crates/kernels/src/lib.rs:1389-1404) */
void bo_rope_table(double theta, int dim, size_t max_pos, float *cosv, float *sinv) {
    int half = dim / 2;
    for (size_t p = 0; p < max_pos; ++p)
        for (int i = 0; i < half; ++i) {
            double inv = 1.0 / pow(theta, (double)(2 * i) / (double)dim);
            double a = (double)p * inv;
            cosv[p * half + i] = (float)cos(a);
            sinv[p * half + i] = (float)sin(a);
        }
}

/* in place on x[T, heads, dim]; pairs (i, i + dim/2) (reference.rs:46-62) */
void bo_rope_neox(float *x, size_t tokens, int heads, int dim, size_t pos0, const float *cosv,
                  const float *sinv) {
    int half = dim / 2;
    for (size_t t = 0; t < tokens; ++t)
        for (int h = 0; h < heads; ++h) {
            float *v = x + (t * heads + h) * dim;
            for (int i = 0; i < half; ++i) {
                double c = cosv[(pos0 + t) * half + i], s = sinv[(pos0 + t) * half + i];
                double a = v[i], b = v[i + half];
                v[i] = (float)(a * c - b * s);
                v[i + half] = (float)(b * c + a * s);
            }
        }
}

/* y[t, r] = sum_k W[r, k] x[t, k]; abs_sum (optional) = sum_k |W x| per output: the tolerance
 * scale of the GEMV/GEMM tests. f16_inputs != 0 rounds dequantised weights and x to f16 first,
 * as the prefill GEMM does (reference.rs:64-114). Rows are independent: OpenMP over them. */
void bo_matmul(int q, const uint8_t *w, size_t rows, size_t cols, const float *x, size_t tokens,
               float *y, float *abs_sum, int f16_inputs) {
    size_t row_bytes = bo_nbytes(q, cols);
    float *xr = (float *)malloc(tokens * cols * sizeof(float));
    for (size_t i = 0; i < tokens * cols; ++i) xr[i] = f16_inputs ? bo_round_f16(x[i]) : x[i];
#pragma omp parallel
    {
        float *wr = (float *)malloc(cols * sizeof(float));
#pragma omp for schedule(static)
        for (long r = 0; r < (long)rows; ++r) {
            bo_dequantize(q, w + (size_t)r * row_bytes, cols, wr);
            if (f16_inputs)
                for (size_t k = 0; k < cols; ++k) wr[k] = bo_round_f16(wr[k]);
            for (size_t t = 0; t < tokens; ++t) {
                const float *xt = xr + t * cols;
                double s = 0.0, a = 0.0;
                for (size_t k = 0; k < cols; ++k) {
                    double p = (double)wr[k] * (double)xt[k];
                    s += p;
                    a += fabs(p);
                }
                y[t * rows + (size_t)r] = (float)s;
                if (abs_sum) abs_sum[t * rows + (size_t)r] = (float)a;
            }
        }
        free(wr);
    }
    free(xr);
}

void bo_embed(int q, const uint8_t *table, size_t h, const uint32_t *ids, size_t tokens, float *out) {
    size_t row_bytes = bo_nbytes(q, h);
    for (size_t t = 0; t < tokens; ++t) bo_dequantize(q, table + (size_t)ids[t] * row_bytes, h, out + t * h);
}

/* Causal GQA attention in double (reference.rs:116-218). q: [T, hq, dim]; k, v: [pos0+T, hkv, dim]
 * with row stride kv_stride floats between positions. q16 != 0: Q*scale rounded to f16 (computed
 * in float) like the prefill attention. vmax (optional): max_j |v_j| per output component. */
void bo_attention(const float *q, const float *k, const float *v, size_t tokens, int hq, int hkv,
                  int dim, size_t pos0, size_t kv_stride, int q16, float *o, float *vmax) {
    int group = hq / hkv;
    float fscale = 1.0f / sqrtf((float)dim);
    double dscale = 1.0 / sqrt((double)dim);
#pragma omp parallel for collapse(2) schedule(dynamic)
    for (long t = 0; t < (long)tokens; ++t)
        for (int h = 0; h < hq; ++h) {
            size_t last = pos0 + (size_t)t;
            int kh = h / group;
            const float *qv = q + ((size_t)t * hq + h) * dim;
            double *s = (double *)malloc((last + 1) * sizeof(double));
            double *qq = (double *)malloc(dim * sizeof(double));
            for (int d = 0; d < dim; ++d) qq[d] = q16 ? (double)bo_round_f16(qv[d] * fscale) : (double)qv[d];
            double m = -INFINITY;
            for (size_t j = 0; j <= last; ++j) {
                const float *kv = k + j * kv_stride + (size_t)kh * dim;
                double acc = 0.0;
                for (int d = 0; d < dim; ++d) acc += qq[d] * (double)kv[d];
                s[j] = q16 ? acc : acc * dscale;
                m = fmax(m, s[j]);
            }
            double z = 0.0;
            for (size_t j = 0; j <= last; ++j) { s[j] = exp(s[j] - m); z += s[j]; }
            for (int d = 0; d < dim; ++d) {
                double acc = 0.0;
                float mx = 0.0f;
                for (size_t j = 0; j <= last; ++j) {
                    float vj = v[j * kv_stride + (size_t)kh * dim + d];
                    acc += s[j] / z * (double)vj;
                    mx = fmaxf(mx, fabsf(vj));
                }
                o[((size_t)t * hq + h) * dim + d] = (float)acc;
                if (vmax) vmax[((size_t)t * hq + h) * dim + d] = mx;
            }
            free(s);
            free(qq);
        }
}

/* ---- deterministic test inputs (crates/kernels/src/testutil.rs:1-83) ----------------------- */

static inline uint64_t xs_next(uint64_t *s) {
    uint64_t x = *s;
    x ^= x >> 12;
    x ^= x << 25;
    x ^= x >> 27;
    *s = x;
    return x * 0x2545F4914F6CDD1DULL;
}

uint64_t bo_rng_new(uint64_t seed) { return seed ? seed : 1; }
uint64_t bo_rng_next_u64(uint64_t *s) { return xs_next(s); }

/* n uniforms in [-scale, scale) */
void bo_rng_vec(uint64_t *s, size_t n, float scale, float *out) {
    for (size_t i = 0; i < n; ++i) out[i] = ((float)(xs_next(s) >> 40) / 8388608.0f - 1.0f) * scale;
}

static void rng_scale(uint64_t *s, uint8_t *p) {
    uint16_t sign = (uint16_t)(xs_next(s) & 1);
    uint16_t ex = (uint16_t)(7 + xs_next(s) % 7);
    uint16_t mant = (uint16_t)(xs_next(s) & 0x3ff);
    wr16(p, (uint16_t)((sign << 15) | (ex << 10) | mant));
}

/* random quantised matrix bytes: scale then payload per block */
void bo_rng_qmatrix(uint64_t *s, int q, size_t rows, size_t cols, uint8_t *out) {
    size_t nb = rows * cols / BO_BLOCK;
    for (size_t b = 0; b < nb; ++b) {
        if (q == BO_Q4_0) {
            rng_scale(s, out); out += 2;
            for (int j = 0; j < 16; ++j) *out++ = (uint8_t)xs_next(s);
        } else if (q == BO_Q6_0) {
            rng_scale(s, out); out += 2;
            for (int j = 0; j < 24; ++j) *out++ = (uint8_t)xs_next(s);
        } else {
            rng_scale(s, out); out += 2;
            for (int j = 0; j < 32; ++j) *out++ = (uint8_t)(int8_t)((int)(xs_next(s) % 255) - 127);
        }
    }
}

/* ---- sampler (crates/runtime/src/sampler.rs:46-170) ---------------------------------------- */

typedef struct { uint64_t state, inc; } BoPcg32;

static uint32_t pcg_next(BoPcg32 *r) {
    uint64_t old = r->state;
    r->state = old * 6364136223846793005ULL + r->inc;
    uint32_t x = (uint32_t)(((old >> 18) ^ old) >> 27);
    uint32_t rot = (uint32_t)(old >> 59);
    return (x >> rot) | (x << ((32 - rot) & 31));
}

void bo_pcg32_new(uint64_t seed, BoPcg32 *r) {
    r->state = 0;
    r->inc = (0xda3e39cb94b95bdbULL << 1) | 1;
    pcg_next(r);
    r->state += seed;
    pcg_next(r);
}
uint32_t bo_pcg32_next_u32(BoPcg32 *r) { return pcg_next(r); }
float bo_pcg32_next_f32(BoPcg32 *r) { return (float)(pcg_next(r) >> 8) / 16777216.0f; }

/* first index of the maximum; NaN never wins; 0 when nothing exceeds -inf (sampler.rs:148-170) */
uint32_t bo_argmax(const float *v, size_t n) {
    float m = -INFINITY;
    for (size_t i = 0; i < n; ++i) if (v[i] > m) m = v[i];
    if (m == -INFINITY) return 0;
    for (size_t i = 0; i < n; ++i) if (v[i] == m) return (uint32_t)i;
    return 0;
}

typedef struct { uint32_t id; float v; } BoCand;

/* f32::total_cmp key: sign-magnitude bits to a monotone signed integer */
static inline int32_t total_key(float f) {
    int32_t b = (int32_t)f2u(f);
    return b ^ (int32_t)(((uint32_t)(b >> 31)) >> 1);
}
/* descending by logit; equal logits keep ascending token id (the reference's unstable sort leaves
 * that order unspecified) */
static int cand_cmp(const void *pa, const void *pb) {
    const BoCand *a = (const BoCand *)pa, *b = (const BoCand *)pb;
    int32_t ka = total_key(a->v), kb = total_key(b->v);
    if (ka != kb) return ka > kb ? -1 : 1;
    return a->id < b->id ? -1 : (a->id > b->id ? 1 : 0);
}

/* One draw. temperature <= 0 is greedy. Sequential f32 sums in sorted order, as sampler.rs:103-146.
 * keep_out (optional) receives the number of candidates kept by top-k/top-p. */
uint32_t bo_sample(BoPcg32 *rng, float temperature, size_t top_k, float top_p, const float *logits,
                   size_t n, size_t *keep_out) {
    if (temperature <= 0.0f) return bo_argmax(logits, n);
    BoCand *c = (BoCand *)malloc(n * sizeof(BoCand));
    for (size_t i = 0; i < n; ++i) { c[i].id = (uint32_t)i; c[i].v = logits[i]; }
    qsort(c, n, sizeof(BoCand), cand_cmp);
    size_t len = (top_k > 0 && top_k < n) ? top_k : n;
    float mx = c[0].v, sum = 0.0f;
    for (size_t i = 0; i < len; ++i) { c[i].v = expf((c[i].v - mx) / temperature); sum += c[i].v; }
    size_t keep = len;
    if (top_p < 1.0f) {
        float acc = 0.0f;
        for (size_t i = 0; i < len; ++i) {
            acc += c[i].v / sum;
            if (acc >= top_p) { keep = i + 1; break; }
        }
    }
    float total = 0.0f;
    for (size_t i = 0; i < keep; ++i) total += c[i].v;
    float r = bo_pcg32_next_f32(rng) * total;
    uint32_t pick = c[keep - 1].id;
    for (size_t i = 0; i < keep; ++i) {
        r -= c[i].v;
        if (r <= 0.0f) { pick = c[i].id; break; }
    }
    if (keep_out) *keep_out = keep;
    free(c);
    return pick;
}

/* ---- whole-model forward (tools/qwen3_ref.py:130-176; crates/models/src/qwen3.rs:549-831) -- */

typedef struct {
    const float *attn_norm, *q_norm, *k_norm, *ffn_norm;
    const uint8_t *wq, *wk, *wv, *wo, *gate, *up, *down;
} BoLayer;

typedef struct {
    int32_t hidden, layers, heads, kv_heads, head_dim, ffn, vocab;
    float eps;
    double rope_theta;
    int32_t layer_qtype;  /* q4_0 for every linear */
    int32_t embed_qtype;  /* q6_0 (or q8_0) */
    int32_t head_qtype;   /* qtype of head (== embed_qtype when tied) */
    const uint8_t *embed;
    const uint8_t *head;  /* lm_head rows; the embedding table when tied */
    const float *final_norm;
    const BoLayer *layer;
} BoModel;

/* KV cache as float values after rounding to the cache type: [layers, ctx, kv_heads*head_dim]. */
typedef struct {
    int32_t kv_type;
    size_t ctx;
    float *k, *v;
} BoCache;

/* Runs `tokens` new ids from position pos0 and writes logits of the last logit_rows positions.
 * f16_prefill != 0 applies the rounding points of the reference's F16 prefill precision
 * (qwen3.rs:516-533,632-669): GEMM inputs (normalised activations, attention output, SwiGLU
 * output) and dequantised weights rounded to f16, Q*scale rounded to f16. hidden_out (optional)
 * receives x after every layer: [layers, tokens, hidden]. Returns 0, or -1 on bad arguments. */
int bo_qwen3_forward(const BoModel *m, BoCache *c, const uint32_t *ids, size_t tokens, size_t pos0,
                     size_t logit_rows, int f16_prefill, float *logits, float *hidden_out) {
    size_t H = (size_t)m->hidden, D = (size_t)m->head_dim, F = (size_t)m->ffn;
    size_t qd = (size_t)m->heads * D, kvd = (size_t)m->kv_heads * D;
    if (tokens == 0 || pos0 + tokens > c->ctx || logit_rows == 0 || logit_rows > tokens) return -1;
    int lq = m->layer_qtype;
    float *x = (float *)malloc(tokens * H * 4), *h = (float *)malloc(tokens * H * 4);
    float *q = (float *)malloc(tokens * qd * 4), *k = (float *)malloc(tokens * kvd * 4);
    float *v = (float *)malloc(tokens * kvd * 4), *att = (float *)malloc(tokens * qd * 4);
    float *g = (float *)malloc(tokens * F * 4), *u = (float *)malloc(tokens * F * 4);
    float *cosv = (float *)malloc((pos0 + tokens) * (D / 2) * 4);
    float *sinv = (float *)malloc((pos0 + tokens) * (D / 2) * 4);
    bo_rope_table(m->rope_theta, (int)D, pos0 + tokens, cosv, sinv);
    bo_embed(m->embed_qtype, m->embed, H, ids, tokens, x);
    for (int li = 0; li < m->layers; ++li) {
        const BoLayer *L = &m->layer[li];
        float *kc = c->k + (size_t)li * c->ctx * kvd, *vc = c->v + (size_t)li * c->ctx * kvd;
        bo_rms_norm(x, L->attn_norm, tokens, H, m->eps, h);
        bo_matmul(lq, L->wq, qd, H, h, tokens, q, NULL, f16_prefill);
        bo_matmul(lq, L->wk, kvd, H, h, tokens, k, NULL, f16_prefill);
        bo_matmul(lq, L->wv, kvd, H, h, tokens, v, NULL, f16_prefill);
        bo_rms_norm(q, L->q_norm, tokens * (size_t)m->heads, D, m->eps, q);
        bo_rms_norm(k, L->k_norm, tokens * (size_t)m->kv_heads, D, m->eps, k);
        bo_rope_neox(q, tokens, m->heads, (int)D, pos0, cosv, sinv);
        bo_rope_neox(k, tokens, m->kv_heads, (int)D, pos0, cosv, sinv);
        bo_round_kv(c->kv_type, k, tokens * kvd, kc + pos0 * kvd);
        bo_round_kv(c->kv_type, v, tokens * kvd, vc + pos0 * kvd);
        bo_attention(q, kc, vc, tokens, m->heads, m->kv_heads, (int)D, pos0, kvd, f16_prefill, att, NULL);
        /* the f16 rounding of the attention output and of SwiGLU happens inside bo_matmul's
         * f16_inputs rounding of x, which is the same value */
        bo_matmul(lq, L->wo, H, qd, att, tokens, h, NULL, f16_prefill);
        for (size_t i = 0; i < tokens * H; ++i) x[i] += h[i];
        bo_rms_norm(x, L->ffn_norm, tokens, H, m->eps, h);
        bo_matmul(lq, L->gate, F, H, h, tokens, g, NULL, f16_prefill);
        bo_matmul(lq, L->up, F, H, h, tokens, u, NULL, f16_prefill);
        if (f16_prefill) {
            /* swiglu_f16 == f16(f32 swiglu) (crates/kernels/tests/ops.rs:319-368) */
            for (size_t i = 0; i < tokens * F; ++i) {
                float gg = g[i];
                g[i] = (gg / (1.0f + expf(-gg))) * u[i];
            }
        } else {
            bo_swiglu(g, u, tokens * F, g);
        }
        bo_matmul(lq, L->down, H, F, g, tokens, h, NULL, f16_prefill);
        for (size_t i = 0; i < tokens * H; ++i) x[i] += h[i];
        if (hidden_out) memcpy(hidden_out + (size_t)li * tokens * H, x, tokens * H * 4);
    }
    size_t first = tokens - logit_rows;
    bo_rms_norm(x + first * H, m->final_norm, logit_rows, H, m->eps, h);
    bo_matmul(m->head_qtype, m->head, (size_t)m->vocab, H, h, logit_rows, logits, NULL, 0);
    free(x); free(h); free(q); free(k); free(v); free(att); free(g); free(u); free(cosv); free(sinv);
    return 0;
}
