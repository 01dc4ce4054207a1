/*
 * CPU oracle — see lisa_oracle.h.  TEST INFRASTRUCTURE ONLY: never linked into
 * or called from the CUDA library.  Build with -O2 -ffp-contract=off so that
 * every a*b+c below is two roundings, as the reference's scalar Rust is.
 */
#include "lisa_oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ */
/* scalar conversions                                                  */
/* ------------------------------------------------------------------ */

static inline uint32_t f32_bits(float v) {
    uint32_t u;
    memcpy(&u, &v, 4);
    return u;
}
static inline float bits_f32(uint32_t u) {
    float v;
    memcpy(&v, &u, 4);
    return v;
}

/* half::bf16::from_f32 (half 2.7.1): round to nearest even, NaN kept quiet. */
uint16_t oracle_f32_to_bf16(float v) {
    uint32_t u = f32_bits(v);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
    uint32_t round_bit = 0x00008000u;
    if ((u & round_bit) != 0 && (u & (3u * round_bit - 1u)) != 0) return (uint16_t)((u >> 16) + 1u);
    return (uint16_t)(u >> 16);
}
float oracle_bf16_to_f32(uint16_t v) { return bits_f32((uint32_t)v << 16); }

float oracle_f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    if (exp == 0) {
        if (man == 0) return bits_f32(sign);
        /* subnormal: value = man * 2^-24 */
        float f = (float)man * (1.0f / 16777216.0f);
        return bits_f32(f32_bits(f) | sign);
    }
    if (exp == 31) return bits_f32(sign | 0x7f800000u | (man << 13));
    return bits_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

uint16_t oracle_f32_to_f16(float v) {
    uint32_t u = f32_bits(v);
    uint32_t sign = (u >> 16) & 0x8000u;
    uint32_t a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);
    if (a >= 0x47800000u) return (uint16_t)(sign | 0x7c00u); /* overflow incl. inf; 65520 rounds up */
    if (a < 0x33000000u) return (uint16_t)sign;               /* below half the smallest subnormal */
    int e = (int)(a >> 23) - 127;
    uint32_t m = (a & 0x7fffffu) | 0x800000u;
    int shift = (e < -14) ? (13 + (-14 - e)) : 13;
    uint32_t half_m = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (half_m & 1u))) half_m++;
    uint32_t out;
    if (e < -14) out = half_m; /* subnormal (may carry into the first normal) */
    else out = ((uint32_t)(e + 15) << 10) + (half_m - 0x400u);
    if (out >= 0x7c00u) out = 0x7c00u;
    return (uint16_t)(sign | out);
}

/* ------------------------------------------------------------------ */
/* threads                                                             */
/* ------------------------------------------------------------------ */

typedef void (*range_fn)(void *ctx, int64_t begin, int64_t end);
typedef struct {
    range_fn fn;
    void *ctx;
    int64_t begin, end;
} range_job;

static void *range_thread(void *p) {
    range_job *j = (range_job *)p;
    j->fn(j->ctx, j->begin, j->end);
    return NULL;
}

/* Contiguous split of [0,total) over `threads` workers, like rayon's chunks. */
static void parallel_rows(int64_t total, int threads, range_fn fn, void *ctx) {
    if (threads < 1) threads = 1;
    if (threads > total) threads = (int)(total > 0 ? total : 1);
    if (threads == 1) {
        fn(ctx, 0, total);
        return;
    }
    pthread_t *tid = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)threads);
    range_job *jobs = (range_job *)malloc(sizeof(range_job) * (size_t)threads);
    int64_t per = (total + threads - 1) / threads;
    int started = 0;
    for (int t = 0; t < threads; ++t) {
        int64_t b = (int64_t)t * per, e = b + per;
        if (b >= total) break;
        if (e > total) e = total;
        jobs[t] = (range_job){fn, ctx, b, e};
        pthread_create(&tid[t], NULL, range_thread, &jobs[t]);
        started++;
    }
    for (int t = 0; t < started; ++t) pthread_join(tid[t], NULL);
    free(tid);
    free(jobs);
}

/* ------------------------------------------------------------------ */
/* affine                                                              */
/* ------------------------------------------------------------------ */

static int affine_args_ok(int64_t k, int group_size, int bits) {
    if (bits != 2 && bits != 4 && bits != 8) return 0;
    if (group_size != 32 && group_size != 64 && group_size != 128) return 0;
    if (k <= 0 || k % group_size != 0) return 0;
    return 1;
}

/* One row of array_ops.rs:66-76. */
static void dequant_row_f32(const uint32_t *wrow, const uint16_t *srow, const uint16_t *brow,
                            int64_t k, int group_size, int bits, int round_bf16, float *out) {
    const int per_word = 32 / bits;
    const uint32_t mask = (bits == 32) ? 0xffffffffu : ((1u << bits) - 1u);
    for (int64_t c = 0; c < k; ++c) {
        uint32_t word = wrow[c / per_word];
        uint32_t qv = (word >> ((c % per_word) * bits)) & mask;
        int64_t g = c / group_size;
        float v = (float)qv * oracle_bf16_to_f32(srow[g]) + oracle_bf16_to_f32(brow[g]);
        out[c] = round_bf16 ? oracle_bf16_to_f32(oracle_f32_to_bf16(v)) : v;
    }
}

int oracle_affine_dequantize_f32(const uint32_t *w, const uint16_t *scales, const uint16_t *biases,
                                 int64_t rows, int64_t k, int group_size, int bits, float *out) {
    if (!affine_args_ok(k, group_size, bits)) return -1;
    const int64_t kq = k * bits / 32, groups = k / group_size;
    for (int64_t r = 0; r < rows; ++r)
        dequant_row_f32(w + r * kq, scales + r * groups, biases + r * groups, k, group_size, bits, 0,
                        out + r * k);
    return 0;
}

int oracle_affine_dequantize_bf16(const uint32_t *w, const uint16_t *scales, const uint16_t *biases,
                                  int64_t rows, int64_t k, int group_size, int bits,
                                  uint16_t *out) {
    if (!affine_args_ok(k, group_size, bits)) return -1;
    const int64_t kq = k * bits / 32, groups = k / group_size;
    float *tmp = (float *)malloc(sizeof(float) * (size_t)k);
    for (int64_t r = 0; r < rows; ++r) {
        dequant_row_f32(w + r * kq, scales + r * groups, biases + r * groups, k, group_size, bits, 0,
                        tmp);
        for (int64_t c = 0; c < k; ++c) out[r * k + c] = oracle_f32_to_bf16(tmp[c]);
    }
    free(tmp);
    return 0;
}

typedef struct {
    const uint16_t *x;
    int64_t m, k, n;
    const uint32_t *w;
    const uint16_t *scales, *biases;
    int group_size, bits, round_w;
    uint16_t *y;
    double *y64;
    const int32_t *ids; /* gather: expert per x row, else NULL */
} matmul_ctx;

/* Output rows [begin,end) of W: dequantize the row once, then the scalar loop
 * of cpu.rs:50-58 for every input row. */
static void matmul_rows(void *p, int64_t begin, int64_t end) {
    matmul_ctx *c = (matmul_ctx *)p;
    const int64_t kq = c->k * c->bits / 32, groups = c->k / c->group_size;
    float *wrow = (float *)malloc(sizeof(float) * (size_t)c->k);
    float *xf = (float *)malloc(sizeof(float) * (size_t)c->k);
    for (int64_t n = begin; n < end; ++n) {
        dequant_row_f32(c->w + n * kq, c->scales + n * groups, c->biases + n * groups, c->k,
                        c->group_size, c->bits, c->round_w, wrow);
        for (int64_t r = 0; r < c->m; ++r) {
            const uint16_t *xr = c->x + r * c->k;
            if (c->y64) {
                double acc = 0.0;
                for (int64_t k = 0; k < c->k; ++k)
                    acc += (double)oracle_bf16_to_f32(xr[k]) * (double)wrow[k];
                c->y64[r * c->n + n] = acc;
            } else {
                for (int64_t k = 0; k < c->k; ++k) xf[k] = oracle_bf16_to_f32(xr[k]);
                float acc = 0.0f;
                for (int64_t k = 0; k < c->k; ++k) acc += xf[k] * wrow[k];
                c->y[r * c->n + n] = oracle_f32_to_bf16(acc);
            }
        }
    }
    free(wrow);
    free(xf);
}

int oracle_affine_matmul(const uint16_t *x, int64_t m, int64_t k, const uint32_t *w,
                         const uint16_t *scales, const uint16_t *biases, int64_t n, int group_size,
                         int bits, int round_weight_bf16, int threads, uint16_t *y) {
    if (!affine_args_ok(k, group_size, bits) || m < 0 || n < 0) return -1;
    matmul_ctx c = {x, m, k, n, w, scales, biases, group_size, bits, round_weight_bf16, y, NULL, NULL};
    parallel_rows(n, threads, matmul_rows, &c);
    return 0;
}

int oracle_affine_matmul_f64(const uint16_t *x, int64_t m, int64_t k, const uint32_t *w,
                             const uint16_t *scales, const uint16_t *biases, int64_t n,
                             int group_size, int bits, int round_weight_bf16, int threads,
                             double *y) {
    if (!affine_args_ok(k, group_size, bits) || m < 0 || n < 0) return -1;
    matmul_ctx c = {x, m, k, n, w, scales, biases, group_size, bits, round_weight_bf16, NULL, y, NULL};
    parallel_rows(n, threads, matmul_rows, &c);
    return 0;
}

int oracle_affine_qmv_factored(const uint16_t *x, int64_t m, int64_t k, const uint32_t *w,
                               const uint16_t *scales, const uint16_t *biases, int64_t n,
                               int group_size, int bits, uint16_t *y) {
    if (!affine_args_ok(k, group_size, bits)) return -1;
    const int per_word = 32 / bits;
    const uint32_t mask = (1u << bits) - 1u;
    const int64_t kq = k * bits / 32, groups = k / group_size;
    for (int64_t r = 0; r < m; ++r)
        for (int64_t o = 0; o < n; ++o) {
            float result = 0.0f;
            for (int64_t g = 0; g < groups; ++g) {
                float accum = 0.0f, xsum = 0.0f;
                for (int64_t c = g * group_size; c < (g + 1) * group_size; ++c) {
                    uint32_t q = (w[o * kq + c / per_word] >> ((c % per_word) * bits)) & mask;
                    float xv = oracle_bf16_to_f32(x[r * k + c]);
                    accum += xv * (float)q;
                    xsum += xv;
                }
                result += oracle_bf16_to_f32(scales[o * groups + g]) * accum +
                          xsum * oracle_bf16_to_f32(biases[o * groups + g]);
            }
            y[r * n + o] = oracle_f32_to_bf16(result);
        }
    return 0;
}

int oracle_affine_quantize(const float *w, int64_t rows, int64_t k, int group_size, int bits,
                           uint32_t *wq, float *scales, float *biases) {
    if (!affine_args_ok(k, group_size, bits) || group_size % (32 / bits) != 0) return -1;
    const int64_t groups = k / group_size;
    const int per_word = 32 / bits;
    const float maxq = (float)((1u << bits) - 1u);
    const float eps = 1e-7f;
    memset(wq, 0, sizeof(uint32_t) * (size_t)(rows * k * bits / 32));
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t g = 0; g < groups; ++g) {
            const int64_t base = r * k + g * group_size;
            float w_min = 3.40282347e+38f, w_max = 0.0f; /* f32::MAX, 0 as array_ops.rs:246-247 */
            for (int i = 0; i < group_size; ++i) {
                float v = w[base + i];
                w_min = fminf(w_min, v);
                w_max = fmaxf(w_max, v);
            }
            float scale = fmaxf((w_max - w_min) / maxq, eps);
            int side = fabsf(w_min) > fabsf(w_max);
            if (!side) scale = -scale;
            float edge = side ? w_min : w_max;
            float q0 = roundf(edge / scale); /* f32::round: half away from zero */
            int at_zero = (q0 == 0.0f);
            if (!at_zero) scale = edge / q0;
            float bias = at_zero ? 0.0f : edge;
            scales[r * groups + g] = scale;
            biases[r * groups + g] = bias;
            for (int i = 0; i < group_size; ++i) {
                float qf = fminf(roundf((w[base + i] - bias) / scale), maxq);
                int32_t q = (int32_t)qf; /* `as i32` saturates; NaN -> 0 */
                if (qf != qf) q = 0;
                int64_t word = base / per_word + i / per_word;
                int shift = (i % per_word) * bits;
                wq[word] |= ((uint32_t)q & ((1u << bits) - 1u)) << shift;
            }
        }
    return 0;
}

void oracle_lcg_fill(uint64_t *seed, float *out, int64_t count) {
    uint64_t s = *seed;
    for (int64_t i = 0; i < count; ++i) {
        s = s * 6364136223846793005ull + 1ull;
        out[i] = (float)((double)(s >> 40) / 8388608.0 - 1.0);
    }
    *seed = s;
}

typedef struct {
    matmul_ctx base;
    int64_t experts;
} gather_ctx;

/* x rows [begin,end): row r uses expert ids[r]; each expert run is the plain
 * quantized matmul of array_ops.rs:591-630. */
static void gather_rows(void *p, int64_t begin, int64_t end) {
    gather_ctx *g = (gather_ctx *)p;
    matmul_ctx *c = &g->base;
    const int64_t kq = c->k * c->bits / 32, groups = c->k / c->group_size;
    float *wrow = (float *)malloc(sizeof(float) * (size_t)c->k);
    float *xf = (float *)malloc(sizeof(float) * (size_t)c->k);
    for (int64_t r = begin; r < end; ++r) {
        int32_t e = c->ids[r];
        for (int64_t k = 0; k < c->k; ++k) xf[k] = oracle_bf16_to_f32(c->x[r * c->k + k]);
        for (int64_t n = 0; n < c->n; ++n) {
            if (e < 0 || e >= g->experts) {
                c->y[r * c->n + n] = 0;
                continue;
            }
            dequant_row_f32(c->w + ((int64_t)e * c->n + n) * kq,
                            c->scales + ((int64_t)e * c->n + n) * groups,
                            c->biases + ((int64_t)e * c->n + n) * groups, c->k, c->group_size,
                            c->bits, c->round_w, wrow);
            float acc = 0.0f;
            for (int64_t k = 0; k < c->k; ++k) acc += xf[k] * wrow[k];
            c->y[r * c->n + n] = oracle_f32_to_bf16(acc);
        }
    }
    free(wrow);
    free(xf);
}

int oracle_gather_qmm(const uint16_t *x, int64_t rows, int64_t k, const uint32_t *w,
                      const uint16_t *scales, const uint16_t *biases, const int32_t *ids,
                      int64_t experts, int64_t n, int group_size, int bits,
                      int round_weight_bf16, int threads, uint16_t *y) {
    if (!affine_args_ok(k, group_size, bits)) return -1;
    gather_ctx g = {{x, rows, k, n, w, scales, biases, group_size, bits, round_weight_bf16, y, NULL, ids},
                    experts};
    parallel_rows(rows, threads, gather_rows, &g);
    return 0;
}

/* ------------------------------------------------------------------ */
/* GGUF K-quants                                                       */
/* ------------------------------------------------------------------ */

int oracle_gguf_block_bytes(int format) {
    switch (format) { /* lib.rs:46-48 */
    case ORACLE_GGUF_Q8_0: return 34;
    case ORACLE_GGUF_Q2_K: return 84;
    case ORACLE_GGUF_Q4_K: return 144;
    case ORACLE_GGUF_Q5_K: return 176;
    default: return -1;
    }
}

int oracle_gguf_block_width(int format) { /* elements of a block, lib.rs:36-70 */
    switch (format) {
    case ORACLE_GGUF_Q8_0: return 32;
    case ORACLE_GGUF_Q2_K:
    case ORACLE_GGUF_Q4_K:
    case ORACLE_GGUF_Q5_K: return 256;
    default: return -1;
    }
}

static float f16_at(const uint8_t *b, int at) {
    return oracle_f16_to_f32((uint16_t)(b[at] | ((uint16_t)b[at + 1] << 8)));
}

/* quant.rs:64-80 */
static void decode_q2_k(const uint8_t *b, float *out) {
    const float d = f16_at(b, 80), min = f16_at(b, 82);
    for (int half = 0; half < 2; ++half)
        for (int shift = 0; shift < 4; ++shift)
            for (int group = 0; group < 2; ++group) {
                uint8_t sc = b[half * 8 + shift * 2 + group];
                float dl = d * (float)(sc & 15);
                float ml = min * (float)(sc >> 4);
                for (int l = 0; l < 16; ++l) {
                    int q = (b[16 + half * 32 + group * 16 + l] >> (2 * shift)) & 3;
                    out[half * 128 + shift * 32 + group * 16 + l] = dl * (float)q - ml;
                }
            }
}

/* quant.rs:82-101 */
static void decode_q4_k(const uint8_t *b, float *out) {
    const float d = f16_at(b, 0), min = f16_at(b, 2);
    for (int group = 0; group < 8; ++group) {
        uint8_t scale, bias;
        if (group < 4) {
            scale = b[4 + group] & 63;
            bias = b[8 + group] & 63;
        } else {
            scale = (uint8_t)((b[8 + group] & 15) | ((b[group] >> 6) << 4));
            bias = (uint8_t)((b[8 + group] >> 4) | ((b[4 + group] >> 6) << 4));
        }
        float dl = d * (float)scale;
        float ml = min * (float)bias;
        for (int l = 0; l < 32; ++l) {
            int q = (b[16 + (group / 2) * 32 + l] >> (4 * (group % 2))) & 15;
            out[group * 32 + l] = dl * (float)q - ml;
        }
    }
}

/* quant.rs:161-182 */
static void decode_q5_k(const uint8_t *b, float *out) {
    const float d = f16_at(b, 0), min = f16_at(b, 2);
    const uint8_t *scales = b + 4;
    for (int group = 0; group < 8; ++group) {
        uint8_t scale, bias;
        if (group < 4) {
            scale = scales[group] & 63;
            bias = scales[group + 4] & 63;
        } else {
            scale = (uint8_t)((scales[group + 4] & 15) | ((scales[group - 4] >> 6) << 4));
            bias = (uint8_t)((scales[group + 4] >> 4) | ((scales[group] >> 6) << 4));
        }
        float ds = d * (float)scale;
        float ms = min * (float)bias;
        for (int j = 0; j < 32; ++j) {
            int low = (b[48 + (group / 2) * 32 + j] >> (4 * (group % 2))) & 15;
            int high = (b[16 + j] & (1 << group)) ? 16 : 0;
            out[group * 32 + j] = ds * (float)(low + high) - ms;
        }
    }
}

/* quant.rs:35-40 */
static void decode_q8_0(const uint8_t *b, float *out) {
    const float scale = f16_at(b, 0);
    for (int i = 0; i < 32; ++i) out[i] = scale * (float)(int8_t)b[i + 2];
}

int oracle_gguf_decode(int format, const uint8_t *packed, int64_t blocks, float *out) {
    const int bytes = oracle_gguf_block_bytes(format), width = oracle_gguf_block_width(format);
    if (bytes < 0 || blocks <= 0) return -1;
    for (int64_t i = 0; i < blocks; ++i) {
        if (format == ORACLE_GGUF_Q2_K) decode_q2_k(packed + i * bytes, out + i * width);
        else if (format == ORACLE_GGUF_Q4_K) decode_q4_k(packed + i * bytes, out + i * width);
        else if (format == ORACLE_GGUF_Q5_K) decode_q5_k(packed + i * bytes, out + i * width);
        else decode_q8_0(packed + i * bytes, out + i * width);
    }
    return 0;
}

static uint32_t xorshift_byte(uint32_t *state) {
    uint32_t s = *state;
    s ^= s << 13;
    s ^= s >> 17;
    s ^= s << 5;
    *state = s;
    return s >> 24;
}

uint64_t oracle_gguf_reference_hash(int format) {
    const int bytes = oracle_gguf_block_bytes(format);
    if (bytes < 0) return 0;
    uint32_t state = 0x12345678u;
    uint64_t hash = 0xcbf29ce484222325ull;
    const int width = oracle_gguf_block_width(format);
    uint8_t packed[176];
    float decoded[256];
    for (int block = 0; block < 128; ++block) {
        for (int i = 0; i < bytes; ++i) packed[i] = (uint8_t)xorshift_byte(&state);
        uint16_t scale = (uint16_t)(0x2800 + (block % 8) * 0x200);
        if (format == ORACLE_GGUF_Q2_K) {
            packed[80] = (uint8_t)(scale & 0xff);
            packed[81] = (uint8_t)(scale >> 8);
            packed[82] = 0x00;
            packed[83] = 0x24;
        } else {
            packed[0] = (uint8_t)(scale & 0xff);
            packed[1] = (uint8_t)(scale >> 8);
            if (format != ORACLE_GGUF_Q8_0) { /* quant.rs:227-230: the K-quants also get a fixed dmin */
                packed[2] = 0x00;
                packed[3] = 0x24;
            }
        }
        oracle_gguf_decode(format, packed, 1, decoded);
        for (int i = 0; i < width; ++i) {
            uint32_t u = f32_bits(decoded[i]);
            for (int b = 0; b < 4; ++b) {
                hash = (hash ^ (uint64_t)((u >> (8 * b)) & 0xffu)) * 0x100000001b3ull;
            }
        }
    }
    return hash;
}

int oracle_gguf_dyadic_blocks(int format, int64_t count, uint8_t *out) {
    const int bytes = oracle_gguf_block_bytes(format);
    if (bytes < 0) return -1;
    uint32_t state = 0x12345678u;
    for (int64_t blk = 0; blk < count; ++blk) {
        uint8_t *b = out + blk * bytes;
        for (int i = 0; i < bytes; ++i) b[i] = (uint8_t)xorshift_byte(&state);
        if (format == ORACLE_GGUF_Q2_K) {
            b[80] = 0x00; b[81] = 0x18; b[82] = 0x00; b[83] = 0x14;
        } else {
            b[0] = 0x00; b[1] = 0x18; b[2] = 0x00; b[3] = 0x14;
        }
    }
    return 0;
}

void oracle_gguf_dyadic_inputs(int64_t count, float *out) {
    for (int64_t i = 0; i < count; ++i) out[i] = (float)((i * 19 + i / 7) % 3) * 0.125f - 0.125f;
}

typedef struct {
    int format;
    const uint8_t *w;
    int64_t experts, rows, row_bytes, tokens, slots, top_k;
    const float *x;
    const int32_t *ids;
    float *y;
} gguf_ctx;

static float dot_f32(const float *w, const float *x, int64_t k) {
    float acc = 0.0f; /* Iterator::sum over f32: left to right from 0.0 */
    for (int64_t i = 0; i < k; ++i) acc += w[i] * x[i];
    return acc;
}

static void gguf_rows(void *p, int64_t begin, int64_t end) {
    gguf_ctx *c = (gguf_ctx *)p;
    const int bytes = oracle_gguf_block_bytes(c->format);
    const int64_t blocks = c->row_bytes / bytes, k = blocks * oracle_gguf_block_width(c->format);
    float *wrow = (float *)malloc(sizeof(float) * (size_t)k);
    for (int64_t r = begin; r < end; ++r) {
        oracle_gguf_decode(c->format, c->w + r * c->row_bytes, blocks, wrow);
        for (int64_t t = 0; t < c->tokens; ++t) c->y[t * c->rows + r] = dot_f32(wrow, c->x + t * k, k);
    }
    free(wrow);
}

int oracle_gguf_matvec(int format, const uint8_t *w, int64_t rows, int64_t row_bytes,
                       const float *x, int64_t tokens, int threads, float *y) {
    const int bytes = oracle_gguf_block_bytes(format);
    if (bytes < 0 || row_bytes <= 0 || row_bytes % bytes != 0 || rows <= 0 || tokens <= 0) return -1;
    gguf_ctx c = {format, w, 1, rows, row_bytes, tokens, 1, 1, x, NULL, y};
    parallel_rows(rows, threads, gguf_rows, &c);
    return 0;
}

static void gguf_expert_slots(void *p, int64_t begin, int64_t end) {
    gguf_ctx *c = (gguf_ctx *)p;
    const int bytes = oracle_gguf_block_bytes(c->format);
    const int64_t blocks = c->row_bytes / bytes, k = blocks * oracle_gguf_block_width(c->format);
    float *wrow = (float *)malloc(sizeof(float) * (size_t)k);
    for (int64_t z = begin; z < end; ++z) { /* z = token * top_k + slot */
        const int64_t token = z / c->top_k, slot = z % c->top_k;
        const int32_t e = c->ids[z];
        const float *xr = c->x + (token * c->slots + slot % c->slots) * k;
        for (int64_t r = 0; r < c->rows; ++r) {
            if (e < 0 || e >= c->experts) {
                c->y[z * c->rows + r] = 0.0f;
                continue;
            }
            oracle_gguf_decode(c->format, c->w + ((int64_t)e * c->rows + r) * c->row_bytes, blocks,
                               wrow);
            c->y[z * c->rows + r] = dot_f32(wrow, xr, k);
        }
    }
    free(wrow);
}

int oracle_gguf_expert_matvec(int format, const uint8_t *w, int64_t experts, int64_t rows,
                              int64_t row_bytes, const float *x, int64_t tokens, int64_t slots,
                              const int32_t *ids, int64_t top_k, int threads, float *y) {
    const int bytes = oracle_gguf_block_bytes(format);
    if (bytes < 0 || row_bytes <= 0 || row_bytes % bytes != 0) return -1;
    if (slots != 1 && slots != top_k) return -1;
    gguf_ctx c = {format, w, experts, rows, row_bytes, tokens, slots, top_k, x, ids, y};
    parallel_rows(tokens * top_k, threads, gguf_expert_slots, &c);
    return 0;
}

/* ------------------------------------------------------------------ */
/* MoE routing                                                         */
/* ------------------------------------------------------------------ */

int oracle_moe_route(const float *logits, int64_t tokens, int64_t experts, int top_k,
                     int32_t *idx, float *weights) {
    if (top_k < 1 || top_k > experts || top_k > 64) return -1;
    uint8_t *taken = (uint8_t *)malloc((size_t)experts);
    for (int64_t t = 0; t < tokens; ++t) {
        const float *l = logits + t * experts;
        memset(taken, 0, (size_t)experts);
        float sel[64];
        for (int j = 0; j < top_k; ++j) {
            int64_t best = -1;
            for (int64_t e = 0; e < experts; ++e)
                if (!taken[e] && (best < 0 || l[e] > l[best])) best = e; /* ties: lowest index */
            taken[best] = 1;
            idx[t * top_k + j] = (int32_t)best;
            sel[j] = l[best];
        }
        float mx = sel[0], sum = 0.0f;
        for (int j = 1; j < top_k; ++j) mx = fmaxf(mx, sel[j]);
        for (int j = 0; j < top_k; ++j) {
            sel[j] = expf(sel[j] - mx);
            sum += sel[j];
        }
        for (int j = 0; j < top_k; ++j) weights[t * top_k + j] = sel[j] / sum;
    }
    free(taken);
    return 0;
}

int oracle_moe_sort(const int32_t *idx, int64_t slots, int64_t experts, int top_k,
                    int32_t *sorted_ids, int32_t *token_rows, int32_t *inverse) {
    int64_t *start = (int64_t *)calloc((size_t)experts + 1, sizeof(int64_t));
    for (int64_t i = 0; i < slots; ++i) {
        if (idx[i] < 0 || idx[i] >= experts) {
            free(start);
            return -1;
        }
        start[idx[i] + 1]++;
    }
    for (int64_t e = 0; e < experts; ++e) start[e + 1] += start[e];
    for (int64_t i = 0; i < slots; ++i) {
        int64_t pos = start[idx[i]]++;
        sorted_ids[pos] = idx[i];
        token_rows[pos] = (int32_t)(i / top_k);
        inverse[i] = (int32_t)pos;
    }
    free(start);
    return 0;
}

int64_t oracle_moe_tile_table(const int32_t *sorted_ids, int64_t rows, int64_t experts,
                              int tile_rows, int32_t *tiles, int64_t capacity) {
    (void)experts;
    memset(tiles, 0, sizeof(int32_t) * 2 * (size_t)capacity);
    int64_t count = 0, s = 0;
    while (s < rows) {
        int64_t e = s + 1;
        while (e < rows && sorted_ids[e] == sorted_ids[s]) e++;
        for (int64_t b = s; b < e; b += tile_rows) {
            if (count >= capacity) return -1;
            tiles[2 * count] = (int32_t)b;
            tiles[2 * count + 1] = (int32_t)((b + tile_rows < e) ? b + tile_rows : e);
            count++;
        }
        s = e;
    }
    return count;
}

static float round_bf16(float v) { return oracle_bf16_to_f32(oracle_f32_to_bf16(v)); }

void oracle_swiglu_bf16(const uint16_t *gate, const uint16_t *up, int64_t count, uint16_t *act) {
    for (int64_t i = 0; i < count; ++i) {
        float g = oracle_bf16_to_f32(gate[i]), u = oracle_bf16_to_f32(up[i]);
        float y = 1.0f / (1.0f + expf(fabsf(g)));
        float s = round_bf16((g < 0.0f) ? y : 1.0f - y);
        float silu = round_bf16(g * s);
        act[i] = oracle_f32_to_bf16(silu * u);
    }
}

int oracle_moe_combine(const uint16_t *down_sorted, const float *weights, const int32_t *inverse,
                       int64_t tokens, int top_k, int64_t hidden, uint16_t *out) {
    if (top_k < 1 || top_k > 64) return -1;
    const int ty = top_k < 8 ? top_k : 8;
    for (int64_t t = 0; t < tokens; ++t)
        for (int64_t h = 0; h < hidden; ++h) {
            float r[64], part[8];
            for (int j = 0; j < top_k; ++j) {
                int64_t row = inverse[t * top_k + j];
                /* a slot that was not sorted (inverse < 0: an expert outside the table or not owned by this
                   rank, the zero rule of deepseek41.rs:204-206 and iq.metal:976-982) adds nothing */
                r[j] = row < 0 ? 0.0f : oracle_bf16_to_f32(down_sorted[row * hidden + h]) * weights[t * top_k + j];
            }
            for (int y = 0; y < ty; ++y) {
                float acc = 0.0f;
                for (int rr = y; rr < top_k; rr += ty) acc = r[rr] + acc;
                part[y] = acc;
            }
            float total = part[0];
            for (int j = 1; j < ty; ++j) total = part[j] + total;
            out[t * hidden + h] = oracle_f32_to_bf16(total);
        }
    return 0;
}
