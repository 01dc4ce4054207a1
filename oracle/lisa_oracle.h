/*
 * CPU oracle for the quantized-weight matmul path of agnosticeng/lisa.
 *
 * TEST INFRASTRUCTURE ONLY.  This is a plain-C restatement of the reference's
 * own arithmetic (Rust host code and the laws its Metal kernels implement).
 * It exists to check the CUDA library and to be timed as the CPU baseline.
 * Nothing in the shipped library links, loads or calls it.
 *
 * Parity is pinned: the GGUF decoders reproduce the reference's frozen
 * FNV-1a-64 hashes (crates/lisa-gguf/src/quant.rs:186-242) and the dyadic
 * exact-dot construction (crates/lisa-engine/src/models/deepseek41/
 * kernel_tests.rs:133-263); the affine law is the reference's host loop
 * (crates/lisa-mlx/src/ops/array_ops.rs:56-83), which has no frozen vectors of
 * its own, only relations between kernels, replayed in tests/.
 */
#ifndef LISA_ORACLE_H
#define LISA_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* GGML tensor type ids (crates/lisa-gguf/src/lib.rs:24-32). */
#define ORACLE_GGUF_Q8_0 8
#define ORACLE_GGUF_Q2_K 10
#define ORACLE_GGUF_Q4_K 12
#define ORACLE_GGUF_Q5_K 13

/* ---- scalar conversions (half 2.7.1 semantics: round-to-nearest-even) ---- */
uint16_t oracle_f32_to_bf16(float v);
float oracle_bf16_to_f32(uint16_t v);
float oracle_f16_to_f32(uint16_t v);
uint16_t oracle_f32_to_f16(float v);

/* ---- affine (MLX) ---- */
/* ops::dequantize host loop, crates/lisa-mlx/src/ops/array_ops.rs:56-83:
 * out[r][c] = (f32)q * (f32)scale + (f32)bias, q = (word >> ((c % pf) * bits)) & mask. */
int oracle_affine_dequantize_f32(const uint32_t *w, const uint16_t *scales, const uint16_t *biases,
                                 int64_t rows, int64_t k, int group_size, int bits, float *out);
/* Same, then cast once to the scales dtype (bf16), array_ops.rs:83. */
int oracle_affine_dequantize_bf16(const uint32_t *w, const uint16_t *scales, const uint16_t *biases,
                                  int64_t rows, int64_t k, int group_size, int bits, uint16_t *out);

/* "Rust dequant + scalar f32 matmul": dequantize a row (optionally rounding the
 * weight to bf16 as ops::dequantize returns it), then acc += x[k]*w[k]
 * sequentially over k (crates/lisa-engine/src/models/laya/cpu.rs:42-60), output
 * rounded to bf16.  Output rows are split over `threads` host threads
 * (the reference uses rayon over rows).  x bf16 [m,k], y bf16 [m,n]. */
int oracle_affine_matmul(const uint16_t *x, int64_t m, int64_t k, const uint32_t *w,
                         const uint16_t *scales, const uint16_t *biases, int64_t n, int group_size,
                         int bits, int round_weight_bf16, int threads, uint16_t *y);
/* Same contraction accumulated in double, not rounded on output. */
int oracle_affine_matmul_f64(const uint16_t *x, int64_t m, int64_t k, const uint32_t *w,
                             const uint16_t *scales, const uint16_t *biases, int64_t n,
                             int group_size, int bits, int round_weight_bf16, int threads,
                             double *y);
/* The qmv kernels' factorisation, quantized.metal:196-295: per group
 * scale * sum(q*x) + bias * sum(x), f32, groups in order; bf16 output. */
int oracle_affine_qmv_factored(const uint16_t *x, int64_t m, int64_t k, const uint32_t *w,
                               const uint16_t *scales, const uint16_t *biases, int64_t n,
                               int group_size, int bits, uint16_t *y);
/* ops::quantize, array_ops.rs:218-290.  w f32 [rows,k] -> packed words and f32
 * scale/bias per group (the caller rounds them to the weight dtype). */
int oracle_affine_quantize(const float *w, int64_t rows, int64_t k, int group_size, int bits,
                           uint32_t *wq, float *scales, float *biases);
/* The reference tests' LCG, array_ops.rs:659-662: returns v in [-1,1). */
void oracle_lcg_fill(uint64_t *seed, float *out, int64_t count);

/* ops::gather_qmm with sorted rhs indices, array_ops.rs:561-642: row r of
 * x [rows,k] uses expert ids[r]; w [experts,n,k*bits/32]. */
int oracle_gather_qmm(const uint16_t *x, int64_t rows, int64_t k, const uint32_t *w,
                      const uint16_t *scales, const uint16_t *biases, const int32_t *ids,
                      int64_t experts, int64_t n, int group_size, int bits,
                      int round_weight_bf16, int threads, uint16_t *y);

/* ---- GGUF K-quants ---- */
int oracle_gguf_block_bytes(int format);
int oracle_gguf_block_width(int format);
/* lisa_gguf::quant::decode, crates/lisa-gguf/src/quant.rs:21-101. */
int oracle_gguf_decode(int format, const uint8_t *packed, int64_t blocks, float *out);
/* The frozen-hash test, quant.rs:186-242: returns FNV-1a-64 over 128 blocks. */
uint64_t oracle_gguf_reference_hash(int format);
/* Block generator of the dyadic tests, kernel_tests.rs:133-162. */
int oracle_gguf_dyadic_blocks(int format, int64_t count, uint8_t *out);
/* Dyadic inputs, kernel_tests.rs:172-176. */
void oracle_gguf_dyadic_inputs(int64_t count, float *out);
/* packed_matvec semantics, crates/lisa-mlx/src/models/deepseek41.rs:93-174, as
 * the CPU check computes it (kernel_tests.rs:196-201): y[t][r] = sum_k w*x, f32. */
int oracle_gguf_matvec(int format, const uint8_t *w, int64_t rows, int64_t row_bytes,
                       const float *x, int64_t tokens, int threads, float *y);
/* expert_matvec semantics, deepseek41.rs:204-283 / kernel_tests.rs:212-263. */
int oracle_gguf_expert_matvec(int format, const uint8_t *w, int64_t experts, int64_t rows,
                              int64_t row_bytes, const float *x, int64_t tokens, int64_t slots,
                              const int32_t *ids, int64_t top_k, int threads, float *y);

/* ---- MoE routing around gather_qmm (crates/lisa-engine/src/models/qwen4/moe.rs) ---- */
/* top-k by value, ties to the lowest expert index, descending-logit order;
 * weights = softmax over the k selected logits (moe.rs:143-146,356-359). */
int oracle_moe_route(const float *logits, int64_t tokens, int64_t experts, int top_k,
                     int32_t *idx, float *weights);
/* Stable sort of slots by expert (moe.rs:368-374): sorted_ids[i] = idx[order[i]],
 * token_rows[i] = order[i] / top_k, inverse[order[i]] = i. */
int oracle_moe_sort(const int32_t *idx, int64_t slots, int64_t experts, int top_k,
                    int32_t *sorted_ids, int32_t *token_rows, int32_t *inverse);
/* Tile table (crates/lisa-mlx/src/models/qwen4/prefill_indirect.rs:16-18,103-133):
 * tiles restart at every expert run; returns the number of tiles used;
 * capacity must be ceil(rows/tile_rows)+experts pairs, unused pairs (0,0). */
int64_t oracle_moe_tile_table(const int32_t *sorted_ids, int64_t rows, int64_t experts,
                              int tile_rows, int32_t *tiles, int64_t capacity);
/* act = bf16(bf16(g*sigmoid(g)) * u), rounding points of exact_header.metal:2-11. */
void oracle_swiglu_bf16(const uint16_t *gate, const uint16_t *up, int64_t count, uint16_t *act);
/* Weighted un-sort and fold, moe.rs:450-481: out[t][h] = bf16(sum_k f32(down[inverse[t*k+j]][h]) * w[t][j]),
 * slots folded left to right in original slot order (mlx_colsum_small_f32). */
int oracle_moe_combine(const uint16_t *down_sorted, const float *weights, const int32_t *inverse,
                       int64_t tokens, int top_k, int64_t hidden, uint16_t *out);

#ifdef __cplusplus
}
#endif
#endif
