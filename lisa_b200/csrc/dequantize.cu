// Standalone affine unpack: out[r, c] = bf16( f32(q) * f32(scale) + f32(bias) ).
//
// Replaces ops::dequantize / jit::affine_dequantize
// (crates/lisa-mlx/src/ops/array_ops.rs:37-84, crates/lisa-mlx/src/jit/matmul.rs:1316-1402).
// The arithmetic is the host law of array_ops.rs:69-83 (f32 multiply, f32 add, one cast),
// which is also what the GEMM tile loaders of the reference compute
// (crates/lisa-mlx/src/shaders/common/matmul/quantized.metal:490-533); the Metal
// affine_dequantize kernel evaluates scale*q+bias in bf16 arithmetic instead
// (quantized.metal:2791) and can differ from it in the last bf16 bit.
#include <cuda_runtime.h>
#include <limits.h>

#include "common.cuh"
#include "kernels.h"

namespace lisa {

// One thread per packed word; a word never straddles a group (group_size >= 32 >= codes per word).
template <int BITS>
__global__ void __launch_bounds__(256) dequantize_kernel(const uint32_t *__restrict__ w,
                                                         const uint16_t *__restrict__ scales,
                                                         const uint16_t *__restrict__ biases, int64_t total_words,
                                                         int words_per_row, int group_size, int groups,
                                                         uint16_t *__restrict__ out) {
    constexpr int CPW = 32 / BITS;
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total_words) return;
    const int64_t row = idx / words_per_row;
    const int wi = static_cast<int>(idx - row * words_per_row);
    const int g = (wi * CPW) / group_size;
    const float sc = bf16_bits_to_f32(__ldg(scales + row * groups + g));
    const float bi = bf16_bits_to_f32(__ldg(biases + row * groups + g));
    const uint32_t word = __ldg(w + idx);
    uint32_t packed[CPW / 2];
#pragma unroll
    for (int j = 0; j < CPW / 2; ++j) {
        const uint32_t q0 = (word >> ((2 * j) * BITS)) & ((1u << BITS) - 1u);
        const uint32_t q1 = (word >> ((2 * j + 1) * BITS)) & ((1u << BITS) - 1u);
        const float v0 = __fadd_rn(__fmul_rn(static_cast<float>(q0), sc), bi);
        const float v1 = __fadd_rn(__fmul_rn(static_cast<float>(q1), sc), bi);
        packed[j] = f32x2_to_bf16x2(v0, v1);
    }
    uint16_t *dst = out + idx * CPW;  // CPW * 2 bytes: 8 (8-bit), 16 (4-bit), 32 (2-bit), aligned likewise
    if constexpr (CPW == 4) {
        *reinterpret_cast<uint2 *>(dst) = make_uint2(packed[0], packed[1]);
    } else {
#pragma unroll
        for (int j = 0; j < CPW / 8; ++j)
            reinterpret_cast<uint4 *>(dst)[j] =
                make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
    }
}

int dequantize_affine(cudaStream_t stream, const uint32_t *w, const void *scales, const void *biases, int64_t rows,
                      int64_t k, int group_size, int bits, void *out) {
    const int words_per_row = static_cast<int>(k * bits / 32);
    const int64_t total = rows * words_per_row;
    const int groups = static_cast<int>(k / group_size);
    const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
    const uint16_t *s = reinterpret_cast<const uint16_t *>(scales);
    const uint16_t *b = reinterpret_cast<const uint16_t *>(biases);
    uint16_t *o = reinterpret_cast<uint16_t *>(out);
    if (bits == 4) dequantize_kernel<4><<<blocks, 256, 0, stream>>>(w, s, b, total, words_per_row, group_size, groups, o);
    else if (bits == 2) dequantize_kernel<2><<<blocks, 256, 0, stream>>>(w, s, b, total, words_per_row, group_size, groups, o);
    else dequantize_kernel<8><<<blocks, 256, 0, stream>>>(w, s, b, total, words_per_row, group_size, groups, o);
    LISA_CUDA_TRY(cudaGetLastError());
    count_launch();
    return LISA_OK;
}

// ---------------------------------------------------------------------------------------
// Row-indexed form for QuantizedEmbedding::forward (crates/lisa-engine/src/core/quant.rs:449-455: take_axis
// of weight, scales and biases by the token ids, then dequantize): out[i, :] = dequantize(row ids[i]).  An id
// outside [0, vocab) writes a row of zeros and reads nothing.
template <int BITS>
__global__ void __launch_bounds__(256) dequantize_rows_kernel(const uint32_t *__restrict__ w, const uint16_t *__restrict__ scales,
                                                              const uint16_t *__restrict__ biases, const int32_t *__restrict__ ids,
                                                              int64_t total_words, int64_t vocab, int words_per_row,
                                                              int group_size, int groups, uint16_t *__restrict__ out) {
    constexpr int CPW = 32 / BITS;
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total_words) return;
    const int64_t i = idx / words_per_row;
    const int wi = static_cast<int>(idx - i * words_per_row);
    const int64_t row = __ldg(ids + i);
    uint16_t *dst = out + idx * CPW;
    if (row < 0 || row >= vocab) {
#pragma unroll
        for (int j = 0; j < CPW; ++j) dst[j] = 0;
        return;
    }
    const int g = (wi * CPW) / group_size;
    const float sc = bf16_bits_to_f32(__ldg(scales + row * groups + g));
    const float bi = bf16_bits_to_f32(__ldg(biases + row * groups + g));
    const uint32_t word = __ldg(w + row * words_per_row + wi);
#pragma unroll
    for (int j = 0; j < CPW; ++j) {
        const uint32_t q = (word >> (j * BITS)) & ((1u << BITS) - 1u);
        dst[j] = static_cast<uint16_t>(f32_to_bf16_bits(__fadd_rn(__fmul_rn(static_cast<float>(q), sc), bi)));
    }
}

int dequantize_affine_rows(cudaStream_t stream, const uint32_t *w, const void *scales, const void *biases, const int32_t *ids,
                           int64_t count, int64_t vocab, int64_t k, int group_size, int bits, void *out) {
    const int words_per_row = static_cast<int>(k * bits / 32);
    const int64_t total = count * words_per_row;
    const int groups = static_cast<int>(k / group_size);
    const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
    const uint16_t *s = reinterpret_cast<const uint16_t *>(scales);
    const uint16_t *b = reinterpret_cast<const uint16_t *>(biases);
    uint16_t *o = reinterpret_cast<uint16_t *>(out);
    if (bits == 4) dequantize_rows_kernel<4><<<blocks, 256, 0, stream>>>(w, s, b, ids, total, vocab, words_per_row, group_size, groups, o);
    else if (bits == 2) dequantize_rows_kernel<2><<<blocks, 256, 0, stream>>>(w, s, b, ids, total, vocab, words_per_row, group_size, groups, o);
    else dequantize_rows_kernel<8><<<blocks, 256, 0, stream>>>(w, s, b, ids, total, vocab, words_per_row, group_size, groups, o);
    LISA_CUDA_TRY(cudaGetLastError());
    count_launch();
    return LISA_OK;
}

// ---------------------------------------------------------------------------------------
// ops::quantize (crates/lisa-mlx/src/ops/array_ops.rs:218-290), the MLX affine quantiser the reference runs on
// the host: per group a signed scale and the outer edge as bias, computed in f32 and cast to the input type at
// the end; codes from the f32 scale.  One thread per (row, group), the reference's operations in its order
// (IEEE division, round half away from zero), so that the packed words and the scales come out bit for bit.
template <int BITS>
__global__ void __launch_bounds__(128) quantize_kernel(const uint16_t *__restrict__ w, int64_t cells, int groups, int group_size,
                                                       uint32_t *__restrict__ wq, uint16_t *__restrict__ scales,
                                                       uint16_t *__restrict__ biases) {
    constexpr int CPW = 32 / BITS;
    const int64_t cell = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;  // row * groups + group
    if (cell >= cells) return;
    const uint16_t *src = w + cell * group_size;
    const float maxq = static_cast<float>((1u << BITS) - 1u);
    float w_min = 3.40282347e+38f, w_max = 0.0f;  // f32::MAX, 0 (array_ops.rs:246-247)
    for (int i = 0; i < group_size; ++i) {
        const float v = bf16_bits_to_f32(__ldg(src + i));
        w_min = fminf(w_min, v);
        w_max = fmaxf(w_max, v);
    }
    float scale = fmaxf(__fdiv_rn(__fsub_rn(w_max, w_min), maxq), 1e-7f);
    const bool side = fabsf(w_min) > fabsf(w_max);
    if (!side) scale = -scale;
    const float edge = side ? w_min : w_max;
    const float q0 = roundf(__fdiv_rn(edge, scale));
    const bool at_zero = q0 == 0.0f;
    if (!at_zero) scale = __fdiv_rn(edge, q0);
    const float bias = at_zero ? 0.0f : edge;
    scales[cell] = static_cast<uint16_t>(f32_to_bf16_bits(scale));
    biases[cell] = static_cast<uint16_t>(f32_to_bf16_bits(bias));
    uint32_t *dst = wq + cell * (group_size / CPW);
    for (int wi = 0; wi < group_size / CPW; ++wi) {
        uint32_t word = 0;
#pragma unroll
        for (int j = 0; j < CPW; ++j) {
            const float v = bf16_bits_to_f32(__ldg(src + wi * CPW + j));
            const float qf = fminf(roundf(__fdiv_rn(__fsub_rn(v, bias), scale)), maxq);
            int q = (qf != qf) ? 0 : (qf <= -2147483648.0f ? INT_MIN : static_cast<int>(qf));  // `as i32`: saturating, NaN -> 0
            word |= (static_cast<uint32_t>(q) & ((1u << BITS) - 1u)) << (j * BITS);
        }
        dst[wi] = word;
    }
}

int quantize_affine(cudaStream_t stream, const void *w, int64_t rows, int64_t k, int group_size, int bits, uint32_t *wq,
                    void *scales, void *biases) {
    const int groups = static_cast<int>(k / group_size);
    const int64_t cells = rows * groups;
    const unsigned blocks = static_cast<unsigned>((cells + 127) / 128);
    const uint16_t *src = reinterpret_cast<const uint16_t *>(w);
    uint16_t *s = reinterpret_cast<uint16_t *>(scales), *b = reinterpret_cast<uint16_t *>(biases);
    if (bits == 4) quantize_kernel<4><<<blocks, 128, 0, stream>>>(src, cells, groups, group_size, wq, s, b);
    else if (bits == 2) quantize_kernel<2><<<blocks, 128, 0, stream>>>(src, cells, groups, group_size, wq, s, b);
    else quantize_kernel<8><<<blocks, 128, 0, stream>>>(src, cells, groups, group_size, wq, s, b);
    LISA_CUDA_TRY(cudaGetLastError());
    count_launch();
    return LISA_OK;
}

}  // namespace lisa
