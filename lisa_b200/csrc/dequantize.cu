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

}  // namespace lisa
