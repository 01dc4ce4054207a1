// f16 and f32 compute dtypes of quantized_matmul and dequantize (ops::quantized_matmul promotes x with the scales'
// dtype and casts x, scales and biases to it, crates/lisa-mlx/src/ops/array_ops.rs:398-404; dequantize returns the
// scales' dtype, array_ops.rs:37-84).  The checkpoints on this path are bf16 and the fast kernels are written for
// it; these two generic kernels make the other two dtypes work -- same laws (qmv factorisation in f32, one
// rounding of q * s + b), one warp per output row and one thread per packed word, no tensor cores.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>

#include "common.cuh"
#include "kernels.h"

namespace lisa {

namespace {

template <typename T>
__device__ __forceinline__ float ty_load(const T *p);
template <>
__device__ __forceinline__ float ty_load<__half>(const __half *p) { return __half2float(__ldg(p)); }
template <>
__device__ __forceinline__ float ty_load<float>(const float *p) { return __ldg(p); }
template <typename T>
__device__ __forceinline__ T ty_store(float v);
template <>
__device__ __forceinline__ __half ty_store<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ float ty_store<float>(float v) { return v; }

// grid (ceil(n / 8), rows of x): warp = output row of the weights
template <typename T, int BITS>
__global__ void __launch_bounds__(256) qmv_typed_kernel(const uint32_t *__restrict__ w, const T *__restrict__ scales,
                                                        const T *__restrict__ biases, const T *__restrict__ x, T *__restrict__ y,
                                                        int n, int k, int group_size) {
    constexpr int CPW = 32 / BITS;
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int64_t mrow = blockIdx.y;
    if (row >= n) return;
    const int nwords = k / CPW, groups = k / group_size;
    const uint32_t *wr = w + static_cast<int64_t>(row) * nwords;
    const T *sr = scales + static_cast<int64_t>(row) * groups, *br = biases + static_cast<int64_t>(row) * groups;
    const T *xr = x + mrow * k;
    float result = 0.f;
    for (int wi = lane; wi < nwords; wi += 32) {
        const uint32_t word = __ldg(wr + wi);
        const int k0 = wi * CPW, gi = k0 / group_size;
        float accum = 0.f, xsum = 0.f;
#pragma unroll
        for (int j = 0; j < CPW; ++j) {
            const float xv = ty_load<T>(xr + k0 + j);
            accum = fmaf(xv, static_cast<float>((word >> (j * BITS)) & ((1u << BITS) - 1u)), accum);
            xsum += xv;
        }
        result = fmaf(ty_load<T>(sr + gi), accum, result);
        result = fmaf(ty_load<T>(br + gi), xsum, result);
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) result += __shfl_xor_sync(0xffffffffu, result, off);
    if (lane == 0) y[mrow * n + row] = ty_store<T>(result);
}

// one thread per packed word: out = T(f32(q) * f32(s) + f32(b)), product and sum each rounded once
template <typename T, int BITS>
__global__ void __launch_bounds__(256) dequantize_typed_kernel(const uint32_t *__restrict__ w, const T *__restrict__ scales,
                                                               const T *__restrict__ biases, int64_t total_words, int words_per_row,
                                                               int group_size, int groups, T *__restrict__ out) {
    constexpr int CPW = 32 / BITS;
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total_words) return;
    const int64_t row = idx / words_per_row;
    const int wi = static_cast<int>(idx - row * words_per_row);
    const int g = (wi * CPW) / group_size;
    const float sc = ty_load<T>(scales + row * groups + g), bi = ty_load<T>(biases + row * groups + g);
    const uint32_t word = __ldg(w + idx);
#pragma unroll
    for (int j = 0; j < CPW; ++j)
        out[idx * CPW + j] = ty_store<T>(__fadd_rn(__fmul_rn(static_cast<float>((word >> (j * BITS)) & ((1u << BITS) - 1u)), sc), bi));
}

template <typename T>
int qmv_typed_launch(cudaStream_t stream, const void *x, int64_t m, int64_t k, const uint32_t *w, const void *scales,
                     const void *biases, int64_t n, int group_size, int bits, void *y) {
    const T *s = reinterpret_cast<const T *>(scales), *b = reinterpret_cast<const T *>(biases);
    for (int64_t done = 0; done < m; done += 65535) {
        const unsigned rows = static_cast<unsigned>(std::min<int64_t>(m - done, 65535));
        const dim3 grid(static_cast<unsigned>((n + 7) / 8), rows);
        const T *xp = reinterpret_cast<const T *>(x) + done * k;
        T *yp = reinterpret_cast<T *>(y) + done * n;
        const int ni = static_cast<int>(n), ki = static_cast<int>(k);
        if (bits == 2) qmv_typed_kernel<T, 2><<<grid, 256, 0, stream>>>(w, s, b, xp, yp, ni, ki, group_size);
        else if (bits == 4) qmv_typed_kernel<T, 4><<<grid, 256, 0, stream>>>(w, s, b, xp, yp, ni, ki, group_size);
        else qmv_typed_kernel<T, 8><<<grid, 256, 0, stream>>>(w, s, b, xp, yp, ni, ki, group_size);
        LISA_CUDA_TRY(cudaGetLastError());
        count_launch();
    }
    return LISA_OK;
}

template <typename T>
int dequantize_typed_launch(cudaStream_t stream, const uint32_t *w, const void *scales, const void *biases, int64_t rows, int64_t k,
                            int group_size, int bits, void *out) {
    const int words_per_row = static_cast<int>(k * bits / 32), groups = static_cast<int>(k / group_size);
    const int64_t total = rows * words_per_row;
    const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
    const T *s = reinterpret_cast<const T *>(scales), *b = reinterpret_cast<const T *>(biases);
    T *o = reinterpret_cast<T *>(out);
    if (bits == 2) dequantize_typed_kernel<T, 2><<<blocks, 256, 0, stream>>>(w, s, b, total, words_per_row, group_size, groups, o);
    else if (bits == 4) dequantize_typed_kernel<T, 4><<<blocks, 256, 0, stream>>>(w, s, b, total, words_per_row, group_size, groups, o);
    else dequantize_typed_kernel<T, 8><<<blocks, 256, 0, stream>>>(w, s, b, total, words_per_row, group_size, groups, o);
    LISA_CUDA_TRY(cudaGetLastError());
    count_launch();
    return LISA_OK;
}

}  // namespace

int qmv_typed(cudaStream_t stream, int dtype, const void *x, int64_t m, int64_t k, const uint32_t *w, const void *scales,
              const void *biases, int64_t n, int group_size, int bits, void *y) {
    if (dtype == LISA_F16) return qmv_typed_launch<__half>(stream, x, m, k, w, scales, biases, n, group_size, bits, y);
    if (dtype == LISA_F32) return qmv_typed_launch<float>(stream, x, m, k, w, scales, biases, n, group_size, bits, y);
    return fail(LISA_ERR_UNSUPPORTED, "qmv_typed: f16 or f32");
}

int dequantize_typed(cudaStream_t stream, int dtype, const uint32_t *w, const void *scales, const void *biases, int64_t rows,
                     int64_t k, int group_size, int bits, void *out) {
    if (dtype == LISA_F16) return dequantize_typed_launch<__half>(stream, w, scales, biases, rows, k, group_size, bits, out);
    if (dtype == LISA_F32) return dequantize_typed_launch<float>(stream, w, scales, biases, rows, k, group_size, bits, out);
    return fail(LISA_ERR_UNSUPPORTED, "dequantize_typed: f16 or f32");
}

}  // namespace lisa
