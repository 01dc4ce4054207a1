// Residual add + RMSNorm as a kernel of its own: sum = bf16(x + r), normed = bf16(w * bf16(f32(sum) * inv)),
// inv = 1 / sqrt(mean(sum^2) + eps) in f32 -- the rounding points of the reference's fused add + rms_norm chain
// (crates/lisa-mlx/src/jit/matmul.rs:304-316 and the shader it names: s, the product with inv, and the product with
// the weight are each rounded to bf16).  The matmul kernels fuse the same arithmetic into their activation
// staging where they can (qmv_tc.cu, NORM form); this kernel serves every other shape.
#include <cuda_runtime.h>

#include "common.cuh"
#include "kernels.h"

namespace lisa {

namespace {

__device__ __forceinline__ float nr_round_bf16(float v) { return bf16_bits_to_f32(f32_to_bf16_bits(v)); }

// one block per row; k a multiple of 8, 16-byte aligned rows
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(const uint4 *__restrict__ x, const uint4 *__restrict__ r,
                                                          const uint4 *__restrict__ w, float eps, int k8, uint4 *__restrict__ sum,
                                                          uint4 *__restrict__ normed) {
    __shared__ float red[8];
    __shared__ float inv_s;
    const int64_t row = blockIdx.x;
    const uint4 *xr = x + row * k8, *rr = r + row * k8;
    uint4 *sr = sum + row * k8;
    float acc = 0.f;
    for (int i = threadIdx.x; i < k8; i += 256) {
        const uint4 a = __ldg(xr + i), b = __ldg(rr + i);
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
        uint32_t sw[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float s0 = nr_round_bf16(bf16_bits_to_f32(aw[q] & 0xffffu) + bf16_bits_to_f32(bw[q] & 0xffffu));
            const float s1 = nr_round_bf16(__uint_as_float(aw[q] & 0xffff0000u) + __uint_as_float(bw[q] & 0xffff0000u));
            acc = fmaf(s0, s0, acc);
            acc = fmaf(s1, s1, acc);
            sw[q] = (__float_as_uint(s0) >> 16) | (__float_as_uint(s1) & 0xffff0000u);
        }
        sr[i] = make_uint4(sw[0], sw[1], sw[2], sw[3]);
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float tot = 0.f;
        for (int i = 0; i < 8; ++i) tot += red[i];
        inv_s = 1.0f / sqrtf(tot / static_cast<float>(k8 * 8) + eps);
    }
    __syncthreads();
    const float inv = inv_s;
    uint4 *nr = normed + row * k8;
    for (int i = threadIdx.x; i < k8; i += 256) {
        const uint4 s = sr[i], wv = __ldg(w + i);  // this thread's own stores
        const uint32_t sw[4] = {s.x, s.y, s.z, s.w}, ww[4] = {wv.x, wv.y, wv.z, wv.w};
        uint32_t nd[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float y0 = bf16_bits_to_f32(ww[q] & 0xffffu) * nr_round_bf16(bf16_bits_to_f32(sw[q] & 0xffffu) * inv);
            const float y1 = __uint_as_float(ww[q] & 0xffff0000u) * nr_round_bf16(__uint_as_float(sw[q] & 0xffff0000u) * inv);
            nd[q] = f32_to_bf16_bits(y0) | (f32_to_bf16_bits(y1) << 16);
        }
        nr[i] = make_uint4(nd[0], nd[1], nd[2], nd[3]);
    }
}

}  // namespace

int add_rmsnorm(cudaStream_t stream, const void *x, const void *residual, const void *weight, float eps, int64_t m, int64_t k,
                void *sum, void *normed) {
    add_rmsnorm_kernel<<<static_cast<unsigned>(m), 256, 0, stream>>>(
        reinterpret_cast<const uint4 *>(x), reinterpret_cast<const uint4 *>(residual), reinterpret_cast<const uint4 *>(weight), eps,
        static_cast<int>(k / 8), reinterpret_cast<uint4 *>(sum), reinterpret_cast<uint4 *>(normed));
    LISA_CUDA_TRY(cudaGetLastError());
    count_launch();
    return LISA_OK;
}

}  // namespace lisa
