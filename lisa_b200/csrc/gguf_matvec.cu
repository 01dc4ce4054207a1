// GGUF K-quant matvec, f32 in / f32 out: y[t, r] = sum_k decode(W[r])[k] * x[t, k].
//
// Replaces lisa_gguf_q2_K_mv / lisa_gguf_q4_K_mv and their expert-indexed forms
// (crates/lisa-mlx/src/shaders/deepseek41/iq.metal:1012-1090,1130-1363; host side
// crates/lisa-mlx/src/models/deepseek41.rs:93-283).  Block layouts follow
// crates/lisa-gguf/src/quant.rs:64-101.  Like the reference kernels, a sub-block contributes
//   d * sc * sum(q * x) - dmin * m * sum(x)
// in f32; on inputs whose products and sums are exactly representable the result equals the
// sequential CPU dot product bit for bit (kernel_tests.rs:178-210).
//
// One warp per output row.  Q4_K: the 32 lanes read the 128 nibble bytes of a block as 32
// consecutive words; Q2_K: two blocks per step, 16 lanes each on the 64 code bytes.  Dense
// calls with several tokens share each decoded word between TT tokens.
#include <cuda_runtime.h>

#include "common.cuh"
#include "kernels.h"

namespace lisa {

struct GgufParams {
    const uint8_t *w;
    const float *x;
    const int32_t *ids;  // nullptr: dense
    float *y;
    int64_t row_bytes;
    int rows, blocks_per_row, experts, tokens, slots, top_k;
};

__device__ __forceinline__ float f16_bits_to_f32(uint32_t h) {
    float f;
    asm("{ .reg .b16 t; cvt.u16.u32 t, %1; cvt.f32.f16 %0, t; }" : "=f"(f) : "r"(h & 0xffffu));
    return f;
}

template <int TT>
__device__ __forceinline__ void q4k_row(const uint8_t *__restrict__ wrow, const float *const (&xr)[TT], int nblocks,
                                        int lane, float (&acc)[TT]) {
    const int pg = lane >> 3;          // pair of sub-blocks: low nibbles -> 2*pg, high -> 2*pg+1
    const int l0 = (lane & 7) * 4;     // element offset within the sub-block
    // several blocks of the row in flight per warp: the loads of a block do not depend on the previous one
#pragma unroll(TT == 1 ? 4 : 2)
    for (int ib = 0; ib < nblocks; ++ib) {
        const uint8_t *blk = wrow + static_cast<size_t>(ib) * 144;
        const uint4 hdr = __ldg(reinterpret_cast<const uint4 *>(blk));
        const uint32_t qs = __ldg(reinterpret_cast<const uint32_t *>(blk + 16) + lane);
        const float d = f16_bits_to_f32(hdr.x), dmin = f16_bits_to_f32(hdr.x >> 16);
        float sc[2], mn[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int g = 2 * pg + h, sh = 8 * (g & 3);
            const uint32_t b0 = (hdr.y >> sh) & 255u, b1 = (hdr.z >> sh) & 255u, b2 = (hdr.w >> sh) & 255u;
            const uint32_t s = (g < 4) ? (b0 & 63u) : ((b2 & 15u) | ((b0 >> 6) << 4));
            const uint32_t m = (g < 4) ? (b1 & 63u) : ((b2 >> 4) | ((b1 >> 6) << 4));
            sc[h] = d * static_cast<float>(s);
            mn[h] = dmin * static_cast<float>(m);
        }
        float ql[4], qh[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            ql[j] = static_cast<float>((qs >> (8 * j)) & 15u);
            qh[j] = static_cast<float>((qs >> (8 * j + 4)) & 15u);
        }
        const int e_lo = ib * 256 + (2 * pg) * 32 + l0;
#pragma unroll
        for (int t = 0; t < TT; ++t) {
            const float4 xl = __ldg(reinterpret_cast<const float4 *>(xr[t] + e_lo));
            const float4 xh = __ldg(reinterpret_cast<const float4 *>(xr[t] + e_lo + 32));
            const float dl = ql[0] * xl.x + ql[1] * xl.y + ql[2] * xl.z + ql[3] * xl.w;
            const float dh = qh[0] * xh.x + qh[1] * xh.y + qh[2] * xh.z + qh[3] * xh.w;
            const float sl = (xl.x + xl.y) + (xl.z + xl.w);
            const float sh = (xh.x + xh.y) + (xh.z + xh.w);
            acc[t] += (sc[0] * dl - mn[0] * sl) + (sc[1] * dh - mn[1] * sh);
        }
    }
}

// Q5_K (crates/lisa-gguf/src/quant.rs:161-182; replaces lisa_gguf_q5_K_mv): the Q4_K block with a fifth bit per
// element: {d, dmin, 12 scale/min bytes, qh[32], qs[128]}; element j of group g is the nibble (g % 2) of
// qs[(g / 2) * 32 + j] plus 16 when bit g of qh[j] is set.  Same lane layout as q4k_row: lane = (pair of groups,
// four consecutive elements).
template <int TT>
__device__ __forceinline__ void q5k_row(const uint8_t *__restrict__ wrow, const float *const (&xr)[TT], int nblocks,
                                        int lane, float (&acc)[TT]) {
    const int pg = lane >> 3;
    const int l0 = (lane & 7) * 4;
#pragma unroll(TT == 1 ? 4 : 2)
    for (int ib = 0; ib < nblocks; ++ib) {
        const uint8_t *blk = wrow + static_cast<size_t>(ib) * 176;
        const uint4 hdr = __ldg(reinterpret_cast<const uint4 *>(blk));
        const uint32_t qh = __ldg(reinterpret_cast<const uint32_t *>(blk + 16 + l0));
        const uint32_t qs = __ldg(reinterpret_cast<const uint32_t *>(blk + 48) + lane);
        const float d = f16_bits_to_f32(hdr.x), dmin = f16_bits_to_f32(hdr.x >> 16);
        float sc[2], mn[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int g = 2 * pg + h, sh = 8 * (g & 3);
            const uint32_t b0 = (hdr.y >> sh) & 255u, b1 = (hdr.z >> sh) & 255u, b2 = (hdr.w >> sh) & 255u;
            const uint32_t s = (g < 4) ? (b0 & 63u) : ((b2 & 15u) | ((b0 >> 6) << 4));
            const uint32_t m = (g < 4) ? (b1 & 63u) : ((b2 >> 4) | ((b1 >> 6) << 4));
            sc[h] = d * static_cast<float>(s);
            mn[h] = dmin * static_cast<float>(m);
        }
        float ql[4], qhi[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t hb = qh >> (8 * j);  // byte qh[l0 + j]
            ql[j] = static_cast<float>(((qs >> (8 * j)) & 15u) + (((hb >> (2 * pg)) & 1u) << 4));
            qhi[j] = static_cast<float>(((qs >> (8 * j + 4)) & 15u) + (((hb >> (2 * pg + 1)) & 1u) << 4));
        }
        const int e_lo = ib * 256 + (2 * pg) * 32 + l0;
#pragma unroll
        for (int t = 0; t < TT; ++t) {
            const float4 xl = __ldg(reinterpret_cast<const float4 *>(xr[t] + e_lo));
            const float4 xh = __ldg(reinterpret_cast<const float4 *>(xr[t] + e_lo + 32));
            const float dl = ql[0] * xl.x + ql[1] * xl.y + ql[2] * xl.z + ql[3] * xl.w;
            const float dh = qhi[0] * xh.x + qhi[1] * xh.y + qhi[2] * xh.z + qhi[3] * xh.w;
            const float sl = (xl.x + xl.y) + (xl.z + xl.w);
            const float sh = (xh.x + xh.y) + (xh.z + xh.w);
            acc[t] += (sc[0] * dl - mn[0] * sl) + (sc[1] * dh - mn[1] * sh);
        }
    }
}

template <int TT>
__device__ __forceinline__ void q2k_row(const uint8_t *__restrict__ wrow, const float *const (&xr)[TT], int nblocks,
                                        int lane, float (&acc)[TT]) {
    const int sub = lane >> 4, t16 = lane & 15;
    const int half = t16 >> 3, group = (t16 & 7) >> 2, pos = (t16 & 7) * 4;
#pragma unroll(TT == 1 ? 4 : 2)
    for (int ib = sub; ib < nblocks; ib += 2) {
        const uint8_t *blk = wrow + static_cast<size_t>(ib) * 84;
        const uint32_t qs = __ldg(reinterpret_cast<const uint32_t *>(blk + 16) + t16);
        const uint32_t dd = __ldg(reinterpret_cast<const uint32_t *>(blk + 80));
        const float d = f16_bits_to_f32(dd), dmin = f16_bits_to_f32(dd >> 16);
        float dl[4], ml[4];
#pragma unroll
        for (int s = 0; s < 4; ++s) {
            const uint32_t scb = __ldg(blk + half * 8 + s * 2 + group);
            dl[s] = d * static_cast<float>(scb & 15u);
            ml[s] = dmin * static_cast<float>(scb >> 4);
        }
        const int e0 = ib * 256 + half * 128 + pos;
#pragma unroll
        for (int t = 0; t < TT; ++t) {
            float a = 0.f;
#pragma unroll
            for (int s = 0; s < 4; ++s) {
                const float4 xv = __ldg(reinterpret_cast<const float4 *>(xr[t] + e0 + s * 32));
                const float q0 = static_cast<float>((qs >> (2 * s)) & 3u);
                const float q1 = static_cast<float>((qs >> (8 + 2 * s)) & 3u);
                const float q2 = static_cast<float>((qs >> (16 + 2 * s)) & 3u);
                const float q3 = static_cast<float>((qs >> (24 + 2 * s)) & 3u);
                const float dq = q0 * xv.x + q1 * xv.y + q2 * xv.z + q3 * xv.w;
                const float sx = (xv.x + xv.y) + (xv.z + xv.w);
                a += dl[s] * dq - ml[s] * sx;
            }
            acc[t] += a;
        }
    }
}

// grid.x: token groups (dense) or token*top_k slots (experts); grid.y: row blocks of 8 warps.
template <int FORMAT, int TT>
__global__ void __launch_bounds__(256) gguf_matvec_kernel(const GgufParams p) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.y * 8 + (threadIdx.x >> 5);
    if (row >= p.rows) return;
    const int64_t k = static_cast<int64_t>(p.blocks_per_row) * 256;
    const uint8_t *wrow;
    const float *xr[TT];
    int64_t out_base[TT];
    bool live[TT];
    if (p.ids) {
        const int z = blockIdx.x;  // token * top_k + slot
        const int token = z / p.top_k, slot = z - token * p.top_k;
        const int e = __ldg(p.ids + z);
        out_base[0] = static_cast<int64_t>(z) * p.rows + row;
        if (e < 0 || e >= p.experts) {  // no weight access for an id outside the table
            if (lane == 0) p.y[out_base[0]] = 0.f;
            return;
        }
        wrow = p.w + (static_cast<int64_t>(e) * p.rows + row) * p.row_bytes;
        xr[0] = p.x + (static_cast<int64_t>(token) * p.slots + (slot % p.slots)) * k;
        live[0] = true;
    } else {
        wrow = p.w + static_cast<int64_t>(row) * p.row_bytes;
#pragma unroll
        for (int t = 0; t < TT; ++t) {
            const int token = blockIdx.x * TT + t;
            live[t] = token < p.tokens;
            const int tk = live[t] ? token : p.tokens - 1;
            xr[t] = p.x + static_cast<int64_t>(tk) * k;
            out_base[t] = static_cast<int64_t>(tk) * p.rows + row;
        }
    }
    float acc[TT];
#pragma unroll
    for (int t = 0; t < TT; ++t) acc[t] = 0.f;
    if (FORMAT == LISA_GGUF_Q4_K) q4k_row<TT>(wrow, xr, p.blocks_per_row, lane, acc);
    else if (FORMAT == LISA_GGUF_Q5_K) q5k_row<TT>(wrow, xr, p.blocks_per_row, lane, acc);
    else q2k_row<TT>(wrow, xr, p.blocks_per_row, lane, acc);
#pragma unroll
    for (int t = 0; t < TT; ++t) {
        float v = acc[t];
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        if (lane == 0 && live[t]) p.y[out_base[t]] = v;
    }
}

int gguf_matvec(cudaStream_t stream, int format, const uint8_t *w, int64_t experts, int64_t rows, int64_t row_bytes,
                const float *x, int64_t tokens, int64_t slots, const int32_t *ids, int64_t top_k, float *y) {
    const int block_bytes = (format == LISA_GGUF_Q2_K) ? 84 : (format == LISA_GGUF_Q5_K) ? 176 : 144;
    if ((reinterpret_cast<uintptr_t>(w) & 15u) != 0)
        return fail(LISA_ERR_MISALIGNED, "gguf matvec: weights must be 16-byte aligned");
    GgufParams p{};
    p.w = w;
    p.x = x;
    p.ids = ids;
    p.y = y;
    p.row_bytes = row_bytes;
    p.rows = static_cast<int>(rows);
    p.blocks_per_row = static_cast<int>(row_bytes / block_bytes);
    p.experts = static_cast<int>(experts);
    p.tokens = static_cast<int>(tokens);
    p.slots = static_cast<int>(slots);
    p.top_k = static_cast<int>(top_k);
    if ((rows + 7) / 8 > 65535) return fail(LISA_ERR_LIMIT, "gguf matvec: more than 524280 rows");
    const unsigned gy = static_cast<unsigned>((rows + 7) / 8);
    dim3 grid;
    int tt = 1;
    if (ids) grid = dim3(static_cast<unsigned>(tokens * top_k), gy);
    else if (tokens == 1) grid = dim3(1, gy);
    else {
        grid = dim3(static_cast<unsigned>((tokens + 3) / 4), gy);
        tt = 4;
    }
    if (format == LISA_GGUF_Q4_K) {
        if (tt == 4) gguf_matvec_kernel<LISA_GGUF_Q4_K, 4><<<grid, 256, 0, stream>>>(p);
        else gguf_matvec_kernel<LISA_GGUF_Q4_K, 1><<<grid, 256, 0, stream>>>(p);
    } else if (format == LISA_GGUF_Q5_K) {
        if (tt == 4) gguf_matvec_kernel<LISA_GGUF_Q5_K, 4><<<grid, 256, 0, stream>>>(p);
        else gguf_matvec_kernel<LISA_GGUF_Q5_K, 1><<<grid, 256, 0, stream>>>(p);
    } else {
        if (tt == 4) gguf_matvec_kernel<LISA_GGUF_Q2_K, 4><<<grid, 256, 0, stream>>>(p);
        else gguf_matvec_kernel<LISA_GGUF_Q2_K, 1><<<grid, 256, 0, stream>>>(p);
    }
    LISA_CUDA_TRY(cudaGetLastError());
    count_launch();
    return LISA_OK;
}

}  // namespace lisa
