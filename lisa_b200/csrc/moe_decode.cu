// The routed-expert block for a handful of tokens (decode), as the reference runs it: no sort, no gathered
// copy of the activations, no per-expert tiles -- every slot (token, j) streams the rows of its own expert.
//
//   moe_gate_up_act      act[slot, :] = swiglu(bf16(x[xrow] . Wg[idx[slot]]^T), bf16(x[xrow] . Wu[idx[slot]]^T))
//   moe_down_combine     out[t, :]    = bf16( fold_j f32(bf16(act[t*k + j] . Wd[idx[t, j]]^T)) * w[t, j] )
//
// replace moe_decode::gate_up_act / down_combine (crates/lisa-mlx/src/models/qwen4/moe_decode.rs:136-298,
// shaders/qwen4/gate_up_reuse.metal, down_combine.metal) without their shared-expert operands, which the routed
// block of the MLX checkpoints does not have.  Rounding points are the reference's: gate and up results each to
// bf16, sigmoid, silu and the product to bf16 (exact_header.metal:2-11), every down result to bf16, the fold of
// mlx_colsum_small_f32 in slot order in f32, the output to bf16 (exact_header.metal:12-24).  With the router
// (moe_route) in front the block is three launches.
//
// Both kernels are weight streams: one warp per output row of one slot, 16-byte loads of packed words (several in
// flight per lane), the activations of the slot staged once per block in shared memory, the qmv factorisation
// scale * sum(q * x) + bias * sum(x) per group (quantized.metal:196-295) in f32.  An id outside [0, experts)
// touches no weights and contributes zeros (deepseek41.rs:204-206).
#include <cuda_runtime.h>

#include <algorithm>

#include "common.cuh"
#include "kernels.h"

namespace lisa {

namespace {

__device__ __forceinline__ float md_round_bf16(float v) { return bf16_bits_to_f32(f32_to_bf16_bits(v)); }

// act = bf16(silu * u), silu = bf16(g * s), s = bf16(sigmoid(g)) evaluated as 1 / (1 + exp(|g|)) mirrored by sign
// (the same function as moe_swiglu's, so the fused and the chained block agree bit for bit on equal inputs)
__device__ __forceinline__ uint16_t md_swiglu_bits(uint16_t gb, uint16_t ub) {
    const float g = bf16_bits_to_f32(gb), u = bf16_bits_to_f32(ub);
    const float y = 1.0f / (1.0f + expf(fabsf(g)));
    const float s = md_round_bf16(g < 0.f ? y : 1.0f - y);
    const float silu = md_round_bf16(g * s);
    return static_cast<uint16_t>(f32_to_bf16_bits(silu * u));
}

// One packed word of each of ROWS rows against the same CPW activations (bf16 in shared memory, 16-byte aligned):
// sum(q * x) per row and sum(x).  A code becomes a float through the mantissa of 2^23 (one logic op and one add,
// both full rate; the integer-to-float conversion runs at a quarter of that): (2^23 + q) - 2^23 = q exactly.
template <int BITS, int ROWS>
__device__ __forceinline__ void md_word(const uint32_t (&word)[ROWS], const uint16_t *xs, float (&accum)[ROWS], float &xsum) {
    constexpr int CPW = 32 / BITS;
    constexpr uint32_t kMask = (1u << BITS) - 1u;
    const uint4 *xv = reinterpret_cast<const uint4 *>(xs);
#pragma unroll
    for (int v = 0; v < CPW / 8; ++v) {
        const uint4 xx = xv[v];
        const uint32_t xw[4] = {xx.x, xx.y, xx.z, xx.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float x0 = bf16_bits_to_f32(xw[j] & 0xffffu), x1 = __uint_as_float(xw[j] & 0xffff0000u);
            const int c = v * 8 + 2 * j;
#pragma unroll
            for (int r = 0; r < ROWS; ++r) {
                const float q0 = __uint_as_float(((word[r] >> (c * BITS)) & kMask) | 0x4b000000u) - 8388608.f;
                const float q1 = __uint_as_float(((word[r] >> ((c + 1) * BITS)) & kMask) | 0x4b000000u) - 8388608.f;
                accum[r] = fmaf(x0, q0, accum[r]);
                accum[r] = fmaf(x1, q1, accum[r]);
            }
            xsum += x0 + x1;
        }
    }
}

// Dot products of ROWS packed rows (words_per_row a multiple of 4, 16-byte aligned) with the staged activations,
// this lane's share: chunks lane, lane + 32, ... of four words; a trip takes two chunks per row (2 * ROWS 16-byte
// loads in flight).  The loads of the first trip are issued by the caller BEFORE it stages the activations, so
// that the two round trips to memory overlap.
template <int ROWS>
__device__ __forceinline__ void md_load(const uint32_t *const (&wr)[ROWS], int chunks, int c0, uint4 (&w0)[ROWS],
                                        uint4 (&w1)[ROWS]) {
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        w0[r] = c0 < chunks ? __ldg(reinterpret_cast<const uint4 *>(wr[r]) + c0) : make_uint4(0, 0, 0, 0);
        w1[r] = c0 + 32 < chunks ? __ldg(reinterpret_cast<const uint4 *>(wr[r]) + c0 + 32) : make_uint4(0, 0, 0, 0);
    }
}

template <int BITS, int ROWS>
__device__ __forceinline__ void md_rows(const uint32_t *const (&wr)[ROWS], const uint16_t *const (&sr)[ROWS],
                                        const uint16_t *const (&br)[ROWS], const uint16_t *xs, int words_per_row,
                                        int group_size, int lane, uint4 (&w0)[ROWS], uint4 (&w1)[ROWS],
                                        float (&result)[ROWS]) {
    constexpr int CPW = 32 / BITS;
    const int chunks = words_per_row >> 2;
#pragma unroll
    for (int r = 0; r < ROWS; ++r) result[r] = 0.f;
    for (int c0 = lane; c0 < chunks; c0 += 64) {
        if (c0 != lane) md_load<ROWS>(wr, chunks, c0, w0, w1);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int c = c0 + 32 * half;
            if (c >= chunks) break;
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) {
                const int k0 = (c * 4 + wi) * CPW;
                const int g = k0 / group_size;
                uint32_t word[ROWS];
                float accum[ROWS], xsum = 0.f;
#pragma unroll
                for (int r = 0; r < ROWS; ++r) {
                    const uint4 &wv = half ? w1[r] : w0[r];
                    word[r] = wi == 0 ? wv.x : wi == 1 ? wv.y : wi == 2 ? wv.z : wv.w;
                    accum[r] = 0.f;
                }
                md_word<BITS, ROWS>(word, xs + k0, accum, xsum);
#pragma unroll
                for (int r = 0; r < ROWS; ++r) {
                    result[r] = fmaf(bf16_bits_to_f32(__ldg(sr[r] + g)), accum[r], result[r]);
                    result[r] = fmaf(bf16_bits_to_f32(__ldg(br[r] + g)), xsum, result[r]);
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r)
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) result[r] += __shfl_xor_sync(0xffffffffu, result[r], off);
}

struct GateUpParams {
    const uint32_t *wg, *wu;
    const uint16_t *sg, *bg, *su, *bu;
    const uint16_t *x;
    const int32_t *idx;   // [slots] expert of every slot
    const int32_t *xrow;  // [slots] row of x of every slot, or null: slot / top_k
    uint16_t *act;        // [slots, n]
    int64_t expert_words, expert_groups;
    int n, k, experts, top_k, group_size, words_per_row, groups_per_row;
};

// grid (ceil(n / 8), slots), 8 warps: warp = output column of the slot
template <int BITS>
__global__ void __launch_bounds__(256) moe_gate_up_act_kernel(const GateUpParams p) {
    extern __shared__ __align__(16) uint8_t md_smem[];
    uint16_t *xs = reinterpret_cast<uint16_t *>(md_smem);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int slot = blockIdx.y;
    const int col = blockIdx.x * 8 + warp;
    const int e = __ldg(p.idx + slot);
    if (e < 0 || e >= p.experts) {  // uniform over the block
        if (lane == 0 && col < p.n) p.act[static_cast<int64_t>(slot) * p.n + col] = 0;
        return;
    }
    const int ccol = min(col, p.n - 1);  // (a column beyond n computes the last one and stores nothing)
    const int64_t wo = e * p.expert_words + static_cast<int64_t>(ccol) * p.words_per_row;
    const int64_t go = e * p.expert_groups + static_cast<int64_t>(ccol) * p.groups_per_row;
    const uint32_t *const wr[2] = {p.wg + wo, p.wu + wo};
    const uint16_t *const sr[2] = {p.sg + go, p.su + go};
    const uint16_t *const br[2] = {p.bg + go, p.bu + go};
    uint4 w0[2], w1[2];
    md_load<2>(wr, p.words_per_row >> 2, lane, w0, w1);
    const int64_t row = p.xrow ? __ldg(p.xrow + slot) : slot / p.top_k;
    const uint4 *xsrc = reinterpret_cast<const uint4 *>(p.x + row * p.k);
    for (int i = threadIdx.x; i < p.k / 8; i += 256) reinterpret_cast<uint4 *>(xs)[i] = __ldg(xsrc + i);
    __syncthreads();
    float res[2];
    md_rows<BITS, 2>(wr, sr, br, xs, p.words_per_row, p.group_size, lane, w0, w1, res);
    if (lane == 0 && col < p.n)
        p.act[static_cast<int64_t>(slot) * p.n + col] =
            md_swiglu_bits(static_cast<uint16_t>(f32_to_bf16_bits(res[0])), static_cast<uint16_t>(f32_to_bf16_bits(res[1])));
}

struct DownParams {
    const uint32_t *wd;
    const uint16_t *sd, *bd;
    const uint16_t *act;     // [tokens * top_k, k]
    const int32_t *idx;      // [tokens, top_k]
    const float *weights;    // [tokens, top_k]
    uint16_t *out;           // [tokens, n]
    int64_t expert_words, expert_groups;
    int n, k, experts, top_k, group_size, words_per_row, groups_per_row;
};

constexpr int kDownCols = 4;  // output columns of one token per block: kDownCols * top_k (column, slot) pairs over 8 warps

// grid (ceil(n / kDownCols), tokens), 8 warps
template <int BITS>
__global__ void __launch_bounds__(256) moe_down_combine_kernel(const DownParams p) {
    extern __shared__ __align__(16) uint8_t md_smem[];
    uint16_t *as = reinterpret_cast<uint16_t *>(md_smem);                                  // [top_k][k]
    float *ds = reinterpret_cast<float *>(md_smem + static_cast<size_t>(p.top_k) * p.k * 2);  // [kDownCols][top_k]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.y;
    const int pairs = kDownCols * p.top_k;
    // (column, slot) pair pi of this warp: its expert row, or null when the column or the id is outside the table
    auto pair_row = [&](int pi, int &j, int64_t &go) -> const uint32_t * {
        const int cl = pi / p.top_k;
        j = pi - cl * p.top_k;
        const int col = blockIdx.x * kDownCols + cl;
        if (pi >= pairs || col >= p.n) return nullptr;
        const int e = __ldg(p.idx + t * p.top_k + j);
        if (e < 0 || e >= p.experts) return nullptr;
        go = e * p.expert_groups + static_cast<int64_t>(col) * p.groups_per_row;
        return p.wd + e * p.expert_words + static_cast<int64_t>(col) * p.words_per_row;
    };
    // the first pair's packed words are requested before the activations are staged
    int j = 0;
    int64_t go = 0;
    const uint32_t *row = pair_row(warp, j, go);
    uint4 w0[1], w1[1];
    {
        const uint32_t *const wr[1] = {row};
        md_load<1>(wr, row ? p.words_per_row >> 2 : 0, lane, w0, w1);
    }
    const uint4 *asrc = reinterpret_cast<const uint4 *>(p.act + static_cast<int64_t>(t) * p.top_k * p.k);
    for (int i = threadIdx.x; i < p.top_k * p.k / 8; i += 256) reinterpret_cast<uint4 *>(as)[i] = __ldg(asrc + i);
    __syncthreads();
    for (int pi = warp; pi < pairs; pi += 8) {
        float d = 0.f;
        int jn = 0;
        int64_t gon = 0;
        const uint32_t *next = pair_row(pi + 8, jn, gon);
        if (row) {
            const uint32_t *const wr[1] = {row};
            const uint16_t *const sr[1] = {p.sd + go};
            const uint16_t *const br[1] = {p.bd + go};
            float res[1];
            md_rows<BITS, 1>(wr, sr, br, as + static_cast<size_t>(j) * p.k, p.words_per_row, p.group_size, lane, w0, w1, res);
            d = md_round_bf16(res[0]);  // the down result is a bf16 tensor in the reference
        }
        if (lane == 0) ds[pi] = d;
        row = next;
        j = jn;
        go = gon;
        if (row) {
            const uint32_t *const wr[1] = {row};
            md_load<1>(wr, p.words_per_row >> 2, lane, w0, w1);
        }
    }
    __syncthreads();
    if (threadIdx.x < kDownCols) {
        const int cl = threadIdx.x, col = blockIdx.x * kDownCols + cl;
        if (col < p.n) {
            // fold of mlx_colsum_small_f32: ty = min(k, 8) strided partial sums, then total = part[j] + total
            const int ty = p.top_k < 8 ? p.top_k : 8;
            float part[8];
#pragma unroll
            for (int y = 0; y < 8; ++y) part[y] = 0.f;
            for (int rr = 0; rr < p.top_k; ++rr) {
                const float r = ds[cl * p.top_k + rr] * __ldg(p.weights + t * p.top_k + rr);
                const int y = rr % ty;
#pragma unroll
                for (int q = 0; q < 8; ++q)
                    if (q == y) part[q] = r + part[q];
            }
            float total = part[0];
#pragma unroll
            for (int q = 1; q < 8; ++q)
                if (q < ty) total = part[q] + total;
            p.out[static_cast<int64_t>(t) * p.n + col] = static_cast<uint16_t>(f32_to_bf16_bits(total));
        }
    }
}

}  // namespace

bool moe_decode_supported(int64_t k, int group_size, int bits, int top_k) {
    if (bits != 2 && bits != 4) return false;
    if (group_size < 32 || group_size % (32 / bits) != 0 || k % group_size != 0) return false;
    if ((k * bits / 32) % 4 != 0 || k % 8 != 0) return false;   // 16-byte chunks of packed words and of activations
    if (top_k < 1 || top_k > 32) return false;
    return static_cast<int64_t>(top_k) * k * 2 + kDownCols * top_k * 4 <= 160 * 1024 && k * 2 <= 160 * 1024;
}

int moe_gate_up_act(cudaStream_t stream, const void *x, const int32_t *idx, const int32_t *xrow, int64_t slots, int top_k,
                    int64_t experts, int64_t k, int64_t n, const uint32_t *wg, const void *sg, const void *bg,
                    const uint32_t *wu, const void *su, const void *bu, int group_size, int bits, void *act) {
    GateUpParams p{};
    p.wg = wg; p.wu = wu;
    p.sg = reinterpret_cast<const uint16_t *>(sg); p.bg = reinterpret_cast<const uint16_t *>(bg);
    p.su = reinterpret_cast<const uint16_t *>(su); p.bu = reinterpret_cast<const uint16_t *>(bu);
    p.x = reinterpret_cast<const uint16_t *>(x);
    p.idx = idx; p.xrow = xrow;
    p.act = reinterpret_cast<uint16_t *>(act);
    p.n = static_cast<int>(n); p.k = static_cast<int>(k); p.experts = static_cast<int>(experts); p.top_k = top_k;
    p.group_size = group_size;
    p.words_per_row = static_cast<int>(k * bits / 32);
    p.groups_per_row = static_cast<int>(k / group_size);
    p.expert_words = n * p.words_per_row;
    p.expert_groups = n * p.groups_per_row;
    const size_t smem = static_cast<size_t>(k) * 2;
    const unsigned gx = static_cast<unsigned>((n + 7) / 8);
    for (int64_t base = 0; base < slots; base += 65535) {
        const unsigned gy = static_cast<unsigned>(std::min<int64_t>(slots - base, 65535));
        GateUpParams q = p;
        q.idx = idx + base;
        q.xrow = xrow ? xrow + base : nullptr;
        q.act = p.act + base * n;
        if (!xrow && base) return fail(LISA_ERR_LIMIT, "moe_gate_up_act: more than 65535 slots need xrow");
        if (bits == 4) {
            LISA_CUDA_TRY(cudaFuncSetAttribute(moe_gate_up_act_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
            moe_gate_up_act_kernel<4><<<dim3(gx, gy), 256, smem, stream>>>(q);
        } else {
            LISA_CUDA_TRY(cudaFuncSetAttribute(moe_gate_up_act_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
            moe_gate_up_act_kernel<2><<<dim3(gx, gy), 256, smem, stream>>>(q);
        }
        LISA_CUDA_TRY(cudaGetLastError());
        count_launch();
    }
    return LISA_OK;
}

int moe_down_combine(cudaStream_t stream, const void *act, const int32_t *idx, const float *weights, int64_t tokens, int top_k,
                     int64_t experts, int64_t k, int64_t n, const uint32_t *wd, const void *sd, const void *bd, int group_size,
                     int bits, void *out) {
    DownParams p{};
    p.wd = wd;
    p.sd = reinterpret_cast<const uint16_t *>(sd); p.bd = reinterpret_cast<const uint16_t *>(bd);
    p.act = reinterpret_cast<const uint16_t *>(act);
    p.idx = idx; p.weights = weights;
    p.out = reinterpret_cast<uint16_t *>(out);
    p.n = static_cast<int>(n); p.k = static_cast<int>(k); p.experts = static_cast<int>(experts); p.top_k = top_k;
    p.group_size = group_size;
    p.words_per_row = static_cast<int>(k * bits / 32);
    p.groups_per_row = static_cast<int>(k / group_size);
    p.expert_words = n * p.words_per_row;
    p.expert_groups = n * p.groups_per_row;
    const size_t smem = static_cast<size_t>(top_k) * k * 2 + kDownCols * top_k * 4;
    const unsigned gx = static_cast<unsigned>((n + kDownCols - 1) / kDownCols);
    for (int64_t base = 0; base < tokens; base += 65535) {
        const unsigned gy = static_cast<unsigned>(std::min<int64_t>(tokens - base, 65535));
        DownParams q = p;
        q.act = p.act + base * top_k * k;
        q.idx = idx + base * top_k;
        q.weights = weights + base * top_k;
        q.out = p.out + base * n;
        if (bits == 4) {
            LISA_CUDA_TRY(cudaFuncSetAttribute(moe_down_combine_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
            moe_down_combine_kernel<4><<<dim3(gx, gy), 256, smem, stream>>>(q);
        } else {
            LISA_CUDA_TRY(cudaFuncSetAttribute(moe_down_combine_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
            moe_down_combine_kernel<2><<<dim3(gx, gy), 256, smem, stream>>>(q);
        }
        LISA_CUDA_TRY(cudaGetLastError());
        count_launch();
    }
    return LISA_OK;
}

}  // namespace lisa
