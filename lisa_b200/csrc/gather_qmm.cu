// MoE routed-expert matmul: y[r, :] = x[r, :] . dequant(W[ids[r]])^T for rows sorted by expert.
//
// Replaces ops::gather_qmm -> gather_qmm_rhs_nax / the per-run host loop
// (crates/lisa-mlx/src/ops/array_ops.rs:561-642, crates/lisa-mlx/src/jit/nax.rs:224-301).
// Unlike the reference's non-NAX path there is no host read-back of the ids: the expert of
// every row is looked up on the device.
//
// Rows-per-expert decides the kernel: up to eight rows per expert on average (decode, small batches) is a
// weight-streaming problem handled by the tensor-memory matvec kernel over a table of (expert, <= 8 rows)
// entries (qmv_tc.cu); more rows per expert is a grouped GEMM over a table of taller tiles (qmm_affine.cu);
// without a workspace, or for shapes those two do not take, gather_qmv_kernel (one warp per output).
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"

namespace lisa {

struct GatherParams {
    const uint32_t *w;
    const uint16_t *scales;
    const uint16_t *biases;
    const uint16_t *x;
    const int32_t *ids;
    uint16_t *y;
    int64_t expert_words;   // n * k * bits / 32
    int64_t expert_groups;  // n * k / group_size
    int n, k, experts, group_size, words_per_row, groups_per_row;
};

template <int BITS>
__global__ void __launch_bounds__(256) gather_qmv_kernel(const GatherParams p, int64_t row_base) {
    constexpr int CPW = 32 / BITS;
    const int lane = threadIdx.x & 31;
    const int col = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int64_t row = row_base + blockIdx.y;
    if (col >= p.n) return;
    const int e = __ldg(p.ids + row);
    if (e < 0 || e >= p.experts) {  // no weight access for an id outside the table
        if (lane == 0) p.y[row * p.n + col] = 0;
        return;
    }
    const uint32_t *wr = p.w + e * p.expert_words + static_cast<int64_t>(col) * p.words_per_row;
    const uint16_t *sr = p.scales + e * p.expert_groups + static_cast<int64_t>(col) * p.groups_per_row;
    const uint16_t *br = p.biases + e * p.expert_groups + static_cast<int64_t>(col) * p.groups_per_row;
    const uint16_t *xr = p.x + row * p.k;
    float result = 0.f;
    for (int wi = lane; wi < p.words_per_row; wi += 32) {
        const uint32_t word = __ldg(wr + wi);
        const int k0 = wi * CPW;
        const int g = k0 / p.group_size;
        float accum = 0.f, xsum = 0.f;
#pragma unroll
        for (int j = 0; j < CPW; j += 2) {
            const uint32_t xx = __ldg(reinterpret_cast<const uint32_t *>(xr + k0 + j));
            const float x0 = bf16_bits_to_f32(xx & 0xffffu), x1 = __uint_as_float(xx & 0xffff0000u);
            const uint32_t q0 = (word >> (j * BITS)) & ((1u << BITS) - 1u);
            const uint32_t q1 = (word >> ((j + 1) * BITS)) & ((1u << BITS) - 1u);
            accum = fmaf(x0, static_cast<float>(q0), accum);
            accum = fmaf(x1, static_cast<float>(q1), accum);
            xsum += x0 + x1;
        }
        result = fmaf(bf16_bits_to_f32(__ldg(sr + g)), accum, result);
        result = fmaf(bf16_bits_to_f32(__ldg(br + g)), xsum, result);
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) result += __shfl_xor_sync(0xffffffffu, result, off);
    if (lane == 0) p.y[row * p.n + col] = static_cast<uint16_t>(f32_to_bf16_bits(result));
}

// ---------------------------------------------------------------------------------------
// Tile table of the grouped GEMM, built on the device from the sorted ids (no host read-back):
// tile = {expert, row_begin, row_end, 0}, at most `bt` rows, never spanning two experts -- the layout
// of the reference's prefill tile table (crates/lisa-engine/src/models/qwen4/prefill_indirect.rs:103-133)
// with the expert added.  Rows whose id is outside [0, experts) get zeros here and no tile.
__device__ __forceinline__ int lower_bound_ids(const int32_t *ids, int rows, int value) {
    int lo = 0, hi = rows;
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (__ldg(ids + mid) < value) lo = mid + 1;
        else hi = mid;
    }
    return lo;
}

constexpr int kTableThreads = 1024;
constexpr int kTableOutputs = 4;

constexpr int kTableFillBlocks = 32;

struct TableOutputs {
    uint16_t *y[kTableOutputs];
    int count;
};

// Zeros over the elements [a, b) of y, spread over `nthreads` threads: 16-byte stores between the aligned ends.
__device__ __forceinline__ void zero_elements(uint16_t *y, int64_t a, int64_t b, int64_t tid, int64_t nthreads) {
    if (b <= a) return;
    const uintptr_t addr = reinterpret_cast<uintptr_t>(y + a);
    int64_t lead = static_cast<int64_t>(((16u - static_cast<unsigned>(addr & 15u)) & 15u) >> 1);
    lead = lead < b - a ? lead : b - a;
    for (int64_t i = tid; i < lead; i += nthreads) y[a + i] = 0;
    const int64_t a2 = a + lead, nvec = (b - a2) >> 3;
    uint4 *v = reinterpret_cast<uint4 *>(y + a2);
    for (int64_t i = tid; i < nvec; i += nthreads) v[i] = make_uint4(0u, 0u, 0u, 0u);
    for (int64_t i = a2 + nvec * 8 + tid; i < b; i += nthreads) y[i] = 0;
}

// Block 0 builds the table; the other blocks write the zeros of the rows whose ids are outside the table (sorted
// ids: negatives first, ids >= experts last -- the padding of an expert-parallel receive buffer can be most of the
// rows).  With at most 1024 experts the run of every expert comes from one coalesced pass over the ids
// (a run starts where ids[i] != ids[i-1]) and the tile counts are scanned with warp shuffles; with more
// experts every thread searches its experts' bounds, 1024 experts per trip.  The table never grows past
// `max_tiles` entries, whatever the ids hold (ids that are not sorted give a wrong table, not a write
// outside it).
__global__ void __launch_bounds__(kTableThreads) gather_tile_table_kernel(const int32_t *__restrict__ ids, int rows, int experts,
                                                                          int bt, int n, int max_tiles, int32_t *tiles,
                                                                          int32_t *tile_count, TableOutputs out) {
    __shared__ int begin_s[kTableThreads], end_s[kTableThreads];
    __shared__ int warp_sum[32];
    __shared__ int running;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (blockIdx.x > 0) {
        const int first_ok = lower_bound_ids(ids, rows, 0);
        const int first_bad = lower_bound_ids(ids, rows, experts);
        if (first_ok == 0 && first_bad == rows) return;
        const int64_t t = static_cast<int64_t>(blockIdx.x - 1) * kTableThreads + tid;
        const int64_t nt = static_cast<int64_t>(gridDim.x - 1) * kTableThreads;
        for (int o = 0; o < out.count; ++o) {
            zero_elements(out.y[o], 0, static_cast<int64_t>(first_ok) * n, t, nt);
            zero_elements(out.y[o], static_cast<int64_t>(first_bad) * n, static_cast<int64_t>(rows) * n, t, nt);
        }
        return;
    }
    const bool one_pass = experts <= kTableThreads;
    if (tid == 0) running = 0;
    begin_s[tid] = 0;
    end_s[tid] = 0;
    __syncthreads();
    if (one_pass) {
        constexpr int kFlight = 8;  // rows per thread and trip, their loads in flight together
        // (whole warps enter a trip: the shuffle below names every lane)
        for (int w0 = tid - lane; w0 < rows; w0 += kFlight * kTableThreads) {
            const int i0 = w0 + lane;
            int cur8[kFlight], edge8[kFlight];
#pragma unroll
            for (int j = 0; j < kFlight; ++j) {
                const int i = i0 + j * kTableThreads;
                cur8[j] = i < rows ? __ldg(ids + i) : 0;
                edge8[j] = (lane == 0 && i < rows && i > 0) ? __ldg(ids + i - 1) : 0;  // the other lanes: their neighbour's row
            }
#pragma unroll
            for (int j = 0; j < kFlight; ++j) {
                const int i = i0 + j * kTableThreads;
                const int left = __shfl_up_sync(0xffffffffu, cur8[j], 1);
                if (i >= rows) continue;
                const int cur = cur8[j], prev = lane == 0 ? edge8[j] : left;
                const bool head = i == 0;
                if (head || prev != cur) {
                    if (cur >= 0 && cur < experts) begin_s[cur] = i;
                    if (!head && prev >= 0 && prev < experts) end_s[prev] = i;
                }
                if (i == rows - 1 && cur >= 0 && cur < experts) end_s[cur] = rows;
            }
        }
        __syncthreads();
    }
    for (int base = 0; base < experts; base += kTableThreads) {
        const int e = base + tid;
        int begin = 0, end = 0;
        if (e < experts) {
            if (one_pass) {
                begin = begin_s[tid];
                end = end_s[tid];
            } else {
                begin = lower_bound_ids(ids, rows, e);
                end = lower_bound_ids(ids, rows, e + 1);
            }
        }
        const int mine = end > begin ? (end - begin + bt - 1) / bt : 0;
        int inc = mine;  // inclusive scan over the block: warps, then the warp sums
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, inc, off);
            if (lane >= off) inc += v;
        }
        if (lane == 31) warp_sum[warp] = inc;
        __syncthreads();
        if (warp == 0) {
            const int w = warp_sum[lane];
            int winc = w;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, winc, off);
                if (lane >= off) winc += v;
            }
            warp_sum[lane] = winc - w;  // exclusive
        }
        __syncthreads();
        int at = running + warp_sum[warp] + inc - mine;
        for (int r = begin; r < end && at < max_tiles; r += bt, ++at)
            reinterpret_cast<int4 *>(tiles)[at] = make_int4(e, r, min(r + bt, end), 0);
        __syncthreads();
        if (tid == kTableThreads - 1) running += warp_sum[warp] + inc;
        __syncthreads();
    }
    if (tid == 0) *tile_count = min(running, max_tiles);
}

// Rows per tile of the grouped GEMM: up to 256 rows the dequantization sets a CTA's pace, beyond that the MMAs, whose
// N follows the rows of the tile; a tile table of 384-row tiles therefore costs what its rows cost plus a little
// (a shallower operand ring), and wins as soon as it saves tiles.  Between 256 and 384 the choice goes by the
// expected number of tiles per expert when the rows spread evenly over the experts (run lengths then scatter
// around the average with a standard deviation of its root).
static int grouped_tile_rows(int64_t rows, int64_t experts) {
    const double avg = static_cast<double>(rows) / static_cast<double>(experts > 0 ? experts : 1);
    if (avg >= 96) {
        const double sd = std::sqrt(avg) + 1e-9;
        auto tiles = [&](double bt) {  // E[ceil(r / bt)], r ~ N(avg, sd)
            double t = 1.0;
            for (int j = 1; j * bt < avg + 6 * sd; ++j) t += 0.5 * std::erfc((j * bt - avg) / (sd * 1.41421356));
            return t;
        };
        return tiles(384.0) * 1.1 < tiles(256.0) ? 384 : 256;
    }
    if (avg >= 40) return 128;
    if (avg >= 12) return 64;
    if (avg >= 4) return 32;
    return 16;
}

size_t gather_qmm_workspace_bytes(int64_t rows, int64_t experts) {
    // Tile table: entries of 4 int32, never more than one per row (every entry holds a row), plus a counter block.
    const int64_t tiles = rows > 0 ? rows : 1;
    return static_cast<size_t>(tiles * 16 + 256);
}

int gather_qmm_affine(cudaStream_t stream, const void *x, int64_t rows, int64_t k, const uint32_t *w,
                      const void *scales, const void *biases, const int32_t *ids, int64_t experts, int64_t n,
                      int group_size, int bits, void *y, void *workspace, size_t workspace_bytes) {
    const uint32_t *ws[1] = {w};
    const void *ss[1] = {scales}, *bs[1] = {biases};
    void *ys[1] = {y};
    return gather_qmm_affine_multi(stream, x, rows, k, 1, ws, ss, bs, ids, experts, n, group_size, bits, ys, workspace, workspace_bytes);
}

int gather_qmm_affine_multi(cudaStream_t stream, const void *x, int64_t rows, int64_t k, int count, const uint32_t *const *w,
                            const void *const *scales, const void *const *biases, const int32_t *ids, int64_t experts, int64_t n,
                            int group_size, int bits, void *const *y, void *workspace, size_t workspace_bytes) {
    // Few rows per expert (decode, short batches): the problem is weight streaming, and the tensor-memory matvec
    // kernel runs one table entry of up to eight rows per CTA, so every live expert is read once.
    const bool have_ws = workspace && workspace_bytes >= gather_qmm_workspace_bytes(rows, experts) && rows < (1ll << 30);
    // (fewer than 24 rows -- one to two decode tokens of a top-8 router -- are quicker through the warp-per-output
    // kernel below: no table, less set-up per CTA; measured cross-over on the 128-expert 2048 x 768 block)
    static const int64_t tc_min_rows = [] {
        const char *v = std::getenv("LISA_GATHER_TC_MIN_ROWS");
        return v ? std::atoll(v) : 24ll;
    }();
    int32_t *tile_count = reinterpret_cast<int32_t *>(workspace);
    int32_t *tiles = tile_count ? tile_count + 64 : nullptr;  // 256 bytes further: 16-byte aligned int4 entries
    // the table kernel also zeroes the rows whose ids are outside the table, in every output
    auto build_table = [&](int bt, int64_t max_tiles) -> int {
        for (int i0 = 0; i0 < count; i0 += kTableOutputs) {
            TableOutputs out{};
            out.count = std::min(count - i0, kTableOutputs);
            for (int i = 0; i < out.count; ++i) out.y[i] = reinterpret_cast<uint16_t *>(y[i0 + i]);
            gather_tile_table_kernel<<<1 + kTableFillBlocks, kTableThreads, 0, stream>>>(ids, static_cast<int>(rows), static_cast<int>(experts), bt,
                                                                     static_cast<int>(n), static_cast<int>(max_tiles), tiles,
                                                                     tile_count, out);
            LISA_CUDA_TRY(cudaGetLastError());
            count_launch();
        }
        return LISA_OK;
    };
    if (have_ws && rows >= tc_min_rows && rows <= 8 * experts && static_cast<int64_t>(experts) * n < (1ll << 31)) {
        const int bt = qmv_tc_grouped_rows(rows, experts, k, n, group_size, bits, count);
        if (bt > 0) {
            const int64_t max_tiles = std::min<int64_t>(rows, (rows + bt - 1) / bt + experts);
            const int rc = build_table(bt, max_tiles);
            if (rc != LISA_OK) return rc;
            return qmv_tc_grouped(stream, x, rows, k, count, w, scales, biases, experts, n, group_size, bits, y, bt, tiles, tile_count,
                                  max_tiles);
        }
    }
    // Grouped tensor-core GEMM once there are enough rows to fill 16-row tiles; otherwise the warp-per-output
    // kernel.
    if (have_ws && rows >= 32 && qmm_affine_supported(rows, k, n, group_size, bits)) {
        const int bt = grouped_tile_rows(rows, experts);
        const int64_t max_tiles = std::min<int64_t>(rows, (rows + bt - 1) / bt + experts);
        if (max_tiles <= 65535) {
            const int rc = build_table(bt, max_tiles);
            if (rc != LISA_OK) return rc;
            if (count == 1)
                return qmm_affine_grouped(stream, x, rows, k, w[0], scales[0], biases[0], experts, n, group_size, bits, y[0], bt, tiles,
                                          tile_count, max_tiles);
            return qmm_affine_grouped_multi(stream, x, rows, k, count, w, scales, biases, experts, n, group_size, bits, y, bt, tiles,
                                            tile_count, max_tiles);
        }
    }
    for (int i = 0; i < count; ++i) {
        GatherParams p{};
        p.w = w[i];
        p.scales = reinterpret_cast<const uint16_t *>(scales[i]);
        p.biases = reinterpret_cast<const uint16_t *>(biases[i]);
        p.x = reinterpret_cast<const uint16_t *>(x);
        p.ids = ids;
        p.y = reinterpret_cast<uint16_t *>(y[i]);
        p.n = static_cast<int>(n);
        p.k = static_cast<int>(k);
        p.experts = static_cast<int>(experts);
        p.group_size = group_size;
        p.words_per_row = static_cast<int>(k * bits / 32);
        p.groups_per_row = static_cast<int>(k / group_size);
        p.expert_words = n * p.words_per_row;
        p.expert_groups = n * p.groups_per_row;
        const unsigned gx = static_cast<unsigned>((n + 7) / 8);
        for (int64_t base = 0; base < rows; base += 65535) {
            const unsigned gy = static_cast<unsigned>(rows - base < 65535 ? rows - base : 65535);
            if (bits == 4) gather_qmv_kernel<4><<<dim3(gx, gy), 256, 0, stream>>>(p, base);
            else gather_qmv_kernel<2><<<dim3(gx, gy), 256, 0, stream>>>(p, base);
            LISA_CUDA_TRY(cudaGetLastError());
            count_launch();
        }
    }
    return LISA_OK;
}

}  // namespace lisa
