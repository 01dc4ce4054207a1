// Routing kernels around gather_qmm: top-k route, stable sort of slots by expert, row
// gather, SwiGLU and the weighted un-sort.
//
// Replaces track_moe_route (crates/lisa-mlx/src/shaders/qwen4/route.metal), the two-launch
// counting sort (crates/lisa-mlx/src/shaders/qwen4/route_counting_scatter.metal,
// crates/lisa-mlx/src/models/qwen4/kernels/moe.rs:72-77), bf16 SwiGLU
// (crates/lisa-mlx/src/shaders/common/exact_header.metal:2-11) and moe_combine without its
// shared-expert term (crates/lisa-mlx/src/shaders/qwen4/moe_combine.metal); the call order
// is that of SparseMoeBlock::forward (crates/lisa-engine/src/models/qwen4/moe.rs:352-481).
#include <cuda_runtime.h>

#include <mutex>

#include "common.cuh"
#include "kernels.h"

namespace lisa {

// ---------------------------------------------------------------- route
// One warp per token.  k rounds of "largest logit not yet taken, ties to the lowest
// expert index"; weights = softmax over the k selected logits in f32.
constexpr int kRouteMaxPerLane = 32;  // experts <= 1024

// PL: logits per lane the kernel is compiled for (the loops over a lane's experts are unrolled over registers):
// 4 serves up to 128 experts, 32 up to 1024.
template <int PL>
__global__ void __launch_bounds__(128) moe_route_kernel(const float *__restrict__ logits, int tokens, int experts,
                                                        int top_k, int32_t *__restrict__ idx,
                                                        float *__restrict__ weights) {
    const int lane = threadIdx.x & 31;
    const int token = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (token >= tokens) return;
    const float *l = logits + static_cast<int64_t>(token) * experts;
    float v[PL];
    const int per_lane = (experts + 31) / 32;
#pragma unroll
    for (int i = 0; i < PL; ++i) {
        const int e = i * 32 + lane;
        v[i] = (i < per_lane && e < experts) ? __ldg(l + e) : -INFINITY;
    }
    uint32_t taken = 0;  // bit i: this lane's i-th expert was selected
    float my_logit = 0.f;
    int my_idx = 0;
    float mx = -INFINITY;
    for (int j = 0; j < top_k; ++j) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < PL; ++i) {
            const int e = i * 32 + lane;
            const bool free_slot = i < per_lane && e < experts && !((taken >> i) & 1u);
            if (free_slot && (v[i] > best || best_e == 0x7fffffff)) {  // first free candidate or strictly larger
                best = v[i];
                best_e = e;
            }
        }
        // warp argmax with ties to the lowest index
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, off);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, off);
            const bool other_valid = oe != 0x7fffffff, mine_valid = best_e != 0x7fffffff;
            if (other_valid && (!mine_valid || ob > best || (ob == best && oe < best_e))) {
                best = ob;
                best_e = oe;
            }
        }
        if ((best_e & 31) == lane) taken |= 1u << (best_e >> 5);
        if (j == 0) mx = best;
        if (lane == j) {
            my_logit = best;
            my_idx = best_e;
        }
    }
    // softmax over the selected logits (lane j holds the j-th)
    float ex = (lane < top_k) ? expf(my_logit - mx) : 0.f;
    float sum = ex;
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    if (lane < top_k) {
        idx[static_cast<int64_t>(token) * top_k + lane] = my_idx;
        weights[static_cast<int64_t>(token) * top_k + lane] = ex / sum;
    }
}

int moe_route(cudaStream_t stream, const float *logits, int64_t tokens, int64_t experts, int top_k, int32_t *idx,
              float *weights) {
    const unsigned blocks = static_cast<unsigned>((tokens + 3) / 4);
    const int t = static_cast<int>(tokens), e = static_cast<int>(experts);
    if (experts <= 128) moe_route_kernel<4><<<blocks, 128, 0, stream>>>(logits, t, e, top_k, idx, weights);
    else if (experts <= 256) moe_route_kernel<8><<<blocks, 128, 0, stream>>>(logits, t, e, top_k, idx, weights);
    else if (experts <= 512) moe_route_kernel<16><<<blocks, 128, 0, stream>>>(logits, t, e, top_k, idx, weights);
    else moe_route_kernel<kRouteMaxPerLane><<<blocks, 128, 0, stream>>>(logits, t, e, top_k, idx, weights);
    LISA_CUDA_TRY(cudaGetLastError());
    count_launch();
    return LISA_OK;
}

// ---------------------------------------------------------------- stable counting sort
// Slots are cut into chunks of 256.  (1) per-chunk histogram -> counts[chunk][expert];
// (2) one block turns counts into start offsets (expert-major, chunk-minor);
// (3) each chunk scatters its slots in order, warp by warp, so equal experts keep their
// original order.  Workspace: counts, (chunks x experts) int32.
constexpr int kSortChunk = 256;

size_t moe_sort_workspace_bytes(int64_t slots, int64_t experts) {
    const int64_t chunks = (slots + kSortChunk - 1) / kSortChunk;
    return static_cast<size_t>(chunks * experts) * sizeof(int32_t);
}

__global__ void __launch_bounds__(kSortChunk) moe_sort_hist_kernel(const int32_t *__restrict__ idx, int slots,
                                                                   int experts, int32_t *__restrict__ counts) {
    extern __shared__ int32_t hist[];
    for (int e = threadIdx.x; e < experts; e += kSortChunk) hist[e] = 0;
    __syncthreads();
    const int i = blockIdx.x * kSortChunk + threadIdx.x;
    if (i < slots) {
        const int e = __ldg(idx + i);
        if (e >= 0 && e < experts) atomicAdd(&hist[e], 1);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += kSortChunk) counts[static_cast<int64_t>(blockIdx.x) * experts + e] = hist[e];
}

// counts[chunk][e] -> exclusive start of (e, chunk) in the sorted order.
// Slots whose id is outside [0, experts) are not sorted: the positions behind the last valid slot are filled
// here with id = experts (gather_qmm writes zeros for it) and token row 0, so that no consumer of the sorted
// arrays reads an index nobody wrote.
__global__ void __launch_bounds__(1024) moe_sort_scan_kernel(int32_t *__restrict__ counts, int chunks, int experts,
                                                             int slots, int32_t *__restrict__ sorted_ids,
                                                             int32_t *__restrict__ token_rows) {
    extern __shared__ int32_t totals[];  // experts + 1
    // exclusive scan over the chunks of every expert: one warp per expert, 128 chunks per trip (the four
    // loads of a trip are issued together: the table is read from global memory once, latency-bound)
    const int lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    for (int e = threadIdx.x >> 5; e < experts; e += nwarps) {
        int run = 0;
        for (int c0 = 0; c0 < chunks; c0 += 128) {
            int v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int c = c0 + 32 * j + lane;
                v[j] = c < chunks ? counts[static_cast<int64_t>(c) * experts + e] : 0;
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int c = c0 + 32 * j + lane;
                int inc = v[j];
#pragma unroll
                for (int off = 1; off < 32; off <<= 1) {
                    const int n = __shfl_up_sync(0xffffffffu, inc, off);
                    if (lane >= off) inc += n;
                }
                if (c < chunks) counts[static_cast<int64_t>(c) * experts + e] = run + inc - v[j];
                run += __shfl_sync(0xffffffffu, inc, 31);
            }
        }
        if (lane == 0) totals[e] = run;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < experts; ++e) {
            const int v = totals[e];
            totals[e] = run;
            run += v;
        }
        totals[experts] = run;  // slots with a valid id
    }
    __syncthreads();
    for (int i = totals[experts] + threadIdx.x; i < slots; i += blockDim.x) {
        sorted_ids[i] = experts;
        token_rows[i] = 0;
    }
    const int64_t cells = static_cast<int64_t>(chunks) * experts;
    for (int64_t i = threadIdx.x; i < cells; i += blockDim.x) counts[i] += totals[i % experts];
}

__global__ void __launch_bounds__(kSortChunk) moe_sort_scatter_kernel(const int32_t *__restrict__ idx, int slots,
                                                                      int experts, int top_k,
                                                                      const int32_t *__restrict__ counts,
                                                                      int32_t *__restrict__ sorted_ids,
                                                                      int32_t *__restrict__ token_rows,
                                                                      int32_t *__restrict__ inverse) {
    extern __shared__ int32_t next[];  // next free position per expert for this chunk
    for (int e = threadIdx.x; e < experts; e += kSortChunk) next[e] = counts[static_cast<int64_t>(blockIdx.x) * experts + e];
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int i = blockIdx.x * kSortChunk + threadIdx.x;
    const bool live = i < slots;
    const int e = live ? __ldg(idx + i) : -1;
    const bool ok = live && e >= 0 && e < experts;
    for (int wv = 0; wv < kSortChunk / 32; ++wv) {
        if (warp == wv) {
            const uint32_t peers = __match_any_sync(0xffffffffu, ok ? e : -1 - lane);
            if (ok) {
                const int rank = __popc(peers & ((1u << lane) - 1u));
                const int pos = next[e] + rank;
                sorted_ids[pos] = e;
                token_rows[pos] = i / top_k;
                inverse[i] = pos;
            } else if (live) {
                inverse[i] = -1;  // not sorted: moe_combine adds nothing for this slot
            }
            __syncwarp();
            if (ok && (peers >> lane) == 1u) next[e] += __popc(peers);  // highest lane of the group
        }
        __syncthreads();
    }
}

// Scan and scatter in one kernel, for tables small enough that every chunk's block can read all of it
// from L2 (chunks <= kPlaceChunks): block b sums, per expert, the counts of all chunks (the expert's total)
// and of the chunks before b, scans the totals over the experts, and places its 256 slots.  One launch and
// one single-block pass less than hist -> scan -> scatter.
constexpr int kPlaceChunks = 256;

__global__ void __launch_bounds__(kSortChunk) moe_sort_place_kernel(const int32_t *__restrict__ idx, int slots, int experts,
                                                                    int top_k, int chunks,
                                                                    const int32_t *__restrict__ counts,
                                                                    int32_t *__restrict__ sorted_ids,
                                                                    int32_t *__restrict__ token_rows,
                                                                    int32_t *__restrict__ inverse) {
    extern __shared__ int32_t place_sm[];
    int32_t *next = place_sm;            // experts: next free position of (expert, this chunk)
    int32_t *total = place_sm + experts;  // experts: slots of the expert over all chunks
    __shared__ int32_t valid;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int e = tid; e < experts; e += kSortChunk) next[e] = 0, total[e] = 0;
    __syncthreads();
    // column sums: thread (g, e) takes the chunks g, g + groups, ... of expert e (coalesced over e)
    const int groups = experts >= kSortChunk ? 1 : kSortChunk / experts;
    for (int e0 = 0; e0 < experts; e0 += kSortChunk) {
        const int g = experts >= kSortChunk ? 0 : tid / experts;
        const int e = experts >= kSortChunk ? e0 + tid : tid - g * experts;
        if (e < experts && g < groups) {
            int all = 0, before = 0;
            for (int c0 = g; c0 < chunks; c0 += 8 * groups) {  // eight loads in flight
                int v[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int c = c0 + j * groups;
                    v[j] = c < chunks ? __ldg(counts + static_cast<int64_t>(c) * experts + e) : 0;
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    all += v[j];
                    before += c0 + j * groups < static_cast<int>(blockIdx.x) ? v[j] : 0;
                }
            }
            if (groups == 1) {
                total[e] = all;
                next[e] = before;
            } else {
                atomicAdd(&total[e], all);
                atomicAdd(&next[e], before);
            }
        }
    }
    __syncthreads();
    // exclusive scan of the totals over the experts (warp 0, 32 experts per trip), added to next[]
    if (warp == 0) {
        int run = 0;
        for (int e0 = 0; e0 < experts; e0 += 32) {
            const int e = e0 + lane;
            const int v = e < experts ? total[e] : 0;
            int inc = v;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const int n = __shfl_up_sync(0xffffffffu, inc, off);
                if (lane >= off) inc += n;
            }
            if (e < experts) next[e] += run + inc - v;
            run += __shfl_sync(0xffffffffu, inc, 31);
        }
        if (lane == 0) valid = run;
    }
    __syncthreads();
    if (blockIdx.x == 0) {  // positions behind the last valid slot: id = experts, token row 0
        for (int i = valid + tid; i < slots; i += kSortChunk) {
            sorted_ids[i] = experts;
            token_rows[i] = 0;
        }
    }
    const int i = blockIdx.x * kSortChunk + tid;
    const bool live = i < slots;
    const int e = live ? __ldg(idx + i) : -1;
    const bool ok = live && e >= 0 && e < experts;
    for (int wv = 0; wv < kSortChunk / 32; ++wv) {
        if (warp == wv) {
            const uint32_t peers = __match_any_sync(0xffffffffu, ok ? e : -1 - lane);
            if (ok) {
                const int rank = __popc(peers & ((1u << lane) - 1u));
                const int pos = next[e] + rank;
                sorted_ids[pos] = e;
                token_rows[pos] = i / top_k;
                inverse[i] = pos;
            } else if (live) {
                inverse[i] = -1;
            }
            __syncwarp();
            if (ok && (peers >> lane) == 1u) next[e] += __popc(peers);
        }
        __syncthreads();
    }
}

static int launch_sort(cudaStream_t stream, const int32_t *idx, int64_t slots, int64_t experts, int top_k,
                       int32_t *sorted_ids, int32_t *token_rows, int32_t *inverse, int32_t *counts) {
    const int chunks = static_cast<int>((slots + kSortChunk - 1) / kSortChunk);
    const size_t esm = static_cast<size_t>(experts) * sizeof(int32_t);
    moe_sort_hist_kernel<<<chunks, kSortChunk, esm, stream>>>(idx, static_cast<int>(slots), static_cast<int>(experts), counts);
    LISA_CUDA_TRY(cudaGetLastError());
    if (chunks <= kPlaceChunks && 2 * esm <= 40 * 1024) {
        moe_sort_place_kernel<<<chunks, kSortChunk, 2 * esm, stream>>>(idx, static_cast<int>(slots), static_cast<int>(experts),
                                                                       top_k, chunks, counts, sorted_ids, token_rows, inverse);
        LISA_CUDA_TRY(cudaGetLastError());
        count_launch(2);
        return LISA_OK;
    }
    moe_sort_scan_kernel<<<1, 1024, esm + sizeof(int32_t), stream>>>(counts, chunks, static_cast<int>(experts),
                                                                      static_cast<int>(slots), sorted_ids, token_rows);
    LISA_CUDA_TRY(cudaGetLastError());
    moe_sort_scatter_kernel<<<chunks, kSortChunk, esm, stream>>>(idx, static_cast<int>(slots), static_cast<int>(experts),
                                                                 top_k, counts, sorted_ids, token_rows, inverse);
    LISA_CUDA_TRY(cudaGetLastError());
    count_launch(3);
    return LISA_OK;
}

int moe_sort(cudaStream_t stream, const int32_t *idx, int64_t slots, int64_t experts, int top_k, int32_t *sorted_ids,
             int32_t *token_rows, int32_t *inverse, void *workspace) {
    return launch_sort(stream, idx, slots, experts, top_k, sorted_ids, token_rows, inverse,
                       reinterpret_cast<int32_t *>(workspace));
}

// ---- the same sort for callers that cannot allocate: the (chunk x expert) count table lives in a
// file-scope device array instead of a caller workspace.  In host code the array's name is only a
// stand-in for the symbol; the device address comes from cudaGetSymbolAddress, once per device.
constexpr int64_t kStaticSortInts = 64 * 1024;  // 256 KiB, held by every GPU that loads the library
static __device__ __align__(256) int32_t g_sort_scratch[kStaticSortInts];
static std::mutex g_sort_scratch_mutex;
static int32_t *g_sort_scratch_ptr[64] = {nullptr};

int64_t moe_sort_static_capacity() { return kStaticSortInts; }

int moe_sort_static(cudaStream_t stream, const int32_t *idx, int64_t slots, int64_t experts, int top_k,
                    int32_t *sorted_ids, int32_t *token_rows, int32_t *inverse) {
    const int64_t chunks = (slots + kSortChunk - 1) / kSortChunk;
    if (chunks * experts > kStaticSortInts)
        return fail(LISA_ERR_LIMIT, "moe_sort_static: ceil(slots/256) * experts exceeds the built-in scratch of 65536 counters");
    int dev = 0;
    LISA_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(LISA_ERR_LIMIT, "moe_sort_static: device ordinal above 63");
    // The scratch address belongs to the CURRENT device: a stream of another GPU would hand its kernels a
    // pointer into the wrong device's copy of the array.
    if (stream != nullptr && stream != cudaStreamLegacy && stream != cudaStreamPerThread) {
        int sdev = -1;
        if (cudaStreamGetDevice(stream, &sdev) == cudaSuccess && sdev != dev)
            return fail(LISA_ERR_BAD_ARG, "moe_sort_static: the stream belongs to another device than the current one");
    }
    int32_t *counts = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_sort_scratch_mutex);
        if (!g_sort_scratch_ptr[dev]) {
            void *ptr = nullptr;
            LISA_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_sort_scratch));  // address on the current device
            g_sort_scratch_ptr[dev] = reinterpret_cast<int32_t *>(ptr);
        }
        counts = g_sort_scratch_ptr[dev];
    }
    // Every counter the scan and scatter kernels read is first written by the histogram kernel of
    // the same call, so nothing has to start at zero.
    return launch_sort(stream, idx, slots, experts, top_k, sorted_ids, token_rows, inverse, counts);
}

// ---------------------------------------------------------------- row gather
__global__ void __launch_bounds__(256) moe_gather_rows_kernel(const uint4 *__restrict__ x,
                                                              const int32_t *__restrict__ token_rows, int64_t rows,
                                                              int vec_per_row, uint4 *__restrict__ out) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= rows * vec_per_row) return;
    const int64_t r = i / vec_per_row;
    const int c = static_cast<int>(i - r * vec_per_row);
    out[i] = __ldg(x + static_cast<int64_t>(__ldg(token_rows + r)) * vec_per_row + c);
}

int moe_gather_rows(cudaStream_t stream, const void *x, const int32_t *token_rows, int64_t rows, int64_t width,
                    void *out) {
    const int vec = static_cast<int>(width / 8);
    const int64_t total = rows * vec;
    moe_gather_rows_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(
        reinterpret_cast<const uint4 *>(x), token_rows, rows, vec, reinterpret_cast<uint4 *>(out));
    LISA_CUDA_TRY(cudaGetLastError());
    count_launch();
    return LISA_OK;
}

// ---------------------------------------------------------------- SwiGLU
__device__ __forceinline__ float round_bf16(float v) { return bf16_bits_to_f32(f32_to_bf16_bits(v)); }

// act = bf16(silu * u), silu = bf16(g * s), s = bf16(sigmoid(g)) evaluated as 1 / (1 + exp(|g|)) mirrored by sign
__device__ __forceinline__ uint16_t swiglu_bits(uint16_t gb, uint16_t ub) {
    const float g = bf16_bits_to_f32(gb), u = bf16_bits_to_f32(ub);
    const float y = 1.0f / (1.0f + expf(fabsf(g)));
    const float s = round_bf16(g < 0.f ? y : 1.0f - y);
    const float silu = round_bf16(g * s);
    return static_cast<uint16_t>(f32_to_bf16_bits(silu * u));
}

__global__ void __launch_bounds__(256) moe_swiglu_kernel(const uint16_t *__restrict__ gate,
                                                         const uint16_t *__restrict__ up, int64_t count,
                                                         uint16_t *__restrict__ act) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= count) return;
    act[i] = swiglu_bits(__ldg(gate + i), __ldg(up + i));
}

// Eight elements per thread (16-byte loads and stores); count8 = count / 8.
__global__ void __launch_bounds__(256) moe_swiglu8_kernel(const uint4 *__restrict__ gate, const uint4 *__restrict__ up,
                                                          int64_t count8, uint4 *__restrict__ act) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= count8) return;
    const uint4 g = __ldg(gate + i), u = __ldg(up + i);
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
        o[j] = static_cast<uint32_t>(swiglu_bits(static_cast<uint16_t>(gw[j] & 0xffffu), static_cast<uint16_t>(uw[j] & 0xffffu))) |
               (static_cast<uint32_t>(swiglu_bits(static_cast<uint16_t>(gw[j] >> 16), static_cast<uint16_t>(uw[j] >> 16))) << 16);
    act[i] = make_uint4(o[0], o[1], o[2], o[3]);
}

int moe_swiglu(cudaStream_t stream, const void *gate, const void *up, int64_t count, void *act) {
    const uint16_t *g16 = reinterpret_cast<const uint16_t *>(gate), *u16 = reinterpret_cast<const uint16_t *>(up);
    uint16_t *a16 = reinterpret_cast<uint16_t *>(act);
    int64_t done = 0;
    if (aligned16(gate) && aligned16(up) && aligned16(act) && count >= 8) {
        const int64_t count8 = count / 8;
        moe_swiglu8_kernel<<<static_cast<unsigned>((count8 + 255) / 256), 256, 0, stream>>>(
            reinterpret_cast<const uint4 *>(gate), reinterpret_cast<const uint4 *>(up), count8, reinterpret_cast<uint4 *>(act));
        LISA_CUDA_TRY(cudaGetLastError());
        count_launch();
        done = count8 * 8;
    }
    if (done < count) {
        moe_swiglu_kernel<<<static_cast<unsigned>((count - done + 255) / 256), 256, 0, stream>>>(g16 + done, u16 + done,
                                                                                                count - done, a16 + done);
        LISA_CUDA_TRY(cudaGetLastError());
        count_launch();
    }
    return LISA_OK;
}

// ---------------------------------------------------------------- combine
// out[t, h] = bf16( fold_j f32(down[inverse[t*k + j], h]) * w[t, j] ), fold order of
// mlx_colsum_small_f32 (exact_header.metal:12-24).
__global__ void __launch_bounds__(256) moe_combine_kernel(const uint16_t *__restrict__ down,
                                                          const float *__restrict__ weights,
                                                          const int32_t *__restrict__ inverse, int64_t tokens,
                                                          int top_k, int64_t hidden, uint16_t *__restrict__ out) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= tokens * hidden) return;
    const int64_t t = i / hidden, h = i - t * hidden;
    const int ty = top_k < 8 ? top_k : 8;
    float part[8];
    for (int y = 0; y < ty; ++y) {
        float acc = 0.f;
        for (int rr = y; rr < top_k; rr += ty) {
            const int64_t row = __ldg(inverse + t * top_k + rr);
            // a slot that was not sorted (inverse < 0: its expert id was out of range or not owned) adds zero
            const float r = row < 0 ? 0.f : bf16_bits_to_f32(__ldg(down + row * hidden + h)) * __ldg(weights + t * top_k + rr);
            acc = r + acc;
        }
        part[y] = acc;
    }
    float total = part[0];
    for (int j = 1; j < ty; ++j) total = part[j] + total;
    out[i] = static_cast<uint16_t>(f32_to_bf16_bits(total));
}

// The same fold for eight consecutive h per thread (hidden a multiple of 8, 16-byte rows): one 16-byte load
// per slot instead of eight 2-byte ones; every element keeps its own sum in the same order.
__global__ void __launch_bounds__(256) moe_combine8_kernel(const uint4 *__restrict__ down, const float *__restrict__ weights,
                                                           const int32_t *__restrict__ inverse, int64_t tokens, int top_k,
                                                           int64_t hidden8, uint4 *__restrict__ out) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= tokens * hidden8) return;
    const int64_t t = i / hidden8, h8 = i - t * hidden8;
    if (top_k == 8) {
        // the usual router: the eight slot rows are fetched together, then folded in the same order as below
        // (part[y] = x * w with one rounding; total = part[0], total = part[y] + total)
        int64_t row[8];
        float w[8];
        uint4 v[8];
#pragma unroll
        for (int y = 0; y < 8; ++y) {
            row[y] = __ldg(inverse + t * 8 + y);
            w[y] = __ldg(weights + t * 8 + y);
        }
#pragma unroll
        for (int y = 0; y < 8; ++y) v[y] = row[y] < 0 ? make_uint4(0, 0, 0, 0) : __ldg(down + row[y] * hidden8 + h8);
        float tot[8];
#pragma unroll
        for (int y = 0; y < 8; ++y) {
            const uint32_t vw[4] = {v[y].x, v[y].y, v[y].z, v[y].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                // (+ 0: the one-term partial sum of the general fold, which turns -0 into +0)
                const float p0 = __fadd_rn(__fmul_rn(bf16_bits_to_f32(vw[e] & 0xffffu), w[y]), 0.f);
                const float p1 = __fadd_rn(__fmul_rn(__uint_as_float(vw[e] & 0xffff0000u), w[y]), 0.f);
                tot[2 * e] = (y == 0) ? p0 : __fadd_rn(p0, tot[2 * e]);
                tot[2 * e + 1] = (y == 0) ? p1 : __fadd_rn(p1, tot[2 * e + 1]);
            }
        }
        uint32_t o8[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) o8[e] = f32_to_bf16_bits(tot[2 * e]) | (f32_to_bf16_bits(tot[2 * e + 1]) << 16);
        out[i] = make_uint4(o8[0], o8[1], o8[2], o8[3]);
        return;
    }
    const int ty = top_k < 8 ? top_k : 8;
    float total[8];
    for (int y = 0; y < ty; ++y) {
        float acc[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = 0.f;
        for (int rr = y; rr < top_k; rr += ty) {
            const int64_t row = __ldg(inverse + t * top_k + rr);
            const float w = __ldg(weights + t * top_k + rr);
            const uint4 v = row < 0 ? make_uint4(0, 0, 0, 0) : __ldg(down + row * hidden8 + h8);
            const uint32_t vw[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                acc[2 * e] = bf16_bits_to_f32(vw[e] & 0xffffu) * w + acc[2 * e];
                acc[2 * e + 1] = __uint_as_float(vw[e] & 0xffff0000u) * w + acc[2 * e + 1];
            }
        }
        // total = part[0]; total = part[j] + total
#pragma unroll
        for (int e = 0; e < 8; ++e) total[e] = (y == 0) ? acc[e] : acc[e] + total[e];
    }
    uint32_t o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) o[e] = f32_to_bf16_bits(total[2 * e]) | (f32_to_bf16_bits(total[2 * e + 1]) << 16);
    out[i] = make_uint4(o[0], o[1], o[2], o[3]);
}

int moe_combine(cudaStream_t stream, const void *down_sorted, const float *weights, const int32_t *inverse,
                int64_t tokens, int top_k, int64_t hidden, void *out) {
    const int64_t total = tokens * hidden;
    if (hidden % 8 == 0 && aligned16(down_sorted) && aligned16(out)) {
        const int64_t total8 = total / 8;
        moe_combine8_kernel<<<static_cast<unsigned>((total8 + 255) / 256), 256, 0, stream>>>(
            reinterpret_cast<const uint4 *>(down_sorted), weights, inverse, tokens, top_k, hidden / 8, reinterpret_cast<uint4 *>(out));
        LISA_CUDA_TRY(cudaGetLastError());
        count_launch();
        return LISA_OK;
    }
    moe_combine_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(
        reinterpret_cast<const uint16_t *>(down_sorted), weights, inverse, tokens, top_k, hidden,
        reinterpret_cast<uint16_t *>(out));
    LISA_CUDA_TRY(cudaGetLastError());
    count_launch();
    return LISA_OK;
}

}  // namespace lisa
