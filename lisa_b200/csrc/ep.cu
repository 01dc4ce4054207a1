// Expert-parallel dispatch and return of routed rows over peer memory (one node, one process per GPU).
//
// The reference runs its routed experts on one device; its only multi-device hook is the contiguous
// ownership rule first = rank * (E / world) (crates/lisa-mlx/src/shaders/deepseek41/iq.metal:976-982), which
// this follows.  Around the single-device block of crates/lisa-engine/src/models/qwen4/moe.rs:352-481 it adds
// the exchange: every rank sorts its own slots by (global) expert -- which also groups them by owner -- and
//   1. publishes how many slots it has for every owner into every rank's count matrix (ep_counts),
//   2. stores the rows and their local expert ids straight into the owners' receive buffers, compactly, at the
//      offsets the count matrix implies (ep_dispatch),
//   3. after the owner has run its experts on exactly the rows it received, the owner stores every result row
//      back into the source rank's buffer at the source's own sorted position (ep_return), where the source
//      folds them with its unchanged `inverse`.
// Plain 16-byte stores to peer mappings; no TMA, no multicast, no collective library.  lisa_cuda_peer_barrier
// between the steps makes the stores visible.  The count matrix is the only thing the host reads (world x world
// ints, to size the owner's launches).
#include <cuda_runtime.h>

#include "common.cuh"
#include "kernels.h"

namespace lisa {

namespace {

constexpr int kEpMaxWorld = 8;

struct EpPeers {
    void *ptr[kEpMaxWorld];
};

__device__ __forceinline__ int ep_lower_bound(const int32_t *ids, int rows, int value) {
    int lo = 0, hi = rows;
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (__ldg(ids + mid) < value) lo = mid + 1;
        else hi = mid;
    }
    return lo;
}

// matrix[r * world + q] = slots rank r has for owner q.  One warp; lane q counts and tells every rank.
__global__ void __launch_bounds__(32) ep_counts_kernel(const int32_t *__restrict__ sorted_ids, int slots, int per, int world,
                                                       int rank, EpPeers matrices) {
    const int q = threadIdx.x;
    if (q >= world) return;
    const int c = ep_lower_bound(sorted_ids, slots, (q + 1) * per) - ep_lower_bound(sorted_ids, slots, q * per);
    for (int p = 0; p < world; ++p) reinterpret_cast<int32_t *>(matrices.ptr[p])[rank * world + q] = c;
}

// One block per sorted slot of this rank: the row goes to its owner's receive buffer.
__global__ void __launch_bounds__(256) ep_dispatch_kernel(const uint4 *__restrict__ x, const int32_t *__restrict__ sorted_ids,
                                                          const int32_t *__restrict__ token_rows, int vec_per_row, int per,
                                                          int world, int rank, const int32_t *__restrict__ matrix,
                                                          EpPeers recv_x, EpPeers recv_ids) {
    const int p = blockIdx.x;
    const int e = __ldg(sorted_ids + p);
    const int q = e / per;
    int start = 0, off = 0;  // first sorted position of owner q here; first row of this rank in q's buffer
    for (int i = 0; i < q; ++i) start += __ldg(matrix + rank * world + i);
    for (int r = 0; r < rank; ++r) off += __ldg(matrix + r * world + q);
    const int64_t j = off + (p - start);
    const uint4 *src = x + static_cast<int64_t>(__ldg(token_rows + p)) * vec_per_row;
    uint4 *dst = reinterpret_cast<uint4 *>(recv_x.ptr[q]) + j * vec_per_row;
    for (int c = threadIdx.x; c < vec_per_row; c += blockDim.x) dst[c] = __ldg(src + c);
    if (threadIdx.x == 0) reinterpret_cast<int32_t *>(recv_ids.ptr[q])[j] = e - q * per;
}

// One block per sorted received row of this owner: the result goes back to the source rank, at the position the
// row has in the source's own sorted order.
__global__ void __launch_bounds__(256) ep_return_kernel(const uint4 *__restrict__ rows, const int32_t *__restrict__ recv_index,
                                                        int vec_per_row, int world, int rank, const int32_t *__restrict__ matrix,
                                                        EpPeers back) {
    const int p = blockIdx.x;
    // the received rows are the first ones of the sorted order (ids of unused buffer rows sort last): a caller
    // that launches over its whole capacity instead of reading the count back stops here
    int received = 0;
    for (int q = 0; q < world; ++q) received += __ldg(matrix + q * world + rank);
    if (p >= received) return;
    const int j = __ldg(recv_index + p);  // index of the row in this owner's receive buffer
    int r = 0, off = 0;
    for (; r < world; ++r) {
        const int c = __ldg(matrix + r * world + rank);
        if (j < off + c) break;
        off += c;
    }
    if (r >= world) return;  // not a received row
    int start = 0;           // first sorted position of this owner on the source rank
    for (int i = 0; i < rank; ++i) start += __ldg(matrix + r * world + i);
    const uint4 *src = rows + static_cast<int64_t>(p) * vec_per_row;
    uint4 *dst = reinterpret_cast<uint4 *>(back.ptr[r]) + static_cast<int64_t>(start + (j - off)) * vec_per_row;
    for (int c = threadIdx.x; c < vec_per_row; c += blockDim.x) dst[c] = __ldg(src + c);
}

}  // namespace

int ep_counts(cudaStream_t stream, const int32_t *sorted_ids, int64_t slots, int64_t experts, int world, int rank,
              void *const *matrices) {
    EpPeers m{};
    for (int i = 0; i < world; ++i) m.ptr[i] = matrices[i];
    ep_counts_kernel<<<1, 32, 0, stream>>>(sorted_ids, static_cast<int>(slots), static_cast<int>(experts / world), world, rank, m);
    LISA_CUDA_TRY(cudaGetLastError());
    count_launch();
    return LISA_OK;
}

int ep_dispatch(cudaStream_t stream, const void *x, const int32_t *sorted_ids, const int32_t *token_rows, int64_t slots,
                int64_t hidden, int64_t experts, int world, int rank, const int32_t *matrix, void *const *recv_x,
                void *const *recv_ids) {
    EpPeers rx{}, ri{};
    for (int i = 0; i < world; ++i) {
        rx.ptr[i] = recv_x[i];
        ri.ptr[i] = recv_ids[i];
    }
    ep_dispatch_kernel<<<static_cast<unsigned>(slots), 256, 0, stream>>>(reinterpret_cast<const uint4 *>(x), sorted_ids, token_rows,
                                                                        static_cast<int>(hidden / 8), static_cast<int>(experts / world),
                                                                        world, rank, matrix, rx, ri);
    LISA_CUDA_TRY(cudaGetLastError());
    count_launch();
    return LISA_OK;
}

int ep_return(cudaStream_t stream, const void *rows, const int32_t *recv_index, int64_t count, int64_t hidden, int world, int rank,
              const int32_t *matrix, void *const *back) {
    if (count == 0) return LISA_OK;
    EpPeers b{};
    for (int i = 0; i < world; ++i) b.ptr[i] = back[i];
    ep_return_kernel<<<static_cast<unsigned>(count), 256, 0, stream>>>(reinterpret_cast<const uint4 *>(rows), recv_index,
                                                                      static_cast<int>(hidden / 8), world, rank, matrix, b);
    LISA_CUDA_TRY(cudaGetLastError());
    count_launch();
    return LISA_OK;
}

}  // namespace lisa
