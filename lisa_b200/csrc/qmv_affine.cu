// Decode GEMV for MLX affine 2-/4-bit weights: y[m, n] = sum_k x[m, k] * (scale * q + bias), m <= 8
// rows of x per launch.
//
// Replaces affine_qmv_fast / affine_qmv / affine_qmv_wide and the small-M verify tiles
// (crates/lisa-mlx/src/shaders/common/matmul/quantized.metal:762-1088, host side
// crates/lisa-mlx/src/jit/matmul.rs:186-302,1799-1869).  Same factorisation as the reference's
// qdot (quantized.metal:196-295): per 64 codes  scale * sum(q*x) + bias * sum(x), in f32, one
// rounding to bf16 at the end.
//
// Two measured facts of sm_100 shape the kernel.  (1) The SM-to-L2 path moves one request of up
// to 128 bytes every few clocks: loads that touch 32 or 64 bytes of a line reach a quarter or a
// half of HBM speed whatever the prefetch depth, so packed rows are fetched as whole 128-byte
// lines by tiled TMA copies, never by per-lane loads shaped like an MMA fragment.  (2) The
// logic/shift pipe issues 64 lanes per clock per SM, half the FMA rate, and a 4-bit stream at
// HBM speed delivers about 45 codes per clock per SM: one LOP3 per code is that pipe's whole
// budget.  Here one LOP3 lifts TWO codes into a bf16 pair (mask 0x000F000F, OR 0x43004300: each
// half is 128 + q exactly), the pairs are the A fragments of mma.sync.m16n8k16 (bf16 x bf16, f32
// accumulate, products exact), the activations are the B fragment, and the constant 128 is
// removed with sum(x):  sum(q*x) = sum((128+q)*x) - 128*sum(x).  The kernel stays a
// weight-streaming GEMV bound by HBM; the tensor pipe is nearly idle.
//
// Streaming kernel (qmv_mma_kernel): persistent CTAs, each owning a contiguous range of output
// rows walked in tiles of 16 rows.  A producer warp fills a shared-memory ring with one 3-D
// tensor copy per stage (box: 128 bytes x L lines x 16 rows, 128-byte swizzle; a ragged last
// tile uses single-row boxes at the same offsets), completing on mbarriers.  With L = 2 mod 4
// (4-bit) or L odd (2-bit) the swizzle makes the fragment-shaped shared-memory reads of the
// eight consumer warps bank-conflict free.  The consumers split the 64-code units of a stage
// between them; scales and biases of the next tile arrive through cp.async while the current
// tile computes; the activations are staged once per CTA and permuted in place into B-fragment
// order.  A tile ends with one cross-warp reduction.  Weights do not depend on the previous
// kernel in the stream, so the producer runs ahead of griddepcontrol.wait: launched with
// programmatic stream serialization, the ring of kernel i+1 fills while kernel i drains.
//
// Generic kernel (qmv_simple_kernel): one warp per output row, direct loads, plain f32 math;
// any shape.  Used for group size 32, for rows that are not whole 128-byte lines and when the
// shared-memory plan does not fit.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>

#include "common.cuh"
#include "kernels.h"
#include "tensor_map.h"

namespace lisa {

static __device__ int g_qmv_status = 0;

int qmv_device_status() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_qmv_status, sizeof(int)) != cudaSuccess) return -1;
    return v;
}
int qmv_clear_status() {
    const int zero = 0;
    return cudaMemcpyToSymbol(g_qmv_status, &zero, sizeof(int)) == cudaSuccess ? LISA_OK : LISA_ERR_CUDA;
}

constexpr int kConsumerWarps = 8;
constexpr int kConsumers = kConsumerWarps * 32;
constexpr int kQmvThreads = kConsumers + 32;  // + producer warp
constexpr int kMaxStages = 8;

struct QmvParams {
    const uint8_t *scales;
    const uint8_t *biases;
    const uint16_t *x;
    uint16_t *y;
    int n, k, m;        // m <= 8
    int mc2;            // m rounded up to even: columns kept in the cross-warp reduction
    int srow_bytes;     // (K / group_size) * 2
    int units;          // K / 64
    int ushift;         // unit >> ushift = group (0 for group 64, 1 for group 128)
    int xstride;        // bytes between rows of the staged activations (padded)
    int s_chunk;        // async-copy granularity of scale rows: 16, 8 or 4 bytes; 0: 2-byte plain copies
    int l1, n1, l2;     // k-segments of a row: n1 segments of l1 lines, then one of l2 lines (l2 may be 0)
    int stages;
    int stage_bytes;    // TR * max(l1, l2) * 128
};

// Shared-memory plan (bytes from the 1024-aligned base), shared by host and device.
// `tr` = rows per tile (16 or 32).
struct QmvSmemPlan {
    int ring, xb, xsum, sc, st, part, bars, total;
};
__host__ __device__ inline QmvSmemPlan qmv_plan(int tr, int units, int m, int mc2, int xstride, int srow_bytes,
                                                int stages, int stage_bytes) {
    QmvSmemPlan p;
    int off = 0;
    p.ring = off;            // stages x stage_bytes, every stage 1024-aligned (swizzle atom)
    off += stages * stage_bytes;
    p.xb = off;
    off += m * xstride;      // activations, permuted in place into B fragments
    off = (off + 15) & ~15;
    p.xsum = off;
    off += units * 8 * 4;    // sum(x) per unit and column
    off = (off + 15) & ~15;
    p.sc = off;              // raw [scales | biases][tr rows][srow_bytes], as fetched
    off += 2 * ((tr * srow_bytes + 15) & ~15);
    p.st = off;              // [2 buffers][tr rows][groups] of f32 {scale, bias - 128 * scale}
    off += 2 * tr * (srow_bytes / 2) * 8;
    p.part = off;            // [2 buffers][warps][tr rows][mc2 columns] partial sums
    off += 2 * kConsumerWarps * tr * mc2 * 4;
    off = (off + 15) & ~15;
    p.bars = off;            // 2 * kMaxStages mbarriers, abort flag
    off += 2 * kMaxStages * 8 + 16;
    p.total = off + 1024;    // slack to align the base
    return p;
}

// Bounded wait: once any thread of the CTA has given up, every later wait returns at once so
// that all threads still reach every barrier and the kernel ends with an error status.
__device__ __forceinline__ void wait_or_abort(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int code) {
    if (*abort_flag) return;
    if (!mbar_wait(bar, parity)) {
        *abort_flag = 1;
        atomicExch(&g_qmv_status, code);
    }
}

__device__ __forceinline__ void tma_load_3d(void *dst, const CUtensorMap *map, int c0, int c1, int c2, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

__device__ __forceinline__ void mma_bf16_16x8x16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                 uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int BITS>
struct UnitGeom {
    static constexpr int kUnitBytes = 64 * BITS / 8;   // packed bytes of 64 codes: 32 (4-bit), 16 (2-bit)
    static constexpr int kLaneBytes = kUnitBytes / 4;  // per lane of a 4-lane group: 8 / 4
    static constexpr int kUnitsPerLine = 128 / kUnitBytes;
};

// Shared-memory loads by 32-bit shared-space address (keeps the address math in 32 bits).
__device__ __forceinline__ uint2 lds_v2(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint4 lds_v4(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ float2 lds_f2(uint32_t a) {
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(a));
    return v;
}

// Eight bf16 pairs (128 + q each) from the 16 codes a lane owns, in the order the four MMAs of
// a unit consume them.  Pair i holds codes (lo_k(i), hi_k(i)) of the lane's 16 consecutive k.
template <int BITS>
__device__ __forceinline__ void decode16(uint32_t src, uint32_t m, uint32_t c, uint32_t (&r)[8]);
// (a & b) | c in one LOP3 with all three operands in registers (two immediates would cost two).
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// A constant the compiler must keep in a register.
__device__ __forceinline__ uint32_t reg_const(uint32_t v) {
    uint32_t d;
    asm volatile("mov.u32 %0, %1;" : "=r"(d) : "r"(v));
    return d;
}
template <>
__device__ __forceinline__ void decode16<4>(uint32_t src, uint32_t m, uint32_t c, uint32_t (&r)[8]) {
    const uint2 v = lds_v2(src);
    r[0] = and_or(v.x, m, c);
    r[1] = and_or(v.x >> 4, m, c);
    r[2] = and_or(v.x >> 8, m, c);
    r[3] = and_or(v.x >> 12, m, c);
    r[4] = and_or(v.y, m, c);
    r[5] = and_or(v.y >> 4, m, c);
    r[6] = and_or(v.y >> 8, m, c);
    r[7] = and_or(v.y >> 12, m, c);
}
template <>
__device__ __forceinline__ void decode16<2>(uint32_t src, uint32_t m, uint32_t c, uint32_t (&r)[8]) {
    const uint32_t v = lds_u32(src);
#pragma unroll
    for (int i = 0; i < 8; ++i) r[i] = and_or(v >> (2 * i), m, c);
}
// The lane's 16 consecutive activations (8 words of two bf16) rearranged into the pair order of
// decode16: pair i = (k_i, k_{i+4}) within each half for 4-bit, (k_i, k_{i+8}) for 2-bit.
template <int BITS>
__device__ __forceinline__ void permute_x(const uint32_t (&raw)[8], uint32_t (&xw)[8]) {
    if (BITS == 4) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            xw[4 * h + 0] = __byte_perm(raw[4 * h + 0], raw[4 * h + 2], 0x5410);
            xw[4 * h + 1] = __byte_perm(raw[4 * h + 0], raw[4 * h + 2], 0x7632);
            xw[4 * h + 2] = __byte_perm(raw[4 * h + 1], raw[4 * h + 3], 0x5410);
            xw[4 * h + 3] = __byte_perm(raw[4 * h + 1], raw[4 * h + 3], 0x7632);
        }
    } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            xw[2 * j] = __byte_perm(raw[j], raw[4 + j], 0x5410);
            xw[2 * j + 1] = __byte_perm(raw[j], raw[4 + j], 0x7632);
        }
    }
}

// Box heights of the code tensor maps, largest first; a tile is fetched with the fewest boxes.
struct QmvMaps {
    CUtensorMap a32, a16, a1;  // segments of l1 lines
    CUtensorMap b32, b16, b1;  // the last segment of l2 lines
};

template <int BITS, int TR>
__global__ void __launch_bounds__(kQmvThreads, 2)
qmv_mma_kernel(const __grid_constant__ QmvMaps maps, const QmvParams p) {
    using U = UnitGeom<BITS>;
    constexpr int NH = TR / 8;  // 8-row groups per tile: lane (g, tig) owns rows g + 8 h
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const QmvSmemPlan plan = qmv_plan(TR, p.units, p.m, p.mc2, p.xstride, p.srow_bytes, p.stages, p.stage_bytes);
    uint8_t *ring = smem + plan.ring;
    uint8_t *xb = smem + plan.xb;
    float *xsum = reinterpret_cast<float *>(smem + plan.xsum);
    uint8_t *scbuf = smem + plan.sc;
    float *part = reinterpret_cast<float *>(smem + plan.part);
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + plan.bars);
    uint64_t *empty = full + kMaxStages;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(empty + kMaxStages);
    const int sc_half = (TR * p.srow_bytes + 15) & ~15;  // bytes of one raw [TR rows] block

    // Rows of this CTA: an even split of n at single-row granularity.
    const int row_begin = static_cast<int>((static_cast<int64_t>(blockIdx.x) * p.n) / gridDim.x);
    const int row_end = static_cast<int>((static_cast<int64_t>(blockIdx.x + 1) * p.n) / gridDim.x);
    const int ntiles = (row_end - row_begin + TR - 1) / TR;
    const int nseg = p.n1 + (p.l2 > 0 ? 1 : 0);
    const int nsteps = ntiles * nseg;  // ring steps: (tile, k-segment)

    if (tid == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kConsumerWarps);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == kConsumerWarps) {
        // ---------------- producer: packed codes do not depend on the previous kernel in the stream
        if (lane == 0) {
            int issued = 0, s = 0, phase = 0, it = 0, sg = 0;
            for (int q = 0; q < nsteps; ++q) {
                if (q >= p.stages) wait_or_abort(&empty[s], phase ^ 1, abort_flag, 1);
                if (*abort_flag) break;
                const int r0 = row_begin + it * TR;
                const int rows = min(TR, row_end - r0);
                const bool first = sg < p.n1;
                const int lines = first ? p.l1 : p.l2;
                const int line0 = first ? sg * p.l1 : p.n1 * p.l1;
                uint8_t *st = ring + static_cast<size_t>(s) * p.stage_bytes;
                mbar_arrive_expect_tx(&full[s], static_cast<uint32_t>(rows * lines * 128));
                // the fewest boxes that cover `rows`: 32, then 16, then single rows, each at the
                // shared-memory offset the full box would put that row (same swizzle)
                int r = 0;
                if (TR == 32 && rows - r >= 32) {
                    tma_load_3d(st, first ? &maps.a32 : &maps.b32, 0, line0, r0, &full[s]);
                    r += 32;
                }
                if (rows - r >= 16) {
                    tma_load_3d(st + r * lines * 128, first ? &maps.a16 : &maps.b16, 0, line0, r0 + r, &full[s]);
                    r += 16;
                }
                for (; r < rows; ++r)
                    tma_load_3d(st + r * lines * 128, first ? &maps.a1 : &maps.b1, 0, line0, r0 + r, &full[s]);
                issued = q + 1;
                if (++s == p.stages) {
                    s = 0;
                    phase ^= 1;
                }
                if (++sg == nseg) {
                    sg = 0;
                    ++it;
                }
            }
            // After an abort, let copies already issued land before the CTA releases its memory.
            if (*abort_flag) {
                for (int q = max(0, issued - p.stages); q < issued; ++q)
                    mbar_wait(&full[q % p.stages], (q / p.stages) & 1, 4000000u);
            }
        }
        return;
    }

    // ---------------- consumers
    const int g = lane >> 2, tig = lane & 3;  // MMA fragment coordinates

    // Scales and biases of tile `it` are fetched raw with asynchronous copies (rows whose size allows
    // no 4-byte granularity are copied synchronously); the thread that fetched a chunk later turns
    // it into f32 pairs {scale, bias - 128 * scale}, the form the inner loop consumes.
    const int groups_row = p.srow_bytes >> 1;
    const int chunk = p.s_chunk ? p.s_chunk : 2;
    uint8_t *raw_s = scbuf, *raw_b = scbuf + sc_half;
    float2 *stbuf = reinterpret_cast<float2 *>(smem + plan.st);
    auto fetch_scales = [&](int it) {
        if (it < ntiles) {
            const int r0 = row_begin + it * TR;
            const int rows = min(TR, row_end - r0);
            const size_t off = static_cast<size_t>(r0) * p.srow_bytes;
            const int nbytes = rows * p.srow_bytes;
            for (int c = tid * chunk; c < nbytes; c += kConsumers * chunk) {
                if (p.s_chunk == 16) {
                    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(smem_u32(raw_s + c)), "l"(p.scales + off + c) : "memory");
                    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(smem_u32(raw_b + c)), "l"(p.biases + off + c) : "memory");
                } else if (p.s_chunk == 8) {
                    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_u32(raw_s + c)), "l"(p.scales + off + c) : "memory");
                    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_u32(raw_b + c)), "l"(p.biases + off + c) : "memory");
                } else if (p.s_chunk == 4) {
                    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(raw_s + c)), "l"(p.scales + off + c) : "memory");
                    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(raw_b + c)), "l"(p.biases + off + c) : "memory");
                } else {
                    *reinterpret_cast<uint16_t *>(raw_s + c) = __ldg(reinterpret_cast<const uint16_t *>(p.scales + off + c));
                    *reinterpret_cast<uint16_t *>(raw_b + c) = __ldg(reinterpret_cast<const uint16_t *>(p.biases + off + c));
                }
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    // Converts the chunks this thread fetched for tile `it` into buffer `b`; call after wait_group.
    auto convert_scales = [&](int it, int b) {
        if (it < ntiles) {
            const int r0 = row_begin + it * TR;
            const int nbytes = min(TR, row_end - r0) * p.srow_bytes;
            float2 *dst = stbuf + b * TR * groups_row;
            for (int c = tid * chunk; c < nbytes; c += kConsumers * chunk) {
                for (int e = 0; e < chunk; e += 2) {
                    const float sv = bf16_bits_to_f32(*reinterpret_cast<const uint16_t *>(raw_s + c + e));
                    const float bv = bf16_bits_to_f32(*reinterpret_cast<const uint16_t *>(raw_b + c + e));
                    dst[(c + e) >> 1] = make_float2(sv, fmaf(-128.f, sv, bv));
                }
            }
        }
    };
    auto scales_landed = [&]() { asm volatile("cp.async.wait_group 0;" ::: "memory"); };
    auto consumer_sync = [&]() { asm volatile("bar.sync 1, %0;" ::"r"(kConsumers) : "memory"); };
    fetch_scales(0);  // weights: independent of the previous kernel

    // ---- activations: produced by the previous kernel in the stream
    pdl_wait();
    {
        const int vec_per_row = p.k / 8;  // uint4 per row of x
        for (int i = tid; i < p.m * vec_per_row; i += kConsumers) {
            const int r = i / vec_per_row, c = i - r * vec_per_row;
            *reinterpret_cast<uint4 *>(xb + r * p.xstride + c * 16) =
                __ldg(reinterpret_cast<const uint4 *>(p.x + static_cast<size_t>(r) * p.k) + c);
        }
    }
    scales_landed();
    convert_scales(0, 0);
    consumer_sync();
    fetch_scales(1);
    // Permute every 16 consecutive k of x in place into B-fragment order, and sum them: one thread
    // per (unit, column, quarter of the unit); the four quarters of a unit sit in adjacent lanes.
    for (int e = tid; e < p.units * 8; e += kConsumers)
        if ((e & 7) >= p.m) xsum[e] = 0.f;  // columns that do not exist
    {
        const int items = p.units * p.m * 4;
        for (int base = 0; base < items; base += kConsumers) {
            const int item = base + tid;
            const bool ok = item < items;
            const int tq = item & 3, un = item >> 2;
            const int u = un / p.m, ncol = un - u * p.m;
            float s16 = 0.f;
            if (ok) {
                uint4 *slot = reinterpret_cast<uint4 *>(xb + ncol * p.xstride + u * 128 + tq * 32);
                const uint4 v0 = slot[0], v1 = slot[1];
                const uint32_t raw[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
                uint32_t xw[8];
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    s16 += bf16_bits_to_f32(raw[i] & 0xffffu) + __uint_as_float(raw[i] & 0xffff0000u);
                permute_x<BITS>(raw, xw);
                slot[0] = make_uint4(xw[0], xw[1], xw[2], xw[3]);
                slot[1] = make_uint4(xw[4], xw[5], xw[6], xw[7]);
            }
            s16 += __shfl_xor_sync(0xffffffffu, s16, 1);
            s16 += __shfl_xor_sync(0xffffffffu, s16, 2);
            if (ok && tq == 0) xsum[u * 8 + ncol] = s16;
        }
    }
    consumer_sync();

    // Columns beyond m read column m-1 again: their results are never stored.
    const uint32_t xlane = smem_u32(xb) + min(g, p.m - 1) * p.xstride + tig * 32;
    const uint32_t xsum_lane = smem_u32(xsum) + 8 * tig;
    const uint32_t ring32 = smem_u32(ring);
    // Unit ul = warp + 8 i of a segment starts at byte b0 + i * step of the row segment: the offset
    // inside the 128-byte line is the same for every i.
    constexpr int kStep = kConsumerWarps * U::kUnitBytes;          // 256 (4-bit) / 128 (2-bit)
    constexpr int kLineStep = kStep >> 7;                          // lines per trip
    const int b0 = warp * U::kUnitBytes + tig * U::kLaneBytes;
    const int line0 = b0 >> 7, chunk0 = (b0 >> 4) & 7, inner = b0 & 15;
    const uint32_t kmask = reg_const(BITS == 4 ? 0x000f000fu : 0x00030003u), kmagic = reg_const(0x43004300u);
    const uint32_t gstep = (kConsumerWarps >> p.ushift) * 8;
    const bool part_writer = 2 * tig < p.mc2;  // lanes whose columns take part in the reduction
    int buf = 0, s = 0, phase = 0;
    for (int it = 0; it < ntiles; ++it) {
        const int r0 = row_begin + it * TR;
        const int rows = min(TR, row_end - r0);
        // rs[2h], rs[2h+1]: (row g + 8h, col 2tig), (row g + 8h, col 2tig + 1)
        float rs[2 * NH];
#pragma unroll
        for (int i = 0; i < 2 * NH; ++i) rs[i] = 0.f;
        const uint32_t st_g = smem_u32(stbuf) + ((buf * TR + g) * groups_row) * 8;
        const uint32_t st_step = 8 * groups_row * 8;  // 8 rows further
        int ubase = 0;  // first unit of the segment
        for (int sg = 0; sg < nseg; ++sg) {
            const int lines = (sg < p.n1) ? p.l1 : p.l2;
            const int nu = lines * U::kUnitsPerLine;
            // lane (g, tig) reads rows g + 8 h of the stage; they share the swizzle key
            const uint32_t rowp = ring32 + s * p.stage_bytes + g * lines * 128 + inner;
            const int keyg = g * lines;
            const uint32_t h_off = 8 * lines * 128;
            wait_or_abort(&full[s], phase, abort_flag, 2);
            const int u0 = ubase + warp;
            uint32_t xo = xlane + u0 * 128, xso = xsum_lane + u0 * 32, go = (u0 >> p.ushift) * 8;
            int line = line0;
            for (int ul = warp; ul < nu; ul += kConsumerWarps) {
                // one unit: TR rows x 64 codes against up to 8 columns of x
                const uint32_t src = rowp + line * 128 + ((chunk0 ^ ((keyg + line) & 7)) << 4);
                const uint4 x0 = lds_v4(xo), x1 = lds_v4(xo + 16);
                const float2 xs = lds_f2(xso);
#pragma unroll
                for (int hp = 0; hp < NH / 2; ++hp) {  // one 16-row MMA tile: row groups 2hp, 2hp+1
                    if (rows > 16 * hp) {              // warp-uniform: skip MMA tiles with no rows
                        uint32_t ra[8], rb[8];
                        decode16<BITS>(src + (2 * hp) * h_off, kmask, kmagic, ra);
                        if (rows > 16 * hp + 8) {
                            decode16<BITS>(src + (2 * hp + 1) * h_off, kmask, kmagic, rb);
                        } else {
#pragma unroll
                            for (int i = 0; i < 8; ++i) rb[i] = 0;
                        }
                        float c[4] = {0.f, 0.f, 0.f, 0.f};
                        mma_bf16_16x8x16(c, ra[0], rb[0], ra[1], rb[1], x0.x, x0.y);
                        mma_bf16_16x8x16(c, ra[2], rb[2], ra[3], rb[3], x0.z, x0.w);
                        mma_bf16_16x8x16(c, ra[4], rb[4], ra[5], rb[5], x1.x, x1.y);
                        mma_bf16_16x8x16(c, ra[6], rb[6], ra[7], rb[7], x1.z, x1.w);
                        const float2 lo = lds_f2(st_g + (2 * hp) * st_step + go);      // {scale, bias - 128 scale}
                        const float2 hi = lds_f2(st_g + (2 * hp + 1) * st_step + go);
                        // scale * (c - 128 sum(x)) + bias * sum(x) == scale * c + (bias - 128 scale) * sum(x)
                        rs[4 * hp + 0] = fmaf(lo.x, c[0], fmaf(lo.y, xs.x, rs[4 * hp + 0]));
                        rs[4 * hp + 1] = fmaf(lo.x, c[1], fmaf(lo.y, xs.y, rs[4 * hp + 1]));
                        rs[4 * hp + 2] = fmaf(hi.x, c[2], fmaf(hi.y, xs.x, rs[4 * hp + 2]));
                        rs[4 * hp + 3] = fmaf(hi.x, c[3], fmaf(hi.y, xs.y, rs[4 * hp + 3]));
                    }
                }
                line += kLineStep;
                xo += kConsumerWarps * 128;
                xso += kConsumerWarps * 32;
                go += gstep;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);  // this warp is done reading the stage
            ubase += nu;
            if (++s == p.stages) {
                s = 0;
                phase ^= 1;
            }
        }
        // cross-warp reduction of the TR x mc2 outputs: part[buf][warp][row][col]
        if (part_writer) {
            float *pw = part + ((buf * kConsumerWarps + warp) * TR + g) * p.mc2 + 2 * tig;
#pragma unroll
            for (int h = 0; h < NH; ++h)
                *reinterpret_cast<float2 *>(pw + 8 * h * p.mc2) = make_float2(rs[2 * h], rs[2 * h + 1]);
        }
        scales_landed();                 // raw scales of the next tile, requested a tile ago
        convert_scales(it + 1, buf ^ 1);
        consumer_sync();
        fetch_scales(it + 2);
        for (int e = tid; e < TR * p.mc2; e += kConsumers) {
            float total = 0.f;
#pragma unroll
            for (int wi = 0; wi < kConsumerWarps; ++wi) total += part[(buf * kConsumerWarps + wi) * TR * p.mc2 + e];
            const int row = e / p.mc2, col = e - row * p.mc2;
            if (row < rows && col < p.m)
                p.y[static_cast<size_t>(col) * p.n + r0 + row] = static_cast<uint16_t>(f32_to_bf16_bits(total));
        }
        buf ^= 1;
    }
}

// ---------------------------------------------------------------------------------------
// Generic kernel: warp per output row, lanes stride over packed words, f32 math with the same
// factorisation.  Any n, any k that is a multiple of the group size, any m (grid.y).
struct SimpleParams {
    const uint8_t *w;
    const uint8_t *scales;
    const uint8_t *biases;
    const uint16_t *x;
    uint16_t *y;
    int n, k, wrow_bytes, srow_bytes, group_size;
};

template <int BITS>
__global__ void __launch_bounds__(256) qmv_simple_kernel(const SimpleParams p) {
    const int group_size = p.group_size;
    constexpr int CPW = 32 / BITS;  // codes per word
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int mrow = blockIdx.y;
    pdl_launch_dependents();
    pdl_wait();
    if (row >= p.n) return;
    const uint32_t *wr = reinterpret_cast<const uint32_t *>(p.w + static_cast<size_t>(row) * p.wrow_bytes);
    const uint16_t *sr = reinterpret_cast<const uint16_t *>(p.scales + static_cast<size_t>(row) * p.srow_bytes);
    const uint16_t *br = reinterpret_cast<const uint16_t *>(p.biases + static_cast<size_t>(row) * p.srow_bytes);
    const uint16_t *xr = p.x + static_cast<size_t>(mrow) * p.k;
    const int nwords = p.k / CPW;
    float result = 0.f;
    for (int wi = lane; wi < nwords; wi += 32) {
        const uint32_t word = __ldg(wr + wi);
        const int k0 = wi * CPW;
        const int gi = k0 / group_size;  // a word never straddles a group (group_size >= 32 >= CPW)
        float accum = 0.f, xsum = 0.f;
#pragma unroll
        for (int j = 0; j < CPW; ++j) {
            const float xv = bf16_bits_to_f32(__ldg(xr + k0 + j));
            const uint32_t qv = (word >> (j * BITS)) & ((1u << BITS) - 1u);
            accum = fmaf(xv, static_cast<float>(qv), accum);
            xsum += xv;
        }
        result = fmaf(bf16_bits_to_f32(__ldg(sr + gi)), accum, result);
        result = fmaf(bf16_bits_to_f32(__ldg(br + gi)), xsum, result);
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) result += __shfl_xor_sync(0xffffffffu, result, off);
    if (lane == 0) p.y[static_cast<size_t>(mrow) * p.n + row] = static_cast<uint16_t>(f32_to_bf16_bits(result));
}

// ---------------------------------------------------------------------------------------
// Host-side planning and launch.

// Splits `lines` (128-byte lines per packed row) into n1 segments of l1 lines plus an optional
// segment of l2 lines, all from the set of line counts whose swizzle keeps the fragment reads
// conflict free: 2 mod 4 for 4-bit (8-byte lane reads), odd for 2-bit (4-byte lane reads).
template <int BITS>
static bool split_lines(int lines, int max_lines, int &l1, int &n1, int &l2) {
    auto valid = [](int l) { return BITS == 4 ? (l % 4 == 2) : (l % 2 == 1); };
    int best_cnt = 1 << 30, best_small = -1;
    for (int a = max_lines; a >= 1; --a) {
        if (!valid(a)) continue;
        for (int cnt = lines / a; cnt >= 1; --cnt) {
            const int rem = lines - cnt * a;
            if (rem != 0 && !(valid(rem) && rem <= max_lines)) continue;
            const int total = cnt + (rem ? 1 : 0);
            const int small = rem ? std::min(a, rem) : a;  // ties: the split with the largest smallest part
            if (total < best_cnt || (total == best_cnt && small > best_small)) {
                best_cnt = total;
                best_small = small;
                l1 = a;
                n1 = cnt;
                l2 = rem;
            }
        }
    }
    return best_cnt != (1 << 30);
}

template <int BITS>
static bool plan_mma(int64_t n, int64_t k, int group_size, int m, QmvParams &p, int &tr, int &grid, int &smem) {
    if (group_size != 64 && group_size != 128) return false;
    if (k % 64 != 0 || k % group_size != 0) return false;
    const int64_t row_bytes = k * BITS / 8;
    if (row_bytes % 128 != 0) return false;  // whole lines only
    const int lines = static_cast<int>(row_bytes / 128);
    p.units = static_cast<int>(k / 64);
    p.mc2 = (m + 1) & ~1;
    p.ushift = (group_size == 128) ? 1 : 0;
    p.s_chunk = (p.srow_bytes % 16 == 0) ? 16 : (p.srow_bytes % 8 == 0) ? 8 : (p.srow_bytes % 4 == 0) ? 4 : 0;
    // rows of staged x sit 16 bytes past a multiple of 128 so that the lanes of different columns
    // hit different banks
    p.xstride = static_cast<int>(((k * 2 + 127) / 128) * 128 + 16);
    const int sms = sm_count();
    const int smem_max = max_smem_optin();
    // Two CTAs per SM when every CTA still gets more than a tile; else one.
    const int per_sm = (n >= static_cast<int64_t>(2) * sms * 24) ? 2 : 1;
    for (int ps = per_sm; ps >= 1; --ps) {
        const int64_t ctas = std::min<int64_t>((n + 15) / 16, static_cast<int64_t>(sms) * ps);
        const int64_t rows_per_cta = (n + ctas - 1) / ctas;
        // 32-row tiles halve the per-unit bookkeeping; worth it once a CTA has more than 16 rows
        for (int t : {32, 16}) {
            if (t == 32 && rows_per_cta <= 16) continue;
            const int budget = (ps == 2) ? smem_max / 2 - 1024 : smem_max;
            // stages of at most ~28 KB so that a ring of three fits beside the rest
            const int max_lines = std::max(2, std::min(14, (28 * 1024) / (t * 128)));
            if (!split_lines<BITS>(lines, max_lines, p.l1, p.n1, p.l2)) continue;
            p.stage_bytes = t * std::max(p.l1, p.l2) * 128;
            for (int stages = kMaxStages; stages >= 2; --stages) {
                if (stages > 4 && stages * p.stage_bytes > 96 * 1024) continue;  // deep rings only while small
                const QmvSmemPlan sp = qmv_plan(t, p.units, m, p.mc2, p.xstride, p.srow_bytes, stages, p.stage_bytes);
                if (sp.total <= budget) {
                    p.stages = stages;
                    smem = sp.total;
                    tr = t;
                    grid = static_cast<int>(ctas);
                    return true;
                }
            }
        }
    }
    return false;
}

static int make_code_map(CUtensorMap *map, const void *w, int64_t n, int64_t row_bytes, int lines_box, int rows_box) {
    const uint64_t dims[3] = {128, static_cast<uint64_t>(row_bytes / 128), static_cast<uint64_t>(n)};
    const uint64_t strides[2] = {128, static_cast<uint64_t>(row_bytes)};
    const uint32_t box[3] = {128, static_cast<uint32_t>(lines_box), static_cast<uint32_t>(rows_box)};
    return make_tensor_map(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, w, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

template <int BITS, int TR>
static int launch_mma(const cudaLaunchConfig_t &cfg, int smem, const QmvMaps &maps, const QmvParams &p) {
    if (smem > 48 * 1024)
        LISA_CUDA_TRY(cudaFuncSetAttribute(qmv_mma_kernel<BITS, TR>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    LISA_CUDA_TRY(cudaLaunchKernelEx(&cfg, qmv_mma_kernel<BITS, TR>, maps, p));
    count_launch();
    return LISA_OK;
}

template <int BITS>
static int qmv_dispatch(cudaStream_t stream, const void *x, int64_t m, int64_t k, const uint32_t *w,
                        const void *scales, const void *biases, int64_t n, int group_size, void *y, unsigned flags) {
    QmvParams p{};
    p.scales = reinterpret_cast<const uint8_t *>(scales);
    p.biases = reinterpret_cast<const uint8_t *>(biases);
    p.n = static_cast<int>(n);
    p.k = static_cast<int>(k);
    p.srow_bytes = static_cast<int>(k / group_size * 2);
    const int64_t row_bytes = k * BITS / 8;
    const bool pdl = (flags & LISA_FLAG_PDL) != 0;
    const bool force_simple = (flags & LISA_FLAG_FORCE_QMV_SIMPLE) != 0;
    const uint16_t *xp = reinterpret_cast<const uint16_t *>(x);
    uint16_t *yp = reinterpret_cast<uint16_t *>(y);

    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;

    QmvMaps maps;
    int maps_l1 = -1, maps_l2 = -1;
    int64_t done = 0;
    while (done < m) {
        const int64_t left = m - done;
        int mc = static_cast<int>(std::min<int64_t>(left, 8));
        int grid = 0, smem = 0, tr = 16;
        bool ok = false;
        if (!force_simple && k % 8 == 0) {
            for (; mc >= 1; mc = (mc > 1) ? (mc + 1) / 2 : 0) {
                if (plan_mma<BITS>(n, k, group_size, mc, p, tr, grid, smem)) {
                    ok = true;
                    break;
                }
            }
        }
        cudaLaunchConfig_t cfg{};
        cfg.stream = stream;
        cfg.attrs = attr;
        cfg.numAttrs = pdl ? 1 : 0;
        if (!ok) {
            // generic kernel, all remaining rows in one launch
            SimpleParams sp{};
            sp.w = reinterpret_cast<const uint8_t *>(w);
            sp.scales = p.scales;
            sp.biases = p.biases;
            sp.x = xp + done * k;
            sp.y = yp + done * n;
            sp.n = p.n;
            sp.k = p.k;
            sp.wrow_bytes = static_cast<int>(row_bytes);
            sp.srow_bytes = p.srow_bytes;
            sp.group_size = group_size;
            if (left > 65535) return fail(LISA_ERR_LIMIT, "qmv: more than 65535 rows for the generic kernel");
            cfg.gridDim = dim3(static_cast<unsigned>((n + 7) / 8), static_cast<unsigned>(left));
            cfg.blockDim = dim3(256);
            LISA_CUDA_TRY(cudaLaunchKernelEx(&cfg, qmv_simple_kernel<BITS>, sp));
            count_launch();
            return LISA_OK;
        }
        if (maps_l1 != p.l1 || maps_l2 != p.l2) {
            const int lb = p.l2 > 0 ? p.l2 : p.l1;
            int rc = make_code_map(&maps.a32, w, n, row_bytes, p.l1, 32);
            if (rc == LISA_OK) rc = make_code_map(&maps.a16, w, n, row_bytes, p.l1, 16);
            if (rc == LISA_OK) rc = make_code_map(&maps.a1, w, n, row_bytes, p.l1, 1);
            if (rc == LISA_OK) rc = make_code_map(&maps.b32, w, n, row_bytes, lb, 32);
            if (rc == LISA_OK) rc = make_code_map(&maps.b16, w, n, row_bytes, lb, 16);
            if (rc == LISA_OK) rc = make_code_map(&maps.b1, w, n, row_bytes, lb, 1);
            if (rc != LISA_OK) return rc;
            maps_l1 = p.l1;
            maps_l2 = p.l2;
        }
        p.x = xp + done * k;
        p.y = yp + done * n;
        p.m = mc;
        cfg.gridDim = dim3(grid);
        cfg.blockDim = dim3(kQmvThreads);
        cfg.dynamicSmemBytes = smem;
        const int rc = (tr == 32) ? launch_mma<BITS, 32>(cfg, smem, maps, p) : launch_mma<BITS, 16>(cfg, smem, maps, p);
        if (rc != LISA_OK) return rc;
        done += mc;
    }
    return LISA_OK;
}

// 8-bit weights (the reference's lm-head case, array_ops.rs test loop over bits 2, 4, 8;
// quantized.metal:102-107,288-292): the generic kernel, one warp per (output row, row of x), for any m.
static int qmv_simple8(cudaStream_t stream, const void *x, int64_t m, int64_t k, const uint32_t *w, const void *scales,
                       const void *biases, int64_t n, int group_size, void *y, unsigned flags) {
    SimpleParams sp{};
    sp.w = reinterpret_cast<const uint8_t *>(w);
    sp.scales = reinterpret_cast<const uint8_t *>(scales);
    sp.biases = reinterpret_cast<const uint8_t *>(biases);
    sp.n = static_cast<int>(n);
    sp.k = static_cast<int>(k);
    sp.wrow_bytes = static_cast<int>(k);
    sp.srow_bytes = static_cast<int>(k / group_size * 2);
    sp.group_size = group_size;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    for (int64_t done = 0; done < m; done += 65535) {
        const int64_t rows = std::min<int64_t>(m - done, 65535);
        sp.x = reinterpret_cast<const uint16_t *>(x) + done * k;
        sp.y = reinterpret_cast<uint16_t *>(y) + done * n;
        cudaLaunchConfig_t cfg{};
        cfg.stream = stream;
        cfg.attrs = attr;
        cfg.numAttrs = (flags & LISA_FLAG_PDL) ? 1 : 0;
        cfg.gridDim = dim3(static_cast<unsigned>((n + 7) / 8), static_cast<unsigned>(rows));
        cfg.blockDim = dim3(256);
        LISA_CUDA_TRY(cudaLaunchKernelEx(&cfg, qmv_simple_kernel<8>, sp));
        count_launch();
    }
    return LISA_OK;
}

int qmv_affine(cudaStream_t stream, const void *x, int64_t m, int64_t k, const uint32_t *w, const void *scales,
               const void *biases, int64_t n, int group_size, int bits, void *y, unsigned flags) {
    if (bits == 8) return qmv_simple8(stream, x, m, k, w, scales, biases, n, group_size, y, flags);
    if (bits == 4) return qmv_dispatch<4>(stream, x, m, k, w, scales, biases, n, group_size, y, flags);
    if (bits == 2) return qmv_dispatch<2>(stream, x, m, k, w, scales, biases, n, group_size, y, flags);
    return fail(LISA_ERR_UNSUPPORTED, "qmv: bits must be 2, 4 or 8");
}

}  // namespace lisa
