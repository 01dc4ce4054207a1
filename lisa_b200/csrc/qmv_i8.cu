// Decode GEMV for MLX affine 2-/4-bit weights, group size 64, on the integer path of mma.sync:
//   y[m, n] = sum_k x[m, k] * (scale * q + bias),  m <= 8 rows of x per pass over the weights.
//
// Same operator as qmv_affine.cu and qmv_tc.cu (replaces affine_qmv_fast / affine_qmv_wide,
// crates/lisa-mlx/src/shaders/common/matmul/quantized.metal:762-1088) and the reference's own factorisation
// (qdot, quantized.metal:196-295): per 64 codes  scale * sum(q*x) + bias * sum(x)  in f32, one rounding to
// bf16 at the end.
//
// A weight-streaming kernel: every packed byte is read once from HBM, and the budget is instructions per
// code.  The codes stay integers.  `w & 0x0F0F0F0F` and `(w >> 4) & 0x0F0F0F0F` turn a packed word into two
// words of four u8 codes (2-bit: four masks of 0x03030303), which are A fragments of
// mma.sync.m16n8k32 (u8 x s8 -> s32) as they are: 16 weight rows x 32 codes per instruction, K in any
// order as long as the activations are stored in the same order.  The activations become integers per
// (token, 64-k group): with E the exponent of the group's largest magnitude, x * 2^(13-E) is rounded to an
// integer below 2^14 and split into two signed bytes, x_int = 256 * hi + lo; column 2t of the B operand is
// the hi plane of token t, column 2t+1 its lo plane (four tokens per MMA, a second set of columns for
// tokens 4..7).  A bf16 value has 8 significant bits: every element within 2^-6 of the group's maximum is
// exact, the rest is rounded to 2^-14 of that maximum.  Products and sums are exact in s32; per (row,
// group, token) the epilogue adds  scale * 2^(E-13) * (256 * D_hi + D_lo) + bias * sum(x)  in f32.
// A group whose largest element towers over the rest (a massive-activation channel) would leave the rest
// with a coarse grid.  The conversion therefore works on 22-bit integers, x_int22 = 65536 p0 + 256 p1 + p2,
// keeps (p0, p1) as the two planes above and flags a group when the dropped bytes, sum|p2|, exceed 2^-12 of
// sum|x_int22| without its largest element; flagged groups (none among Gaussian activations: the largest
// element must be about ten times the typical one) run two more MMAs on the p2 plane, which makes every element within 2^-14 of the
// maximum exact and bounds the rest by 2^-22 of it.
//
// Structure: persistent CTAs own a contiguous range of output rows (even split at single-row granularity)
// and walk it in tiles of up to 64 rows.  A producer warp streams the packed rows through a shared-memory ring
// with tiled TMA copies (one box of 128 bytes x rows per 128-byte line, 128-byte swizzle, no multicast; a
// ragged last tile uses 32- and 16-row boxes and single-row boxes at the same offsets) and the tile's scales
// and biases (contiguous in memory) with two bulk copies.  The eight consumer warps are (16-row group of the
// tile, quad-warp) pairs: a warp keeps its 16 rows for the whole kernel and takes one quad (four 64-code
// units, 256 codes) of every 16 KiB ring stage; lane (g, tig) owns two rows of the group and the 16 codes
// 16*tig .. 16*tig+15 of each unit.  With one token the eight MMA columns hold four units side by side
// (column = (unit, byte plane); a unit's B operand is zero outside its own columns), so a quad is eight MMAs
// into one accumulator tile and one f32 step per lane; two tokens share a tile between two units, four and
// more take one unit per tile.  A lane sums by unit class (unit index mod 4) and the classes are added in the
// same tree, (c0 + c1) + (c2 + c3), for every token count, then the quad-warps in order: a row's result does
// not depend on m or on the row's position (it does depend on the tile height of the launch).  Packed
// weights, scales and biases do not depend on the previous kernel in the stream, so the producer runs ahead of
// griddepcontrol.wait: launched with programmatic stream serialization, the ring of kernel i+1 fills while
// kernel i computes.
//
// Measured on B200 against the tensor-memory kernel (qmv_tc.cu), per launch in a dependent chain, one token:
// q|k|v 8.1 us (6.1), o 5.3 (5.2), gate|up 12.3 (10.8), down 10.0 (8.0); 38912 x 2560: 19.8 (21.0).  Staging
// the activations (22-bit integers, three planes) costs 1.4 us at k = 2560 and 4.4 us at k = 9728 after
// griddepcontrol.wait, which is why the tensor-memory kernel stays the default where both apply.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>

#include "common.cuh"
#include "kernels.h"
#include "tensor_map.h"

namespace lisa {

static __device__ int g_qmv_i8_status = 0;

int qmv_i8_device_status() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_qmv_i8_status, sizeof(int)) != cudaSuccess) return -1;
    return v;
}
int qmv_i8_clear_status() {
    const int zero = 0;
    return cudaMemcpyToSymbol(g_qmv_i8_status, &zero, sizeof(int)) == cudaSuccess ? LISA_OK : LISA_ERR_CUDA;
}

namespace {

constexpr int kNW = 8;                       // consumer warps
constexpr int kConsumersI8 = kNW * 32;
constexpr int kThreadsI8 = kConsumersI8 + 32;  // + producer warp
constexpr int kTR = 64;                      // rows per tile: up to four 16-row MMA tiles
constexpr int kMaxStagesI8 = 8;
constexpr int kMaxSegI8 = 3;                 // sibling linears of one launch
constexpr int kXI = 4;                       // activation items a thread has in flight while staging x

struct I8Seg {
    const uint8_t *scales;   // bf16 [n, groups]
    const uint8_t *biases;
    uint16_t *out[8];        // row r of this linear is column col0 + r of every out[i] (leading dimension ldy)
    int n, cta0, ctas, ldy, col0;
};
struct I8Params {
    const uint16_t *x;
    int k, m;
    int groups;              // k / 64 = units per row
    int rows_cap;            // rows of the tallest tile of the launch, rounded up to 16 (<= 64): sizes the buffers
    int l1, n1, l2;          // k-segments of a row: n1 ring stages of l1 lines, then one of l2 lines (may be 0)
    int stages, stage_bytes;
    int nsb;                 // buffers for the scales and biases of a tile: 1 or 2
    int nseg, nout;
    I8Seg seg[kMaxSegI8];
};
struct I8Maps {
    CUtensorMap m[kMaxSegI8][4];  // per linear: boxes of 64, 32, 16 and 1 rows
};

// Shared-memory plan, bytes from the 1024-aligned base.
struct I8Plan {
    int ring, sb, sb_half, sb_bytes, xq, xq3, xflag, xs, part, bars, total;
};
__host__ __device__ inline I8Plan i8_plan(int groups, int m, int rows_cap, int stages, int stage_bytes, int nsb) {
    I8Plan p;
    int off = 0;
    p.ring = off;
    off += stages * stage_bytes;
    p.sb = off;                               // [nsb][scales | biases][rows_cap][groups] bf16, as in memory
    p.sb_half = rows_cap * groups * 2;
    p.sb_bytes = 2 * p.sb_half;
    off += nsb * p.sb_bytes;
    p.xq = off;                               // [unit][2m columns][4 tig][16 bytes] activation bytes in B-fragment order
    off += groups * 2 * m * 64;
    p.xq3 = off;                              // [unit][m columns][4 tig][16 bytes] third byte plane (flagged units)
    off += groups * m * 64;
    p.xflag = off;                            // [unit][m] non-zero: the token's group needs the third plane
    off += groups * m * 4;
    p.xs = off;                               // [unit][m] {2^(E-13), sum(x)} f32 pairs
    off += groups * m * 8;
    p.part = off;                             // [2][quad-warps of a row group][m][rows_cap] f32 partial sums
    off += 2 * (kNW * 16 / rows_cap) * m * rows_cap * 4;
    off = (off + 15) & ~15;
    p.bars = off;                             // 2 * kMaxStagesI8 + 4 mbarriers, abort flag
    off += (2 * kMaxStagesI8 + 4) * 8 + 16;
    p.total = off + 1024;                     // slack to align the base
    return p;
}

// Bounded waits.  Once any thread of the CTA has given up, every later wait returns at once, so that all
// threads still reach every barrier and the kernel ends with an error status instead of hanging.
__device__ __forceinline__ void i8_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int code) {
    if (*abort_flag) return;
    for (int i = 0; i < 64; ++i)
        if (mbar_try_wait(bar, parity)) return;
    // a wait that lasts (the ring is empty while the previous kernel of the stream still runs): sleep
    // between polls, give up after a few seconds
    if (!mbar_wait_relaxed(bar, parity, 32, 1u << 25)) {
        *abort_flag = 1;
        atomicExch(&g_qmv_i8_status, code);
    }
}

__device__ __forceinline__ void i8_tma_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint2 i8_lds_v2(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t i8_lds_u32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t i8_lds_u16(uint32_t a) {
    uint32_t v;
    asm volatile("{ .reg .b16 t; ld.shared.u16 t, [%1]; cvt.u32.u16 %0, t; }" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint4 i8_lds_v4(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ float2 i8_lds_f2(uint32_t a) {
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(a));
    return v;
}
template <int N>
struct I8C {
    static constexpr int value = N;
};

// MP: tokens per pass rounded up to a power of two (1, 2, 4, 8).  The eight columns of an MMA hold GS = 4 / min(MP, 4)
// consecutive 64-code units side by side (column = (unit slot, token, byte plane); the B operand of a unit is
// zero outside its own slot), so one accumulator tile serves GS units and the f32 part runs once per GS units:
// for one token, once per 256 codes and 16 rows.  MP = 8 takes a second B operand for tokens 4..7.
template <int BITS, int MP>
__global__ void __launch_bounds__(kThreadsI8, 2)
qmv_i8_kernel(const __grid_constant__ I8Maps maps, const __grid_constant__ I8Params p) {
    constexpr int UPL = 128 * 8 / BITS / 64;   // 64-code units per 128-byte line: 4 (4-bit) / 8 (2-bit)
    constexpr int QPL = UPL / 4;               // quads (four units, 256 codes) per line: 1 / 2
    constexpr int QPW = QPL;                   // quads a warp takes per stage: a stage is one line per quad-warp
    constexpr int NSET = (MP == 8) ? 2 : 1;
    constexpr int MPC = (MP == 8) ? 4 : MP;    // tokens per B operand
    constexpr int GS = 4 / MPC;                // units per accumulator tile
    constexpr int ND = 4 / GS;                 // accumulator tiles per quad
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const I8Plan plan = i8_plan(p.groups, p.m, p.rows_cap, p.stages, p.stage_bytes, p.nsb);
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + plan.bars);
    uint64_t *empty = full + kMaxStagesI8;
    uint64_t *sfull = empty + kMaxStagesI8;   // [2]
    uint64_t *sempty = sfull + 2;             // [2]
    volatile int *abort_flag = reinterpret_cast<volatile int *>(sempty + 2);

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);  // warp-uniform for the compiler too

    // the linear this CTA belongs to (one, unless the launch is the sibling form) and its rows
    int si = 0;
    if (p.nseg > 1 && static_cast<int>(blockIdx.x) >= p.seg[1].cta0) si = 1;
    if (p.nseg > 2 && static_cast<int>(blockIdx.x) >= p.seg[2].cta0) si = 2;
    const I8Seg &sg = p.seg[si];
    const int cta = static_cast<int>(blockIdx.x) - sg.cta0;
    const int row_begin = static_cast<int>((static_cast<int64_t>(cta) * sg.n) / sg.ctas);
    const int row_end = static_cast<int>((static_cast<int64_t>(cta + 1) * sg.n) / sg.ctas);
    const int ntiles = (row_end - row_begin + kTR - 1) / kTR;
    const int nkseg = p.n1 + (p.l2 > 0 ? 1 : 0);
    const int srow = p.groups * 2;            // bytes of a row of scales
    const int line_box = p.rows_cap * 128;    // bytes of one 128-byte line of a tile in the ring

    if (tid == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kNW);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&sfull[b], 1);
            mbar_init(&sempty[b], kNW);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == kNW) {
        // ---------------- producer: nothing it reads depends on the previous kernel in the stream.  The whole
        // warp runs the loop (waits and counters stay warp-uniform); an elected lane arms the barrier, lane l
        // issues the copies of line l of the stage.
        const CUtensorMap *m64 = &maps.m[si][0], *m32 = &maps.m[si][1], *m16 = &maps.m[si][2], *m1 = &maps.m[si][3];
        if (lane < 4) asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&maps.m[si][lane])) : "memory");
        const uint32_t ring32 = smem_u32(smem + plan.ring);
        int s = 0, phase = 0, q = 0;
        bool ok = true;
        for (int it = 0; it < ntiles && ok; ++it) {
            const int r0 = row_begin + it * kTR;
            const int rows = min(kTR, row_end - r0);
            {
                const int b = it % p.nsb, use = it / p.nsb;
                if (use > 0) i8_wait(&sempty[b], (use - 1) & 1, abort_flag, 1);
                if (*abort_flag) break;
                if (elect_one()) {
                    uint8_t *dst = smem + plan.sb + b * plan.sb_bytes;
                    const uint32_t bytes = static_cast<uint32_t>(rows * srow);
                    mbar_arrive_expect_tx(&sfull[b], 2 * bytes);
                    bulk_g2s(dst, sg.scales + static_cast<size_t>(r0) * srow, bytes, &sfull[b]);
                    bulk_g2s(dst + plan.sb_half, sg.biases + static_cast<size_t>(r0) * srow, bytes, &sfull[b]);
                }
                __syncwarp();
            }
            for (int ks = 0; ks < nkseg; ++ks, ++q) {
                if (q >= p.stages) i8_wait(&empty[s], phase ^ 1, abort_flag, 2);
                if (*abort_flag) {
                    ok = false;
                    break;
                }
                const bool first = ks < p.n1;
                const int lines = first ? p.l1 : p.l2;
                const int line0 = first ? ks * p.l1 : p.n1 * p.l1;
                if (elect_one()) mbar_arrive_expect_tx(&full[s], static_cast<uint32_t>(rows * lines * 128));
                __syncwarp();
                for (int l = lane; l < lines; l += 32) {
                    const uint32_t dst = ring32 + s * p.stage_bytes + l * line_box;
                    const int cx = (line0 + l) * 128;
                    int r = 0;
                    if (rows == kTR) {
                        i8_tma_2d(dst, m64, cx, r0, &full[s]);
                        r = kTR;
                    }
                    if (rows - r >= 32) {
                        i8_tma_2d(dst + r * 128, m32, cx, r0 + r, &full[s]);
                        r += 32;
                    }
                    if (rows - r >= 16) {
                        i8_tma_2d(dst + r * 128, m16, cx, r0 + r, &full[s]);
                        r += 16;
                    }
                    for (; r < rows; ++r) i8_tma_2d(dst + r * 128, m1, cx, r0 + r, &full[s]);
                }
                __syncwarp();
                if (++s == p.stages) {
                    s = 0;
                    phase ^= 1;
                }
            }
        }
        // after an abort, let the copies already issued land before the CTA gives its memory back
        if (*abort_flag && lane == 0) {
            for (int qq = max(0, q - p.stages); qq < q; ++qq) mbar_wait(&full[qq % p.stages], (qq / p.stages) & 1, 4000000u);
            mbar_wait(&sfull[0], 0, 1000000u);
            mbar_wait(&sfull[1], 0, 1000000u);
        }
        return;
    }

    // ---------------- consumers
    const int g = lane >> 2, tig = lane & 3;
    const int m = p.m;
    const int ncols = 2 * m;
    const int rcap = p.rows_cap;
    const uint32_t xq32 = smem_u32(smem + plan.xq), xs32 = smem_u32(smem + plan.xs), xq332 = smem_u32(smem + plan.xq3);
    int *xflag = reinterpret_cast<int *>(smem + plan.xflag);
    float *part = reinterpret_cast<float *>(smem + plan.part);
    auto consumer_sync = [&]() { asm volatile("bar.sync 1, %0;" ::"r"(kConsumersI8) : "memory"); };

    pdl_wait();  // the activations come from the previous kernel in the stream
    {
        // One item = 8 consecutive activations of one (token, unit): loaded, turned into integer bytes in the K
        // order of the unpacked codes, stored in B-fragment order.  The eight items of a (token, unit) sit in
        // adjacent lanes and share the group's exponent and sum through shuffles.  A thread has kXI loads in
        // flight: this runs after griddepcontrol.wait, on the critical path of the launch.
        const int items = m * p.groups * 8;
        for (int base = 0; base < items; base += kConsumersI8 * kXI) {
            uint4 vv[kXI];
#pragma unroll
            for (int jj = 0; jj < kXI; ++jj) {
                const int item = base + jj * kConsumersI8 + tid;
                vv[jj] = make_uint4(0, 0, 0, 0);
                if (item < items) {
                    const int tu = item >> 3;
                    const int t = tu / p.groups, u = tu - t * p.groups;
                    vv[jj] = __ldg(reinterpret_cast<const uint4 *>(p.x + static_cast<size_t>(t) * p.k + u * 64 + (item & 7) * 8));
                }
            }
#pragma unroll
            for (int jj = 0; jj < kXI; ++jj) {
                const int item = base + jj * kConsumersI8 + tid;
                if (base + jj * kConsumersI8 >= items) break;  // uniform
                const bool in = item < items;
                const int p8 = item & 7, tu = item >> 3;
                const int t = in ? tu / p.groups : 0, u = in ? tu - t * p.groups : 0;
                const uint32_t r[4] = {vv[jj].x, vv[jj].y, vv[jj].z, vv[jj].w};
                float xf[8];
                float s = 0.f;
                uint32_t amax = 0;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    xf[2 * i] = bf16_bits_to_f32(r[i] & 0xffffu);
                    xf[2 * i + 1] = __uint_as_float(r[i] & 0xffff0000u);
                    s += xf[2 * i] + xf[2 * i + 1];
                    amax = max(amax, max(r[i] & 0x7fffu, (r[i] >> 16) & 0x7fffu));
                }
#pragma unroll
                for (int off = 1; off < 8; off <<= 1) {
                    s += __shfl_xor_sync(0xffffffffu, s, off);
                    amax = max(amax, __shfl_xor_sync(0xffffffffu, amax, off));
                }
                // E: biased exponent of the group's largest magnitude.  Groups below 2^-105 count as zero; an
                // infinity or NaN makes the group's factor NaN.
                const uint32_t e = amax >> 7;
                const bool live = e >= 22u && e < 255u;
                const float up = __uint_as_float((275u - e) << 23);  // 2^(21 - (E - 127))
                int hb[8], lb[8], tb[8];
                int sabs = 0, mabs = 0, sp2 = 0;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int xi = live ? __float2int_rn(xf[i] * up) : 0;  // |xi| < 2^22
                    const int r1 = (xi + 128) >> 8;                        // xi = 256 r1 + p2
                    tb[i] = xi - (r1 << 8);
                    hb[i] = (r1 + 128) >> 8;                               // r1 = 256 h + l; three signed bytes
                    lb[i] = r1 - (hb[i] << 8);
                    sabs += abs(xi);
                    mabs = max(mabs, abs(xi));
                    sp2 += abs(tb[i]);
                }
#pragma unroll
                for (int off = 1; off < 8; off <<= 1) {
                    sabs += __shfl_xor_sync(0xffffffffu, sabs, off);
                    mabs = max(mabs, __shfl_xor_sync(0xffffffffu, mabs, off));
                    sp2 += __shfl_xor_sync(0xffffffffu, sp2, off);
                }
                const bool need3 = sp2 * 4096 > sabs - mabs;  // the dropped bytes against the group without its largest element
                if (in) {
                    // element kk = 8 * (p8 & 1) + i of lane-group tg = p8 >> 1 of the unit
                    const int tg = p8 >> 1, odd = p8 & 1;
                    const uint32_t hi_at = xq32 + ((u * ncols + 2 * t) * 4 + tg) * 16, lo_at = hi_at + 64;
                    const uint32_t p2_at = xq332 + ((u * m + t) * 4 + tg) * 16;
                    if (BITS == 4) {
                        // word 0/1: even codes of packed word 0/1; word 2/3: odd codes
                        uint32_t he = 0, ho = 0, le = 0, lo = 0, te = 0, to = 0;
#pragma unroll
                        for (int i = 0; i < 8; i += 2) {
                            he |= (static_cast<uint32_t>(hb[i]) & 0xffu) << (4 * i);
                            ho |= (static_cast<uint32_t>(hb[i + 1]) & 0xffu) << (4 * i);
                            le |= (static_cast<uint32_t>(lb[i]) & 0xffu) << (4 * i);
                            lo |= (static_cast<uint32_t>(lb[i + 1]) & 0xffu) << (4 * i);
                            te |= (static_cast<uint32_t>(tb[i]) & 0xffu) << (4 * i);
                            to |= (static_cast<uint32_t>(tb[i + 1]) & 0xffu) << (4 * i);
                        }
                        asm volatile("st.shared.u32 [%0], %1;" ::"r"(hi_at + odd * 4), "r"(he) : "memory");
                        asm volatile("st.shared.u32 [%0], %1;" ::"r"(hi_at + 8 + odd * 4), "r"(ho) : "memory");
                        asm volatile("st.shared.u32 [%0], %1;" ::"r"(lo_at + odd * 4), "r"(le) : "memory");
                        asm volatile("st.shared.u32 [%0], %1;" ::"r"(lo_at + 8 + odd * 4), "r"(lo) : "memory");
                        asm volatile("st.shared.u32 [%0], %1;" ::"r"(p2_at + odd * 4), "r"(te) : "memory");
                        asm volatile("st.shared.u32 [%0], %1;" ::"r"(p2_at + 8 + odd * 4), "r"(to) : "memory");
                    } else {
                        // word j holds codes j, j+4, j+8, j+12 of the lane-group's packed word: this item supplies
                        // bytes 2*odd and 2*odd+1 of every word
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const uint32_t h2 = (static_cast<uint32_t>(hb[j]) & 0xffu) | ((static_cast<uint32_t>(hb[j + 4]) & 0xffu) << 8);
                            const uint32_t l2 = (static_cast<uint32_t>(lb[j]) & 0xffu) | ((static_cast<uint32_t>(lb[j + 4]) & 0xffu) << 8);
                            const uint32_t t2 = (static_cast<uint32_t>(tb[j]) & 0xffu) | ((static_cast<uint32_t>(tb[j + 4]) & 0xffu) << 8);
                            asm volatile("{ .reg .b16 t; cvt.u16.u32 t, %1; st.shared.u16 [%0], t; }" ::"r"(hi_at + j * 4 + odd * 2), "r"(h2) : "memory");
                            asm volatile("{ .reg .b16 t; cvt.u16.u32 t, %1; st.shared.u16 [%0], t; }" ::"r"(lo_at + j * 4 + odd * 2), "r"(l2) : "memory");
                            asm volatile("{ .reg .b16 t; cvt.u16.u32 t, %1; st.shared.u16 [%0], t; }" ::"r"(p2_at + j * 4 + odd * 2), "r"(t2) : "memory");
                        }
                    }
                    if (p8 == 0) {
                        xflag[u * m + t] = need3 ? 1 : 0;
                        const float xscale = live ? __uint_as_float((e - 13u) << 23)  // 2^(E - 127 - 13)
                                                  : (e == 255u ? __uint_as_float(0x7fc00000u) : 0.f);
                        asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(xs32 + (u * m + t) * 8), "f"(xscale), "f"(s) : "memory");
                    }
                }
            }
        }
    }
    consumer_sync();

    // ---- roles: warp = (16-row group h of the tile, quad-warp qd).  A warp keeps its rows for the whole kernel
    // and takes QPW quads (four units each) of every stage.
    const int nhc = p.rows_cap >> 4;           // 16-row groups of a tile: 1, 2 or 4
    const int nq = kNW / nhc;                  // quad-warps per row group
    const int h = warp % nhc, qd = warp / nhc;
    // The two rows of the group this lane owns (MMA rows g and g + 8).  The 128-byte swizzle XORs the 16-byte
    // chunk index with (row & 7): with 8-byte reads (4-bit) rows 2g, 2g+1 keep a half warp on 32 distinct
    // banks, with 4-byte reads (2-bit) rows g, g+8 keep a whole warp on them.
    const int rowA = 16 * h + ((BITS == 4) ? 2 * g : g), rowB = 16 * h + ((BITS == 4) ? 2 * g + 1 : g + 8);
    const int keyA = rowA & 7, keyB = rowB & 7;
    // byte offset, inside a line of the stage, of the lane's 16 codes of unit j of the line's first quad (the
    // second quad of a 2-bit line is chunks 4..7: the same offsets with bit 6 flipped)
    uint32_t offA[4], offB[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int chunk = (BITS == 4) ? 2 * j + (tig >> 1) : j;
        const int inner = (BITS == 4) ? (tig & 1) * 8 : tig * 4;
        offA[j] = rowA * 128 + ((chunk ^ keyA) << 4) + inner;
        offB[j] = rowB * 128 + ((chunk ^ keyB) << 4) + inner;
    }
    uint32_t kmask;
    asm volatile("mov.u32 %0, %1;" : "=r"(kmask) : "r"(BITS == 4 ? 0x0f0f0f0fu : 0x03030303u));
    // B operand: column g = (unit slot, token, plane).  The lane supplies activation bytes for the unit of its slot
    // only; for the other units of the accumulator tile its B registers are zero (bmask).
    const int slot_b = g / (2 * MPC), tok_b = (g % (2 * MPC)) >> 1, plane_b = g & 1;
    // tokens that do not exist read another token's bytes: their columns are never stored
    const int tok_b0 = tok_b % min(m, MPC);
    const int tok_b1 = (MP == 8) ? 4 + tok_b % (m - 4) : 0;
    uint32_t bmask[GS];
#pragma unroll
    for (int sl = 0; sl < GS; ++sl) bmask[sl] = (slot_b == sl) ? 0xffffffffu : 0u;
    const uint32_t xq_b0 = xq32 + (((2 * tok_b0 + plane_b) * 4) + tig) * 16 + slot_b * ncols * 64;
    const uint32_t xq_b1 = (MP == 8) ? xq32 + (((2 * tok_b1 + plane_b) * 4) + tig) * 16 : 0u;
    // third plane: column 2 * (slot, token) carries it, odd columns are zero
    const uint32_t xq3_b0 = xq332 + (tok_b0 * 4 + tig) * 16 + slot_b * m * 64;
    const uint32_t xq3_b1 = (MP == 8) ? xq332 + (tok_b1 * 4 + tig) * 16 : 0u;
    const uint32_t b3mask = plane_b ? 0u : 0xffffffffu;
    // f32 part: the lane reads back columns 2 tig, 2 tig + 1 = (slot, token) of rows A and B
    const int slot_e = tig / MPC, tok_e = tig % MPC;
    const int tok_e0 = min(tok_e, min(m, MPC) - 1), tok_e1 = (MP == 8) ? 4 + min(tok_e, m - 5) : 0;
    const uint32_t ring32 = smem_u32(smem + plan.ring);
    const uint32_t xflag32 = smem_u32(xflag);

    uint16_t *const *outs = sg.out;
    const int ldy = sg.ldy, col0 = sg.col0;

    int buf = 0, s = 0, phase = 0;
    for (int it = 0; it < ntiles; ++it) {
        const int r0 = row_begin + it * kTR;
        const int rows = min(kTR, row_end - r0);
        const bool active = 16 * h < rows;     // a row group without rows only keeps the barriers going
        const int sbuf = it % p.nsb;
        i8_wait(&sfull[sbuf], (it / p.nsb) & 1, abort_flag, 3);
        const uint32_t sc32 = smem_u32(smem + plan.sb + sbuf * plan.sb_bytes);
        const uint32_t scA = sc32 + rowA * srow, scB = sc32 + rowB * srow;
        float rs[NSET][ND][2];   // [column set][accumulator tile of the quad][row A / row B]: unit class d * GS + slot_e
#pragma unroll
        for (int a = 0; a < NSET; ++a)
#pragma unroll
            for (int d = 0; d < ND; ++d) rs[a][d][0] = rs[a][d][1] = 0.f;
        int ubase = 0;
        for (int ks = 0; ks < nkseg; ++ks) {
            const int lines = (ks < p.n1) ? p.l1 : p.l2;
            i8_wait(&full[s], phase, abort_flag, 4);
            const uint32_t stage32 = ring32 + s * p.stage_bytes;
#pragma unroll
            for (int qi = 0; qi < QPW; ++qi) {
                const int quad = qd * QPW + qi;            // quad of the stage
                const int line = quad / QPL;
                if (active && line < lines) {
                    const int j0 = (quad % QPL) * 4;       // first unit of the quad inside its line
                    const int u0 = ubase + quad * 4;       // first unit of the quad inside the row
                    const uint32_t lbase = stage32 + line * line_box;
                    // all shared-memory loads of the quad first
                    uint32_t wa[4][BITS == 4 ? 2 : 1], wb[4][BITS == 4 ? 2 : 1];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (BITS == 4) {
                            const uint2 va = i8_lds_v2(lbase + offA[j]), vb = i8_lds_v2(lbase + offB[j]);
                            wa[j][0] = va.x; wa[j][BITS == 4 ? 1 : 0] = va.y;
                            wb[j][0] = vb.x; wb[j][BITS == 4 ? 1 : 0] = vb.y;
                        } else {
                            wa[j][0] = i8_lds_u32(lbase + (offA[j] ^ (j0 << 4)));
                            wb[j][0] = i8_lds_u32(lbase + (offB[j] ^ (j0 << 4)));
                        }
                    }
                    uint4 xr0[ND], xr1[ND];
#pragma unroll
                    for (int d = 0; d < ND; ++d) {
                        xr0[d] = i8_lds_v4(xq_b0 + (u0 + d * GS) * ncols * 64);
                        if (MP == 8) xr1[d] = i8_lds_v4(xq_b1 + (u0 + d) * ncols * 64);
                    }
                    // per accumulator tile the lane's f32 part belongs to unit u0 + d * GS + slot_e
                    float2 xs0[ND], xs1[ND];
                    uint32_t sA[ND], bA[ND], sB[ND], bB[ND], fl0[ND], fl1[ND];
#pragma unroll
                    for (int d = 0; d < ND; ++d) {
                        const int ue = u0 + d * GS + slot_e;
                        xs0[d] = i8_lds_f2(xs32 + (ue * m + tok_e0) * 8);
                        fl0[d] = i8_lds_u32(xflag32 + (ue * m + tok_e0) * 4);
                        if (MP == 8) {
                            xs1[d] = i8_lds_f2(xs32 + (ue * m + tok_e1) * 8);
                            fl1[d] = i8_lds_u32(xflag32 + (ue * m + tok_e1) * 4);
                        }
                        sA[d] = i8_lds_u16(scA + ue * 2);
                        bA[d] = i8_lds_u16(scA + plan.sb_half + ue * 2);
                        sB[d] = i8_lds_u16(scB + ue * 2);
                        bB[d] = i8_lds_u16(scB + plan.sb_half + ue * 2);
                    }
                    // unpack: the lane's 16 codes of rows A and B of every unit as four words of four u8
                    uint32_t fa[4][4], fb[4][4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (BITS == 4) {
                            fa[j][0] = wa[j][0] & kmask; fa[j][1] = wa[j][BITS == 4 ? 1 : 0] & kmask;
                            fa[j][2] = (wa[j][0] >> 4) & kmask; fa[j][3] = (wa[j][BITS == 4 ? 1 : 0] >> 4) & kmask;
                            fb[j][0] = wb[j][0] & kmask; fb[j][1] = wb[j][BITS == 4 ? 1 : 0] & kmask;
                            fb[j][2] = (wb[j][0] >> 4) & kmask; fb[j][3] = (wb[j][BITS == 4 ? 1 : 0] >> 4) & kmask;
                        } else {
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                fa[j][i] = (wa[j][0] >> (2 * i)) & kmask;
                                fb[j][i] = (wb[j][0] >> (2 * i)) & kmask;
                            }
                        }
                    }
                    bool third = false;
#pragma unroll
                    for (int d = 0; d < ND; ++d) third = third || fl0[d] != 0 || (MP == 8 && fl1[d] != 0);
                    third = __any_sync(0xffffffffu, third);
#pragma unroll
                    for (int d = 0; d < ND; ++d) {
                        // two chains per tile (even and odd codes), added at the end
                        int ce[4] = {0, 0, 0, 0}, co[4] = {0, 0, 0, 0}, ce1[4] = {0, 0, 0, 0}, co1[4] = {0, 0, 0, 0};
#pragma unroll
                        for (int sl = 0; sl < GS; ++sl) {
                            const int j = d * GS + sl;
                            const uint32_t bx = (GS > 1) ? (xr0[d].x & bmask[sl]) : xr0[d].x, by = (GS > 1) ? (xr0[d].y & bmask[sl]) : xr0[d].y;
                            const uint32_t bz = (GS > 1) ? (xr0[d].z & bmask[sl]) : xr0[d].z, bw = (GS > 1) ? (xr0[d].w & bmask[sl]) : xr0[d].w;
                            mma_u8s8(ce, fa[j][0], fb[j][0], fa[j][1], fb[j][1], bx, by);
                            mma_u8s8(co, fa[j][2], fb[j][2], fa[j][3], fb[j][3], bz, bw);
                            if (MP == 8) {
                                mma_u8s8(ce1, fa[j][0], fb[j][0], fa[j][1], fb[j][1], xr1[d].x, xr1[d].y);
                                mma_u8s8(co1, fa[j][2], fb[j][2], fa[j][3], fb[j][3], xr1[d].z, xr1[d].w);
                            }
                        }
                        // sum(q * x_int) = 256 * (hi column) + (lo column), below 2^24: exact as a float
                        float qa0 = static_cast<float>((ce[0] + co[0]) * 256 + (ce[1] + co[1]));
                        float qb0 = static_cast<float>((ce[2] + co[2]) * 256 + (ce[3] + co[3]));
                        float qa1 = 0.f, qb1 = 0.f;
                        if (MP == 8) {
                            qa1 = static_cast<float>((ce1[0] + co1[0]) * 256 + (ce1[1] + co1[1]));
                            qb1 = static_cast<float>((ce1[2] + co1[2]) * 256 + (ce1[3] + co1[3]));
                        }
                        if (third) {  // rare: the p2 plane of a group with a towering element; column 2 * (slot, token)
                            int t3[4] = {0, 0, 0, 0}, t31[4] = {0, 0, 0, 0};
                            const uint4 xt0 = i8_lds_v4(xq3_b0 + (u0 + d * GS) * m * 64);
                            uint4 xt1 = make_uint4(0, 0, 0, 0);
                            if (MP == 8) xt1 = i8_lds_v4(xq3_b1 + (u0 + d) * m * 64);
#pragma unroll
                            for (int sl = 0; sl < GS; ++sl) {
                                const int j = d * GS + sl;
                                const uint32_t mk = b3mask & bmask[sl];
                                mma_u8s8(t3, fa[j][0], fb[j][0], fa[j][1], fb[j][1], xt0.x & mk, xt0.y & mk);
                                mma_u8s8(t3, fa[j][2], fb[j][2], fa[j][3], fb[j][3], xt0.z & mk, xt0.w & mk);
                                if (MP == 8) {
                                    mma_u8s8(t31, fa[j][0], fb[j][0], fa[j][1], fb[j][1], xt1.x & b3mask, xt1.y & b3mask);
                                    mma_u8s8(t31, fa[j][2], fb[j][2], fa[j][3], fb[j][3], xt1.z & b3mask, xt1.w & b3mask);
                                }
                            }
                            if (fl0[d]) {
                                qa0 = fmaf(static_cast<float>(t3[0]), 0.00390625f, qa0);
                                qb0 = fmaf(static_cast<float>(t3[2]), 0.00390625f, qb0);
                            }
                            if (MP == 8 && fl1[d]) {
                                qa1 = fmaf(static_cast<float>(t31[0]), 0.00390625f, qa1);
                                qb1 = fmaf(static_cast<float>(t31[2]), 0.00390625f, qb1);
                            }
                        }
                        const float sAf = bf16_bits_to_f32(sA[d]), bAf = bf16_bits_to_f32(bA[d]);
                        const float sBf = bf16_bits_to_f32(sB[d]), bBf = bf16_bits_to_f32(bB[d]);
                        rs[0][d][0] = fmaf(sAf * xs0[d].x, qa0, fmaf(bAf, xs0[d].y, rs[0][d][0]));
                        rs[0][d][1] = fmaf(sBf * xs0[d].x, qb0, fmaf(bBf, xs0[d].y, rs[0][d][1]));
                        if (MP == 8) {
                            rs[NSET - 1][d][0] = fmaf(sAf * xs1[d].x, qa1, fmaf(bAf, xs1[d].y, rs[NSET - 1][d][0]));
                            rs[NSET - 1][d][1] = fmaf(sBf * xs1[d].x, qb1, fmaf(bBf, xs1[d].y, rs[NSET - 1][d][1]));
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);  // this warp is done reading the stage
            ubase += lines * UPL;
            if (++s == p.stages) {
                s = 0;
                phase ^= 1;
            }
        }
        if (lane == 0) mbar_arrive(&sempty[sbuf]);  // (after the __syncwarp above: the warp has read its last scale)
        // The lane holds, per token, the sums of its unit classes (unit index mod 4).  They are added in the same
        // tree whatever MP is -- (c0 + c1) + (c2 + c3) -- so that a row's result does not depend on how many
        // rows of x the call has; then the quad-warps of the row group are added in order.
        {
            float tot[NSET][2];
#pragma unroll
            for (int a = 0; a < NSET; ++a)
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    if (GS == 4) {
                        float v = rs[a][0][r];
                        v += __shfl_xor_sync(0xffffffffu, v, 1);
                        v += __shfl_xor_sync(0xffffffffu, v, 2);
                        tot[a][r] = v;
                    } else if (GS == 2) {
                        const float v0 = rs[a][0][r] + __shfl_xor_sync(0xffffffffu, rs[a][0][r], 2);
                        const float v1 = rs[a][ND - 1][r] + __shfl_xor_sync(0xffffffffu, rs[a][ND - 1][r], 2);
                        tot[a][r] = v0 + v1;
                    } else {
                        tot[a][r] = (rs[a][0][r] + rs[a][1 % ND][r]) + (rs[a][2 % ND][r] + rs[a][3 % ND][r]);
                    }
                }
            float *pw = part + (buf * nq + qd) * m * rcap;
            if (active && slot_e == 0 && tok_e < min(m, MPC)) {
                pw[tok_e * rcap + rowA] = tot[0][0];
                pw[tok_e * rcap + rowB] = tot[0][1];
            }
            if (MP == 8 && active && tok_e < m - 4) {
                pw[(4 + tok_e) * rcap + rowA] = tot[NSET - 1][0];
                pw[(4 + tok_e) * rcap + rowB] = tot[NSET - 1][1];
            }
        }
        consumer_sync();
        for (int e = tid; e < m * rows; e += kConsumersI8) {
            const int t = e / rows, row = e - t * rows;
            float total = 0.f;
            for (int wi = 0; wi < nq; ++wi) total += part[((buf * nq + wi) * m + t) * rcap + row];
            const uint16_t v = static_cast<uint16_t>(f32_to_bf16_bits(total));
            const size_t at = static_cast<size_t>(t) * ldy + col0 + r0 + row;
            for (int o = 0; o < p.nout; ++o) outs[o][at] = v;  // plain stores; peers' memory in the all-gather form
        }
        buf ^= 1;
    }
}

}  // namespace

// CTAs of a linear with n rows when `budget` CTAs are available: one CTA per 16 rows at most; when an even
// split would give 17 to 20 rows per CTA and n is a multiple of 16, exactly 16 rows each (a few CTAs more
// than the budget: no MMA tile with a single row, no ragged boxes).
static int i8_ctas(int64_t n, int budget) {
    const int64_t by16 = (n + 15) / 16;
    if (by16 <= budget) return static_cast<int>(by16);
    const int64_t per = (n + budget - 1) / budget;
    if (per <= 20 && n % 16 == 0 && by16 <= budget + budget / 8) return static_cast<int>(by16);
    return budget;
}

// CTAs of a launch of `count` linears: one per SM over all of them, shared out by rows.
static void i8_split(int count, const int64_t *n, int *cta0, int *ctas, int &grid, int &rows_max) {
    const int sms = sm_count();
    int64_t n_all = 0;
    for (int i = 0; i < count; ++i) n_all += n[i];
    grid = 0;
    rows_max = 1;
    for (int i = 0; i < count; ++i) {
        const int budget = (count == 1) ? sms : std::max<int>(1, static_cast<int>((static_cast<int64_t>(sms) * n[i] + n_all / 2) / n_all));
        cta0[i] = grid;
        ctas[i] = i8_ctas(n[i], budget);
        grid += ctas[i];
        rows_max = std::max(rows_max, static_cast<int>((n[i] + ctas[i] - 1) / ctas[i]));
    }
}

// `m` rows are wanted; `mc` (<= 8) is how many one pass takes.  `rows_max`: rows of the launch's largest CTA.
static bool i8_make_plan(int64_t k, int group_size, int bits, int m, int rows_max, I8Params &p, int &smem, int &mc) {
    if (bits != 2 && bits != 4) return false;
    if (group_size != 64 || m < 1) return false;
    const int64_t row_bytes = k * bits / 8;
    if (k % 512 != 0 || row_bytes % 128 != 0) return false;  // whole lines; rows of scales are multiples of 16 bytes
    if (k > (1 << 20)) return false;
    p.k = static_cast<int>(k);
    p.groups = static_cast<int>(k / 64);
    p.rows_cap = rows_max <= 16 ? 16 : rows_max <= 32 ? 32 : kTR;
    const int lines = static_cast<int>(row_bytes / 128);
    const int line_box = p.rows_cap * 128;
    // a stage is one line per quad-warp of a row group: 8 warps over rows_cap / 16 row groups (16 KiB)
    const int lps = std::min(kNW * 16 / p.rows_cap, lines);
    p.l1 = lps;
    p.n1 = lines / lps;
    p.l2 = lines - p.n1 * lps;
    p.stage_bytes = lps * line_box;
    const bool one_tile = rows_max <= kTR;
    const int budget = max_smem_optin() / 2 - 1024;  // two CTAs (of consecutive kernels) per SM
    for (mc = std::min(m, 8); mc >= 1; mc = (mc > 4) ? 4 : mc - 1) {
        // two buffers for the scales of a tile when a CTA has several tiles and a ring of three stages still fits
        for (int nsb = one_tile ? 1 : 2; nsb >= 1; --nsb) {
            const int fixed = i8_plan(p.groups, mc, p.rows_cap, 0, p.stage_bytes, nsb).total;
            const int stages = std::min(kMaxStagesI8, (budget - fixed) / p.stage_bytes);
            if (stages >= (nsb == 2 ? 3 : 2)) {
                p.stages = stages;
                p.nsb = nsb;
                smem = i8_plan(p.groups, mc, p.rows_cap, stages, p.stage_bytes, nsb).total;
                return true;
            }
        }
    }
    return false;
}

bool qmv_i8_multi_supported(int64_t m, int64_t k, int count, const int64_t *n, int group_size, int bits) {
    if (count < 1 || count > kMaxSegI8 || m < 1) return false;
    for (int i = 0; i < count; ++i)
        if (n[i] < 1 || n[i] > (1 << 24)) return false;
    int cta0[kMaxSegI8], ctas[kMaxSegI8], grid = 0, rows_max = 1;
    i8_split(count, n, cta0, ctas, grid, rows_max);
    I8Params p{};
    int smem = 0, mc = 0;
    return i8_make_plan(k, group_size, bits, static_cast<int>(std::min<int64_t>(m, 8)), rows_max, p, smem, mc);
}

bool qmv_i8_supported(int64_t m, int64_t k, int64_t n, int group_size, int bits) {
    return qmv_i8_multi_supported(m, k, 1, &n, group_size, bits);
}

template <int BITS, int MP>
static int i8_launch_t(const cudaLaunchConfig_t &cfg, int smem, const I8Maps &maps, const I8Params &p) {
    LISA_CUDA_TRY(cudaFuncSetAttribute(qmv_i8_kernel<BITS, MP>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    LISA_CUDA_TRY(cudaLaunchKernelEx(&cfg, qmv_i8_kernel<BITS, MP>, maps, p));
    count_launch();
    return LISA_OK;
}

// count linears (1..3) that share x: linear i has n[i] rows; y holds count x nout pointers (linear i, output r at
// y[i * nout + r]); row r of linear i is column col0[i] + r of an [m, ldy[i]] output.
static int i8_run(cudaStream_t stream, const void *x, int64_t m, int64_t k, int count, const uint32_t *const *w,
                  const void *const *scales, const void *const *biases, const int64_t *n, int group_size, int bits,
                  void *const *y, int nout, const int64_t *ldy, const int64_t *col0, unsigned flags) {
    if (count < 1 || count > kMaxSegI8 || nout < 1 || nout > 8) return fail(LISA_ERR_UNSUPPORTED, "qmv_i8: one to three linears, one to eight outputs");
    I8Maps maps{};
    const int64_t row_bytes = k * bits / 8;
    int cta0[kMaxSegI8], ctas[kMaxSegI8], grid = 0, rows_max = 1;
    i8_split(count, n, cta0, ctas, grid, rows_max);
    for (int i = 0; i < count; ++i) {
        const uint64_t dims[2] = {static_cast<uint64_t>(row_bytes), static_cast<uint64_t>(n[i])};
        const uint64_t strides[1] = {static_cast<uint64_t>(row_bytes)};
        const uint32_t heights[4] = {kTR, 32, 16, 1};
        for (int b = 0; b < 4; ++b) {
            const uint32_t box[2] = {128, heights[b]};
            const int rc = make_tensor_map(&maps.m[i][b], CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, w[i], dims, strides, box,
                                           CU_TENSOR_MAP_SWIZZLE_128B);
            if (rc != LISA_OK) return rc;
        }
    }
    const uint16_t *xp = reinterpret_cast<const uint16_t *>(x);
    int mc = 0;
    for (int64_t done = 0; done < m; done += mc) {
        I8Params p{};
        int smem = 0;
        if (!i8_make_plan(k, group_size, bits, static_cast<int>(std::min<int64_t>(m - done, 8)), rows_max, p, smem, mc))
            return fail(LISA_ERR_UNSUPPORTED, "qmv_i8: shape not supported");
        p.x = xp + done * k;
        p.m = mc;
        p.nseg = count;
        p.nout = nout;
        for (int i = 0; i < count; ++i) {
            I8Seg &sg = p.seg[i];
            sg.scales = reinterpret_cast<const uint8_t *>(scales[i]);
            sg.biases = reinterpret_cast<const uint8_t *>(biases[i]);
            sg.n = static_cast<int>(n[i]);
            sg.ldy = static_cast<int>(ldy[i]);
            sg.col0 = static_cast<int>(col0[i]);
            for (int r = 0; r < nout; ++r) sg.out[r] = reinterpret_cast<uint16_t *>(y[i * nout + r]) + done * ldy[i];
            sg.cta0 = cta0[i];
            sg.ctas = ctas[i];
        }
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(grid);
        cfg.blockDim = dim3(kThreadsI8);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = (flags & LISA_FLAG_PDL) ? 1 : 0;
        int rc;
        if (bits == 4)
            rc = (mc > 4) ? i8_launch_t<4, 8>(cfg, smem, maps, p) : (mc > 2) ? i8_launch_t<4, 4>(cfg, smem, maps, p)
                 : (mc == 2) ? i8_launch_t<4, 2>(cfg, smem, maps, p) : i8_launch_t<4, 1>(cfg, smem, maps, p);
        else
            rc = (mc > 4) ? i8_launch_t<2, 8>(cfg, smem, maps, p) : (mc > 2) ? i8_launch_t<2, 4>(cfg, smem, maps, p)
                 : (mc == 2) ? i8_launch_t<2, 2>(cfg, smem, maps, p) : i8_launch_t<2, 1>(cfg, smem, maps, p);
        if (rc != LISA_OK) return rc;
    }
    return LISA_OK;
}

int qmv_i8(cudaStream_t stream, const void *x, int64_t m, int64_t k, const uint32_t *w, const void *scales,
           const void *biases, int64_t n, int group_size, int bits, void *y, unsigned flags) {
    const int64_t zero = 0;
    return i8_run(stream, x, m, k, 1, &w, &scales, &biases, &n, group_size, bits, &y, 1, &n, &zero, flags);
}

int qmv_i8_allgather(cudaStream_t stream, const void *x, int64_t m, int64_t k, const uint32_t *w, const void *scales,
                     const void *biases, int64_t n, int group_size, int bits, void *const *outs, int world,
                     int64_t n_total, int64_t col0, unsigned flags) {
    return i8_run(stream, x, m, k, 1, &w, &scales, &biases, &n, group_size, bits, outs, world, &n_total, &col0, flags);
}

int qmv_i8_multi(cudaStream_t stream, const void *x, int64_t m, int64_t k, int count, const uint32_t *const *w,
                 const void *const *scales, const void *const *biases, const int64_t *n, int group_size, int bits,
                 void *const *y, unsigned flags, int world, const int64_t *n_total, const int64_t *col0) {
    if (world > 0) return i8_run(stream, x, m, k, count, w, scales, biases, n, group_size, bits, y, world, n_total, col0, flags);
    const int64_t zeros[kMaxSegI8] = {0, 0, 0};
    return i8_run(stream, x, m, k, count, w, scales, biases, n, group_size, bits, y, 1, n, zeros, flags);
}

}  // namespace lisa
