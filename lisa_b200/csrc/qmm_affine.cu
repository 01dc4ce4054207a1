// Prefill GEMM for MLX affine 2-/4-bit weights on the 5th-generation tensor cores:
//   y[m, n] = sum_k x[m, k] * bf16( f32(q[n, k]) * scale + bias ),  f32 accumulate, bf16 out.
//
// Replaces affine_qmm_t / affine_qmm_t_splitk / affine_qmm_t_nax
// (crates/lisa-mlx/src/shaders/common/matmul/quantized.metal:1200-1326,1902-2032,
//  crates/lisa-mlx/src/shaders/nax/quant_header.metal:3657-3790,3931-3978; host side
//  crates/lisa-mlx/src/jit/matmul.rs:1885-2055, crates/lisa-mlx/src/jit/nax.rs:304-406).
// The weight tile is dequantized to bf16 with the law of the reference's tile loaders
// (quantized.metal:490-533): one f32 multiply-add, one rounding to bf16.
//
// One CTA computes a 128 (weight rows) x BT (tokens, <= 256) output tile.  The dequantized
// weight tile is the A operand (M = 128 of the MMA), the activation tile the B operand
// (N = BT), so every dequantized weight is reused for BT tokens.  Warp roles:
//   warp 0      TMA producer: activation tiles [BT x 64] bf16 (128-byte swizzle) and packed
//               weight tiles [128 rows x 128 bytes] (128-byte swizzle), both tiled
//               cp.async.bulk.tensor loads completing on mbarriers (no multicast);
//   warp 1      allocates TMEM and issues tcgen05.mma (one thread), four K=16 steps per
//               64-wide k-block, accumulating in TMEM;
//   warps 2..9  dequantize: thread (row, half) turns 32 codes of its row into bf16 and stores
//               them in the K-major 128-byte-swizzled layout the MMA descriptor expects, then
//               fence.proxy.async + mbarrier arrive; after the main loop the same warps read
//               the accumulator with tcgen05.ld and store bf16 rows.
#include <cuda.h>
#include <cuda_runtime.h>

#include "common.cuh"
#include "kernels.h"
#include "tensor_map.h"

namespace lisa {

static __device__ int g_qmm_status = 0;

int qmm_device_status() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_qmm_status, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

constexpr int kBN = 128;        // weight rows per CTA (MMA M)
constexpr int kBK = 64;         // k per MMA stage: 64 bf16 = one 128-byte swizzle row
constexpr int kXStages = 4;     // activation ring
constexpr int kWpStages = 2;    // packed-weight ring
constexpr int kWdStages = 3;    // dequantized-weight ring
constexpr int kDequantWarps = 8;
constexpr int kThreads = (2 + kDequantWarps) * 32;
constexpr int kWdBytes = kBN * kBK * 2;   // 16 KiB
constexpr int kWpBytes = kBN * 128;       // 16 KiB

struct QmmParams {
    const uint16_t *scales;
    const uint16_t *biases;
    uint16_t *y;
    int m, n, k;
    int groups;       // k / group_size
    int gshift_kb;    // group index of (k-block kb, half h): see dequant
    int group_size;
    int bt;           // tokens per CTA tile, multiple of 16, <= 256
    int tmem_cols;    // power of two >= 32, >= bt
    int num_kb;       // k / 64 (rounded up)
};

// ---- tcgen05 / TMA wrappers ----
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t *dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]; bf16 operands, f32 accumulate.
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3fffu);  // start address
    d |= static_cast<uint64_t>(1) << 16;                      // leading byte offset (unused for swizzled K-major)
    d |= static_cast<uint64_t>(1024 >> 4) << 32;              // stride byte offset between 8-row groups
    d |= static_cast<uint64_t>(1) << 46;                      // descriptor version (Blackwell)
    d |= static_cast<uint64_t>(2) << 61;                      // SWIZZLE_128B
    return d;
}
// Instruction descriptor: D f32, A and B bf16, both K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t umma_idesc_bf16(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
           (static_cast<uint32_t>(128 >> 4) << 24);
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void qmm_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int code) {
    if (*abort_flag) return;
    if (!mbar_wait(bar, parity)) {
        *abort_flag = 1;
        atomicExch(&g_qmm_status, code);
    }
}

// d = a + b on two packed f32 lanes.
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
    unsigned long long ra, rb, rd;
    ra = (static_cast<unsigned long long>(__float_as_uint(a.y)) << 32) | __float_as_uint(a.x);
    rb = (static_cast<unsigned long long>(__float_as_uint(b.y)) << 32) | __float_as_uint(b.x);
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(rd) : "l"(ra), "l"(rb));
    return make_float2(__uint_as_float(static_cast<uint32_t>(rd)), __uint_as_float(static_cast<uint32_t>(rd >> 32)));
}

// Eight bf16 weights (one 16-byte chunk of the A tile) from codes of `word`.
// 4-bit: code j is masked in place (bits 4j..4j+3, j <= 3 after an optional >>16), turned into the
// float 2^23 + q*16^j by OR-ing the exponent of 2^23, and q*16^j * (s/16^j) + b is evaluated with
// one rounding: the same real number as q*s + b, hence the same f32 and the same bf16.
template <int BITS>
struct Dequant;

template <>
struct Dequant<4> {
    static constexpr int kWordsPer32 = 4;  // words holding 32 codes
    // sj[j] = s / 16^j, j = 0..3
    __device__ __forceinline__ static uint4 chunk(uint32_t word, const float (&sj)[4], float b) {
        const float magic = 8388608.0f;
        const uint32_t mbits = 0x4b000000u;
        const uint32_t hi = word >> 16;
        uint32_t out[4];
#pragma unroll
        for (int p = 0; p < 4; ++p) {  // codes 2p, 2p+1
            const uint32_t src = (p < 2) ? word : hi;
            const int j0 = (2 * p) & 3, j1 = (2 * p + 1) & 3;
            const float f0 = __uint_as_float((src & (0xfu << (4 * j0))) | mbits);
            const float f1 = __uint_as_float((src & (0xfu << (4 * j1))) | mbits);
            const float2 q = fadd2(make_float2(f0, f1), make_float2(-magic, -magic));
            const float2 v = ffma2(q, make_float2(sj[j0], sj[j1]), make_float2(b, b));
            out[p] = f32x2_to_bf16x2(v.x, v.y);
        }
        return make_uint4(out[0], out[1], out[2], out[3]);
    }
};

template <>
struct Dequant<2> {
    static constexpr int kWordsPer32 = 2;
    // 2-bit: codes 0..7 of `half16` (a 16-bit half of a word); sj[j] = s / 4^j, j = 0..7
    __device__ __forceinline__ static uint4 chunk(uint32_t half16, const float (&sj)[8], float b) {
        const float magic = 8388608.0f;
        const uint32_t mbits = 0x4b000000u;
        uint32_t out[4];
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            const float f0 = __uint_as_float((half16 & (0x3u << (4 * p))) | mbits);
            const float f1 = __uint_as_float((half16 & (0x3u << (4 * p + 2))) | mbits);
            const float2 q = fadd2(make_float2(f0, f1), make_float2(-magic, -magic));
            const float2 v = ffma2(q, make_float2(sj[2 * p], sj[2 * p + 1]), make_float2(b, b));
            out[p] = f32x2_to_bf16x2(v.x, v.y);
        }
        return make_uint4(out[0], out[1], out[2], out[3]);
    }
};

struct QmmSmem {
    // byte offsets from the 1024-aligned base
    static constexpr int kXs = 0;                                   // kXStages * bt * 128
    __host__ __device__ static int wp(int bt) { return kXStages * bt * 128; }
    __host__ __device__ static int wd(int bt) { return wp(bt) + kWpStages * kWpBytes; }
    __host__ __device__ static int bars(int bt) { return wd(bt) + kWdStages * kWdBytes; }
    __host__ __device__ static int total(int bt) { return bars(bt) + 256 + 1024; }  // + alignment slack
};

template <int BITS>
__global__ void __launch_bounds__(kThreads, 1)
qmm_affine_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                  const QmmParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *xs = smem + QmmSmem::kXs;
    uint8_t *wp = smem + QmmSmem::wp(p.bt);
    uint8_t *wd = smem + QmmSmem::wd(p.bt);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + QmmSmem::bars(p.bt));
    uint64_t *x_full = bars, *x_empty = bars + kXStages;
    uint64_t *wp_full = bars + 2 * kXStages, *wp_empty = wp_full + kWpStages;
    uint64_t *wd_full = wp_empty + kWpStages, *wd_empty = wd_full + kWdStages;
    uint64_t *acc_full = wd_empty + kWdStages;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_full + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    constexpr int KBW = (128 * 8 / BITS) / kBK;  // k-blocks per packed-weight stage: 4 (4-bit), 8 (2-bit)
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n0 = blockIdx.x * kBN;
    const int t0 = blockIdx.y * p.bt;
    const int num_kb = p.num_kb;

    if (tid == 0) {
        for (int i = 0; i < kXStages; ++i) {
            mbar_init(&x_full[i], 1);
            mbar_init(&x_empty[i], 1);
        }
        for (int i = 0; i < kWpStages; ++i) {
            mbar_init(&wp_full[i], 1);
            mbar_init(&wp_empty[i], kDequantWarps);
        }
        for (int i = 0; i < kWdStages; ++i) {
            mbar_init(&wd_full[i], kDequantWarps);
            mbar_init(&wd_empty[i], 1);
        }
        mbar_init(acc_full, 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, static_cast<uint32_t>(p.tmem_cols));
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();
    pdl_wait();

    if (warp == 0) {
        // ---------------- TMA producer
        if (lane == 0) {
            for (int kb = 0; kb < num_kb; ++kb) {
                const int s = kb % kXStages;
                if (kb >= kXStages) qmm_wait(&x_empty[s], ((kb / kXStages) - 1) & 1, abort_flag, 1);
                if (*abort_flag) break;
                if (kb % KBW == 0) {
                    const int wi = kb / KBW, ws = wi % kWpStages;
                    if (wi >= kWpStages) qmm_wait(&wp_empty[ws], ((wi / kWpStages) - 1) & 1, abort_flag, 2);
                    if (*abort_flag) break;
                    mbar_arrive_expect_tx(&wp_full[ws], kWpBytes);
                    tma_load_2d(wp + ws * kWpBytes, &map_w, wi * 128, n0, &wp_full[ws]);
                }
                mbar_arrive_expect_tx(&x_full[s], static_cast<uint32_t>(p.bt) * 128u);
                tma_load_2d(xs + static_cast<size_t>(s) * p.bt * 128, &map_x, kb * kBK, t0, &x_full[s]);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_bf16(p.bt);
            for (int kb = 0; kb < num_kb; ++kb) {
                const int s = kb % kXStages, b = kb % kWdStages;
                qmm_wait(&x_full[s], (kb / kXStages) & 1, abort_flag, 3);
                qmm_wait(&wd_full[b], (kb / kWdStages) & 1, abort_flag, 4);
                if (*abort_flag) break;
                tc_fence_after();
                const uint32_t a_addr = smem_u32(wd + b * kWdBytes);
                const uint32_t b_addr = smem_u32(xs + static_cast<size_t>(s) * p.bt * 128);
#pragma unroll
                for (int ks = 0; ks < kBK / 16; ++ks) {
                    umma_bf16(tmem_base, umma_desc_sw128(a_addr + ks * 32), umma_desc_sw128(b_addr + ks * 32), idesc,
                              (kb > 0 || ks > 0) ? 1u : 0u);
                }
                umma_commit(&x_empty[s]);
                umma_commit(&wd_empty[b]);
            }
            umma_commit(acc_full);
        }
    } else {
        // ---------------- dequantize, then epilogue
        const int dq = tid - 64;            // 0..255
        const int row = dq & 127;           // weight row of the tile
        const int half = dq >> 7;           // which 32 of the 64 k of a k-block
        const int grow = n0 + row;
        const bool row_ok = grow < p.n;
        const int swz = row & 7;
        const uint16_t *srow = p.scales + static_cast<size_t>(row_ok ? grow : 0) * p.groups;
        const uint16_t *brow = p.biases + static_cast<size_t>(row_ok ? grow : 0) * p.groups;
        // group of (kb, half): k = kb*64 + half*32
        auto group_of = [&](int kb) { return (kb * kBK + half * 32) / p.group_size; };
        float s_next = 0.f, b_next = 0.f;
        {
            const int g = group_of(0);
            if (row_ok && g < p.groups) {
                s_next = bf16_bits_to_f32(__ldg(srow + g));
                b_next = bf16_bits_to_f32(__ldg(brow + g));
            }
        }
        for (int kb = 0; kb < num_kb; ++kb) {
            const int wi = kb / KBW, ws = wi % kWpStages, sub = kb % KBW, b = kb % kWdStages;
            const float sc = s_next, bi = b_next;
            if (kb + 1 < num_kb) {
                const int g = group_of(kb + 1);
                if (row_ok && g < p.groups) {
                    s_next = bf16_bits_to_f32(__ldg(srow + g));
                    b_next = bf16_bits_to_f32(__ldg(brow + g));
                } else {
                    s_next = 0.f;
                    b_next = 0.f;
                }
            }
            if (sub == 0) qmm_wait(&wp_full[ws], (wi / kWpStages) & 1, abort_flag, 5);
            // packed codes of (row, k-block, half): 32 codes
            const uint8_t *prow = wp + ws * kWpBytes + row * 128;
            uint32_t words[4];
            if (BITS == 4) {
                const int c = sub * 2 + half;  // 16-byte chunk of the 128-byte packed row
                const uint4 v = *reinterpret_cast<const uint4 *>(prow + ((c ^ swz) << 4));
                words[0] = v.x; words[1] = v.y; words[2] = v.z; words[3] = v.w;
            } else {
                const int c = sub;
                const uint2 v = *reinterpret_cast<const uint2 *>(prow + ((c ^ swz) << 4) + half * 8);
                words[0] = v.x; words[1] = v.y; words[2] = 0; words[3] = 0;
            }
            if (sub == KBW - 1 || kb == num_kb - 1) {
                __syncwarp();
                if (lane == 0) mbar_arrive(&wp_empty[ws]);
            }
            if (kb >= kWdStages) qmm_wait(&wd_empty[b], ((kb / kWdStages) - 1) & 1, abort_flag, 6);
            uint8_t *drow = wd + b * kWdBytes + (row >> 3) * 1024 + swz * 128;
            if (BITS == 4) {
                float sj[4];
                sj[0] = sc; sj[1] = sc * 0.0625f; sj[2] = sc * 0.00390625f; sj[3] = sc * 0.000244140625f;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint4 o = Dequant<4>::chunk(words[j], sj, bi);
                    *reinterpret_cast<uint4 *>(drow + (((half * 4 + j) ^ swz) << 4)) = o;
                }
            } else {
                float sj[8];
                float f = sc;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    sj[j] = f;
                    f *= 0.25f;
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t h16 = (j & 1) ? (words[j >> 1] >> 16) : (words[j >> 1] & 0xffffu);
                    const uint4 o = Dequant<2>::chunk(h16, sj, bi);
                    *reinterpret_cast<uint4 *>(drow + (((half * 4 + j) ^ swz) << 4)) = o;
                }
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&wd_full[b]);
        }

        // ---------------- epilogue: TMEM -> registers -> bf16 rows of y
        qmm_wait(acc_full, 0, abort_flag, 7);
        tc_fence_after();
        const int quad = warp & 3;                 // TMEM lanes 32*quad .. 32*quad+31
        const int egroup = (warp - 2) >> 2;        // two warps share a quadrant: interleave column chunks
        const int out_row = n0 + quad * 32 + lane;
        const int chunks = p.bt / 16;
        for (int ci = egroup; ci < chunks; ci += 2) {
            uint32_t r[16];
            tmem_ld16(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(ci * 16), r);
            tmem_ld_wait();
            if (out_row < p.n && !*abort_flag) {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int tok = t0 + ci * 16 + j;
                    if (tok < p.m)
                        p.y[static_cast<size_t>(tok) * p.n + out_row] =
                            static_cast<uint16_t>(f32_to_bf16_bits(__uint_as_float(r[j])));
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, static_cast<uint32_t>(p.tmem_cols));
    }
}

// ---------------------------------------------------------------------------------------
// Host side: tensor maps and launch.

static int make_map_2d(CUtensorMap *map, CUtensorMapDataType dt, const void *base, uint64_t inner, uint64_t outer,
                       uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer) {
    const uint64_t dims[2] = {inner, outer};
    const uint64_t strides[1] = {row_stride_bytes};
    const uint32_t box[2] = {box_inner, box_outer};
    return make_tensor_map(map, dt, 2, base, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

bool qmm_affine_supported(int64_t m, int64_t k, int64_t n, int group_size, int bits) {
    (void)m;
    (void)n;
    if (bits != 2 && bits != 4) return false;
    if (group_size != 32 && group_size != 64 && group_size != 128) return false;
    // row strides of both tensor maps must be multiples of 16 bytes
    if ((k * 2) % 16 != 0 || (k * bits / 8) % 16 != 0) return false;
    return true;
}

int qmm_affine(cudaStream_t stream, const void *x, int64_t m, int64_t k, const uint32_t *w, const void *scales,
               const void *biases, int64_t n, int group_size, int bits, void *y, unsigned flags) {
    QmmParams p{};
    p.scales = reinterpret_cast<const uint16_t *>(scales);
    p.biases = reinterpret_cast<const uint16_t *>(biases);
    p.y = reinterpret_cast<uint16_t *>(y);
    p.m = static_cast<int>(m);
    p.n = static_cast<int>(n);
    p.k = static_cast<int>(k);
    p.groups = static_cast<int>(k / group_size);
    p.group_size = group_size;
    int bt = static_cast<int>(m >= 256 ? 256 : ((m + 15) / 16) * 16);
    p.bt = bt;
    int cols = 32;
    while (cols < bt) cols <<= 1;
    p.tmem_cols = cols;
    p.num_kb = static_cast<int>((k + kBK - 1) / kBK);

    CUtensorMap map_x, map_w;
    int rc = make_map_2d(&map_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, x, static_cast<uint64_t>(k),
                         static_cast<uint64_t>(m), static_cast<uint64_t>(k) * 2, kBK, static_cast<uint32_t>(bt));
    if (rc != LISA_OK) return rc;
    const uint64_t wrow_bytes = static_cast<uint64_t>(k) * bits / 8;
    rc = make_map_2d(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, w, wrow_bytes, static_cast<uint64_t>(n), wrow_bytes, 128,
                     kBN);
    if (rc != LISA_OK) return rc;

    const size_t smem = static_cast<size_t>(QmmSmem::total(bt));
    dim3 grid(static_cast<unsigned>((n + kBN - 1) / kBN), static_cast<unsigned>((m + bt - 1) / bt));
    if (grid.y > 65535) return fail(LISA_ERR_LIMIT, "qmm: too many row tiles");
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (flags & LISA_FLAG_PDL) ? 1 : 0;
    if (bits == 4) {
        LISA_CUDA_TRY(cudaFuncSetAttribute(qmm_affine_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        LISA_CUDA_TRY(cudaLaunchKernelEx(&cfg, qmm_affine_kernel<4>, map_x, map_w, p));
    } else {
        LISA_CUDA_TRY(cudaFuncSetAttribute(qmm_affine_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        LISA_CUDA_TRY(cudaLaunchKernelEx(&cfg, qmm_affine_kernel<2>, map_x, map_w, p));
    }
    count_launch();
    return LISA_OK;
}

}  // namespace lisa
