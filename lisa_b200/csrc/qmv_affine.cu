// Decode GEMV for MLX affine 2-/4-bit weights: y[m, n] = sum_k x[m, k] * (scale * q + bias).
//
// Replaces affine_qmv_fast / affine_qmv / affine_qmv_wide
// (crates/lisa-mlx/src/shaders/common/matmul/quantized.metal:762-1088, host side
// crates/lisa-mlx/src/jit/matmul.rs:186-302,1799-1869).  Same factorisation as the
// reference's qdot (quantized.metal:196-295): per group  scale * sum(q*x) + bias * sum(x),
// accumulated in f32, rounded once to bf16.
//
// Streaming kernel (qmv_stream_kernel): one persistent CTA per SM (or two), each owning a
// contiguous range of output rows, so the packed rows, scales and biases it needs are three
// contiguous byte ranges.  A producer warp moves them into a shared-memory ring with bulk
// async copies (TMA, untiled) that complete on mbarriers; consumer warps split K between
// all their threads, decode codes in registers (qmv_math.h) and keep one accumulator per
// row of the tile; a transposed warp-shuffle reduction plus one cross-warp step finishes a
// tile.  Weights never depend on the previous kernel in the stream, so the producer starts
// before griddepcontrol.wait: launched with programmatic stream serialization the ring of
// kernel i+1 fills while kernel i drains.
//
// Generic kernel (qmv_simple_kernel): one warp per output row, direct coalesced loads; any
// shape, any m.  Used when the streaming kernel's shared-memory plan does not fit.
#include <cuda_runtime.h>

#include <algorithm>

#include "common.cuh"
#include "qmv_math.h"

namespace lisa {

static __device__ int g_qmv_status = 0;

int qmv_device_status() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_qmv_status, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

struct QmvParams {
    const uint8_t *w;
    const uint8_t *scales;
    const uint8_t *biases;
    const uint16_t *x;
    uint16_t *y;
    int n, k, m;
    int wrow_bytes;   // K * bits / 8
    int srow_bytes;   // (K / group_size) * 2
    int nchunks;      // 8-byte chunks per packed row
    int gshift;       // chunk index >> gshift = group index
    int stages;       // ring depth
    int stage_bytes;  // bytes of one ring stage (multiple of 128)
    int w_region;     // bytes reserved for packed rows in a stage (multiple of 16)
    int s_region;     // bytes reserved for scales (and for biases) in a stage
    int consumers;    // consumer threads (multiple of 32)
    int w_bulk, s_bulk;  // 1: rows are multiples of 16 bytes, bulk copies allowed
};

template <int BITS>
struct QmvGeom {
    static constexpr int kCodesPerChunk = 64 / BITS;       // one chunk = two words = 8 bytes
    static constexpr int kQuads = kCodesPerChunk / 4;      // float4 of pre-scaled x per chunk
    static constexpr int kPairsPerWord = QmvCode<BITS>::kPairsPerWord;
};

// Shared-memory plan (bytes), shared by host and device.
struct QmvSmemPlan {
    int bars, xt, sx, xu, part, ring, total;
};
template <int BITS>
__host__ __device__ inline QmvSmemPlan qmv_plan(int k, int m, int nwarps, int tr, int stages,
                                                int stage_bytes) {
    QmvSmemPlan p;
    const int nchunks = k / QmvGeom<BITS>::kCodesPerChunk;
    p.bars = 0;
    int off = 256;  // [0,128): 2 * stages mbarriers (stages <= 8); [128,132): abort flag
    p.xt = off;
    off += m * k * 4;
    p.sx = off;
    off += m * nchunks * 4;
    p.xu = off;
    off += m * nchunks * 4;
    off = (off + 15) & ~15;
    p.part = off;
    off += 2 * nwarps * tr * m * 4;
    off = (off + 127) & ~127;
    p.ring = off;
    off += stages * stage_bytes;
    p.total = off;
    return p;
}

// Bounded wait shared by producer and consumers: once any thread of the CTA has given up,
// every later wait returns at once so that all threads still reach every barrier.
__device__ __forceinline__ void wait_or_abort(uint64_t *bar, uint32_t parity, volatile int *abort_flag,
                                              int code) {
    if (*abort_flag) return;
    if (!mbar_wait(bar, parity)) {
        *abort_flag = 1;
        atomicExch(&g_qmv_status, code);
    }
}

// Transposed butterfly: on return lane l holds in v[0] the warp-wide sum of value index
// `reduced_index<NV>(l)`.
template <int NV>
__device__ __forceinline__ void warp_reduce_many(float (&v)[NV], int lane) {
    int n = NV;
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
        if (n > 1) {
            n >>= 1;
            const bool upper = (lane & off) != 0;
#pragma unroll
            for (int i = 0; i < NV / 2; ++i) {
                if (i < n) {
                    const float send = upper ? v[i] : v[i + n];
                    const float keep = upper ? v[i + n] : v[i];
                    v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
                }
            }
        } else {
            v[0] += __shfl_xor_sync(0xffffffffu, v[0], off);
        }
    }
}
template <int NV>
__device__ __forceinline__ int reduced_index(int lane) {
    int n = NV, idx = 0;
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
        if (n > 1) {
            n >>= 1;
            if (lane & off) idx += n;
        }
    }
    return idx;
}

template <int BITS, int TR, int MT>
__global__ void __launch_bounds__(288, 1) qmv_stream_kernel(const QmvParams p) {
    using G = QmvGeom<BITS>;
    using Code = QmvCode<BITS>;
    constexpr int NV = TR * MT;
    extern __shared__ __align__(128) uint8_t smem[];

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int T = p.consumers;
    const int nwarps = T >> 5;  // consumer warps; warp `nwarps` is the producer
    const QmvSmemPlan plan = qmv_plan<BITS>(p.k, MT, nwarps, TR, p.stages, p.stage_bytes);

    uint64_t *full = reinterpret_cast<uint64_t *>(smem);
    uint64_t *empty = full + p.stages;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + 128);
    float4 *xt = reinterpret_cast<float4 *>(smem + plan.xt);
    float *sx = reinterpret_cast<float *>(smem + plan.sx);
    float *xu = reinterpret_cast<float *>(smem + plan.xu);
    float *part = reinterpret_cast<float *>(smem + plan.part);
    uint8_t *ring = smem + plan.ring;

    // Rows of this CTA: an even split of n at single-row granularity.
    const int row_begin = static_cast<int>((static_cast<int64_t>(blockIdx.x) * p.n) / gridDim.x);
    const int row_end = static_cast<int>((static_cast<int64_t>(blockIdx.x + 1) * p.n) / gridDim.x);
    const int ntiles = (row_end - row_begin + TR - 1) / TR;

    if (tid == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], nwarps);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == nwarps) {
        // ---------------- producer warp: weights do not depend on the previous kernel.
        int issued = 0;
        for (int it = 0; it < ntiles; ++it) {
            const int s = it % p.stages;
            if (it >= p.stages) wait_or_abort(&empty[s], ((it / p.stages) - 1) & 1, abort_flag, 1);
            if (*abort_flag) break;
            const int r0 = row_begin + it * TR;
            const int rows = min(TR, row_end - r0);
            uint8_t *st = ring + static_cast<size_t>(s) * p.stage_bytes;
            const uint8_t *gw = p.w + static_cast<size_t>(r0) * p.wrow_bytes;
            const uint8_t *gs = p.scales + static_cast<size_t>(r0) * p.srow_bytes;
            const uint8_t *gb = p.biases + static_cast<size_t>(r0) * p.srow_bytes;
            const uint32_t wbytes = rows * p.wrow_bytes, sbytes = rows * p.srow_bytes;
            // Rows that are not multiples of 16 bytes cannot use bulk copies: plain copy.
            if (!p.w_bulk) {
                for (uint32_t i = lane * 4; i < wbytes; i += 128)
                    *reinterpret_cast<uint32_t *>(st + i) = *reinterpret_cast<const uint32_t *>(gw + i);
            }
            if (!p.s_bulk) {
                for (uint32_t i = lane * 2; i < sbytes; i += 64) {
                    *reinterpret_cast<uint16_t *>(st + p.w_region + i) =
                        *reinterpret_cast<const uint16_t *>(gs + i);
                    *reinterpret_cast<uint16_t *>(st + p.w_region + p.s_region + i) =
                        *reinterpret_cast<const uint16_t *>(gb + i);
                }
            }
            __syncwarp();
            if (lane == 0) {
                const uint32_t tx = (p.w_bulk ? wbytes : 0u) + (p.s_bulk ? 2u * sbytes : 0u);
                mbar_arrive_expect_tx(&full[s], tx);
                if (p.w_bulk) bulk_g2s(st, gw, wbytes, &full[s]);
                if (p.s_bulk) {
                    bulk_g2s(st + p.w_region, gs, sbytes, &full[s]);
                    bulk_g2s(st + p.w_region + p.s_region, gb, sbytes, &full[s]);
                }
            }
            issued = it + 1;
        }
        // After an abort, let copies already issued land before the CTA releases its memory.
        if (*abort_flag && lane == 0) {
            for (int it = max(0, issued - p.stages); it < issued; ++it)
                mbar_wait(&full[it % p.stages], (it / p.stages) & 1, 4000000u);
        }
        return;
    }

    // ---------------- consumers
    pdl_wait();  // x is produced by the previous kernel in the stream

    // Stage the activations: pre-scaled and permuted to the decode order, with the
    // per-chunk sums the factorisation needs.
    for (int item = tid; item < MT * p.nchunks; item += T) {
        const int mrow = item / p.nchunks, c = item - mrow * p.nchunks;
        float xs_sum = 0.f, x_sum = 0.f;
        float xv[G::kCodesPerChunk];
        if (mrow < p.m) {
            const uint4 *src =
                reinterpret_cast<const uint4 *>(p.x + static_cast<size_t>(mrow) * p.k + c * G::kCodesPerChunk);
#pragma unroll
            for (int i = 0; i < G::kCodesPerChunk / 8; ++i) {
                const uint4 v = __ldg(src + i);
                const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    xv[i * 8 + j * 2] = bf16_bits_to_f32(u[j] & 0xffffu);
                    xv[i * 8 + j * 2 + 1] = __uint_as_float(u[j] & 0xffff0000u);
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < G::kCodesPerChunk; ++i) xv[i] = 0.f;
        }
#pragma unroll
        for (int q = 0; q < G::kQuads; ++q) {
            float o[4];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int pair = q * 2 + h;            // pair index within the chunk
                const int word = pair / G::kPairsPerWord;
                const int pw = pair % G::kPairsPerWord;
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int kk = word * Code::kCodesPerWord + Code::code_of(pw, e);
                    const float v = xv[kk] * Code::xscale_of(pw, e);
                    o[h * 2 + e] = v;
                    xs_sum += v;
                }
            }
            xt[(mrow * G::kQuads + q) * p.nchunks + c] = make_float4(o[0], o[1], o[2], o[3]);
        }
#pragma unroll
        for (int i = 0; i < G::kCodesPerChunk; ++i) x_sum += xv[i];
        sx[mrow * p.nchunks + c] = xs_sum;
        xu[mrow * p.nchunks + c] = x_sum;
    }
    asm volatile("bar.sync 1, %0;" ::"r"(T) : "memory");

    int buf = 0;
    for (int it = 0; it < ntiles; ++it) {
        const int s = it % p.stages;
        const int r0 = row_begin + it * TR;
        const int rows = min(TR, row_end - r0);
        const uint8_t *st = ring + static_cast<size_t>(s) * p.stage_bytes;
        const uint8_t *st_s = st + p.w_region;
        const uint8_t *st_b = st_s + p.s_region;

        float rsum[NV];
#pragma unroll
        for (int i = 0; i < NV; ++i) rsum[i] = 0.f;

        wait_or_abort(&full[s], (it / p.stages) & 1, abort_flag, 2);

        for (int c = tid; c < p.nchunks; c += T) {
            // pre-scaled activations of this chunk, one set per input row
            float2 xq[MT][G::kQuads * 2];
            float sxc[MT], xuc[MT];
#pragma unroll
            for (int mm = 0; mm < MT; ++mm) {
#pragma unroll
                for (int q = 0; q < G::kQuads; ++q) {
                    const float4 v = xt[(mm * G::kQuads + q) * p.nchunks + c];
                    xq[mm][q * 2] = make_float2(v.x, v.y);
                    xq[mm][q * 2 + 1] = make_float2(v.z, v.w);
                }
                sxc[mm] = sx[mm * p.nchunks + c];
                xuc[mm] = xu[mm * p.nchunks + c];
            }
            const int g2 = (c >> p.gshift) * 2;
#pragma unroll
            for (int r = 0; r < TR; ++r) {
                if (r < rows) {
                    const uint2 wv = *reinterpret_cast<const uint2 *>(st + r * p.wrow_bytes + c * 8);
                    const float sc = bf16_bits_to_f32(
                        *reinterpret_cast<const uint16_t *>(st_s + r * p.srow_bytes + g2));
                    const float bi = bf16_bits_to_f32(
                        *reinterpret_cast<const uint16_t *>(st_b + r * p.srow_bytes + g2));
                    uint32_t lo[2][G::kPairsPerWord], hi[2][G::kPairsPerWord];
                    Code::decode(wv.x, lo[0], hi[0]);
                    Code::decode(wv.y, lo[1], hi[1]);
#pragma unroll
                    for (int mm = 0; mm < MT; ++mm) {
                        float2 a0 = make_float2(0.f, 0.f), a1 = make_float2(0.f, 0.f);
#pragma unroll
                        for (int wd = 0; wd < 2; ++wd) {
#pragma unroll
                            for (int pp = 0; pp < G::kPairsPerWord; ++pp) {
                                const float2 t =
                                    make_float2(__uint_as_float(lo[wd][pp]), __uint_as_float(hi[wd][pp]));
                                const float2 xv2 = xq[mm][wd * G::kPairsPerWord + pp];
                                if (pp & 1) a1 = ffma2(t, xv2, a1);
                                else a0 = ffma2(t, xv2, a0);
                            }
                        }
                        const float acc = (a0.x + a0.y) + (a1.x + a1.y);
                        float rs = rsum[r * MT + mm];
                        rs = fmaf(sc, acc - sxc[mm], rs);
                        rs = fmaf(bi, xuc[mm], rs);
                        rsum[r * MT + mm] = rs;
                    }
                }
            }
        }

        // this warp is done reading the stage
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);

        warp_reduce_many<NV>(rsum, lane);
        const int ridx = reduced_index<NV>(lane);
        constexpr int kHolders = 32 / NV;  // lanes holding the same reduced value (NV <= 32)
        if ((lane % (kHolders > 0 ? kHolders : 1)) == 0)
            part[(buf * nwarps + warp) * NV + ridx] = rsum[0];
        asm volatile("bar.sync 1, %0;" ::"r"(T) : "memory");
        if (tid < NV) {
            float total = 0.f;
            for (int wi = 0; wi < nwarps; ++wi) total += part[(buf * nwarps + wi) * NV + tid];
            const int r = tid / MT, mm = tid - r * MT;
            if (r < rows && mm < p.m)
                p.y[static_cast<size_t>(mm) * p.n + r0 + r] = static_cast<uint16_t>(f32_to_bf16_bits(total));
        }
        buf ^= 1;
    }
}

// ---------------------------------------------------------------------------------------
// Generic kernel: warp per output row, lanes stride over 8-byte chunks, f32 math with the
// same factorisation.  Handles any n, any k that is a multiple of the group size, any m.
template <int BITS>
__global__ void __launch_bounds__(256) qmv_simple_kernel(const QmvParams p, int group_size) {
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
        const int g = k0 / group_size;  // a word never straddles a group (group_size >= 32 >= CPW)
        float accum = 0.f, xsum = 0.f;
#pragma unroll
        for (int j = 0; j < CPW; ++j) {
            const float xv = bf16_bits_to_f32(__ldg(xr + k0 + j));
            const uint32_t q = (word >> (j * BITS)) & ((1u << BITS) - 1u);
            accum = fmaf(xv, static_cast<float>(q), accum);
            xsum += xv;
        }
        result = fmaf(bf16_bits_to_f32(__ldg(sr + g)), accum, result);
        result = fmaf(bf16_bits_to_f32(__ldg(br + g)), xsum, result);
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) result += __shfl_xor_sync(0xffffffffu, result, off);
    if (lane == 0) p.y[static_cast<size_t>(mrow) * p.n + row] = static_cast<uint16_t>(f32_to_bf16_bits(result));
}

// ---------------------------------------------------------------------------------------
// Host-side planning and launch.

struct QmvLaunchPlan {
    bool ok;
    int tr, stages, stage_bytes, w_region, s_region, consumers, grid, smem;
};

template <int BITS>
static QmvLaunchPlan plan_stream(int64_t n, int64_t k, int group_size, int mt) {
    QmvLaunchPlan lp{};
    lp.ok = false;
    const int cpc = QmvGeom<BITS>::kCodesPerChunk;
    if (k % cpc != 0 || k % 8 != 0) return lp;  // chunks must tile a row; x rows must be 16-byte multiples
    const int nchunks = static_cast<int>(k / cpc);
    const int wrow = static_cast<int>(k * BITS / 8), srow = static_cast<int>(k / group_size * 2);
    const int sms = sm_count();
    const int smem_max = max_smem_optin();
    // consumer threads: enough to cover the chunks of a row with few idle lanes, at most 256
    int best_t = 32;
    double best_u = 0.0;
    for (int t = 256; t >= 32; t -= 32) {
        const int iters = (nchunks + t - 1) / t;
        const double u = static_cast<double>(nchunks) / (static_cast<double>(iters) * t);
        if (u > best_u + 0.02) {
            best_u = u;
            best_t = t;
        }
    }
    lp.consumers = best_t;
    const int nwarps = best_t / 32;
    // Two CTAs per SM when every CTA still gets a few full tiles; else one.
    const int per_sm = (n / (2 * sms) >= 16) ? 2 : 1;
    lp.grid = static_cast<int>(std::min<int64_t>(n, static_cast<int64_t>(sms) * per_sm));
    const int budget = (per_sm == 2 ? smem_max / 2 - 2048 : smem_max) ;
    for (int tr : {16, 8}) {
        if (tr * mt > 32) continue;
        const int w_region = (tr * wrow + 15) & ~15;
        const int s_region = (tr * srow + 15) & ~15;
        const int stage_bytes = (w_region + 2 * s_region + 127) & ~127;
        for (int stages = 8; stages >= 2; --stages) {
            if (stages * stage_bytes > 96 * 1024 && stages > 3) continue;  // deep rings only while small
            const QmvSmemPlan sp = qmv_plan<BITS>(static_cast<int>(k), mt, nwarps, tr, stages, stage_bytes);
            if (sp.total <= budget) {
                lp.ok = true;
                lp.tr = tr;
                lp.stages = stages;
                lp.stage_bytes = stage_bytes;
                lp.w_region = w_region;
                lp.s_region = s_region;
                lp.smem = sp.total;
                return lp;
            }
        }
    }
    if (per_sm == 2) {
        // retry with the whole SM
        lp.grid = static_cast<int>(std::min<int64_t>(n, sms));
        for (int tr : {16, 8}) {
            if (tr * mt > 32) continue;
            const int w_region = (tr * wrow + 15) & ~15;
            const int s_region = (tr * srow + 15) & ~15;
            const int stage_bytes = (w_region + 2 * s_region + 127) & ~127;
            for (int stages = 4; stages >= 2; --stages) {
                const QmvSmemPlan sp = qmv_plan<BITS>(static_cast<int>(k), mt, nwarps, tr, stages, stage_bytes);
                if (sp.total <= smem_max) {
                    lp.ok = true;
                    lp.tr = tr;
                    lp.stages = stages;
                    lp.stage_bytes = stage_bytes;
                    lp.w_region = w_region;
                    lp.s_region = s_region;
                    lp.smem = sp.total;
                    return lp;
                }
            }
        }
    }
    return lp;
}

template <typename Kern>
static int launch_kernel(Kern kern, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, bool pdl,
                         const QmvParams &p) {
    if (smem > 48 * 1024) {
        LISA_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    LISA_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, p));
    count_launch();
    return LISA_OK;
}

template <int BITS, int TR, int MT>
static int launch_stream(const QmvParams &p, const QmvLaunchPlan &lp, cudaStream_t stream, bool pdl) {
    return launch_kernel(qmv_stream_kernel<BITS, TR, MT>, dim3(lp.grid), dim3(lp.consumers + 32), lp.smem,
                         stream, pdl, p);
}

template <int BITS>
static int qmv_dispatch(cudaStream_t stream, const void *x, int64_t m, int64_t k, const uint32_t *w,
                        const void *scales, const void *biases, int64_t n, int group_size, void *y,
                        unsigned flags) {
    QmvParams p{};
    p.w = reinterpret_cast<const uint8_t *>(w);
    p.scales = reinterpret_cast<const uint8_t *>(scales);
    p.biases = reinterpret_cast<const uint8_t *>(biases);
    p.n = static_cast<int>(n);
    p.k = static_cast<int>(k);
    p.wrow_bytes = static_cast<int>(k * BITS / 8);
    p.srow_bytes = static_cast<int>(k / group_size * 2);
    const int cpc = QmvGeom<BITS>::kCodesPerChunk;
    p.nchunks = static_cast<int>(k / cpc);
    int gshift = 0;
    while ((cpc << gshift) < group_size) ++gshift;
    p.gshift = gshift;
    p.w_bulk = (p.wrow_bytes % 16 == 0) ? 1 : 0;
    p.s_bulk = (p.srow_bytes % 16 == 0) ? 1 : 0;
    const bool pdl = (flags & LISA_FLAG_PDL) != 0;
    const bool force_simple = (flags & LISA_FLAG_FORCE_QMV_SIMPLE) != 0;

    const uint16_t *xp = reinterpret_cast<const uint16_t *>(x);
    uint16_t *yp = reinterpret_cast<uint16_t *>(y);
    int64_t done = 0;
    while (done < m) {
        const int64_t left = m - done;
        int mt = left >= 4 ? 4 : (left >= 2 ? 2 : 1);
        QmvLaunchPlan lp{};
        if (!force_simple && group_size >= cpc) {
            for (; mt >= 1; mt >>= 1) {
                lp = plan_stream<BITS>(n, k, group_size, mt);
                if (lp.ok) break;
            }
        }
        if (!lp.ok) {
            // generic kernel, all remaining rows in one launch
            p.x = xp + done * k;
            p.y = yp + done * n;
            p.m = static_cast<int>(left);
            if (left > 65535) return fail(LISA_ERR_LIMIT, "qmv: more than 65535 rows for the generic kernel");
            const int rows_per_block = 8;
            dim3 grid(static_cast<unsigned>((n + rows_per_block - 1) / rows_per_block), static_cast<unsigned>(left));
            cudaLaunchConfig_t cfg{};
            cfg.gridDim = grid;
            cfg.blockDim = dim3(rows_per_block * 32);
            cfg.stream = stream;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[0].val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs = attr;
            cfg.numAttrs = pdl ? 1 : 0;
            LISA_CUDA_TRY(cudaLaunchKernelEx(&cfg, qmv_simple_kernel<BITS>, p, group_size));
            count_launch();
            return LISA_OK;
        }
        p.x = xp + done * k;
        p.y = yp + done * n;
        p.m = static_cast<int>(std::min<int64_t>(left, mt));
        p.stages = lp.stages;
        p.stage_bytes = lp.stage_bytes;
        p.w_region = lp.w_region;
        p.s_region = lp.s_region;
        p.consumers = lp.consumers;
        int rc = LISA_OK;
        if (lp.tr == 16 && mt == 1) rc = launch_stream<BITS, 16, 1>(p, lp, stream, pdl);
        else if (lp.tr == 16 && mt == 2) rc = launch_stream<BITS, 16, 2>(p, lp, stream, pdl);
        else if (lp.tr == 8 && mt == 1) rc = launch_stream<BITS, 8, 1>(p, lp, stream, pdl);
        else if (lp.tr == 8 && mt == 2) rc = launch_stream<BITS, 8, 2>(p, lp, stream, pdl);
        else if (lp.tr == 8 && mt == 4) rc = launch_stream<BITS, 8, 4>(p, lp, stream, pdl);
        else return fail(LISA_ERR_UNSUPPORTED, "qmv: no kernel for the planned tile");
        if (rc != LISA_OK) return rc;
        done += p.m;
    }
    return LISA_OK;
}

int qmv_affine(cudaStream_t stream, const void *x, int64_t m, int64_t k, const uint32_t *w, const void *scales,
               const void *biases, int64_t n, int group_size, int bits, void *y, unsigned flags) {
    if (bits == 4) return qmv_dispatch<4>(stream, x, m, k, w, scales, biases, n, group_size, y, flags);
    if (bits == 2) return qmv_dispatch<2>(stream, x, m, k, w, scales, biases, n, group_size, y, flags);
    return fail(LISA_ERR_UNSUPPORTED, "qmv: bits must be 2 or 4");
}

}  // namespace lisa
