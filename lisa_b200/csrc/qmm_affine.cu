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
// (N = BT), so every dequantized weight is reused for BT tokens.  The A operand lives in
// TENSOR MEMORY: the dequantize warps write bf16 pairs with tcgen05.st next to the accumulator,
// and tcgen05.mma reads A from there.  Shared memory therefore carries only the TMA writes and
// the B-operand reads: with A in shared memory as well (16 KiB stored and 16 KiB re-read per
// k-block on top of 32 KiB of B reads and 36 KiB of TMA writes per 524 tensor-pipe clocks) the
// 128 B/clk shared-memory port, not the tensor pipe, set the pace.  Warp roles:
//   warp 0       TMA producer: activation tiles [BT x 64] bf16 (128-byte swizzle) and packed
//                weight tiles [128 rows x 128 bytes] (128-byte swizzle), both tiled
//                cp.async.bulk.tensor loads completing on mbarriers (no multicast);
//   warp 1       allocates TMEM and issues tcgen05.mma (one thread), four K=16 steps per
//                64-wide k-block, accumulating in TMEM;
//   warps 2..17  dequantize: warps 2..9 take the even k-blocks, warps 10..17 the odd ones; thread
//                (row, half) turns 32 codes of its row into 16 bf16 pairs (packed f32x2 arithmetic)
//                and stores them to its TMEM lane (row) with tcgen05.st.32x32b.x16, then
//                tcgen05.wait::st + fence + mbarrier arrive; after the main loop the same warps
//                read the accumulator with tcgen05.ld and store bf16 rows.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdlib>

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
int qmm_clear_status() {
    const int zero = 0;
    return cudaMemcpyToSymbol(g_qmm_status, &zero, sizeof(int)) == cudaSuccess ? LISA_OK : LISA_ERR_CUDA;
}

constexpr int kBN = 128;        // weight rows per CTA (MMA M)
constexpr int kWideBt = 384;    // the tall token tile (template WIDE)
constexpr int kBK = 64;         // k per MMA stage: 64 bf16 = one 128-byte swizzle row
constexpr int kStages = 5;      // operand ring: stage s = activation tile in shared memory + A tile in tensor memory
constexpr int kWpStages = 4;    // packed-weight ring: loads run a whole ring (12+ k-blocks) ahead of their use
constexpr int kQ4kBlock = 144;  // GGUF Q4_K: bytes of a 256-element block = one packed stage row (4 k-blocks)
constexpr int kQ2kBlock = 84;   // GGUF Q2_K: bytes of a block; a packed stage row is four of them (16 k-blocks)
constexpr int kACols = kBK / 2; // one k-block of A: 64 bf16 per lane = 32 columns
constexpr int kDequantWarps = 16;  // two sets of 8 warps (even / odd k-blocks); 2 threads per weight row, 32 codes each
constexpr int kWarpsPerKb = kDequantWarps / 2;
constexpr int kThreads = (2 + kDequantWarps) * 32;
constexpr int kWpBytes = kBN * 128;       // 16 KiB

constexpr int kMaxSeg = 3;  // linears of one launch in the sibling form (q|k|v, gate|up)
struct QmmParams {
    const uint16_t *scales;
    const uint16_t *biases;
    uint16_t *y;
    int m, n, k;
    int groups;       // k / group_size
    int group_size;
    int bt;           // tokens per CTA tile, multiple of 16, <= 256
    int acc_cols;     // accumulator columns: power of two >= 32, >= bt; the A ring starts there
    int tmem_cols;    // allocation: power of two >= acc_cols + kStages * 32
    int num_kb;       // k / 64 (rounded up)
    // Grouped (MoE) form: tile blockIdx.y is {expert, row_begin, row_end, -} of the rows sorted by expert;
    // the weights of expert e are rows [e*n, (e+1)*n) of the packed matrix.  Null for the dense GEMM.
    const int32_t *tiles;
    const int32_t *tile_count;
    float *yf;        // GGUF form: f32 output [m, n]
    // Dense affine form only: 1 or 2 k-slices per output tile.  The two CTAs of a tile (blockIdx.z) are a
    // cluster; slice 1 hands its f32 accumulators to slice 0 through distributed shared memory.
    int ksplit;
    // Sibling form (dense affine only): up to kMaxSeg linears that share x, m, k in one launch; segment s owns
    // row tiles [seg_tile[s], seg_tile[s + 1]) and has its own packed rows (tensor map s), scales, biases, y.
    int nseg;
    int seg_tile[kMaxSeg];
    int seg_n[kMaxSeg];
    const uint16_t *seg_scales[kMaxSeg];
    const uint16_t *seg_biases[kMaxSeg];
    uint16_t *seg_y[kMaxSeg];
    // N-sharded form fused with its all-gather (dense affine, one linear): the tile is stored at columns
    // col0 + row of every rank's [m, ldy] output (outs[0 .. nout): this GPU's buffer and peer mappings).
    int nout, ldy, col0;
    int vec_out;  // every output 16-byte aligned, ldy, col0 and n multiples of 8: whole 16-byte runs of 8 rows
    uint16_t *outs[8];
    // Persistent form (one k-slice, no all-gather): the grid is one CTA per SM and CTA b takes the tiles
    // b, b + gridDim.x, ... of the list (token tile major, `ntx` row tiles each, `ntotal` in all).  Barriers,
    // tensor memory and the rings are set up once; the loads of the next tile run during the epilogue.
    int persist, ntx, ntotal;
};
struct QmmMaps {
    CUtensorMap m[kMaxSeg];
};

__device__ __forceinline__ uint32_t qmm_cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void qmm_cluster_arrive() { asm volatile("barrier.cluster.arrive.release;" ::: "memory"); }
__device__ __forceinline__ void qmm_cluster_wait() { asm volatile("barrier.cluster.wait.acquire;" ::: "memory"); }
// Store into the shared memory of CTA `rank` of the cluster, at the address `local_addr` has there.
__device__ __forceinline__ void qmm_st_cluster_f32(uint32_t local_addr, uint32_t rank, float v) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}

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
// D[tmem] (+)= A[tmem] * B[smem descriptor {desc_lo, desc_hi}]; bf16 operands, f32 accumulate.
// A: lane = row, two consecutive k per 32-bit column (low half = even k), 8 columns per K=16 step.
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint32_t desc_lo, uint32_t desc_hi,
                                             uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        ".reg .b64 d;\n\t"
        "mov.b64 d, {%2, %3};\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], d, %4, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "r"(tmem_a), "r"(desc_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "r"(r[0]),
                 "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::
            "r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
        "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// Shared-memory matrix descriptor, K-major, 128-byte swizzle, 8-row groups 1024 bytes apart, in two
// halves: low = start address >> 4 (bits 0-13) | leading byte offset 1 (bit 16, unused for swizzled
// K-major); high = stride byte offset 1024 >> 4 (bits 32-45) | version 1 (bit 46) | SWIZZLE_128B (2 << 61).
// Advancing k by 16 bf16 inside the 128-byte row adds 32 bytes = 2 to the low half.
__device__ __forceinline__ uint32_t umma_desc_lo(uint32_t smem_addr) { return (smem_addr >> 4) | (1u << 16); }
constexpr uint32_t kUmmaDescHiSw128 = (1024u >> 4) | (1u << 14) | (2u << 29);
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

// Every wait is bounded; one that runs out records which wait it was, and the role that hit it leaves
// its loop.  The other roles then run out at their own next wait, so the kernel always ends.
__device__ __forceinline__ bool qmm_wait(uint64_t *bar, uint32_t parity, int code) {
    if (mbar_wait(bar, parity)) return true;
    atomicExch(&g_qmm_status, code);
    return false;
}
// For the sixteen dequantize warps, which run several k-blocks ahead of the MMA issuer: polls spaced
// by a short sleep keep the shared-memory pipeline free for the single MMA-issuing thread.
__device__ __forceinline__ bool qmm_wait_relaxed(uint64_t *bar, uint32_t parity, int code) {
    if (mbar_wait_relaxed(bar, parity)) return true;
    atomicExch(&g_qmm_status, code);
    return false;
}

// (a & b) | c in one LOP3 with all three operands in registers.
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

__device__ __forceinline__ unsigned long long pack_f32x2(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
// Two codes of `src` -> one word of two bf16 weights.  Code j sits at bit offset BITS*j of `src` and
// is masked in place (m0, m1), turned into the float 2^23 + q * 2^(BITS*j) by OR-ing the exponent of
// 2^23 (one LOP3 each), then both lanes at once: f - 2^23 (exact), (f - 2^23) * (s / 2^(BITS*j)) + b
// with one rounding -- the same real number as q * s + b, hence the same f32 and the same bf16.
__device__ __forceinline__ uint32_t dequant_pair(uint32_t src, uint32_t m0, uint32_t m1, uint32_t mbits,
                                                 unsigned long long neg_magic2, unsigned long long s2,
                                                 unsigned long long b2) {
    uint32_t out;
    asm("{\n\t"
        ".reg .b32 q0, q1;\n\t"
        ".reg .f32 f0, f1;\n\t"
        ".reg .b64 t;\n\t"
        "lop3.b32 q0, %1, %2, %4, 0xEA;\n\t"
        "lop3.b32 q1, %1, %3, %4, 0xEA;\n\t"
        "mov.b64 t, {q0, q1};\n\t"
        "add.rn.f32x2 t, t, %5;\n\t"
        "fma.rn.f32x2 t, t, %6, %7;\n\t"
        "mov.b64 {f0, f1}, t;\n\t"
        "cvt.rn.bf16x2.f32 %0, f1, f0;\n\t"
        "}\n"
        : "=r"(out)
        : "r"(src), "r"(m0), "r"(m1), "r"(mbits), "l"(neg_magic2), "l"(s2), "l"(b2));
    return out;
}

// The same two weights as dequant_pair, as a bf16 pair `hi` and the bf16 pair `lo` of what the rounding to
// bf16 left over: hi + lo carries 16 significant bits of each f32 weight.
__device__ __forceinline__ void dequant_pair_split(uint32_t src, uint32_t m0, uint32_t m1, uint32_t mbits,
                                                   unsigned long long neg_magic2, unsigned long long s2,
                                                   unsigned long long b2, uint32_t &hi, uint32_t &lo) {
    asm("{\n\t"
        ".reg .b32 q0, q1, h0, h1;\n\t"
        ".reg .f32 f0, f1;\n\t"
        ".reg .b64 t;\n\t"
        "lop3.b32 q0, %2, %3, %5, 0xEA;\n\t"
        "lop3.b32 q1, %2, %4, %5, 0xEA;\n\t"
        "mov.b64 t, {q0, q1};\n\t"
        "add.rn.f32x2 t, t, %6;\n\t"
        "fma.rn.f32x2 t, t, %7, %8;\n\t"
        "mov.b64 {f0, f1}, t;\n\t"
        "cvt.rn.bf16x2.f32 %0, f1, f0;\n\t"
        "shl.b32 h0, %0, 16;\n\t"
        "and.b32 h1, %0, 0xffff0000;\n\t"
        "sub.rn.f32 f0, f0, h0;\n\t"
        "sub.rn.f32 f1, f1, h1;\n\t"
        "cvt.rn.bf16x2.f32 %1, f1, f0;\n\t"
        "}\n"
        : "=r"(hi), "=r"(lo)
        : "r"(src), "r"(m0), "r"(m1), "r"(mbits), "l"(neg_magic2), "l"(s2), "l"(b2));
}

struct QmmSmem {
    // byte offsets from the 1024-aligned base
    static constexpr int kXs = 0;                                   // kStages * bt * 128
    __host__ __device__ static int wp(int bt, int xplanes = 1, int stages = kStages) { return stages * xplanes * bt * 128; }
    __host__ __device__ static int bars(int bt, int wstages = kWpStages, int wbytes = kWpBytes, int xplanes = 1,
                                        int stages = kStages) {
        return wp(bt, xplanes, stages) + wstages * wbytes;
    }
    __host__ __device__ static int total(int bt, int wstages = kWpStages, int wbytes = kWpBytes, int xplanes = 1,
                                         int stages = kStages) {
        return bars(bt, wstages, wbytes, xplanes, stages) + 256 + 1024;  // + alignment slack
    }
};

// GGUF = 4 (with BITS = 4): the packed rows are GGUF Q4_K blocks (crates/lisa-gguf/src/quant.rs:82-101):
// a stage row is one 144-byte block {f16 d, f16 dmin, 12 bytes of 6-bit scales and mins, 128 nibble bytes},
// a (k-block, half) is one 32-element sub-block g = 2*sub + half -- nibble `half` of bytes 32*sub .. +31 --
// i.e. an affine group with scale = d*sc_g and bias = -dmin*m_g, taken from the block header in shared
// memory.  GGUF = 2 (with BITS = 2): Q2_K blocks (quant.rs:64-80), four 84-byte blocks {16 scale/min
// bytes, 64 code bytes, f16 d, f16 dmin} per stage row; the 32 elements of (k-block, half) are the 2-bit
// fields at bit offset 2*shift of bytes 32*(kb4/2) .. +31, shift = 2*(kb4&1) + half, the first 16 under scale
// byte [half_of_block*8 + shift*2], the last 16 under the next one.  The output is f32.
//
// WIDE: a token tile of 384 (the dequantization sets a CTA's pace whatever the token tile, so a taller tile is
// that many fewer passes over the weights): two MMAs per k-step (N = 256 and N = 128, into columns 0 and 256
// of the accumulator), three loads of 128 activation rows per stage, a three-stage operand ring (48 KiB
// a stage), all 512 tensor-memory columns (384 accumulator + 3 x 32 of A).
template <int BITS, int GGUF = 0, bool WIDE = false>
__global__ void __launch_bounds__(kThreads, 1)
qmm_affine_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ QmmMaps maps_w,
                  const QmmParams p) {
    constexpr int ST = (GGUF == 2 || WIDE) ? 3 : kStages;              // operand ring stages
    constexpr int WS = (GGUF == 4) ? 3 : (GGUF == 2) ? 2 : kWpStages;  // packed ring stages
    constexpr int ROWB = (GGUF == 4) ? kQ4kBlock : (GGUF == 2) ? 4 * kQ2kBlock : 128;  // bytes of a packed stage row
    constexpr int WPB = kBN * ROWB;                       // bytes of a packed stage
    // GGUF activations are f32: they come as two bf16 planes, x = hi + lo (rows [0, m) and [m, 2m) of the
    // activation tensor map), both multiplied with the same A tile into the same accumulator, so that only
    // the rounding of the decoded weights is left
    constexpr int XP = GGUF ? 2 : 1;
    // ... and the decoded weights as two bf16 planes as well (hi in columns 0..31 of an A stage, lo in
    // 32..63); the products hi*hi, hi*lo and lo*hi go into the same accumulator
    constexpr int ACOLS = GGUF ? 2 * kACols : kACols;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *xs = smem + QmmSmem::kXs;
    uint8_t *wp = smem + QmmSmem::wp(p.bt, XP, ST);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + QmmSmem::bars(p.bt, WS, WPB, XP, ST));
    // full[s]: activation tile landed (1 arrival + bytes) and the eight dequantize warps of the k-block
    // stored their parts of the A tile; empty[s]: the MMAs that read stage s completed (tcgen05.commit).
    uint64_t *full = bars, *empty = bars + ST;
    uint64_t *wp_full = bars + 2 * ST, *wp_empty = wp_full + WS;
    uint64_t *acc_full = wp_empty + WS;
    uint64_t *acc_empty = acc_full + 1;  // persistent form: the sixteen epilogue warps have read the accumulator
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty + 1);

    constexpr int KBW = (GGUF == 2) ? 16 : (128 * 8 / BITS) / kBK;  // k-blocks per packed-weight stage: 4 (4-bit), 8 (2-bit), 16 (Q2_K)
    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);  // warp-uniform for the compiler too
    // Tiles of this CTA: tile (blockIdx.x, blockIdx.y) in the plain form, a strided walk over the list in the
    // persistent one.
    const int ntx = p.persist ? p.ntx : static_cast<int>(gridDim.x);
    const int tile_first = p.persist ? static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.y * gridDim.x + blockIdx.x);
    const int tile_step = p.persist ? static_cast<int>(gridDim.x) : 0x40000000;
    const int tile_total = p.persist ? p.ntotal : tile_first + 1;
    const int live_y = p.tiles ? __ldg(p.tile_count) : 0x7fffffff;  // grouped form: token tiles in the table
    if (tile_first / ntx >= live_y) return;  // whole CTA, before any barrier
    struct Tile {
        int seg;     // the linear this row tile belongs to (0, unless the launch is the sibling form)
        int seg_n;   // its rows
        int n0;      // first weight row of the tile within the linear
        int t0, t_end;  // tokens
        int wrow0;   // first row of the packed matrix (grouped: the expert's rows)
    };
    auto tile_at = [&](int L, Tile &c) -> bool {
        const int ytile = L / ntx;
        int xtile = L - ytile * ntx;
        if (ytile >= live_y) return false;  // token-tile major: every later tile is outside the table too
        c.seg = 0;
        if (!GGUF && p.nseg > 1) {
            c.seg = (xtile >= p.seg_tile[1]) ? 1 : 0;
            if (p.nseg > 2 && xtile >= p.seg_tile[2]) c.seg = 2;
            xtile -= (c.seg == 0) ? 0 : (c.seg == 1) ? p.seg_tile[1] : p.seg_tile[2];
        }
        c.seg_n = (c.seg == 0) ? p.n : (c.seg == 1) ? p.seg_n[1] : p.seg_n[2];
        c.n0 = xtile * kBN;
        c.t0 = ytile * p.bt;
        c.t_end = p.m;
        c.wrow0 = c.n0;
        if (p.tiles) {
            const int4 tile = __ldg(reinterpret_cast<const int4 *>(p.tiles) + ytile);
            c.wrow0 = tile.x * c.seg_n + c.n0;  // (sibling linears of a grouped launch have their own [experts * n, k] matrices)
            c.t0 = tile.y;
            c.t_end = tile.z;
        }
        return true;
    };
    // this CTA's k-slice: whole packed stages, [kb_off, kb_off + num_kb)
    const bool split = !GGUF && p.ksplit > 1;
    const uint32_t krank = split ? qmm_cluster_rank() : 0u;
    int kb_off = 0, num_kb = p.num_kb;
    if (split) {
        const int total_wi = (p.num_kb + KBW - 1) / KBW;
        const int wi0 = static_cast<int>(krank) * total_wi / p.ksplit, wi1 = static_cast<int>(krank + 1) * total_wi / p.ksplit;
        kb_off = wi0 * KBW;
        num_kb = min(wi1 * KBW, p.num_kb) - kb_off;
    }
    const int wi_off = kb_off / KBW;

    if (tid == 0) {
        for (int i = 0; i < ST; ++i) {
            mbar_init(&full[i], 1 + kWarpsPerKb);
            mbar_init(&empty[i], 1);
        }
        for (int i = 0; i < WS; ++i) {
            mbar_init(&wp_full[i], 1);
            mbar_init(&wp_empty[i], kDequantWarps);
        }
        mbar_init(acc_full, 1);
        mbar_init(acc_empty, kDequantWarps);
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
    const uint32_t tmem_a = tmem_base + static_cast<uint32_t>(p.acc_cols);
    // Launched as a dependent, only what reads or writes activations waits for the previous kernel: the
    // activation loads of the producer and the stores of the epilogue.  Packed weights, scales and biases
    // are constants of the model.
    pdl_launch_dependents();

    if (warp == 0) {
        // ---------------- TMA producer
        if (lane == 0) {
            const int num_wi = (num_kb + KBW - 1) / KBW;
            const uint32_t x_bytes = static_cast<uint32_t>(p.bt) * 128u * XP;
            int wcnt = 0;  // packed stages issued, over all tiles: stage c lives in slot c % WS
            int xcnt = 0;  // activation stages issued
            int s = 0;
            uint32_t ph = 1;  // parity of the lap before: the first lap does not wait
            bool ok = true, first = true;
            Tile c;
            for (int L = tile_first; L < tile_total && ok; L += tile_step) {
                if (!tile_at(L, c)) break;
                const CUtensorMap *map_w = &maps_w.m[c.seg];
                const int t0 = c.t0;
                const int boxes = (min(c.t_end - c.t0, p.bt) + 127) >> 7;
                int next_wi = 0;
                // Packed weights come from HBM: their loads are issued a whole ring ahead, independent of
                // how far the operand ring has drained.
                auto issue_w = [&]() {
                    const int ws = wcnt % WS;
                    if (wcnt >= WS) ok = qmm_wait(&wp_empty[ws], ((wcnt / WS) - 1) & 1, 2);
                    if (!ok) return;
                    mbar_arrive_expect_tx(&wp_full[ws], WPB);
                    // x coordinate in elements of the map: bytes, or 32-bit words for Q2_K
                    tma_load_2d(wp + ws * WPB, map_w, (next_wi + wi_off) * (GGUF == 2 ? ROWB / 4 : ROWB), c.wrow0, &wp_full[ws]);
                    ++next_wi;
                    ++wcnt;
                };
                for (int kb = 0; kb < num_kb && ok; ++kb) {
                    if (kb % KBW == 0) {
                        // (a later tile starts one stage short of the ring: its last slot frees only when the
                        // tile before has been dequantized to the end, and the activation loads must not queue
                        // behind that wait)
                        const int want = kb / KBW + ((kb == 0 && !first) ? WS - 1 : WS);
                        while (ok && next_wi < num_wi && next_wi < want) issue_w();
                        if (first) {
                            pdl_wait();
                            first = false;
                        }
                    }
                    if (xcnt >= ST && ok) ok = qmm_wait(&empty[s], ph, 1);
                    if (!ok) break;
                    if (WIDE) {
                        // the map's box is 128 rows; a ragged tile (the last of a dense launch, a short expert run)
                        // loads only the boxes that hold its rows, and the MMAs below stop at the same row
                        mbar_arrive_expect_tx(&full[s], static_cast<uint32_t>(boxes) * (128u * 128u));
#pragma unroll
                        for (int r = 0; r < 3; ++r)
                            if (r < boxes) tma_load_2d(xs + static_cast<size_t>(s) * x_bytes + r * (128 * 128), &map_x, (kb + kb_off) * kBK, t0 + 128 * r, &full[s]);
                    } else {
                        mbar_arrive_expect_tx(&full[s], x_bytes);
                        tma_load_2d(xs + static_cast<size_t>(s) * x_bytes, &map_x, (kb + kb_off) * kBK, t0, &full[s]);
                    }
                    if (GGUF) tma_load_2d(xs + static_cast<size_t>(s) * x_bytes + x_bytes / 2, &map_x, kb * kBK, p.m + t0, &full[s]);
                    ++xcnt;
                    if (++s == ST) { s = 0; ph ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: the whole warp runs the loop, so that waits, counters and operand
        // addresses stay warp-uniform, and one elected lane issues the four MMAs and the commit of a
        // k-block.  (Issued from inside an `if (lane == 0)` the same loop took ~450 of the 512 clocks
        // that four N = 256 MMAs last.)
        {
            const uint32_t b_lo0 = umma_desc_lo(smem_u32(xs));
            const uint32_t b_step = static_cast<uint32_t>(p.bt) * 8u * XP;  // one stage, in 16-byte units
            int s = 0, it = 0;
            uint32_t ph = 0, acc = 0;
            bool ok = true;
            Tile c;
            for (int L = tile_first; L < tile_total; L += tile_step, ++it) {
            if (!tile_at(L, c)) break;
            if (it > 0) {  // the epilogue of the tile before has read the accumulator
                ok = __all_sync(0xffffffffu, qmm_wait(acc_empty, (it - 1) & 1, 8));
                if (!ok) break;
                tc_fence_after();
            }
            acc = 0;
            // N of the MMAs: the rows of this tile rounded up to 16 (the tensor pipe's time goes with N, and a ragged
            // tile costs what its rows cost); WIDE: rows 256.. are a second MMA into column 256 of the accumulator
            const int r16 = (min(c.t_end - c.t0, p.bt) + 15) & ~15;
            const uint32_t idesc = umma_idesc_bf16(WIDE ? min(r16, 256) : r16);
            const bool second = WIDE && r16 > 256;
            const uint32_t idesc_b = umma_idesc_bf16(second ? r16 - 256 : 16);
            for (int kb = 0; kb < num_kb; ++kb) {
                ok = __all_sync(0xffffffffu, qmm_wait(&full[s], ph, 3));
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_addr = tmem_a + static_cast<uint32_t>(s * ACOLS);
                const uint32_t b_lo = b_lo0 + static_cast<uint32_t>(s) * b_step;
                if (elect_one()) {
#pragma unroll
                    for (int ks = 0; ks < kBK / 16; ++ks) {
                        umma_bf16_ts(tmem_base, a_addr + ks * 8, b_lo + ks * 2, kUmmaDescHiSw128, idesc, acc);
                        if (second) umma_bf16_ts(tmem_base + 256, a_addr + ks * 8, b_lo + (256 * 128 / 16) + ks * 2, kUmmaDescHiSw128, idesc_b, acc);
                        acc = 1;
                        if (GGUF) {
                            // x_lo (half a stage further) with w_hi, then x_hi with w_lo
                            umma_bf16_ts(tmem_base, a_addr + ks * 8, b_lo + b_step / 2 + ks * 2, kUmmaDescHiSw128, idesc, 1u);
                            umma_bf16_ts(tmem_base, a_addr + kACols + ks * 8, b_lo + ks * 2, kUmmaDescHiSw128, idesc, 1u);
                        }
                    }
                    umma_commit(&empty[s]);
                }
                acc = 1;
                __syncwarp();
                if (++s == ST) { s = 0; ph ^= 1; }
            }
            if (!ok) break;
            if (elect_one()) umma_commit(acc_full);
            __syncwarp();
            }
        }
    } else {
        // ---------------- dequantize, then epilogue
        const int dw = warp - 2;             // 0..15
        const int quad = warp & 3;           // this warp's TMEM lanes: 32*quad .. 32*quad+31
        const int half = (dw >> 2) & 1;      // which 32 of the 64 k of a k-block
        const int kpar = dw >> 3;            // this warp's k-blocks: kpar, kpar + 2, ...
        const int row = quad * 32 + lane;    // weight row of the tile = TMEM lane
        const int swz = row & 7;
        // scale and bias of (k-block, half): group (kb*64 + half*32) >> log2(group_size); rows past n and
        // groups past k read a valid element instead: their products meet zero activations or unused rows
        const int gshift = (p.group_size == 32) ? 5 : (p.group_size == 64) ? 6 : 7;
        const int g_last = p.groups - 1;
        // masks and the exponent of 2^23, pinned in registers so that every extraction is one LOP3
        uint32_t mk[8], mbits;
#pragma unroll
        for (int j = 0; j < 8; ++j)
            asm volatile("mov.u32 %0, %1;" : "=r"(mk[j]) : "r"(BITS == 4 ? (0xfu << (4 * (j & 3))) : (0x3u << (2 * j))));
        asm volatile("mov.u32 %0, %1;" : "=r"(mbits) : "r"(0x4b000000u));
        const unsigned long long neg_magic2 = pack_f32x2(-8388608.0f, -8388608.0f);
        const uint32_t wp32 = smem_u32(wp) + row * ROWB;
        const uint32_t a_lane = tmem_a + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(half * 16);
        const int num_wi = (num_kb + KBW - 1) / KBW;
        // epilogue geometry (the same for every tile)
        const int chunks = p.bt / 16;
        // Two k-slices: once both have finished their loops (both operand rings are idle), each slice
        // writes the accumulators of the token chunks the OTHER one owns (slice 0: the first half of the
        // chunks) as part[token of the tile][row] f32 over the owner's operand ring; the owner adds them to
        // its own and stores that half of the tile.
        const uint32_t part32 = smem_u32(xs);
        // k-slices: slice r owns the token chunks [r * chunks / S, (r + 1) * chunks / S); `own_max` bounds a share
        const int S = split ? p.ksplit : 1;
        const int own_lo = static_cast<int>(krank) * chunks / S, own_hi = static_cast<int>(krank + 1) * chunks / S;
        const int own_max = (chunks + S - 1) / S;
        const uint32_t region = static_cast<uint32_t>(own_max) * 16u * kBN * 4u;  // what one slice sends to an owner
        // 16-byte stores of the all-gather form need 16-byte aligned runs of 8 rows and room for the stage
        const bool vec_out = !GGUF && p.nout > 0 && p.vec_out && (!split || p.bt >= 128);
        int kb_base = 0, wi_base = 0, it = 0;  // k-blocks and packed stages of the tiles before, tiles done
        bool ok = true;
        Tile c;
        for (int L = tile_first; L < tile_total; L += tile_step, ++it, kb_base += num_kb, wi_base += num_wi) {
        if (!tile_at(L, c)) break;
        const int seg = c.seg, seg_n = c.seg_n, n0 = c.n0, t0 = c.t0, t_end = c.t_end;
        const int grow = n0 + row;
        const size_t srow_off = static_cast<size_t>(c.wrow0 - n0 + (grow < seg_n ? grow : 0)) * p.groups;
        const uint16_t *srow = ((seg == 0) ? p.scales : (seg == 1) ? p.seg_scales[1] : p.seg_scales[2]) + srow_off;
        const uint16_t *brow = ((seg == 0) ? p.biases : (seg == 1) ? p.seg_biases[1] : p.seg_biases[2]) + srow_off;
        auto load_sb = [&](int kb, uint32_t &sb, uint32_t &bb) {
            int g = ((kb + kb_off) * kBK + half * 32) >> gshift;
            g = g < g_last ? g : g_last;
            sb = __ldg(srow + g);
            bb = __ldg(brow + g);
        };
        uint32_t s_next = 0, b_next = 0;
        if (!GGUF && kpar < num_kb) load_sb(kpar, s_next, b_next);
        for (int kb = kpar; kb < num_kb; kb += 2) {
            const int wi = kb / KBW, wr = wi_base + wi, ws = wr % WS, sub = kb % KBW;
            const int ar = kb_base + kb, a = ar % ST;  // stage of the operand ring, counted over all tiles
            float sc = bf16_bits_to_f32(s_next), bi = bf16_bits_to_f32(b_next);
            float sc1 = 0.f, bi1 = 0.f;  // Q2_K: scale and bias of the second 16 elements
            int qshift = 0;              // Q2_K: which 2-bit field of every byte
            if (!GGUF && kb + 2 < num_kb) load_sb(kb + 2, s_next, b_next);
            // first visit of this packed-weight stage
            if (sub < 2) ok = __all_sync(0xffffffffu, qmm_wait_relaxed(&wp_full[ws], (wr / WS) & 1, 5));
            if (!ok) break;

            // packed codes of (row, k-block, half): 32 codes
            uint32_t w[4];
            uint32_t wq[8];  // GGUF: the 32 bytes whose nibble `half` are this thread's codes
            if (GGUF == 2) {
                const int bq = sub >> 2, kb4 = sub & 3;  // block of the stage row, k-block of the block
                const uint32_t blk = wp32 + ws * WPB + bq * kQ2kBlock;  // 4-byte aligned only
                const int hb = kb4 >> 1, shift = 2 * (kb4 & 1) + half;
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(wq[i]) : "r"(blk + 16 + hb * 32 + 4 * i));
                uint32_t sw, dd;
                asm volatile("ld.shared.u32 %0, [%1];" : "=r"(sw) : "r"(blk + hb * 8 + (shift >> 1) * 4));
                asm volatile("ld.shared.u32 %0, [%1];" : "=r"(dd) : "r"(blk + 80));
                // scale bytes [hb*8 + shift*2 + group], group 0 / 1 = first / last 16 elements
                const uint32_t sb0 = (sw >> (16 * (shift & 1))) & 255u, sb1 = (sw >> (16 * (shift & 1) + 8)) & 255u;
                float d, dmin;
                asm("{ .reg .b16 lo, hi; mov.b32 {lo, hi}, %2; cvt.f32.f16 %0, lo; cvt.f32.f16 %1, hi; }" : "=f"(d), "=f"(dmin) : "r"(dd));
                sc = d * static_cast<float>(sb0 & 15u);
                bi = -(dmin * static_cast<float>(sb0 >> 4));
                sc1 = d * static_cast<float>(sb1 & 15u);
                bi1 = -(dmin * static_cast<float>(sb1 >> 4));
                qshift = shift;
                w[0] = w[1] = w[2] = w[3] = 0;
            } else if (GGUF == 4) {
                const uint32_t blk = wp32 + ws * WPB;
                uint32_t h0, h1, h2, h3;
                asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(h0), "=r"(h1), "=r"(h2), "=r"(h3) : "r"(blk));
                asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(wq[0]), "=r"(wq[1]), "=r"(wq[2]), "=r"(wq[3])
                             : "r"(blk + 16 + sub * 32));
                asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(wq[4]), "=r"(wq[5]), "=r"(wq[6]), "=r"(wq[7])
                             : "r"(blk + 32 + sub * 32));
                // 6-bit scale and min of sub-block g (quant.rs:88-96)
                const int g = 2 * sub + half, sh = 8 * (g & 3);
                const uint32_t b0 = (h1 >> sh) & 255u, b1 = (h2 >> sh) & 255u, b2 = (h3 >> sh) & 255u;
                const uint32_t sq = (g < 4) ? (b0 & 63u) : ((b2 & 15u) | ((b0 >> 6) << 4));
                const uint32_t mq = (g < 4) ? (b1 & 63u) : ((b2 >> 4) | ((b1 >> 6) << 4));
                float d, dmin;
                asm("{ .reg .b16 lo, hi; mov.b32 {lo, hi}, %2; cvt.f32.f16 %0, lo; cvt.f32.f16 %1, hi; }" : "=f"(d), "=f"(dmin) : "r"(h0));
                sc = d * static_cast<float>(sq);            // exact: 11 x 6 significant bits
                bi = -(dmin * static_cast<float>(mq));
                w[0] = w[1] = w[2] = w[3] = 0;
            } else if (BITS == 4) {
                const int c = sub * 2 + half;  // 16-byte chunk of the 128-byte packed row
                asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3])
                             : "r"(wp32 + ws * WPB + ((c ^ swz) << 4)));
            } else {
                uint32_t v0, v1;
                asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v0), "=r"(v1)
                             : "r"(wp32 + ws * WPB + ((sub ^ swz) << 4) + half * 8));
                w[0] = v0;        // 2-bit: each 16-bit half holds 8 codes; the masks reach bits 0..15 only
                w[1] = v0 >> 16;
                w[2] = v1;
                w[3] = v1 >> 16;
            }
            const bool last_visit = sub >= KBW - 2 || kb + 2 >= num_kb;
            uint32_t o[16];
            uint32_t olo[16];  // GGUF only
            const unsigned long long b2 = pack_f32x2(bi, bi);
            if (GGUF == 2) {
                // element 4i + b is the field at bit offset 2*shift of byte b of word i: offsets 2*shift and
                // 2*shift + 8 of each 16-bit half; mk[j] = 3 << 2j
                const float down = __uint_as_float((127u - 2u * qshift) << 23);  // 2^(-2*shift)
                const unsigned long long sg0 = pack_f32x2(sc * down, sc * down * 0.00390625f);
                const unsigned long long sg1 = pack_f32x2(sc1 * down, sc1 * down * 0.00390625f);
                const unsigned long long b21 = pack_f32x2(bi1, bi1);
                uint32_t m0 = mk[0], m1 = mk[4];
                if (qshift == 1) { m0 = mk[1]; m1 = mk[5]; }
                if (qshift == 2) { m0 = mk[2]; m1 = mk[6]; }
                if (qshift == 3) { m0 = mk[3]; m1 = mk[7]; }
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    dequant_pair_split(wq[i], m0, m1, mbits, neg_magic2, i < 4 ? sg0 : sg1, i < 4 ? b2 : b21, o[2 * i + 0], olo[2 * i + 0]);
                    dequant_pair_split(wq[i] >> 16, m0, m1, mbits, neg_magic2, i < 4 ? sg0 : sg1, i < 4 ? b2 : b21, o[2 * i + 1], olo[2 * i + 1]);
                }
            } else if (GGUF == 4) {
                // element 4i + b of the sub-block is nibble `half` of byte b of word i: bit offsets 4*half and
                // 4*half + 8 of each 16-bit half of the word
                const unsigned long long sg = half ? pack_f32x2(sc * 0.0625f, sc * 0.000244140625f)
                                                   : pack_f32x2(sc, sc * 0.00390625f);
                const uint32_t m0 = half ? mk[1] : mk[0], m1 = half ? mk[3] : mk[2];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    dequant_pair_split(wq[i], m0, m1, mbits, neg_magic2, sg, b2, o[2 * i + 0], olo[2 * i + 0]);
                    dequant_pair_split(wq[i] >> 16, m0, m1, mbits, neg_magic2, sg, b2, o[2 * i + 1], olo[2 * i + 1]);
                }
            } else if (BITS == 4) {
                const unsigned long long s01 = pack_f32x2(sc, sc * 0.0625f);
                const unsigned long long s23 = pack_f32x2(sc * 0.00390625f, sc * 0.000244140625f);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint32_t lo = w[i], hi = w[i] >> 16;
                    o[4 * i + 0] = dequant_pair(lo, mk[0], mk[1], mbits, neg_magic2, s01, b2);
                    o[4 * i + 1] = dequant_pair(lo, mk[2], mk[3], mbits, neg_magic2, s23, b2);
                    o[4 * i + 2] = dequant_pair(hi, mk[0], mk[1], mbits, neg_magic2, s01, b2);
                    o[4 * i + 3] = dequant_pair(hi, mk[2], mk[3], mbits, neg_magic2, s23, b2);
                }
            } else {
                unsigned long long s2[4];
                float f = sc;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    s2[j] = pack_f32x2(f, f * 0.25f);
                    f *= 0.0625f;
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) {
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        o[4 * i + j] = dequant_pair(w[i], mk[2 * j], mk[2 * j + 1], mbits, neg_magic2, s2[j], b2);
                }
            }
            // the MMAs that read this stage of the A ring a lap ago must have completed
            if (ar >= ST) {
                ok = __all_sync(0xffffffffu, qmm_wait_relaxed(&empty[a], ((ar / ST) - 1) & 1, 6));  // warp-uniform: tcgen05.st is warp-wide
                if (!ok) break;
                tc_fence_after();
            }
            tmem_st16(a_lane + static_cast<uint32_t>(a * ACOLS), o);
            if (GGUF) tmem_st16(a_lane + static_cast<uint32_t>(a * ACOLS + kACols), olo);
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&full[a]);
                // last visit of the packed stage: hand it back to the producer only now that its words
                // have been consumed (an arrival placed right after the loads let the refill overtake them)
                if (last_visit) mbar_arrive(&wp_empty[ws]);
            }
        }

        // ---------------- epilogue: TMEM -> registers -> bf16 rows of y
        pdl_wait();  // y may still be read by the previous kernel
        if (ok) ok = qmm_wait_relaxed(acc_full, it & 1, 7);
        ok = __all_sync(0xffffffffu, ok);  // tcgen05.ld is warp-wide
        tc_fence_after();
        const int out_row = n0 + row;
        uint16_t *yseg = (seg == 0) ? p.y : (seg == 1) ? p.seg_y[1] : p.seg_y[2];
        const int live = min(chunks, (t_end - t0 + 15) >> 4);  // chunks that hold rows of the tile
        if (split) {
            fence_proxy_async_smem();
            qmm_cluster_arrive();
            qmm_cluster_wait();
            for (int ci = dw >> 2; ci < live && ok; ci += kDequantWarps / 4) {
                if (ci >= own_lo && ci < own_hi) continue;
                uint32_t r[16];
                tmem_ld16(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(ci * 16), r);
                tmem_ld_wait();
                // the owner of chunk ci, the first chunk it owns, and this slice's slot among the owner's senders
                int owner = 0;
                while ((owner + 1) * chunks / S <= ci) ++owner;
                const int olo = owner * chunks / S;
                const uint32_t slot = krank < static_cast<uint32_t>(owner) ? krank : krank - 1u;
                const uint32_t dst = part32 + slot * region;
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    qmm_st_cluster_f32(dst + static_cast<uint32_t>((((ci - olo) * 16 + j) * kBN + row) * 4), static_cast<uint32_t>(owner), __uint_as_float(r[j]));
            }
            qmm_cluster_arrive();
            qmm_cluster_wait();
        }
        // (the 16-byte store path synchronises the four warps of a chunk group with a named barrier, so its
        // trip count must not depend on a per-warp `ok`: after a timed-out wait the values are undefined anyway)
        for (int ci = dw >> 2; ci < live && (ok || vec_out); ci += kDequantWarps / 4) {
            if (ci < own_lo || ci >= own_hi) continue;
            uint32_t r[16];
            tmem_ld16(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(ci * 16), r);
            tmem_ld_wait();
            if (split) {
                // own partial sums first, then the other slices' in rank order
                for (int sl = 0; sl < S - 1; ++sl) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        float v;
                        asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v)
                                     : "r"(part32 + sl * region + static_cast<uint32_t>((((ci - own_lo) * 16 + j) * kBN + row) * 4)));
                        r[j] = __float_as_uint(__uint_as_float(r[j]) + v);
                    }
                }
            }
            if (vec_out) {
                // All-gather form: the chunk (128 rows x 16 tokens) is transposed through shared memory so that
                // every thread stores 16 bytes and a token's 128 rows leave as one 256-byte run per output
                // (2-byte lanes made 64-byte writes over NVLink).  The four warps of a chunk group share a
                // 4 KiB stage behind whatever the k-slice exchange used.
                uint8_t *stage = xs + (split ? (S - 1) * region : 0u) + (dw >> 2) * 4096;
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    *reinterpret_cast<uint16_t *>(stage + j * 256 + row * 2) = static_cast<uint16_t>(f32_to_bf16_bits(__uint_as_float(r[j])));
                asm volatile("bar.sync %0, 128;" ::"r"(1 + (dw >> 2)) : "memory");
#pragma unroll
                for (int v = 0; v < 2; ++v) {
                    const int item = v * 128 + row, j = item >> 4, sg8 = (item & 15) * 8;
                    const int tok = t0 + ci * 16 + j;
                    if (tok < t_end && n0 + sg8 < seg_n) {
                        const uint4 val = *reinterpret_cast<const uint4 *>(stage + j * 256 + sg8 * 2);
                        const size_t at = static_cast<size_t>(tok) * p.ldy + p.col0 + n0 + sg8;
                        for (int o = 0; o < p.nout; ++o) *reinterpret_cast<uint4 *>(p.outs[o] + at) = val;  // peers' memory included
                    }
                }
                asm volatile("bar.sync %0, 128;" ::"r"(1 + (dw >> 2)) : "memory");
            } else if (out_row < seg_n) {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int tok = t0 + ci * 16 + j;
                    if (tok < t_end) {
                        if (GGUF) {
                            p.yf[static_cast<size_t>(tok) * p.n + out_row] = __uint_as_float(r[j]);
                        } else if (p.nout > 0) {
                            const uint16_t v = static_cast<uint16_t>(f32_to_bf16_bits(__uint_as_float(r[j])));
                            const size_t at = static_cast<size_t>(tok) * p.ldy + p.col0 + out_row;
                            for (int o = 0; o < p.nout; ++o) p.outs[o][at] = v;  // plain stores, peers' memory included
                        } else {
                            yseg[static_cast<size_t>(tok) * seg_n + out_row] =
                                static_cast<uint16_t>(f32_to_bf16_bits(__uint_as_float(r[j])));
                        }
                    }
                }
            }
        }
        if (!ok) break;
        if (p.persist) {  // this warp's accumulator reads are done: the next tile's MMAs may overwrite it
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty);
        }
        }
    }
    if (split && warp < 2) {
        // producer and MMA warps: both phases of the cluster barrier count every thread
        qmm_cluster_arrive();
        qmm_cluster_wait();
        qmm_cluster_arrive();
        qmm_cluster_wait();
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

static int qmm_launch(cudaStream_t stream, const void *x, int64_t m, int64_t k, const uint32_t *w, const void *scales,
                      const void *biases, int64_t n, int64_t experts, int group_size, int bits, void *y, unsigned flags,
                      int bt, const int32_t *tiles, const int32_t *tile_count, int64_t max_tiles, int nseg = 1,
                      const uint32_t *const *seg_w = nullptr, const void *const *seg_scales = nullptr,
                      const void *const *seg_biases = nullptr, const int64_t *seg_n = nullptr, void *const *seg_y = nullptr,
                      void *const *outs = nullptr, int nout = 0, int64_t ldy = 0, int64_t col0 = 0) {
    QmmParams p{};
    p.nout = nout;
    p.ldy = static_cast<int>(ldy);
    p.col0 = static_cast<int>(col0);
    for (int o = 0; o < nout; ++o) p.outs[o] = reinterpret_cast<uint16_t *>(outs[o]);
    p.vec_out = (nout > 0 && ldy % 8 == 0 && col0 % 8 == 0 && n % 8 == 0) ? 1 : 0;
    for (int o = 0; o < nout; ++o)
        if (!aligned16(outs[o])) p.vec_out = 0;
    p.scales = reinterpret_cast<const uint16_t *>(scales);
    p.biases = reinterpret_cast<const uint16_t *>(biases);
    p.y = reinterpret_cast<uint16_t *>(y);
    p.m = static_cast<int>(m);
    p.n = static_cast<int>(n);
    p.k = static_cast<int>(k);
    p.groups = static_cast<int>(k / group_size);
    p.group_size = group_size;
    p.bt = bt;
    const bool wide = bt == kWideBt;
    int acc = 32;
    while (acc < bt) acc <<= 1;
    if (wide) acc = kWideBt;  // the A ring follows the 384 accumulator columns
    p.acc_cols = acc;
    int cols = 32;
    while (cols < acc + (wide ? 3 : kStages) * kACols) cols <<= 1;
    p.tmem_cols = cols;
    p.num_kb = static_cast<int>((k + kBK - 1) / kBK);
    p.tiles = tiles;
    p.tile_count = tile_count;

    CUtensorMap map_x;
    QmmMaps maps_w{};
    int rc = make_map_2d(&map_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, x, static_cast<uint64_t>(k),
                         static_cast<uint64_t>(m), static_cast<uint64_t>(k) * 2, kBK, static_cast<uint32_t>(wide ? 128 : bt));
    if (rc != LISA_OK) return rc;
    const uint64_t wrow_bytes = static_cast<uint64_t>(k) * bits / 8;
    rc = make_map_2d(&maps_w.m[0], CU_TENSOR_MAP_DATA_TYPE_UINT8, w, wrow_bytes, static_cast<uint64_t>(n * experts), wrow_bytes,
                     128, kBN);
    if (rc != LISA_OK) return rc;
    int64_t ntiles = (n + kBN - 1) / kBN;
    p.nseg = 1;
    if (nseg > 1) {
        // sibling linears: segment 0 is (w, scales, biases, n, y) above
        p.nseg = nseg;
        p.seg_tile[0] = 0;
        p.seg_n[0] = static_cast<int>(n);
        for (int i = 1; i < nseg; ++i) {
            rc = make_map_2d(&maps_w.m[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, seg_w[i], wrow_bytes, static_cast<uint64_t>(seg_n[i] * experts),
                             wrow_bytes, 128, kBN);
            if (rc != LISA_OK) return rc;
            p.seg_tile[i] = static_cast<int>(ntiles);
            p.seg_n[i] = static_cast<int>(seg_n[i]);
            p.seg_scales[i] = reinterpret_cast<const uint16_t *>(seg_scales[i]);
            p.seg_biases[i] = reinterpret_cast<const uint16_t *>(seg_biases[i]);
            p.seg_y[i] = reinterpret_cast<uint16_t *>(seg_y[i]);
            ntiles += (seg_n[i] + kBN - 1) / kBN;
        }
    }

    const size_t smem = static_cast<size_t>(wide ? QmmSmem::total(bt, kWpStages, kWpBytes, 1, 3) : QmmSmem::total(bt));
    const int64_t ytiles = tiles ? max_tiles : (m + bt - 1) / bt;
    if (ytiles > 65535) return fail(LISA_ERR_LIMIT, "qmm: too many row tiles");
    // Two k-slices per tile (a cluster of two CTAs) when the tiles fill the SMs badly: a CTA's time is its
    // number of k-blocks (the dequantization sets the pace whatever the token tile), a launch's time the
    // number of waves times that plus about six k-blocks of prologue and store, and the exchange of half
    // of the 128 x bt accumulators costs about five more (measured on the configs[1] prefill shapes).
    p.ksplit = 1;
    if (!tiles && !wide) {
        const int kbw = (128 * 8 / bits) / kBK;
        const int64_t sms = sm_count(), ctas = ntiles * ytiles;
        const int64_t t1 = ((ctas + sms - 1) / sms) * (p.num_kb + 6);          // + prologue and store
        int64_t best = t1 * 93;  // a split has to win by 7 %
        for (int sl = 2; sl <= 4; ++sl) {
            if (p.num_kb < 2 * sl * kbw) break;
            // the slices exchange (sl - 1) / sl of the accumulators through the idle operand ring, which has to hold them
            const int chunks = bt / 16, own_max = (chunks + sl - 1) / sl;
            if (static_cast<int64_t>(sl - 1) * own_max * 16 * kBN * 4 + 4 * 4096 > static_cast<int64_t>(kStages) * bt * 128) continue;
            const int64_t ts = ((sl * ctas + sms - 1) / sms) * (p.num_kb / sl + 6 + 3 + 2 * sl);  // + the exchange
            if (ts * 100 < best) {
                best = ts * 100;
                p.ksplit = sl;
            }
        }
    }
    dim3 grid(static_cast<unsigned>(ntiles), static_cast<unsigned>(ytiles), static_cast<unsigned>(p.ksplit));
    // More tiles than SMs, one k-slice, no all-gather stage in the operand ring: one CTA per SM walks the tile list
    // (LISA_QMM_PERSIST=0: one CTA per tile, for comparison).
    static const bool persist_on = [] {
        const char *v = std::getenv("LISA_QMM_PERSIST");
        return !(v && v[0] == '0');
    }();
    // (a last packed stage of one k-block is visited by one of the two dequantize sets only and never handed back in
    // full: harmless at the end of a CTA, not in front of another tile)
    const bool lone_kb = p.num_kb % ((128 * 8 / bits) / kBK) == 1;
    if (persist_on && !lone_kb && p.ksplit == 1 && nout == 0 && ntiles * ytiles > sm_count() && ntiles * ytiles < (1ll << 30)) {
        p.persist = 1;
        p.ntx = static_cast<int>(ntiles);
        p.ntotal = static_cast<int>(ntiles * ytiles);
        grid = dim3(static_cast<unsigned>(sm_count()), 1, 1);
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (flags & LISA_FLAG_PDL) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    if (p.ksplit > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = 1;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = static_cast<unsigned>(p.ksplit);
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    if (wide && bits == 4) {
        LISA_CUDA_TRY(cudaFuncSetAttribute(qmm_affine_kernel<4, 0, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        LISA_CUDA_TRY(cudaLaunchKernelEx(&cfg, qmm_affine_kernel<4, 0, true>, map_x, maps_w, p));
    } else if (wide) {
        LISA_CUDA_TRY(cudaFuncSetAttribute(qmm_affine_kernel<2, 0, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        LISA_CUDA_TRY(cudaLaunchKernelEx(&cfg, qmm_affine_kernel<2, 0, true>, map_x, maps_w, p));
    } else if (bits == 4) {
        LISA_CUDA_TRY(cudaFuncSetAttribute(qmm_affine_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        LISA_CUDA_TRY(cudaLaunchKernelEx(&cfg, qmm_affine_kernel<4>, map_x, maps_w, p));
    } else {
        LISA_CUDA_TRY(cudaFuncSetAttribute(qmm_affine_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        LISA_CUDA_TRY(cudaLaunchKernelEx(&cfg, qmm_affine_kernel<2>, map_x, maps_w, p));
    }
    count_launch();
    return LISA_OK;
}

// ---------------------------------------------------------------------------------------
// GGUF Q4_K GEMM: f32 activations are first rounded to bf16 into the caller's workspace, then the same
// tensor-core kernel runs with the Q4_K block decoder; f32 output.
// x (f32) -> hi = bf16(x), lo = bf16(x - hi): hi + lo carries 16 significant bits of x.
__global__ void __launch_bounds__(256) f32_to_bf16_planes_kernel(const float4 *__restrict__ src, uint2 *__restrict__ hi,
                                                                 uint2 *__restrict__ lo, int64_t n4) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n4) {
        const float4 v = __ldg(src + i);
        const uint32_t h0 = f32x2_to_bf16x2(v.x, v.y), h1 = f32x2_to_bf16x2(v.z, v.w);
        const float rx = v.x - bf16_bits_to_f32(h0 & 0xffffu), ry = v.y - __uint_as_float(h0 & 0xffff0000u);
        const float rz = v.z - bf16_bits_to_f32(h1 & 0xffffu), rw = v.w - __uint_as_float(h1 & 0xffff0000u);
        hi[i] = make_uint2(h0, h1);
        lo[i] = make_uint2(f32x2_to_bf16x2(rx, ry), f32x2_to_bf16x2(rz, rw));
    }
}

bool qmm_gguf_supported(int format, int64_t tokens, int64_t rows, int64_t row_bytes) {
    if (tokens < 1 || rows < 1) return false;
    if (format == LISA_GGUF_Q4_K) {
        if (row_bytes % kQ4kBlock != 0) return false;
    } else if (format == LISA_GGUF_Q2_K) {
        if (row_bytes % (4 * kQ2kBlock) != 0) return false;  // whole stage rows of four blocks; 16-byte row pitch
    } else {
        return false;
    }
    const int64_t k = row_bytes / (format == LISA_GGUF_Q4_K ? kQ4kBlock : kQ2kBlock) * 256;
    return tokens * k < (1ll << 40);
}

size_t qmm_gguf_workspace_bytes(int64_t tokens, int64_t k) { return static_cast<size_t>(2 * tokens * k * 2 + 256); }

int qmm_gguf(cudaStream_t stream, int format, const uint8_t *w, int64_t rows, int64_t row_bytes, const float *x,
             int64_t tokens, float *y, void *workspace) {
    const bool q4 = format == LISA_GGUF_Q4_K;
    const int64_t k = row_bytes / (q4 ? kQ4kBlock : kQ2kBlock) * 256;
    uint16_t *xb = reinterpret_cast<uint16_t *>(workspace);
    const int64_t n4 = tokens * k / 4;
    f32_to_bf16_planes_kernel<<<static_cast<unsigned>((n4 + 255) / 256), 256, 0, stream>>>(
        reinterpret_cast<const float4 *>(x), reinterpret_cast<uint2 *>(xb), reinterpret_cast<uint2 *>(xb + tokens * k), n4);
    LISA_CUDA_TRY(cudaGetLastError());
    count_launch();

    const int stages = q4 ? kStages : 3, wstages = q4 ? 3 : 2;
    const int row_stage_bytes = q4 ? kQ4kBlock : 4 * kQ2kBlock;
    QmmParams p{};
    p.yf = y;
    p.m = static_cast<int>(tokens);
    p.n = static_cast<int>(rows);
    p.k = static_cast<int>(k);
    p.groups = 1;
    p.group_size = 32;
    // two activation planes per stage: token tiles of at most 128
    const int bt = static_cast<int>(tokens >= 128 ? 128 : ((tokens + 15) / 16) * 16);
    p.bt = bt;
    int acc = 32;
    while (acc < bt) acc <<= 1;
    p.acc_cols = acc;
    int cols = 32;
    while (cols < acc + stages * 2 * kACols) cols <<= 1;  // two weight planes per A stage
    p.tmem_cols = cols;
    p.num_kb = static_cast<int>(k / kBK);

    CUtensorMap map_x;
    QmmMaps maps_w{};
    CUtensorMap &map_w = maps_w.m[0];
    int rc = make_map_2d(&map_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, xb, static_cast<uint64_t>(k), static_cast<uint64_t>(2 * tokens),
                         static_cast<uint64_t>(k) * 2, kBK, static_cast<uint32_t>(bt));
    if (rc != LISA_OK) return rc;
    {
        // Q4_K: bytes, one block per box row; Q2_K: 32-bit words (a 336-byte box row is over the 256-element limit in bytes)
        const uint64_t dims[2] = {static_cast<uint64_t>(q4 ? row_bytes : row_bytes / 4), static_cast<uint64_t>(rows)};
        const uint64_t strides[1] = {static_cast<uint64_t>(row_bytes)};
        const uint32_t box[2] = {static_cast<uint32_t>(q4 ? kQ4kBlock : kQ2kBlock), kBN};
        rc = make_tensor_map(&map_w, q4 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, w, dims, strides,
                             box, CU_TENSOR_MAP_SWIZZLE_NONE);
        if (rc != LISA_OK) return rc;
    }
    const int smem = QmmSmem::total(bt, wstages, kBN * row_stage_bytes, 2, stages);
    const int64_t ytiles = (tokens + bt - 1) / bt;
    if (ytiles > 65535) return fail(LISA_ERR_LIMIT, "gguf matmul: too many row tiles");
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>((rows + kBN - 1) / kBN), static_cast<unsigned>(ytiles));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    if (q4) {
        LISA_CUDA_TRY(cudaFuncSetAttribute(qmm_affine_kernel<4, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        LISA_CUDA_TRY(cudaLaunchKernelEx(&cfg, qmm_affine_kernel<4, 4>, map_x, maps_w, p));
    } else {
        LISA_CUDA_TRY(cudaFuncSetAttribute(qmm_affine_kernel<2, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        LISA_CUDA_TRY(cudaLaunchKernelEx(&cfg, qmm_affine_kernel<2, 2>, map_x, maps_w, p));
    }
    count_launch();
    return LISA_OK;
}

// Token tile of a dense launch: the whole of m up to 256; beyond that 256 or 384, whichever gives fewer
// wave x k-block units (a CTA's time is its k-blocks, whatever the tile; the 256 form may run as two k-slices,
// see qmm_launch; a taller tile has a longer epilogue).  LISA_QMM_BT = 256 / 384 overrides the choice.
static int dense_tile_rows(int64_t m, int64_t ntiles, int64_t k, int bits) {
    if (m <= 256) return static_cast<int>((m + 15) / 16 * 16);
    static const int forced = [] {
        const char *v = std::getenv("LISA_QMM_BT");
        return v ? std::atoi(v) : 0;
    }();
    if (forced == 256 || forced == kWideBt) return forced;
    const int64_t num_kb = (k + kBK - 1) / kBK, kbw = (128 * 8 / bits) / kBK, sms = sm_count();
    auto waves = [&](int64_t ctas) { return (ctas + sms - 1) / sms; };
    const int64_t y256 = (m + 255) / 256, y384 = (m + kWideBt - 1) / kWideBt;
    int64_t t256 = waves(ntiles * y256) * (num_kb + 6);
    const int64_t t256s = waves(2 * ntiles * y256) * (num_kb / 2 + 6 + 5);
    if (num_kb >= 4 * kbw && t256s * 100 < t256 * 93) t256 = t256s;
    // a 384-token CTA takes 1.25-1.3 times as long per k-block (tensor-bound, measured; the lower end inside a chain
    // of dependent launches, where the next launch's CTAs fill the ragged last wave) and has a longer epilogue
    const int64_t t384 = waves(ntiles * y384) * (num_kb * 125 / 100 + 9);
    return t384 < t256 ? kWideBt : 256;
}

int qmm_affine(cudaStream_t stream, const void *x, int64_t m, int64_t k, const uint32_t *w, const void *scales,
               const void *biases, int64_t n, int group_size, int bits, void *y, unsigned flags) {
    const int bt = dense_tile_rows(m, (n + kBN - 1) / kBN, k, bits);
    return qmm_launch(stream, x, m, k, w, scales, biases, n, 1, group_size, bits, y, flags, bt, nullptr, nullptr, 0);
}

// N-sharded GEMM fused with its all-gather: this rank's rows [col0, col0 + n) of an n_total-row linear, stored
// by the epilogue as columns of every rank's [m, n_total] output (outs[0 .. world), peer pointers included).
int qmm_affine_allgather(cudaStream_t stream, const void *x, int64_t m, int64_t k, const uint32_t *w, const void *scales,
                         const void *biases, int64_t n, int group_size, int bits, void *const *outs, int world,
                         int64_t n_total, int64_t col0, unsigned flags) {
    const int bt = dense_tile_rows(m, (n + kBN - 1) / kBN, k, bits);
    return qmm_launch(stream, x, m, k, w, scales, biases, n, 1, group_size, bits, outs[0], flags, bt, nullptr, nullptr, 0, 1,
                      nullptr, nullptr, nullptr, nullptr, nullptr, outs, world, n_total, col0);
}

// Sibling linears (2 or 3 that share x, m, k, group size, bits) as one GEMM launch: linear i writes its own
// [m, n[i]] output.  The row tiles of all of them fill the waves together.
int qmm_affine_multi(cudaStream_t stream, const void *x, int64_t m, int64_t k, int count, const uint32_t *const *w,
                     const void *const *scales, const void *const *biases, const int64_t *n, int group_size, int bits,
                     void *const *y, unsigned flags) {
    if (count < 2 || count > kMaxSeg) return fail(LISA_ERR_UNSUPPORTED, "qmm_affine_multi: two or three linears per launch");
    int64_t ntiles = 0;
    for (int i = 0; i < count; ++i) ntiles += (n[i] + kBN - 1) / kBN;
    const int bt = dense_tile_rows(m, ntiles, k, bits);
    return qmm_launch(stream, x, m, k, w[0], scales[0], biases[0], n[0], 1, group_size, bits, y[0], flags, bt, nullptr, nullptr, 0,
                      count, w, scales, biases, n, y);
}

// Grouped GEMM over a tile table: rows of x sorted by expert, tile i = {expert, row_begin, row_end} with
// row_end - row_begin <= bt; tiles[max_tiles][4] and *tile_count live in device memory.
int qmm_affine_grouped(cudaStream_t stream, const void *x, int64_t rows, int64_t k, const uint32_t *w,
                       const void *scales, const void *biases, int64_t experts, int64_t n, int group_size, int bits,
                       void *y, int bt, const int32_t *tiles, const int32_t *tile_count, int64_t max_tiles) {
    return qmm_launch(stream, x, rows, k, w, scales, biases, n, experts, group_size, bits, y, 0, bt, tiles, tile_count,
                      max_tiles);
}

// The same over `count` sibling linears (2 or 3, one n: gate | up of a routed block) in one launch.
int qmm_affine_grouped_multi(cudaStream_t stream, const void *x, int64_t rows, int64_t k, int count, const uint32_t *const *w,
                             const void *const *scales, const void *const *biases, int64_t experts, int64_t n, int group_size,
                             int bits, void *const *y, int bt, const int32_t *tiles, const int32_t *tile_count, int64_t max_tiles) {
    if (count < 2 || count > kMaxSeg) return fail(LISA_ERR_UNSUPPORTED, "qmm_affine_grouped_multi: two or three linears per launch");
    int64_t ns[kMaxSeg];
    for (int i = 0; i < count; ++i) ns[i] = n;
    return qmm_launch(stream, x, rows, k, w[0], scales[0], biases[0], n, experts, group_size, bits, y[0], 0, bt, tiles, tile_count,
                      max_tiles, count, w, scales, biases, ns, y);
}

}  // namespace lisa
