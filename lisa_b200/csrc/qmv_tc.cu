// Decode GEMV for MLX affine 2-/4-bit weights through tcgen05 with the weights in tensor memory:
//   y[m, n] = sum_k x[m, k] * (scale * q + bias),  m <= 8 rows of x per launch, group size 64.
//
// Same operator as qmv_affine.cu (replaces affine_qmv_fast / affine_qmv_wide,
// crates/lisa-mlx/src/shaders/common/matmul/quantized.metal:762-1088) and the same factorisation as the
// reference's qdot (quantized.metal:196-295): per 64 codes  scale * sum(q*x) + bias * sum(x)  in f32.
//
// Why a second GEMV kernel.  The mma.sync kernel spends about 0.12 warp-instructions per code: the
// fragment loads, the per-lane shifts and the four MMAs of every 16 rows x 64 codes are issued by the
// same warps that unpack, and a 4-bit stream at HBM speed (45 codes per clock per SM) would need 5.5
// warp-instructions per clock of the 4 an SM has.  Here the codes go to the tensor core as what they
// are, unsigned 8-bit integers: two instructions spread the eight nibbles of a word over two words of
// bytes (w & 0x0F0F0F0F, (w >> 4) & 0x0F0F0F0F), thread (row) writes the 16 words of a 64-code k-block
// straight to its lane of tensor memory with tcgen05.st, and tcgen05.mma.kind::i8 multiplies A = that
// tile (128 rows x 64 k, u8, in TMEM) with B = the activations (in shared memory), D = a 128 x 16 s32
// tile in TMEM -- one D per 64-code group, so that scale and bias are applied by the epilogue warps.
//
// The activations become integers per (token, 64-k group): with E the exponent of the group's largest
// magnitude, x * 2^(13-E) is rounded to an integer below 2^14 and split into two signed bytes,
// x_int = 256 * hi + lo; rows 0..7 of the B tile hold the hi bytes of up to 8 tokens, rows 8..15 the lo
// bytes.  A bf16 value has 8 significant bits, so every element within 2^-6 of the group maximum is
// represented exactly and the rest to 2^-14 of that maximum; products and sums are exact in s32:
//   sum(q*x) = 2^(E-13) * (256 * D[:, t] + D[:, 8+t]),   y += scale * sum(q*x) + bias * sum(x)
// with sum(x) the f32 sum of the bf16 activations.  About 0.03 warp-instructions per code.
//
// Work split: CTA = (128-row tile, k-slice); the k-slices of a tile form a thread-block cluster and their
// partial sums are written into the shared memory of the cluster's rank 0, which adds them in rank
// order.  CTAs use under half an SM, and the weights do not depend on the previous kernel in the
// stream: launched with programmatic stream serialization, kernel i+1 fills its ring and unpacks while
// kernel i still computes.
//
// Warp roles (14 warps):
//   warp 0        TMA producer: packed tiles [128 rows x 128 bytes], 128-byte swizzle, no multicast;
//   warp 1        TMEM allocation; runs the MMA loop warp-uniformly, an elected lane issues the MMAs of
//                 two k-blocks and their commits;
//   warps 2..9    unpack: warps 2..5 the even k-blocks, 6..9 the odd ones;
//   warps 10..13  stage scales and biases, then (after griddepcontrol.wait) the activations as byte
//                 pairs in the K order of the unpacked words; epilogue per pair of k-blocks; final store.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"
#include "tensor_map.h"

namespace lisa {

static __device__ int g_qmv_tc_status = 0;

int qmv_tc_device_status() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_qmv_tc_status, sizeof(int)) != cudaSuccess) return -1;
    return v;
}
int qmv_tc_clear_status() {
    const int zero = 0;
    return cudaMemcpyToSymbol(g_qmv_tc_status, &zero, sizeof(int)) == cudaSuccess ? LISA_OK : LISA_ERR_CUDA;
}

namespace {

constexpr int kRows = 128;            // weight rows per CTA = MMA M = TMEM lanes
// Everything downstream of the packed ring moves in PAIRS of k-blocks (one B tile, one hand-over):
constexpr int kNP = 4;                // ring of pair stages: A (tensor memory, 2 x 16 columns) and D (2 x 16 s32 columns)
constexpr int kACols = 16, kDCols = 16;
constexpr int kTmemCols = 256;        // kNP * 32 + kNP * 32
constexpr int kMaxWStages = 6;        // packed-weight ring (shared memory), 16 KiB per stage
constexpr int kWBytes = kRows * 128;
constexpr int kUnpackWarps = 8, kEpilogueWarps = 4;
constexpr int kThreads = (2 + kUnpackWarps + kEpilogueWarps) * 32;
constexpr bool kDeferHandOver = false;  // hand a pair to the MMA warp only after the next one is unpacked
constexpr int kMaxSeg = 3;            // linears of one launch in the sibling form (q|k|v, gate|up)
constexpr int kXTile = 2048;          // B tile of TWO k-blocks: 16 rows (8 hi, 8 lo) x 128 bytes (2 x 64 k)

struct TcParams {
    const uint16_t *scales;
    const uint16_t *biases;
    const uint16_t *x;
    int n, k, m;
    int groups;      // k / 64
    int num_kb;      // k / 64
    int splits;      // cluster size: k-slices per row tile
    int wstages;     // stages of the packed ring
    int max_l;       // k-blocks of the longest slice (sizes the shared-memory plan)
    // Output: row r of this matrix is column col0 + r of every buffer in `out` (leading dimension ldy).
    // One buffer (the caller's y, col0 = 0, ldy = n) for the plain GEMV; for the N-sharded form the
    // buffers of all ranks, this rank's own among them: the all-gather is the epilogue's stores.
    uint16_t *out[8];
    int nout, ldy, col0;
    int wbytes;      // bytes of a packed stage: 128 rows x 128 (affine) or x 144 (Q4_K blocks)
    // GGUF form (f32 in, f32 out; the packed rows are Q4_K blocks, row pitch row_bytes)
    const float *xf;
    float *yf;
    const uint8_t *wg;
    long long row_bytes;
    // sibling form: up to kMaxSeg linears that share x, m, k in one launch; segment s owns row tiles
    // [seg_tile[s], seg_tile[s + 1]) and has its own packed rows (tensor map s), scales, biases and output
    int nseg;
    int seg_tile[kMaxSeg];
    int seg_n[kMaxSeg];
    const uint16_t *seg_scales[kMaxSeg];
    const uint16_t *seg_biases[kMaxSeg];
    uint16_t *seg_out[kMaxSeg];
    // sibling form fused with the all-gather of N-sharded linears: segment s is stored at columns
    // seg_col0[s] + row of every rank's [m, seg_ldy[s]] output of that linear (seg_nout of them; 0: not used)
    int seg_nout;
    int seg_ldy[kMaxSeg];
    int seg_col0[kMaxSeg];
    uint16_t *seg_outs[kMaxSeg][8];
    // grouped form (gather_qmm with few rows per expert): row tile y of the grid belongs to entry g_tiles[y / g_ntiles]
    // = {expert, row_begin, row_end} of the sorted rows (at most 8 rows per entry); the packed matrix is addressed as
    // [experts * g_n, k], x and the output are the sorted rows; entries beyond *g_count do nothing
    // scales and biases of a tile by two tiled TMA copies (box sc_box groups x 128 rows, dense rows of sc_words
    // words) instead of per-thread copies: needs rows of whole 16-byte pieces (groups a multiple of 8); a slice
    // that starts at a group index 4 mod 8 loads from 4 groups earlier
    int sc_tma, sc_box, sc_words;
    // GGUF expert form (one token per CTA): row tile y of the grid belongs to slot z = y / e_ntiles of the flat
    // [tokens, top_k] id table; its expert's rows start at ids[z] * n of the packed matrix, its activations are row
    // (z / e_topk) * e_slots + (z % e_topk) % e_slots of x, its output row z of y; an id outside [0, e_experts)
    // stores zeros and touches no weights
    const int *e_ids;
    int e_experts, e_slots, e_topk, e_ntiles;
    // NORM form: residual [m, k], norm weight [k], eps; outputs: the sum [m, k] and (or null) the normed row [m, k]
    const uint16_t *nr, *nw;
    float neps;
    uint16_t *nsum, *nnorm;
    const int4 *g_tiles;
    const int *g_count;
    int g_ntiles;   // row tiles of one expert
    int g_n;        // rows of one expert (sibling linears of a grouped launch share it)
};
struct TcMaps {
    CUtensorMap m[kMaxSeg];  // packed rows of every segment
    CUtensorMap s[kMaxSeg];  // its scales and biases as [rows, groups] bf16 (used when TcParams::sc_tma)
    CUtensorMap b[kMaxSeg];
};

// Shared-memory plan, bytes from the 1024-aligned base.
struct TcPlan {
    int ring, xb, zero, xsum, sc, part, bars, total;
};
// Bytes of the B tile of a pair of k-blocks.  Affine form with up to four tokens: hi bytes in rows t, lo bytes
// in rows 4 + t of ONE 8-row group (1024 bytes); the MMA still reads N = 16 rows, the second group being
// whatever follows (the next pair's tile, or the staging area behind the last one): its eight accumulator
// columns are never read.
// Words per row of the staged scales (and of the staged biases): the bf16 values of the slice's groups as they lie
// in memory, four per 8-byte asynchronous copy, the row pitch an odd number of such copies so that the 32 rows
// of a warp spread over the banks (two rows per bank).
__host__ __device__ inline int tc_sc_stride(int max_l) { return 2 * (((max_l + 3) / 4) | 1); }
__host__ __device__ inline int tc_xtile(int m, int wbytes) { return (wbytes == kWBytes && m <= 4) ? 1024 : kXTile; }
__host__ __device__ inline TcPlan tc_plan(int wstages, int max_l, int splits, int m, int wbytes = kWBytes, int sc_words = 0) {
    TcPlan p;
    int off = 0;
    p.ring = off;
    off += wstages * wbytes;
    p.xb = off;                       // one B tile per pair of k-blocks (swizzled)
    off += ((max_l + 1) / 2) * tc_xtile(m, wbytes);
    p.zero = off;                     // (unused)
    p.xsum = off;                     // [max_l][8] f32 sum(x), then [max_l][8] f32 2^(E-13)
    off += 2 * max_l * 8 * 4;
    off = (off + 127) & ~127;         // (a TMA destination)
    p.sc = off;                       // affine: scales [128][S] then biases [128][S] (S = sc_words, or tc_sc_stride words a row); GGUF: block headers
    off += (wbytes == kWBytes) ? 2 * kRows * (sc_words ? sc_words : tc_sc_stride(max_l)) * 4 : max_l * kRows * 4;
    if (wbytes == kRows * 336) off += (max_l / 4 + 1) * kRows * 4;  // Q2_K: {d, dmin} of every block, after the scale bytes
    p.part = off;                     // rank 0 of the cluster: [splits][128][m] f32 partial sums of all k-slices
    off += splits * kRows * m * 4;
    off = (off + 15) & ~15;
    p.bars = off;                     // 33 mbarriers and the TMEM address
    off += 512;
    p.total = off + 1024;
    return p;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem descriptor {lo, hi}], u8 x s8 operands, s32 accumulate, K = 32.
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint32_t desc_lo, uint32_t desc_hi,
                                        uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        ".reg .b64 d;\n\t"
        "mov.b64 d, {%2, %3};\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], d, %4, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "r"(tmem_a), "r"(desc_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t *r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::
            "r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
        "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
// tcgen05.ld.32x32b of N consecutive columns of the warp's 32 lanes (N = 1, 2, 4, 8).
template <int N>
__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t *r);
template <>
__device__ __forceinline__ void tmem_ld<1>(uint32_t taddr, uint32_t *r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(r[0]) : "r"(taddr));
}
template <>
__device__ __forceinline__ void tmem_ld<2>(uint32_t taddr, uint32_t *r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x2.b32 {%0, %1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(taddr));
}
template <>
__device__ __forceinline__ void tmem_ld<4>(uint32_t taddr, uint32_t *r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(taddr));
}
template <>
__device__ __forceinline__ void tmem_ld<8>(uint32_t taddr, uint32_t *r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr));
}
template <int N>
struct IntC {
    static constexpr int value = N;
};
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire;" ::: "memory"); }
// Store into the shared memory of CTA `rank` of the cluster, at the address `local_addr` has there.
__device__ __forceinline__ void st_cluster_f32(uint32_t local_addr, uint32_t rank, float v) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}

__device__ __forceinline__ bool tc_wait(uint64_t *bar, uint32_t parity, int code) {
    if (mbar_wait(bar, parity)) return true;
    atomicExch(&g_qmv_tc_status, code);
    return false;
}
// The producer and the unpack warps run ahead of griddepcontrol.wait, so their waits can last as long as
// the previous kernel in the stream: polls spaced by a short sleep, and a limit of a few seconds.
__device__ __forceinline__ bool tc_wait_relaxed(uint64_t *bar, uint32_t parity, int code) {
    // in the steady state a wait is short: poll first, sleep between polls only when it lasts
    for (int i = 0; i < 64; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    if (mbar_wait_relaxed(bar, parity, 32, 1u << 26)) return true;
    atomicExch(&g_qmv_tc_status, code);
    return false;
}

// K order of the unpacked bytes.  4-bit: word j of a k-block (8 codes) becomes the words
// (c0, c2, c4, c6) and (c1, c3, c5, c7).  2-bit: word j (16 codes) becomes four words, word i holding
// (c_i, c_{4+i}, c_{8+i}, c_{12+i}).  The activation bytes are stored in the same order.
//
// GG = 4 (with BITS = 4): GGUF Q4_K matvec, f32 activations and output, one or two tokens
// (replaces lisa_gguf_q4_K_mv, crates/lisa-mlx/src/shaders/deepseek41/iq.metal:1239-1363; block layout
// crates/lisa-gguf/src/quant.rs:82-101).  A packed stage row is one 144-byte block = 4 k-blocks; the low
// nibbles of code bytes 32j .. 32j+31 are sub-block 2j, the high nibbles sub-block 2j+1, so the unpacked
// bytes are already in K order.  Each 32-element sub-block has its own scale and min: the two K=32 MMAs
// of a k-block accumulate into ONE D whose columns 0..7 see only sub-block 0 and columns 8..15 only
// sub-block 1, because the B tile is block diagonal (rows 0..7 hold activation bytes for k 0..31 and
// zeros for k 32..63, rows 8..15 the reverse).  An activation is three signed bytes,
// x_int = rn(x * 2^(21-E)) = 65536 p0 + 256 p1 + p2 (22 bits; exact on the reference's dyadic inputs),
// row 3t + q of a half holding piece q of token t.
//
// GG = 2 (with BITS = 2): GGUF Q2_K matvec, one token (replaces lisa_gguf_q2_K_mv, iq.metal:1130-1237; block
// layout quant.rs:64-80).  A packed stage row is four 84-byte blocks (16 k-blocks); the 64 elements of
// k-block kb4 of a block are the 2-bit fields at shifts 2*(kb4&1) and 2*(kb4&1)+1 of code bytes
// 32*(kb4/2) .. +31, so a pair of k-blocks is the four fields of the same 32 bytes.  Sub-blocks are 16
// elements: four per k-block, D columns 4*g + q (piece q), B rows 4*g + q non-zero only for k 16g .. 16g+15.
//
// NORM (affine only): the activations are rms_norm(bf16(x + r)) * w, computed by the staging warps
// (affine_qmv_fast_addnorm, crates/lisa-mlx/src/jit/matmul.rs:304-470 and its shader's rounding points:
// s = bf16(x + r), inv = 1 / sqrt(mean(s^2) + eps) in f32 over the whole row, normed = bf16(w * bf16(s * inv))).
// Every CTA reads the whole row of x and r once for the mean square (its own k-slice a second time for the
// values); the CTAs of the first row tile also write s (the new residual) and, if asked, the normed row.
//
// NORM = 2 (affine only): the activations are swiglu(x, nr) = bf16(bf16(g * bf16(sigmoid(g))) * u) with g = x and
// u = nr (crates/lisa-mlx/src/shaders/common/exact_header.metal:2-11): the down projection of an MLP reads the
// gate and up outputs directly; the CTAs of the first row tile write the activation row if asked (nnorm).
template <int BITS, int GG = 0, int NORM = 0>
__global__ void __launch_bounds__(kThreads, 2)
qmv_tc_kernel(const __grid_constant__ TcMaps maps, const TcParams p) {
    constexpr int ROWB = (GG == 4) ? 144 : (GG == 2) ? 336 : 128;  // bytes of a packed stage row
    constexpr int CPW = 32 / BITS;             // codes per word
    constexpr int KBW = (GG == 2) ? 16 : (128 * 8 / BITS) / 64;  // k-blocks per packed stage: 4 / 8 (affine), 4 (Q4_K), 16 (Q2_K)
    constexpr int KB_BYTES = 64 * BITS / 8;    // packed bytes of one row of a k-block: 32 / 16
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const TcPlan plan = tc_plan(p.wstages, p.max_l, p.splits, p.m, p.wbytes, p.sc_words);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + plan.bars);
    uint64_t *wp_full = bars;                      // [kMaxWStages]
    uint64_t *wp_empty = wp_full + kMaxWStages;    // [kMaxWStages], 8 unpack warps
    uint64_t *a_full = wp_empty + kMaxWStages;     // [kNP], 4 unpack warps of the pair's set
    uint64_t *done = a_full + kNP;                 // [kNP], tcgen05.commit of the pair's MMAs: D ready
    uint64_t *d_empty = done + kNP;                // [kNP], 4 epilogue warps: D read, hence A stage and D buffer free
    uint64_t *x_ready = d_empty + kNP;             // 4 epilogue warps
    uint64_t *sc_full = x_ready + 1;               // scales and biases of the tile (TMA)
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(sc_full + 1);

    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);  // warp-uniform for the compiler too
    const uint32_t rank = (p.splits > 1) ? cluster_ctarank() : 0u;
    int tile = blockIdx.x / p.splits;
    // the linear this row tile belongs to (one, unless the launch is the sibling form)
    int seg = 0;
    if (!GG && p.nseg > 1) {
        seg = (tile >= p.seg_tile[1]) ? 1 : 0;
        if (p.nseg > 2 && tile >= p.seg_tile[2]) seg = 2;
        tile -= (seg == 0) ? 0 : (seg == 1) ? p.seg_tile[1] : p.seg_tile[2];
    }
    // grouped form: this CTA's table entry; the k-slices of a tile (one cluster) share it, so they leave together
    int m_cta = p.m, g_row0 = 0, g_first = 0;
    if (!GG && p.g_tiles) {
        const int entry = tile / p.g_ntiles;
        pdl_wait();  // the table comes from the kernel before this one
        if (entry >= *p.g_count) return;
        const int4 t = p.g_tiles[entry];
        tile -= entry * p.g_ntiles;
        g_row0 = t.x * p.g_n;     // first row of the expert in the packed matrix
        g_first = t.y;            // first sorted row of the entry
        m_cta = t.z - t.y;
    }
    const float *xf_cta = p.xf;
    float *yf_cta = p.yf;
    if (GG && p.e_ids) {
        const int z = tile / p.e_ntiles;
        tile -= z * p.e_ntiles;
        pdl_wait();  // the ids may come from the kernel before this one
        const int e = p.e_ids[z];
        if (e < 0 || e >= p.e_experts) {  // the k-slices of a tile share the slot: the cluster leaves together
            if (rank == 0 && tid < kRows && tile * kRows + tid < p.n) p.yf[static_cast<size_t>(z) * p.n + tile * kRows + tid] = 0.f;
            return;
        }
        g_row0 = e * p.n;
        const int token = z / p.e_topk, slot = z - token * p.e_topk;
        xf_cta = p.xf + (static_cast<size_t>(token) * p.e_slots + slot % p.e_slots) * p.k;
        yf_cta = p.yf + static_cast<size_t>(z) * p.n;
    }
    const uint16_t *x_cta = p.x + static_cast<size_t>(g_first) * p.k;
    const CUtensorMap *map_w = &maps.m[seg];
    const int seg_n = (seg == 0) ? p.n : (seg == 1) ? p.seg_n[1] : p.seg_n[2];
    const int n0 = tile * kRows;
    // this CTA's k-slice, in packed stages and in k-blocks
    const int total_ws = (p.num_kb + KBW - 1) / KBW;
    const int ws0 = static_cast<int>((static_cast<int64_t>(rank) * total_ws) / p.splits);
    const int ws1 = static_cast<int>((static_cast<int64_t>(rank + 1) * total_ws) / p.splits);
    const int kb0 = ws0 * KBW;
    const int L = min(ws1 * KBW, p.num_kb) - kb0;  // k-blocks of this slice (>= 0)

    pdl_launch_dependents();
    if (warp == 0) {
        // one barrier per lane (26 of them): a single thread took ~500 clocks over the same initialisations
        constexpr int kNB = 2 * kMaxWStages + 3 * kNP + 2;
        static_assert(kNB <= 32, "one lane per barrier");
        if (lane < kNB) {
            uint32_t count = 1;                                                       // wp_full, done, sc_full
            if (lane >= kMaxWStages && lane < 2 * kMaxWStages) count = kUnpackWarps;  // wp_empty
            else if (lane >= 2 * kMaxWStages && lane < 2 * kMaxWStages + kNP) count = kUnpackWarps / 2;  // a_full
            else if (lane >= 2 * kMaxWStages + 2 * kNP && lane < 2 * kMaxWStages + 3 * kNP) count = kEpilogueWarps;  // d_empty
            else if (lane == 2 * kMaxWStages + 3 * kNP) count = kEpilogueWarps;       // x_ready
            mbar_init(&bars[lane], count);
        }
        mbar_fence_init();
        __syncwarp();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // first cluster phase: every CTA of the cluster is running (its shared memory exists) before any
    // partial sum is sent to rank 0; arrived here, waited for just before the stores
    if (p.splits > 1) cluster_arrive();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_a = tmem_base, tmem_d = tmem_base + kNP * 2 * kACols;
    const int P = (L + 1) / 2;  // pairs of k-blocks of this slice
    const bool compact = !GG && p.m <= 4;  // B tile of a pair in one 8-row group (see tc_xtile)
    const uint32_t xtile = compact ? 1024u : static_cast<uint32_t>(kXTile);
    const uint32_t ring32 = smem_u32(smem + plan.ring);
    const uint32_t xb32 = smem_u32(smem + plan.xb);
    float *xsum = reinterpret_cast<float *>(smem + plan.xsum);
    float *xscale = xsum + p.max_l * 8;
    uint32_t *sc = reinterpret_cast<uint32_t *>(smem + plan.sc);
    float *part = reinterpret_cast<float *>(smem + plan.part);

    // Staging of the affine activations, callable by any warp: thread `sidx` of `kstep` staging threads (whole
    // warps: the items of a (token, k-block) are adjacent lanes and share the group's exponent and sum through
    // shuffles).  The epilogue warps alone stage one to four tokens (the unpack warps meanwhile run ahead of
    // griddepcontrol.wait); with more tokens, and in the grouped form, the unpack warps help: the conversion is
    // then the longest phase of the CTA and the unpacked stages it delays are few.
    const bool helpers = !GG && (p.g_tiles != nullptr || p.m > 4);
    constexpr int kStageAll = (kEpilogueWarps + kUnpackWarps) * 32;
    auto stage_affine = [&](int sidx, int kstep) {
        // one item = one word's worth of codes (CPW activations) of one token: loaded, turned into
        // integer byte pairs in the K order of the unpacked words, stored swizzled; the items of a
        // (token, k-block) are adjacent lanes and share the group's exponent and sum through
        // shuffles.  Two rounds of loads are in flight at a time: this runs after
        // griddepcontrol.wait, on the critical path.
        constexpr int IPK = 64 / CPW;  // items per k-block: 8 / 4
        constexpr int NV = CPW / 8;    // 16-byte vectors per item: 1 / 2
        const int items = m_cta * L * IPK;
        const int per_token = L * IPK;
        float *red = part;  // NORM: [staging warps][8] partial sums of squares, then 1 / rms of token t at red[96 + t]
        if constexpr (NORM == 1) {
            auto rb = [](float f) { return bf16_bits_to_f32(f32_to_bf16_bits(f)); };
            const int bar_id = (kstep == kStageAll) ? 2 : 1;
            for (int t = 0; t < m_cta; ++t) {
                const uint4 *xr = reinterpret_cast<const uint4 *>(x_cta + static_cast<size_t>(t) * p.k);
                const uint4 *rr = reinterpret_cast<const uint4 *>(p.nr + static_cast<size_t>(t) * p.k);
                float acc = 0.f;
                // three chunks per trip, their six loads issued together (a 2560-wide row is one trip for 128 threads)
                for (int i0 = sidx; i0 < p.k / 8; i0 += 3 * kstep) {
                    uint4 a[3], b[3];
#pragma unroll
                    for (int u = 0; u < 3; ++u) {
                        const int i = i0 + u * kstep;
                        const bool in = i < p.k / 8;
                        a[u] = in ? __ldg(xr + i) : make_uint4(0, 0, 0, 0);
                        b[u] = in ? __ldg(rr + i) : make_uint4(0, 0, 0, 0);
                    }
#pragma unroll
                    for (int u = 0; u < 3; ++u) {
                        const uint32_t aw[4] = {a[u].x, a[u].y, a[u].z, a[u].w}, bw[4] = {b[u].x, b[u].y, b[u].z, b[u].w};
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const float s0 = rb(bf16_bits_to_f32(aw[q] & 0xffffu) + bf16_bits_to_f32(bw[q] & 0xffffu));
                            const float s1 = rb(__uint_as_float(aw[q] & 0xffff0000u) + __uint_as_float(bw[q] & 0xffff0000u));
                            acc = fmaf(s0, s0, acc);
                            acc = fmaf(s1, s1, acc);
                        }
                    }
                }
#pragma unroll
                for (int off = 16; off >= 1; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
                if (lane == 0) red[(sidx >> 5) * 8 + t] = acc;
            }
            asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(kstep) : "memory");
            if (sidx < m_cta) {
                float tot = 0.f;
                for (int w = 0; w < (kstep >> 5); ++w) tot += red[w * 8 + sidx];  // fixed order
                red[96 + sidx] = 1.0f / sqrtf(tot / static_cast<float>(p.k) + p.neps);
            }
            asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(kstep) : "memory");
        }
        auto load_item = [&](int item, uint4 (&v)[NV]) {
            if (item < items) {
                const int t = item / per_token, u = item - t * per_token;
                const size_t at = static_cast<size_t>(t) * p.k + kb0 * 64 + u * CPW;
                const uint4 *src = reinterpret_cast<const uint4 *>(x_cta + at);
#pragma unroll
                for (int i = 0; i < NV; ++i) v[i] = __ldg(src + i);
                if constexpr (NORM == 2) {
                    auto rb = [](float f) { return bf16_bits_to_f32(f32_to_bf16_bits(f)); };
                    auto act = [&](float gv, float uv) {  // the same function as moe_swiglu's
                        const float y = 1.0f / (1.0f + expf(fabsf(gv)));
                        const float sg = rb(gv < 0.f ? y : 1.0f - y);
                        return rb(gv * sg) * uv;
                    };
                    const bool writer = n0 == 0 && seg == 0 && p.nnorm;
#pragma unroll
                    for (int i = 0; i < NV; ++i) {
                        const uint4 uv = __ldg(reinterpret_cast<const uint4 *>(p.nr + at) + i);
                        const uint32_t gw[4] = {v[i].x, v[i].y, v[i].z, v[i].w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
                        uint32_t a[4];
#pragma unroll
                        for (int q = 0; q < 4; ++q)
                            a[q] = f32_to_bf16_bits(act(bf16_bits_to_f32(gw[q] & 0xffffu), bf16_bits_to_f32(uw[q] & 0xffffu))) |
                                   (f32_to_bf16_bits(act(__uint_as_float(gw[q] & 0xffff0000u), __uint_as_float(uw[q] & 0xffff0000u))) << 16);
                        v[i] = make_uint4(a[0], a[1], a[2], a[3]);
                        if (writer) reinterpret_cast<uint4 *>(p.nnorm + at)[i] = v[i];
                    }
                }
                if constexpr (NORM == 1) {
                    auto rb = [](float f) { return bf16_bits_to_f32(f32_to_bf16_bits(f)); };
                    const float inv = red[96 + t];
                    const bool writer = n0 == 0 && seg == 0;  // the first row tile's k-slices cover the row once
#pragma unroll
                    for (int i = 0; i < NV; ++i) {
                        const uint4 rv = __ldg(reinterpret_cast<const uint4 *>(p.nr + at) + i);
                        const uint4 wv = __ldg(reinterpret_cast<const uint4 *>(p.nw + kb0 * 64 + u * CPW) + i);
                        const uint32_t xw[4] = {v[i].x, v[i].y, v[i].z, v[i].w}, rw[4] = {rv.x, rv.y, rv.z, rv.w};
                        const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
                        uint32_t sw[4], nd[4];
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const float s0 = rb(bf16_bits_to_f32(xw[q] & 0xffffu) + bf16_bits_to_f32(rw[q] & 0xffffu));
                            const float s1 = rb(__uint_as_float(xw[q] & 0xffff0000u) + __uint_as_float(rw[q] & 0xffff0000u));
                            const float y0 = bf16_bits_to_f32(ww[q] & 0xffffu) * rb(s0 * inv);
                            const float y1 = __uint_as_float(ww[q] & 0xffff0000u) * rb(s1 * inv);
                            sw[q] = (__float_as_uint(s0) >> 16) | (__float_as_uint(s1) & 0xffff0000u);
                            nd[q] = f32_to_bf16_bits(y0) | (f32_to_bf16_bits(y1) << 16);
                        }
                        v[i] = make_uint4(nd[0], nd[1], nd[2], nd[3]);
                        if (writer) {
                            reinterpret_cast<uint4 *>(p.nsum + at)[i] = make_uint4(sw[0], sw[1], sw[2], sw[3]);
                            if (p.nnorm) reinterpret_cast<uint4 *>(p.nnorm + at)[i] = v[i];
                        }
                    }
                }
            }
        };
        auto store_item = [&](int item, const uint4 (&v)[NV]) {
            const bool in = item < items;
            const int t = in ? item / per_token : 0, u = in ? item - t * per_token : 0;
            const int kbl = u / IPK, j = u - kbl * IPK;
            uint32_t r[CPW / 2];
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                r[4 * i + 0] = in ? v[i].x : 0u;
                r[4 * i + 1] = in ? v[i].y : 0u;
                r[4 * i + 2] = in ? v[i].z : 0u;
                r[4 * i + 3] = in ? v[i].w : 0u;
            }
            float xf[CPW];
            float s = 0.f;
            uint32_t amax = 0;
#pragma unroll
            for (int i = 0; i < CPW / 2; ++i) {
                xf[2 * i] = bf16_bits_to_f32(r[i] & 0xffffu);
                xf[2 * i + 1] = __uint_as_float(r[i] & 0xffff0000u);
                s += xf[2 * i] + xf[2 * i + 1];
                amax = max(amax, max(r[i] & 0x7fffu, (r[i] >> 16) & 0x7fffu));
            }
#pragma unroll
            for (int off = 1; off < IPK; off <<= 1) {
                s += __shfl_xor_sync(0xffffffffu, s, off);
                amax = max(amax, __shfl_xor_sync(0xffffffffu, amax, off));
            }
            // E: biased exponent of the group's largest magnitude.  Groups below 2^-113 count as zero;
            // an infinity or NaN makes the group's factor NaN.
            const uint32_t e = amax >> 7;
            const bool live = e >= 14u && e < 255u;
            const float up = __uint_as_float((267u - e) << 23);  // 2^(13 - (E - 127))
            uint32_t hi[CPW / 4], lo[CPW / 4];
#pragma unroll
            for (int i = 0; i < CPW / 4; ++i) hi[i] = lo[i] = 0;
#pragma unroll
            for (int i = 0; i < CPW; ++i) {
                // rn(x * 2^(13-E)) through the mantissa of 1.5 * 2^23 (one full-rate FMA instead of a quarter-rate
                // conversion; the product is exact, the sum rounds to nearest even at unit weight)
                const int xi = live ? __float_as_int(fmaf(xf[i], up, 12582912.f)) - 0x4b400000 : 0;  // |xi| < 2^14
                const int h = (xi + 128) >> 8, l = xi - (h << 8);      // xi = 256 h + l, both signed bytes
                // byte position of element i in the unpacked order
                const int pos = (BITS == 4) ? ((i & 1) * 4 + (i >> 1)) : ((i & 3) * 4 + (i >> 2));
                hi[pos >> 2] |= (static_cast<uint32_t>(h) & 0xffu) << (8 * (pos & 3));
                lo[pos >> 2] |= (static_cast<uint32_t>(l) & 0xffu) << (8 * (pos & 3));
            }
            if (in) {
                // hi bytes: row t of the first group; lo bytes: row t of the second group, or row 4 + t of the first
                const uint32_t tile = xb32 + (kbl >> 1) * xtile;
                const int rl = compact ? t + 4 : t;
                const uint32_t rowh = tile + t * 128, rowl = tile + (compact ? 0u : 1024u) + rl * 128;
                const int par = kbl & 1;
                if (BITS == 4) {
                    const int chunk = par * 4 + (j >> 1), off8 = (j & 1) * 8;
                    asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(rowh + ((chunk ^ t) << 4) + off8), "r"(hi[0]), "r"(hi[1]) : "memory");
                    asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(rowl + ((chunk ^ rl) << 4) + off8), "r"(lo[0]), "r"(lo[1]) : "memory");
                } else {
                    const int chunk = par * 4 + j;
                    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(rowh + ((chunk ^ t) << 4)), "r"(hi[0]), "r"(hi[1]), "r"(hi[CPW / 4 - 2]), "r"(hi[CPW / 4 - 1]) : "memory");
                    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(rowl + ((chunk ^ rl) << 4)), "r"(lo[0]), "r"(lo[1]), "r"(lo[CPW / 4 - 2]), "r"(lo[CPW / 4 - 1]) : "memory");
                }
                if (j == 0) {
                    xsum[kbl * 8 + t] = s;
                    xscale[kbl * 8 + t] = live ? __uint_as_float((e - 13u) << 23)  // 2^(E - 127 - 13)
                                               : (e == 255u ? __uint_as_float(0x7fc00000u) : 0.f);
                }
            }
        };
        // (more rounds in flight -- four, or the three that a 2560-wide 4-bit slice needs -- were measured three times,
        // alone and with the helping warps: 2 % slower every time)
        for (int base = 0; base < items; base += 2 * kstep) {
            uint4 va[NV], vb[NV];
            load_item(base + sidx, va);
            load_item(base + kstep + sidx, vb);
            store_item(base + sidx, va);
            if (base + kstep < items) store_item(base + kstep + sidx, vb);
        }
    };

    if (warp == 0) {
        // ---------------- producer: packed codes do not depend on the previous kernel in the stream
        int s = 0;
        uint32_t ph = 1;
        auto issue = [&](int wi) {
            mbar_arrive_expect_tx(&wp_full[s], kRows * ROWB);
            // x coordinate in elements of the map: bytes, or 32-bit words for Q2_K
            tma_load_2d(ring32 + s * (kRows * ROWB), map_w, wi * (GG == 2 ? ROWB / 4 : ROWB), g_row0 + n0, &wp_full[s]);
            if (++s == p.wstages) { s = 0; ph ^= 1; }
        };
        const int ws_ring = min(ws1, ws0 + p.wstages);
        if (lane == 0)
            for (int wi = ws0; wi < ws_ring; ++wi) issue(wi);
        if (!GG && p.sc_tma && lane == 0) {
            // scales and biases of the tile: rows g_row0 + n0 .., groups from the 8-aligned index at or below kb0
            const uint32_t bytes = static_cast<uint32_t>(kRows * p.sc_box * 2);
            const uint32_t sc32 = smem_u32(sc);
            mbar_arrive_expect_tx(sc_full, 2 * bytes);
            tma_load_2d(sc32, &maps.s[seg], kb0 & ~7, g_row0 + n0, sc_full);
            tma_load_2d(sc32 + bytes, &maps.b[seg], kb0 & ~7, g_row0 + n0, sc_full);
        }
        if (lane == 0) {
            for (int wi = ws_ring; wi < ws1; ++wi) {
                if (!tc_wait_relaxed(&wp_empty[s], ph, 1)) break;
                issue(wi);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: the whole warp runs the loop (uniform waits and addresses), one
        // elected lane issues the four MMAs and the commit of a k-block
        if (L > 0) {
            // instruction descriptor: D s32 (2 << 4), A u8 (0 << 7), B s8 (1 << 10), K-major, M = 128, N = 16
            const uint32_t idesc = (2u << 4) | (0u << 7) | (1u << 10) | ((16u >> 3) << 17) | ((128u >> 4) << 24);
            // B descriptor, K-major, 128-byte swizzle: rows 0..7 (hi bytes) and rows 8..15 (lo bytes) are 1024 apart
            const uint32_t desc_hi = (1024u >> 4) | (1u << 14) | (2u << 29);
            pdl_wait();  // the bounded waits below start counting once the previous kernel is done
            bool ok = tc_wait(x_ready, 0, 2);
            int st = 0;
            uint32_t ph = 0;
            // One pair of k-blocks per trip (they share a B tile), their MMAs interleaved: the two K=32 steps
            // of a k-block accumulate into the same D; steps of different k-blocks can overlap.
            // the poll of the next pair's barrier is issued before this pair's MMAs and looked at after them
            bool ready = false;
            for (int pr = 0; pr < P; ++pr) {
                const bool two = 2 * pr + 1 < L;
                if (!__all_sync(0xffffffffu, ready)) ok = __all_sync(0xffffffffu, ok && tc_wait(&a_full[st], ph, 3));
                if (!ok) break;
                {
                    const int nst = (st + 1 == kNP) ? 0 : st + 1;
                    ready = (pr + 1 < P) && mbar_test_wait(&a_full[nst], nst == 0 ? ph ^ 1u : ph);
                }
                tc_fence_after();
                const uint32_t lo0 = ((xb32 + pr * xtile) >> 4) | (1u << 16), lo1 = lo0 + 4;  // +64 bytes: second k-block
                const uint32_t a0_addr = tmem_a + st * 2 * kACols, a1_addr = a0_addr + kACols;
                const uint32_t d0_addr = tmem_d + st * 2 * kDCols, d1_addr = d0_addr + kDCols;
                if (elect_one()) {
                    if (two) {
#pragma unroll
                        for (int ks = 0; ks < 2; ++ks) {
                            umma_ts(d0_addr, a0_addr + ks * 8, lo0 + ks * 2, desc_hi, idesc, ks > 0);
                            umma_ts(d1_addr, a1_addr + ks * 8, lo1 + ks * 2, desc_hi, idesc, ks > 0);
                        }
                    } else {
#pragma unroll
                        for (int ks = 0; ks < 2; ++ks) umma_ts(d0_addr, a0_addr + ks * 8, lo0 + ks * 2, desc_hi, idesc, ks > 0);
                    }
                    umma_commit(&done[st]);
                }
                __syncwarp();
                if (++st == kNP) { st = 0; ph ^= 1; }
            }
        }
    } else if (warp < 2 + kUnpackWarps) {
        // ---------------- unpack: thread = weight row = TMEM lane; one pair of k-blocks (128 codes) per trip
        const int uw = warp - 2;
        const int set = uw >> 2;       // pairs set, set + 2, ...
        const int quad = warp & 3;     // TMEM lanes 32*quad .. +31
        const int row = quad * 32 + lane;
        const int swz = row & 7;
        uint32_t kmask;
        asm volatile("mov.u32 %0, %1;" : "=r"(kmask) : "r"(BITS == 4 ? 0x0f0f0f0fu : 0x03030303u));
        const uint32_t row32 = ring32 + row * ROWB;
        const uint32_t a_lane = tmem_a + (static_cast<uint32_t>(quad * 32) << 16);
        bool ok = true;
        if (helpers) {
            asm volatile("bar.sync 2, %0;" ::"r"(kStageAll) : "memory");  // the tiles are zeroed
            pdl_wait();
            stage_affine(kEpilogueWarps * 32 + (tid - 64), kStageAll);
            fence_proxy_async_smem();
            asm volatile("bar.sync 2, %0;" ::"r"(kStageAll) : "memory");
        }
        // The TMEM stores of one pair complete while the next one is loaded and unpacked: their
        // completion wait, the hand-over to the MMA warp and the release of the packed stage are deferred
        // to the next trip (`pend_*`).
        bool pending = false;
        int pend_st = 0;
        auto finish_pending = [&]() {
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&a_full[pend_st]);
            pending = false;
        };
        constexpr int kChunksPerKb = KB_BYTES / 16;  // 16-byte chunks of one row of a k-block: 2 / 1
        // packed stage of the pair, kept incrementally (no division in the loop): slot s of the ring, the
        // parity of its `full` barrier, and the first k-block of the pair inside the stage (even)
        int sub = 2 * set, s = 0;
        uint32_t wpar = 0;
        for (int pr = set; pr < P; pr += 2) {
            const bool two = 2 * pr + 1 < L;
            if (sub < 4) {
                // first visit of this set to the stage.  If it has not landed yet, the previous pair is handed
                // over first (its hand-over is otherwise deferred to overlap the TMEM stores with this pair's
                // unpacking)
                if (!__all_sync(0xffffffffu, mbar_test_wait(&wp_full[s], wpar))) {
                    if (pending) finish_pending();
                    ok = __all_sync(0xffffffffu, tc_wait_relaxed(&wp_full[s], wpar, 4));
                }
            }
            if (!ok) break;
            // A stage and D buffer of this pair are free once the epilogue has read pair pr - kNP: polled here,
            // looked at after the unpacking (a poll takes about as long as the unpacking)
            const int stg = pr % kNP;
            const uint32_t dpar = ((pr / kNP) - 1) & 1;
            bool slot_free = true;
            if (pr >= kNP) slot_free = mbar_test_wait(&d_empty[stg], dpar);
            uint32_t o[32];
            if (GG && set == 0) {
                // first visit of this block of the row (a block is two pairs, this set takes the even ones): its
                // header moves from the packed stage to the epilogue's table before the pair is handed over
                const int bq = pr >> 1;
                if (GG == 4) {
                    const uint32_t src = row32 + s * (kRows * ROWB);
                    uint32_t h0, h1, h2, h3;
                    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(h0), "=r"(h1), "=r"(h2), "=r"(h3) : "r"(src));
                    reinterpret_cast<uint4 *>(sc)[bq * kRows + row] = make_uint4(h0, h1, h2, h3);
                } else {
                    const uint32_t src = row32 + s * (kRows * ROWB) + (sub >> 2) * 84;
                    uint32_t h[5];
#pragma unroll
                    for (int i = 0; i < 4; ++i) asm volatile("ld.shared.u32 %0, [%1];" : "=r"(h[i]) : "r"(src + 4 * i));
                    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(h[4]) : "r"(src + 80));
                    reinterpret_cast<uint4 *>(sc)[bq * kRows + row] = make_uint4(h[0], h[1], h[2], h[3]);
                    sc[p.max_l * kRows + bq * kRows + row] = h[4];
                }
            }
            if (GG == 2) {
                // the pair's 128 elements are the four 2-bit fields of 32 code bytes of one block
                const uint32_t blk = row32 + s * (kRows * ROWB) + (sub >> 2) * 84 + 16 + ((sub & 3) >> 1) * 32;
                uint32_t w[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w[i]) : "r"(blk + 4 * i));
#pragma unroll
                for (int f = 0; f < 4; ++f)
#pragma unroll
                    for (int i = 0; i < 8; ++i) o[8 * f + i] = (w[i] >> (2 * f)) & kmask;
            } else {
                const uint32_t base = row32 + s * (kRows * ROWB);
                uint32_t w[8 * kChunksPerKb];  // 16 (4-bit) / 8 (2-bit) words of the pair
#pragma unroll
                for (int c = 0; c < 2 * kChunksPerKb; ++c)
                    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                                 : "=r"(w[4 * c]), "=r"(w[4 * c + 1]), "=r"(w[4 * c + 2]), "=r"(w[4 * c + 3])
                                 : "r"(GG ? base + 16 + (sub * kChunksPerKb + c) * 16  // Q4_K: code bytes follow the 16-byte header, no swizzle
                                          : base + (((sub * kChunksPerKb + c) ^ swz) << 4)));
                if (GG == 4) {
                    // k-block h of the pair = code bytes 32h .. 32h+31 = words 8h .. 8h+7: low nibbles are its
                    // first 32 elements, high nibbles its last 32
#pragma unroll
                    for (int h = 0; h < 2; ++h)
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            o[16 * h + i] = w[8 * h + i] & kmask;
                            o[16 * h + 8 + i] = (w[8 * h + i] >> 4) & kmask;
                        }
                } else if (BITS == 4) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        o[2 * j + 0] = w[j] & kmask;         // codes 0, 2, 4, 6 of the word, one per byte
                        o[2 * j + 1] = (w[j] >> 4) & kmask;  // codes 1, 3, 5, 7
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j)
#pragma unroll
                        for (int i = 0; i < 4; ++i) o[4 * j + i] = (w[j] >> (2 * i)) & kmask;  // codes i, 4+i, 8+i, 12+i
                }
            }
            if (pending) finish_pending();
            if (!__all_sync(0xffffffffu, slot_free)) ok = __all_sync(0xffffffffu, tc_wait_relaxed(&d_empty[stg], dpar, 6));
            if (!ok) break;  // (warp-uniform: tcgen05.st is warp-wide)
            tc_fence_after();
            const uint32_t dst = a_lane + static_cast<uint32_t>(stg * 2 * kACols);
            tmem_st16(dst, o);
            if (two) tmem_st16(dst + kACols, o + 16);
            // last visit of the packed stage: back to the producer.  The TMEM stores above were issued with
            // the unpacked words as operands, so the shared-memory loads of the stage have completed (an
            // arrival placed right after the loads let the refill overtake them).
            if ((sub >= KBW - 4 || pr + 2 >= P) && lane == 0) mbar_arrive(&wp_empty[s]);
            pending = true;
            pend_st = stg;
            if (!kDeferHandOver) finish_pending();
            // next pair of this set: four k-blocks on
            sub += 4;
            while (sub >= KBW) {
                sub -= KBW;
                if (++s == p.wstages) { s = 0; wpar ^= 1; }
            }
        }
        if (pending) finish_pending();
    } else {
        // ---------------- staging, epilogue, reduction
        const int quad = warp & 3;
        const int row = quad * 32 + lane;
        const int et = tid - (2 + kUnpackWarps) * 32;  // 0..127
        const int grow = g_row0 + min(n0 + row, seg_n - 1);
        // scales and biases of (row, group) of the slice: weights, no dependency on the previous kernel
        if (GG) {
            // the block headers (Q4_K: {d, dmin, 6-bit scales and mins}; Q2_K: 16 scale/min bytes and {d, dmin}) come
            // with the packed stage: the unpack warp that first visits a block copies them to `sc` ([block][row])
        } else if (!p.sc_tma) {
            const uint16_t *sbase = (seg == 0) ? p.scales : (seg == 1) ? p.seg_scales[1] : p.seg_scales[2];
            const uint16_t *bbase = (seg == 0) ? p.biases : (seg == 1) ? p.seg_biases[1] : p.seg_biases[2];
            // as they lie in memory: row r of the scales at sc + r * S, of the biases kRows * S words further
            const int S = tc_sc_stride(p.max_l);
            if ((p.groups & 3) == 0 && (kb0 & 3) == 0) {
                // four groups per 8-byte asynchronous copy (a row holds a multiple of four groups, so the last copy
                // of a short slice stays inside the row); consecutive threads copy consecutive pieces of a row, so a
                // warp touches a few sectors per instruction instead of one per lane.  Nothing waits for the copies
                // until the activations are staged.
                const int c = (L + 3) / 4;
                const uint32_t sc32 = smem_u32(sc);
                int r = et / c, ch = et - r * c;            // this thread's first (row, piece)
                const int dr = (kEpilogueWarps * 32) / c, dch = (kEpilogueWarps * 32) - dr * c;
                for (; r < kRows;) {
                    const size_t at = static_cast<size_t>(g_row0 + min(n0 + r, seg_n - 1)) * p.groups + kb0 + 4 * ch;
                    const uint32_t dst = sc32 + (r * S + 2 * ch) * 4;
                    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(sbase + at) : "memory");
                    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst + kRows * S * 4), "l"(bbase + at) : "memory");
                    r += dr;
                    ch += dch;
                    if (ch >= c) { ch -= c; ++r; }
                }
                asm volatile("cp.async.commit_group;" ::: "memory");
            } else {
                const uint16_t *sr = sbase + static_cast<size_t>(grow) * p.groups + kb0;
                const uint16_t *br = bbase + static_cast<size_t>(grow) * p.groups + kb0;
                uint16_t *s16 = reinterpret_cast<uint16_t *>(sc + row * S), *b16 = reinterpret_cast<uint16_t *>(sc + (kRows + row) * S);
#pragma unroll 4
                for (int g = 0; g < L; ++g) {
                    s16[g] = __ldg(sr + g);
                    b16[g] = __ldg(br + g);
                }
            }
        }
        // activation tiles: zero everything (rows of tokens >= m and the half of an odd last tile stay zero)
        {
            uint4 *z = reinterpret_cast<uint4 *>(smem + plan.xb);
            const int n16 = ((L + 1) / 2) * static_cast<int>(xtile) / 16;
            for (int i = et; i < n16; i += kEpilogueWarps * 32) z[i] = make_uint4(0, 0, 0, 0);
        }
        if (helpers) asm volatile("bar.sync 2, %0;" ::"r"(kStageAll) : "memory");  // the unpack warps may write the tiles now
        else asm volatile("bar.sync 1, %0;" ::"r"(kEpilogueWarps * 32) : "memory");
        pdl_wait();  // activations come from the previous kernel
        if (!GG) stage_affine(et, helpers ? kStageAll : kEpilogueWarps * 32);
        if (GG) {
            // one item = 8 consecutive f32 activations of one token; the four items of a 32-element
            // sub-block are adjacent lanes and share its exponent and sum through shuffles
            const int items = p.m * L * 8;
            const int per_token = L * 8;
            constexpr int kStep = kEpilogueWarps * 32;
            for (int base = 0; base < items; base += kStep) {
                const int item = base + et;
                const bool in = item < items;
                const int t = in ? item / per_token : 0, u = in ? item - t * per_token : 0;
                const int kbl = u >> 3, j = u & 7;  // k-block, 8-element run of it
                float xv[8];
                if (in) {
                    const float4 *src = reinterpret_cast<const float4 *>(xf_cta + static_cast<size_t>(t) * p.k + (kb0 + kbl) * 64 + j * 8);
                    const float4 v0 = __ldg(src), v1 = __ldg(src + 1);
                    xv[0] = v0.x; xv[1] = v0.y; xv[2] = v0.z; xv[3] = v0.w;
                    xv[4] = v1.x; xv[5] = v1.y; xv[6] = v1.z; xv[7] = v1.w;
                } else {
#pragma unroll
                    for (int i = 0; i < 8; ++i) xv[i] = 0.f;
                }
                float sum = 0.f;
                uint32_t amax = 0;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    sum += xv[i];
                    amax = max(amax, __float_as_uint(xv[i]) & 0x7fffffffu);
                }
#pragma unroll
                for (int off = 1; off < (GG == 2 ? 2 : 4); off <<= 1) {  // items per sub-block: 2 (Q2_K) / 4 (Q4_K)
                    sum += __shfl_xor_sync(0xffffffffu, sum, off);
                    amax = max(amax, __shfl_xor_sync(0xffffffffu, amax, off));
                }
                // E: biased exponent of the sub-block's largest magnitude; below 2^-105 the sub-block counts
                // as zero, an infinity or NaN makes its factor NaN
                const uint32_t e = amax >> 23;
                const bool live = e >= 22u && e < 255u;
                const float up = __uint_as_float((275u - e) << 23);  // 2^(21 - (E - 127))
                uint32_t pc[3][2] = {{0, 0}, {0, 0}, {0, 0}};        // piece q, bytes of the 8 elements
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int xi = live ? __float2int_rn(xv[i] * up) : 0;  // |xi| < 2^22
                    const int r1 = (xi + 128) >> 8, p2 = xi - (r1 << 8);   // xi = 256 r1 + p2
                    const int p0 = (r1 + 128) >> 8, p1 = r1 - (p0 << 8);   // r1 = 256 p0 + p1
                    pc[0][i >> 2] |= (static_cast<uint32_t>(p0) & 0xffu) << (8 * (i & 3));
                    pc[1][i >> 2] |= (static_cast<uint32_t>(p1) & 0xffu) << (8 * (i & 3));
                    pc[2][i >> 2] |= (static_cast<uint32_t>(p2) & 0xffu) << (8 * (i & 3));
                }
                if (in && GG == 2) {
                    const int g4 = j >> 1;                      // 16-element sub-block of the k-block
                    const int par = kbl & 1;
                    const int chunk = par * 4 + g4, off8 = (j & 1) * 8;  // a sub-block is one 16-byte chunk
                    const uint32_t tile = xb32 + (kbl >> 1) * kXTile + (g4 >> 1) * 1024;  // rows 4*g4 + q
#pragma unroll
                    for (int q = 0; q < 3; ++q) {
                        const int r = 4 * (g4 & 1) + q;         // row within the 8-row group
                        asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(tile + r * 128 + ((chunk ^ r) << 4) + off8),
                                     "r"(pc[q][0]), "r"(pc[q][1]) : "memory");
                    }
                    if ((j & 1) == 0) {
                        xsum[kbl * 8 + g4] = sum;
                        xscale[kbl * 8 + g4] = live ? __uint_as_float((e - 21u) << 23)
                                                    : (e == 255u ? __uint_as_float(0x7fc00000u) : 0.f);
                    }
                } else if (in) {
                    const int h = j >> 2;                       // sub-block of the k-block
                    const int par = kbl & 1;                    // k-block of the pair (64-byte half of a B row)
                    const int chunk = par * 4 + 2 * h + ((j & 3) >> 1), off8 = (j & 1) * 8;
                    const uint32_t tile = xb32 + (kbl >> 1) * kXTile + h * 1024;  // rows 8h .. 8h+7
#pragma unroll
                    for (int q = 0; q < 3; ++q) {
                        const int r = 3 * t + q;                // row within the 8-row group
                        asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(tile + r * 128 + ((chunk ^ r) << 4) + off8),
                                     "r"(pc[q][0]), "r"(pc[q][1]) : "memory");
                    }
                    if ((j & 3) == 0) {
                        xsum[kbl * 8 + h * 4 + t] = sum;
                        xscale[kbl * 8 + h * 4 + t] = live ? __uint_as_float((e - 21u) << 23)  // 2^(E - 127 - 21)
                                                             : (e == 255u ? __uint_as_float(0x7fc00000u) : 0.f);
                    }
                }
            }
        }
        fence_proxy_async_smem();  // the MMA reads the tiles through the async proxy
        asm volatile("cp.async.wait_all;" ::: "memory");  // this thread's copies of scales and biases (other rows' too: hence before the barrier)
        if (helpers) asm volatile("bar.sync 2, %0;" ::"r"(kStageAll) : "memory");
        else asm volatile("bar.sync 1, %0;" ::"r"(kEpilogueWarps * 32) : "memory");
        if (lane == 0) mbar_arrive(x_ready);

        float rs[8];
#pragma unroll
        for (int t = 0; t < 8; ++t) rs[t] = 0.f;
        const uint32_t d_lane = tmem_d + (static_cast<uint32_t>(quad * 32) << 16);
        bool ok = true;
        // One pair of k-blocks per trip; only the columns of the tokens that exist are read (MT = m rounded
        // up to a power of two): hi bytes in columns [0, MT), lo bytes in columns [8, 8 + MT) of each D.
        const int sc_boff = kRows * (p.sc_tma ? p.sc_words : tc_sc_stride(p.max_l));  // words from a row's scales to its biases
        const uint32_t *sc_row = sc + row * (sc_boff / kRows) + (p.sc_tma ? (kb0 & 7) >> 1 : 0);
        auto run = [&](auto mt) {
            constexpr int MT = decltype(mt)::value;
            int st = 0;
            uint32_t ph = 0;
            bool ready = false;  // poll of the next pair's barrier, issued before this pair's arithmetic
            // staged scales and biases of this row, two groups a word, from the slice's first group on
            if (p.sc_tma) ok = __all_sync(0xffffffffu, tc_wait_relaxed(sc_full, 0, 9));
            const uint32_t *srow_e = sc_row;
            for (int pr = 0; pr < P; ++pr) {
                const bool two = 2 * pr + 1 < L;
                if (!__all_sync(0xffffffffu, ready)) ok = __all_sync(0xffffffffu, tc_wait_relaxed(&done[st], ph, 7));
                if (!ok) break;
                tc_fence_after();
                uint32_t c[2][2][MT];  // [k-block of the pair][hi, lo][token]
                const uint32_t dp = d_lane + st * 2 * kDCols;
                const uint32_t lo_col = compact ? 4u : 8u;  // accumulator column = row of the B tile
                tmem_ld<MT>(dp, c[0][0]);
                tmem_ld<MT>(dp + lo_col, c[0][1]);
                tmem_ld<MT>(dp + kDCols, c[1][0]);
                tmem_ld<MT>(dp + kDCols + lo_col, c[1][1]);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&d_empty[st]);
                {
                    const int nst = (st + 1 == kNP) ? 0 : st + 1;
                    ready = (pr + 1 < P) && mbar_test_wait(&done[nst], nst == 0 ? ph ^ 1u : ph);
                }
                const uint32_t sp = srow_e[pr], bp = srow_e[sc_boff + pr];  // scales / biases of the pair's two groups
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    if (h == 1 && !two) break;
                    const int kk = 2 * pr + h;
                    const float sv = h ? __uint_as_float(sp & 0xffff0000u) : bf16_bits_to_f32(sp & 0xffffu);
                    const float bv = h ? __uint_as_float(bp & 0xffff0000u) : bf16_bits_to_f32(bp & 0xffffu);
#pragma unroll
                    for (int t = 0; t < MT; ++t) {
                        // sum(q * x_int) = 256 * (hi column) + (lo column), below 2^24: exact as a float
                        const int qx = static_cast<int>(c[h][0][t]) * 256 + static_cast<int>(c[h][1][t]);
                        rs[t] = fmaf(sv * xscale[kk * 8 + t], static_cast<float>(qx), fmaf(bv, xsum[kk * 8 + t], rs[t]));
                    }
                }
                if (++st == kNP) { st = 0; ph ^= 1; }
            }
        };
        // Q4_K: columns 3t + q of each half of a D are the pieces of token t against one sub-block; its scale
        // d * sc_g and min dmin * m_g come from the staged block header (quant.rs:88-96)
        auto run_gguf = [&](auto mt) {
            constexpr int MT = decltype(mt)::value;  // columns read per half: 4 (one token) or 8 (two)
            const uint4 *hdr = reinterpret_cast<const uint4 *>(sc);
            int st = 0;
            uint32_t ph = 0;
            for (int pr = 0; pr < P; ++pr) {
                const bool two = 2 * pr + 1 < L;
                ok = __all_sync(0xffffffffu, tc_wait_relaxed(&done[st], ph, 7));
                if (!ok) break;
                tc_fence_after();
                uint32_t c[2][2][MT];  // [k-block of the pair][sub-block][piece columns]
                const uint32_t dp = d_lane + st * 2 * kDCols;
                tmem_ld<MT>(dp, c[0][0]);
                tmem_ld<MT>(dp + 8, c[0][1]);
                tmem_ld<MT>(dp + kDCols, c[1][0]);
                tmem_ld<MT>(dp + kDCols + 8, c[1][1]);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&d_empty[st]);
                const uint4 hd = hdr[((2 * pr) >> 2) * kRows + row];  // both k-blocks of a pair sit in one block
                float d, dmin;
                asm("{ .reg .b16 lo, hi; mov.b32 {lo, hi}, %2; cvt.f32.f16 %0, lo; cvt.f32.f16 %1, hi; }" : "=f"(d), "=f"(dmin) : "r"(hd.x));
#pragma unroll
                for (int hk = 0; hk < 2; ++hk) {
                    if (hk == 1 && !two) break;
                    const int kk = 2 * pr + hk;
#pragma unroll
                    for (int hs = 0; hs < 2; ++hs) {
                        const int g = 2 * (kk & 3) + hs, sh = 8 * (g & 3);
                        const uint32_t b0 = (hd.y >> sh) & 255u, b1 = (hd.z >> sh) & 255u, b2 = (hd.w >> sh) & 255u;
                        const uint32_t sq = (g < 4) ? (b0 & 63u) : ((b2 & 15u) | ((b0 >> 6) << 4));
                        const uint32_t mq = (g < 4) ? (b1 & 63u) : ((b2 >> 4) | ((b1 >> 6) << 4));
                        const float ds = d * static_cast<float>(sq), dm = dmin * static_cast<float>(mq);
#pragma unroll
                        for (int t = 0; t < MT / 4; ++t) {  // MT = 4: one token, MT = 8: two
                            // sum(q * x_int) = 65536 c0 + 256 c1 + c2
                            const float val = static_cast<float>(static_cast<int>(c[hk][hs][3 * t])) * 65536.f +
                                              static_cast<float>(static_cast<int>(c[hk][hs][3 * t + 1]) * 256 +
                                                                 static_cast<int>(c[hk][hs][3 * t + 2]));
                            rs[t] += ds * (val * xscale[kk * 8 + hs * 4 + t]) - dm * xsum[kk * 8 + hs * 4 + t];
                        }
                    }
                }
                if (++st == kNP) { st = 0; ph ^= 1; }
            }
        };
        // Q2_K, one token: columns 4*g + q of a D are piece q against sub-block g (16 elements) of the k-block
        auto run_q2k = [&]() {
            const uint4 *hdr = reinterpret_cast<const uint4 *>(sc);
            const uint32_t *dd = sc + p.max_l * kRows;
            int st = 0;
            uint32_t ph = 0;
            for (int pr = 0; pr < P; ++pr) {
                const bool two = 2 * pr + 1 < L;
                ok = __all_sync(0xffffffffu, tc_wait_relaxed(&done[st], ph, 7));
                if (!ok) break;
                tc_fence_after();
                uint32_t c[2][2][8];  // [k-block of the pair][rows 0..7 / 8..15][columns]
                const uint32_t dp = d_lane + st * 2 * kDCols;
                tmem_ld<8>(dp, c[0][0]);
                tmem_ld<8>(dp + 8, c[0][1]);
                tmem_ld<8>(dp + kDCols, c[1][0]);
                tmem_ld<8>(dp + kDCols + 8, c[1][1]);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&d_empty[st]);
                const int blk = (2 * pr) >> 2;
                const uint4 sb16 = hdr[blk * kRows + row];
                float d, dmin;
                asm("{ .reg .b16 lo, hi; mov.b32 {lo, hi}, %2; cvt.f32.f16 %0, lo; cvt.f32.f16 %1, hi; }" : "=f"(d), "=f"(dmin) : "r"(dd[blk * kRows + row]));
#pragma unroll
                for (int hk = 0; hk < 2; ++hk) {
                    if (hk == 1 && !two) break;
                    const int kk = 2 * pr + hk, kb4 = kk & 3;
#pragma unroll
                    for (int g4 = 0; g4 < 4; ++g4) {
                        // scale byte [half*8 + shift*2 + group], shift = 2*(kb4&1) + g4/2, group = g4&1
                        const int si = (kb4 >> 1) * 8 + (2 * (kb4 & 1) + (g4 >> 1)) * 2 + (g4 & 1);
                        const int wi4 = si >> 2;  // selects instead of a dynamically indexed array
                        const uint32_t sword = wi4 == 0 ? sb16.x : wi4 == 1 ? sb16.y : wi4 == 2 ? sb16.z : sb16.w;
                        const uint32_t sbyte = (sword >> (8 * (si & 3))) & 255u;
                        const float ds = d * static_cast<float>(sbyte & 15u), dm = dmin * static_cast<float>(sbyte >> 4);
                        const uint32_t *cc = c[hk][g4 >> 1] + 4 * (g4 & 1);
                        const float val = static_cast<float>(static_cast<int>(cc[0])) * 65536.f +
                                          static_cast<float>(static_cast<int>(cc[1]) * 256 + static_cast<int>(cc[2]));
                        rs[0] += ds * (val * xscale[kk * 8 + g4]) - dm * xsum[kk * 8 + g4];
                    }
                }
                if (++st == kNP) { st = 0; ph ^= 1; }
            }
        };
        if (GG == 2) {
            run_q2k();
        } else if (GG) {
            if (p.m == 1) run_gguf(IntC<4>{});
            else run_gguf(IntC<8>{});
        } else if (p.g_tiles) {
            // grouped form: the B tile layout is the plan's (eight tokens), the columns read are the entry's
            if (m_cta == 1) run(IntC<1>{});
            else if (m_cta == 2) run(IntC<2>{});
            else if (m_cta <= 4) run(IntC<4>{});
            else run(IntC<8>{});
        }
        else if (p.m == 1) run(IntC<1>{});
        else if (p.m == 2) run(IntC<2>{});
        else if (p.m <= 4) run(IntC<4>{});
        else run(IntC<8>{});
        // this slice's partial sums go to rank 0 of the cluster (slot [rank][row][t] of its `part`)
        if (p.splits > 1) cluster_wait();  // first phase: rank 0 is running
        const uint32_t slot = smem_u32(part) + ((rank * kRows + row) * p.m) * 4;
#pragma unroll
        for (int t = 0; t < 8; ++t) {
            if (t < p.m) {
                if (p.splits > 1) st_cluster_f32(slot + 4 * t, 0u, rs[t]);
                else part[row * p.m + t] = rs[t];
            }
        }
    }
    if (p.splits > 1 && warp < 2 + kUnpackWarps) cluster_wait();  // the other warps close the first phase too

    // ---------------- sum of the k-slices in rank order (cluster rank 0), store
    tc_fence_before();
    __syncthreads();
    if (p.splits > 1) {
        cluster_arrive();            // second phase: this CTA's partial sums are on their way (release)
        if (rank == 0) cluster_wait();  // rank 0 alone waits for all of them; the others may leave
    }
    if (rank == 0 && warp >= 2 + kUnpackWarps) {
        const int row = (warp & 3) * 32 + lane;
        if (n0 + row < seg_n) {
            // sibling form: the segment's own [m, n] output; else outs[0 .. nout) with pitch ldy
            uint16_t *out0 = (seg == 0) ? p.out[0] : (seg == 1) ? p.seg_out[1] : p.seg_out[2];
            const int ldy = (p.nseg > 1) ? seg_n : p.ldy;
#pragma unroll
            for (int t = 0; t < 8; ++t) {
                if (t < m_cta) {
                    float tot = 0.f;
                    for (int r = 0; r < p.splits; ++r) tot += part[(r * kRows + row) * p.m + t];
                    const size_t at = static_cast<size_t>(g_first + t) * ldy + p.col0 + n0 + row;
                    if (GG) {
                        // f32 out; the N-sharded form stores the column block into every rank's output (plain stores)
                        yf_cta[at] = tot;
                        for (int o = 1; o < p.nout; ++o) reinterpret_cast<float *>(p.out[o])[at] = tot;
                    } else if (p.nseg > 1 && p.seg_nout > 0) {
                        const uint16_t v = static_cast<uint16_t>(f32_to_bf16_bits(tot));
                        const size_t ag = static_cast<size_t>(t) * p.seg_ldy[seg] + p.seg_col0[seg] + n0 + row;
                        for (int o = 0; o < p.seg_nout; ++o) p.seg_outs[seg][o][ag] = v;  // peers' memory included
                    } else {
                        const uint16_t v = static_cast<uint16_t>(f32_to_bf16_bits(tot));
                        out0[at] = v;
                        for (int o = 1; o < p.nout; ++o) p.out[o][at] = v;  // plain stores, peers' memory included
                    }
                }
            }
        }
    }
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

}  // namespace

// Shapes the kernel takes: group size 64, packed rows addressable by a tensor map, and a k-slice whose
// staging fits half an SM's shared memory.  `m` rows are wanted; `mc` (<= 8) is how many one launch takes.
static bool tc_make_plan(int64_t n, int64_t k, int group_size, int bits, int m, TcParams &p, int &smem, int &grid, int &mc,
                         int wbytes = kWBytes, int kbw_stage = 0, int64_t tiles_all = 0) {
    if (bits != 2 && bits != 4) return false;
    if (group_size != 64 || k % 64 != 0 || m < 1) return false;
    if ((k * bits / 8) % 16 != 0 || (k * 2) % 16 != 0) return false;
    const int kbw = kbw_stage ? kbw_stage : (128 * 8 / bits) / 64;  // k-blocks per packed stage
    const int num_kb = static_cast<int>(k / 64);
    const int total_ws = (num_kb + kbw - 1) / kbw;
    const int64_t tiles = tiles_all ? tiles_all : (n + kRows - 1) / kRows;  // row tiles of the launch
    int budget = max_smem_optin() / 2 - 2048;  // two CTAs (of consecutive kernels) per SM
    if (wbytes == kRows * 336) budget = max_smem_optin() - 2048;  // Q2_K stages are 42 KB: one CTA per SM, two stages or more
    // as many k-slices as keep the grid near one CTA per SM; more when the slice would not fit
    int splits = 1;
    while (splits < 8 && tiles * (splits * 2) <= sm_count() + 20 && splits * 2 <= total_ws) splits *= 2;
    // The number of k-slices must not depend on m (a row's result is the sum of its slices in rank order,
    // and a row of an m-row call has to equal its own m = 1 call bit for bit): it is the first one whose
    // shallowest ring fits beside the staging of ONE token; a call with more rows than fit beside that
    // runs as several launches of fewer rows, each with the same slices.
    for (; splits <= 8; splits *= 2) {
        if (splits > total_ws) break;
        const int max_ws = (total_ws + splits - 1) / splits;
        const int max_l = std::min(max_ws * kbw, num_kb);
        const int ws_min = std::min(2, max_ws);
        // scales and biases by TMA when their rows are whole 16-byte pieces; the box covers the longest slice, plus
        // four groups when some slice starts at a group index that is 4 mod 8
        static const bool sc_tma_on = [] { const char *v = std::getenv("LISA_TC_SC_TMA"); return !(v && v[0] == '0'); }();
        const bool sc_tma = sc_tma_on && wbytes == kWBytes && num_kb % 8 == 0;
        bool sc_off = false;
        for (int r = 0; r < splits; ++r) sc_off = sc_off || ((static_cast<int64_t>(r) * total_ws / splits) * kbw) % 8 != 0;
        const int sc_box = (max_l + (sc_off ? 4 : 0) + 7) / 8 * 8;
        const int scw = sc_tma ? sc_box / 2 : 0;
        if (tc_plan(ws_min, max_l, splits, 1, wbytes, scw).total > budget) continue;
        mc = std::min(m, 8);
        while (mc > 1 && tc_plan(ws_min, max_l, splits, mc, wbytes, scw).total > budget) mc = (mc + 1) / 2;
        for (int ws = std::min(kMaxWStages, max_ws); ws >= ws_min; --ws) {
            const TcPlan plan = tc_plan(ws, max_l, splits, mc, wbytes, scw);
            if (plan.total <= budget) {
                p.sc_tma = sc_tma ? 1 : 0;
                p.sc_box = sc_box;
                p.sc_words = scw;
                p.splits = splits;
                p.wstages = ws;
                p.max_l = max_l;
                p.num_kb = num_kb;
                p.groups = num_kb;
                p.wbytes = wbytes;
                smem = plan.total;
                grid = static_cast<int>(tiles * splits);
                return true;
            }
        }
        return false;
    }
    return false;
}

bool qmv_tc_supported(int64_t m, int64_t k, int64_t n, int group_size, int bits) {
    TcParams p{};
    int smem = 0, grid = 0, mc = 0;
    if (n < 1 || n > (1 << 24) || m < 1) return false;
    return tc_make_plan(n, k, group_size, bits, static_cast<int>(std::min<int64_t>(m, 8)), p, smem, grid, mc);
}

static int affine_tensor_map(CUtensorMap *map, const uint32_t *w, int64_t n, int64_t k, int bits) {
    const uint64_t row_bytes = static_cast<uint64_t>(k) * bits / 8;
    const uint64_t dims[2] = {row_bytes, static_cast<uint64_t>(n)};
    const uint64_t strides[1] = {row_bytes};
    const uint32_t box[2] = {128, kRows};
    return make_tensor_map(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, w, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

// Tensor maps of one segment's scales and biases, [rows, groups] bf16, box sc_box groups x 128 rows, no swizzle.
static int scale_tensor_maps(TcMaps &maps, int seg, const void *scales, const void *biases, int64_t rows, int64_t groups, int box) {
    const uint64_t dims[2] = {static_cast<uint64_t>(groups), static_cast<uint64_t>(rows)};
    const uint64_t strides[1] = {static_cast<uint64_t>(groups) * 2};
    const uint32_t bx[2] = {static_cast<uint32_t>(box), kRows};
    int rc = make_tensor_map(&maps.s[seg], CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, scales, dims, strides, bx, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc != LISA_OK) return rc;
    return make_tensor_map(&maps.b[seg], CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, biases, dims, strides, bx, CU_TENSOR_MAP_SWIZZLE_NONE);
}

static int tc_launch_kernel(cudaStream_t stream, int bits, const TcMaps &maps, const TcParams &p, int grid, int smem, unsigned flags) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (p.splits > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = p.splits;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    if (flags & LISA_FLAG_PDL) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    if (p.nr && !p.nw && bits == 4) {  // (no norm weight: the second input is the up projection of a SwiGLU)
        LISA_CUDA_TRY(cudaFuncSetAttribute(qmv_tc_kernel<4, 0, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        LISA_CUDA_TRY(cudaLaunchKernelEx(&cfg, qmv_tc_kernel<4, 0, 2>, maps, p));
    } else if (p.nr && !p.nw) {
        LISA_CUDA_TRY(cudaFuncSetAttribute(qmv_tc_kernel<2, 0, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        LISA_CUDA_TRY(cudaLaunchKernelEx(&cfg, qmv_tc_kernel<2, 0, 2>, maps, p));
    } else if (p.nr && bits == 4) {
        LISA_CUDA_TRY(cudaFuncSetAttribute(qmv_tc_kernel<4, 0, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        LISA_CUDA_TRY(cudaLaunchKernelEx(&cfg, qmv_tc_kernel<4, 0, 1>, maps, p));
    } else if (p.nr) {
        LISA_CUDA_TRY(cudaFuncSetAttribute(qmv_tc_kernel<2, 0, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        LISA_CUDA_TRY(cudaLaunchKernelEx(&cfg, qmv_tc_kernel<2, 0, 1>, maps, p));
    } else if (bits == 4) {
        LISA_CUDA_TRY(cudaFuncSetAttribute(qmv_tc_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        LISA_CUDA_TRY(cudaLaunchKernelEx(&cfg, qmv_tc_kernel<4>, maps, p));
    } else {
        LISA_CUDA_TRY(cudaFuncSetAttribute(qmv_tc_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        LISA_CUDA_TRY(cudaLaunchKernelEx(&cfg, qmv_tc_kernel<2>, maps, p));
    }
    count_launch();
    return LISA_OK;
}

static void tc_set_norm(TcParams &p, const TcNormArgs *norm, int64_t done, int64_t k) {
    if (!norm) return;
    p.nr = reinterpret_cast<const uint16_t *>(norm->residual) + done * k;
    p.nw = reinterpret_cast<const uint16_t *>(norm->weight);
    p.neps = norm->eps;
    p.nsum = norm->sum ? reinterpret_cast<uint16_t *>(norm->sum) + done * k : nullptr;
    p.nnorm = norm->normed ? reinterpret_cast<uint16_t *>(norm->normed) + done * k : nullptr;
}

static int qmv_tc_launch(cudaStream_t stream, const void *x, int64_t m, int64_t k, const uint32_t *w, const void *scales,
                         const void *biases, int64_t n, int group_size, int bits, void *const *outs, int nout, int64_t ldy,
                         int64_t col0, unsigned flags, const TcNormArgs *norm = nullptr) {
    const uint16_t *xp = reinterpret_cast<const uint16_t *>(x);
    TcMaps maps{};
    {
        const int rc = affine_tensor_map(&maps.m[0], w, n, k, bits);
        if (rc != LISA_OK) return rc;
    }
    int mc = 0;
    for (int64_t done = 0; done < m; done += mc) {
        TcParams p{};
        int smem = 0, grid = 0;
        if (!tc_make_plan(n, k, group_size, bits, static_cast<int>(std::min<int64_t>(m - done, 8)), p, smem, grid, mc))
            return fail(LISA_ERR_UNSUPPORTED, "qmv_tc: shape not supported");
        if (p.sc_tma && done == 0) {
            const int rc = scale_tensor_maps(maps, 0, scales, biases, n, k / 64, p.sc_box);
            if (rc != LISA_OK) return rc;
        }
        p.scales = reinterpret_cast<const uint16_t *>(scales);
        p.biases = reinterpret_cast<const uint16_t *>(biases);
        p.x = xp + done * k;
        p.nout = nout;
        p.ldy = static_cast<int>(ldy);
        p.col0 = static_cast<int>(col0);
        for (int o = 0; o < nout; ++o) p.out[o] = reinterpret_cast<uint16_t *>(outs[o]) + done * ldy;
        p.n = static_cast<int>(n);
        p.k = static_cast<int>(k);
        p.m = mc;
        tc_set_norm(p, norm, done, k);
        const int rc = tc_launch_kernel(stream, bits, maps, p, grid, smem, flags);
        if (rc != LISA_OK) return rc;
    }
    return LISA_OK;
}

// Grouped form: `rows` sorted rows, expert of row r = the table entry that covers r; entries hold at most
// `*bt_out` rows (the caller builds the table with that height after asking qmv_tc_grouped_rows).
static int64_t grouped_live_tiles(int64_t rows, int64_t experts, int64_t n, int count) {
    // what the split heuristic sees: the row tiles of the experts that can be live, not the table's capacity
    return std::max<int64_t>(1, std::min(rows, experts)) * ((n + kRows - 1) / kRows) * count;
}

int qmv_tc_grouped_rows(int64_t rows, int64_t experts, int64_t k, int64_t n, int group_size, int bits, int count) {
    TcParams p{};
    int smem = 0, grid = 0, mc = 0;
    if (n < 1 || n > (1 << 24) || count < 1 || count > kMaxSeg) return 0;
    if (!tc_make_plan(n, k, group_size, bits, 8, p, smem, grid, mc, kWBytes, 0, grouped_live_tiles(rows, experts, n, count))) return 0;
    return mc;
}

// `count` sibling linears (1 to 3, the same n and k: gate | up of a routed block) in one launch: segment i owns the
// i-th block of max_tiles * ntiles row tiles of the grid, and inside its block the tiles are (entry, row tile).
int qmv_tc_grouped(cudaStream_t stream, const void *x, int64_t rows, int64_t k, int count, const uint32_t *const *w,
                   const void *const *scales, const void *const *biases, int64_t experts, int64_t n, int group_size, int bits,
                   void *const *y, int bt, const int32_t *tiles, const int32_t *tile_count, int64_t max_tiles) {
    if (count < 1 || count > kMaxSeg) return fail(LISA_ERR_UNSUPPORTED, "qmv_tc_grouped: one to three linears per launch");
    TcMaps maps{};
    for (int i = 0; i < count; ++i) {
        const int rc = affine_tensor_map(&maps.m[i], w[i], experts * n, k, bits);
        if (rc != LISA_OK) return rc;
    }
    const int64_t ntiles = (n + kRows - 1) / kRows;
    TcParams p{};
    int smem = 0, grid = 0, mc = 0;
    if (!tc_make_plan(n, k, group_size, bits, 8, p, smem, grid, mc, kWBytes, 0, grouped_live_tiles(rows, experts, n, count)) || mc != bt)
        return fail(LISA_ERR_UNSUPPORTED, "qmv_tc_grouped: shape not supported");
    if (max_tiles * ntiles * count * p.splits > (1ll << 30)) return fail(LISA_ERR_OVERFLOW, "qmv_tc_grouped: grid too large");
    p.x = reinterpret_cast<const uint16_t *>(x);
    p.nout = 1;
    p.ldy = static_cast<int>(n);
    p.col0 = 0;
    p.n = static_cast<int>(n);
    p.k = static_cast<int>(k);
    p.m = bt;
    p.nseg = count;
    for (int i = 0; i < count; ++i) {
        p.seg_tile[i] = static_cast<int>(i * max_tiles * ntiles);
        p.seg_n[i] = static_cast<int>(n);
        p.seg_scales[i] = reinterpret_cast<const uint16_t *>(scales[i]);
        p.seg_biases[i] = reinterpret_cast<const uint16_t *>(biases[i]);
        p.seg_out[i] = reinterpret_cast<uint16_t *>(y[i]);
        if (p.sc_tma) {
            const int rc = scale_tensor_maps(maps, i, scales[i], biases[i], experts * n, k / 64, p.sc_box);
            if (rc != LISA_OK) return rc;
        }
    }
    p.scales = p.seg_scales[0];
    p.biases = p.seg_biases[0];
    p.out[0] = p.seg_out[0];
    p.g_tiles = reinterpret_cast<const int4 *>(tiles);
    p.g_count = tile_count;
    p.g_ntiles = static_cast<int>(ntiles);
    p.g_n = static_cast<int>(n);
    return tc_launch_kernel(stream, bits, maps, p, static_cast<int>(max_tiles * ntiles * count * p.splits), smem, 0);
}

int qmv_tc(cudaStream_t stream, const void *x, int64_t m, int64_t k, const uint32_t *w, const void *scales,
           const void *biases, int64_t n, int group_size, int bits, void *y, unsigned flags, const TcNormArgs *norm) {
    void *outs[1] = {y};
    return qmv_tc_launch(stream, x, m, k, w, scales, biases, n, group_size, bits, outs, 1, n, 0, flags, norm);
}

// N-sharded GEMV fused with its all-gather: this rank's rows [col0, col0 + n) of an n_total-row linear,
// stored as columns of every rank's [m, n_total] output (outs[0 .. world), peer pointers included).
int qmv_tc_allgather(cudaStream_t stream, const void *x, int64_t m, int64_t k, const uint32_t *w, const void *scales,
                     const void *biases, int64_t n, int group_size, int bits, void *const *outs, int world,
                     int64_t n_total, int64_t col0, unsigned flags) {
    return qmv_tc_launch(stream, x, m, k, w, scales, biases, n, group_size, bits, outs, world, n_total, col0, flags);
}

// Sibling linears: `count` (2 or 3) weight matrices with the same k, group size and bit width applied to the
// same x in ONE launch (q|k|v, gate|up of a decoder layer); linear i writes its own [m, n[i]] output.
bool qmv_tc_multi_supported(int64_t m, int64_t k, int count, const int64_t *n, int group_size, int bits) {
    if (count < 2 || count > kMaxSeg || m < 1) return false;
    int64_t tiles = 0;
    for (int i = 0; i < count; ++i) {
        if (n[i] < 1 || n[i] > (1 << 24)) return false;
        tiles += (n[i] + kRows - 1) / kRows;
    }
    TcParams p{};
    int smem = 0, grid = 0, mc = 0;
    return tc_make_plan(n[0], k, group_size, bits, static_cast<int>(std::min<int64_t>(m, 8)), p, smem, grid, mc, kWBytes, 0, tiles);
}

// With `world` > 0 the launch is also the all-gather of N-sharded siblings: y holds count x world pointers
// (linear i, rank r at y[i * world + r]), linear i's rows are columns [col0[i], col0[i] + n[i]) of n_total[i].
int qmv_tc_multi(cudaStream_t stream, const void *x, int64_t m, int64_t k, int count, const uint32_t *const *w,
                 const void *const *scales, const void *const *biases, const int64_t *n, int group_size, int bits,
                 void *const *y, unsigned flags, int world, const int64_t *n_total, const int64_t *col0, const TcNormArgs *norm) {
    if (count < 2 || count > kMaxSeg) return fail(LISA_ERR_UNSUPPORTED, "qmv_tc_multi: two or three linears per launch");
    const uint16_t *xp = reinterpret_cast<const uint16_t *>(x);
    TcMaps maps{};
    int64_t tiles = 0;
    int first[kMaxSeg] = {0, 0, 0};
    for (int i = 0; i < count; ++i) {
        const int rc = affine_tensor_map(&maps.m[i], w[i], n[i], k, bits);
        if (rc != LISA_OK) return rc;
        first[i] = static_cast<int>(tiles);
        tiles += (n[i] + kRows - 1) / kRows;
    }
    int mc = 0;
    for (int64_t done = 0; done < m; done += mc) {
        TcParams p{};
        int smem = 0, grid = 0;
        if (!tc_make_plan(n[0], k, group_size, bits, static_cast<int>(std::min<int64_t>(m - done, 8)), p, smem, grid, mc, kWBytes, 0, tiles))
            return fail(LISA_ERR_UNSUPPORTED, "qmv_tc_multi: shape not supported");
        if (p.sc_tma && done == 0) {
            for (int i = 0; i < count; ++i) {
                const int rc = scale_tensor_maps(maps, i, scales[i], biases[i], n[i], k / 64, p.sc_box);
                if (rc != LISA_OK) return rc;
            }
        }
        p.x = xp + done * k;
        p.k = static_cast<int>(k);
        p.m = mc;
        p.nout = 1;
        p.col0 = 0;
        p.nseg = count;
        for (int i = 0; i < count; ++i) {
            p.seg_tile[i] = first[i];
            p.seg_n[i] = static_cast<int>(n[i]);
            p.seg_scales[i] = reinterpret_cast<const uint16_t *>(scales[i]);
            p.seg_biases[i] = reinterpret_cast<const uint16_t *>(biases[i]);
            if (world > 0) {
                p.seg_ldy[i] = static_cast<int>(n_total[i]);
                p.seg_col0[i] = static_cast<int>(col0[i]);
                for (int r = 0; r < world; ++r)
                    p.seg_outs[i][r] = reinterpret_cast<uint16_t *>(y[i * world + r]) + done * n_total[i];
                p.seg_out[i] = p.seg_outs[i][0];
            } else {
                p.seg_out[i] = reinterpret_cast<uint16_t *>(y[i]) + done * n[i];
            }
        }
        p.seg_nout = world > 0 ? world : 0;
        p.scales = p.seg_scales[0];
        p.biases = p.seg_biases[0];
        p.out[0] = p.seg_out[0];
        p.n = p.seg_n[0];
        p.ldy = p.seg_n[0];
        tc_set_norm(p, norm, done, k);
        const int rc = tc_launch_kernel(stream, bits, maps, p, grid, smem, flags);
        if (rc != LISA_OK) return rc;
    }
    return LISA_OK;
}

// GGUF matvec through the same kernel (f32 in, f32 out): Q4_K for one or two tokens, Q2_K for one.
static bool gguf_tc_plan(int format, int64_t tokens, int64_t rows, int64_t row_bytes, TcParams &p, int &smem, int &grid,
                         int64_t tiles_all = 0) {
    if (tokens < 1 || rows < 1 || rows > (1 << 24)) return false;
    int mc = 0;
    if (format == LISA_GGUF_Q4_K) {
        if (tokens > 2 || row_bytes % 144 != 0) return false;
        if (!tc_make_plan(rows, row_bytes / 144 * 256, 64, 4, static_cast<int>(tokens), p, smem, grid, mc, kRows * 144, 4, tiles_all)) return false;
    } else if (format == LISA_GGUF_Q2_K) {
        if (tokens > 1 || row_bytes % 336 != 0) return false;  // whole stage rows of four blocks
        if (!tc_make_plan(rows, row_bytes / 84 * 256, 64, 2, 1, p, smem, grid, mc, kRows * 336, 16, tiles_all)) return false;
    } else {
        return false;
    }
    return mc == tokens;
}

bool qmv_tc_gguf_supported(int format, int64_t tokens, int64_t rows, int64_t row_bytes) {
    TcParams p{};
    int smem = 0, grid = 0;
    return gguf_tc_plan(format, tokens, rows, row_bytes, p, smem, grid);
}

int qmv_tc_gguf(cudaStream_t stream, int format, const uint8_t *w, int64_t rows, int64_t row_bytes, const float *x,
                int64_t tokens, float *y) {
    float *outs[1] = {y};
    return qmv_tc_gguf_allgather(stream, format, w, rows, row_bytes, x, tokens, outs, 1, rows, 0);
}

// Expert form (deepseek41::expert_matvec): every (token, j) slot is a one-token matvec against the rows of its own
// expert.  One launch over all slots; meant for decode-sized id tables.
bool qmv_tc_gguf_expert_supported(int format, int64_t slots_total, int64_t experts, int64_t rows, int64_t row_bytes) {
    TcParams p{};
    int smem = 0, grid = 0;
    if (slots_total < 1 || slots_total > 256 || experts * rows > (1ll << 31) - kRows) return false;
    return gguf_tc_plan(format, 1, rows, row_bytes, p, smem, grid, slots_total * ((rows + kRows - 1) / kRows));
}

int qmv_tc_gguf_expert(cudaStream_t stream, int format, const uint8_t *w, int64_t experts, int64_t rows, int64_t row_bytes,
                       const float *x, int64_t tokens, int64_t slots, const int32_t *ids, int64_t top_k, float *y) {
    const bool q4 = format == LISA_GGUF_Q4_K;
    const int64_t k = row_bytes / (q4 ? 144 : 84) * 256, z = tokens * top_k, ntiles = (rows + kRows - 1) / kRows;
    TcParams p{};
    int smem = 0, grid = 0;
    if (!gguf_tc_plan(format, 1, rows, row_bytes, p, smem, grid, z * ntiles))
        return fail(LISA_ERR_UNSUPPORTED, "gguf expert matvec: shape not supported by the tensor-memory kernel");
    TcMaps maps{};
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(q4 ? row_bytes : row_bytes / 4), static_cast<uint64_t>(experts * rows)};
        const uint64_t strides[1] = {static_cast<uint64_t>(row_bytes)};
        const uint32_t box[2] = {static_cast<uint32_t>(q4 ? 144 : 84), kRows};
        const int rc = make_tensor_map(&maps.m[0], q4 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, w, dims,
                                       strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
        if (rc != LISA_OK) return rc;
    }
    p.xf = x;
    p.yf = y;
    p.wg = w;
    p.row_bytes = row_bytes;
    p.n = static_cast<int>(rows);
    p.k = static_cast<int>(k);
    p.m = 1;
    p.nout = 1;
    p.out[0] = reinterpret_cast<uint16_t *>(y);
    p.ldy = static_cast<int>(rows);
    p.col0 = 0;
    p.e_ids = ids;
    p.e_experts = static_cast<int>(experts);
    p.e_slots = static_cast<int>(slots);
    p.e_topk = static_cast<int>(top_k);
    p.e_ntiles = static_cast<int>(ntiles);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(z * ntiles * p.splits));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    int na = 0;
    if (p.splits > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = p.splits;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    if (q4) {
        LISA_CUDA_TRY(cudaFuncSetAttribute(qmv_tc_kernel<4, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        LISA_CUDA_TRY(cudaLaunchKernelEx(&cfg, qmv_tc_kernel<4, 4>, maps, p));
    } else {
        LISA_CUDA_TRY(cudaFuncSetAttribute(qmv_tc_kernel<2, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        LISA_CUDA_TRY(cudaLaunchKernelEx(&cfg, qmv_tc_kernel<2, 2>, maps, p));
    }
    count_launch();
    return LISA_OK;
}

// The same launch as the all-gather of an N-sharded GGUF matrix: rows [col0, col0 + rows) of a rows_total-row
// matrix, stored as columns of every rank's f32 [tokens, rows_total] output (outs[0 .. world), peers included).
int qmv_tc_gguf_allgather(cudaStream_t stream, int format, const uint8_t *w, int64_t rows, int64_t row_bytes, const float *x,
                          int64_t tokens, float *const *outs, int world, int64_t rows_total, int64_t col0) {
    float *y = outs[0];
    const bool q4 = format == LISA_GGUF_Q4_K;
    const int64_t k = row_bytes / (q4 ? 144 : 84) * 256;
    TcParams p{};
    int smem = 0, grid = 0;
    if (!gguf_tc_plan(format, tokens, rows, row_bytes, p, smem, grid))
        return fail(LISA_ERR_UNSUPPORTED, "gguf matvec: shape not supported by the tensor-memory kernel");
    TcMaps maps{};
    CUtensorMap &map_w = maps.m[0];
    {
        // Q4_K: bytes, one block per box row; Q2_K: 32-bit words, four blocks (336 bytes) per box row
        const uint64_t dims[2] = {static_cast<uint64_t>(q4 ? row_bytes : row_bytes / 4), static_cast<uint64_t>(rows)};
        const uint64_t strides[1] = {static_cast<uint64_t>(row_bytes)};
        const uint32_t box[2] = {static_cast<uint32_t>(q4 ? 144 : 84), kRows};
        const int rc = make_tensor_map(&map_w, q4 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, w, dims,
                                       strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
        if (rc != LISA_OK) return rc;
    }
    p.xf = x;
    p.yf = y;
    p.wg = w;
    p.row_bytes = row_bytes;
    p.n = static_cast<int>(rows);
    p.k = static_cast<int>(k);
    p.m = static_cast<int>(tokens);
    p.nout = world;
    for (int o = 0; o < world; ++o) p.out[o] = reinterpret_cast<uint16_t *>(outs[o]);
    p.ldy = static_cast<int>(rows_total);
    p.col0 = static_cast<int>(col0);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    int na = 0;
    if (p.splits > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = p.splits;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    if (q4) {
        LISA_CUDA_TRY(cudaFuncSetAttribute(qmv_tc_kernel<4, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        LISA_CUDA_TRY(cudaLaunchKernelEx(&cfg, qmv_tc_kernel<4, 4>, maps, p));
    } else {
        LISA_CUDA_TRY(cudaFuncSetAttribute(qmv_tc_kernel<2, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        LISA_CUDA_TRY(cudaLaunchKernelEx(&cfg, qmv_tc_kernel<2, 2>, maps, p));
    }
    count_launch();
    return LISA_OK;
}

// ---------------------------------------------------------------------------------------
// Barrier between the GPUs of one node over peer memory, one launch per rank: every rank writes `epoch`
// into its slot of every rank's flag array (plain system-scope stores after a system fence; the stores of
// the kernels before it in the stream have completed by stream order), then waits until all slots of its
// own array have reached `epoch`.  The wait is bounded: after about a second it records an error status
// and returns, so a rank that never arrives costs an error, not a hung GPU.
static __device__ int g_peer_status = 0;

int peer_device_status() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_peer_status, sizeof(int)) != cudaSuccess) return -1;
    return v;
}
int peer_clear_status() {
    const int zero = 0;
    return cudaMemcpyToSymbol(g_peer_status, &zero, sizeof(int)) == cudaSuccess ? LISA_OK : LISA_ERR_CUDA;
}

struct PeerBarrierParams {
    unsigned long long *slots[8];  // slots[p]: the flag array of rank p (peer pointer), this rank writes [rank]
    const unsigned long long *mine;  // this rank's own flag array
    int rank, world;
    unsigned long long epoch;
};

__global__ void __launch_bounds__(32) peer_barrier_kernel(const PeerBarrierParams p) {
    const int lane = threadIdx.x;
    // epoch 0: count the barriers in slot 8 of this rank's own array (every rank runs the same sequence
    // of barriers, so the counts agree); the launch can then be replayed from a CUDA graph
    unsigned long long epoch = p.epoch;
    if (epoch == 0) {
        unsigned long long *counter = const_cast<unsigned long long *>(p.mine) + 8;
        if (lane == 0) epoch = atomicAdd(counter, 1ull) + 1ull;
        epoch = __shfl_sync(0xffffffffu, epoch, 0);
    }
    if (lane < p.world) {
        __threadfence_system();
        asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p.slots[lane] + p.rank), "l"(epoch) : "memory");
        bool ok = false;
        for (int i = 0; i < 4000000 && !ok; ++i) {
            unsigned long long v;
            asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p.mine + lane) : "memory");
            ok = v >= epoch;
            if (!ok) __nanosleep(200);
        }
        if (!ok) atomicExch(&g_peer_status, 1 + lane);
    }
}

int peer_barrier(cudaStream_t stream, int rank, int world, void *const *flag_arrays, unsigned long long epoch) {
    PeerBarrierParams p{};
    for (int i = 0; i < world; ++i) p.slots[i] = reinterpret_cast<unsigned long long *>(flag_arrays[i]);
    p.mine = reinterpret_cast<const unsigned long long *>(flag_arrays[rank]);
    p.rank = rank;
    p.world = world;
    p.epoch = epoch;
    peer_barrier_kernel<<<1, 32, 0, stream>>>(p);
    LISA_CUDA_TRY(cudaGetLastError());
    count_launch();
    return LISA_OK;
}

}  // namespace lisa
