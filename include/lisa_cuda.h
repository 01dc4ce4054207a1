/*
 * lisa_cuda — C ABI of the B200 (sm_100a) quantized-weight matmul library.
 *
 * One entry point per operator that lisa-engine dispatches on this path.  Each
 * comment names the reference interface the entry point replaces (paths are
 * relative to the agnosticeng/lisa repository).
 *
 * Conventions
 *  - Every pointer is a DEVICE pointer to contiguous row-major memory that the
 *    caller owns; the library never allocates, frees or retains memory.
 *    Weights are read-only.  Workspaces, where an op needs one, are sized by a
 *    *_workspace_bytes query and passed in by the caller.
 *  - `stream` is a cudaStream_t.  Calls validate their arguments on the host,
 *    enqueue work on `stream` and return; they do not synchronise.
 *  - Return value: 0 on success, a negative lisa_status otherwise; nothing has
 *    been enqueued when a call fails.  lisa_cuda_last_error_string() describes
 *    the calling thread's last failure.
 *  - bf16 / f16 tensors are 16-bit, f32 32-bit, packed weights are uint32 words
 *    with code i of a word in bits [bits*i, bits*i+bits) (low code first).
 *  - Alignment: x, w, scales, biases, y must be 16-byte aligned.
 */
#ifndef LISA_CUDA_H
#define LISA_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void *lisa_stream_t; /* cudaStream_t */

typedef enum lisa_status {
    LISA_OK = 0,
    LISA_ERR_BAD_ARG = -1,     /* null pointer, non-positive size, inconsistent shapes */
    LISA_ERR_UNSUPPORTED = -2, /* bits / group size / dtype / transpose=false / lhs_indices ... */
    LISA_ERR_MISALIGNED = -3,
    LISA_ERR_OVERFLOW = -4,
    LISA_ERR_CUDA = -5,
    LISA_ERR_WORKSPACE = -6, /* workspace missing or too small */
    LISA_ERR_LIMIT = -7      /* a documented size limit was exceeded */
} lisa_status;

typedef enum lisa_dtype { LISA_BF16 = 0, LISA_F16 = 1, LISA_F32 = 2 } lisa_dtype;

/* GGML tensor type ids, crates/lisa-gguf/src/lib.rs:24-32. */
typedef enum lisa_gguf_format { LISA_GGUF_Q2_K = 10, LISA_GGUF_Q4_K = 12, LISA_GGUF_Q5_K = 13 } lisa_gguf_format;

/* Dispatch overrides for lisa_cuda_quantized_matmul_ex. */
enum {
    LISA_FLAG_NONE = 0,
    LISA_FLAG_FORCE_QMV = 1 << 0,     /* mma.sync streaming kernel (staged ring) */
    LISA_FLAG_FORCE_QMV_SIMPLE = 1 << 1, /* CUDA-core generic kernel (direct loads) */
    LISA_FLAG_FORCE_QMM = 1 << 2,     /* tcgen05 tensor-core kernel */
    LISA_FLAG_PDL = 1 << 3,           /* launch with programmatic stream serialization: the
                                         kernel prefetches weights before waiting on the
                                         previous kernel in the stream */
    LISA_FLAG_FORCE_QMV_TC = 1 << 4,  /* streaming kernel with the unpacked weights in tensor memory
                                         (tcgen05): fail instead of falling back when the shape is
                                         not supported */
    LISA_FLAG_FORCE_QMV_I8 = 1 << 5   /* streaming kernel on the integer mma.sync path (u8 codes x s8
                                         activation planes; group size 64, k a multiple of 512): fail
                                         instead of falling back when the shape is not supported */
};

const char *lisa_cuda_last_error_string(void);
int lisa_cuda_version(void);
/* Number of kernels this library has launched from the calling process. */
uint64_t lisa_cuda_launch_count(void);
/* Device-side status word: 0, or non-zero after a kernel gave up on one of its bounded
 * waits (its output is then undefined).  Synchronises the current device. */
int lisa_cuda_device_status(void);
/* The status word is sticky: once a kernel has given up on a wait, every later query reports it.  A caller
 * that has handled the failure (dropped the outputs of the affected calls) resets it here.  Synchronises
 * the current device.  No counterpart in the reference, whose kernels have no bounded waits. */
int lisa_cuda_clear_device_status(void);

/* ops::quantized_matmul(x, w, scales, biases, transpose, group_size, bits)
 *   crates/lisa-mlx/src/ops/array_ops.rs:378-493
 * y[m, n] = x[m, k] . dequant(W)[n, k]^T, fp32 accumulate, output in `dtype`.
 *   x [m,k] dtype; w uint32 [n, k*bits/32]; scales, biases dtype [n, k/group_size];
 *   y [m,n] dtype.  m >= 1.  Like the reference: transpose must be non-zero and
 *   biases non-null (array_ops.rs:387-392).  bits in {2,4,8}, group_size in
 *   {32,64,128}, dtype LISA_BF16, or LISA_F16 / LISA_F32 (x, scales, biases and y all in it, as the
 *   reference casts them to the promoted dtype, array_ops.rs:398-404; these two, and 8-bit weights -- the
 *   lm-head case -- run on generic weight-streaming kernels at every row count; the other entry points of
 *   this header are bf16 only).  Dispatch by m mirrors array_ops.rs:405-488:
 *   up to 8 rows stream the weights once (group size 64: the tensor-memory GEMV; other group sizes: the
 *   bf16 mma.sync or the generic kernel), more rows run the tcgen05 GEMM.
 *   Numerics of the group-64 GEMV: products and sums are exact integers, but the activations of a (row of
 *   x, 64-k group) are first put on an integer grid of 2^-13 of the group's largest power of two (two
 *   signed bytes), so an element is off by at most 2^-14 of the group's largest magnitude; bf16
 *   activations within 2^-6 of that maximum are exact.  For Gaussian-like activations this is below the
 *   bf16 rounding of the output; a group with one element 2^10 times the rest loses the rest to about
 *   10 %.  LISA_FLAG_FORCE_QMV_I8 selects a kernel that adds a third byte (2^-22) for such groups,
 *   LISA_FLAG_FORCE_QMV one that keeps the bf16 activations exactly. */
int lisa_cuda_quantized_matmul(lisa_stream_t stream, const void *x, int64_t m, int64_t k,
                               const uint32_t *w, const void *scales, const void *biases,
                               int64_t n, int transpose, int group_size, int bits, int dtype,
                               void *y);
int lisa_cuda_quantized_matmul_ex(lisa_stream_t stream, const void *x, int64_t m, int64_t k,
                                  const uint32_t *w, const void *scales, const void *biases,
                                  int64_t n, int transpose, int group_size, int bits, int dtype,
                                  void *y, unsigned flags);

/* ops::quantized_matmul_serial_rows, array_ops.rs:500-555: independent decode
 * rows; every row's result is bit-identical to its own m=1 call. */
int lisa_cuda_quantized_matmul_serial_rows(lisa_stream_t stream, const void *x, int64_t rows,
                                           int64_t k, const uint32_t *w, const void *scales,
                                           const void *biases, int64_t n, int transpose,
                                           int group_size, int bits, int dtype, void *y);

/* Sibling linears: `count` (1..3) quantized linears with the same k, group size, bit width and dtype
 * applied to the SAME x -- q_proj | k_proj | v_proj of an attention block
 * (crates/lisa-engine/src/models/qwen4/attention.rs:111-128 calls the three `forward(x)` one after
 * another) or gate_proj | up_proj of an MLP.  Linear i is (w[i], scales[i], biases[i]) with n[i]
 * output rows and writes its own [m, n[i]] output y[i]; results are those of `count` calls of
 * lisa_cuda_quantized_matmul within the f32 summation order.  For m <= 8 and shapes the
 * tensor-memory GEMV takes this is ONE launch (a decode launch costs microseconds whatever its size);
 * for more than 8 rows it is one tensor-core GEMM launch whose row tiles cover all the linears (small
 * ones no longer leave most SMs idle); otherwise the linears run one after another through the
 * dispatch of lisa_cuda_quantized_matmul. */
int lisa_cuda_quantized_matmul_siblings(lisa_stream_t stream, const void *x, int64_t m, int64_t k,
                                        int count, const uint32_t *const *w,
                                        const void *const *scales, const void *const *biases,
                                        const int64_t *n, int transpose, int group_size, int bits,
                                        int dtype, void *const *y, unsigned flags);

/* N-sharded decode linear fused with its all-gather (one node, up to 8 GPUs, one process per GPU).
 * No counterpart in the reference, which runs on one device: this is the multi-GPU form of
 * ops::quantized_matmul: up to 8 rows (group size 64) through the tensor-memory GEMV, more rows through
 * the tensor-core GEMM; in both the kernel's own epilogue does the all-gather.  The caller holds rows
 * [col0, col0 + n_local) of an n_total-row linear; y_all[r] is rank r's [m, n_total] output buffer as
 * seen from this GPU (its own buffer and peer mappings of the others', e.g. CUDA IPC or
 * cuMemMap'd symmetric memory with peer access enabled).  The kernel's epilogue stores this rank's
 * column block into all of them with plain stores; no collective library is involved.
 * lisa_cuda_peer_barrier, enqueued after it on every rank, makes the blocks of all ranks visible:
 * flag_arrays[r] is rank r's array of 16 uint64 (zero-initialised, peer-mapped like the outputs;
 * slots 0..7 are written by the peers, slot 8 counts this rank's barriers), `epoch` a number that
 * grows with every barrier, or 0 to use the count in slot 8 (the same launch can then be replayed
 * from a CUDA graph).  Its wait is bounded (about a second), after which
 * lisa_cuda_device_status() reports the failure.
 * Reuse of the output buffers: the barrier orders this call's stores (of all ranks) before the reads that
 * follow it; it does NOT order one rank's reads of call i before another rank's stores of call i+1.  A
 * caller that issues call i+1 into the same y_all buffers must either alternate between two sets of buffers
 * (the stores of call i+2 then come after the barrier of call i+1, which no rank passes before every rank
 * has enqueued it behind its own reads of call i) or enqueue a second lisa_cuda_peer_barrier between the
 * reads of call i and call i+1. */
int lisa_cuda_quantized_matmul_allgather(lisa_stream_t stream, const void *x, int64_t m, int64_t k,
                                         const uint32_t *w, const void *scales, const void *biases,
                                         int64_t n_local, int transpose, int group_size, int bits, int dtype,
                                         void *const *y_all, int world, int64_t n_total, int64_t col0,
                                         unsigned flags);
/* Residual add + RMSNorm in front of one to three linears that read the normed row (the attention or MLP input of
 * a transformer block): replaces the fused add + rms_norm + qmv chain, affine_qmv_fast_addnorm
 * (crates/lisa-mlx/src/jit/matmul.rs:304-470) and its sibling form.
 *   sum    = dtype(x + residual)                                   [m, k], always written (the new residual)
 *   normed = dtype(norm_weight * dtype(f32(sum) * inv)),  inv = 1 / sqrt(mean(sum^2) + eps) in f32, per row
 *   y[i]   = normed . dequant(w[i])^T
 * The three roundings (sum, the product with inv, the product with the weight) are the reference's.  With up to 8
 * rows and shapes the tensor-memory kernel takes, add and norm run inside its activation staging: one launch, and
 * `normed` may be null.  Every other shape runs lisa_cuda_add_rmsnorm and then the linears, and needs `normed`
 * (LISA_ERR_WORKSPACE without it).  norm_weight: dtype [k].  k a multiple of 8. */
int lisa_cuda_quantized_matmul_addnorm(lisa_stream_t stream, const void *x, const void *residual, const void *norm_weight, float eps,
                                       int64_t m, int64_t k, int count, const uint32_t *const *w, const void *const *scales,
                                       const void *const *biases, const int64_t *n, int transpose, int group_size, int bits,
                                       int dtype, void *const *y, void *sum, void *normed, unsigned flags);
/* SwiGLU in front of a linear (the down projection of an MLP reading its gate and up outputs):
 *   act = dtype(dtype(gate * dtype(sigmoid(gate))) * up)  (crates/lisa-mlx/src/shaders/common/exact_header.metal:2-11)
 *   y   = act . dequant(w)^T
 * With up to 8 rows and shapes the tensor-memory kernel takes, the activation is formed in its staging: one
 * launch, `act` may be null (if given, it receives the activation rows).  Other shapes run lisa_cuda_swiglu and the
 * ordinary dispatch and need `act` (LISA_ERR_WORKSPACE without it).  gate, up: dtype [m, k]. */
int lisa_cuda_quantized_matmul_swiglu(lisa_stream_t stream, const void *gate, const void *up, int64_t m, int64_t k, const uint32_t *w,
                                      const void *scales, const void *biases, int64_t n, int transpose, int group_size, int bits,
                                      int dtype, void *y, void *act, unsigned flags);
/* The same add and norm as a call of its own: sum and normed [m, k]. */
int lisa_cuda_add_rmsnorm(lisa_stream_t stream, const void *x, const void *residual, const void *norm_weight, float eps, int64_t m,
                          int64_t k, int dtype, void *sum, void *normed);

/* Sibling linears (lisa_cuda_quantized_matmul_siblings) that are N-sharded and fused with their
 * all-gather: linear i holds rows [col0[i], col0[i] + n_local[i]) of an n_total[i]-row linear and
 * y_all[i * world + r] is rank r's [m, n_total[i]] output buffer of linear i as seen from this GPU.
 * One launch for up to 8 rows; otherwise one lisa_cuda_quantized_matmul_allgather per linear.  One
 * lisa_cuda_peer_barrier after it covers all the linears. */
int lisa_cuda_quantized_matmul_siblings_allgather(lisa_stream_t stream, const void *x, int64_t m, int64_t k,
                                                  int count, const uint32_t *const *w,
                                                  const void *const *scales, const void *const *biases,
                                                  const int64_t *n_local, int transpose, int group_size,
                                                  int bits, int dtype, void *const *y_all, int world,
                                                  const int64_t *n_total, const int64_t *col0,
                                                  unsigned flags);

int lisa_cuda_peer_barrier(lisa_stream_t stream, int rank, int world, void *const *flag_arrays,
                           uint64_t epoch);

/* ops::dequantize(w, scales, biases, group_size, bits), array_ops.rs:37-84 and
 * jit::affine_dequantize, crates/lisa-mlx/src/jit/matmul.rs:1316-1402.
 * out[r, c] = dtype( f32(q) * f32(scale) + f32(bias) ): the host law of
 * array_ops.rs:69-83, which is also what the GEMM tiles use. */
int lisa_cuda_dequantize(lisa_stream_t stream, const uint32_t *w, const void *scales,
                         const void *biases, int64_t rows, int64_t k, int group_size, int bits,
                         int dtype, void *out);

/* QuantizedEmbedding::forward, crates/lisa-engine/src/core/quant.rs:449-455 (take_axis of weight, scales and
 * biases by the token ids, then ops::dequantize): out[i, :] = dequantize(row ids[i]) for `count` int32 ids into
 * a [vocab, ...] table; an id outside [0, vocab) gives a row of zeros.  out dtype [count, k].  bits in {2,4,8}. */
int lisa_cuda_dequantize_rows(lisa_stream_t stream, const uint32_t *w, const void *scales,
                              const void *biases, const int32_t *ids, int64_t count, int64_t vocab,
                              int64_t k, int group_size, int bits, int dtype, void *out);

/* ops::quantize(w, group_size, bits), array_ops.rs:218-290: the MLX affine quantiser (signed scale, outer edge
 * as bias, computed in f32; scales and biases returned in w's dtype).  w dtype [rows, k]; wq uint32
 * [rows, k*bits/32]; scales, biases dtype [rows, k/group_size].  Same refusal as the reference when the group
 * size does not divide k or is not a whole number of words.  Bit for bit the reference's host loop. */
int lisa_cuda_quantize(lisa_stream_t stream, const void *w, int64_t rows, int64_t k, int group_size,
                       int bits, int dtype, uint32_t *wq, void *scales, void *biases);

/* ops::gather_qmm(x, w, scales, biases, lhs_indices, rhs_indices, transpose,
 *                 group_size, bits, sorted_indices), array_ops.rs:561-642.
 * x [rows,k]; w uint32 [experts, n, k*bits/32]; scales/biases [experts, n, k/gs];
 * rhs_indices int32 [rows], non-decreasing; y [rows,n].  Row r uses expert
 * rhs_indices[r]; an id outside [0,experts) writes zeros and touches no weight.
 * Like the reference: transpose non-zero, lhs_indices null, sorted_indices
 * non-zero, rhs_indices and biases non-null (array_ops.rs:573-585). */
size_t lisa_cuda_gather_qmm_workspace_bytes(int64_t rows, int64_t experts);
int lisa_cuda_gather_qmm(lisa_stream_t stream, const void *x, int64_t rows, int64_t k,
                         const uint32_t *w, const void *scales, const void *biases,
                         const int32_t *lhs_indices, const int32_t *rhs_indices, int64_t experts,
                         int64_t n, int transpose, int group_size, int bits, int sorted_indices,
                         int dtype, void *y, void *workspace, size_t workspace_bytes);

/* The same for one to three linears that share x, the ids, n and k (the gate and up projections of a routed
 * block, which the reference's prefill path runs as one grouped launch, models/qwen4/prefill_indirect.rs:127-170):
 * one tile table, and one launch wherever a grouped kernel runs (the matvec form up to eight rows per expert on
 * average, the GEMM form beyond).  w, scales, biases, y: tables of `count` pointers; the workspace is
 * lisa_cuda_gather_qmm_workspace_bytes(rows, experts) as for one linear. */
int lisa_cuda_gather_qmm_siblings(lisa_stream_t stream, const void *x, int64_t rows, int64_t k, int count, const uint32_t *const *w,
                                  const void *const *scales, const void *const *biases, const int32_t *rhs_indices, int64_t experts,
                                  int64_t n, int transpose, int group_size, int bits, int sorted_indices, int dtype, void *const *y,
                                  void *workspace, size_t workspace_bytes);

/* deepseek41::packed_matvec(format, weights, input), crates/lisa-mlx/src/models/deepseek41.rs:93-110.
 * w uint8 [rows, row_bytes] of GGUF blocks; x f32 [tokens, K], K = row_bytes/block*256;
 * y f32 [tokens, rows].  Same limits: rows % 8 == 0, row_bytes % block == 0,
 * 1 <= tokens <= 65535 (deepseek41.rs:50-65,100-101).  Formats: Q2_K (84-byte blocks), Q4_K (144), Q5_K (176);
 * one or two tokens of Q4_K and one token of Q2_K (rows of whole 336-byte groups) run through the tensor-memory
 * kernel, everything else one warp per row; both are exact on inputs whose products and sums are exact. */
int lisa_cuda_gguf_packed_matvec(lisa_stream_t stream, int format, const uint8_t *w, int64_t rows,
                                 int64_t row_bytes, const float *x, int64_t tokens, float *y);

/* N-sharded GGUF matvec fused with its all-gather (one node, up to 8 GPUs, one process per GPU): the caller holds
 * rows [row0, row0 + rows_local) of a rows_total-row matrix (rows are independent, as in the dense case); y_all[r]
 * is rank r's f32 [tokens, rows_total] output as seen from this GPU (own buffer + peer mappings); the kernel's
 * epilogue stores this rank's column block into all of them with plain stores; lisa_cuda_peer_barrier after it.
 * No counterpart in the reference (one device).  Takes what the tensor-memory kernel takes: Q4_K with one or
 * two tokens, Q2_K with one token and rows of whole 336-byte groups; LISA_ERR_UNSUPPORTED otherwise (run the
 * local matvec and a collective all-gather of the f32 blocks instead).  Same buffer reuse rule as
 * lisa_cuda_quantized_matmul_allgather. */
int lisa_cuda_gguf_packed_matvec_allgather(lisa_stream_t stream, int format, const uint8_t *w, int64_t rows_local,
                                           int64_t row_bytes, const float *x, int64_t tokens, void *const *y_all,
                                           int world, int64_t rows_total, int64_t row0);

/* The same operator for many tokens (prefill, target-verify: the reference runs these rows as
 * independent matvecs, deepseek41.rs:165-171) with a device workspace from the caller's pool
 * (lisa_cuda_gguf_packed_matmul_workspace_bytes, 16-byte aligned).  With a workspace and 32 tokens
 * or more (Q4_K; Q2_K with row_bytes a multiple of 336; not Q5_K) the product runs on the tensor cores: activations and
 * decoded weights each enter as two bf16 planes (value = hi + lo, 16 significant bits), f32
 * accumulate, f32 out; results agree with the matvec to ~1e-4 max-relative, not bit for bit (on
 * the reference's dyadic test inputs they are exact).  Any other case is the matvec above, exactly. */
size_t lisa_cuda_gguf_packed_matmul_workspace_bytes(int64_t tokens, int64_t row_bytes, int format);
int lisa_cuda_gguf_packed_matmul(lisa_stream_t stream, int format, const uint8_t *w, int64_t rows,
                                 int64_t row_bytes, const float *x, int64_t tokens, float *y,
                                 void *workspace, size_t workspace_bytes);

/* deepseek41::expert_matvec(format, weights, input, ids), deepseek41.rs:204-283.
 * w uint8 [experts, rows, row_bytes]; x f32 [tokens, slots, K], slots in {1, top_k};
 * ids int32 [tokens, top_k], top_k <= 32; y f32 [tokens, top_k, rows].
 * An id < 0 or >= experts writes zeros without touching weight memory. */
int lisa_cuda_gguf_expert_matvec(lisa_stream_t stream, int format, const uint8_t *w,
                                 int64_t experts, int64_t rows, int64_t row_bytes, const float *x,
                                 int64_t tokens, int64_t slots, const int32_t *ids, int64_t top_k,
                                 float *y);

/* Routing around gather_qmm, crates/lisa-engine/src/models/qwen4/moe.rs:352-481.
 * moe_route: top-k by value (ties to the lowest expert), idx in descending-logit
 *   order, weights = softmax over the k selected logits (moe.rs:143-146;
 *   crates/lisa-mlx/src/shaders/qwen4/route.metal).  logits f32 [tokens, experts]. */
int lisa_cuda_moe_route(lisa_stream_t stream, const float *logits, int64_t tokens, int64_t experts,
                        int top_k, int32_t *idx, float *weights);
/* moe_sort: stable sort of the tokens*top_k slots by expert (moe.rs:368-374;
 *   crates/lisa-mlx/src/models/qwen4/kernels/moe.rs:72-77).  sorted_ids[i],
 *   token_rows[i] = slot/top_k, inverse[slot] = position.  workspace: see query. */
size_t lisa_cuda_moe_sort_workspace_bytes(int64_t slots, int64_t experts);
int lisa_cuda_moe_sort(lisa_stream_t stream, const int32_t *idx, int64_t slots, int64_t experts,
                       int top_k, int32_t *sorted_ids, int32_t *token_rows, int32_t *inverse,
                       void *workspace, size_t workspace_bytes);
/* lisa_cuda_moe_sort_static: the same stable sort, for callers that must not allocate device
 *   memory.  It has no counterpart in the reference.  Some hosts of this library run where
 *   cudaMalloc is off limits: a real-time decode loop that may not stall on the allocator, an
 *   engine that has already handed the whole GPU to its own pool, a plugin that is only given
 *   the buffers of its inputs and outputs.  For them the (chunk x expert) count table lives in
 *   a device array built into the library (256 KiB, resident on every GPU that loads the
 *   library until the process exits) instead of a caller workspace.
 *   Limit: ceil(slots / 256) * experts <= 65536; larger problems are refused with
 *   LISA_ERR_LIMIT (use lisa_cuda_moe_sort with a workspace).  The call allocates and frees
 *   nothing.  Its first call on a device looks up the array's device address (a blocking
 *   runtime query), so make that first call outside any stream capture.  All calls on a device
 *   share the one array, which keeps whatever the last call left in it; every counter a call
 *   reads is written earlier by the same call, so nothing needs clearing, but two calls that
 *   may overlap on the GPU (different streams) race on it and must be ordered by the caller.
 *   `stream` must belong to the current device (checked: LISA_ERR_BAD_ARG otherwise; the array is
 *   per device).  The looked-up address is cached per device for the life of the process: after
 *   cudaDeviceReset() it is stale, and the library must not be called again on that device without
 *   being reloaded. */
int lisa_cuda_moe_sort_static(lisa_stream_t stream, const int32_t *idx, int64_t slots, int64_t experts,
                              int top_k, int32_t *sorted_ids, int32_t *token_rows, int32_t *inverse);
/* x_sorted[i, :] = x[token_rows[i], :] (gatherSort, moe.rs:375-377). */
int lisa_cuda_gather_rows(lisa_stream_t stream, const void *x, const int32_t *token_rows,
                          int64_t rows, int64_t width, int dtype, void *out);
/* act = bf16(bf16(g * sigmoid(g)) * u), crates/lisa-mlx/src/shaders/common/exact_header.metal:2-11. */
int lisa_cuda_swiglu(lisa_stream_t stream, const void *gate, const void *up, int64_t count,
                     int dtype, void *act);
/* moe_combine without the shared expert (moe.rs:436-481): out[t, h] =
 *   dtype( sum_j f32(down_sorted[inverse[t*top_k + j], h]) * weights[t, j] ), slots
 *   folded in original order. */
int lisa_cuda_moe_combine(lisa_stream_t stream, const void *down_sorted, const float *weights,
                          const int32_t *inverse, int64_t tokens, int top_k, int64_t hidden,
                          int dtype, void *out);

/* The routed block for a handful of tokens (decode), three launches with lisa_cuda_moe_route in front: no sort,
 * no gathered copy of x, no tile table.  Replace moe_decode::gate_up_act and moe_decode::down_combine
 * (crates/lisa-mlx/src/models/qwen4/moe_decode.rs:136-298; shaders/qwen4/gate_up_reuse.metal, down_combine.metal)
 * without their shared-expert operands.
 *   gate_up_act:  act[s, :] = swiglu(bf16(x[r] . Wg[idx[s]]^T), bf16(x[r] . Wu[idx[s]]^T)) for every slot s, with
 *                 r = xrow[s], or s / top_k when xrow is null; idx int32 [slots] (the router's [tokens, top_k]
 *                 output read flat), Wg / Wu [experts, inter, hidden * bits / 32], act bf16 [slots, inter];
 *   down_combine: out[t, :] = dtype( fold_j f32(bf16(act[t * top_k + j] . Wd[idx[t, j]]^T)) * weights[t, j] ),
 *                 slots folded in original order (exact_header.metal:12-24), Wd [experts, hidden, inter * bits / 32].
 * Rounding points as in the reference (every matmul result, sigmoid, silu, their product and the fold to bf16).
 * An id outside [0, experts) reads no weights and contributes zeros.  2- or 4-bit, group size a multiple of
 * 32, bf16.  Meant for tokens * top_k below a few dozen; the sorted path (moe_sort + gather_qmm) reads every
 * expert once and wins beyond that. */
int lisa_cuda_moe_gate_up_act(lisa_stream_t stream, const void *x, const int32_t *idx, const int32_t *xrow, int64_t slots,
                              int top_k, int64_t experts, int64_t hidden, int64_t inter, const uint32_t *wg, const void *sg,
                              const void *bg, const uint32_t *wu, const void *su, const void *bu, int group_size, int bits,
                              int dtype, void *act);
int lisa_cuda_moe_down_combine(lisa_stream_t stream, const void *act, const int32_t *idx, const float *weights, int64_t tokens,
                               int top_k, int64_t experts, int64_t inter, int64_t hidden, const uint32_t *wd, const void *sd,
                               const void *bd, int group_size, int bits, int dtype, void *out);

/* Expert-parallel exchange over peer memory (one node, up to 8 GPUs, one process per GPU).  No counterpart in
 * the reference, which runs one device; ownership is its contiguous rule first = rank * (experts / world)
 * (crates/lisa-mlx/src/shaders/deepseek41/iq.metal:976-982).  Tokens are data-parallel, experts are owned.
 * Every rank routes and sorts its own slots by GLOBAL expert (lisa_cuda_moe_route, lisa_cuda_moe_sort), which
 * groups them by owner, then:
 *   ep_counts    publishes how many of its slots belong to each owner: entry [rank * world + q] of every rank's
 *                int32 [world, world] count matrix (count_matrices[r]: rank r's matrix as seen from this GPU);
 *   -- lisa_cuda_peer_barrier; the caller may now read its matrix (column `rank` sums to the rows it receives) --
 *   ep_dispatch  stores row token_rows[p] of x and the local expert id of every sorted slot p into its owner's
 *                receive buffers (recv_x[q]: bf16 [capacity, hidden], recv_ids[q]: int32 [capacity]; capacity >= the
 *                owner's total, at most world * slots), compactly: source ranks in order, slots in sorted order;
 *   -- lisa_cuda_peer_barrier; the owner sorts recv_ids (moe_sort with top_k = 1: token_rows is then the index into
 *      recv_x), runs gather_rows / gather_qmm / swiglu / gather_qmm on exactly the rows it received --
 *   ep_return    stores result row p (sorted order; recv_index = that sort's token_rows) into the source rank's
 *                `back` buffer (back[r]: bf16 [slots of r, hidden]) at the position the slot has in the source's own
 *                sorted order, so that the source folds with lisa_cuda_moe_combine and its own `inverse`;
 *   -- lisa_cuda_peer_barrier --
 * Plain stores into peer mappings; every buffer is reused from step to step (the three barriers order the reuse).
 * Without a host read (so that the whole step can be captured in a CUDA graph): fill recv_ids with an id outside
 * the owner's table before the first barrier, then run the owner's sort, gather_rows, gather_qmm and ep_return
 * over the whole capacity: unused rows sort last, get no tile and no weight access, and ep_return stops at the
 * received count, which it reads from the matrix on the device (count may be any value >= it). */
int lisa_cuda_ep_counts(lisa_stream_t stream, const int32_t *sorted_ids, int64_t slots, int64_t experts, int world,
                        int rank, void *const *count_matrices);
int lisa_cuda_ep_dispatch(lisa_stream_t stream, const void *x, const int32_t *sorted_ids, const int32_t *token_rows,
                          int64_t slots, int64_t hidden, int64_t experts, int world, int rank,
                          const int32_t *count_matrix, void *const *recv_x, void *const *recv_ids, int dtype);
int lisa_cuda_ep_return(lisa_stream_t stream, const void *rows, const int32_t *recv_index, int64_t count, int64_t hidden,
                        int world, int rank, const int32_t *count_matrix, void *const *back, int dtype);

#ifdef __cplusplus
}
#endif
#endif
