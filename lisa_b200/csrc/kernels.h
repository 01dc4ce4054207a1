// Internal launch functions, one group per translation unit.  Arguments are already
// validated by api.cu; every function enqueues on `stream` and returns a lisa_status.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace lisa {

// qmv_affine.cu
int qmv_affine(cudaStream_t stream, const void *x, int64_t m, int64_t k, const uint32_t *w, const void *scales,
               const void *biases, int64_t n, int group_size, int bits, void *y, unsigned flags);
int qmv_device_status();
int qmv_clear_status();

// qmv_tc.cu: the same GEMV with the unpacked weights in tensor memory (tcgen05), group size 64, m <= 8 per pass
bool qmv_tc_supported(int64_t m, int64_t k, int64_t n, int group_size, int bits);
// residual add + RMSNorm in front of the matmul (the kernel's NORM form): the activations are
// rms_norm(bf16(x + residual)) * weight; `sum` receives bf16(x + residual), `normed` (or null) the normed rows.
// With a null weight the form is the SwiGLU one: activations = swiglu(x, residual), `normed` (or null) receives them.
struct TcNormArgs {
    const void *residual;
    const void *weight;
    float eps;
    void *sum;
    void *normed;
};
int qmv_tc(cudaStream_t stream, const void *x, int64_t m, int64_t k, const uint32_t *w, const void *scales,
           const void *biases, int64_t n, int group_size, int bits, void *y, unsigned flags, const TcNormArgs *norm = nullptr);
int qmv_tc_device_status();
int qmv_tc_clear_status();
int qmv_tc_allgather(cudaStream_t stream, const void *x, int64_t m, int64_t k, const uint32_t *w, const void *scales,
                     const void *biases, int64_t n, int group_size, int bits, void *const *outs, int world,
                     int64_t n_total, int64_t col0, unsigned flags);
bool qmv_tc_multi_supported(int64_t m, int64_t k, int count, const int64_t *n, int group_size, int bits);
int qmv_tc_multi(cudaStream_t stream, const void *x, int64_t m, int64_t k, int count, const uint32_t *const *w,
                 const void *const *scales, const void *const *biases, const int64_t *n, int group_size, int bits,
                 void *const *y, unsigned flags, int world = 0, const int64_t *n_total = nullptr,
                 const int64_t *col0 = nullptr, const TcNormArgs *norm = nullptr);
// f16 / f32 compute dtypes (typed.cu): generic kernels, any m
int qmv_typed(cudaStream_t stream, int dtype, const void *x, int64_t m, int64_t k, const uint32_t *w, const void *scales,
              const void *biases, int64_t n, int group_size, int bits, void *y);
int dequantize_typed(cudaStream_t stream, int dtype, const uint32_t *w, const void *scales, const void *biases, int64_t rows,
                     int64_t k, int group_size, int bits, void *out);
// bf16(x + r) and rms_norm of it times w, as a kernel of its own (the unfused form)
int add_rmsnorm(cudaStream_t stream, const void *x, const void *residual, const void *weight, float eps, int64_t m, int64_t k,
                void *sum, void *normed);
bool qmv_tc_gguf_supported(int format, int64_t tokens, int64_t rows, int64_t row_bytes);
bool qmv_tc_gguf_expert_supported(int format, int64_t slots_total, int64_t experts, int64_t rows, int64_t row_bytes);
int qmv_tc_gguf_expert(cudaStream_t stream, int format, const uint8_t *w, int64_t experts, int64_t rows, int64_t row_bytes,
                       const float *x, int64_t tokens, int64_t slots, const int32_t *ids, int64_t top_k, float *y);
// grouped (sorted rows, one expert per table entry) form of the tensor-memory matvec: rows per entry it can take
// for this shape (0 = unsupported), and the launch over a device tile table {expert, row_begin, row_end, 0}
int qmv_tc_grouped_rows(int64_t rows, int64_t experts, int64_t k, int64_t n, int group_size, int bits, int count = 1);
int qmv_tc_grouped(cudaStream_t stream, const void *x, int64_t rows, int64_t k, int count, const uint32_t *const *w,
                   const void *const *scales, const void *const *biases, int64_t experts, int64_t n, int group_size, int bits,
                   void *const *y, int bt, const int32_t *tiles, const int32_t *tile_count, int64_t max_tiles);
int qmv_tc_gguf(cudaStream_t stream, int format, const uint8_t *w, int64_t rows, int64_t row_bytes, const float *x,
                int64_t tokens, float *y);
int qmv_tc_gguf_allgather(cudaStream_t stream, int format, const uint8_t *w, int64_t rows, int64_t row_bytes, const float *x,
                          int64_t tokens, float *const *outs, int world, int64_t rows_total, int64_t col0);
int peer_barrier(cudaStream_t stream, int rank, int world, void *const *flag_arrays, unsigned long long epoch);
int peer_device_status();
int peer_clear_status();

// qmv_i8.cu: the same GEMV on the integer path of mma.sync (u8 codes x s8 activation planes), group size 64,
// k a multiple of 512, m <= 8 per pass; one to three sibling linears per launch; all-gather form with peer outputs
bool qmv_i8_supported(int64_t m, int64_t k, int64_t n, int group_size, int bits);
bool qmv_i8_multi_supported(int64_t m, int64_t k, int count, const int64_t *n, int group_size, int bits);
int qmv_i8(cudaStream_t stream, const void *x, int64_t m, int64_t k, const uint32_t *w, const void *scales,
           const void *biases, int64_t n, int group_size, int bits, void *y, unsigned flags);
int qmv_i8_allgather(cudaStream_t stream, const void *x, int64_t m, int64_t k, const uint32_t *w, const void *scales,
                     const void *biases, int64_t n, int group_size, int bits, void *const *outs, int world,
                     int64_t n_total, int64_t col0, unsigned flags);
int qmv_i8_multi(cudaStream_t stream, const void *x, int64_t m, int64_t k, int count, const uint32_t *const *w,
                 const void *const *scales, const void *const *biases, const int64_t *n, int group_size, int bits,
                 void *const *y, unsigned flags, int world = 0, const int64_t *n_total = nullptr,
                 const int64_t *col0 = nullptr);
int qmv_i8_device_status();
int qmv_i8_clear_status();

// qmm_affine.cu
bool qmm_affine_supported(int64_t m, int64_t k, int64_t n, int group_size, int bits);
int qmm_affine(cudaStream_t stream, const void *x, int64_t m, int64_t k, const uint32_t *w, const void *scales,
               const void *biases, int64_t n, int group_size, int bits, void *y, unsigned flags);
int qmm_affine_multi(cudaStream_t stream, const void *x, int64_t m, int64_t k, int count, const uint32_t *const *w,
                     const void *const *scales, const void *const *biases, const int64_t *n, int group_size, int bits,
                     void *const *y, unsigned flags);
int qmm_affine_allgather(cudaStream_t stream, const void *x, int64_t m, int64_t k, const uint32_t *w, const void *scales,
                         const void *biases, int64_t n, int group_size, int bits, void *const *outs, int world,
                         int64_t n_total, int64_t col0, unsigned flags);
int qmm_affine_grouped(cudaStream_t stream, const void *x, int64_t rows, int64_t k, const uint32_t *w,
                       const void *scales, const void *biases, int64_t experts, int64_t n, int group_size, int bits,
                       void *y, int bt, const int32_t *tiles, const int32_t *tile_count, int64_t max_tiles);
int qmm_affine_grouped_multi(cudaStream_t stream, const void *x, int64_t rows, int64_t k, int count, const uint32_t *const *w,
                             const void *const *scales, const void *const *biases, int64_t experts, int64_t n, int group_size,
                             int bits, void *const *y, int bt, const int32_t *tiles, const int32_t *tile_count, int64_t max_tiles);
int qmm_device_status();
int qmm_clear_status();
// GGUF Q4_K GEMM on the same kernel (bf16 operands: the caller opts in by giving a workspace)
bool qmm_gguf_supported(int format, int64_t tokens, int64_t rows, int64_t row_bytes);
size_t qmm_gguf_workspace_bytes(int64_t tokens, int64_t k);
int qmm_gguf(cudaStream_t stream, int format, const uint8_t *w, int64_t rows, int64_t row_bytes, const float *x,
             int64_t tokens, float *y, void *workspace);

// dequantize.cu
int dequantize_affine(cudaStream_t stream, const uint32_t *w, const void *scales, const void *biases, int64_t rows,
                      int64_t k, int group_size, int bits, void *out);

int dequantize_affine_rows(cudaStream_t stream, const uint32_t *w, const void *scales, const void *biases, const int32_t *ids,
                           int64_t count, int64_t vocab, int64_t k, int group_size, int bits, void *out);
int quantize_affine(cudaStream_t stream, const void *w, int64_t rows, int64_t k, int group_size, int bits, uint32_t *wq,
                    void *scales, void *biases);

// gather_qmm.cu
size_t gather_qmm_workspace_bytes(int64_t rows, int64_t experts);
int gather_qmm_affine(cudaStream_t stream, const void *x, int64_t rows, int64_t k, const uint32_t *w,
                      const void *scales, const void *biases, const int32_t *ids, int64_t experts, int64_t n,
                      int group_size, int bits, void *y, void *workspace, size_t workspace_bytes);
// the same for `count` sibling linears (one n, one k, one set of ids: gate | up): one table, one launch where a grouped kernel runs
int gather_qmm_affine_multi(cudaStream_t stream, const void *x, int64_t rows, int64_t k, int count, const uint32_t *const *w,
                            const void *const *scales, const void *const *biases, const int32_t *ids, int64_t experts, int64_t n,
                            int group_size, int bits, void *const *y, void *workspace, size_t workspace_bytes);

// gguf_matvec.cu: ids == nullptr selects the dense matvec (experts = slots = top_k = 1).
int gguf_matvec(cudaStream_t stream, int format, const uint8_t *w, int64_t experts, int64_t rows, int64_t row_bytes,
                const float *x, int64_t tokens, int64_t slots, const int32_t *ids, int64_t top_k, float *y);

// moe.cu
int moe_route(cudaStream_t stream, const float *logits, int64_t tokens, int64_t experts, int top_k, int32_t *idx,
              float *weights);
size_t moe_sort_workspace_bytes(int64_t slots, int64_t experts);
int moe_sort(cudaStream_t stream, const int32_t *idx, int64_t slots, int64_t experts, int top_k, int32_t *sorted_ids,
             int32_t *token_rows, int32_t *inverse, void *workspace);
int64_t moe_sort_static_capacity();
int moe_sort_static(cudaStream_t stream, const int32_t *idx, int64_t slots, int64_t experts, int top_k,
                    int32_t *sorted_ids, int32_t *token_rows, int32_t *inverse);
int moe_gather_rows(cudaStream_t stream, const void *x, const int32_t *token_rows, int64_t rows, int64_t width,
                    void *out);
int moe_swiglu(cudaStream_t stream, const void *gate, const void *up, int64_t count, void *act);
// the routed block for a handful of tokens (moe_decode.cu): per-slot gate|up + SwiGLU, per-token down + fold
bool moe_decode_supported(int64_t k, int group_size, int bits, int top_k);
int moe_gate_up_act(cudaStream_t stream, const void *x, const int32_t *idx, const int32_t *xrow, int64_t slots, int top_k,
                    int64_t experts, int64_t k, int64_t n, const uint32_t *wg, const void *sg, const void *bg,
                    const uint32_t *wu, const void *su, const void *bu, int group_size, int bits, void *act);
int moe_down_combine(cudaStream_t stream, const void *act, const int32_t *idx, const float *weights, int64_t tokens, int top_k,
                     int64_t experts, int64_t k, int64_t n, const uint32_t *wd, const void *sd, const void *bd, int group_size,
                     int bits, void *out);
int moe_combine(cudaStream_t stream, const void *down_sorted, const float *weights, const int32_t *inverse,
                int64_t tokens, int top_k, int64_t hidden, void *out);

// ep.cu: expert-parallel dispatch / return over peer memory
int ep_counts(cudaStream_t stream, const int32_t *sorted_ids, int64_t slots, int64_t experts, int world, int rank,
              void *const *matrices);
int ep_dispatch(cudaStream_t stream, const void *x, const int32_t *sorted_ids, const int32_t *token_rows, int64_t slots,
                int64_t hidden, int64_t experts, int world, int rank, const int32_t *matrix, void *const *recv_x,
                void *const *recv_ids);
int ep_return(cudaStream_t stream, const void *rows, const int32_t *recv_index, int64_t count, int64_t hidden, int world, int rank,
              const int32_t *matrix, void *const *back);

}  // namespace lisa
