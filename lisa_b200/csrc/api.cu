// C ABI of the library (include/lisa_cuda.h): argument validation, error reporting and the
// dispatch rules of the reference's operator layer
// (crates/lisa-mlx/src/ops/array_ops.rs:378-642, crates/lisa-mlx/src/models/deepseek41.rs:50-283).
// Nothing here allocates device memory or synchronises.
#include <cuda_runtime.h>

#include <stdlib.h>

#include <atomic>
#include <mutex>
#include <sstream>
#include <string>

#include "common.cuh"
#include "kernels.h"

namespace lisa {

static thread_local std::string t_last_error;
static std::atomic<uint64_t> g_launches{0};

void set_error(const std::string &msg) { t_last_error = msg; }
int fail(int code, const std::string &msg) {
    t_last_error = msg;
    return code;
}
int cuda_fail(cudaError_t err, const char *what) {
    std::ostringstream os;
    os << "CUDA error " << static_cast<int>(err) << " (" << cudaGetErrorString(err) << ") in " << what;
    t_last_error = os.str();
    return LISA_ERR_CUDA;
}
void count_launch(unsigned n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

struct DeviceInfo {
    int sms = 0;
    int smem_optin = 0;
};
static DeviceInfo g_dev[64];
static std::once_flag g_dev_once[64];

static const DeviceInfo &device_info() {
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    std::call_once(g_dev_once[dev], [dev]() {
        cudaDeviceGetAttribute(&g_dev[dev].sms, cudaDevAttrMultiProcessorCount, dev);
        cudaDeviceGetAttribute(&g_dev[dev].smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    });
    return g_dev[dev];
}
int sm_count() { return device_info().sms > 0 ? device_info().sms : 148; }
int max_smem_optin() { return device_info().smem_optin > 0 ? device_info().smem_optin : 232448; }

static int check_affine(const char *op, const void *x, int64_t m, int64_t k, const uint32_t *w, const void *scales,
                        const void *biases, int64_t n, int group_size, int bits, int dtype, const void *y,
                        bool allow8 = false, bool any_dtype = false) {
    std::string name(op);
    if (!biases) return fail(LISA_ERR_BAD_ARG, name + ": affine biases required");
    if (!x || !w || !scales || !y) return fail(LISA_ERR_BAD_ARG, name + ": null pointer");
    if (m < 1 || n < 1 || k < 1) return fail(LISA_ERR_BAD_ARG, name + ": sizes must be positive");
    if (bits != 2 && bits != 4 && !(allow8 && bits == 8))
        return fail(LISA_ERR_UNSUPPORTED, name + (allow8 ? ": bits must be 2, 4 or 8" : ": bits must be 2 or 4"));
    if (group_size != 32 && group_size != 64 && group_size != 128)
        return fail(LISA_ERR_UNSUPPORTED, name + ": group_size must be 32, 64 or 128");
    if (dtype != LISA_BF16 && !(any_dtype && (dtype == LISA_F16 || dtype == LISA_F32)))
        return fail(LISA_ERR_UNSUPPORTED, name + (any_dtype ? ": unsupported compute dtype" : ": unsupported compute dtype (bf16 only)"));
    if (k % group_size != 0) return fail(LISA_ERR_BAD_ARG, name + ": k is not a multiple of group_size");
    if (m > (1ll << 30) || n > (1ll << 30) || k > (1ll << 30) || m * n > (1ll << 40) || n * k > (1ll << 42))
        return fail(LISA_ERR_OVERFLOW, name + ": shape too large");
    if (!aligned16(x) || !aligned16(w) || !aligned16(scales) || !aligned16(biases) || !aligned16(y))
        return fail(LISA_ERR_MISALIGNED, name + ": pointers must be 16-byte aligned");
    return LISA_OK;
}

// Row count from which the tensor-core GEMM takes over from the weight-streaming kernel.
// The reference switches at qmv_batch_limit (crates/lisa-mlx/src/jit/matmul.rs:1873-1881).  Here the
// streaming kernel takes up to 8 rows in one pass over the weights while their activations fit its
// shared-memory staging (m * k <= 8 * 9728, measured crossover); a GEMM CTA costs the same for any
// tile of up to 256 rows, so it wins as soon as the streaming kernel would need a second pass.
static const int64_t kQmvMaxRows = 8;
static const int64_t kQmvMaxStaged = 8 * 9728;
static bool prefer_qmv(int64_t m, int64_t k, bool tc_ok) {
    // the tensor-memory GEMV takes up to 8 rows for about the cost of one
    if (tc_ok) return m <= kQmvMaxRows;
    return m <= kQmvMaxRows && (m <= 4 || m * k <= kQmvMaxStaged);
}

// Which weight-streaming kernel takes a call that both support: the tensor-memory kernel (measured faster on
// every decode shape of the 4-bit stack), the integer mma.sync kernel when the environment says
// LISA_QMV_KERNEL=i8 (read once; for side-by-side measurements) or LISA_FLAG_FORCE_QMV_I8 is given.
static bool prefer_i8() {
    static const bool v = []() {
        const char *e = getenv("LISA_QMV_KERNEL");
        return e && e[0] == 'i' && e[1] == '8';
    }();
    return v;
}

static int quantized_matmul_impl(cudaStream_t stream, const void *x, int64_t m, int64_t k, const uint32_t *w,
                                 const void *scales, const void *biases, int64_t n, int transpose, int group_size,
                                 int bits, int dtype, void *y, unsigned flags) {
    if (!transpose) return fail(LISA_ERR_UNSUPPORTED, "quantized_matmul: only transpose=true supported");
    int rc = check_affine("quantized_matmul", x, m, k, w, scales, biases, n, group_size, bits, dtype, y, true, true);
    if (rc != LISA_OK) return rc;
    if (dtype != LISA_BF16) {
        // f16 / f32 activations, scales and biases (array_ops.rs:398-404): the generic kernel for every row count
        if (flags & (LISA_FLAG_FORCE_QMM | LISA_FLAG_FORCE_QMV | LISA_FLAG_FORCE_QMV_TC | LISA_FLAG_FORCE_QMV_I8))
            return fail(LISA_ERR_UNSUPPORTED, "quantized_matmul: f16 and f32 run on the generic kernel only");
        return qmv_typed(stream, dtype, x, m, k, w, scales, biases, n, group_size, bits, y);
    }
    if (bits == 8) {
        // 8-bit weights (lm heads): the generic weight-streaming kernel for every row count
        if (flags & (LISA_FLAG_FORCE_QMM | LISA_FLAG_FORCE_QMV_TC | LISA_FLAG_FORCE_QMV_I8))
            return fail(LISA_ERR_UNSUPPORTED, "quantized_matmul: 8-bit weights run on the generic kernel only");
        return qmv_affine(stream, x, m, k, w, scales, biases, n, group_size, bits, y, flags);
    }
    const bool force_tc = (flags & LISA_FLAG_FORCE_QMV_TC) != 0;
    const bool force_i8 = (flags & LISA_FLAG_FORCE_QMV_I8) != 0;
    const bool force_qmv = (flags & (LISA_FLAG_FORCE_QMV | LISA_FLAG_FORCE_QMV_SIMPLE)) != 0 || force_tc || force_i8;
    const bool force_qmm = (flags & LISA_FLAG_FORCE_QMM) != 0;
    if (force_qmv && force_qmm) return fail(LISA_ERR_BAD_ARG, "quantized_matmul: contradictory flags");
    const bool qmm_ok = qmm_affine_supported(m, k, n, group_size, bits);
    if (force_qmm && !qmm_ok) return fail(LISA_ERR_UNSUPPORTED, "quantized_matmul: shape not supported by the GEMM kernel");
    const bool tc_ok = qmv_tc_supported(m, k, n, group_size, bits);
    const bool i8_ok = qmv_i8_supported(m, k, n, group_size, bits);
    if (force_qmm || (!force_qmv && !prefer_qmv(m, k, tc_ok || i8_ok) && qmm_ok))
        return qmm_affine(stream, x, m, k, w, scales, biases, n, group_size, bits, y, flags);
    if (force_tc && !tc_ok)
        return fail(LISA_ERR_UNSUPPORTED, "quantized_matmul: shape not supported by the tensor-memory GEMV");
    if (force_i8 && !i8_ok)
        return fail(LISA_ERR_UNSUPPORTED, "quantized_matmul: shape not supported by the integer GEMV");
    // Group size 64: the tensor-memory GEMV where it applies, else the integer mma.sync GEMV (k a multiple of
    // 512); LISA_FLAG_FORCE_QMV and LISA_FLAG_FORCE_QMV_SIMPLE select the bf16 mma.sync and the generic kernel.
    const bool plain_forced = (flags & (LISA_FLAG_FORCE_QMV | LISA_FLAG_FORCE_QMV_SIMPLE)) != 0;
    if (force_i8 || (i8_ok && !plain_forced && !force_tc && (prefer_i8() || !tc_ok)))
        return qmv_i8(stream, x, m, k, w, scales, biases, n, group_size, bits, y, flags);
    if (force_tc || (tc_ok && !plain_forced)) return qmv_tc(stream, x, m, k, w, scales, biases, n, group_size, bits, y, flags);
    return qmv_affine(stream, x, m, k, w, scales, biases, n, group_size, bits, y, flags);
}

}  // namespace lisa

using namespace lisa;

extern "C" {

const char *lisa_cuda_last_error_string(void) { return t_last_error.c_str(); }
int lisa_cuda_version(void) { return 100; }
uint64_t lisa_cuda_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int lisa_cuda_device_status(void) {
    // Non-zero after a kernel gave up on a bounded wait.  Synchronises the device.
    const int a = qmv_device_status();
    const int b = qmm_device_status();
    const int c = qmv_tc_device_status();
    const int d = peer_device_status();
    const int e = qmv_i8_device_status();
    if (a < 0 || b < 0 || c < 0 || d < 0 || e < 0) return -1;
    return a | (e << 4) | (b << 8) | (c << 16) | (d << 24);
}

int lisa_cuda_clear_device_status(void) {
    // The status words are sticky: a caller that has handled a failure resets them here.
    const int rc[5] = {qmv_clear_status(), qmm_clear_status(), qmv_tc_clear_status(), peer_clear_status(), qmv_i8_clear_status()};
    for (int i = 0; i < 5; ++i)
        if (rc[i] != LISA_OK) return fail(LISA_ERR_CUDA, "clear_device_status: could not reset a status word");
    return LISA_OK;
}

int lisa_cuda_quantized_matmul(lisa_stream_t stream, const void *x, int64_t m, int64_t k, const uint32_t *w,
                               const void *scales, const void *biases, int64_t n, int transpose, int group_size,
                               int bits, int dtype, void *y) {
    return quantized_matmul_impl(static_cast<cudaStream_t>(stream), x, m, k, w, scales, biases, n, transpose,
                                 group_size, bits, dtype, y, LISA_FLAG_NONE);
}

int lisa_cuda_quantized_matmul_ex(lisa_stream_t stream, const void *x, int64_t m, int64_t k, const uint32_t *w,
                                  const void *scales, const void *biases, int64_t n, int transpose, int group_size,
                                  int bits, int dtype, void *y, unsigned flags) {
    return quantized_matmul_impl(static_cast<cudaStream_t>(stream), x, m, k, w, scales, biases, n, transpose,
                                 group_size, bits, dtype, y, flags);
}

int lisa_cuda_quantized_matmul_serial_rows(lisa_stream_t stream, const void *x, int64_t rows, int64_t k,
                                           const uint32_t *w, const void *scales, const void *biases, int64_t n,
                                           int transpose, int group_size, int bits, int dtype, void *y) {
    if (!transpose) return fail(LISA_ERR_UNSUPPORTED, "quantized_matmul_serial_rows: only transpose=true supported");
    // Outside 2..8 rows the reference hands over to quantized_matmul (array_ops.rs:521-523).
    if (rows <= 1 || rows > 8)
        return quantized_matmul_impl(static_cast<cudaStream_t>(stream), x, rows, k, w, scales, biases, n, transpose,
                                     group_size, bits, dtype, y, LISA_FLAG_NONE);
    int rc = check_affine("quantized_matmul_serial_rows", x, rows, k, w, scales, biases, n, group_size, bits, dtype, y);
    if (rc != LISA_OK) return rc;
    // Both streaming kernels accumulate every input row in the same order whatever the row count, so
    // each row equals its own m=1 call bit for bit -- as long as it is the kernel an m=1 call takes.
    if (qmv_i8_supported(1, k, n, group_size, bits) && (prefer_i8() || !qmv_tc_supported(1, k, n, group_size, bits)))
        return qmv_i8(static_cast<cudaStream_t>(stream), x, rows, k, w, scales, biases, n, group_size, bits, y,
                      LISA_FLAG_NONE);
    if (qmv_tc_supported(1, k, n, group_size, bits))
        return qmv_tc(static_cast<cudaStream_t>(stream), x, rows, k, w, scales, biases, n, group_size, bits, y,
                      LISA_FLAG_NONE);
    return qmv_affine(static_cast<cudaStream_t>(stream), x, rows, k, w, scales, biases, n, group_size, bits, y,
                      LISA_FLAG_NONE);
}

int lisa_cuda_quantized_matmul_allgather(lisa_stream_t stream, const void *x, int64_t m, int64_t k, const uint32_t *w,
                                         const void *scales, const void *biases, int64_t n_local, int transpose,
                                         int group_size, int bits, int dtype, void *const *y_all, int world,
                                         int64_t n_total, int64_t col0, unsigned flags) {
    if (!transpose) return fail(LISA_ERR_UNSUPPORTED, "quantized_matmul_allgather: only transpose=true supported");
    if (!y_all || world < 1 || world > 8) return fail(LISA_ERR_BAD_ARG, "quantized_matmul_allgather: 1 to 8 output buffers");
    for (int r = 0; r < world; ++r)
        if (!y_all[r] || (reinterpret_cast<uintptr_t>(y_all[r]) & 1u)) return fail(LISA_ERR_BAD_ARG, "quantized_matmul_allgather: null or misaligned output buffer");
    int rc = check_affine("quantized_matmul_allgather", x, m, k, w, scales, biases, n_local, group_size, bits, dtype, y_all[0]);
    if (rc != LISA_OK) return rc;
    if (col0 < 0 || n_total < 1 || col0 + n_local > n_total || n_total > (1ll << 30))
        return fail(LISA_ERR_BAD_ARG, "quantized_matmul_allgather: column block outside the output");
    if (m > kQmvMaxRows) {
        // many rows: the tensor-core GEMM, whose epilogue stores the tile into every rank's output
        if (!qmm_affine_supported(m, k, n_local, group_size, bits))
            return fail(LISA_ERR_UNSUPPORTED, "quantized_matmul_allgather: shape not supported by the GEMM kernel");
        return qmm_affine_allgather(static_cast<cudaStream_t>(stream), x, m, k, w, scales, biases, n_local, group_size, bits,
                                    y_all, world, n_total, col0, flags);
    }
    if (!qmv_tc_supported(m, k, n_local, group_size, bits))
        return fail(LISA_ERR_UNSUPPORTED, "quantized_matmul_allgather: up to 8 rows need a shape the tensor-memory GEMV takes");
    return qmv_tc_allgather(static_cast<cudaStream_t>(stream), x, m, k, w, scales, biases, n_local, group_size, bits, y_all,
                            world, n_total, col0, flags);
}

int lisa_cuda_quantized_matmul_siblings(lisa_stream_t stream, const void *x, int64_t m, int64_t k, int count,
                                        const uint32_t *const *w, const void *const *scales,
                                        const void *const *biases, const int64_t *n, int transpose, int group_size,
                                        int bits, int dtype, void *const *y, unsigned flags) {
    if (!transpose) return fail(LISA_ERR_UNSUPPORTED, "quantized_matmul_siblings: only transpose=true supported");
    if (count < 1 || count > 3 || !w || !scales || !biases || !n || !y)
        return fail(LISA_ERR_BAD_ARG, "quantized_matmul_siblings: one to three linears, non-null tables");
    for (int i = 0; i < count; ++i) {
        const int rc = check_affine("quantized_matmul_siblings", x, m, k, w[i], scales[i], biases[i], n[i], group_size, bits, dtype, y[i]);
        if (rc != LISA_OK) return rc;
    }
    // one launch when the tensor-memory GEMV takes the rows; otherwise the linears one after another,
    // each through the dispatch of quantized_matmul
    if (count >= 2 && m <= 8 && !(flags & (LISA_FLAG_FORCE_QMM | LISA_FLAG_FORCE_QMV | LISA_FLAG_FORCE_QMV_SIMPLE))) {
        const bool tc_ok = !(flags & LISA_FLAG_FORCE_QMV_I8) && qmv_tc_multi_supported(m, k, count, n, group_size, bits);
        const bool i8_ok = !(flags & LISA_FLAG_FORCE_QMV_TC) && qmv_i8_multi_supported(m, k, count, n, group_size, bits);
        if (i8_ok && ((flags & LISA_FLAG_FORCE_QMV_I8) || prefer_i8() || !tc_ok))
            return qmv_i8_multi(static_cast<cudaStream_t>(stream), x, m, k, count, w, scales, biases, n, group_size, bits, y, flags);
        if (tc_ok)
            return qmv_tc_multi(static_cast<cudaStream_t>(stream), x, m, k, count, w, scales, biases, n, group_size, bits, y, flags);
    }
    // many rows: one GEMM launch whose row tiles cover all the linears (they fill the waves together)
    if (count >= 2 && m > kQmvMaxRows &&
        !(flags & (LISA_FLAG_FORCE_QMV | LISA_FLAG_FORCE_QMV_SIMPLE | LISA_FLAG_FORCE_QMV_TC | LISA_FLAG_FORCE_QMV_I8))) {
        bool gemm_ok = true;
        for (int i = 0; i < count; ++i) gemm_ok = gemm_ok && qmm_affine_supported(m, k, n[i], group_size, bits);
        if (gemm_ok)
            return qmm_affine_multi(static_cast<cudaStream_t>(stream), x, m, k, count, w, scales, biases, n, group_size, bits, y, flags);
    }
    for (int i = 0; i < count; ++i) {
        const int rc = quantized_matmul_impl(static_cast<cudaStream_t>(stream), x, m, k, w[i], scales[i], biases[i], n[i],
                                             transpose, group_size, bits, dtype, y[i], flags);
        if (rc != LISA_OK) return rc;
    }
    return LISA_OK;
}

int lisa_cuda_add_rmsnorm(lisa_stream_t stream, const void *x, const void *residual, const void *norm_weight, float eps, int64_t m,
                          int64_t k, int dtype, void *sum, void *normed) {
    if (!x || !residual || !norm_weight || !sum || !normed) return fail(LISA_ERR_BAD_ARG, "add_rmsnorm: null pointer");
    if (m < 1 || m > (1ll << 31) - 1 || k < 8 || k % 8 != 0 || k > (1 << 24)) return fail(LISA_ERR_BAD_ARG, "add_rmsnorm: k must be a multiple of 8");
    if (dtype != LISA_BF16) return fail(LISA_ERR_UNSUPPORTED, "add_rmsnorm: bf16 only");
    if (!(eps >= 0.f)) return fail(LISA_ERR_BAD_ARG, "add_rmsnorm: eps must not be negative");
    if (!aligned16(x) || !aligned16(residual) || !aligned16(norm_weight) || !aligned16(sum) || !aligned16(normed))
        return fail(LISA_ERR_MISALIGNED, "add_rmsnorm: pointers must be 16-byte aligned");
    return add_rmsnorm(static_cast<cudaStream_t>(stream), x, residual, norm_weight, eps, m, k, sum, normed);
}

int lisa_cuda_quantized_matmul_addnorm(lisa_stream_t stream, const void *x, const void *residual, const void *norm_weight, float eps,
                                       int64_t m, int64_t k, int count, const uint32_t *const *w, const void *const *scales,
                                       const void *const *biases, const int64_t *n, int transpose, int group_size, int bits,
                                       int dtype, void *const *y, void *sum, void *normed, unsigned flags) {
    if (!transpose) return fail(LISA_ERR_UNSUPPORTED, "quantized_matmul_addnorm: only transpose=true supported");
    if (count < 1 || count > 3 || !w || !scales || !biases || !n || !y)
        return fail(LISA_ERR_BAD_ARG, "quantized_matmul_addnorm: one to three linears, non-null tables");
    if (!residual || !norm_weight || !sum) return fail(LISA_ERR_BAD_ARG, "quantized_matmul_addnorm: null pointer");
    if (!(eps >= 0.f)) return fail(LISA_ERR_BAD_ARG, "quantized_matmul_addnorm: eps must not be negative");
    for (int i = 0; i < count; ++i) {
        const int rc = check_affine("quantized_matmul_addnorm", x, m, k, w[i], scales[i], biases[i], n[i], group_size, bits, dtype, y[i]);
        if (rc != LISA_OK) return rc;
    }
    if (k % 8 != 0 || !aligned16(residual) || !aligned16(norm_weight) || !aligned16(sum) || (normed && !aligned16(normed)))
        return fail(LISA_ERR_MISALIGNED, "quantized_matmul_addnorm: k must be a multiple of 8 and the pointers 16-byte aligned");
    const cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned forced = LISA_FLAG_FORCE_QMM | LISA_FLAG_FORCE_QMV | LISA_FLAG_FORCE_QMV_SIMPLE | LISA_FLAG_FORCE_QMV_I8;
    // decode rows through the tensor-memory kernel: the add and the norm happen in its activation staging
    if (m <= kQmvMaxRows && bits != 8 && !(flags & forced)) {
        const TcNormArgs norm{residual, norm_weight, eps, sum, normed};
        if (count == 1 && qmv_tc_supported(m, k, n[0], group_size, bits))
            return qmv_tc(st, x, m, k, w[0], scales[0], biases[0], n[0], group_size, bits, y[0], flags, &norm);
        if (count >= 2 && qmv_tc_multi_supported(m, k, count, n, group_size, bits))
            return qmv_tc_multi(st, x, m, k, count, w, scales, biases, n, group_size, bits, y, flags, 0, nullptr, nullptr, &norm);
    }
    // every other shape: the norm as a kernel of its own (it needs somewhere to put the normed rows), then the linears
    if (!normed) return fail(LISA_ERR_WORKSPACE, "quantized_matmul_addnorm: this shape runs unfused and needs the normed output buffer");
    int rc = add_rmsnorm(st, x, residual, norm_weight, eps, m, k, sum, normed);
    if (rc != LISA_OK) return rc;
    return lisa_cuda_quantized_matmul_siblings(stream, normed, m, k, count, w, scales, biases, n, transpose, group_size, bits, dtype, y, flags);
}

int lisa_cuda_quantized_matmul_swiglu(lisa_stream_t stream, const void *gate, const void *up, int64_t m, int64_t k, const uint32_t *w,
                                      const void *scales, const void *biases, int64_t n, int transpose, int group_size, int bits,
                                      int dtype, void *y, void *act, unsigned flags) {
    if (!transpose) return fail(LISA_ERR_UNSUPPORTED, "quantized_matmul_swiglu: only transpose=true supported");
    if (!up) return fail(LISA_ERR_BAD_ARG, "quantized_matmul_swiglu: null pointer");
    const int rc = check_affine("quantized_matmul_swiglu", gate, m, k, w, scales, biases, n, group_size, bits, dtype, y);
    if (rc != LISA_OK) return rc;
    if (k % 8 != 0 || !aligned16(up) || (act && !aligned16(act)))
        return fail(LISA_ERR_MISALIGNED, "quantized_matmul_swiglu: k must be a multiple of 8 and the pointers 16-byte aligned");
    const cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned forced = LISA_FLAG_FORCE_QMM | LISA_FLAG_FORCE_QMV | LISA_FLAG_FORCE_QMV_SIMPLE | LISA_FLAG_FORCE_QMV_I8;
    // decode rows: the activation is formed in the staging of the tensor-memory kernel
    if (m <= kQmvMaxRows && bits != 8 && !(flags & forced) && qmv_tc_supported(m, k, n, group_size, bits)) {
        const TcNormArgs fuse{up, nullptr, 0.f, nullptr, act};
        return qmv_tc(st, gate, m, k, w, scales, biases, n, group_size, bits, y, flags, &fuse);
    }
    if (!act) return fail(LISA_ERR_WORKSPACE, "quantized_matmul_swiglu: this shape runs unfused and needs the activation buffer");
    const int rs = moe_swiglu(st, gate, up, m * k, act);
    if (rs != LISA_OK) return rs;
    return quantized_matmul_impl(st, act, m, k, w, scales, biases, n, transpose, group_size, bits, dtype, y, flags);
}

int lisa_cuda_quantized_matmul_siblings_allgather(lisa_stream_t stream, const void *x, int64_t m, int64_t k, int count,
                                                  const uint32_t *const *w, const void *const *scales,
                                                  const void *const *biases, const int64_t *n_local, int transpose,
                                                  int group_size, int bits, int dtype, void *const *y_all, int world,
                                                  const int64_t *n_total, const int64_t *col0, unsigned flags) {
    if (!transpose) return fail(LISA_ERR_UNSUPPORTED, "quantized_matmul_siblings_allgather: only transpose=true supported");
    if (count < 1 || count > 3 || !w || !scales || !biases || !n_local || !y_all || !n_total || !col0)
        return fail(LISA_ERR_BAD_ARG, "quantized_matmul_siblings_allgather: one to three linears, non-null tables");
    if (world < 1 || world > 8) return fail(LISA_ERR_BAD_ARG, "quantized_matmul_siblings_allgather: 1 to 8 output buffers per linear");
    for (int i = 0; i < count; ++i) {
        for (int r = 0; r < world; ++r)
            if (!y_all[i * world + r] || (reinterpret_cast<uintptr_t>(y_all[i * world + r]) & 1u))
                return fail(LISA_ERR_BAD_ARG, "quantized_matmul_siblings_allgather: null or misaligned output buffer");
        const int rc = check_affine("quantized_matmul_siblings_allgather", x, m, k, w[i], scales[i], biases[i], n_local[i], group_size,
                                    bits, dtype, y_all[i * world]);
        if (rc != LISA_OK) return rc;
        if (col0[i] < 0 || n_total[i] < 1 || col0[i] + n_local[i] > n_total[i] || n_total[i] > (1ll << 30))
            return fail(LISA_ERR_BAD_ARG, "quantized_matmul_siblings_allgather: column block outside the output");
    }
    // one launch when the tensor-memory GEMV takes the rows; otherwise one fused launch per linear
    if (count >= 2 && m <= kQmvMaxRows && qmv_tc_multi_supported(m, k, count, n_local, group_size, bits))
        return qmv_tc_multi(static_cast<cudaStream_t>(stream), x, m, k, count, w, scales, biases, n_local, group_size, bits, y_all,
                            flags, world, n_total, col0);
    for (int i = 0; i < count; ++i) {
        const int rc = lisa_cuda_quantized_matmul_allgather(stream, x, m, k, w[i], scales[i], biases[i], n_local[i], transpose,
                                                            group_size, bits, dtype, y_all + i * world, world, n_total[i], col0[i], flags);
        if (rc != LISA_OK) return rc;
    }
    return LISA_OK;
}

int lisa_cuda_peer_barrier(lisa_stream_t stream, int rank, int world, void *const *flag_arrays, uint64_t epoch) {
    if (!flag_arrays || world < 1 || world > 8 || rank < 0 || rank >= world)
        return fail(LISA_ERR_BAD_ARG, "peer_barrier: bad rank or world");
    for (int r = 0; r < world; ++r)
        if (!flag_arrays[r] || (reinterpret_cast<uintptr_t>(flag_arrays[r]) & 7u)) return fail(LISA_ERR_BAD_ARG, "peer_barrier: null or misaligned flag array");
    return peer_barrier(static_cast<cudaStream_t>(stream), rank, world, flag_arrays, epoch);
}

int lisa_cuda_dequantize(lisa_stream_t stream, const uint32_t *w, const void *scales, const void *biases,
                         int64_t rows, int64_t k, int group_size, int bits, int dtype, void *out) {
    if (!w || !scales || !biases || !out) return fail(LISA_ERR_BAD_ARG, "dequantize: null pointer");
    if (rows < 1 || k < 1) return fail(LISA_ERR_BAD_ARG, "dequantize: sizes must be positive");
    if (bits != 2 && bits != 4 && bits != 8) return fail(LISA_ERR_UNSUPPORTED, "dequantize: bits must be 2, 4 or 8");
    if (group_size != 32 && group_size != 64 && group_size != 128)
        return fail(LISA_ERR_UNSUPPORTED, "dequantize: group_size must be 32, 64 or 128");
    if (dtype != LISA_BF16 && dtype != LISA_F16 && dtype != LISA_F32) return fail(LISA_ERR_UNSUPPORTED, "dequantize: unsupported dtype");
    if (k % group_size != 0) return fail(LISA_ERR_BAD_ARG, "dequantize: k is not a multiple of group_size");
    if (rows * k > (1ll << 42)) return fail(LISA_ERR_OVERFLOW, "dequantize: shape too large");
    if (!aligned16(w) || !aligned16(scales) || !aligned16(biases) || !aligned16(out))
        return fail(LISA_ERR_MISALIGNED, "dequantize: pointers must be 16-byte aligned");
    if (dtype != LISA_BF16) return dequantize_typed(static_cast<cudaStream_t>(stream), dtype, w, scales, biases, rows, k, group_size, bits, out);
    return dequantize_affine(static_cast<cudaStream_t>(stream), w, scales, biases, rows, k, group_size, bits, out);
}

int lisa_cuda_dequantize_rows(lisa_stream_t stream, const uint32_t *w, const void *scales, const void *biases,
                              const int32_t *ids, int64_t count, int64_t vocab, int64_t k, int group_size, int bits, int dtype,
                              void *out) {
    if (!w || !scales || !biases || !ids || !out) return fail(LISA_ERR_BAD_ARG, "dequantize_rows: null pointer");
    if (count < 1 || vocab < 1 || k < 1) return fail(LISA_ERR_BAD_ARG, "dequantize_rows: sizes must be positive");
    if (bits != 2 && bits != 4 && bits != 8) return fail(LISA_ERR_UNSUPPORTED, "dequantize_rows: bits must be 2, 4 or 8");
    if (group_size != 32 && group_size != 64 && group_size != 128)
        return fail(LISA_ERR_UNSUPPORTED, "dequantize_rows: group_size must be 32, 64 or 128");
    if (dtype != LISA_BF16) return fail(LISA_ERR_UNSUPPORTED, "dequantize_rows: unsupported dtype (bf16 only)");
    if (k % group_size != 0) return fail(LISA_ERR_BAD_ARG, "dequantize_rows: k is not a multiple of group_size");
    if (count * k > (1ll << 42) || vocab * k > (1ll << 44)) return fail(LISA_ERR_OVERFLOW, "dequantize_rows: shape too large");
    if (!aligned16(w) || !aligned16(scales) || !aligned16(biases) || !aligned16(out) || (reinterpret_cast<uintptr_t>(ids) & 3u))
        return fail(LISA_ERR_MISALIGNED, "dequantize_rows: pointers must be 16-byte aligned (ids 4-byte)");
    return dequantize_affine_rows(static_cast<cudaStream_t>(stream), w, scales, biases, ids, count, vocab, k, group_size, bits, out);
}

int lisa_cuda_quantize(lisa_stream_t stream, const void *w, int64_t rows, int64_t k, int group_size, int bits, int dtype,
                       uint32_t *wq, void *scales, void *biases) {
    if (!w || !wq || !scales || !biases) return fail(LISA_ERR_BAD_ARG, "quantize: null pointer");
    if (rows < 1 || k < 1) return fail(LISA_ERR_BAD_ARG, "quantize: sizes must be positive");
    if (bits != 2 && bits != 4 && bits != 8) return fail(LISA_ERR_UNSUPPORTED, "quantize: bits must be 2, 4 or 8");
    if (group_size < 1 || k % group_size != 0 || group_size % (32 / bits) != 0) {
        std::ostringstream os;  // array_ops.rs:226-228
        os << "quantize: group size " << group_size << " incompatible with K=" << k << ", bits=" << bits;
        return fail(LISA_ERR_BAD_ARG, os.str());
    }
    if (dtype != LISA_BF16) return fail(LISA_ERR_UNSUPPORTED, "quantize: unsupported dtype (bf16 only)");
    if (rows * k > (1ll << 42)) return fail(LISA_ERR_OVERFLOW, "quantize: shape too large");
    if (!aligned16(w) || !aligned16(wq) || !aligned16(scales) || !aligned16(biases))
        return fail(LISA_ERR_MISALIGNED, "quantize: pointers must be 16-byte aligned");
    return quantize_affine(static_cast<cudaStream_t>(stream), w, rows, k, group_size, bits, wq, scales, biases);
}

size_t lisa_cuda_gather_qmm_workspace_bytes(int64_t rows, int64_t experts) {
    return gather_qmm_workspace_bytes(rows, experts);
}

int lisa_cuda_gather_qmm(lisa_stream_t stream, const void *x, int64_t rows, int64_t k, const uint32_t *w,
                         const void *scales, const void *biases, const int32_t *lhs_indices,
                         const int32_t *rhs_indices, int64_t experts, int64_t n, int transpose, int group_size,
                         int bits, int sorted_indices, int dtype, void *y, void *workspace, size_t workspace_bytes) {
    if (!transpose) return fail(LISA_ERR_UNSUPPORTED, "gather_qmm: only transpose=true supported");
    if (lhs_indices) return fail(LISA_ERR_UNSUPPORTED, "gather_qmm: lhs_indices path not ported");
    if (!sorted_indices) return fail(LISA_ERR_UNSUPPORTED, "gather_qmm: only sorted_indices=true supported");
    if (!rhs_indices) return fail(LISA_ERR_BAD_ARG, "gather_qmm: rhs_indices required");
    int rc = check_affine("gather_qmm", x, rows, k, w, scales, biases, n, group_size, bits, dtype, y);
    if (rc != LISA_OK) return rc;
    if (experts < 1 || experts > (1 << 20)) return fail(LISA_ERR_BAD_ARG, "gather_qmm: bad expert count");
    if (experts * n * k > (1ll << 44)) return fail(LISA_ERR_OVERFLOW, "gather_qmm: shape too large");
    const size_t need = gather_qmm_workspace_bytes(rows, experts);
    if (need > 0 && (!workspace || workspace_bytes < need))
        return fail(LISA_ERR_WORKSPACE, "gather_qmm: workspace missing or too small");
    if (workspace && !aligned16(workspace)) return fail(LISA_ERR_MISALIGNED, "gather_qmm: workspace must be 16-byte aligned");
    return gather_qmm_affine(static_cast<cudaStream_t>(stream), x, rows, k, w, scales, biases, rhs_indices, experts, n,
                             group_size, bits, y, workspace, workspace_bytes);
}

int lisa_cuda_gather_qmm_siblings(lisa_stream_t stream, const void *x, int64_t rows, int64_t k, int count, const uint32_t *const *w,
                                  const void *const *scales, const void *const *biases, const int32_t *rhs_indices, int64_t experts,
                                  int64_t n, int transpose, int group_size, int bits, int sorted_indices, int dtype, void *const *y,
                                  void *workspace, size_t workspace_bytes) {
    if (!transpose) return fail(LISA_ERR_UNSUPPORTED, "gather_qmm_siblings: only transpose=true supported");
    if (!sorted_indices) return fail(LISA_ERR_UNSUPPORTED, "gather_qmm_siblings: only sorted_indices=true supported");
    if (!rhs_indices) return fail(LISA_ERR_BAD_ARG, "gather_qmm_siblings: rhs_indices required");
    if (count < 1 || count > 3 || !w || !scales || !biases || !y)
        return fail(LISA_ERR_BAD_ARG, "gather_qmm_siblings: one to three linears, non-null tables");
    for (int i = 0; i < count; ++i) {
        const int rc = check_affine("gather_qmm_siblings", x, rows, k, w[i], scales[i], biases[i], n, group_size, bits, dtype, y[i]);
        if (rc != LISA_OK) return rc;
    }
    if (experts < 1 || experts > (1 << 20)) return fail(LISA_ERR_BAD_ARG, "gather_qmm_siblings: bad expert count");
    if (experts * n * k > (1ll << 44)) return fail(LISA_ERR_OVERFLOW, "gather_qmm_siblings: shape too large");
    const size_t need = gather_qmm_workspace_bytes(rows, experts);
    if (need > 0 && (!workspace || workspace_bytes < need))
        return fail(LISA_ERR_WORKSPACE, "gather_qmm_siblings: workspace missing or too small");
    if (workspace && !aligned16(workspace)) return fail(LISA_ERR_MISALIGNED, "gather_qmm_siblings: workspace must be 16-byte aligned");
    return gather_qmm_affine_multi(static_cast<cudaStream_t>(stream), x, rows, k, count, w, scales, biases, rhs_indices, experts, n,
                                   group_size, bits, y, workspace, workspace_bytes);
}

static int gguf_geometry(const char *op, int format, int64_t rows, int64_t row_bytes, int *block_bytes) {
    std::string name(op);
    if (format == LISA_GGUF_Q2_K) *block_bytes = 84;
    else if (format == LISA_GGUF_Q4_K) *block_bytes = 144;
    else if (format == LISA_GGUF_Q5_K) *block_bytes = 176;
    else return fail(LISA_ERR_UNSUPPORTED, name + ": unsupported GGUF block format");
    // deepseek41.rs:50-65
    if (rows <= 0 || row_bytes <= 0 || rows % 8 != 0 || row_bytes % *block_bytes != 0)
        return fail(LISA_ERR_BAD_ARG, name + ": unsupported GGUF quantized matvec layout");
    if (row_bytes / *block_bytes > (1 << 22)) return fail(LISA_ERR_OVERFLOW, name + ": GGUF quantized input width overflow");
    return LISA_OK;
}

int lisa_cuda_gguf_packed_matvec(lisa_stream_t stream, int format, const uint8_t *w, int64_t rows, int64_t row_bytes,
                                 const float *x, int64_t tokens, float *y) {
    int block = 0;
    int rc = gguf_geometry("packed_matvec", format, rows, row_bytes, &block);
    if (rc != LISA_OK) return rc;
    if (!w || !x || !y) return fail(LISA_ERR_BAD_ARG, "packed_matvec: null pointer");
    if (tokens < 1 || tokens > 65535) return fail(LISA_ERR_BAD_ARG, "invalid GGUF matvec input rows");
    if ((reinterpret_cast<uintptr_t>(w) & 1u) != 0) return fail(LISA_ERR_MISALIGNED, "packed_matvec: weights must be 2-byte aligned");
    if (!aligned16(x) || (reinterpret_cast<uintptr_t>(y) & 3u) != 0)
        return fail(LISA_ERR_MISALIGNED, "packed_matvec: x must be 16-byte and y 4-byte aligned");
    // one or two tokens of a Q4_K matrix: the tensor-memory kernel (exact on dyadic inputs like the warp-per-row one)
    if (aligned16(w) && row_bytes % 16 == 0 && qmv_tc_gguf_supported(format, tokens, rows, row_bytes))
        return qmv_tc_gguf(static_cast<cudaStream_t>(stream), format, w, rows, row_bytes, x, tokens, y);
    return gguf_matvec(static_cast<cudaStream_t>(stream), format, w, 1, rows, row_bytes, x, tokens, 1, nullptr, 1, y);
}

int lisa_cuda_gguf_packed_matvec_allgather(lisa_stream_t stream, int format, const uint8_t *w, int64_t rows_local,
                                           int64_t row_bytes, const float *x, int64_t tokens, void *const *y_all, int world,
                                           int64_t rows_total, int64_t row0) {
    int block = 0;
    int rc = gguf_geometry("packed_matvec_allgather", format, rows_local, row_bytes, &block);
    if (rc != LISA_OK) return rc;
    if (!w || !x || !y_all) return fail(LISA_ERR_BAD_ARG, "packed_matvec_allgather: null pointer");
    if (world < 1 || world > 8) return fail(LISA_ERR_BAD_ARG, "packed_matvec_allgather: 1 to 8 output buffers");
    for (int r = 0; r < world; ++r)
        if (!y_all[r] || (reinterpret_cast<uintptr_t>(y_all[r]) & 3u)) return fail(LISA_ERR_BAD_ARG, "packed_matvec_allgather: null or misaligned output buffer");
    if (tokens < 1 || tokens > 65535) return fail(LISA_ERR_BAD_ARG, "invalid GGUF matvec input rows");
    if (row0 < 0 || rows_total < 1 || row0 + rows_local > rows_total || rows_total > (1ll << 30))
        return fail(LISA_ERR_BAD_ARG, "packed_matvec_allgather: row block outside the output");
    if (!aligned16(w) || !aligned16(x) || row_bytes % 16 != 0) return fail(LISA_ERR_MISALIGNED, "packed_matvec_allgather: w and x must be 16-byte aligned");
    if (!qmv_tc_gguf_supported(format, tokens, rows_local, row_bytes))
        return fail(LISA_ERR_UNSUPPORTED, "packed_matvec_allgather: the fused form takes what the tensor-memory kernel takes "
                                          "(Q4_K: one or two tokens; Q2_K: one token, rows of whole 336-byte groups that fit its stages)");
    return qmv_tc_gguf_allgather(static_cast<cudaStream_t>(stream), format, w, rows_local, row_bytes, x, tokens,
                                 reinterpret_cast<float *const *>(y_all), world, rows_total, row0);
}

size_t lisa_cuda_gguf_packed_matmul_workspace_bytes(int64_t tokens, int64_t row_bytes, int format) {
    const int block = (format == LISA_GGUF_Q2_K) ? 84 : (format == LISA_GGUF_Q5_K) ? 176 : 144;
    if (tokens < 1 || row_bytes < block) return 0;
    return qmm_gguf_workspace_bytes(tokens, row_bytes / block * 256);
}

// Tokens from which the tensor-core product replaces the per-token matvecs.
static const int64_t kGgufGemmMinTokens = 32;

int lisa_cuda_gguf_packed_matmul(lisa_stream_t stream, int format, const uint8_t *w, int64_t rows, int64_t row_bytes,
                                 const float *x, int64_t tokens, float *y, void *workspace, size_t workspace_bytes) {
    int block = 0;
    int rc = gguf_geometry("packed_matmul", format, rows, row_bytes, &block);
    if (rc != LISA_OK) return rc;
    const bool gemm = workspace && tokens >= kGgufGemmMinTokens && qmm_gguf_supported(format, tokens, rows, row_bytes) &&
                      aligned16(w) && row_bytes % 16 == 0;
    if (!gemm) return lisa_cuda_gguf_packed_matvec(stream, format, w, rows, row_bytes, x, tokens, y);
    if (!w || !x || !y) return fail(LISA_ERR_BAD_ARG, "packed_matmul: null pointer");
    if (tokens > 65535) return fail(LISA_ERR_BAD_ARG, "invalid GGUF matvec input rows");
    if (!aligned16(x) || (reinterpret_cast<uintptr_t>(y) & 3u) != 0 || !aligned16(workspace))
        return fail(LISA_ERR_MISALIGNED, "packed_matmul: x and workspace must be 16-byte and y 4-byte aligned");
    if (workspace_bytes < lisa_cuda_gguf_packed_matmul_workspace_bytes(tokens, row_bytes, format))
        return fail(LISA_ERR_WORKSPACE, "packed_matmul: workspace too small");
    return qmm_gguf(static_cast<cudaStream_t>(stream), format, w, rows, row_bytes, x, tokens, y, workspace);
}

int lisa_cuda_gguf_expert_matvec(lisa_stream_t stream, int format, const uint8_t *w, int64_t experts, int64_t rows,
                                 int64_t row_bytes, const float *x, int64_t tokens, int64_t slots, const int32_t *ids,
                                 int64_t top_k, float *y) {
    int block = 0;
    int rc = gguf_geometry("expert_matvec", format, rows, row_bytes, &block);
    if (rc != LISA_OK) return rc;
    if (!w || !x || !y || !ids) return fail(LISA_ERR_BAD_ARG, "expert_matvec: null pointer");
    // deepseek41.rs:216-228
    if (experts < 1 || tokens < 1 || tokens > 65535 || top_k < 1 || top_k > 32 || (slots != 1 && slots != top_k))
        return fail(LISA_ERR_BAD_ARG, "invalid GGUF expert matvec geometry");
    if ((reinterpret_cast<uintptr_t>(w) & 1u) != 0) return fail(LISA_ERR_MISALIGNED, "expert_matvec: weights must be 2-byte aligned");
    if (!aligned16(x) || (reinterpret_cast<uintptr_t>(y) & 3u) != 0 || (reinterpret_cast<uintptr_t>(ids) & 3u) != 0)
        return fail(LISA_ERR_MISALIGNED, "expert_matvec: x must be 16-byte, y and ids 4-byte aligned");
    // decode-sized id tables: every slot as a one-token launch tile of the tensor-memory kernel (exact on dyadic
    // inputs like the warp-per-row kernel; ids outside the table store zeros and touch no weights there too)
    if (aligned16(w) && row_bytes % 16 == 0 && qmv_tc_gguf_expert_supported(format, tokens * top_k, experts, rows, row_bytes))
        return qmv_tc_gguf_expert(static_cast<cudaStream_t>(stream), format, w, experts, rows, row_bytes, x, tokens, slots, ids,
                                  top_k, y);
    return gguf_matvec(static_cast<cudaStream_t>(stream), format, w, experts, rows, row_bytes, x, tokens, slots, ids, top_k, y);
}

int lisa_cuda_moe_route(lisa_stream_t stream, const float *logits, int64_t tokens, int64_t experts, int top_k,
                        int32_t *idx, float *weights) {
    if (!logits || !idx || !weights) return fail(LISA_ERR_BAD_ARG, "moe_route: null pointer");
    if (tokens < 1 || experts < 1 || top_k < 1 || top_k > experts) return fail(LISA_ERR_BAD_ARG, "moe_route: bad sizes");
    if (top_k > 32 || experts > 1024) return fail(LISA_ERR_LIMIT, "moe_route: top_k <= 32 and experts <= 1024");
    return moe_route(static_cast<cudaStream_t>(stream), logits, tokens, experts, top_k, idx, weights);
}

size_t lisa_cuda_moe_sort_workspace_bytes(int64_t slots, int64_t experts) { return moe_sort_workspace_bytes(slots, experts); }

int lisa_cuda_moe_sort(lisa_stream_t stream, const int32_t *idx, int64_t slots, int64_t experts, int top_k,
                       int32_t *sorted_ids, int32_t *token_rows, int32_t *inverse, void *workspace,
                       size_t workspace_bytes) {
    if (!idx || !sorted_ids || !token_rows || !inverse) return fail(LISA_ERR_BAD_ARG, "moe_sort: null pointer");
    if (slots < 1 || experts < 1 || top_k < 1 || slots > (1ll << 30)) return fail(LISA_ERR_BAD_ARG, "moe_sort: bad sizes");
    if (experts > 4096) return fail(LISA_ERR_LIMIT, "moe_sort: experts <= 4096");
    if (!workspace || workspace_bytes < moe_sort_workspace_bytes(slots, experts))
        return fail(LISA_ERR_WORKSPACE, "moe_sort: workspace missing or too small");
    if (!aligned16(workspace)) return fail(LISA_ERR_MISALIGNED, "moe_sort: workspace must be 16-byte aligned");
    return moe_sort(static_cast<cudaStream_t>(stream), idx, slots, experts, top_k, sorted_ids, token_rows, inverse,
                    workspace);
}

int lisa_cuda_moe_sort_static(lisa_stream_t stream, const int32_t *idx, int64_t slots, int64_t experts, int top_k,
                              int32_t *sorted_ids, int32_t *token_rows, int32_t *inverse) {
    if (!idx || !sorted_ids || !token_rows || !inverse) return fail(LISA_ERR_BAD_ARG, "moe_sort_static: null pointer");
    if (slots < 1 || experts < 1 || top_k < 1 || slots > (1ll << 30)) return fail(LISA_ERR_BAD_ARG, "moe_sort_static: bad sizes");
    if (experts > 4096) return fail(LISA_ERR_LIMIT, "moe_sort_static: experts <= 4096");
    return moe_sort_static(static_cast<cudaStream_t>(stream), idx, slots, experts, top_k, sorted_ids, token_rows, inverse);
}

int lisa_cuda_gather_rows(lisa_stream_t stream, const void *x, const int32_t *token_rows, int64_t rows, int64_t width,
                          int dtype, void *out) {
    if (!x || !token_rows || !out) return fail(LISA_ERR_BAD_ARG, "gather_rows: null pointer");
    if (rows < 1 || width < 1) return fail(LISA_ERR_BAD_ARG, "gather_rows: bad sizes");
    if (dtype != LISA_BF16) return fail(LISA_ERR_UNSUPPORTED, "gather_rows: bf16 only");
    if (width % 8 != 0 || !aligned16(x) || !aligned16(out))
        return fail(LISA_ERR_MISALIGNED, "gather_rows: width must be a multiple of 8 and pointers 16-byte aligned");
    return moe_gather_rows(static_cast<cudaStream_t>(stream), x, token_rows, rows, width, out);
}

int lisa_cuda_swiglu(lisa_stream_t stream, const void *gate, const void *up, int64_t count, int dtype, void *act) {
    if (!gate || !up || !act) return fail(LISA_ERR_BAD_ARG, "swiglu: null pointer");
    if (count < 1) return fail(LISA_ERR_BAD_ARG, "swiglu: bad size");
    if (dtype != LISA_BF16) return fail(LISA_ERR_UNSUPPORTED, "swiglu: bf16 only");
    return moe_swiglu(static_cast<cudaStream_t>(stream), gate, up, count, act);
}

int lisa_cuda_moe_combine(lisa_stream_t stream, const void *down_sorted, const float *weights, const int32_t *inverse,
                          int64_t tokens, int top_k, int64_t hidden, int dtype, void *out) {
    if (!down_sorted || !weights || !inverse || !out) return fail(LISA_ERR_BAD_ARG, "moe_combine: null pointer");
    if (tokens < 1 || top_k < 1 || hidden < 1) return fail(LISA_ERR_BAD_ARG, "moe_combine: bad sizes");
    if (top_k > 32) return fail(LISA_ERR_LIMIT, "moe_combine: top_k <= 32");
    if (dtype != LISA_BF16) return fail(LISA_ERR_UNSUPPORTED, "moe_combine: bf16 only");
    return moe_combine(static_cast<cudaStream_t>(stream), down_sorted, weights, inverse, tokens, top_k, hidden, out);
}

static int check_moe_decode(const char *op, int64_t experts, int64_t k, int64_t n, int top_k, int group_size, int bits, int dtype) {
    std::string name(op);
    if (dtype != LISA_BF16) return fail(LISA_ERR_UNSUPPORTED, name + ": bf16 only");
    if (experts < 1 || experts > (1 << 20) || k < 1 || n < 1) return fail(LISA_ERR_BAD_ARG, name + ": bad sizes");
    if (experts * n * k > (1ll << 44)) return fail(LISA_ERR_OVERFLOW, name + ": shape too large");
    if (top_k < 1 || top_k > 32) return fail(LISA_ERR_LIMIT, name + ": top_k must be 1..32");
    if (!moe_decode_supported(k, group_size, bits, top_k))
        return fail(LISA_ERR_UNSUPPORTED, name + ": needs 2- or 4-bit codes, a group size that is a multiple of 32, "
                                                 "rows of whole 16-byte chunks and top_k rows of activations within 160 KiB");
    return LISA_OK;
}

int lisa_cuda_moe_gate_up_act(lisa_stream_t stream, const void *x, const int32_t *idx, const int32_t *xrow, int64_t slots,
                              int top_k, int64_t experts, int64_t hidden, int64_t inter, const uint32_t *wg, const void *sg,
                              const void *bg, const uint32_t *wu, const void *su, const void *bu, int group_size, int bits,
                              int dtype, void *act) {
    if (!x || !idx || !wg || !sg || !bg || !wu || !su || !bu || !act) return fail(LISA_ERR_BAD_ARG, "moe_gate_up_act: null pointer");
    if (slots < 1 || slots > (1 << 24)) return fail(LISA_ERR_BAD_ARG, "moe_gate_up_act: bad slot count");
    const int rc = check_moe_decode("moe_gate_up_act", experts, hidden, inter, top_k, group_size, bits, dtype);
    if (rc != LISA_OK) return rc;
    if (!aligned16(x) || !aligned16(wg) || !aligned16(wu)) return fail(LISA_ERR_MISALIGNED, "moe_gate_up_act: pointers must be 16-byte aligned");
    return moe_gate_up_act(static_cast<cudaStream_t>(stream), x, idx, xrow, slots, top_k, experts, hidden, inter, wg, sg, bg, wu, su,
                           bu, group_size, bits, act);
}

int lisa_cuda_moe_down_combine(lisa_stream_t stream, const void *act, const int32_t *idx, const float *weights, int64_t tokens,
                               int top_k, int64_t experts, int64_t inter, int64_t hidden, const uint32_t *wd, const void *sd,
                               const void *bd, int group_size, int bits, int dtype, void *out) {
    if (!act || !idx || !weights || !wd || !sd || !bd || !out) return fail(LISA_ERR_BAD_ARG, "moe_down_combine: null pointer");
    if (tokens < 1 || tokens > (1 << 24)) return fail(LISA_ERR_BAD_ARG, "moe_down_combine: bad token count");
    const int rc = check_moe_decode("moe_down_combine", experts, inter, hidden, top_k, group_size, bits, dtype);
    if (rc != LISA_OK) return rc;
    if (!aligned16(act) || !aligned16(wd)) return fail(LISA_ERR_MISALIGNED, "moe_down_combine: pointers must be 16-byte aligned");
    return moe_down_combine(static_cast<cudaStream_t>(stream), act, idx, weights, tokens, top_k, experts, inter, hidden, wd, sd, bd,
                            group_size, bits, out);
}

static int check_ep(const char *op, int world, int rank, int64_t experts, int64_t hidden, void *const *a, void *const *b) {
    std::string name(op);
    if (world < 1 || world > 8 || rank < 0 || rank >= world) return fail(LISA_ERR_BAD_ARG, name + ": bad rank or world");
    if (experts < world || experts % world != 0) return fail(LISA_ERR_BAD_ARG, name + ": the experts do not split over the ranks");
    if (hidden < 8 || hidden % 8 != 0) return fail(LISA_ERR_MISALIGNED, name + ": hidden must be a multiple of 8");
    for (int r = 0; r < world; ++r) {
        if (!a || !a[r] || !aligned16(a[r])) return fail(LISA_ERR_BAD_ARG, name + ": null or misaligned peer buffer");
        if (b && (!b[r] || (reinterpret_cast<uintptr_t>(b[r]) & 3u))) return fail(LISA_ERR_BAD_ARG, name + ": null or misaligned peer buffer");
    }
    return LISA_OK;
}

int lisa_cuda_ep_counts(lisa_stream_t stream, const int32_t *sorted_ids, int64_t slots, int64_t experts, int world, int rank,
                        void *const *count_matrices) {
    if (!sorted_ids || slots < 1 || slots > (1ll << 30)) return fail(LISA_ERR_BAD_ARG, "ep_counts: null ids or bad slot count");
    const int rc = check_ep("ep_counts", world, rank, experts, 8, count_matrices, nullptr);
    if (rc != LISA_OK) return rc;
    return ep_counts(static_cast<cudaStream_t>(stream), sorted_ids, slots, experts, world, rank, count_matrices);
}

int lisa_cuda_ep_dispatch(lisa_stream_t stream, const void *x, const int32_t *sorted_ids, const int32_t *token_rows,
                          int64_t slots, int64_t hidden, int64_t experts, int world, int rank, const int32_t *count_matrix,
                          void *const *recv_x, void *const *recv_ids, int dtype) {
    if (!x || !sorted_ids || !token_rows || !count_matrix || slots < 1 || slots > (1ll << 30))
        return fail(LISA_ERR_BAD_ARG, "ep_dispatch: null pointer or bad slot count");
    if (dtype != LISA_BF16) return fail(LISA_ERR_UNSUPPORTED, "ep_dispatch: bf16 only");
    if (!aligned16(x)) return fail(LISA_ERR_MISALIGNED, "ep_dispatch: x must be 16-byte aligned");
    const int rc = check_ep("ep_dispatch", world, rank, experts, hidden, recv_x, recv_ids);
    if (rc != LISA_OK) return rc;
    return ep_dispatch(static_cast<cudaStream_t>(stream), x, sorted_ids, token_rows, slots, hidden, experts, world, rank,
                       count_matrix, recv_x, recv_ids);
}

int lisa_cuda_ep_return(lisa_stream_t stream, const void *rows, const int32_t *recv_index, int64_t count, int64_t hidden,
                        int world, int rank, const int32_t *count_matrix, void *const *back, int dtype) {
    if (count < 0 || count > (1ll << 30)) return fail(LISA_ERR_BAD_ARG, "ep_return: bad row count");
    if (count > 0 && (!rows || !recv_index)) return fail(LISA_ERR_BAD_ARG, "ep_return: null pointer");
    if (!count_matrix) return fail(LISA_ERR_BAD_ARG, "ep_return: null count matrix");
    if (dtype != LISA_BF16) return fail(LISA_ERR_UNSUPPORTED, "ep_return: bf16 only");
    if (count > 0 && !aligned16(rows)) return fail(LISA_ERR_MISALIGNED, "ep_return: rows must be 16-byte aligned");
    const int rc = check_ep("ep_return", world, rank, world, hidden, back, nullptr);
    if (rc != LISA_OK) return rc;
    return ep_return(static_cast<cudaStream_t>(stream), rows, recv_index, count, hidden, world, rank, count_matrix, back);
}

}  // extern "C"
