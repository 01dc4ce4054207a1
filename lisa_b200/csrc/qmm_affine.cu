// Placeholder translation unit: the tcgen05 GEMM is not built yet.
#include <cuda_runtime.h>

#include "common.cuh"
#include "kernels.h"

namespace lisa {
bool qmm_affine_supported(int64_t, int64_t, int64_t, int, int) { return false; }
int qmm_affine(cudaStream_t, const void *, int64_t, int64_t, const uint32_t *, const void *, const void *, int64_t,
               int, int, void *, unsigned) {
    return fail(LISA_ERR_UNSUPPORTED, "qmm: not built");
}
int qmm_device_status() { return 0; }
}  // namespace lisa
