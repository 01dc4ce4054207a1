// Host-side construction of TMA tensor maps (cuTensorMapEncodeTiled through the runtime's
// driver entry point, so the library does not link against libcuda).
#pragma once

#include <cuda.h>
#include <stdint.h>

namespace lisa {

// rank <= 3.  dims[0] is the contiguous dimension (elements); strides_bytes[i] is the byte
// stride of dims[i + 1].  Returns a lisa_status and records the error string on failure.
int make_tensor_map(CUtensorMap *map, CUtensorMapDataType dtype, int rank, const void *base, const uint64_t *dims,
                    const uint64_t *strides_bytes, const uint32_t *box, CUtensorMapSwizzle swizzle);

}  // namespace lisa
