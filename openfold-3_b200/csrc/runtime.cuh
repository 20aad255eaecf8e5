// Host-side runtime pieces shared by the entry points: tensor-map encoding through the
// driver entry point (no link-time dependency on libcuda), launch-attribute helpers.
#pragma once
#include <cuda.h>
#include "common.cuh"

namespace of3 {

// Encodes a tiled bf16 tensor map. dims/strides are innermost-first; strides_bytes has
// rank-1 entries (stride of dim 1.., the innermost is dense). Returns OF3_OK or an error code.
int make_tmap_bf16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                   const uint64_t* strides_bytes, const uint32_t* box, bool swizzle128);

// Number of SMs of the current device (cached per device).
int sm_count();

}  // namespace of3
