// Host-side runtime pieces shared by the entry points: tensor-map encoding through the
// driver entry point (no link-time dependency on libcuda), launch-attribute helpers.
#pragma once
#include <cuda.h>
#include "common.cuh"

namespace of3 {

// Encodes a tiled bf16 tensor map. dims/strides are innermost-first; strides_bytes has
// rank-1 entries (stride of dim 1.., the innermost is dense). Returns OF3_OK or an error code.
// swizzle: 0 none, 1 (or true) 128-byte, 2 64-byte. Encoded maps are kept in a locked cache keyed by
// every argument, so a steady-state launch costs a lookup instead of a driver call per operand.
int make_tmap_bf16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                   const uint64_t* strides_bytes, const uint32_t* box, int swizzle);

// Per-kernel launch accounting. Every launch site of this library opens a LaunchScope with its
// kernel id: launches are always counted; when timing is enabled (of3_profile_enable) a CUDA event
// pair is recorded around the launch on the launching stream, and of3_profile_read sums their
// elapsed times. Ids: 1 contract, 2 trimul_in, 3 trimul_out, 4 transition, 5 triattn_proj,
// 6 triattn_core, 7 triattn_out, 8 single-track kernels, 9 pair-bias projection, 10 linear layers of the
// single track (the contraction kernel as a plain GEMM), 20 the shape-generic SIMT kernels, 30 / 31 peer
// barrier / pull.
constexpr int kMaxKernelIds = 32;
struct LaunchScope {
    int kid;
    cudaStream_t stream;
    void* rec;
    LaunchScope(int kernel_id, cudaStream_t st);
    ~LaunchScope();
};

// Number of SMs of the current device (cached per device).
int sm_count();

// Function attributes (e.g. the dynamic shared-memory limit) are per device: a launch site asks whether
// its kernels (identified by `key`, one per launch site, < 32) are configured on the CURRENT device and
// marks them once cudaFuncSetAttribute has succeeded there. Guarded by the runtime's mutex.
bool device_configured(int key);
void device_mark_configured(int key);

}  // namespace of3
