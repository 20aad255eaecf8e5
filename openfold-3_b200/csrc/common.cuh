// Shared host/device helpers for the Pairformer hot-path library.
//
// Error convention of every extern "C" entry point: 0 = ok, negative = bad
// argument / unsupported shape (OF3_ERR_*), positive = a cudaError_t value.
// Nothing here throws or aborts.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stddef.h>

#include "of3b200.h"

namespace of3 {

// Records the first error message of this thread; read by of3_last_error_string().
void set_error(const char* fmt, ...);

// Device status block: written by kernels whose bounded waits run out.
// word 0: non-zero error code, word 1: kernel id, word 2: blockIdx.x, word 3: site id.
int* device_status_ptr();  // lazily allocated once per device (not on the hot path after the first call)

#define OF3_CUDA_CHECK(expr)                                                       \
    do {                                                                           \
        cudaError_t _e = (expr);                                                   \
        if (_e != cudaSuccess) {                                                   \
            of3::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), \
                           __FILE__, __LINE__);                                    \
            return (int)_e;                                                        \
        }                                                                          \
    } while (0)

#define OF3_REQUIRE(cond, code, ...)      \
    do {                                  \
        if (!(cond)) {                    \
            of3::set_error(__VA_ARGS__);  \
            return (code);                \
        }                                 \
    } while (0)

static inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Bump allocator over a caller-owned workspace.
struct Arena {
    char* base;
    size_t cap;
    size_t off;
    Arena(void* p, size_t n) : base((char*)p), cap(n), off(0) {}
    void* take(size_t bytes) {
        size_t o = align_up(off, 256);
        off = o + bytes;
        return base ? (void*)(base + o) : nullptr;
    }
    bool ok() const { return off <= cap; }
};

}  // namespace of3

#ifdef __CUDACC__
namespace of3 {

__device__ __forceinline__ float sigmoidf_fast(float x) { return 1.0f / (1.0f + __expf(-x)); }

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float bf16lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

template <typename T>
__device__ __forceinline__ float ld_as_float(const T* p);
template <>
__device__ __forceinline__ float ld_as_float<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float ld_as_float<__nv_bfloat16>(const __nv_bfloat16* p) {
    return __bfloat162float(*p);
}
template <typename T>
__device__ __forceinline__ void st_from_float(T* p, float v);
template <>
__device__ __forceinline__ void st_from_float<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void st_from_float<__nv_bfloat16>(__nv_bfloat16* p, float v) {
    *p = __float2bfloat16_rn(v);
}

}  // namespace of3
#endif
