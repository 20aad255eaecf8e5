// Device helpers shared by the "row tile" kernels: a tile is 128 rows (pair positions) of 128
// bf16 channels held in shared memory as a K-major, 128-byte-swizzled tcgen05 A operand made of
// two k-blocks [128 rows x 64 channels] (16 KB each) -- exactly what two TMA boxes {64, 128}
// with CU_TENSOR_MAP_SWIZZLE_128B deposit. One thread owns one row.
#pragma once
#include "umma.cuh"

namespace of3 {
namespace rowtile {

constexpr int kRows = 128;
constexpr int kC = 128;
constexpr int kKBlockBytes = kRows * 64 * 2;  // 16384
constexpr int kTileBytes = 2 * kKBlockBytes;  // 32768
constexpr float kLnEps = 1e-5f;

__device__ __forceinline__ float tanh_approx(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// sigmoid through one MUFU op (tanh.approx); absolute error ~5e-4, well inside bf16 rounding.
__device__ __forceinline__ float sigmoid_fast(float x) {
    return fmaf(0.5f, tanh_approx(0.5f * x), 0.5f);
}
// max of three (one instruction on sm_100)
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// (x0, x1) += (y0, y1) as one packed instruction (half the issue slots of two scalar adds)
__device__ __forceinline__ void add2(float& x0, float& x1, float y0, float y1) {
    unsigned long long a, b;
    asm("mov.b64 %0, {%1, %2};" : "=l"(a) : "f"(x0), "f"(x1));
    asm("mov.b64 %0, {%1, %2};" : "=l"(b) : "f"(y0), "f"(y1));
    asm("add.rn.f32x2 %0, %0, %1;" : "+l"(a) : "l"(b));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(x0), "=f"(x1) : "l"(a));
}

// Named barrier for a subset of the CTA's warps (id 1..15; nthreads multiple of 32).
__device__ __forceinline__ void group_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// Shared-memory address of 16-byte chunk `chunk` (0..15, 8 channels each) of row `row`.
__device__ __forceinline__ uint32_t chunk_addr(uint32_t tile, int row, int chunk) {
    return tile + (uint32_t)((chunk >> 3) * kKBlockBytes + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}
// Same for a tile with 64-byte rows (32 bf16) in the 64-byte swizzle: chunk 0..3, XORed with (row/2)%4.
__device__ __forceinline__ uint32_t chunk_addr64(uint32_t tile, int row, int chunk) {
    return tile + (uint32_t)(row * 64 + ((chunk ^ ((row >> 1) & 3)) << 4));
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z),
                 "r"(v.w)
                 : "memory");
}

// Reads this thread's row (128 bf16) of a swizzled tile into 64 packed registers.
__device__ __forceinline__ void load_row(uint32_t tile, int row, uint32_t (&raw)[64]) {
#pragma unroll
    for (int ch = 0; ch < 16; ++ch) {
        const uint4 v = lds128(chunk_addr(tile, row, ch));
        raw[ch * 4 + 0] = v.x;
        raw[ch * 4 + 1] = v.y;
        raw[ch * 4 + 2] = v.z;
        raw[ch * 4 + 3] = v.w;
    }
}

// LayerNorm statistics of 128 packed bf16 values (fp32, two-pass on registers). Eight independent partial sums (a
// single accumulator is a 128-deep dependent chain, which with two warps per scheduler is pure latency), associated
// exactly like the two-threads-per-row variant below -- four partial sums per half row, the halves added last -- so
// that kernels that split a row over two threads and kernels that do not produce the same bits.
__device__ __forceinline__ void row_stats(const uint32_t (&raw)[64], float& mean, float& rstd) {
    float s[8];
#pragma unroll
    for (int a = 0; a < 8; ++a) s[a] = 0.f;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
#pragma unroll
            for (int a = 0; a < 4; ++a) s[h * 4 + a] += bf16lo(raw[h * 32 + i + a]) + bf16hi(raw[h * 32 + i + a]);
        }
    }
    mean = (((s[0] + s[1]) + (s[2] + s[3])) + ((s[4] + s[5]) + (s[6] + s[7]))) * (1.0f / kC);
    float v[8];
#pragma unroll
    for (int a = 0; a < 8; ++a) v[a] = 0.f;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                const float x0 = bf16lo(raw[h * 32 + i + a]) - mean, x1 = bf16hi(raw[h * 32 + i + a]) - mean;
                v[h * 4 + a] = fmaf(x0, x0, v[h * 4 + a]);
                v[h * 4 + a] = fmaf(x1, x1, v[h * 4 + a]);
            }
        }
    }
    const float var = (((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]))) * (1.0f / kC);
    rstd = rsqrtf(var + kLnEps);
}

// Writes LN(raw) * gamma + beta (bf16) as this thread's row of a swizzled tile.
// gamma/beta: fp32 arrays of 128 in shared memory, 16-byte aligned (broadcast vector reads).
__device__ __forceinline__ void store_normalized_row(uint32_t tile, int row, const uint32_t (&raw)[64],
                                                     float mean, float rstd, const float* gamma,
                                                     const float* beta) {
    const float nm = -mean * rstd;
#pragma unroll
    for (int ch = 0; ch < 16; ++ch) {
        const float4 g0 = *reinterpret_cast<const float4*>(gamma + ch * 8);
        const float4 g1 = *reinterpret_cast<const float4*>(gamma + ch * 8 + 4);
        const float4 b0 = *reinterpret_cast<const float4*>(beta + ch * 8);
        const float4 b1 = *reinterpret_cast<const float4*>(beta + ch * 8 + 4);
        const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
        const float bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            // (x - mean) * rstd as one fma: x * rstd + (-mean * rstd)
            const float a = fmaf(fmaf(bf16lo(raw[ch * 4 + j]), rstd, nm), gg[j * 2], bb[j * 2]);
            const float b = fmaf(fmaf(bf16hi(raw[ch * 4 + j]), rstd, nm), gg[j * 2 + 1], bb[j * 2 + 1]);
            o[j] = pack_bf16x2(a, b);
        }
        sts128(chunk_addr(tile, row, ch), make_uint4(o[0], o[1], o[2], o[3]));
    }
}

// The same three steps with TWO threads per row: lanes 0..15 of a warp hold channels 0..63 of 16 rows, lanes
// 16..31 channels 64..127 of the same rows (half = lane >> 4); the statistics are joined by one shuffle.
__device__ __forceinline__ void load_half_row(uint32_t tile, int row, int half, uint32_t (&raw)[32]) {
#pragma unroll
    for (int ch = 0; ch < 8; ++ch) {
        const uint4 v = lds128(chunk_addr(tile, row, half * 8 + ch));
        raw[ch * 4 + 0] = v.x;
        raw[ch * 4 + 1] = v.y;
        raw[ch * 4 + 2] = v.z;
        raw[ch * 4 + 3] = v.w;
    }
}
// Sum, and sum of squared deviations, of this thread's 64 of a row's 128 values.
__device__ __forceinline__ float half_row_sum(const uint32_t (&raw)[32]) {
    float s[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
#pragma unroll
        for (int a = 0; a < 4; ++a) s[a] += bf16lo(raw[i + a]) + bf16hi(raw[i + a]);
    }
    return (s[0] + s[1]) + (s[2] + s[3]);
}
__device__ __forceinline__ float half_row_sqdev(const uint32_t (&raw)[32], float mean) {
    float v[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
#pragma unroll
        for (int a = 0; a < 4; ++a) {
            const float x0 = bf16lo(raw[i + a]) - mean, x1 = bf16hi(raw[i + a]) - mean;
            v[a] = fmaf(x0, x0, v[a]);
            v[a] = fmaf(x1, x1, v[a]);
        }
    }
    return (v[0] + v[1]) + (v[2] + v[3]);
}
// the two halves of a row sit 16 lanes apart in one warp
__device__ __forceinline__ void half_row_stats(const uint32_t (&raw)[32], float& mean, float& rstd) {
    float sum = half_row_sum(raw);
    sum += __shfl_xor_sync(0xffffffffu, sum, 16);
    mean = sum * (1.0f / kC);
    float var = half_row_sqdev(raw, mean);
    var += __shfl_xor_sync(0xffffffffu, var, 16);
    rstd = rsqrtf(var * (1.0f / kC) + kLnEps);
}
// the two halves of a row belong to the same lane of two warps of a group of `nthreads` threads: the partial
// results cross through xch (2 x 256 floats of shared memory) and two named barriers (id)
__device__ __forceinline__ void half_row_stats_xwarp(const uint32_t (&raw)[32], int row, int half, float* xch, int bar_id,
                                                     int nthreads, float& mean, float& rstd) {
    const float sum = half_row_sum(raw);
    xch[half * 128 + row] = sum;
    group_sync(bar_id, nthreads);
    mean = (sum + xch[(half ^ 1) * 128 + row]) * (1.0f / kC);
    const float var = half_row_sqdev(raw, mean);
    xch[256 + half * 128 + row] = var;
    group_sync(bar_id, nthreads);
    rstd = rsqrtf((var + xch[256 + (half ^ 1) * 128 + row]) * (1.0f / kC) + kLnEps);
}
__device__ __forceinline__ void store_normalized_half_row(uint32_t tile, int row, int half, const uint32_t (&raw)[32],
                                                          float mean, float rstd, const float* gamma,
                                                          const float* beta) {
    const float nm = -mean * rstd;
#pragma unroll
    for (int ch = 0; ch < 8; ++ch) {
        const int c0 = (half * 8 + ch) * 8;
        const float4 g0 = *reinterpret_cast<const float4*>(gamma + c0);
        const float4 g1 = *reinterpret_cast<const float4*>(gamma + c0 + 4);
        const float4 b0 = *reinterpret_cast<const float4*>(beta + c0);
        const float4 b1 = *reinterpret_cast<const float4*>(beta + c0 + 4);
        const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
        const float bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float a = fmaf(fmaf(bf16lo(raw[ch * 4 + j]), rstd, nm), gg[j * 2], bb[j * 2]);
            const float b = fmaf(fmaf(bf16hi(raw[ch * 4 + j]), rstd, nm), gg[j * 2 + 1], bb[j * 2 + 1]);
            o[j] = pack_bf16x2(a, b);
        }
        sts128(chunk_addr(tile, row, half * 8 + ch), make_uint4(o[0], o[1], o[2], o[3]));
    }
}

// 8 tcgen05.mma (K = 128 in steps of 16) of one row tile against a weight slab:
// D[128 x N] (+)= A[128 x 128] * W[N x 128]^T. `w_kb_stride` = bytes between the slab's k-blocks.
__device__ __forceinline__ void mma_k128(uint32_t d_tmem, uint32_t a_tile, uint32_t w_slab,
                                         uint32_t w_kb_stride, uint32_t idesc, bool accumulate) {
#pragma unroll
    for (int kb = 0; kb < 2; ++kb) {
        const uint64_t ad = umma::smem_desc_k_sw128(a_tile + kb * kKBlockBytes);
        const uint64_t bd = umma::smem_desc_k_sw128(w_slab + kb * w_kb_stride);
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4)
            umma::mma_bf16(d_tmem, ad + 2u * k4, bd + 2u * k4, idesc,
                           (accumulate || kb != 0 || k4 != 0) ? 1u : 0u);
    }
}

}  // namespace rowtile
}  // namespace of3
