// Pair-bias projection of the single track on the tensor pipe (bf16 z, c_z = 128, 16 heads):
//   bias[h][pos] = sum_c LayerNorm_z(z[pos])[c] * W[h][c]          (attention_pair_bias.py:154-163)
// One pass over z. Row tiles of 128 pair positions: TMA -> LayerNorm in place in the swizzled A operand
// (one thread per row) -> one 128 x 16 x 128 tcgen05 GEMM against the resident 4 KB weight -> fp32 rows
// written head-major. The LayerNorm pass is the long pole of every row-tile kernel here, so TWO sets of
// four LayerNorm warps work on alternate tiles over a four-deep ring of z tiles; the thread-per-row SIMT
// version (2048 FMAs and 512 shared-memory reads per row) took 188 us at N = 768.
#include "modules.cuh"
#include "rowtile.cuh"
#include "runtime.cuh"

namespace of3 {
namespace fast {
namespace {

using namespace umma;
using namespace rowtile;

constexpr int kKidPairBias = 9;
constexpr int kStages = 4;
constexpr int kHeads = 16;
constexpr int kPbThreads = 32 * (2 + 8 + 4);  // producer, MMA, 2 x 4 LayerNorm warps, 4 epilogue warps

struct PbSmem {
    static constexpr uint32_t kZ = 0;                              // 4 stages x 32 KB
    static constexpr uint32_t kW = kStages * kTileBytes;           // 2 k-blocks x [16 rows x 128 B]
    static constexpr uint32_t kGamma = kW + 4096;
    static constexpr uint32_t kBeta = kGamma + 512;
    static constexpr uint32_t kBars = kBeta + 512;
    static constexpr uint32_t kTotal = kBars + 256;
    static constexpr uint32_t kDyn = kTotal + 1024;
};

__global__ void __launch_bounds__(kPbThreads, 1)
pair_bias_tc_kernel(const __grid_constant__ CUtensorMap tmZ, const __grid_constant__ CUtensorMap tmW,
                    const __nv_bfloat16* __restrict__ ln_w, const __nv_bfloat16* __restrict__ ln_b,
                    float* __restrict__ dst, __nv_bfloat16* __restrict__ tiles, int n_tok, long long rows, long long nn,
                    int* status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gbase = smem_raw + (sbase - smem_u32(smem_raw));
    float* gamma = reinterpret_cast<float*>(gbase + PbSmem::kGamma);
    float* beta = reinterpret_cast<float*>(gbase + PbSmem::kBeta);
    const uint32_t bars = sbase + PbSmem::kBars;
    const uint32_t w_full = bars;
    auto z_full = [&](int s) { return bars + 8u * (1 + s); };
    auto z_empty = [&](int s) { return bars + 8u * (1 + kStages + s); };
    auto a_ready = [&](int s) { return bars + 8u * (1 + 2 * kStages + s); };
    auto slot_full = [&](int q) { return bars + 8u * (1 + 3 * kStages + q); };
    auto slot_empty = [&](int q) { return bars + 8u * (3 + 3 * kStages + q); };
    volatile uint32_t* tmem_ptr = reinterpret_cast<volatile uint32_t*>(gbase + PbSmem::kBars + 160);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + PbSmem::kBars + 168);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long num_tiles = (rows + kRows - 1) / kRows;

    if (threadIdx.x == 0) {
        mbar_init(w_full, 1);
        for (int s = 0; s < kStages; ++s) {
            mbar_init(z_full(s), 1);
            mbar_init(z_empty(s), 1);
            mbar_init(a_ready(s), 4);
        }
        for (int q = 0; q < 2; ++q) {
            mbar_init(slot_full(q), 1);
            mbar_init(slot_empty(q), 4);
        }
        *abort_flag = 0;
        mbar_fence_init();
        prefetch_tmap(&tmZ);
    }
    if (threadIdx.x < 128) {
        gamma[threadIdx.x] = ln_w ? __bfloat162float(ln_w[threadIdx.x]) : 1.0f;
        beta[threadIdx.x] = ln_b ? __bfloat162float(ln_b[threadIdx.x]) : 0.0f;
    }
    if (warp == 1) {
        tmem_alloc(smem_u32((const void*)tmem_ptr), 32);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_ptr;  // slot q = columns [16 q, 16 q + 16)

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            mbar_arrive_expect_tx(w_full, 4096);
            for (int kb = 0; kb < 2; ++kb) tma_load_2d(sbase + PbSmem::kW + kb * 2048, &tmW, w_full, kb * 64, 0);
            uint32_t it = 0;
            for (long long t = blockIdx.x; t < num_tiles; t += gridDim.x, ++it) {
                const int s = it % kStages;
                if (!mbar_wait(z_empty(s), ((it / kStages) & 1u) ^ 1u, abort_flag)) {
                    report_wait_failure(status, abort_flag, kKidPairBias, 1);
                    break;
                }
                mbar_arrive_expect_tx(z_full(s), kTileBytes);
                const uint32_t d = sbase + PbSmem::kZ + s * kTileBytes;
                for (int kb = 0; kb < 2; ++kb) tma_load_2d(d + kb * kKBlockBytes, &tmZ, z_full(s), kb * 64, (int)(t * kRows));
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = idesc_bf16_f32(128, kHeads);
            bool ok = mbar_wait(w_full, 0, abort_flag);
            if (!ok) report_wait_failure(status, abort_flag, kKidPairBias, 2);
            uint32_t it = 0;
            for (long long t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
                const int s = it % kStages, q = it & 1;
                if (!mbar_wait(a_ready(s), (it / kStages) & 1u, abort_flag)) {
                    report_wait_failure(status, abort_flag, kKidPairBias, 3);
                    break;
                }
                if (!mbar_wait(slot_empty(q), ((it >> 1) & 1u) ^ 1u, abort_flag)) {
                    report_wait_failure(status, abort_flag, kKidPairBias, 4);
                    break;
                }
                tc_fence_after_sync();
                mma_k128(tmem_base + q * kHeads, sbase + PbSmem::kZ + s * kTileBytes, sbase + PbSmem::kW, 2048, idesc,
                         false);
                mma_commit(slot_full(q));
                mma_commit(z_empty(s));
            }
        }
    } else if (warp < 10) {
        // ---------------------------------------------------------------- two LayerNorm sets, alternate tiles
        const int set = (warp - 2) >> 2;
        const int row = (warp & 3) * 32 + lane;  // any bijection warp -> 32 rows works here (no TMEM access)
        uint32_t it = 0;
        for (long long t = blockIdx.x; t < num_tiles; t += gridDim.x, ++it) {
            if ((int)(it & 1u) != set) continue;
            const int s = it % kStages;
            if (!mbar_wait(z_full(s), (it / kStages) & 1u, abort_flag)) {
                if (lane == 0) report_wait_failure(status, abort_flag, kKidPairBias, 5);
                break;
            }
            const uint32_t tile = sbase + PbSmem::kZ + s * kTileBytes;
            uint32_t raw[64];
            load_row(tile, row, raw);
            float mean, rstd;
            row_stats(raw, mean, rstd);
            store_normalized_row(tile, row, raw, mean, rstd, gamma, beta);
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(a_ready(s));
        }
    } else {
        // ---------------------------------------------------------------- epilogue warps (10..13)
        const int quad = warp & 3;
        const int row = quad * 32 + lane;
        uint32_t it = 0;
        for (long long t = blockIdx.x; t < num_tiles; t += gridDim.x, ++it) {
            const int q = it & 1;
            if (!mbar_wait(slot_full(q), (it >> 1) & 1u, abort_flag)) {
                if (lane == 0) report_wait_failure(status, abort_flag, kKidPairBias, 6);
                break;
            }
            tc_fence_after_sync();
            uint32_t r[16];
            tmem_ld16(tmem_base + ((uint32_t)(quad * 32) << 16) + q * kHeads, r);
            tmem_ld_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(slot_empty(q));
            const long long pos = t * kRows + row;
            if (pos < rows) {
                const long long b = pos / nn, qk = pos - b * nn;
                if (tiles != nullptr) {
                    // the attention kernel's bias image: bf16, times log2(e), [b*16 + h][key block of 32][query row][32
                    // keys], each 64-byte row in the 64-byte swizzle of a K-major A operand
                    const int i = (int)(qk / n_tok), j = (int)(qk - (long long)i * n_tok);
                    const long long nkb = (n_tok + 31) >> 5;
                    const long long hs = nkb * n_tok * 32;   // elements per (sample, head)
                    __nv_bfloat16* d = tiles + (b * kHeads) * hs + ((long long)(j >> 5) * n_tok + i) * 32 +
                                       (((((j & 31) >> 3) ^ ((i >> 1) & 3)) << 3) | (j & 7));
#pragma unroll
                    for (int h = 0; h < kHeads; ++h)
                        d[h * hs] = __float2bfloat16_rn(__uint_as_float(r[h]) * 1.4426950408889634f);
                } else {
                    float* d = dst + (b * kHeads) * nn + qk;
#pragma unroll
                    for (int h = 0; h < kHeads; ++h) d[h * nn] = __uint_as_float(r[h]);
                }
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 32);
    }
}

}  // namespace

namespace {
int pair_bias_launch(const __nv_bfloat16* z, const __nv_bfloat16* ln_w, const __nv_bfloat16* ln_b,
                     const __nv_bfloat16* w, float* dst, __nv_bfloat16* tiles, int n_tok, long long B, long long nn,
                     cudaStream_t st);
}

// dst[b][h][pos] (fp32) for B samples of nn pair positions each; z [B * nn][128] bf16.
int pair_bias_c128_h16(const __nv_bfloat16* z, const __nv_bfloat16* ln_w, const __nv_bfloat16* ln_b,
                       const __nv_bfloat16* w, float* dst, long long B, long long nn, cudaStream_t st) {
    return pair_bias_launch(z, ln_w, ln_b, w, dst, nullptr, 0, B, nn, st);
}

// The same projection written straight into the bias image of the single-track attention kernel (bf16 tiles
// [b*16 + h][key block of 32][N query rows][32], times log2(e)): no fp32 tensor in between. z [B][N][N][128].
int pair_bias_tiles_c128_h16(const __nv_bfloat16* z, const __nv_bfloat16* ln_w, const __nv_bfloat16* ln_b,
                             const __nv_bfloat16* w, __nv_bfloat16* tiles, long long B, int N, cudaStream_t st) {
    if (N % 32 != 0) {   // the key padding of the last block must read as zeros
        const size_t bytes = (size_t)B * kHeads * ((N + 31) / 32) * N * 32 * sizeof(__nv_bfloat16);
        OF3_CUDA_CHECK(cudaMemsetAsync(tiles, 0, bytes, st));
    }
    return pair_bias_launch(z, ln_w, ln_b, w, nullptr, tiles, N, B, (long long)N * N, st);
}

namespace {
int pair_bias_launch(const __nv_bfloat16* z, const __nv_bfloat16* ln_w, const __nv_bfloat16* ln_b,
                     const __nv_bfloat16* w, float* dst, __nv_bfloat16* tiles, int n_tok, long long B, long long nn,
                     cudaStream_t st) {
    const long long rows = B * nn;
    if (rows <= 0) return OF3_OK;
    OF3_REQUIRE(((uintptr_t)z & 15) == 0 && ((uintptr_t)w & 15) == 0, OF3_ERR_ALIGN,
                "pair_bias: z and the weight must be 16-byte aligned");
    OF3_REQUIRE(rows < (1LL << 31) - 256, OF3_ERR_SHAPE, "pair_bias: too many pair positions");
    int rc;
    CUtensorMap tmZ, tmW;
    {
        uint64_t dims[2] = {128, (uint64_t)rows};
        uint64_t str[1] = {256};
        uint32_t box[2] = {64, 128};
        if ((rc = make_tmap_bf16(&tmZ, z, 2, dims, str, box, 1))) return rc;
    }
    {
        uint64_t dims[2] = {128, (uint64_t)kHeads};
        uint64_t str[1] = {256};
        uint32_t box[2] = {64, (uint32_t)kHeads};
        if ((rc = make_tmap_bf16(&tmW, w, 2, dims, str, box, 1))) return rc;
    }
    if (!device_configured(3)) {
        OF3_CUDA_CHECK(cudaFuncSetAttribute(pair_bias_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            PbSmem::kDyn));
        device_mark_configured(3);
    }
    const long long num_tiles = (rows + kRows - 1) / kRows;
    const int grid = (int)(num_tiles < sm_count() ? num_tiles : sm_count());
    LaunchScope scope(kKidPairBias, st);
    pair_bias_tc_kernel<<<grid, kPbThreads, PbSmem::kDyn, st>>>(tmZ, tmW, ln_w, ln_b, dst, tiles, n_tok, rows, nn,
                                                                device_status_ptr());
    OF3_CUDA_CHECK(cudaGetLastError());
    return OF3_OK;
}
}  // namespace

}  // namespace fast
}  // namespace of3
