// Triangle multiplicative update, bf16 / tcgen05 family (c_z = c_hidden = 128).
//
// Three kernels per layer, all fed by TMA:
//   trimul_in   z tile -> LayerNorm_in (in place) -> the four projections a_p, a_g, b_p, b_g TRANSPOSED
//               (tcgen05: the weights are the A operand, the normalised tile the B operand, so a TMEM lane is an
//               output channel and its columns are the tile's 128 positions) -> mask * sigmoid(gate) * proj ->
//               a, b stored CHANNEL-MAJOR with the contracted index innermost, a_t[c][i][k], b_t[c][j][k]:
//               every epilogue thread writes its channel's 256 contiguous bytes with 16-byte stores.
//               For the incoming update the tile walks z along its first index instead, so that
//               both directions feed the same K-major x K-major contraction.
//   contract    x_t[c][i][j] = sum_k a_t[c][i][k] * b_t[c][j][k]      (contract.cu)
//   trimul_out  x tile (all channels of 128 positions) -> LayerNorm_out -> linear_z, and in the
//               same pass z tile -> LayerNorm_in -> linear_g (recomputing the gate is one more
//               128^3 MMA and saves writing and re-reading an N^2 x 128 gate tensor);
//               out = z + sigmoid(gate) * update, TMA-stored.
// Reference: openfold3/core/model/layers/triangular_multiplicative_update.py:421-503.
#include "modules.cuh"
#include "rowtile.cuh"
#include "runtime.cuh"

namespace of3 {
namespace fast {
namespace {

using namespace umma;
using namespace rowtile;

constexpr int kKidIn = 2;
constexpr int kKidOut = 3;

struct TileCoord {
    int b, fixed, t0;  // sample, fixed index (i), first row of the tile along the walking index
};
// R = lines per sample (R == N for a whole pair tensor, N / P for a row shard)
__device__ __forceinline__ TileCoord tile_coord(long long t, int R, int tiles_per_line) {
    TileCoord c;
    c.t0 = (int)(t % tiles_per_line) * kRows;
    const long long line = t / tiles_per_line;
    c.fixed = (int)(line % R);
    c.b = (int)(line / R);
    return c;
}

// =====================================================================================
// trimul_in
// =====================================================================================
struct InSmem {
    static constexpr uint32_t kW = 0;                          // 2 k-blocks x [512 rows x 128 B]
    static constexpr uint32_t kWKb = 512 * 128;                // 65536
    static constexpr uint32_t kZ = 2 * kWKb;                   // 2 stages x 32768
    static constexpr uint32_t kGamma = kZ + 2 * kTileBytes;    // 128 floats
    static constexpr uint32_t kBeta = kGamma + 512;
    static constexpr uint32_t kMask = kBeta + 512;             // 4 x 128 floats: 0.5 * mask of the tile's positions
    static constexpr uint32_t kBars = kMask + 4 * 512;
    static constexpr uint32_t kTotal = kBars + 128;
    static constexpr uint32_t kDyn = kTotal + 1024;
};

// outgoing: tmZ is 3-D {c, second index, b*N + first index}; incoming: 4-D {c, second, first, b}
constexpr int kInLnWarps = 8;    // two threads per position
constexpr int kInEpiSets = 2;    // epilogue warp sets: a / b projection x first / second half of the tile's positions
constexpr int kInThreads = 32 * (2 + kInLnWarps + 4 * kInEpiSets);  // producer, MMA, LayerNorm and epilogue warps

template <bool kOutgoing>
__global__ void __launch_bounds__(kInThreads, 1)
trimul_in_kernel(const __grid_constant__ CUtensorMap tmZ, const __grid_constant__ CUtensorMap tmWap,
                 const __grid_constant__ CUtensorMap tmWag, const __grid_constant__ CUtensorMap tmWbp,
                 const __grid_constant__ CUtensorMap tmWbg, const __nv_bfloat16* __restrict__ mask,
                 const __nv_bfloat16* __restrict__ ln_w, const __nv_bfloat16* __restrict__ ln_b,
                 __nv_bfloat16* __restrict__ a_t, __nv_bfloat16* __restrict__ b_t, int B, int R,
                 int N, int ld, int group_shift, long long group_stride, int wide_stores, int* status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gbase = smem_raw + (sbase - smem_u32(smem_raw));
    float* gamma = reinterpret_cast<float*>(gbase + InSmem::kGamma);
    float* beta = reinterpret_cast<float*>(gbase + InSmem::kBeta);
    float* mask05 = reinterpret_cast<float*>(gbase + InSmem::kMask);
    const uint32_t bars = sbase + InSmem::kBars;
    const uint32_t w_full = bars;
    auto z_full = [&](int s) { return bars + 8u * (1 + s); };
    auto z_empty = [&](int s) { return bars + 8u * (3 + s); };
    auto a_ready = [&](int s) { return bars + 8u * (5 + s); };
    auto slot_full = [&](int q) { return bars + 8u * (7 + q); };
    auto slot_empty = [&](int q) { return bars + 8u * (9 + q); };
    volatile uint32_t* tmem_ptr = reinterpret_cast<volatile uint32_t*>(gbase + InSmem::kBars + 96);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + InSmem::kBars + 104);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_per_line = (N + kRows - 1) / kRows;
    const long long num_tiles = (long long)B * R * tiles_per_line;

    if (threadIdx.x == 0) {
        mbar_init(w_full, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(z_full(s), 1);
            mbar_init(z_empty(s), 1);
            mbar_init(a_ready(s), kInLnWarps);
            mbar_init(slot_full(s), 1);
            mbar_init(slot_empty(s), 2 * kInEpiSets);
        }
        *abort_flag = 0;
        mbar_fence_init();
        prefetch_tmap(&tmZ);
    }
    if (threadIdx.x < 128) {
        gamma[threadIdx.x] = __bfloat162float(ln_w[threadIdx.x]);
        beta[threadIdx.x] = __bfloat162float(ln_b[threadIdx.x]);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32((const void*)tmem_ptr), 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_ptr;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            mbar_arrive_expect_tx(w_full, 2 * InSmem::kWKb);
            const CUtensorMap* wm[4] = {&tmWap, &tmWag, &tmWbp, &tmWbg};
            for (int w = 0; w < 4; ++w)
                for (int kb = 0; kb < 2; ++kb)
                    tma_load_2d(sbase + InSmem::kW + kb * InSmem::kWKb + w * 128 * 128, wm[w], w_full,
                                kb * 64, 0);
            uint32_t it = 0;
            for (long long t = blockIdx.x; t < num_tiles; t += gridDim.x, ++it) {
                const int s = it & 1;
                if (!mbar_wait(z_empty(s), ((it >> 1) & 1u) ^ 1u, abort_flag)) {
                    report_wait_failure(status, abort_flag, kKidIn, 1);
                    break;
                }
                const TileCoord tc = tile_coord(t, R, tiles_per_line);
                mbar_arrive_expect_tx(z_full(s), kTileBytes);
                const uint32_t dst = sbase + InSmem::kZ + s * kTileBytes;
                for (int kb = 0; kb < 2; ++kb) {
                    if (kOutgoing)
                        tma_load_3d(dst + kb * kKBlockBytes, &tmZ, z_full(s), kb * 64, tc.t0,
                                    tc.b * R + tc.fixed);
                    else
                        tma_load_4d(dst + kb * kKBlockBytes, &tmZ, z_full(s), kb * 64, tc.fixed, tc.t0,
                                    tc.b);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = idesc_bf16_f32(128, 128);
            bool ok = mbar_wait(w_full, 0, abort_flag);
            if (!ok) report_wait_failure(status, abort_flag, kKidIn, 2);
            uint32_t it = 0;
            for (long long t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
                const int s = it & 1;
                if (!mbar_wait(a_ready(s), (it >> 1) & 1u, abort_flag)) {
                    report_wait_failure(status, abort_flag, kKidIn, 3);
                    break;
                }
                const uint32_t ztile = sbase + InSmem::kZ + s * kTileBytes;
                for (int q = 0; q < 2; ++q) {
                    if (!mbar_wait(slot_empty(q), (it & 1u) ^ 1u, abort_flag)) {
                        report_wait_failure(status, abort_flag, kKidIn, 4);
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    // D[channel][position] = W[channel][:] . LN(z)[position][:]: projection, then gate
                    for (int hg = 0; hg < 2; ++hg) {
                        const uint32_t w_tile = sbase + InSmem::kW + (q * 2 + hg) * 128 * 128;
#pragma unroll
                        for (int kb = 0; kb < 2; ++kb) {
                            const uint64_t ad = smem_desc_k_sw128(w_tile + kb * InSmem::kWKb);
                            const uint64_t bd = smem_desc_k_sw128(ztile + kb * kKBlockBytes);
#pragma unroll
                            for (int k4 = 0; k4 < 4; ++k4)
                                mma_bf16(tmem_base + q * 256 + hg * 128, ad + 2u * k4, bd + 2u * k4, idesc,
                                         (kb != 0 || k4 != 0) ? 1u : 0u);
                        }
                    }
                    mma_commit(slot_full(q));
                }
                if (ok) mma_commit(z_empty(s));
            }
        }
    } else if (warp < 2 + kInLnWarps) {
        // ---------------------------------------------------------------- LayerNorm warps: a warp takes 16 positions,
        // lanes 0..15 their first 64 channels, lanes 16..31 the other 64 (statistics joined by one shuffle)
        const int row = (warp - 2) * 16 + (lane & 15);
        const int half = lane >> 4;
        uint32_t it = 0;
        for (long long t = blockIdx.x; t < num_tiles; t += gridDim.x, ++it) {
            const int s = it & 1;
            if (!mbar_wait(z_full(s), (it >> 1) & 1u, abort_flag)) {
                if (lane == 0) report_wait_failure(status, abort_flag, kKidIn, 5);
                break;
            }
            const uint32_t tile = sbase + InSmem::kZ + s * kTileBytes;
            uint32_t raw[32];
            load_half_row(tile, row, half, raw);
            float mean, rstd;
            half_row_stats(raw, mean, rstd);
            store_normalized_half_row(tile, row, half, raw, mean, rstd, gamma, beta);
            const TileCoord tc = tile_coord(t, R, tiles_per_line);
            const int k = tc.t0 + row;
            float m = 0.f;   // positions past the end of the line are never stored
            if (k < N) {
                m = 0.5f;
                if (mask != nullptr) {
                    const long long lin = kOutgoing ? ((long long)(tc.b * R + tc.fixed) * N + k)
                                                    : ((long long)(tc.b * N + k) * R + tc.fixed);
                    m = 0.5f * __bfloat162float(mask[lin]);
                }
            }
            // four mask buffers: the epilogue of tile `it` may still read its buffer while tile it + 2 is normalised;
            // tile it + 4 cannot get here before that epilogue has released its TMEM slot
            if (half == 0) mask05[(it & 3) * 128 + row] = m;
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(a_ready(s));
        }
    } else {
        // ---------------------------------------------------------------- epilogue warps: the first four take the a
        // projection (TMEM slot 0), the other four the b projection (slot 1); thread = output channel, columns =
        // positions
        const int set = (warp - 2 - kInLnWarps) >> 2;
        const int q = set / (kInEpiSets / 2), khalf = set % (kInEpiSets / 2);
        constexpr int kSpan = kRows / (kInEpiSets / 2);   // positions per set
        const int quad = warp & 3;
        const int c = quad * 32 + lane;
        const long long cs = (long long)R * ld;
        // channel c lives at (c >> group_shift) * group_stride + (c & group_mask) * R * ld: one contiguous plane
        // [128][R][ld] by default, or one group of channels per destination rank when the planes are about to be
        // exchanged
        __nv_bfloat16* plane = (q == 0 ? a_t : b_t) + (long long)(c >> group_shift) * group_stride +
                               (long long)(c & ((1 << group_shift) - 1)) * cs;
        const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + q * 256;
        uint32_t it = 0;
        for (long long t = blockIdx.x; t < num_tiles; t += gridDim.x, ++it) {
            const TileCoord tc = tile_coord(t, R, tiles_per_line);
            const int kmax = (N - tc.t0 < kRows) ? N - tc.t0 : kRows;   // positions of the tile that exist
            if (!mbar_wait(slot_full(q), it & 1u, abort_flag)) {
                if (lane == 0) report_wait_failure(status, abort_flag, kKidIn, 6);
                break;
            }
            tc_fence_after_sync();
            const float* mk = mask05 + (it & 3) * 128;
            // the line pitch ld is a multiple of 8 elements, so a 16-byte store that starts below N ends inside the
            // row; with a pitch that is a multiple of 16 (and 32-byte aligned planes) the same holds for 32 bytes
            __nv_bfloat16* dst = plane + (long long)tc.b * ((kC >> group_shift) * group_stride) +
                                 (long long)tc.fixed * ld + tc.t0;
            // 16 positions per pass; the TMEM load of the next pass is in flight while this one is computed
            auto emit = [&](const uint32_t (&p)[16], const uint32_t (&g)[16], int k0) {
                uint32_t o[8];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const float4 m0 = *reinterpret_cast<const float4*>(mk + k0 + j * 8);
                    const float4 m1 = *reinterpret_cast<const float4*>(mk + k0 + j * 8 + 4);
                    const float mm[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
                    float v[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        // mask * p * sigmoid(g) = pm * tanh(g / 2) + pm with pm = (mask / 2) * p
                        const float pm = mm[e] * __uint_as_float(p[j * 8 + e]);
                        v[e] = fmaf(tanh_approx(0.5f * __uint_as_float(g[j * 8 + e])), pm, pm);
                    }
#pragma unroll
                    for (int e = 0; e < 4; ++e) o[j * 4 + e] = pack_bf16x2(v[2 * e], v[2 * e + 1]);
                }
                if (wide_stores) {   // one full 32-byte sector per thread
                    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst + k0), "r"(o[0]),
                                 "r"(o[1]), "r"(o[2]), "r"(o[3]), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7])
                                 : "memory");
                } else {
                    *reinterpret_cast<uint4*>(dst + k0) = make_uint4(o[0], o[1], o[2], o[3]);
                    if (k0 + 8 < kmax) *reinterpret_cast<uint4*>(dst + k0 + 8) = make_uint4(o[4], o[5], o[6], o[7]);
                }
            };
            const int k_begin = khalf * kSpan;
            const int k_end = (kmax < (khalf + 1) * kSpan) ? kmax : (khalf + 1) * kSpan;
            uint32_t pa[16], ga[16], pb[16], gb[16];
            if (k_begin < k_end) {
                tmem_ld16(taddr + k_begin, pa);
                tmem_ld16(taddr + 128 + k_begin, ga);
            }
#pragma unroll 1
            for (int k0 = k_begin; k0 < k_end; k0 += 32) {
                tmem_ld_wait();
                if (k0 + 16 < k_end) {
                    tmem_ld16(taddr + k0 + 16, pb);
                    tmem_ld16(taddr + 128 + k0 + 16, gb);
                }
                emit(pa, ga, k0);
                if (k0 + 16 < k_end) {
                    tmem_ld_wait();
                    if (k0 + 32 < k_end) {
                        tmem_ld16(taddr + k0 + 32, pa);
                        tmem_ld16(taddr + 128 + k0 + 32, ga);
                    }
                    emit(pb, gb, k0 + 16);
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(slot_empty(q));
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 512);
    }
}

// The same layer with the projections the other way round (the normalised tile is the A operand, a TMEM lane is a
// position, its columns the output channels; N = 256 per MMA): a warp's store covers 32 consecutive positions of ONE
// channel plane. Slower than the kernel above while a channel plane stays within a 2 MB page or so (170 against
// 151 us at N = 768: one 2-byte store per value), faster beyond (1.13 against 2.02 ms at N = 2048, where the 32
// planes one store of the kernel above touches lie megabytes apart).
constexpr int kInRowsThreads = 448;  // producer, MMA, 4 LayerNorm warps, 2 x 4 epilogue warps

template <bool kOutgoing>
__global__ void __launch_bounds__(kInRowsThreads, 1)
trimul_in_rows_kernel(const __grid_constant__ CUtensorMap tmZ, const __grid_constant__ CUtensorMap tmWap,
                 const __grid_constant__ CUtensorMap tmWag, const __grid_constant__ CUtensorMap tmWbp,
                 const __grid_constant__ CUtensorMap tmWbg, const __nv_bfloat16* __restrict__ mask,
                 const __nv_bfloat16* __restrict__ ln_w, const __nv_bfloat16* __restrict__ ln_b,
                 __nv_bfloat16* __restrict__ a_t, __nv_bfloat16* __restrict__ b_t, int B, int R,
                 int N, int ld, int group_shift, long long group_stride, int* status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gbase = smem_raw + (sbase - smem_u32(smem_raw));
    float* gamma = reinterpret_cast<float*>(gbase + InSmem::kGamma);
    float* beta = reinterpret_cast<float*>(gbase + InSmem::kBeta);
    const uint32_t bars = sbase + InSmem::kBars;
    const uint32_t w_full = bars;
    auto z_full = [&](int s) { return bars + 8u * (1 + s); };
    auto z_empty = [&](int s) { return bars + 8u * (3 + s); };
    auto a_ready = [&](int s) { return bars + 8u * (5 + s); };
    auto slot_full = [&](int q) { return bars + 8u * (7 + q); };
    auto slot_empty = [&](int q) { return bars + 8u * (9 + q); };
    volatile uint32_t* tmem_ptr = reinterpret_cast<volatile uint32_t*>(gbase + InSmem::kBars + 96);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + InSmem::kBars + 104);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_per_line = (N + kRows - 1) / kRows;
    const long long num_tiles = (long long)B * R * tiles_per_line;

    if (threadIdx.x == 0) {
        mbar_init(w_full, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(z_full(s), 1);
            mbar_init(z_empty(s), 1);
            mbar_init(a_ready(s), 4);
            mbar_init(slot_full(s), 1);
            mbar_init(slot_empty(s), 4);
        }
        *abort_flag = 0;
        mbar_fence_init();
        prefetch_tmap(&tmZ);
    }
    if (threadIdx.x < 128) {
        gamma[threadIdx.x] = __bfloat162float(ln_w[threadIdx.x]);
        beta[threadIdx.x] = __bfloat162float(ln_b[threadIdx.x]);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32((const void*)tmem_ptr), 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_ptr;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            mbar_arrive_expect_tx(w_full, 2 * InSmem::kWKb);
            const CUtensorMap* wm[4] = {&tmWap, &tmWag, &tmWbp, &tmWbg};
            for (int w = 0; w < 4; ++w)
                for (int kb = 0; kb < 2; ++kb)
                    tma_load_2d(sbase + InSmem::kW + kb * InSmem::kWKb + w * 128 * 128, wm[w], w_full,
                                kb * 64, 0);
            uint32_t it = 0;
            for (long long t = blockIdx.x; t < num_tiles; t += gridDim.x, ++it) {
                const int s = it & 1;
                if (!mbar_wait(z_empty(s), ((it >> 1) & 1u) ^ 1u, abort_flag)) {
                    report_wait_failure(status, abort_flag, kKidIn, 1);
                    break;
                }
                const TileCoord tc = tile_coord(t, R, tiles_per_line);
                mbar_arrive_expect_tx(z_full(s), kTileBytes);
                const uint32_t dst = sbase + InSmem::kZ + s * kTileBytes;
                for (int kb = 0; kb < 2; ++kb) {
                    if (kOutgoing)
                        tma_load_3d(dst + kb * kKBlockBytes, &tmZ, z_full(s), kb * 64, tc.t0,
                                    tc.b * R + tc.fixed);
                    else
                        tma_load_4d(dst + kb * kKBlockBytes, &tmZ, z_full(s), kb * 64, tc.fixed, tc.t0,
                                    tc.b);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = idesc_bf16_f32(128, 256);
            bool ok = mbar_wait(w_full, 0, abort_flag);
            if (!ok) report_wait_failure(status, abort_flag, kKidIn, 2);
            uint32_t it = 0;
            for (long long t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
                const int s = it & 1;
                if (!mbar_wait(a_ready(s), (it >> 1) & 1u, abort_flag)) {
                    report_wait_failure(status, abort_flag, kKidIn, 3);
                    break;
                }
                for (int q = 0; q < 2; ++q) {
                    if (!mbar_wait(slot_empty(q), (it & 1u) ^ 1u, abort_flag)) {
                        report_wait_failure(status, abort_flag, kKidIn, 4);
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    mma_k128(tmem_base + q * 256, sbase + InSmem::kZ + s * kTileBytes,
                             sbase + InSmem::kW + q * 256 * 128, InSmem::kWKb, idesc, false);
                    mma_commit(slot_full(q));
                }
                if (ok) mma_commit(z_empty(s));
            }
        }
    } else if (warp < 6) {
        // ---------------------------------------------------------------- LayerNorm warps (2..5)
        const int row = (warp - 2) * 32 + lane;
        uint32_t it = 0;
        for (long long t = blockIdx.x; t < num_tiles; t += gridDim.x, ++it) {
            const int s = it & 1;
            if (!mbar_wait(z_full(s), (it >> 1) & 1u, abort_flag)) {
                if (lane == 0) report_wait_failure(status, abort_flag, kKidIn, 5);
                break;
            }
            const uint32_t tile = sbase + InSmem::kZ + s * kTileBytes;
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
        // ---------------------------------------------------------------- epilogue warps: 6..9 take the a
        // projection (TMEM slot 0), 10..13 the b projection (slot 1). One set of four warps doing both
        // (2 x 128 sigmoid / multiply / convert / store per row and tile on one thread) was the longest
        // chain of the kernel.
        const int qset = (warp - 6) >> 2;
        const int quad = warp & 3;
        const int row = quad * 32 + lane;
        uint32_t it = 0;
        bool ok = true;
        for (long long t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
            const TileCoord tc = tile_coord(t, R, tiles_per_line);
            const int k = tc.t0 + row;
            const bool valid = k < N;
            float m = 1.0f;
            if (valid && mask != nullptr) {
                const long long lin = kOutgoing ? ((long long)(tc.b * R + tc.fixed) * N + k)
                                                : ((long long)(tc.b * N + k) * R + tc.fixed);
                m = __bfloat162float(mask[lin]);
            }
            const float mh = 0.5f * m;
            for (int q = qset; q <= qset; ++q) {
                if (!mbar_wait(slot_full(q), it & 1u, abort_flag)) {
                    if (lane == 0) report_wait_failure(status, abort_flag, kKidIn, 6);
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                // channel c lives at (c >> group_shift) * group_stride + (c & group_mask) * R * ld: one
                // contiguous plane [128][R][ld] by default, or one group of channels per destination
                // rank when the planes are about to be exchanged
                const long long cs = (long long)R * ld;
                __nv_bfloat16* dst = (q == 0 ? a_t : b_t) +
                                     (long long)tc.b * ((kC >> group_shift) * group_stride) +
                                     (long long)tc.fixed * ld + k;
                const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + q * 256;
#pragma unroll 1
                for (int cb = 0; cb < 4; ++cb) {
                    uint32_t p[32], g[32];
                    tmem_ld32(taddr + cb * 32, p);
                    tmem_ld32(taddr + 128 + cb * 32, g);
                    tmem_ld_wait();
                    if (valid) {
#pragma unroll
                        for (int hf = 0; hf < 2; ++hf) {  // groups hold >= 16 channels: no boundary inside a half
                            const int c0 = cb * 32 + hf * 16;
                            __nv_bfloat16* d0 = dst + (long long)(c0 >> group_shift) * group_stride +
                                                (long long)(c0 & ((1 << group_shift) - 1)) * cs;
#pragma unroll
                            for (int e = 0; e < 16; ++e) {
                                // the same expression as the kernel above, so that both give the same bits:
                                // mask * p * sigmoid(g) = pm * tanh(g / 2) + pm with pm = (mask / 2) * p
                                const float pm = mh * __uint_as_float(p[hf * 16 + e]);
                                const float v = fmaf(tanh_approx(0.5f * __uint_as_float(g[hf * 16 + e])), pm, pm);
                                d0[(long long)e * cs] = __float2bfloat16_rn(v);
                            }
                        }
                    }
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(slot_empty(q));
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 512);
    }
}

// =====================================================================================
// trimul_out
// =====================================================================================
struct OutSmem {
    static constexpr uint32_t kWg = 0;                        // [128 x 128] as 2 k-blocks of 16 KB
    static constexpr uint32_t kWz = kTileBytes;
    static constexpr uint32_t kZ = 2 * kTileBytes;            // 2 groups x 32768 (z tile, then output)
    static constexpr uint32_t kX = kZ + 2 * kTileBytes;       // 2 groups x 32768 (x tile [c][j], then A)
    static constexpr uint32_t kParams = kX + 2 * kTileBytes;  // gamma_in, beta_in, gamma_out, beta_out
    static constexpr uint32_t kBars = kParams + 4 * 512;
    static constexpr uint32_t kTotal = kBars + 128;
    static constexpr uint32_t kDyn = kTotal + 1024;
};

__global__ void __launch_bounds__(320, 1)
trimul_out_kernel(const __grid_constant__ CUtensorMap tmZ, const __grid_constant__ CUtensorMap tmX,
                  const __grid_constant__ CUtensorMap tmOut, const __grid_constant__ CUtensorMap tmWg,
                  const __grid_constant__ CUtensorMap tmWz, const __nv_bfloat16* __restrict__ ln_in_w,
                  const __nv_bfloat16* __restrict__ ln_in_b, const __nv_bfloat16* __restrict__ ln_out_w,
                  const __nv_bfloat16* __restrict__ ln_out_b, int B, int R, int N, int add_residual,
                  int* status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gbase = smem_raw + (sbase - smem_u32(smem_raw));
    float* prm = reinterpret_cast<float*>(gbase + OutSmem::kParams);
    const uint32_t bars = sbase + OutSmem::kBars;
    const uint32_t w_full = bars;
    // The x buffer is free as soon as the group's GEMMs have read it (the result goes over the z buffer), so
    // the next x tile is fetched during the epilogue; the z buffer is free once the output store has read it,
    // and its next tile lands while the group gathers and normalises x. Fetched together after the store,
    // the two loads cost every tile 2200 cycles of waiting.
    auto x_full = [&](int g) { return bars + 8u * (1 + g); };   // TMA landed: x tile
    auto z_empty = [&](int g) { return bars + 8u * (3 + g); };  // output store has read the z buffer
    auto a_ready = [&](int g) { return bars + 8u * (5 + g); };  // both A operands written
    auto d_full = [&](int g) { return bars + 8u * (7 + g); };   // MMAs of the group's tile done
    auto z_full = [&](int g) { return bars + 8u * (9 + g); };   // TMA landed: z tile
    auto x_empty = [&](int g) { return bars + 8u * (11 + g); };  // MMAs have read the x buffer
    volatile uint32_t* tmem_ptr = reinterpret_cast<volatile uint32_t*>(gbase + OutSmem::kBars + 112);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + OutSmem::kBars + 116);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_per_line = (N + kRows - 1) / kRows;
    const long long num_tiles = (long long)B * R * tiles_per_line;
    // tiles of this CTA alternate between the two groups: local tile index lt -> group lt & 1
    const long long my_tiles = (num_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x;

    if (threadIdx.x == 0) {
        mbar_init(w_full, 1);
        for (int g = 0; g < 2; ++g) {
            mbar_init(x_full(g), 1);
            mbar_init(z_full(g), 1);
            mbar_init(x_empty(g), 1);
            mbar_init(z_empty(g), 1);
            mbar_init(a_ready(g), 4);
            mbar_init(d_full(g), 1);
        }
        *abort_flag = 0;
        mbar_fence_init();
        prefetch_tmap(&tmZ);
        prefetch_tmap(&tmX);
        prefetch_tmap(&tmOut);
    }
    if (threadIdx.x < 128) {
        prm[threadIdx.x] = __bfloat162float(ln_in_w[threadIdx.x]);
        prm[128 + threadIdx.x] = __bfloat162float(ln_in_b[threadIdx.x]);
        prm[256 + threadIdx.x] = __bfloat162float(ln_out_w[threadIdx.x]);
        prm[384 + threadIdx.x] = __bfloat162float(ln_out_b[threadIdx.x]);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32((const void*)tmem_ptr), 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_ptr;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            mbar_arrive_expect_tx(w_full, 2 * kTileBytes);
            for (int kb = 0; kb < 2; ++kb) {
                tma_load_2d(sbase + OutSmem::kWg + kb * kKBlockBytes, &tmWg, w_full, kb * 64, 0);
                tma_load_2d(sbase + OutSmem::kWz + kb * kKBlockBytes, &tmWz, w_full, kb * 64, 0);
            }
            for (long long lt = 0; lt < my_tiles; ++lt) {
                const int g = (int)(lt & 1);
                const uint32_t use = (uint32_t)(lt >> 1);
                const TileCoord tc = tile_coord(blockIdx.x + lt * gridDim.x, R, tiles_per_line);
                if (!mbar_wait(x_empty(g), (use & 1u) ^ 1u, abort_flag)) {
                    report_wait_failure(status, abort_flag, kKidOut, 1);
                    break;
                }
                // x tile: all 128 channels of positions (fixed, t0 .. t0+127), layout [c][j]
                mbar_arrive_expect_tx(x_full(g), kTileBytes);
                tma_load_3d(sbase + OutSmem::kX + g * kTileBytes, &tmX, x_full(g), tc.t0, tc.fixed, tc.b * kC);
                if (!mbar_wait(z_empty(g), (use & 1u) ^ 1u, abort_flag)) {
                    report_wait_failure(status, abort_flag, kKidOut, 6);
                    break;
                }
                mbar_arrive_expect_tx(z_full(g), kTileBytes);
                const uint32_t zdst = sbase + OutSmem::kZ + g * kTileBytes;
                for (int kb = 0; kb < 2; ++kb)
                    tma_load_3d(zdst + kb * kKBlockBytes, &tmZ, z_full(g), kb * 64, tc.t0, tc.b * R + tc.fixed);
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = idesc_bf16_f32(128, 128);
            bool ok = mbar_wait(w_full, 0, abort_flag);
            if (!ok) report_wait_failure(status, abort_flag, kKidOut, 2);
            for (long long lt = 0; lt < my_tiles && ok; ++lt) {
                const int g = (int)(lt & 1);
                const uint32_t use = (uint32_t)(lt >> 1);
                if (!mbar_wait(a_ready(g), use & 1u, abort_flag)) {
                    report_wait_failure(status, abort_flag, kKidOut, 3);
                    break;
                }
                tc_fence_after_sync();
                // gate = LN_in(z) W_g^T -> columns [0,128); update = LN_out(x) W_z^T -> [128,256)
                mma_k128(tmem_base + g * 256, sbase + OutSmem::kZ + g * kTileBytes, sbase + OutSmem::kWg,
                         kKBlockBytes, idesc, false);
                mma_k128(tmem_base + g * 256 + 128, sbase + OutSmem::kX + g * kTileBytes,
                         sbase + OutSmem::kWz, kKBlockBytes, idesc, false);
                mma_commit(d_full(g));
                mma_commit(x_empty(g));
            }
        }
    } else {
        // ---------------------------------------------------------------- two row groups (warps 2..5, 6..9)
        const int g = (warp - 2) >> 2;
        const int quad = warp & 3;
        const int row = quad * 32 + lane;
        const int gtid = (warp - 2 - g * 4) * 32 + lane;  // 0..127 inside the group
        const uint32_t ztile = sbase + OutSmem::kZ + g * kTileBytes;
        const uint32_t xtile = sbase + OutSmem::kX + g * kTileBytes;
        for (long long lt = g; lt < my_tiles; lt += 2) {
            const uint32_t use = (uint32_t)(lt >> 1);
            const TileCoord tc = tile_coord(blockIdx.x + lt * gridDim.x, R, tiles_per_line);
            if (!mbar_wait(x_full(g), use & 1u, abort_flag)) {
                if (lane == 0) report_wait_failure(status, abort_flag, kKidOut, 4);
                break;
            }
            float mean, rstd;
            // --- x column of this position: 128 channels, [c][j] layout, stride 256 B
            {
                uint32_t xraw[64];
                const uint32_t col = xtile + row * 2;
#pragma unroll
                for (int i = 0; i < 64; ++i) {
                    uint32_t lo, hi;
                    if ((i & 7) == 0) asm volatile("" ::: "memory");  // cap the loads in flight per batch
                    asm volatile("ld.shared.u16 %0, [%1];" : "=r"(lo) : "r"(col + (2 * i) * 256));
                    asm volatile("ld.shared.u16 %0, [%1];" : "=r"(hi) : "r"(col + (2 * i + 1) * 256));
                    xraw[i] = lo | (hi << 16);
                }
                row_stats(xraw, mean, rstd);
                group_sync(1 + g, 128);  // everyone has read its column before rows overwrite the buffer
                store_normalized_row(xtile, row, xraw, mean, rstd, prm + 256, prm + 384);
            }
            // --- z row: keep the raw values for the residual, normalise in place (A operand 1)
            if (!mbar_wait(z_full(g), use & 1u, abort_flag)) {
                if (lane == 0) report_wait_failure(status, abort_flag, kKidOut, 7);
                break;
            }
            uint32_t zraw[64];
            load_row(ztile, row, zraw);
            row_stats(zraw, mean, rstd);
            store_normalized_row(ztile, row, zraw, mean, rstd, prm, prm + 128);
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(a_ready(g));
            // --- wait for both GEMMs, combine, write the output tile over the z buffer
            if (!mbar_wait(d_full(g), use & 1u, abort_flag)) {
                if (lane == 0) report_wait_failure(status, abort_flag, kKidOut, 5);
                break;
            }
            tc_fence_after_sync();
            const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + g * 256;
#pragma unroll
            for (int cb = 0; cb < 8; ++cb) {  // 16 channels per step
                uint32_t gate[16], upd[16];
                tmem_ld16(taddr + cb * 16, gate);
                tmem_ld16(taddr + 128 + cb * 16, upd);
                tmem_ld_wait();
#pragma unroll
                for (int ch = 0; ch < 2; ++ch) {
                    uint32_t o[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int e = ch * 8 + j * 2;
                        const uint32_t zr = zraw[cb * 8 + ch * 4 + j];
                        float v0 = sigmoid_fast(__uint_as_float(gate[e])) * __uint_as_float(upd[e]);
                        float v1 = sigmoid_fast(__uint_as_float(gate[e + 1])) * __uint_as_float(upd[e + 1]);
                        if (add_residual) {
                            v0 += bf16lo(zr);
                            v1 += bf16hi(zr);
                        }
                        o[j] = pack_bf16x2(v0, v1);
                    }
                    sts128(chunk_addr(ztile, row, cb * 2 + ch), make_uint4(o[0], o[1], o[2], o[3]));
                }
            }
            tc_fence_before_sync();
            fence_proxy_async_smem();
            group_sync(1 + g, 128);
            if (gtid == 0) {
                for (int kb = 0; kb < 2; ++kb)
                    tma_store_3d(&tmOut, ztile + kb * kKBlockBytes, kb * 64, tc.t0, tc.b * R + tc.fixed);
                tma_store_commit();
                tma_store_wait_read<0>();
                mbar_arrive(z_empty(g));
            }
        }
        if (gtid == 0) tma_store_wait_all<0>();
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 512);
    }
}

int weight_tmap(CUtensorMap* m, const void* w, int rows) {
    uint64_t dims[2] = {128, (uint64_t)rows};
    uint64_t str[1] = {256};
    uint32_t box[2] = {64, 128};
    return make_tmap_bf16(m, w, 2, dims, str, box, true);
}

}  // namespace


bool trimul_supported(int c_z, int c_h) { return c_z == 128 && c_h == 128; }

static int set_attrs() {
    if (!device_configured(5)) {
        OF3_CUDA_CHECK(cudaFuncSetAttribute(trimul_in_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, InSmem::kDyn));
        OF3_CUDA_CHECK(cudaFuncSetAttribute(trimul_in_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, InSmem::kDyn));
        OF3_CUDA_CHECK(cudaFuncSetAttribute(trimul_in_rows_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, InSmem::kDyn));
        OF3_CUDA_CHECK(cudaFuncSetAttribute(trimul_in_rows_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, InSmem::kDyn));
        OF3_CUDA_CHECK(cudaFuncSetAttribute(trimul_out_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, OutSmem::kDyn));
        device_mark_configured(5);
    }
    return OF3_OK;
}

// z as lines: {c, position, b*R + line}
static int line_tmap(CUtensorMap* m, const void* z, int B, int R, int N) {
    uint64_t dims[3] = {128, (uint64_t)N, (uint64_t)B * R};
    uint64_t str[2] = {256, (uint64_t)N * 256};
    uint32_t box[3] = {64, 128, 1};
    return make_tmap_bf16(m, z, 3, dims, str, box, 1);
}

// a_t[(b*128 + c)][line][k], b_t likewise, from R lines of N positions per sample: z is [B][R][N][128].
// transposed_walk: z is [B][N][R][128] and a line runs along its FIRST index (line = second index),
// which makes the incoming update the same K-major contraction as the outgoing one; with R != N this
// is a row shard of N rows seen as R lines of N positions each.
// groups > 1: the 128 channels are written as `groups` equal groups, group q of a_t at
// a_t + q * group_stride (b_t likewise), so that each group can be sent to another rank as one block.
int trimul_project(const __nv_bfloat16* z, const __nv_bfloat16* mask, __nv_bfloat16* a_t, __nv_bfloat16* b_t,
                   int B, int R, int N, int ld, bool transposed_walk, const of3_trimul_params* p,
                   cudaStream_t st, int groups, long long group_stride) {
    OF3_REQUIRE(((uintptr_t)z & 15) == 0, OF3_ERR_ALIGN, "trimul: z must be 16-byte aligned");
    OF3_REQUIRE(groups == 1 || groups == 2 || groups == 4 || groups == 8, OF3_ERR_ARG,
                "trimul: channel groups must be 1, 2, 4 or 8 (got %d)", groups);
    int group_shift = 7;
    for (int g = groups; g > 1; g >>= 1) --group_shift;
    if (groups == 1) group_stride = (long long)kC * R * ld;
    int rc;
    CUtensorMap tmZ, tmW[4];
    if (!transposed_walk) {
        if ((rc = line_tmap(&tmZ, z, B, R, N))) return rc;
    } else {  // {c, second (line), first (position), b}
        uint64_t dims[4] = {128, (uint64_t)R, (uint64_t)N, (uint64_t)B};
        uint64_t str[3] = {256, (uint64_t)R * 256, (uint64_t)N * R * 256};
        uint32_t box[4] = {64, 1, 128, 1};
        if ((rc = make_tmap_bf16(&tmZ, z, 4, dims, str, box, 1))) return rc;
    }
    const void* w4[4] = {p->w_a_p, p->w_a_g, p->w_b_p, p->w_b_g};
    for (int i = 0; i < 4; ++i)
        if ((rc = weight_tmap(&tmW[i], w4[i], 128))) return rc;
    if ((rc = set_attrs())) return rc;
    const long long tiles = (long long)B * R * ceil_div(N, kRows);
    const int grid = (int)(tiles < sm_count() ? tiles : sm_count());
    // 32-byte stores need every channel row of a_t / b_t to start on a 32-byte boundary
    const int wide = (ld % 16 == 0 && (group_stride % 16) == 0 && ((uintptr_t)a_t & 31) == 0 && ((uintptr_t)b_t & 31) == 0) ? 1 : 0;
    // a channel plane of R lines: beyond about one 2 MB page the kernel whose stores stay inside one plane wins
    const bool planes_far_apart = (long long)R * ld * (long long)sizeof(__nv_bfloat16) > (2LL << 20);
    LaunchScope scope(kKidIn, st);
    const __nv_bfloat16* lw = (const __nv_bfloat16*)p->ln_in_w;
    const __nv_bfloat16* lb = (const __nv_bfloat16*)p->ln_in_b;
    if (planes_far_apart) {
        if (!transposed_walk)
            trimul_in_rows_kernel<true><<<grid, kInRowsThreads, InSmem::kDyn, st>>>(
                tmZ, tmW[0], tmW[1], tmW[2], tmW[3], mask, lw, lb, a_t, b_t, B, R, N, ld, group_shift, group_stride,
                device_status_ptr());
        else
            trimul_in_rows_kernel<false><<<grid, kInRowsThreads, InSmem::kDyn, st>>>(
                tmZ, tmW[0], tmW[1], tmW[2], tmW[3], mask, lw, lb, a_t, b_t, B, R, N, ld, group_shift, group_stride,
                device_status_ptr());
    } else if (!transposed_walk) {
        trimul_in_kernel<true><<<grid, kInThreads, InSmem::kDyn, st>>>(
            tmZ, tmW[0], tmW[1], tmW[2], tmW[3], mask, lw, lb, a_t, b_t, B, R, N, ld, group_shift, group_stride, wide,
            device_status_ptr());
    } else {
        trimul_in_kernel<false><<<grid, kInThreads, InSmem::kDyn, st>>>(
            tmZ, tmW[0], tmW[1], tmW[2], tmW[3], mask, lw, lb, a_t, b_t, B, R, N, ld, group_shift, group_stride, wide,
            device_status_ptr());
    }
    OF3_CUDA_CHECK(cudaGetLastError());
    return OF3_OK;
}

// x = a_t . b_t^T per channel (a_t: R lines, b_t: all N lines), then LN_out / linear_z / gate / residual
// on the R lines of z -> out (may alias z).
int trimul_finish(const __nv_bfloat16* z, __nv_bfloat16* out, const __nv_bfloat16* a_t,
                  const __nv_bfloat16* b_t, __nv_bfloat16* x_t, int B, int R, int N, int ld, int add_residual,
                  const of3_trimul_params* p, cudaStream_t st) {
    OF3_REQUIRE(((uintptr_t)z & 15) == 0 && ((uintptr_t)out & 15) == 0, OF3_ERR_ALIGN,
                "trimul: z/out must be 16-byte aligned");
    int rc = contract_nt_bf16(a_t, b_t, x_t, B * kC, R, N, N, ld, ld, ld, (long long)R * ld, (long long)N * ld,
                              (long long)R * ld, st);
    if (rc) return rc;
    return trimul_output(z, out, x_t, B, R, N, ld, add_residual, p, st);
}

// LN_out(x) -> linear_z, gate from LN_in(z), residual: the part of the update after the contraction,
// on R lines of z with x_t[b*128 + c][line][j] (pitch ld)
int trimul_output(const __nv_bfloat16* z, __nv_bfloat16* out, const __nv_bfloat16* x_t, int B, int R, int N, int ld,
                  int add_residual, const of3_trimul_params* p, cudaStream_t st) {
    OF3_REQUIRE(((uintptr_t)z & 15) == 0 && ((uintptr_t)out & 15) == 0 && ((uintptr_t)x_t & 15) == 0, OF3_ERR_ALIGN,
                "trimul: z/out/x must be 16-byte aligned");
    int rc;
    CUtensorMap tmZ, tmOut, tmX, tmWg, tmWz;
    if ((rc = line_tmap(&tmZ, z, B, R, N))) return rc;
    if ((rc = line_tmap(&tmOut, out, B, R, N))) return rc;
    {   // x_t[b*128 + c][line][j], pitch ld: box = 128 positions j x 1 x 128 channels, no swizzle
        uint64_t dims[3] = {(uint64_t)N, (uint64_t)R, (uint64_t)B * kC};
        uint64_t str[2] = {(uint64_t)ld * 2, (uint64_t)R * ld * 2};
        uint32_t box[3] = {128, 1, 128};
        if ((rc = make_tmap_bf16(&tmX, x_t, 3, dims, str, box, 0))) return rc;
    }
    if ((rc = weight_tmap(&tmWg, p->w_g, 128))) return rc;
    if ((rc = weight_tmap(&tmWz, p->w_z, 128))) return rc;
    if ((rc = set_attrs())) return rc;
    const long long tiles = (long long)B * R * ceil_div(N, kRows);
    const int grid = (int)(tiles < sm_count() ? tiles : sm_count());
    LaunchScope scope(kKidOut, st);
    trimul_out_kernel<<<grid, 320, OutSmem::kDyn, st>>>(
        tmZ, tmX, tmOut, tmWg, tmWz, (const __nv_bfloat16*)p->ln_in_w, (const __nv_bfloat16*)p->ln_in_b,
        (const __nv_bfloat16*)p->ln_out_w, (const __nv_bfloat16*)p->ln_out_b, B, R, N, add_residual,
        device_status_ptr());
    OF3_CUDA_CHECK(cudaGetLastError());
    return OF3_OK;
}

int trimul(const __nv_bfloat16* z, const __nv_bfloat16* mask, __nv_bfloat16* out, int B, int N,
           int flags, const of3_trimul_params* p, Arena& ws, cudaStream_t st) {
    const int ld = (int)align_up(N, 8);
    const size_t plane = (size_t)B * kC * N * ld * sizeof(__nv_bfloat16);
    __nv_bfloat16* a_t = (__nv_bfloat16*)ws.take(plane);
    __nv_bfloat16* b_t = (__nv_bfloat16*)ws.take(plane);
    __nv_bfloat16* x_t = (__nv_bfloat16*)ws.take(plane);
    if (!ws.base) return OF3_OK;
    OF3_REQUIRE(ws.ok(), OF3_ERR_WORKSPACE, "trimul: workspace too small (%zu needed)", ws.off);
    const bool outgoing = (flags & OF3_FLAG_OUTGOING) != 0;
    int rc = trimul_project(z, mask, a_t, b_t, B, N, N, ld, !outgoing, p, st);
    if (rc) return rc;
    return trimul_finish(z, out, a_t, b_t, x_t, B, N, N, ld, (flags & OF3_FLAG_ADD_RESIDUAL) ? 1 : 0, p, st);
}

}  // namespace fast
}  // namespace of3
