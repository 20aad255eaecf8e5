// SwiGLU pair transition, bf16 / tcgen05 family (c = 128, expansion 4 -> hidden 512).
//
// One fused kernel: x tile -> LayerNorm (in place in the A operand) -> per 64-wide hidden chunk
//   G1: [a|b] = LN(x) [W_a;W_b]_chunk^T  (128x128x128, accumulators in TMEM)
//   h  = silu(a) * b  -> bf16 -> shared memory as the next A operand (never leaves the SM)
//   G2: y += h W_out[:, chunk]^T         (128x128x64, accumulated over the 8 chunks in TMEM)
// then out = x + mask * y, TMA-stored. The 512-wide hidden activation (604 MB at N = 768 in the
// reference's unfused path) never touches HBM. Two 128-row groups ping-pong on the tensor pipe
// and share every weight chunk (streamed from L2 by TMA, double-buffered), which halves the
// weight traffic per row.
// Reference: openfold3/core/model/layers/transition.py:225-271,
//            openfold3/core/model/primitives/activations.py:33-61.
#include "modules.cuh"
#include "rowtile.cuh"
#include "runtime.cuh"

namespace of3 {
namespace fast {
namespace {

using namespace umma;
using namespace rowtile;

constexpr int kKidTrans = 4;
constexpr int kHidden = 512;
constexpr int kChunk = 64;
constexpr int kNumChunks = kHidden / kChunk;  // 8


struct TrSmem {
    static constexpr uint32_t kWStage = 49152;                 // [Wa|Wb] slab 32 KB + Wout chunk 16 KB
    static constexpr uint32_t kW = 0;                          // 2 stages
    static constexpr uint32_t kX = 2 * kWStage;                // 2 groups x 32 KB (x tile / A / output)
    static constexpr uint32_t kH = kX + 2 * kTileBytes;        // 2 groups x 16 KB
    static constexpr uint32_t kParams = kH + 2 * kKBlockBytes; // gamma, beta
    static constexpr uint32_t kXch = kParams + 1024;           // 2 groups x 512 floats: LayerNorm partial sums
    static constexpr uint32_t kBars = kXch + 4096;
    static constexpr uint32_t kTotal = kBars + 256;
    static constexpr uint32_t kDyn = kTotal + 1024;
};

// warps: 0 producer, 1 and 2 the MMA issuers of row group 0 and 1, 3..10 and 11..18 the two row groups: two
// threads share a row (TMEM lane) and take half of its channels each through LayerNorm, half of every hidden chunk
// through silu * mul, and half of the output row -- the per-row chains were the longest thing in the kernel.
// One issuing thread for both groups was the critical path (in-kernel clock64 phases: 5000 cycles per hidden
// chunk for 1536 cycles of tensor work -- it waited for one group's silu pass while the other group's next
// GEMM was ready to go); each group now has its own issuer and the tensor pipe interleaves the two chains.
constexpr int kTrThreads = 32 * (3 + 2 * 8);

__global__ void __launch_bounds__(kTrThreads, 1)
transition_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmOut,
                  const __grid_constant__ CUtensorMap tmWa, const __grid_constant__ CUtensorMap tmWb,
                  const __grid_constant__ CUtensorMap tmWo, const __nv_bfloat16* __restrict__ mask,
                  const __nv_bfloat16* __restrict__ ln_w, const __nv_bfloat16* __restrict__ ln_b,
                  long long rows, int add_residual, int* status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gbase = smem_raw + (sbase - smem_u32(smem_raw));
    float* prm = reinterpret_cast<float*>(gbase + TrSmem::kParams);
    const uint32_t bars = sbase + TrSmem::kBars;
    auto w_full = [&](int s) { return bars + 8u * (0 + s); };
    auto w_empty = [&](int s) { return bars + 8u * (2 + s); };
    auto x_full = [&](int g) { return bars + 8u * (4 + g); };
    auto x_empty = [&](int g) { return bars + 8u * (6 + g); };
    auto a_ready = [&](int g) { return bars + 8u * (8 + g); };
    auto d1_full = [&](int g) { return bars + 8u * (10 + g); };
    auto d1_empty = [&](int g) { return bars + 8u * (12 + g); };
    auto h_ready = [&](int g) { return bars + 8u * (14 + g); };
    auto h_free = [&](int g) { return bars + 8u * (16 + g); };
    auto d2_full = [&](int g) { return bars + 8u * (18 + g); };
    auto d2_empty = [&](int g) { return bars + 8u * (20 + g); };
    auto wo_full = [&](int s) { return bars + 8u * (22 + s); };   // W_out chunk of a weight stage (its own ring:
    auto wo_empty = [&](int s) { return bars + 8u * (24 + s); };  // the slab is free long before the chunk's 2nd GEMM)
    volatile uint32_t* tmem_ptr = reinterpret_cast<volatile uint32_t*>(gbase + TrSmem::kBars + 224);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + TrSmem::kBars + 232);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long num_tiles = (rows + kRows - 1) / kRows;
    const long long my_tiles = (num_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x;
    const long long my_pairs = (my_tiles + 1) / 2;

    if (threadIdx.x == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(w_full(i), 1);
            mbar_init(w_empty(i), 2);  // both groups' issuers have consumed the [W_a|W_b] slab
            mbar_init(wo_full(i), 1);
            mbar_init(wo_empty(i), 2);
            mbar_init(x_full(i), 1);
            mbar_init(x_empty(i), 1);
            mbar_init(a_ready(i), 8);
            mbar_init(d1_full(i), 1);
            mbar_init(d1_empty(i), 8);
            mbar_init(h_ready(i), 8);
            mbar_init(h_free(i), 1);
            mbar_init(d2_full(i), 1);
            mbar_init(d2_empty(i), 8);
        }
        *abort_flag = 0;
        mbar_fence_init();
        prefetch_tmap(&tmX);
        prefetch_tmap(&tmWa);
        prefetch_tmap(&tmWb);
        prefetch_tmap(&tmWo);
    }
    if (threadIdx.x < 128) {
        prm[threadIdx.x] = __bfloat162float(ln_w[threadIdx.x]);
        prm[128 + threadIdx.x] = __bfloat162float(ln_b[threadIdx.x]);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32((const void*)tmem_ptr), 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_ptr;
    // TMEM columns: group g -> D1 at g*256 + [0,128) ([a 64 | b 64]), D2 at g*256 + [128,256)

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            uint32_t wi = 0;
            bool ok = true;
            for (long long pi = 0; pi < my_pairs && ok; ++pi) {
                for (int g = 0; g < 2; ++g) {
                    const long long lt = pi * 2 + g;
                    if (lt >= my_tiles) break;
                    if (!mbar_wait(x_empty(g), ((uint32_t)pi & 1u) ^ 1u, abort_flag)) {
                        report_wait_failure(status, abort_flag, kKidTrans, 1);
                        ok = false;
                        break;
                    }
                    const long long tile = blockIdx.x + lt * gridDim.x;
                    mbar_arrive_expect_tx(x_full(g), kTileBytes);
                    const uint32_t dst = sbase + TrSmem::kX + g * kTileBytes;
                    // rows can exceed 2^31 only beyond any realistic N; tile*128 fits in int for N <= 46340
                    tma_load_2d(dst, &tmX, x_full(g), 0, (int)(tile * kRows));
                    tma_load_2d(dst + kKBlockBytes, &tmX, x_full(g), 64, (int)(tile * kRows));
                }
                for (int c = 0; c < kNumChunks && ok; ++c, ++wi) {
                    const int s = wi & 1;
                    if (!mbar_wait(w_empty(s), ((wi >> 1) & 1u) ^ 1u, abort_flag)) {
                        report_wait_failure(status, abort_flag, kKidTrans, 2);
                        ok = false;
                        break;
                    }
                    mbar_arrive_expect_tx(w_full(s), 2 * kKBlockBytes);
                    const uint32_t w = sbase + TrSmem::kW + s * TrSmem::kWStage;
                    for (int kb = 0; kb < 2; ++kb) {
                        // slab k-block kb: rows [0,64) = W_a chunk, rows [64,128) = W_b chunk
                        tma_load_2d(w + kb * kKBlockBytes, &tmWa, w_full(s), kb * 64, c * kChunk);
                        tma_load_2d(w + kb * kKBlockBytes + 64 * 128, &tmWb, w_full(s), kb * 64, c * kChunk);
                    }
                    if (!mbar_wait(wo_empty(s), ((wi >> 1) & 1u) ^ 1u, abort_flag)) {
                        report_wait_failure(status, abort_flag, kKidTrans, 12);
                        ok = false;
                        break;
                    }
                    mbar_arrive_expect_tx(wo_full(s), kKBlockBytes);
                    tma_load_2d(w + 2 * kKBlockBytes, &tmWo, wo_full(s), c * kChunk, 0);
                }
            }
        }
    } else if (warp <= 2) {
        // ---------------------------------------------------------------- MMA issuer of row group g
        if (lane == 0) {
            const int g = warp - 1;
            constexpr uint32_t idesc = idesc_bf16_f32(128, 128);
            uint32_t wi = 0;
            bool ok = true;
            auto fail = [&](int site) {
                report_wait_failure(status, abort_flag, kKidTrans, site);
                ok = false;
            };
            // Software-pipelined per tile: G1 of chunk c+1 is issued as soon as the row group has read D1 of
            // chunk c, BEFORE waiting for that chunk's silu pass and its G2, so the row group finds its next
            // accumulator ready when it comes back (the serial G2 -> weights -> G1 hop cost ~1900 cycles per chunk).
            auto issue_g1 = [&](uint32_t widx, uint32_t c) -> bool {
                const int s = widx & 1;
                if (!mbar_wait(w_full(s), (widx >> 1) & 1u, abort_flag)) { fail(3); return false; }
                if (!mbar_wait(d1_empty(g), (c & 1u) ^ 1u, abort_flag)) { fail(5); return false; }
                tc_fence_after_sync();
                mma_k128(tmem_base + g * 256, sbase + TrSmem::kX + g * kTileBytes,
                         sbase + TrSmem::kW + s * TrSmem::kWStage, kKBlockBytes, idesc, false);
                mma_commit(d1_full(g));
                mma_commit(w_empty(s));
                return true;
            };
            for (long long pi = 0; pi < my_pairs && ok; ++pi) {
                const bool have_tile = pi * 2 + g < my_tiles;  // the last pair may hold one tile only
                const uint32_t ppar = (uint32_t)pi & 1u;
                if (!have_tile) {  // keep both weight rings moving
                    for (int c = 0; c < kNumChunks && ok; ++c, ++wi) {
                        const int s = wi & 1;
                        if (!mbar_wait(w_full(s), (wi >> 1) & 1u, abort_flag)) { fail(3); break; }
                        mbar_arrive(w_empty(s));
                        if (!mbar_wait(wo_full(s), (wi >> 1) & 1u, abort_flag)) { fail(13); break; }
                        mbar_arrive(wo_empty(s));
                    }
                    continue;
                }
                if (!mbar_wait(a_ready(g), ppar, abort_flag)) { fail(4); break; }
                if (!issue_g1(wi, 0)) break;
                for (int c = 0; c < kNumChunks && ok; ++c, ++wi) {
                    const int s = wi & 1;
                    const uint32_t cpar = (uint32_t)c & 1u;  // 8 chunks per tile: chunk parity is global
                    if (c + 1 < kNumChunks && !issue_g1(wi + 1, c + 1)) break;
                    if (c == 0 && !mbar_wait(d2_empty(g), ppar ^ 1u, abort_flag)) { fail(6); break; }
                    if (!mbar_wait(wo_full(s), (wi >> 1) & 1u, abort_flag)) { fail(13); break; }
                    if (!mbar_wait(h_ready(g), cpar, abort_flag)) { fail(7); break; }
                    tc_fence_after_sync();
                    const uint64_t ad = smem_desc_k_sw128(sbase + TrSmem::kH + g * kKBlockBytes);
                    const uint64_t bd = smem_desc_k_sw128(sbase + TrSmem::kW + s * TrSmem::kWStage + 2 * kKBlockBytes);
#pragma unroll
                    for (int k4 = 0; k4 < 4; ++k4)
                        mma_bf16(tmem_base + g * 256 + 128, ad + 2u * k4, bd + 2u * k4, idesc,
                                 (c != 0 || k4 != 0) ? 1u : 0u);
                    mma_commit(h_free(g));
                    if (c == kNumChunks - 1) mma_commit(d2_full(g));
                    mma_commit(wo_empty(s));
                }
            }
        }
    } else {
        // ---------------------------------------------------------------- two row groups
        const int g = (warp - 3) >> 3;
        const int quad = warp & 3;
        const int half = ((warp - 3) >> 2) & 1;
        const int row = quad * 32 + lane;
        const int gtid = (warp - 3 - g * 8) * 32 + lane;
        float* xch = reinterpret_cast<float*>(gbase + TrSmem::kXch) + g * 512;
        const uint32_t xtile = sbase + TrSmem::kX + g * kTileBytes;
        const uint32_t htile = sbase + TrSmem::kH + g * kKBlockBytes;
        const uint32_t t_d1 = tmem_base + ((uint32_t)(quad * 32) << 16) + g * 256;
        const uint32_t t_d2 = t_d1 + 128;
        bool ok = true;
        for (long long pi = 0; pi * 2 + g < my_tiles && ok; ++pi) {
            const uint32_t ppar = (uint32_t)pi & 1u;
            const long long tile = blockIdx.x + (pi * 2 + g) * gridDim.x;
            const long long grow = tile * kRows + row;
            if (!mbar_wait(x_full(g), ppar, abort_flag)) {
                if (lane == 0) report_wait_failure(status, abort_flag, kKidTrans, 8);
                break;
            }
            uint32_t raw[32];   // this thread's 64 channels of the row: kept for the residual
            load_half_row(xtile, row, half, raw);
            {
                float mean, rstd;
                half_row_stats_xwarp(raw, row, half, xch, 1 + g, 256, mean, rstd);
                store_normalized_half_row(xtile, row, half, raw, mean, rstd, prm, prm + 128);
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(a_ready(g));
            float m = 1.0f;
            if (mask != nullptr && grow < rows) m = __bfloat162float(mask[grow]);

            for (int c = 0; c < kNumChunks; ++c) {
                const uint32_t cpar = (uint32_t)c & 1u;
                if (!mbar_wait(d1_full(g), cpar, abort_flag)) {
                    if (lane == 0) report_wait_failure(status, abort_flag, kKidTrans, 9);
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                uint32_t hpk[16];  // 32 of the chunk's 64 hidden values of this row, packed bf16x2
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    uint32_t a[16], b[16];
                    tmem_ld16(t_d1 + half * 32 + q * 16, a);
                    tmem_ld16(t_d1 + 64 + half * 32 + q * 16, b);
                    tmem_ld_wait();
#pragma unroll
                    for (int e = 0; e < 16; e += 2) {
                        const float a0 = __uint_as_float(a[e]), a1 = __uint_as_float(a[e + 1]);
                        const float h0 = a0 * sigmoid_fast(a0) * __uint_as_float(b[e]);
                        const float h1 = a1 * sigmoid_fast(a1) * __uint_as_float(b[e + 1]);
                        hpk[q * 8 + e / 2] = pack_bf16x2(h0, h1);
                    }
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(d1_empty(g));
                // the previous chunk's G2 must have consumed the H buffer before it is overwritten
                if (!mbar_wait(h_free(g), cpar ^ 1u, abort_flag)) {
                    if (lane == 0) report_wait_failure(status, abort_flag, kKidTrans, 10);
                    ok = false;
                    break;
                }
#pragma unroll
                for (int ch = 0; ch < 4; ++ch)
                    sts128(chunk_addr(htile, row, half * 4 + ch),
                           make_uint4(hpk[ch * 4], hpk[ch * 4 + 1], hpk[ch * 4 + 2], hpk[ch * 4 + 3]));
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(h_ready(g));
            }
            if (!ok) break;
            if (!mbar_wait(d2_full(g), ppar, abort_flag)) {
                if (lane == 0) report_wait_failure(status, abort_flag, kKidTrans, 11);
                break;
            }
            tc_fence_after_sync();
#pragma unroll
            for (int cb = 0; cb < 4; ++cb) {
                uint32_t y[16];
                tmem_ld16(t_d2 + half * 64 + cb * 16, y);
                tmem_ld_wait();
#pragma unroll
                for (int ch = 0; ch < 2; ++ch) {
                    uint32_t o[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int e = ch * 8 + j * 2;
                        const uint32_t xr = raw[cb * 8 + ch * 4 + j];
                        float v0 = m * __uint_as_float(y[e]);
                        float v1 = m * __uint_as_float(y[e + 1]);
                        if (add_residual) {
                            v0 += bf16lo(xr);
                            v1 += bf16hi(xr);
                        }
                        o[j] = pack_bf16x2(v0, v1);
                    }
                    sts128(chunk_addr(xtile, row, half * 8 + cb * 2 + ch), make_uint4(o[0], o[1], o[2], o[3]));
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(d2_empty(g));
            fence_proxy_async_smem();
            group_sync(1 + g, 256);
            if (gtid == 0) {
                tma_store_3d(&tmOut, xtile, 0, (int)(tile * kRows), 0);
                tma_store_3d(&tmOut, xtile + kKBlockBytes, 64, (int)(tile * kRows), 0);
                tma_store_commit();
                tma_store_wait_read<0>();
                mbar_arrive(x_empty(g));
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

}  // namespace


bool transition_supported(int c, int n) { return c == 128 && n == 4; }

int transition(const __nv_bfloat16* x, const __nv_bfloat16* mask, __nv_bfloat16* out, long long rows,
               int flags, const of3_transition_params* p, Arena& ws, cudaStream_t st) {
    (void)ws.take(16);
    if (!ws.base) return OF3_OK;
    OF3_REQUIRE(rows < (1LL << 31) - 256, OF3_ERR_SHAPE, "transition: too many rows");
    int rc;
    CUtensorMap tmX, tmOut, tmWa, tmWb, tmWo;
    {
        uint64_t dims[2] = {128, (uint64_t)rows};
        uint64_t str[1] = {256};
        uint32_t box[2] = {64, 128};
        if ((rc = make_tmap_bf16(&tmX, x, 2, dims, str, box, true))) return rc;
        // the store map is 3-D only to share tma_store_3d with the other kernels
        uint64_t dims3[3] = {128, (uint64_t)rows, 1};
        uint64_t str3[2] = {256, (uint64_t)rows * 256};
        uint32_t box3[3] = {64, 128, 1};
        if ((rc = make_tmap_bf16(&tmOut, out, 3, dims3, str3, box3, true))) return rc;
    }
    {
        uint64_t dims[2] = {128, kHidden};
        uint64_t str[1] = {256};
        uint32_t box[2] = {64, kChunk};
        if ((rc = make_tmap_bf16(&tmWa, p->w_a, 2, dims, str, box, true))) return rc;
        if ((rc = make_tmap_bf16(&tmWb, p->w_b, 2, dims, str, box, true))) return rc;
        uint64_t dimo[2] = {kHidden, 128};
        uint64_t stro[1] = {kHidden * 2};
        uint32_t boxo[2] = {kChunk, 128};
        if ((rc = make_tmap_bf16(&tmWo, p->w_out, 2, dimo, stro, boxo, true))) return rc;
    }
    if (!device_configured(4)) {
        OF3_CUDA_CHECK(cudaFuncSetAttribute(transition_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            TrSmem::kDyn));
        device_mark_configured(4);
    }
    const long long tiles = (rows + kRows - 1) / kRows;
    // two tiles per CTA pass share each weight chunk: aim for an even number of tiles per CTA
    long long grid = sm_count();
    if (tiles < 2 * grid) grid = (tiles + 1) / 2;
    if (grid < 1) grid = 1;
    LaunchScope scope(kKidTrans, st);
    transition_kernel<<<(int)grid, kTrThreads, TrSmem::kDyn, st>>>(
        tmX, tmOut, tmWa, tmWb, tmWo, mask, (const __nv_bfloat16*)p->ln_w, (const __nv_bfloat16*)p->ln_b,
        rows, (flags & OF3_FLAG_ADD_RESIDUAL) ? 1 : 0, device_status_ptr());
    OF3_CUDA_CHECK(cudaGetLastError());
    return OF3_OK;
}

}  // namespace fast
}  // namespace of3
