// Batched NT contraction on tcgen05:  X[b][i][j] = sum_k A[b][i][k] * B[b][j][k]
// (bf16 operands, fp32 accumulation in TMEM, bf16 result).
//
// This is the N^3*c part of the triangle multiplicative update: one "batch" entry per
// (sample, hidden channel); the prologue kernel writes the gated projections a, b
// channel-major with the contracted index innermost, so the outgoing and the incoming
// update are the same K-major x K-major GEMM
// (reference: openfold3/core/model/layers/triangular_multiplicative_update.py:71-97).
//
// Persistent, warp-specialised CTA (one per SM):
//   warp 0     TMA producer     A tile 128x64, B tile BNx64 per k-block, 128B swizzle
//   warp 1     MMA issuer       tcgen05.mma 128 x BN x 16, accumulators double-buffered in TMEM
//   warps 2-5  epilogue         tcgen05.ld -> bf16 -> global (overlaps the next tile's main loop)
#include "runtime.cuh"
#include "umma.cuh"

namespace of3 {
namespace {

using namespace umma;

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kKernelIdContract = 1;

template <int BN>
struct ContractCfg {
    static constexpr int kStages = (BN == 256) ? 4 : 6;
    static constexpr int kABytes = kBM * kBK * 2;
    static constexpr int kBBytes = BN * kBK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kTmemCols = 2 * BN;
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align slack*/ + 256 /*barriers*/;
};

template <int BN>
__global__ void __launch_bounds__(192, 1)
contract_nt_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                   __nv_bfloat16* __restrict__ out, int M, int N, int K, int batch,
                   long long out_batch_stride, int ldo, int rows_per_block, long long row_block_stride,
                   int a_shared, int* status) {
    using Cfg = ContractCfg<BN>;
    constexpr int S = Cfg::kStages;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar_base = smem_base + S * Cfg::kStageBytes;
    // barrier block: full[S], empty[S], tmem_full[2], tmem_empty[2] (8 B each), then tmem ptr, abort
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (S + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * S + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * S + 2 + a); };
    uint8_t* gen_base = smem_raw + (smem_base - smem_u32(smem_raw));
    volatile uint32_t* tmem_ptr_smem =
        reinterpret_cast<volatile uint32_t*>(gen_base + S * Cfg::kStageBytes + 8 * (2 * S + 4));
    volatile int* abort_flag =
        reinterpret_cast<volatile int*>(gen_base + S * Cfg::kStageBytes + 8 * (2 * S + 4) + 8);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    const int num_mt = (M + kBM - 1) / kBM;
    const int num_nt = (N + BN - 1) / BN;
    const int num_kb = (K + kBK - 1) / kBK;
    const long long num_tiles = (long long)batch * num_mt * num_nt;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 4);
        }
        *abort_flag = 0;
        mbar_fence_init();
        prefetch_tmap(&tmA);
        prefetch_tmap(&tmB);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32((const void*)tmem_ptr_smem), Cfg::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_ptr_smem;

    if (warp == 0) {
        // ------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (long long t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                const int nt = (int)(t % num_nt);
                const int mt = (int)((t / num_nt) % num_mt);
                const int b = (int)(t / ((long long)num_nt * num_mt));
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % S;
                    const uint32_t ph = (it / S) & 1u;
                    if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag)) {
                        report_wait_failure(status, abort_flag, kKernelIdContract, 1);
                        ok = false;
                        break;
                    }
                    mbar_arrive_expect_tx(full_bar(s), Cfg::kStageBytes);
                    const uint32_t sa = smem_base + s * Cfg::kStageBytes;
                    tma_load_3d(sa, &tmA, full_bar(s), kb * kBK, mt * kBM, a_shared ? 0 : b);
                    tma_load_3d(sa + Cfg::kABytes, &tmB, full_bar(s), kb * kBK, nt * BN, b);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = idesc_bf16_f32(kBM, BN);
            uint32_t it = 0, tcount = 0;
            bool ok = true;
            for (long long t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tcount) {
                const uint32_t acc = tcount & 1u;
                const uint32_t acc_ph = (tcount >> 1) & 1u;
                if (!mbar_wait(tempty_bar(acc), acc_ph ^ 1u, abort_flag)) {
                    report_wait_failure(status, abort_flag, kKernelIdContract, 2);
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % S;
                    const uint32_t ph = (it / S) & 1u;
                    if (!mbar_wait(full_bar(s), ph, abort_flag)) {
                        report_wait_failure(status, abort_flag, kKernelIdContract, 3);
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t sa = smem_base + s * Cfg::kStageBytes;
                    const uint64_t adesc = smem_desc_k_sw128(sa);
                    const uint64_t bdesc = smem_desc_k_sw128(sa + Cfg::kABytes);
#pragma unroll
                    for (int k4 = 0; k4 < kBK / 16; ++k4) {
                        // +32 B per 16-element K step == +2 in the 16-byte-unit address field
                        mma_bf16(d_tmem, adesc + 2u * k4, bdesc + 2u * k4, idesc,
                                 (kb | k4) != 0 ? 1u : 0u);
                    }
                    mma_commit(empty_bar(s));
                }
                if (ok) mma_commit(tfull_bar(acc));
            }
        }
    } else {
        // ------------------------------------------------ epilogue (warps 2..5)
        const int quad = warp & 3;  // TMEM lane quarter this warp may read
        uint32_t tcount = 0;
        bool ok = true;
        for (long long t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tcount) {
            const int nt = (int)(t % num_nt);
            const int mt = (int)((t / num_nt) % num_mt);
            const int b = (int)(t / ((long long)num_nt * num_mt));
            const uint32_t acc = tcount & 1u;
            const uint32_t acc_ph = (tcount >> 1) & 1u;
            if (!mbar_wait(tfull_bar(acc), acc_ph, abort_flag)) {
                if (lane == 0) report_wait_failure(status, abort_flag, kKernelIdContract, 4);
                ok = false;
                break;
            }
            tc_fence_after_sync();
            const int row = mt * kBM + quad * 32 + lane;
            // rows_per_block > 0: output rows are grouped in blocks of that many rows and block q starts
            // at q * row_block_stride (the layout a row-sharding all-to-all sends without a repack)
            long long roff = (long long)row * ldo;
            if (rows_per_block > 0) {
                const int q = row / rows_per_block;
                roff = (long long)q * row_block_stride + (long long)(row - q * rows_per_block) * ldo;
            }
            __nv_bfloat16* orow = out + (long long)b * out_batch_stride + roff;
            const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * BN;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t r[32];
                tmem_ld32(taddr + c * 32, r);
                tmem_ld_wait();
                const int col0 = nt * BN + c * 32;
                if (row < M) {
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        const int col = col0 + g * 8;
                        if (col < N) {
                            uint4 v;
                            v.x = pack_bf16x2(__uint_as_float(r[g * 8 + 0]), __uint_as_float(r[g * 8 + 1]));
                            v.y = pack_bf16x2(__uint_as_float(r[g * 8 + 2]), __uint_as_float(r[g * 8 + 3]));
                            v.z = pack_bf16x2(__uint_as_float(r[g * 8 + 4]), __uint_as_float(r[g * 8 + 5]));
                            v.w = pack_bf16x2(__uint_as_float(r[g * 8 + 6]), __uint_as_float(r[g * 8 + 7]));
                            *reinterpret_cast<uint4*>(orow + col) = v;
                        }
                    }
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(acc));
        }
    }

    // ---------------------------------------------------- teardown
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
}

template <int BN>
int launch_contract(const __nv_bfloat16* a, const __nv_bfloat16* b, __nv_bfloat16* out, int batch,
                    int M, int N, int K, int lda, int ldb, int ldo, long long a_bs, long long b_bs,
                    long long o_bs, int rows_per_block, long long row_block_stride, cudaStream_t stream,
                    int account_as) {
    using Cfg = ContractCfg<BN>;
    CUtensorMap tmA, tmB;
    {
        // a_bs == 0: every batch entry multiplies the same A (several linear layers on one input)
        uint64_t dims[3] = {(uint64_t)K, (uint64_t)M, (uint64_t)(a_bs == 0 ? 1 : batch)};
        uint64_t str[2] = {(uint64_t)lda * 2, (uint64_t)(a_bs == 0 ? (long long)lda * M : a_bs) * 2};
        uint32_t box[3] = {kBK, kBM, 1};
        int rc = make_tmap_bf16(&tmA, a, 3, dims, str, box, true);
        if (rc) return rc;
    }
    {
        uint64_t dims[3] = {(uint64_t)K, (uint64_t)N, (uint64_t)batch};
        uint64_t str[2] = {(uint64_t)ldb * 2, (uint64_t)b_bs * 2};
        uint32_t box[3] = {kBK, BN, 1};
        int rc = make_tmap_bf16(&tmB, b, 3, dims, str, box, true);
        if (rc) return rc;
    }
    constexpr int kAttrKey = BN == 256 ? 0 : (BN == 128 ? 1 : 2);  // per-device function attributes
    if (!device_configured(kAttrKey)) {
        OF3_CUDA_CHECK(cudaFuncSetAttribute(contract_nt_kernel<BN>,
                                            cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            Cfg::kSmemBytes));
        device_mark_configured(kAttrKey);
    }
    const long long tiles = (long long)batch * ceil_div(M, kBM) * ceil_div(N, BN);
    const int grid = (int)(tiles < sm_count() ? tiles : sm_count());
    int* status = device_status_ptr();
    LaunchScope scope(account_as, stream);  // launch accounting: the triangle einsum or a plain linear layer
    contract_nt_kernel<BN><<<grid, 192, Cfg::kSmemBytes, stream>>>(tmA, tmB, out, M, N, K, batch,
                                                                   o_bs, ldo, rows_per_block, row_block_stride,
                                                                   a_bs == 0 ? 1 : 0, status);
    OF3_CUDA_CHECK(cudaGetLastError());
    return OF3_OK;
}

}  // namespace

int contract_nt_bf16(const __nv_bfloat16* a, const __nv_bfloat16* b, __nv_bfloat16* out, int batch,
                     int M, int N, int K, int lda, int ldb, int ldo, long long a_bs, long long b_bs,
                     long long o_bs, cudaStream_t stream, int rows_per_block, long long row_block_stride,
                     int account_as) {
    OF3_REQUIRE(a && b && out, OF3_ERR_ARG, "contract: null pointer");
    OF3_REQUIRE(batch > 0 && M > 0 && N > 0 && K > 0, OF3_ERR_ARG, "contract: non-positive size");
    OF3_REQUIRE(lda % 8 == 0 && ldb % 8 == 0 && ldo % 8 == 0 && a_bs % 8 == 0 && b_bs % 8 == 0 &&
                    o_bs % 8 == 0,
                OF3_ERR_ALIGN, "contract: pitches must be multiples of 8 elements");
    OF3_REQUIRE(ldo >= (int)align_up(N, 8), OF3_ERR_ALIGN, "contract: ldo < round_up(N, 8)");
    OF3_REQUIRE(((uintptr_t)out & 15) == 0, OF3_ERR_ALIGN, "contract: out not 16-byte aligned");
    OF3_REQUIRE(rows_per_block >= 0 && row_block_stride % 8 == 0, OF3_ERR_ALIGN,
                "contract: row block stride must be a multiple of 8 elements");
    if (N > 128)
        return launch_contract<256>(a, b, out, batch, M, N, K, lda, ldb, ldo, a_bs, b_bs, o_bs, rows_per_block,
                                    row_block_stride, stream, account_as);
    return launch_contract<128>(a, b, out, batch, M, N, K, lda, ldb, ldo, a_bs, b_bs, o_bs, rows_per_block,
                                row_block_stride, stream, account_as);
}

}  // namespace of3

// X[b][i][j] = sum_k A[b][i][k] * B[b][j][k]; element pitches lda/ldb/ldo, batch strides in elements.
extern "C" int of3_contract_nt_bf16(const void* a, const void* b, void* out, int batch, int M, int N,
                                    int K, int lda, int ldb, int ldo, long long a_batch_stride,
                                    long long b_batch_stride, long long out_batch_stride,
                                    void* stream) {
    return of3::contract_nt_bf16((const __nv_bfloat16*)a, (const __nv_bfloat16*)b,
                                 (__nv_bfloat16*)out, batch, M, N, K, lda, ldb, ldo, a_batch_stride,
                                 b_batch_stride, out_batch_stride, (cudaStream_t)stream, 0, 0, 1);
}
