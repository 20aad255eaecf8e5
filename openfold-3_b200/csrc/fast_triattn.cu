// Triangle attention, bf16 / tcgen05 family (c_z = 128, 4 heads x 32).
//
//   triattn_proj   z tile -> LayerNorm (in place in the A operand) -> [q|k|v] projection on
//                  tcgen05; the 4-wide triangle-bias projection is a fourth small GEMM. q is
//                  stored pre-scaled by log2(e)/sqrt(d), the bias pre-scaled by log2(e), so the
//                  softmax runs on exp2. Layouts: q, k, v as pre-swizzled operand tiles (see the
//                  epilogue), bias as fp32 tiles [head][key block of 32][q][36].
//   triattn_core   streaming attention for (2 lines, head, 128 queries): S = Q K^T on tcgen05 into
//                  TMEM, online softmax (fp32, exp2) by one thread per query row, P written back
//                  to TMEM as bf16 over S and used from there as the A operand of O += P V; the row
//                  sums of P come out of the same GEMM (a constant row of ones appended to V). Mask
//                  and pair bias are added in fp32; N^3 logits are never materialised.
//   triattn_out    z tile -> LayerNorm -> linear_g (gate recomputed instead of stored), o tile
//                  * sigmoid(gate) -> linear_o -> + z, TMA-stored.
// "line" is the leading index of the (possibly transposed) pair tensor: with kTransposed the
// kernels read and write z through transposed TMA boxes, which gives the ending-node layer
// (and PairBlock's transpose / tri_att_end / transpose) without moving z.
// Reference: openfold3/core/model/layers/triangular_attention.py:102-167,
//            openfold3/core/model/primitives/attention.py:94-135, 270-310.
#include "modules.cuh"
#include "rowtile.cuh"
#include "runtime.cuh"

namespace of3 {
namespace fast {
namespace {

using namespace umma;
using namespace rowtile;

constexpr int kH = 4;
constexpr int kD = 32;
constexpr int kKidProj = 5;
constexpr int kKidCore = 6;
constexpr int kKidOut = 7;
constexpr float kLog2e = 1.4426950408889634f;

struct LineTile {
    int b, line, t0;
};
// R = lines per sample (R == N for a whole pair tensor, N / P for a row shard)
__device__ __forceinline__ LineTile line_tile(long long t, int R, int tiles_per_line) {
    LineTile c;
    c.t0 = (int)(t % tiles_per_line) * kRows;
    const long long l = t / tiles_per_line;
    c.line = (int)(l % R);
    c.b = (int)(l / R);
    return c;
}
// z tile of a line: rows (line, t0..t0+127) of the view; transposed view = z[b, t, line, :]
template <bool kTransposed>
__device__ __forceinline__ void load_z_tile(uint32_t dst, const CUtensorMap* tm, uint32_t bar,
                                            const LineTile& c, int R) {
    for (int kb = 0; kb < 2; ++kb) {
        if (kTransposed)
            tma_load_4d(dst + kb * kKBlockBytes, tm, bar, kb * 64, c.line, c.t0, c.b);
        else
            tma_load_3d(dst + kb * kKBlockBytes, tm, bar, kb * 64, c.t0, c.b * R + c.line);
    }
}

// =====================================================================================
// triattn_proj
// =====================================================================================
struct ProjSmem {
    static constexpr uint32_t kWKb = 384 * 128;               // one k-block of [q|k|v]: 49152
    static constexpr uint32_t kW = 0;
    static constexpr uint32_t kZ = 2 * kWKb;                  // 2 stages x 32768
    static constexpr uint32_t kGamma = kZ + 2 * kTileBytes;
    static constexpr uint32_t kBeta = kGamma + 512;
    static constexpr uint32_t kWb = kBeta + 512;              // bias weight as a B operand: 2 k-blocks x [16 x 128 B]
    static constexpr uint32_t kBars = kWb + 4096;
    static constexpr uint32_t kTotal = kBars + 128;
    static constexpr uint32_t kDyn = kTotal + 1024;
};

// warps: 0 producer, 1 MMA issuer, 2..5 LayerNorm (one thread per row), 6..9 epilogue (TMEM slot 0: q, k;
// slot 1: v and the 4-wide triangle bias). The bias projection is a fourth GEMM (N = 16 with 12 zero rows)
// instead of 1024 FMAs per row inside the LayerNorm pass.
constexpr int kProjThreads = 320;
constexpr int kBiasK = 32;  // keys per bias row = keys per attention step
// Pair-bias image: bf16, pre-scaled by log2(e), [b*4 + head][key block of 32][query row][32 keys]: the 128 rows
// of a query tile and one key block are contiguous (one untiled bulk copy) and each 64-byte row is stored in the
// 64-byte swizzle of a K-major tcgen05 A operand (16-byte chunk c of query row q at chunk c ^ ((q / 2) % 4)),
// because the attention kernel adds the bias on the tensor pipe: S += bias_tile * I_32^T.

template <bool kTransposed>
__global__ void __launch_bounds__(kProjThreads, 1)
triattn_proj_kernel(const __grid_constant__ CUtensorMap tmZ, const __grid_constant__ CUtensorMap tmWq,
                    const __grid_constant__ CUtensorMap tmWk, const __grid_constant__ CUtensorMap tmWv,
                    const __grid_constant__ CUtensorMap tmWb,
                    const __nv_bfloat16* __restrict__ ln_w, const __nv_bfloat16* __restrict__ ln_b,
                    __nv_bfloat16* __restrict__ q_out,
                    __nv_bfloat16* __restrict__ k_out, __nv_bfloat16* __restrict__ vt_out,
                    __nv_bfloat16* __restrict__ tb_out, int B, int R, int N, int npad, int row0, int* status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gbase = smem_raw + (sbase - smem_u32(smem_raw));
    float* gamma = reinterpret_cast<float*>(gbase + ProjSmem::kGamma);
    float* beta = reinterpret_cast<float*>(gbase + ProjSmem::kBeta);
    const uint32_t bars = sbase + ProjSmem::kBars;
    const uint32_t w_full = bars;
    auto z_full = [&](int s) { return bars + 8u * (1 + s); };
    auto z_empty = [&](int s) { return bars + 8u * (3 + s); };
    auto a_ready = [&](int s) { return bars + 8u * (5 + s); };
    auto slot_full = [&](int q) { return bars + 8u * (7 + q); };
    auto slot_empty = [&](int q) { return bars + 8u * (9 + q); };
    volatile uint32_t* tmem_ptr = reinterpret_cast<volatile uint32_t*>(gbase + ProjSmem::kBars + 96);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + ProjSmem::kBars + 104);

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
    // TMEM: slot 0 = [q|k] columns [0,256), slot 1 = v columns [256,384) + triangle bias [384,400)

    if (warp == 0) {
        if (lane == 0) {
            mbar_arrive_expect_tx(w_full, 2 * ProjSmem::kWKb + 4096);
            const CUtensorMap* wm[3] = {&tmWq, &tmWk, &tmWv};
            for (int w = 0; w < 3; ++w)
                for (int kb = 0; kb < 2; ++kb)
                    tma_load_2d(sbase + ProjSmem::kW + kb * ProjSmem::kWKb + w * 128 * 128, wm[w], w_full,
                                kb * 64, 0);
            // rows 4..15 of the box lie outside the [4 x 128] weight: the copy fills them with zeros
            for (int kb = 0; kb < 2; ++kb) tma_load_2d(sbase + ProjSmem::kWb + kb * 2048, &tmWb, w_full, kb * 64, 0);
            uint32_t it = 0;
            for (long long t = blockIdx.x; t < num_tiles; t += gridDim.x, ++it) {
                const int s = it & 1;
                if (!mbar_wait(z_empty(s), ((it >> 1) & 1u) ^ 1u, abort_flag)) {
                    report_wait_failure(status, abort_flag, kKidProj, 1);
                    break;
                }
                const LineTile tc = line_tile(t, R, tiles_per_line);
                mbar_arrive_expect_tx(z_full(s), kTileBytes);
                load_z_tile<kTransposed>(sbase + ProjSmem::kZ + s * kTileBytes, &tmZ, z_full(s), tc, R);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = mbar_wait(w_full, 0, abort_flag);
            if (!ok) report_wait_failure(status, abort_flag, kKidProj, 2);
            uint32_t it = 0;
            for (long long t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
                const int s = it & 1;
                if (!mbar_wait(a_ready(s), (it >> 1) & 1u, abort_flag)) {
                    report_wait_failure(status, abort_flag, kKidProj, 3);
                    break;
                }
                for (int q = 0; q < 2; ++q) {
                    if (!mbar_wait(slot_empty(q), (it & 1u) ^ 1u, abort_flag)) {
                        report_wait_failure(status, abort_flag, kKidProj, 4);
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    mma_k128(tmem_base + q * 256, sbase + ProjSmem::kZ + s * kTileBytes,
                             sbase + ProjSmem::kW + q * 256 * 128, ProjSmem::kWKb,
                             q == 0 ? idesc_bf16_f32(128, 256) : idesc_bf16_f32(128, 128), false);
                    if (q == 1)
                        mma_k128(tmem_base + 384, sbase + ProjSmem::kZ + s * kTileBytes, sbase + ProjSmem::kWb, 2048,
                                 idesc_bf16_f32(128, 16), false);
                    mma_commit(slot_full(q));
                }
                if (ok) mma_commit(z_empty(s));
            }
        }
    } else if (warp < 6) {
        // LayerNorm warps: normalise in place (the A operand of all four GEMMs)
        const int row = (warp - 2) * 32 + lane;
        uint32_t it = 0;
        for (long long t = blockIdx.x; t < num_tiles; t += gridDim.x, ++it) {
            const int s = it & 1;
            if (!mbar_wait(z_full(s), (it >> 1) & 1u, abort_flag)) {
                if (lane == 0) report_wait_failure(status, abort_flag, kKidProj, 5);
                break;
            }
            const uint32_t tile = sbase + ProjSmem::kZ + s * kTileBytes;
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
        // epilogue warps
        const int quad = warp & 3;
        const int row = quad * 32 + lane;
        const float qscale = kLog2e * rsqrtf((float)kD);
        uint32_t it = 0;
        bool ok = true;
        for (long long t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
            const LineTile tc = line_tile(t, R, tiles_per_line);
            const int pos = tc.t0 + row;
            const bool valid = pos < npad;   // positions in [N, npad) are written as zeros (key padding)
            const bool live = pos < N;
            // Images are tile-major with the line inside the tile index, so the tiles of four consecutive
            // lines (one attention CTA) are contiguous and arrive with ONE bulk copy:
            //   q [b][h][query tile of 128][line < rpad][128][32]
            //   k [b][h][key block of 32 ][line < rpad][32][32]      v likewise with [32 d][32 keys]
            const int rpad = (R + 3) & ~3;
            const int nkb = npad >> 5;
            // ---- slot 0: q (columns 0..127) and k (128..255), [line][head][pos][32], stored as the
            // 64-byte-swizzled shared-memory image (16-byte chunk c of row pos at chunk c ^ ((pos/2)%4)),
            // so that the attention kernel fetches whole tiles with one untiled bulk copy each
            const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16);
            if (!mbar_wait(slot_full(0), it & 1u, abort_flag)) {
                if (lane == 0) report_wait_failure(status, abort_flag, kKidProj, 6);
                break;
            }
            tc_fence_after_sync();
#pragma unroll 1
            for (int qk = 0; qk < 2; ++qk) {
                __nv_bfloat16* base = qk == 0 ? q_out : k_out;
                const float sc = qk == 0 ? qscale : 1.0f;
#pragma unroll 1
                for (int h = 0; h < kH; ++h) {
                    uint32_t r[32];
                    tmem_ld32(taddr + qk * 128 + h * 32, r);
                    tmem_ld_wait();
                    if (valid || qk == 0) {
                        const long long bh = (long long)tc.b * kH + h;
                        const long long rowidx = qk == 0
                            ? ((bh * tiles_per_line + (pos >> 7)) * rpad + tc.line) * 128 + (pos & 127)
                            : ((bh * nkb + (pos >> 5)) * rpad + tc.line) * 32 + (pos & 31);
                        uint4* dst = reinterpret_cast<uint4*>(base + rowidx * kD);
                        const float sl = live ? sc : 0.f;
#pragma unroll
                        for (int v4 = 0; v4 < 4; ++v4) {
                            uint4 v;
                            v.x = pack_bf16x2(sl * __uint_as_float(r[v4 * 8 + 0]), sl * __uint_as_float(r[v4 * 8 + 1]));
                            v.y = pack_bf16x2(sl * __uint_as_float(r[v4 * 8 + 2]), sl * __uint_as_float(r[v4 * 8 + 3]));
                            v.z = pack_bf16x2(sl * __uint_as_float(r[v4 * 8 + 4]), sl * __uint_as_float(r[v4 * 8 + 5]));
                            v.w = pack_bf16x2(sl * __uint_as_float(r[v4 * 8 + 6]), sl * __uint_as_float(r[v4 * 8 + 7]));
                            dst[v4 ^ ((pos >> 1) & 3)] = v;
                        }
                    }
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(slot_empty(0));
            // ---- slot 1: v, stored as tiles [line][head][key block of 32][32 d][32 keys], each tile the
            // 64-byte-swizzled image of the K-major B operand of P V (row d, chunk (key%32)/8)
            if (!mbar_wait(slot_full(1), it & 1u, abort_flag)) {
                if (lane == 0) report_wait_failure(status, abort_flag, kKidProj, 7);
                ok = false;
                break;
            }
            tc_fence_after_sync();
#pragma unroll 1
            for (int h = 0; h < kH; ++h) {
                uint32_t r[32];
                tmem_ld32(taddr + 256 + h * 32, r);
                tmem_ld_wait();
                if (valid) {
                    __nv_bfloat16* tile =
                        vt_out + (((((long long)tc.b * kH + h) * nkb + (pos >> 5)) * rpad + tc.line) << 10);
                    const int c = (pos & 31) >> 3, w = pos & 7;
#pragma unroll
                    for (int e = 0; e < 32; ++e)
                        tile[e * 32 + (((c ^ ((e >> 1) & 3)) << 3) | w)] =
                            __float2bfloat16_rn(live ? __uint_as_float(r[e]) : 0.f);
                }
            }
            uint32_t tbr[16];  // triangle bias of this position: columns 384..387, pre-scaled for exp2
            tmem_ld16(taddr + 384, tbr);
            tmem_ld_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(slot_empty(1));
            if (valid) {  // key padding [N, npad) is read by the attention kernel: zeros
                // row0 = index of this shard's first line among all query rows (the swizzle follows the global row)
                const int kc = (((pos & 31) >> 3) ^ (((row0 + tc.line) >> 1) & 3)) * 8 + (pos & 7);
#pragma unroll
                for (int h = 0; h < kH; ++h)
                    tb_out[((((long long)tc.b * kH + h) * nkb + (pos >> 5)) * R + tc.line) * kBiasK + kc] =
                        __float2bfloat16_rn(live ? __uint_as_float(tbr[h]) * kLog2e : 0.f);
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
// triattn_core
// =====================================================================================
// One CTA = one head, 128 queries and TWO lines of the pair tensor, 32 keys per step; two CTAs share an SM
// (their prologues, epilogues and waits interleave). Per line and step j:
//   MMA warp      S_j = Q K_j^T + Tb_j I^T into one of two TMEM slots: 128 x 32 logits, K = 32, and the pair-bias
//                 tile [128 q x 32 k] (bf16, shared by both lines) as a second A operand against a 32 x 32
//                 identity, so the tensor pipe adds the bias (a bf16 value times 1.0 accumulated in fp32 is exact)
//                 and the softmax threads never touch it. S_{j+2} is issued as soon as P_j V_j, which reads P_j
//                 out of the same slot, is done: a whole step before the softmax warps want it.
//   softmax warps thread = query row = TMEM lane: S -> registers [+ mask bias where the block has masked keys],
//                 row maximum, P = exp2(S - m), rounded to bf16 and written over S (the first 16 columns of the
//                 slot, bf16 pairs)
//   MMA warp      O[128 x 48] += P [V; 1; 0] with P read from TMEM as the A operand: columns 0..31 are the head's
//                 channels, column 32 -- a row of ones under the V tile in shared memory -- is the row sum of the
//                 rounded P. A GEMM of N = 48 occupies the tensor pipe no longer than one of N = 32, and the
//                 softmax threads keep no running sum.
// TMEM columns of a line (112 of 128): S / P slots [0,32) [32,64), O [64,112).
// The running maximum m used for scaling is only raised when the row maximum exceeds it by more than 8
// (2^8 head room in P): then, and only then, the thread rescales its O row (channels and row sum) in TMEM.
// The result is exact: numerator and denominator always share one scale.
constexpr int kBQ = 128;      // queries per CTA
constexpr int kBK = 32;       // keys per step
constexpr int kMaxKeys = 2048;   // one CTA keeps a mask-bias row per line in shared memory
constexpr int kKbStages = 4;     // ring of K tiles + bias tile (read by S_j, two steps ahead of the softmax)
constexpr int kVStages = 4;      // ring of V tiles (read by P_j V_j)
constexpr int kLines = 2;     // lines per CTA
constexpr int kLinePad = 4;   // the operand images pad the line count of a sample to a multiple of this
constexpr int kCoreThreads = 32 * (1 + kLines + 4 * kLines);  // producer, one MMA warp per line, softmax
constexpr float kRescaleThreshold = 8.0f;
constexpr uint32_t kTbTileBytes = kBQ * kBiasK * 2;    // 8192
constexpr uint32_t kVSlot = 3072;                      // V tile [32 d][32 keys] + a row of ones + 15 unused rows
constexpr int kON = 48;                                // N of the P V GEMM: 32 output channels, the row sum, padding
constexpr uint32_t kColO = 64;                         // O [64, 112): 32 channels, column 32 = sum of the row's P

struct CoreSmem {
    static constexpr uint32_t kQ = 0;                                   // lines x 8 KB
    static constexpr uint32_t kK = kQ + kLines * 8192;                  // stages x lines x 2 KB
    static constexpr uint32_t kTb = kK + kKbStages * kLines * 2048;     // stages x 8 KB: bias tiles [128 q][32 k] bf16
    static constexpr uint32_t kV = kTb + kKbStages * kTbTileBytes;      // stages x lines x 3 KB
    static constexpr uint32_t kIdent = kV + kVStages * kLines * kVSlot; // 2 KB: 32 x 32 identity (B operand)
    static constexpr uint32_t kBars = kIdent + 2048;
    static constexpr uint32_t kFlags = kBars + 320;                     // lines x 128 block flags (bytes)
    static constexpr uint32_t kMb = kFlags + kLines * 128;              // lines x nkeys_pad floats
    static uint32_t dyn_bytes(int nblk) { return kMb + kLines * nblk * kBK * 4 + 1024; }
};

template <bool kTransposed>
__global__ void __launch_bounds__(kCoreThreads, 2)
triattn_core_kernel(const __nv_bfloat16* __restrict__ q_img, const __nv_bfloat16* __restrict__ k_img,
                    const __nv_bfloat16* __restrict__ v_img, const __nv_bfloat16* __restrict__ tb_img,
                    const __nv_bfloat16* __restrict__ mask, __nv_bfloat16* __restrict__ o_out, int B,
                    int R, int N, int npad, float inf, int* status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gbase = smem_raw + (sbase - smem_u32(smem_raw));
    float* mbs = reinterpret_cast<float*>(gbase + CoreSmem::kMb);
    volatile uint8_t* mbflag = gbase + CoreSmem::kFlags;
    const uint32_t bars = sbase + CoreSmem::kBars;
    const uint32_t q_full = bars;
    auto kb_full = [&](int s) { return bars + 8u * (1 + s); };
    auto kb_empty = [&](int s) { return bars + 8u * (1 + kKbStages + s); };
    constexpr int kB1 = 1 + 2 * kKbStages;
    auto v_full = [&](int s) { return bars + 8u * (kB1 + s); };
    auto v_empty = [&](int s) { return bars + 8u * (kB1 + kVStages + s); };
    constexpr int kB2 = kB1 + 2 * kVStages;
    auto s_full = [&](int L, int s) { return bars + 8u * (kB2 + L * 2 + s); };
    auto p_ready = [&](int L, int s) { return bars + 8u * (kB2 + 2 * kLines + L * 2 + s); };
    auto pv_done = [&](int L, int s) { return bars + 8u * (kB2 + 4 * kLines + L * 2 + s); };
    constexpr int kNumBars = kB2 + 6 * kLines;
    static_assert(8 * kNumBars + 16 <= 320, "barrier block");
    volatile uint32_t* tmem_ptr = reinterpret_cast<volatile uint32_t*>(gbase + CoreSmem::kBars + 8 * kNumBars);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + CoreSmem::kBars + 8 * kNumBars + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_qt = (N + kBQ - 1) / kBQ;
    const int groups_per_b = (R + kLines - 1) / kLines;
    const int qt = blockIdx.x % n_qt;
    const int h = (blockIdx.x / n_qt) % kH;
    const int lg = blockIdx.x / (n_qt * kH);
    const int b = lg / groups_per_b;
    const int line0 = (lg % groups_per_b) * kLines;
    const int q0 = qt * kBQ;
    const int nblk = (N + kBK - 1) / kBK;
    const int nkp = nblk * kBK;
    // lines past the end of the sample recompute the first line of the group and are not stored
    auto line_of = [&](int L) { return (line0 + L < R) ? line0 + L : line0; };

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < kKbStages; ++s) {
            mbar_init(kb_full(s), 1);
            mbar_init(kb_empty(s), 4 * kLines);  // every softmax warp has read the S that consumed the stage
        }
        for (int s = 0; s < kVStages; ++s) {
            mbar_init(v_full(s), 1);
            mbar_init(v_empty(s), kLines);       // each line's commit after the P V that read the stage
        }
        for (int L = 0; L < kLines; ++L) {
            for (int s = 0; s < 2; ++s) {
                mbar_init(s_full(L, s), 1);
                mbar_init(p_ready(L, s), 4);
                mbar_init(pv_done(L, s), 1);
            }
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    // 32 x 32 identity, bf16, K-major with the 64-byte swizzle: element (n, n) of row n
    for (int idx = threadIdx.x; idx < 32 * 16; idx += blockDim.x) {
        const int n = idx >> 4, w = idx & 15;  // row, 32-bit word of the row (2 elements)
        const int k = w * 2;                   // first element of the word
        uint32_t v = 0;
        if (k == n) v = 0x00003F80u;
        if (k + 1 == n) v = 0x3F800000u;
        const int chunk = (k >> 3) ^ ((n >> 1) & 3);
        *reinterpret_cast<uint32_t*>(gbase + CoreSmem::kIdent + n * 64 + chunk * 16 + (w & 3) * 4) = v;
    }
    // rows 32..47 of every V slot: a row of ones (column 32 of O then accumulates the row sum of P on the tensor
    // pipe, rounded exactly like the numerator) and 15 rows of zeros; the bulk copies only ever write rows 0..31
    for (int idx = threadIdx.x; idx < kVStages * kLines * 64; idx += blockDim.x) {
        const int slot = idx >> 6, w = idx & 63;   // 64 uint4 = 1 KB per slot
        const uint32_t v = (w < 4) ? 0x3F803F80u : 0u;
        *reinterpret_cast<uint4*>(gbase + CoreSmem::kV + slot * kVSlot + 2048 + w * 16) = make_uint4(v, v, v, v);
    }
    fence_proxy_async_smem();
    if (warp == 1) {
        tmem_alloc(smem_u32((const void*)tmem_ptr), kLines * 128);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();  // the only CTA-wide barrier before the teardown: the copies and GEMMs start right behind it
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_ptr;

    if (warp == 0) {
        if (lane == 0) {
            const int nkb = npad / kBK;
            const int rpad = (R + kLinePad - 1) / kLinePad * kLinePad;
            const long long bh = (long long)b * kH + h;
            mbar_arrive_expect_tx(q_full, kLines * kBQ * 64);
            bulk_load(sbase + CoreSmem::kQ, q_img + (((bh * n_qt + qt) * rpad + line0) * kBQ) * kD, kLines * kBQ * 64,
                      q_full);
            const int q_rows = (N - q0 < kBQ) ? N - q0 : kBQ;  // rows of the bias tile that exist
            const uint32_t tb_bytes = (uint32_t)q_rows * kBiasK * 2;
            for (int j = 0; j < nblk; ++j) {
                const long long tile0 = ((bh * nkb + j) * rpad + line0) << 10;  // first of the lines' tiles
                {   // K tiles of both lines + the pair-bias tile of key block j (shared by the lines)
                    const int s = j % kKbStages;
                    if (!mbar_wait(kb_empty(s), ((j / kKbStages) & 1u) ^ 1u, abort_flag)) {
                        report_wait_failure(status, abort_flag, kKidCore, 1);
                        break;
                    }
                    mbar_arrive_expect_tx(kb_full(s), kLines * 2048 + tb_bytes);
                    bulk_load(sbase + CoreSmem::kK + s * kLines * 2048, k_img + tile0, kLines * 2048, kb_full(s));
                    bulk_load(sbase + CoreSmem::kTb + s * kTbTileBytes,
                              tb_img + ((bh * nkb + j) * (long long)N + q0) * kBiasK, tb_bytes, kb_full(s));
                }
                {   // V tiles
                    const int s = j % kVStages;
                    if (!mbar_wait(v_empty(s), ((j / kVStages) & 1u) ^ 1u, abort_flag)) {
                        report_wait_failure(status, abort_flag, kKidCore, 11);
                        break;
                    }
                    mbar_arrive_expect_tx(v_full(s), kLines * 2048);
                    for (int L = 0; L < kLines; ++L)
                        bulk_load(sbase + CoreSmem::kV + (s * kLines + L) * kVSlot, v_img + tile0 + L * 1024, 2048,
                                  v_full(s));
                }
            }
        }
    } else if (warp <= kLines) {
        // ---------------------------------------------------------------- one MMA-issuing warp per line
        // The whole warp walks the loop and lane 0 issues: with warp-uniform control flow and operands (the
        // shuffles tell the compiler so) descriptors and addresses live in uniform registers, instead of being
        // moved there one by one in front of every tcgen05.mma of a single-lane loop.
        const int L = __shfl_sync(0xffffffffu, warp, 0) - 1;
        const uint32_t tm = __shfl_sync(0xffffffffu, tmem_base, 0);
        const uint32_t sb = __shfl_sync(0xffffffffu, sbase, 0);
        constexpr uint32_t idesc_s = idesc_bf16_f32(128, kBK);  // S: 128 x 32, K = 32
        constexpr uint32_t idesc_o = idesc_bf16_f32(128, kON);  // O: 128 x 48 (channels, row sum, padding), K = 32
        bool ok = mbar_wait(q_full, 0, abort_flag);
        if (!ok && lane == 0) report_wait_failure(status, abort_flag, kKidCore, 2);
        const uint64_t qdesc = smem_desc_k_sw64(sb + CoreSmem::kQ + L * 8192);
        const uint64_t identdesc = smem_desc_k_sw64(sb + CoreSmem::kIdent);
        const uint32_t t_line = tm + L * 128;
        // S_i = Q K_i^T + Tb_i into slot i % 2, free once P_{i-2} V_{i-2} (which read P out of it) is done
        auto issue_s = [&](int i) -> bool {
            const int s = i & 1;
            const int ks = i % kKbStages;
            if (i >= 2 && !mbar_wait(pv_done(L, s), ((i - 2) >> 1) & 1u, abort_flag)) {
                if (lane == 0) report_wait_failure(status, abort_flag, kKidCore, 4);
                return false;
            }
            if (!mbar_wait(kb_full(ks), (i / kKbStages) & 1u, abort_flag)) {
                if (lane == 0) report_wait_failure(status, abort_flag, kKidCore, 3);
                return false;
            }
            tc_fence_after_sync();
            const uint64_t kdesc = smem_desc_k_sw64(sb + CoreSmem::kK + (ks * kLines + L) * 2048);
            const uint64_t tbdesc = smem_desc_k_sw64(sb + CoreSmem::kTb + ks * kTbTileBytes);
            const uint32_t d = t_line + s * kBK;
            if (lane == 0) {
                mma_bf16(d, qdesc, kdesc, idesc_s, 0u);
                mma_bf16(d, qdesc + 2u, kdesc + 2u, idesc_s, 1u);
                mma_bf16(d, tbdesc, identdesc, idesc_s, 1u);            // + pair bias
                mma_bf16(d, tbdesc + 2u, identdesc + 2u, idesc_s, 1u);
                mma_commit(s_full(L, s));
            }
            __syncwarp();
            return true;
        };
        ok = ok && issue_s(0);
        if (ok && nblk > 1) ok = issue_s(1);
        for (int j = 0; j < nblk && ok; ++j) {
            // O += P_j V_j at the end of step j, then S_{j+2} into the slot P_j was read from
            const int vs = j % kVStages;
            if (!mbar_wait(v_full(vs), (j / kVStages) & 1u, abort_flag)) {
                if (lane == 0) report_wait_failure(status, abort_flag, kKidCore, 12);
                break;
            }
            if (!mbar_wait(p_ready(L, j & 1), (j >> 1) & 1u, abort_flag)) {
                if (lane == 0) report_wait_failure(status, abort_flag, kKidCore, 5);
                break;
            }
            tc_fence_after_sync();
            const uint64_t vdesc = smem_desc_k_sw64(sb + CoreSmem::kV + (vs * kLines + L) * kVSlot);
            if (lane == 0) {
                const uint32_t a_p = t_line + (j & 1) * kBK;
                mma_bf16_ts(t_line + kColO, a_p, vdesc, idesc_o, j != 0 ? 1u : 0u);
                mma_bf16_ts(t_line + kColO, a_p + 8u, vdesc + 2u, idesc_o, 1u);
                mma_commit(pv_done(L, j & 1));
                mma_commit(v_empty(vs));
            }
            __syncwarp();
            if (j + 2 < nblk && !issue_s(j + 2)) break;
        }
    } else {
        // ---------------------------------------------------------------- softmax warpgroups
        const int L = (warp - 1 - kLines) >> 2;
        const int quad = warp & 3;
        const int row = quad * 32 + lane;
        const int qpos = q0 + row;
        const bool line_valid = line0 + L < R;
        const long long bl = (long long)b * R + line_of(L);
        const uint32_t trow = tmem_base + ((uint32_t)(quad * 32) << 16) + L * 128;
        float* mbl = mbs + L * nkp;
        // Additive key mask of this line, pre-scaled for exp2: inf * (mask - 1) * log2(e), -inf beyond N. The four
        // warps of the line prepare it for themselves (eight keys per thread and pass, the loads of a pass
        // independent of each other) while the first copies and GEMMs are already under way.
        {
            const int gt = (warp - 1 - kLines - 4 * L) * 32 + lane;  // 0..127 within the line's warps
            const int line = line_of(L);
            for (int base = 0; base < nkp; base += 128 * 8) {   // warp-uniform trip count (ballot below)
                const int c0 = base + gt * 8;
                const bool active = c0 < nkp;
                float v[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const int k = c0 + e;
                    float m = 1.0f;
                    if (mask != nullptr && k < N) {
                        const long long mi = kTransposed ? ((long long)b * N + k) * N + line
                                                         : ((long long)b * R + line) * N + k;
                        m = __bfloat162float(mask[mi]);
                    }
                    v[e] = (k < N) ? inf * (m - 1.0f) * kLog2e : -INFINITY;
                }
                bool any = false;
#pragma unroll
                for (int e = 0; e < 8; ++e) any |= (v[e] != 0.f);
                if (active) {
                    *reinterpret_cast<float4*>(mbl + c0) = make_float4(v[0], v[1], v[2], v[3]);
                    *reinterpret_cast<float4*>(mbl + c0 + 4) = make_float4(v[4], v[5], v[6], v[7]);
                }
                // a key block of 32 = four consecutive threads: does any of its keys carry a non-zero bias?
                const unsigned bal = __ballot_sync(0xffffffffu, any);
                if (active && (lane & 3) == 0) mbflag[L * 128 + (c0 >> 5)] = ((bal >> lane) & 0xFu) ? 1 : 0;
            }
            group_sync(1 + L, 128);
        }
        unsigned long long mflags = 0ull;  // bit j: key block j of this line has a masked (or padding) key
        {
            const unsigned lo = __ballot_sync(0xffffffffu, lane < nblk && mbflag[L * 128 + lane]);
            const unsigned hi = __ballot_sync(0xffffffffu, lane + 32 < nblk && mbflag[L * 128 + 32 + lane]);
            mflags = ((unsigned long long)hi << 32) | lo;
        }
        float m_used = 0.f;
        bool ok = true;
        for (int j = 0; j < nblk && ok; ++j) {
            const int s = j & 1;
            if (!mbar_wait(s_full(L, s), (j >> 1) & 1u, abort_flag)) {
                if (lane == 0) report_wait_failure(status, abort_flag, kKidCore, 7);
                ok = false;
                break;
            }
            tc_fence_after_sync();
            uint32_t sr[32];
            tmem_ld32(trow + s * kBK, sr);
            tmem_ld_wait();
            // S_j is in registers: the K / bias stage its GEMM read can be refilled
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(kb_empty(j % kKbStages));
            float sv[kBK];
#pragma unroll
            for (int e = 0; e < 32; ++e) sv[e] = __uint_as_float(sr[e]);
            // + mask bias (blocks without a masked key skip it): (q.k + pair bias) + inf * (mask - 1); a masked
            // key ends at the same -1.44e9 in either order of the two additions, an unmasked one adds exactly 0
            if ((mflags >> j) & 1ull) {
                const int k0 = j * kBK;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float4 mb = *reinterpret_cast<const float4*>(mbl + k0 + i * 4);
                    sv[i * 4] += mb.x;
                    sv[i * 4 + 1] += mb.y;
                    sv[i * 4 + 2] += mb.z;
                    sv[i * 4 + 3] += mb.w;
                }
            }
            float mx0 = max3(sv[0], sv[1], sv[2]), mx1 = max3(sv[3], sv[4], sv[5]);
#pragma unroll
            for (int e = 6; e < 30; e += 4) {
                mx0 = max3(mx0, sv[e], sv[e + 1]);
                mx1 = max3(mx1, sv[e + 2], sv[e + 3]);
            }
            const float mx = max3(mx0, mx1, fmaxf(sv[30], sv[31]));
            bool rescale = false;
            if (j == 0) {
                m_used = mx;  // finite: block 0 always holds a key < N, masked keys are -1e9-ish, not -inf
            } else {
                rescale = __any_sync(0xffffffffu, mx - m_used > kRescaleThreshold);
            }
            if (rescale) {
                float f = 1.0f;
                if (mx - m_used > kRescaleThreshold) {
                    f = ex2_approx(m_used - mx);
                    m_used = mx;
                }
                // every P V issued so far must have landed in O before it is rescaled
                if (!mbar_wait(pv_done(L, (j - 1) & 1), ((j - 1) >> 1) & 1u, abort_flag)) {
                    if (lane == 0) report_wait_failure(status, abort_flag, kKidCore, 8);
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                uint32_t orow[32];
                tmem_ld32(trow + kColO, orow);
                const uint32_t lsum = tmem_ld1(trow + kColO + 32);   // the row sum rides in column 32 of O
                tmem_ld_wait();
#pragma unroll
                for (int e = 0; e < 32; ++e) orow[e] = __float_as_uint(__uint_as_float(orow[e]) * f);
                tmem_st32(trow + kColO, orow);
                tmem_st1(trow + kColO + 32, __float_as_uint(__uint_as_float(lsum) * f));
                tmem_st_wait();
            }
            uint32_t pk[16];
            const float nm = -m_used;
#pragma unroll
            for (int e = 0; e < 32; e += 2) {
                add2(sv[e], sv[e + 1], nm, nm);
                pk[e >> 1] = pack_bf16x2(ex2_approx(sv[e]), ex2_approx(sv[e + 1]));
            }
            // P_j goes where S_j was (every thread of the warp has its S row in registers: the load above is
            // warp-wide); the row sum is taken by the tensor pipe from the rounded P (the ones row of the V tile)
            tmem_st16(trow + s * kBK, pk);
            tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_ready(L, s));
        }
        if (ok) {
            if (mbar_wait(pv_done(L, (nblk - 1) & 1), ((nblk - 1) >> 1) & 1u, abort_flag)) {
                tc_fence_after_sync();
                uint32_t r[32];
                tmem_ld32(trow + kColO, r);
                const uint32_t lsum = tmem_ld1(trow + kColO + 32);
                tmem_ld_wait();
                const float inv = 1.0f / __uint_as_float(lsum);
                if (qpos < N && line_valid) {
                    uint4* dst = reinterpret_cast<uint4*>(o_out + ((bl * N + qpos) * (long long)kC) + h * kD);
#pragma unroll
                    for (int v4 = 0; v4 < 4; ++v4) {
                        float fo[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) fo[e] = __uint_as_float(r[v4 * 8 + e]) * inv;
                        dst[v4] = make_uint4(pack_bf16x2(fo[0], fo[1]), pack_bf16x2(fo[2], fo[3]),
                                             pack_bf16x2(fo[4], fo[5]), pack_bf16x2(fo[6], fo[7]));
                    }
                }
            } else if (lane == 0) {
                report_wait_failure(status, abort_flag, kKidCore, 10);
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kLines * 128);
    }
}

// =====================================================================================
// triattn_out
// =====================================================================================
struct AOutSmem {
    static constexpr uint32_t kWg = 0;
    static constexpr uint32_t kWo = kTileBytes;
    static constexpr uint32_t kZ = 2 * kTileBytes;            // 2 groups: z tile, then output
    static constexpr uint32_t kO = kZ + 2 * kTileBytes;       // 2 groups: o tile, gated in place
    static constexpr uint32_t kParams = kO + 2 * kTileBytes;  // gamma, beta
    static constexpr uint32_t kXch = kParams + 1024;          // 2 groups x 512 floats: LayerNorm partial sums
    static constexpr uint32_t kBars = kXch + 4096;
    static constexpr uint32_t kTotal = kBars + 160;
    static constexpr uint32_t kDyn = kTotal + 1024;
};

// producer, MMA issuer, 2 groups x 8 warps: a group alternates tiles with the other one; inside a group two threads
// share a row (TMEM lane), each with 64 of its 128 channels through LayerNorm, gating and the output pass
constexpr int kAOutThreads = 32 * (2 + 2 * 8);

template <bool kTransposed>
__global__ void __launch_bounds__(kAOutThreads, 1)
triattn_out_kernel(const __grid_constant__ CUtensorMap tmZ, const __grid_constant__ CUtensorMap tmO,
                   const __grid_constant__ CUtensorMap tmOut, const __grid_constant__ CUtensorMap tmWg,
                   const __grid_constant__ CUtensorMap tmWo, const __nv_bfloat16* __restrict__ ln_w,
                   const __nv_bfloat16* __restrict__ ln_b, int B, int R, int N, int add_residual, int* status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gbase = smem_raw + (sbase - smem_u32(smem_raw));
    float* prm = reinterpret_cast<float*>(gbase + AOutSmem::kParams);
    const uint32_t bars = sbase + AOutSmem::kBars;
    const uint32_t w_full = bars;
    // The z buffer is free once the gate GEMM has read it (the result goes over the o buffer), so the next
    // z tile is fetched while this one is still being gated and projected; the o buffer is free once the output
    // store has read it, and its next tile lands during the next LayerNorm + gate GEMM.
    auto z_full = [&](int g) { return bars + 8u * (1 + g); };
    auto o_empty = [&](int g) { return bars + 8u * (3 + g); };
    auto o_full = [&](int g) { return bars + 8u * (13 + g); };
    auto z_empty = [&](int g) { return bars + 8u * (15 + g); };
    auto a1_ready = [&](int g) { return bars + 8u * (5 + g); };
    auto g_full = [&](int g) { return bars + 8u * (7 + g); };
    auto a2_ready = [&](int g) { return bars + 8u * (9 + g); };
    auto d_full = [&](int g) { return bars + 8u * (11 + g); };
    volatile uint32_t* tmem_ptr = reinterpret_cast<volatile uint32_t*>(gbase + AOutSmem::kBars + 144);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + AOutSmem::kBars + 148);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_per_line = (N + kRows - 1) / kRows;
    const long long num_tiles = (long long)B * R * tiles_per_line;
    const long long my_tiles = (num_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x;

    if (threadIdx.x == 0) {
        mbar_init(w_full, 1);
        for (int g = 0; g < 2; ++g) {
            mbar_init(z_full(g), 1);
            mbar_init(o_full(g), 1);
            mbar_init(z_empty(g), 1);
            mbar_init(o_empty(g), 1);
            mbar_init(a1_ready(g), 8);
            mbar_init(g_full(g), 1);
            mbar_init(a2_ready(g), 8);
            mbar_init(d_full(g), 1);
        }
        *abort_flag = 0;
        mbar_fence_init();
        prefetch_tmap(&tmZ);
        prefetch_tmap(&tmO);
        prefetch_tmap(&tmOut);
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

    if (warp == 0) {
        if (lane == 0) {
            mbar_arrive_expect_tx(w_full, 2 * kTileBytes);
            for (int kb = 0; kb < 2; ++kb) {
                tma_load_2d(sbase + AOutSmem::kWg + kb * kKBlockBytes, &tmWg, w_full, kb * 64, 0);
                tma_load_2d(sbase + AOutSmem::kWo + kb * kKBlockBytes, &tmWo, w_full, kb * 64, 0);
            }
            for (long long lt = 0; lt < my_tiles; ++lt) {
                const int g = (int)(lt & 1);
                const uint32_t use = (uint32_t)(lt >> 1);
                const LineTile tc = line_tile(blockIdx.x + lt * gridDim.x, R, tiles_per_line);
                if (!mbar_wait(z_empty(g), (use & 1u) ^ 1u, abort_flag)) {
                    report_wait_failure(status, abort_flag, kKidOut, 1);
                    break;
                }
                mbar_arrive_expect_tx(z_full(g), kTileBytes);
                load_z_tile<kTransposed>(sbase + AOutSmem::kZ + g * kTileBytes, &tmZ, z_full(g), tc, R);
                if (!mbar_wait(o_empty(g), (use & 1u) ^ 1u, abort_flag)) {
                    report_wait_failure(status, abort_flag, kKidOut, 8);
                    break;
                }
                mbar_arrive_expect_tx(o_full(g), kTileBytes);
                const uint32_t odst = sbase + AOutSmem::kO + g * kTileBytes;
                for (int kb = 0; kb < 2; ++kb)
                    tma_load_3d(odst + kb * kKBlockBytes, &tmO, o_full(g), kb * 64, tc.t0, tc.b * R + tc.line);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = idesc_bf16_f32(128, 128);
            bool ok = mbar_wait(w_full, 0, abort_flag);
            if (!ok) report_wait_failure(status, abort_flag, kKidOut, 2);
            // gate GEMM of tile lt is issued before the output GEMM of tile lt-1, so the two groups
            // overlap: one gates its o tile while the other's gate GEMM runs
            for (long long lt = 0; lt <= my_tiles && ok; ++lt) {
                if (lt < my_tiles) {
                    const int g = (int)(lt & 1);
                    if (!mbar_wait(a1_ready(g), (uint32_t)(lt >> 1) & 1u, abort_flag)) {
                        report_wait_failure(status, abort_flag, kKidOut, 3);
                        break;
                    }
                    tc_fence_after_sync();
                    mma_k128(tmem_base + g * 256, sbase + AOutSmem::kZ + g * kTileBytes, sbase + AOutSmem::kWg,
                             kKBlockBytes, idesc, false);
                    mma_commit(g_full(g));
                    mma_commit(z_empty(g));
                }
                if (lt >= 1) {
                    const long long pt = lt - 1;
                    const int g = (int)(pt & 1);
                    if (!mbar_wait(a2_ready(g), (uint32_t)(pt >> 1) & 1u, abort_flag)) {
                        report_wait_failure(status, abort_flag, kKidOut, 4);
                        break;
                    }
                    tc_fence_after_sync();
                    mma_k128(tmem_base + g * 256 + 128, sbase + AOutSmem::kO + g * kTileBytes,
                             sbase + AOutSmem::kWo, kKBlockBytes, idesc, false);
                    mma_commit(d_full(g));
                }
            }
        }
    } else {
        const int g = (warp - 2) >> 3;
        const int quad = warp & 3;
        const int half = ((warp - 2) >> 2) & 1;   // channels [64 * half, 64 * half + 64) of the row
        const int row = quad * 32 + lane;
        const int gtid = (warp - 2 - g * 8) * 32 + lane;
        float* xch = reinterpret_cast<float*>(gbase + AOutSmem::kXch) + g * 512;
        const uint32_t ztile = sbase + AOutSmem::kZ + g * kTileBytes;
        const uint32_t otile = sbase + AOutSmem::kO + g * kTileBytes;
        const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + g * 256 + half * 64;
        for (long long lt = g; lt < my_tiles; lt += 2) {
            const uint32_t use = (uint32_t)(lt >> 1);
            const LineTile tc = line_tile(blockIdx.x + lt * gridDim.x, R, tiles_per_line);
            if (!mbar_wait(z_full(g), use & 1u, abort_flag)) {
                if (lane == 0) report_wait_failure(status, abort_flag, kKidOut, 5);
                break;
            }
            uint32_t zraw[32];
            load_half_row(ztile, row, half, zraw);
            {
                float mean, rstd;
                half_row_stats_xwarp(zraw, row, half, xch, 1 + g, 256, mean, rstd);
                store_normalized_half_row(ztile, row, half, zraw, mean, rstd, prm, prm + 128);
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(a1_ready(g));
            // ---- gate: o <- o * sigmoid(LN(z) W_g^T), in place in the o tile
            if (!mbar_wait(g_full(g), use & 1u, abort_flag)) {
                if (lane == 0) report_wait_failure(status, abort_flag, kKidOut, 6);
                break;
            }
            tc_fence_after_sync();
            if (!mbar_wait(o_full(g), use & 1u, abort_flag)) {
                if (lane == 0) report_wait_failure(status, abort_flag, kKidOut, 9);
                break;
            }
#pragma unroll
            for (int cb = 0; cb < 4; ++cb) {
                uint32_t gate[16];
                tmem_ld16(taddr + cb * 16, gate);
                tmem_ld_wait();
#pragma unroll
                for (int ch = 0; ch < 2; ++ch) {
                    const uint32_t addr = chunk_addr(otile, row, half * 8 + cb * 2 + ch);
                    const uint4 ov = lds128(addr);
                    const uint32_t w[4] = {ov.x, ov.y, ov.z, ov.w};
                    uint32_t o[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int e = ch * 8 + j * 2;
                        o[j] = pack_bf16x2(bf16lo(w[j]) * sigmoid_fast(__uint_as_float(gate[e])),
                                           bf16hi(w[j]) * sigmoid_fast(__uint_as_float(gate[e + 1])));
                    }
                    sts128(addr, make_uint4(o[0], o[1], o[2], o[3]));
                }
            }
            tc_fence_before_sync();
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(a2_ready(g));
            // ---- output projection + residual, written over the o tile (its GEMM is done) and TMA-stored
            if (!mbar_wait(d_full(g), use & 1u, abort_flag)) {
                if (lane == 0) report_wait_failure(status, abort_flag, kKidOut, 7);
                break;
            }
            tc_fence_after_sync();
#pragma unroll
            for (int cb = 0; cb < 4; ++cb) {
                uint32_t upd[16];
                tmem_ld16(taddr + 128 + cb * 16, upd);
                tmem_ld_wait();
#pragma unroll
                for (int ch = 0; ch < 2; ++ch) {
                    uint32_t o[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int e = ch * 8 + j * 2;
                        const uint32_t zr = zraw[cb * 8 + ch * 4 + j];
                        float v0 = __uint_as_float(upd[e]), v1 = __uint_as_float(upd[e + 1]);
                        if (add_residual) {
                            v0 += bf16lo(zr);
                            v1 += bf16hi(zr);
                        }
                        o[j] = pack_bf16x2(v0, v1);
                    }
                    sts128(chunk_addr(otile, row, half * 8 + cb * 2 + ch), make_uint4(o[0], o[1], o[2], o[3]));
                }
            }
            tc_fence_before_sync();
            fence_proxy_async_smem();
            group_sync(1 + g, 256);
            if (gtid == 0) {
                for (int kb = 0; kb < 2; ++kb) {
                    if (kTransposed) {
                        asm volatile(
                            "cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::
                                "l"(reinterpret_cast<uint64_t>(&tmOut)),
                            "r"(otile + kb * kKBlockBytes), "r"(kb * 64), "r"(tc.line), "r"(tc.t0), "r"(tc.b)
                            : "memory");
                    } else {
                        tma_store_3d(&tmOut, otile + kb * kKBlockBytes, kb * 64, tc.t0, tc.b * R + tc.line);
                    }
                }
                tma_store_commit();
                tma_store_wait_read<0>();
                mbar_arrive(o_empty(g));
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

int weight_tmap128(CUtensorMap* m, const void* w) {
    uint64_t dims[2] = {128, 128};
    uint64_t str[1] = {256};
    uint32_t box[2] = {64, 128};
    return make_tmap_bf16(m, w, 2, dims, str, box, 1);
}

int z_tmap(CUtensorMap* m, const void* z, int B, int R, int N, bool transposed) {
    if (!transposed) {
        uint64_t dims[3] = {128, (uint64_t)N, (uint64_t)B * R};
        uint64_t str[2] = {256, (uint64_t)N * 256};
        uint32_t box[3] = {64, 128, 1};
        return make_tmap_bf16(m, z, 3, dims, str, box, 1);
    }
    uint64_t dims[4] = {128, (uint64_t)N, (uint64_t)N, (uint64_t)B};
    uint64_t str[3] = {256, (uint64_t)N * 256, (uint64_t)N * N * 256};
    uint32_t box[4] = {64, 1, 128, 1};
    return make_tmap_bf16(m, z, 4, dims, str, box, 1);
}

template <bool kT>
int set_attrs() {
    constexpr int kAttrKey = kT ? 7 : 6;  // per-device function attributes
    if (!device_configured(kAttrKey)) {
        OF3_CUDA_CHECK(cudaFuncSetAttribute(triattn_proj_kernel<kT>, cudaFuncAttributeMaxDynamicSharedMemorySize, ProjSmem::kDyn));
        OF3_CUDA_CHECK(cudaFuncSetAttribute(triattn_core_kernel<kT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            CoreSmem::dyn_bytes(kMaxKeys / kBK)));
        OF3_CUDA_CHECK(cudaFuncSetAttribute(triattn_out_kernel<kT>, cudaFuncAttributeMaxDynamicSharedMemorySize, AOutSmem::kDyn));
        device_mark_configured(kAttrKey);
    }
    return OF3_OK;
}

template <bool kT>
int project_impl(const __nv_bfloat16* z, __nv_bfloat16* q, __nv_bfloat16* k, __nv_bfloat16* vt,
                 __nv_bfloat16* tb, int B, int R, int N, int row0, const of3_triattn_params* p, cudaStream_t st) {
    int rc;
    CUtensorMap tmZ, tmW[3], tmWb;
    if ((rc = z_tmap(&tmZ, z, B, R, N, kT))) return rc;
    const void* w3[3] = {p->w_q, p->w_k, p->w_v};
    for (int i = 0; i < 3; ++i)
        if ((rc = weight_tmap128(&tmW[i], w3[i]))) return rc;
    {   // linear_z.weight [4, 128]: box of 16 rows, the 12 rows past the end are zero-filled
        OF3_REQUIRE(((uintptr_t)p->w_bias & 15) == 0, OF3_ERR_ALIGN, "triattn: linear_z.weight must be 16-byte aligned");
        uint64_t dims[2] = {128, (uint64_t)kH};
        uint64_t str[1] = {256};
        uint32_t box[2] = {64, 16};
        if ((rc = make_tmap_bf16(&tmWb, p->w_bias, 2, dims, str, box, 1))) return rc;
    }
    if ((rc = set_attrs<kT>())) return rc;
    const long long tiles = (long long)B * R * ceil_div(N, kRows);
    const int grid = (int)(tiles < sm_count() ? tiles : sm_count());
    LaunchScope scope(kKidProj, st);
    triattn_proj_kernel<kT><<<grid, kProjThreads, ProjSmem::kDyn, st>>>(
        tmZ, tmW[0], tmW[1], tmW[2], tmWb, (const __nv_bfloat16*)p->ln_w, (const __nv_bfloat16*)p->ln_b, q, k, vt,
        tb, B, R, N, (int)align_up(N, kBK), row0, device_status_ptr());
    OF3_CUDA_CHECK(cudaGetLastError());
    return OF3_OK;
}

template <bool kT>
int finish_impl(const __nv_bfloat16* z, const __nv_bfloat16* mask, __nv_bfloat16* out, const __nv_bfloat16* q,
                const __nv_bfloat16* k, const __nv_bfloat16* vt, const __nv_bfloat16* tb, __nv_bfloat16* o, int B,
                int R, int N, float inf, int add_residual, const of3_triattn_params* p, cudaStream_t st) {
    int rc;
    CUtensorMap tmZ, tmOut, tmO, tmWg, tmWo;
    if ((rc = z_tmap(&tmZ, z, B, R, N, kT))) return rc;
    if ((rc = z_tmap(&tmOut, out, B, R, N, kT))) return rc;
    if ((rc = z_tmap(&tmO, o, B, R, N, false))) return rc;  // o is [line][pos][128] in view order
    if ((rc = weight_tmap128(&tmWg, p->w_g))) return rc;
    if ((rc = weight_tmap128(&tmWo, p->w_o))) return rc;
    if ((rc = set_attrs<kT>())) return rc;
    int* status = device_status_ptr();
    const long long ctas = (long long)B * ceil_div(R, kLines) * kH * ceil_div(N, kBQ);
    OF3_REQUIRE(ctas < (1LL << 31), OF3_ERR_SHAPE, "triattn: too many attention tiles");
    {
        LaunchScope scope(kKidCore, st);
        triattn_core_kernel<kT><<<(unsigned)ctas, kCoreThreads, CoreSmem::dyn_bytes(ceil_div(N, kBK)), st>>>(
            q, k, vt, tb, mask, o, B, R, N, (int)align_up(N, kBK), inf, status);
    }
    OF3_CUDA_CHECK(cudaGetLastError());
    const long long tiles = (long long)B * R * ceil_div(N, kRows);
    const int grid = (int)(tiles < sm_count() ? tiles : sm_count());
    LaunchScope scope(kKidOut, st);
    triattn_out_kernel<kT><<<grid, kAOutThreads, AOutSmem::kDyn, st>>>(
        tmZ, tmO, tmOut, tmWg, tmWo, (const __nv_bfloat16*)p->ln_w, (const __nv_bfloat16*)p->ln_b, B, R, N,
        add_residual, status);
    OF3_CUDA_CHECK(cudaGetLastError());
    return OF3_OK;
}

}  // namespace


bool triattn_supported(int c_z, int H, int d, int N) {
    return c_z == 128 && H == kH && d == kD && N <= kMaxKeys;
}

// Elements of each of the q / k / v image buffers for B samples of R lines and N positions: 4 heads x
// (query tiles of 128) x (R rounded up to 4 lines) x 128 x 32; the k / v images need no more than that.
size_t triattn_image_elems(int B, int R, int N) {
    return (size_t)B * kH * ceil_div(N, kBQ) * align_up(R, kLinePad) * kBQ * kD;
}

// Elements (bf16) of the pair-bias image of B samples with R query rows and N keys: [B*4][key blocks of 32][R][32].
size_t triattn_bias_elems(int B, int R, int N) {
    return (size_t)B * kH * ceil_div(N, kBK) * R * kBiasK;
}

// q, k, v operand images and this shard's rows of the pair-bias image tb[(b*H + h)][key block][line][32]
// from R lines of N positions; row0 = index of the shard's first line among all N query rows (0 for a whole
// tensor). transposed: whole square tensors only.
int triattn_project(const __nv_bfloat16* z, __nv_bfloat16* q, __nv_bfloat16* k, __nv_bfloat16* vt,
                    __nv_bfloat16* tb, int B, int R, int N, int row0, bool transposed,
                    const of3_triattn_params* p, cudaStream_t st) {
    OF3_REQUIRE(((uintptr_t)z & 15) == 0, OF3_ERR_ALIGN, "triattn: z must be 16-byte aligned");
    OF3_REQUIRE(!transposed || R == N, OF3_ERR_SHAPE, "triattn: transposed view needs the whole tensor");
    return transposed ? project_impl<true>(z, q, k, vt, tb, B, R, N, row0, p, st)
                      : project_impl<false>(z, q, k, vt, tb, B, R, N, row0, p, st);
}

// attention over the R lines with the pair-bias image of all N query rows (tb [(b*H + h)][key block][N][32]),
// gate, output projection, residual.
int triattn_finish(const __nv_bfloat16* z, const __nv_bfloat16* mask, __nv_bfloat16* out,
                   const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* vt,
                   const __nv_bfloat16* tb, __nv_bfloat16* o, int B, int R, int N, float inf,
                   bool transposed, int add_residual, const of3_triattn_params* p, cudaStream_t st) {
    OF3_REQUIRE(((uintptr_t)tb & 15) == 0, OF3_ERR_ALIGN, "triattn: the pair-bias image must be 16-byte aligned");
    OF3_REQUIRE(((uintptr_t)z & 15) == 0 && ((uintptr_t)out & 15) == 0, OF3_ERR_ALIGN,
                "triattn: z/out must be 16-byte aligned");
    OF3_REQUIRE(N <= kMaxKeys, OF3_ERR_SHAPE, "triattn: N %d above the %d keys one CTA keeps a mask row for", N,
                kMaxKeys);
    OF3_REQUIRE(!transposed || R == N, OF3_ERR_SHAPE, "triattn: transposed view needs the whole tensor");
    return transposed ? finish_impl<true>(z, mask, out, q, k, vt, tb, o, B, R, N, inf, add_residual, p, st)
                      : finish_impl<false>(z, mask, out, q, k, vt, tb, o, B, R, N, inf, add_residual, p, st);
}

int triattn(const __nv_bfloat16* z, const __nv_bfloat16* mask, __nv_bfloat16* out, int B, int N,
            float inf, int flags, const of3_triattn_params* p, Arena& ws, cudaStream_t st) {
    const size_t plane = (size_t)B * N * N * kC * sizeof(__nv_bfloat16);
    const size_t img = triattn_image_elems(B, N, N) * sizeof(__nv_bfloat16);
    __nv_bfloat16* q = (__nv_bfloat16*)ws.take(img);
    __nv_bfloat16* k = (__nv_bfloat16*)ws.take(img);
    __nv_bfloat16* vt = (__nv_bfloat16*)ws.take(img);
    __nv_bfloat16* o = (__nv_bfloat16*)ws.take(plane);
    __nv_bfloat16* tb = (__nv_bfloat16*)ws.take(triattn_bias_elems(B, N, N) * sizeof(__nv_bfloat16));
    if (!ws.base) return OF3_OK;
    OF3_REQUIRE(ws.ok(), OF3_ERR_WORKSPACE, "triattn: workspace too small (%zu needed)", ws.off);
    const bool tr = (flags & OF3_FLAG_TRANSPOSED) != 0;
    int rc = triattn_project(z, q, k, vt, tb, B, N, N, 0, tr, p, st);
    if (rc) return rc;
    return triattn_finish(z, mask, out, q, k, vt, tb, o, B, N, N, inf, tr,
                          (flags & OF3_FLAG_ADD_RESIDUAL) ? 1 : 0, p, st);
}

}  // namespace fast
}  // namespace of3
