// Attention of the single track and of the diffusion token stack on the tensor pipe (bf16, 16 heads of 24 or 48):
// the streaming core of the triangle attention (csrc/fast_triattn.cu) with one (pair tensor, head, 128 queries) and
// two samples per CTA.
//
//   single_pack     q / k / v rows [rows, H*d] (outputs of the linear layers) -> pre-swizzled operand tiles: q with
//                   its bias added and scaled by log2(e)/sqrt(d), K-dim padded with zeros to 32 (d = 24) or 64
//                   (d = 48); k likewise per key block of 32; v transposed [d rows][32 keys]; keys >= N are zeros
//   single_bias     pair bias fp32 [zh][nq][N] -> bf16 tiles [zh][key block][nq][32], pre-scaled by log2(e), each
//                   64-byte row in the 64-byte swizzle of a K-major A operand (callers that project the bias
//                   themselves get these tiles straight from csrc/fast_pairbias.cu and skip this kernel)
//   single_core     per CTA and 32-key step: S = Q K^T + bias I^T (tcgen05, TMEM), online softmax by one thread per
//                   query row (exp2, lazy rescaling), P (bf16) back into TMEM over S as the A operand of
//                   O += P [V; 1] (the row of ones makes the tensor pipe accumulate the row sum l); epilogue
//                   O / l * sigmoid(gate) -> og [rows, H*d]
// Queries may be a window of nq rows of the sample (row-sharded callers); keys and values are always all N rows.
// Reference: openfold3/core/model/layers/attention_pair_bias.py:123-227,
//            openfold3/core/model/primitives/attention.py:94-135, 270-310.
#include "modules.cuh"
#include "rowtile.cuh"
#include "runtime.cuh"

namespace of3 {
namespace fast {
namespace {

using namespace umma;
using namespace rowtile;
typedef __nv_bfloat16 bf16;

constexpr int kKidSingleAttn = 8;    // operand images: accounted with the single track's small kernels
constexpr int kKidSingleCore = 11;   // the attention core
constexpr float kLog2e = 1.4426950408889634f;
constexpr int kBQ = 128;   // queries per CTA and line
constexpr int kBK = 32;    // keys per step
constexpr int kLines = 2;  // samples per CTA: they share the pair-bias tiles
constexpr int kThreads = 32 * (1 + kLines + 4 * kLines);  // producer, one MMA warp per line, softmax warps
constexpr float kRescaleThreshold = 8.0f;
constexpr int kMaxKeysSingle = 8192;  // one flag byte per key block, 256 of them

template <int D>
struct Cfg {
    static constexpr int kKD = (D <= 32) ? 32 : 64;      // K dim of Q K^T after zero padding
    static constexpr int kKSteps = (D + 15) / 16;        // K = 16 steps that hold data
    static constexpr int kDV = (D <= 32) ? 32 : 48;      // rows of the V^T tile = columns of O
    static constexpr int kStages = (D <= 32) ? 4 : 3;    // ring of K + bias tiles
    static constexpr int kVStages = (D <= 32) ? 4 : 2;   // ring of V tiles (two CTAs of 16 x 48 heads must fit an SM)
    static constexpr uint32_t kQBytes = kBQ * kKD * 2;   // 8 or 16 KB
    static constexpr uint32_t kKBytes = kBK * kKD * 2;   // 2 or 4 KB
    static constexpr uint32_t kVBytes = kDV * kBK * 2;   // 2 or 3 KB: the tile a bulk copy brings
    static constexpr int kON = kDV + 16;                 // N of the P V GEMM: channels, a row of ones (-> row sum), padding
    static constexpr uint32_t kVSlot = kON * kBK * 2;    // 3 or 4 KB: rows kDV .. kDV + 15 are written once per CTA
    static constexpr uint32_t kTbBytes = kBQ * kBK * 2;  // 8 KB
    // shared memory (offsets from a 1024-byte boundary)
    static constexpr uint32_t kQ = 0;
    static constexpr uint32_t kK = kQ + kLines * kQBytes;
    static constexpr uint32_t kTb = kK + kStages * kLines * kKBytes;
    static constexpr uint32_t kV = kTb + kStages * kTbBytes;
    static constexpr uint32_t kIdent = kV + kVStages * kLines * kVSlot;
    static constexpr uint32_t kBars = kIdent + 2048;
    static constexpr uint32_t kFlags = kBars + 320;       // lines x 256 key-block flags (bytes)
    static constexpr uint32_t kMb = kFlags + kLines * 256;
    static uint32_t dyn_bytes(int nkp) { return kMb + kLines * nkp * 4 + 1024; }
    // TMEM columns of a line (128): S slots [0,32) [32,64), each taking the step's P (16 columns of bf16 pairs)
    // in place once S has been read out; O [64, 64 + kON): kDV channels, then the sum of the row's P
    static constexpr uint32_t kColO = 64;
};

// 16-byte chunk c of row r inside a K-major tile with rows of kKD bf16: 64-byte rows use the 64-byte swizzle,
// 128-byte rows the 128-byte swizzle (what the tcgen05 descriptors of umma.cuh expect).
template <int KD>
__device__ __forceinline__ uint32_t tile_chunk_off(int r, int c) {
    return KD == 32 ? (uint32_t)(r * 64 + ((c ^ ((r >> 1) & 3)) << 4)) : (uint32_t)(r * 128 + ((c ^ (r & 7)) << 4));
}


// ---------------------------------------------------------------- operand images
// q and k: one thread per 16-byte chunk of a tile row (reads of a warp run along the rows of the source, each
// tile row is written whole). blockIdx.y: 0 = q tiles [bh][query tile][128][KD], 1 = k tiles [bh][key block][32][KD].
template <int D>
__global__ void __launch_bounds__(256)
single_pack_qk_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ q_bias,
                      bf16* __restrict__ q_img, bf16* __restrict__ k_img, int BB, int N, int nq, int H, float qscale) {
    constexpr int KD = Cfg<D>::kKD, CH = KD / 8;
    const bool is_q = blockIdx.y == 0;
    const int rows_src = is_q ? nq : N;
    const int tile_rows = is_q ? kBQ : kBK;
    const int rows_pad = (rows_src + tile_rows - 1) / tile_rows * tile_rows;
    const long long idx = (long long)blockIdx.x * 256 + threadIdx.x;
    const int c = (int)(idx % CH);
    const int h = (int)((idx / CH) % H);
    const int pos = (int)((idx / ((long long)CH * H)) % rows_pad);
    const long long bb = idx / ((long long)CH * H * rows_pad);
    if (bb >= BB) return;
    uint4 w = make_uint4(0u, 0u, 0u, 0u);
    if (pos < rows_src && c * 8 < D) {
        const long long off = (bb * rows_src + pos) * (long long)(H * D) + h * D + c * 8;
        w = *reinterpret_cast<const uint4*>((is_q ? q : k) + off);
        if (is_q) {
            uint4 bq = make_uint4(0u, 0u, 0u, 0u);
            if (q_bias) bq = *reinterpret_cast<const uint4*>(q_bias + h * D + c * 8);
            w.x = pack_bf16x2((bf16lo(w.x) + bf16lo(bq.x)) * qscale, (bf16hi(w.x) + bf16hi(bq.x)) * qscale);
            w.y = pack_bf16x2((bf16lo(w.y) + bf16lo(bq.y)) * qscale, (bf16hi(w.y) + bf16hi(bq.y)) * qscale);
            w.z = pack_bf16x2((bf16lo(w.z) + bf16lo(bq.z)) * qscale, (bf16hi(w.z) + bf16hi(bq.z)) * qscale);
            w.w = pack_bf16x2((bf16lo(w.w) + bf16lo(bq.w)) * qscale, (bf16hi(w.w) + bf16hi(bq.w)) * qscale);
        }
    }
    const long long tile = (bb * H + h) * (rows_pad / tile_rows) + pos / tile_rows;
    uint8_t* dst = reinterpret_cast<uint8_t*>(is_q ? q_img : k_img) + tile * tile_rows * (long long)(KD * 2);
    *reinterpret_cast<uint4*>(dst + tile_chunk_off<KD>(pos % tile_rows, c)) = w;
}

// v: block = (key block of 32, sample); the 32 source rows pass through shared memory and leave transposed,
// v tiles [bh][key block][DV][32 keys] with the 64-byte swizzle. Dynamic shared memory: 32 * H * D * 2 bytes.
template <int D>
__global__ void __launch_bounds__(256)
single_pack_v_kernel(const bf16* __restrict__ v, bf16* __restrict__ v_img, int N, int H) {
    constexpr int DV = Cfg<D>::kDV;
    extern __shared__ __align__(16) uint8_t vs_raw[];
    bf16* vs = reinterpret_cast<bf16*>(vs_raw);
    const int kb = blockIdx.x, nkb = gridDim.x;
    const long long bb = blockIdx.y;
    const int HD = H * D, cpr = HD / 8;
    for (int idx = threadIdx.x; idx < kBK * cpr; idx += 256) {
        const int r = idx / cpr, c = idx % cpr;
        const int key = kb * kBK + r;
        uint4 w = make_uint4(0u, 0u, 0u, 0u);
        if (key < N) w = *reinterpret_cast<const uint4*>(v + (bb * N + key) * (long long)HD + c * 8);
        *reinterpret_cast<uint4*>(vs + r * HD + c * 8) = w;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < H * DV * 4; idx += 256) {
        const int kc = idx & 3, dd = (idx >> 2) % DV, h = idx / (4 * DV);
        uint32_t w[4] = {0u, 0u, 0u, 0u};
        if (dd < D) {
            const unsigned short* col = reinterpret_cast<const unsigned short*>(vs) + h * D + dd;
#pragma unroll
            for (int e = 0; e < 4; ++e)
                w[e] = (uint32_t)col[(kc * 8 + 2 * e) * HD] | ((uint32_t)col[(kc * 8 + 2 * e + 1) * HD] << 16);
        }
        bf16* tile = v_img + (((bb * H + h) * nkb + kb) * (long long)DV + dd) * kBK;
        *reinterpret_cast<uint4*>(tile + ((kc ^ ((dd >> 1) & 3)) << 3)) = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

// pair bias fp32 [zh][nq][N] -> bf16 tiles [zh][key block][nq][32], times log2(e); block = (query row, zh)
__global__ void __launch_bounds__(256)
single_bias_kernel(const float* __restrict__ pair_bias, bf16* __restrict__ tb_img, int N, int nq, int nkb) {
    const int qrow = blockIdx.x;
    const long long zh = blockIdx.y;
    const float* src = pair_bias + (zh * nq + qrow) * (long long)N;
    for (int key = threadIdx.x; key < nkb * kBK; key += 256) {
        const float val = key < N ? src[key] * kLog2e : 0.f;
        const int kb = key >> 5, kk = key & 31;
        const int c = (kk >> 3) ^ ((qrow >> 1) & 3);
        tb_img[((zh * nkb + kb) * (long long)nq + qrow) * kBK + c * 8 + (kk & 7)] = __float2bfloat16_rn(val);
    }
}

// ---------------------------------------------------------------- single_core
// One CTA = (pair tensor z, head, 128 queries) for TWO samples ("lines") that share the pair bias; two CTAs per SM.
// Per line and 32-key step j:
//   MMA warp      S_j = Q K_j^T + Tb_j I^T into TMEM slot j % 2 (the bias tile is a second A operand against a
//                 32 x 32 identity: the tensor pipe adds it, exactly, in fp32)
//   softmax warps thread = query row = TMEM lane: S -> registers [+ key-mask bias], row maximum, P = exp2(S - m),
//                 P rounded to bf16 into the first 16 columns of the slot S_j came from
//   MMA warp      O += P_j V_j with P read from TMEM as the A operand; when that GEMM is done the slot takes S_{j+2}
// The running maximum m used for scaling is only raised when a row maximum exceeds it by more than 8 (2^8 head
// room in P): then the thread rescales its O row in TMEM and its running sum. Numerator and denominator always
// share one scale, so the result is exact.
template <int D>
__global__ void __launch_bounds__(kThreads, 2)
single_core_kernel(const bf16* __restrict__ q_img, const bf16* __restrict__ k_img, const bf16* __restrict__ v_img,
                   const bf16* __restrict__ tb_img, const bf16* __restrict__ mask, const bf16* __restrict__ gate,
                   bf16* __restrict__ out, int N, int nq, int H, int rpb, float inf, int* status) {
    using C = Cfg<D>;
    constexpr int KD = C::kKD, DV = C::kDV, kSt = C::kStages, kVSt = C::kVStages;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gbase = smem_raw + (sbase - smem_u32(smem_raw));
    float* mbs = reinterpret_cast<float*>(gbase + C::kMb);
    volatile uint8_t* mbflag = gbase + C::kFlags;
    const uint32_t bars = sbase + C::kBars;
    const uint32_t q_full = bars;
    auto kb_full = [&](int s) { return bars + 8u * (1 + s); };
    auto kb_empty = [&](int s) { return bars + 8u * (1 + kSt + s); };
    constexpr int kB1 = 1 + 2 * kSt;
    auto v_full = [&](int s) { return bars + 8u * (kB1 + s); };
    auto v_empty = [&](int s) { return bars + 8u * (kB1 + kVSt + s); };
    constexpr int kB2 = kB1 + 2 * kVSt;
    auto s_full = [&](int L, int s) { return bars + 8u * (kB2 + L * 2 + s); };
    auto p_ready = [&](int L, int s) { return bars + 8u * (kB2 + 2 * kLines + L * 2 + s); };
    auto pv_done = [&](int L, int s) { return bars + 8u * (kB2 + 4 * kLines + L * 2 + s); };
    constexpr int kNumBars = kB2 + 6 * kLines;
    static_assert(8 * kNumBars + 16 <= 320, "barrier block");
    volatile uint32_t* tmem_ptr = reinterpret_cast<volatile uint32_t*>(gbase + C::kBars + 8 * kNumBars);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + C::kBars + 8 * kNumBars + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_qt = (nq + kBQ - 1) / kBQ;
    const int gpz = (rpb + kLines - 1) / kLines;   // CTAs per (z, head, query tile)
    const int grp = blockIdx.x % gpz;
    const int qt = (blockIdx.x / gpz) % n_qt;
    const int h = (blockIdx.x / (gpz * n_qt)) % H;
    const int z = blockIdx.x / (gpz * n_qt * H);
    const int q0 = qt * kBQ;
    const int nblk = (N + kBK - 1) / kBK;
    const int nkp = nblk * kBK;
    // a line past the last sample of z recomputes the group's first sample and is not stored
    auto sample_of = [&](int L) { return (long long)z * rpb + ((grp * kLines + L < rpb) ? grp * kLines + L : grp * kLines); };

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < kSt; ++s) {
            mbar_init(kb_full(s), 1);
            mbar_init(kb_empty(s), 4 * kLines);  // every softmax warp has read the S that consumed the stage
        }
        for (int s = 0; s < kVSt; ++s) {
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
    // 32 x 32 identity, bf16, K-major with the 64-byte swizzle
    for (int idx = threadIdx.x; idx < 32 * 16; idx += blockDim.x) {
        const int n = idx >> 4, w = idx & 15;
        const int k = w * 2;
        uint32_t v = 0;
        if (k == n) v = 0x00003F80u;
        if (k + 1 == n) v = 0x3F800000u;
        const int chunk = (k >> 3) ^ ((n >> 1) & 3);
        *reinterpret_cast<uint32_t*>(gbase + C::kIdent + n * 64 + chunk * 16 + (w & 3) * 4) = v;
    }
    // rows kDV .. kDV + 15 of every V slot: a row of ones (column kDV of O then accumulates the row sum of P on the
    // tensor pipe, rounded exactly like the numerator) and 15 rows of zeros; the bulk copies write rows 0 .. kDV - 1
    for (int idx = threadIdx.x; idx < kVSt * kLines * 64; idx += blockDim.x) {
        const int slot = idx >> 6, w = idx & 63;   // 64 uint4 = 1 KB per slot
        const uint32_t v = (w < 4) ? 0x3F803F80u : 0u;
        *reinterpret_cast<uint4*>(gbase + C::kV + slot * C::kVSlot + C::kVBytes + w * 16) = make_uint4(v, v, v, v);
    }
    fence_proxy_async_smem();
    if (warp == 1) {
        tmem_alloc(smem_u32((const void*)tmem_ptr), kLines * 128);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_ptr;

    if (warp == 0) {
        if (lane == 0) {
            const long long zh = (long long)z * H + h;
            mbar_arrive_expect_tx(q_full, kLines * C::kQBytes);
            for (int L = 0; L < kLines; ++L)
                bulk_load(sbase + C::kQ + L * C::kQBytes,
                          q_img + (((sample_of(L) * H + h) * n_qt + qt) * kBQ) * (long long)KD, C::kQBytes, q_full);
            const int q_rows = (nq - q0 < kBQ) ? nq - q0 : kBQ;   // rows of the bias tile that exist
            const uint32_t tb_bytes = (uint32_t)q_rows * kBK * 2;
            for (int j = 0; j < nblk; ++j) {
                const int s = j % kSt;
                const uint32_t ph = ((j / kSt) & 1u) ^ 1u;
                if (!mbar_wait(kb_empty(s), ph, abort_flag)) {
                    report_wait_failure(status, abort_flag, kKidSingleCore, 1);
                    break;
                }
                mbar_arrive_expect_tx(kb_full(s), kLines * C::kKBytes + tb_bytes);
                for (int L = 0; L < kLines; ++L)
                    bulk_load(sbase + C::kK + (s * kLines + L) * C::kKBytes,
                              k_img + (((sample_of(L) * H + h) * nblk + j) * kBK) * (long long)KD, C::kKBytes,
                              kb_full(s));
                bulk_load(sbase + C::kTb + s * C::kTbBytes, tb_img + ((zh * nblk + j) * (long long)nq + q0) * kBK,
                          tb_bytes, kb_full(s));
                const int sv = j % kVSt;
                if (!mbar_wait(v_empty(sv), ((j / kVSt) & 1u) ^ 1u, abort_flag)) {
                    report_wait_failure(status, abort_flag, kKidSingleCore, 11);
                    break;
                }
                mbar_arrive_expect_tx(v_full(sv), kLines * C::kVBytes);
                for (int L = 0; L < kLines; ++L)
                    bulk_load(sbase + C::kV + (sv * kLines + L) * C::kVSlot,
                              v_img + (((sample_of(L) * H + h) * nblk + j) * (long long)DV) * kBK, C::kVBytes,
                              v_full(sv));
            }
        }
    } else if (warp <= kLines) {
        // ---------------------------------------------------------------- one MMA-issuing warp per line
        // The whole warp walks the loop and lane 0 issues: with warp-uniform control flow and operands descriptors
        // and addresses live in uniform registers.
        const int L = __shfl_sync(0xffffffffu, warp, 0) - 1;
        const uint32_t tm = __shfl_sync(0xffffffffu, tmem_base, 0);
        const uint32_t sb = __shfl_sync(0xffffffffu, sbase, 0);
        constexpr uint32_t idesc_s = idesc_bf16_f32(128, kBK);
        constexpr uint32_t idesc_o = idesc_bf16_f32(128, C::kON);
        auto kdesc_of = [](uint32_t a) { return KD == 32 ? smem_desc_k_sw64(a) : smem_desc_k_sw128(a); };
        bool ok = mbar_wait(q_full, 0, abort_flag);
        if (!ok && lane == 0) report_wait_failure(status, abort_flag, kKidSingleCore, 2);
        const uint64_t qdesc = kdesc_of(sb + C::kQ + L * C::kQBytes);
        const uint64_t identdesc = smem_desc_k_sw64(sb + C::kIdent);
        const uint32_t t_line = tm + L * 128;
        // S_i = Q K_i^T + Tb_i into slot i % 2, free once P_{i-2} V_{i-2} (which read P out of it) is done
        auto issue_s = [&](int i) -> bool {
            const int s = i & 1;
            const int ks = i % kSt;
            if (i >= 2 && !mbar_wait(pv_done(L, s), ((i - 2) >> 1) & 1u, abort_flag)) {
                if (lane == 0) report_wait_failure(status, abort_flag, kKidSingleCore, 4);
                return false;
            }
            if (!mbar_wait(kb_full(ks), (i / kSt) & 1u, abort_flag)) {
                if (lane == 0) report_wait_failure(status, abort_flag, kKidSingleCore, 3);
                return false;
            }
            tc_fence_after_sync();
            const uint64_t kdesc = kdesc_of(sb + C::kK + (ks * kLines + L) * C::kKBytes);
            const uint64_t tbdesc = smem_desc_k_sw64(sb + C::kTb + ks * C::kTbBytes);
            const uint32_t d = t_line + s * kBK;
            if (lane == 0) {
#pragma unroll
                for (int kk = 0; kk < C::kKSteps; ++kk)
                    mma_bf16(d, qdesc + 2u * kk, kdesc + 2u * kk, idesc_s, kk ? 1u : 0u);
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
            const int vs = j % kVSt;
            if (!mbar_wait(v_full(vs), (j / kVSt) & 1u, abort_flag)) {
                if (lane == 0) report_wait_failure(status, abort_flag, kKidSingleCore, 12);
                break;
            }
            if (!mbar_wait(p_ready(L, j & 1), (j >> 1) & 1u, abort_flag)) {
                if (lane == 0) report_wait_failure(status, abort_flag, kKidSingleCore, 5);
                break;
            }
            tc_fence_after_sync();
            const uint64_t vdesc = smem_desc_k_sw64(sb + C::kV + (vs * kLines + L) * C::kVSlot);
            if (lane == 0) {
                const uint32_t a_p = t_line + (j & 1) * kBK;
                mma_bf16_ts(t_line + C::kColO, a_p, vdesc, idesc_o, j != 0 ? 1u : 0u);
                mma_bf16_ts(t_line + C::kColO, a_p + 8u, vdesc + 2u, idesc_o, 1u);
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
        const bool line_valid = grp * kLines + L < rpb;
        const long long bb = sample_of(L);
        const uint32_t trow = tmem_base + ((uint32_t)(quad * 32) << 16) + L * 128;
        float* mbl = mbs + L * nkp;
        // Additive key mask of this sample, pre-scaled for exp2: inf * (mask - 1) * log2(e), -inf beyond N; one flag
        // per key block tells whether the block has any non-zero entry.
        {
            const int gt = (warp - 1 - kLines - 4 * L) * 32 + lane;  // 0..127 within the line's warps
            for (int base = 0; base < nkp; base += 128 * 8) {        // warp-uniform trip count (ballot below)
                const int c0 = base + gt * 8;
                const bool active = c0 < nkp;
                float v[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const int k = c0 + e;
                    float m = 1.0f;
                    if (mask != nullptr && k < N) m = __bfloat162float(mask[bb * N + k]);
                    v[e] = (k < N) ? inf * (m - 1.0f) * kLog2e : -INFINITY;
                }
                bool any = false;
#pragma unroll
                for (int e = 0; e < 8; ++e) any |= (v[e] != 0.f);
                if (active) {
                    *reinterpret_cast<float4*>(mbl + c0) = make_float4(v[0], v[1], v[2], v[3]);
                    *reinterpret_cast<float4*>(mbl + c0 + 4) = make_float4(v[4], v[5], v[6], v[7]);
                }
                const unsigned bal = __ballot_sync(0xffffffffu, any);
                if (active && (lane & 3) == 0) mbflag[L * 256 + (c0 >> 5)] = ((bal >> lane) & 0xFu) ? 1 : 0;
            }
            group_sync(1 + L, 128);
        }
        float m_used = 0.f;
        bool ok = true;
        for (int j = 0; j < nblk && ok; ++j) {
            const int s = j & 1;
            if (!mbar_wait(s_full(L, s), (j >> 1) & 1u, abort_flag)) {
                if (lane == 0) report_wait_failure(status, abort_flag, kKidSingleCore, 7);
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
            if (lane == 0) mbar_arrive(kb_empty(j % kSt));
            float sv[kBK];
#pragma unroll
            for (int e = 0; e < 32; ++e) sv[e] = __uint_as_float(sr[e]);
            if (mbflag[L * 256 + j]) {
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
                    if (lane == 0) report_wait_failure(status, abort_flag, kKidSingleCore, 8);
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                uint32_t orow[32];
                tmem_ld32(trow + C::kColO, orow);
                tmem_ld_wait();
#pragma unroll
                for (int e = 0; e < 32; ++e) orow[e] = __float_as_uint(__uint_as_float(orow[e]) * f);
                tmem_st32(trow + C::kColO, orow);
                if (DV > 32) {
                    uint32_t o2[16];
                    tmem_ld16(trow + C::kColO + 32, o2);
                    tmem_ld_wait();
#pragma unroll
                    for (int e = 0; e < 16; ++e) o2[e] = __float_as_uint(__uint_as_float(o2[e]) * f);
                    tmem_st16(trow + C::kColO + 32, o2);
                }
                const uint32_t lsum = tmem_ld1(trow + C::kColO + DV);   // the row sum rides in column kDV of O
                tmem_ld_wait();
                tmem_st1(trow + C::kColO + DV, __float_as_uint(__uint_as_float(lsum) * f));
                tmem_st_wait();
            }
            uint32_t pk[16];
            const float nm = -m_used;
#pragma unroll
            for (int e = 0; e < 32; e += 2) {
                add2(sv[e], sv[e + 1], nm, nm);
                pk[e >> 1] = pack_bf16x2(ex2_approx(sv[e]), ex2_approx(sv[e + 1]));
            }
            // P_j goes where S_j was: every thread of the warp has its S row in registers (the load above is
            // warp-wide), other warps own other lanes; the row sum is taken by the tensor pipe from the rounded P
            tmem_st16(trow + s * kBK, pk);
            tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_ready(L, s));
        }
        if (ok) {
            if (mbar_wait(pv_done(L, (nblk - 1) & 1), ((nblk - 1) >> 1) & 1u, abort_flag)) {
                tc_fence_after_sync();
                const uint32_t lsum = tmem_ld1(trow + C::kColO + DV);
                tmem_ld_wait();
                const float inv = 1.0f / __uint_as_float(lsum);
                const bool store = qpos < nq && line_valid;
                const long long off = (bb * nq + qpos) * (long long)(H * D) + h * D;
#pragma unroll
                for (int part = 0; part < DV / 16; ++part) {
                    uint32_t r[16];
                    tmem_ld16(trow + C::kColO + part * 16, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int v8 = 0; v8 < 2; ++v8) {
                        const int c0 = part * 16 + v8 * 8;
                        if (c0 < D && store) {
                            float fo[8];
#pragma unroll
                            for (int e = 0; e < 8; ++e) fo[e] = __uint_as_float(r[v8 * 8 + e]) * inv;
                            if (gate != nullptr) {
                                const uint4 gw = *reinterpret_cast<const uint4*>(gate + off + c0);
                                fo[0] *= sigmoidf_fast(bf16lo(gw.x)); fo[1] *= sigmoidf_fast(bf16hi(gw.x));
                                fo[2] *= sigmoidf_fast(bf16lo(gw.y)); fo[3] *= sigmoidf_fast(bf16hi(gw.y));
                                fo[4] *= sigmoidf_fast(bf16lo(gw.z)); fo[5] *= sigmoidf_fast(bf16hi(gw.z));
                                fo[6] *= sigmoidf_fast(bf16lo(gw.w)); fo[7] *= sigmoidf_fast(bf16hi(gw.w));
                            }
                            *reinterpret_cast<uint4*>(out + off + c0) =
                                make_uint4(pack_bf16x2(fo[0], fo[1]), pack_bf16x2(fo[2], fo[3]),
                                           pack_bf16x2(fo[4], fo[5]), pack_bf16x2(fo[6], fo[7]));
                        }
                    }
                }
            } else if (lane == 0) {
                report_wait_failure(status, abort_flag, kKidSingleCore, 10);
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

template <int D>
struct Images {
    size_t q, k, v, tb;  // bytes
    Images(int BB, int Bz, int N, int nq, int H) {
        const size_t n_qt = ceil_div(nq, kBQ), nkb = ceil_div(N, kBK);
        q = (size_t)BB * H * n_qt * Cfg<D>::kQBytes;
        k = (size_t)BB * H * nkb * Cfg<D>::kKBytes;
        v = (size_t)BB * H * nkb * Cfg<D>::kVBytes;
        tb = (size_t)Bz * H * nkb * nq * kBK * sizeof(bf16);
    }
};

template <int D>
int attn_tc_impl(const bf16* q, const bf16* k, const bf16* v, const bf16* g, const bf16* q_bias, const float* pb,
                 const bf16* mask, bf16* out, int BB, int N, int nq, int H, float inf, int rpb, Arena& ws,
                 cudaStream_t st, const bf16* z, const bf16* ln_z_w, const bf16* ln_z_b, const bf16* w_z,
                 const bf16* bias_tiles) {
    const int Bz = BB / rpb;
    const Images<D> im(BB, Bz, N, nq, H);
    bf16* q_img = (bf16*)ws.take(im.q);
    bf16* k_img = (bf16*)ws.take(im.k);
    bf16* v_img = (bf16*)ws.take(im.v);
    bf16* tb_img = (bf16*)ws.take(im.tb);
    if (!ws.base) return OF3_OK;
    OF3_REQUIRE(ws.ok(), OF3_ERR_WORKSPACE, "single attention: workspace too small (%zu needed)", ws.off);
    const int nkb = ceil_div(N, kBK), n_qt = ceil_div(nq, kBQ);
    constexpr int CH = Cfg<D>::kKD / 8;
    {
        const long long nq_chunks = (long long)BB * n_qt * kBQ * H * CH, nk_chunks = (long long)BB * nkb * kBK * H * CH;
        const long long most = nq_chunks > nk_chunks ? nq_chunks : nk_chunks;
        LaunchScope scope(kKidSingleAttn, st);
        single_pack_qk_kernel<D><<<dim3((unsigned)((most + 255) / 256), 2), 256, 0, st>>>(
            q, k, q_bias, q_img, k_img, BB, N, nq, H, kLog2e * rsqrtf((float)D));
    }
    {
        const size_t smem = (size_t)kBK * H * D * sizeof(bf16);
        OF3_CUDA_CHECK(cudaFuncSetAttribute(single_pack_v_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            (int)smem));
        LaunchScope scope(kKidSingleAttn, st);
        single_pack_v_kernel<D><<<dim3(nkb, BB), 256, smem, st>>>(v, v_img, N, H);
    }
    if (bias_tiles != nullptr) {
        tb_img = const_cast<bf16*>(bias_tiles);   // projected earlier, in this kernel's layout
    } else if (pb != nullptr) {
        LaunchScope scope(kKidSingleAttn, st);
        single_bias_kernel<<<dim3(nq, Bz * H), 256, 0, st>>>(pb, tb_img, N, nq, nkb);
    } else {   // straight from the pair tensor: no fp32 bias in between
        OF3_REQUIRE(z != nullptr && w_z != nullptr && nq == N && H == 16, OF3_ERR_ARG,
                    "single attention: neither a pair bias nor a whole pair tensor to project it from");
        const int rc = pair_bias_tiles_c128_h16(z, ln_z_w, ln_z_b, w_z, tb_img, Bz, N, st);
        if (rc) return rc;
    }
    OF3_CUDA_CHECK(cudaGetLastError());
    const uint32_t smem = Cfg<D>::dyn_bytes(nkb * kBK);
    // the size depends on N and function attributes are per device: set on every launch (a host-side store)
    OF3_CUDA_CHECK(cudaFuncSetAttribute(single_core_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const long long grid = (long long)Bz * H * n_qt * ceil_div(rpb, kLines);
    LaunchScope scope(kKidSingleCore, st);
    single_core_kernel<D><<<(unsigned)grid, kThreads, smem, st>>>(q_img, k_img, v_img, tb_img, mask, g, out, N, nq, H,
                                                                  rpb, inf, device_status_ptr());
    OF3_CUDA_CHECK(cudaGetLastError());
    return OF3_OK;
}

}  // namespace

// d in {24, 48}; H * d a multiple of 8 (16-byte rows per head); N within the mask row a CTA keeps.
bool single_attn_tc_supported(int N, int H, int d) {
    if (!(d == 24 || d == 48) || N < 1 || N > kMaxKeysSingle) return false;
    const size_t smem = d == 24 ? Cfg<24>::dyn_bytes(ceil_div(N, kBK) * kBK) : Cfg<48>::dyn_bytes(ceil_div(N, kBK) * kBK);
    return smem <= 227 * 1024 && (size_t)kBK * H * d * sizeof(bf16) <= 160 * 1024;
}

// Gated attention with pair bias over BB samples of N keys and nq query rows each:
//   out[bb, i, h, :] = sigmoid(g[bb, i, h, :]) * softmax_j((q[bb, i, h] + q_bias[h]) . k[bb, j, h] / sqrt(d)
//                                                       + inf * (mask[bb, j] - 1) + pair_bias[bb / rpb, h, i, j]) v
// q, g, out: [BB, nq, H*d]; k, v: [BB, N, H*d]; pair_bias fp32 [BB / rpb, H, nq, N]; mask [BB, N] or null.
// With ws.base == nullptr only the workspace need is accumulated.
int single_attn_tc(const bf16* q, const bf16* k, const bf16* v, const bf16* g, const bf16* q_bias,
                   const float* pair_bias, const bf16* mask, bf16* out, int BB, int N, int nq, int H, int d, float inf,
                   int rows_per_bias, Arena& ws, cudaStream_t st, const bf16* z, const bf16* ln_z_w, const bf16* ln_z_b,
                   const bf16* w_z, const bf16* bias_tiles) {
    OF3_REQUIRE(single_attn_tc_supported(N, H, d), OF3_ERR_SHAPE, "single attention: N %d, H %d, d %d not supported",
                N, H, d);
    OF3_REQUIRE(rows_per_bias > 0 && BB % rows_per_bias == 0, OF3_ERR_SHAPE,
                "single attention: %d samples do not divide into groups of %d", BB, rows_per_bias);
    return d == 24 ? attn_tc_impl<24>(q, k, v, g, q_bias, pair_bias, mask, out, BB, N, nq, H, inf, rows_per_bias, ws, st,
                                      z, ln_z_w, ln_z_b, w_z, bias_tiles)
                   : attn_tc_impl<48>(q, k, v, g, q_bias, pair_bias, mask, out, BB, N, nq, H, inf, rows_per_bias, ws, st,
                                      z, ln_z_w, ln_z_b, w_z, bias_tiles);
}

}  // namespace fast
}  // namespace of3
