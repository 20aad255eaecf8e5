// Single-track layers of the Pairformer block in bf16 (c_s = 384 in OpenFold3): attention with pair bias
// (LayerNorm variant) and the SwiGLU transition for widths without a fused row-tile kernel.
//
// The token dimension is tiny next to the pair tensor (N x 384 against N x N x 128), so these are
// launch/latency-bound chains, not roofline kernels. The linears run on the tcgen05 contraction
// kernel (activation rows x weight rows, both K-major), the attention on the streaming tensor-pipe
// kernel of fast_single_attn.cu, and everything in between is bf16 in HBM with fp32 arithmetic.
// Reference: openfold3/core/model/layers/attention_pair_bias.py:123-227,
//            openfold3/core/model/primitives/attention.py:94-135, 270-310,
//            openfold3/core/model/layers/transition.py:225-271.
#include "generic_ops.cuh"
#include "modules.cuh"
#include "runtime.cuh"

namespace of3 {
namespace fast {
namespace {

typedef __nv_bfloat16 bf16;
constexpr int kKidSingle = 8;
constexpr int kKidLinear = 10;  // linear layers on the contraction kernel: accounted apart from the triangle einsum

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
// ---------------------------------------------------------------- LayerNorm rows -> bf16
__global__ void __launch_bounds__(256) ln_rows_kernel(const bf16* __restrict__ x, const bf16* __restrict__ gamma,
                                                      const bf16* __restrict__ beta, bf16* __restrict__ y,
                                                      long long rows, int C) {
    const int lane = threadIdx.x & 31;
    const long long r = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (r >= rows) return;
    const bf16* xr = x + r * C;
    float s = 0.f;
    for (int c = lane; c < C; c += 32) s += __bfloat162float(xr[c]);
    const float mean = warp_sum(s) / (float)C;
    float v = 0.f;
    for (int c = lane; c < C; c += 32) {
        const float d = __bfloat162float(xr[c]) - mean;
        v += d * d;
    }
    const float rstd = rsqrtf(warp_sum(v) / (float)C + 1e-5f);
    for (int c = lane; c < C; c += 32) {
        float o = (__bfloat162float(xr[c]) - mean) * rstd;
        if (gamma) o *= __bfloat162float(gamma[c]);
        if (beta) o += __bfloat162float(beta[c]);
        y[r * C + c] = __float2bfloat16_rn(o);
    }
}

// ---------------------------------------------------------------- elementwise
__global__ void silu_mul_bf16_kernel(const bf16* __restrict__ a, const bf16* __restrict__ b, bf16* __restrict__ dst,
                                     long long n) {
    const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 2;
    if (i >= n) return;
    const uint32_t av = *reinterpret_cast<const uint32_t*>(a + i), bv = *reinterpret_cast<const uint32_t*>(b + i);
    const float a0 = bf16lo(av), a1 = bf16hi(av);
    const float h0 = a0 / (1.0f + __expf(-a0)) * bf16lo(bv);
    const float h1 = a1 / (1.0f + __expf(-a1)) * bf16hi(bv);
    *reinterpret_cast<uint32_t*>(dst + i) = pack_bf16x2(h0, h1);
}
// out[r, :] = (residual ? residual[r, :] : 0) + upd[r, :] * (mask ? mask[r] : 1)
__global__ void residual_bf16_kernel(const bf16* __restrict__ upd, const bf16* residual, const bf16* __restrict__ mask,
                                     bf16* out, long long rows, int C) {
    const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 2;
    if (i >= rows * C) return;
    const long long r = i / C;
    const float mk = mask ? __bfloat162float(mask[r]) : 1.0f;
    const uint32_t u = *reinterpret_cast<const uint32_t*>(upd + i);
    float v0 = bf16lo(u) * mk, v1 = bf16hi(u) * mk;
    if (residual) {
        const uint32_t z = *reinterpret_cast<const uint32_t*>(residual + i);
        v0 += bf16lo(z);
        v1 += bf16hi(z);
    }
    *reinterpret_cast<uint32_t*>(out + i) = pack_bf16x2(v0, v1);
}

// AdaLN combine (normalization.py:121-140): dst = sigmoid(g_lin + b_g[c]) * ln_a + s_lin
__global__ void ada_combine_bf16_kernel(const bf16* __restrict__ g_lin, const bf16* __restrict__ b_g,
                                        const bf16* __restrict__ ln_a, const bf16* __restrict__ s_lin,
                                        bf16* __restrict__ dst, long long n, int C) {
    const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 2;
    if (i >= n) return;
    const int c = (int)(i % C);
    const uint32_t gv = *reinterpret_cast<const uint32_t*>(g_lin + i), av = *reinterpret_cast<const uint32_t*>(ln_a + i);
    const uint32_t sv = *reinterpret_cast<const uint32_t*>(s_lin + i), bv = *reinterpret_cast<const uint32_t*>(b_g + c);
    const float r0 = bf16lo(av) / (1.0f + __expf(-(bf16lo(gv) + bf16lo(bv)))) + bf16lo(sv);
    const float r1 = bf16hi(av) / (1.0f + __expf(-(bf16hi(gv) + bf16hi(bv)))) + bf16hi(sv);
    *reinterpret_cast<uint32_t*>(dst + i) = pack_bf16x2(r0, r1);
}
// out[r, c] = (residual ? residual[r, c] : 0) + sigmoid(gate_lin[r, c] + gate_b[c]) * upd[r, c] * (mask ? mask[r] : 1)
__global__ void gate_residual_bf16_kernel(const bf16* __restrict__ upd, const bf16* __restrict__ gate_lin,
                                          const bf16* __restrict__ gate_b, const bf16* residual,
                                          const bf16* __restrict__ mask, bf16* out, long long rows, int C) {
    const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 2;
    if (i >= rows * C) return;
    const long long r = i / C;
    const int c = (int)(i - r * C);
    const float mk = mask ? __bfloat162float(mask[r]) : 1.0f;
    const uint32_t u = *reinterpret_cast<const uint32_t*>(upd + i), gv = *reinterpret_cast<const uint32_t*>(gate_lin + i);
    const uint32_t bv = *reinterpret_cast<const uint32_t*>(gate_b + c);
    float v0 = bf16lo(u) * mk / (1.0f + __expf(-(bf16lo(gv) + bf16lo(bv))));
    float v1 = bf16hi(u) * mk / (1.0f + __expf(-(bf16hi(gv) + bf16hi(bv))));
    if (residual) {
        const uint32_t z = *reinterpret_cast<const uint32_t*>(residual + i);
        v0 += bf16lo(z);
        v1 += bf16hi(z);
    }
    *reinterpret_cast<uint32_t*>(out + i) = pack_bf16x2(v0, v1);
}

int linear_bf16(const bf16* x, const bf16* w, bf16* y, long long rows, int out_dim, int in_dim, cudaStream_t st) {
    return contract_nt_bf16(x, w, y, 1, (int)rows, out_dim, in_dim, in_dim, in_dim, out_dim, rows * in_dim,
                            (long long)out_dim * in_dim, rows * out_dim, st, 0, 0, kKidLinear);
}

// `count` linear layers of equal shape on ONE input: y[i] = x w[i]^T with w[i] = w[0] + i * out_dim * in_dim and
// y[i] = y[0] + i * rows * out_dim. One launch when the caller's weights lie back to back in memory (the Python
// modules pack them that way), one launch per layer otherwise.
int linear_group_bf16(const bf16* x, const bf16* const* w, bf16* y, int count, long long rows, int out_dim, int in_dim,
                      cudaStream_t st) {
    const long long w_elems = (long long)out_dim * in_dim;
    bool adjacent = true;
    for (int i = 1; i < count; ++i) adjacent = adjacent && (w[i] == w[0] + i * w_elems);
    if (adjacent && count > 1)
        return contract_nt_bf16(x, w[0], y, count, (int)rows, out_dim, in_dim, in_dim, in_dim, out_dim, 0, w_elems,
                                rows * out_dim, st, 0, 0, kKidLinear);
    for (int i = 0; i < count; ++i) {
        const int rc = linear_bf16(x, w[i], y + i * rows * out_dim, rows, out_dim, in_dim, st);
        if (rc) return rc;
    }
    return OF3_OK;
}

// an = AdaLN(a, s) (normalization.py:89-140): LN(a) without affine, LN_s(s) with scale only, two linears
// from it, combine. t_ln / t_sn / t_g / t_s: scratch [rows, c_a], [rows, c_s], [rows, c_a], [rows, c_a].
int ada_ln_bf16(const bf16* a, const bf16* s, bf16* an, bf16* t_sn, bf16* t_g, bf16* t_s, long long rows, int c_a,
                int c_s, const bf16* ln_s_w, const bf16* w_g, const bf16* b_g, const bf16* w_s, cudaStream_t st) {
    {
        LaunchScope scope(kKidSingle, st);
        ln_rows_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(a, nullptr, nullptr, an, rows, c_a);
    }
    {
        LaunchScope scope(kKidSingle, st);
        ln_rows_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(s, ln_s_w, nullptr, t_sn, rows, c_s);
    }
    OF3_CUDA_CHECK(cudaGetLastError());
    int rc;
    if (t_s == t_g + rows * c_a) {   // the two projections of LN_s(s) as one launch
        const bf16* w2[2] = {w_g, w_s};
        if ((rc = linear_group_bf16(t_sn, w2, t_g, 2, rows, c_a, c_s, st))) return rc;
    } else {
        if ((rc = linear_bf16(t_sn, w_g, t_g, rows, c_a, c_s, st))) return rc;
        if ((rc = linear_bf16(t_sn, w_s, t_s, rows, c_a, c_s, st))) return rc;
    }
    {
        LaunchScope scope(kKidSingle, st);
        const long long n2 = rows * c_a / 2;
        ada_combine_bf16_kernel<<<(unsigned)((n2 + 255) / 256), 256, 0, st>>>(t_g, b_g, an, t_s, an, rows * c_a, c_a);
    }
    OF3_CUDA_CHECK(cudaGetLastError());
    return OF3_OK;
}

}  // namespace

// bf16, one pair tensor per group of samples; c_a = H * d a multiple of 64; d in {24, 48}.
bool attn_pair_bias_supported(int Ba, int Bz, int N, int c_a, int c_s, int c_z, int H, int d, int flags) {
    if (flags & OF3_FLAG_FORCE_GENERIC) return false;
    if ((flags & OF3_FLAG_ADA_LN) && (c_s <= 0 || c_s % 64 != 0)) return false;
    if (!(d == 24 || d == 48) || H * d != c_a || c_a % 64 != 0) return false;
    if (c_z != 128 || H != 16 || Bz <= 0 || Ba % Bz != 0) return false;
    return single_attn_tc_supported(N, H, d);
}

int attn_pair_bias(const bf16* a, const bf16* z, const bf16* s, const bf16* mask, bf16* out, int Ba, int Bz, int N,
                   int c_a, int c_s, int H, int d, float inf, int flags, const of3_attn_pair_bias_params* p, Arena& ws,
                   cudaStream_t st, const float* pair_bias, const bf16* bias_tiles) {
    const long long rows = (long long)Ba * N;
    const bool ada = (flags & OF3_FLAG_ADA_LN) != 0;
    bf16* t_sn = ada ? (bf16*)ws.take(rows * c_s * sizeof(bf16)) : nullptr;
    bf16* t_g = ada ? (bf16*)ws.take(2 * rows * c_a * sizeof(bf16)) : nullptr;   // t_g, t_s back to back
    bf16* t_s = ada ? t_g + rows * c_a : nullptr;
    bf16* an = (bf16*)ws.take(rows * c_a * sizeof(bf16));
    bf16* q = (bf16*)ws.take(4 * rows * c_a * sizeof(bf16));   // q, g, k, v back to back
    bf16* g = q + rows * c_a;
    bf16* k = g + rows * c_a;
    bf16* v = k + rows * c_a;
    bf16* og = (bf16*)ws.take(rows * c_a * sizeof(bf16));
    bf16* y = (bf16*)ws.take(rows * c_a * sizeof(bf16));
    float* zb = (float*)ws.take((size_t)Bz * H * N * N * sizeof(float));
    if (!ws.base)   // sizing pass: the operand images of the attention come last
        return single_attn_tc(nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, Ba, N, N, H, d, inf,
                              Ba / Bz, ws, st);
    OF3_REQUIRE(ws.ok(), OF3_ERR_WORKSPACE, "attn_pair_bias: workspace too small (%zu needed)", ws.off);
    int rc;
    (void)zb;   // pair_bias == nullptr: the attention projects its bias tiles straight from z (no fp32 bias tensor)
    if (ada) {
        if ((rc = ada_ln_bf16(a, s, an, t_sn, t_g, t_s, rows, c_a, c_s, (const bf16*)p->ada_ln_s_w,
                              (const bf16*)p->ada_w_g, (const bf16*)p->ada_b_g, (const bf16*)p->ada_w_s, st)))
            return rc;
    } else {
        LaunchScope scope(kKidSingle, st);
        ln_rows_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(a, (const bf16*)p->ln_a_w, (const bf16*)p->ln_a_b,
                                                                   an, rows, c_a);
    }
    OF3_CUDA_CHECK(cudaGetLastError());
    {
        const bf16* w4[4] = {(const bf16*)p->w_q, (const bf16*)p->w_g, (const bf16*)p->w_k, (const bf16*)p->w_v};
        if ((rc = linear_group_bf16(an, w4, q, 4, rows, c_a, c_a, st))) return rc;
    }
    if ((rc = single_attn_tc(q, k, v, g, (const bf16*)p->b_q, pair_bias, mask, og, Ba, N, N, H, d, inf, Ba / Bz, ws, st,
                             z, (const bf16*)p->ln_z_w, (const bf16*)p->ln_z_b, (const bf16*)p->w_z, bias_tiles)))
        return rc;
    if ((rc = linear_bf16(og, (const bf16*)p->w_o, y, rows, c_a, c_a, st))) return rc;
    if (ada) {  // output gate from the raw conditioning: sigmoid(linear_ada_out(s)) * y
        if ((rc = linear_bf16(s, (const bf16*)p->w_ada_out, t_g, rows, c_a, c_s, st))) return rc;
        LaunchScope scope(kKidSingle, st);
        const long long n2 = rows * c_a / 2;
        gate_residual_bf16_kernel<<<(unsigned)((n2 + 255) / 256), 256, 0, st>>>(
            y, t_g, (const bf16*)p->b_ada_out, (flags & OF3_FLAG_ADD_RESIDUAL) ? a : nullptr, nullptr, out, rows, c_a);
    } else {
        LaunchScope scope(kKidSingle, st);
        const long long n2 = rows * c_a / 2;
        residual_bf16_kernel<<<(unsigned)((n2 + 255) / 256), 256, 0, st>>>(
            y, (flags & OF3_FLAG_ADD_RESIDUAL) ? a : nullptr, nullptr, out, rows, c_a);
    }
    OF3_CUDA_CHECK(cudaGetLastError());
    return OF3_OK;
}

// ConditionedTransitionBlock (transition.py:325-339): AdaLN -> SwiGLU -> linear_out, gated by sigmoid(linear_g(s)).
bool cond_transition_supported(int c_a, int c_s, int n, int flags) {
    return !(flags & OF3_FLAG_FORCE_GENERIC) && c_a % 64 == 0 && c_s % 64 == 0 && (n * c_a) % 64 == 0;
}
int cond_transition(const bf16* a, const bf16* s, const bf16* mask, bf16* out, long long rows, int c_a, int c_s, int n,
                    int flags, const of3_cond_transition_params* p, Arena& ws, cudaStream_t st) {
    const int hid = n * c_a;
    bf16* an = (bf16*)ws.take(rows * c_a * sizeof(bf16));
    bf16* t_sn = (bf16*)ws.take(rows * c_s * sizeof(bf16));
    bf16* t_g = (bf16*)ws.take(2 * rows * c_a * sizeof(bf16));   // t_g, t_s back to back
    bf16* t_s = t_g + rows * c_a;
    bf16* ha = (bf16*)ws.take(2 * rows * hid * sizeof(bf16));    // ha, hb back to back
    bf16* hb = ha + rows * hid;
    if (!ws.base) return OF3_OK;
    OF3_REQUIRE(ws.ok(), OF3_ERR_WORKSPACE, "cond_transition: workspace too small (%zu needed)", ws.off);
    int rc;
    if ((rc = ada_ln_bf16(a, s, an, t_sn, t_g, t_s, rows, c_a, c_s, (const bf16*)p->ada_ln_s_w, (const bf16*)p->ada_w_g,
                          (const bf16*)p->ada_b_g, (const bf16*)p->ada_w_s, st)))
        return rc;
    {
        const bf16* w2[2] = {(const bf16*)p->w_a, (const bf16*)p->w_b};
        if ((rc = linear_group_bf16(an, w2, ha, 2, rows, hid, c_a, st))) return rc;
    }
    {
        LaunchScope scope(kKidSingle, st);
        const long long n2 = rows * hid / 2;
        silu_mul_bf16_kernel<<<(unsigned)((n2 + 255) / 256), 256, 0, st>>>(ha, hb, ha, rows * hid);
    }
    OF3_CUDA_CHECK(cudaGetLastError());
    if ((rc = linear_bf16(ha, (const bf16*)p->w_out, t_s, rows, c_a, hid, st))) return rc;
    if ((rc = linear_bf16(s, (const bf16*)p->w_g, t_g, rows, c_a, c_s, st))) return rc;
    {
        LaunchScope scope(kKidSingle, st);
        const long long n2 = rows * c_a / 2;
        gate_residual_bf16_kernel<<<(unsigned)((n2 + 255) / 256), 256, 0, st>>>(
            t_s, t_g, (const bf16*)p->b_g, (flags & OF3_FLAG_ADD_RESIDUAL) ? a : nullptr, mask, out, rows, c_a);
    }
    OF3_CUDA_CHECK(cudaGetLastError());
    return OF3_OK;
}

// The same layer for a window of R query rows [row0, row0 + R) of one sample: keys and values come from
// all N rows of `a`, queries / gate / output only from the window; pair_bias_rows is [H][R][N] (the
// projected pair bias of exactly those rows) and out_rows is [R][c_a]. Used when the pair tensor, and
// with it the pair bias, is split by rows over several GPUs.
int attn_pair_bias_rows(const bf16* a, const float* pair_bias_rows, const bf16* mask, bf16* out_rows, int N, int row0,
                        int R, int c_a, int H, int d, float inf, int flags, const of3_attn_pair_bias_params* p,
                        Arena& ws, cudaStream_t st) {
    bf16* an = (bf16*)ws.take((size_t)N * c_a * sizeof(bf16));
    bf16* k = (bf16*)ws.take((size_t)2 * N * c_a * sizeof(bf16));   // k, v back to back
    bf16* v = k + (size_t)N * c_a;
    bf16* q = (bf16*)ws.take((size_t)2 * R * c_a * sizeof(bf16));   // q, g back to back
    bf16* g = q + (size_t)R * c_a;
    bf16* og = (bf16*)ws.take((size_t)R * c_a * sizeof(bf16));
    bf16* y = (bf16*)ws.take((size_t)R * c_a * sizeof(bf16));
    if (!ws.base)
        return single_attn_tc(nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, 1, N, R, H, d, inf, 1,
                              ws, st);
    OF3_REQUIRE(ws.ok(), OF3_ERR_WORKSPACE, "attn_pair_bias_rows: workspace too small (%zu needed)", ws.off);
    OF3_REQUIRE(row0 >= 0 && R > 0 && row0 + R <= N, OF3_ERR_ARG, "attn_pair_bias_rows: window [%d, %d) outside %d rows",
                row0, row0 + R, N);
    int rc;
    {
        LaunchScope scope(kKidSingle, st);
        ln_rows_kernel<<<(unsigned)((N + 7) / 8), 256, 0, st>>>(a, (const bf16*)p->ln_a_w, (const bf16*)p->ln_a_b, an, N,
                                                                c_a);
    }
    OF3_CUDA_CHECK(cudaGetLastError());
    const bf16* an_w = an + (long long)row0 * c_a;
    {
        const bf16* wkv[2] = {(const bf16*)p->w_k, (const bf16*)p->w_v};
        const bf16* wqg[2] = {(const bf16*)p->w_q, (const bf16*)p->w_g};
        if ((rc = linear_group_bf16(an, wkv, k, 2, N, c_a, c_a, st))) return rc;
        if ((rc = linear_group_bf16(an_w, wqg, q, 2, R, c_a, c_a, st))) return rc;
    }
    if ((rc = single_attn_tc(q, k, v, g, (const bf16*)p->b_q, pair_bias_rows, mask, og, 1, N, R, H, d, inf, 1, ws, st)))
        return rc;
    if ((rc = linear_bf16(og, (const bf16*)p->w_o, y, R, c_a, c_a, st))) return rc;
    {
        LaunchScope scope(kKidSingle, st);
        const long long n2 = (long long)R * c_a / 2;
        residual_bf16_kernel<<<(unsigned)((n2 + 255) / 256), 256, 0, st>>>(
            y, (flags & OF3_FLAG_ADD_RESIDUAL) ? a + (long long)row0 * c_a : nullptr, nullptr, out_rows, R, c_a);
    }
    OF3_CUDA_CHECK(cudaGetLastError());
    return OF3_OK;
}

// SwiGLU transition for widths without the fused row-tile kernel (bf16, c and n*c multiples of 64).
bool transition_wide_supported(int c, int n) { return c % 64 == 0 && !(c == 128 && n == 4); }

int transition_wide(const bf16* x, const bf16* mask, bf16* out, long long rows, int c, int n, int flags,
                    const of3_transition_params* p, Arena& ws, cudaStream_t st) {
    const int hid = n * c;
    bf16* xn = (bf16*)ws.take(rows * c * sizeof(bf16));
    bf16* ha = (bf16*)ws.take(2 * rows * hid * sizeof(bf16));   // ha, hb back to back
    bf16* hb = ha + rows * hid;
    bf16* y = (bf16*)ws.take(rows * c * sizeof(bf16));
    if (!ws.base) return OF3_OK;
    OF3_REQUIRE(ws.ok(), OF3_ERR_WORKSPACE, "transition: workspace too small (%zu needed)", ws.off);
    OF3_REQUIRE(rows < (1LL << 31), OF3_ERR_SHAPE, "transition: too many rows");
    int rc;
    {
        LaunchScope scope(kKidSingle, st);
        ln_rows_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(x, (const bf16*)p->ln_w, (const bf16*)p->ln_b, xn,
                                                                   rows, c);
    }
    OF3_CUDA_CHECK(cudaGetLastError());
    {
        const bf16* w2[2] = {(const bf16*)p->w_a, (const bf16*)p->w_b};
        if ((rc = linear_group_bf16(xn, w2, ha, 2, rows, hid, c, st))) return rc;
    }
    {
        LaunchScope scope(kKidSingle, st);
        const long long n2 = rows * hid / 2;
        silu_mul_bf16_kernel<<<(unsigned)((n2 + 255) / 256), 256, 0, st>>>(ha, hb, ha, rows * hid);
    }
    OF3_CUDA_CHECK(cudaGetLastError());
    if ((rc = linear_bf16(ha, (const bf16*)p->w_out, y, rows, c, hid, st))) return rc;
    {
        LaunchScope scope(kKidSingle, st);
        const long long n2 = rows * c / 2;
        residual_bf16_kernel<<<(unsigned)((n2 + 255) / 256), 256, 0, st>>>(
            y, (flags & OF3_FLAG_ADD_RESIDUAL) ? x : nullptr, mask, out, rows, c);
    }
    OF3_CUDA_CHECK(cudaGetLastError());
    return OF3_OK;
}

}  // namespace fast
}  // namespace of3
