// Single-track layers of the Pairformer block in bf16 (c_s = 384 in OpenFold3): attention with pair bias
// (LayerNorm variant) and the SwiGLU transition for widths without a fused row-tile kernel.
//
// The token dimension is tiny next to the pair tensor (N x 384 against N x N x 128), so these are
// launch/latency-bound chains, not roofline kernels. The linears run on the tcgen05 contraction
// kernel (activation rows x weight rows, both K-major), the attention keeps one head's K and V
// resident in shared memory, and everything in between is bf16 in HBM with fp32 arithmetic.
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
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
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

// ---------------------------------------------------------------- attention, one head resident
// grid (query chunks of 16, H, BB); 8 warps, each warp owns TWO queries (they share every K / V read).
// K and V of (bb, h) sit in shared memory as bf16 rows at a 16-byte-aligned pitch chosen so that eight
// lanes reading eight consecutive rows with 128-bit loads touch all 32 banks once (48 B for d = 24,
// 112 B for d = 48). A lane owns the keys lane, lane + 32, ...: logits, exponentials and the P V
// accumulation are lane-private (no shuffles per key); per chunk of 256 keys the warp agrees on the
// running maximum (one max-reduction), and the 2 x d partial outputs are summed over lanes once at the end.
// q, g, out and the pair bias hold nq query rows per sample (nq = N, or a window of the rows when the
// queries are split over ranks); k, v and the mask always hold all N keys.
constexpr int kQPB = 16;  // queries per block

template <int D>
struct AttnCfg {
    static constexpr int kPitch = (D == 24) ? 48 : 112;  // bytes per K / V row in shared memory
    static constexpr int kVec = D / 8;                    // 16-byte vectors per row
};

__device__ __forceinline__ void unpack8(const uint4& w, float* f) {
    f[0] = bf16lo(w.x); f[1] = bf16hi(w.x); f[2] = bf16lo(w.y); f[3] = bf16hi(w.y);
    f[4] = bf16lo(w.z); f[5] = bf16hi(w.z); f[6] = bf16lo(w.w); f[7] = bf16hi(w.w);
}

template <int D>
__global__ void __launch_bounds__(256, (D <= 24) ? 2 : 1)
single_attn_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v,
                   const bf16* __restrict__ g, const bf16* __restrict__ q_bias, const float* __restrict__ pair_bias,
                   const bf16* __restrict__ mask, bf16* __restrict__ out, int N, int nq, int H, float scale, float inf,
                   long long rows_per_bias, int passes) {
    constexpr int PB = AttnCfg<D>::kPitch, NV = AttnCfg<D>::kVec;
    constexpr int kChunk = 8;  // keys per lane between two agreements on the running maximum
    extern __shared__ __align__(16) uint8_t smem[];
    uint8_t* Ks = smem;
    uint8_t* Vs = Ks + (size_t)N * PB;
    float* mb = reinterpret_cast<float*>(Vs + (size_t)N * PB);  // additive key mask
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long bb = blockIdx.z;
    const int h = blockIdx.y;
    const int HD = H * D;
    for (int idx = threadIdx.x; idx < N * NV; idx += 256) {
        const int kk = idx / NV, c = idx % NV;
        const long long off = (bb * N + kk) * HD + h * D + c * 8;
        *reinterpret_cast<uint4*>(Ks + kk * PB + c * 16) = *reinterpret_cast<const uint4*>(k + off);
        *reinterpret_cast<uint4*>(Vs + kk * PB + c * 16) = *reinterpret_cast<const uint4*>(v + off);
    }
    const int npad = (N + 31) & ~31;
    for (int kk = threadIdx.x; kk < npad; kk += 256)
        mb[kk] = kk < N ? (mask ? inf * (__bfloat162float(mask[bb * N + kk]) - 1.0f) : 0.f) : -INFINITY;
    __syncthreads();

    // a block serves `passes` groups of 16 queries with one load of the head's K and V
    for (int pass = 0; pass < passes; ++pass) {
    const int qa = (blockIdx.x * passes + pass) * kQPB + warp * 2;  // this warp's queries qa, qa + 1
    if (qa >= nq) break;
    const bool has_b = qa + 1 < nq;
    const int qb = has_b ? qa + 1 : qa;
    const float* pb_base = pair_bias + ((bb / rows_per_bias) * H + h) * (long long)nq * N;
    const float* pba = pb_base + (long long)qa * N;
    const float* pbb = pb_base + (long long)qb * N;
    const long long offa = (bb * nq + qa) * HD + h * D, offb = (bb * nq + qb) * HD + h * D;
    float fa[D], fb[D];
#pragma unroll
    for (int c = 0; c < D; ++c) {
        const float bq = q_bias ? __bfloat162float(q_bias[h * D + c]) : 0.f;
        fa[c] = (__bfloat162float(q[offa + c]) + bq) * scale;
        fb[c] = (__bfloat162float(q[offb + c]) + bq) * scale;
    }
    float oa[D], ob[D];
#pragma unroll
    for (int c = 0; c < D; ++c) oa[c] = ob[c] = 0.f;
    float ma = -INFINITY, mbq = -INFINITY, la = 0.f, lb = 0.f;

    for (int k0 = 0; k0 < npad; k0 += 32 * kChunk) {
        float sa[kChunk], sb[kChunk];
        float cma = -INFINITY, cmb = -INFINITY;
#pragma unroll
        for (int i = 0; i < kChunk; ++i) {
            const int kk = k0 + i * 32 + lane;
            sa[i] = sb[i] = -INFINITY;
            if (kk < N) {
                float da = 0.f, db = 0.f;
#pragma unroll
                for (int c8 = 0; c8 < NV; ++c8) {
                    float kf[8];
                    unpack8(*reinterpret_cast<const uint4*>(Ks + kk * PB + c8 * 16), kf);
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        da = fmaf(fa[c8 * 8 + e], kf[e], da);
                        db = fmaf(fb[c8 * 8 + e], kf[e], db);
                    }
                }
                const float m = mb[kk];
                sa[i] = (da + m) + pba[kk];  // the reference's order: (q.k + mask bias) + pair bias
                sb[i] = (db + m) + pbb[kk];
            }
            cma = fmaxf(cma, sa[i]);
            cmb = fmaxf(cmb, sb[i]);
        }
        const float na = fmaxf(ma, warp_max(cma)), nb = fmaxf(mbq, warp_max(cmb));  // finite: key k0 exists
        const float ca = __expf(ma - na), cb = __expf(mbq - nb);                     // 0 on the first chunk
        ma = na;
        mbq = nb;
        la *= ca;
        lb *= cb;
#pragma unroll
        for (int c = 0; c < D; ++c) {
            oa[c] *= ca;
            ob[c] *= cb;
        }
#pragma unroll
        for (int i = 0; i < kChunk; ++i) {
            const int kk = k0 + i * 32 + lane;
            if (kk < N) {
                const float pa = __expf(sa[i] - ma), pq = __expf(sb[i] - mbq);
                la += pa;
                lb += pq;
#pragma unroll
                for (int c8 = 0; c8 < NV; ++c8) {
                    float vf[8];
                    unpack8(*reinterpret_cast<const uint4*>(Vs + kk * PB + c8 * 16), vf);
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        oa[c8 * 8 + e] = fmaf(pa, vf[e], oa[c8 * 8 + e]);
                        ob[c8 * 8 + e] = fmaf(pq, vf[e], ob[c8 * 8 + e]);
                    }
                }
            }
        }
    }
    la = warp_sum(la);
    lb = warp_sum(lb);
    float ra = 0.f, rb = 0.f;  // lane c keeps output dim c (and c + 32 for d = 48)
    float ra2 = 0.f, rb2 = 0.f;
#pragma unroll
    for (int c = 0; c < D; ++c) {
        const float ta = warp_sum(oa[c]), tb = warp_sum(ob[c]);
        if (c < 32) {
            if (lane == c) { ra = ta; rb = tb; }
        } else {
            if (lane == c - 32) { ra2 = ta; rb2 = tb; }
        }
    }
    const float ia = 1.0f / la, ib = 1.0f / lb;
    if (lane < D) {
        float r = ra * ia;
        if (g) r *= 1.0f / (1.0f + __expf(-__bfloat162float(g[offa + lane])));
        out[offa + lane] = __float2bfloat16_rn(r);
        if (has_b) {
            float r2 = rb * ib;
            if (g) r2 *= 1.0f / (1.0f + __expf(-__bfloat162float(g[offb + lane])));
            out[offb + lane] = __float2bfloat16_rn(r2);
        }
    }
    if (D > 32 && lane + 32 < D) {
        float r = ra2 * ia;
        if (g) r *= 1.0f / (1.0f + __expf(-__bfloat162float(g[offa + lane + 32])));
        out[offa + lane + 32] = __float2bfloat16_rn(r);
        if (has_b) {
            float r2 = rb2 * ib;
            if (g) r2 *= 1.0f / (1.0f + __expf(-__bfloat162float(g[offb + lane + 32])));
            out[offb + lane + 32] = __float2bfloat16_rn(r2);
        }
    }
    }  // passes
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

template <int D>
int launch_attn(const bf16* q, const bf16* k, const bf16* v, const bf16* g, const bf16* q_bias, const float* pb,
                const bf16* mask, bf16* out, int BB, int N, int nq, int H, float inf, long long rows_per_bias,
                cudaStream_t st) {
    const size_t smem = (size_t)N * AttnCfg<D>::kPitch * 2 + (size_t)((N + 31) & ~31) * 4;
    // the limit depends on N and function attributes are per device: set on every launch (a host-side store)
    OF3_CUDA_CHECK(cudaFuncSetAttribute(single_attn_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)smem));
    // enough blocks for a few waves, as few loads of K / V as that allows
    int passes = 1;
    while (passes < 8 && (long long)ceil_div(nq, kQPB * passes * 2) * H * BB >= 4LL * sm_count()) passes *= 2;
    dim3 grid(ceil_div(nq, kQPB * passes), H, BB);
    LaunchScope scope(kKidSingle, st);
    single_attn_kernel<D><<<grid, 256, smem, st>>>(q, k, v, g, q_bias, pb, mask, out, N, nq, H, rsqrtf((float)D),
                                                   inf, rows_per_bias, passes);
    OF3_CUDA_CHECK(cudaGetLastError());
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
    if ((rc = linear_bf16(t_sn, w_g, t_g, rows, c_a, c_s, st))) return rc;
    if ((rc = linear_bf16(t_sn, w_s, t_s, rows, c_a, c_s, st))) return rc;
    {
        LaunchScope scope(kKidSingle, st);
        const long long n2 = rows * c_a / 2;
        ada_combine_bf16_kernel<<<(unsigned)((n2 + 255) / 256), 256, 0, st>>>(t_g, b_g, an, t_s, an, rows * c_a, c_a);
    }
    OF3_CUDA_CHECK(cudaGetLastError());
    return OF3_OK;
}

}  // namespace

// bf16, LayerNorm variant, one pair tensor per sample; c_a = H * d a multiple of 64; d in {24, 48};
// K and V of one head must fit in shared memory.
bool attn_pair_bias_supported(int Ba, int Bz, int N, int c_a, int c_s, int c_z, int H, int d, int flags) {
    if (flags & OF3_FLAG_FORCE_GENERIC) return false;
    if ((flags & OF3_FLAG_ADA_LN) && (c_s <= 0 || c_s % 64 != 0)) return false;
    if (!(d == 24 || d == 48) || H * d != c_a || c_a % 64 != 0) return false;
    if (c_z != 128 || H != 16 || Bz <= 0 || Ba % Bz != 0) return false;
    return (size_t)N * (d == 24 ? 48 : 112) * 2 + (size_t)N * 4 + 1024 <= 200 * 1024;
}

int attn_pair_bias(const bf16* a, const bf16* z, const bf16* s, const bf16* mask, bf16* out, int Ba, int Bz, int N,
                   int c_a, int c_s, int H, int d, float inf, int flags, const of3_attn_pair_bias_params* p, Arena& ws,
                   cudaStream_t st, const float* pair_bias) {
    const long long rows = (long long)Ba * N;
    const bool ada = (flags & OF3_FLAG_ADA_LN) != 0;
    bf16* t_sn = ada ? (bf16*)ws.take(rows * c_s * sizeof(bf16)) : nullptr;
    bf16* t_g = ada ? (bf16*)ws.take(rows * c_a * sizeof(bf16)) : nullptr;
    bf16* t_s = ada ? (bf16*)ws.take(rows * c_a * sizeof(bf16)) : nullptr;
    bf16* an = (bf16*)ws.take(rows * c_a * sizeof(bf16));
    bf16* q = (bf16*)ws.take(rows * c_a * sizeof(bf16));
    bf16* k = (bf16*)ws.take(rows * c_a * sizeof(bf16));
    bf16* v = (bf16*)ws.take(rows * c_a * sizeof(bf16));
    bf16* g = (bf16*)ws.take(rows * c_a * sizeof(bf16));
    bf16* og = (bf16*)ws.take(rows * c_a * sizeof(bf16));
    bf16* y = (bf16*)ws.take(rows * c_a * sizeof(bf16));
    float* zb = (float*)ws.take((size_t)Bz * H * N * N * sizeof(float));
    if (!ws.base) return OF3_OK;
    OF3_REQUIRE(ws.ok(), OF3_ERR_WORKSPACE, "attn_pair_bias: workspace too small (%zu needed)", ws.off);
    int rc;
    if (pair_bias == nullptr) {
        if ((rc = fast::pair_bias_c128_h16(z, (const bf16*)p->ln_z_w, (const bf16*)p->ln_z_b, (const bf16*)p->w_z, zb,
                                           Bz, (long long)N * N, st)))
            return rc;
        pair_bias = zb;
    }
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
    if ((rc = linear_bf16(an, (const bf16*)p->w_q, q, rows, c_a, c_a, st))) return rc;
    if ((rc = linear_bf16(an, (const bf16*)p->w_k, k, rows, c_a, c_a, st))) return rc;
    if ((rc = linear_bf16(an, (const bf16*)p->w_v, v, rows, c_a, c_a, st))) return rc;
    if ((rc = linear_bf16(an, (const bf16*)p->w_g, g, rows, c_a, c_a, st))) return rc;
    const long long rpb = Ba / Bz;
    if (d == 24)
        rc = launch_attn<24>(q, k, v, g, (const bf16*)p->b_q, pair_bias, mask, og, Ba, N, N, H, inf, rpb, st);
    else
        rc = launch_attn<48>(q, k, v, g, (const bf16*)p->b_q, pair_bias, mask, og, Ba, N, N, H, inf, rpb, st);
    if (rc) return rc;
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
    bf16* t_g = (bf16*)ws.take(rows * c_a * sizeof(bf16));
    bf16* t_s = (bf16*)ws.take(rows * c_a * sizeof(bf16));
    bf16* ha = (bf16*)ws.take(rows * hid * sizeof(bf16));
    bf16* hb = (bf16*)ws.take(rows * hid * sizeof(bf16));
    if (!ws.base) return OF3_OK;
    OF3_REQUIRE(ws.ok(), OF3_ERR_WORKSPACE, "cond_transition: workspace too small (%zu needed)", ws.off);
    int rc;
    if ((rc = ada_ln_bf16(a, s, an, t_sn, t_g, t_s, rows, c_a, c_s, (const bf16*)p->ada_ln_s_w, (const bf16*)p->ada_w_g,
                          (const bf16*)p->ada_b_g, (const bf16*)p->ada_w_s, st)))
        return rc;
    if ((rc = linear_bf16(an, (const bf16*)p->w_a, ha, rows, hid, c_a, st))) return rc;
    if ((rc = linear_bf16(an, (const bf16*)p->w_b, hb, rows, hid, c_a, st))) return rc;
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
    bf16* k = (bf16*)ws.take((size_t)N * c_a * sizeof(bf16));
    bf16* v = (bf16*)ws.take((size_t)N * c_a * sizeof(bf16));
    bf16* q = (bf16*)ws.take((size_t)R * c_a * sizeof(bf16));
    bf16* g = (bf16*)ws.take((size_t)R * c_a * sizeof(bf16));
    bf16* og = (bf16*)ws.take((size_t)R * c_a * sizeof(bf16));
    bf16* y = (bf16*)ws.take((size_t)R * c_a * sizeof(bf16));
    if (!ws.base) return OF3_OK;
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
    if ((rc = linear_bf16(an, (const bf16*)p->w_k, k, N, c_a, c_a, st))) return rc;
    if ((rc = linear_bf16(an, (const bf16*)p->w_v, v, N, c_a, c_a, st))) return rc;
    if ((rc = linear_bf16(an_w, (const bf16*)p->w_q, q, R, c_a, c_a, st))) return rc;
    if ((rc = linear_bf16(an_w, (const bf16*)p->w_g, g, R, c_a, c_a, st))) return rc;
    if (d == 24)
        rc = launch_attn<24>(q, k, v, g, (const bf16*)p->b_q, pair_bias_rows, mask, og, 1, N, R, H, inf, 1, st);
    else
        rc = launch_attn<48>(q, k, v, g, (const bf16*)p->b_q, pair_bias_rows, mask, og, 1, N, R, H, inf, 1, st);
    if (rc) return rc;
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
    bf16* ha = (bf16*)ws.take(rows * hid * sizeof(bf16));
    bf16* hb = (bf16*)ws.take(rows * hid * sizeof(bf16));
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
    if ((rc = linear_bf16(xn, (const bf16*)p->w_a, ha, rows, hid, c, st))) return rc;
    if ((rc = linear_bf16(xn, (const bf16*)p->w_b, hb, rows, hid, c, st))) return rc;
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
