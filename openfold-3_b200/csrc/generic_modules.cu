// Module-level compositions of the shape-generic kernels (fp32 validation mode, and bf16
// storage for shapes without a tcgen05 kernel). Each function restates one reference module
// as a short chain of kernels on fp32 intermediates in the caller's workspace; with
// `ws.base == nullptr` it only measures the workspace it would use.
#include "modules.cuh"
#include "generic_ops.cuh"

namespace of3 {
namespace generic {

#define TRY(x)                  \
    do {                        \
        int _rc = (x);          \
        if (_rc) return _rc;    \
    } while (0)

static inline GemmDesc row_gemm(long long rows, int out_dim, int in_dim, int lda, int ldo) {
    GemmDesc g;
    g.batch = 1;
    g.M = (int)rows;
    g.N = out_dim;
    g.K = in_dim;
    g.a_b = 0; g.a_m = lda; g.a_k = 1;
    g.w_b = 0; g.w_n = in_dim; g.w_k = 1;
    g.o_b = 0; g.o_m = ldo; g.o_n = 1;
    return g;
}

// y[rows, out_dim] = x[rows, in_dim] W^T (+ bias), W of storage type T
template <typename T>
static int linear(const float* x, const T* W, const T* bias, float* y, long long rows, int out_dim,
                  int in_dim, cudaStream_t st) {
    // gemm_nt indexes M with an int and grid.y <= 65535 tiles of 64 rows: split long row counts
    const long long kChunk = 65535LL * 64;
    for (long long r0 = 0; r0 < rows; r0 += kChunk) {
        const long long nr = rows - r0 < kChunk ? rows - r0 : kChunk;
        GemmDesc g = row_gemm(nr, out_dim, in_dim, in_dim, out_dim);
        TRY(gemm_nt<T>(x + r0 * in_dim, W, bias, y + r0 * out_dim, g, st));
    }
    return OF3_OK;
}

// ------------------------------------------------------------------ triangle multiplication
template <typename T>
int trimul(const T* z, const T* mask, T* out, int B, int N, int c_z, int c_h, int flags,
           const of3_trimul_params* p, Arena& ws, cudaStream_t st) {
    const long long rows = (long long)B * N * N;
    const int cm = c_z > c_h ? c_z : c_h;
    float* zn = (float*)ws.take(rows * c_z * sizeof(float));
    float* t1 = (float*)ws.take(rows * cm * sizeof(float));
    float* t2 = (float*)ws.take(rows * cm * sizeof(float));
    float* a = (float*)ws.take(rows * cm * sizeof(float));
    float* b = (float*)ws.take(rows * cm * sizeof(float));
    float* x = (float*)ws.take(rows * c_h * sizeof(float));
    if (!ws.base) return OF3_OK;
    OF3_REQUIRE(ws.ok(), OF3_ERR_WORKSPACE, "trimul: workspace too small (%zu needed)", ws.off);
    const bool outgoing = (flags & OF3_FLAG_OUTGOING) != 0;

    TRY((layernorm<T, T>(z, (const T*)p->ln_in_w, (const T*)p->ln_in_b, zn, rows, c_z, 1e-5f, rows, 0,
                         c_z, st)));
    TRY(linear<T>(zn, (const T*)p->w_a_g, nullptr, t1, rows, c_h, c_z, st));
    TRY(linear<T>(zn, (const T*)p->w_a_p, nullptr, t2, rows, c_h, c_z, st));
    TRY(gate_mul_mask<T>(t1, t2, c_h, mask, a, rows, c_h, st));
    TRY(linear<T>(zn, (const T*)p->w_b_g, nullptr, t1, rows, c_h, c_z, st));
    TRY(linear<T>(zn, (const T*)p->w_b_p, nullptr, t2, rows, c_h, c_z, st));
    TRY(gate_mul_mask<T>(t1, t2, c_h, mask, b, rows, c_h, st));
    // one GEMM per hidden channel, operands read in place from the [N, N, c_h] tensors
    for (int s = 0; s < B; ++s) {
        const long long off = (long long)s * N * N * c_h;
        GemmDesc g;
        g.batch = c_h; g.M = N; g.N = N; g.K = N;
        g.a_b = 1; g.w_b = 1; g.o_b = 1;
        g.o_m = (long long)N * c_h; g.o_n = c_h;
        if (outgoing) {  // x[i,j] = sum_k a[i,k] b[j,k]
            g.a_m = (long long)N * c_h; g.a_k = c_h;
            g.w_n = (long long)N * c_h; g.w_k = c_h;
        } else {         // x[i,j] = sum_k a[k,i] b[k,j]
            g.a_m = c_h; g.a_k = (long long)N * c_h;
            g.w_n = c_h; g.w_k = (long long)N * c_h;
        }
        for (int c0 = 0; c0 < c_h; c0 += 32768) {
            GemmDesc gc = g;
            gc.batch = c_h - c0 < 32768 ? c_h - c0 : 32768;
            TRY(gemm_nt<float>(a + off + c0, b + off + c0, nullptr, x + off + c0, gc, st));
        }
    }
    TRY((layernorm<float, T>(x, (const T*)p->ln_out_w, (const T*)p->ln_out_b, t1, rows, c_h, 1e-5f,
                             rows, 0, c_h, st)));
    TRY(linear<T>(t1, (const T*)p->w_z, nullptr, t2, rows, c_z, c_h, st));
    TRY(linear<T>(zn, (const T*)p->w_g, nullptr, a, rows, c_z, c_z, st));
    TRY(finalize<T>(t2, a, (flags & OF3_FLAG_ADD_RESIDUAL) ? z : nullptr, nullptr, out, rows, c_z,
                    rows, 0, c_z, st));
    return OF3_OK;
}

// ------------------------------------------------------------------ triangle attention
template <typename T>
int triattn(const T* z, const T* mask, T* out, int B, int N, int c_z, int H, int d, float inf,
            int flags, const of3_triattn_params* p, Arena& ws, cudaStream_t st) {
    const long long rows = (long long)N * N;  // one sample at a time
    const int hd = H * d;
    float* xn = (float*)ws.take(rows * c_z * sizeof(float));
    float* q = (float*)ws.take(rows * hd * sizeof(float));
    float* k = (float*)ws.take(rows * hd * sizeof(float));
    float* v = (float*)ws.take(rows * hd * sizeof(float));
    float* g = (float*)ws.take(rows * hd * sizeof(float));
    float* o = (float*)ws.take(rows * hd * sizeof(float));
    float* tb_raw = (float*)ws.take(rows * H * sizeof(float));
    float* tb = (float*)ws.take(rows * H * sizeof(float));
    float* mb = (float*)ws.take(rows * sizeof(float));
    float* y = (float*)ws.take(rows * c_z * sizeof(float));
    if (!ws.base) return OF3_OK;
    OF3_REQUIRE(ws.ok(), OF3_ERR_WORKSPACE, "triattn: workspace too small (%zu needed)", ws.off);
    const bool tr = (flags & OF3_FLAG_TRANSPOSED) != 0;
    // row r = (i', j') of the (possibly transposed) view: source element z[j', i'] when transposed
    const long long outer = tr ? c_z : (long long)N * c_z;
    const long long inner = tr ? (long long)N * c_z : c_z;
    const float scale = 1.0f / sqrtf((float)d);
    for (int s = 0; s < B; ++s) {
        const T* zs = z + (long long)s * rows * c_z;
        T* os = out + (long long)s * rows * c_z;
        TRY((layernorm<T, T>(zs, (const T*)p->ln_w, (const T*)p->ln_b, xn, rows, c_z, 1e-5f, N, outer,
                             inner, st)));
        TRY(linear<T>(xn, (const T*)p->w_q, nullptr, q, rows, hd, c_z, st));
        TRY(linear<T>(xn, (const T*)p->w_k, nullptr, k, rows, hd, c_z, st));
        TRY(linear<T>(xn, (const T*)p->w_v, nullptr, v, rows, hd, c_z, st));
        TRY(linear<T>(xn, (const T*)p->w_g, nullptr, g, rows, hd, c_z, st));
        TRY(linear<T>(xn, (const T*)p->w_bias, nullptr, tb_raw, rows, H, c_z, st));
        TRY(permute_bias(tb_raw, tb, 1, N, H, st));
        const float* mbp = nullptr;
        if (mask) {
            const T* ms = mask + (long long)s * rows;
            TRY(mask_to_bias<T>(ms, mb, N, N, inf, tr ? 1 : N, tr ? N : 1, st));
            mbp = mb;
        }
        TRY(attention(q, k, v, mbp, tb, o, N, N, H, d, scale, N, st));
        TRY(sigmoid_mul(o, hd, g, hd, q, rows, hd, st));
        TRY(linear<T>(q, (const T*)p->w_o, nullptr, y, rows, c_z, hd, st));
        TRY(finalize<T>(y, nullptr, (flags & OF3_FLAG_ADD_RESIDUAL) ? zs : nullptr, nullptr, os, rows,
                        c_z, N, outer, inner, st));
    }
    return OF3_OK;
}

// ------------------------------------------------------------------ SwiGLU transition
template <typename T>
int transition(const T* x, const T* mask, T* out, long long rows, int c, int n, int flags,
               const of3_transition_params* p, Arena& ws, cudaStream_t st) {
    const int hid = n * c;
    float* xn = (float*)ws.take(rows * c * sizeof(float));
    float* a = (float*)ws.take(rows * hid * sizeof(float));
    float* b = (float*)ws.take(rows * hid * sizeof(float));
    float* y = (float*)ws.take(rows * c * sizeof(float));
    if (!ws.base) return OF3_OK;
    OF3_REQUIRE(ws.ok(), OF3_ERR_WORKSPACE, "transition: workspace too small (%zu needed)", ws.off);
    TRY((layernorm<T, T>(x, (const T*)p->ln_w, (const T*)p->ln_b, xn, rows, c, 1e-5f, rows, 0, c, st)));
    TRY(linear<T>(xn, (const T*)p->w_a, nullptr, a, rows, hid, c, st));
    TRY(linear<T>(xn, (const T*)p->w_b, nullptr, b, rows, hid, c, st));
    TRY(silu_mul(a, b, hid, a, rows, hid, st));
    TRY(linear<T>(a, (const T*)p->w_out, nullptr, y, rows, c, hid, st));
    TRY(finalize<T>(y, nullptr, (flags & OF3_FLAG_ADD_RESIDUAL) ? x : nullptr, mask, out, rows, c,
                    rows, 0, c, st));
    return OF3_OK;
}

// adaptive LayerNorm: dst = sigmoid(W_g LN_s(s) + b_g) * LN(a) + W_s LN_s(s); also returns nothing else
template <typename T>
static int ada_ln(const T* a, const T* s, float* dst, float* sn, float* t1, float* t2,
                  long long rows, int c_a, int c_s, const T* ln_s_w, const T* w_g, const T* b_g,
                  const T* w_s, cudaStream_t st) {
    TRY((layernorm<T, T>(a, nullptr, nullptr, dst, rows, c_a, 1e-5f, rows, 0, c_a, st)));
    TRY((layernorm<T, T>(s, ln_s_w, nullptr, sn, rows, c_s, 1e-5f, rows, 0, c_s, st)));
    TRY(linear<T>(sn, w_g, b_g, t1, rows, c_a, c_s, st));
    TRY(linear<T>(sn, w_s, nullptr, t2, rows, c_a, c_s, st));
    TRY(ada_combine(t1, dst, t2, dst, rows * c_a, st));
    return OF3_OK;
}

// ------------------------------------------------------------------ attention with pair bias
template <typename T>
int attn_pair_bias(const T* a, const T* z, const T* s, const T* mask, T* out, int Ba, int Bz, int N,
                   int c_a, int c_s, int c_z, int H, int d, float inf, int flags,
                   const of3_attn_pair_bias_params* p, Arena& ws, cudaStream_t st, const float* pair_bias) {
    const long long rows = (long long)Ba * N;
    const long long zrows = (long long)Bz * N * N;
    const int hd = H * d;
    const bool ada = (flags & OF3_FLAG_ADA_LN) != 0;
    float* an = (float*)ws.take(rows * c_a * sizeof(float));
    float* q = (float*)ws.take(rows * hd * sizeof(float));
    float* k = (float*)ws.take(rows * hd * sizeof(float));
    float* v = (float*)ws.take(rows * hd * sizeof(float));
    float* g = (float*)ws.take(rows * hd * sizeof(float));
    float* o = (float*)ws.take(rows * hd * sizeof(float));
    float* y = (float*)ws.take(rows * c_a * sizeof(float));
    float* mb = (float*)ws.take(rows * sizeof(float));
    float* zb = (float*)ws.take(zrows * H * sizeof(float));
    float* sn = ada ? (float*)ws.take(rows * c_s * sizeof(float)) : nullptr;
    float* t1 = ada ? (float*)ws.take(rows * c_a * sizeof(float)) : nullptr;
    float* t2 = ada ? (float*)ws.take(rows * c_a * sizeof(float)) : nullptr;
    // the pair-bias projection streams z in row panels so its scratch stays small
    const long long panel = 65536;
    float* zn = (float*)ws.take(panel * c_z * sizeof(float));
    float* zp = (float*)ws.take(zrows * H * sizeof(float));
    if (!ws.base) return OF3_OK;
    OF3_REQUIRE(ws.ok(), OF3_ERR_WORKSPACE, "attn_pair_bias: workspace too small (%zu needed)", ws.off);
    OF3_REQUIRE(Bz > 0 && Ba % Bz == 0, OF3_ERR_SHAPE, "attn_pair_bias: Ba %d not a multiple of Bz %d",
                Ba, Bz);
    if (ada) {
        OF3_REQUIRE(s != nullptr, OF3_ERR_ARG, "attn_pair_bias: AdaLN needs s");
        TRY(ada_ln<T>(a, s, an, sn, t1, t2, rows, c_a, c_s, (const T*)p->ada_ln_s_w,
                      (const T*)p->ada_w_g, (const T*)p->ada_b_g, (const T*)p->ada_w_s, st));
    } else {
        TRY((layernorm<T, T>(a, (const T*)p->ln_a_w, (const T*)p->ln_a_b, an, rows, c_a, 1e-5f, rows, 0,
                             c_a, st)));
    }
    if (pair_bias != nullptr) {
        zb = const_cast<float*>(pair_bias);
    } else if (c_z == 128 && H == 16 && ((uintptr_t)z & 15) == 0) {
        // one pass over z: LayerNorm statistics and all 16 head projections per pair position
        TRY(pair_bias_c128_h16<T>(z, (const T*)p->ln_z_w, (const T*)p->ln_z_b, (const T*)p->w_z, zb, Bz,
                                      (long long)N * N, st));
    } else {
        for (long long r0 = 0; r0 < zrows; r0 += panel) {
            const long long nr = zrows - r0 < panel ? zrows - r0 : panel;
            TRY((layernorm<T, T>(z + r0 * c_z, (const T*)p->ln_z_w, (const T*)p->ln_z_b, zn, nr, c_z, 1e-5f,
                                 nr, 0, c_z, st)));
            TRY(linear<T>(zn, (const T*)p->w_z, nullptr, zp + r0 * H, nr, H, c_z, st));
        }
        TRY(permute_bias(zp, zb, Bz, N, H, st));
    }
    TRY(linear<T>(an, (const T*)p->w_q, (const T*)p->b_q, q, rows, hd, c_a, st));
    TRY(linear<T>(an, (const T*)p->w_k, nullptr, k, rows, hd, c_a, st));
    TRY(linear<T>(an, (const T*)p->w_v, nullptr, v, rows, hd, c_a, st));
    TRY(linear<T>(an, (const T*)p->w_g, nullptr, g, rows, hd, c_a, st));
    const float* mbp = nullptr;
    if (mask) {
        TRY(mask_to_bias<T>(mask, mb, Ba, N, inf, N, 1, st));
        mbp = mb;
    }
    TRY(attention(q, k, v, mbp, zb, o, Ba, N, H, d, 1.0f / sqrtf((float)d), Ba / Bz, st));
    TRY(sigmoid_mul(o, hd, g, hd, q, rows, hd, st));
    TRY(linear<T>(q, (const T*)p->w_o, nullptr, y, rows, c_a, hd, st));
    const float* gate = nullptr;
    if (ada) {
        TRY(to_f32<T>(s, sn, rows * c_s, st));
        TRY(linear<T>(sn, (const T*)p->w_ada_out, (const T*)p->b_ada_out, t1, rows, c_a, c_s, st));
        gate = t1;
    }
    TRY(finalize<T>(y, gate, (flags & OF3_FLAG_ADD_RESIDUAL) ? a : nullptr, nullptr, out, rows, c_a,
                    rows, 0, c_a, st));
    return OF3_OK;
}

// ------------------------------------------------------------------ conditioned transition
template <typename T>
int cond_transition(const T* a, const T* s, const T* mask, T* out, long long rows, int c_a, int c_s,
                    int n, int flags, const of3_cond_transition_params* p, Arena& ws,
                    cudaStream_t st) {
    const int hid = n * c_a;
    float* an = (float*)ws.take(rows * c_a * sizeof(float));
    float* sn = (float*)ws.take(rows * c_s * sizeof(float));
    float* t1 = (float*)ws.take(rows * c_a * sizeof(float));
    float* t2 = (float*)ws.take(rows * c_a * sizeof(float));
    float* ha = (float*)ws.take(rows * hid * sizeof(float));
    float* hb = (float*)ws.take(rows * hid * sizeof(float));
    if (!ws.base) return OF3_OK;
    OF3_REQUIRE(ws.ok(), OF3_ERR_WORKSPACE, "cond_transition: workspace too small (%zu needed)", ws.off);
    TRY(ada_ln<T>(a, s, an, sn, t1, t2, rows, c_a, c_s, (const T*)p->ada_ln_s_w, (const T*)p->ada_w_g,
                  (const T*)p->ada_b_g, (const T*)p->ada_w_s, st));
    TRY(linear<T>(an, (const T*)p->w_a, nullptr, ha, rows, hid, c_a, st));
    TRY(linear<T>(an, (const T*)p->w_b, nullptr, hb, rows, hid, c_a, st));
    TRY(silu_mul(ha, hb, hid, ha, rows, hid, st));
    TRY(linear<T>(ha, (const T*)p->w_out, nullptr, t1, rows, c_a, hid, st));
    TRY(to_f32<T>(s, sn, rows * c_s, st));
    TRY(linear<T>(sn, (const T*)p->w_g, (const T*)p->b_g, t2, rows, c_a, c_s, st));
    TRY(finalize<T>(t1, t2, (flags & OF3_FLAG_ADD_RESIDUAL) ? a : nullptr, mask, out, rows, c_a, rows,
                    0, c_a, st));
    return OF3_OK;
}

#define INSTANTIATE(T)                                                                               \
    template int trimul<T>(const T*, const T*, T*, int, int, int, int, int, const of3_trimul_params*, \
                           Arena&, cudaStream_t);                                                    \
    template int triattn<T>(const T*, const T*, T*, int, int, int, int, int, float, int,             \
                            const of3_triattn_params*, Arena&, cudaStream_t);                        \
    template int transition<T>(const T*, const T*, T*, long long, int, int, int,                     \
                               const of3_transition_params*, Arena&, cudaStream_t);                  \
    template int attn_pair_bias<T>(const T*, const T*, const T*, const T*, T*, int, int, int, int,   \
                                   int, int, int, int, float, int, const of3_attn_pair_bias_params*, \
                                   Arena&, cudaStream_t, const float*);                                          \
    template int cond_transition<T>(const T*, const T*, const T*, T*, long long, int, int, int, int, \
                                    const of3_cond_transition_params*, Arena&, cudaStream_t);
INSTANTIATE(float)
INSTANTIATE(__nv_bfloat16)

}  // namespace generic
}  // namespace of3
