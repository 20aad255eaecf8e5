// Shape-generic SIMT kernels (any channel width, head count, sequence length).
//
// They back (1) the fp32 validation mode, where every product and sum is true fp32 (no
// tensor cores, no TF32), and (2) bf16 storage with shapes the tcgen05 kernels do not
// cover. Storage type T is float or __nv_bfloat16; intermediates are always fp32.
#pragma once
#include "common.cuh"

namespace of3 {
namespace generic {

// y[r, :] = LN(x[r, :]) * gamma + beta (gamma/beta may be null); y is dense fp32 [rows, C].
// Source row r lives at x + (r / inner) * outer_stride + (r % inner) * inner_stride (elements),
// so a transposed [N, N, C] view is normalised without materialising it.
template <typename TX, typename TP>
int layernorm(const TX* x, const TP* gamma, const TP* beta, float* y, long long rows, int C,
              float eps, long long inner, long long outer_stride, long long inner_stride,
              cudaStream_t stream);

// out[b][m][n] = sum_k A[b][m][k] * W[b][n][k] (+ bias[n]); all strides in elements.
// A fp32, W and bias of type TW (fp32 or bf16), out fp32.
struct GemmDesc {
    int batch, M, N, K;
    long long a_b, a_m, a_k;
    long long w_b, w_n, w_k;
    long long o_b, o_m, o_n;
};
template <typename TW>
int gemm_nt(const float* A, const TW* W, const TW* bias, float* out, const GemmDesc& d,
            cudaStream_t stream);

// Streaming (online-softmax) attention, one warp per query:
//   o[bb, q, h, :] = softmax_k( scale * q.k + mask_bias[bb, k] + pair_bias[bb / rows_per_bias, h, q, k] ) v
// q,k,v,out: [BB, N, H*d] fp32; mask_bias: [BB, N] fp32 additive or null;
// pair_bias: [BB / rows_per_bias, H, N, N] fp32 or null. d <= 64.
int attention(const float* q, const float* k, const float* v, const float* mask_bias,
              const float* pair_bias, float* out, long long BB, int N, int H, int d, float scale,
              long long rows_per_bias, cudaStream_t stream);

// dst[r, c] = (mask ? mask[r] : 1) * sigmoid(g[r, c]) * p[r, c]; g/p rows have pitch ld.
template <typename T>
int gate_mul_mask(const float* g, const float* p, int ld, const T* mask, float* dst, long long rows,
                  int C, cudaStream_t stream);
// dst[r, c] = x[r, c] * sigmoid(g[r, c]) with row pitches ldx / ldg, dst dense.
int sigmoid_mul(const float* x, int ldx, const float* g, int ldg, float* dst, long long rows, int C,
                cudaStream_t stream);
// dst[r, c] = silu(a[r, c]) * b[r, c], a/b rows have pitch ld, dst dense.
int silu_mul(const float* a, const float* b, int ld, float* dst, long long rows, int C,
             cudaStream_t stream);
// dst = sigmoid(g) * a + s   (adaptive LayerNorm combine), all dense, n elements.
int ada_combine(const float* g, const float* a, const float* s, float* dst, long long n,
                cudaStream_t stream);
// dst[r, k] = inf * (mask[r * row_stride + k * k_stride] - 1)
template <typename T>
int mask_to_bias(const T* mask, float* dst, long long rows, int N, float inf, long long row_stride,
                 long long k_stride, cudaStream_t stream);
// out_row(r) = (residual ? residual_row(r) : 0) + upd[r, :] * (gate ? sigmoid(gate[r, :]) : 1)
//              * (mask ? mask[r] : 1)
// upd/gate dense fp32 [rows, C]; residual/out rows addressed like layernorm's source rows
// (residual and out may alias); mask dense [rows] of type T.
template <typename T>
int finalize(const float* upd, const float* gate, const T* residual, const T* mask, T* out,
             long long rows, int C, long long inner, long long outer_stride,
             long long inner_stride, cudaStream_t stream);
// Fused pair-bias projection for 128-channel pair tensors and 16 heads:
// dst[b][h][pos] = sum_c LN(z[b, pos, :])[c] * w[h][c] for pos < positions_per_sample (N*N for a whole
// tensor, R*N for a row shard), one thread per pair position, one pass over z.
// gamma/beta may be null. Returns OF3_ERR_SHAPE for other widths (callers fall back to the chain).
template <typename T>
int pair_bias_c128_h16(const T* z, const T* gamma, const T* beta, const T* w, float* dst, long long B,
                       long long positions_per_sample, cudaStream_t stream);
// dst[b][h][q][k] = src[b][q][k][h]
int permute_bias(const float* src, float* dst, long long B, int N, int H, cudaStream_t stream);
// dense fp32 copy of a storage-type tensor
template <typename T>
int to_f32(const T* src, float* dst, long long n, cudaStream_t stream);

}  // namespace generic
}  // namespace of3
