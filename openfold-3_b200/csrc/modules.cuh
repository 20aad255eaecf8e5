// Internal module-level interfaces behind the C ABI: the shape-generic family (any shape,
// fp32 or bf16 storage) and the tcgen05 family (bf16, the OpenFold3 Pairformer widths).
#pragma once
#include "common.cuh"
#include "of3b200.h"

namespace of3 {

namespace generic {
template <typename T>
int trimul(const T* z, const T* mask, T* out, int B, int N, int c_z, int c_h, int flags,
           const of3_trimul_params* p, Arena& ws, cudaStream_t st);
template <typename T>
int triattn(const T* z, const T* mask, T* out, int B, int N, int c_z, int H, int d, float inf,
            int flags, const of3_triattn_params* p, Arena& ws, cudaStream_t st);
template <typename T>
int transition(const T* x, const T* mask, T* out, long long rows, int c, int n, int flags,
               const of3_transition_params* p, Arena& ws, cudaStream_t st);
template <typename T>
int attn_pair_bias(const T* a, const T* z, const T* s, const T* mask, T* out, int Ba, int Bz, int N,
                   int c_a, int c_s, int c_z, int H, int d, float inf, int flags,
                   const of3_attn_pair_bias_params* p, Arena& ws, cudaStream_t st,
                   const float* pair_bias = nullptr);  // [Bz][H][N][N] already projected (z unused)
template <typename T>
int cond_transition(const T* a, const T* s, const T* mask, T* out, long long rows, int c_a, int c_s,
                    int n, int flags, const of3_cond_transition_params* p, Arena& ws,
                    cudaStream_t st);
}  // namespace generic

namespace fast {
// bf16, c_z = c_hidden = 128
bool trimul_supported(int c_z, int c_h);
int trimul(const __nv_bfloat16* z, const __nv_bfloat16* mask, __nv_bfloat16* out, int B, int N,
           int flags, const of3_trimul_params* p, Arena& ws, cudaStream_t st);
// bf16, c_z = 128, 4 heads x 32
bool triattn_supported(int c_z, int H, int d, int N);
int triattn(const __nv_bfloat16* z, const __nv_bfloat16* mask, __nv_bfloat16* out, int B, int N,
            float inf, int flags, const of3_triattn_params* p, Arena& ws, cudaStream_t st);
// bf16, c = 128, n = 4
// phases of the two layers above on R lines of N positions (R == N: whole tensor; R = N / P: a row shard)
int trimul_project(const __nv_bfloat16* z, const __nv_bfloat16* mask, __nv_bfloat16* a_t, __nv_bfloat16* b_t,
                   int B, int R, int N, int ld, bool transposed_walk, const of3_trimul_params* p,
                   cudaStream_t st, int groups = 1, long long group_stride = 0);
int trimul_output(const __nv_bfloat16* z, __nv_bfloat16* out, const __nv_bfloat16* x_t, int B, int R, int N, int ld,
                  int add_residual, const of3_trimul_params* p, cudaStream_t st);
int trimul_finish(const __nv_bfloat16* z, __nv_bfloat16* out, const __nv_bfloat16* a_t,
                  const __nv_bfloat16* b_t, __nv_bfloat16* x_t, int B, int R, int N, int ld, int add_residual,
                  const of3_trimul_params* p, cudaStream_t st);
size_t triattn_image_elems(int B, int R, int N);
size_t triattn_bias_elems(int B, int R, int N);  // bf16 elements of the pair-bias image [B*4][key blocks][R][32]
int triattn_project(const __nv_bfloat16* z, __nv_bfloat16* q, __nv_bfloat16* k, __nv_bfloat16* vt,
                    __nv_bfloat16* tb, int B, int R, int N, int row0, bool transposed,
                    const of3_triattn_params* p, cudaStream_t st);
int triattn_finish(const __nv_bfloat16* z, const __nv_bfloat16* mask, __nv_bfloat16* out,
                   const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* vt,
                   const __nv_bfloat16* tb, __nv_bfloat16* o, int B, int R, int N, float inf,
                   bool transposed, int add_residual, const of3_triattn_params* p, cudaStream_t st);
bool transition_supported(int c, int n);
int transition(const __nv_bfloat16* x, const __nv_bfloat16* mask, __nv_bfloat16* out, long long rows,
               int flags, const of3_transition_params* p, Arena& ws, cudaStream_t st);
// gated attention with pair bias on the tensor pipe: q, g, out [BB, nq, H*d]; k, v [BB, N, H*d]; pair_bias fp32
// [BB / rows_per_bias, H, nq, N]; with ws.base == nullptr only the workspace need is accumulated
bool single_attn_tc_supported(int N, int H, int d);
// pair_bias == nullptr: the bias tiles are projected straight from z (whole pair tensors only: nq == N) with the
// LayerNorm weight / bias ln_z_w / ln_z_b and linear_z.weight w_z
int single_attn_tc(const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* v, const __nv_bfloat16* g,
                   const __nv_bfloat16* q_bias, const float* pair_bias, const __nv_bfloat16* mask, __nv_bfloat16* out,
                   int BB, int N, int nq, int H, int d, float inf, int rows_per_bias, Arena& ws, cudaStream_t st,
                   const __nv_bfloat16* z = nullptr, const __nv_bfloat16* ln_z_w = nullptr,
                   const __nv_bfloat16* ln_z_b = nullptr, const __nv_bfloat16* w_z = nullptr,
                   const __nv_bfloat16* bias_tiles = nullptr);   // bias_tiles: from pair_bias_tiles_c128_h16
// single-track layers (bf16): linears on the tcgen05 contraction kernel, attention on single_attn_tc
// (LayerNorm variant of the trunk, or with OF3_FLAG_ADA_LN the conditioned variant of the diffusion stack)
bool attn_pair_bias_supported(int Ba, int Bz, int N, int c_a, int c_s, int c_z, int H, int d, int flags);
int attn_pair_bias(const __nv_bfloat16* a, const __nv_bfloat16* z, const __nv_bfloat16* s, const __nv_bfloat16* mask,
                   __nv_bfloat16* out, int Ba, int Bz, int N, int c_a, int c_s, int H, int d, float inf, int flags,
                   const of3_attn_pair_bias_params* p, Arena& ws, cudaStream_t st, const float* pair_bias,
                   const __nv_bfloat16* bias_tiles = nullptr);
bool cond_transition_supported(int c_a, int c_s, int n, int flags);
int cond_transition(const __nv_bfloat16* a, const __nv_bfloat16* s, const __nv_bfloat16* mask, __nv_bfloat16* out,
                    long long rows, int c_a, int c_s, int n, int flags, const of3_cond_transition_params* p, Arena& ws,
                    cudaStream_t st);
int attn_pair_bias_rows(const __nv_bfloat16* a, const float* pair_bias_rows, const __nv_bfloat16* mask,
                        __nv_bfloat16* out_rows, int N, int row0, int R, int c_a, int H, int d, float inf, int flags,
                        const of3_attn_pair_bias_params* p, Arena& ws, cudaStream_t st);
// pair-bias projection of the single track on the tensor pipe: dst [B][16][nn] fp32 from z [B*nn][128] bf16
int pair_bias_c128_h16(const __nv_bfloat16* z, const __nv_bfloat16* ln_w, const __nv_bfloat16* ln_b,
                       const __nv_bfloat16* w, float* dst, long long B, long long nn, cudaStream_t st);
// the same projection written as the single-track attention kernel's bf16 bias tiles (z [B][N][N][128])
int pair_bias_tiles_c128_h16(const __nv_bfloat16* z, const __nv_bfloat16* ln_w, const __nv_bfloat16* ln_b,
                             const __nv_bfloat16* w, __nv_bfloat16* tiles, long long B, int N, cudaStream_t st);
bool transition_wide_supported(int c, int n);
int transition_wide(const __nv_bfloat16* x, const __nv_bfloat16* mask, __nv_bfloat16* out, long long rows, int c,
                    int n, int flags, const of3_transition_params* p, Arena& ws, cudaStream_t st);
}  // namespace fast

int contract_nt_bf16(const __nv_bfloat16* a, const __nv_bfloat16* b, __nv_bfloat16* out, int batch,
                     int M, int N, int K, int lda, int ldb, int ldo, long long a_bs, long long b_bs,
                     long long o_bs, cudaStream_t stream, int rows_per_block = 0, long long row_block_stride = 0,
                     int account_as = 1);  // kernel id of the launch accounting: 1 triangle einsum, 10 linear layer

}  // namespace of3
