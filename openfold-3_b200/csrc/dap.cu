// Entry points for the row-sharded ("DAP") pair stack: each rank owns R = N / P consecutive rows of
// the pair tensor z[N, N, 128] (bf16, one sample) and runs every layer in two phases around the one
// exchange step the layer needs. The exchange itself (NCCL all-gather / all-to-all through
// torch.distributed) is done by the caller between the phases; remote data always lands in this
// GPU's own memory first and the kernels only ever read local memory.
//
//   triangle update  project: local rows -> a_t, b_t (channel-major) | all-gather b_t | finish:
//                    contraction of the local rows of a against ALL rows of b, LN / gate / residual
//   triangle attn    project: q, k, v^T and the local rows of the pair bias | all-gather bias |
//                    finish: attention over the local lines, gate, output projection, residual
//   incoming update / ending-node attention run the same phases on the all-to-all-transposed shard.
#include "generic_ops.cuh"
#include "modules.cuh"

using namespace of3;

extern "C" {

int of3_dap_pitch(int N, int multiple) { return (int)align_up((size_t)N, (size_t)multiple); }

long long of3_dap_triattn_image_elems(int R, int N) { return (long long)fast::triattn_image_elems(1, R, N); }

int of3_dap_trimul_project(const void* z_rows, const void* mask_rows, void* a_t, void* b_t, int R, int N,
                           const of3_trimul_params* p, void* stream) {
    OF3_REQUIRE(z_rows && a_t && b_t && p, OF3_ERR_ARG, "dap_trimul_project: null pointer argument");
    OF3_REQUIRE(R > 0 && N > 0, OF3_ERR_ARG, "dap_trimul_project: non-positive size");
    return fast::trimul_project((const __nv_bfloat16*)z_rows, (const __nv_bfloat16*)mask_rows, (__nv_bfloat16*)a_t,
                                (__nv_bfloat16*)b_t, 1, R, N, (int)align_up(N, 8), false, p, (cudaStream_t)stream);
}

int of3_dap_trimul_finish(const void* z_rows, void* out_rows, const void* a_t, const void* b_all, void* x_scratch,
                          int R, int N, int flags, const of3_trimul_params* p, void* stream) {
    OF3_REQUIRE(z_rows && out_rows && a_t && b_all && x_scratch && p, OF3_ERR_ARG,
                "dap_trimul_finish: null pointer argument");
    OF3_REQUIRE(R > 0 && N > 0, OF3_ERR_ARG, "dap_trimul_finish: non-positive size");
    return fast::trimul_finish((const __nv_bfloat16*)z_rows, (__nv_bfloat16*)out_rows, (const __nv_bfloat16*)a_t,
                               (const __nv_bfloat16*)b_all, (__nv_bfloat16*)x_scratch, 1, R, N, (int)align_up(N, 8),
                               (flags & OF3_FLAG_ADD_RESIDUAL) ? 1 : 0, p, (cudaStream_t)stream);
}

int of3_dap_triattn_project(const void* z_rows, void* q, void* k, void* vt, void* bias_rows, int R, int N,
                            const of3_triattn_params* p, void* stream) {
    OF3_REQUIRE(z_rows && q && k && vt && bias_rows && p, OF3_ERR_ARG, "dap_triattn_project: null pointer argument");
    OF3_REQUIRE(R > 0 && N > 0, OF3_ERR_ARG, "dap_triattn_project: non-positive size");
    return fast::triattn_project((const __nv_bfloat16*)z_rows, (__nv_bfloat16*)q, (__nv_bfloat16*)k,
                                 (__nv_bfloat16*)vt, (__nv_bfloat16*)bias_rows, 1, R, N, (int)align_up(N, 64), false, p,
                                 (cudaStream_t)stream);
}

int of3_dap_triattn_finish(const void* z_rows, const void* mask_rows, void* out_rows, const void* q, const void* k,
                           const void* vt, const void* bias_all, void* o_scratch, int R, int N, float inf, int flags,
                           const of3_triattn_params* p, void* stream) {
    OF3_REQUIRE(z_rows && out_rows && q && k && vt && bias_all && o_scratch && p, OF3_ERR_ARG,
                "dap_triattn_finish: null pointer argument");
    OF3_REQUIRE(R > 0 && N > 0, OF3_ERR_ARG, "dap_triattn_finish: non-positive size");
    return fast::triattn_finish((const __nv_bfloat16*)z_rows, (const __nv_bfloat16*)mask_rows,
                                (__nv_bfloat16*)out_rows, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k,
                                (const __nv_bfloat16*)vt, (const __nv_bfloat16*)bias_all, (__nv_bfloat16*)o_scratch, 1, R,
                                N, (int)align_up(N, 64), inf, false, (flags & OF3_FLAG_ADD_RESIDUAL) ? 1 : 0, p,
                                (cudaStream_t)stream);
}

int of3_pair_bias_project(const void* z_rows, const void* ln_w, const void* ln_b, const void* w, float* bias_rows,
                          long long positions, int c_z, int H, int dtype, void* stream) {
    OF3_REQUIRE(z_rows && w && bias_rows, OF3_ERR_ARG, "pair_bias_project: null pointer argument");
    OF3_REQUIRE(c_z == 128 && H == 16, OF3_ERR_SHAPE, "pair_bias_project: only c_z = 128, 16 heads");
    if (dtype == OF3_DTYPE_BF16)
        return generic::pair_bias_c128_h16<__nv_bfloat16>((const __nv_bfloat16*)z_rows, (const __nv_bfloat16*)ln_w,
                                                          (const __nv_bfloat16*)ln_b, (const __nv_bfloat16*)w,
                                                          bias_rows, 1, positions, (cudaStream_t)stream);
    OF3_REQUIRE(dtype == OF3_DTYPE_F32, OF3_ERR_ARG, "pair_bias_project: bad dtype %d", dtype);
    return generic::pair_bias_c128_h16<float>((const float*)z_rows, (const float*)ln_w, (const float*)ln_b,
                                              (const float*)w, bias_rows, 1, positions, (cudaStream_t)stream);
}

int of3_attn_pair_bias_forward_prebias(const void* a, const float* pair_bias, const void* s, const void* mask,
                                       void* out, int Ba, int Bz, int N, int c_a, int c_s, int H, int d, float inf,
                                       int dtype, int flags, const of3_attn_pair_bias_params* p, void* workspace,
                                       size_t workspace_bytes, void* stream) {
    OF3_REQUIRE(a && pair_bias && out && p && workspace, OF3_ERR_ARG, "attn_pair_bias_prebias: null pointer argument");
    OF3_REQUIRE(Ba > 0 && Bz > 0 && Ba % Bz == 0 && N > 0, OF3_ERR_ARG, "attn_pair_bias_prebias: bad sizes");
    Arena ws(workspace, workspace_bytes);
    if (dtype == OF3_DTYPE_BF16 && fast::attn_pair_bias_supported(Ba, Bz, N, c_a, 128, H, d, flags))
        return fast::attn_pair_bias((const __nv_bfloat16*)a, nullptr, (const __nv_bfloat16*)mask, (__nv_bfloat16*)out,
                                    Ba, Bz, N, c_a, H, d, inf, flags, p, ws, (cudaStream_t)stream, pair_bias);
    if (dtype == OF3_DTYPE_BF16)
        return generic::attn_pair_bias<__nv_bfloat16>((const __nv_bfloat16*)a, nullptr, (const __nv_bfloat16*)s,
                                                      (const __nv_bfloat16*)mask, (__nv_bfloat16*)out, Ba, Bz, N, c_a,
                                                      c_s, 128, H, d, inf, flags, p, ws, (cudaStream_t)stream, pair_bias);
    OF3_REQUIRE(dtype == OF3_DTYPE_F32, OF3_ERR_ARG, "attn_pair_bias_prebias: bad dtype %d", dtype);
    return generic::attn_pair_bias<float>((const float*)a, nullptr, (const float*)s, (const float*)mask, (float*)out, Ba,
                                          Bz, N, c_a, c_s, 128, H, d, inf, flags, p, ws, (cudaStream_t)stream, pair_bias);
}

}  // extern "C"
