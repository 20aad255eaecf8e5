// extern "C" entry points: argument checks, kernel-family selection, workspace sizing.
#include "modules.cuh"

using namespace of3;

namespace {

bool use_fast(int dtype, int flags) {
    return dtype == OF3_DTYPE_BF16 && !(flags & OF3_FLAG_FORCE_GENERIC);
}

#define CHECK_DTYPE(dtype)                                                                     \
    OF3_REQUIRE((dtype) == OF3_DTYPE_BF16 || (dtype) == OF3_DTYPE_F32, OF3_ERR_ARG,            \
                "dtype %d is neither OF3_DTYPE_BF16 nor OF3_DTYPE_F32", (dtype))

int trimul_dispatch(const void* z, const void* mask, void* out, int B, int N, int c_z, int c_h,
                    int dtype, int flags, const of3_trimul_params* p, Arena& ws, cudaStream_t st) {
    if (use_fast(dtype, flags) && fast::trimul_supported(c_z, c_h))
        return fast::trimul((const __nv_bfloat16*)z, (const __nv_bfloat16*)mask, (__nv_bfloat16*)out,
                            B, N, flags, p, ws, st);
    if (dtype == OF3_DTYPE_BF16)
        return generic::trimul<__nv_bfloat16>((const __nv_bfloat16*)z, (const __nv_bfloat16*)mask,
                                              (__nv_bfloat16*)out, B, N, c_z, c_h, flags, p, ws, st);
    return generic::trimul<float>((const float*)z, (const float*)mask, (float*)out, B, N, c_z, c_h,
                                  flags, p, ws, st);
}

int triattn_dispatch(const void* z, const void* mask, void* out, int B, int N, int c_z, int H, int d,
                     float inf, int dtype, int flags, const of3_triattn_params* p, Arena& ws,
                     cudaStream_t st) {
    if (use_fast(dtype, flags) && fast::triattn_supported(c_z, H, d, N))
        return fast::triattn((const __nv_bfloat16*)z, (const __nv_bfloat16*)mask, (__nv_bfloat16*)out,
                             B, N, inf, flags, p, ws, st);
    if (dtype == OF3_DTYPE_BF16)
        return generic::triattn<__nv_bfloat16>((const __nv_bfloat16*)z, (const __nv_bfloat16*)mask,
                                               (__nv_bfloat16*)out, B, N, c_z, H, d, inf, flags, p,
                                               ws, st);
    return generic::triattn<float>((const float*)z, (const float*)mask, (float*)out, B, N, c_z, H, d,
                                   inf, flags, p, ws, st);
}

int transition_dispatch(const void* x, const void* mask, void* out, long long rows, int c, int n,
                        int dtype, int flags, const of3_transition_params* p, Arena& ws,
                        cudaStream_t st) {
    if (use_fast(dtype, flags) && fast::transition_supported(c, n))
        return fast::transition((const __nv_bfloat16*)x, (const __nv_bfloat16*)mask,
                                (__nv_bfloat16*)out, rows, flags, p, ws, st);
    if (use_fast(dtype, flags) && fast::transition_wide_supported(c, n))
        return fast::transition_wide((const __nv_bfloat16*)x, (const __nv_bfloat16*)mask, (__nv_bfloat16*)out, rows,
                                     c, n, flags, p, ws, st);
    if (dtype == OF3_DTYPE_BF16)
        return generic::transition<__nv_bfloat16>((const __nv_bfloat16*)x, (const __nv_bfloat16*)mask,
                                                  (__nv_bfloat16*)out, rows, c, n, flags, p, ws, st);
    return generic::transition<float>((const float*)x, (const float*)mask, (float*)out, rows, c, n,
                                      flags, p, ws, st);
}

int apb_dispatch(const void* a, const void* z, const void* s, const void* mask, void* out, int Ba,
                 int Bz, int N, int c_a, int c_s, int c_z, int H, int d, float inf, int dtype,
                 int flags, const of3_attn_pair_bias_params* p, Arena& ws, cudaStream_t st) {
    if (dtype == OF3_DTYPE_BF16 && fast::attn_pair_bias_supported(Ba, Bz, N, c_a, c_s, c_z, H, d, flags))
        return fast::attn_pair_bias((const __nv_bfloat16*)a, (const __nv_bfloat16*)z, (const __nv_bfloat16*)s,
                                    (const __nv_bfloat16*)mask, (__nv_bfloat16*)out, Ba, Bz, N, c_a, c_s, H, d, inf,
                                    flags, p, ws, st, nullptr);
    if (dtype == OF3_DTYPE_BF16)
        return generic::attn_pair_bias<__nv_bfloat16>(
            (const __nv_bfloat16*)a, (const __nv_bfloat16*)z, (const __nv_bfloat16*)s,
            (const __nv_bfloat16*)mask, (__nv_bfloat16*)out, Ba, Bz, N, c_a, c_s, c_z, H, d, inf,
            flags, p, ws, st);
    return generic::attn_pair_bias<float>((const float*)a, (const float*)z, (const float*)s,
                                          (const float*)mask, (float*)out, Ba, Bz, N, c_a, c_s, c_z,
                                          H, d, inf, flags, p, ws, st);
}

int cond_dispatch(const void* a, const void* s, const void* mask, void* out, long long rows, int c_a,
                  int c_s, int n, int dtype, int flags, const of3_cond_transition_params* p,
                  Arena& ws, cudaStream_t st) {
    if (dtype == OF3_DTYPE_BF16 && fast::cond_transition_supported(c_a, c_s, n, flags))
        return fast::cond_transition((const __nv_bfloat16*)a, (const __nv_bfloat16*)s, (const __nv_bfloat16*)mask,
                                     (__nv_bfloat16*)out, rows, c_a, c_s, n, flags, p, ws, st);
    if (dtype == OF3_DTYPE_BF16)
        return generic::cond_transition<__nv_bfloat16>(
            (const __nv_bfloat16*)a, (const __nv_bfloat16*)s, (const __nv_bfloat16*)mask,
            (__nv_bfloat16*)out, rows, c_a, c_s, n, flags, p, ws, st);
    return generic::cond_transition<float>((const float*)a, (const float*)s, (const float*)mask,
                                           (float*)out, rows, c_a, c_s, n, flags, p, ws, st);
}

}  // namespace

extern "C" {

int of3_fast_path_available(int module_id, int dtype, int c, int c_hidden, int heads, int head_dim) {
    if (dtype != OF3_DTYPE_BF16) return 0;
    switch (module_id) {
        case OF3_MODULE_TRIMUL: return fast::trimul_supported(c, c_hidden) ? 1 : 0;
        case OF3_MODULE_TRIATTN: return fast::triattn_supported(c, heads, head_dim, 1) ? 1 : 0;
        case OF3_MODULE_TRANSITION: return fast::transition_supported(c, c_hidden) ? 1 : 0;
        default: return 0;
    }
}

size_t of3_trimul_workspace_bytes(int B, int N, int c_z, int c_h, int dtype, int flags) {
    Arena ws(nullptr, 0);
    of3_trimul_params p = {};
    if (trimul_dispatch(nullptr, nullptr, nullptr, B, N, c_z, c_h, dtype, flags, &p, ws, nullptr)) return 0;
    return ws.off + 256;
}
int of3_trimul_forward(const void* z, const void* mask, void* out, int B, int N, int c_z, int c_h,
                       int dtype, int flags, const of3_trimul_params* p, void* workspace,
                       size_t workspace_bytes, void* stream) {
    CHECK_DTYPE(dtype);
    OF3_REQUIRE(z && out && p && workspace, OF3_ERR_ARG, "trimul: null pointer argument");
    OF3_REQUIRE(B > 0 && N > 0 && c_z > 0 && c_h > 0, OF3_ERR_ARG, "trimul: non-positive size");
    OF3_REQUIRE(p->ln_in_w && p->ln_in_b && p->w_a_p && p->w_a_g && p->w_b_p && p->w_b_g && p->w_g &&
                    p->ln_out_w && p->ln_out_b && p->w_z,
                OF3_ERR_ARG, "trimul: null parameter pointer");
    Arena ws(workspace, workspace_bytes);
    return trimul_dispatch(z, mask, out, B, N, c_z, c_h, dtype, flags, p, ws, (cudaStream_t)stream);
}

size_t of3_triattn_workspace_bytes(int B, int N, int c_z, int H, int d, int dtype, int flags) {
    Arena ws(nullptr, 0);
    of3_triattn_params p = {};
    if (triattn_dispatch(nullptr, nullptr, nullptr, B, N, c_z, H, d, 1e9f, dtype, flags, &p, ws, nullptr))
        return 0;
    return ws.off + 256;
}
int of3_triattn_forward(const void* z, const void* mask, void* out, int B, int N, int c_z, int H,
                        int d, float inf, int dtype, int flags, const of3_triattn_params* p,
                        void* workspace, size_t workspace_bytes, void* stream) {
    CHECK_DTYPE(dtype);
    OF3_REQUIRE(z && out && p && workspace, OF3_ERR_ARG, "triattn: null pointer argument");
    OF3_REQUIRE(B > 0 && N > 0 && c_z > 0 && H > 0 && d > 0, OF3_ERR_ARG, "triattn: non-positive size");
    OF3_REQUIRE(p->ln_w && p->ln_b && p->w_bias && p->w_q && p->w_k && p->w_v && p->w_g && p->w_o,
                OF3_ERR_ARG, "triattn: null parameter pointer");
    Arena ws(workspace, workspace_bytes);
    return triattn_dispatch(z, mask, out, B, N, c_z, H, d, inf, dtype, flags, p, ws,
                            (cudaStream_t)stream);
}

size_t of3_transition_workspace_bytes(long long rows, int c, int n, int dtype, int flags) {
    Arena ws(nullptr, 0);
    of3_transition_params p = {};
    if (transition_dispatch(nullptr, nullptr, nullptr, rows, c, n, dtype, flags, &p, ws, nullptr)) return 0;
    return ws.off + 256;
}
int of3_transition_forward(const void* x, const void* mask, void* out, long long rows, int c, int n,
                           int dtype, int flags, const of3_transition_params* p, void* workspace,
                           size_t workspace_bytes, void* stream) {
    CHECK_DTYPE(dtype);
    OF3_REQUIRE(x && out && p && workspace, OF3_ERR_ARG, "transition: null pointer argument");
    OF3_REQUIRE(rows > 0 && c > 0 && n > 0, OF3_ERR_ARG, "transition: non-positive size");
    OF3_REQUIRE(p->ln_w && p->ln_b && p->w_a && p->w_b && p->w_out, OF3_ERR_ARG,
                "transition: null parameter pointer");
    Arena ws(workspace, workspace_bytes);
    return transition_dispatch(x, mask, out, rows, c, n, dtype, flags, p, ws, (cudaStream_t)stream);
}

size_t of3_attn_pair_bias_workspace_bytes(int Ba, int Bz, int N, int c_a, int c_s, int c_z, int H,
                                          int d, int dtype, int flags) {
    Arena ws(nullptr, 0);
    of3_attn_pair_bias_params p = {};
    if (apb_dispatch(nullptr, nullptr, nullptr, nullptr, nullptr, Ba, Bz, N, c_a, c_s, c_z, H, d, 1e9f,
                     dtype, flags, &p, ws, nullptr))
        return 0;
    return ws.off + 256;
}
int of3_attn_pair_bias_forward(const void* a, const void* z, const void* s, const void* mask,
                               void* out, int Ba, int Bz, int N, int c_a, int c_s, int c_z, int H,
                               int d, float inf, int dtype, int flags,
                               const of3_attn_pair_bias_params* p, void* workspace,
                               size_t workspace_bytes, void* stream) {
    CHECK_DTYPE(dtype);
    OF3_REQUIRE(a && z && out && p && workspace, OF3_ERR_ARG, "attn_pair_bias: null pointer argument");
    OF3_REQUIRE(Ba > 0 && Bz > 0 && N > 0 && c_a > 0 && c_z > 0 && H > 0 && d > 0, OF3_ERR_ARG,
                "attn_pair_bias: non-positive size");
    OF3_REQUIRE(Ba % Bz == 0, OF3_ERR_SHAPE, "attn_pair_bias: Ba %d not a multiple of Bz %d", Ba, Bz);
    const bool ada = (flags & OF3_FLAG_ADA_LN) != 0;
    if (ada) {
        OF3_REQUIRE(s && c_s > 0 && p->ada_ln_s_w && p->ada_w_g && p->ada_b_g && p->ada_w_s &&
                        p->w_ada_out && p->b_ada_out,
                    OF3_ERR_ARG, "attn_pair_bias: AdaLN variant needs s and the ada_* parameters");
    } else {
        OF3_REQUIRE(p->ln_a_w && p->ln_a_b, OF3_ERR_ARG, "attn_pair_bias: null layer_norm_a parameter");
    }
    OF3_REQUIRE(p->ln_z_w && p->w_z && p->w_q && p->w_k && p->w_v && p->w_g && p->w_o, OF3_ERR_ARG,
                "attn_pair_bias: null parameter pointer");
    Arena ws(workspace, workspace_bytes);
    return apb_dispatch(a, z, s, mask, out, Ba, Bz, N, c_a, c_s, c_z, H, d, inf, dtype, flags, p, ws,
                        (cudaStream_t)stream);
}

size_t of3_cond_transition_workspace_bytes(long long rows, int c_a, int c_s, int n, int dtype,
                                           int flags) {
    Arena ws(nullptr, 0);
    of3_cond_transition_params p = {};
    if (cond_dispatch(nullptr, nullptr, nullptr, nullptr, rows, c_a, c_s, n, dtype, flags, &p, ws, nullptr))
        return 0;
    return ws.off + 256;
}
int of3_cond_transition_forward(const void* a, const void* s, const void* mask, void* out,
                                long long rows, int c_a, int c_s, int n, int dtype, int flags,
                                const of3_cond_transition_params* p, void* workspace,
                                size_t workspace_bytes, void* stream) {
    CHECK_DTYPE(dtype);
    OF3_REQUIRE(a && s && out && p && workspace, OF3_ERR_ARG, "cond_transition: null pointer argument");
    OF3_REQUIRE(rows > 0 && c_a > 0 && c_s > 0 && n > 0, OF3_ERR_ARG, "cond_transition: non-positive size");
    OF3_REQUIRE(p->ada_ln_s_w && p->ada_w_g && p->ada_b_g && p->ada_w_s && p->w_a && p->w_b && p->w_g &&
                    p->b_g && p->w_out,
                OF3_ERR_ARG, "cond_transition: null parameter pointer");
    Arena ws(workspace, workspace_bytes);
    return cond_dispatch(a, s, mask, out, rows, c_a, c_s, n, dtype, flags, p, ws, (cudaStream_t)stream);
}

}  // extern "C"
