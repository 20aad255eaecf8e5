// Entry points for the row-sharded ("DAP") pair stack: each rank owns R = N / P consecutive rows of
// the pair tensor z[N, N, 128] (bf16, one sample) and runs every layer in two phases around the one
// exchange step the layer needs. The exchange itself (NCCL all-gather / all-to-all through
// torch.distributed) is done by the caller between the phases; remote data always lands in this
// GPU's own memory first and the kernels only ever read local memory.
//
//   triangle update  project: local rows -> a_t, b_t (channel-major, one group of 128 / P channels per
//                    destination rank) | all-to-all: rows -> channels | contract: this rank's channels
//                    over ALL rows, output grouped by the rank that owns each row | all-to-all back |
//                    output: LN / linear / gate / residual on the local rows
//   triangle attn    project: q, k, v^T and the local rows of the pair bias | all-gather bias |
//                    finish: attention over the local lines, gate, output projection, residual
//   The incoming update projects with a transposed walk over the local rows (no transposed copy of
//   z); ending-node attention runs the same phases on the all-to-all-transposed shard.
#include "generic_ops.cuh"
#include "modules.cuh"
#include "runtime.cuh"

using namespace of3;

namespace {
// Rows of `row_bytes` bytes indexed by (i0, i1, i2); byte strides per index on both sides. The rows are
// cut into vectors V (16 bytes when everything is 16-byte aligned, else 2 bytes) and the vectors are
// dealt to threads in flat order, so short rows still fill a warp; four independent vectors per thread
// and step keep enough loads in flight.
template <typename V>
__global__ void __launch_bounds__(256)
copy_rows_3d_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, long long n_rows, int n1, int n2,
                    long long s0, long long s1, long long s2, long long t0, long long t1, long long t2,
                    int vec_per_row) {
    const long long total = n_rows * vec_per_row;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long base = (long long)blockIdx.x * blockDim.x + threadIdx.x; base < total; base += 4 * stride) {
        V val[4];
        long long doff[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const long long idx = base + u * stride;
            doff[u] = -1;
            if (idx < total) {
                const long long row = idx / vec_per_row;
                const int v = (int)(idx - row * vec_per_row);
                const int i2 = (int)(row % n2);
                const long long r1 = row / n2;
                const int i1 = (int)(r1 % n1);
                const long long i0 = r1 / n1;
                val[u] = reinterpret_cast<const V*>(src + i0 * s0 + i1 * s1 + i2 * s2)[v];
                doff[u] = i0 * t0 + i1 * t1 + i2 * t2 + (long long)v * (long long)sizeof(V);
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (doff[u] >= 0) *reinterpret_cast<V*>(dst + doff[u]) = val[u];
    }
}
}  // namespace

extern "C" {

int of3_copy_rows_3d(const void* src, void* dst, int n0, int n1, int n2, long long s0, long long s1, long long s2,
                     long long t0, long long t1, long long t2, int row_bytes, void* stream) {
    OF3_REQUIRE(src && dst, OF3_ERR_ARG, "copy_rows_3d: null pointer argument");
    OF3_REQUIRE(n0 > 0 && n1 > 0 && n2 > 0 && row_bytes > 0 && row_bytes % 2 == 0, OF3_ERR_ARG,
                "copy_rows_3d: bad sizes");
    const long long n_rows = (long long)n0 * n1 * n2;
    const bool vec = (((uintptr_t)src | (uintptr_t)dst | (uintptr_t)s0 | (uintptr_t)s1 | (uintptr_t)s2 |
                       (uintptr_t)t0 | (uintptr_t)t1 | (uintptr_t)t2 | (uintptr_t)row_bytes) & 15) == 0;
    const int vpr = vec ? row_bytes / 16 : row_bytes / 2;
    long long blocks = (n_rows * vpr + 4 * 256 - 1) / (4 * 256);
    const long long cap = (long long)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    LaunchScope scope(20, (cudaStream_t)stream);
    if (vec)
        copy_rows_3d_kernel<uint4><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
            (const uint8_t*)src, (uint8_t*)dst, n_rows, n1, n2, s0, s1, s2, t0, t1, t2, vpr);
    else
        copy_rows_3d_kernel<uint16_t><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
            (const uint8_t*)src, (uint8_t*)dst, n_rows, n1, n2, s0, s1, s2, t0, t1, t2, vpr);
    OF3_CUDA_CHECK(cudaGetLastError());
    return OF3_OK;
}

size_t of3_attn_pair_bias_rows_workspace_bytes(int N, int R, int c_a) {
    Arena ws(nullptr, 0);
    fast::attn_pair_bias_rows(nullptr, nullptr, nullptr, nullptr, N, 0, R, c_a, 16, c_a / 16, 0.f, 0, nullptr, ws, 0);
    return ws.off + 256;
}

int of3_attn_pair_bias_forward_rows(const void* a, const float* pair_bias_rows, const void* mask, void* out_rows,
                                    int N, int row0, int R, int c_a, int H, int d, float inf, int dtype, int flags,
                                    const of3_attn_pair_bias_params* p, void* workspace, size_t workspace_bytes,
                                    void* stream) {
    OF3_REQUIRE(a && pair_bias_rows && out_rows && p && workspace, OF3_ERR_ARG,
                "attn_pair_bias_rows: null pointer argument");
    OF3_REQUIRE(dtype == OF3_DTYPE_BF16 && !(flags & OF3_FLAG_ADA_LN) &&
                    fast::attn_pair_bias_supported(1, 1, N, c_a, 0, 128, H, d, flags),
                OF3_ERR_SHAPE, "attn_pair_bias_rows: bf16, 16 heads of 24 or 48 only");
    Arena ws(workspace, workspace_bytes);
    return fast::attn_pair_bias_rows((const __nv_bfloat16*)a, pair_bias_rows, (const __nv_bfloat16*)mask,
                                     (__nv_bfloat16*)out_rows, N, row0, R, c_a, H, d, inf, flags, p, ws,
                                     (cudaStream_t)stream);
}

int of3_dap_pitch(int N, int multiple) { return (int)align_up((size_t)N, (size_t)multiple); }

long long of3_dap_triattn_image_elems(int R, int N) { return (long long)fast::triattn_image_elems(1, R, N); }

long long of3_dap_triattn_bias_elems(int R, int N) { return (long long)fast::triattn_bias_elems(1, R, N); }

int of3_dap_trimul_project(const void* z_rows, const void* mask, void* ab, int lines, int positions, int transposed,
                           int world, const of3_trimul_params* p, void* stream) {
    OF3_REQUIRE(z_rows && ab && p, OF3_ERR_ARG, "dap_trimul_project: null pointer argument");
    OF3_REQUIRE(lines > 0 && positions > 0, OF3_ERR_ARG, "dap_trimul_project: non-positive size");
    OF3_REQUIRE(world == 1 || world == 2 || world == 4 || world == 8, OF3_ERR_ARG,
                "dap_trimul_project: world must be 1, 2, 4 or 8 (got %d)", world);
    const int ld = (int)align_up(positions, 8);
    const long long plane = (long long)(128 / world) * lines * ld;  // one rank's channels of a (or b)
    __nv_bfloat16* a_t = (__nv_bfloat16*)ab;
    return fast::trimul_project((const __nv_bfloat16*)z_rows, (const __nv_bfloat16*)mask, a_t, a_t + plane, 1, lines,
                                positions, ld, transposed != 0, p, (cudaStream_t)stream, world, 2 * plane);
}

int of3_dap_trimul_contract(const void* ab_all, void* x_blocks, int N, int channels, int rows_per_rank,
                            void* stream) {
    OF3_REQUIRE(ab_all && x_blocks, OF3_ERR_ARG, "dap_trimul_contract: null pointer argument");
    OF3_REQUIRE(N > 0 && channels > 0 && rows_per_rank > 0 && N % rows_per_rank == 0, OF3_ERR_ARG,
                "dap_trimul_contract: bad sizes N=%d channels=%d rows_per_rank=%d", N, channels, rows_per_rank);
    const int ld = (int)align_up(N, 8);
    const __nv_bfloat16* a = (const __nv_bfloat16*)ab_all;
    const long long plane = (long long)N * ld;
    return contract_nt_bf16(a, a + (long long)channels * plane, (__nv_bfloat16*)x_blocks, channels, N, N, N, ld, ld, ld,
                            plane, plane, (long long)rows_per_rank * ld, (cudaStream_t)stream, rows_per_rank,
                            (long long)channels * rows_per_rank * ld);
}

int of3_dap_trimul_output(const void* z_rows, void* out_rows, const void* x_t, int R, int N, int flags,
                          const of3_trimul_params* p, void* stream) {
    OF3_REQUIRE(z_rows && out_rows && x_t && p, OF3_ERR_ARG, "dap_trimul_output: null pointer argument");
    OF3_REQUIRE(R > 0 && N > 0, OF3_ERR_ARG, "dap_trimul_output: non-positive size");
    return fast::trimul_output((const __nv_bfloat16*)z_rows, (__nv_bfloat16*)out_rows, (const __nv_bfloat16*)x_t, 1, R,
                               N, (int)align_up(N, 8), (flags & OF3_FLAG_ADD_RESIDUAL) ? 1 : 0, p,
                               (cudaStream_t)stream);
}

int of3_dap_triattn_project(const void* z_rows, void* q, void* k, void* vt, void* bias_rows, int R, int N, int row0,
                            const of3_triattn_params* p, void* stream) {
    OF3_REQUIRE(z_rows && q && k && vt && bias_rows && p, OF3_ERR_ARG, "dap_triattn_project: null pointer argument");
    OF3_REQUIRE(R > 0 && N > 0 && row0 >= 0 && row0 + R <= N, OF3_ERR_ARG,
                "dap_triattn_project: bad sizes R=%d N=%d row0=%d", R, N, row0);
    return fast::triattn_project((const __nv_bfloat16*)z_rows, (__nv_bfloat16*)q, (__nv_bfloat16*)k,
                                 (__nv_bfloat16*)vt, (__nv_bfloat16*)bias_rows, 1, R, N, row0, false, p,
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
                                N, inf, false, (flags & OF3_FLAG_ADD_RESIDUAL) ? 1 : 0, p, (cudaStream_t)stream);
}

int of3_pair_bias_project(const void* z_rows, const void* ln_w, const void* ln_b, const void* w, float* bias_rows,
                          long long positions, int c_z, int H, int dtype, void* stream) {
    OF3_REQUIRE(z_rows && w && bias_rows, OF3_ERR_ARG, "pair_bias_project: null pointer argument");
    OF3_REQUIRE(c_z == 128 && H == 16, OF3_ERR_SHAPE, "pair_bias_project: only c_z = 128, 16 heads");
    if (dtype == OF3_DTYPE_BF16)
        return fast::pair_bias_c128_h16((const __nv_bfloat16*)z_rows, (const __nv_bfloat16*)ln_w,
                                        (const __nv_bfloat16*)ln_b, (const __nv_bfloat16*)w, bias_rows, 1, positions,
                                        (cudaStream_t)stream);
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
    if (dtype == OF3_DTYPE_BF16 && fast::attn_pair_bias_supported(Ba, Bz, N, c_a, c_s, 128, H, d, flags))
        return fast::attn_pair_bias((const __nv_bfloat16*)a, nullptr, (const __nv_bfloat16*)s,
                                    (const __nv_bfloat16*)mask, (__nv_bfloat16*)out, Ba, Bz, N, c_a, c_s, H, d, inf,
                                    flags, p, ws, (cudaStream_t)stream, pair_bias);
    if (dtype == OF3_DTYPE_BF16)
        return generic::attn_pair_bias<__nv_bfloat16>((const __nv_bfloat16*)a, nullptr, (const __nv_bfloat16*)s,
                                                      (const __nv_bfloat16*)mask, (__nv_bfloat16*)out, Ba, Bz, N, c_a,
                                                      c_s, 128, H, d, inf, flags, p, ws, (cudaStream_t)stream, pair_bias);
    OF3_REQUIRE(dtype == OF3_DTYPE_F32, OF3_ERR_ARG, "attn_pair_bias_prebias: bad dtype %d", dtype);
    return generic::attn_pair_bias<float>((const float*)a, nullptr, (const float*)s, (const float*)mask, (float*)out, Ba,
                                          Bz, N, c_a, c_s, 128, H, d, inf, flags, p, ws, (cudaStream_t)stream, pair_bias);
}

long long of3_pair_bias_tiles_elems(int N) { return 16LL * ((N + 31) / 32) * N * 32; }

int of3_pair_bias_project_tiles(const void* z, const void* ln_w, const void* ln_b, const void* w, void* tiles, int N,
                                int c_z, int H, int dtype, void* stream) {
    OF3_REQUIRE(z && w && tiles, OF3_ERR_ARG, "pair_bias_project_tiles: null pointer argument");
    OF3_REQUIRE(c_z == 128 && H == 16 && dtype == OF3_DTYPE_BF16 && N > 0, OF3_ERR_SHAPE,
                "pair_bias_project_tiles: only bf16, c_z = 128, 16 heads");
    return fast::pair_bias_tiles_c128_h16((const __nv_bfloat16*)z, (const __nv_bfloat16*)ln_w, (const __nv_bfloat16*)ln_b,
                                          (const __nv_bfloat16*)w, (__nv_bfloat16*)tiles, 1, N, (cudaStream_t)stream);
}

int of3_attn_pair_bias_forward_pretiles(const void* a, const void* bias_tiles, const void* s, const void* mask,
                                        void* out, int Ba, int Bz, int N, int c_a, int c_s, int H, int d, float inf,
                                        int dtype, int flags, const of3_attn_pair_bias_params* p, void* workspace,
                                        size_t workspace_bytes, void* stream) {
    OF3_REQUIRE(a && bias_tiles && out && p && workspace, OF3_ERR_ARG, "attn_pair_bias_pretiles: null pointer argument");
    OF3_REQUIRE(Ba > 0 && Bz > 0 && Ba % Bz == 0 && N > 0, OF3_ERR_ARG, "attn_pair_bias_pretiles: bad sizes");
    OF3_REQUIRE(dtype == OF3_DTYPE_BF16 && fast::attn_pair_bias_supported(Ba, Bz, N, c_a, c_s, 128, H, d, flags),
                OF3_ERR_SHAPE, "attn_pair_bias_pretiles: bias tiles only feed the bf16 tensor-core attention");
    Arena ws(workspace, workspace_bytes);
    return fast::attn_pair_bias((const __nv_bfloat16*)a, nullptr, (const __nv_bfloat16*)s, (const __nv_bfloat16*)mask,
                                (__nv_bfloat16*)out, Ba, Bz, N, c_a, c_s, H, d, inf, flags, p, ws, (cudaStream_t)stream,
                                nullptr, (const __nv_bfloat16*)bias_tiles);
}

}  // extern "C"
