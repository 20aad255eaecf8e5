// Shape-generic SIMT kernels: see generic_ops.cuh. True fp32 arithmetic throughout.
#include "generic_ops.cuh"
#include "runtime.cuh"

namespace of3 {
namespace generic {
namespace {

constexpr int kThreads = 256;

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
__device__ __forceinline__ float sigmoid_acc(float x) { return 1.0f / (1.0f + expf(-x)); }

inline unsigned grid_for(long long n, int per_block) {
    long long g = (n + per_block - 1) / per_block;
    return (unsigned)(g < 1 ? 1 : g);
}

// ------------------------------------------------------------------ LayerNorm
template <typename TX, typename TP>
__global__ void layernorm_kernel(const TX* __restrict__ x, const TP* __restrict__ gamma,
                                 const TP* __restrict__ beta, float* __restrict__ y, long long rows,
                                 int C, float eps, long long inner, long long outer_stride,
                                 long long inner_stride) {
    const int lane = threadIdx.x & 31;
    const long long r = (long long)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
    if (r >= rows) return;
    const TX* xr = x + (r / inner) * outer_stride + (r % inner) * inner_stride;
    float s = 0.f;
    for (int c = lane; c < C; c += 32) s += ld_as_float(xr + c);
    const float mean = warp_sum(s) / (float)C;
    float v = 0.f;
    for (int c = lane; c < C; c += 32) {
        const float d = ld_as_float(xr + c) - mean;
        v += d * d;
    }
    const float rstd = 1.0f / sqrtf(warp_sum(v) / (float)C + eps);
    float* yr = y + r * C;
    for (int c = lane; c < C; c += 32) {
        float o = (ld_as_float(xr + c) - mean) * rstd;
        if (gamma) o *= ld_as_float(gamma + c);
        if (beta) o += ld_as_float(beta + c);
        yr[c] = o;
    }
}

// ------------------------------------------------------------------ strided batched NT GEMM
constexpr int kTM = 64, kTN = 64, kTK = 16;

template <typename TW>
__global__ void __launch_bounds__(256) gemm_nt_kernel(const float* __restrict__ A,
                                                      const TW* __restrict__ W,
                                                      const TW* __restrict__ bias,
                                                      float* __restrict__ out, GemmDesc d) {
    __shared__ float As[kTK][kTM + 1];
    __shared__ float Ws[kTK][kTN + 1];
    const int b = blockIdx.z;
    const int m0 = blockIdx.y * kTM;
    const int n0 = blockIdx.x * kTN;
    const float* Ab = A + (long long)b * d.a_b;
    const TW* Wb = W + (long long)b * d.w_b;
    const int tx = threadIdx.x & 15;  // n micro index
    const int ty = threadIdx.x >> 4;  // m micro index
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < d.K; k0 += kTK) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int idx = threadIdx.x + e * 256;
            const int kk = idx & 15;
            const int mm = idx >> 4;
            const int gm = m0 + mm, gk = k0 + kk;
            As[kk][mm] = (gm < d.M && gk < d.K) ? Ab[(long long)gm * d.a_m + (long long)gk * d.a_k] : 0.f;
            const int gn = n0 + mm;
            Ws[kk][mm] = (gn < d.N && gk < d.K)
                             ? ld_as_float(Wb + (long long)gn * d.w_n + (long long)gk * d.w_k)
                             : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kTK; ++kk) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
    float* ob = out + (long long)b * d.o_b;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= d.M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn >= d.N) continue;
            float v = acc[i][j];
            if (bias) v += ld_as_float(bias + gn);
            ob[(long long)gm * d.o_m + (long long)gn * d.o_n] = v;
        }
    }
}

// ------------------------------------------------------------------ streaming attention
constexpr int kAttWarps = 8;
constexpr int kAttMaxD = 64;

__global__ void __launch_bounds__(kAttWarps * 32)
attention_kernel(const float* __restrict__ q, const float* __restrict__ k,
                 const float* __restrict__ v, const float* __restrict__ mask_bias,
                 const float* __restrict__ pair_bias, float* __restrict__ out, int N, int H, int d,
                 float scale, long long rows_per_bias) {
    __shared__ float Ks[32][kAttMaxD + 1];
    __shared__ float Vs[32][kAttMaxD + 1];
    __shared__ float Qs[kAttWarps][kAttMaxD];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long bb = blockIdx.x;
    const int h = blockIdx.y;
    const int qi = blockIdx.z * kAttWarps + warp;
    const bool q_valid = qi < N;
    const long long row_pitch = (long long)H * d;
    const float* qrow = q + (bb * N + (q_valid ? qi : 0)) * row_pitch + (long long)h * d;
    for (int c = lane; c < d; c += 32) Qs[warp][c] = qrow[c];
    const float* pb = pair_bias
                          ? pair_bias + (((bb / rows_per_bias) * H + h) * (long long)N +
                                         (q_valid ? qi : 0)) * N
                          : nullptr;
    const float* mb = mask_bias ? mask_bias + bb * N : nullptr;
    float m = -INFINITY, l = 0.f, o0 = 0.f, o1 = 0.f;
    for (int k0 = 0; k0 < N; k0 += 32) {
        __syncthreads();
        for (int idx = threadIdx.x; idx < 32 * d; idx += kAttWarps * 32) {
            const int kk = idx / d, c = idx % d;
            const int gk = k0 + kk;
            float kv = 0.f, vv = 0.f;
            if (gk < N) {
                const long long off = (bb * N + gk) * row_pitch + (long long)h * d + c;
                kv = k[off];
                vv = v[off];
            }
            Ks[kk][c] = kv;
            Vs[kk][c] = vv;
        }
        __syncthreads();
        const int gk = k0 + lane;
        float s = -INFINITY;
        if (gk < N) {
            float dot = 0.f;
            for (int c = 0; c < d; ++c) dot = fmaf(Qs[warp][c], Ks[lane][c], dot);
            s = dot * scale;
            if (mb) s += mb[gk];
            if (pb) s += pb[gk];
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float p = (gk < N) ? expf(s - m_new) : 0.f;
        const float corr = expf(m - m_new);
        l = l * corr + warp_sum(p);
        o0 *= corr;
        o1 *= corr;
#pragma unroll 8
        for (int j = 0; j < 32; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            o0 = fmaf(pj, Vs[j][lane], o0);
            if (d > 32) o1 = fmaf(pj, Vs[j][(lane + 32) < kAttMaxD ? lane + 32 : 0], o1);
        }
        m = m_new;
    }
    if (q_valid) {
        float* orow = out + (bb * N + qi) * row_pitch + (long long)h * d;
        const float inv = 1.0f / l;
        if (lane < d) orow[lane] = o0 * inv;
        if (lane + 32 < d) orow[lane + 32] = o1 * inv;
    }
}


// ------------------------------------------------------------------ fused pair-bias projection
// LN(x).w_h = rstd * sum_c (x_c - mean) * (gamma_c w_hc) + sum_c beta_c w_hc
template <typename T>
__global__ void __launch_bounds__(128) pair_bias_c128_h16_kernel(const T* __restrict__ z,
                                                                 const T* __restrict__ gamma,
                                                                 const T* __restrict__ beta,
                                                                 const T* __restrict__ w,
                                                                 float* __restrict__ dst, long long rows,
                                                                 long long nn) {
    __shared__ float ws[16][128];
    __shared__ float cs[16];
    for (int i = threadIdx.x; i < 16 * 128; i += 128) {
        const int c = i & 127;
        ws[i >> 7][c] = ld_as_float(w + i) * (gamma ? ld_as_float(gamma + c) : 1.0f);
    }
    if (threadIdx.x < 16) {
        float a = 0.f;
        if (beta)
            for (int c = 0; c < 128; ++c) a += ld_as_float(beta + c) * ld_as_float(w + threadIdx.x * 128 + c);
        cs[threadIdx.x] = a;
    }
    __syncthreads();
    const long long r = (long long)blockIdx.x * 128 + threadIdx.x;
    if (r >= rows) return;
    float x[128];
    const T* zr = z + r * 128;
    if constexpr (sizeof(T) == 2) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const uint4 v = __ldg(reinterpret_cast<const uint4*>(zr) + i);
            const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                x[i * 8 + j * 2] = bf16lo(u[j]);
                x[i * 8 + j * 2 + 1] = bf16hi(u[j]);
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const float4 v = __ldg(reinterpret_cast<const float4*>(zr) + i);
            x[i * 4] = v.x; x[i * 4 + 1] = v.y; x[i * 4 + 2] = v.z; x[i * 4 + 3] = v.w;
        }
    }
    // four independent partial sums / four heads at a time: the single chains of 128 dependent
    // operations were the critical path at the 8-12 warps per SM that 128 row registers allow
    float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int c = 0; c < 128; c += 4) {
        s4[0] += x[c]; s4[1] += x[c + 1]; s4[2] += x[c + 2]; s4[3] += x[c + 3];
    }
    const float mean = ((s4[0] + s4[1]) + (s4[2] + s4[3])) * (1.0f / 128.0f);
    float v4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int c = 0; c < 128; c += 4) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            x[c + e] -= mean;
            v4[e] = fmaf(x[c + e], x[c + e], v4[e]);
        }
    }
    const float rstd = 1.0f / sqrtf(((v4[0] + v4[1]) + (v4[2] + v4[3])) * (1.0f / 128.0f) + 1e-5f);
    const long long b = r / nn;
    const long long qk = r % nn;
#pragma unroll 1
    for (int h = 0; h < 16; h += 4) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < 128; c += 4) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float4 wv = *reinterpret_cast<const float4*>(&ws[h + e][c]);
                acc[e] = fmaf(x[c], wv.x, acc[e]);
                acc[e] = fmaf(x[c + 1], wv.y, acc[e]);
                acc[e] = fmaf(x[c + 2], wv.z, acc[e]);
                acc[e] = fmaf(x[c + 3], wv.w, acc[e]);
            }
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) dst[(b * 16 + h + e) * nn + qk] = fmaf(acc[e], rstd, cs[h + e]);
    }
}

// ------------------------------------------------------------------ elementwise
template <typename T>
__global__ void gate_mul_mask_kernel(const float* __restrict__ g, const float* __restrict__ p,
                                     int ld, const T* __restrict__ mask, float* __restrict__ dst,
                                     long long rows, int C) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * C) return;
    const long long r = i / C;
    const int c = (int)(i % C);
    const float mk = mask ? ld_as_float(mask + r) : 1.0f;
    dst[i] = mk * sigmoid_acc(g[r * ld + c]) * p[r * ld + c];
}
__global__ void sigmoid_mul_kernel(const float* __restrict__ x, int ldx, const float* __restrict__ g,
                                   int ldg, float* __restrict__ dst, long long rows, int C) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * C) return;
    const long long r = i / C;
    const int c = (int)(i % C);
    dst[i] = x[r * ldx + c] * sigmoid_acc(g[r * ldg + c]);
}
__global__ void silu_mul_kernel(const float* __restrict__ a, const float* __restrict__ b, int ld,
                                float* __restrict__ dst, long long rows, int C) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * C) return;
    const long long r = i / C;
    const int c = (int)(i % C);
    const float av = a[r * ld + c];
    dst[i] = av * sigmoid_acc(av) * b[r * ld + c];
}
__global__ void ada_combine_kernel(const float* __restrict__ g, const float* __restrict__ a,
                                   const float* __restrict__ s, float* __restrict__ dst,
                                   long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = sigmoid_acc(g[i]) * a[i] + s[i];
}
template <typename T>
__global__ void mask_to_bias_kernel(const T* __restrict__ mask, float* __restrict__ dst,
                                    long long rows, int N, float inf, long long row_stride,
                                    long long k_stride) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * N) return;
    const long long r = i / N;
    const int kk = (int)(i % N);
    dst[i] = inf * (ld_as_float(mask + r * row_stride + kk * k_stride) - 1.0f);
}
template <typename T>
__global__ void finalize_kernel(const float* __restrict__ upd, const float* __restrict__ gate,
                                const T* residual, const T* __restrict__ mask, T* out,
                                long long rows, int C, long long inner, long long outer_stride,
                                long long inner_stride) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * C) return;
    const long long r = i / C;
    const int c = (int)(i % C);
    const long long off = (r / inner) * outer_stride + (r % inner) * inner_stride + c;
    float v = upd[i];
    if (gate) v *= sigmoid_acc(gate[i]);
    if (mask) v *= ld_as_float(mask + r);
    if (residual) v += ld_as_float(residual + off);
    st_from_float(out + off, v);
}
__global__ void permute_bias_kernel(const float* __restrict__ src, float* __restrict__ dst,
                                    long long B, int N, int H) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long total = B * H * (long long)N * N;
    if (i >= total) return;
    const int kk = (int)(i % N);
    const int qq = (int)((i / N) % N);
    const int h = (int)((i / ((long long)N * N)) % H);
    const long long b = i / ((long long)N * N * H);
    dst[i] = src[((b * N + qq) * N + kk) * H + h];
}
template <typename T>
__global__ void to_f32_kernel(const T* __restrict__ src, float* __restrict__ dst, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = ld_as_float(src + i);
}

}  // namespace

// ------------------------------------------------------------------ host wrappers
template <typename TX, typename TP>
int layernorm(const TX* x, const TP* gamma, const TP* beta, float* y, long long rows, int C,
              float eps, long long inner, long long outer_stride, long long inner_stride,
              cudaStream_t stream) {
    if (rows <= 0) return OF3_OK;
    LaunchScope scope(20, stream);
    layernorm_kernel<TX, TP><<<grid_for(rows, kThreads / 32), kThreads, 0, stream>>>(
        x, gamma, beta, y, rows, C, eps, inner, outer_stride, inner_stride);
    OF3_CUDA_CHECK(cudaGetLastError());
    return OF3_OK;
}
template int layernorm<float, float>(const float*, const float*, const float*, float*, long long, int,
                                     float, long long, long long, long long, cudaStream_t);
template int layernorm<__nv_bfloat16, __nv_bfloat16>(const __nv_bfloat16*, const __nv_bfloat16*,
                                                     const __nv_bfloat16*, float*, long long, int,
                                                     float, long long, long long, long long,
                                                     cudaStream_t);
template int layernorm<float, __nv_bfloat16>(const float*, const __nv_bfloat16*, const __nv_bfloat16*,
                                             float*, long long, int, float, long long, long long,
                                             long long, cudaStream_t);

template <typename TW>
int gemm_nt(const float* A, const TW* W, const TW* bias, float* out, const GemmDesc& d,
            cudaStream_t stream) {
    if (d.batch <= 0 || d.M <= 0 || d.N <= 0) return OF3_OK;
    OF3_REQUIRE(d.batch <= 65535, OF3_ERR_SHAPE, "gemm_nt: batch %d > 65535", d.batch);
    dim3 grid(ceil_div(d.N, kTN), ceil_div(d.M, kTM), d.batch);
    OF3_REQUIRE(grid.y <= 65535, OF3_ERR_SHAPE, "gemm_nt: M %d too large for one launch", d.M);
    LaunchScope scope(20, stream);
    gemm_nt_kernel<TW><<<grid, 256, 0, stream>>>(A, W, bias, out, d);
    OF3_CUDA_CHECK(cudaGetLastError());
    return OF3_OK;
}
template int gemm_nt<float>(const float*, const float*, const float*, float*, const GemmDesc&,
                            cudaStream_t);
template int gemm_nt<__nv_bfloat16>(const float*, const __nv_bfloat16*, const __nv_bfloat16*, float*,
                                    const GemmDesc&, cudaStream_t);

int attention(const float* q, const float* k, const float* v, const float* mask_bias,
              const float* pair_bias, float* out, long long BB, int N, int H, int d, float scale,
              long long rows_per_bias, cudaStream_t stream) {
    OF3_REQUIRE(d >= 1 && d <= kAttMaxD, OF3_ERR_SHAPE, "attention: head dim %d not in [1, %d]", d,
                kAttMaxD);
    OF3_REQUIRE(H <= 65535, OF3_ERR_SHAPE, "attention: too many heads");
    OF3_REQUIRE(ceil_div(N, kAttWarps) <= 65535, OF3_ERR_SHAPE, "attention: N %d too large", N);
    if (BB <= 0) return OF3_OK;
    dim3 grid((unsigned)BB, H, ceil_div(N, kAttWarps));
    LaunchScope scope(20, stream);
    attention_kernel<<<grid, kAttWarps * 32, 0, stream>>>(q, k, v, mask_bias, pair_bias, out, N, H, d,
                                                          scale, rows_per_bias);
    OF3_CUDA_CHECK(cudaGetLastError());
    return OF3_OK;
}

template <typename T>
int gate_mul_mask(const float* g, const float* p, int ld, const T* mask, float* dst, long long rows,
                  int C, cudaStream_t stream) {
    if (rows <= 0) return OF3_OK;
    LaunchScope scope(20, stream);
    gate_mul_mask_kernel<T><<<grid_for(rows * C, kThreads), kThreads, 0, stream>>>(g, p, ld, mask, dst,
                                                                                  rows, C);
    OF3_CUDA_CHECK(cudaGetLastError());
    return OF3_OK;
}
template int gate_mul_mask<float>(const float*, const float*, int, const float*, float*, long long,
                                  int, cudaStream_t);
template int gate_mul_mask<__nv_bfloat16>(const float*, const float*, int, const __nv_bfloat16*,
                                          float*, long long, int, cudaStream_t);

int sigmoid_mul(const float* x, int ldx, const float* g, int ldg, float* dst, long long rows, int C,
                cudaStream_t stream) {
    if (rows <= 0) return OF3_OK;
    LaunchScope scope(20, stream);
    sigmoid_mul_kernel<<<grid_for(rows * C, kThreads), kThreads, 0, stream>>>(x, ldx, g, ldg, dst,
                                                                             rows, C);
    OF3_CUDA_CHECK(cudaGetLastError());
    return OF3_OK;
}
int silu_mul(const float* a, const float* b, int ld, float* dst, long long rows, int C,
             cudaStream_t stream) {
    if (rows <= 0) return OF3_OK;
    LaunchScope scope(20, stream);
    silu_mul_kernel<<<grid_for(rows * C, kThreads), kThreads, 0, stream>>>(a, b, ld, dst, rows, C);
    OF3_CUDA_CHECK(cudaGetLastError());
    return OF3_OK;
}
int ada_combine(const float* g, const float* a, const float* s, float* dst, long long n,
                cudaStream_t stream) {
    if (n <= 0) return OF3_OK;
    LaunchScope scope(20, stream);
    ada_combine_kernel<<<grid_for(n, kThreads), kThreads, 0, stream>>>(g, a, s, dst, n);
    OF3_CUDA_CHECK(cudaGetLastError());
    return OF3_OK;
}
template <typename T>
int mask_to_bias(const T* mask, float* dst, long long rows, int N, float inf, long long row_stride,
                 long long k_stride, cudaStream_t stream) {
    if (rows <= 0) return OF3_OK;
    LaunchScope scope(20, stream);
    mask_to_bias_kernel<T><<<grid_for(rows * N, kThreads), kThreads, 0, stream>>>(
        mask, dst, rows, N, inf, row_stride, k_stride);
    OF3_CUDA_CHECK(cudaGetLastError());
    return OF3_OK;
}
template int mask_to_bias<float>(const float*, float*, long long, int, float, long long, long long,
                                 cudaStream_t);
template int mask_to_bias<__nv_bfloat16>(const __nv_bfloat16*, float*, long long, int, float,
                                         long long, long long, cudaStream_t);

template <typename T>
int finalize(const float* upd, const float* gate, const T* residual, const T* mask, T* out,
             long long rows, int C, long long inner, long long outer_stride,
             long long inner_stride, cudaStream_t stream) {
    if (rows <= 0) return OF3_OK;
    LaunchScope scope(20, stream);
    finalize_kernel<T><<<grid_for(rows * C, kThreads), kThreads, 0, stream>>>(
        upd, gate, residual, mask, out, rows, C, inner, outer_stride, inner_stride);
    OF3_CUDA_CHECK(cudaGetLastError());
    return OF3_OK;
}
template int finalize<float>(const float*, const float*, const float*, const float*, float*,
                             long long, int, long long, long long, long long, cudaStream_t);
template int finalize<__nv_bfloat16>(const float*, const float*, const __nv_bfloat16*,
                                     const __nv_bfloat16*, __nv_bfloat16*, long long, int, long long,
                                     long long, long long, cudaStream_t);


template <typename T>
int pair_bias_c128_h16(const T* z, const T* gamma, const T* beta, const T* w, float* dst, long long B,
                       long long positions_per_sample, cudaStream_t stream) {
    const long long nn = positions_per_sample;
    const long long rows = B * nn;
    if (rows <= 0) return OF3_OK;
    OF3_REQUIRE(((uintptr_t)z & 15) == 0, OF3_ERR_ALIGN, "pair_bias: z must be 16-byte aligned");
    LaunchScope scope(20, stream);
    pair_bias_c128_h16_kernel<T><<<grid_for(rows, 128), 128, 0, stream>>>(z, gamma, beta, w, dst, rows, nn);
    OF3_CUDA_CHECK(cudaGetLastError());
    return OF3_OK;
}
template int pair_bias_c128_h16<float>(const float*, const float*, const float*, const float*, float*,
                                       long long, long long, cudaStream_t);
template int pair_bias_c128_h16<__nv_bfloat16>(const __nv_bfloat16*, const __nv_bfloat16*, const __nv_bfloat16*,
                                               const __nv_bfloat16*, float*, long long, long long, cudaStream_t);

int permute_bias(const float* src, float* dst, long long B, int N, int H, cudaStream_t stream) {
    const long long total = B * H * (long long)N * N;
    if (total <= 0) return OF3_OK;
    LaunchScope scope(20, stream);
    permute_bias_kernel<<<grid_for(total, kThreads), kThreads, 0, stream>>>(src, dst, B, N, H);
    OF3_CUDA_CHECK(cudaGetLastError());
    return OF3_OK;
}

template <typename T>
int to_f32(const T* src, float* dst, long long n, cudaStream_t stream) {
    if (n <= 0) return OF3_OK;
    LaunchScope scope(20, stream);
    to_f32_kernel<T><<<grid_for(n, kThreads), kThreads, 0, stream>>>(src, dst, n);
    OF3_CUDA_CHECK(cudaGetLastError());
    return OF3_OK;
}
template int to_f32<float>(const float*, float*, long long, cudaStream_t);
template int to_f32<__nv_bfloat16>(const __nv_bfloat16*, float*, long long, cudaStream_t);

}  // namespace generic
}  // namespace of3
