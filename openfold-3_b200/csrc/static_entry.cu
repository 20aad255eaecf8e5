// of3_trimul_forward_static: the triangle multiplicative update for callers that cannot allocate.
//
// Some hosts of this library cannot call cudaMalloc (or hand over a workspace they got from an
// allocator): a serving process that froze its device-memory budget after start-up, a plugin that
// runs inside somebody else's stream-ordered region where allocating would synchronise the device,
// an embedder that only passes the tensors it was given. For them this one entry point brings its
// own scratch: a fixed 16 MiB array in device global memory that is part of the library image, so
// every GPU that loads the library holds those 16 MiB until the process exits.
//
// It runs the shape-generic kernel chain (fp32 arithmetic, fp32 or bf16 storage), whose
// intermediates all live in that array, and it calls no cudaMalloc / cudaFree and no allocating
// library routine. Limits and rules:
//   * B * N * N * max(c_z, c_hidden) * 24 bytes (+ alignment) must fit in 16 MiB, e.g. N <= 73 for
//     B = 1, c = 128; larger problems are rejected with OF3_ERR_WORKSPACE and a message.
//   * The first call on a device looks the array's device address up (cudaGetSymbolAddress, with
//     that device current) and caches it; make that first call outside any stream capture.
//   * All calls share the one array, and it keeps whatever the last call left in it. Nothing in
//     the chain needs zero-initialised scratch (every buffer is fully written before it is read),
//     but two calls whose kernels overlap on the GPU (different streams, or graphs replayed
//     concurrently) race on it: serialise them.
//   * Launch timing (of3_profile_enable) creates CUDA events on demand; leave it off here.
#include <mutex>

#include "modules.cuh"

namespace {

constexpr size_t kStaticScratchBytes = 16u << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDev = 64;
std::mutex g_setup_mu;
void* g_scratch_addr[kMaxDev] = {nullptr};

// Device address of the scratch array on the current device. In host code the array's name is
// only a handle for the runtime, never a pointer a kernel could use.
int static_scratch(void** out) {
    int dev = 0;
    OF3_CUDA_CHECK(cudaGetDevice(&dev));
    OF3_REQUIRE(dev >= 0 && dev < kMaxDev, OF3_ERR_ARG, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lk(g_setup_mu);
    if (g_scratch_addr[dev] == nullptr) {
        void* p = nullptr;
        OF3_CUDA_CHECK(cudaGetSymbolAddress(&p, g_static_scratch));
        OF3_REQUIRE(p != nullptr, OF3_ERR_DRIVER, "cudaGetSymbolAddress returned a null address");
        g_scratch_addr[dev] = p;
    }
    *out = g_scratch_addr[dev];
    return OF3_OK;
}

}  // namespace

extern "C" size_t of3_trimul_static_scratch_bytes(void) { return kStaticScratchBytes; }

extern "C" int of3_trimul_forward_static(const void* z, const void* mask, void* out, int B, int N, int c_z,
                                         int c_h, int dtype, int flags, const of3_trimul_params* p,
                                         void* stream) {
    using namespace of3;
    OF3_REQUIRE(dtype == OF3_DTYPE_BF16 || dtype == OF3_DTYPE_F32, OF3_ERR_ARG,
                "dtype %d is neither OF3_DTYPE_BF16 nor OF3_DTYPE_F32", dtype);
    OF3_REQUIRE(z && out && p, OF3_ERR_ARG, "trimul_static: null pointer argument");
    OF3_REQUIRE(B > 0 && N > 0 && c_z > 0 && c_h > 0, OF3_ERR_ARG, "trimul_static: non-positive size");
    OF3_REQUIRE(p->ln_in_w && p->ln_in_b && p->w_a_p && p->w_a_g && p->w_b_p && p->w_b_g && p->w_g &&
                    p->ln_out_w && p->ln_out_b && p->w_z,
                OF3_ERR_ARG, "trimul_static: null parameter pointer");
    // size the chain first (no device work), reject what does not fit
    Arena probe(nullptr, 0);
    int rc = dtype == OF3_DTYPE_BF16
                 ? generic::trimul<__nv_bfloat16>(nullptr, nullptr, nullptr, B, N, c_z, c_h, flags, p, probe, nullptr)
                 : generic::trimul<float>(nullptr, nullptr, nullptr, B, N, c_z, c_h, flags, p, probe, nullptr);
    if (rc) return rc;
    OF3_REQUIRE(probe.off <= kStaticScratchBytes, OF3_ERR_WORKSPACE,
                "trimul_static: B=%d N=%d c_z=%d c_hidden=%d needs %zu bytes of scratch, the built-in array "
                "holds %zu; use of3_trimul_forward with a caller-owned workspace",
                B, N, c_z, c_h, probe.off, kStaticScratchBytes);
    void* scratch = nullptr;
    if ((rc = static_scratch(&scratch))) return rc;
    Arena ws(scratch, kStaticScratchBytes);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == OF3_DTYPE_BF16)
        return generic::trimul<__nv_bfloat16>((const __nv_bfloat16*)z, (const __nv_bfloat16*)mask,
                                              (__nv_bfloat16*)out, B, N, c_z, c_h, flags, p, ws, st);
    return generic::trimul<float>((const float*)z, (const float*)mask, (float*)out, B, N, c_z, c_h, flags, p,
                                  ws, st);
}
