// Runtime support: per-thread error string, per-device status block, tensor-map encoding.
#include "runtime.cuh"

#include <cudaTypedefs.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

namespace of3 {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

static const int kMaxDevices = 64;
static int* g_status[kMaxDevices] = {nullptr};
static int g_sm_count[kMaxDevices] = {0};
static std::mutex g_mu;

int* device_status_ptr() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_status[dev] == nullptr) {
        int* p = nullptr;
        if (cudaMalloc(&p, 16 * sizeof(int)) != cudaSuccess) return nullptr;
        if (cudaMemset(p, 0, 16 * sizeof(int)) != cudaSuccess) return nullptr;
        g_status[dev] = p;
    }
    return g_status[dev];
}

int sm_count() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_sm_count[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
        g_sm_count[dev] = n;
    }
    return g_sm_count[dev];
}

static unsigned g_configured[kMaxDevices] = {0};

bool device_configured(int key) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices || key < 0 || key >= 32) return false;
    std::lock_guard<std::mutex> lk(g_mu);
    return (g_configured[dev] >> key) & 1u;
}

void device_mark_configured(int key) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices || key < 0 || key >= 32) return;
    std::lock_guard<std::mutex> lk(g_mu);
    g_configured[dev] |= 1u << key;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    std::lock_guard<std::mutex> lk(g_mu);
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
                cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

static std::unordered_map<std::string, CUtensorMap> g_tmaps;
static const size_t kMaxCachedTmaps = 8192;

int make_tmap_bf16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                   const uint64_t* strides_bytes, const uint32_t* box, int swizzle) {
    EncodeTiledFn fn = encode_fn();
    OF3_REQUIRE(fn != nullptr, OF3_ERR_DRIVER, "cuTensorMapEncodeTiled entry point unavailable");
    OF3_REQUIRE(((uintptr_t)base & 15) == 0, OF3_ERR_ALIGN, "tensor map base not 16-byte aligned");
    cuuint64_t gdim[5];
    cuuint64_t gstr[5];
    cuuint32_t bx[5];
    cuuint32_t es[5];
    for (int i = 0; i < rank; ++i) {
        gdim[i] = dims[i];
        bx[i] = box[i];
        es[i] = 1;
        if (i > 0) {
            OF3_REQUIRE((strides_bytes[i - 1] & 15) == 0, OF3_ERR_ALIGN,
                        "tensor map stride %d (%llu B) not a multiple of 16", i,
                        (unsigned long long)strides_bytes[i - 1]);
            gstr[i - 1] = strides_bytes[i - 1];
        }
    }
    // cache key: every argument of the encoding (a tensor map holds no device state: the same
    // arguments give the same 128 bytes on every device of the process)
    std::string key;
    key.reserve(8 + 4 + rank * 20 + 4);
    auto put = [&key](const void* p, size_t n) { key.append((const char*)p, n); };
    put(&base, sizeof(base));
    put(&rank, sizeof(rank));
    put(gdim, rank * sizeof(cuuint64_t));
    put(gstr, (rank - 1) * sizeof(cuuint64_t));
    put(bx, rank * sizeof(cuuint32_t));
    put(&swizzle, sizeof(swizzle));
    {
        std::lock_guard<std::mutex> lk(g_mu);
        auto it = g_tmaps.find(key);
        if (it != g_tmaps.end()) {
            *out = it->second;
            return OF3_OK;
        }
    }
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base),
                    gdim, gstr, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle == 1 ? CU_TENSOR_MAP_SWIZZLE_128B
                                 : (swizzle == 2 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE),
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    OF3_REQUIRE(r == CUDA_SUCCESS, OF3_ERR_DRIVER, "cuTensorMapEncodeTiled failed with CUresult %d",
                (int)r);
    {
        std::lock_guard<std::mutex> lk(g_mu);
        if (g_tmaps.size() >= kMaxCachedTmaps) g_tmaps.clear();  // bounded: callers with ever-new buffers
        g_tmaps.emplace(std::move(key), *out);
    }
    return OF3_OK;
}

// ------------------------------------------------------------------ launch accounting
struct ProfRec {
    cudaEvent_t a, b;
    int kid;
};
static std::vector<ProfRec> g_recs;      // event pairs of the current profiling window
static std::vector<cudaEvent_t> g_pool;  // recycled events
static long long g_launches[kMaxKernelIds] = {0};
static bool g_prof_on = false;

static cudaEvent_t take_event() {
    if (!g_pool.empty()) {
        cudaEvent_t e = g_pool.back();
        g_pool.pop_back();
        return e;
    }
    cudaEvent_t e = nullptr;
    cudaEventCreate(&e);
    return e;
}

LaunchScope::LaunchScope(int kernel_id, cudaStream_t st) : kid(kernel_id), stream(st), rec(nullptr) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (kid >= 0 && kid < kMaxKernelIds) g_launches[kid]++;
    if (g_prof_on) {
        ProfRec r{take_event(), take_event(), kid};
        if (r.a && r.b) {
            cudaEventRecord(r.a, stream);
            g_recs.push_back(r);
            rec = (void*)(uintptr_t)g_recs.size();  // index + 1
        }
    }
}
LaunchScope::~LaunchScope() {
    if (rec) {
        std::lock_guard<std::mutex> lk(g_mu);
        const size_t idx = (size_t)(uintptr_t)rec - 1;
        if (idx < g_recs.size()) cudaEventRecord(g_recs[idx].b, stream);
    }
}

}  // namespace of3

extern "C" int of3_profile_enable(int on) {
    std::lock_guard<std::mutex> lk(of3::g_mu);
    of3::g_prof_on = on != 0;
    return OF3_OK;
}

extern "C" int of3_profile_reset(void) {
    std::lock_guard<std::mutex> lk(of3::g_mu);
    for (auto& r : of3::g_recs) {
        of3::g_pool.push_back(r.a);
        of3::g_pool.push_back(r.b);
    }
    of3::g_recs.clear();
    for (int i = 0; i < of3::kMaxKernelIds; ++i) of3::g_launches[i] = 0;
    return OF3_OK;
}

extern "C" int of3_profile_read(int kernel_id, long long* launches, float* total_ms) {
    OF3_REQUIRE(kernel_id >= 0 && kernel_id < of3::kMaxKernelIds && launches && total_ms, OF3_ERR_ARG,
                "of3_profile_read: bad argument");
    OF3_CUDA_CHECK(cudaDeviceSynchronize());
    std::lock_guard<std::mutex> lk(of3::g_mu);
    *launches = of3::g_launches[kernel_id];
    float sum = 0.f;
    for (auto& r : of3::g_recs) {
        if (r.kid != kernel_id) continue;
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, r.a, r.b) == cudaSuccess) sum += ms;
    }
    *total_ms = sum;
    return OF3_OK;
}

extern "C" const char* of3_last_error_string(void) { return of3::g_err; }

extern "C" int of3_device_status(int* out4) {
    int* p = of3::device_status_ptr();
    OF3_REQUIRE(p != nullptr, OF3_ERR_ARG, "no device status block (no CUDA device?)");
    OF3_REQUIRE(out4 != nullptr, OF3_ERR_ARG, "out4 is null");
    OF3_CUDA_CHECK(cudaMemcpy(out4, p, 4 * sizeof(int), cudaMemcpyDeviceToHost));
    return OF3_OK;
}

// Stream-ordered copy of the status block into pinned host memory (no synchronisation): callers that replay
// CUDA graphs read it one step late instead of stalling the stream.
extern "C" int of3_device_status_async(int* host4, void* stream) {
    int* p = of3::device_status_ptr();
    OF3_REQUIRE(p != nullptr, OF3_ERR_ARG, "no device status block (no CUDA device?)");
    OF3_REQUIRE(host4 != nullptr, OF3_ERR_ARG, "host4 is null");
    OF3_CUDA_CHECK(cudaMemcpyAsync(host4, p, 4 * sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    return OF3_OK;
}

extern "C" int of3_device_status_clear(void) {
    int* p = of3::device_status_ptr();
    OF3_REQUIRE(p != nullptr, OF3_ERR_ARG, "no device status block (no CUDA device?)");
    OF3_CUDA_CHECK(cudaMemset(p, 0, 16 * sizeof(int)));
    return OF3_OK;
}
