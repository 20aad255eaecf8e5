// Exchanges between the GPUs of one node over NVLink peer memory, without a collective library:
//
//   * every rank owns one "peer heap" (cudaMalloc, exported with cudaIpcGetMemHandle and mapped by the
//     other ranks' processes with cudaIpcOpenMemHandle); the same byte offset names the same logical
//     buffer on every rank;
//   * an exchange is  barrier  ->  pull: after the barrier every rank's producer kernels have finished,
//     and each rank then reads what it needs straight out of its peers' heaps (plain 16-byte loads over
//     NVLink) and writes it, already in the layout its next kernel reads, into its own memory. The
//     all-to-all, the all-gather and the repack that used to follow them are one kernel;
//   * the barrier is a kernel of one warp: lane p stores this rank's epoch into peer p's flag word and
//     spins, for at most two seconds, until peer p's epoch has arrived in its own flag words. When the
//     limit runs out the kernel records a status word (kernel id 30) and returns; nothing waits forever.
//     The pull kernels that follow see the status word and move nothing, the host raises on its next status
//     check: a step with a failed barrier never yields a silently wrong result. The first barrier of a step
//     (of3_peer_barrier_step_entry) has a one-minute limit, because there the ranks' hosts may be far apart.
//     Each rank runs on its own GPU, so the waiting kernels are always co-resident.
//
// A buffer may be overwritten by its owner only after another barrier has been passed since the peers
// pulled from it; the callers' exchange sequences have that property (see dap.py).
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"
#include "of3b200.h"
#include "runtime.cuh"

using namespace of3;

namespace {

constexpr int kMaxPeers = 8;
constexpr int kKidBarrier = 30;
constexpr uint64_t kBarrierLimitNs = 2000000000ull;         // between the layers of a step: ranks are in lock step
constexpr uint64_t kStepEntryLimitNs = 60000000000ull;      // first barrier of a step: covers host skew between ranks

struct PeerPtrs {
    void* p[kMaxPeers];
};

__device__ __forceinline__ uint64_t gtimer() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// flags.p[r] -> rank r's flag block: words [0, 8) = epoch last announced by rank 0..7, word 8 = r's own epoch
__global__ void __launch_bounds__(32) peer_barrier_kernel(PeerPtrs flags, int world, int rank, uint64_t limit_ns,
                                                          int* status) {
    unsigned* mine = reinterpret_cast<unsigned*>(flags.p[rank]);
    unsigned epoch = 0;
    if (threadIdx.x == 0) {
        epoch = mine[8] + 1;
        mine[8] = epoch;
    }
    epoch = __shfl_sync(0xffffffffu, epoch, 0);
    if ((int)threadIdx.x < world && (int)threadIdx.x != rank) {
        __threadfence_system();  // everything earlier kernels of this GPU wrote is visible before the flag
        st_release_sys(reinterpret_cast<unsigned*>(flags.p[threadIdx.x]) + rank, epoch);
        // a step that has already failed announces its epoch (the peers are not held up) but waits no more
        if (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0) return;
        const uint64_t t0 = gtimer();
        unsigned spins = 0;
        while ((int)(ld_acquire_sys(mine + threadIdx.x) - epoch) < 0) {
            if ((++spins & 255u) == 0 && gtimer() - t0 > limit_ns) {
                if (status != nullptr && atomicCAS(status, 0, 1) == 0) {
                    status[1] = kKidBarrier;
                    status[2] = (int)threadIdx.x;  // the peer that did not arrive
                    status[3] = (int)epoch;
                    __threadfence();
                }
                break;
            }
        }
    }
}

// Rows of row_bytes bytes indexed (i0, i1, i2); i0 selects the SOURCE RANK: row (i0, i1, i2) is read at
// srcs.p[i0] + src_off + i1*s1 + i2*s2 and written at dst + i0*t0 + i1*t1 + i2*t2. Vectors are dealt
// to threads in flat order with the source index rotated by this rank, so that at any moment the ranks
// read from different peers.
// kPush: the same index space with the roles swapped -- the row is read from the LOCAL buffer `dst` and
// written into rank i0's heap (posted writes instead of read round trips).
template <typename V, bool kPush>
__global__ void __launch_bounds__(256)
peer_pull_rows_kernel(PeerPtrs srcs, long long src_off, uint8_t* __restrict__ dst, int n0, int n1, int n2,
                      long long s1, long long s2, long long t0, long long t1, long long t2, int vec_per_row,
                      int rank, const int* __restrict__ status) {
    // a barrier that gave up (or any other bounded wait of this step) has recorded a status word: the peers'
    // buffers may be stale or half written, so nothing is moved and the step's result stays visibly unfinished
    if (status != nullptr && *reinterpret_cast<const volatile int*>(status) != 0) return;
    const long long total = (long long)n0 * n1 * n2 * vec_per_row;
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
                const int i0 = ((int)(r1 / n1) + rank) % n0;
                uint8_t* remote = reinterpret_cast<uint8_t*>(srcs.p[i0]) + src_off + i1 * s1 + i2 * s2 +
                                  (long long)v * (long long)sizeof(V);
                const long long loff = i0 * t0 + i1 * t1 + i2 * t2 + (long long)v * (long long)sizeof(V);
                if (kPush) {
                    val[u] = *reinterpret_cast<const V*>(dst + loff);
                    doff[u] = reinterpret_cast<long long>(remote);
                } else {
                    val[u] = *reinterpret_cast<const V*>(remote);
                    doff[u] = loff;
                }
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (doff[u] < 0) continue;
            if (kPush)
                *reinterpret_cast<V*>(doff[u]) = val[u];
            else
                *reinterpret_cast<V*>(dst + doff[u]) = val[u];
        }
    }
}

}  // namespace

extern "C" {

int of3_peer_heap_alloc(size_t bytes, void** ptr, void* handle64) {
    OF3_REQUIRE(ptr && handle64 && bytes > 0, OF3_ERR_ARG, "peer_heap_alloc: bad argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    OF3_CUDA_CHECK(cudaMalloc(ptr, bytes));
    OF3_CUDA_CHECK(cudaMemset(*ptr, 0, bytes));
    OF3_CUDA_CHECK(cudaDeviceSynchronize());
    OF3_CUDA_CHECK(cudaIpcGetMemHandle(reinterpret_cast<cudaIpcMemHandle_t*>(handle64), *ptr));
    return OF3_OK;
}

int of3_peer_heap_open(const void* handle64, void** ptr) {
    OF3_REQUIRE(ptr && handle64, OF3_ERR_ARG, "peer_heap_open: bad argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    OF3_CUDA_CHECK(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return OF3_OK;
}

int of3_peer_heap_close(void* ptr) {
    OF3_REQUIRE(ptr, OF3_ERR_ARG, "peer_heap_close: null pointer");
    OF3_CUDA_CHECK(cudaIpcCloseMemHandle(ptr));
    return OF3_OK;
}

int of3_peer_heap_free(void* ptr) {
    OF3_REQUIRE(ptr, OF3_ERR_ARG, "peer_heap_free: null pointer");
    OF3_CUDA_CHECK(cudaFree(ptr));
    return OF3_OK;
}

static int peer_barrier(void* const* flag_blocks, int world, int rank, uint64_t limit_ns, void* stream) {
    OF3_REQUIRE(flag_blocks && world >= 1 && world <= kMaxPeers && rank >= 0 && rank < world, OF3_ERR_ARG,
                "peer_barrier: bad argument (world %d, rank %d)", world, rank);
    PeerPtrs f{};
    for (int r = 0; r < world; ++r) {
        OF3_REQUIRE(flag_blocks[r] && ((uintptr_t)flag_blocks[r] & 3) == 0, OF3_ERR_ARG, "peer_barrier: bad flag block");
        f.p[r] = flag_blocks[r];
    }
    LaunchScope scope(kKidBarrier, (cudaStream_t)stream);
    peer_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(f, world, rank, limit_ns, device_status_ptr());
    OF3_CUDA_CHECK(cudaGetLastError());
    return OF3_OK;
}

int of3_peer_barrier(void* const* flag_blocks, int world, int rank, void* stream) {
    return peer_barrier(flag_blocks, world, rank, kBarrierLimitNs, stream);
}

int of3_peer_barrier_step_entry(void* const* flag_blocks, int world, int rank, void* stream) {
    return peer_barrier(flag_blocks, world, rank, kStepEntryLimitNs, stream);
}

static int peer_rows(void* const* srcs, long long src_off, void* dst, int world, int rank, int n1, int n2,
                     long long s1, long long s2, long long t0, long long t1, long long t2, int row_bytes,
                     void* stream, bool push) {
    OF3_REQUIRE(srcs && dst && world >= 1 && world <= kMaxPeers && rank >= 0 && rank < world, OF3_ERR_ARG,
                "peer_pull_rows: bad argument (world %d, rank %d)", world, rank);
    OF3_REQUIRE(n1 > 0 && n2 > 0 && row_bytes > 0 && row_bytes % 2 == 0 && src_off >= 0, OF3_ERR_ARG,
                "peer_pull_rows: bad sizes");
    PeerPtrs s{};
    uintptr_t all = (uintptr_t)dst | (uintptr_t)src_off | (uintptr_t)s1 | (uintptr_t)s2 | (uintptr_t)t0 |
                    (uintptr_t)t1 | (uintptr_t)t2 | (uintptr_t)row_bytes;
    for (int r = 0; r < world; ++r) {
        OF3_REQUIRE(srcs[r], OF3_ERR_ARG, "peer_pull_rows: null source %d", r);
        s.p[r] = srcs[r];
        all |= (uintptr_t)srcs[r];
    }
    const bool vec = (all & 15) == 0;
    const int vpr = vec ? row_bytes / 16 : row_bytes / 2;
    const long long total = (long long)world * n1 * n2 * vpr;
    long long blocks = (total + 4 * 256 - 1) / (4 * 256);
    const long long cap = (long long)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    LaunchScope scope(31, (cudaStream_t)stream);
    cudaStream_t st = (cudaStream_t)stream;
    uint8_t* d = (uint8_t*)dst;
    const int* status = device_status_ptr();
    if (vec && push)
        peer_pull_rows_kernel<uint4, true><<<(unsigned)blocks, 256, 0, st>>>(s, src_off, d, world, n1, n2, s1, s2, t0, t1,
                                                                             t2, vpr, rank, status);
    else if (vec)
        peer_pull_rows_kernel<uint4, false><<<(unsigned)blocks, 256, 0, st>>>(s, src_off, d, world, n1, n2, s1, s2, t0,
                                                                              t1, t2, vpr, rank, status);
    else if (push)
        peer_pull_rows_kernel<uint16_t, true><<<(unsigned)blocks, 256, 0, st>>>(s, src_off, d, world, n1, n2, s1, s2, t0,
                                                                                t1, t2, vpr, rank, status);
    else
        peer_pull_rows_kernel<uint16_t, false><<<(unsigned)blocks, 256, 0, st>>>(s, src_off, d, world, n1, n2, s1, s2,
                                                                                 t0, t1, t2, vpr, rank, status);
    OF3_CUDA_CHECK(cudaGetLastError());
    return OF3_OK;
}

int of3_peer_pull_rows(void* const* srcs, long long src_off, void* dst, int world, int rank, int n1, int n2,
                       long long s1, long long s2, long long t0, long long t1, long long t2, int row_bytes,
                       void* stream) {
    return peer_rows(srcs, src_off, dst, world, rank, n1, n2, s1, s2, t0, t1, t2, row_bytes, stream, false);
}

int of3_peer_push_rows(void* const* dsts, long long dst_off, const void* src, int world, int rank, int n1, int n2,
                       long long s1, long long s2, long long t0, long long t1, long long t2, int row_bytes,
                       void* stream) {
    return peer_rows(dsts, dst_off, const_cast<void*>(src), world, rank, n1, n2, s1, s2, t0, t1, t2, row_bytes, stream,
                     true);
}

}  // extern "C"
