// Placeholders for tcgen05 module kernels that are not written yet: report "unsupported" so
// the entry points select the shape-generic kernels.
#include "modules.cuh"
namespace of3 {
namespace fast {
bool triattn_supported(int, int, int) { return false; }
int triattn(const __nv_bfloat16*, const __nv_bfloat16*, __nv_bfloat16*, int, int, float, int,
            const of3_triattn_params*, Arena&, cudaStream_t) { return OF3_ERR_SHAPE; }
}  // namespace fast
}  // namespace of3
