// Kernel-family selection for the projection ops.
#include "qx_common.cuh"
#include "qx_kernels.h"

namespace qx {

void launch_projection(cudaStream_t st, const GemvArgs& a) {
  launch_gemv_generic(st, a);
}

}  // namespace qx
