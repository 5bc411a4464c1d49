// Kernel-family selection for the projection ops.
#include <cstdlib>

#include "qx_common.cuh"
#include "qx_kernels.h"

namespace qx {

void launch_projection(cudaStream_t st, const GemvArgs& a) {
  // QX_FORCE_GENERIC=1 keeps every call on the shape-generic kernel (A/B comparisons)
  static const bool force_generic = [] {
    const char* e = getenv("QX_FORCE_GENERIC");
    return e && e[0] == '1';
  }();
  if (!force_generic && stream_path_ok(a) && launch_gemv_stream(st, a)) return;
  launch_gemv_generic(st, a);
}

}  // namespace qx
