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
  // QX_ENABLE_TC=0 keeps batch > 16 off the tcgen05 kernel
  static const bool tc_enabled = [] {
    const char* e = getenv("QX_ENABLE_TC");
    return !(e && e[0] == '0');
  }();
  if (!force_generic && stream_path_ok(a) && launch_gemv_stream(st, a)) return;
  if (!force_generic && stream_passes_ok(a) && launch_gemv_stream_passes(st, a)) return;
  if (!force_generic && tc_enabled && tc_path_ok(a) && launch_gemm_tc(st, a)) return;
  launch_gemv_generic(st, a);
}

}  // namespace qx
