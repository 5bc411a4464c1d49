// Kernel-family selection for the projection ops.
#include "qx_common.cuh"
#include "qx_kernels.h"

namespace qx {

size_t projection_scratch_bytes(const GemvArgs& a) {
  if (options().force_generic) return 0;
  const size_t s = stream_scratch_bytes(a);
  const size_t t = tc_scratch_bytes(a);
  return s > t ? s : t;
}

// Returns true when the kernel that ran also wrote the requested MXFP8 output rows; every other
// output quantisation is a second launch by the caller.
bool launch_projection(cudaStream_t st, const GemvArgs& a) {
  const bool fusable = a.out_quant == OQ_MXFP8 && !a.out_f32 && a.N % 32 == 0 && a.q_codes;
  if (!options().force_generic) {
    if (stream_path_ok(a) && launch_gemv_stream(st, a)) return fusable;
    if (stream_passes_ok(a) && launch_gemv_stream_passes(st, a)) return fusable;
    if (tc_path_ok(a)) {
      bool fused = false;
      if (launch_gemm_tc(st, a, &fused)) return fusable && fused;
    }
  }
  launch_gemv_generic(st, a);
  return false;
}

}  // namespace qx
