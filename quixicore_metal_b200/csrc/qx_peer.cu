// Exchange of the per-shard LM-head candidates between GPUs by plain peer stores over NVLink,
// in place of an all-gather: every rank copies its slot of the gather buffer into the same slot of
// every peer's buffer (symmetric allocation), then publishes a step number in a flag word on every
// peer; the merge stage of a rank starts once the flags of all peers carry the current step.
//
//   push:  grid of copy CTAs; 16-byte loads from the local slot, one 16-byte store per peer.  Every
//          CTA fences its stores system-wide and takes a ticket; the CTA that takes the last ticket
//          fences again and writes the step number to flag[self] on every peer.
//   wait:  one warp, lane r polls flag[r] (acquire, system scope) until it is at least the step
//          number.  The wait is bounded: when it runs out the kernel writes 1 to *status and returns,
//          so a missing peer costs the call its result but never hangs the GPU; later waits on the
//          same status word return at once.
//
// Buffers alternate between two halves by step parity: a peer may already push step n + 1 while this
// rank still merges step n, but never step n + 2 (its merge of n + 1 needs this rank's push of n + 1,
// which is enqueued behind this rank's merge of n).  No multicast / multimem is used.
#include "qx_common.cuh"
#include "qx_kernels.h"

namespace qx {

namespace {

constexpr int PEER_MAX = 16;
struct PeerPtrs { void* p[PEER_MAX]; };

__global__ void __launch_bounds__(256)
peer_push_kernel(const uint4* __restrict__ src, PeerPtrs dst, PeerPtrs flags, size_t n16, int world, int self,
                 int step, unsigned* __restrict__ tickets) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (size_t)gridDim.x * blockDim.x) {
    const uint4 v = src[i];
    for (int r = 0; r < world; ++r)
      if (r != self) reinterpret_cast<uint4*>(dst.p[r])[i] = v;
  }
  __threadfence_system();                       // this thread's peer stores before the ticket
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned t = atomicAdd(tickets, 1u);
    if (t == gridDim.x - 1) {                   // every CTA has fenced its stores
      *tickets = 0u;                            // ready for the next launch (stream order)
      __threadfence_system();
      for (int r = 0; r < world; ++r)
        if (r != self) {
          volatile int* f = reinterpret_cast<volatile int*>(flags.p[r]) + self;
          *f = step;
        }
      __threadfence_system();
    }
  }
}

__global__ void __launch_bounds__(32)
peer_wait_kernel(const int* __restrict__ flags, int world, int self, int step, int max_polls, int* __restrict__ status) {
  const int r = threadIdx.x;
  bool ok = true;
  if (*reinterpret_cast<volatile int*>(status) != 0) return;   // an earlier wait already ran out: do not wait again
  if (r < world && r != self) {
    const volatile int* f = flags + r;
    ok = false;
    for (int i = 0; i < max_polls; ++i) {
      if (*f - step >= 0) { ok = true; break; }      // wrap-safe "at least this step"
      __nanosleep(200);
    }
  }
  __threadfence_system();                              // acquire: the peers' data stores precede their flags
  if (!__all_sync(0xffffffffu, ok) && threadIdx.x == 0) *status = 1;
}

// ---- all-reduce of fp32 partial sums with the residual add fused into the consumer ----------------------
// Symmetric buffer per rank: two halves (step parity) of `world` slots of slot_floats floats.  The
// step number lives in device memory (*counter, one word per rank, advanced by the push kernel), so
// the same launches can be replayed from a CUDA graph: nothing step-dependent is a kernel argument.
//   push:   s = *counter + 1; the rank's partial goes into slot [s & 1][self] of EVERY rank's buffer
//           (its own included); the CTA with the last ticket publishes s in flag[self] on every rank
//           and stores s to *counter.
//   finish: s = *counter; every CTA waits (bounded) until all flags carry s, then
//           out[i] = T(sum over ranks r = 0..world-1 of slot[s & 1][r][i] + residual[i]): the same
//           order on every rank, so all ranks hold bit-identical results.
__global__ void __launch_bounds__(256)
peer_sum_push_kernel(const float4* __restrict__ src, PeerPtrs bufs, PeerPtrs flags, size_t n4, size_t slot_floats,
                     int world, int self, int* __restrict__ counter, unsigned* __restrict__ tickets) {
  const int s = *reinterpret_cast<volatile int*>(counter) + 1;
  const size_t slot = ((size_t)(s & 1) * world + self) * slot_floats / 4;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
    const float4 v = src[i];
    for (int r = 0; r < world; ++r) reinterpret_cast<float4*>(bufs.p[r])[slot + i] = v;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned t = atomicAdd(tickets, 1u);
    if (t == gridDim.x - 1) {
      *tickets = 0u;
      __threadfence_system();
      for (int r = 0; r < world; ++r) {
        volatile int* f = reinterpret_cast<volatile int*>(flags.p[r]) + self;
        *f = s;
      }
      *reinterpret_cast<volatile int*>(counter) = s;
      __threadfence_system();
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
peer_sum_finish_kernel(const float* __restrict__ buf, const int* __restrict__ flags, const int* __restrict__ counter,
                       const T* __restrict__ residual, T* __restrict__ out, size_t n, size_t slot_floats, int world,
                       int max_polls, int* __restrict__ status) {
  __shared__ int timed_out;
  const int s = *reinterpret_cast<const volatile int*>(counter);
  if (threadIdx.x == 0) timed_out = 0;
  __syncthreads();
  if (threadIdx.x < world && *reinterpret_cast<volatile int*>(status) == 0) {
    const volatile int* f = flags + threadIdx.x;
    bool ok = false;
    for (int i = 0; i < max_polls; ++i) {
      if (*f - s >= 0) { ok = true; break; }
      __nanosleep(100);
    }
    if (!ok) timed_out = 1;
  }
  __threadfence_system();
  __syncthreads();
  if (timed_out && threadIdx.x == 0) *status = 1;      // the sums below are then not valid; nothing hangs
  const float* half = buf + (size_t)(s & 1) * world * slot_floats;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float acc = 0.f;
    for (int r = 0; r < world; ++r) acc += half[(size_t)r * slot_floats + i];
    out[i] = from_f32<T>(acc + to_f32<T>(residual[i]));
  }
}

}  // namespace

bool launch_peer_sum_push(cudaStream_t st, const float* src, size_t n, void* const* peer_bufs, void* const* peer_flags,
                          int world, int self, int* counter, unsigned* tickets) {
  if (world < 1 || world > PEER_MAX || n % 4 != 0 || ((uintptr_t)src & 15) != 0) return false;
  PeerPtrs b{}, f{};
  for (int r = 0; r < world; ++r) {
    b.p[r] = peer_bufs[r]; f.p[r] = peer_flags[r];
    if (((uintptr_t)peer_bufs[r] & 15) != 0 || !peer_flags[r]) return false;
  }
  int blocks = (int)((n / 4 + 255) / 256);
  if (blocks > sm_count()) blocks = sm_count();
  if (blocks < 1) blocks = 1;
  peer_sum_push_kernel<<<blocks, 256, 0, st>>>((const float4*)src, b, f, n / 4, n, world, self, counter, tickets);
  note_launch();
  return true;
}

void launch_peer_sum_finish(cudaStream_t st, const float* buf, const int* flags, const int* counter, const void* residual,
                            void* out, size_t n, int world, qx_dtype dtype, int max_polls, int* status) {
  int blocks = (int)((n + 255) / 256);
  if (blocks > sm_count()) blocks = sm_count();
  if (blocks < 1) blocks = 1;
  if (dtype == QX_DTYPE_F32)
    peer_sum_finish_kernel<float><<<blocks, 256, 0, st>>>(buf, flags, counter, (const float*)residual, (float*)out, n, n, world, max_polls, status);
  else if (dtype == QX_DTYPE_F16)
    peer_sum_finish_kernel<__half><<<blocks, 256, 0, st>>>(buf, flags, counter, (const __half*)residual, (__half*)out, n, n, world, max_polls, status);
  else
    peer_sum_finish_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(buf, flags, counter, (const __nv_bfloat16*)residual, (__nv_bfloat16*)out, n, n, world, max_polls, status);
  note_launch();
}

bool launch_peer_push(cudaStream_t st, const void* src, size_t bytes, void* const* peer_dst, void* const* peer_flags,
                      int world, int self, int step, unsigned* tickets) {
  if (world < 1 || world > PEER_MAX || bytes % 16 != 0 || ((uintptr_t)src & 15) != 0) return false;
  PeerPtrs d{}, f{};
  for (int r = 0; r < world; ++r) {
    d.p[r] = peer_dst[r]; f.p[r] = peer_flags[r];
    if (r != self && (((uintptr_t)peer_dst[r] & 15) != 0 || !peer_flags[r])) return false;
  }
  const size_t n16 = bytes / 16;
  int blocks = (int)((n16 + 255) / 256);
  if (blocks > 2 * sm_count()) blocks = 2 * sm_count();
  if (blocks < 1) blocks = 1;
  peer_push_kernel<<<blocks, 256, 0, st>>>((const uint4*)src, d, f, n16, world, self, step, tickets);
  note_launch();
  return true;
}

void launch_peer_wait(cudaStream_t st, const int* flags, int world, int self, int step, int max_polls, int* status) {
  peer_wait_kernel<<<1, 32, 0, st>>>(flags, world, self, step, max_polls, status);
  note_launch();
}

}  // namespace qx
