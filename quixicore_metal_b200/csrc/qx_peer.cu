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

}  // namespace

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
