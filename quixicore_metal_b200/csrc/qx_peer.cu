// Exchanges between GPUs by plain peer stores over NVLink into symmetric allocations, in place of the
// collectives of a decode step: the all-gather of the per-shard LM-head candidates and the all-reduce of
// the row-parallel projections' fp32 partials.  No multicast / multimem is used.  Two forms:
//
//   flag-in-data (peer_gather_kernel, peer_allreduce_kernel; small messages): every 16-byte store carries
//          two floats and, beside each, the step number; the receiver polls the data words themselves.
//          One launch, one NVLink crossing, no fence and no separate flag.  Described at the kernels.
//   push + wait (peer_push_kernel, peer_wait_kernel; large slots, where doubling the bytes costs more
//          than a fence): every rank copies its slot of the gather buffer into the same slot of every
//          peer's buffer, then publishes the step number in a flag word on every peer; the merge stage
//          of a rank starts once the flags of all peers carry the current step.
//          push:  grid of copy CTAs; 16-byte loads from the local slot, one 16-byte store per peer.  Every
//                 CTA fences its stores system-wide and takes a ticket; the CTA that takes the last
//                 ticket fences again and writes the step number to flag[self] on every peer.
//          wait:  one warp, lane r polls flag[r] (acquire, system scope) until it is at least the step.
//
// Every wait is bounded: when it runs out the kernel writes 1 to *status and carries on, so a missing peer
// costs the call its result but never hangs the GPU; later waits on the same status word return at once.
// Buffers alternate between two halves by step parity: a peer may already send step n + 1 while this
// rank still consumes step n, but never step n + 2 (that needs this rank's data of step n + 1, which is
// enqueued behind this rank's consumer of n).  All kernels are programmatic dependent launches: they may
// be scheduled while the producer of their input still runs and touch nothing before
// griddepcontrol.wait; each lets its own dependent be scheduled as soon as it has started.
#include "qx_common.cuh"
#include "qx_kernels.h"

namespace qx {

namespace {

constexpr int PEER_MAX = 16;
struct PeerPtrs { void* p[PEER_MAX]; };

__global__ void __launch_bounds__(256)
peer_push_kernel(const uint4* __restrict__ src, PeerPtrs dst, PeerPtrs flags, size_t n16, int world, int self,
                 int step, unsigned* __restrict__ tickets) {
  asm volatile("griddepcontrol.wait;" ::: "memory");     // launched as a programmatic dependent of the producer of src
  asm volatile("griddepcontrol.launch_dependents;");
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
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;");
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

// ---- all-reduce of fp32 partial sums with the residual add and the cast fused, ONE launch, flag-in-data ----
// Latency form for decode-sized partials (row-parallel projections): every 16-byte store carries two floats and, beside each, the step
// number {x, s, y, s}; the receiver polls the data words themselves until both step fields match, so there
// is no separate flag, no fence and no barrier between the store and its use - one NVLink crossing per
// all-reduce.  8-byte halves are single-copy atomic, and each half carries its own step field.
// Every rank owns a buffer of two halves (step parity) of `world` slots of n / 2 such 16-byte words; a
// slot's stale content is from step s - 2, never s.  A thread stores its elements of the rank's partial into
// slot [s & 1][self] of every rank (its own included), then reads slot [s & 1][r] of its own buffer for
// r = 0 .. world - 1 in order (bounded polls; on expiry *status = 1, the thread stops waiting and the result
// is not valid), adds the residual and casts.  A thread waits only for stores of the same element by the
// other GPUs and has stored before it waits: no CTA depends on another CTA of its grid.  The last CTA of the
// grid stores s to *counter (device-side step: the launch can be replayed from a CUDA graph).  blockIdx.y
// selects the rank when several ranks whose buffers live on ONE GPU run as one cooperative launch
// (separate launches that wait for one another on one GPU are not guaranteed to overlap).
struct PeerSumRank {
  const float2* src; const void* residual; void* out; int* counter; unsigned* tickets; int* status;
};
struct PeerSumRanks { PeerSumRank r[PEER_MAX]; };

__device__ __forceinline__ void st_volatile_v4(uint4* p, uint4 v) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 ld_volatile_v4(const uint4* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

template <typename T>
__global__ void __launch_bounds__(256)
peer_allreduce_kernel(const PeerSumRanks ranks, const PeerPtrs bufs, size_t n2, int world, int self0, int max_polls) {
  // Programmatic dependent launch on both sides: this grid may be scheduled while the projection before it
  // still runs (nothing is read or written before that kernel has completed), and the projection after it
  // may be scheduled and fetch its first weights while this grid waits for the peers.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;");
  const PeerSumRank me = ranks.r[blockIdx.y];
  const int self = self0 + (int)blockIdx.y;
  const int s = *reinterpret_cast<volatile int*>(me.counter) + 1;
  const bool may_wait = *reinterpret_cast<volatile int*>(me.status) == 0;   // an earlier wait ran out: do not wait again
  const size_t half = (size_t)(s & 1) * world * n2;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t j0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (size_t j = j0; j < n2; j += stride) {
    const float2 v = me.src[j];
    const uint4 w = make_uint4(__float_as_uint(v.x), (uint32_t)s, __float_as_uint(v.y), (uint32_t)s);
    for (int r = 0; r < world; ++r) st_volatile_v4(reinterpret_cast<uint4*>(bufs.p[r]) + half + (size_t)self * n2 + j, w);
  }
  const uint4* in = reinterpret_cast<const uint4*>(bufs.p[self]) + half;
  const T* res = reinterpret_cast<const T*>(me.residual);
  T* out = reinterpret_cast<T*>(me.out);
  bool dead = !may_wait;
  for (size_t j = j0; j < n2; j += stride) {
    float ax = 0.f, ay = 0.f;
    for (int r = 0; r < world; ++r) {
      const uint4* p = in + (size_t)r * n2 + j;
      uint4 w = ld_volatile_v4(p);
      if (!dead) {
        int polls = 0;
        while (w.y != (uint32_t)s || w.w != (uint32_t)s) {
          if (++polls > max_polls) { dead = true; break; }
          w = ld_volatile_v4(p);
        }
      }
      ax += __uint_as_float(w.x);
      ay += __uint_as_float(w.z);
    }
    out[2 * j] = from_f32<T>(ax + to_f32<T>(res[2 * j]));
    out[2 * j + 1] = from_f32<T>(ay + to_f32<T>(res[2 * j + 1]));
  }
  if (dead && may_wait) *me.status = 1;                    // nothing hangs; the sums are not valid
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned t = atomicAdd(me.tickets, 1u);
    if (t == gridDim.x - 1) {                              // every CTA of this rank has read *counter
      *me.tickets = 0u;
      *reinterpret_cast<volatile int*>(me.counter) = s;
    }
  }
}


// ---- all-gather of small slots, ONE launch, flag-in-data ---------------------------------------------------
// The latency form of push + wait for candidate slots of a few KB (argmax / top-k candidates, top-p pools of
// a single row): same 16-byte words {x, step, y, step} as the all-reduce above.  A thread sends its pair of
// floats of the local slot [self] of `gather` to the word buffer of every peer, then polls its own word
// buffer for the same pair of every peer (bounded; on expiry *status = 1 and the thread stops waiting) and
// writes it into slot [r] of `gather`, which the merge stage reads as plain floats.  Word buffer of a rank:
// two halves (step parity) of `world` slots of n2 words.  blockIdx.y = rank when all ranks live on one GPU
// and run as one cooperative launch.
struct PeerGatherRank { float2* gather; int* status; };
struct PeerGatherRanks { PeerGatherRank r[PEER_MAX]; };

__global__ void __launch_bounds__(256)
peer_gather_kernel(const PeerGatherRanks ranks, const PeerPtrs words, size_t n2, int world, int self0, int step,
                   int max_polls) {
  asm volatile("griddepcontrol.wait;" ::: "memory");     // launched as a programmatic dependent of the producer of the slot
  asm volatile("griddepcontrol.launch_dependents;");
  const PeerGatherRank me = ranks.r[blockIdx.y];
  const int self = self0 + (int)blockIdx.y;
  const bool may_wait = *reinterpret_cast<volatile int*>(me.status) == 0;
  const size_t half = (size_t)(step & 1) * world * n2;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t j0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (size_t j = j0; j < n2; j += stride) {
    const float2 v = me.gather[(size_t)self * n2 + j];
    const uint4 w = make_uint4(__float_as_uint(v.x), (uint32_t)step, __float_as_uint(v.y), (uint32_t)step);
    for (int r = 0; r < world; ++r)
      if (r != self) st_volatile_v4(reinterpret_cast<uint4*>(words.p[r]) + half + (size_t)self * n2 + j, w);
  }
  const uint4* in = reinterpret_cast<const uint4*>(words.p[self]) + half;
  bool dead = !may_wait;
  for (size_t j = j0; j < n2; j += stride) {
    for (int r = 0; r < world; ++r) {
      if (r == self) continue;
      const uint4* p = in + (size_t)r * n2 + j;
      uint4 w = ld_volatile_v4(p);
      if (!dead) {
        int polls = 0;
        while (w.y != (uint32_t)step || w.w != (uint32_t)step) {
          if (++polls > max_polls) { dead = true; break; }
          w = ld_volatile_v4(p);
        }
      }
      me.gather[(size_t)r * n2 + j] = make_float2(__uint_as_float(w.x), __uint_as_float(w.z));
    }
  }
  if (dead && may_wait) *me.status = 1;
}

}  // namespace

// Launch as a programmatic dependent of the kernel before it on the stream (plain launch if refused).
static cudaError_t launch_dependent(const void* fn, dim3 grid, dim3 block, void** args, cudaStream_t st) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelExC(&cfg, fn, args);
  if (e != cudaSuccess) { cudaGetLastError(); e = cudaLaunchKernel(fn, grid, block, args, 0, st); }
  return e;
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
  const uint4* src16 = (const uint4*)src;
  size_t n16v = n16;
  void* args[] = {&src16, &d, &f, &n16v, &world, &self, &step, &tickets};
  if (launch_dependent((const void*)peer_push_kernel, dim3((unsigned)blocks), dim3(256), args, st) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  note_launch();
  return true;
}

void launch_peer_wait(cudaStream_t st, const int* flags, int world, int self, int step, int max_polls, int* status) {
  void* args[] = {&flags, &world, &self, &step, &max_polls, &status};
  if (launch_dependent((const void*)peer_wait_kernel, dim3(1), dim3(32), args, st) != cudaSuccess) cudaGetLastError();
  note_launch();
}

}  // namespace qx

namespace qx {

// local_ranks == 1: this process is rank `self`.  local_ranks == world: all ranks live on this GPU and
// run as one cooperative launch (rank = blockIdx.y); src / residual / out / counter / tickets / status
// are then arrays of `world` pointers, else arrays of one.
bool launch_peer_allreduce(cudaStream_t st, const float* const* src, const void* const* residual, void* const* out,
                           size_t n, void* const* peer_bufs, int world, int self, int local_ranks,
                           int* const* counter, unsigned* const* tickets, int* const* status, qx_dtype dtype,
                           int max_polls) {
  if (world < 1 || world > PEER_MAX || n % 2 != 0 || n == 0) return false;
  if (local_ranks != 1 && local_ranks != world) return false;
  PeerSumRanks ranks{};
  PeerPtrs b{};
  for (int r = 0; r < world; ++r) {
    b.p[r] = peer_bufs[r];
    if (!peer_bufs[r] || ((uintptr_t)peer_bufs[r] & 15) != 0) return false;
  }
  for (int r = 0; r < local_ranks; ++r) {
    if (!src[r] || !residual[r] || !out[r] || !counter[r] || !tickets[r] || !status[r]) return false;
    if (((uintptr_t)src[r] & 7) != 0) return false;
    ranks.r[r] = PeerSumRank{(const float2*)src[r], residual[r], out[r], counter[r], tickets[r], status[r]};
  }
  size_t n2 = n / 2;
  int chunks = (int)((n2 + 255) / 256);
  if (chunks > sm_count()) chunks = sm_count();
  if (local_ranks > 1 && chunks * local_ranks > sm_count()) chunks = sm_count() / local_ranks;
  if (chunks < 1) chunks = 1;
  int self0 = local_ranks > 1 ? 0 : self;
  dim3 grid((unsigned)chunks, (unsigned)local_ranks);
  void* args[] = {&ranks, &b, &n2, &world, &self0, &max_polls};
  const void* fn = dtype == QX_DTYPE_F32 ? (const void*)peer_allreduce_kernel<float>
                   : dtype == QX_DTYPE_F16 ? (const void*)peer_allreduce_kernel<__half>
                                           : (const void*)peer_allreduce_kernel<__nv_bfloat16>;
  cudaError_t e;
  if (local_ranks > 1) {
    e = cudaLaunchCooperativeKernel(fn, grid, dim3(256), args, 0, st);
  } else {
    e = launch_dependent(fn, grid, dim3(256), args, st);
  }
  if (e != cudaSuccess) { cudaGetLastError(); return false; }
  note_launch();
  return true;
}

}  // namespace qx

namespace qx {

// local_ranks == 1: this process is rank `self`; local_ranks == world: all ranks on this GPU, one
// cooperative launch, gather / status arrays of `world` pointers.
bool launch_peer_gather(cudaStream_t st, float* const* gather, size_t slot_floats, void* const* peer_words, int world,
                        int self, int local_ranks, int step, int* const* status, int max_polls) {
  if (world < 1 || world > PEER_MAX || slot_floats % 2 != 0 || slot_floats == 0) return false;
  if (local_ranks != 1 && local_ranks != world) return false;
  PeerGatherRanks ranks{};
  PeerPtrs w{};
  for (int r = 0; r < world; ++r) {
    w.p[r] = peer_words[r];
    if (!peer_words[r] || ((uintptr_t)peer_words[r] & 15) != 0) return false;
  }
  for (int r = 0; r < local_ranks; ++r) {
    if (!gather[r] || !status[r] || ((uintptr_t)gather[r] & 7) != 0) return false;
    ranks.r[r] = PeerGatherRank{(float2*)gather[r], status[r]};
  }
  size_t n2 = slot_floats / 2;
  int chunks = (int)((n2 + 255) / 256);
  if (chunks > sm_count()) chunks = sm_count();
  if (local_ranks > 1 && chunks * local_ranks > sm_count()) chunks = sm_count() / local_ranks;
  if (chunks < 1) chunks = 1;
  int self0 = local_ranks > 1 ? 0 : self;
  dim3 grid((unsigned)chunks, (unsigned)local_ranks);
  void* args[] = {&ranks, &w, &n2, &world, &self0, &step, &max_polls};
  cudaError_t e = local_ranks > 1 ? cudaLaunchCooperativeKernel((const void*)peer_gather_kernel, grid, dim3(256), args, 0, st)
                                  : launch_dependent((const void*)peer_gather_kernel, grid, dim3(256), args, st);
  if (e != cudaSuccess) { cudaGetLastError(); return false; }
  note_launch();
  return true;
}

}  // namespace qx
