// Host-side services shared by the entry points: device scratch for calls that bring no workspace,
// the tensor-map cache, and the path options.
#include <atomic>
#include <cstring>
#include <mutex>
#include <vector>

#include "qx_common.cuh"
#include "qx_kernels.h"
#include "qx_tmap.h"

namespace qx {

// ---- path options -----------------------------------------------------------------------------
static Options g_options;
const Options& options() { return g_options; }
bool set_option(const char* name, int value) {
  if (!name) return false;
  if (std::strcmp(name, "stream_passes") == 0 && value >= 0 && value <= 2) { g_options.stream_passes = value; return true; }
  if (std::strcmp(name, "force_generic") == 0) { g_options.force_generic = value != 0; return true; }
  if (std::strcmp(name, "tc_pipeline") == 0) { g_options.tc_pipeline = value != 0; return true; }
  if (std::strcmp(name, "lm_head_ksplit") == 0) { g_options.lm_head_ksplit = value != 0; return true; }
  return false;
}

// ---- library-managed scratch ------------------------------------------------------------------
// Used only when the caller passes no workspace.  Calls on one stream are ordered, so a buffer tied
// to (device, stream) can serve every call on that stream.  Up to 16 (device, stream) pairs get
// such a buffer.  It grows by allocating a larger one; the smaller one stays allocated until the
// process exits (work already enqueued may still read it), so growth never synchronises or frees:
// the total is below twice the largest request.  cudaStreamPerThread (one handle, a different
// stream in every thread), streams that are being captured, and pairs beyond the 16th take a
// stream-ordered allocation per call instead (*must_free: release with cudaFreeAsync on `st`).
struct ScratchSlot { int dev; cudaStream_t st; void* ptr; size_t bytes; };
static ScratchSlot g_scratch[16] = {};
static std::mutex g_scratch_mu;
static std::atomic<uint64_t> g_scratch_allocs{0};

uint64_t scratch_alloc_count() { return g_scratch_allocs.load(std::memory_order_relaxed); }

void* default_scratch(cudaStream_t st, size_t bytes, bool* must_free) {
  *must_free = false;
  if (bytes == 0) bytes = 256;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return nullptr; }
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(st, &cap) != cudaSuccess) { cudaGetLastError(); cap = cudaStreamCaptureStatusNone; }
  if (cap == cudaStreamCaptureStatusNone && st != cudaStreamPerThread) {
    std::lock_guard<std::mutex> lock(g_scratch_mu);
    ScratchSlot* slot = nullptr;
    for (auto& s : g_scratch) {
      if (s.ptr && s.dev == dev && s.st == st) { slot = &s; break; }
      if (!s.ptr && !slot) slot = &s;
    }
    if (slot && slot->ptr && slot->bytes >= bytes) return slot->ptr;
    if (slot) {
      size_t want = bytes < (1u << 20) ? (1u << 20) : bytes;
      if (slot->ptr && want < 2 * slot->bytes) want = 2 * slot->bytes;
      void* p = nullptr;
      if (cudaMalloc(&p, want) == cudaSuccess) {
        g_scratch_allocs.fetch_add(1, std::memory_order_relaxed);
        *slot = ScratchSlot{dev, st, p, want};      // a smaller predecessor stays allocated on purpose
        return p;
      }
      cudaGetLastError();
    }
  }
  void* p = nullptr;
  if (cudaMallocAsync(&p, bytes, st) != cudaSuccess) { cudaGetLastError(); return nullptr; }
  g_scratch_allocs.fetch_add(1, std::memory_order_relaxed);
  *must_free = true;
  return p;
}

// ---- tensor-map cache ---------------------------------------------------------------------------
// Encoding a tensor map is a driver call of a few microseconds; a decode loop calls the same weights
// every step.  Maps are cached per (device, base pointer, rows, row bytes, box).  A weight freed
// and another allocated at the same address with the same geometry yields the same map, so stale
// entries are harmless; the table is a small direct-mapped cache, collisions simply re-encode.
struct MapEntry { int dev; const void* w; int64_t rows; size_t row_bytes; int box_bytes, box_rows; bool valid; CUtensorMap map; };
static MapEntry g_maps[256];
static std::mutex g_maps_mu;

bool cached_weight_map(CUtensorMap* map, const void* w, int64_t rows, size_t row_bytes, int box_bytes,
                       int box_rows) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return false; }
  uint64_t h = (uint64_t)(uintptr_t)w * 0x9E3779B97F4A7C15ull;
  h ^= (uint64_t)rows * 0xC2B2AE3D27D4EB4Full + (uint64_t)box_bytes * 31u + (uint64_t)box_rows * 131u + (uint64_t)dev * 7u;
  MapEntry& e = g_maps[(h >> 40) & 255u];
  {
    std::lock_guard<std::mutex> lock(g_maps_mu);
    if (e.valid && e.dev == dev && e.w == w && e.rows == rows && e.row_bytes == row_bytes &&
        e.box_bytes == box_bytes && e.box_rows == box_rows) {
      *map = e.map;
      return true;
    }
  }
  if (!make_weight_map(map, w, rows, row_bytes, box_bytes, box_rows)) return false;
  std::lock_guard<std::mutex> lock(g_maps_mu);
  e = MapEntry{dev, w, rows, row_bytes, box_bytes, box_rows, true, *map};
  return true;
}

}  // namespace qx
