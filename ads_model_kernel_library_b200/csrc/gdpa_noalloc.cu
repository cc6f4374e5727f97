// gdpa_fwd_noalloc: the GDPA forward for callers that cannot give the library a scratch buffer.
//
// The ordinary forward needs a work schedule in device memory that the caller allocates.  Some
// callers have no allocator to ask: a serving process that has handed every byte of device memory
// to its own arena, or host code that runs where a device allocation would stall or is forbidden.
// For them the schedule lives in a fixed array that is part of this library's device image.
//
//  - The array holds at most GDPA_NOALLOC_MAX_ITEMS work items (1 MiB + 16 bytes).  Every GPU that
//    loads the library carries it until the process exits.
//  - All calls on a device share the array, and it keeps what the last call wrote.  Nothing in it
//    has to start at zero: the schedule builder rewrites the header and every item it will use on
//    each call.  Two calls whose kernels overlap on the GPU (different streams, or different
//    threads) race on the array; callers must order them.
//  - The first call on a device looks up the array's device address (cudaGetSymbolAddress) and
//    sets the kernels' shared-memory attribute.  Make that first call outside any stream capture.
//    The address is cached for the life of the process: after cudaDeviceReset() on that device the
//    cached value is stale and this entry point must not be used again in the process.
//  - No cudaMalloc / cudaFree / allocating library routine is called, on any path.
#include <atomic>
#include <mutex>

#include "../../include/gdpa_b200.h"
#include "gdpa_common.cuh"
#include "gdpa_launch.h"

namespace gdpa {
namespace {

constexpr long long kNoallocMaxItems = GDPA_NOALLOC_MAX_ITEMS;

// In host code this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) int g_noalloc_schedule[kSchedHeaderInts + 4 * kNoallocMaxItems];

constexpr int kMaxDev = 64;
std::mutex g_setup_mutex;
int* g_sched_ptr[kMaxDev];  // device address of g_noalloc_schedule on each device, 0 until set up

// Once per device, with that device current: resolve the array's device address.
int noalloc_schedule_ptr(int** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return GDPA_ERR_DEVICE;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_sched_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_noalloc_schedule) != cudaSuccess || ptr == nullptr) {
      (void)cudaGetLastError();
      return GDPA_ERR_DEVICE;
    }
    g_sched_ptr[dev] = static_cast<int*>(ptr);
  }
  *out = g_sched_ptr[dev];
  return GDPA_OK;
}

}  // namespace
}  // namespace gdpa

using namespace gdpa;

#pragma GCC visibility push(default)
extern "C" int gdpa_fwd_noalloc(const GdpaFwdParams* p, gdpa_stream_t stream) {
  // The same host-side checks as gdpa_fwd, first: a call that gdpa_fwd would refuse must not have touched the
  // shared array (nor launched anything) by the time it is refused.
  int rc = fwd_check_params(p, false, false);
  if (rc != GDPA_OK) return rc;
  if (p->total_q == 0 || p->batch == 0) return GDPA_OK;
  // Upper bound on the number of work items, the same arithmetic gdpa_schedule_bytes() uses.
  const long long need = static_cast<long long>(p->heads) * (p->total_q / kFwdQBlock + p->batch);
  if (need > kNoallocMaxItems) return GDPA_ERR_NOALLOC_TOO_LARGE;
  int* sched = nullptr;
  rc = noalloc_schedule_ptr(&sched);
  if (rc != GDPA_OK) return rc;

  GdpaSchedParams sp;
  sp.struct_size = sizeof(sp);
  sp.mode = GDPA_SCHED_FWD;
  sp.q_offsets = p->q_offsets;
  sp.kv_offsets = p->kv_offsets;
  sp.offsets_are_int64 = p->offsets_are_int64;
  sp.batch = p->batch;
  sp.heads = p->heads;
  sp.max_seq_len_q = p->max_seq_len_q;
  sp.max_seq_len_kv = p->max_seq_len_kv;
  sp.kv_batch = p->kv_batch;
  sp.schedule = sched;
  sp.schedule_bytes = static_cast<int64_t>(sizeof(int)) * (kSchedHeaderInts + 4 * kNoallocMaxItems);
  sp.kv_seq_index = p->kv_seq_index;
  rc = gdpa_build_schedule(&sp, stream);
  if (rc != GDPA_OK) return rc;
  GdpaFwdParams fp = *p;
  fp.schedule = sched;
  return gdpa_fwd(&fp, stream);
}
#pragma GCC visibility pop
