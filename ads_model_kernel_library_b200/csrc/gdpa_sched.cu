// Device-side builder of the longest-first work list walked by the persistent GDPA kernels.
//
// Forward items are (sequence, head, 256-row Q block) weighted by the number of KV tiles of the
// sequence; backward items are (sequence, head, 128-row KV tile) weighted by the number of Q tiles.
// The list is a counting sort by weight, heaviest first, built by one thread block without any
// host synchronisation.  Buffer layout: int32 header {count, mode, 0, 0}, then one int4
// {sequence, head, block, weight} per item.
#include "gdpa_common.cuh"
#include "gdpa_launch.h"

namespace gdpa {

namespace {

constexpr int kSchedThreads = 1024;
constexpr int kBins = 4096;

__device__ __forceinline__ void seq_geometry(const SchedArgs& a, int b, int& nblk, int& weight) {
  long long s0, e0;
  seq_bounds(a.q_off, b, a.off64, s0, e0);
  long long lq = e0 - s0;
  int kb = b;
  if (a.kv_index != nullptr) {  // an entry beyond the KV batch is clamped, as the kernels do
    kb = static_cast<int>(load_offset(a.kv_index, b, a.off64));
    kb = kb < 0 ? 0 : (kb >= a.kv_batch ? a.kv_batch - 1 : kb);
  }
  seq_bounds(a.kv_off, kb, a.off64, s0, e0);
  long long lkv = e0 - s0;
  lq = lq < 0 ? 0 : (lq < a.max_q ? lq : a.max_q);
  lkv = lkv < 0 ? 0 : (lkv < a.max_kv ? lkv : a.max_kv);
  const int nq = static_cast<int>((lq + kTile - 1) / kTile);
  const int nkv = static_cast<int>((lkv + kTile - 1) / kTile);
  if (a.mode == 0) {
    nblk = static_cast<int>((lq + kFwdQBlock - 1) / kFwdQBlock);
    weight = nkv;
  } else {
    nblk = nkv;
    weight = nq;
  }
  if (weight > kBins - 1) weight = kBins - 1;
}

__global__ void __launch_bounds__(kSchedThreads, 1) gdpa_build_schedule_kernel(const SchedArgs a) {
  __shared__ int hist[kBins];
  __shared__ int total;
  for (int i = threadIdx.x; i < kBins; i += kSchedThreads) hist[i] = 0;
  __syncthreads();
  for (int b = threadIdx.x; b < a.batch; b += kSchedThreads) {
    int nblk, w;
    seq_geometry(a, b, nblk, w);
    if (nblk > 0) atomicAdd(&hist[w], nblk * a.heads);
  }
  __syncthreads();
  // Exclusive prefix over bins from the heaviest down: hist[w] becomes the first slot of weight w.
  if (threadIdx.x < 32) {
    // Each lane owns a contiguous run of bins (heaviest first); lane totals are scanned by shuffles.
    constexpr int per = kBins / 32;
    const int hi = kBins - 1 - threadIdx.x * per;  // this lane walks hi, hi-1, ..., hi-per+1
    int sum = 0;
    for (int i = 0; i < per; ++i) sum += hist[hi - i];
    int incl = sum;
    for (int d = 1; d < 32; d <<= 1) {
      int n = __shfl_up_sync(0xffffffffu, incl, d);
      if (threadIdx.x >= d) incl += n;
    }
    int run = incl - sum;
    for (int i = 0; i < per; ++i) {
      const int c = hist[hi - i];
      hist[hi - i] = run;
      run += c;
    }
    if (threadIdx.x == 31) total = incl;
  }
  __syncthreads();
  const long long cap = a.capacity_items;
  int4* items = reinterpret_cast<int4*>(a.sched + kSchedHeaderInts);
  for (int b = threadIdx.x; b < a.batch; b += kSchedThreads) {
    int nblk, w;
    seq_geometry(a, b, nblk, w);
    if (nblk == 0) continue;
    const int base = atomicAdd(&hist[w], nblk * a.heads);
    for (int h = 0; h < a.heads; ++h)
      for (int blk = 0; blk < nblk; ++blk) {
        const long long slot = static_cast<long long>(base) + h * nblk + blk;
        if (slot < cap) items[slot] = make_int4(b, h, blk, w);
      }
  }
  if (threadIdx.x == 0) {
    a.sched[0] = static_cast<int>(total < cap ? total : cap);
    a.sched[1] = a.mode;
    a.sched[2] = total;  // items the batch needs; larger than [0] only if the buffer was too small
    a.sched[3] = 0;
  }
}

}  // namespace

int launch_build_schedule(const SchedArgs& a, cudaStream_t stream) {
  gdpa_build_schedule_kernel<<<1, kSchedThreads, 0, stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : GDPA_ERR_LAUNCH_;
}

}  // namespace gdpa
