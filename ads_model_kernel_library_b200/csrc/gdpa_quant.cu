// Producer of the low-precision inputs of gdpa_fwd_fp8: a jagged [total, H, D] tensor (bf16 or fp32) is quantised
// to FP8 e4m3 with one fp32 scale per (sequence-local 128-token block, head), scale = max(amax / 448, 1e-12) over
// the block, value = e4m3(clamp(x / scale, -448, 448)) with round-to-nearest-even.  Block j of sequence b is row
// block_offsets[b] + j of the scale tensor, block_offsets being the exclusive prefix sum of ceil(len / 128), which
// the first kernel builds on the device (no host synchronisation).  HBM-bound byte work: one CTA of 128 threads
// per (block, head), a thread per token row.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "gdpa_common.cuh"
#include "gdpa_launch.h"

namespace gdpa {

namespace {

__global__ void gdpa_block_offsets_kernel(const void* offsets, void* block_offsets, int off64, int batch) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  long long run = 0;
  for (int b = 0; b <= batch; ++b) {
    if (off64) static_cast<long long*>(block_offsets)[b] = run;
    else static_cast<int*>(block_offsets)[b] = static_cast<int>(run);
    if (b < batch) {
      long long len = load_offset(offsets, b + 1, off64) - load_offset(offsets, b, off64);
      if (len < 0) len = 0;
      run += (len + kTile - 1) / kTile;
    }
  }
}

__device__ __forceinline__ float load_elem(const float* p, long long i) { return p[i]; }
__device__ __forceinline__ float load_elem(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }

template <typename T>
__global__ void __launch_bounds__(kTile) gdpa_quant_fp8_kernel(const QuantArgs a) {
  __shared__ float s_max[kTile / 32];
  __shared__ float s_scale;
  const long long g = blockIdx.x;  // block index over the batch
  const int h = blockIdx.y;
  if (g >= load_offset(a.block_offsets, a.batch, a.off64)) return;
  // the sequence that owns block g: last b with block_offsets[b] <= g
  int lo = 0, hi = a.batch;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (load_offset(a.block_offsets, mid, a.off64) <= g) lo = mid;
    else hi = mid;
  }
  const int b = lo;
  const long long seq_start = load_offset(a.offsets, b, a.off64), seq_end = load_offset(a.offsets, b + 1, a.off64);
  const long long row = seq_start + (g - load_offset(a.block_offsets, b, a.off64)) * kTile + threadIdx.x;
  const bool valid = row < seq_end;
  const T* x = static_cast<const T*>(a.x);
  const long long base = (row * a.heads + h) * static_cast<long long>(a.head_dim);
  float amax = 0.f;
  if (valid)
    for (int d = 0; d < a.head_dim; ++d) amax = fmaxf(amax, fabsf(load_elem(x, base + d)));
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, s));
  if ((threadIdx.x & 31) == 0) s_max[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = s_max[0];
    for (int i = 1; i < kTile / 32; ++i) m = fmaxf(m, s_max[i]);
    const float scale = fmaxf(m / 448.f, 1e-12f);
    s_scale = scale;
    a.scales[g * a.heads + h] = scale;
  }
  __syncthreads();
  if (!valid) return;
  const float scale = s_scale;
  uint32_t* out = reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(a.x8) + base);
  for (int d = 0; d < a.head_dim; d += 4) {
    float v[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) v[e] = fminf(fmaxf(load_elem(x, base + d + e) / scale, -448.f), 448.f);
    out[d >> 2] = pack_e4m3x4(v[0], v[1], v[2], v[3]);
  }
}

}  // namespace

int launch_quant_fp8(const QuantArgs& a, int in_is_fp32, cudaStream_t stream) {
  gdpa_block_offsets_kernel<<<1, 32, 0, stream>>>(a.offsets, a.block_offsets, a.off64, a.batch);
  if (cudaGetLastError() != cudaSuccess) return GDPA_ERR_LAUNCH_;
  if (a.max_blocks == 0) return 0;
  const dim3 grid(static_cast<unsigned>(a.max_blocks), static_cast<unsigned>(a.heads));
  if (in_is_fp32) gdpa_quant_fp8_kernel<float><<<grid, kTile, 0, stream>>>(a);
  else gdpa_quant_fp8_kernel<__nv_bfloat16><<<grid, kTile, 0, stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : GDPA_ERR_LAUNCH_;
}

}  // namespace gdpa
