// Producer of the low-precision inputs of gdpa_fwd_fp8: a jagged [total, H, D] tensor (bf16 or fp32) is quantised
// to FP8 e4m3 with one fp32 scale per (sequence-local 128-token block, head), scale = max(amax / 448, 1e-12) over
// the block, value = e4m3(clamp(x / scale, -448, 448)) with round-to-nearest-even.  Block j of sequence b is row
// block_offsets[b] + j of the scale tensor, block_offsets being the exclusive prefix sum of ceil(len / 128), which
// the first kernel builds on the device (no host synchronisation).  HBM-bound byte work: one CTA of 128 threads
// per (block, head), a thread per token row.
//
// Second format: MXFP8 (e4m3 elements, one e8m0 power-of-two scale per 32 elements along the contraction
// dimension), the wire format of the reference's block-scaled variant (gdpa/src/flash_fwd_sm100.py:746-833,
// gdpa/src/interface.py:714-750).  The element tensor keeps the jagged [total, H, D] shape; only the scale
// tensor is padded, every sequence to a multiple of 128 rows, and stored in 512-byte atoms of 128 rows x 4
// scales: byte 16 * (row % 32) + 4 * (row / 32) + k of an atom is the scale of row `row` and 32-element block k.
// With the scales along the head dim (Q, K) the rows are tokens and atoms are ordered [head][token block][ceil(D / 128)];
// with the scales along the tokens (V) the rows are head-dim indices and atoms are ordered
// [head][ceil(D / 128)][token block].  e8m0 follows the reference's round-up rule for its P tile
// (gdpa/src/activation_utils.py:444-517): t = amax * (1 / 448) in fp32, exponent field of t, plus one when the
// mantissa is not zero; elements are x * 2^(127 - e8m0) rounded to nearest even, saturating.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
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
__device__ __forceinline__ void store_elem(float* p, long long i, float v) { p[i] = v; }
__device__ __forceinline__ void store_elem(__nv_bfloat16* p, long long i, float v) { p[i] = __float2bfloat16_rn(v); }

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


// e8m0 code of a block with absolute maximum `amax`, and 2^(127 - code)
__device__ __forceinline__ uint32_t mx_e8m0_of(float amax, float& inv_scale) {
  const uint32_t bits = __float_as_uint(amax * (1.f / 448.f));
  uint32_t e = (bits >> 23) & 0xffu;
  if ((bits & 0x7fffffu) != 0u) ++e;
  e = min(e, 254u);  // 255 is the NaN code of e8m0
  inv_scale = e == 254u ? __uint_as_float(0x00400000u) /* 2^-127 */ : __uint_as_float((254u - e) << 23);
  return e;
}
// 2^(code - 127); code 0 is a denormal of fp32, which the shift cannot build
__device__ __forceinline__ float mx_scale_of(uint32_t e) { return e == 0u ? 5.877471754111438e-39f : __uint_as_float(e << 23); }

__device__ __forceinline__ float e4m3_to_float(uint8_t v) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(v, __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}

// the sequence that owns token block g (last b with block_offsets[b] <= g)
__device__ __forceinline__ int owner_of_block(const void* block_offsets, int off64, int batch, long long g) {
  int lo = 0, hi = batch;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (load_offset(block_offsets, mid, off64) <= g) lo = mid;
    else hi = mid;
  }
  return lo;
}

// One CTA of 128 threads per (128-token block, head).  AXIS 0: a thread per token row, scales along the head
// dim.  AXIS 1: a thread per head-dim index, scales along the tokens.  QUANT: x -> (x8, sf); else (x8, sf) -> x.
template <typename T, int AXIS, bool QUANT>
__global__ void __launch_bounds__(kTile) gdpa_mxfp8_kernel(const MxArgs a) {
  const long long g = blockIdx.x;
  const int h = blockIdx.y;
  if (g >= load_offset(a.block_offsets, a.batch, a.off64)) return;
  const int b = owner_of_block(a.block_offsets, a.off64, a.batch, g);
  const long long seq_end = load_offset(a.offsets, b + 1, a.off64);
  const long long row0 = load_offset(a.offsets, b, a.off64) + (g - load_offset(a.block_offsets, b, a.off64)) * kTile;
  const int t = threadIdx.x;
  const int d_atoms = (a.head_dim + 127) / 128;
  T* x = static_cast<T*>(a.x);
  uint8_t* x8 = static_cast<uint8_t*>(a.x8);
  const uint32_t atom_byte = 16u * (t & 31) + 4u * (t >> 5);
  if constexpr (AXIS == 0) {
    const long long row = row0 + t;
    const bool valid = row < seq_end;
    const long long base = (row * a.heads + h) * static_cast<long long>(a.head_dim);
    for (int da = 0; da < d_atoms; ++da) {
      uint32_t* sf_word = reinterpret_cast<uint32_t*>(a.sf + ((static_cast<long long>(h) * a.sf_blocks + g) * d_atoms + da) * 512 + atom_byte);
      uint32_t word = QUANT ? 0u : *sf_word;
      for (int k = 0; k < 4; ++k) {
        const int d0 = da * 128 + k * 32;
        if (d0 >= a.head_dim || !valid) continue;
        if constexpr (QUANT) {
          float v[32];
          float amax = 0.f;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            v[i] = load_elem(x, base + d0 + i);
            amax = fmaxf(amax, fabsf(v[i]));
          }
          float inv;
          word |= mx_e8m0_of(amax, inv) << (8 * k);
          uint32_t* out = reinterpret_cast<uint32_t*>(x8 + base + d0);
#pragma unroll
          for (int i = 0; i < 8; ++i) out[i] = pack_e4m3x4(v[4 * i] * inv, v[4 * i + 1] * inv, v[4 * i + 2] * inv, v[4 * i + 3] * inv);
        } else {
          const float sc = mx_scale_of((word >> (8 * k)) & 0xffu);
#pragma unroll
          for (int i = 0; i < 32; ++i) store_elem(x, base + d0 + i, e4m3_to_float(x8[base + d0 + i]) * sc);
        }
      }
      if constexpr (QUANT) *sf_word = word;  // rows past the sequence end carry zeros
    }
  } else {
    for (int da = 0; da < d_atoms; ++da) {
      const int d = da * 128 + t;
      const bool valid_d = d < a.head_dim;
      uint32_t* sf_word = reinterpret_cast<uint32_t*>(a.sf + ((static_cast<long long>(h) * d_atoms + da) * a.sf_blocks + g) * 512 + atom_byte);
      uint32_t word = QUANT ? 0u : *sf_word;
      for (int k = 0; k < 4; ++k) {
        const long long r0 = row0 + k * 32;
        if (!valid_d || r0 >= seq_end) continue;
        const int n = static_cast<int>(min(32LL, seq_end - r0));
        const long long stride = static_cast<long long>(a.heads) * a.head_dim;
        const long long base = (r0 * a.heads + h) * static_cast<long long>(a.head_dim) + d;
        if constexpr (QUANT) {
          float v[32];
          float amax = 0.f;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            v[i] = i < n ? load_elem(x, base + i * stride) : 0.f;
            amax = fmaxf(amax, fabsf(v[i]));
          }
          float inv;
          word |= mx_e8m0_of(amax, inv) << (8 * k);
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (i < n) x8[base + i * stride] = static_cast<uint8_t>(pack_e4m3x4(v[i] * inv, 0.f, 0.f, 0.f) & 0xffu);
        } else {
          const float sc = mx_scale_of((word >> (8 * k)) & 0xffu);
          for (int i = 0; i < n; ++i) store_elem(x, base + i * stride, e4m3_to_float(x8[base + i * stride]) * sc);
        }
      }
      if constexpr (QUANT) *sf_word = word;
    }
  }
}

template <typename T>
int launch_mx_t(const MxArgs& a, int quantize, cudaStream_t stream) {
  const dim3 grid(static_cast<unsigned>(a.max_blocks), static_cast<unsigned>(a.heads));
  if (a.scale_axis == 0) {
    if (quantize) gdpa_mxfp8_kernel<T, 0, true><<<grid, kTile, 0, stream>>>(a);
    else gdpa_mxfp8_kernel<T, 0, false><<<grid, kTile, 0, stream>>>(a);
  } else {
    if (quantize) gdpa_mxfp8_kernel<T, 1, true><<<grid, kTile, 0, stream>>>(a);
    else gdpa_mxfp8_kernel<T, 1, false><<<grid, kTile, 0, stream>>>(a);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : GDPA_ERR_LAUNCH_;
}

}  // namespace

int launch_mxfp8(const MxArgs& a, int quantize, int x_is_fp32, cudaStream_t stream) {
  gdpa_block_offsets_kernel<<<1, 32, 0, stream>>>(a.offsets, a.block_offsets, a.off64, a.batch);
  if (cudaGetLastError() != cudaSuccess) return GDPA_ERR_LAUNCH_;
  if (a.max_blocks == 0) return 0;
  return x_is_fp32 ? launch_mx_t<float>(a, quantize, stream) : launch_mx_t<__nv_bfloat16>(a, quantize, stream);
}

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
