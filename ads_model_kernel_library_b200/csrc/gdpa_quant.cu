// Producer of the low-precision inputs of gdpa_fwd_fp8: a jagged [total, H, D] tensor (bf16 or fp32) is quantised
// to FP8 e4m3 with one fp32 scale per (sequence-local 128-token block, head), scale = max(amax / 448, 1e-12) over
// the block, value = e4m3(clamp(x / scale, -448, 448)) with round-to-nearest-even.  Block j of sequence b is row
// block_offsets[b] + j of the scale tensor, block_offsets being the exclusive prefix sum of ceil(len / 128), which
// the first kernel builds on the device (no host synchronisation).  HBM-bound byte work: one CTA of 128 threads
// per (block, head), the 128 x D tile moved in 16-element pieces.
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

// block_offsets = exclusive prefix sum of ceil(len / 128): one CTA, a run of sequences per thread, scan of the
// per-thread sums through warp shuffles.
constexpr int kScanThreads = 1024;
__global__ void __launch_bounds__(kScanThreads) gdpa_block_offsets_kernel(const void* offsets, void* block_offsets, int off64,
                                                                        int batch) {
  __shared__ long long s_warp[kScanThreads / 32];
  const int t = threadIdx.x, lane = t & 31, wp = t >> 5;
  const int per = (batch + kScanThreads - 1) / kScanThreads;
  const int b0 = min(batch, t * per), b1 = min(batch, b0 + per);
  auto blocks_of = [&](int b) {
    long long len = load_offset(offsets, b + 1, off64) - load_offset(offsets, b, off64);
    if (len < 0) len = 0;
    return (len + kTile - 1) / kTile;
  };
  long long sum = 0;
  for (int b = b0; b < b1; ++b) sum += blocks_of(b);
  long long incl = sum;
#pragma unroll
  for (int s = 1; s < 32; s <<= 1) {
    const long long o = __shfl_up_sync(0xffffffffu, incl, s);
    if (lane >= s) incl += o;
  }
  if (lane == 31) s_warp[wp] = incl;
  __syncthreads();
  if (wp == 0) {
    long long w = s_warp[lane];
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) {
      const long long o = __shfl_up_sync(0xffffffffu, w, s);
      if (lane >= s) w += o;
    }
    s_warp[lane] = w;  // inclusive over warps
  }
  __syncthreads();
  incl += wp > 0 ? s_warp[wp - 1] : 0;
  long long run = incl - sum;
  auto put = [&](int b, long long v) {
    if (off64) static_cast<long long*>(block_offsets)[b] = v;
    else static_cast<int*>(block_offsets)[b] = static_cast<int>(v);
  };
  for (int b = b0; b < b1; ++b) {
    put(b, run);
    run += blocks_of(b);
  }
  if (t == kScanThreads - 1) put(batch, incl);
}

__device__ __forceinline__ float load_elem(const float* p, long long i) { return p[i]; }
__device__ __forceinline__ float load_elem(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }

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

// 16 consecutive elements <-> fp32 registers
__device__ __forceinline__ void load16(const float* p, float (&v)[16]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float4 f = reinterpret_cast<const float4*>(p)[i];
    v[4 * i] = f.x, v[4 * i + 1] = f.y, v[4 * i + 2] = f.z, v[4 * i + 3] = f.w;
  }
}
__device__ __forceinline__ void load16(const __nv_bfloat16* p, float (&v)[16]) {
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const uint4 u = reinterpret_cast<const uint4*>(p)[i];
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      v[8 * i + 2 * e] = __uint_as_float(w[e] << 16);
      v[8 * i + 2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
    }
  }
}
__device__ __forceinline__ void store16(float* p, const float (&v)[16]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) reinterpret_cast<float4*>(p)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
}
__device__ __forceinline__ void store16(__nv_bfloat16* p, const float (&v)[16]) {
#pragma unroll
  for (int i = 0; i < 2; ++i)
    reinterpret_cast<uint4*>(p)[i] = make_uint4(pack_bf16x2(v[8 * i], v[8 * i + 1]), pack_bf16x2(v[8 * i + 2], v[8 * i + 3]),
                                                pack_bf16x2(v[8 * i + 4], v[8 * i + 5]), pack_bf16x2(v[8 * i + 6], v[8 * i + 7]));
}
// 16 e4m3 codes -> fp32
__device__ __forceinline__ void unpack_e4m3x16(const uint4 raw, float (&v)[16]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
#pragma unroll
    for (int hlf = 0; hlf < 2; ++hlf) {
      const __half2_raw h2 = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>((w[e] >> (16 * hlf)) & 0xffffu), __NV_E4M3);
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h2));
      v[4 * e + 2 * hlf] = f.x;
      v[4 * e + 2 * hlf + 1] = f.y;
    }
  }
}
__device__ __forceinline__ uint4 pack_e4m3x16(const float (&v)[16]) {
  return make_uint4(pack_e4m3x4(v[0], v[1], v[2], v[3]), pack_e4m3x4(v[4], v[5], v[6], v[7]),
                    pack_e4m3x4(v[8], v[9], v[10], v[11]), pack_e4m3x4(v[12], v[13], v[14], v[15]));
}

constexpr int kMxMaxAtoms = 4;  // head_dim <= 512

// One CTA of 128 threads per (128-token block, head): a 128 x D tile, moved in 16-element pieces (a row of the
// tile is D / 16 consecutive pieces, so 8 lanes cover 128 contiguous bytes of e4m3).  The tile's scale atoms pass
// through shared memory and are read / written as whole 512-byte lines.  AXIS 0: scales along the head dim (a
// 32-element block is two pieces of neighbouring lanes).  AXIS 1: scales along the tokens (a block is 32 rows of one
// head-dim index; thread = (32-row block, 8-row quarter, 16-wide head-dim piece), maxima combined through shared
// memory, the tile read twice: it stays in L1 / L2).  QUANT: x -> (x8, sf); else (x8, sf) -> x.
template <typename T, int AXIS, bool QUANT>
__global__ void __launch_bounds__(kTile) gdpa_mxfp8_kernel(const MxArgs a) {
  __shared__ __align__(16) uint8_t s_sf[kMxMaxAtoms][512];
  __shared__ float s_amax[(AXIS == 1 && QUANT) ? 4 * 4 * 128 : 1];
  const long long g = blockIdx.x;
  const int h = blockIdx.y;
  if (g >= load_offset(a.block_offsets, a.batch, a.off64)) return;
  const int b = owner_of_block(a.block_offsets, a.off64, a.batch, g);
  const long long seq_end = load_offset(a.offsets, b + 1, a.off64);
  const long long row0 = load_offset(a.offsets, b, a.off64) + (g - load_offset(a.block_offsets, b, a.off64)) * kTile;
  const int nrows = static_cast<int>(min(static_cast<long long>(kTile), seq_end - row0));
  const int t = threadIdx.x;
  const int D = a.head_dim;
  const int d_atoms = (D + 127) / 128;
  const int cpr = D / 16;  // pieces per row
  T* x = static_cast<T*>(a.x);
  uint8_t* x8 = static_cast<uint8_t*>(a.x8);
  auto atom_words = [&](int da) {
    const long long atom = AXIS == 0 ? (static_cast<long long>(h) * a.sf_blocks + g) * d_atoms + da
                                     : (static_cast<long long>(h) * d_atoms + da) * a.sf_blocks + g;
    return reinterpret_cast<uint32_t*>(a.sf + atom * 512);
  };
  auto elem_base = [&](int row) { return ((row0 + row) * a.heads + h) * static_cast<long long>(D); };
  for (int da = 0; da < d_atoms; ++da) reinterpret_cast<uint32_t*>(s_sf[da])[t] = QUANT ? 0u : atom_words(da)[t];
  __syncthreads();

  if constexpr (AXIS == 0) {
    const int limit = nrows * cpr;  // even: D is a multiple of 32
    for (int i0 = 0; i0 < limit; i0 += kTile) {
      const int idx = i0 + t;
      const bool active = idx < limit;
      const int row = idx / cpr, c = idx % cpr;
      const int d0 = c * 16;
      uint8_t* code_at = &s_sf[d0 >> 7][16 * (row & 31) + 4 * (row >> 5) + ((d0 & 127) >> 5)];
      float v[16];
      if constexpr (QUANT) {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = 0.f;
        if (active) load16(x + elem_base(row) + d0, v);
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));  // the other half of the 32-element block
        float inv;
        const uint32_t code = mx_e8m0_of(amax, inv);
        if (active) {
          if ((c & 1) == 0) *code_at = static_cast<uint8_t>(code);
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] *= inv;
          *reinterpret_cast<uint4*>(x8 + elem_base(row) + d0) = pack_e4m3x16(v);
        }
      } else if (active) {
        const float sc = mx_scale_of(*code_at);
        unpack_e4m3x16(*reinterpret_cast<const uint4*>(x8 + elem_base(row) + d0), v);
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] *= sc;
        store16(x + elem_base(row) + d0, v);
      }
    }
  } else if constexpr (!QUANT) {
    // scales of (32-row block kb, head-dim index d) regrouped so that a piece reads its 16 codes as one vector
    __shared__ __align__(16) uint8_t s_code[kMxMaxAtoms][4][128];
    for (int da = 0; da < d_atoms; ++da) {
      const uint32_t word = reinterpret_cast<const uint32_t*>(s_sf[da])[t];  // bytes of head-dim index (t / 4) + 32 * (t % 4)
#pragma unroll
      for (int kb = 0; kb < 4; ++kb) s_code[da][kb][(t >> 2) + 32 * (t & 3)] = static_cast<uint8_t>(word >> (8 * kb));
    }
    __syncthreads();
    const int limit = nrows * cpr;
    for (int idx = t; idx < limit; idx += kTile) {
      const int row = idx / cpr, d0 = (idx % cpr) * 16;
      const uint4 cw = *reinterpret_cast<const uint4*>(&s_code[d0 >> 7][row >> 5][d0 & 127]);
      const uint32_t cws[4] = {cw.x, cw.y, cw.z, cw.w};
      float v[16];
      unpack_e4m3x16(*reinterpret_cast<const uint4*>(x8 + elem_base(row) + d0), v);
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] *= mx_scale_of((cws[i >> 2] >> (8 * (i & 3))) & 0xffu);
      store16(x + elem_base(row) + d0, v);
    }
  } else {
    const int kb = t >> 5, tq = (t >> 3) & 3, dc = t & 7;
    for (int da = 0; da < d_atoms; ++da) {
      const int d0 = da * 128 + dc * 16;
      const bool has_d = d0 < D;
      float amax[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) amax[i] = 0.f;
      for (int r = 0; r < 8; ++r) {
        const int row = kb * 32 + tq * 8 + r;
        if (has_d && row < nrows) {
          float v[16];
          load16(x + elem_base(row) + d0, v);
#pragma unroll
          for (int i = 0; i < 16; ++i) amax[i] = fmaxf(amax[i], fabsf(v[i]));
        }
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) s_amax[(kb * 4 + tq) * 128 + dc * 16 + i] = amax[i];
      __syncthreads();
      float inv[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        float m = 0.f;
#pragma unroll
        for (int q = 0; q < 4; ++q) m = fmaxf(m, s_amax[(kb * 4 + q) * 128 + dc * 16 + i]);
        const uint32_t code = mx_e8m0_of(m, inv[i]);
        const int dl = dc * 16 + i;  // head-dim index inside the atom
        if (tq == 0 && has_d) s_sf[da][16 * (dl & 31) + 4 * (dl >> 5) + kb] = static_cast<uint8_t>(code);
      }
      for (int r = 0; r < 8; ++r) {
        const int row = kb * 32 + tq * 8 + r;
        if (has_d && row < nrows) {
          float v[16];
          load16(x + elem_base(row) + d0, v);
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] *= inv[i];
          *reinterpret_cast<uint4*>(x8 + elem_base(row) + d0) = pack_e4m3x16(v);
        }
      }
      __syncthreads();  // s_amax is reused by the next atom
    }
  }
  if constexpr (QUANT) {
    __syncthreads();
    for (int da = 0; da < d_atoms; ++da) atom_words(da)[t] = reinterpret_cast<const uint32_t*>(s_sf[da])[t];
  }
}

// One CTA of 128 threads per (128-token block, head): the 128 x D tile is read twice in 16-element pieces (8 lanes
// cover 256 contiguous bytes of bf16), first for the block maximum, then (from L1 / L2) to quantise.
template <typename T>
__global__ void __launch_bounds__(kTile) gdpa_quant_fp8_kernel(const QuantArgs a) {
  __shared__ float s_max[kTile / 32];
  __shared__ float s_scale;
  const long long g = blockIdx.x;  // block index over the batch
  const int h = blockIdx.y;
  if (g >= load_offset(a.block_offsets, a.batch, a.off64)) return;
  const int b = owner_of_block(a.block_offsets, a.off64, a.batch, g);
  const long long seq_end = load_offset(a.offsets, b + 1, a.off64);
  const long long row0 = load_offset(a.offsets, b, a.off64) + (g - load_offset(a.block_offsets, b, a.off64)) * kTile;
  const int nrows = static_cast<int>(min(static_cast<long long>(kTile), seq_end - row0));
  const int t = threadIdx.x;
  const int D = a.head_dim;
  const T* x = static_cast<const T*>(a.x);
  uint8_t* x8 = static_cast<uint8_t*>(a.x8);
  auto elem_base = [&](int row) { return ((row0 + row) * a.heads + h) * static_cast<long long>(D); };
  float amax = 0.f;
  if (a.vec16) {
    const int cpr = D / 16, limit = nrows * cpr;
    for (int idx = t; idx < limit; idx += kTile) {
      float v[16];
      load16(x + elem_base(idx / cpr) + (idx % cpr) * 16, v);
#pragma unroll
      for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
    }
  } else if (t < nrows) {
    for (int d = 0; d < D; ++d) amax = fmaxf(amax, fabsf(load_elem(x, elem_base(t) + d)));
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, s));
  if ((t & 31) == 0) s_max[t >> 5] = amax;
  __syncthreads();
  if (t == 0) {
    float m = s_max[0];
    for (int i = 1; i < kTile / 32; ++i) m = fmaxf(m, s_max[i]);
    const float scale = fmaxf(m / 448.f, 1e-12f);
    s_scale = scale;
    a.scales[g * a.heads + h] = scale;
  }
  __syncthreads();
  const float scale = s_scale;
  if (a.vec16) {
    const int cpr = D / 16, limit = nrows * cpr;
    for (int idx = t; idx < limit; idx += kTile) {
      const long long at = elem_base(idx / cpr) + (idx % cpr) * 16;
      float v[16];
      load16(x + at, v);
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] = fminf(fmaxf(v[i] / scale, -448.f), 448.f);
      *reinterpret_cast<uint4*>(x8 + at) = pack_e4m3x16(v);
    }
  } else if (t < nrows) {
    uint32_t* out = reinterpret_cast<uint32_t*>(x8 + elem_base(t));
    for (int d = 0; d < D; d += 4) {
      float v[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) v[e] = fminf(fmaxf(load_elem(x, elem_base(t) + d + e) / scale, -448.f), 448.f);
      out[d >> 2] = pack_e4m3x4(v[0], v[1], v[2], v[3]);
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
  gdpa_block_offsets_kernel<<<1, kScanThreads, 0, stream>>>(a.offsets, a.block_offsets, a.off64, a.batch);
  if (cudaGetLastError() != cudaSuccess) return GDPA_ERR_LAUNCH_;
  if (a.max_blocks == 0) return 0;
  return x_is_fp32 ? launch_mx_t<float>(a, quantize, stream) : launch_mx_t<__nv_bfloat16>(a, quantize, stream);
}

int launch_quant_fp8(const QuantArgs& a, int in_is_fp32, cudaStream_t stream) {
  gdpa_block_offsets_kernel<<<1, kScanThreads, 0, stream>>>(a.offsets, a.block_offsets, a.off64, a.batch);
  if (cudaGetLastError() != cudaSuccess) return GDPA_ERR_LAUNCH_;
  if (a.max_blocks == 0) return 0;
  const dim3 grid(static_cast<unsigned>(a.max_blocks), static_cast<unsigned>(a.heads));
  if (in_is_fp32) gdpa_quant_fp8_kernel<float><<<grid, kTile, 0, stream>>>(a);
  else gdpa_quant_fp8_kernel<__nv_bfloat16><<<grid, kTile, 0, stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : GDPA_ERR_LAUNCH_;
}

}  // namespace gdpa
