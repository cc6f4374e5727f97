// Row-wise norms either side of the GDPA forward, for the fused pipeline
//
//   ln_q = LayerNorm(Q) over all heads of a token      -> gdpa_layernorm_rows_kernel
//   x    = GDPA(ln_q, K, V) + ln_q                      (residual add and the per-row sum of x^2 are fused
//                                                        into the epilogue of gdpa_fwd_kernel)
//   out  = x * rsqrt(mean(x^2) + eps) * w (+ residual)  -> gdpa_rmsnorm_rows_kernel
//
// which is what the reference's GDPA-plus-norm kernel computes in one launch with a cluster of one CTA per
// head (gdpa_megakernel/src/tlx_gdpa_megakernel.py:359-405 RMS norm, :412-500 layer norm, :1076-1135
// epilogue order; checked by gdpa_megakernel/tests/test_tlx_gdpa_megakernel.py:50-145).  Both kernels are
// HBM-bound streaming passes: one warp per token row of N = heads * head_dim bf16 values, 16-byte loads,
// fp32 statistics, the row kept in registers between the statistics and the write when N <= 2048.  The backward
// of both norms (gdpa_norm_rows_bwd_kernel) follows the same row-per-warp scheme on a persistent grid.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "gdpa_launch.h"

namespace gdpa {

namespace {

constexpr int kNormThreads = 256;         // 8 rows per block

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
  return v;
}

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    f[2 * j] = __uint_as_float(w[j] << 16);
    f[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
  }
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  return make_uint4(pack2(f[0], f[1]), pack2(f[2], f[3]), pack2(f[4], f[5]), pack2(f[6], f[7]));
}

__device__ __forceinline__ void load8(const float* p, float (&f)[8]) {
  const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

// y = (x - mean) * rstd * weight + bias per row; mean and the (biased) variance over the N values of the row,
// variance from the centred values like torch.nn.functional.layer_norm.  A lane keeps up to kCachedChunks
// 16-byte chunks of the row in registers between the passes (rows of up to 256 * kCachedChunks values; the
// instantiation is chosen by the row length, fewer registers giving more rows in flight); longer rows are
// read again.
template <int kCachedChunks>
__global__ void __launch_bounds__(kNormThreads) gdpa_layernorm_rows_kernel(const NormArgs a) {
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * (kNormThreads / 32) + (threadIdx.x >> 5);
  if (row >= a.rows) return;
  const int chunks = a.n / 8;
  const uint4* src = reinterpret_cast<const uint4*>(a.x + row * a.n);
  uint4* dst = reinterpret_cast<uint4*>(a.out + row * a.n);
  const bool cached = chunks <= 32 * kCachedChunks;
  uint4 keep[kCachedChunks];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < kCachedChunks; ++i) {
    const int c = lane + 32 * i;
    keep[i] = make_uint4(0, 0, 0, 0);
    if (c < chunks) {
      keep[i] = src[c];
      float f[8];
      unpack8(keep[i], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) sum += f[j];
    }
  }
  for (int c = lane + 32 * kCachedChunks; c < chunks; c += 32) {
    float f[8];
    unpack8(src[c], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) sum += f[j];
  }
  const float mean = warp_sum(sum) / static_cast<float>(a.n);
  float var = 0.f;
#pragma unroll
  for (int i = 0; i < kCachedChunks; ++i) {
    if (lane + 32 * i < chunks) {
      float f[8];
      unpack8(keep[i], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) var = fmaf(f[j] - mean, f[j] - mean, var);
    }
  }
  for (int c = lane + 32 * kCachedChunks; c < chunks; c += 32) {
    float f[8];
    unpack8(src[c], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) var = fmaf(f[j] - mean, f[j] - mean, var);
  }
  const float rstd = rsqrtf(warp_sum(var) / static_cast<float>(a.n) + a.eps);
  if (a.row_mean != nullptr && lane == 0) {
    a.row_mean[row] = mean;
    a.row_rstd[row] = rstd;
  }
  for (int c = lane; c < chunks; c += 32) {
    float f[8];
    const int i = c >> 5;
    uint4 v;
    if (cached) {
      // select from the register copy without dynamic indexing
      v = keep[0];
#pragma unroll
      for (int k = 1; k < kCachedChunks; ++k)
        if (i == k) v = keep[k];
    } else {
      v = src[c];
    }
    unpack8(v, f);
    float w[8], b[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      w[j] = 1.f;
      b[j] = 0.f;
    }
    if (a.weight != nullptr) load8(a.weight + 8 * c, w);
    if (a.bias != nullptr) load8(a.bias + 8 * c, b);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = fmaf((f[j] - mean) * rstd, w[j], b[j]);
    dst[c] = pack8(f);
  }
}

// out = x * rsqrt(sumsq / N + eps) * weight (+ residual).  `row_sumsq` holds the per-row sum of squares when
// the producer of x accumulated it (the forward kernel's fused epilogue); when it is null the kernel sums the
// squares of the bf16 values of x itself.
__global__ void __launch_bounds__(kNormThreads) gdpa_rmsnorm_rows_kernel(const NormArgs a) {
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * (kNormThreads / 32) + (threadIdx.x >> 5);
  if (row >= a.rows) return;
  const int chunks = a.n / 8;
  const uint4* src = reinterpret_cast<const uint4*>(a.x + row * a.n);
  uint4* dst = reinterpret_cast<uint4*>(a.out + row * a.n);
  const uint4* res = a.residual != nullptr ? reinterpret_cast<const uint4*>(a.residual + row * a.n) : nullptr;
  float ssq;
  if (a.row_sumsq != nullptr) {
    ssq = a.row_sumsq[row];
  } else {
    float s = 0.f;
    for (int c = lane; c < chunks; c += 32) {
      float f[8];
      unpack8(src[c], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) s = fmaf(f[j], f[j], s);
    }
    ssq = warp_sum(s);
  }
  const float rrms = rsqrtf(ssq / static_cast<float>(a.n) + a.eps);
  if (a.row_rstd != nullptr && lane == 0) a.row_rstd[row] = rrms;
  for (int c = lane; c < chunks; c += 32) {
    float f[8], w[8], r[8];
    unpack8(src[c], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      w[j] = 1.f;
      r[j] = 0.f;
    }
    if (a.weight != nullptr) load8(a.weight + 8 * c, w);
    if (res != nullptr) unpack8(res[c], r);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = fmaf(f[j] * rrms, w[j], r[j]);
    dst[c] = pack8(f);
  }
}

// ------------------------------------------------------------------------------------------------------------
// Backward of the two row norms.  One warp per row, persistent grid; lanes own fixed columns, so the weight / bias
// gradients (sums over rows) are collected per block in shared memory and flushed with one global atomic per
// column and block.
constexpr int kNormBwdMaxN = 4096;  // weight / bias gradients are supported up to this row length

// RMS norm  y = x r w,  r = rsqrt(mean(x^2) + eps)  (r saved by the forward):
//   g = dy w;  dx = r g - x r^3 mean(g x);  dw += dy x r.
// Layer norm  y = xh rstd' ...  with xh = (x - mean) rstd (mean, rstd saved by the forward):
//   g = (dy + dy_add) w;  dx = rstd (g - mean(g) - xh mean(g xh));  dw += (dy + dy_add) xh;  db += dy + dy_add.
// `dy_add` is an optional second incoming gradient of the same shape (the Q-residual branch of the pipeline).
// With mode 2 there is no norm: dx = dy + dy_add.
template <int MODE>  // 0 = RMS norm, 1 = layer norm, 2 = plain sum
__global__ void __launch_bounds__(kNormThreads) gdpa_norm_rows_bwd_kernel(const NormBwdArgs a) {
  __shared__ float s_dw[MODE == 2 ? 1 : kNormBwdMaxN];
  __shared__ float s_db[MODE == 1 ? kNormBwdMaxN : 1];
  const int lane = threadIdx.x & 31;
  const int chunks = a.n / 8;
  const bool want_dw = MODE != 2 && a.dweight != nullptr;
  const bool want_db = MODE == 1 && a.dbias != nullptr;
  if (want_dw || want_db) {
    for (int i = threadIdx.x; i < a.n; i += kNormThreads) {
      if (want_dw) s_dw[i] = 0.f;
      if (want_db) s_db[i] = 0.f;
    }
    __syncthreads();
  }
  const long long warps = static_cast<long long>(gridDim.x) * (kNormThreads / 32);
  const float inv_n = 1.f / static_cast<float>(a.n);
  for (long long row = static_cast<long long>(blockIdx.x) * (kNormThreads / 32) + (threadIdx.x >> 5); row < a.rows; row += warps) {
    const uint4* dy = reinterpret_cast<const uint4*>(a.dy + row * a.n);
    const uint4* dy2 = a.dy_add != nullptr ? reinterpret_cast<const uint4*>(a.dy_add + row * a.n) : nullptr;
    const uint4* x = MODE != 2 ? reinterpret_cast<const uint4*>(a.x + row * a.n) : nullptr;
    uint4* dx = reinterpret_cast<uint4*>(a.dx + row * a.n);
    const float rstd = MODE != 2 ? a.row_rstd[row] : 1.f;
    const float mean = MODE == 1 ? a.row_mean[row] : 0.f;
    // pass 1: the row sums
    float s1 = 0.f, s2 = 0.f;
    if (MODE != 2) {
      for (int c = lane; c < chunks; c += 32) {
        float g[8], xv[8], w[8];
        unpack8(dy[c], g);
        if (dy2 != nullptr) {
          float t[8];
          unpack8(dy2[c], t);
#pragma unroll
          for (int j = 0; j < 8; ++j) g[j] += t[j];
        }
        unpack8(x[c], xv);
#pragma unroll
        for (int j = 0; j < 8; ++j) w[j] = 1.f;
        if (a.weight != nullptr) load8(a.weight + 8 * c, w);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float gw = g[j] * w[j];
          const float xh = MODE == 1 ? (xv[j] - mean) * rstd : xv[j];
          s1 += gw;
          s2 = fmaf(gw, xh, s2);
        }
      }
      s1 = warp_sum(s1) * inv_n;
      s2 = warp_sum(s2) * inv_n;
    }
    // pass 2: dx and the column sums (the row is read again; it sits in L1 / L2)
    for (int c = lane; c < chunks; c += 32) {
      float g[8], xv[8], w[8], o[8];
      unpack8(dy[c], g);
      if (dy2 != nullptr) {
        float t[8];
        unpack8(dy2[c], t);
#pragma unroll
        for (int j = 0; j < 8; ++j) g[j] += t[j];
      }
      if (MODE == 2) {
        dx[c] = pack8(g);
        continue;
      }
      unpack8(x[c], xv);
#pragma unroll
      for (int j = 0; j < 8; ++j) w[j] = 1.f;
      if (a.weight != nullptr) load8(a.weight + 8 * c, w);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float gw = g[j] * w[j];
        if (MODE == 0) {
          // dx = r g - x r^3 mean(g x)
          o[j] = rstd * (gw - xv[j] * rstd * rstd * s2);
          if (want_dw) atomicAdd(&s_dw[8 * c + j], g[j] * xv[j] * rstd);
        } else {
          const float xh = (xv[j] - mean) * rstd;
          o[j] = rstd * (gw - s1 - xh * s2);
          if (want_dw) atomicAdd(&s_dw[8 * c + j], g[j] * xh);
          if (want_db) atomicAdd(&s_db[8 * c + j], g[j]);
        }
      }
      dx[c] = pack8(o);
    }
  }
  if (want_dw || want_db) {
    __syncthreads();
    for (int i = threadIdx.x; i < a.n; i += kNormThreads) {
      if (want_dw) atomicAdd(a.dweight + i, s_dw[i]);
      if (want_db) atomicAdd(a.dbias + i, s_db[i]);
    }
  }
}

}  // namespace

int launch_layernorm_rows(const NormArgs& a, cudaStream_t stream) {
  if (a.rows == 0) return 0;
  const long long blocks = (a.rows + kNormThreads / 32 - 1) / (kNormThreads / 32);
  const unsigned grid = static_cast<unsigned>(blocks);
  if (a.n <= 512) gdpa_layernorm_rows_kernel<2><<<grid, kNormThreads, 0, stream>>>(a);
  else if (a.n <= 1024) gdpa_layernorm_rows_kernel<4><<<grid, kNormThreads, 0, stream>>>(a);
  else gdpa_layernorm_rows_kernel<8><<<grid, kNormThreads, 0, stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : GDPA_ERR_LAUNCH_;
}

int launch_rmsnorm_rows(const NormArgs& a, cudaStream_t stream) {
  if (a.rows == 0) return 0;
  const long long blocks = (a.rows + kNormThreads / 32 - 1) / (kNormThreads / 32);
  gdpa_rmsnorm_rows_kernel<<<static_cast<unsigned>(blocks), kNormThreads, 0, stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : GDPA_ERR_LAUNCH_;
}

// mode: 0 = RMS norm, 1 = layer norm, 2 = plain sum of the two incoming gradients
int launch_norm_rows_bwd(const NormBwdArgs& a, int mode, cudaStream_t stream) {
  if (a.rows == 0) return 0;
  long long blocks = (a.rows + kNormThreads / 32 - 1) / (kNormThreads / 32);
  if (blocks > 148 * 8) blocks = 148 * 8;
  const unsigned grid = static_cast<unsigned>(blocks);
  if (mode == 0) gdpa_norm_rows_bwd_kernel<0><<<grid, kNormThreads, 0, stream>>>(a);
  else if (mode == 1) gdpa_norm_rows_bwd_kernel<1><<<grid, kNormThreads, 0, stream>>>(a);
  else gdpa_norm_rows_bwd_kernel<2><<<grid, kNormThreads, 0, stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : GDPA_ERR_LAUNCH_;
}

}  // namespace gdpa
