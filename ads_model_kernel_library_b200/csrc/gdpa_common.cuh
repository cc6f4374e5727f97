// Definitions shared by the GDPA schedule builder, the forward and the backward kernels.
#pragma once

#include "gdpa_launch.h"
#include "sm100_ptx.cuh"

namespace gdpa {

constexpr int kTile = 128;          // rows of one Q tile / KV tile
constexpr int kFwdQBlock = 256;     // Q rows of one forward work item (two Q tiles)
constexpr int kSchedHeaderInts = 4; // schedule buffer: int32 header, then int4 work items

// Activation classes the kernels are specialised on (several reference names share one class).
enum ActClass : int {
  ACT_RAW = 0,
  ACT_GELU_ERF = 1,
  ACT_GELU_TANH = 2,
  ACT_LEAKY_RELU = 3,
  ACT_RELU = 4,
  ACT_SILU = 5,
  ACT_HARDSWISH = 6,
  ACT_RELU_SQUARE = 7,
  ACT_SOFTMAX = 8,
  ACT_NUM_CLASSES = 9
};

__host__ __device__ inline int act_class_from_id(int id) {
  switch (id) {
    case 0: return ACT_RAW;
    case 1: return ACT_GELU_ERF;
    case 2: case 3: case 6: case 11: return ACT_GELU_TANH;
    case 4: return ACT_LEAKY_RELU;
    case 5: return ACT_RELU;
    case 7: case 8: return ACT_SILU;
    case 9: return ACT_HARDSWISH;
    case 10: return ACT_RELU_SQUARE;
    case 100: return ACT_SOFTMAX;
    default: return -1;
  }
}

// Offset flags: bit 0 = 64-bit entries; bit 1 = the array holds [start, end] pairs, two entries per sequence (the
// reference's use_start_end_offsets, gdpa/triton/triton_generalized_dot_product_attention.py:943-946, :4270-4274:
// sequences may then share or overlap K / V rows), instead of batch + 1 prefix sums.
constexpr int kOffsets64 = 1, kOffsetsPairs = 2;
__device__ __forceinline__ long long load_offset(const void* p, int i, int flags) {
  return (flags & kOffsets64) ? static_cast<const long long*>(p)[i] : static_cast<long long>(static_cast<const int*>(p)[i]);
}
// first row and row past the end of sequence b
__device__ __forceinline__ void seq_bounds(const void* p, int b, int flags, long long& start, long long& end) {
  const int i = (flags & kOffsetsPairs) ? 2 * b : b;
  start = load_offset(p, i, flags);
  end = load_offset(p, i + 1, flags);
}

// Cycle stamps for performance analysis: one CTA (GDPA_TRACE_CTA, default 0) writes clock64() into slot `slot` of the trace buffer
// when one was registered with gdpa_debug_set_trace().  Compiled in only in builds with -DGDPA_ENABLE_TRACE
// (the pointer tests sit in the MMA-issuing threads, which are on the critical path of every tile); the
// default build has none.
constexpr int kTraceSlots = 16384;
#ifdef GDPA_ENABLE_TRACE
#ifndef GDPA_TRACE_CTA
#define GDPA_TRACE_CTA 0
#endif
#define GDPA_TRACE(args, slot)                                                                  \
  do {                                                                                          \
    if ((args).trace != nullptr && blockIdx.x == GDPA_TRACE_CTA && (slot) >= 0 && (slot) < kTraceSlots) \
      (args).trace[(slot)] = clock64();                                                         \
  } while (0)
#else
#define GDPA_TRACE(args, slot) do { } while (0)
#endif

// One work item of a schedule, with the sequence geometry it refers to.
struct Work {
  int b, h, blk;
  int kb;  // entry of the KV offsets the sequence reads (b unless a kv_index is given)
  long long q_start, kv_start;
  int lq, lkv;
};

// What the offsets may address: rows of the Q-side and KV-side tensors and entries of the KV offsets.  Sequence
// bounds read from the offset arrays are clamped to these, so that a malformed offset array (an entry beyond the
// tensor, a decreasing pair, a kv_index entry beyond the KV batch) cannot make a kernel store outside a tensor; the
// result for such a sequence is unspecified but in bounds.  Validation proper is the host's job.
struct SeqLimits {
  long long total_q, total_kv;
  int kv_batch;  // sequences the KV offsets describe
};

__device__ __forceinline__ long long clamp_ll(long long x, long long lo, long long hi) { return x < lo ? lo : (x > hi ? hi : x); }

// `kv_index` (optional, same integer type as the offsets) maps a sequence to the entry of the KV offsets
// it reads: the reference's ad_to_request_offset, where many Q sequences share one KV sequence
// (gdpa/triton/triton_generalized_dot_product_attention.py:3961-3966).
__device__ __forceinline__ Work load_work(const int* sched, int idx, const void* q_off, const void* kv_off, int is64,
                                          int max_q, int max_kv, const SeqLimits& lim, const void* kv_index = nullptr) {
  const int4 it = reinterpret_cast<const int4*>(sched + kSchedHeaderInts)[idx];
  Work w;
  w.b = it.x;
  w.h = it.y;
  w.blk = it.z;
  int kb = w.b;
  if (kv_index != nullptr) {
    kb = static_cast<int>(load_offset(kv_index, w.b, is64));
    kb = kb < 0 ? 0 : (kb >= lim.kv_batch ? lim.kv_batch - 1 : kb);
  }
  long long q_end, kv_end;
  seq_bounds(q_off, w.b, is64, w.q_start, q_end);
  seq_bounds(kv_off, kb, is64, w.kv_start, kv_end);
  w.kb = kb;
  w.q_start = clamp_ll(w.q_start, 0, lim.total_q);
  w.kv_start = clamp_ll(w.kv_start, 0, lim.total_kv);
  q_end = clamp_ll(q_end, w.q_start, lim.total_q);
  kv_end = clamp_ll(kv_end, w.kv_start, lim.total_kv);
  const long long lq = q_end - w.q_start;
  const long long lkv = kv_end - w.kv_start;
  w.lq = static_cast<int>(lq < max_q ? lq : max_q);
  w.lkv = static_cast<int>(lkv < max_kv ? lkv : max_kv);
  return w;
}

// Banded attention (the reference's window_size): a pair (q, kv) of sequence-local positions takes part
// only if |q - kv| <= window; window < 0 means no band.  A forward work item (256 Q rows) then visits
// only the KV tiles that can hold such a pair, a backward work item (128 KV rows) only such Q tiles.
__device__ __forceinline__ void fwd_kv_range(const Work& w, int window, int& first, int& count) {
  const int nkv = (w.lkv + kTile - 1) / kTile;
  first = 0;
  count = nkv;
  if (window >= 0 && nkv > 0) {
    const int q_lo = w.blk * kFwdQBlock;
    const int q_hi = min(w.lq, q_lo + kFwdQBlock) - 1;
    const int lo = max(0, q_lo - window) / kTile;
    const int hi = min(nkv, (q_hi + window) / kTile + 1);
    first = lo < hi ? lo : 0;
    count = lo < hi ? hi - lo : 0;
  }
}
__device__ __forceinline__ void bwd_q_range(const Work& w, int window, int& first, int& count) {
  const int nq = (w.lq + kTile - 1) / kTile;
  first = 0;
  count = nq;
  if (window >= 0 && nq > 0) {
    const int kv_lo = w.blk * kTile;
    const int kv_hi = min(w.lkv, kv_lo + kTile) - 1;
    const int lo = max(0, kv_lo - window) / kTile;
    const int hi = min(nq, (kv_hi + window) / kTile + 1);
    first = lo < hi ? lo : 0;
    count = lo < hi ? hi - lo : 0;
  }
}
__device__ __forceinline__ bool in_window(int q_pos, int kv_pos, int window) {
  const int d = q_pos - kv_pos;
  return window < 0 || (d <= window && -d <= window);
}

// Zero-padded tiles.  A tile of a sequence is 128 rows; the last tile of a sequence holds fewer, and the rows after
// them in the packed tensor belong to the next sequence.  The reference reads such rows as zero (per-sequence block
// loads, gdpa/triton/triton_generalized_dot_product_attention.py:270, :317, :1575-1600), and so do these kernels: the
// loader warp fetches a ragged tile as full boxes onto a barrier of its own, overwrites the rows past the sequence end
// with zeros in shared memory, and only then releases the tile to its consumers.  Everything downstream sees a full
// tile whose padding is exactly zero: score entries outside the sequence are act(0) = 0 and their gradients
// act'(0) x 0 = 0 with no masking, and nothing of a neighbouring sequence (Inf and NaN included) can reach this one.

// Persistent CTAs walk the longest-first list in a zigzag: round r gives CTA c the item
// r*G + c on even rounds and r*G + (G-1-c) on odd rounds, so the CTA that drew the longest item of
// one round draws the shortest of the next.
struct WorkWalker {
  int round, grid, cta, count;
  __device__ WorkWalker(int count_) : round(0), grid(gridDim.x), cta(blockIdx.x), count(count_) {}
  __device__ __forceinline__ bool next(int& idx) {
    idx = round * grid + ((round & 1) ? (grid - 1 - cta) : cta);
    ++round;
    return idx < count;
  }
};

// act(x) * scale for the elementwise activation classes.  `hscale` = 0.5 * scale.
template <int ACT>
__device__ __forceinline__ float act_scaled(float x, float scale, float hscale) {
  if constexpr (ACT == ACT_RAW) {
    return x * scale;
  } else if constexpr (ACT == ACT_RELU) {
    return fmaxf(x, 0.f) * scale;
  } else if constexpr (ACT == ACT_LEAKY_RELU) {
    return (x > 0.f ? x : 0.01f * x) * scale;
  } else if constexpr (ACT == ACT_RELU_SQUARE) {
    float r = fmaxf(x, 0.f);
    return r * r * scale;
  } else if constexpr (ACT == ACT_HARDSWISH) {
    float r = fminf(fmaxf(x + 3.f, 0.f), 6.f);
    return x * r * (scale * (1.f / 6.f));
  } else if constexpr (ACT == ACT_GELU_ERF) {
    float xs = x * hscale;
    return fmaf(xs, erff(x * 0.70710678118654752f), xs);
  } else if constexpr (ACT == ACT_GELU_TANH) {
    // 0.5 x (1 + tanh(sqrt(2/pi) x (1 + 0.044715 x^2)))
    float x2 = x * x;
    float inner = fmaf(x2, 0.7978845608028654f * 0.044715f, 0.7978845608028654f);
    float t = tanh_approx(x * inner);
    float xs = x * hscale;
    return fmaf(xs, t, xs);
  } else if constexpr (ACT == ACT_SILU) {
    // x sigmoid(x) = 0.5 x (1 + tanh(x / 2))
    float t = tanh_approx(0.5f * x);
    float xs = x * hscale;
    return fmaf(xs, t, xs);
  } else {
    return x;
  }
}

// Two activations at once, packed bf16x2 result (x0 in the low half).  GELU-tanh and SiLU use packed
// f32x2 arithmetic around the two MUFU evaluations (fewer issue slots; tanh.approx.f32 is the cheapest
// tanh per element on this part); the other classes fall back to the scalar form.
template <int ACT>
__device__ __forceinline__ uint32_t act_scaled_pair_bf16(float x0, float x1, float scale, float hscale) {
  if constexpr (ACT == ACT_GELU_TANH) {
    const uint64_t X = pack_f32x2(x0, x1);
    const uint64_t X2 = mul_f32x2(X, X);
    const uint64_t INNER = fma_f32x2(X2, pack_f32x2(0.7978845608028654f * 0.044715f, 0.7978845608028654f * 0.044715f),
                                     pack_f32x2(0.7978845608028654f, 0.7978845608028654f));
    float u0, u1;
    unpack_f32x2(mul_f32x2(X, INNER), u0, u1);
    const uint64_t T = pack_f32x2(tanh_approx(u0), tanh_approx(u1));
    const uint64_t XS = mul_f32x2(X, pack_f32x2(hscale, hscale));
    float p0, p1;
    unpack_f32x2(fma_f32x2(XS, T, XS), p0, p1);
    return pack_bf16x2(p0, p1);
  } else if constexpr (ACT == ACT_SILU) {
    const uint64_t X = pack_f32x2(x0, x1);
    float h0, h1;
    unpack_f32x2(mul_f32x2(X, pack_f32x2(0.5f, 0.5f)), h0, h1);
    const uint64_t T = pack_f32x2(tanh_approx(h0), tanh_approx(h1));
    const uint64_t XS = mul_f32x2(X, pack_f32x2(hscale, hscale));
    float p0, p1;
    unpack_f32x2(fma_f32x2(XS, T, XS), p0, p1);
    return pack_bf16x2(p0, p1);
  } else {
    return pack_bf16x2(act_scaled<ACT>(x0, scale, hscale), act_scaled<ACT>(x1, scale, hscale));
  }
}

// act(x) and act'(x), both already multiplied by `scale`.
template <int ACT>
__device__ __forceinline__ void act_and_grad_scaled(float x, float scale, float hscale, float& p, float& g) {
  if constexpr (ACT == ACT_RAW) {
    p = x * scale;
    g = scale;
  } else if constexpr (ACT == ACT_RELU) {
    p = fmaxf(x, 0.f) * scale;
    g = x > 0.f ? scale : 0.f;
  } else if constexpr (ACT == ACT_LEAKY_RELU) {
    p = (x > 0.f ? x : 0.01f * x) * scale;
    g = x > 0.f ? scale : 0.01f * scale;
  } else if constexpr (ACT == ACT_RELU_SQUARE) {
    float r = fmaxf(x, 0.f);
    p = r * r * scale;
    g = 2.f * r * scale;
  } else if constexpr (ACT == ACT_HARDSWISH) {
    float r = fminf(fmaxf(x + 3.f, 0.f), 6.f);
    p = x * r * (scale * (1.f / 6.f));
    g = x < -3.f ? 0.f : (x > 3.f ? scale : fmaf(x, 2.f, 3.f) * (scale * (1.f / 6.f)));
  } else if constexpr (ACT == ACT_GELU_ERF) {
    float cdf = fmaf(0.5f, erff(x * 0.70710678118654752f), 0.5f);
    float pdf = __expf(-0.5f * x * x) * 0.3989422804014327f;
    p = x * cdf * scale;
    g = fmaf(x, pdf, cdf) * scale;
  } else if constexpr (ACT == ACT_GELU_TANH) {
    // p = 0.5 x (1 + t);  p' = 0.5 (1 + t) + 0.5 x (1 - t^2) c0 (1 + 3 c1 x^2)
    constexpr float c0 = 0.7978845608028654f, c1 = 0.044715f;
    float x2 = x * x;
    float t = tanh_approx(x * fmaf(x2, c0 * c1, c0));
    float xs = x * hscale;
    p = fmaf(xs, t, xs);
    float du = fmaf(x2, 3.f * c0 * c1, c0);
    float sech2 = fmaf(-t, t, 1.f);
    g = fmaf(xs * sech2, du, fmaf(hscale, t, hscale));
  } else if constexpr (ACT == ACT_SILU) {
    // sg = 0.5 (1 + tanh(x/2));  p = x sg;  p' = sg (1 + x (1 - sg))
    float t = tanh_approx(0.5f * x);
    float sg = fmaf(0.5f, t, 0.5f);
    p = x * sg * scale;
    g = sg * fmaf(x, 1.f - sg, 1.f) * scale;
  } else {
    p = x;
    g = 1.f;
  }
}

// Two elements at once: packed bf16x2 of act * scale (x0 in the low half) and the packed fp32 pair
// of act' * scale.  `m0` / `m1` = element is inside the sequence; masked elements give 0 and 0.
template <int ACT, bool MASKED>
__device__ __forceinline__ void act_and_grad_pair(float x0, float x1, float scale, float hscale, bool m0, bool m1,
                                                  uint32_t& p_bf16x2, uint64_t& g2) {
  float p0, p1, g0, g1;
  if constexpr (ACT == ACT_GELU_TANH) {
    constexpr float c0 = 0.7978845608028654f, c1 = 0.044715f;
    const uint64_t X = pack_f32x2(x0, x1);
    const uint64_t X2 = mul_f32x2(X, X);
    float u0, u1;
    unpack_f32x2(mul_f32x2(X, fma_f32x2(X2, pack_f32x2(c0 * c1, c0 * c1), pack_f32x2(c0, c0))), u0, u1);
    const uint64_t T = pack_f32x2(tanh_approx(u0), tanh_approx(u1));
    const uint64_t HS = pack_f32x2(hscale, hscale);
    // with s = hscale (1 + t):  p = x s  and  p' = s + p (1 - t) du   (1 - t^2 = (1 - t)(1 + t)); nine packed
    // operations per pair instead of thirteen, and the element-wise phase is bound by the FMA pipe
    const uint64_t S = fma_f32x2(T, HS, HS);
    const uint64_t P = mul_f32x2(X, S);
    const uint64_t DU = fma_f32x2(X2, pack_f32x2(3.f * c0 * c1, 3.f * c0 * c1), pack_f32x2(c0, c0));
    const uint64_t OMT = fma_f32x2(T, pack_f32x2(-1.f, -1.f), pack_f32x2(1.f, 1.f));
    const uint64_t G = fma_f32x2(mul_f32x2(P, DU), OMT, S);
    unpack_f32x2(P, p0, p1);
    if constexpr (!MASKED) {
      p_bf16x2 = pack_bf16x2(p0, p1);
      g2 = G;
      return;
    }
    unpack_f32x2(G, g0, g1);
  } else if constexpr (ACT == ACT_SILU) {
    const uint64_t X = pack_f32x2(x0, x1);
    float h0, h1;
    unpack_f32x2(mul_f32x2(X, pack_f32x2(0.5f, 0.5f)), h0, h1);
    const uint64_t T = pack_f32x2(tanh_approx(h0), tanh_approx(h1));
    // sg * scale and 1 - sg, each one fma of t
    const uint64_t SGS = fma_f32x2(T, pack_f32x2(hscale, hscale), pack_f32x2(hscale, hscale));
    const uint64_t P = mul_f32x2(X, SGS);
    const uint64_t OM = fma_f32x2(T, pack_f32x2(-0.5f, -0.5f), pack_f32x2(0.5f, 0.5f));
    const uint64_t G = mul_f32x2(SGS, fma_f32x2(X, OM, pack_f32x2(1.f, 1.f)));
    unpack_f32x2(P, p0, p1);
    if constexpr (!MASKED) {
      p_bf16x2 = pack_bf16x2(p0, p1);
      g2 = G;
      return;
    }
    unpack_f32x2(G, g0, g1);
  } else {
    act_and_grad_scaled<ACT>(x0, scale, hscale, p0, g0);
    act_and_grad_scaled<ACT>(x1, scale, hscale, p1, g1);
  }
  if constexpr (MASKED) {
    p0 = m0 ? p0 : 0.f;
    p1 = m1 ? p1 : 0.f;
    g0 = m0 ? g0 : 0.f;
    g1 = m1 ? g1 : 0.f;
  }
  p_bf16x2 = pack_bf16x2(p0, p1);
  g2 = pack_f32x2(g0, g1);
}

}  // namespace gdpa
