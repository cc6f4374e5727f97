// Internal interface between the C-ABI entry points (gdpa_api.cu) and the kernel translation
// units.  Plain structs only.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace gdpa {

// Internal copies of the public return codes (include/gdpa_b200.h).
constexpr int GDPA_ERR_UNSUPPORTED_DIM_ = 2;
constexpr int GDPA_ERR_UNSUPPORTED_ACT_ = 4;
constexpr int GDPA_ERR_LAUNCH_ = 6;

// The tensor map of one operand tensor: boxes of 128 rows x 128 bytes (128-byte swizzle).
constexpr int kTmapHeights = 1;
constexpr int kTmapRows[kTmapHeights] = {128};
struct TmapSet {
  CUtensorMap m[kTmapHeights];
};

// The maps of the fp32 dQ accumulator: boxes of 32 columns x 32, 16, 8, 4, 2, 1 rows, so that the reduce-add of a
// ragged tile covers exactly the rows of its sequence.
constexpr int kDqTmapHeights = 6;
struct DqTmapSet {
  CUtensorMap m[kDqTmapHeights];
};

// The map of the forward's output: boxes of 32 columns x 32 rows (64-byte swizzle), one warp's staging slab.  A slab with fewer than 32 rows of its sequence is stored from registers
// instead: further maps for smaller boxes, on top of the loaders' own, made the TMA unit refetch descriptors.
struct OutTmap {
  CUtensorMap m;
};

struct FwdArgs {
  __nv_bfloat16* o;
  const void* q_off;
  const void* kv_off;
  int off64;
  int heads;
  int max_q;
  int max_kv;
  float scale;
  const int* sched;
  int* status;
  // FP8 path: per-(128-token block, head) fp32 scales and per-sequence block offsets.
  const float* q_scales;
  const float* k_scales;
  const float* v_scales;
  const void* q_blk_off;
  const void* kv_blk_off;
  long long* trace;  // optional cycle-stamp buffer of CTA 0 (performance analysis); null in normal use
  float* lse;        // softmax: optional [heads, total_q] log-sum-exp output (base 2)
  long long total_q;
  int kv_heads;      // K / V heads; query head h reads K / V head h / kv_group
  int kv_group;      // heads / kv_heads
  const void* kv_index;  // optional: sequence -> entry of the KV offsets (shared KV sequences)
  int window;            // band |q - kv| <= window of sequence-local positions; -1 = none
  // norm pipeline: optional [total_q, heads, D] bf16 tensor added to O before it is stored, and optional
  // [total_q] fp32 array that receives the sum over heads and columns of the squares of what is stored
  const __nv_bfloat16* residual;
  float* row_sumsq;
  long long total_kv;    // rows of K / V (bounds the sequence ranges read from the offsets)
  int kv_batch;          // sequences the KV offsets describe (bounds kv_index entries)
};

struct NormArgs {
  const __nv_bfloat16* x;
  __nv_bfloat16* out;
  const float* weight;
  const float* bias;
  const __nv_bfloat16* residual;
  const float* row_sumsq;
  float* row_mean;
  float* row_rstd;
  long long rows;
  int n;
  float eps;
};

struct QuantArgs {
  const void* x;
  void* x8;
  float* scales;
  const void* offsets;
  void* block_offsets;
  int off64;
  int batch;
  int heads;
  int head_dim;
  long long max_blocks;  // rows of `scales`: at least total / 128 + batch
  int vec16;             // head_dim a multiple of 16 and x, x8 16-byte aligned: 16-element vector accesses
};

struct MxArgs {
  void* x;        // [total, H, D] bf16 or fp32: input of the quantiser, output of the de-quantiser
  void* x8;       // [total, H, D] e4m3
  uint8_t* sf;    // e8m0 scales in 512-byte atoms
  const void* offsets;
  void* block_offsets;
  int off64;
  int batch;
  int heads;
  int head_dim;
  int scale_axis;       // 0: scales along the head dim (Q, K); 1: along the tokens (V)
  long long sf_blocks;  // 128-row token blocks the scale tensor is laid out for (its head stride)
  long long max_blocks; // grid bound: at least total / 128 + batch
};

struct NormBwdArgs {
  const __nv_bfloat16* dy;
  const __nv_bfloat16* dy_add;
  const __nv_bfloat16* x;
  __nv_bfloat16* dx;
  const float* weight;
  const float* row_mean;
  const float* row_rstd;
  float* dweight;
  float* dbias;
  long long rows;
  int n;
};

struct FwdLaunch {
  TmapSet tm_q, tm_k, tm_v;
  OutTmap tm_o;
  FwdArgs args;
  int grid;
  cudaStream_t stream;
};

struct BwdArgs {
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  float* dq_accum;
  const void* q_off;
  const void* kv_off;
  int off64;
  int heads;
  int max_q;
  int max_kv;
  float scale;
  const int* sched;
  int* status;
  long long* trace;  // optional cycle-stamp buffer of CTA 0; null in normal use
  const float* lse;    // softmax backward: [heads, total_q] log-sum-exp of the forward (base 2)
  const float* dpsum;  // softmax backward: [heads, total_q] rowsum(dO * O)
  long long total_q;
  int q_heads;         // query heads; `heads` above is the number of K / V heads (the work items' heads)
  int kv_group;        // q_heads / heads: a work item walks the Q tiles of every query head of its group
  int window;          // band |q - kv| <= window of sequence-local positions; -1 = none
  float* dk_acc;       // start / end offsets: fp32 accumulators the dK / dV tiles are added into (else null)
  float* dv_acc;
  long long total_kv;  // rows of K / V (bounds the sequence ranges read from the offsets)
};

struct BwdLaunch {
  TmapSet tm_q, tm_k, tm_v, tm_do;
  DqTmapSet tm_dq;
  BwdArgs args;
  int grid;
  cudaStream_t stream;
};

struct SchedArgs {
  const void* q_off;
  const void* kv_off;
  int off64;
  int batch;
  int heads;
  int max_q;
  int max_kv;
  int mode;
  int* sched;
  long long capacity_items;
  const void* kv_index;  // optional: sequence -> entry of the KV offsets
  int kv_batch;          // sequences the KV offsets describe (bounds kv_index entries)
};

}  // namespace gdpa
struct GdpaFwdParams;
namespace gdpa {
// Host-side argument checks of the forward entry points (no CUDA call): the return code gdpa_fwd / gdpa_fwd_fp8 would
// give for these parameters before they launch anything (`needs_schedule`: a null schedule pointer is an error).
int fwd_check_params(const GdpaFwdParams* p, bool fp8, bool needs_schedule);

int launch_fwd_bf16(const FwdLaunch& l, int head_dim, int act_class);
int launch_fwd_softmax_bf16(const FwdLaunch& l, int head_dim);
int launch_fwd_fp8(const FwdLaunch& l, int head_dim, int act_class);
int launch_bwd_bf16(const BwdLaunch& l, int head_dim, int act_class);
int launch_dpsum(const __nv_bfloat16* d_o, const __nv_bfloat16* o, float* dpsum, long long total_q, int heads, int head_dim,
                 cudaStream_t stream);
int launch_dq_convert(const float* acc, __nv_bfloat16* dq, long long n, cudaStream_t stream);
int launch_layernorm_rows(const NormArgs& a, cudaStream_t stream);
int launch_rmsnorm_rows(const NormArgs& a, cudaStream_t stream);
int launch_quant_fp8(const QuantArgs& a, int in_is_fp32, cudaStream_t stream);
int launch_mxfp8(const MxArgs& a, int quantize, int x_is_fp32, cudaStream_t stream);
int launch_norm_rows_bwd(const NormBwdArgs& a, int mode, cudaStream_t stream);
int launch_build_schedule(const SchedArgs& a, cudaStream_t stream);

}  // namespace gdpa
