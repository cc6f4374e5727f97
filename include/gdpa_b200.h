/*
 * gdpa_b200.h -- C ABI of the B200 (sm_100a) GDPA kernel library (libgdpa_b200.so).
 *
 * GDPA = Generalized Dot Product Attention over jagged batches: for every sequence b and head h
 *     S = Q_b,h K_b,h^T            (fp32 accumulate)
 *     P = act(S) * qk_scale        (elementwise activation, scale AFTER the activation)
 *     O = cast(P) V_b,h
 * or, for GDPA_ACT_SOFTMAX, P = softmax(qk_scale * S) with online rescaling.
 *
 * The reference library (facebookresearch/ads_model_kernel_library) has no native boundary: its
 * kernels are Python DSL objects called from Python.  The entry points below are what a binding
 * for the reference's operator `gdpa::generalized_dot_product_attention` would call; each one
 * cites the reference interface it replaces (paths are relative to the reference's root).
 *
 * Conventions
 *  - Every pointer in the parameter structs is a DEVICE pointer unless its name ends in `_host`.
 *  - Q is [total_q, heads, head_dim], K and V are [total_kv, heads, head_dim], row-major and
 *    contiguous; offsets are [batch + 1] exclusive prefix sums of the sequence lengths, int32 or
 *    int64.  The field `offsets_are_int64` of the parameter structs is a set of flags: GDPA_OFFSETS_INT64 (1) for
 *    64-bit entries, GDPA_OFFSETS_PAIRS (2) when both offset arrays hold 2 * batch entries [start_0, end_0,
 *    start_1, end_1, ...] instead (the reference's use_start_end_offsets,
 *    gdpa/triton/triton_generalized_dot_product_attention.py:943-946, :4270-4274): sequences may then share or
 *    overlap K / V rows, Q rows must not overlap.  Pairs are accepted by gdpa_build_schedule, gdpa_fwd,
 *    gdpa_fwd_noalloc and gdpa_bwd (which then needs `dkv_accum`), not together with kv_seq_index or FP8.
 *  - The library allocates nothing and never synchronises the stream.  Scratch buffers
 *    (schedule, fp32 dQ accumulator, status word) are supplied by the caller; their sizes come
 *    from gdpa_schedule_bytes() and gdpa_bwd_workspace_bytes().
 *  - Entry points return 0 on success or a GDPA_ERR_* code; no C++ exception crosses the
 *    boundary.  gdpa_strerror() turns a code into text.
 *  - Every in-kernel wait is bounded.  A wait that runs out writes a non-zero code to
 *    `status` (if given), the kernel frees its tensor memory and returns; the context stays
 *    usable.
 *  - Offsets are trusted to be monotone prefix sums inside the tensors.  The kernels clamp every sequence range
 *    they read from an offset array to [0, total_q] / [0, total_kv], so a malformed array gives unspecified values
 *    for the sequences concerned but no access outside the tensors; checking the arrays is the host's business.
 *  - A sequence's result depends on that sequence's rows only: rows of other sequences that share a 128-row tile
 *    with it never reach its output, whatever they hold (Inf and NaN included), as with the reference's
 *    zero-padded per-sequence loads.
 */
#ifndef GDPA_B200_H_
#define GDPA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* A CUDA stream handle (cudaStream_t) passed as an opaque pointer. */
typedef void* gdpa_stream_t;

/* Return codes. */
enum {
  GDPA_OK = 0,
  GDPA_ERR_BAD_ARG = 1,        /* null pointer, negative size, struct_size mismatch            */
  GDPA_ERR_UNSUPPORTED_DIM = 2,/* head_dim not in {64, 128}                                    */
  GDPA_ERR_UNSUPPORTED_DTYPE = 3,
  GDPA_ERR_UNSUPPORTED_ACT = 4,
  GDPA_ERR_MISALIGNED = 5,     /* a tensor base is not 16-byte aligned                         */
  GDPA_ERR_LAUNCH = 6,         /* cudaGetLastError() after a launch was not cudaSuccess        */
  GDPA_ERR_DRIVER = 7,         /* tensor-map encoding entry point unavailable or failed        */
  GDPA_ERR_CAPACITY = 8,       /* schedule buffer too small for this batch                     */
  GDPA_ERR_DEVICE = 9,         /* current device is not compute capability 10.x               */
  GDPA_ERR_NOALLOC_TOO_LARGE = 10 /* gdpa_fwd_noalloc: batch needs more than GDPA_NOALLOC_MAX_ITEMS */
};

/* Activation ids.  0..11 are the reference's enumeration order
 * (gdpa/triton/math.py:43-55, :77-78); 100 is this library's name for the behaviour of the
 * reference's CPU kernel (softmax, gdpa/triton/triton_generalized_dot_product_attention.py:3973). */
enum {
  GDPA_ACT_RAW = 0,
  GDPA_ACT_GELU = 1,            /* exact erf GELU */
  GDPA_ACT_GELU_APPROX = 2,     /* tanh GELU      */
  GDPA_ACT_FAST_GELU = 3,       /* tanh GELU      */
  GDPA_ACT_LEAKY_RELU = 4,      /* slope 0.01     */
  GDPA_ACT_RELU = 5,
  GDPA_ACT_FAST_GELU_BF16 = 6,  /* tanh GELU      */
  GDPA_ACT_SILU = 7,
  GDPA_ACT_FAST_SILU = 8,
  GDPA_ACT_HARDSWISH = 9,
  GDPA_ACT_RELU_SQUARE = 10,
  GDPA_ACT_FAST_GELU_TAYLOR = 11, /* evaluated as tanh GELU, as the reference's eager table does */
  GDPA_ACT_SOFTMAX = 100
};

enum { GDPA_DTYPE_BF16 = 0, GDPA_DTYPE_FP8_E4M3 = 1 };

/* Which pass a schedule is for. */
enum {
  GDPA_SCHED_FWD = 0, /* one work item per (sequence, head, 256-row Q block)  */
  GDPA_SCHED_BWD = 1  /* one work item per (sequence, head, 128-row KV tile)  */
};

/* ---------------------------------------------------------------------------------------------
 * Work schedule: the list of tiles the persistent kernels walk, longest first.
 * Replaces precompute_for_varline_load_balancing (gdpa/src/interface.py:219-325), which builds
 * the same kind of list with torch ops and host synchronisations; this one is built on the device
 * without a host sync.
 * ------------------------------------------------------------------------------------------- */
typedef struct GdpaSchedParams {
  uint32_t struct_size;       /* sizeof(GdpaSchedParams) */
  int32_t mode;               /* GDPA_SCHED_FWD or GDPA_SCHED_BWD */
  const void* q_offsets;      /* [batch + 1] */
  const void* kv_offsets;     /* [batch + 1] */
  int32_t offsets_are_int64;
  int32_t batch;
  int32_t heads;
  int32_t max_seq_len_q;      /* lengths are clamped to these, as the reference does          */
  int32_t max_seq_len_kv;     /*   (gdpa/triton/triton_generalized_dot_product_attention.py:599-624) */
  int32_t kv_batch;           /* with kv_seq_index: sequences kv_offsets describes (its entries - 1); 0 = batch */
  void* schedule;             /* out: gdpa_schedule_bytes() bytes, 16-byte aligned             */
  int64_t schedule_bytes;     /* size of that buffer                                           */
  /* Optional [batch] map from a Q sequence to the entry of kv_offsets it attends to (the reference's
   * ad_to_request_offset: many Q sequences share one KV sequence, forward / inference only;
   * gdpa/triton/triton_generalized_dot_product_attention.py:3961-3966).  Same integer type as the
   * offsets.  Null = sequence b reads KV sequence b.  Entries outside [0, kv_batch) are clamped into it. */
  const void* kv_seq_index;
} GdpaSchedParams;

/* Bytes needed for a schedule of the given pass.  total_rows is total_q for GDPA_SCHED_FWD and
 * total_kv for GDPA_SCHED_BWD.  Pure host arithmetic. */
size_t gdpa_schedule_bytes(int32_t mode, int64_t total_rows, int32_t batch, int32_t heads);

/* Build the schedule on `stream`.  No host synchronisation. */
int gdpa_build_schedule(const GdpaSchedParams* params, gdpa_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * Forward.  Replaces the launch half of torch.ops.gdpa.generalized_dot_product_attention
 * (gdpa/triton/triton_generalized_dot_product_attention.py:3099-3335) and of _flash_attn_fwd
 * (gdpa/src/interface.py:931-1254): one persistent tcgen05 kernel.
 * ------------------------------------------------------------------------------------------- */
#define GDPA_OFFSETS_INT64 1
#define GDPA_OFFSETS_PAIRS 2

typedef struct GdpaFwdParams {
  uint32_t struct_size;       /* sizeof(GdpaFwdParams) */
  int32_t dtype;              /* GDPA_DTYPE_BF16 */
  const void* q;              /* [total_q,  heads, head_dim] */
  const void* k;              /* [total_kv, heads, head_dim] */
  const void* v;              /* [total_kv, heads, head_dim] */
  void* o;                    /* out [total_q, heads, head_dim], bf16 */
  const void* q_offsets;
  const void* kv_offsets;
  int32_t offsets_are_int64;
  int32_t batch;
  int64_t total_q;
  int64_t total_kv;
  int32_t heads;
  int32_t head_dim;           /* 64 or 128 */
  int32_t max_seq_len_q;
  int32_t max_seq_len_kv;
  int32_t activation;         /* GDPA_ACT_* */
  float qk_scale;             /* multiplies act(S); for softmax multiplies S before exp */
  const void* schedule;       /* from gdpa_build_schedule(GDPA_SCHED_FWD) */
  int32_t* status;            /* optional int32 in device memory, or in pinned host memory mapped into the device's
                                 address space (the host can then poll it without a synchronisation); written
                                 non-zero if a wait ran out */
  /* FP8 path only (gdpa_fwd_fp8): one fp32 scale per (sequence-local 128-token block, head),
   * laid out [number of blocks over the batch, heads]; block b of sequence s sits at row
   * block_offsets[s] + b where block_offsets is the exclusive prefix sum of ceil(len / 128). */
  const float* q_scales;
  const float* k_scales;
  const float* v_scales;
  const void* q_block_offsets;  /* [batch + 1], same integer type as the offsets */
  const void* kv_block_offsets; /* [batch + 1] */
  /* Optional cudaEvent_t pair recorded on `stream` immediately before and after the main kernel
   * launch, so that a benchmark can time that kernel alone.  Null = not recorded. */
  void* timing_start_event;
  void* timing_stop_event;
  /* Optional, GDPA_ACT_SOFTMAX with bf16 inputs only: fp32 [heads, total_q] log-sum-exp of the scaled
   * scores in base 2 (log2 sum_kv 2^(qk_scale log2(e) S)), which gdpa_bwd needs for the softmax
   * backward.  Null = not written. */
  float* lse;
  /* Grouped-query attention: number of K / V heads (heads must be a multiple of it; query head h reads
   * K / V head h / (heads / kv_heads)).  0 = same as heads.  K, V (and the FP8 K / V scales) are then
   * [total_kv, kv_heads, head_dim]. */
  int32_t kv_heads;
  /* Banded attention, the reference's window_size
   * (gdpa/triton/triton_generalized_dot_product_attention.py:209-211, :274-278): a pair of sequence-local
   * positions (q, kv) takes part only if |q - kv| <= window_size; scores outside are treated as 0 before
   * the activation (excluded from the softmax).  Stored as window_size + 1; 0 = no band. */
  int32_t window_plus_one;
  /* Optional [batch] map from a Q sequence to its KV sequence, as in GdpaSchedParams (forward only). */
  const void* kv_seq_index;
  /* Strides of Q, K, V in elements: {between rows (tokens), between heads}; the head dimension is always
   * contiguous.  0 = the contiguous default {heads * head_dim, head_dim}.  Packed layouts (the reference's
   * fused QKV / fused KV tensors, gdpa/triton/triton_generalized_dot_product_attention.py:605-622) are
   * passed as three base pointers into one buffer with the packed strides.  Strides in bytes must be
   * multiples of 16.  O is always written contiguously. */
  int64_t q_strides[2];
  int64_t k_strides[2];
  int64_t v_strides[2];
  /* Fused epilogue of the norm pipeline (gdpa_fwd with an element-wise activation only; GDPA_ERR_BAD_ARG
   * with softmax or FP8): when `residual` is set
   * ([total_q, heads, head_dim] bf16, contiguous) the kernel stores O + residual instead of O (the
   * reference's fused_q_residual_add, gdpa_megakernel/src/tlx_gdpa_megakernel.py:1076-1082); when
   * `row_sumsq` is set ([total_q] fp32, zeroed by the caller) every row's sum over heads and columns of the
   * squares of the stored values (taken before rounding to bf16) is added to it, which gdpa_rmsnorm_rows()
   * then turns into the RMS norm over heads * head_dim (:359-405).  Null = plain O. */
  const void* residual;
  float* row_sumsq;
  /* With kv_seq_index: the number of sequences kv_offsets describes (its entries minus one); entries of
   * kv_seq_index outside [0, kv_batch) are clamped into it.  0 = batch. */
  int32_t kv_batch;
  int32_t reserved;
} GdpaFwdParams;

int gdpa_fwd(const GdpaFwdParams* params, gdpa_stream_t stream);

/* Forward for callers that cannot allocate device memory.  No counterpart in the reference, whose
 * Python host code allocates freely through torch.  Same contract as gdpa_fwd() except that
 * `schedule` is ignored: the work schedule is built into a fixed array inside the library's device
 * image, so the caller passes only inputs and outputs.  Meant for hosts that own all device memory
 * through an arena of their own, or that run where an allocation would stall the device.
 *  - Limit: heads * (total_q / 256 + batch) <= GDPA_NOALLOC_MAX_ITEMS, otherwise
 *    GDPA_ERR_NOALLOC_TOO_LARGE is returned and nothing is launched.
 *  - The array (1 MiB) is shared by every call on a device and keeps the previous call's contents;
 *    calls whose kernels may overlap on the GPU race on it and must be ordered by the caller.
 *  - The first call on a device resolves the array's address; make it before any stream capture.
 *  - Calls no cudaMalloc / cudaFree and no allocating library routine. */
#define GDPA_NOALLOC_MAX_ITEMS 65536
int gdpa_fwd_noalloc(const GdpaFwdParams* params, gdpa_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * Row norms either side of the forward, for the reference's GDPA-plus-norm pipeline
 * (gdpa_megakernel/src/tlx_gdpa_megakernel.py:8155-8192: fused_layernorm, fused_q_residual_add,
 * fused_rms_norm, fused_residual_add).  Rows are tokens, `n` = heads * head_dim bf16 values per row
 * (a multiple of 8, rows contiguous and 16-byte aligned).
 * ------------------------------------------------------------------------------------------- */
typedef struct GdpaNormParams {
  uint32_t struct_size;   /* sizeof(GdpaNormParams) */
  int32_t n;              /* values per row */
  int64_t rows;
  const void* x;          /* [rows, n] bf16 */
  void* out;              /* [rows, n] bf16; may alias x */
  const float* weight;    /* optional [n] fp32 */
  const float* bias;      /* optional [n] fp32 (layer norm only) */
  const void* residual;   /* optional [rows, n] bf16 added AFTER the RMS norm (fused_residual_add) */
  const float* row_sumsq; /* RMS norm: optional [rows] fp32 sums of squares from gdpa_fwd; null = computed here */
  float* row_mean;        /* optional [rows] fp32 outputs: layer-norm mean ...                    */
  float* row_rstd;        /*   ... and 1 / sqrt(var + eps), or 1 / rms for the RMS norm            */
  float eps;
  int32_t reserved;
} GdpaNormParams;

/* out = (x - mean(x)) / sqrt(var(x) + eps) * weight + bias per row (biased variance, as torch layer_norm). */
int gdpa_layernorm_rows(const GdpaNormParams* params, gdpa_stream_t stream);
/* out = x / sqrt(mean(x^2) + eps) * weight + residual per row. */
int gdpa_rmsnorm_rows(const GdpaNormParams* params, gdpa_stream_t stream);

/* Backward of the two row norms (and the plain sum of two incoming gradients), for training through the
 * GDPA-plus-norm pipeline.  `mode`: 0 = RMS norm, 1 = layer norm, 2 = dx = dy + dy_add.
 *   RMS norm:   g = dy w;             dx = r (g - x r^2 mean(g x));            dweight += dy x r
 *   layer norm: g = (dy + dy_add) w;  dx = rstd (g - mean(g) - xh mean(g xh));  dweight += (dy + dy_add) xh;
 *               dbias += dy + dy_add,  xh = (x - mean) rstd
 * with r / mean / rstd the per-row statistics the forward entry points write (row_rstd, row_mean).  dweight and
 * dbias ([n] fp32, optional, n <= 4096) are added to: the caller zeroes them. */
typedef struct GdpaNormBwdParams {
  uint32_t struct_size;   /* sizeof(GdpaNormBwdParams) */
  int32_t mode;
  int64_t rows;
  int32_t n;
  int32_t reserved;
  const void* dy;         /* [rows, n] bf16 */
  const void* dy_add;     /* optional [rows, n] bf16, added to dy */
  const void* x;          /* [rows, n] bf16: the input of the norm (modes 0, 1) */
  void* dx;               /* [rows, n] bf16 */
  const float* weight;    /* optional [n] fp32 */
  const float* row_mean;  /* [rows] fp32 (mode 1) */
  const float* row_rstd;  /* [rows] fp32 (modes 0, 1) */
  float* dweight;         /* optional [n] fp32 */
  float* dbias;           /* optional [n] fp32 (mode 1) */
} GdpaNormBwdParams;

int gdpa_norm_rows_bwd(const GdpaNormBwdParams* params, gdpa_stream_t stream);

/* Producer of the FP8 inputs: quantises a jagged [total, heads, head_dim] tensor (bf16, or fp32 with
 * in_is_fp32) to e4m3 with one fp32 scale per (sequence-local 128-token block, head):
 * scale = max(amax / 448, 1e-12), value = e4m3(clamp(x / scale, -448, 448)).  Writes block_offsets
 * ([batch + 1], the integer type of the offsets: exclusive prefix sum of ceil(len / 128)) and scales
 * ([scale_rows, heads] fp32, scale_rows >= total / 128 + batch; rows past block_offsets[batch] are left
 * untouched).  No counterpart in the reference, whose quantisation helper for its low-precision variant is
 * missing from its tree (gdpa/src/interface.py:715-724 refers to it).  No host synchronisation. */
typedef struct GdpaQuantParams {
  uint32_t struct_size;   /* sizeof(GdpaQuantParams) */
  int32_t in_is_fp32;
  const void* x;
  void* x8;               /* [total, heads, head_dim] e4m3 */
  float* scales;
  const void* offsets;    /* [batch + 1] */
  void* block_offsets;    /* out: [batch + 1] */
  int32_t offsets_are_int64;
  int32_t batch;
  int64_t total;
  int32_t heads;
  int32_t head_dim;       /* a multiple of 4 */
  int64_t scale_rows;
} GdpaQuantParams;

int gdpa_quantize_fp8_blockwise(const GdpaQuantParams* params, gdpa_stream_t stream);

/* MXFP8 wire format of the reference's block-scaled variant (gdpa/src/interface.py:714-750,
 * gdpa/src/flash_fwd_sm100.py:746-833): e4m3 elements in the jagged [total, heads, head_dim] shape plus one
 * e8m0 scale (2^(code - 127)) per 32 elements along the contraction dimension.  Only the scale tensor is
 * padded, every sequence to a multiple of 128 rows; block_offsets[b] * 128 is the reference's
 * cu_seqlens_sf[b].  Scales live in 512-byte atoms of 128 rows x 4 scales, byte
 * 16 * (row % 32) + 4 * (row / 32) + k for row `row` and 32-element block k of the atom:
 *   scale_axis 0 (Q, K: scales along head_dim): rows are tokens, atom index
 *     (head * sf_blocks + token_block) * ceil(head_dim / 128) + head_dim_atom;
 *   scale_axis 1 (V: scales along the tokens): rows are head-dim indices, atom index
 *     (head * ceil(head_dim / 128) + head_dim_atom) * sf_blocks + token_block.
 * sf_blocks is the number of 128-row token blocks the scale tensor is laid out for: block_offsets[batch] for
 * the reference's layout (known to a caller that has the sequence lengths on the host), or any upper bound such
 * as total / 128 + batch (fewer than ceil(total / 128) is GDPA_ERR_CAPACITY; blocks past sf_blocks are left
 * unprocessed).  gdpa_quantize_mxfp8 is the producer the reference refers to but does not contain
 * (quantize_varlen_mxfp8_sf_only, gdpa/src/interface.py:715-724): code = exponent field of amax * (1 / 448) in
 * fp32, plus one when its mantissa is not zero (the reference's rule for its P tile,
 * gdpa/src/activation_utils.py:444-517), element = e4m3(x * 2^(127 - code)) to nearest even, saturating; scale
 * bytes of rows past a sequence's end are zero.  gdpa_dequantize_mxfp8 is the exact inverse map into bf16 or fp32
 * (every e4m3 value times a power of two is a bf16 number).  Both write block_offsets ([batch + 1], the integer
 * type of the offsets).  head_dim a multiple of 32, at most 512; x, x8 and sf 16-byte aligned.  No host synchronisation. */
typedef struct GdpaMxParams {
  uint32_t struct_size;   /* sizeof(GdpaMxParams) */
  int32_t x_is_fp32;      /* type of x: 0 bf16, 1 fp32 */
  void* x;                /* [total, heads, head_dim]: in (quantise) / out (de-quantise) */
  void* x8;               /* [total, heads, head_dim] e4m3: out / in */
  void* sf;               /* heads * ceil(head_dim / 128) * sf_blocks * 512 bytes: out / in */
  const void* offsets;    /* [batch + 1] */
  void* block_offsets;    /* out: [batch + 1] */
  int32_t offsets_are_int64;
  int32_t batch;
  int64_t total;
  int32_t heads;
  int32_t head_dim;
  int32_t scale_axis;
  int32_t reserved;
  int64_t sf_blocks;
} GdpaMxParams;

int gdpa_quantize_mxfp8(const GdpaMxParams* params, gdpa_stream_t stream);
int gdpa_dequantize_mxfp8(const GdpaMxParams* params, gdpa_stream_t stream);

/* Low-precision forward: Q, K, V are FP8 e4m3 with the per-block fp32 scales above, O is bf16; every
 * activation, head_dim 128.
 * Mirrors the reference's FP8 variant (gdpa/src/flash_fwd_sm100.py:326-352, output dtype rule
 * gdpa/src/interface.py:1053). */
int gdpa_fwd_fp8(const GdpaFwdParams* params, gdpa_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * Backward.  Replaces torch.ops.gdpa.generalized_dot_product_attention_backward
 * (gdpa/triton/triton_generalized_dot_product_attention.py:3461-3788) and _flash_attn_bwd
 * (gdpa/src/interface.py:1257-1685): S and P are recomputed, dQ, dK, dV come out of one
 * persistent kernel (for GDPA_ACT_SOFTMAX: dS = qk_scale P (dP - dPsum), with P rebuilt from the
 * forward's log-sum-exp); dQ is accumulated in fp32 (the reference reduces into bf16,
 * gdpa/src/flash_bwd_sm100.py:2267-2287) and rounded once by a second, bandwidth-bound kernel.
 * ------------------------------------------------------------------------------------------- */
typedef struct GdpaBwdParams {
  uint32_t struct_size;       /* sizeof(GdpaBwdParams) */
  int32_t dtype;              /* GDPA_DTYPE_BF16 */
  const void* q;
  const void* k;
  const void* v;
  const void* d_o;            /* [total_q, heads, head_dim] gradient of O */
  void* dq;                   /* out [total_q,  heads, head_dim] bf16 */
  void* dk;                   /* out [total_kv, heads, head_dim] bf16 */
  void* dv;                   /* out [total_kv, heads, head_dim] bf16 */
  const void* q_offsets;
  const void* kv_offsets;
  int32_t offsets_are_int64;
  int32_t batch;
  int64_t total_q;
  int64_t total_kv;
  int32_t heads;
  int32_t head_dim;
  int32_t max_seq_len_q;
  int32_t max_seq_len_kv;
  int32_t activation;
  float qk_scale;
  const void* schedule;       /* from gdpa_build_schedule(GDPA_SCHED_BWD).  gdpa_bwd writes one word of its header:
                               * the kernel hands work items to its CTAs through a counter there, which gdpa_bwd
                               * zeroes on the stream before the launch.  The list itself is only read and may be
                               * reused by later calls, but two gdpa_bwd calls that can run at the same time need
                               * a schedule buffer each. */
  void* dq_accum;             /* scratch: gdpa_bwd_workspace_bytes() bytes; zeroed by gdpa_bwd */
  int32_t* status;
  /* Optional cudaEvent_t pair recorded around the main backward kernel only (not around the
   * accumulator memset and the fp32 -> bf16 dQ rounding kernel).  Null = not recorded. */
  void* timing_start_event;
  void* timing_stop_event;
  /* GDPA_ACT_SOFTMAX only (the softmax backward, which the reference leaves unimplemented:
   * gdpa/src/flash_bwd_sm100.py:2038-2058 keeps the dPsum term commented out): the forward output O
   * [total_q, heads, head_dim] bf16, the forward's lse [heads, total_q] fp32, and a scratch buffer of
   * total_q * heads floats that receives dPsum = rowsum(dO * O). */
  const void* o;
  const float* lse;
  float* dpsum;
  /* Grouped-query attention: number of K / V heads, 0 = same as heads.  dK, dV are
   * [total_kv, kv_heads, head_dim] and sum the contributions of the query heads of a group; the
   * schedule must have been built with heads = kv_heads. */
  int32_t kv_heads;
  int32_t window_plus_one;    /* banded attention, as in GdpaFwdParams: window_size + 1, 0 = no band */
  /* Strides of Q, K, V in elements, as in GdpaFwdParams (0 = contiguous).  dO, dQ, dK, dV are contiguous. */
  int64_t q_strides[2];
  int64_t k_strides[2];
  int64_t v_strides[2];
  /* With GDPA_OFFSETS_PAIRS a K / V row can belong to several sequences, so dK and dV are summed in fp32:
   * scratch of 2 * total_kv * kv_heads * head_dim floats (dK then dV), 16-byte aligned, zeroed by gdpa_bwd, which
   * also rounds it into dk / dv (the reference adds with atomics into zeroed gradients,
   * gdpa/triton/triton_generalized_dot_product_attention.py:2369-2387, :3514).  Null otherwise. */
  void* dkv_accum;
} GdpaBwdParams;

/* Bytes of the fp32 dQ accumulator for a backward over total_q rows. */
size_t gdpa_bwd_workspace_bytes(int64_t total_q, int32_t heads, int32_t head_dim);

int gdpa_bwd(const GdpaBwdParams* params, gdpa_stream_t stream);

/* Text for a return code (static storage). */
const char* gdpa_strerror(int code);

/* Number of kernels launched by this library in this process so far (all entry points).
 * Used by benchmarks to report how many of this library's kernels ran in a timed region. */
int64_t gdpa_launch_count(void);

/* Diagnostic: launch a one-warp kernel whose single wait can never be satisfied and gives up after
 * `limit_ns` nanoseconds (at most 1 s): it must write a non-zero code to *status (device int32) and
 * return normally, leaving the context usable.  This is the give-up path of every in-kernel wait of
 * the library, exercised without hanging or faulting the GPU. */
int gdpa_debug_wait_probe(int32_t* status, uint64_t limit_ns, gdpa_stream_t stream);

/* Diagnostic hook for performance analysis: register a device buffer of 16384 int64 slots into which
 * CTA 0 of the forward kernel (and of the backward kernel in a library built with -DGDPA_ENABLE_TRACE)
 * writes SM cycle stamps at fixed points of its pipeline (slot layout in csrc/gdpa_fwd.cu and
 * csrc/gdpa_bwd.cu), or null to switch tracing off (default).  Process-wide; not meant for production use. */
void gdpa_debug_set_trace(void* device_buffer);

/* Library version: major * 10000 + minor * 100 + patch. */
int32_t gdpa_version(void);

#ifdef __cplusplus
}
#endif
#endif /* GDPA_B200_H_ */
