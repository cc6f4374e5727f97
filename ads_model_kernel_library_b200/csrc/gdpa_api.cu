// C-ABI entry points of libgdpa_b200.so (declared in include/gdpa_b200.h): argument checks,
// TMA tensor-map encoding, kernel selection and launch.  Nothing here allocates device memory or
// synchronises a stream.
#include <atomic>
#include <cstring>

#include "../../include/gdpa_b200.h"
#include "gdpa_common.cuh"
#include "gdpa_launch.h"

namespace gdpa {
namespace {

std::atomic<long long> g_launches{0};
std::atomic<long long*> g_trace{nullptr};

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver's tensor-map encoder, looked up through the runtime so that the library does not
// link against libcuda.  The result is immutable once set.
EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) return nullptr;
    if (q != cudaDriverEntryPointSuccess) return nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

struct DeviceInfo {
  int sm_count = 0;
  int cc_major = 0;
};

// Immutable per-device attributes, read once per device.
int device_info(DeviceInfo* out) {
  constexpr int kMaxDev = 64;
  static std::atomic<int> ready[kMaxDev];
  static DeviceInfo info[kMaxDev];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return GDPA_ERR_DEVICE;
  if (!ready[dev].load(std::memory_order_acquire)) {
    DeviceInfo d;
    if (cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return GDPA_ERR_DEVICE;
    if (cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return GDPA_ERR_DEVICE;
    info[dev] = d;  // racing writers store identical values
    ready[dev].store(1, std::memory_order_release);
  }
  *out = info[dev];
  return out->cc_major == 10 ? GDPA_OK : GDPA_ERR_DEVICE;
}

// Tensor map over a [rows, heads, head_dim] row-major tensor; a box is `box_rows` rows of one
// head by `box_cols` elements, stored with the 128-byte swizzle (box_cols * elem_bytes == 128)
// or unswizzled.
// `row_stride` / `head_stride` are in elements; 0 means the contiguous default (heads * head_dim and
// head_dim).  Packed layouts (Q, K, V interleaved along the last dimension) are views with larger strides.
int make_tmap(CUtensorMap* m, const void* base, CUtensorMapDataType dt, int elem_bytes, long long rows, int heads,
              int head_dim, int box_cols, int box_rows, int swizzle_bytes, long long row_stride = 0,
              long long head_stride = 0) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (enc == nullptr) return GDPA_ERR_DRIVER;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) return GDPA_ERR_MISALIGNED;
  if (head_stride <= 0) head_stride = head_dim;
  if (row_stride <= 0) row_stride = static_cast<long long>(heads) * head_dim;
  if (head_stride < head_dim || row_stride < head_stride * heads) return GDPA_ERR_BAD_ARG;
  if ((head_stride * elem_bytes) % 16 != 0 || (row_stride * elem_bytes) % 16 != 0) return GDPA_ERR_MISALIGNED;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(head_dim), static_cast<cuuint64_t>(heads),
                        static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(head_stride) * elem_bytes,
                           static_cast<cuuint64_t>(row_stride) * elem_bytes};
  cuuint32_t box[3] = {static_cast<cuuint32_t>(box_cols), 1u, static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[3] = {1u, 1u, 1u};
  CUresult r = enc(m, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                   : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                   : swizzle_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? GDPA_OK : GDPA_ERR_DRIVER;
}

// The map of one operand tensor (TmapSet).
int make_tmap_set(TmapSet* set, const void* base, CUtensorMapDataType dt, int elem_bytes, long long rows, int heads,
                  int head_dim, int box_cols, long long row_stride = 0, long long head_stride = 0) {
  for (int i = 0; i < kTmapHeights; ++i) {
    const int rc = make_tmap(&set->m[i], base, dt, elem_bytes, rows, heads, head_dim, box_cols, kTmapRows[i], 128, row_stride,
                             head_stride);
    if (rc != GDPA_OK) return rc;
  }
  return GDPA_OK;
}

// A wait that nothing satisfies: one thread waits on an mbarrier nobody arrives on, with a short
// limit, so that the give-up path of the kernels' bounded waits (status word written, normal return)
// can be exercised without hanging or faulting the GPU.
__global__ void gdpa_wait_probe_kernel(int* status, unsigned long long limit_ns) {
  __shared__ unsigned long long bar;
  __shared__ int abort_flag;
  const uint32_t bar_addr = smem_u32(&bar);
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(bar_addr, 1);
    mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) (void)mbar_wait_limit(bar_addr, 0, &abort_flag, status, 0x7700 | ST_ROLE_LOAD, limit_ns);
  __syncthreads();
}

template <class P>
int check_common(const P* p) {
  if (p == nullptr || p->struct_size != sizeof(P)) return GDPA_ERR_BAD_ARG;
  if (p->batch < 0 || p->heads <= 0 || p->total_q < 0 || p->total_kv < 0) return GDPA_ERR_BAD_ARG;
  if (p->max_seq_len_q < 0 || p->max_seq_len_kv < 0) return GDPA_ERR_BAD_ARG;
  if (p->window_plus_one < 0 || p->window_plus_one > (1 << 29)) return GDPA_ERR_BAD_ARG;
  if (p->head_dim != 64 && p->head_dim != 128) return GDPA_ERR_UNSUPPORTED_DIM;
  if (p->q_offsets == nullptr || p->kv_offsets == nullptr) return GDPA_ERR_BAD_ARG;
  if ((p->offsets_are_int64 & ~(GDPA_OFFSETS_INT64 | GDPA_OFFSETS_PAIRS)) != 0) return GDPA_ERR_BAD_ARG;
  // TMA coordinates are 32-bit row indices (the padding of a ragged tile is fetched from up to 127 rows past the end).
  if (p->total_q >= (1ll << 31) - 128 || p->total_kv >= (1ll << 31) - 128) return GDPA_ERR_BAD_ARG;
  return GDPA_OK;
}

}  // namespace
}  // namespace gdpa

using namespace gdpa;

#pragma GCC visibility push(default)
extern "C" {

const char* gdpa_strerror(int code) {
  switch (code) {
    case GDPA_OK: return "ok";
    case GDPA_ERR_BAD_ARG: return "bad argument (null pointer, negative size or struct_size mismatch)";
    case GDPA_ERR_UNSUPPORTED_DIM: return "unsupported head_dim (supported: 64, 128)";
    case GDPA_ERR_UNSUPPORTED_DTYPE: return "unsupported dtype";
    case GDPA_ERR_UNSUPPORTED_ACT: return "unsupported activation for this entry point";
    case GDPA_ERR_MISALIGNED: return "tensor base address is not 16-byte aligned";
    case GDPA_ERR_LAUNCH: return "kernel launch failed";
    case GDPA_ERR_DRIVER: return "tensor-map encoding unavailable or failed";
    case GDPA_ERR_CAPACITY: return "schedule buffer too small";
    case GDPA_ERR_DEVICE: return "current device is not a compute-capability 10.x GPU";
    case GDPA_ERR_NOALLOC_TOO_LARGE:
      return "gdpa_fwd_noalloc: heads * (total_q / 256 + batch) exceeds GDPA_NOALLOC_MAX_ITEMS (65536); use gdpa_fwd with a caller-allocated schedule";
    default: return "unknown error code";
  }
}

int32_t gdpa_version(void) { return 100; }

int gdpa_debug_wait_probe(int32_t* status, uint64_t limit_ns, gdpa_stream_t stream) {
  if (status == nullptr || limit_ns == 0 || limit_ns > 1000000000ull) return GDPA_ERR_BAD_ARG;
  gdpa_wait_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(status, limit_ns);
  return cudaGetLastError() == cudaSuccess ? GDPA_OK : GDPA_ERR_LAUNCH;
}

void gdpa_debug_set_trace(void* device_buffer) { g_trace.store(static_cast<long long*>(device_buffer)); }

int64_t gdpa_launch_count(void) { return g_launches.load(); }

size_t gdpa_schedule_bytes(int32_t mode, int64_t total_rows, int32_t batch, int32_t heads) {
  if (total_rows < 0 || batch < 0 || heads <= 0) return 0;
  const int64_t tile = (mode == GDPA_SCHED_FWD) ? kFwdQBlock : kTile;
  const int64_t items = static_cast<int64_t>(heads) * (total_rows / tile + batch);
  return static_cast<size_t>(kSchedHeaderInts * 4 + 16 * (items > 0 ? items : 1));
}

size_t gdpa_bwd_workspace_bytes(int64_t total_q, int32_t heads, int32_t head_dim) {
  if (total_q < 0 || heads <= 0 || head_dim <= 0) return 0;
  return static_cast<size_t>(total_q) * heads * head_dim * sizeof(float);
}

int gdpa_build_schedule(const GdpaSchedParams* p, gdpa_stream_t stream) {
  if (p == nullptr || p->struct_size != sizeof(GdpaSchedParams)) return GDPA_ERR_BAD_ARG;
  if (p->batch < 0 || p->heads <= 0 || p->schedule == nullptr) return GDPA_ERR_BAD_ARG;
  if (p->mode != GDPA_SCHED_FWD && p->mode != GDPA_SCHED_BWD) return GDPA_ERR_BAD_ARG;
  if (p->batch > 0 && (p->q_offsets == nullptr || p->kv_offsets == nullptr)) return GDPA_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(p->schedule) & 15u) != 0) return GDPA_ERR_MISALIGNED;
  if (p->schedule_bytes < kSchedHeaderInts * 4 + 16) return GDPA_ERR_CAPACITY;
  if ((p->offsets_are_int64 & ~(GDPA_OFFSETS_INT64 | GDPA_OFFSETS_PAIRS)) != 0) return GDPA_ERR_BAD_ARG;
  if ((p->offsets_are_int64 & GDPA_OFFSETS_PAIRS) != 0 && p->kv_seq_index != nullptr) return GDPA_ERR_BAD_ARG;
  SchedArgs a;
  a.q_off = p->q_offsets;
  a.kv_off = p->kv_offsets;
  a.off64 = p->offsets_are_int64;
  a.batch = p->batch;
  a.heads = p->heads;
  a.max_q = p->max_seq_len_q;
  a.max_kv = p->max_seq_len_kv;
  a.mode = p->mode;
  a.sched = static_cast<int*>(p->schedule);
  a.capacity_items = (p->schedule_bytes - kSchedHeaderInts * 4) / 16;
  a.kv_index = p->kv_seq_index;
  if (p->kv_batch < 0) return GDPA_ERR_BAD_ARG;
  a.kv_batch = (p->kv_seq_index != nullptr && p->kv_batch > 0) ? p->kv_batch : p->batch;
  int rc = launch_build_schedule(a, static_cast<cudaStream_t>(stream));
  if (rc == 0) g_launches.fetch_add(1);
  return rc;
}

}  // extern "C"
#pragma GCC visibility pop

// Everything gdpa_fwd / gdpa_fwd_fp8 check on the host before they touch the device, in one place so that
// gdpa_fwd_noalloc can run the same checks before it writes its shared schedule array.
int gdpa::fwd_check_params(const GdpaFwdParams* p, bool fp8, bool needs_schedule) {
  int rc = check_common(p);
  if (rc != GDPA_OK) return rc;
  if (needs_schedule && p->schedule == nullptr) return GDPA_ERR_BAD_ARG;
  if (p->dtype != (fp8 ? GDPA_DTYPE_FP8_E4M3 : GDPA_DTYPE_BF16)) return GDPA_ERR_UNSUPPORTED_DTYPE;
  const int act = act_class_from_id(p->activation);
  if (act < 0) return GDPA_ERR_UNSUPPORTED_ACT;
  if (p->kv_batch < 0) return GDPA_ERR_BAD_ARG;
  if (p->total_q == 0 || p->batch == 0) return GDPA_OK;
  if (p->q == nullptr || p->o == nullptr) return GDPA_ERR_BAD_ARG;
  if (p->total_kv > 0 && (p->k == nullptr || p->v == nullptr)) return GDPA_ERR_BAD_ARG;
  if (((reinterpret_cast<uintptr_t>(p->o) | reinterpret_cast<uintptr_t>(p->q) | reinterpret_cast<uintptr_t>(p->k) |
        reinterpret_cast<uintptr_t>(p->v)) & 15u) != 0)
    return GDPA_ERR_MISALIGNED;
  if (fp8 && (p->q_scales == nullptr || p->k_scales == nullptr || p->v_scales == nullptr ||
              p->q_block_offsets == nullptr || p->kv_block_offsets == nullptr))
    return GDPA_ERR_BAD_ARG;
  const int kv_heads = p->kv_heads > 0 ? p->kv_heads : p->heads;
  if (p->heads % kv_heads != 0) return GDPA_ERR_BAD_ARG;
  if ((p->residual != nullptr || p->row_sumsq != nullptr) && (fp8 || act == ACT_SOFTMAX)) return GDPA_ERR_BAD_ARG;
  if ((p->offsets_are_int64 & GDPA_OFFSETS_PAIRS) != 0 && (fp8 || p->kv_seq_index != nullptr)) return GDPA_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(p->residual) & 15u) != 0) return GDPA_ERR_MISALIGNED;
  return GDPA_OK;
}

#pragma GCC visibility push(default)
extern "C" {

static int fwd_common(const GdpaFwdParams* p, gdpa_stream_t stream, bool fp8) {
  int rc = fwd_check_params(p, fp8, true);
  if (rc != GDPA_OK) return rc;
  if (p->total_q == 0 || p->batch == 0) return GDPA_OK;
  const int act = act_class_from_id(p->activation);
  const int kv_heads = p->kv_heads > 0 ? p->kv_heads : p->heads;
  DeviceInfo di;
  rc = device_info(&di);
  if (rc != GDPA_OK) return rc;

  FwdLaunch l;
  std::memset(&l, 0, sizeof(l));
  const CUtensorMapDataType dt = fp8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const int eb = fp8 ? 1 : 2;
  const int box_cols = 128 / eb;
  // An empty K/V still needs valid maps for the kernel parameters: point them at Q.
  const void* kp = p->total_kv > 0 ? p->k : p->q;
  const void* vp = p->total_kv > 0 ? p->v : p->q;
  const long long kv_rows = p->total_kv > 0 ? p->total_kv : p->total_q;
  const bool no_kv = p->total_kv == 0;
  if ((rc = make_tmap_set(&l.tm_q, p->q, dt, eb, p->total_q, p->heads, p->head_dim, box_cols, p->q_strides[0],
                          p->q_strides[1])) != GDPA_OK)
    return rc;
  const int kvh_map = p->total_kv > 0 ? kv_heads : p->heads;
  if ((rc = make_tmap_set(&l.tm_k, kp, dt, eb, kv_rows, kvh_map, p->head_dim, box_cols,
                          no_kv ? p->q_strides[0] : p->k_strides[0], no_kv ? p->q_strides[1] : p->k_strides[1])) != GDPA_OK)
    return rc;
  if ((rc = make_tmap_set(&l.tm_v, vp, dt, eb, kv_rows, kvh_map, p->head_dim, box_cols,
                          no_kv ? p->q_strides[0] : p->v_strides[0], no_kv ? p->q_strides[1] : p->v_strides[1])) != GDPA_OK)
    return rc;
  // output, stored by 32-column x 32-row boxes from the activation warps' staging slabs (64-byte swizzled); the bf16
  // softmax kernel at head_dim 128 has room for 16-column slabs only (32-byte swizzled)
  const bool narrow_out = !fp8 && act == ACT_SOFTMAX && p->head_dim == 128;
  if ((rc = make_tmap(&l.tm_o.m, p->o, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p->total_q, p->heads, p->head_dim, narrow_out ? 16 : 32,
                      32, narrow_out ? 32 : 64)) != GDPA_OK)
    return rc;
  l.args.o = static_cast<__nv_bfloat16*>(p->o);
  l.args.q_off = p->q_offsets;
  l.args.kv_off = p->kv_offsets;
  l.args.off64 = p->offsets_are_int64;
  l.args.heads = p->heads;
  l.args.max_q = p->max_seq_len_q;
  l.args.max_kv = p->max_seq_len_kv;
  l.args.scale = p->qk_scale;
  l.args.sched = static_cast<const int*>(p->schedule);
  l.args.status = p->status;
  l.args.trace = g_trace.load();
  l.args.lse = (!fp8 && act == ACT_SOFTMAX) ? p->lse : nullptr;
  l.args.total_q = p->total_q;
  l.args.kv_heads = kv_heads;
  l.args.kv_group = p->heads / kv_heads;
  l.args.kv_index = p->kv_seq_index;
  l.args.window = p->window_plus_one > 0 ? p->window_plus_one - 1 : -1;
  l.args.residual = static_cast<const __nv_bfloat16*>(p->residual);
  l.args.row_sumsq = p->row_sumsq;
  l.args.total_kv = p->total_kv;
  l.args.kv_batch = (p->kv_seq_index != nullptr && p->kv_batch > 0) ? p->kv_batch : p->batch;
  l.args.q_scales = p->q_scales;
  l.args.k_scales = p->k_scales;
  l.args.v_scales = p->v_scales;
  l.args.q_blk_off = p->q_block_offsets;
  l.args.kv_blk_off = p->kv_block_offsets;
  l.grid = di.sm_count;
  l.stream = static_cast<cudaStream_t>(stream);
  if (p->timing_start_event != nullptr) cudaEventRecord(static_cast<cudaEvent_t>(p->timing_start_event), l.stream);
  if (fp8) {
    rc = launch_fwd_fp8(l, p->head_dim, act);
  } else if (act == ACT_SOFTMAX) {
    rc = launch_fwd_softmax_bf16(l, p->head_dim);
  } else {
    rc = launch_fwd_bf16(l, p->head_dim, act);
  }
  if (p->timing_stop_event != nullptr) cudaEventRecord(static_cast<cudaEvent_t>(p->timing_stop_event), l.stream);
  if (rc == 0) g_launches.fetch_add(1);
  return rc;
}

int gdpa_fwd(const GdpaFwdParams* p, gdpa_stream_t stream) { return fwd_common(p, stream, false); }

int gdpa_fwd_fp8(const GdpaFwdParams* p, gdpa_stream_t stream) { return fwd_common(p, stream, true); }

static int norm_args(const GdpaNormParams* p, NormArgs* a) {
  if (p == nullptr || p->struct_size != sizeof(GdpaNormParams)) return GDPA_ERR_BAD_ARG;
  if (p->rows < 0 || p->n <= 0 || p->n % 8 != 0 || !(p->eps >= 0.f)) return GDPA_ERR_BAD_ARG;
  if (p->rows > 0 && (p->x == nullptr || p->out == nullptr)) return GDPA_ERR_BAD_ARG;
  if ((p->row_mean == nullptr) != (p->row_rstd == nullptr) && p->row_mean != nullptr) return GDPA_ERR_BAD_ARG;
  const uintptr_t align = reinterpret_cast<uintptr_t>(p->x) | reinterpret_cast<uintptr_t>(p->out) |
                          reinterpret_cast<uintptr_t>(p->residual) | reinterpret_cast<uintptr_t>(p->weight) |
                          reinterpret_cast<uintptr_t>(p->bias);
  if ((align & 15u) != 0) return GDPA_ERR_MISALIGNED;
  a->x = static_cast<const __nv_bfloat16*>(p->x);
  a->out = static_cast<__nv_bfloat16*>(p->out);
  a->weight = p->weight;
  a->bias = p->bias;
  a->residual = static_cast<const __nv_bfloat16*>(p->residual);
  a->row_sumsq = p->row_sumsq;
  a->row_mean = p->row_mean;
  a->row_rstd = p->row_rstd;
  a->rows = p->rows;
  a->n = p->n;
  a->eps = p->eps;
  return GDPA_OK;
}

int gdpa_layernorm_rows(const GdpaNormParams* p, gdpa_stream_t stream) {
  NormArgs a;
  int rc = norm_args(p, &a);
  if (rc != GDPA_OK) return rc;
  if (a.row_mean == nullptr) a.row_rstd = nullptr;
  rc = launch_layernorm_rows(a, static_cast<cudaStream_t>(stream));
  if (rc == 0 && a.rows > 0) g_launches.fetch_add(1);
  return rc;
}

int gdpa_rmsnorm_rows(const GdpaNormParams* p, gdpa_stream_t stream) {
  NormArgs a;
  int rc = norm_args(p, &a);
  if (rc != GDPA_OK) return rc;
  rc = launch_rmsnorm_rows(a, static_cast<cudaStream_t>(stream));
  if (rc == 0 && a.rows > 0) g_launches.fetch_add(1);
  return rc;
}

int gdpa_quantize_fp8_blockwise(const GdpaQuantParams* p, gdpa_stream_t stream) {
  if (p == nullptr || p->struct_size != sizeof(GdpaQuantParams)) return GDPA_ERR_BAD_ARG;
  if (p->batch < 0 || p->total < 0 || p->heads <= 0 || p->head_dim <= 0 || p->head_dim % 4 != 0) return GDPA_ERR_BAD_ARG;
  if (p->offsets == nullptr || p->block_offsets == nullptr) return GDPA_ERR_BAD_ARG;
  if (p->total > 0 && (p->x == nullptr || p->x8 == nullptr || p->scales == nullptr)) return GDPA_ERR_BAD_ARG;
  if (p->scale_rows < p->total / kTile + p->batch) return GDPA_ERR_CAPACITY;
  if (p->heads > 65535) return GDPA_ERR_BAD_ARG;
  if (((reinterpret_cast<uintptr_t>(p->x8) | reinterpret_cast<uintptr_t>(p->x)) & 3u) != 0) return GDPA_ERR_MISALIGNED;
  QuantArgs a;
  a.x = p->x;
  a.x8 = p->x8;
  a.scales = p->scales;
  a.offsets = p->offsets;
  a.block_offsets = p->block_offsets;
  a.off64 = p->offsets_are_int64;
  a.batch = p->batch;
  a.heads = p->heads;
  a.head_dim = p->head_dim;
  a.max_blocks = p->total > 0 ? p->total / kTile + p->batch : 0;
  a.vec16 = p->head_dim % 16 == 0 && ((reinterpret_cast<uintptr_t>(p->x8) | reinterpret_cast<uintptr_t>(p->x)) & 15u) == 0;
  const int rc = launch_quant_fp8(a, p->in_is_fp32, static_cast<cudaStream_t>(stream));
  if (rc == 0) g_launches.fetch_add(a.max_blocks > 0 ? 2 : 1);
  return rc;
}

namespace {
int run_mxfp8(const GdpaMxParams* p, int quantize, gdpa_stream_t stream) {
  if (p == nullptr || p->struct_size != sizeof(GdpaMxParams)) return GDPA_ERR_BAD_ARG;
  if (p->batch < 0 || p->total < 0 || p->heads <= 0 || p->heads > 65535 || p->head_dim <= 0 || p->head_dim % 32 != 0 ||
      p->head_dim > 512)
    return GDPA_ERR_BAD_ARG;
  if (p->scale_axis != 0 && p->scale_axis != 1) return GDPA_ERR_BAD_ARG;
  if (p->offsets == nullptr || p->block_offsets == nullptr) return GDPA_ERR_BAD_ARG;
  if (p->total > 0 && (p->x == nullptr || p->x8 == nullptr || p->sf == nullptr)) return GDPA_ERR_BAD_ARG;
  if (p->sf_blocks < 0) return GDPA_ERR_BAD_ARG;
  // a batch of `total` rows has at least ceil(total / 128) blocks, whatever its sequence lengths
  if (p->sf_blocks < (p->total + kTile - 1) / kTile) return GDPA_ERR_CAPACITY;
  if (((reinterpret_cast<uintptr_t>(p->x8) | reinterpret_cast<uintptr_t>(p->x) | reinterpret_cast<uintptr_t>(p->sf)) & 15u) != 0)
    return GDPA_ERR_MISALIGNED;
  MxArgs a;
  a.x = p->x;
  a.x8 = p->x8;
  a.sf = static_cast<uint8_t*>(p->sf);
  a.offsets = p->offsets;
  a.block_offsets = p->block_offsets;
  a.off64 = p->offsets_are_int64;
  a.batch = p->batch;
  a.heads = p->heads;
  a.head_dim = p->head_dim;
  a.scale_axis = p->scale_axis;
  a.sf_blocks = p->sf_blocks;
  // the grid covers every block a batch of this size can have, clipped to the blocks the scale tensor holds
  a.max_blocks = p->total > 0 ? p->total / kTile + p->batch : 0;
  if (a.max_blocks > a.sf_blocks) a.max_blocks = a.sf_blocks;
  const int rc = launch_mxfp8(a, quantize, p->x_is_fp32, static_cast<cudaStream_t>(stream));
  if (rc == 0) g_launches.fetch_add(a.max_blocks > 0 ? 2 : 1);
  return rc;
}
}  // namespace

int gdpa_quantize_mxfp8(const GdpaMxParams* p, gdpa_stream_t stream) { return run_mxfp8(p, 1, stream); }
int gdpa_dequantize_mxfp8(const GdpaMxParams* p, gdpa_stream_t stream) { return run_mxfp8(p, 0, stream); }

int gdpa_norm_rows_bwd(const GdpaNormBwdParams* p, gdpa_stream_t stream) {
  if (p == nullptr || p->struct_size != sizeof(GdpaNormBwdParams)) return GDPA_ERR_BAD_ARG;
  if (p->mode < 0 || p->mode > 2 || p->rows < 0 || p->n <= 0 || p->n % 8 != 0) return GDPA_ERR_BAD_ARG;
  if (p->rows > 0 && (p->dy == nullptr || p->dx == nullptr)) return GDPA_ERR_BAD_ARG;
  if (p->rows > 0 && p->mode != 2 && (p->x == nullptr || p->row_rstd == nullptr)) return GDPA_ERR_BAD_ARG;
  if (p->rows > 0 && p->mode == 1 && p->row_mean == nullptr) return GDPA_ERR_BAD_ARG;
  if (p->mode == 2 && p->dy_add == nullptr) return GDPA_ERR_BAD_ARG;
  if ((p->dweight != nullptr || p->dbias != nullptr) && p->n > 4096) return GDPA_ERR_BAD_ARG;
  const uintptr_t align = reinterpret_cast<uintptr_t>(p->dy) | reinterpret_cast<uintptr_t>(p->dy_add) |
                          reinterpret_cast<uintptr_t>(p->x) | reinterpret_cast<uintptr_t>(p->dx) |
                          reinterpret_cast<uintptr_t>(p->weight);
  if ((align & 15u) != 0) return GDPA_ERR_MISALIGNED;
  NormBwdArgs a;
  a.dy = static_cast<const __nv_bfloat16*>(p->dy);
  a.dy_add = static_cast<const __nv_bfloat16*>(p->dy_add);
  a.x = static_cast<const __nv_bfloat16*>(p->x);
  a.dx = static_cast<__nv_bfloat16*>(p->dx);
  a.weight = p->mode == 2 ? nullptr : p->weight;
  a.row_mean = p->row_mean;
  a.row_rstd = p->row_rstd;
  a.dweight = p->dweight;
  a.dbias = p->dbias;
  a.rows = p->rows;
  a.n = p->n;
  const int rc = launch_norm_rows_bwd(a, p->mode, static_cast<cudaStream_t>(stream));
  if (rc == 0 && a.rows > 0) g_launches.fetch_add(1);
  return rc;
}

int gdpa_bwd(const GdpaBwdParams* p, gdpa_stream_t stream) {
  int rc = check_common(p);
  if (rc != GDPA_OK) return rc;
  if (p->schedule == nullptr) return GDPA_ERR_BAD_ARG;
  if (p->dtype != GDPA_DTYPE_BF16) return GDPA_ERR_UNSUPPORTED_DTYPE;
  const int act = act_class_from_id(p->activation);
  if (act < 0) return GDPA_ERR_UNSUPPORTED_ACT;
  if (act == ACT_SOFTMAX && (p->o == nullptr || p->lse == nullptr || p->dpsum == nullptr)) return GDPA_ERR_BAD_ARG;
  if (p->batch == 0 || (p->total_q == 0 && p->total_kv == 0)) return GDPA_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int kv_heads = p->kv_heads > 0 ? p->kv_heads : p->heads;
  if (p->heads % kv_heads != 0) return GDPA_ERR_BAD_ARG;
  const size_t elems_q = static_cast<size_t>(p->total_q) * p->heads * p->head_dim;
  const size_t elems_kv = static_cast<size_t>(p->total_kv) * kv_heads * p->head_dim;
  if (p->total_q == 0) {
    // No query rows: dK = dV = 0.
    if (p->dk == nullptr || p->dv == nullptr) return GDPA_ERR_BAD_ARG;
    if (cudaMemsetAsync(p->dk, 0, elems_kv * 2, st) != cudaSuccess) return GDPA_ERR_LAUNCH;
    if (cudaMemsetAsync(p->dv, 0, elems_kv * 2, st) != cudaSuccess) return GDPA_ERR_LAUNCH;
    return GDPA_OK;
  }
  if (p->q == nullptr || p->d_o == nullptr || p->dq == nullptr || p->dq_accum == nullptr) return GDPA_ERR_BAD_ARG;
  if (p->total_kv == 0) {
    // No key rows: dQ = 0.
    if (cudaMemsetAsync(p->dq, 0, elems_q * 2, st) != cudaSuccess) return GDPA_ERR_LAUNCH;
    return GDPA_OK;
  }
  if (p->k == nullptr || p->v == nullptr || p->dk == nullptr || p->dv == nullptr) return GDPA_ERR_BAD_ARG;
  if (((reinterpret_cast<uintptr_t>(p->dk) | reinterpret_cast<uintptr_t>(p->dv) | reinterpret_cast<uintptr_t>(p->dq)) & 15u) != 0)
    return GDPA_ERR_MISALIGNED;
  const bool pairs = (p->offsets_are_int64 & GDPA_OFFSETS_PAIRS) != 0;
  if (pairs && p->dkv_accum == nullptr) return GDPA_ERR_BAD_ARG;
  if (pairs && (reinterpret_cast<uintptr_t>(p->dkv_accum) & 15u) != 0) return GDPA_ERR_MISALIGNED;
  DeviceInfo di;
  rc = device_info(&di);
  if (rc != GDPA_OK) return rc;

  BwdLaunch l;
  std::memset(&l, 0, sizeof(l));
  const CUtensorMapDataType dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if ((rc = make_tmap_set(&l.tm_q, p->q, dt, 2, p->total_q, p->heads, p->head_dim, 64, p->q_strides[0], p->q_strides[1])) != GDPA_OK)
    return rc;
  if ((rc = make_tmap_set(&l.tm_k, p->k, dt, 2, p->total_kv, kv_heads, p->head_dim, 64, p->k_strides[0], p->k_strides[1])) != GDPA_OK)
    return rc;
  if ((rc = make_tmap_set(&l.tm_v, p->v, dt, 2, p->total_kv, kv_heads, p->head_dim, 64, p->v_strides[0], p->v_strides[1])) != GDPA_OK)
    return rc;
  if ((rc = make_tmap_set(&l.tm_do, p->d_o, dt, 2, p->total_q, p->heads, p->head_dim, 64)) != GDPA_OK) return rc;
  // fp32 dQ accumulator, reduced into by 32-column x 32-row boxes (128-byte swizzled staging).
  for (int i = 0; i < kDqTmapHeights; ++i)
    if ((rc = make_tmap(&l.tm_dq.m[i], p->dq_accum, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, p->total_q, p->heads, p->head_dim, 32,
                        32 >> i, 128)) != GDPA_OK)
      return rc;
  l.args.dk = static_cast<__nv_bfloat16*>(p->dk);
  l.args.dv = static_cast<__nv_bfloat16*>(p->dv);
  l.args.dq_accum = static_cast<float*>(p->dq_accum);
  l.args.q_off = p->q_offsets;
  l.args.kv_off = p->kv_offsets;
  l.args.off64 = p->offsets_are_int64;
  l.args.heads = kv_heads;
  l.args.q_heads = p->heads;
  l.args.kv_group = p->heads / kv_heads;
  l.args.window = p->window_plus_one > 0 ? p->window_plus_one - 1 : -1;
  l.args.max_q = p->max_seq_len_q;
  l.args.max_kv = p->max_seq_len_kv;
  l.args.scale = p->qk_scale;
  l.args.sched = static_cast<const int*>(p->schedule);
  l.args.status = p->status;
  l.args.trace = g_trace.load();
  l.args.lse = p->lse;
  l.args.dpsum = p->dpsum;
  l.args.total_q = p->total_q;
  l.args.dk_acc = pairs ? static_cast<float*>(p->dkv_accum) : nullptr;
  l.args.dv_acc = pairs ? static_cast<float*>(p->dkv_accum) + elems_kv : nullptr;
  l.args.total_kv = p->total_kv;
  l.grid = di.sm_count;
  l.stream = st;
  if (cudaMemsetAsync(p->dq_accum, 0, elems_q * sizeof(float), st) != cudaSuccess) return GDPA_ERR_LAUNCH;
  // the kernel hands work items out through a counter in the schedule header (word 3)
  if (cudaMemsetAsync(static_cast<int*>(const_cast<void*>(p->schedule)) + 3, 0, sizeof(int), st) != cudaSuccess) return GDPA_ERR_LAUNCH;
  if (pairs && cudaMemsetAsync(p->dkv_accum, 0, 2 * elems_kv * sizeof(float), st) != cudaSuccess) return GDPA_ERR_LAUNCH;
  if (act == ACT_SOFTMAX) {
    rc = launch_dpsum(static_cast<const __nv_bfloat16*>(p->d_o), static_cast<const __nv_bfloat16*>(p->o), p->dpsum,
                      p->total_q, p->heads, p->head_dim, st);
    if (rc != 0) return rc;
    g_launches.fetch_add(1);
  }
  if (p->timing_start_event != nullptr) cudaEventRecord(static_cast<cudaEvent_t>(p->timing_start_event), st);
  rc = launch_bwd_bf16(l, p->head_dim, act);
  if (p->timing_stop_event != nullptr) cudaEventRecord(static_cast<cudaEvent_t>(p->timing_stop_event), st);
  if (rc != 0) return rc;
  rc = launch_dq_convert(static_cast<const float*>(p->dq_accum), static_cast<__nv_bfloat16*>(p->dq),
                         static_cast<long long>(elems_q), st);
  if (rc == 0) g_launches.fetch_add(2);
  if (rc == 0 && pairs) {
    rc = launch_dq_convert(l.args.dk_acc, static_cast<__nv_bfloat16*>(p->dk), static_cast<long long>(elems_kv), st);
    if (rc == 0) rc = launch_dq_convert(l.args.dv_acc, static_cast<__nv_bfloat16*>(p->dv), static_cast<long long>(elems_kv), st);
    if (rc == 0) g_launches.fetch_add(2);
  }
  return rc;
}

}  // extern "C"
#pragma GCC visibility pop
