// GDPA forward for sm_100a:  O = cast(act(Q K^T) * scale) V  over a jagged batch.
//
// One persistent CTA per SM walks a longest-first list of work items (sequence, head, 256-row
// Q block).  A work item keeps two 128-row Q tiles resident in shared memory and streams the
// sequence's K and V tiles through a shared-memory ring.  Roles (20 warps, 96 registers each):
//
//   warps 0-7   activation of Q tile 0: S0 (TMEM) -> registers -> act * scale -> bf16 P0 (TMEM); two
//               warps per TMEM lane quarter, each owning 64 of the 128 S columns.  At the end of a work
//               item the same warps drain their half of O0 (TMEM -> bf16 -> a staging slab in shared memory ->
//               TMA store).
//   warps 8-15  the same for Q tile 1
//   warp  16    MMA issuer (one lane): S_s = Q_s K^T (tcgen05.mma, operands in shared memory),
//               O_s += P_s V (A operand P read from TMEM)
//   warp  17    TMA loader (lane 0 issues the copies, the warp zeroes the tails of ragged tiles);  warps 18-19 idle
//
// TMEM (512 columns): S0 [0,128)  S1 [128,256)  O0 [256,256+D)  O1 [384,384+D).  P_s (bf16, two
// values per column) of column half h overwrites the first 32 columns of that half's own S columns.
// While the warps of one Q tile run their activation the tensor cores run the other tile's P V and
// next Q K^T, so activation and MMA overlap.
//
// Variants of the same kernel: softmax with online rescaling (the two column halves exchange their row
// maxima through shared memory, keep partial row sums and write the log-sum-exp for the backward), and
// FP8 e4m3 operands with per-128-token-block scales.
//
// Tiles reach their consumers zero-padded (the loader zeroes the tail of a ragged tile in shared memory): rows of a
// tile beyond the end of its sequence are zeros, not the next sequence's tokens, as with the reference's per-sequence block loads
// (gdpa/triton/triton_generalized_dot_product_attention.py:270, :317).  So S columns beyond the KV length are
// exactly 0 and act(0) = 0 for every supported element-wise activation: no masking, and nothing a neighbouring
// sequence holds (Inf and NaN included) reaches this one.  Only the softmax (where a padded column must not count)
// and the band (window_size) test columns.  Q rows beyond the Q length are computed and never stored.
#include "gdpa_common.cuh"
#include "gdpa_launch.h"

namespace gdpa {

namespace {

// 20 warps: warps 0-7 / 8-15 activation of Q tile 0 / 1 (two warps per TMEM lane quarter, each owning 64
// of the 128 S columns; they also drain their half of O at the end of a work item), 16 MMA, 17 TMA,
// 18-19 idle.  A single warp cannot overlap its MUFU instructions with its FMA-pipe instructions, so two
// activation warps per SM sub-partition and Q tile halve the activation time.
constexpr int kFwdThreads = 20 * 32;
constexpr int kKvStages = 4;

// Barrier indices inside the shared barrier array.
enum FwdBar : int {
  B_Q_FULL = 0,                        // [2] TMA -> MMA
  B_Q_EMPTY = 2,                       // [2] MMA commit -> TMA
  B_KV_FULL = 4,                       // [kKvStages]
  B_KV_EMPTY = 4 + kKvStages,          // [kKvStages]
  B_S_FULL = 4 + 2 * kKvStages,        // [2] MMA commit -> activation group
  B_P_FULL = 6 + 2 * kKvStages,        // [2] activation group (128 arrivals) -> MMA
  B_O_FULL = 8 + 2 * kKvStages,        // [2] MMA commit -> epilogue
  B_O_EMPTY = 10 + 2 * kKvStages,      // [2] epilogue (128 arrivals) -> MMA
  B_L_FULL = 12 + 2 * kKvStages,       // [2] softmax: activation group -> epilogue (row sums)
  B_M_FULL = 14 + 2 * kKvStages,       // [2] softmax, wide layout: both column halves have published their row maxima
  B_LD_TMP = 16 + 2 * kKvStages,       // the loader's own: a ragged tile has landed and can have its padding rows zeroed
  B_COUNT = 17 + 2 * kKvStages
};

template <int D, int EB>
struct FwdSmem {
  static constexpr int kTileBytes = kTile * D * EB;      // one 128 x D tile of EB-byte elements
  static constexpr int kHalfBytes = kTile * 128;         // one swizzled box: 128 rows x 128 bytes
  static constexpr int kBoxes = D * EB / 128;            // boxes per tile
  static constexpr int kBoxCols = 128 / EB;              // elements per box row
  static constexpr int kQOff = 0;
  static constexpr int kKvOff = 2 * kTileBytes;
  static constexpr int kRowSumOff = kKvOff + kKvStages * kTileBytes;  // softmax: float[2 Q tiles][2 halves][128]
  static constexpr int kRowMaxOff = kRowSumOff + 4 * kTile * 4;       // softmax, wide: float[2 parity][2][2][128]
  // Output staging: one slab of 32 rows x 32 bf16 per activation warp, 64-byte swizzled, from which that warp's O
  // rows leave by TMA store.  Where shared memory has room the slabs follow the softmax arrays (kSeparate); with
  // 32 KB bf16 tiles (head_dim 128) it has not, the slabs lie over those arrays, and the softmax kernels of that
  // shape store O from registers instead.
  static constexpr int kOutSlabBytes = 32 * 64;
  static constexpr int kStatBytes = 12 * kTile * 4;
  static constexpr bool kSeparate = kRowSumOff + kStatBytes + 16 * kOutSlabBytes + 2048 <= 227 * 1024;
  static constexpr int kOutOff = kSeparate ? kRowSumOff + kStatBytes : kRowSumOff;
  // ... and there the softmax kernel has narrow slabs of its own behind its arrays: 32 rows x 16 bf16 (32-byte swizzle)
  static constexpr int kNarrowSlabBytes = 32 * 32;
  static constexpr int kNarrowOff = kRowSumOff + kStatBytes;
  static_assert(kStatBytes + 16 * kNarrowSlabBytes <= 16 * kOutSlabBytes, "the narrow slabs fit in the staging region");
  static constexpr int kBarOff = kOutOff + 16 * kOutSlabBytes;
  static_assert(16 * kOutSlabBytes >= kStatBytes, "the softmax arrays fit in the staging region");
  static constexpr int kTmemPtrOff = kBarOff + B_COUNT * 8;
  static constexpr int kAbortOff = kTmemPtrOff + 4;
  static constexpr int kBytes = kAbortOff + 4;
  static constexpr int kDynBytes = kBytes + 1024;        // slack to align the base to 1024 bytes
};

#define GDPA_WAIT(bar_idx, parity, role)                                                                   \
  if (!mbar_wait(bar_base + 8u * (bar_idx), (parity), abort_flag, a.status, ((bar_idx) << 8) | (role))) \
    goto role_done;
// The same for roles whose whole warp waits and then executes warp-collective tcgen05.ld / st: the
// decision to leave is taken by the warp as a whole, so no lane runs ahead into a collective instruction.
#define GDPA_WAIT_WARP(bar_idx, parity, role)                                                                       \
  {                                                                                                                 \
    const bool ok_ = mbar_wait(bar_base + 8u * (bar_idx), (parity), abort_flag, a.status, ((bar_idx) << 8) | (role)); \
    if (!__all_sync(0xffffffffu, ok_)) goto role_done;                                                              \
  }

// Sum of squares of eight bf16 values packed in a uint4.
__device__ __forceinline__ float sumsq_bf16x8(const uint4& v) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float lo = __uint_as_float(w[j] << 16), hi = __uint_as_float(w[j] & 0xffff0000u);
    s = fmaf(lo, lo, fmaf(hi, hi, s));
  }
  return s;
}

// FUSE = the epilogue of the norm pipeline (residual add, row sums of squares) compiled in: a template parameter
// rather than a run-time branch, so that the plain forward carries none of it.
template <int D, int ACT, bool FP8, bool FUSE>
__global__ void __launch_bounds__(kFwdThreads, 1)
gdpa_fwd_kernel(const __grid_constant__ TmapSet tm_q, const __grid_constant__ TmapSet tm_k,
                const __grid_constant__ TmapSet tm_v, const __grid_constant__ OutTmap tm_o, const FwdArgs a) {
  constexpr int EB = FP8 ? 1 : 2;
  constexpr bool kSoftmax = (ACT == ACT_SOFTMAX);
  // O leaves through shared memory and TMA stores (whole 64-byte row pieces per transaction); the bf16 softmax
  // kernel at head_dim 128 (its row statistics hold that shared memory) has narrower slabs of its own (32-byte row
  // pieces); the norm-pipeline epilogue has its own path through the wide slabs
  constexpr bool kNarrowOut = !FUSE && kSoftmax && !FwdSmem<D, FP8 ? 1 : 2>::kSeparate;
  constexpr bool kTmaOut = !FUSE && !kNarrowOut;
  constexpr int kActWarps = 16;
  constexpr int kMmaWarp = 16;
  constexpr int kLoadWarp = 17;
  constexpr uint32_t kStageThreads = 256u;  // threads that work on one Q tile's S / O
  using L = FwdSmem<D, EB>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + L::kBarOff;
  volatile uint32_t* tmem_ptr = reinterpret_cast<volatile uint32_t*>(smem + L::kTmemPtrOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kAbortOff);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < B_COUNT; ++i) {
      const bool many = (i >= B_P_FULL && i < B_P_FULL + 2) || (i >= B_O_EMPTY && i < B_O_EMPTY + 2) ||
                        (i >= B_L_FULL && i < B_L_FULL + 2);
      uint32_t cnt = many ? 128u : 1u;
      if ((i >= B_P_FULL && i < B_P_FULL + 2) || (i >= B_O_EMPTY && i < B_O_EMPTY + 2) ||
          (i >= B_L_FULL && i < B_L_FULL + 2) || (i >= B_M_FULL && i < B_M_FULL + 2))
        cnt = kStageThreads;
      mbar_init(bar_base + 8u * i, cnt);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_base + L::kTmemPtrOff, 512);
    tmem_relinquish();
  }
  if (warp == kLoadWarp && lane == 0) {
    tma_prefetch_desc(&tm_q.m[0]);
    tma_prefetch_desc(&tm_k.m[0]);
    tma_prefetch_desc(&tm_v.m[0]);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr;
  const int n_items = a.sched[0];
  const SeqLimits lim = {a.total_q, a.total_kv, a.kv_batch};

  // Operand format code: 1 = bf16 for kind::f16, 0 = e4m3 for kind::f8f6f4.
  constexpr uint32_t kFmt = FP8 ? 0u : 1u;
  // QK: A = Q tile (K-major), B = K tile (K-major), M = 128, N = 128.
  constexpr uint32_t kIdescQK = umma_idesc(kFmt, kFmt, 0, 0, kTile, kTile);
  // PV: A = P in TMEM, B = V tile (MN-major: head dim contiguous), M = 128, N = D.
  constexpr uint32_t kIdescPV = umma_idesc(kFmt, kFmt, 0, 1, kTile, D);

  if (warp >= kMmaWarp) {
   if (warp == kLoadWarp) {
    // ------------------------------------------------------------------ TMA loader
    // The whole warp walks the items; lane 0 issues the copies.  A full tile goes straight to its consumers' barrier.
    // A ragged tile (the last of its sequence) is fetched as the same full boxes onto the loader's own barrier -- its
    // rows past the sequence end are the next sequence's, or, past the tensor's end, the TMA unit's zero fill -- then
    // the warp overwrites those rows with zeros in shared memory and only then releases the tile: the consumers see a
    // zero-padded tile and nothing of the neighbour reaches them.
    {
      uint32_t kv_stage = 0, kv_phase = 0, q_phase = 0, tmp_phase = 0;  // bit s of q_phase = parity of Q stage s
      [[maybe_unused]] int ltr = 0;  // KV tiles before this item (trace rows)
      // one tile = L::kBoxes boxes of 128 rows x 128 bytes; `ragged`: onto the loader's barrier, then zero rows >= valid
      auto load_tile = [&](uint32_t dst_off, const CUtensorMap* tm, int full_bar, int y, int row0, int valid) -> bool {
        const bool ragged = valid < kTile;
        if (lane == 0) {
          const uint32_t bar = bar_base + 8u * (ragged ? B_LD_TMP : full_bar);
          mbar_arrive_expect_tx(bar, L::kTileBytes);
#pragma unroll
          for (int hf = 0; hf < L::kBoxes; ++hf)
            tma_load_3d(smem_base + dst_off + hf * L::kHalfBytes, tm, bar, hf * L::kBoxCols, y, row0);
        }
        if (ragged) {
          const bool ok = mbar_wait(bar_base + 8u * B_LD_TMP, tmp_phase, abort_flag, a.status, (B_LD_TMP << 8) | ST_ROLE_LOAD);
          if (!__all_sync(0xffffffffu, ok)) return false;
          tmp_phase ^= 1u;
          for (int bx = 0; bx < L::kBoxes; ++bx)
            for (int off = valid * 128 + lane * 16; off < L::kHalfBytes; off += 512)
              *reinterpret_cast<uint4*>(smem + dst_off + bx * L::kHalfBytes + off) = make_uint4(0, 0, 0, 0);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_base + 8u * full_bar);
        }
        return true;
      };
      WorkWalker walker(n_items);
      int idx;
      while (walker.next(idx)) {
        const Work w = load_work(a.sched, idx, a.q_off, a.kv_off, a.off64, a.max_q, a.max_kv, lim, a.kv_index);
        int j0, nkv;  // first KV tile and number of KV tiles this item visits
        fwd_kv_range(w, a.window, j0, nkv);
        if (nkv == 0) continue;
        const int q0 = w.blk * kFwdQBlock;
        const int nst = (w.lq - q0 > kTile) ? 2 : 1;
        const int q_row = static_cast<int>(w.q_start) + q0;
        const int kv_row = static_cast<int>(w.kv_start) + j0 * kTile;
        // Issue order Q0, K0, Q1, V0, K1, V1, ...
        for (int step = 0; step < 2 * nkv + 2; ++step) {
          if (step == 0 || step == 2) {
            const int s = step >> 1;
            if (s >= nst) continue;
            if (lane == 0) GDPA_TRACE(a, ltr * 32 + 24 + s * 2);
            GDPA_WAIT_WARP(B_Q_EMPTY + s, ((q_phase >> s) & 1u) ^ 1u, ST_ROLE_LOAD);
            if (lane == 0) GDPA_TRACE(a, ltr * 32 + 25 + s * 2);
            q_phase ^= 1u << s;
            if (!load_tile(L::kQOff + s * L::kTileBytes, &tm_q.m[0], B_Q_FULL + s, w.h, q_row + s * kTile,
                           w.lq - q0 - s * kTile))
              goto role_done;
          } else {
            const int t = (step == 1) ? 0 : step - 2;  // 0 = K0, 1 = V0, 2 = K1, ...
            const int j = t >> 1;
            GDPA_WAIT_WARP(B_KV_EMPTY + kv_stage, kv_phase ^ 1u, ST_ROLE_LOAD);
            if (!load_tile(L::kKvOff + kv_stage * L::kTileBytes, (t & 1) ? &tm_v.m[0] : &tm_k.m[0], B_KV_FULL + kv_stage,
                           w.h / a.kv_group, kv_row + j * kTile, w.lkv - (j0 + j) * kTile))
              goto role_done;
            if (++kv_stage == kKvStages) {
              kv_stage = 0;
              kv_phase ^= 1u;
            }
          }
        }
        ltr += nkv;
      }
    }
   } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      uint32_t kv_stage = 0, kv_phase = 0;
      // bit s of q_phase / p_phase / o_phase = parity of that barrier of Q tile s (registers, not arrays indexed by s)
      uint32_t q_phase = 0, p_phase = 0, o_phase = 0;
      int tr = 0;
      // Descriptors of stage 0 / ring slot 0, built once; per MMA only the low word moves.
      const uint64_t dq0 = umma_smem_desc_sw128(smem_base + L::kQOff, 16, 1024);
      const uint64_t dk0 = umma_smem_desc_sw128(smem_base + L::kKvOff, 16, 1024);
      const uint64_t dv0 = umma_smem_desc_sw128(smem_base + L::kKvOff, L::kHalfBytes, 1024);
      auto issue_qk = [&](int s, uint32_t k_stage) {
        const uint64_t da = umma_desc_advance(dq0, s * L::kTileBytes);
        const uint64_t db = umma_desc_advance(dk0, k_stage * L::kTileBytes);
        const uint32_t d_tmem = tmem_base + s * kTile;
        // one K slice = 32 bytes of the head dim (16 bf16 or 32 e4m3), four slices per 128-byte box
#pragma unroll
        for (int kk = 0; kk < D * EB / 32; ++kk) {
          const uint32_t off = (kk >> 2) * L::kHalfBytes + (kk & 3) * 32;
          if constexpr (FP8) umma_ss_f8(d_tmem, umma_desc_advance(da, off), umma_desc_advance(db, off), kIdescQK, kk > 0 ? 1u : 0u);
          else umma_ss_f16(d_tmem, umma_desc_advance(da, off), umma_desc_advance(db, off), kIdescQK, kk > 0 ? 1u : 0u);
        }
      };
      auto issue_pv = [&](int s, uint32_t v_stage, bool accumulate) {
        const uint64_t db = umma_desc_advance(dv0, v_stage * L::kTileBytes);
        const uint32_t d_tmem = tmem_base + 256 + s * kTile, a_tmem = tmem_base + s * kTile;
        // one K slice = 16 (bf16) or 32 (e4m3) KV rows of 128 bytes; P holds it in 8 TMEM columns
        constexpr int kRowsPerSlice = 32 / EB;
#pragma unroll
        for (int kk = 0; kk < kTile / kRowsPerSlice; ++kk) {
          const uint32_t acc = (accumulate || kk > 0) ? 1u : 0u;
          // the P slices of column half h sit at the start of that half's own S columns
          const uint32_t a_col = FP8 ? (kk >> 1) * 64 + (kk & 1) * 8 : (kk >> 2) * 64 + (kk & 3) * 8;
          if constexpr (FP8) umma_ts_f8(d_tmem, a_tmem + a_col, umma_desc_advance(db, kk * kRowsPerSlice * 128), kIdescPV, acc);
          else umma_ts_f16(d_tmem, a_tmem + a_col, umma_desc_advance(db, kk * kRowsPerSlice * 128), kIdescPV, acc);
        }
      };
      WorkWalker walker(n_items);
      int idx;
      while (walker.next(idx)) {
        const Work w = load_work(a.sched, idx, a.q_off, a.kv_off, a.off64, a.max_q, a.max_kv, lim, a.kv_index);
        int j0, nkv;
        fwd_kv_range(w, a.window, j0, nkv);
        if (nkv == 0) continue;
        const int nst = (w.lq - w.blk * kFwdQBlock > kTile) ? 2 : 1;
        // First S tiles: S_s = Q_s K_0^T.
        {
          const uint32_t k_stage = kv_stage;
          for (int s = 0; s < nst; ++s) {
            GDPA_WAIT(B_Q_FULL + s, (q_phase >> s) & 1u, ST_ROLE_MMA);
            q_phase ^= 1u << s;
            if (s == 0) GDPA_WAIT(B_KV_FULL + k_stage, kv_phase, ST_ROLE_MMA);
            tc_fence_after();
            issue_qk(s, k_stage);
            tc_commit(bar_base + 8u * (B_S_FULL + s));
            if (nkv == 1) tc_commit(bar_base + 8u * (B_Q_EMPTY + s));
          }
          tc_commit(bar_base + 8u * (B_KV_EMPTY + k_stage));
          if (++kv_stage == kKvStages) { kv_stage = 0; kv_phase ^= 1u; }
        }
        for (int j = 0; j < nkv; ++j) {
          const bool more = (j + 1 < nkv);
          const uint32_t v_stage = kv_stage, v_phase = kv_phase;
          if (++kv_stage == kKvStages) { kv_stage = 0; kv_phase ^= 1u; }
          const uint32_t k_stage = kv_stage, k_phase = kv_phase;  // K_{j+1}, valid if more
          if (more) { if (++kv_stage == kKvStages) { kv_stage = 0; kv_phase ^= 1u; } }
          GDPA_WAIT(B_KV_FULL + v_stage, v_phase, ST_ROLE_MMA);
          for (int s = 0; s < nst; ++s) {
            GDPA_TRACE(a, tr * 32 + 16 + s * 4 + 0);
            GDPA_WAIT(B_P_FULL + s, (p_phase >> s) & 1u, ST_ROLE_MMA);
            GDPA_TRACE(a, tr * 32 + 16 + s * 4 + 1);
            p_phase ^= 1u << s;
            if (j == 0) {
              GDPA_WAIT(B_O_EMPTY + s, ((o_phase >> s) & 1u) ^ 1u, ST_ROLE_MMA);
              o_phase ^= 1u << s;
            }
            tc_fence_after();
            issue_pv(s, v_stage, j > 0);
            if (more) {
              if (s == 0) {
                GDPA_WAIT(B_KV_FULL + k_stage, k_phase, ST_ROLE_MMA);
                tc_fence_after();
              }
              issue_qk(s, k_stage);
              tc_commit(bar_base + 8u * (B_S_FULL + s));
              if (j + 2 == nkv) tc_commit(bar_base + 8u * (B_Q_EMPTY + s));
            } else {
              tc_commit(bar_base + 8u * (B_O_FULL + s));
            }
            GDPA_TRACE(a, tr * 32 + 16 + s * 4 + 2);
          }
          ++tr;
          tc_commit(bar_base + 8u * (B_KV_EMPTY + v_stage));
          if (more) tc_commit(bar_base + 8u * (B_KV_EMPTY + k_stage));
        }
      }
    }
   }
  } else if (warp < kActWarps) {
    // ------------------------------------------------------------------ activation + epilogue
    const int s = warp >> 3;           // Q tile
    const int half = (warp >> 2) & 1;  // which 64 of the 128 S columns
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t s_tmem = tmem_base + lane_base + s * kTile + half * 64;
    const uint32_t o_tmem = tmem_base + lane_base + 256 + s * kTile + half * (D / 2);
    const float scale = a.scale, hscale = 0.5f * a.scale;
    uint32_t s_phase = 0, o_phase = 0;
    int tr = 0;
    WorkWalker walker(n_items);
    int idx;
    while (walker.next(idx)) {
      const Work w = load_work(a.sched, idx, a.q_off, a.kv_off, a.off64, a.max_q, a.max_kv, lim, a.kv_index);
      int j0, nkv;
      fwd_kv_range(w, a.window, j0, nkv);
      const int q0 = w.blk * kFwdQBlock;
      const int nst = (w.lq - q0 > kTile) ? 2 : 1;
      if (s >= nst) continue;
      const int qr = q0 + s * kTile + row;
      const bool row_valid = qr < w.lq;
      const long long o_elem = ((w.q_start + qr) * a.heads + w.h) * static_cast<long long>(D) + half * (D / 2);
      uint4* dst = reinterpret_cast<uint4*>(a.o + o_elem);
      // fused epilogue of the norm pipeline: x = O + residual, and the sum of x^2 over this thread's half row is
      // added to the row's entry of row_sumsq (the RMS norm over all heads is finished by a second kernel)
      const uint4* res = (FUSE && a.residual != nullptr) ? reinterpret_cast<const uint4*>(a.residual + o_elem) : nullptr;
      float* const row_sumsq = FUSE ? a.row_sumsq : nullptr;
      float ssq = 0.f;
      if (nkv == 0) {
        if (row_valid) {
#pragma unroll
          for (int i = 0; i < D / 16; ++i) {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (res != nullptr) {
              v = res[i];
              ssq += sumsq_bf16x8(v);
            }
            dst[i] = v;
          }
          if (row_sumsq != nullptr) atomicAdd(row_sumsq + w.q_start + qr, ssq);
        }
        continue;
      }
      float inv_l = 1.f;
      if constexpr (kSoftmax) {
        // ---- softmax, one row split over two warps (64 columns each): the halves publish their partial
        // row maxima through shared memory and an mbarrier, take the common maximum, and keep partial row
        // sums that the epilogue adds.  P = exp2(c S + bias - m); the O accumulator is rescaled only when
        // the running maximum m grew by more than kThr.  FP8: c carries the Q- and K-block scales and
        // bias = log2(V-block scale), so P contains the V scale and uses the whole e4m3 range; the row
        // sum divides it out again.
        constexpr float kThr = FP8 ? 1.f : 8.f;
        constexpr float kPScale = FP8 ? 128.f : 1.f;
        constexpr float kLog2e = 1.4426950408889634f;
        float* rowmax = reinterpret_cast<float*>(smem + L::kRowMaxOff);
        float* rowsum = reinterpret_cast<float*>(smem + L::kRowSumOff);
        float m_used = -INFINITY, row_sum = 0.f;
        float sq = 1.f;
        long long kv_blk0 = 0;
        if constexpr (FP8) {
          sq = a.q_scales[(load_offset(a.q_blk_off, w.b, a.off64) + w.blk * 2 + s) * a.heads + w.h];
          kv_blk0 = load_offset(a.kv_blk_off, w.kb, a.off64);
        }
        for (int j = 0; j < nkv; ++j) {
          // columns [clo, chi) of this warp's 64 take part: inside the KV length and inside the band
          const int kbase = (j0 + j) * kTile + half * 64;
          int clo = 0, chi = min(kTile, w.lkv - (j0 + j) * kTile) - half * 64;
          if (a.window >= 0) {
            clo = max(clo, qr - a.window - kbase);
            chi = min(chi, qr + a.window - kbase + 1);
          }
          float c = a.scale * kLog2e, bias = 0.f, inv_sv = 1.f;
          if constexpr (FP8) {
            const float sk = a.k_scales[(kv_blk0 + j0 + j) * a.kv_heads + w.h / a.kv_group];
            const float sv = a.v_scales[(kv_blk0 + j0 + j) * a.kv_heads + w.h / a.kv_group];
            c *= sq * sk;
            bias = log2f(sv);
            inv_sv = 1.f / sv;
          }
          GDPA_WAIT_WARP(B_S_FULL + s, s_phase, ST_ROLE_ACT);
          tc_fence_after();
          uint32_t ra[32], rb[32];
          // pass 1: partial row maximum of c * S over this warp's valid columns (chunk 1 in flight
          // while chunk 0 is scanned)
          float pmax = -INFINITY;
          tmem_ld32(s_tmem, ra);
#pragma unroll
          for (int ch = 0; ch < 2; ++ch) {
            uint32_t(&cur)[32] = ch ? rb : ra;
            tmem_wait_ld();
            tmem_regs_ready(cur);
            if (ch == 0) tmem_ld32(s_tmem + 32, rb);
            // a chunk wholly inside [clo, chi) for every row of the warp needs no predicates; without a band
            // the lower bound is 0
            if (__all_sync(0xffffffffu, clo <= ch * 32 && chi >= (ch + 1) * 32)) {
#pragma unroll
              for (int i = 0; i < 32; ++i) pmax = fmaxf(pmax, __uint_as_float(cur[i]) * c);
            } else if (a.window < 0) {
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                const float t = __uint_as_float(cur[i]) * c;
                pmax = (ch * 32 + i < chi) ? fmaxf(pmax, t) : pmax;
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                const float t = __uint_as_float(cur[i]) * c;
                pmax = (ch * 32 + i >= clo && ch * 32 + i < chi) ? fmaxf(pmax, t) : pmax;
              }
            }
          }
          float* slot = rowmax + (((s_phase * 2 + s) * 2) * kTile);
          slot[half * kTile + row] = pmax;
          mbar_arrive(bar_base + 8u * (B_M_FULL + s));
          GDPA_WAIT_WARP(B_M_FULL + s, s_phase, ST_ROLE_ACT);
          const float rmax = fmaxf(pmax, reinterpret_cast<volatile float*>(slot)[(half ^ 1) * kTile + row]);
          s_phase ^= 1u;
          const float m_new = fmaxf(m_used, rmax + bias);
          if (j == 0) {
            m_used = m_new;
          } else if (__any_sync(0xffffffffu, m_new > m_used + kThr)) {
            // a row that has not seen a key yet (both maxima -inf) keeps its zeros
            const float alpha = (m_new == -INFINITY) ? 1.f : ex2_approx(m_used - m_new);
            row_sum *= alpha;
            m_used = m_new;
#pragma unroll
            for (int ch = 0; ch < D / 64; ++ch) {
              uint32_t ro[32];
              tmem_ld32(o_tmem + ch * 32, ro);
              tmem_wait_ld();
              tmem_regs_ready(ro);
#pragma unroll
              for (int i = 0; i < 32; ++i) ro[i] = __float_as_uint(__uint_as_float(ro[i]) * alpha);
              tmem_st32(o_tmem + ch * 32, ro);
            }
          }
          // pass 2: reload the scores, P = exp2(c S + bias - m), partial row sum, quantise, store over
          // columns of this half that have been read
          const float off = (m_used == -INFINITY) ? 0.f : bias - m_used;  // a row may have seen no column yet
          float psum = 0.f;
          tmem_ld32(s_tmem, ra);
#pragma unroll
          for (int ch = 0; ch < 2; ++ch) {
            uint32_t(&cur)[32] = ch ? rb : ra;
            tmem_wait_ld();
            tmem_regs_ready(cur);
            if (ch == 0) tmem_ld32(s_tmem + 32, rb);
            // P of this chunk with the column test `inside`; three instantiations so that the common case (the
            // chunk wholly inside [clo, chi) for every row of the warp) carries no predicates at all
            auto emit = [&](auto inside) {
              auto prob = [&](int i) {
                const float e = ex2_approx(fmaf(__uint_as_float(cur[i]), c, off));
                const float p = inside(i) ? e : 0.f;
                psum += p;
                return p;
              };
              if constexpr (FP8) {
                uint32_t pk[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  const float p0 = prob(4 * i), p1 = prob(4 * i + 1), p2 = prob(4 * i + 2), p3 = prob(4 * i + 3);
                  pk[i] = pack_e4m3x4(p0 * kPScale, p1 * kPScale, p2 * kPScale, p3 * kPScale);
                }
                tmem_st8(s_tmem + ch * 8, pk);
              } else {
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                  const float p0 = prob(2 * i), p1 = prob(2 * i + 1);
                  pk[i] = pack_bf16x2(p0, p1);
                }
                tmem_st16(s_tmem + ch * 16, pk);
              }
            };
            if (__all_sync(0xffffffffu, clo <= ch * 32 && chi >= (ch + 1) * 32)) emit([](int) { return true; });
            else if (a.window < 0) emit([&](int i) { return ch * 32 + i < chi; });  // without a band the lower bound is 0
            else emit([&](int i) { return ch * 32 + i >= clo && ch * 32 + i < chi; });
          }
          row_sum = fmaf(psum, inv_sv, row_sum);
          tmem_wait_st();
          tc_fence_before();
          mbar_arrive(bar_base + 8u * (B_P_FULL + s));
        }
        // both halves publish their partial row sums; each then divides its half of O by the total
        rowsum[(s * 2 + half) * kTile + row] = row_sum * kPScale;
        mbar_arrive(bar_base + 8u * (B_L_FULL + s));
        GDPA_WAIT_WARP(B_L_FULL + s, o_phase, ST_ROLE_EPI);
        const float l_total = row_sum * kPScale + reinterpret_cast<volatile float*>(rowsum)[(s * 2 + (half ^ 1)) * kTile + row];
        inv_l = l_total > 0.f ? 1.f / l_total : 0.f;  // a row whose band holds no key gives zeros
        if constexpr (!FP8) {
          // log-sum-exp of the scaled scores in base 2, for the softmax backward (+inf for a row without
          // keys, which makes every P of that row zero there)
          if (half == 0 && row_valid && a.lse != nullptr)
            a.lse[static_cast<long long>(w.h) * a.total_q + w.q_start + qr] = l_total > 0.f ? m_used + log2f(l_total) : INFINITY;
        }
      }
      // FP8 with an element-wise activation: S = sq sk (Q8 K8^T) per tile, and P is stored as
      // e4m3(act(S) sv_j / sv_max) with sv_max the largest V-block scale the item visits, so that every KV tile
      // adds into the same accumulator; O = qk_scale sv_max sum_j P_j V8_j (the factor goes into the epilogue).
      float fp8_sq = 1.f, fp8_inv_svmax = 1.f;
      long long fp8_kv_blk0 = 0;
      if constexpr (FP8 && !kSoftmax) {
        const int hkv = w.h / a.kv_group;
        fp8_sq = a.q_scales[(load_offset(a.q_blk_off, w.b, a.off64) + w.blk * 2 + s) * a.heads + w.h];
        fp8_kv_blk0 = load_offset(a.kv_blk_off, w.kb, a.off64);
        float sv_max = 0.f;
        for (int j = 0; j < nkv; ++j) sv_max = fmaxf(sv_max, a.v_scales[(fp8_kv_blk0 + j0 + j) * a.kv_heads + hkv]);
        fp8_inv_svmax = sv_max > 0.f ? 1.f / sv_max : 0.f;
        inv_l = a.scale * sv_max;
      }
      for (int j = 0; !kSoftmax && j < nkv; ++j) {
        // columns [clo, chi) of this warp's 64 take part: inside the KV length and inside the band
        const int kbase = (j0 + j) * kTile + half * 64;
        int clo = 0, chi = min(kTile, w.lkv - (j0 + j) * kTile) - half * 64;
        if (a.window >= 0) {
          clo = max(clo, qr - a.window - kbase);
          chi = min(chi, qr + a.window - kbase + 1);
        }
        float fp8_xs = 1.f, fp8_g = 1.f;
        if constexpr (FP8 && !kSoftmax) {
          const int hkv = w.h / a.kv_group;
          fp8_xs = fp8_sq * a.k_scales[(fp8_kv_blk0 + j0 + j) * a.kv_heads + hkv];
          fp8_g = a.v_scales[(fp8_kv_blk0 + j0 + j) * a.kv_heads + hkv] * fp8_inv_svmax;
        }
        if ((threadIdx.x & 255) == 0) GDPA_TRACE(a, tr * 32 + s * 8 + 0);
        GDPA_WAIT_WARP(B_S_FULL + s, s_phase, ST_ROLE_ACT);
        s_phase ^= 1u;
        tc_fence_after();
        if ((threadIdx.x & 255) == 0) GDPA_TRACE(a, tr * 32 + s * 8 + 1);
        uint32_t ra[32], rb[32];
        tmem_ld32(s_tmem, ra);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t(&cur)[32] = c ? rb : ra;
          uint32_t pk[16];
          tmem_wait_ld();
          tmem_regs_ready(cur);
          if (c == 0) tmem_ld32(s_tmem + 32, rb);
          if constexpr (FP8) {
            // 32 values -> 32 e4m3 in 8 registers, over the first columns of this half
            uint32_t p8[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              float pv[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int c0 = c * 32 + 4 * i + e;
                const float x = (c0 >= clo && c0 < chi) ? __uint_as_float(cur[4 * i + e]) * fp8_xs : 0.f;
                pv[e] = act_scaled<ACT>(x, fp8_g, 0.5f * fp8_g);
              }
              p8[i] = pack_e4m3x4(pv[0], pv[1], pv[2], pv[3]);
            }
            tmem_st8(s_tmem + c * 8, p8);
            continue;
          }
          // without a band nothing is masked (the tile's padding is zero, act(0) = 0); with one, the unmasked path
          // is taken by the warp as a whole
          if (a.window < 0 || __all_sync(0xffffffffu, clo <= c * 32 && chi >= (c + 1) * 32)) {
#pragma unroll
            for (int i = 0; i < 16; ++i)
              pk[i] = act_scaled_pair_bf16<ACT>(__uint_as_float(cur[2 * i]), __uint_as_float(cur[2 * i + 1]), scale, hscale);
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int c0 = c * 32 + 2 * i;
              const float x0 = (c0 >= clo && c0 < chi) ? __uint_as_float(cur[2 * i]) : 0.f;
              const float x1 = (c0 + 1 >= clo && c0 + 1 < chi) ? __uint_as_float(cur[2 * i + 1]) : 0.f;
              pk[i] = act_scaled_pair_bf16<ACT>(x0, x1, scale, hscale);
            }
          }
          tmem_st16(s_tmem + c * 16, pk);  // over columns of this half that have been read
        }
        if ((threadIdx.x & 255) == 0) GDPA_TRACE(a, tr * 32 + s * 8 + 2);
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(bar_base + 8u * (B_P_FULL + s));
        if ((threadIdx.x & 255) == 0) GDPA_TRACE(a, tr * 32 + s * 8 + 3);
        ++tr;
      }
      // Norm pipeline, a warp whose 32 rows all belong to the sequence: its residual rows are fetched now, under the
      // wait for the last P V, as whole 64-byte row pieces (four neighbouring lanes per piece), and turned into one row
      // per thread through the staging slab below.  Piece p = i * 32 + lane: row p / 4, 16-byte chunk p % 4.
      [[maybe_unused]] uint4 rres[D / 64][4];
      [[maybe_unused]] const bool fuse_staged = FUSE && (w.lq - (qr - lane) >= 32);
      if constexpr (FUSE) {
        if (fuse_staged && a.residual != nullptr) {
#pragma unroll
          for (int c = 0; c < D / 64; ++c)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int p = i * 32 + lane;
              rres[c][i] = *reinterpret_cast<const uint4*>(
                  a.residual + ((w.q_start + (qr - lane) + (p >> 2)) * a.heads + w.h) * static_cast<long long>(D) + half * (D / 2) +
                  c * 32 + (p & 3) * 8);
            }
        }
      }
      // epilogue: this warp's half of the O tile, TMEM -> bf16 -> global
      GDPA_WAIT_WARP(B_O_FULL + s, o_phase, ST_ROLE_EPI);
      o_phase ^= 1u;
      tc_fence_after();
      if ((threadIdx.x & 255) == 0) GDPA_TRACE(a, (tr - 1) * 32 + s * 8 + 4);
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        uint32_t r[32];
        tmem_ld32(o_tmem + c * 32, r);
        tmem_wait_ld();
        tmem_regs_ready(r);
        if (c == D / 64 - 1) {
          tc_fence_before();
          mbar_arrive(bar_base + 8u * (B_O_EMPTY + s));
        }
        // rows of this warp's 32 inside the sequence (the same for every lane)
        const int slab_rows = w.lq - (qr - lane);
        if (kTmaOut && slab_rows >= 32) {
          // this warp's 32 rows x 32 columns: registers -> its slab (row = 64 bytes, 16-byte pieces XORed with bits 1-2
          // of the row, the 64-byte swizzle of the tensor map) -> one TMA store.  (A slab that the sequence ends in is
          // stored from registers below.)
          const uint32_t slab = smem_base + L::kOutOff + warp * L::kOutSlabBytes;
          uint8_t* const slab_row = smem + L::kOutOff + warp * L::kOutSlabBytes + lane * 64;
          if (lane == 0) tma_store_wait_read<0>();  // the store that read this slab last has finished reading it
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(r[8 * i + 0]) * inv_l, __uint_as_float(r[8 * i + 1]) * inv_l);
            v.y = pack_bf16x2(__uint_as_float(r[8 * i + 2]) * inv_l, __uint_as_float(r[8 * i + 3]) * inv_l);
            v.z = pack_bf16x2(__uint_as_float(r[8 * i + 4]) * inv_l, __uint_as_float(r[8 * i + 5]) * inv_l);
            v.w = pack_bf16x2(__uint_as_float(r[8 * i + 6]) * inv_l, __uint_as_float(r[8 * i + 7]) * inv_l);
            *reinterpret_cast<uint4*>(slab_row + ((i ^ ((lane >> 1) & 3)) << 4)) = v;
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_3d(&tm_o.m, slab, half * (D / 2) + c * 32, w.h, static_cast<int>(w.q_start) + qr);
            tma_store_commit();
          }
        } else if (kNarrowOut && slab_rows >= 32) {
          // the same with this variant's narrow slab: 16 columns at a time, 32-byte rows whose two 16-byte pieces swap
          // places in every other group of four rows (the tensor map's 32-byte swizzle)
          const uint32_t slab = smem_base + L::kNarrowOff + warp * L::kNarrowSlabBytes;
          uint8_t* const slab_row = smem + L::kNarrowOff + warp * L::kNarrowSlabBytes + lane * 32;
#pragma unroll
          for (int h2 = 0; h2 < 2; ++h2) {
            if (lane == 0) tma_store_wait_read<0>();
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              const int e = 16 * h2 + 8 * i;
              uint4 v;
              v.x = pack_bf16x2(__uint_as_float(r[e + 0]) * inv_l, __uint_as_float(r[e + 1]) * inv_l);
              v.y = pack_bf16x2(__uint_as_float(r[e + 2]) * inv_l, __uint_as_float(r[e + 3]) * inv_l);
              v.z = pack_bf16x2(__uint_as_float(r[e + 4]) * inv_l, __uint_as_float(r[e + 5]) * inv_l);
              v.w = pack_bf16x2(__uint_as_float(r[e + 6]) * inv_l, __uint_as_float(r[e + 7]) * inv_l);
              *reinterpret_cast<uint4*>(slab_row + ((i ^ ((lane >> 2) & 1)) << 4)) = v;
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_3d(&tm_o.m, slab, half * (D / 2) + c * 32 + h2 * 16, w.h, static_cast<int>(w.q_start) + qr);
              tma_store_commit();
            }
          }
        } else if (FUSE && fuse_staged) {
          // the norm pipeline's epilogue through the same slab: residual pieces in, one row per thread out, x = O + residual
          // and its bf16 back in, one TMA store
          const uint32_t slab = smem_base + L::kOutOff + warp * L::kOutSlabBytes;
          uint8_t* const slab_base = smem + L::kOutOff + warp * L::kOutSlabBytes;
          uint8_t* const slab_row = slab_base + lane * 64;
          if (lane == 0) tma_store_wait_read<0>();
          __syncwarp();
          uint4 own[4] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
          if (a.residual != nullptr) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int p = i * 32 + lane, prow = p >> 2;
              *reinterpret_cast<uint4*>(slab_base + prow * 64 + (((p & 3) ^ ((prow >> 1) & 3)) << 4)) = rres[c][i];
            }
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 4; ++i) own[i] = *reinterpret_cast<const uint4*>(slab_row + ((i ^ ((lane >> 1) & 3)) << 4));
            __syncwarp();
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t rw[4] = {own[i].x, own[i].y, own[i].z, own[i].w};
            uint32_t ow[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float x0 = fmaf(__uint_as_float(r[8 * i + 2 * j]), inv_l, __uint_as_float(rw[j] << 16));
              const float x1 = fmaf(__uint_as_float(r[8 * i + 2 * j + 1]), inv_l, __uint_as_float(rw[j] & 0xffff0000u));
              ssq = fmaf(x0, x0, fmaf(x1, x1, ssq));
              ow[j] = pack_bf16x2(x0, x1);
            }
            *reinterpret_cast<uint4*>(slab_row + ((i ^ ((lane >> 1) & 3)) << 4)) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_3d(&tm_o.m, slab, half * (D / 2) + c * 32, w.h, static_cast<int>(w.q_start) + qr);
            tma_store_commit();
          }
        } else if (row_valid) {
          if (!FUSE || (res == nullptr && row_sumsq == nullptr)) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 v;
              v.x = pack_bf16x2(__uint_as_float(r[8 * i + 0]) * inv_l, __uint_as_float(r[8 * i + 1]) * inv_l);
              v.y = pack_bf16x2(__uint_as_float(r[8 * i + 2]) * inv_l, __uint_as_float(r[8 * i + 3]) * inv_l);
              v.z = pack_bf16x2(__uint_as_float(r[8 * i + 4]) * inv_l, __uint_as_float(r[8 * i + 5]) * inv_l);
              v.w = pack_bf16x2(__uint_as_float(r[8 * i + 6]) * inv_l, __uint_as_float(r[8 * i + 7]) * inv_l);
              dst[c * 4 + i] = v;
            }
          } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 rv = make_uint4(0, 0, 0, 0);
              if (res != nullptr) rv = res[c * 4 + i];
              const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
              uint32_t ow[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float x0 = fmaf(__uint_as_float(r[8 * i + 2 * j]), inv_l, __uint_as_float(rw[j] << 16));
                const float x1 = fmaf(__uint_as_float(r[8 * i + 2 * j + 1]), inv_l, __uint_as_float(rw[j] & 0xffff0000u));
                ssq = fmaf(x0, x0, fmaf(x1, x1, ssq));
                ow[j] = pack_bf16x2(x0, x1);
              }
              dst[c * 4 + i] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
            }
          }
        }
      }
      if (row_sumsq != nullptr && row_valid) atomicAdd(row_sumsq + w.q_start + qr, ssq);
      if ((threadIdx.x & 255) == 0) GDPA_TRACE(a, (tr - 1) * 32 + s * 8 + 5);
    }
  }

role_done:
  // Teardown: everyone meets here (also after a wait ran out), then the allocating warp frees TMEM.
  __syncwarp();
  if (*abort_flag != 0) {
    // a wait ran out: give this CTA's TMA copies and MMAs in flight a bounded time (1 ms) to finish
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 1000000ull) {}
  }
  if ((kTmaOut || kNarrowOut || FUSE) && warp < kActWarps && lane == 0) tma_store_wait_all<0>();  // this warp's stores have left shared memory
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

#undef GDPA_WAIT
#undef GDPA_WAIT_WARP

template <int D, int ACT, bool FP8, bool FUSE>
int launch_fwd_fuse(const FwdLaunch& l) {
  using L = FwdSmem<D, FP8 ? 1 : 2>;
  auto kernel = gdpa_fwd_kernel<D, ACT, FP8, FUSE>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynBytes);
  if (e != cudaSuccess) return GDPA_ERR_LAUNCH_;
  kernel<<<l.grid, kFwdThreads, L::kDynBytes, l.stream>>>(l.tm_q, l.tm_k, l.tm_v, l.tm_o, l.args);
  return cudaGetLastError() == cudaSuccess ? 0 : GDPA_ERR_LAUNCH_;
}

template <int D, int ACT, bool FP8>
int launch_fwd_inst(const FwdLaunch& l) {
  // the fused epilogue exists for bf16 operands and the element-wise activations (the entry point refuses the rest)
  if constexpr (!FP8 && ACT != ACT_SOFTMAX) {
    if (l.args.residual != nullptr || l.args.row_sumsq != nullptr) return launch_fwd_fuse<D, ACT, FP8, true>(l);
  }
  return launch_fwd_fuse<D, ACT, FP8, false>(l);
}

template <int D>
int launch_fwd_d(const FwdLaunch& l, int act_class) {
  switch (act_class) {
    case ACT_RAW: return launch_fwd_inst<D, ACT_RAW, false>(l);
    case ACT_GELU_ERF: return launch_fwd_inst<D, ACT_GELU_ERF, false>(l);
    case ACT_GELU_TANH: return launch_fwd_inst<D, ACT_GELU_TANH, false>(l);
    case ACT_LEAKY_RELU: return launch_fwd_inst<D, ACT_LEAKY_RELU, false>(l);
    case ACT_RELU: return launch_fwd_inst<D, ACT_RELU, false>(l);
    case ACT_SILU: return launch_fwd_inst<D, ACT_SILU, false>(l);
    case ACT_HARDSWISH: return launch_fwd_inst<D, ACT_HARDSWISH, false>(l);
    case ACT_RELU_SQUARE: return launch_fwd_inst<D, ACT_RELU_SQUARE, false>(l);
    case ACT_SOFTMAX: return launch_fwd_inst<D, ACT_SOFTMAX, false>(l);
    default: return GDPA_ERR_UNSUPPORTED_ACT_;
  }
}

}  // namespace

int launch_fwd_bf16(const FwdLaunch& l, int head_dim, int act_class) {
  if (head_dim == 128) return launch_fwd_d<128>(l, act_class);
  if (head_dim == 64) return launch_fwd_d<64>(l, act_class);
  return GDPA_ERR_UNSUPPORTED_DIM_;
}

int launch_fwd_softmax_bf16(const FwdLaunch& l, int head_dim) { return launch_fwd_bf16(l, head_dim, ACT_SOFTMAX); }

// FP8 e4m3 operands: head_dim 128 only (a 64-byte row would need the 64-byte swizzle).
int launch_fwd_fp8(const FwdLaunch& l, int head_dim, int act_class) {
  if (head_dim != 128) return GDPA_ERR_UNSUPPORTED_DIM_;
  switch (act_class) {
    case ACT_RAW: return launch_fwd_inst<128, ACT_RAW, true>(l);
    case ACT_GELU_ERF: return launch_fwd_inst<128, ACT_GELU_ERF, true>(l);
    case ACT_GELU_TANH: return launch_fwd_inst<128, ACT_GELU_TANH, true>(l);
    case ACT_LEAKY_RELU: return launch_fwd_inst<128, ACT_LEAKY_RELU, true>(l);
    case ACT_RELU: return launch_fwd_inst<128, ACT_RELU, true>(l);
    case ACT_SILU: return launch_fwd_inst<128, ACT_SILU, true>(l);
    case ACT_HARDSWISH: return launch_fwd_inst<128, ACT_HARDSWISH, true>(l);
    case ACT_RELU_SQUARE: return launch_fwd_inst<128, ACT_RELU_SQUARE, true>(l);
    case ACT_SOFTMAX: return launch_fwd_inst<128, ACT_SOFTMAX, true>(l);
    default: return GDPA_ERR_UNSUPPORTED_ACT_;
  }
}

}  // namespace gdpa
