// GDPA backward for sm_100a: dQ, dK, dV of  O = cast(act(Q K^T) * scale) V  over a jagged batch,
// with S and P recomputed (nothing but Q, K, V, dO is read).
//
// One persistent CTA per SM takes work items (sequence, head, 128-row KV tile) from a longest-first list: its first
// by its index, the following ones from a counter in the list's header.  The item's K and V tiles stay resident in shared memory; the Q tiles of the sequence stream
// through a two-stage ring, the dO tiles through one stage (with grouped-query attention the item walks
// the Q tiles of every query head of its group; with a band only the Q tiles the band can reach).
// Per Q tile m the tensor cores run five contractions, with the KV rows as the M dimension of the
// "transposed" score tiles:
//
//   S^T  = K Q_m^T          (smem x smem)        -> TMEM [0,128)
//   dP^T = V dO_m^T         (smem x smem)        -> TMEM [128,256)
//   dV  += P^T dO_m         (P^T bf16 in TMEM, overwriting S^T)  -> TMEM [256,256+D)
//   dK  += dS^T Q_m         (dS^T bf16 in TMEM, overwriting dP^T)  -> TMEM [384,384+D)
//   dQ_m = dS K             (dS^T bf16 in smem, read MN-major)   -> TMEM [128,128+D), aliasing dP^T
//
// issued in the order S(m), dK(m-1), dQ(m-1), dP(m), dV(m) (dK reads dS^T from TMEM, where it sits
// over the dP^T columns that dQ then overwrites) so that the element-wise work of tile m
// (P = act(S) scale, act'(S) scale, dS = act' dP) overlaps the contractions of tile m-1 and m+1.
// dQ tiles are drained by a dedicated warpgroup (whole tile into registers, TMEM released, then each
// warp stages its 32 rows in shared memory) and added into an fp32 accumulator by TMA reduce-add; a
// second kernel rounds the accumulator to bf16.  Q rows of a ragged tile beyond the sequence are not touched: the
// reduce of such a tile covers exactly the rows of the sequence (smaller boxes).
//
// Softmax: P^T = 2^(c S^T - lse[q]) from the forward's log-sum-exp and dS = scale P (dP - dPsum[q]); the
// per-column statistics of a Q tile reach the element-wise warps through shared memory.
//
// Roles (16 warps, setmaxnreg 144 / 144 / 80): warps 0-3 dQ reduce, warps 4-11 element-wise (warp w:
// TMEM lanes 32*(w%4), score columns 64*((w-4)/4); at the end of a work item they write dK and dV out through their own
// part of the dS^T buffer), warp 12 MMA issuer (one lane), warp 13 TMA loader (lane 0 issues the copies and draws the
// work items, the warp zeroes the tails of ragged tiles), warps 14-15 idle.
// P^T of column half h is written over the first 32 columns of that half's own S^T columns
// ([64h, 64h+32)), so the two halves never touch each other's unread scores.
//
// Tiles reach their consumers zero-padded (the loader zeroes the tail of a ragged tile in shared memory): rows of a
// Q, dO, K or V tile beyond the end of its sequence are zeros, not the next sequence's tokens, as with the reference's per-sequence block loads
// (gdpa/triton/triton_generalized_dot_product_attention.py:1575-1600).  Score entries outside the sequence are
// therefore S = 0, P = act(0) = 0 and dS = act'(0) x dP with dP = 0: exact zeros with no masking anywhere, and nothing
// a neighbouring sequence holds (Inf and NaN included) reaches this one.  (Softmax: P = 2^(0 - lse) is not zero there,
// but every product it enters has a zero partner: the padded dO, K and V rows and the zero dPsum.)  Only the band
// (window_size) tests columns.
#include "gdpa_common.cuh"
#include "gdpa_launch.h"

namespace gdpa {

namespace {

constexpr int kBwdThreads = 16 * 32;
constexpr int kBwdMmaWarp = 12;
constexpr int kBwdLoadWarp = 13;
constexpr int kRegsCompute = 144;
constexpr int kRegsReduce = 144;
constexpr int kRegsOther = 80;
// setmaxnreg only moves registers inside the CTA's own allocation (512 threads x 128 registers): what the
// increases ask for must not exceed what the decreases free, or the increase never returns.
static_assert(8 * 32 * kRegsCompute + 4 * 32 * kRegsReduce + 4 * 32 * kRegsOther <= kBwdThreads * 128,
              "setmaxnreg budget exceeds the CTA's register allocation");
constexpr int kDqWarpSlabBytes = 32 * 32 * 4;  // one warp's staging slab: 32 rows x 32 fp32

enum BwdBar : int {
  BB_KV_FULL = 0,
  BB_KV_EMPTY = 1,
  BB_Q_FULL = 2,    // [2]
  BB_Q_EMPTY = 4,   // [2]
  BB_DO_FULL = 6,   // one stage
  BB_DO_EMPTY = 8,
  BB_S_FULL = 10,
  BB_P_FULL = 11,   // 256 arrivals
  BB_DP_FULL = 12,
  BB_DS_FULL = 13,  // 256 arrivals
  BB_DQ_FULL = 14,
  BB_DQ_EMPTY = 15, // 128 arrivals
  BB_DKV_FULL = 16,
  BB_DKV_EMPTY = 17,// 256 arrivals
  BB_ST_FULL = 18,  // 256 arrivals: softmax, the per-column statistics of a Q tile are in shared memory
  BB_LD_TMP = 19,   // the loader's own: a ragged tile has landed and can have its padding rows zeroed
  BB_WORK_FULL = 20,   // [kWorkSlots] the loader has published the index of a work item
  BB_WORK_EMPTY = 24,  // [kWorkSlots] 13 arrivals: the MMA thread, 8 element-wise and 4 drain warps have read it
  BB_COUNT = 28
};
constexpr int kWorkSlots = 4;


template <int D>
struct BwdSmem {
  static constexpr int kTileBytes = kTile * D * 2;
  static constexpr int kHalfBytes = kTile * 64 * 2;
  static constexpr int kKOff = 0;
  static constexpr int kVOff = kTileBytes;
  static constexpr int kQOff = 2 * kTileBytes;            // 2 stages
  static constexpr int kDoOff = 4 * kTileBytes;           // 1 stage
  static constexpr int kDsOff = 5 * kTileBytes;           // 128 x 128 bf16, two swizzled boxes
  static constexpr int kDsBytes = kTile * kTile * 2;
  static constexpr int kDqOff = kDsOff + kDsBytes;        // 2 staging slabs of 128 rows x 32 fp32
  static constexpr int kDqSlabBytes = kTile * 32 * 4;
  static constexpr int kBarOff = kDqOff + 2 * kDqSlabBytes;
  static constexpr int kTmemPtrOff = kBarOff + BB_COUNT * 8;
  static constexpr int kAbortOff = kTmemPtrOff + 4;
  static constexpr int kStatOff = (kAbortOff + 4 + 15) / 16 * 16;  // softmax: float lse[128], dpsum[2][128]
  static constexpr int kWorkOff = kStatOff + 3 * kTile * 4;  // int[kWorkSlots]: indices of the work items in flight
  static constexpr int kBytes = kWorkOff + kWorkSlots * 4;
  static constexpr int kDynBytes = kBytes + 1024;
};

// How dQ tiles leave the SM: staged in shared memory (per-warp 32 x 32 fp32 slabs) and added into the fp32
// accumulator by TMA reduce, which writes full 128-byte lines at L2; vector reductions straight from registers
// saturate the LSU / L2 atomic path.  The thread that issues the MMAs is on the critical path of every Q tile:
// whatever it executes between two waits delays the tensor pipe, so its per-tile state lives in registers (stage
// parities as bits of one word, operand descriptors built once per role) and full tiles take a path with no test
// per MMA.

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

// ACC: dK / dV tiles are added into fp32 accumulators instead of stored (K / V rows shared between sequences).
template <int D, int ACT, bool ACC>
__global__ void __launch_bounds__(kBwdThreads, 1)
gdpa_bwd_kernel(const __grid_constant__ TmapSet tm_q, const __grid_constant__ TmapSet tm_k,
                const __grid_constant__ TmapSet tm_v, const __grid_constant__ TmapSet tm_do,
                const __grid_constant__ DqTmapSet tm_dq, const BwdArgs a) {
  using L = BwdSmem<D>;
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
    for (int i = 0; i < BB_COUNT; ++i) {
      uint32_t cnt = 1;
      if (i == BB_P_FULL || i == BB_DS_FULL || i == BB_DKV_EMPTY || i == BB_ST_FULL) cnt = 256;
      if (i == BB_DQ_EMPTY) cnt = 128;
      if (i >= BB_WORK_EMPTY && i < BB_WORK_EMPTY + kWorkSlots) cnt = 13;
      mbar_init(bar_base + 8u * i, cnt);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == kBwdMmaWarp) {
    tmem_alloc(smem_base + L::kTmemPtrOff, 512);
    tmem_relinquish();
  }
  if (warp == kBwdLoadWarp && lane == 0) {
    tma_prefetch_desc(&tm_q.m[0]);
    tma_prefetch_desc(&tm_k.m[0]);
    tma_prefetch_desc(&tm_v.m[0]);
    tma_prefetch_desc(&tm_do.m[0]);
    tma_prefetch_desc(&tm_dq.m[0]);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr;
  const int n_items = a.sched[0];
  const SeqLimits lim = {a.total_q, a.total_kv, 0};
#ifdef GDPA_ENABLE_TRACE
  // every CTA's start and end time (ns) in the last 512 slots of the trace buffer
  if (a.trace != nullptr && threadIdx.x == 0 && blockIdx.x < 256) a.trace[kTraceSlots - 512 + 2 * blockIdx.x] = global_timer_ns();
#endif

  // Work items are handed out dynamically: the list is longest first, every CTA starts with item blockIdx.x and takes
  // its next one from a counter in the schedule header (word 3, zeroed by the entry point before the launch), so a
  // CTA that runs slower -- SMs differ in what memory latency they see, ragged tiles cost extra -- takes fewer items
  // instead of finishing late.  The loader warp draws the index and publishes it to the other roles through a small
  // ring in shared memory; -1 ends the walk.
  const uint32_t work_ring = smem_base + L::kWorkOff;
  int* const work_counter = const_cast<int*>(a.sched) + 3;
  uint32_t work_pos = 0;  // items this role has taken: ring slot = work_pos % kWorkSlots, parity = (work_pos / kWorkSlots) & 1
  // Consumer side: the index of this role's next work item, -1 at the end of the list, -2 if the wait ran out.
  // `warp_wide`: called by a whole warp, whose lane 0 releases the slot.  (A function that is not inlined would keep
  // this out of the roles' code, but register allocation fails for calls in a kernel with fixed register counts.)
  auto take_work_item = [&](int role, bool warp_wide) -> int {
    const uint32_t slot = work_pos % kWorkSlots, parity = (work_pos / kWorkSlots) & 1u;
    ++work_pos;
    bool ok = mbar_wait(bar_base + 8u * (BB_WORK_FULL + slot), parity, abort_flag, a.status, ((BB_WORK_FULL + slot) << 8) | role);
    if (warp_wide) ok = __all_sync(0xffffffffu, ok);
    if (!ok) return -2;
    int idx;
    asm volatile("ld.volatile.shared.s32 %0, [%1];" : "=r"(idx) : "r"(work_ring + 4u * slot) : "memory");
    if (warp_wide) __syncwarp();
    if (!warp_wide || lane == 0) mbar_arrive(bar_base + 8u * (BB_WORK_EMPTY + slot));
    return idx;
  };

  constexpr uint32_t kColS = 0, kColDP = 128, kColDV = 256, kColDK = 384;
  // S^T / dP^T: A and B both K-major (head dim contiguous), M = N = 128.
  constexpr uint32_t kIdescKK = umma_idesc(1, 1, 0, 0, kTile, kTile);
  // dV, dK: A K-major (TMEM or smem), B MN-major (dO / Q rows hold the head dim), N = D.
  constexpr uint32_t kIdescKM = umma_idesc(1, 1, 0, 1, kTile, D);
  // dQ: A = dS read MN-major (Q index contiguous in smem), B = K tile MN-major, N = D.
  constexpr uint32_t kIdescMM = umma_idesc(1, 1, 1, 1, kTile, D);

  if (warp >= 12) {
    setmaxnreg_dec<kRegsOther>();
    if (warp == kBwdLoadWarp) {
      // ---------------------------------------------------------------- TMA loader
      // The whole warp walks the items; lane 0 issues the copies.  A full tile goes straight to its consumers'
      // barrier.  A ragged tile (the last of its sequence) is fetched as the same full boxes onto the loader's own
      // barrier -- its rows past the sequence end are the next sequence's, or, past the tensor's end, the TMA unit's
      // zero fill -- then the warp overwrites those rows with zeros in shared memory and only then releases the tile:
      // the consumers see a zero-padded tile, nothing of the neighbour reaches them, and the tile costs D / 64 copies
      // plus at most 16 KB of zero stores per box (decomposing it into boxes of its valid rows took up to eleven copies
      // per box, ~250 cycles each to issue).
      {
        uint32_t kv_phase = 0, q_phase = 0 /* bit st = parity of Q stage st */, do_phase = 0, st = 0, tmp_phase = 0;
        [[maybe_unused]] int ltr = 0;  // trace: Q tiles of the items before this one
        // zero rows [valid, 128) of `nbox` consecutive boxes at `base` (a box's rows are contiguous 128-byte lines)
        auto zero_tail = [&](uint8_t* base, int nbox, int valid) {
          for (int bx = 0; bx < nbox; ++bx)
            for (int off = valid * 128 + lane * 16; off < L::kHalfBytes; off += 512)
              *reinterpret_cast<uint4*>(base + bx * L::kHalfBytes + off) = make_uint4(0, 0, 0, 0);
          fence_proxy_async_smem();
          __syncwarp();
        };
        // producer side of the work ring: the slot must have been read by every consumer of its previous use
        auto draw_item = [&](int& idx) -> bool {
          const uint32_t slot = work_pos % kWorkSlots, parity = (work_pos / kWorkSlots) & 1u;
          const bool ok = mbar_wait(bar_base + 8u * (BB_WORK_EMPTY + slot), parity ^ 1u, abort_flag, a.status,
                                    ((BB_WORK_EMPTY + slot) << 8) | ST_ROLE_LOAD);
          if (!__all_sync(0xffffffffu, ok)) return false;
          int i = 0;
          if (lane == 0) {
            i = work_pos == 0 ? static_cast<int>(blockIdx.x) : static_cast<int>(gridDim.x) + atomicAdd(work_counter, 1);
            if (i >= n_items) i = -1;
            asm volatile("st.volatile.shared.s32 [%0], %1;" ::"r"(work_ring + 4u * slot), "r"(i) : "memory");
            mbar_arrive(bar_base + 8u * (BB_WORK_FULL + slot));
          }
          idx = __shfl_sync(0xffffffffu, i, 0);
          ++work_pos;
          return true;
        };
        int idx, idx_next;
        if (!draw_item(idx)) goto role_done;
        for (; idx >= 0; idx = idx_next) {
          // the next index is drawn now, a whole work item ahead of its use
          if (!draw_item(idx_next)) goto role_done;
          const Work w = load_work(a.sched, idx, a.q_off, a.kv_off, a.off64, a.max_q, a.max_kv, lim);
          int m0, nq1;  // first Q tile and number of Q tiles of one query head this item visits
          bwd_q_range(w, a.window, m0, nq1);
          const int nq = nq1 * a.kv_group;  // ... over every query head of this K / V head's group
          if (nq == 0) continue;
          const int kv_row = static_cast<int>(w.kv_start) + w.blk * kTile;
          const int q_row = static_cast<int>(w.q_start);
          if (lane == 0) GDPA_TRACE(a, ltr * 32 + 20);
          GDPA_WAIT_WARP(BB_KV_EMPTY, kv_phase ^ 1u, ST_ROLE_LOAD);
          if (lane == 0) GDPA_TRACE(a, ltr * 32 + 21);
          kv_phase ^= 1u;
          const int kv_valid = w.lkv - w.blk * kTile;  // rows of this KV tile that belong to the sequence
          {
            const bool ragged = kv_valid < kTile;
            if (lane == 0) {
              const uint32_t bar = bar_base + 8u * (ragged ? BB_LD_TMP : BB_KV_FULL);
              mbar_arrive_expect_tx(bar, 2 * L::kTileBytes);
#pragma unroll
              for (int hf = 0; hf < D / 64; ++hf)
                tma_load_3d(smem_base + L::kKOff + hf * L::kHalfBytes, &tm_k.m[0], bar, hf * 64, w.h, kv_row);
#pragma unroll
              for (int hf = 0; hf < D / 64; ++hf)
                tma_load_3d(smem_base + L::kVOff + hf * L::kHalfBytes, &tm_v.m[0], bar, hf * 64, w.h, kv_row);
            }
            if (ragged) {
              GDPA_WAIT_WARP(BB_LD_TMP, tmp_phase, ST_ROLE_LOAD);
              tmp_phase ^= 1u;
              zero_tail(smem + L::kKOff, 2 * (D / 64), kv_valid);  // K and V are neighbours in shared memory
              if (lane == 0) mbar_arrive(bar_base + 8u * BB_KV_FULL);
            }
          }
          if (lane == 0) GDPA_TRACE(a, ltr * 32 + 22);
          ltr += nq;
          for (int m = 0; m < nq; ++m) {
            const int hq = w.h * a.kv_group + m / nq1, mm = m0 + m % nq1;
            const int q_valid = w.lq - mm * kTile;  // rows of this Q / dO tile that belong to the sequence
            const bool ragged = q_valid < kTile;
            GDPA_WAIT_WARP(BB_Q_EMPTY + st, ((q_phase >> st) & 1u) ^ 1u, ST_ROLE_LOAD);
            q_phase ^= 1u << st;
            if (lane == 0) {
              const uint32_t bar = bar_base + 8u * (ragged ? BB_LD_TMP : BB_Q_FULL + st);
              mbar_arrive_expect_tx(bar, L::kTileBytes);
#pragma unroll
              for (int hf = 0; hf < D / 64; ++hf)
                tma_load_3d(smem_base + L::kQOff + st * L::kTileBytes + hf * L::kHalfBytes, &tm_q.m[0], bar, hf * 64, hq,
                            q_row + mm * kTile);
            }
            if (ragged) {
              GDPA_WAIT_WARP(BB_LD_TMP, tmp_phase, ST_ROLE_LOAD);
              tmp_phase ^= 1u;
              zero_tail(smem + L::kQOff + st * L::kTileBytes, D / 64, q_valid);
              if (lane == 0) mbar_arrive(bar_base + 8u * (BB_Q_FULL + st));
            }
            GDPA_WAIT_WARP(BB_DO_EMPTY, do_phase ^ 1u, ST_ROLE_LOAD);
            do_phase ^= 1u;
            if (lane == 0) {
              const uint32_t bar = bar_base + 8u * (ragged ? BB_LD_TMP : BB_DO_FULL);
              mbar_arrive_expect_tx(bar, L::kTileBytes);
#pragma unroll
              for (int hf = 0; hf < D / 64; ++hf)
                tma_load_3d(smem_base + L::kDoOff + hf * L::kHalfBytes, &tm_do.m[0], bar, hf * 64, hq, q_row + mm * kTile);
            }
            if (ragged) {
              GDPA_WAIT_WARP(BB_LD_TMP, tmp_phase, ST_ROLE_LOAD);
              tmp_phase ^= 1u;
              zero_tail(smem + L::kDoOff, D / 64, q_valid);
              if (lane == 0) mbar_arrive(bar_base + 8u * BB_DO_FULL);
            }
            st ^= 1u;
          }
        }
      }
    } else if (warp == kBwdMmaWarp) {
      // ---------------------------------------------------------------- MMA issuer
      if (lane == 0) {
        uint32_t kv_phase = 0, q_phase = 0 /* bit st = parity of Q stage st */, do_phase = 0, st = 0;
        uint32_t p_phase = 0, ds_phase = 0, dqe_phase = 0, dkve_phase = 0;
        int tr = 0;  // trace: Q tiles seen so far (slot layout: tr * 32 + event, events 0-7 MMA, 8-12 element-wise, 13-16 reduce)
        const uint32_t sK = smem_base + L::kKOff, sV = smem_base + L::kVOff, sDs = smem_base + L::kDsOff;
        // Descriptors of the operand buffers, built once; per MMA only the start address moves.
        const uint64_t dK_k = umma_smem_desc_sw128(sK, 16, 1024), dV_k = umma_smem_desc_sw128(sV, 16, 1024);
        const uint64_t dK_mn = umma_smem_desc_sw128(sK, L::kHalfBytes, 1024), dDs_mn = umma_smem_desc_sw128(sDs, L::kHalfBytes, 1024);
        const uint64_t dQ0_k = umma_smem_desc_sw128(smem_base + L::kQOff, 16, 1024);
        const uint64_t dQ0_mn = umma_smem_desc_sw128(smem_base + L::kQOff, L::kHalfBytes, 1024);
        const uint64_t dDo_k = umma_smem_desc_sw128(smem_base + L::kDoOff, 16, 1024);
        const uint64_t dDo_mn = umma_smem_desc_sw128(smem_base + L::kDoOff, L::kHalfBytes, 1024);
        // A, B K-major over the head dim: D / 16 slices.
        auto mma_kmajor_pair = [&](uint32_t d_col, uint64_t a_desc, uint64_t b_desc) {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t off = (kk >> 2) * L::kHalfBytes + (kk & 3) * 32;
            umma_ss_f16(tmem_base + d_col, umma_desc_advance(a_desc, off), umma_desc_advance(b_desc, off), kIdescKK,
                        kk > 0 ? 1u : 0u);
          }
        };
        int idx;
        while (true) {
          idx = take_work_item(ST_ROLE_MMA, false);
          if (idx == -2) goto role_done;
          if (idx < 0) break;
          const Work w = load_work(a.sched, idx, a.q_off, a.kv_off, a.off64, a.max_q, a.max_kv, lim);
          int m0, nq1;
          bwd_q_range(w, a.window, m0, nq1);
          const int nq = nq1 * a.kv_group;
          if (nq == 0) continue;
          GDPA_WAIT(BB_KV_FULL, kv_phase, ST_ROLE_MMA);
          kv_phase ^= 1u;
          for (int m = 0; m <= nq; ++m) {
            const uint64_t dQ_k = umma_desc_advance(dQ0_k, st * L::kTileBytes);
            if (m < nq) {
              GDPA_TRACE(a, tr * 32 + 0);
              GDPA_WAIT(BB_Q_FULL + st, (q_phase >> st) & 1u, ST_ROLE_MMA);
              q_phase ^= 1u << st;
              tc_fence_after();
              mma_kmajor_pair(kColS, dK_k, dQ_k);  // S^T = K Q_m^T
              tc_commit(bar_base + 8u * BB_S_FULL);
              GDPA_TRACE(a, tr * 32 + 1);
            }
            if (m > 0) {
              const uint32_t pst = st ^ 1u;
              const uint64_t dQp_mn = umma_desc_advance(dQ0_mn, pst * L::kTileBytes);
              GDPA_WAIT(BB_DS_FULL, ds_phase, ST_ROLE_MMA);
              ds_phase ^= 1u;
              tc_fence_after();
              GDPA_TRACE(a, tr * 32 + 2);
              // dK += dS^T Q_{m-1} : A = dS^T (bf16 in TMEM over the dP^T columns this half has read),
              // B = Q tile MN-major.  Issued before dQ, which overwrites those columns.
#pragma unroll
              for (int kk = 0; kk < kTile / 16; ++kk)
                umma_ts_f16(tmem_base + kColDK, tmem_base + kColDP + (kk >> 2) * 64 + (kk & 3) * 8,
                            umma_desc_advance(dQp_mn, kk * 2048), kIdescKM,
                            (m > 1 || kk > 0) ? 1u : 0u);
              // dQ_{m-1} = dS K : A = dS^T tile in shared memory read MN-major, B = K tile MN-major
#pragma unroll
              for (int kk = 0; kk < kTile / 16; ++kk)
                umma_ss_f16(tmem_base + kColDP, umma_desc_advance(dDs_mn, kk * 2048), umma_desc_advance(dK_mn, kk * 2048),
                            kIdescMM, kk > 0 ? 1u : 0u);
              tc_commit(bar_base + 8u * BB_DQ_FULL);
              tc_commit(bar_base + 8u * (BB_Q_EMPTY + pst));
              GDPA_TRACE(a, tr * 32 + 3);
            }
            if (m < nq) {
              GDPA_WAIT(BB_DO_FULL, do_phase, ST_ROLE_MMA);
              do_phase ^= 1u;
              GDPA_WAIT(BB_DQ_EMPTY, dqe_phase ^ 1u, ST_ROLE_MMA);
              dqe_phase ^= 1u;
              tc_fence_after();
              GDPA_TRACE(a, tr * 32 + 4);
              mma_kmajor_pair(kColDP, dV_k, dDo_k);  // dP^T = V dO_m^T
              tc_commit(bar_base + 8u * BB_DP_FULL);
              GDPA_TRACE(a, tr * 32 + 5);
              GDPA_WAIT(BB_P_FULL, p_phase, ST_ROLE_MMA);
              p_phase ^= 1u;
              GDPA_TRACE(a, tr * 32 + 6);
              if (m == 0) {
                GDPA_WAIT(BB_DKV_EMPTY, dkve_phase ^ 1u, ST_ROLE_MMA);
                dkve_phase ^= 1u;
              }
              tc_fence_after();
              // dV += P^T dO_m : A = P^T (bf16 in TMEM over the S^T columns), B = dO tile MN-major
#pragma unroll
              for (int kk = 0; kk < kTile / 16; ++kk)
                umma_ts_f16(tmem_base + kColDV, tmem_base + kColS + (kk >> 2) * 64 + (kk & 3) * 8,
                            umma_desc_advance(dDo_mn, kk * 2048), kIdescKM,
                            (m > 0 || kk > 0) ? 1u : 0u);
              tc_commit(bar_base + 8u * BB_DO_EMPTY);
              GDPA_TRACE(a, tr * 32 + 7);
              ++tr;
              st ^= 1u;
            }
          }
          tc_commit(bar_base + 8u * BB_DKV_FULL);
          tc_commit(bar_base + 8u * BB_KV_EMPTY);
        }
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ element-wise warps
    setmaxnreg_inc<kRegsCompute>();
    const int quarter = warp & 3;
    const int half = (warp - 4) >> 2;
    const int row = quarter * 32 + lane;  // KV row of the tile == TMEM lane
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t tS = tmem_base + lane_base + kColS, tDP = tmem_base + lane_base + kColDP;
    const float scale = a.scale, hscale = 0.5f * a.scale;
    uint8_t* sds_row = smem + L::kDsOff + half * L::kHalfBytes + row * 128;
    uint32_t s_phase = 0, dp_phase = 0, dkv_phase = 0, st_phase = 0;
    int tr = 0;
    const bool tracer = (threadIdx.x == 128);
    constexpr bool kSoftmax = (ACT == ACT_SOFTMAX);
    float* stat_lse = reinterpret_cast<float*>(smem + L::kStatOff);
    float* stat_dps = stat_lse + kTile;  // two buffers, by parity of the Q tile
    const int ew_tid = threadIdx.x - 128;  // 0..255 among the element-wise threads
    const float c2 = a.scale * 1.4426950408889634f;
    int idx;
    while (true) {
      idx = take_work_item(ST_ROLE_ACT, true);
      if (idx == -2) goto role_done;
      if (idx < 0) break;
      const Work w = load_work(a.sched, idx, a.q_off, a.kv_off, a.off64, a.max_q, a.max_kv, lim);
      int m0, nq1;
      bwd_q_range(w, a.window, m0, nq1);
      const int nq = nq1 * a.kv_group;
      const int kv_local = w.blk * kTile + row;
      const bool row_valid = kv_local < w.lkv;
      __nv_bfloat16* dk_row = a.dk + ((w.kv_start + kv_local) * a.heads + w.h) * static_cast<long long>(D);
      __nv_bfloat16* dv_row = a.dv + ((w.kv_start + kv_local) * a.heads + w.h) * static_cast<long long>(D);
      if (nq == 0) {
        if (row_valid) {
#pragma unroll
          for (int i = 0; i < D / 16; ++i) {
            reinterpret_cast<uint4*>(dk_row)[half * (D / 16) + i] = make_uint4(0, 0, 0, 0);
            reinterpret_cast<uint4*>(dv_row)[half * (D / 16) + i] = make_uint4(0, 0, 0, 0);
          }
        }
        continue;
      }
      for (int m = 0; m < nq; ++m) {
        const int hq = w.h * a.kv_group + m / nq1, mm = m0 + m % nq1;
        // Without a band nothing is masked: the tiles are zero-padded, so score entries outside the sequence are
        // act(0) = 0 and their dS is act'(0) x 0 = 0.  With a band, columns [clo, chi) of the tile take part for this
        // thread's KV row, and the unmasked path is taken by the warp as a whole.
        int clo = 0, chi = row_valid ? min(kTile, w.lq - mm * kTile) : 0;
        bool full = true;
        if (a.window >= 0) {
          clo = max(clo, kv_local - a.window - mm * kTile);
          chi = min(chi, kv_local + a.window - mm * kTile + 1);
          full = __all_sync(0xffffffffu, clo <= 0 && chi >= kTile);
        }
        uint64_t g2[32];  // act'(S) * scale of this thread's 64 columns, as packed pairs
        uint32_t ra[32], rb[32];
        if (tracer) GDPA_TRACE(a, tr * 32 + 8);
        float stat = 0.f;
        if constexpr (kSoftmax) {
          // this thread's share of the Q tile's column statistics: lse for threads 0-127, dPsum for 128-255
          const int qc = mm * kTile + (ew_tid & 127);
          if (qc < w.lq) {
            const long long at = static_cast<long long>(hq) * a.total_q + w.q_start + qc;
            stat = (ew_tid < 128) ? a.lse[at] : a.dpsum[at];
          }
        }
        GDPA_WAIT_WARP(BB_S_FULL, s_phase, ST_ROLE_ACT);
        s_phase ^= 1u;
        tc_fence_after();
        if (tracer) GDPA_TRACE(a, tr * 32 + 9);
        if constexpr (kSoftmax) {
          // S(m) ready means every thread has left phase 1 of tile m-1 (lse buffer free) and phase 2 of tile
          // m-2 (dPsum buffer of this parity free)
          if (ew_tid < 128) stat_lse[ew_tid] = stat;
          else stat_dps[(m & 1) * kTile + (ew_tid - 128)] = stat;
          mbar_arrive(bar_base + 8u * BB_ST_FULL);
          GDPA_WAIT_WARP(BB_ST_FULL, st_phase, ST_ROLE_ACT);
          st_phase ^= 1u;
        }
        tmem_ld32(tS + half * 64, ra);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t(&cur)[32] = c ? rb : ra;
          uint32_t pk[16];
          tmem_wait_ld();
          tmem_regs_ready(cur);
          if (c == 0) tmem_ld32(tS + half * 64 + 32, rb);
          if constexpr (kSoftmax) {
            // P^T = 2^(c S^T - lse[q]) (already normalised); kept in g2 for dS = scale P (dP - dPsum)
            // the column test in two instantiations: none, or the per-thread range of a band
            auto emit = [&](auto inside) {
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                const int col = half * 64 + c * 32 + 2 * i;
                const float2 l2 = *reinterpret_cast<const float2*>(stat_lse + col);
                float p0 = ex2_approx(fmaf(__uint_as_float(cur[2 * i]), c2, -l2.x));
                float p1 = ex2_approx(fmaf(__uint_as_float(cur[2 * i + 1]), c2, -l2.y));
                p0 = inside(col) ? p0 : 0.f;
                p1 = inside(col + 1) ? p1 : 0.f;
                pk[i] = pack_bf16x2(p0, p1);
                g2[c * 16 + i] = pack_f32x2(p0, p1);
              }
            };
            if (full) emit([](int) { return true; });
            else emit([&](int col) { return col >= clo && col < chi; });
          } else if (full) {
#pragma unroll
            for (int i = 0; i < 16; ++i)
              act_and_grad_pair<ACT, false>(__uint_as_float(cur[2 * i]), __uint_as_float(cur[2 * i + 1]), scale, hscale,
                                            true, true, pk[i], g2[c * 16 + i]);
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int col = half * 64 + c * 32 + 2 * i;
              act_and_grad_pair<ACT, true>(__uint_as_float(cur[2 * i]), __uint_as_float(cur[2 * i + 1]), scale, hscale,
                                           col >= clo && col < chi, col + 1 >= clo && col + 1 < chi, pk[i], g2[c * 16 + i]);
            }
          }
          // P^T chunk c of this half goes over columns this half has already read
          tmem_st16(tS + half * 64 + c * 16, pk);
        }
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(bar_base + 8u * BB_P_FULL);
        if (tracer) GDPA_TRACE(a, tr * 32 + 10);

        GDPA_WAIT_WARP(BB_DP_FULL, dp_phase, ST_ROLE_ACT);
        dp_phase ^= 1u;
        tc_fence_after();
        if (tracer) GDPA_TRACE(a, tr * 32 + 11);
        // dS^T = act'(S^T) * dP^T for this thread's 64 columns (dP^T is finite everywhere: the operands are zero-padded)
        tmem_ld32(tDP + half * 64, ra);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t(&cur)[32] = c ? rb : ra;
          tmem_wait_ld();
          tmem_regs_ready(cur);
          if (c == 0) tmem_ld32(tDP + half * 64 + 32, rb);
          uint32_t pk[16];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint32_t d[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float d0, d1;
              if constexpr (kSoftmax) {
                const float2 ps = *reinterpret_cast<const float2*>(stat_dps + (m & 1) * kTile + half * 64 + c * 32 + 8 * j + 2 * e);
                float p0, p1;
                unpack_f32x2(g2[c * 16 + 4 * j + e], p0, p1);
                d0 = p0 * (__uint_as_float(cur[8 * j + 2 * e]) - ps.x) * scale;
                d1 = p1 * (__uint_as_float(cur[8 * j + 2 * e + 1]) - ps.y) * scale;
              } else {
                unpack_f32x2(mul_f32x2(g2[c * 16 + 4 * j + e],
                                       pack_f32x2(__uint_as_float(cur[8 * j + 2 * e]), __uint_as_float(cur[8 * j + 2 * e + 1]))),
                             d0, d1);
              }
              d[e] = pack_bf16x2(d0, d1);
            }
            // 16-byte chunk (4c + j) of this row's 128-byte line, XOR-swizzled by the row index
            *reinterpret_cast<uint4*>(sds_row + (((c * 4 + j) ^ (row & 7)) << 4)) = make_uint4(d[0], d[1], d[2], d[3]);
            pk[4 * j + 0] = d[0];
            pk[4 * j + 1] = d[1];
            pk[4 * j + 2] = d[2];
            pk[4 * j + 3] = d[3];
          }
          // the same values as the A operand of dK, over dP^T columns this half has already read
          tmem_st16(tDP + half * 64 + c * 16, pk);
        }
        tmem_wait_st();
        fence_proxy_async_smem();
        tc_fence_before();
        mbar_arrive(bar_base + 8u * BB_DS_FULL);
        if (tracer) GDPA_TRACE(a, tr * 32 + 12);
        ++tr;
      }
      // dK / dV of this KV tile: TMEM -> bf16 -> global, rows inside the sequence only.
      if (tracer) GDPA_TRACE(a, (tr - 1) * 32 + 17);
      GDPA_WAIT_WARP(BB_DKV_FULL, dkv_phase, ST_ROLE_ACT);
      dkv_phase ^= 1u;
      tc_fence_after();
      if (tracer) GDPA_TRACE(a, (tr - 1) * 32 + 18);
      // Rolled over the two tensors: this runs once per work item, and the kernel's code size is what the instruction
      // cache sees in every Q tile.
#pragma unroll 1
      for (int t = 0; t < 2; ++t) {
        const uint32_t tcol = tmem_base + lane_base + (t == 0 ? kColDV : kColDK) + half * (D / 2);
        if constexpr (ACC) {
          // K / V rows shared between sequences (start / end offsets): every owner adds into fp32 accumulators
          __nv_bfloat16* dst_row = (t == 0 ? dv_row : dk_row) + half * (D / 2);
#pragma unroll 1
          for (int c = 0; c < D / 64; ++c) {
            uint32_t r[32];
            tmem_ld32(tcol + c * 32, r);
            tmem_wait_ld();
            if (row_valid) {
              float* acc_row = (t == 0 ? a.dv_acc : a.dk_acc) + (dst_row - (t == 0 ? a.dv : a.dk)) + c * 32;
#pragma unroll
              for (int j = 0; j < 8; ++j)
                atomicAdd(reinterpret_cast<float4*>(acc_row) + j,
                          make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]),
                                      __uint_as_float(r[4 * j + 3])));
            }
          }
        } else {
          // This warp's 32 rows x D/2 columns go through shared memory so that they leave as whole row pieces: 16-byte
          // stores straight from registers, one row per thread, touch 32 lines per instruction and flood the load/store
          // unit (measured: the stores and the loads queued behind them cost ~7 000 cycles per work item).  The
          // staging slab is this warp's own 4 KB of the dS^T buffer, which nothing reads once the item's last dQ
          // product has completed (it precedes the commit this warp has just waited for); its 16-byte pieces are
          // XORed with row bits so that neither the row-per-thread writes nor the piece-per-thread reads conflict.
          // (TMA stores from the slab did the same job on full tiles but, with their two more tensor maps beside the
          // loader's, slowed ragged KV tiles several-fold.)
          constexpr int kPieces = D / 16;  // 16-byte pieces per row of D/2 bf16
          uint8_t* const slab = smem + L::kDsOff + half * L::kHalfBytes + quarter * 4096;
          auto piece = [](int row_, int chunk) { return row_ * (kPieces * 16) + ((chunk ^ (D == 128 ? (row_ & 7) : ((row_ >> 1) & 3))) << 4); };
#pragma unroll
          for (int c = 0; c < D / 64; ++c) {
            uint32_t r[32];
            tmem_ld32(tcol + c * 32, r);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 v;
              v.x = pack_bf16x2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
              v.y = pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
              v.z = pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
              v.w = pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
              *reinterpret_cast<uint4*>(slab + piece(lane, c * 4 + j)) = v;
            }
          }
          __syncwarp();
          // piece p = i * 32 + lane of the slab: row p / kPieces, 16-byte piece p % kPieces; kPieces neighbouring lanes
          // write one row's D bytes
          const int slab_rows = w.lkv - (kv_local - lane);  // rows of this warp's 32 inside the sequence
          __nv_bfloat16* const out0 = (t == 0 ? dv_row : dk_row) - static_cast<long long>(lane) * a.heads * D + half * (D / 2);
#pragma unroll 2
          for (int i = 0; i < kPieces; ++i) {
            const int prow = (i * 32 + lane) / kPieces, chunk = lane % kPieces;
            if (prow < slab_rows)
              *reinterpret_cast<uint4*>(out0 + static_cast<long long>(prow) * a.heads * D + chunk * 8) =
                  *reinterpret_cast<const uint4*>(slab + piece(prow, chunk));
          }
          __syncwarp();  // the slab is rewritten for the next tensor, and by the next item's dS^T
        }
      }
      tc_fence_before();
      mbar_arrive(bar_base + 8u * BB_DKV_EMPTY);
      if (tracer) GDPA_TRACE(a, (tr - 1) * 32 + 19);
    }
  } else {
    // ------------------------------------------------------------------ dQ reduce warps 0-3
    setmaxnreg_inc<kRegsReduce>();  // above the 128 registers per thread the kernel is launched with
    // Each warp drains its own 32 Q rows: TMEM -> registers -> its private staging slab (32 rows x
    // 32 fp32, 128-byte swizzled, two buffers) -> one TMA reduce-add per slab.  No cross-warp barrier.
    const uint32_t tDQ = tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + kColDP;
    uint8_t* stage_row = smem + L::kDqOff + warp * (2 * kDqWarpSlabBytes) + lane * 128;
    const uint32_t stage_base = smem_base + L::kDqOff + warp * (2 * kDqWarpSlabBytes);
    uint32_t dq_phase = 0, slab = 0;
    int tr = 0;
    int idx;
    while (true) {
      idx = take_work_item(ST_ROLE_RED, true);
      if (idx == -2) goto role_done;
      if (idx < 0) break;
      const Work w = load_work(a.sched, idx, a.q_off, a.kv_off, a.off64, a.max_q, a.max_kv, lim);
      int m0, nq1;
      bwd_q_range(w, a.window, m0, nq1);
      const int nq = nq1 * a.kv_group;
      for (int m = 0; m < nq; ++m) {
        const int hq = w.h * a.kv_group + m / nq1, mm = m0 + m % nq1;
        const int q_row0 = static_cast<int>(w.q_start) + mm * kTile + warp * 32;
        uint32_t r[D / 32][32];
        if (threadIdx.x == 0) GDPA_TRACE(a, tr * 32 + 13);
        {
          const bool ok = mbar_wait(bar_base + 8u * BB_DQ_FULL, dq_phase, abort_flag, a.status, (BB_DQ_FULL << 8) | ST_ROLE_RED);
          if (!__all_sync(0xffffffffu, ok)) goto role_done;  // warp-uniform decision
        }
        dq_phase ^= 1u;
        tc_fence_after();
        if (threadIdx.x == 0) GDPA_TRACE(a, tr * 32 + 14);
        // Pull the whole dQ tile into registers with back-to-back loads and release the TMEM columns
        // (they alias dP^T of the next Q tile) before any staging work.
#pragma unroll
        for (int c = 0; c < D / 32; ++c) tmem_ld32(tDQ + c * 32, r[c]);
        tmem_wait_ld();
#pragma unroll
        for (int c = 0; c < D / 32; ++c) tmem_regs_ready(r[c]);
        tc_fence_before();
        mbar_arrive(bar_base + 8u * BB_DQ_EMPTY);
        if (threadIdx.x == 0) GDPA_TRACE(a, tr * 32 + 15);
        // Rows of a ragged tile beyond the sequence belong to the next one and must not be touched (their dS is zero, but
        // a zero times a non-finite K row of THIS sequence is not): the reduce-add of a slab with fewer than 32 rows of
        // the sequence is issued as boxes of 16, 8, 4, 2, 1 rows that cover exactly those rows.
        const int slab_rows = w.lq - mm * kTile - warp * 32;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          const uint32_t buf = slab & 1u;
          // the reduce that read this staging buffer two slabs ago must have finished reading it
          if (lane == 0) tma_store_wait_read<1>();
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(stage_row + buf * kDqWarpSlabBytes + ((j ^ (lane & 7)) << 4)) =
                make_uint4(r[c][4 * j], r[c][4 * j + 1], r[c][4 * j + 2], r[c][4 * j + 3]);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (slab_rows >= 32) {
              tma_reduce_add_3d(&tm_dq.m[0], stage_base + buf * kDqWarpSlabBytes, c * 32, hq, q_row0);
            } else {
              int done = 0;
#pragma unroll 1
              for (int k = 1; k < kDqTmapHeights; ++k) {
                const int h = 32 >> k;
                if (slab_rows - done >= h) {
                  tma_reduce_add_3d(&tm_dq.m[k], stage_base + buf * kDqWarpSlabBytes + done * 128, c * 32, hq, q_row0 + done);
                  done += h;
                }
              }
            }
            tma_store_commit();
          }
          ++slab;
        }
        if (threadIdx.x == 0) GDPA_TRACE(a, tr * 32 + 16);
        ++tr;
      }
    }
  }

role_done:
  __syncwarp();
  if (*abort_flag != 0) {
    // a wait ran out: give this CTA's TMA copies and MMAs in flight a bounded time (1 ms) to finish
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 1000000ull) {}
  }
  if (warp < 4 && lane == 0) tma_store_wait_all<0>();  // this warp's reduce-adds have left shared memory
  tc_fence_before();
  __syncthreads();
#ifdef GDPA_ENABLE_TRACE
  if (a.trace != nullptr && threadIdx.x == 0 && blockIdx.x < 256) a.trace[kTraceSlots - 511 + 2 * blockIdx.x] = global_timer_ns();
#endif
  if (warp == kBwdMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

#undef GDPA_WAIT
#undef GDPA_WAIT_WARP

__global__ void __launch_bounds__(256) gdpa_dq_convert_kernel(const float4* __restrict__ acc, uint2* __restrict__ dq,
                                                              long long n4) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += stride) {
    const float4 v = acc[i];
    uint2 o;
    o.x = pack_bf16x2(v.x, v.y);
    o.y = pack_bf16x2(v.z, v.w);
    dq[i] = o;
  }
}

// dPsum[h, t] = sum_d dO[t, h, d] * O[t, h, d] (fp32), one warp per (token, head) row.
__global__ void __launch_bounds__(256) gdpa_dpsum_kernel(const __nv_bfloat16* __restrict__ d_o, const __nv_bfloat16* __restrict__ o,
                                                         float* __restrict__ dpsum, long long total_q, int heads, int head_dim) {
  const long long rows = total_q * heads;
  const int lane = threadIdx.x & 31;
  const long long warps = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  for (long long r = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); r < rows; r += warps) {
    const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(d_o + r * head_dim);
    const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(o + r * head_dim);
    float acc = 0.f;
    for (int i = lane; i < head_dim / 2; i += 32) {
      const float2 x = __bfloat1622float2(a2[i]), y = __bfloat1622float2(b2[i]);
      acc = fmaf(x.x, y.x, fmaf(x.y, y.y, acc));
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
    if (lane == 0) dpsum[(r % heads) * total_q + r / heads] = acc;
  }
}

template <int D, int ACT, bool ACC>
int launch_bwd_acc(const BwdLaunch& l) {
  using L = BwdSmem<D>;
  auto kernel = gdpa_bwd_kernel<D, ACT, ACC>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynBytes);
  if (e != cudaSuccess) return GDPA_ERR_LAUNCH_;
  kernel<<<l.grid, kBwdThreads, L::kDynBytes, l.stream>>>(l.tm_q, l.tm_k, l.tm_v, l.tm_do, l.tm_dq, l.args);
  return cudaGetLastError() == cudaSuccess ? 0 : GDPA_ERR_LAUNCH_;
}

template <int D, int ACT>
int launch_bwd_inst(const BwdLaunch& l) {
  return l.args.dk_acc != nullptr ? launch_bwd_acc<D, ACT, true>(l) : launch_bwd_acc<D, ACT, false>(l);
}

template <int D>
int launch_bwd_d(const BwdLaunch& l, int act_class) {
  switch (act_class) {
    case ACT_RAW: return launch_bwd_inst<D, ACT_RAW>(l);
    case ACT_GELU_ERF: return launch_bwd_inst<D, ACT_GELU_ERF>(l);
    case ACT_GELU_TANH: return launch_bwd_inst<D, ACT_GELU_TANH>(l);
    case ACT_LEAKY_RELU: return launch_bwd_inst<D, ACT_LEAKY_RELU>(l);
    case ACT_RELU: return launch_bwd_inst<D, ACT_RELU>(l);
    case ACT_SILU: return launch_bwd_inst<D, ACT_SILU>(l);
    case ACT_HARDSWISH: return launch_bwd_inst<D, ACT_HARDSWISH>(l);
    case ACT_RELU_SQUARE: return launch_bwd_inst<D, ACT_RELU_SQUARE>(l);
    case ACT_SOFTMAX: return launch_bwd_inst<D, ACT_SOFTMAX>(l);
    default: return GDPA_ERR_UNSUPPORTED_ACT_;
  }
}

}  // namespace

int launch_bwd_bf16(const BwdLaunch& l, int head_dim, int act_class) {
  if (head_dim == 128) return launch_bwd_d<128>(l, act_class);
  if (head_dim == 64) return launch_bwd_d<64>(l, act_class);
  return GDPA_ERR_UNSUPPORTED_DIM_;
}

int launch_dpsum(const __nv_bfloat16* d_o, const __nv_bfloat16* o, float* dpsum, long long total_q, int heads, int head_dim,
                 cudaStream_t stream) {
  const long long rows = total_q * heads;
  if (rows == 0) return 0;
  long long blocks = (rows + 7) / 8;
  if (blocks > 148 * 16) blocks = 148 * 16;
  gdpa_dpsum_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(d_o, o, dpsum, total_q, heads, head_dim);
  return cudaGetLastError() == cudaSuccess ? 0 : GDPA_ERR_LAUNCH_;
}

int launch_dq_convert(const float* acc, __nv_bfloat16* dq, long long n, cudaStream_t stream) {
  const long long n4 = n / 4;  // heads * head_dim is a multiple of 64
  if (n4 == 0) return 0;
  long long blocks = (n4 + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  gdpa_dq_convert_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(reinterpret_cast<const float4*>(acc),
                                                                      reinterpret_cast<uint2*>(dq), n4);
  return cudaGetLastError() == cudaSuccess ? 0 : GDPA_ERR_LAUNCH_;
}


}  // namespace gdpa
