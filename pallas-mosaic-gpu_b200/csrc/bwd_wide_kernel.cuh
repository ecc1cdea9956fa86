// Splash attention fused backward over the column (per-KV-block) schedule with 128 q
// rows per step, head_dim 128, sm_100a.
//
// Why a second column kernel.  The 64-row-per-step kernel (bwd_col_kernel.cuh) is bound
// by the shared-memory data pipe, not by the tensor core: a tcgen05.mma that reads both
// operands from shared memory streams M x 16 + N x 16 16-bit values per instruction, and
// with N = 64 that is 6 KB for 32 cycles of arithmetic -- more than the 128 bytes per
// cycle the pipe delivers.  Taking a whole 128-row q block per step makes every
// score-shaped product N = 128 (8 KB for 64 cycles: exactly the pipe's rate) and reads
// the stationary K / V tile once per 128 q rows instead of twice; shared-memory traffic
// per visited block pair drops by about a quarter.
//
// One CTA owns one 128-row KV block of one KV head and walks every q block that sees it,
// for every q head of the KV head's group (GQA/MQA heads are reduced in tensor memory).
// Per step (one 128 x 128 block pair):
//   S^T  = K Q^T        smem x smem -> TMEM region R1 (f32, 128 columns)
//   dP^T = V dO^T       smem x smem -> TMEM region R2
//   phase A (needs S^T):   P^T = exp2((S^T - lse) log2e), packed 16-bit over R1
//   phase B (needs dP^T):  dS^T = P^T (dP^T - delta) [(1 - tanh^2) with soft-cap], packed
//                          over R2 and staged in shared memory as an MMA operand
//   dV  += P^T dO       TMEM x smem
//   dK  += dS^T Q       TMEM x smem
//   dQ^T = K^T dS^T     smem x smem -> R2, drained by a writer warpgroup that
//                       reduce-adds it into the f32 accumulator [batch*heads*128, q_len]
//
// Tensor memory holds R1, R2, dK and dV (4 x 128 = 512 columns), so the scores are not
// double-buffered; the overlap comes from the issue order instead:
//   dP^T(t)  dV(t)  S^T(t+1)  dK(t)  dQ^T(t)  [writer drains R2]  dP^T(t+1) ...
// Phase B of step t runs under dV(t) and S^T(t+1); phase A of step t+1 runs under dK(t),
// dQ^T(t), the drain and dP^T(t+1).  The only gap in the tensor core's queue is the drain
// of R2.  Q has two slots (Q(t) lives from S^T(t) to dK(t), across S^T(t+1)); dO has one
// (it lives from dP^T(t) to dV(t), which are adjacent) and is refilled under S^T(t+1),
// dK(t) and dQ^T(t).  The writer stages f32 dQ^T tiles in 32 KB of its own, so it only
// has to keep up with the step rate.
//
// Behaviour follows the reference kernel (splash_attention_mgpu/backward_fused.py:64-512);
// the code shares nothing with it.
#pragma once

#include <stddef.h>

#include <type_traits>

#include "bwd_col_kernel.cuh"  // BwdArgs, ColSteps, math constants
#include "ptx.cuh"

// Timeline marks for debugging builds; empty in the product.
#ifndef SPLASH_TRACE_MARK
#define SPLASH_TRACE_MARK(role, t, k)
#define SPLASH_TRACE_NS(role, t, k)
#endif

namespace splash {

enum WideSite : int {
  kWSiteQEmpty = 61, kWSiteDoEmpty, kWSiteMmaKV, kWSiteMmaQ, kWSiteMmaDo, kWSiteMmaP, kWSiteMmaDs, kWSiteMmaDqFree,
  kWSiteEwQ, kWSiteEwS, kWSiteEwDp, kWSiteEwStage, kWSiteEwDone, kWSiteEwEpi,
  kWSiteWrReady,
};

template <int D_>
struct WideLayout {
  static_assert(D_ == 64 || D_ == 128, "head_dim 64 or 128");
  static constexpr int D = D_;
  static constexpr int kRows = 128;  // kv rows per CTA
  static constexpr int BC = 128;     // q rows per step
  static constexpr int kBox = kRows * 128;        // one 64-element-wide box of a 128-row tile: 16 KB
  static constexpr int kTile = kRows * D * 2;     // a K, V, Q or dO tile
  // At head_dim 64 the dQ^T product keeps M = 128: its A operand's second 64 rows are a second
  // copy of the K tile, so the upper half of the result repeats the lower half and is not stored.
  static constexpr int kKDupBytes = D == 64 ? kBox : 0;
  static constexpr int kDsBytes = kRows * BC * 2;  // dS^T as an MMA operand
  static constexpr int kSlots = 2;
  static constexpr int kVecBytes = BC * 4;
  // Shared memory map (bytes from the 1024-aligned base).
  static constexpr int kOffK = 0, kOffV = kTile + kKDupBytes, kOffQ = kOffV + kTile, kOffDo = kOffQ + kSlots * kTile;
  static constexpr int kOffDs = kOffDo + kTile;
  static constexpr int kOffDqStage = kOffDs + kDsBytes;  // per writer warp: kDqBufs f32 tiles of [32 d, 32 q]
  static constexpr int kDqBufs = 2;
  static constexpr int kDqBoxBytes = 32 * 32 * 4;
  static constexpr int kOffLse = kOffDqStage + 4 * kDqBufs * kDqBoxBytes, kOffDelta = kOffLse + kSlots * kVecBytes;
  // Folded operands (head_dim 64, where shared memory has the room): -lse and -delta are subtracted
  // inside the S^T and dP^T products by one extra K = 16 slice each.  Per q row eight 16-bit values
  // {hi, mid, lo, 0, ...} whose sum is -lse (or -delta) to f32 precision -- the first 8 x 8 core
  // matrices of an unswizzled K-major tile -- against {1, 1, 1, 0, ...} per kv row; the second half of
  // K is a shared block of zeros.
  static constexpr bool kFold = D == 64;
  static constexpr int kAuxTile = BC * 16;
  static constexpr int kOffAux = kOffDelta + kSlots * kVecBytes;                  // per Q slot: [-lse tile | -delta tile]
  static constexpr int kOffOnes = kOffAux + (kFold ? kSlots * 2 * kAuxTile : 0);
  static constexpr int kOffZeros = kOffOnes + (kFold ? kAuxTile : 0);
  static constexpr int kOffBars = kOffZeros + (kFold ? kAuxTile : 0);
  static constexpr int kBarBytes = 256;
  static constexpr int kListSteps = 256;  // capacity of the list of block steps that survive segment skipping
  static constexpr int kOffList = kOffBars + kBarBytes;
  static constexpr int kSmemBytes = kOffList + kListSteps * 2;
  // Tensor memory columns.
  static constexpr int kColS = 0, kColDp = 128, kColDk = 256, kColDv = 256 + D;
  static constexpr int kTmemCols = 512;
  static constexpr int kEwThreads = 256;
  static constexpr int kThreads = 512;  // 2 elementwise warpgroups, writer warpgroup, producer warpgroup
  // Registers per thread after the warpgroups have traded: 256 * 160 + 128 * 152 + 128 * 40 = 64 K.
  static constexpr int kEwRegs = 160, kWriterRegs = 152, kProducerRegs = 40;
};

struct WideBarriers {
  uint64_t kv_full;
  uint64_t q_full[2], q_empty[2], do_full, do_empty;
  uint64_t s_ready, dp_ready, p_ready, ds_ready;
  uint64_t dq_ready, dq_free;
  uint64_t acc_done, epi[2];
  uint32_t tmem_base;
  uint32_t abort_flag;
  uint32_t dead;
  uint32_t n_eff;  // block steps left after segment skipping
};
static_assert(sizeof(WideBarriers) <= WideLayout<128>::kBarBytes, "barrier block");

#define SPLASH_WBAR(field, idx) \
  (bars_u32 + static_cast<uint32_t>(offsetof(WideBarriers, field)) + 8u * static_cast<uint32_t>(idx))

// PLAIN: no soft-cap and no segment ids -- that code is compiled out.  Streamed (dense
// int8) mask blocks are not handled here; calls that carry them take the 64-row kernel.
template <int HEAD_DIM, bool PLAIN, bool BF16>
__global__ void __launch_bounds__(WideLayout<HEAD_DIM>::kThreads, 1)
splash_bwd_wide_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                       const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                       const __grid_constant__ CUtensorMap tm_dk, const __grid_constant__ CUtensorMap tm_dv,
                       const __grid_constant__ CUtensorMap tm_dqacc, const BwdArgs a) {
  using L = WideLayout<HEAD_DIM>;
  constexpr int D = L::D;
  constexpr int kRows = L::kRows;
  constexpr int kEwWarps = 8;
  constexpr int kWriterWarp0 = 8;
  constexpr int kProducerWarp0 = 12;  // +0 Q/K/V producer, +1 MMA issuer, +2 dO producer

  const bool has_seg = !PLAIN && a.has_seg;
  const float soft_cap = PLAIN ? 0.f : a.soft_cap;
  extern __shared__ __align__(1024) uint8_t smem_wide[];
  const uint32_t base_u32 = smem_u32(smem_wide);
  const uint32_t k_u32 = base_u32 + L::kOffK;
  const uint32_t v_u32 = base_u32 + L::kOffV;
  const uint32_t q_u32 = base_u32 + L::kOffQ;
  const uint32_t do_u32 = base_u32 + L::kOffDo;
  const uint32_t ds_u32 = base_u32 + L::kOffDs;
  const uint32_t dqs_u32 = base_u32 + L::kOffDqStage;
  const uint32_t lse_u32 = base_u32 + L::kOffLse;
  const uint32_t delta_u32 = base_u32 + L::kOffDelta;
  const uint32_t aux_u32 = base_u32 + L::kOffAux;
  const uint32_t ones_u32 = base_u32 + L::kOffOnes;
  const uint32_t zeros_u32 = base_u32 + L::kOffZeros;
  // With soft-capping lse has to be subtracted after the cap, so only delta is folded then.
  const bool fold_lse = L::kFold && !(soft_cap > 0.f);
  const uint32_t bars_u32 = base_u32 + L::kOffBars;
  const uint32_t abort_u32 = bars_u32 + static_cast<uint32_t>(offsetof(WideBarriers, abort_flag));
  const uint32_t dead_u32 = bars_u32 + static_cast<uint32_t>(offsetof(WideBarriers, dead));
  const uint32_t tmem_slot_u32 = bars_u32 + static_cast<uint32_t>(offsetof(WideBarriers, tmem_base));
  const uint32_t neff_u32 = bars_u32 + static_cast<uint32_t>(offsetof(WideBarriers, n_eff));
  const uint32_t list_u32 = base_u32 + L::kOffList;
  const bool has_list = has_seg && a.seg_q_ranges != nullptr;

  const int warp = uniform_warp_index();
  const int lane = threadIdx.x & 31;

  // ---- which KV block ----------------------------------------------------------
  const int group = a.heads / a.kv_heads;
  int hb, order_idx;
  decode_work_item(blockIdx.x, a.kv_blocks, a.kv_heads * a.batch, a.head_group, hb, order_idx);
  const int kvh = hb % a.kv_heads;
  const int b = hb / a.kv_heads;
  const int head0 = kvh * group;
  const int mh0 = a.mask_heads > 1 ? head0 : 0;
  const int kj = a.block_order[mh0 * a.kv_blocks + order_idx];
  const int kv_row0 = (b * a.kv_heads + kvh) * a.kv_len + kj * kRows;  // row in the [B*KVH*Skv, D] view

  ColSteps<1> it;
  it.bind(&a, kj, head0, group);
  const int scheduled = it.scheduled();

  // One warp initialises the barriers while the MMA warp allocates tensor memory.  Thread
  // 0 reads the status word once and shares it, so the whole CTA agrees on whether an
  // earlier launch already gave up; the tiles need a 1024-byte aligned base, which the
  // same thread checks.
  if (warp == 0) {
    constexpr uint32_t kNumBarriers = offsetof(WideBarriers, tmem_base) / 8;
    for (uint32_t i = lane; i < kNumBarriers; i += 32) {
      const uint32_t off = 8u * i;
      uint32_t count = 1;
      if (off >= offsetof(WideBarriers, q_empty) && off < offsetof(WideBarriers, do_full)) count = 1 + kEwWarps;  // dK + vector readers
      if (off == offsetof(WideBarriers, p_ready) || off == offsetof(WideBarriers, ds_ready)) count = L::kEwThreads;
      if (off == offsetof(WideBarriers, dq_free) || off >= offsetof(WideBarriers, epi)) count = 128;
      mbar_init(bars_u32 + off, count);
    }
    if (lane == 0) {
      sts32(abort_u32, 0);
      uint32_t dead_word = a.status[0] != 0;
      if (base_u32 & 1023u) {
        if (atomicCAS(a.status, 0, kDevBadSchedule) == 0) {
          a.status[1] = 0;
          a.status[2] = static_cast<int>(blockIdx.x);
          a.status[3] = static_cast<int>(base_u32 & 1023u);
        }
        dead_word = 1;
      }
      sts32(dead_u32, dead_word);
    }
    fence_mbar_init();
    fence_proxy_async_smem();
  } else if (warp == kProducerWarp0 + 1) {
    tmem_alloc(tmem_slot_u32, L::kTmemCols);
    tmem_relinquish();
  } else if (warp == 1 && has_list) {
    // Block steps whose q and kv segment-id ranges can meet; the others are left out by every role.
    const int2* qt = a.seg_q_ranges + static_cast<size_t>(b) * (a.q_len / kSegChunk);
    const int2* kt = a.seg_kv_ranges + static_cast<size_t>(b) * (a.kv_len / kSegChunk);
    const SegRange kr = seg_range(kt, kj * (kRows / kSegChunk), kRows / kSegChunk);
    const int kept = build_step_list(list_u32, scheduled, lane, [&](int f) {
      const int qblk = a.block_list[it.off_of_flat(f)];
      return seg_classify(seg_range(qt, qblk * (128 / kSegChunk), 128 / kSegChunk), kr);
    });
    if (lane == 0) sts32(neff_u32, static_cast<uint32_t>(kept));
  }
  if constexpr (L::kFold) {
    if (threadIdx.x >= 64 && threadIdx.x < 64 + 256) {
      // 128 rows of {1, 1, 1, 0, 0, 0, 0, 0}, and 2 KB of zeros.
      const uint32_t i = threadIdx.x - 64;
      const uint32_t one = BF16 ? 0x3f80u : 0x3c00u;
      if (i < 128) sts128(ones_u32 + i * 16, make_uint4(one | (one << 16), one, 0u, 0u));
      else sts128(zeros_u32 + (i - 128) * 16, make_uint4(0u, 0u, 0u, 0u));
      fence_proxy_async_smem();
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = lds32(tmem_slot_u32);
  const WaitCtx ctx{abort_u32};
  it.start(list_u32, has_list, has_list ? static_cast<int>(lds32(neff_u32)) : scheduled);
  const int total = it.total();
  if (lds32(dead_u32)) {
    if (warp == kProducerWarp0 + 1) {
      __syncwarp();
      tmem_dealloc(tmem, L::kTmemCols);
    }
    return;
  }
  constexpr uint32_t kDescHi = desc_hi(1024);

  if (warp >= kProducerWarp0) {
    setmaxnreg_dec<L::kProducerRegs>();
    if (warp == kProducerWarp0 && total > 0) {
      // -------------------- K, V once; then the Q ring (with lse, delta) --------------------
      if (elect_one()) {
        prefetch_tensormap(&tm_q);
        prefetch_tensormap(&tm_k);
        prefetch_tensormap(&tm_v);
        mbar_arrive_expect_tx(SPLASH_WBAR(kv_full, 0), 2 * L::kTile + L::kKDupBytes);
#pragma unroll
        for (int c = 0; c < D / 64; ++c) tma_load_2d(k_u32 + c * L::kBox, &tm_k, c * 64, kv_row0, SPLASH_WBAR(kv_full, 0));
        if constexpr (L::kKDupBytes > 0) tma_load_2d(k_u32 + L::kTile, &tm_k, 0, kv_row0, SPLASH_WBAR(kv_full, 0));
#pragma unroll
        for (int c = 0; c < D / 64; ++c) tma_load_2d(v_u32 + c * L::kBox, &tm_v, c * 64, kv_row0, SPLASH_WBAR(kv_full, 0));
      }
      for (int t = 0; it.valid(); it.next(), ++t) {
        const int slot = t & 1;
        const int qblk = a.block_list[it.off()];
        const int q_row = (b * a.heads + it.head()) * a.q_len + qblk * 128;
        if (t >= 2 && !warp_wait(SPLASH_WBAR(q_empty, slot), ((t >> 1) & 1) ^ 1, ctx, kWSiteQEmpty, t)) break;
        if (elect_one()) {
          const uint32_t bar = SPLASH_WBAR(q_full, slot);
          mbar_arrive_expect_tx(bar, L::kTile + (L::kFold ? 2 * L::kAuxTile + L::kVecBytes : 2 * L::kVecBytes));
#pragma unroll
          for (int c = 0; c < D / 64; ++c) tma_load_2d(q_u32 + slot * L::kTile + c * L::kBox, &tm_q, c * 64, q_row, bar);
          bulk_load_1d(lse_u32 + slot * L::kVecBytes, a.lse + q_row, L::kVecBytes, bar);
          if constexpr (L::kFold) {
            const size_t aux_off = static_cast<size_t>(q_row) * 16;
            bulk_load_1d(aux_u32 + slot * 2 * L::kAuxTile, a.aux_lse + aux_off, L::kAuxTile, bar);
            bulk_load_1d(aux_u32 + slot * 2 * L::kAuxTile + L::kAuxTile, a.aux_delta + aux_off, L::kAuxTile, bar);
          } else {
            bulk_load_1d(delta_u32 + slot * L::kVecBytes, a.delta + q_row, L::kVecBytes, bar);
          }
        }
      }
    } else if (warp == kProducerWarp0 + 2 && total > 0) {
      // ------------------------------------ dO ring ------------------------------------
      if (elect_one()) prefetch_tensormap(&tm_do);
      for (int t = 0; it.valid(); it.next(), ++t) {
        const int qblk = a.block_list[it.off()];
        const int q_row = (b * a.heads + it.head()) * a.q_len + qblk * 128;
        if (t >= 1 && !warp_wait(SPLASH_WBAR(do_empty, 0), (t & 1) ^ 1, ctx, kWSiteDoEmpty, t)) break;
        if (elect_one()) {
          const uint32_t bar = SPLASH_WBAR(do_full, 0);
          mbar_arrive_expect_tx(bar, L::kTile);
#pragma unroll
          for (int c = 0; c < D / 64; ++c) tma_load_2d(do_u32 + c * L::kBox, &tm_do, c * 64, q_row, bar);
        }
      }
    } else if (warp == kProducerWarp0 + 1 && total > 0) {
      // ----------------------------------- MMA issuer -----------------------------------
      // All lanes run the loop; one elected lane issues each instruction.
      constexpr uint32_t kIdescScore = make_idesc(BF16, 128, 128, false, false);  // K Q^T, V dO^T
      constexpr uint32_t kIdescAcc = make_idesc(BF16, 128, D, false, true);        // P^T dO, dS^T Q
      constexpr uint32_t kIdescDq = make_idesc(BF16, 128, 128, true, true);        // K^T dS^T
      // K-major tiles: 64-element boxes side by side, 32 bytes per 16-element slice.
      auto issue_scores = [&](uint32_t d_col, uint32_t a_tile, uint32_t b_tile) {
        const uint32_t a_lo = desc_lo(a_tile, 16), b_lo = desc_lo(b_tile, 16);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t o = ((kk / 4) * L::kBox + (kk % 4) * 32) >> 4;
          umma_ss2_w(tmem + d_col, a_lo + o, kDescHi, b_lo + o, kDescHi, kIdescScore, kk > 0);
        }
      };
      // One more K = 16 slice: D[kv, q] += sum_k ones[kv, k] * aux[q, k] = -lse[q] (or -delta[q]);
      // both operands unswizzled K-major, the second half of K read from the block of zeros.
      auto issue_fold = [&](uint32_t d_col, uint32_t b_tile) {
        umma_ss2_w(tmem + d_col, desc_lo_plain(ones_u32, zeros_u32 - ones_u32), desc_hi_plain(128),
                   desc_lo_plain(b_tile, zeros_u32 - b_tile), desc_hi_plain(128), kIdescScore, 1u);
      };
      // A = packed 16-bit values the elementwise warps left in tensor memory: q columns
      // 0-63 packed into columns 0-31 of the region, q columns 64-127 into columns 64-95
      // (each warpgroup packs into its own half).  B = a [128 q, 128 d] tile read MN-major.
      auto issue_acc = [&](uint32_t d_col, uint32_t a_col, uint32_t b_tile, bool first) {
        const uint32_t b_lo = desc_lo(b_tile, L::kBox);
#pragma unroll
        for (int kk = 0; kk < 128 / 16; ++kk)
          umma_ts2_w(tmem + d_col, tmem + a_col + (kk >> 2) * 64 + (kk & 3) * 8, b_lo + ((kk * 2048) >> 4), kDescHi,
                     kIdescAcc, (!first || kk > 0) ? 1u : 0u);
      };
      // dQ^T[d, q] = sum_kv K[kv, d] dS^T[kv, q]: both operands read MN-major.
      auto issue_dq = [&]() {
        const uint32_t k_lo = desc_lo(k_u32, L::kBox), ds_lo = desc_lo(ds_u32, L::kBox);
#pragma unroll
        for (int kk = 0; kk < kRows / 16; ++kk)
          umma_ss2_w(tmem + L::kColDp, k_lo + ((kk * 2048) >> 4), kDescHi, ds_lo + ((kk * 2048) >> 4), kDescHi, kIdescDq,
                     kk > 0);
      };
      bool ok = warp_wait(SPLASH_WBAR(kv_full, 0), 0, ctx, kWSiteMmaKV, 0) &&
                warp_wait(SPLASH_WBAR(q_full, 0), 0, ctx, kWSiteMmaQ, 0);
      if (ok) {
        tc_fence_after();
        issue_scores(L::kColS, k_u32, q_u32);
        if (fold_lse) issue_fold(L::kColS, aux_u32);
        umma_commit_w(SPLASH_WBAR(s_ready, 0));
        ok = warp_wait(SPLASH_WBAR(do_full, 0), 0, ctx, kWSiteMmaDo, 0);
      }
      if (ok) {
        tc_fence_after();
        issue_scores(L::kColDp, v_u32, do_u32);
        if constexpr (L::kFold) issue_fold(L::kColDp, aux_u32 + L::kAuxTile);
        umma_commit_w(SPLASH_WBAR(dp_ready, 0));
        for (int t = 0; t < total; ++t) {
          const int slot = t & 1, nslot = slot ^ 1;
          const uint32_t par = t & 1;
          SPLASH_TRACE_MARK(0, t, 0);
          if (!warp_wait(SPLASH_WBAR(p_ready, 0), par, ctx, kWSiteMmaP, t)) break;
          SPLASH_TRACE_MARK(0, t, 1);
          tc_fence_after();
          issue_acc(L::kColDv, L::kColS, do_u32, t == 0);                      // dV += P^T dO
          umma_commit_w(SPLASH_WBAR(do_empty, 0));
          if (t + 1 < total) {
            if (!warp_wait(SPLASH_WBAR(q_full, nslot), ((t + 1) >> 1) & 1, ctx, kWSiteMmaQ, t + 1)) break;
            SPLASH_TRACE_MARK(0, t, 2);
            tc_fence_after();
            issue_scores(L::kColS, k_u32, q_u32 + nslot * L::kTile);         // S^T(t+1) over P^T(t)
            if (fold_lse) issue_fold(L::kColS, aux_u32 + nslot * 2 * L::kAuxTile);
            umma_commit_w(SPLASH_WBAR(s_ready, 0));
          }
          SPLASH_TRACE_MARK(0, t, 3);
          if (!warp_wait(SPLASH_WBAR(ds_ready, 0), par, ctx, kWSiteMmaDs, t)) break;
          SPLASH_TRACE_MARK(0, t, 4);
          tc_fence_after();
          issue_acc(L::kColDk, L::kColDp, q_u32 + slot * L::kTile, t == 0);   // dK += dS^T Q
          umma_commit_w(SPLASH_WBAR(q_empty, slot));
          issue_dq();                                                          // dQ^T(t) over dS^T(t)
          umma_commit_w(SPLASH_WBAR(dq_ready, 0));
          SPLASH_TRACE_MARK(0, t, 5);
          if (t + 1 < total && !warp_wait(SPLASH_WBAR(do_full, 0), par ^ 1, ctx, kWSiteMmaDo, t + 1)) break;
          SPLASH_TRACE_MARK(0, t, 6);
          // The writer must have taken dQ^T(t) out of R2 (every phase of dq_free is observed).
          if (!warp_wait(SPLASH_WBAR(dq_free, 0), par, ctx, kWSiteMmaDqFree, t)) break;
          SPLASH_TRACE_MARK(0, t, 7);
          if (t + 1 < total) {
            tc_fence_after();
            issue_scores(L::kColDp, v_u32, do_u32);                            // dP^T(t+1)
            if constexpr (L::kFold) issue_fold(L::kColDp, aux_u32 + nslot * 2 * L::kAuxTile + L::kAuxTile);
            umma_commit_w(SPLASH_WBAR(dp_ready, 0));
          }
        }
        umma_commit_w(SPLASH_WBAR(acc_done, 0));
      }
    }
  } else if (warp >= kWriterWarp0) {
    // ================================ dQ writer ==================================
    setmaxnreg_inc<L::kWriterRegs>();
    // Each warp drains its own 32 head-dim rows (its quarter of the TMEM lanes) through
    // staging tiles of its own, so the writer warps never wait for one another.
    const int wq = warp & 3;
    const uint32_t dq_tmem = tmem + (static_cast<uint32_t>(wq * 32) << 16) + L::kColDp;
    const uint32_t my_stage = dqs_u32 + wq * (L::kDqBufs * L::kDqBoxBytes);
    int t = 0;
    for (; it.valid(); it.next(), ++t) {
      const int qblk = a.block_list[it.off()];
      SPLASH_TRACE_MARK(2, t, 0);
      if (!warp_wait(SPLASH_WBAR(dq_ready, 0), t & 1, ctx, kWSiteWrReady, t)) break;
      SPLASH_TRACE_MARK(2, t, 1);
      tc_fence_after();
      uint32_t acc[128];
      const bool mine = wq * 32 < D;  // at head_dim 64 the upper two quarters repeat the lower ones
      if (mine) {
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32(dq_tmem + c * 32, acc + c * 32);
        tmem_wait_ld();
      }
      tc_fence_before();
      mbar_arrive(SPLASH_WBAR(dq_free, 0));
      if (!mine) continue;
      SPLASH_TRACE_MARK(2, t, 2);
      const int x = qblk * 128;
      const int y = (b * a.heads + it.head()) * D + wq * 32;
      // Four passes of 32 q columns: [32 d, 32 q] f32 tiles, 128-byte rows, 128-byte swizzle.
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t stage = my_stage + (j % L::kDqBufs) * L::kDqBoxBytes;
        // The reduction that last used this tile must have read it.
        if (lane == 0 && (t > 0 || j >= L::kDqBufs)) bulk_wait_group_read<L::kDqBufs - 1>();
        __syncwarp();
#pragma unroll
        for (int c = 0; c < 8; ++c)
          sts128(stage + swz128(lane, c), make_uint4(acc[j * 32 + c * 4], acc[j * 32 + c * 4 + 1],
                                                     acc[j * 32 + c * 4 + 2], acc[j * 32 + c * 4 + 3]));
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_reduce_add_2d(&tm_dqacc, stage, x + j * 32, y);
          bulk_commit_group();
        }
      }
      SPLASH_TRACE_MARK(2, t, 3);
    }
    if (lane == 0) bulk_wait_group_read<0>();
  } else {
    // ========================== elementwise warpgroups ===========================
    setmaxnreg_inc<L::kEwRegs>();
    const int w = warp >> 2;                 // which half of the 128 q columns
    const int wq = warp & 3;
    const int row = wq * 32 + lane;          // kv row inside the block
    const int kv_pos = kj * kRows + row;
    const uint32_t tmem_row = tmem + (static_cast<uint32_t>(wq * 32) << 16);
    const int col0 = w * 64;                 // first q column this thread handles

    if (total == 0) {
      // No q block sees this KV block: its gradients are zero.
      uint8_t* base = static_cast<uint8_t*>(w == 0 ? a.dk : a.dv);
      uint4* dst = reinterpret_cast<uint4*>(base + static_cast<size_t>(kv_row0 + row) * (D * 2));
#pragma unroll
      for (int c = 0; c < D * 2 / 16; ++c) dst[c] = make_uint4(0, 0, 0, 0);
    } else {
      const int my_seg = has_seg ? a.seg_kv[static_cast<size_t>(b) * a.kv_len + kv_pos] : 0;
      const bool cap_on = soft_cap > 0.f;
      const float cap = soft_cap, inv_cap = cap_on ? 1.f / soft_cap : 0.f;
      bool alive = true;
      int cur_mh = -1;
      int band_lo = -(1 << 30), band_hi = (1 << 30);  // allowed range of kv_pos - q_pos for this kv row

      for (int t = 0; it.valid(); it.next(), ++t) {
        const int slot = t & 1;
        const uint32_t par = t & 1;
        const int off = it.off();
        const int qblk = a.block_list[off];
        const bool partial = a.block_kind[off] == SPLASH_BLOCK_PARTIAL;
        if (a.mask_desc && it.mask_head(it.g) != cur_mh) {
          cur_mh = it.mask_head(it.g);
          band_lo = a.mask_desc[cur_mh * 4 + 0];
          band_hi = a.mask_desc[cur_mh * 4 + 1];
          const int chunk = a.mask_desc[cur_mh * 4 + 2];
          if (chunk > 0) {
            // q must share the kv row's chunk: start <= q_pos <= start + chunk - 1.
            const int start = (kv_pos / chunk) * chunk;
            band_lo = max(band_lo, kv_pos - (start + chunk - 1));
            band_hi = min(band_hi, kv_pos - start);
          }
        }
        const int q0 = qblk * 128 + col0;  // sequence position of this thread's first column
        // Visibility of this thread's 64 columns (bit i of word c: column c * 32 + i).
        uint32_t vis[2] = {0xffffffffu, 0xffffffffu};
        const bool seg_compare = has_seg && !it.uniform();
        const bool plain_step = !partial && !seg_compare && !cap_on;
        if (!plain_step) {
          if (partial) {
            // Column i of word c is visible iff band_lo <= d0 - i <= band_hi: a run of bits.
#pragma unroll
            for (int c = 0; c < 2; ++c) {
              const int d0 = kv_pos - (q0 + c * 32);
              const int first = max(0, d0 - band_hi), last = min(31, d0 - band_lo);
              vis[c] = first <= last ? ((0xffffffffu >> (31 - last)) & (0xffffffffu << first)) : 0u;
            }
          }
          if (seg_compare) {
            const int4* sq = reinterpret_cast<const int4*>(a.seg_q + static_cast<size_t>(b) * a.q_len + q0);
#pragma unroll
            for (int g = 0; g < 16; ++g) {
              const int4 sg = __ldg(sq + g);
              const int c = g >> 3, i = (g & 7) * 4;
              if (sg.x != my_seg) vis[c] &= ~(1u << (i + 0));
              if (sg.y != my_seg) vis[c] &= ~(1u << (i + 1));
              if (sg.z != my_seg) vis[c] &= ~(1u << (i + 2));
              if (sg.w != my_seg) vis[c] &= ~(1u << (i + 3));
            }
          }
        }
        SPLASH_TRACE_MARK(1, t, 0);
        SPLASH_TRACE_NS(1, t, 7);
        if (!warp_wait(SPLASH_WBAR(q_full, slot), (t >> 1) & 1, ctx, kWSiteEwQ, t)) { alive = false; break; }
        if (!warp_wait(SPLASH_WBAR(s_ready, 0), par, ctx, kWSiteEwS, t)) { alive = false; break; }
        SPLASH_TRACE_MARK(1, t, 1);
        tc_fence_after();

        // ---- phase A: P^T from S^T; the factor that dS^T needs stays in registers ----
        float pf[64];
        {
          uint32_t* sraw = reinterpret_cast<uint32_t*>(pf);
          tmem_ld32(tmem_row + L::kColS + col0, sraw);
          tmem_ld32(tmem_row + L::kColS + col0 + 32, sraw + 32);
          tmem_wait_ld();
          uint32_t ppk[32];
          const uint32_t vec = lse_u32 + slot * L::kVecBytes + col0 * 4;
          // One straight-line body per (soft-cap, masking) combination; the step picks one.
          // Masked entries and rows that saw no key (lse == mask_value) get an exponent of
          // -inf, i.e. P = 0.  FULL blocks without segment ids need neither test: a row whose
          // lse is mask_value never meets a FULL block.
          // Where the products fold lse in (head_dim 64, no soft-cap) the scores arrive with lse
          // already subtracted and rows that saw no key carry a large negative value: P = exp2(S^T log2e).
          auto body = [&](auto cap_c, auto mask_c) {
            constexpr bool kCap = decltype(cap_c)::value, kMask = decltype(mask_c)::value;
            constexpr bool kNeedLse = kCap || !L::kFold;
#pragma unroll
            for (int g = 0; g < 16; ++g) {
              float nl[4] = {0.f, 0.f, 0.f, 0.f};
              if constexpr (kNeedLse) {
                const uint4 lw = lds128(vec + g * 16);
                const uint32_t lraw[4] = {lw.x, lw.y, lw.z, lw.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float lse_e = __uint_as_float(lraw[e]);
                  nl[e] = lse_e * -kLog2e;
                  if constexpr (kMask) {
                    if (lse_e == a.mask_value) nl[e] = -INFINITY;
                  }
                }
              }
              float pv[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int i = g * 4 + e;
                float sval = pf[i], keep = 1.f;
                if constexpr (kCap) {
                  const float th = tanh_approx(sval * inv_cap);
                  sval = cap * th;
                  keep = fmaf(-th, th, 1.f);
                }
                float x = kNeedLse ? fmaf(sval, kLog2e, nl[e]) : sval * kLog2e;
                if constexpr (kMask) {
                  if (!((vis[i >> 5] >> (i & 31)) & 1u)) x = -INFINITY;
                }
                const float p = ex2_approx(x);
                pv[e] = p;
                pf[i] = kCap ? p * keep : p;
              }
              ppk[g * 2] = pack2<BF16>(pv[0], pv[1]);
              ppk[g * 2 + 1] = pack2<BF16>(pv[2], pv[3]);
            }
          };
          using T = std::true_type;
          using F = std::false_type;
          const bool masked = partial || seg_compare;
          if (!cap_on && !masked) body(F{}, F{});
          else if (!cap_on) body(F{}, T{});
          else if (!masked) body(T{}, F{});
          else body(T{}, T{});
          // Packed P^T goes over the first half of the columns this thread just read.
          tmem_st32(tmem_row + L::kColS + col0, ppk);
          tmem_wait_st();
          tc_fence_before();
          mbar_arrive(SPLASH_WBAR(p_ready, 0));
        }
        SPLASH_TRACE_MARK(1, t, 2);

        // ---- phase B: dS^T from dP^T ---------------------------------------------------
        if (!warp_wait(SPLASH_WBAR(dp_ready, 0), par, ctx, kWSiteEwDp, t)) { alive = false; break; }
        SPLASH_TRACE_MARK(1, t, 3);
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t dpraw[32];
          tmem_ld32(tmem_row + L::kColDp + col0 + c * 32, dpraw);
          tmem_wait_ld();
          uint32_t dspk[16];
          if constexpr (L::kFold) {
            // dP^T arrives with delta already subtracted.
#pragma unroll
            for (int g = 0; g < 8; ++g) {
              const int i = c * 32 + g * 4;
              dspk[g * 2] = pack2<BF16>(pf[i + 0] * __uint_as_float(dpraw[g * 4 + 0]),
                                        pf[i + 1] * __uint_as_float(dpraw[g * 4 + 1]));
              dspk[g * 2 + 1] = pack2<BF16>(pf[i + 2] * __uint_as_float(dpraw[g * 4 + 2]),
                                            pf[i + 3] * __uint_as_float(dpraw[g * 4 + 3]));
            }
          } else {
            const uint32_t vec = delta_u32 + slot * L::kVecBytes + (col0 + c * 32) * 4;
#pragma unroll
            for (int g = 0; g < 8; ++g) {
              const uint4 dw = lds128(vec + g * 16);
              const int i = c * 32 + g * 4;
              dspk[g * 2] = pack2<BF16>(pf[i + 0] * (__uint_as_float(dpraw[g * 4 + 0]) - __uint_as_float(dw.x)),
                                        pf[i + 1] * (__uint_as_float(dpraw[g * 4 + 1]) - __uint_as_float(dw.y)));
              dspk[g * 2 + 1] = pack2<BF16>(pf[i + 2] * (__uint_as_float(dpraw[g * 4 + 2]) - __uint_as_float(dw.z)),
                                            pf[i + 3] * (__uint_as_float(dpraw[g * 4 + 3]) - __uint_as_float(dw.w)));
            }
          }
          tmem_st16(tmem_row + L::kColDp + col0 + c * 16, dspk);
          // dS^T staged as [kv row][q], two boxes of 64 q columns, 128-byte swizzle.
#pragma unroll
          for (int g = 0; g < 4; ++g)
            sts128(ds_u32 + w * L::kBox + swz128(row, c * 4 + g),
                   make_uint4(dspk[g * 4], dspk[g * 4 + 1], dspk[g * 4 + 2], dspk[g * 4 + 3]));
        }
        // The slot's vectors have been read.
        __syncwarp();
        if (lane == 0) mbar_arrive(SPLASH_WBAR(q_empty, slot));
        tmem_wait_st();
        fence_proxy_async_smem();
        tc_fence_before();
        mbar_arrive(SPLASH_WBAR(ds_ready, 0));
        SPLASH_TRACE_MARK(1, t, 4);
      }

      // ---- epilogue: dK by warpgroup 0, dV by warpgroup 1 ---------------------------
      if (alive) alive = warp_wait(SPLASH_WBAR(acc_done, 0), 0, ctx, kWSiteEwDone, total);
      if (alive) {
        tc_fence_after();
        const uint32_t stage = w == 0 ? k_u32 : v_u32;  // K / V tiles are dead once every MMA has finished
        const uint32_t acc_tmem = tmem_row + (w == 0 ? L::kColDk : L::kColDv);
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t o[32];
          tmem_ld32(acc_tmem + c * 32, o);
          tmem_wait_ld();
          const uint32_t box = stage + (c / 2) * L::kBox;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 wv;
            wv.x = pack2<BF16>(__uint_as_float(o[g * 8 + 0]), __uint_as_float(o[g * 8 + 1]));
            wv.y = pack2<BF16>(__uint_as_float(o[g * 8 + 2]), __uint_as_float(o[g * 8 + 3]));
            wv.z = pack2<BF16>(__uint_as_float(o[g * 8 + 4]), __uint_as_float(o[g * 8 + 5]));
            wv.w = pack2<BF16>(__uint_as_float(o[g * 8 + 6]), __uint_as_float(o[g * 8 + 7]));
            sts128(box + swz128(row, (c & 1) * 4 + g), wv);
          }
        }
        fence_proxy_async_smem();
        mbar_arrive(SPLASH_WBAR(epi, w));
        if (row == 0) {
          if (mbar_wait(SPLASH_WBAR(epi, w), 0, ctx, kWSiteEwEpi, total)) {
#pragma unroll
            for (int c = 0; c < D / 64; ++c) tma_store_2d(w == 0 ? &tm_dk : &tm_dv, stage + c * L::kBox, c * 64, kv_row0);
            bulk_commit_group();
            bulk_wait_group_read<0>();
          }
        }
      }
    }
  }

  // ---- teardown ---------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (const uint32_t gave_up = lds32(abort_u32)) {
    if (threadIdx.x == 0) report_abort(a.status, gave_up);
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000) {}
  }
  if (warp == kProducerWarp0 + 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem, L::kTmemCols);
  }
}

#undef SPLASH_WBAR

}  // namespace splash
