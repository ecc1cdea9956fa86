// Splash attention forward for sm_100a: one warp-specialised kernel template that
// covers the forward variants.
//
//   NT = 1, AW = 1  one 128-row q tile per CTA, one softmax warpgroup.  The two S
//           buffers in tensor memory alternate between KV steps, so Q.K^T of step
//           s+1 runs while the warpgroup works on step s.  With 64-wide KV blocks and
//           a two-stage ring two such CTAs share an SM.
//   NT = 1, AW = 2  the same tile with two softmax warpgroups that take the KV steps
//           in turn (128-wide KV blocks).  The groups hand the stale row maximum to
//           one another through shared memory, keep partial row sums and split the
//           epilogue; P has tensor-memory columns of its own, so the S buffer of step
//           s is free as soon as its softmax has read it and Q.K^T of step s+2 runs
//           under the softmax of step s.
//   NT = 2  two 128-row q tiles per CTA ("ping-pong").  Each tile has its own S
//           buffer and its own softmax warpgroup; every K/V block fetched is
//           used by both tiles, and the tensor core works for one tile while the
//           other tile's softmax runs.
//
// Roles inside a CTA
//   softmax warpgroups    warps [0, 4*NT*AW): one thread per q row (= TMEM lane)
//   K/Q producer          next warp: Q once, then K (+ KV segment ids, + the int8 block
//                         of a dense partial mask) per visited block
//   MMA issuer            next warp: all tcgen05.mma / commit, one elected lane
//   V producer            next warp: V per visited block
//
// Data flow per visited KV block:  S = Q K^T (smem x smem -> TMEM f32), softmax in
// registers (exp2 domain, running max kept stale until it moves by more than 2^8),
// P written to tensor memory as packed 16-bit (over S, or into its own columns with
// AW = 2), O += P V (TMEM x smem -> TMEM f32).
// Empty blocks are never touched, FULL blocks skip masking, PARTIAL blocks are
// masked in registers from a band descriptor or a dense int8 block.
//
// Behaviour follows the reference kernels (splash_attention_mgpu/kernel.py:132-537,
// forward_pingpong.py:131-681); the code shares nothing with them.
#pragma once

#include <stddef.h>


#include "../../include/splash_sm100.h"
#include "ptx.cuh"
#include "seg_skip.cuh"

// Timeline marks for debugging builds; empty in the product.
#ifndef SPLASH_TRACE_MARK
#define SPLASH_TRACE_MARK(role, t, k)
#define SPLASH_TRACE_NS(role, t, k)
#endif

namespace splash {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRescaleThreshold = 8.0f;  // in powers of two

struct FwdArgs {
  const int32_t* num_steps;
  const int32_t* block_order;
  const int32_t* block_list;
  const int32_t* block_kind;
  const int32_t* mask_block;
  const int32_t* mask_desc;
  const int32_t* seg_q;
  const int32_t* seg_kv;
  const uint8_t* partial_blocks;  // bit-packed dense partial blocks [n, block_q, block_kv / 8], or null
  const int2* seg_q_ranges;   // [batch, q_len / 64] (min, max) segment ids, or null: no block skipping
  const int2* seg_kv_ranges;  // [batch, kv_len / 64]
  void* out;
  float* lse_out;
  int32_t* status;
  int32_t batch, heads, kv_heads, q_len, kv_len;
  int32_t mask_heads, max_steps, q_blocks, stages;
  int32_t has_dense, has_seg;
  int32_t head_group;  // heads whose blocks are interleaved in the launch order
  float mask_value, soft_cap;
};

// Wait sites, reported in the status word when a wait runs out.
enum FwdSite : int {
  kSiteTmaKEmpty = 1, kSiteTmaVEmpty, kSiteTmaAuxEmpty,
  kSiteMmaQ, kSiteMmaK, kSiteMmaV, kSiteMmaP, kSiteMmaSFree,
  kSiteSmxS, kSiteSmxAux, kSiteSmxPv, kSiteSmxDone, kSiteSmxEpi, kSiteSmxM, kSiteSmxFin,
};

// AW softmax warpgroups take the KV steps of a tile in turn (one-tile kernel only).
template <int D, int DV, int BKV, int NT, int AW = 1>
struct FwdLayout {
  static_assert(AW == 1 || (AW == 2 && NT == 1), "alternating warpgroups need the one-tile kernel");
  static constexpr int kTile = 128;
  static constexpr int kQBytes = NT * kTile * D * 2;
  static constexpr int kKStage = BKV * D * 2;
  static constexpr int kVStage = BKV * DV * 2;
  static constexpr int kMaskStage = NT * kTile * BKV / 8;  // one bit per element
  static constexpr int kSegStage = BKV * 4;
  // Tensor-memory columns: S (two buffers) | P when it has columns of its own | O.
  // P lies over its S except with alternating warpgroups, where freeing S(t) as soon as
  // it has been read lets the scores of step t + 2 run under the softmax of step t.
  static constexpr int kPCol = AW == 2 ? 2 * BKV : 0;     // first column of P buffer 0
  static constexpr int kPStride = AW == 2 ? BKV / 2 : BKV;  // from P buffer 0 to buffer 1
  static constexpr int kOCol = AW == 2 ? 3 * BKV : 2 * BKV;
  static constexpr int kTmemUsed = kOCol + NT * DV;
  static constexpr int kTmemCols = kTmemUsed <= 128 ? 128 : (kTmemUsed <= 256 ? 256 : 512);
  static_assert(kTmemUsed <= 512, "tensor memory has 512 columns");
  static constexpr int kSoftmaxGroups = NT * AW;
  static constexpr int kThreads = (kSoftmaxGroups + 1) * 128;
  // Row maxima shared by the alternating warpgroups, and their partial row sums.
  static constexpr int kShareBytes = AW > 1 ? 3 * kTile * 4 : 0;
  static constexpr bool kOStageInQ = (NT == 2) || (DV <= D);
  // Register split between the warpgroups when there are two softmax warpgroups
  // (multiples of 8; 2 * 128 * softmax + 128 * producer <= 64K).
  static constexpr bool kSplitRegs = kSoftmaxGroups == 2;
  static constexpr int kSoftmaxRegs = 216;
  static constexpr int kProducerRegs = 72;

  // `list_steps`: capacity of the list of steps that survive segment skipping (0 = no list).
  __host__ __device__ static size_t smem_bytes(int stages, bool dense, bool seg, int list_steps = 0) {
    size_t b = 1024;  // alignment slack
    b += kQBytes + static_cast<size_t>(stages) * (kKStage + kVStage);
    if (dense) b += static_cast<size_t>(stages) * kMaskStage;
    if (seg) b += static_cast<size_t>(stages) * kSegStage;
    b += 1024;  // barriers, TMEM slot, flags
    b += kShareBytes;
    b += (static_cast<size_t>(list_steps) * 2 + 15) & ~static_cast<size_t>(15);
    return b;
  }
};

constexpr int kFwdMaxStages = 8;

struct FwdBarriers {
  uint64_t q_full;
  uint64_t k_full[kFwdMaxStages], k_empty[kFwdMaxStages];
  uint64_t v_full[kFwdMaxStages], v_empty[kFwdMaxStages];
  uint64_t aux_full[kFwdMaxStages], aux_empty[kFwdMaxStages];
  uint64_t s_ready[2], p_ready[2];
  uint64_t pv_done[2], o_done;  // pv_done by step parity: a waiter meets every phase of a barrier in turn
  uint64_t epi[2];
  uint64_t s_free[2];   // alternating warpgroups: S buffer read into registers
  uint64_t m_ready[2];  // alternating warpgroups: the row maxima after step s stand in shared memory
  uint64_t fin;         // alternating warpgroups: partial row sums posted
  uint32_t tmem_base;
  uint32_t abort_flag;
  uint32_t dead;
  uint32_t n_eff;  // steps left after segment skipping
};

#define SPLASH_BAR(field, idx) \
  (bars_u32 + static_cast<uint32_t>(offsetof(FwdBarriers, field)) + 8u * static_cast<uint32_t>(idx))

// PLAIN: no soft-cap, no segment ids, no streamed mask blocks -- those blocks of the
// softmax loop are compiled out, which shortens the instruction stream of the common case.
template <int D, int DV, int BKV, int NT, int AW, bool PLAIN, bool BF16>
__global__ void __launch_bounds__((NT * AW + 1) * 128, 1)
splash_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                  const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                  const FwdArgs a) {
  using L = FwdLayout<D, DV, BKV, NT, AW>;
  constexpr int kTile = 128;
  constexpr int kBq = NT * kTile;
  constexpr int kSoftmaxWarps = 4 * NT * AW;

  const bool has_dense = !PLAIN && a.has_dense;
  const bool has_seg = !PLAIN && a.has_seg;
  const float soft_cap = PLAIN ? 0.f : a.soft_cap;
  extern __shared__ uint8_t smem_raw[];
  const int stages = a.stages;
  // Shared-window addresses (32-bit) of the buffers; tiles are 1024-byte aligned.
  const uint32_t q_u32 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t k_u32 = q_u32 + L::kQBytes;
  const uint32_t v_u32 = k_u32 + stages * L::kKStage;
  const uint32_t mask_u32 = v_u32 + stages * L::kVStage;
  const uint32_t seg_u32 = mask_u32 + (has_dense ? stages * L::kMaskStage : 0);
  const uint32_t bars_u32 = seg_u32 + (has_seg ? stages * L::kSegStage : 0);
  const uint32_t share_u32 = bars_u32 + 1024;  // [row maxima | partial sums of group 0 | of group 1]
  const uint32_t abort_u32 = bars_u32 + static_cast<uint32_t>(offsetof(FwdBarriers, abort_flag));
  const uint32_t tmem_slot_u32 = bars_u32 + static_cast<uint32_t>(offsetof(FwdBarriers, tmem_base));
  const uint32_t dead_u32 = bars_u32 + static_cast<uint32_t>(offsetof(FwdBarriers, dead));
  const uint32_t neff_u32 = bars_u32 + static_cast<uint32_t>(offsetof(FwdBarriers, n_eff));
  const uint32_t list_u32 = share_u32 + L::kShareBytes;  // surviving steps, 16 bits each
  const bool has_list = has_seg && a.seg_q_ranges != nullptr;

  const int warp = uniform_warp_index();
  const int lane = threadIdx.x & 31;

  // ---- which tile of work ---------------------------------------------------
  int hb, order_idx;
  decode_work_item(blockIdx.x, a.q_blocks, a.heads * a.batch, a.head_group, hb, order_idx);
  const int h = hb % a.heads;
  const int b = hb / a.heads;
  const int mh = a.mask_heads > 1 ? h : 0;
  const int qi = a.block_order[mh * a.q_blocks + order_idx];
  const int n_sched = a.num_steps[mh * a.q_blocks + qi];
  const bool has_aux = has_dense || has_seg;
  const int sched_off = (mh * a.q_blocks + qi) * a.max_steps;  // offset into the step lists
  const int q_row0 = (b * a.heads + h) * a.q_len + qi * kBq;   // row in the [B*H*Sq, D] view

  // ---- set-up -----------------------------------------------------------------
  // One warp initialises the barriers, a lane each, while the MMA warp allocates tensor
  // memory; one CTA barrier later every role starts.  A launch that finds the status
  // word already set (an earlier kernel gave up a wait) returns without touching data; one
  // thread reads the word and shares it, so every role of the CTA takes the same branch.
  if (warp == 0) {
    constexpr uint32_t kNumBarriers = offsetof(FwdBarriers, tmem_base) / 8;
    for (uint32_t i = lane; i < kNumBarriers; i += 32) {
      const uint32_t off = 8u * i;
      uint32_t count = 1;
      if (off >= offsetof(FwdBarriers, aux_empty) && off < offsetof(FwdBarriers, s_ready)) count = 4 * NT;  // the warps that consume one step
      if (off >= offsetof(FwdBarriers, p_ready) && off < offsetof(FwdBarriers, pv_done)) count = kTile;
      if (off >= offsetof(FwdBarriers, epi) && off < offsetof(FwdBarriers, s_free)) count = kTile * AW;
      if (off >= offsetof(FwdBarriers, s_free) && off < offsetof(FwdBarriers, fin)) count = kTile;  // s_free, m_ready
      if (off == offsetof(FwdBarriers, fin)) count = kTile * AW;
      mbar_init(bars_u32 + off, count);
    }
    if (lane == 0) {
      sts32(abort_u32, 0);
      sts32(dead_u32, a.status[0] != 0);
    }
    fence_mbar_init();
    fence_proxy_async_smem();
  } else if (warp == kSoftmaxWarps + 1) {
    tmem_alloc(tmem_slot_u32, L::kTmemCols);
    tmem_relinquish();
  } else if (warp == 1 && has_list) {
    // Steps whose q and kv segment-id ranges can meet; the others are left out by every role.
    const int2* qt = a.seg_q_ranges + static_cast<size_t>(b) * (a.q_len / kSegChunk);
    const int2* kt = a.seg_kv_ranges + static_cast<size_t>(b) * (a.kv_len / kSegChunk);
    const SegRange qr = seg_range(qt, qi * (kBq / kSegChunk), kBq / kSegChunk);
    const int kept = build_step_list(list_u32, n_sched, lane, [&](int s) {
      const int j = a.block_list[sched_off + s];
      return seg_classify(qr, seg_range(kt, j * (BKV / kSegChunk), BKV / kSegChunk));
    });
    if (lane == 0) sts32(neff_u32, static_cast<uint32_t>(kept));
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = lds32(tmem_slot_u32);
  const WaitCtx ctx{abort_u32};
  const int n = has_list ? static_cast<int>(lds32(neff_u32)) : n_sched;
  // Entry e of the CTA's step sequence: index into the schedule lists, and whether the
  // block needs no segment comparison.
  auto step_at = [&](int e) -> uint32_t { return has_list ? lds16(list_u32 + 2u * e) : static_cast<uint32_t>(e); };
  if (lds32(dead_u32)) {
    if (warp == kSoftmaxWarps + 1) {
      __syncwarp();
      tmem_dealloc(tmem, L::kTmemCols);
    }
    return;
  }

  constexpr uint32_t kIdescQK = make_idesc(BF16, 128, BKV, false, false);
  constexpr uint32_t kIdescPV = make_idesc(BF16, 128, DV, false, true);
  constexpr uint32_t kDescHi = desc_hi(1024);

  if (warp >= kSoftmaxWarps) {
    // =========================== producer warpgroup ============================
    if constexpr (L::kSplitRegs) setmaxnreg_dec<L::kProducerRegs>();
    if (warp == kSoftmaxWarps && n > 0) {
      // ------------------------------ TMA producer ------------------------------
      // The whole warp runs the loop (warp-uniform control flow); one elected lane
      // issues each group of copies.
      const int kv_row0 = (b * a.kv_heads + h / (a.heads / a.kv_heads)) * a.kv_len;
      if (elect_one()) {
        prefetch_tensormap(&tm_q);
        prefetch_tensormap(&tm_k);
        mbar_arrive_expect_tx(SPLASH_BAR(q_full, 0), L::kQBytes);
#pragma unroll
        for (int t = 0; t < NT; ++t)
#pragma unroll
          for (int c = 0; c < D / 64; ++c)
            tma_load_2d(q_u32 + t * (kTile * D * 2) + c * (kTile * 128), &tm_q, c * 64, q_row0 + t * kTile,
                        SPLASH_BAR(q_full, 0));
      }
      int slot = 0;
      uint32_t phase = 0;
      int st_next = static_cast<int>(step_at(0) & 0x7fffu);
      int j_next = a.block_list[sched_off + st_next];
      for (int s = 0; s < n; ++s) {
        const int j = j_next, st = st_next;
        if (s + 1 < n) {
          st_next = static_cast<int>(step_at(s + 1) & 0x7fffu);
          j_next = a.block_list[sched_off + st_next];
        }
        const int kv_row = kv_row0 + j * BKV;
        if (s >= stages && !warp_wait(SPLASH_BAR(k_empty, slot), phase ^ 1, ctx, kSiteTmaKEmpty, s)) break;
        if (elect_one()) {
          mbar_arrive_expect_tx(SPLASH_BAR(k_full, slot), L::kKStage);
#pragma unroll
          for (int c = 0; c < D / 64; ++c)
            tma_load_2d(k_u32 + slot * L::kKStage + c * (BKV * 128), &tm_k, c * 64, kv_row, SPLASH_BAR(k_full, slot));
        }
        if (has_aux) {
          if (s >= stages && !warp_wait(SPLASH_BAR(aux_empty, slot), phase ^ 1, ctx, kSiteTmaAuxEmpty, s)) break;
          const bool partial_dense = has_dense && a.block_kind[sched_off + st] == SPLASH_BLOCK_PARTIAL;
          const uint32_t bytes = (has_seg ? L::kSegStage : 0) + (partial_dense ? L::kMaskStage : 0);
          const size_t mblock = partial_dense ? static_cast<size_t>(a.mask_block[sched_off + st]) : 0;
          if (elect_one()) {
            mbar_arrive_expect_tx(SPLASH_BAR(aux_full, slot), bytes);
            if (has_seg)
              bulk_load_1d(seg_u32 + slot * L::kSegStage, a.seg_kv + static_cast<size_t>(b) * a.kv_len + j * BKV,
                           L::kSegStage, SPLASH_BAR(aux_full, slot));
            if (partial_dense)
              bulk_load_1d(mask_u32 + slot * L::kMaskStage, a.partial_blocks + mblock * L::kMaskStage, L::kMaskStage,
                           SPLASH_BAR(aux_full, slot));
          }
        }
        if (++slot == stages) { slot = 0; phase ^= 1; }
      }
    } else if (warp == kSoftmaxWarps + 2 && n > 0) {
      // ------------------------------ V producer --------------------------------
      // A warp of its own, so that a V slot still held by P.V never delays the K
      // blocks behind it, which the tensor core needs first.
      const int kv_row0 = (b * a.kv_heads + h / (a.heads / a.kv_heads)) * a.kv_len;
      if (elect_one()) prefetch_tensormap(&tm_v);
      int slot = 0;
      uint32_t phase = 0;
      int j_next = a.block_list[sched_off + (step_at(0) & 0x7fffu)];
      for (int s = 0; s < n; ++s) {
        const int kv_row = kv_row0 + j_next * BKV;
        if (s + 1 < n) j_next = a.block_list[sched_off + (step_at(s + 1) & 0x7fffu)];
        if (s >= stages && !warp_wait(SPLASH_BAR(v_empty, slot), phase ^ 1, ctx, kSiteTmaVEmpty, s)) break;
        if (elect_one()) {
          mbar_arrive_expect_tx(SPLASH_BAR(v_full, slot), L::kVStage);
#pragma unroll
          for (int c = 0; c < DV / 64; ++c)
            tma_load_2d(v_u32 + slot * L::kVStage + c * (BKV * 128), &tm_v, c * 64, kv_row, SPLASH_BAR(v_full, slot));
        }
        if (++slot == stages) { slot = 0; phase ^= 1; }
      }
    } else if (warp == kSoftmaxWarps + 1 && n > 0) {
      // ------------------------------- MMA issuer -------------------------------
      // All lanes run the loop; one elected lane issues each instruction.
      // S_t = Q_t K^T: both operands K-major, 64-element (128-byte) boxes side by side.
      auto issue_qk = [&](int t, int kslot, uint32_t s_dst) {
        const uint32_t a_lo = desc_lo(q_u32 + t * (kTile * D * 2), 16);
        const uint32_t b_lo = desc_lo(k_u32 + kslot * L::kKStage, 16);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t ao = ((kk / 4) * (kTile * 128) + (kk % 4) * 32) >> 4;
          const uint32_t bo = ((kk / 4) * (BKV * 128) + (kk % 4) * 32) >> 4;
          umma_ss2_w(s_dst, a_lo + ao, kDescHi, b_lo + bo, kDescHi, kIdescQK, kk > 0);
        }
      };
      // O_t (+)= P_t V: P from tensor memory (8 columns per 16 keys), V MN-major.
      auto issue_pv = [&](int t, int vslot, uint32_t p_src, uint32_t acc) {
        const uint32_t b_lo = desc_lo(v_u32 + vslot * L::kVStage, BKV * 128);
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk)
          umma_ts2_w(tmem + L::kOCol + t * DV, p_src + kk * 8, b_lo + ((kk * 2048) >> 4), kDescHi, kIdescPV,
                   kk > 0 ? 1u : acc);
      };
      bool ok = warp_wait(SPLASH_BAR(q_full, 0), 0, ctx, kSiteMmaQ, 0) &&
                warp_wait(SPLASH_BAR(k_full, 0), 0, ctx, kSiteMmaK, 0);
      if (ok) {
        tc_fence_after();
        issue_qk(0, 0, tmem);
        umma_commit_w(SPLASH_BAR(s_ready, 0));
        if constexpr (NT == 2) {
          issue_qk(1, 0, tmem + BKV);
          umma_commit_w(SPLASH_BAR(s_ready, 1));
        }
        umma_commit_w(SPLASH_BAR(k_empty, 0));
        int slot = 0;
        uint32_t phase = 0;
        if constexpr (AW == 2) {
          // The scores run two steps ahead of P.V: S(s + 2) goes into the buffer that the
          // softmax of step s has read into registers, under that softmax.
          int ks = 1;  // K ring position of the next scores to issue (stages >= 2)
          uint32_t kp = 0;
          if (n > 1) {
            ok = warp_wait(SPLASH_BAR(k_full, ks), kp, ctx, kSiteMmaK, 1);
            if (ok) {
              tc_fence_after();
              issue_qk(0, ks, tmem + BKV);
              umma_commit_w(SPLASH_BAR(s_ready, 1));
              umma_commit_w(SPLASH_BAR(k_empty, ks));
              if (++ks == stages) { ks = 0; kp ^= 1; }
            }
          }
          for (int s = 0; s < n && ok; ++s) {
            const int cur = s & 1;
            const uint32_t par = (s >> 1) & 1;
            SPLASH_TRACE_MARK(0, s, 0);
            if (s + 2 < n) {
              if (!warp_wait(SPLASH_BAR(k_full, ks), kp, ctx, kSiteMmaK, s + 2)) break;
              SPLASH_TRACE_MARK(0, s, 1);
              if (!warp_wait(SPLASH_BAR(s_free, cur), par, ctx, kSiteMmaSFree, s)) break;
              SPLASH_TRACE_MARK(0, s, 2);
              tc_fence_after();
              issue_qk(0, ks, tmem + cur * BKV);
              umma_commit_w(SPLASH_BAR(s_ready, cur));
              umma_commit_w(SPLASH_BAR(k_empty, ks));
              if (++ks == stages) { ks = 0; kp ^= 1; }
            }
            SPLASH_TRACE_MARK(0, s, 3);
            if (!warp_wait(SPLASH_BAR(v_full, slot), phase, ctx, kSiteMmaV, s)) break;
            SPLASH_TRACE_MARK(0, s, 4);
            if (!warp_wait(SPLASH_BAR(p_ready, cur), par, ctx, kSiteMmaP, s)) break;
            SPLASH_TRACE_MARK(0, s, 5);
            tc_fence_after();
            issue_pv(0, slot, tmem + L::kPCol + cur * L::kPStride, s > 0);
            umma_commit_w(SPLASH_BAR(v_empty, slot));
            umma_commit_w(SPLASH_BAR(pv_done, cur));
            if (++slot == stages) { slot = 0; phase ^= 1; }
          }
        } else
        for (int s = 0; s < n; ++s) {
          int slot1 = slot + 1;
          uint32_t phase1 = phase;
          if (slot1 == stages) { slot1 = 0; phase1 ^= 1; }
          const bool next = s + 1 < n;
          if constexpr (NT == 1) {
            const int cur = s & 1;
            if (next) {
              if (!warp_wait(SPLASH_BAR(k_full, slot1), phase1, ctx, kSiteMmaK, s + 1)) break;
              tc_fence_after();
              issue_qk(0, slot1, tmem + (cur ^ 1) * BKV);
              umma_commit_w(SPLASH_BAR(s_ready, cur ^ 1));
              umma_commit_w(SPLASH_BAR(k_empty, slot1));
            }
            if (!warp_wait(SPLASH_BAR(v_full, slot), phase, ctx, kSiteMmaV, s)) break;
            if (!warp_wait(SPLASH_BAR(p_ready, cur), (s >> 1) & 1, ctx, kSiteMmaP, s)) break;
            tc_fence_after();
            issue_pv(0, slot, tmem + cur * BKV, s > 0);
            umma_commit_w(SPLASH_BAR(v_empty, slot));
            umma_commit_w(SPLASH_BAR(pv_done, cur));
          } else {
            if (!warp_wait(SPLASH_BAR(v_full, slot), phase, ctx, kSiteMmaV, s)) break;
            if (!warp_wait(SPLASH_BAR(p_ready, 0), s & 1, ctx, kSiteMmaP, s)) break;
            tc_fence_after();
            issue_pv(0, slot, tmem, s > 0);
            if (next) {
              if (!warp_wait(SPLASH_BAR(k_full, slot1), phase1, ctx, kSiteMmaK, s + 1)) break;
              tc_fence_after();
              issue_qk(0, slot1, tmem);
              umma_commit_w(SPLASH_BAR(s_ready, 0));
            }
            if (!warp_wait(SPLASH_BAR(p_ready, 1), s & 1, ctx, kSiteMmaP, s)) break;
            tc_fence_after();
            issue_pv(1, slot, tmem + BKV, s > 0);
            umma_commit_w(SPLASH_BAR(v_empty, slot));
            if (next) {
              issue_qk(1, slot1, tmem + BKV);
              umma_commit_w(SPLASH_BAR(s_ready, 1));
              umma_commit_w(SPLASH_BAR(k_empty, slot1));
            }
          }
          slot = slot1;
          phase = phase1;
        }
        if constexpr (NT == 2) umma_commit_w(SPLASH_BAR(o_done, 0));
      }
    }
  } else {
    // ============================ softmax warpgroups ============================
    if constexpr (L::kSplitRegs) setmaxnreg_inc<L::kSoftmaxRegs>();
    // Two tiles: warpgroup g owns tile g.  One tile with AW warpgroups: group g takes the
    // KV steps g, g + AW, ... of the tile, so that AW steps are in the softmax at a time;
    // the groups pass the (stale) row maxima to one another through shared memory, keep
    // partial row sums, and split the columns of O in the epilogue.
    const int grp = warp >> 2;
    const int t = (NT == 2) ? grp : 0;             // which q tile
    const int row = (warp & 3) * 32 + lane;        // row inside the tile
    const int q_pos = qi * kBq + t * kTile + row;  // position in the sequence
    // TMEM address of this thread's lane quarter, column 0.
    const uint32_t tmem_row = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    const uint32_t o_tmem = tmem_row + L::kOCol + t * DV;
    const uint32_t m_sh = share_u32 + row * 4;                    // the row's maximum after the latest step
    const uint32_t l_sh = share_u32 + (1 + grp) * kTile * 4 + row * 4;  // this group's partial row sum
    constexpr int kEpiCols = DV / AW;                             // columns of O per thread in the epilogue
    const int epi_col0 = (AW == 2) ? grp * kEpiCols : 0;

    if (n == 0) {
      // No visible block: zeros and lse = mask_value, nothing else runs.
      const size_t out_row = static_cast<size_t>(q_row0) + t * kTile + row;
      const uint4 z = make_uint4(0, 0, 0, 0);
      uint4* dst = reinterpret_cast<uint4*>(static_cast<uint8_t*>(a.out) + out_row * (DV * 2)) + epi_col0 * 2 / 16;
#pragma unroll
      for (int c = 0; c < kEpiCols * 2 / 16; ++c) dst[c] = z;
      if (a.lse_out && epi_col0 == 0) a.lse_out[out_row] = a.mask_value;
    } else {
      // Per-row band in units of (kv_pos - q_pos); a chunk restriction folds in.
      int band_lo = -(1 << 30), band_hi = (1 << 30);
      if (a.mask_desc) {
        band_lo = a.mask_desc[mh * 4 + 0];
        band_hi = a.mask_desc[mh * 4 + 1];
        const int chunk = a.mask_desc[mh * 4 + 2];
        if (chunk > 0) {
          const int start = (q_pos / chunk) * chunk;
          band_lo = max(band_lo, start - q_pos);
          band_hi = min(band_hi, start + chunk - 1 - q_pos);
        }
      }
      const int my_seg = has_seg ? a.seg_q[static_cast<size_t>(b) * a.q_len + q_pos] : 0;

      float m_run = -INFINITY;  // stale running max, raw logit units
      float l_run = 0.f;
      const int s_first = (AW == 2) ? grp : 0;
      int slot = s_first % stages;
      uint32_t phase = (s_first / stages) & 1;
      uint32_t entry = s_first < n ? step_at(s_first) : 0u;
      int kind = s_first < n ? a.block_kind[sched_off + (entry & 0x7fffu)] : 0;
      int jblk = s_first < n ? a.block_list[sched_off + (entry & 0x7fffu)] : 0;
      bool alive = true;
      float sv[BKV];  // the current row of S
      auto load_row = [&](int buf, uint32_t par, int step) {
        if (!warp_wait(SPLASH_BAR(s_ready, buf), par, ctx, kSiteSmxS, step)) return false;
        tc_fence_after();
        uint32_t* raw = reinterpret_cast<uint32_t*>(sv);
#pragma unroll
        for (int c = 0; c < BKV / 32; ++c) tmem_ld32(tmem_row + buf * BKV + c * 32, raw + c * 32);
        return true;
      };

      for (int s = s_first; s < n; s += AW) {
        const int kind_now = kind, j_now = jblk;
        const bool seg_compare = has_seg && !(entry & kSegUniformBit);
        if (s + AW < n) {
          entry = step_at(s + AW);
          kind = a.block_kind[sched_off + (entry & 0x7fffu)];
          jblk = a.block_list[sched_off + (entry & 0x7fffu)];
        }
        const int buf = (NT == 2) ? t : (s & 1);
        const uint32_t par = (NT == 2) ? (s & 1) : ((s >> 1) & 1);
        const uint32_t p_tmem = tmem_row + L::kPCol + buf * L::kPStride;
        if ((warp & 3) == 0) { SPLASH_TRACE_MARK(1 + grp, s, 0); SPLASH_TRACE_NS(1 + grp, s, 7); }
        if (!load_row(buf, par, s)) { alive = false; break; }
        tmem_wait_ld();
        if ((warp & 3) == 0) SPLASH_TRACE_MARK(1 + grp, s, 1);
        if constexpr (AW == 2) {
          // The row is in registers: the tensor core may write the scores of step s + 2.
          tc_fence_before();
          mbar_arrive(SPLASH_BAR(s_free, buf));
        }
        if (soft_cap > 0.f) {
          const float cap = soft_cap, inv_cap = 1.f / soft_cap;
#pragma unroll
          for (int i = 0; i < BKV; ++i) sv[i] = cap * tanh_approx(sv[i] * inv_cap);
        }
        if (has_aux) {
          if (!warp_wait(SPLASH_BAR(aux_full, slot), phase, ctx, kSiteSmxAux, s)) { alive = false; break; }
        }
        const bool partial = kind_now == SPLASH_BLOCK_PARTIAL;
        if (partial && !has_dense) {
          const int d0 = j_now * BKV - q_pos;
#pragma unroll
          for (int i = 0; i < BKV; ++i) {
            const int d = d0 + i;
            if (d < band_lo || d > band_hi) sv[i] = -INFINITY;
          }
        }
        if (partial && has_dense) {
          // One bit per element, BKV / 8 bytes per q row, rows of the tile(s) back to back.
          const uint32_t mrow = mask_u32 + slot * L::kMaskStage + (t * kTile + row) * (BKV / 8);
          uint32_t bits[BKV / 32];
          if constexpr (BKV == 128) {
            const uint4 w = lds128(mrow);
            bits[0] = w.x; bits[1] = w.y; bits[2] = w.z; bits[3] = w.w;
          } else {
            bits[0] = lds32(mrow);
            bits[1] = lds32(mrow + 4);
          }
#pragma unroll
          for (int i = 0; i < BKV; ++i)
            if (!((bits[i >> 5] >> (i & 31)) & 1u)) sv[i] = -INFINITY;
        }
        if (seg_compare) {
          const uint32_t segs = seg_u32 + slot * L::kSegStage;
#pragma unroll
          for (int c = 0; c < BKV / 4; ++c) {
            const uint4 g = lds128(segs + c * 16);
            if (static_cast<int>(g.x) != my_seg) sv[c * 4 + 0] = -INFINITY;
            if (static_cast<int>(g.y) != my_seg) sv[c * 4 + 1] = -INFINITY;
            if (static_cast<int>(g.z) != my_seg) sv[c * 4 + 2] = -INFINITY;
            if (static_cast<int>(g.w) != my_seg) sv[c * 4 + 3] = -INFINITY;
          }
        }
        if (has_aux) {
          __syncwarp();
          if (lane == 0) mbar_arrive(SPLASH_BAR(aux_empty, slot));
        }

        // ---- online softmax with a stale maximum --------------------------------
        if ((warp & 3) == 0) SPLASH_TRACE_MARK(1 + grp, s, 6);
        float mx0 = max3(sv[0], sv[1], sv[2]), mx1 = max3(sv[3], sv[4], sv[5]);
        float mx2 = fmaxf(sv[6], sv[7]), mx3 = sv[8];
#pragma unroll
        for (int i = 9; i + 7 < BKV; i += 8) {
          mx0 = max3(mx0, sv[i], sv[i + 1]);
          mx1 = max3(mx1, sv[i + 2], sv[i + 3]);
          mx2 = max3(mx2, sv[i + 4], sv[i + 5]);
          mx3 = max3(mx3, sv[i + 6], sv[i + 7]);
        }
        // BKV = 64 or 128: elements BKV-7 .. BKV-1 remain.
        mx0 = max3(mx0, sv[BKV - 7], sv[BKV - 6]);
        mx1 = max3(mx1, sv[BKV - 5], sv[BKV - 4]);
        mx2 = max3(mx2, sv[BKV - 3], sv[BKV - 2]);
        mx3 = fmaxf(mx3, sv[BKV - 1]);
        if constexpr (AW == 2) {
          // The maximum the previous step settled on (the other group's); this group's
          // partial sum moves to that scale first.
          if (s > 0) {
            if (!warp_wait(SPLASH_BAR(m_ready, (s - 1) & 1), ((s - 1) >> 1) & 1, ctx, kSiteSmxM, s)) { alive = false; break; }
            const float m_prev = __uint_as_float(lds32(m_sh));
            if (m_prev != m_run) {
              l_run = (m_run == -INFINITY) ? 0.f : l_run * ex2_approx((m_run - m_prev) * kLog2e);
              m_run = m_prev;
            }
          }
        }
        if ((warp & 3) == 0) SPLASH_TRACE_MARK(1 + grp, s, 2);
        const float m_new = fmaxf(m_run, fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)));
        const bool moved = (m_new - m_run) * kLog2e > kRescaleThreshold;  // false for NaN (-inf - -inf)
        float alpha = 1.f;
        if (moved) {
          alpha = ex2_approx((m_run - m_new) * kLog2e);  // 0 when m_run was -inf
          m_run = m_new;
          l_run *= alpha;
        }
        if constexpr (AW == 2) {
          if (moved || s == 0) sts32(m_sh, __float_as_uint(m_run));
          mbar_arrive(SPLASH_BAR(m_ready, s & 1));
        }
        if constexpr (AW == 2) {
          // P has its own columns: they are free once P.V of this group's previous step is done.
          if (s >= 2 && !warp_wait(SPLASH_BAR(pv_done, s & 1), ((s - 2) >> 1) & 1, ctx, kSiteSmxPv, s)) { alive = false; break; }
        }
        if ((warp & 3) == 0) SPLASH_TRACE_MARK(1 + grp, s, 3);
        const float m_scaled = (m_run == -INFINITY) ? 0.f : m_run * kLog2e;
        const float2 scale2 = make_float2(kLog2e, kLog2e), shift2 = make_float2(-m_scaled, -m_scaled);
        float2 sum_a = make_float2(0.f, 0.f), sum_b = make_float2(0.f, 0.f);
        // P is packed 32 columns of S (16 words) at a time, so that only one small staging
        // group is live beside the row itself.
#pragma unroll
        for (int c = 0; c < BKV / 32; ++c) {
          uint32_t pk[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float2 x = fma2(make_float2(sv[c * 32 + 2 * j], sv[c * 32 + 2 * j + 1]), scale2, shift2);
            float2 pr;
            pr.x = ex2_approx(x.x);
            pr.y = ex2_approx(x.y);
            if (j & 1) sum_b = add2(sum_b, pr); else sum_a = add2(sum_a, pr);
            pk[j] = pack2<BF16>(pr.x, pr.y);
          }
          tmem_st16(p_tmem + c * 16, pk);
        }
        l_run += (sum_a.x + sum_a.y) + (sum_b.x + sum_b.y);
        if ((warp & 3) == 0) SPLASH_TRACE_MARK(1 + grp, s, 4);

        // O may only be touched once P.V of the previous step has finished.  With two
        // tiles the s_ready wait above already certifies that (the tensor core runs
        // its instructions in issue order); with one tile it is signalled explicitly.
        if constexpr (NT == 1) {
          if (s > 0 && !warp_wait(SPLASH_BAR(pv_done, (s - 1) & 1), ((s - 1) >> 1) & 1, ctx, kSiteSmxPv, s)) { alive = false; break; }
        }
        if (s > 0 && __any_sync(0xffffffffu, moved)) {
          tc_fence_after();
          // Rare after the first steps: kept as a rolled loop so that it does not pad the
          // instruction stream of the common case.
#pragma unroll 1
          for (int c = 0; c < DV / 32; ++c) {
            uint32_t o[32];
            tmem_ld32(o_tmem + c * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st32(o_tmem + c * 32, o);
          }
        }
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(SPLASH_BAR(p_ready, buf));
        if ((warp & 3) == 0) SPLASH_TRACE_MARK(1 + grp, s, 5);
#pragma unroll
        for (int i = 0; i < AW; ++i)
          if (++slot == stages) { slot = 0; phase ^= 1; }
      }

      // ---- epilogue: O / l, cast, stage in shared memory, TMA store ---------------
      if (alive) {
        if constexpr (NT == 2) alive = warp_wait(SPLASH_BAR(o_done, 0), 0, ctx, kSiteSmxDone, n);
        else alive = warp_wait(SPLASH_BAR(pv_done, (n - 1) & 1), ((n - 1) >> 1) & 1, ctx, kSiteSmxDone, n);
      }
      float l_tot = l_run;
      if constexpr (AW == 2) {
        // Bring both partial sums to the final maximum and add them.  The group that did
        // not run the last step learns that maximum at the last step's barrier.
        if (alive && ((n - 1) & 1) != grp)
          alive = warp_wait(SPLASH_BAR(m_ready, (n - 1) & 1), ((n - 1) >> 1) & 1, ctx, kSiteSmxM, n);
        if (alive) {
          const float m_fin = __uint_as_float(lds32(m_sh));
          if (m_fin != m_run) {
            l_run = (m_run == -INFINITY) ? 0.f : l_run * ex2_approx((m_run - m_fin) * kLog2e);
            m_run = m_fin;
          }
          sts32(l_sh, __float_as_uint(l_run));
          mbar_arrive(SPLASH_BAR(fin, 0));
          alive = warp_wait(SPLASH_BAR(fin, 0), 0, ctx, kSiteSmxFin, n);
        }
        if (alive) l_tot = l_run + __uint_as_float(lds32(share_u32 + (1 + (grp ^ 1)) * kTile * 4 + row * 4));
      }
      if (alive) {
        tc_fence_after();
        const float inv_l = l_tot > 0.f ? 1.f / l_tot : 0.f;
        const uint32_t stage = L::kOStageInQ ? (q_u32 + t * (kTile * D * 2)) : v_u32;
#pragma unroll
        for (int cc = 0; cc < kEpiCols / 32; ++cc) {
          const int c = epi_col0 / 32 + cc;
          uint32_t o[32];
          tmem_ld32(o_tmem + c * 32, o);
          tmem_wait_ld();
          const uint32_t box = stage + (c / 2) * (kTile * 128);
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 w;
            w.x = pack2<BF16>(__uint_as_float(o[g * 8 + 0]) * inv_l, __uint_as_float(o[g * 8 + 1]) * inv_l);
            w.y = pack2<BF16>(__uint_as_float(o[g * 8 + 2]) * inv_l, __uint_as_float(o[g * 8 + 3]) * inv_l);
            w.z = pack2<BF16>(__uint_as_float(o[g * 8 + 4]) * inv_l, __uint_as_float(o[g * 8 + 5]) * inv_l);
            w.w = pack2<BF16>(__uint_as_float(o[g * 8 + 6]) * inv_l, __uint_as_float(o[g * 8 + 7]) * inv_l);
            sts128(box + swz128(row, (c & 1) * 4 + g), w);
          }
        }
        if (a.lse_out && epi_col0 == 0)
          a.lse_out[static_cast<size_t>(q_row0) + t * kTile + row] =
              l_tot > 0.f ? m_run + lg2_approx(l_tot) * kLn2 : a.mask_value;
        fence_proxy_async_smem();
        mbar_arrive(SPLASH_BAR(epi, t));
        if (row == 0 && epi_col0 == 0) {
          if (mbar_wait(SPLASH_BAR(epi, t), 0, ctx, kSiteSmxEpi, n)) {
#pragma unroll
            for (int c = 0; c < DV / 64; ++c)
              tma_store_2d(&tm_o, stage + c * (kTile * 128), c * 64, q_row0 + t * kTile);
            bulk_commit_group();
            bulk_wait_group_read<0>();
          }
        }
      }
    }
  }

  // ---- teardown: every thread of every role ends up here --------------------------
  tc_fence_before();
  __syncthreads();
  if (const uint32_t gave_up = lds32(abort_u32)) {
    if (threadIdx.x == 0) report_abort(a.status, gave_up);
    // Give copies that were still in flight time to land before the CTA's shared
    // memory is handed to another CTA.
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000) {}
  }
  if (warp == kSoftmaxWarps + 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem, L::kTmemCols);
  }
}

#undef SPLASH_BAR

}  // namespace splash
