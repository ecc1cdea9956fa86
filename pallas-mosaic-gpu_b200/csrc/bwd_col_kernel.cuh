// Splash attention backward over the column (per-KV-block) schedule, sm_100a.
//
// One CTA owns one 128-row KV block of one KV head and walks every q block that
// sees it, for every q head of the KV head's group, so dK and dV are complete when
// the CTA ends: GQA/MQA heads are reduced in tensor memory, not across CTAs.
//
//   FUSED = false   dK, dV only (the split backward; dQ comes from bwd_row_kernel).
//   FUSED = true    also dQ: each step's dQ^T = K^T dS^T tile is reduce-added into an
//                   f32 accumulator laid out [batch, heads, head_dim, q_len] with a
//                   TMA add-reduction (64 q rows per step).
//
// Per step (64 q rows of one q block):
//   S^T  = K Q^T        smem x smem -> TMEM f32   [128 kv, 64]
//   dP^T = V dO^T       smem x smem -> TMEM f32
//   elementwise (thread = kv row, two warpgroups split the 64 columns):
//     P^T  = exp2((S^T - lse) log2e)   masked entries 0
//     dS^T = P^T (dP^T - delta) [ (1 - tanh^2) with soft-cap ]
//     both written back over the columns they came from as packed 16-bit; FUSED also
//     stages dS^T in shared memory
//   dV  += P^T dO       TMEM x smem
//   dK  += dS^T Q       TMEM x smem
//   dQ^T = K^T dS^T     smem x smem (FUSED), written over the dead dP^T columns and
//                       drained by a writer warpgroup
//
// S^T and dP^T are double-buffered in tensor memory: the scores of step t+2 are issued
// while the elementwise warps work on step t+1, so the tensor core and the elementwise
// warps overlap instead of taking turns.  That needs three Q/dO tiles in flight.
//
// Behaviour follows the reference kernels (splash_attention_mgpu/backward.py:377-785,
// backward_fused.py:64-512); the code shares nothing with them.
#pragma once

#include <stddef.h>

#include "../../include/splash_sm100.h"
#include "fwd_kernel.cuh"  // math constants
#include "ptx.cuh"
#include "seg_skip.cuh"

namespace splash {

struct BwdArgs {
  const int32_t* num_steps;
  const int32_t* block_order;
  const int32_t* block_list;
  const int32_t* block_kind;
  const int32_t* mask_block;
  const int32_t* mask_desc;
  const int32_t* seg_q;
  const int32_t* seg_kv;
  const uint8_t* partial_blocks;  // bit-packed dense partial blocks [n, 128, 16 bytes], or null
  const int2* seg_q_ranges;   // [batch, q_len / 64] (min, max) segment ids, or null: no block skipping
  const int2* seg_kv_ranges;  // [batch, kv_len / 64]
  const float* lse;
  const float* delta;
  const uint8_t* aux_lse;    // 128-row fused kernel at head_dim 64: per q row {hi, mid, lo, 0 x 5} 16-bit parts of -lse
  const uint8_t* aux_delta;  // ... and of -delta (16 bytes per row each)
  void* dq;
  void* dk;
  void* dv;
  int32_t* status;
  int32_t batch, heads, kv_heads, q_len, kv_len;
  int32_t mask_heads, max_steps, q_blocks, kv_blocks, stages;
  int32_t has_dense, has_seg;
  int32_t head_group;  // heads whose blocks are interleaved in the launch order
  float mask_value, soft_cap;
};

enum BwdSite : int {
  kBSiteTmaEmpty = 21, kBSiteMmaKV, kBSiteMmaFull, kBSiteMmaP, kBSiteMmaDqFree,
  kBSiteEwFull, kBSiteEwS, kBSiteEwDone, kBSiteEwEpi,
  kBSiteWrReady, kBSiteWrBarA, kBSiteWrBarB,
};

constexpr int kColBC = 64;  // q rows per step

template <int D, int DV, bool FUSED>
struct ColLayout {
  static_assert(!FUSED || D == DV, "the fused kernel needs head_dim == head_dim_v");
  static constexpr int kRows = 128;  // kv rows per CTA
  static constexpr int BC = kColBC;
  static constexpr int kSub = 128 / BC;
  static constexpr int kKBytes = kRows * D * 2;
  static constexpr int kVBytes = kRows * DV * 2;
  // FUSED at head_dim 64: dQ^T = K^T dS^T is issued with M = 128 like at head_dim 128, and
  // the second 64 rows of its A operand are a second copy of the K tile, so the upper half
  // of the result repeats the lower half and is simply not stored.  That keeps one
  // accumulator layout and one writer for both head dims at the price of idle MMA rows.
  static constexpr int kKDupBytes = (FUSED && D == 64) ? kRows * 128 : 0;
  static constexpr int kQStage = BC * D * 2;
  static constexpr int kDoStage = BC * DV * 2;
  static constexpr int kVecStage = BC * 4;          // lse, delta, q segment ids: BC words each
  static constexpr int kMaskStage = kRows * 128 / 8;  // a whole transposed block, one bit per element
  static constexpr int kDsStage = kRows * BC * 2;   // FUSED: dS^T as an MMA operand
  static constexpr int kDqStage = 128 * 32 * 4;     // FUSED: half a dQ^T tile (32 q columns), f32
  // Tensor memory columns: two S^T buffers, two dP^T buffers, dK, dV.  P^T lives in the
  // S^T buffer it came from, dS^T in the dP^T buffer, dQ^T reuses the dP^T buffer.
  static constexpr int kColS = 0, kColDp = 2 * BC, kColDk = 4 * BC, kColDv = 4 * BC + D;
  static constexpr int kTmemUsed = 4 * BC + D + DV;
  static constexpr int kTmemCols = 512;
  static constexpr int kEwThreads = 256;
  static constexpr int kThreads = kEwThreads + (FUSED ? 128 : 0) + 128;
  static_assert(kTmemUsed <= 512, "tensor memory budget");

  // `list_steps`: capacity of the list of block steps that survive segment skipping (0 = no list).
  __host__ __device__ static size_t smem_bytes(int stages, bool dense, bool seg, int list_steps = 0) {
    size_t b = 1024;
    b += (static_cast<size_t>(list_steps) * 2 + 15) & ~static_cast<size_t>(15);
    b += kKBytes + kKDupBytes + kVBytes;
    b += static_cast<size_t>(stages) * (kQStage + kDoStage + 2 * kVecStage);
    if (seg) b += static_cast<size_t>(stages) * kVecStage;
    if (dense) b += static_cast<size_t>(stages) * kMaskStage;
    if (FUSED) b += 2 * kDsStage + kDqStage;
    b += 1024;
    return b;
  }
};

constexpr int kBwdMaxStages = 4;

struct ColBarriers {
  uint64_t kv_full;
  uint64_t full[kBwdMaxStages], empty[kBwdMaxStages];
  uint64_t s_ready[2], p_ready[2], acc_done;
  uint64_t dq_ready, dq_free, wr_a, wr_b;
  uint64_t epi[2];
  uint32_t tmem_base;
  uint32_t abort_flag;
  uint32_t dead;
  uint32_t n_eff;  // block steps left after segment skipping
};

#define SPLASH_CBAR(field, idx) \
  (bars_u32 + static_cast<uint32_t>(offsetof(ColBarriers, field)) + 8u * static_cast<uint32_t>(idx))

// Enumerates the steps of one CTA: q heads of the group x visited q blocks x sub-blocks.
// A "block step" is one (head, visited q block) pair, numbered in that order ("flat"
// index); with segment skipping the CTA walks the list of surviving flat indices that one
// of its warps put in shared memory, otherwise all of them.
template <int SUB>
struct ColSteps {
  const BwdArgs* a;
  int kj, head0, group;
  uint32_t list_u32;
  bool has_list;
  int count;   // block steps to walk
  int e;       // position in that sequence
  int g, s, sb, n, base;  // head, step inside the head, sub-step, steps of head g, flat index of (g, 0)
  uint32_t entry;

  __device__ __forceinline__ int mask_head(int gg) const { return a->mask_heads > 1 ? head0 + gg : 0; }
  __device__ __forceinline__ int steps_of(int gg) const { return a->num_steps[mask_head(gg) * a->kv_blocks + kj]; }
  __device__ __forceinline__ void bind(const BwdArgs* args, int kj_, int head0_, int group_) {
    a = args; kj = kj_; head0 = head0_; group = group_;
  }
  // Scheduled block steps of the CTA, before any skipping.
  __device__ __forceinline__ int scheduled() const {
    int t = 0;
    for (int gg = 0; gg < group; ++gg) t += steps_of(gg);
    return t;
  }
  // Offset into the step lists of flat index f (used while the list is being built).
  __device__ __forceinline__ int off_of_flat(int f) const {
    int gg = 0, bb = 0, nn = steps_of(0);
    while (f >= bb + nn) { bb += nn; ++gg; nn = steps_of(gg); }
    return (mask_head(gg) * a->kv_blocks + kj) * a->max_steps + (f - bb);
  }
  __device__ __forceinline__ void seek() {
    entry = has_list ? lds16(list_u32 + 2u * e) : static_cast<uint32_t>(e);
    const int flat = static_cast<int>(entry & 0x7fffu);
    while (flat >= base + n) { base += n; ++g; n = steps_of(g); }
    s = flat - base;
  }
  __device__ __forceinline__ void start(uint32_t list, bool with_list, int count_) {
    list_u32 = list; has_list = with_list; count = count_;
    e = 0; g = 0; s = 0; sb = 0; base = 0; entry = 0;
    n = steps_of(0);
    if (count > 0) seek();
  }
  __device__ __forceinline__ bool valid() const { return e < count; }
  __device__ __forceinline__ void next() {
    if (++sb == SUB) {
      sb = 0;
      if (++e < count) seek();
    }
  }
  __device__ __forceinline__ int head() const { return head0 + g; }
  __device__ __forceinline__ int off() const { return (mask_head(g) * a->kv_blocks + kj) * a->max_steps + s; }
  __device__ __forceinline__ int total() const { return count * SUB; }
  // Both sides of the block carry one and the same segment id: nothing to compare.
  __device__ __forceinline__ bool uniform() const { return has_list && (entry & kSegUniformBit); }
};

// PLAIN: no soft-cap, no segment ids, no streamed mask blocks -- that code is compiled out.
template <int D, int DV, bool FUSED, bool PLAIN, bool BF16>
__global__ void __launch_bounds__(ColLayout<D, DV, FUSED>::kThreads, 1)
splash_bwd_col_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                      const __grid_constant__ CUtensorMap tm_dk, const __grid_constant__ CUtensorMap tm_dv,
                      const __grid_constant__ CUtensorMap tm_dqacc, const BwdArgs a) {
  using L = ColLayout<D, DV, FUSED>;
  constexpr int kRows = 128;
  constexpr int BC = kColBC;
  constexpr int kSub = L::kSub;
  constexpr int kEwWarps = 8;
  constexpr int kWriterWarp0 = kEwWarps;                       // FUSED only
  constexpr int kProducerWarp0 = kEwWarps + (FUSED ? 4 : 0);

  const bool has_dense = !PLAIN && a.has_dense;
  const bool has_seg = !PLAIN && a.has_seg;
  const float soft_cap = PLAIN ? 0.f : a.soft_cap;
  extern __shared__ uint8_t smem_raw[];
  const int stages = a.stages;
  const uint32_t k_u32 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t v_u32 = k_u32 + L::kKBytes + L::kKDupBytes;
  const uint32_t q_u32 = v_u32 + L::kVBytes;
  const uint32_t do_u32 = q_u32 + stages * L::kQStage;
  const uint32_t ds_u32 = do_u32 + stages * L::kDoStage;              // FUSED: 2 x dS^T
  const uint32_t dqs_u32 = ds_u32 + (FUSED ? 2 * L::kDsStage : 0);    // FUSED: dQ^T staging
  const uint32_t mask_u32 = dqs_u32 + (FUSED ? L::kDqStage : 0);
  const uint32_t lse_u32 = mask_u32 + (has_dense ? stages * L::kMaskStage : 0);
  const uint32_t delta_u32 = lse_u32 + stages * L::kVecStage;
  const uint32_t segq_u32 = delta_u32 + stages * L::kVecStage;
  const uint32_t bars_u32 = (segq_u32 + (has_seg ? stages * L::kVecStage : 0) + 15u) & ~15u;
  const uint32_t list_u32 = (bars_u32 + static_cast<uint32_t>(sizeof(ColBarriers)) + 15u) & ~15u;  // surviving block steps
  const uint32_t neff_u32 = bars_u32 + static_cast<uint32_t>(offsetof(ColBarriers, n_eff));
  const bool has_list = has_seg && a.seg_q_ranges != nullptr;
  const uint32_t abort_u32 = bars_u32 + static_cast<uint32_t>(offsetof(ColBarriers, abort_flag));
  const uint32_t tmem_slot_u32 = bars_u32 + static_cast<uint32_t>(offsetof(ColBarriers, tmem_base));
  const uint32_t dead_u32 = bars_u32 + static_cast<uint32_t>(offsetof(ColBarriers, dead));

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

  ColSteps<kSub> it;
  it.bind(&a, kj, head0, group);
  const int scheduled = it.scheduled();

  // One warp initialises the barriers, a lane each, while the MMA warp allocates tensor
  // memory; one CTA barrier later every role starts.  A launch that finds the status
  // word already set returns without touching data; one thread reads the word and shares
  // it, so every role of the CTA takes the same branch.
  if (warp == 0) {
    constexpr uint32_t kNumBarriers = offsetof(ColBarriers, tmem_base) / 8;
    for (uint32_t i = lane; i < kNumBarriers; i += 32) {
      const uint32_t off = 8u * i;
      uint32_t count = 1;
      if (off >= offsetof(ColBarriers, empty) && off < offsetof(ColBarriers, s_ready)) count = 1 + kEwWarps;
      if (off >= offsetof(ColBarriers, p_ready) && off < offsetof(ColBarriers, acc_done)) count = L::kEwThreads;
      if (off >= offsetof(ColBarriers, dq_free) && off < offsetof(ColBarriers, tmem_base)) count = 128;  // dq_free, wr_a, wr_b, epi
      mbar_init(bars_u32 + off, count);
    }
    if (lane == 0) {
      sts32(abort_u32, 0);
      sts32(dead_u32, a.status[0] != 0);
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
    if (warp == kProducerWarp0 && total > 0) {
      // ------------------------------ TMA producer ------------------------------
      // Warp-uniform loop; one elected lane issues each group of copies.
      if (elect_one()) {
        prefetch_tensormap(&tm_q);
        prefetch_tensormap(&tm_do);
        mbar_arrive_expect_tx(SPLASH_CBAR(kv_full, 0), L::kKBytes + L::kKDupBytes + L::kVBytes);
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
          tma_load_2d(k_u32 + c * (kRows * 128), &tm_k, c * 64, kv_row0, SPLASH_CBAR(kv_full, 0));
        if constexpr (L::kKDupBytes > 0) tma_load_2d(k_u32 + L::kKBytes, &tm_k, 0, kv_row0, SPLASH_CBAR(kv_full, 0));
#pragma unroll
        for (int c = 0; c < DV / 64; ++c)
          tma_load_2d(v_u32 + c * (kRows * 128), &tm_v, c * 64, kv_row0, SPLASH_CBAR(kv_full, 0));
      }
      int slot = 0;
      uint32_t phase = 0;
      for (int t = 0; it.valid(); it.next(), ++t) {
        const int off = it.off();
        const int qblk = a.block_list[off];
        const int q_row = (b * a.heads + it.head()) * a.q_len + qblk * 128 + it.sb * BC;
        if (t >= stages && !warp_wait(SPLASH_CBAR(empty, slot), phase ^ 1, ctx, kBSiteTmaEmpty, t)) break;
        const bool partial_dense = has_dense && a.block_kind[off] == SPLASH_BLOCK_PARTIAL;
        const uint32_t bytes = L::kQStage + L::kDoStage + 2 * L::kVecStage + (has_seg ? L::kVecStage : 0) +
                               (partial_dense ? L::kMaskStage : 0);
        const uint32_t bar = SPLASH_CBAR(full, slot);
        const size_t mblock = partial_dense ? static_cast<size_t>(a.mask_block[off]) : 0;
        if (elect_one()) {
          mbar_arrive_expect_tx(bar, bytes);
#pragma unroll
          for (int c = 0; c < D / 64; ++c)
            tma_load_2d(q_u32 + slot * L::kQStage + c * (BC * 128), &tm_q, c * 64, q_row, bar);
#pragma unroll
          for (int c = 0; c < DV / 64; ++c)
            tma_load_2d(do_u32 + slot * L::kDoStage + c * (BC * 128), &tm_do, c * 64, q_row, bar);
          bulk_load_1d(lse_u32 + slot * L::kVecStage, a.lse + q_row, L::kVecStage, bar);
          bulk_load_1d(delta_u32 + slot * L::kVecStage, a.delta + q_row, L::kVecStage, bar);
          if (has_seg)
            bulk_load_1d(segq_u32 + slot * L::kVecStage,
                         a.seg_q + static_cast<size_t>(b) * a.q_len + qblk * 128 + it.sb * BC, L::kVecStage, bar);
          if (partial_dense)
            bulk_load_1d(mask_u32 + slot * L::kMaskStage, a.partial_blocks + mblock * L::kMaskStage, L::kMaskStage, bar);
        }
        if (++slot == stages) { slot = 0; phase ^= 1; }
      }
    } else if (warp == kProducerWarp0 + 1 && total > 0) {
      // ------------------------------- MMA issuer -------------------------------
      // All lanes run the loop; one elected lane issues each instruction.
      constexpr uint32_t kIdescScore = make_idesc(BF16, 128, BC, false, false);   // K Q^T, V dO^T
      constexpr uint32_t kIdescAcc = make_idesc(BF16, 128, D, false, true);       // dS^T Q
      constexpr uint32_t kIdescAccV = make_idesc(BF16, 128, DV, false, true);     // P^T dO
      constexpr uint32_t kIdescDq = make_idesc(BF16, 128, BC, true, true);        // K^T dS^T
      auto issue_s = [&](int slot, int buf) {
        const uint32_t k_lo = desc_lo(k_u32, 16), q_lo = desc_lo(q_u32 + slot * L::kQStage, 16);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_ss2_w(tmem + L::kColS + buf * BC, k_lo + (((kk / 4) * (kRows * 128) + (kk % 4) * 32) >> 4), kDescHi,
                     q_lo + (((kk / 4) * (BC * 128) + (kk % 4) * 32) >> 4), kDescHi, kIdescScore, kk > 0);
      };
      auto issue_dp = [&](int slot, int buf) {
        const uint32_t v_lo = desc_lo(v_u32, 16), do_lo = desc_lo(do_u32 + slot * L::kDoStage, 16);
#pragma unroll
        for (int kk = 0; kk < DV / 16; ++kk)
          umma_ss2_w(tmem + L::kColDp + buf * BC, v_lo + (((kk / 4) * (kRows * 128) + (kk % 4) * 32) >> 4), kDescHi,
                     do_lo + (((kk / 4) * (BC * 128) + (kk % 4) * 32) >> 4), kDescHi, kIdescScore, kk > 0);
      };
      int s_slot = 0;        // ring position of the next step whose scores get issued
      uint32_t s_phase = 0;
      bool ok = warp_wait(SPLASH_CBAR(kv_full, 0), 0, ctx, kBSiteMmaKV, 0);
      // Prologue: scores of steps 0 and 1 fill the two buffers.
      for (int u = 0; u < 2 && u < total && ok; ++u) {
        ok = warp_wait(SPLASH_CBAR(full, s_slot), s_phase, ctx, kBSiteMmaFull, u);
        if (!ok) break;
        tc_fence_after();
        issue_dp(s_slot, u);
        issue_s(s_slot, u);
        umma_commit_w(SPLASH_CBAR(s_ready, u));
        if (++s_slot == stages) { s_slot = 0; s_phase ^= 1; }
      }
      if (ok) {
        int c_slot = 0;  // ring position of the step whose P^T / dS^T get consumed
        for (int t = 0; t < total; ++t) {
          const int buf = t & 1;
          if (!warp_wait(SPLASH_CBAR(p_ready, buf), (t >> 1) & 1, ctx, kBSiteMmaP, t)) break;
          tc_fence_after();
          // A operands of dK / dV are the packed 16-bit values the elementwise warps wrote
          // over dP^T / S^T: keys 0-31 sit in columns 0-15 of the buffer, keys 32-63 in
          // columns 32-47 (each warpgroup packs into its own half).  B operands MN-major:
          // boxes of 64 columns, BC rows each.
          {
            // dK += dS^T Q
            const uint32_t q_lo = desc_lo(q_u32 + c_slot * L::kQStage, BC * 128);
#pragma unroll
            for (int kk = 0; kk < BC / 16; ++kk)
              umma_ts2_w(tmem + L::kColDk, tmem + L::kColDp + buf * BC + (kk >> 1) * 32 + (kk & 1) * 8,
                         q_lo + ((kk * 2048) >> 4), kDescHi, kIdescAcc, (t > 0 || kk > 0) ? 1u : 0u);
          }
          if constexpr (FUSED) {
            // dQ^T[d, q] = sum_kv K[kv, d] dS^T[kv, q]: A = K read MN-major, B = staged dS^T
            // MN-major.  The result replaces dP^T / dS^T of this step, which dK has consumed
            // (the tensor core runs its instructions in issue order).  It is issued this
            // early so that the writer has drained it long before the next dP^T needs the
            // columns.
            const uint32_t k_lo = desc_lo(k_u32, kRows * 128);
            const uint32_t ds_lo = desc_lo(ds_u32 + buf * L::kDsStage, kRows * 128);
#pragma unroll
            for (int kk = 0; kk < kRows / 16; ++kk)
              umma_ss2_w(tmem + L::kColDp + buf * BC, k_lo + ((kk * 2048) >> 4), kDescHi, ds_lo + ((kk * 2048) >> 4),
                         kDescHi, kIdescDq, kk > 0);
            umma_commit_w(SPLASH_CBAR(dq_ready, 0));
          }
          {
            // dV += P^T dO
            const uint32_t do_lo = desc_lo(do_u32 + c_slot * L::kDoStage, BC * 128);
#pragma unroll
            for (int kk = 0; kk < BC / 16; ++kk)
              umma_ts2_w(tmem + L::kColDv, tmem + L::kColS + buf * BC + (kk >> 1) * 32 + (kk & 1) * 8,
                         do_lo + ((kk * 2048) >> 4), kDescHi, kIdescAccV, (t > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit_w(SPLASH_CBAR(empty, c_slot));
          if (t + 2 < total) {
            // Scores of step t+2 go into the buffers step t has just vacated.
            if (!warp_wait(SPLASH_CBAR(full, s_slot), s_phase, ctx, kBSiteMmaFull, t + 2)) break;
            tc_fence_after();
            issue_s(s_slot, buf);
            if constexpr (FUSED) {
              // The writer must have taken dQ^T of step t out of the dP^T buffer.
              if (!warp_wait(SPLASH_CBAR(dq_free, 0), t & 1, ctx, kBSiteMmaDqFree, t)) break;
              tc_fence_after();
            }
            issue_dp(s_slot, buf);
            umma_commit_w(SPLASH_CBAR(s_ready, buf));
            if (++s_slot == stages) { s_slot = 0; s_phase ^= 1; }
          } else if constexpr (FUSED) {
            // Tail steps: still observe every phase of dq_free, so that dq_ready never
            // runs two phases ahead of the writer.
            if (!warp_wait(SPLASH_CBAR(dq_free, 0), t & 1, ctx, kBSiteMmaDqFree, t)) break;
          }
          if (++c_slot == stages) c_slot = 0;
        }
        umma_commit_w(SPLASH_CBAR(acc_done, 0));
      }
    }
  } else if (FUSED && warp >= kWriterWarp0) {
    // ================================ dQ writer ==================================
    if constexpr (FUSED) {
      const int wq = warp & 3;
      const int drow = wq * 32 + lane;  // head-dim index = TMEM lane
      const uint32_t dq_tmem = tmem + (static_cast<uint32_t>(wq * 32) << 16) + L::kColDp;
      const bool leader = (warp == kWriterWarp0 && lane == 0);
      bool alive = true;
      int t = 0;
      for (; it.valid() && alive; it.next(), ++t) {
        const int qblk = a.block_list[it.off()];
        if (!warp_wait(SPLASH_CBAR(dq_ready, 0), t & 1, ctx, kBSiteWrReady, t)) break;
        tc_fence_after();
        uint32_t acc[BC];
#pragma unroll
        for (int c = 0; c < BC / 32; ++c) tmem_ld32(dq_tmem + (t & 1) * BC + c * 32, acc + c * 32);
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(SPLASH_CBAR(dq_free, 0));
        const int x = qblk * 128 + it.sb * BC;
        const int y = (b * a.heads + it.head()) * D;
        // Two passes of 32 q columns through one 16 KB staging tile (128 rows of 128 bytes).
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const uint32_t par = (2 * t + half) & 1;
          // The previous reduction must have read the staging tile.
          if (leader) bulk_wait_group_read<0>();
          mbar_arrive(SPLASH_CBAR(wr_a, 0));
          if (!warp_wait(SPLASH_CBAR(wr_a, 0), par, ctx, kBSiteWrBarA, t)) { alive = false; break; }
          if (drow < D) {  // at head_dim 64 the upper rows repeat the lower ones
#pragma unroll
            for (int c = 0; c < 8; ++c)
              sts128(dqs_u32 + swz128(drow, c), make_uint4(acc[half * 32 + c * 4], acc[half * 32 + c * 4 + 1],
                                                           acc[half * 32 + c * 4 + 2], acc[half * 32 + c * 4 + 3]));
          }
          fence_proxy_async_smem();
          mbar_arrive(SPLASH_CBAR(wr_b, 0));
          if (!warp_wait(SPLASH_CBAR(wr_b, 0), par, ctx, kBSiteWrBarB, t)) { alive = false; break; }
          if (leader) {
            tma_reduce_add_2d(&tm_dqacc, dqs_u32, x + half * 32, y);
            bulk_commit_group();
          }
        }
      }
      if (leader) bulk_wait_group_read<0>();
    }
  } else {
    // ========================== elementwise warpgroups ===========================
    const int w = warp >> 2;                 // which half of the 64 columns
    const int wq = warp & 3;
    const int row = wq * 32 + lane;          // kv row inside the block
    const int kv_pos = kj * kRows + row;
    const uint32_t tmem_row = tmem + (static_cast<uint32_t>(wq * 32) << 16);
    const int col0 = w * 32;                 // first column this thread handles

    if (total == 0) {
      // No q block sees this KV block: its gradients are zero.
      if (w == 0) {
        uint4* dst = reinterpret_cast<uint4*>(static_cast<uint8_t*>(a.dk) + static_cast<size_t>(kv_row0 + row) * (D * 2));
#pragma unroll
        for (int c = 0; c < D * 2 / 16; ++c) dst[c] = make_uint4(0, 0, 0, 0);
      } else {
        uint4* dst = reinterpret_cast<uint4*>(static_cast<uint8_t*>(a.dv) + static_cast<size_t>(kv_row0 + row) * (DV * 2));
#pragma unroll
        for (int c = 0; c < DV * 2 / 16; ++c) dst[c] = make_uint4(0, 0, 0, 0);
      }
    } else {
      const int my_seg = has_seg ? a.seg_kv[static_cast<size_t>(b) * a.kv_len + kv_pos] : 0;
      const bool cap_on = soft_cap > 0.f;
      const float cap = soft_cap, inv_cap = cap_on ? 1.f / soft_cap : 0.f;
      bool alive = true;
      int slot = 0;
      uint32_t phase = 0;
      int cur_mh = -1;
      int band_lo = -(1 << 30), band_hi = (1 << 30);  // allowed range of kv_pos - q_pos for this kv row

      for (int t = 0; it.valid(); it.next(), ++t) {
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
        if (!warp_wait(SPLASH_CBAR(full, slot), phase, ctx, kBSiteEwFull, t)) { alive = false; break; }
        const int buf = t & 1;
        if (!warp_wait(SPLASH_CBAR(s_ready, buf), (t >> 1) & 1, ctx, kBSiteEwS, t)) { alive = false; break; }
        tc_fence_after();
        const int q0 = qblk * 128 + it.sb * BC + col0;  // sequence position of this thread's first column
        {
          constexpr int c = 0;  // one 32-column chunk per thread and step
          uint32_t sraw[32], dpraw[32];
          tmem_ld32(tmem_row + L::kColS + buf * BC + col0, sraw);
          tmem_ld32(tmem_row + L::kColDp + buf * BC + col0, dpraw);
          tmem_wait_ld();
          uint32_t ppk[16], dspk[16];
          const uint32_t vec_off = slot * L::kVecStage + (col0 + c * 32) * 4;
          if (!partial && (!has_seg || it.uniform()) && !cap_on) {
            // FULL block, no segment ids (or one id on both sides), no soft-cap: nothing to
            // mask.  (A row whose lse is mask_value never meets such a block, so no guard is
            // needed here.)
#pragma unroll
            for (int g = 0; g < 8; ++g) {
              const uint4 lw = lds128(lse_u32 + vec_off + g * 16);
              const uint4 dw = lds128(delta_u32 + vec_off + g * 16);
              const float nl0 = __uint_as_float(lw.x) * -kLog2e, nl1 = __uint_as_float(lw.y) * -kLog2e;
              const float nl2 = __uint_as_float(lw.z) * -kLog2e, nl3 = __uint_as_float(lw.w) * -kLog2e;
              const float p0 = ex2_approx(fmaf(__uint_as_float(sraw[g * 4 + 0]), kLog2e, nl0));
              const float p1 = ex2_approx(fmaf(__uint_as_float(sraw[g * 4 + 1]), kLog2e, nl1));
              const float p2 = ex2_approx(fmaf(__uint_as_float(sraw[g * 4 + 2]), kLog2e, nl2));
              const float p3 = ex2_approx(fmaf(__uint_as_float(sraw[g * 4 + 3]), kLog2e, nl3));
              ppk[g * 2] = pack2<BF16>(p0, p1);
              ppk[g * 2 + 1] = pack2<BF16>(p2, p3);
              dspk[g * 2] = pack2<BF16>(p0 * (__uint_as_float(dpraw[g * 4 + 0]) - __uint_as_float(dw.x)),
                                        p1 * (__uint_as_float(dpraw[g * 4 + 1]) - __uint_as_float(dw.y)));
              dspk[g * 2 + 1] = pack2<BF16>(p2 * (__uint_as_float(dpraw[g * 4 + 2]) - __uint_as_float(dw.z)),
                                            p3 * (__uint_as_float(dpraw[g * 4 + 3]) - __uint_as_float(dw.w)));
            }
          } else {
            uint32_t vis = 0xffffffffu;  // bit i: column i of this chunk is visible
            if (partial && !has_dense) {
              const int d0 = kv_pos - (q0 + c * 32);
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                const int d = d0 - i;
                if (d < band_lo || d > band_hi) vis &= ~(1u << i);
              }
            }
            if (partial && has_dense) {
              // Transposed block, one bit per element: 16 bytes per kv row, bit = q column.
              vis &= lds32(mask_u32 + slot * L::kMaskStage + row * 16 + (it.sb * BC + col0 + c * 32) / 8);
            }
            if (has_seg && !it.uniform()) {
#pragma unroll
              for (int g = 0; g < 8; ++g) {
                const uint4 sg = lds128(segq_u32 + vec_off + g * 16);
                if (static_cast<int>(sg.x) != my_seg) vis &= ~(1u << (g * 4 + 0));
                if (static_cast<int>(sg.y) != my_seg) vis &= ~(1u << (g * 4 + 1));
                if (static_cast<int>(sg.z) != my_seg) vis &= ~(1u << (g * 4 + 2));
                if (static_cast<int>(sg.w) != my_seg) vis &= ~(1u << (g * 4 + 3));
              }
            }
#pragma unroll
            for (int g = 0; g < 8; ++g) {
              const uint4 lw = lds128(lse_u32 + vec_off + g * 16);
              const uint4 dw = lds128(delta_u32 + vec_off + g * 16);
              const float lses[4] = {__uint_as_float(lw.x), __uint_as_float(lw.y), __uint_as_float(lw.z), __uint_as_float(lw.w)};
              const float dels[4] = {__uint_as_float(dw.x), __uint_as_float(dw.y), __uint_as_float(dw.z), __uint_as_float(dw.w)};
              float pv[4], dsv[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int i = g * 4 + e;
                float sval = __uint_as_float(sraw[i]);
                float tanh_v = 0.f;
                if (cap_on) {
                  tanh_v = tanh_approx(sval * inv_cap);
                  sval = cap * tanh_v;
                }
                // Rows that saw no key carry lse = mask_value; they contribute nothing.
                const bool on = ((vis >> i) & 1u) && lses[e] != a.mask_value;
                const float p = on ? ex2_approx(fmaf(sval, kLog2e, lses[e] * -kLog2e)) : 0.f;  // same rounding as the unmasked path
                float ds = p * (__uint_as_float(dpraw[i]) - dels[e]);
                if (cap_on) ds *= (1.f - tanh_v * tanh_v);
                pv[e] = p;
                dsv[e] = ds;
              }
              ppk[g * 2] = pack2<BF16>(pv[0], pv[1]);
              ppk[g * 2 + 1] = pack2<BF16>(pv[2], pv[3]);
              dspk[g * 2] = pack2<BF16>(dsv[0], dsv[1]);
              dspk[g * 2 + 1] = pack2<BF16>(dsv[2], dsv[3]);
            }
          }
          // Packed results go over the first half of the columns this thread just read.
          tmem_st16(tmem_row + L::kColS + buf * BC + col0, ppk);
          tmem_st16(tmem_row + L::kColDp + buf * BC + col0, dspk);
          if constexpr (FUSED) {
            // dS^T staged as [kv row][64 q], 128 bytes per row, 128-byte swizzle.
            const uint32_t stage = ds_u32 + buf * L::kDsStage;
            const int chunk0 = (col0 + c * 32) / 8;  // 16-byte chunk index of this thread's first column
#pragma unroll
            for (int g = 0; g < 4; ++g)
              sts128(stage + swz128(row, chunk0 + g),
                     make_uint4(dspk[g * 4], dspk[g * 4 + 1], dspk[g * 4 + 2], dspk[g * 4 + 3]));
          }
        }
        // The slot's vectors and mask slice have been read.
        __syncwarp();
        if (lane == 0) mbar_arrive(SPLASH_CBAR(empty, slot));
        tmem_wait_st();
        if constexpr (FUSED) fence_proxy_async_smem();
        tc_fence_before();
        mbar_arrive(SPLASH_CBAR(p_ready, buf));
        if (++slot == stages) { slot = 0; phase ^= 1; }
      }

      // ---- epilogue: dK by warpgroup 0, dV by warpgroup 1 ---------------------------
      if (alive) alive = warp_wait(SPLASH_CBAR(acc_done, 0), 0, ctx, kBSiteEwDone, total);
      if (alive) {
        tc_fence_after();
        const uint32_t stage = w == 0 ? k_u32 : v_u32;  // K / V tiles are dead once every MMA has finished
        const uint32_t acc_tmem = tmem_row + (w == 0 ? L::kColDk : L::kColDv);
        constexpr int kMaxCols = D > DV ? D : DV;
        const int cols = w == 0 ? D : DV;  // uniform per warpgroup
#pragma unroll
        for (int c = 0; c < kMaxCols / 32; ++c) {
          if (c * 32 >= cols) break;
          uint32_t o[32];
          tmem_ld32(acc_tmem + c * 32, o);
          tmem_wait_ld();
          const uint32_t box = stage + (c / 2) * (kRows * 128);
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
        mbar_arrive(SPLASH_CBAR(epi, w));
        if (row == 0) {
          if (mbar_wait(SPLASH_CBAR(epi, w), 0, ctx, kBSiteEwEpi, total)) {
#pragma unroll
            for (int c = 0; c < kMaxCols / 64; ++c)
              if (c * 64 < cols) tma_store_2d(w == 0 ? &tm_dk : &tm_dv, stage + c * (kRows * 128), c * 64, kv_row0);
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

#undef SPLASH_CBAR

}  // namespace splash
