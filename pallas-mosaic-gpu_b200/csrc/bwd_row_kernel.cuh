// Splash attention backward, dQ over the row (per-q-block) schedule, sm_100a.
//
// One CTA owns one 128-row q block of one head and walks the KV blocks that row
// visits, in sub-blocks of BC keys:
//   S  = Q K^T          smem x smem -> TMEM f32   [128 q, BC]
//   dP = dO V^T         smem x smem -> TMEM f32
//   elementwise (thread = q row; two warpgroups split the BC columns):
//     P  = exp2((S - lse) log2e), masked entries 0
//     dS = P (dP - delta) [ (1 - tanh^2) with soft-cap ], written to TMEM as packed 16-bit
//   dQ += dS K          TMEM x smem -> TMEM f32
// dS is double-buffered so that dQ of step t runs while the elementwise warps work on
// step t+1.
//
// Behaviour follows the reference kernel (splash_attention_mgpu/backward.py:87-374);
// the code shares nothing with it.
#pragma once

#include <stddef.h>

#include "../../include/splash_sm100.h"
#include "bwd_col_kernel.cuh"  // BwdArgs, kBwdMaxStages
#include "ptx.cuh"

namespace splash {

enum BwdRowSite : int {
  kRSiteTmaEmpty = 41, kRSiteMmaQ, kRSiteMmaFull, kRSiteMmaDs,
  kRSiteEwFull, kRSiteEwS, kRSiteEwDone, kRSiteEwEpi,
};

template <int D, int DV, int BC>
struct RowLayout {
  static constexpr int kRows = 128;  // q rows per CTA
  static constexpr int kSub = 128 / BC;
  static constexpr int kQBytes = kRows * D * 2;
  static constexpr int kDoBytes = kRows * DV * 2;
  static constexpr int kKStage = BC * D * 2;
  static constexpr int kVStage = BC * DV * 2;
  static constexpr int kVecStage = BC * 4;       // kv segment ids
  static constexpr int kMaskStage = kRows * 128 / 8;  // a whole block, one bit per element
  static constexpr int kColS = 0, kColDp = BC, kColDs = 2 * BC, kColDq = 3 * BC;  // two dS buffers of BC/2
  static constexpr int kTmemUsed = 3 * BC + D;
  static constexpr int kTmemCols = kTmemUsed <= 256 ? 256 : 512;
  static constexpr int kThreads = 384;
  static_assert(kTmemUsed <= 512, "tensor memory budget");

  // `list_steps`: capacity of the list of block steps that survive segment skipping (0 = no list).
  __host__ __device__ static size_t smem_bytes(int stages, bool dense, bool seg, int list_steps = 0) {
    size_t b = 1024;
    b += (static_cast<size_t>(list_steps) * 2 + 15) & ~static_cast<size_t>(15);
    b += kQBytes + kDoBytes;
    b += static_cast<size_t>(stages) * (kKStage + kVStage);
    if (seg) b += static_cast<size_t>(stages) * kVecStage;
    if (dense) b += static_cast<size_t>(stages) * kMaskStage;
    b += 1024;
    return b;
  }
};

struct RowBarriers {
  uint64_t q_full;
  uint64_t full[kBwdMaxStages], empty[kBwdMaxStages];
  uint64_t s_ready, ds_ready, acc_done;
  uint64_t epi;
  uint32_t tmem_base;
  uint32_t abort_flag;
  uint32_t dead;
  uint32_t n_eff;  // block steps left after segment skipping
};

#define SPLASH_RBAR(field, idx) \
  (bars_u32 + static_cast<uint32_t>(offsetof(RowBarriers, field)) + 8u * static_cast<uint32_t>(idx))

template <int D, int DV, int BC, bool BF16>
__global__ void __launch_bounds__(384, 1)
splash_bwd_row_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                      const __grid_constant__ CUtensorMap tm_dq, const BwdArgs a) {
  using L = RowLayout<D, DV, BC>;
  constexpr int kRows = 128;
  constexpr int kSub = L::kSub;
  constexpr int kEwWarps = 8;
  constexpr int kHalf = BC / 2;

  extern __shared__ uint8_t smem_raw[];
  const int stages = a.stages;
  const uint32_t q_u32 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t do_u32 = q_u32 + L::kQBytes;
  const uint32_t k_u32 = do_u32 + L::kDoBytes;
  const uint32_t v_u32 = k_u32 + stages * L::kKStage;
  const uint32_t mask_u32 = v_u32 + stages * L::kVStage;
  const uint32_t seg_u32 = mask_u32 + (a.has_dense ? stages * L::kMaskStage : 0);
  const uint32_t bars_u32 = (seg_u32 + (a.has_seg ? stages * L::kVecStage : 0) + 15u) & ~15u;
  const uint32_t abort_u32 = bars_u32 + static_cast<uint32_t>(offsetof(RowBarriers, abort_flag));
  const uint32_t dead_u32 = bars_u32 + static_cast<uint32_t>(offsetof(RowBarriers, dead));
  const uint32_t tmem_slot_u32 = bars_u32 + static_cast<uint32_t>(offsetof(RowBarriers, tmem_base));
  const uint32_t neff_u32 = bars_u32 + static_cast<uint32_t>(offsetof(RowBarriers, n_eff));
  const uint32_t list_u32 = bars_u32 + 128u;  // surviving block steps, 16 bits each
  static_assert(sizeof(RowBarriers) <= 128, "step list overlaps the barriers");
  const bool has_list = a.has_seg && a.seg_q_ranges != nullptr;

  const int warp = uniform_warp_index();
  const int lane = threadIdx.x & 31;

  int hb, order_idx;
  decode_work_item(blockIdx.x, a.q_blocks, a.heads * a.batch, a.head_group, hb, order_idx);
  const int h = hb % a.heads;
  const int b = hb / a.heads;
  const int mh = a.mask_heads > 1 ? h : 0;
  const int qi = a.block_order[mh * a.q_blocks + order_idx];
  const int n_sched = a.num_steps[mh * a.q_blocks + qi];
  const int sched_off = (mh * a.q_blocks + qi) * a.max_steps;
  const int q_row0 = (b * a.heads + h) * a.q_len + qi * kRows;

  if (threadIdx.x == 0) {
    sts32(abort_u32, 0);
    sts32(dead_u32, a.status[0] != 0);
    mbar_init(SPLASH_RBAR(q_full, 0), 1);
    for (int i = 0; i < stages; ++i) {
      mbar_init(SPLASH_RBAR(full, i), 1);
      mbar_init(SPLASH_RBAR(empty, i), 1 + kEwWarps);
    }
    mbar_init(SPLASH_RBAR(s_ready, 0), 1);
    mbar_init(SPLASH_RBAR(ds_ready, 0), 256);
    mbar_init(SPLASH_RBAR(acc_done, 0), 1);
    mbar_init(SPLASH_RBAR(epi, 0), 256);
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  __syncthreads();
  if (lds32(dead_u32)) return;
  if (warp == kEwWarps + 1) {
    tmem_alloc(tmem_slot_u32, L::kTmemCols);
    tmem_relinquish();
  } else if (warp == 1 && has_list) {
    // Block steps whose q and kv segment-id ranges can meet; every role leaves out the others.
    const int2* qt = a.seg_q_ranges + static_cast<size_t>(b) * (a.q_len / kSegChunk);
    const int2* kt = a.seg_kv_ranges + static_cast<size_t>(b) * (a.kv_len / kSegChunk);
    const SegRange qr = seg_range(qt, qi * (kRows / kSegChunk), kRows / kSegChunk);
    const int kept = build_step_list(list_u32, n_sched, lane, [&](int s) {
      const int j = a.block_list[sched_off + s];
      return seg_classify(qr, seg_range(kt, j * (128 / kSegChunk), 128 / kSegChunk));
    });
    if (lane == 0) sts32(neff_u32, static_cast<uint32_t>(kept));
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = lds32(tmem_slot_u32);
  const WaitCtx ctx{abort_u32};
  const int n = has_list ? static_cast<int>(lds32(neff_u32)) : n_sched;
  const int total = n * kSub;
  // Entry e of the CTA's block-step sequence: index into the schedule lists, top bit set
  // when the block needs no segment comparison.
  auto step_at = [&](int e) -> uint32_t { return has_list ? lds16(list_u32 + 2u * e) : static_cast<uint32_t>(e); };
  constexpr uint32_t kDescHi = desc_hi(1024);

  if (warp >= kEwWarps) {
    if (warp == kEwWarps && total > 0) {
      // ------------------------------ TMA producer ------------------------------
      // Warp-uniform loop; one elected lane issues each group of copies.
      const int kv_row0 = (b * a.kv_heads + h / (a.heads / a.kv_heads)) * a.kv_len;
      if (elect_one()) {
        prefetch_tensormap(&tm_k);
        prefetch_tensormap(&tm_v);
        mbar_arrive_expect_tx(SPLASH_RBAR(q_full, 0), L::kQBytes + L::kDoBytes);
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
          tma_load_2d(q_u32 + c * (kRows * 128), &tm_q, c * 64, q_row0, SPLASH_RBAR(q_full, 0));
#pragma unroll
        for (int c = 0; c < DV / 64; ++c)
          tma_load_2d(do_u32 + c * (kRows * 128), &tm_do, c * 64, q_row0, SPLASH_RBAR(q_full, 0));
      }
      int slot = 0;
      uint32_t phase = 0;
      for (int t = 0; t < total; ++t) {
        const int s = static_cast<int>(step_at(t / kSub) & 0x7fffu), sb = t % kSub;
        const int j = a.block_list[sched_off + s];
        const int kv_row = kv_row0 + j * 128 + sb * BC;
        if (t >= stages && !warp_wait(SPLASH_RBAR(empty, slot), phase ^ 1, ctx, kRSiteTmaEmpty, t)) break;
        const bool partial_dense = a.has_dense && a.block_kind[sched_off + s] == SPLASH_BLOCK_PARTIAL;
        const uint32_t bytes = L::kKStage + L::kVStage + (a.has_seg ? L::kVecStage : 0) +
                               (partial_dense ? L::kMaskStage : 0);
        const uint32_t bar = SPLASH_RBAR(full, slot);
        const size_t mblock = partial_dense ? static_cast<size_t>(a.mask_block[sched_off + s]) : 0;
        if (elect_one()) {
          mbar_arrive_expect_tx(bar, bytes);
#pragma unroll
          for (int c = 0; c < D / 64; ++c)
            tma_load_2d(k_u32 + slot * L::kKStage + c * (BC * 128), &tm_k, c * 64, kv_row, bar);
#pragma unroll
          for (int c = 0; c < DV / 64; ++c)
            tma_load_2d(v_u32 + slot * L::kVStage + c * (BC * 128), &tm_v, c * 64, kv_row, bar);
          if (a.has_seg)
            bulk_load_1d(seg_u32 + slot * L::kVecStage,
                         a.seg_kv + static_cast<size_t>(b) * a.kv_len + j * 128 + sb * BC, L::kVecStage, bar);
          if (partial_dense)
            bulk_load_1d(mask_u32 + slot * L::kMaskStage, a.partial_blocks + mblock * L::kMaskStage, L::kMaskStage, bar);
        }
        if (++slot == stages) { slot = 0; phase ^= 1; }
      }
    } else if (warp == kEwWarps + 1 && total > 0) {
      // ------------------------------- MMA issuer -------------------------------
      constexpr uint32_t kIdescScore = make_idesc(BF16, 128, BC, false, false);
      constexpr uint32_t kIdescDq = make_idesc(BF16, 128, D, false, true);
      auto issue_scores = [&](int slot) {
        const uint32_t q_lo = desc_lo(q_u32, 16), k_lo = desc_lo(k_u32 + slot * L::kKStage, 16);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_ss2_w(tmem + L::kColS, q_lo + (((kk / 4) * (kRows * 128) + (kk % 4) * 32) >> 4), kDescHi,
                   k_lo + (((kk / 4) * (BC * 128) + (kk % 4) * 32) >> 4), kDescHi, kIdescScore, kk > 0);
        const uint32_t do_lo = desc_lo(do_u32, 16), v_lo = desc_lo(v_u32 + slot * L::kVStage, 16);
#pragma unroll
        for (int kk = 0; kk < DV / 16; ++kk)
          umma_ss2_w(tmem + L::kColDp, do_lo + (((kk / 4) * (kRows * 128) + (kk % 4) * 32) >> 4), kDescHi,
                   v_lo + (((kk / 4) * (BC * 128) + (kk % 4) * 32) >> 4), kDescHi, kIdescScore, kk > 0);
      };
      bool ok = warp_wait(SPLASH_RBAR(q_full, 0), 0, ctx, kRSiteMmaQ, 0) &&
                warp_wait(SPLASH_RBAR(full, 0), 0, ctx, kRSiteMmaFull, 0);
      if (ok) {
        tc_fence_after();
        issue_scores(0);
        umma_commit_w(SPLASH_RBAR(s_ready, 0));
        int slot = 0;
        uint32_t phase = 0;
        for (int t = 0; t < total; ++t) {
          int slot1 = slot + 1;
          uint32_t phase1 = phase;
          if (slot1 == stages) { slot1 = 0; phase1 ^= 1; }
          if (!warp_wait(SPLASH_RBAR(ds_ready, 0), t & 1, ctx, kRSiteMmaDs, t)) break;
          tc_fence_after();
          auto issue_dq = [&]() {
            // dQ += dS K  (K tile read MN-major: boxes of 64 head-dim columns, BC rows each)
            const uint32_t k_lo = desc_lo(k_u32 + slot * L::kKStage, BC * 128);
#pragma unroll
            for (int kk = 0; kk < BC / 16; ++kk)
              umma_ts2_w(tmem + L::kColDq, tmem + L::kColDs + (t & 1) * (BC / 2) + kk * 8, k_lo + ((kk * 2048) >> 4),
                       kDescHi, kIdescDq, (t > 0 || kk > 0) ? 1u : 0u);
            umma_commit_w(SPLASH_RBAR(empty, slot));
          };
          // With a single stage the next K/V tile can only arrive once dQ has released
          // this one; with more, the next scores go first so that dQ overlaps the
          // elementwise work on them.
          if (stages == 1) issue_dq();
          if (t + 1 < total) {
            // S / dP of step t have been read: the next scores may overwrite them.
            if (!warp_wait(SPLASH_RBAR(full, slot1), phase1, ctx, kRSiteMmaFull, t + 1)) break;
            tc_fence_after();
            issue_scores(slot1);
            umma_commit_w(SPLASH_RBAR(s_ready, 0));
          }
          if (stages != 1) issue_dq();
          slot = slot1;
          phase = phase1;
        }
        umma_commit_w(SPLASH_RBAR(acc_done, 0));
      }
    }
  } else {
    // ========================== elementwise warpgroups ===========================
    const int w = warp >> 2;
    const int wq = warp & 3;
    const int row = wq * 32 + lane;
    const int q_pos = qi * kRows + row;
    const uint32_t tmem_row = tmem + (static_cast<uint32_t>(wq * 32) << 16);
    const int col0 = w * kHalf;
    const size_t out_row = static_cast<size_t>(q_row0) + row;

    if (total == 0) {
      if (w == 0) {
        uint4* dst = reinterpret_cast<uint4*>(static_cast<uint8_t*>(a.dq) + out_row * (D * 2));
#pragma unroll
        for (int c = 0; c < D * 2 / 16; ++c) dst[c] = make_uint4(0, 0, 0, 0);
      }
    } else {
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
      const int my_seg = a.has_seg ? a.seg_q[static_cast<size_t>(b) * a.q_len + q_pos] : 0;
      const float lse = a.lse[out_row];
      const float delta = a.delta[out_row];
      const bool row_on = lse != a.mask_value;  // rows that saw no key contribute nothing
      const float lse2 = lse * kLog2e;
      const bool cap_on = a.soft_cap > 0.f;
      const float cap = a.soft_cap, inv_cap = cap_on ? 1.f / a.soft_cap : 0.f;
      bool alive = true;
      int slot = 0;
      uint32_t phase = 0;

      for (int t = 0; t < total; ++t) {
        const uint32_t entry = step_at(t / kSub);
        const int s = static_cast<int>(entry & 0x7fffu), sb = t % kSub;
        const bool seg_compare = a.has_seg && !(entry & kSegUniformBit);
        const int j = a.block_list[sched_off + s];
        const bool partial = a.block_kind[sched_off + s] == SPLASH_BLOCK_PARTIAL;
        if (!warp_wait(SPLASH_RBAR(full, slot), phase, ctx, kRSiteEwFull, t)) { alive = false; break; }
        if (!warp_wait(SPLASH_RBAR(s_ready, 0), t & 1, ctx, kRSiteEwS, t)) { alive = false; break; }
        tc_fence_after();
        const int kv0 = j * 128 + sb * BC + col0;  // position of this thread's first column
#pragma unroll
        for (int c = 0; c < kHalf / 32; ++c) {
          uint32_t sraw[32], dpraw[32];
          tmem_ld32(tmem_row + L::kColS + col0 + c * 32, sraw);
          tmem_ld32(tmem_row + L::kColDp + col0 + c * 32, dpraw);
          tmem_wait_ld();
          uint32_t vis = row_on ? 0xffffffffu : 0u;
          if (partial && !a.has_dense) {
            const int d0 = kv0 + c * 32 - q_pos;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int d = d0 + i;
              if (d < band_lo || d > band_hi) vis &= ~(1u << i);
            }
          }
          if (partial && a.has_dense) {
            // One bit per element: 16 bytes per q row, bit = kv column inside the block.
            vis &= lds32(mask_u32 + slot * L::kMaskStage + row * 16 + (sb * BC + col0 + c * 32) / 8);
          }
          if (seg_compare) {
#pragma unroll
            for (int g = 0; g < 8; ++g) {
              const uint4 sg = lds128(seg_u32 + slot * L::kVecStage + (col0 + c * 32 + g * 4) * 4);
              if (static_cast<int>(sg.x) != my_seg) vis &= ~(1u << (g * 4 + 0));
              if (static_cast<int>(sg.y) != my_seg) vis &= ~(1u << (g * 4 + 1));
              if (static_cast<int>(sg.z) != my_seg) vis &= ~(1u << (g * 4 + 2));
              if (static_cast<int>(sg.w) != my_seg) vis &= ~(1u << (g * 4 + 3));
            }
          }
          uint32_t dspk[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float dsv[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              float sval = __uint_as_float(sraw[i + e]);
              float tanh_v = 0.f;
              if (cap_on) {
                tanh_v = tanh_approx(sval * inv_cap);
                sval = cap * tanh_v;
              }
              const float p = ((vis >> (i + e)) & 1u) ? ex2_approx(fmaf(sval, kLog2e, -lse2)) : 0.f;
              float ds = p * (__uint_as_float(dpraw[i + e]) - delta);
              if (cap_on) ds *= (1.f - tanh_v * tanh_v);
              dsv[e] = ds;
            }
            dspk[i / 2] = pack2<BF16>(dsv[0], dsv[1]);
          }
          tmem_st16(tmem_row + L::kColDs + (t & 1) * (BC / 2) + (col0 + c * 32) / 2, dspk);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(SPLASH_RBAR(empty, slot));
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(SPLASH_RBAR(ds_ready, 0));
        if (++slot == stages) { slot = 0; phase ^= 1; }
      }

      // ---- epilogue: each warpgroup casts half of the dQ columns --------------------
      if (alive) alive = warp_wait(SPLASH_RBAR(acc_done, 0), 0, ctx, kRSiteEwDone, total);
      if (alive) {
        tc_fence_after();
        constexpr int kColsPerWg = D / 2;
#pragma unroll
        for (int c = 0; c < kColsPerWg / 32; ++c) {
          const int cc = w * (kColsPerWg / 32) + c;  // 32-column chunk index within D
          uint32_t o[32];
          tmem_ld32(tmem_row + L::kColDq + cc * 32, o);
          tmem_wait_ld();
          const uint32_t box = q_u32 + (cc / 2) * (kRows * 128);  // Q tile is dead: reuse it for staging
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 wv;
            wv.x = pack2<BF16>(__uint_as_float(o[g * 8 + 0]), __uint_as_float(o[g * 8 + 1]));
            wv.y = pack2<BF16>(__uint_as_float(o[g * 8 + 2]), __uint_as_float(o[g * 8 + 3]));
            wv.z = pack2<BF16>(__uint_as_float(o[g * 8 + 4]), __uint_as_float(o[g * 8 + 5]));
            wv.w = pack2<BF16>(__uint_as_float(o[g * 8 + 6]), __uint_as_float(o[g * 8 + 7]));
            sts128(box + swz128(row, (cc & 1) * 4 + g), wv);
          }
        }
        fence_proxy_async_smem();
        mbar_arrive(SPLASH_RBAR(epi, 0));
        if (threadIdx.x == 0) {
          if (mbar_wait(SPLASH_RBAR(epi, 0), 0, ctx, kRSiteEwEpi, total)) {
#pragma unroll
            for (int c = 0; c < D / 64; ++c) tma_store_2d(&tm_dq, q_u32 + c * (kRows * 128), c * 64, q_row0);
            bulk_commit_group();
            bulk_wait_group_read<0>();
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (const uint32_t gave_up = lds32(abort_u32)) {
    if (threadIdx.x == 0) report_abort(a.status, gave_up);
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000) {}
  }
  if (warp == kEwWarps + 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem, L::kTmemCols);
  }
}

#undef SPLASH_RBAR

}  // namespace splash
