// Host launcher for the forward kernel template: builds the TMA tensor maps for one
// call and enqueues the grid.  Included by the translation units that instantiate
// the kernel for a given (head_dim, head_dim_v, block_kv, tiles) combination.
#pragma once

#include <cstdlib>

#include "dispatch.h"
#include "fwd_kernel.cuh"
#include "host_common.cuh"

namespace splash {

template <int D, int DV, int BKV, int NT, int AW, bool PLAIN, bool BF16>
int launch_fwd_plain(const SplashParams& p, cudaStream_t stream) {
  using L = FwdLayout<D, DV, BKV, NT, AW>;
  const bool dense = p.partial_blocks != nullptr;
  const bool seg = p.seg_q != nullptr;
  // The list of steps that survive segment skipping needs max_steps 16-bit entries; without room
  // for it (or with more than 2^15 steps) every scheduled block is computed.
  bool skipping = seg && p.seg_ranges != nullptr && p.max_steps < (1 << 15);
  if (skipping && L::smem_bytes(p.num_stages, dense, seg, p.max_steps) > kMaxDynamicSmem) skipping = false;
  const size_t smem = L::smem_bytes(p.num_stages, dense, seg, skipping ? p.max_steps : 0);
  if (smem > kMaxDynamicSmem) {
    char d[96];
    snprintf(d, sizeof d, "%zu > %zu bytes; reduce num_stages or block_kv", smem, kMaxDynamicSmem);
    return fail(SPLASH_BUDGET_EXCEEDED, "Shared memory budget exceeded", d);
  }
  if (!L::kOStageInQ && p.num_stages * BKV < 128)
    return fail(SPLASH_BUDGET_EXCEEDED, "Shared memory budget exceeded", "output staging needs num_stages * block_kv >= 128");

  const CUtensorMapDataType dt = tmap_dtype(p.dtype);
  const uint64_t q_rows = static_cast<uint64_t>(p.batch) * p.heads * p.q_len;
  const uint64_t kv_rows = static_cast<uint64_t>(p.batch) * p.kv_heads * p.kv_len;
  CUtensorMap tm_q, tm_k, tm_v, tm_o;
  int rc;
  if ((rc = make_tmap_2d(&tm_q, p.q, dt, 2, q_rows, D, 128, 64, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  if ((rc = make_tmap_2d(&tm_k, p.k, dt, 2, kv_rows, D, BKV, 64, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  if ((rc = make_tmap_2d(&tm_v, p.v, dt, 2, kv_rows, DV, BKV, 64, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  if ((rc = make_tmap_2d(&tm_o, p.out, dt, 2, q_rows, DV, 128, 64, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  if (dense && (reinterpret_cast<uintptr_t>(p.partial_blocks) & 15))
    return fail(SPLASH_INVALID_ARGUMENT, "partial_blocks not 16-byte aligned");

  FwdArgs a;
  a.num_steps = p.num_steps;
  a.block_order = p.block_order;
  a.block_list = p.block_list;
  a.block_kind = p.block_kind;
  a.mask_block = p.mask_block;
  a.mask_desc = p.mask_desc;
  a.seg_q = p.seg_q;
  a.seg_kv = p.seg_kv;
  a.partial_blocks = reinterpret_cast<const uint8_t*>(p.partial_blocks);
  a.seg_q_ranges = skipping ? seg_q_ranges(p) : nullptr;
  a.seg_kv_ranges = skipping ? seg_kv_ranges(p) : nullptr;
  a.out = p.out;
  a.lse_out = p.lse_out;
  a.status = p.status;
  a.batch = p.batch;
  a.heads = p.heads;
  a.kv_heads = p.kv_heads;
  a.q_len = p.q_len;
  a.kv_len = p.kv_len;
  a.mask_heads = p.mask_heads;
  a.max_steps = p.max_steps;
  a.q_blocks = p.q_len / (128 * NT);
  a.stages = p.num_stages;
  a.has_dense = dense;
  a.has_seg = seg;
  a.head_group = 8;
  a.mask_value = p.mask_value;
  a.soft_cap = p.soft_cap;

  auto kernel = splash_fwd_kernel<D, DV, BKV, NT, AW, PLAIN, BF16>;
  if ((rc = opt_in_smem(kernel, smem))) return rc;
  const unsigned grid = static_cast<unsigned>(a.q_blocks) * p.heads * p.batch;
  kernel<<<grid, L::kThreads, smem, stream>>>(tm_q, tm_k, tm_v, tm_o, a);
  SPLASH_CUDA_CHECK(cudaGetLastError());
  return SPLASH_OK;
}

// The kernel without its soft-cap, segment and streamed-mask code when the call uses none.
template <int D, int DV, int BKV, int NT, int AW, bool BF16>
int launch_fwd_typed(const SplashParams& p, cudaStream_t stream) {
  const bool plain = p.soft_cap == 0.f && p.seg_q == nullptr && p.partial_blocks == nullptr;
  if (plain) return launch_fwd_plain<D, DV, BKV, NT, AW, true, BF16>(p, stream);
  return launch_fwd_plain<D, DV, BKV, NT, AW, false, BF16>(p, stream);
}

// Softmax warpgroups that alternate over the KV steps of a one-tile kernel;
// SPLASH_FWD_AW=1|2 overrides the default (experiments).
inline int fwd_alternating_groups() {
  static const int forced = [] {
    const char* e = getenv("SPLASH_FWD_AW");
    return e ? atoi(e) : 0;
  }();
  return (forced == 1 || forced == 2) ? forced : 2;
}

template <int D, int DV, int BKV, int NT>
int launch_fwd(const SplashParams& p, cudaStream_t stream) {
  const bool bf16 = p.dtype == SPLASH_DTYPE_BF16;
  // Two alternating groups with 128-column blocks; with 64-column blocks one group
  // keeps the kernel small enough for two CTAs per SM, which serves that tiling better.
  if constexpr (NT == 1 && BKV == 128 && 3 * BKV + DV <= 512) {
    if (fwd_alternating_groups() == 2) {
      if (bf16) return launch_fwd_typed<D, DV, BKV, NT, 2, true>(p, stream);
      return launch_fwd_typed<D, DV, BKV, NT, 2, false>(p, stream);
    }
  }
  if (bf16) return launch_fwd_typed<D, DV, BKV, NT, 1, true>(p, stream);
  return launch_fwd_typed<D, DV, BKV, NT, 1, false>(p, stream);
}

}  // namespace splash
