// Host launchers for the backward kernel templates.
#pragma once

#include "bwd_col_kernel.cuh"
#include "bwd_row_kernel.cuh"
#include "dispatch.h"
#include "host_common.cuh"

namespace splash {

inline void fill_bwd_args(BwdArgs& a, const SplashParams& p, bool dense, bool seg) {
  a.num_steps = p.num_steps;
  a.block_order = p.block_order;
  a.block_list = p.block_list;
  a.block_kind = p.block_kind;
  a.mask_block = p.mask_block;
  a.mask_desc = p.mask_desc;
  a.seg_q = p.seg_q;
  a.seg_kv = p.seg_kv;
  a.partial_blocks = reinterpret_cast<const uint8_t*>(p.partial_blocks);
  a.seg_q_ranges = nullptr;
  a.seg_kv_ranges = nullptr;
  a.lse = p.lse;
  a.delta = p.delta;
  a.aux_lse = nullptr;
  a.aux_delta = nullptr;
  a.dq = p.dq;
  a.dk = p.dk;
  a.dv = p.dv;
  a.status = p.status;
  a.batch = p.batch;
  a.heads = p.heads;
  a.kv_heads = p.kv_heads;
  a.q_len = p.q_len;
  a.kv_len = p.kv_len;
  a.mask_heads = p.mask_heads;
  a.max_steps = p.max_steps;
  a.q_blocks = p.q_len / 128;
  a.kv_blocks = p.kv_len / 128;
  a.stages = p.num_stages;
  a.has_dense = dense;
  a.has_seg = seg;
  a.head_group = 4;
  a.mask_value = p.mask_value;
  a.soft_cap = p.soft_cap;
}

template <int D, int DV, bool FUSED, bool BF16>
int launch_bwd_col_typed(const SplashParams& p, cudaStream_t stream) {
  using L = ColLayout<D, DV, FUSED>;
  constexpr int BC = kColBC;
  const bool dense = p.partial_blocks != nullptr;
  const bool seg = p.seg_q != nullptr;
  // Ring depth: the kernel keeps the Q/dO tiles of three consecutive steps in flight, so
  // three stages (or the caller's larger request) are used when they fit, two otherwise.
  int stages = p.num_stages < 3 ? 3 : (p.num_stages > kBwdMaxStages ? kBwdMaxStages : p.num_stages);
  while (stages > 2 && L::smem_bytes(stages, dense, seg) > kMaxDynamicSmem) --stages;
  // Segment skipping keeps a list of up to group * max_steps block steps per CTA (16-bit entries);
  // without room for it every scheduled block is computed.
  const int list_steps = (p.heads / p.kv_heads) * p.max_steps;
  const bool skipping = seg && p.seg_ranges != nullptr && list_steps < (1 << 15) &&
                        L::smem_bytes(stages, dense, seg, list_steps) <= kMaxDynamicSmem;
  const size_t smem = L::smem_bytes(stages, dense, seg, skipping ? list_steps : 0);
  if (smem > kMaxDynamicSmem) {
    char d[96];
    snprintf(d, sizeof d, "%zu > %zu bytes", smem, kMaxDynamicSmem);
    return fail(SPLASH_BUDGET_EXCEEDED, "shared memory budget exceeded", d);
  }
  const CUtensorMapDataType dt = tmap_dtype(p.dtype);
  const uint64_t q_rows = static_cast<uint64_t>(p.batch) * p.heads * p.q_len;
  const uint64_t kv_rows = static_cast<uint64_t>(p.batch) * p.kv_heads * p.kv_len;
  CUtensorMap tm_q, tm_k, tm_v, tm_do, tm_dk, tm_dv, tm_dqacc;
  memset(&tm_dqacc, 0, sizeof tm_dqacc);
  if (dense && (reinterpret_cast<uintptr_t>(p.partial_blocks) & 15))
    return fail(SPLASH_INVALID_ARGUMENT, "partial_blocks not 16-byte aligned");
  int rc;
  if ((rc = make_tmap_2d(&tm_q, p.q, dt, 2, q_rows, D, BC, 64, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  if ((rc = make_tmap_2d(&tm_do, p.d_out, dt, 2, q_rows, DV, BC, 64, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  if ((rc = make_tmap_2d(&tm_k, p.k, dt, 2, kv_rows, D, 128, 64, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  if ((rc = make_tmap_2d(&tm_v, p.v, dt, 2, kv_rows, DV, 128, 64, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  if ((rc = make_tmap_2d(&tm_dk, p.dk, dt, 2, kv_rows, D, 128, 64, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  if ((rc = make_tmap_2d(&tm_dv, p.dv, dt, 2, kv_rows, DV, 128, 64, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  if (FUSED) {
    // f32 accumulator viewed as [batch * heads * head_dim, q_len]; tiles of 32 q columns.
    const uint64_t acc_rows = static_cast<uint64_t>(p.batch) * p.heads * D;
    if ((rc = make_tmap_2d(&tm_dqacc, p.dq_acc, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, acc_rows, p.q_len, D, 32,
                           CU_TENSOR_MAP_SWIZZLE_128B)))
      return rc;
  }
  BwdArgs a;
  fill_bwd_args(a, p, dense, seg);
  a.stages = stages;
  a.seg_q_ranges = skipping ? seg_q_ranges(p) : nullptr;
  a.seg_kv_ranges = skipping ? seg_kv_ranges(p) : nullptr;
  // The kernel without its soft-cap, segment and streamed-mask code when the call uses none.
  const bool plain = p.soft_cap == 0.f && !seg && !dense;
  auto kernel = plain ? splash_bwd_col_kernel<D, DV, FUSED, true, BF16> : splash_bwd_col_kernel<D, DV, FUSED, false, BF16>;
  if ((rc = opt_in_smem(kernel, smem))) return rc;
  const unsigned grid = static_cast<unsigned>(a.kv_blocks) * p.kv_heads * p.batch;
  kernel<<<grid, L::kThreads, smem, stream>>>(tm_q, tm_k, tm_v, tm_do, tm_dk, tm_dv, tm_dqacc, a);
  SPLASH_CUDA_CHECK(cudaGetLastError());
  return SPLASH_OK;
}

template <int D, int DV, bool FUSED>
int launch_bwd_col(const SplashParams& p, cudaStream_t stream) {
  if (p.dtype == SPLASH_DTYPE_BF16) return launch_bwd_col_typed<D, DV, FUSED, true>(p, stream);
  return launch_bwd_col_typed<D, DV, FUSED, false>(p, stream);
}

template <int D, int DV, int BC>
size_t bwd_row_smem(const SplashParams& p) {
  return RowLayout<D, DV, BC>::smem_bytes(p.num_stages, p.partial_blocks != nullptr, p.seg_q != nullptr);
}

template <int D, int DV, int BC, bool BF16>
int launch_bwd_row_typed(const SplashParams& p, cudaStream_t stream) {
  using L = RowLayout<D, DV, BC>;
  const bool dense = p.partial_blocks != nullptr;
  const bool seg = p.seg_q != nullptr;
  // The list of block steps that survive segment skipping needs max_steps 16-bit entries;
  // without room for it the kernel runs every scheduled step.
  const bool skipping = seg && p.seg_ranges != nullptr && p.max_steps < (1 << 15) &&
                        L::smem_bytes(p.num_stages, dense, seg, p.max_steps) <= kMaxDynamicSmem;
  const size_t smem = L::smem_bytes(p.num_stages, dense, seg, skipping ? p.max_steps : 0);
  if (smem > kMaxDynamicSmem) {
    char d[96];
    snprintf(d, sizeof d, "%zu > %zu bytes; reduce num_stages or the sub-block sizes", smem, kMaxDynamicSmem);
    return fail(SPLASH_BUDGET_EXCEEDED, "shared memory budget exceeded", d);
  }
  const CUtensorMapDataType dt = tmap_dtype(p.dtype);
  const uint64_t q_rows = static_cast<uint64_t>(p.batch) * p.heads * p.q_len;
  const uint64_t kv_rows = static_cast<uint64_t>(p.batch) * p.kv_heads * p.kv_len;
  CUtensorMap tm_q, tm_k, tm_v, tm_do, tm_dq;
  if (dense && (reinterpret_cast<uintptr_t>(p.partial_blocks) & 15))
    return fail(SPLASH_INVALID_ARGUMENT, "partial_blocks not 16-byte aligned");
  int rc;
  if ((rc = make_tmap_2d(&tm_q, p.q, dt, 2, q_rows, D, 128, 64, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  if ((rc = make_tmap_2d(&tm_do, p.d_out, dt, 2, q_rows, DV, 128, 64, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  if ((rc = make_tmap_2d(&tm_k, p.k, dt, 2, kv_rows, D, BC, 64, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  if ((rc = make_tmap_2d(&tm_v, p.v, dt, 2, kv_rows, DV, BC, 64, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  if ((rc = make_tmap_2d(&tm_dq, p.dq, dt, 2, q_rows, D, 128, 64, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  BwdArgs a;
  fill_bwd_args(a, p, dense, seg);
  a.seg_q_ranges = skipping ? seg_q_ranges(p) : nullptr;
  a.seg_kv_ranges = skipping ? seg_kv_ranges(p) : nullptr;
  auto kernel = splash_bwd_row_kernel<D, DV, BC, BF16>;
  if ((rc = opt_in_smem(kernel, smem))) return rc;
  const unsigned grid = static_cast<unsigned>(a.q_blocks) * p.heads * p.batch;
  kernel<<<grid, L::kThreads, smem, stream>>>(tm_q, tm_k, tm_v, tm_do, tm_dq, a);
  SPLASH_CUDA_CHECK(cudaGetLastError());
  return SPLASH_OK;
}

template <int D, int DV, int BC>
int launch_bwd_row(const SplashParams& p, cudaStream_t stream) {
  if (p.dtype == SPLASH_DTYPE_BF16) return launch_bwd_row_typed<D, DV, BC, true>(p, stream);
  return launch_bwd_row_typed<D, DV, BC, false>(p, stream);
}

}  // namespace splash
