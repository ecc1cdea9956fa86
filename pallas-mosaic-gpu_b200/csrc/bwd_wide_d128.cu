// Launcher of the 128-row-per-step fused backward (bwd_wide_kernel.cuh).
#include "bwd_launch.cuh"
#include "bwd_wide_kernel.cuh"
#include "dispatch.h"

namespace splash {

bool bwd_wide_supported(const SplashParams& p) {
  return p.head_dim == 128 && p.head_dim_v == 128 && p.partial_blocks == nullptr;
}

template <bool BF16>
static int launch_bwd_wide_typed(const SplashParams& p, cudaStream_t stream) {
  using L = WideLayout;
  const bool seg = p.seg_q != nullptr;
  const CUtensorMapDataType dt = tmap_dtype(p.dtype);
  const uint64_t q_rows = static_cast<uint64_t>(p.batch) * p.heads * p.q_len;
  const uint64_t kv_rows = static_cast<uint64_t>(p.batch) * p.kv_heads * p.kv_len;
  CUtensorMap tm_q, tm_k, tm_v, tm_do, tm_dk, tm_dv, tm_dqacc;
  int rc;
  if ((rc = make_tmap_2d(&tm_q, p.q, dt, 2, q_rows, 128, 128, 64, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  if ((rc = make_tmap_2d(&tm_do, p.d_out, dt, 2, q_rows, 128, 128, 64, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  if ((rc = make_tmap_2d(&tm_k, p.k, dt, 2, kv_rows, 128, 128, 64, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  if ((rc = make_tmap_2d(&tm_v, p.v, dt, 2, kv_rows, 128, 128, 64, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  if ((rc = make_tmap_2d(&tm_dk, p.dk, dt, 2, kv_rows, 128, 128, 64, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  if ((rc = make_tmap_2d(&tm_dv, p.dv, dt, 2, kv_rows, 128, 128, 64, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  // f32 accumulator viewed as [batch * heads * head_dim, q_len]; tiles of 32 rows x 32 q columns.
  const uint64_t acc_rows = static_cast<uint64_t>(p.batch) * p.heads * 128;
  if ((rc = make_tmap_2d(&tm_dqacc, p.dq_acc, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, acc_rows, p.q_len, 32, 32,
                         CU_TENSOR_MAP_SWIZZLE_128B)))
    return rc;
  BwdArgs a;
  fill_bwd_args(a, p, false, seg);
  a.stages = L::kSlots;
  // Segment skipping when the CTA's list of block steps fits the room set aside for it.
  const bool skipping = seg && p.seg_ranges != nullptr && (p.heads / p.kv_heads) * p.max_steps <= L::kListSteps;
  a.seg_q_ranges = skipping ? seg_q_ranges(p) : nullptr;
  a.seg_kv_ranges = skipping ? seg_kv_ranges(p) : nullptr;
  const bool plain = p.soft_cap == 0.f && !seg;
  auto kernel = plain ? splash_bwd_wide_kernel<true, BF16> : splash_bwd_wide_kernel<false, BF16>;
  if ((rc = opt_in_smem(kernel, L::kSmemBytes))) return rc;
  const unsigned grid = static_cast<unsigned>(a.kv_blocks) * p.kv_heads * p.batch;
  kernel<<<grid, L::kThreads, L::kSmemBytes, stream>>>(tm_q, tm_k, tm_v, tm_do, tm_dk, tm_dv, tm_dqacc, a);
  SPLASH_CUDA_CHECK(cudaGetLastError());
  return SPLASH_OK;
}

int launch_bwd_wide(const SplashParams& p, cudaStream_t stream) {
  if (!bwd_wide_supported(p)) return fail(SPLASH_UNSUPPORTED, "the 128-row fused backward needs head_dim 128 and no streamed mask blocks");
  if (p.dtype == SPLASH_DTYPE_BF16) return launch_bwd_wide_typed<true>(p, stream);
  return launch_bwd_wide_typed<false>(p, stream);
}

}  // namespace splash
