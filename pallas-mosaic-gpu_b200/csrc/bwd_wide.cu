// Launcher of the 128-row-per-step fused backward (bwd_wide_kernel.cuh).
#include "bwd_launch.cuh"
#include "bwd_wide_kernel.cuh"
#include "dispatch.h"

namespace splash {

bool bwd_wide_supported(const SplashParams& p) {
  return (p.head_dim == 128 || p.head_dim == 64) && p.head_dim_v == p.head_dim && p.partial_blocks == nullptr;
}

template <int D, bool BF16>
static int launch_bwd_wide_typed(const SplashParams& p, cudaStream_t stream) {
  using L = WideLayout<D>;
  const bool seg = p.seg_q != nullptr;
  const CUtensorMapDataType dt = tmap_dtype(p.dtype);
  const uint64_t q_rows = static_cast<uint64_t>(p.batch) * p.heads * p.q_len;
  const uint64_t kv_rows = static_cast<uint64_t>(p.batch) * p.kv_heads * p.kv_len;
  CUtensorMap tm_q, tm_k, tm_v, tm_do, tm_dk, tm_dv, tm_dqacc;
  int rc;
  if ((rc = make_tmap_2d(&tm_q, p.q, dt, 2, q_rows, D, 128, 64, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  if ((rc = make_tmap_2d(&tm_do, p.d_out, dt, 2, q_rows, D, 128, 64, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  if ((rc = make_tmap_2d(&tm_k, p.k, dt, 2, kv_rows, D, 128, 64, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  if ((rc = make_tmap_2d(&tm_v, p.v, dt, 2, kv_rows, D, 128, 64, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  if ((rc = make_tmap_2d(&tm_dk, p.dk, dt, 2, kv_rows, D, 128, 64, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  if ((rc = make_tmap_2d(&tm_dv, p.dv, dt, 2, kv_rows, D, 128, 64, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  // f32 accumulator viewed as [batch * heads * head_dim, q_len]; tiles of 32 rows x 32 q columns.
  const uint64_t acc_rows = static_cast<uint64_t>(p.batch) * p.heads * D;
  if ((rc = make_tmap_2d(&tm_dqacc, p.dq_acc, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, acc_rows, p.q_len, 32, 32,
                         CU_TENSOR_MAP_SWIZZLE_128B)))
    return rc;
  BwdArgs a;
  fill_bwd_args(a, p, false, seg);
  a.stages = L::kSlots;
  if (L::kFold) {
    // The scratch holds the f32 dQ accumulator, then the folded -lse and -delta operands.
    const long long rows = static_cast<long long>(p.batch) * p.heads * p.q_len;
    uint8_t* aux = reinterpret_cast<uint8_t*>(p.dq_acc) + rows * D * 4;
    a.aux_lse = aux;
    a.aux_delta = aux + rows * 16;
    if ((rc = launch_fold_operands(p.lse, p.delta, aux, aux + rows * 16, rows, p.mask_value, p.dtype, stream))) return rc;
  }
  // Segment skipping when the CTA's list of block steps fits the room set aside for it.
  const bool skipping = seg && p.seg_ranges != nullptr && (p.heads / p.kv_heads) * p.max_steps <= L::kListSteps;
  a.seg_q_ranges = skipping ? seg_q_ranges(p) : nullptr;
  a.seg_kv_ranges = skipping ? seg_kv_ranges(p) : nullptr;
  const bool plain = p.soft_cap == 0.f && !seg;
  auto kernel = plain ? splash_bwd_wide_kernel<D, true, BF16> : splash_bwd_wide_kernel<D, false, BF16>;
  if ((rc = opt_in_smem(kernel, L::kSmemBytes))) return rc;
  const unsigned grid = static_cast<unsigned>(a.kv_blocks) * p.kv_heads * p.batch;
  kernel<<<grid, L::kThreads, L::kSmemBytes, stream>>>(tm_q, tm_k, tm_v, tm_do, tm_dk, tm_dv, tm_dqacc, a);
  SPLASH_CUDA_CHECK(cudaGetLastError());
  return SPLASH_OK;
}

int launch_bwd_wide(const SplashParams& p, cudaStream_t stream) {
  if (!bwd_wide_supported(p))
    return fail(SPLASH_UNSUPPORTED, "the 128-row fused backward needs head_dim == head_dim_v in {64, 128} and no streamed mask blocks");
  if (p.head_dim == 64) {
    if (p.dtype == SPLASH_DTYPE_BF16) return launch_bwd_wide_typed<64, true>(p, stream);
    return launch_bwd_wide_typed<64, false>(p, stream);
  }
  if (p.dtype == SPLASH_DTYPE_BF16) return launch_bwd_wide_typed<128, true>(p, stream);
  return launch_bwd_wide_typed<128, false>(p, stream);
}

}  // namespace splash
