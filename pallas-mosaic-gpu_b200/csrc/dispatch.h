// Declarations of the per-configuration launchers; each is explicitly instantiated
// in exactly one translation unit so the kernels compile in parallel.
#pragma once

#include <cuda_runtime.h>

#include "../../include/splash_sm100.h"

namespace splash {

template <int D, int DV, int BKV, int NT>
int launch_fwd(const SplashParams& p, cudaStream_t stream);

}  // namespace splash

namespace splash {

template <int D, int DV, bool FUSED>
int launch_bwd_col(const SplashParams& p, cudaStream_t stream);

template <int D, int DV, int BC>
int launch_bwd_row(const SplashParams& p, cudaStream_t stream);

template <int D, int DV, int BC>
size_t bwd_row_smem(const SplashParams& p);

// Fused backward with 128 q rows per step (head_dim 128, no streamed mask blocks).
bool bwd_wide_supported(const SplashParams& p);
int launch_bwd_wide(const SplashParams& p, cudaStream_t stream);

// delta = rowsum(dO * O); dq = cast(transpose(dq_acc)).
// When `zero` is non-null the same pass also clears zero_floats_per_row floats per row of it.
int launch_delta(const void* o, const void* d_out, float* delta, long long rows, int head_dim_v, int dtype,
                 cudaStream_t stream, float* zero = nullptr, int zero_floats_per_row = 0);
int launch_dq_transpose_cast(const float* acc, void* dq, long long batch_heads, int head_dim, int q_len, int dtype,
                             cudaStream_t stream);
// -lse and -delta of every q row as three 16-bit parts each (16 bytes per row and array): the
// operands of the slice that the 128-row fused backward adds to its score products at head_dim 64.
int launch_fold_operands(const float* lse, const float* delta, void* aux_lse, void* aux_delta, long long rows,
                         float mask_value, int dtype, cudaStream_t stream);
// Bytes of those two arrays together (they follow the f32 dQ accumulator in the fused backward's scratch).
inline long long fold_operand_bytes(const SplashParams& p) {
  return p.head_dim == 64 ? 2ll * 16 * p.batch * p.heads * p.q_len : 0;
}

// Fills p.seg_ranges (when given, with segment ids) with the (min, max) id of every 64 positions.
int launch_seg_ranges(const SplashParams& p, cudaStream_t stream);

// The two halves of p.seg_ranges as the kernels read them, or nulls when skipping is off.
inline const int2* seg_q_ranges(const SplashParams& p) {
  return (p.seg_q && p.seg_ranges) ? reinterpret_cast<const int2*>(p.seg_ranges) : nullptr;
}
inline const int2* seg_kv_ranges(const SplashParams& p) {
  return (p.seg_q && p.seg_ranges)
             ? reinterpret_cast<const int2*>(p.seg_ranges) + static_cast<long long>(p.batch) * (p.q_len / 64)
             : nullptr;
}

}  // namespace splash
