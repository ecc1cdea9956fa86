// Small memory-bound passes around the backward kernels:
//   delta = rowsum(dO * O) in f32 (what the reference leaves to XLA,
//           splash_attention_mgpu/splash_attention.py:289-290);
//   dq    = cast(transpose(dq_acc)): the fused backward accumulates dQ^T in f32 as
//           [batch*heads, head_dim, q_len] (reference backward_fused.py:506-511).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "dispatch.h"
#include "host_common.cuh"

namespace splash {

template <bool BF16>
__device__ __forceinline__ float2 unpack2(uint32_t w) {
  if constexpr (BF16) {
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
  } else {
    const __half2 h = *reinterpret_cast<const __half2*>(&w);
    return __half22float2(h);
  }
}

// One warp per group of kRows rows; each lane handles 16-byte chunks (8 elements) and
// keeps the loads of all its rows in flight together.  When `zero` is given, the warp
// also clears `zero_vec_per_row` float4 per row of it: the fused backward gets its f32
// dQ accumulator cleared by the pass that already streams O and dO.
constexpr int kDeltaRows = 4;

template <bool BF16>
__global__ void __launch_bounds__(256) delta_kernel(const uint4* __restrict__ o, const uint4* __restrict__ d_out,
                                                    float* __restrict__ delta, long long rows, int chunks_per_row,
                                                    float4* __restrict__ zero, int zero_vec_per_row) {
  const long long row0 = (static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5)) * kDeltaRows;
  const int lane = threadIdx.x & 31;
  if (row0 >= rows) return;
  float acc[kDeltaRows];
#pragma unroll
  for (int r = 0; r < kDeltaRows; ++r) acc[r] = 0.f;
  for (int c = lane; c < chunks_per_row; c += 32) {
    uint4 a[kDeltaRows], b[kDeltaRows];
#pragma unroll
    for (int r = 0; r < kDeltaRows; ++r) {
      const bool live = row0 + r < rows;
      a[r] = live ? o[(row0 + r) * chunks_per_row + c] : make_uint4(0, 0, 0, 0);
      b[r] = live ? d_out[(row0 + r) * chunks_per_row + c] : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int r = 0; r < kDeltaRows; ++r) {
      const uint32_t aw[4] = {a[r].x, a[r].y, a[r].z, a[r].w}, bw[4] = {b[r].x, b[r].y, b[r].z, b[r].w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 x = unpack2<BF16>(aw[i]), y = unpack2<BF16>(bw[i]);
        acc[r] = fmaf(x.x, y.x, acc[r]);
        acc[r] = fmaf(x.y, y.y, acc[r]);
      }
    }
  }
  if (zero) {
    const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int r = 0; r < kDeltaRows; ++r)
      if (row0 + r < rows)
        for (int c = lane; c < zero_vec_per_row; c += 32) zero[(row0 + r) * zero_vec_per_row + c] = z;
  }
#pragma unroll
  for (int r = 0; r < kDeltaRows; ++r) {
    float v = acc[r];
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
    if (lane == 0 && row0 + r < rows) delta[row0 + r] = v;
  }
}

int launch_delta(const void* o, const void* d_out, float* delta, long long rows, int head_dim_v, int dtype,
                 cudaStream_t stream, float* zero, int zero_floats_per_row) {
  if (!o || !d_out || !delta || rows <= 0 || head_dim_v % 8) return fail(SPLASH_INVALID_ARGUMENT, "bad delta arguments");
  if (zero && zero_floats_per_row % 4) return fail(SPLASH_INVALID_ARGUMENT, "bad delta arguments");
  const unsigned grid = static_cast<unsigned>((rows + 8 * kDeltaRows - 1) / (8 * kDeltaRows));
  if (dtype == SPLASH_DTYPE_BF16)
    delta_kernel<true><<<grid, 256, 0, stream>>>(static_cast<const uint4*>(o), static_cast<const uint4*>(d_out), delta,
                                                  rows, head_dim_v / 8, reinterpret_cast<float4*>(zero),
                                                  zero_floats_per_row / 4);
  else
    delta_kernel<false><<<grid, 256, 0, stream>>>(static_cast<const uint4*>(o), static_cast<const uint4*>(d_out), delta,
                                                   rows, head_dim_v / 8, reinterpret_cast<float4*>(zero),
                                                   zero_floats_per_row / 4);
  SPLASH_CUDA_CHECK(cudaGetLastError());
  return SPLASH_OK;
}

// acc: [bh, d, q] f32  ->  dq: [bh, q, d] 16-bit, in tiles of 64 (d) x 64 (q).  Reads are
// 256-byte runs along q; each warp store covers 128 contiguous bytes along d.
template <bool BF16>
__global__ void __launch_bounds__(256) dq_transpose_cast_kernel(const float* __restrict__ acc, uint16_t* __restrict__ dq,
                                                                int head_dim, int q_len) {
  __shared__ float tile[64][65];
  // blockIdx.x runs over (batch * heads, q tiles): the z extent of a grid stops at 65535.
  const int q_tiles = q_len / 64;
  const long long bh = blockIdx.x / q_tiles;
  const int d0 = blockIdx.y * 64, q0 = (blockIdx.x % q_tiles) * 64;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float* src = acc + (bh * head_dim + d0) * static_cast<long long>(q_len) + q0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int d = warp * 8 + i;
    const float2 v = *reinterpret_cast<const float2*>(src + static_cast<long long>(d) * q_len + 2 * lane);
    tile[d][2 * lane] = v.x;
    tile[d][2 * lane + 1] = v.y;
  }
  __syncthreads();
  uint16_t* dst = dq + (bh * q_len + q0) * static_cast<long long>(head_dim) + d0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int q = warp * 8 + i;
    const float lo = tile[2 * lane][q], hi = tile[2 * lane + 1][q];
    uint32_t w;
    if constexpr (BF16) {
      const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
      w = *reinterpret_cast<const uint32_t*>(&v);
    } else {
      const __half2 v = __floats2half2_rn(lo, hi);
      w = *reinterpret_cast<const uint32_t*>(&v);
    }
    *reinterpret_cast<uint32_t*>(dst + static_cast<long long>(q) * head_dim + 2 * lane) = w;
  }
}

// Splits -x into three 16-bit floats whose sum is -x to f32 precision, as the eight 16-bit
// values {hi, mid, lo, 0, 0, 0, 0, 0} per row that the 128-row fused backward (head_dim 64)
// multiplies by {1, 1, 1, 0, ...} in one extra K = 16 slice of its score products.  Rows whose
// lse is mask_value (they saw no key) get a large negative value instead, which makes their P zero.
template <bool BF16>
__device__ __forceinline__ uint4 split3_neg(float x, bool sentinel) {
  float v = sentinel ? (BF16 ? -1.0e30f : -60000.f) : -x;
  uint32_t h[3];
#pragma unroll
  for (int i = 0; i < 3; ++i) {
    if constexpr (BF16) {
      const __nv_bfloat16 b = __float2bfloat16_rn(v);
      h[i] = *reinterpret_cast<const uint16_t*>(&b);
      v -= __bfloat162float(b);
    } else {
      const __half b = __float2half_rn(v);
      h[i] = *reinterpret_cast<const uint16_t*>(&b);
      v -= __half2float(b);
    }
  }
  return make_uint4(h[0] | (h[1] << 16), h[2], 0u, 0u);
}

template <bool BF16>
__global__ void __launch_bounds__(256) fold_operands_kernel(const float* __restrict__ lse, const float* __restrict__ delta,
                                                            uint4* __restrict__ aux_lse, uint4* __restrict__ aux_delta,
                                                            long long rows, float mask_value) {
  const long long r = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
  if (r >= rows) return;
  const float l = lse[r];
  aux_lse[r] = split3_neg<BF16>(l, l == mask_value);
  aux_delta[r] = split3_neg<BF16>(delta[r], false);
}

int launch_fold_operands(const float* lse, const float* delta, void* aux_lse, void* aux_delta, long long rows,
                         float mask_value, int dtype, cudaStream_t stream) {
  const unsigned grid = static_cast<unsigned>((rows + 255) / 256);
  if (dtype == SPLASH_DTYPE_BF16)
    fold_operands_kernel<true><<<grid, 256, 0, stream>>>(lse, delta, static_cast<uint4*>(aux_lse),
                                                         static_cast<uint4*>(aux_delta), rows, mask_value);
  else
    fold_operands_kernel<false><<<grid, 256, 0, stream>>>(lse, delta, static_cast<uint4*>(aux_lse),
                                                          static_cast<uint4*>(aux_delta), rows, mask_value);
  SPLASH_CUDA_CHECK(cudaGetLastError());
  return SPLASH_OK;
}

// (min, max) of every 64 consecutive segment ids: one warp per chunk, two ids per lane.
// `out` holds the q part [batch, q_len / 64] followed by the kv part [batch, kv_len / 64].
__global__ void __launch_bounds__(256) seg_ranges_kernel(const int32_t* __restrict__ seg_q,
                                                         const int32_t* __restrict__ seg_kv, int2* __restrict__ out,
                                                         long long q_chunks, long long kv_chunks) {
  const long long chunk = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (chunk >= q_chunks + kv_chunks) return;
  const int32_t* src = chunk < q_chunks ? seg_q + chunk * 64 : seg_kv + (chunk - q_chunks) * 64;
  const int2 v = *reinterpret_cast<const int2*>(src + 2 * lane);
  int lo = min(v.x, v.y), hi = max(v.x, v.y);
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) {
    lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, s));
    hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, s));
  }
  if (lane == 0) out[chunk] = make_int2(lo, hi);
}

int launch_seg_ranges(const SplashParams& p, cudaStream_t stream) {
  if (!p.seg_q || !p.seg_kv || !p.seg_ranges) return SPLASH_OK;
  if (p.q_len % 64 || p.kv_len % 64) return fail(SPLASH_INVALID_ARGUMENT, "segment ranges need sequence lengths that are multiples of 64");
  const long long q_chunks = static_cast<long long>(p.batch) * (p.q_len / 64);
  const long long kv_chunks = static_cast<long long>(p.batch) * (p.kv_len / 64);
  const unsigned grid = static_cast<unsigned>((q_chunks + kv_chunks + 7) / 8);
  seg_ranges_kernel<<<grid, 256, 0, stream>>>(p.seg_q, p.seg_kv, reinterpret_cast<int2*>(p.seg_ranges), q_chunks,
                                               kv_chunks);
  SPLASH_CUDA_CHECK(cudaGetLastError());
  return SPLASH_OK;
}

int launch_dq_transpose_cast(const float* acc, void* dq, long long batch_heads, int head_dim, int q_len, int dtype,
                             cudaStream_t stream) {
  if (!acc || !dq || head_dim % 64 || q_len % 64) return fail(SPLASH_INVALID_ARGUMENT, "bad dq cast arguments");
  if (batch_heads * (q_len / 64) >= (1ll << 31)) return fail(SPLASH_INVALID_ARGUMENT, "batch * heads * q_len too large");
  dim3 grid(static_cast<unsigned>(batch_heads * (q_len / 64)), head_dim / 64, 1);
  if (dtype == SPLASH_DTYPE_BF16)
    dq_transpose_cast_kernel<true><<<grid, 256, 0, stream>>>(acc, static_cast<uint16_t*>(dq), head_dim, q_len);
  else
    dq_transpose_cast_kernel<false><<<grid, 256, 0, stream>>>(acc, static_cast<uint16_t*>(dq), head_dim, q_len);
  SPLASH_CUDA_CHECK(cudaGetLastError());
  return SPLASH_OK;
}

}  // namespace splash
