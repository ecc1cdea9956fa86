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

// One warp per row; each lane handles 16-byte chunks (8 elements).
template <bool BF16>
__global__ void __launch_bounds__(256) delta_kernel(const uint4* __restrict__ o, const uint4* __restrict__ d_out,
                                                    float* __restrict__ delta, long long rows, int chunks_per_row) {
  const long long row = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  float acc = 0.f;
  for (int c = lane; c < chunks_per_row; c += 32) {
    const uint4 a = o[row * chunks_per_row + c];
    const uint4 b = d_out[row * chunks_per_row + c];
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 x = unpack2<BF16>(aw[i]), y = unpack2<BF16>(bw[i]);
      acc = fmaf(x.x, y.x, acc);
      acc = fmaf(x.y, y.y, acc);
    }
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
  if (lane == 0) delta[row] = acc;
}

int launch_delta(const void* o, const void* d_out, float* delta, long long rows, int head_dim_v, int dtype,
                 cudaStream_t stream) {
  if (!o || !d_out || !delta || rows <= 0 || head_dim_v % 8) return fail(SPLASH_INVALID_ARGUMENT, "bad delta arguments");
  const unsigned grid = static_cast<unsigned>((rows + 7) / 8);
  if (dtype == SPLASH_DTYPE_BF16)
    delta_kernel<true><<<grid, 256, 0, stream>>>(static_cast<const uint4*>(o), static_cast<const uint4*>(d_out), delta,
                                                  rows, head_dim_v / 8);
  else
    delta_kernel<false><<<grid, 256, 0, stream>>>(static_cast<const uint4*>(o), static_cast<const uint4*>(d_out), delta,
                                                   rows, head_dim_v / 8);
  SPLASH_CUDA_CHECK(cudaGetLastError());
  return SPLASH_OK;
}

// acc: [bh, d, q] f32  ->  dq: [bh, q, d] 16-bit.  Tiles of 32 (d) x 64 (q).
template <bool BF16>
__global__ void __launch_bounds__(256) dq_transpose_cast_kernel(const float* __restrict__ acc, uint16_t* __restrict__ dq,
                                                                int head_dim, int q_len) {
  __shared__ float tile[32][65];
  const long long bh = blockIdx.z;
  const int d0 = blockIdx.y * 32, q0 = blockIdx.x * 64;
  const float* src = acc + (bh * head_dim + d0) * static_cast<long long>(q_len) + q0;
  for (int i = threadIdx.x; i < 32 * 64; i += 256) {
    const int d = i / 64, q = i % 64;
    tile[d][q] = src[static_cast<long long>(d) * q_len + q];
  }
  __syncthreads();
  uint16_t* dst = dq + (bh * q_len + q0) * static_cast<long long>(head_dim) + d0;
  for (int i = threadIdx.x; i < 64 * 16; i += 256) {
    const int q = i / 16, dp = (i % 16) * 2;
    uint32_t w;
    if constexpr (BF16) {
      const __nv_bfloat162 v = __floats2bfloat162_rn(tile[dp][q], tile[dp + 1][q]);
      w = *reinterpret_cast<const uint32_t*>(&v);
    } else {
      const __half2 v = __floats2half2_rn(tile[dp][q], tile[dp + 1][q]);
      w = *reinterpret_cast<const uint32_t*>(&v);
    }
    *reinterpret_cast<uint32_t*>(dst + static_cast<long long>(q) * head_dim + dp) = w;
  }
}

int launch_dq_transpose_cast(const float* acc, void* dq, long long batch_heads, int head_dim, int q_len, int dtype,
                             cudaStream_t stream) {
  if (!acc || !dq || head_dim % 32 || q_len % 64) return fail(SPLASH_INVALID_ARGUMENT, "bad dq cast arguments");
  dim3 grid(q_len / 64, head_dim / 32, static_cast<unsigned>(batch_heads));
  if (dtype == SPLASH_DTYPE_BF16)
    dq_transpose_cast_kernel<true><<<grid, 256, 0, stream>>>(acc, static_cast<uint16_t*>(dq), head_dim, q_len);
  else
    dq_transpose_cast_kernel<false><<<grid, 256, 0, stream>>>(acc, static_cast<uint16_t*>(dq), head_dim, q_len);
  SPLASH_CUDA_CHECK(cudaGetLastError());
  return SPLASH_OK;
}

}  // namespace splash
