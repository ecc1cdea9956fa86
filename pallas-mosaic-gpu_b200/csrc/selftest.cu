// Single-tile tcgen05 GEMM that exercises every operand form the attention kernels
// use: K-major and MN-major shared-memory descriptors (128-byte swizzle, filled by
// TMA) and an A operand staged through tensor memory as packed 16-bit values.
// The test-suite compares its output with a plain matmul, which pins the
// descriptor encodings independently of the attention kernels.
#include "host_common.cuh"
#include "ptx.cuh"

namespace splash {

struct SelftestBars {
  uint64_t full, done;
  uint32_t tmem_base;
  int abort_flag;
};

__global__ void __launch_bounds__(128, 1)
selftest_umma_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                     const void* a_gmem, const void* b_gmem, float* d_gmem, int n, int kd, int a_mode, int b_mode, int bf16,
                     int32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* a_smem = smem;                  // up to 128 x 256 x 2 bytes
  uint8_t* b_smem = smem + 64 * 1024;      // up to 256 x 256 x 2 bytes
  SelftestBars* bars = reinterpret_cast<SelftestBars*>(smem + 192 * 1024);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    bars->abort_flag = 0;
    mbar_init(smem_u32(&bars->full), 1);
    mbar_init(smem_u32(&bars->done), 1);
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  __syncthreads();
  if (warp == 0) {
    tmem_alloc(smem_u32(&bars->tmem_base), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;
  WaitCtx ctx{smem_u32(&bars->abort_flag)};
  const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
  const int row = warp * 32 + lane;
  const uint32_t a_tmem_col = 256;  // A operand columns when staged in tensor memory

  if (a_mode == 2) {
    // Each thread packs its own row of A and stores it into tensor memory.
    const uint16_t* arow = static_cast<const uint16_t*>(a_gmem) + static_cast<size_t>(row) * kd;
    for (int c = 0; c < kd / 32; ++c) {
      uint32_t w[16];
#pragma unroll
      for (int i = 0; i < 16; ++i)
        w[i] = static_cast<uint32_t>(arow[c * 32 + 2 * i]) | (static_cast<uint32_t>(arow[c * 32 + 2 * i + 1]) << 16);
      tmem_st16(tmem + lane_base + a_tmem_col + c * 16, w);
    }
    tmem_wait_st();
  }
  if (a_mode == 4) {
    // Unswizzled core-matrix layout, written by the threads themselves.
    const uint16_t* arow = static_cast<const uint16_t*>(a_gmem) + static_cast<size_t>(row) * kd;
    for (int k = 0; k < kd; ++k) *reinterpret_cast<uint16_t*>(a_smem + core_matrix_offset(row, k, kd)) = arow[k];
  }
  if (b_mode == 2) {
    for (int r = row; r < n; r += 128) {
      const uint16_t* brow = static_cast<const uint16_t*>(b_gmem) + static_cast<size_t>(r) * kd;
      for (int k = 0; k < kd; ++k) *reinterpret_cast<uint16_t*>(b_smem + core_matrix_offset(r, k, kd)) = brow[k];
    }
  }
  if (a_mode == 4 || b_mode == 2) fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  if (a_mode == 3) {
    // Wait-limit check: nothing ever arrives on this barrier, so the bounded wait runs
    // out (about a second), records site 102 / step 7 and the kernel unwinds normally.
    if (warp == 0) warp_wait(smem_u32(&bars->full), 0, ctx, 102, 7);
  } else if (threadIdx.x == 0) {
    uint32_t bytes = (b_mode == 2 ? 0 : n * kd * 2) + ((a_mode == 2 || a_mode == 4) ? 0 : 128 * kd * 2);
    const uint32_t full = smem_u32(&bars->full);
    if (bytes > 0) mbar_arrive_expect_tx(full, bytes);
    if (a_mode == 0) {
      for (int c = 0; c < kd / 64; ++c) tma_load_2d(smem_u32(a_smem) + c * (128 * 128), &tm_a, c * 64, 0, full);
    } else if (a_mode == 1) {
      for (int c = 0; c < 2; ++c) tma_load_2d(smem_u32(a_smem) + c * (kd * 128), &tm_a, c * 64, 0, full);
    }
    if (b_mode == 0) {
      for (int c = 0; c < kd / 64; ++c) tma_load_2d(smem_u32(b_smem) + c * (n * 128), &tm_b, c * 64, 0, full);
    } else if (b_mode == 1) {
      for (int c = 0; c < n / 64; ++c) tma_load_2d(smem_u32(b_smem) + c * (kd * 128), &tm_b, c * 64, 0, full);
    }
    if (bytes == 0) mbar_arrive(full);
    if (mbar_wait(full, 0, ctx, 100, 0)) {
      tc_fence_after();
      const uint32_t idesc = make_idesc(bf16 != 0, 128, n, a_mode == 1, b_mode == 1);
      const uint32_t a_addr = smem_u32(a_smem), b_addr = smem_u32(b_smem);
      for (int kk = 0; kk < kd / 16; ++kk) {
        const uint32_t plain_hi = desc_hi_plain((kd / 8) * 128);
        uint64_t bdesc;
        if (b_mode == 0)
          bdesc = make_smem_desc(b_addr + (kk / 4) * (n * 128) + (kk % 4) * 32, 16, 1024);
        else if (b_mode == 1)
          bdesc = make_smem_desc(b_addr + kk * 2048, kd * 128, 1024);
        else
          bdesc = (static_cast<uint64_t>(plain_hi) << 32) | desc_lo_plain(b_addr + kk * 256, 128);
        if (a_mode == 2) {
          umma_ts(tmem, tmem + a_tmem_col + kk * 8, bdesc, idesc, kk > 0);
        } else {
          uint64_t adesc;
          if (a_mode == 0)
            adesc = make_smem_desc(a_addr + (kk / 4) * (128 * 128) + (kk % 4) * 32, 16, 1024);
          else if (a_mode == 1)
            adesc = make_smem_desc(a_addr + kk * 2048, kd * 128, 1024);
          else
            adesc = (static_cast<uint64_t>(plain_hi) << 32) | desc_lo_plain(a_addr + kk * 256, 128);
          umma_ss(tmem, adesc, bdesc, idesc, kk > 0);
        }
      }
      umma_commit(smem_u32(&bars->done));
    }
  }
  __syncwarp();
  if (a_mode != 3 && warp_wait(smem_u32(&bars->done), 0, ctx, 101, 0)) {
    tc_fence_after();
    for (int c = 0; c < n / 16; ++c) {
      uint32_t r[16];
      tmem_ld16(tmem + lane_base + c * 16, r);
      tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 16; ++i) d_gmem[static_cast<size_t>(row) * n + c * 16 + i] = __uint_as_float(r[i]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && bars->abort_flag) report_abort(status, static_cast<uint32_t>(bars->abort_flag));
  if (warp == 0) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace splash

extern "C" int splash_selftest_umma(const void* a, const void* b, float* d, int32_t n, int32_t kd, int32_t a_mode,
                                    int32_t b_mode, int32_t dtype, int32_t* status, void* stream) {
  using namespace splash;
  if (!a || !b || !d || !status) return fail(SPLASH_INVALID_ARGUMENT, "null pointer");
  if (n % 64 || n < 64 || n > 256 || kd % 64 || kd < 64 || kd > 256) return fail(SPLASH_INVALID_ARGUMENT, "n, kd must be multiples of 64 in [64, 256]");
  if (a_mode < 0 || a_mode > 4 || b_mode < 0 || b_mode > 2) return fail(SPLASH_INVALID_ARGUMENT, "bad operand mode");
  const CUtensorMapDataType dt = tmap_dtype(dtype);
  CUtensorMap tm_a, tm_b;
  int rc;
  if (a_mode == 1) rc = make_tmap_2d(&tm_a, a, dt, 2, kd, 128, kd, 64, CU_TENSOR_MAP_SWIZZLE_128B);  // a_mode 3 (wait-limit check) never loads
  else rc = make_tmap_2d(&tm_a, a, dt, 2, 128, kd, 128, 64, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  if (b_mode == 1) rc = make_tmap_2d(&tm_b, b, dt, 2, kd, n, kd, 64, CU_TENSOR_MAP_SWIZZLE_128B);
  else rc = make_tmap_2d(&tm_b, b, dt, 2, n, kd, n, 64, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  const size_t smem = 193 * 1024 + 1024;
  if ((rc = opt_in_smem(selftest_umma_kernel, smem))) return rc;
  selftest_umma_kernel<<<1, 128, smem, static_cast<cudaStream_t>(stream)>>>(
      tm_a, tm_b, a, b, d, n, kd, a_mode, b_mode, dtype == SPLASH_DTYPE_BF16, status);
  SPLASH_CUDA_CHECK(cudaGetLastError());
  return SPLASH_OK;
}
