// extern "C" entry points of libsplash_sm100.so: argument validation, dispatch to
// the compiled kernel configuration, status helpers.
#include <cstdlib>

#include "dispatch.h"
#include "host_common.cuh"

namespace splash {

constexpr int kBwdStagesMax = 4;

static int check_common(const SplashParams* p, bool backward) {
  if (!p) return fail(SPLASH_INVALID_ARGUMENT, "params is null");
  if (!p->q || !p->k || !p->v || !p->status) return fail(SPLASH_INVALID_ARGUMENT, "q, k, v and status must be non-null");
  if (!p->num_steps || !p->block_order || !p->block_list || !p->block_kind)
    return fail(SPLASH_INVALID_ARGUMENT, "schedule arrays must be non-null");
  if (p->batch <= 0 || p->heads <= 0 || p->kv_heads <= 0 || p->q_len <= 0 || p->kv_len <= 0)
    return fail(SPLASH_INVALID_ARGUMENT, "sizes must be positive");
  if (p->heads % p->kv_heads) return fail(SPLASH_INVALID_ARGUMENT, "heads not a multiple of kv_heads");
  if (p->dtype != SPLASH_DTYPE_BF16 && p->dtype != SPLASH_DTYPE_F16) return fail(SPLASH_UNSUPPORTED, "Only bf16/f16 are supported");
  if (p->head_dim % 64 || p->head_dim_v % 64 || p->head_dim > 256 || p->head_dim_v > 256 || p->head_dim <= 0 ||
      p->head_dim_v <= 0)
    return fail(SPLASH_UNSUPPORTED, "head dims must be multiples of 64 and <= 256");
  if (p->mask_heads != 1 && p->mask_heads != p->heads) return fail(SPLASH_INVALID_ARGUMENT, "mask_heads must be 1 or heads");
  if (p->max_steps < 1) return fail(SPLASH_INVALID_ARGUMENT, "max_steps must be >= 1");
  if ((p->seg_q == nullptr) != (p->seg_kv == nullptr)) return fail(SPLASH_INVALID_ARGUMENT, "seg_q and seg_kv go together");
  if (p->partial_blocks && (!p->mask_block || p->num_partial_blocks <= 0))
    return fail(SPLASH_INVALID_ARGUMENT, "dense partial blocks need mask_block ids");
  if (p->partial_blocks && p->mask_desc) return fail(SPLASH_INVALID_ARGUMENT, "give dense partial blocks or a band descriptor, not both");
  if (static_cast<int64_t>(p->batch) * p->heads * p->q_len >= (1ll << 31) ||
      static_cast<int64_t>(p->batch) * p->kv_heads * p->kv_len >= (1ll << 31))
    return fail(SPLASH_INVALID_ARGUMENT, "batch * heads * length must fit in 31 bits");
  if (backward && (!p->d_out || !p->lse || !p->delta)) return fail(SPLASH_INVALID_ARGUMENT, "backward needs d_out, lse and delta");
  return SPLASH_OK;
}

static int check_fwd(const SplashParams* p, int tiles) {
  if (int rc = check_common(p, false)) return rc;
  if (!p->out) return fail(SPLASH_INVALID_ARGUMENT, "out is null");
  if (p->block_q != 128 * tiles) return fail(SPLASH_INVALID_ARGUMENT, "block_q does not match this entry point");
  if (p->block_kv != 64 && p->block_kv != 128) return fail(SPLASH_INVALID_ARGUMENT, "block_kv must be 64 or 128");
  if (p->num_stages < 2 || p->num_stages > 8) return fail(SPLASH_INVALID_ARGUMENT, "num_stages must be in [2, 8]");
  if (p->q_len % p->block_q || p->kv_len % p->block_kv)
    return fail(SPLASH_INVALID_ARGUMENT, "Sequence lengths must be multiples of the block sizes");
  return SPLASH_OK;
}

#define SPLASH_FWD_CASE(D_, DV_, NT_)                                                               \
  if (p->head_dim == D_ && p->head_dim_v == DV_) {                                                  \
    return p->block_kv == 64 ? launch_fwd<D_, DV_, 64, NT_>(*p, st) : launch_fwd<D_, DV_, 128, NT_>(*p, st); \
  }

}  // namespace splash

using namespace splash;

extern "C" int64_t splash_seg_ranges_bytes(const SplashParams* p) {
  if (!p || !p->seg_q || p->q_len % 64 || p->kv_len % 64) return 0;
  return static_cast<int64_t>(p->batch) * (p->q_len / 64 + p->kv_len / 64) * 8;
}

extern "C" int splash_fwd128(const SplashParams* p, void* stream) {
  if (int rc = check_fwd(p, 1)) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (int rc = launch_seg_ranges(*p, st)) return rc;
  SPLASH_FWD_CASE(64, 64, 1)
  SPLASH_FWD_CASE(64, 128, 1)
  SPLASH_FWD_CASE(128, 128, 1)
  SPLASH_FWD_CASE(128, 64, 1)
  SPLASH_FWD_CASE(192, 192, 1)
  SPLASH_FWD_CASE(256, 256, 1)
  return fail(SPLASH_UNSUPPORTED, "this (head_dim, head_dim_v) pair is not compiled for the 128-row forward");
}

extern "C" int splash_fwd256(const SplashParams* p, void* stream) {
  if (int rc = check_fwd(p, 2)) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (int rc = launch_seg_ranges(*p, st)) return rc;
  if (p->head_dim != p->head_dim_v) return fail(SPLASH_UNSUPPORTED, "ping-pong kernel needs head_dim == head_dim_v");
  SPLASH_FWD_CASE(64, 64, 2)
  SPLASH_FWD_CASE(128, 128, 2)
  return fail(SPLASH_UNSUPPORTED, "ping-pong kernel supports head_dim 64/128");
}

static int check_bwd(const SplashParams* p) {
  if (int rc = check_common(p, true)) return rc;
  if (p->block_q != 128 || p->block_kv != 128) return fail(SPLASH_INVALID_ARGUMENT, "the backward schedule is 128x128");
  if (p->num_stages < 1 || p->num_stages > kBwdStagesMax) return fail(SPLASH_INVALID_ARGUMENT, "num_stages_bwd must be in [1, 4]");
  if (p->q_len % 128 || p->kv_len % 128) return fail(SPLASH_INVALID_ARGUMENT, "Sequence lengths must be multiples of 128");
  if (p->sub_block != 0 && p->sub_block != 64 && p->sub_block != 128)
    return fail(SPLASH_INVALID_ARGUMENT, "sub_block must be 0, 64 or 128");
  if ((p->head_dim != 64 && p->head_dim != 128) || (p->head_dim_v != 64 && p->head_dim_v != 128))
    return fail(SPLASH_UNSUPPORTED, "the backward pass supports head dims 64 and 128");
  return SPLASH_OK;
}

static int check_bwd_fused(const SplashParams* p) {
  if (int rc = check_bwd(p)) return rc;
  if (p->head_dim != p->head_dim_v) return fail(SPLASH_UNSUPPORTED, "the fused backward needs head_dim == head_dim_v");
  return SPLASH_OK;
}

extern "C" int splash_bwd_delta(const void* o, const void* d_out, float* delta, int64_t rows, int32_t head_dim_v,
                                int32_t dtype, void* stream) {
  return launch_delta(o, d_out, delta, rows, head_dim_v, dtype, static_cast<cudaStream_t>(stream));
}

extern "C" int splash_bwd_dq(const SplashParams* p, void* stream) {
  if (int rc = check_bwd(p)) return rc;
  if (!p->dq) return fail(SPLASH_INVALID_ARGUMENT, "dq is null");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (int rc = launch_seg_ranges(*p, st)) return rc;
  // The requested sub-block is a preference: 128 keys per step when it fits in shared
  // memory, else 64.
  const bool want128 = p->sub_block != 64;
#define SPLASH_DQ_CASE(D_, DV_)                                                                                  \
  if (p->head_dim == D_ && p->head_dim_v == DV_) {                                                               \
    if (want128 && bwd_row_smem<D_, DV_, 128>(*p) <= kMaxDynamicSmem) return launch_bwd_row<D_, DV_, 128>(*p, st); \
    return launch_bwd_row<D_, DV_, 64>(*p, st);                                                                  \
  }
  SPLASH_DQ_CASE(64, 64)
  SPLASH_DQ_CASE(128, 128)
  SPLASH_DQ_CASE(128, 64)
  SPLASH_DQ_CASE(64, 128)
#undef SPLASH_DQ_CASE
  return fail(SPLASH_UNSUPPORTED, "this (head_dim, head_dim_v) pair is not compiled for the dQ kernel");
}

extern "C" int splash_bwd_dkv(const SplashParams* p, void* stream) {
  if (int rc = check_bwd(p)) return rc;
  if (!p->dk || !p->dv) return fail(SPLASH_INVALID_ARGUMENT, "dk / dv is null");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (int rc = launch_seg_ranges(*p, st)) return rc;
  // The kernel works in steps of 64 q rows with double-buffered scores; `sub_block`
  // is accepted for compatibility and does not change the tiling.
  if (p->head_dim == 64) return p->head_dim_v == 64 ? launch_bwd_col<64, 64, false>(*p, st) : launch_bwd_col<64, 128, false>(*p, st);
  return p->head_dim_v == 128 ? launch_bwd_col<128, 128, false>(*p, st) : launch_bwd_col<128, 64, false>(*p, st);
}

// The f32 dQ accumulator alone.
static int64_t dq_acc_bytes(const SplashParams* p) {
  return static_cast<int64_t>(p->batch) * p->heads * p->q_len * p->head_dim * 4;
}

extern "C" int64_t splash_bwd_fused_workspace_bytes(const SplashParams* p) {
  if (!p) return 0;
  // Accumulator; at head_dim 64 also 32 bytes per q row for the folded lse / delta operands.
  return dq_acc_bytes(p) + fold_operand_bytes(*p);
}

extern "C" int splash_bwd_fused(const SplashParams* p, void* stream) {
  if (int rc = check_bwd_fused(p)) return rc;
  if (!p->dq || !p->dk || !p->dv || !p->dq_acc) return fail(SPLASH_INVALID_ARGUMENT, "dq, dk, dv and dq_acc must be non-null");

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (int rc = launch_seg_ranges(*p, st)) return rc;
  if (p->out) {
    // One pass streams O and dO for delta and clears the accumulator on the way.
    if (int rc = launch_delta(p->out, p->d_out, p->delta, static_cast<long long>(p->batch) * p->heads * p->q_len,
                              p->head_dim_v, p->dtype, st, p->dq_acc, p->head_dim))
      return rc;
  } else {
    SPLASH_CUDA_CHECK(cudaMemsetAsync(p->dq_acc, 0, static_cast<size_t>(dq_acc_bytes(p)), st));
  }
  // Head dim 128 takes the kernel that works on whole 128-row q blocks; streamed mask blocks
  // and head dim 64 take the 64-row one.  SPLASH_BWD_WIDE=0 forces the latter (experiments).
  const char* wide_env = getenv("SPLASH_BWD_WIDE");
  const bool wide_off = wide_env && wide_env[0] == '0';
  int rc;
  if (!wide_off && bwd_wide_supported(*p)) rc = launch_bwd_wide(*p, st);
  else rc = p->head_dim == 64 ? launch_bwd_col<64, 64, true>(*p, st) : launch_bwd_col<128, 128, true>(*p, st);
  if (rc) return rc;
  return launch_dq_transpose_cast(p->dq_acc, p->dq, static_cast<long long>(p->batch) * p->heads, p->head_dim, p->q_len,
                                  p->dtype, st);
}

// ---------------------------------------------------------------------------
// Fused backward for callers that cannot allocate
// ---------------------------------------------------------------------------
// The f32 dQ accumulator lives in a fixed array inside the library image instead of
// caller-provided scratch.  In host code `g_static_dq_acc` is only a handle for the
// symbol, not a device address; the address a kernel can use comes from
// cudaGetSymbolAddress, looked up once per device with that device current.
constexpr size_t kStaticDqAccBytes = SPLASH_STATIC_DQ_ACC_BYTES;
static __device__ __align__(256) float g_static_dq_acc[kStaticDqAccBytes / sizeof(float)];

static int static_dq_acc_address(float** out) {
  constexpr int kMaxDevices = 64;
  static float* cache[kMaxDevices] = {};
  int dev = -1;
  SPLASH_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(SPLASH_INVALID_ARGUMENT, "device ordinal out of range");
  float* ptr = __atomic_load_n(&cache[dev], __ATOMIC_ACQUIRE);
  if (!ptr) {
    void* sym = nullptr;
    SPLASH_CUDA_CHECK(cudaGetSymbolAddress(&sym, g_static_dq_acc));
    if (!sym) return fail(SPLASH_CUDA_ERROR, "cudaGetSymbolAddress returned a null address");
    ptr = static_cast<float*>(sym);
    __atomic_store_n(&cache[dev], ptr, __ATOMIC_RELEASE);
  }
  *out = ptr;
  return SPLASH_OK;
}

extern "C" int splash_bwd_fused_static(const SplashParams* p, void* stream) {
  if (int rc = check_bwd_fused(p)) return rc;
  SplashParams q = *p;
  const int64_t need = splash_bwd_fused_workspace_bytes(&q);
  if (need <= 0 || static_cast<uint64_t>(need) > kStaticDqAccBytes) {
    char d[160];
    snprintf(d, sizeof d, "the scratch for these shapes is %lld bytes, the built-in one holds %zu",
             static_cast<long long>(need), kStaticDqAccBytes);
    return fail(SPLASH_BUDGET_EXCEEDED, "problem too large for splash_bwd_fused_static", d);
  }
  float* acc = nullptr;
  if (int rc = static_dq_acc_address(&acc)) return rc;
  q.dq_acc = acc;  // whatever the caller put there is ignored
  return splash_bwd_fused(&q, stream);
}

extern "C" int splash_read_status(const int32_t* status, int32_t* host_out, void* stream) {
  int32_t h[4] = {0, 0, 0, 0};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  SPLASH_CUDA_CHECK(cudaMemcpyAsync(h, status, sizeof h, cudaMemcpyDeviceToHost, st));
  SPLASH_CUDA_CHECK(cudaStreamSynchronize(st));
  if (host_out) memcpy(host_out, h, sizeof h);
  if (h[0] != 0) {
    char d[128];
    snprintf(d, sizeof d, "code %d at wait site %d, block %d, step %d", h[0], h[1], h[2], h[3]);
    return fail(SPLASH_DEVICE_TIMEOUT, "a kernel gave up waiting", d);
  }
  return SPLASH_OK;
}

extern "C" const char* splash_status_string(int status) {
  switch (status) {
    case SPLASH_OK: return "ok";
    case SPLASH_INVALID_ARGUMENT: return "invalid argument";
    case SPLASH_UNSUPPORTED: return "unsupported configuration";
    case SPLASH_BUDGET_EXCEEDED: return "shared/tensor memory budget exceeded";
    case SPLASH_CUDA_ERROR: return "CUDA error";
    case SPLASH_DEVICE_TIMEOUT: return "device-side wait timed out";
    default: return "unknown status";
  }
}

extern "C" const char* splash_last_error(void) { return last_error_buf(); }
