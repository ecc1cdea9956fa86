/* C ABI of libsplash_sm100.so: block-sparse flash attention ("splash attention")
 * forward and backward for NVIDIA B200 (sm_100a).
 *
 * Each entry point stands in for one device-kernel call site of the reference
 * project kuym/Pallas-Mosaic-GPU, whose boundary is a `plgpu.kernel(...)(*inputs)`
 * call that JAX turns into an XLA GPU custom call.  The operand lists below keep
 * the reference's operand order; the Python mask callable of the reference is
 * replaced by a small per-head band descriptor (see `mask_desc`).
 *
 * Conventions
 *   - Plain pointers and sizes only; every buffer is owned by the caller and lives
 *     in device memory unless stated otherwise.  Except where an entry point says
 *     so, the library allocates no device memory and keeps no state besides what it
 *     remembers per device: the shared-memory limit already granted to each kernel
 *     and (splash_bwd_fused_static) the address of its built-in scratch.
 *   - Calls enqueue work on `stream` (a cudaStream_t passed as void*) and return
 *     without synchronising.
 *   - Return value: SPLASH_OK or a negative SplashStatus.  Nothing is thrown
 *     across the ABI and nothing aborts.
 *   - `status` points at 4 int32 in device memory, zeroed by the caller.  A kernel
 *     whose bounded waits run out writes {code, site, block, step} there and
 *     unwinds instead of spinning; once the word is non-zero later CTAs (and later
 *     launches given the same word) return at once.
 */
#ifndef SPLASH_SM100_H_
#define SPLASH_SM100_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum SplashStatus {
  SPLASH_OK = 0,
  SPLASH_INVALID_ARGUMENT = -1, /* shapes, divisibility, null pointers */
  SPLASH_UNSUPPORTED = -2,      /* dtype / head_dim / tile combination not built */
  SPLASH_BUDGET_EXCEEDED = -3,  /* shared or tensor memory budget */
  SPLASH_CUDA_ERROR = -4,       /* a CUDA runtime/driver call failed */
  SPLASH_DEVICE_TIMEOUT = -5    /* reported by splash_read_status only */
} SplashStatus;

enum { SPLASH_DTYPE_BF16 = 0, SPLASH_DTYPE_F16 = 1 };
enum { SPLASH_BLOCK_EMPTY = 0, SPLASH_BLOCK_PARTIAL = 1, SPLASH_BLOCK_FULL = 2 };

typedef struct SplashParams {
  /* ---- operands, in the reference's order -------------------------------- */
  const void* q;           /* [batch, heads, q_len, head_dim]          bf16/f16 */
  const void* k;           /* [batch, kv_heads, kv_len, head_dim]               */
  const void* v;           /* [batch, kv_heads, kv_len, head_dim_v]             */
  const void* d_out;       /* backward: [batch, heads, q_len, head_dim_v]       */
  const float* lse;        /* backward: [batch, heads, q_len], natural log      */
  float* delta;            /* backward: [batch, heads, q_len] = sum(dO * O); written
                            * by splash_bwd_fused when `out` is set, read otherwise */
  const int32_t* seg_q;    /* [batch, q_len] or NULL                            */
  const int32_t* seg_kv;   /* [batch, kv_len] or NULL                           */
  /* Sparse schedule.  Forward and dQ use the per-q-block ("row") lists; dK/dV
   * and the fused backward use the per-kv-block ("column") lists.  All int32. */
  const int32_t* num_steps;   /* [mask_heads, blocks]                           */
  const int32_t* block_order; /* [mask_heads, blocks], heaviest first           */
  const int32_t* block_list;  /* [mask_heads, blocks, max_steps] visited blocks */
  const int32_t* block_kind;  /* [mask_heads, blocks, max_steps] PARTIAL/FULL   */
  const int32_t* mask_block;  /* [mask_heads, blocks, max_steps] or NULL        */
  /* Dense partial blocks, one bit per element (1 = attend), bit i of byte j standing for
   * column 8 * j + i: [n, block_q, block_kv / 8] bytes for the row kernels,
   * [n, block_kv, block_q / 8] (transposed) for the column kernels; 16-byte aligned.
   * NULL when partial blocks are computed from `mask_desc`.  (The reference streams
   * int8 blocks, splash_attention_mgpu/mask_info.py:113-120.) */
  const int8_t* partial_blocks;
  /* [mask_heads, 4] int32 {lo, hi, chunk, 0}: a key is visible iff
   * lo <= kv_pos - q_pos <= hi and (chunk == 0 or q_pos/chunk == kv_pos/chunk).
   * NULL when partial blocks are dense or when there are no partial blocks. */
  const int32_t* mask_desc;
  /* ---- results ------------------------------------------------------------ */
  void* out;        /* forward: [batch, heads, q_len, head_dim_v]               */
  float* lse_out;   /* forward: [batch, heads, q_len] or NULL                   */
  void* dq;         /* backward: like q                                         */
  void* dk;         /* backward: like k                                         */
  void* dv;         /* backward: like v                                         */
  float* dq_acc;    /* fused backward scratch: f32, transposed -- [batch, heads, head_dim, q_len],
                     * i.e. [batch * heads * head_dim, q_len] row-major; size from
                     * splash_bwd_fused_workspace_bytes()                         */
  int32_t* status;  /* 4 x int32, see above                                     */
  /* ---- static configuration ---------------------------------------------- */
  int32_t batch, heads, kv_heads, q_len, kv_len, head_dim, head_dim_v;
  int32_t dtype;              /* SPLASH_DTYPE_*                                  */
  int32_t mask_heads;         /* 1 (shared schedule) or heads                    */
  int32_t max_steps;          /* last dimension of block_list                    */
  int32_t num_partial_blocks; /* first dimension of partial_blocks               */
  int32_t block_q, block_kv;  /* schedule granularity                            */
  int32_t num_stages;         /* shared-memory ring depth                        */
  int32_t sub_block;          /* backward contraction sub-block (64/128), 0=auto */
  float mask_value;           /* lse reported for rows that see no key           */
  float soft_cap;             /* logits -> cap * tanh(logits / cap); 0 = off     */
  /* ---- optional scratch (appended; zero/NULL keeps the behaviour without it) ---- */
  /* Segment-aware block skipping.  With segment ids, int32 scratch of
   * splash_seg_ranges_bytes() bytes: every entry point that is given it first fills it with
   * the smallest and largest segment id of every 64 positions of seg_q and seg_kv, and its
   * CTAs then leave out scheduled blocks whose q and kv id ranges cannot meet, and skip the
   * per-element comparison in blocks where both sides carry one and the same id.  The
   * reference computes every scheduled block and masks by comparison
   * (splash_attention_mgpu/kernel.py:392-395); results are the same.  NULL: as the reference. */
  int32_t* seg_ranges;
} SplashParams;

/* Bytes of `seg_ranges` scratch for these shapes (0 when there are no segment ids).  No
 * counterpart in the reference, which computes every scheduled block and masks by
 * comparing ids (splash_attention_mgpu/kernel.py:392-395). */
int64_t splash_seg_ranges_bytes(const SplashParams* p);

/* Forward, one 128-row q tile per CTA.  Replaces the custom call made by
 * `_splash_attention_forward` (reference splash_attention_mgpu/kernel.py:521-537). */
int splash_fwd128(const SplashParams* p, void* stream);

/* Forward, two 128-row q tiles per CTA sharing every K/V block ("ping-pong").
 * Replaces `splash_attention_forward_pingpong`
 * (reference splash_attention_mgpu/forward_pingpong.py:667-681). */
int splash_fwd256(const SplashParams* p, void* stream);

/* delta = rowsum(dO * O) in f32, the reduction the reference leaves to XLA
 * (reference splash_attention_mgpu/splash_attention.py:289-290).
 * `o` and `d_out` are [rows, head_dim_v] of `dtype`; `delta` is [rows] f32. */
int splash_bwd_delta(const void* o, const void* d_out, float* delta, int64_t rows, int32_t head_dim_v,
                     int32_t dtype, void* stream);

/* dQ over the row schedule.  Replaces `splash_attention_bwd_dq`
 * (reference splash_attention_mgpu/backward.py:368-374). */
int splash_bwd_dq(const SplashParams* p, void* stream);

/* dK and dV over the column schedule, looping the q heads of a KV head inside the
 * CTA.  Replaces `splash_attention_bwd_dkv`
 * (reference splash_attention_mgpu/backward.py:777-785). */
int splash_bwd_dkv(const SplashParams* p, void* stream);

/* Fused backward (dQ, dK, dV in one kernel; dQ reduce-added into `dq_acc`, which
 * this call zeroes first and converts into `dq` afterwards).  head_dim == head_dim_v
 * in {64, 128}; other pairs of 64/128 go through splash_bwd_dq + splash_bwd_dkv.  Replaces
 * `splash_attention_bwd_fused` together with its accumulator zero-fill and
 * transpose/cast passes (reference splash_attention_mgpu/backward_fused.py:492-511).
 * With `out` null, `delta` must already hold rowsum(dO * O) (splash_bwd_delta); with
 * `out` set to the forward output, this call fills `delta` itself in the pass that
 * clears the accumulator (what the reference leaves to XLA,
 * splash_attention_mgpu/splash_attention.py:289-290). */
int splash_bwd_fused(const SplashParams* p, void* stream);

/* Bytes of `dq_acc` scratch splash_bwd_fused needs for these shapes: the f32 accumulator
 * batch * heads * q_len * head_dim * 4, and at head_dim 64 another 32 bytes per q row behind it
 * (lse and delta split into 16-bit parts, operands of the 128-row kernel). */
int64_t splash_bwd_fused_workspace_bytes(const SplashParams* p);

/* Size of the scratch built into the library for splash_bwd_fused_static. */
#define SPLASH_STATIC_DQ_ACC_BYTES (16u << 20)

/* splash_bwd_fused without caller scratch and without any allocation.  (No counterpart
 * in the reference: there the f32 dQ accumulator is an ordinary XLA buffer.)
 *
 * Who needs it: code that runs where device allocation is off limits -- the execute
 * callback of another runtime (an XLA custom call, an inference-server plugin's
 * enqueue hook), or a process whose memory pool is sealed after start-up.  Calling
 * cudaMalloc there can stall the whole device, bypasses the host runtime's memory
 * accounting, or is simply forbidden, and such callers often have no spare workspace
 * to hand over either.
 *
 * The dQ accumulator is a fixed SPLASH_STATIC_DQ_ACC_BYTES (16 MiB) array inside the
 * library image; every GPU that loads the library carries it until the process exits.
 * `p->dq_acc` is ignored; all other fields are as for splash_bwd_fused.  Shapes whose
 * splash_bwd_fused_workspace_bytes() exceeds SPLASH_STATIC_DQ_ACC_BYTES are refused with
 * SPLASH_BUDGET_EXCEEDED.  The call performs no cudaMalloc / cudaFree and no allocating
 * library call.  The first call on each device looks up the array's device address
 * (cudaGetSymbolAddress); make that first call outside any stream capture.  The address
 * is remembered per device ordinal for the life of the process and does not survive
 * cudaDeviceReset or the destruction of the device's primary context: a process that
 * does either must not call this entry point on that device again.
 *
 * All calls share the one array: it is cleared at the start of each call, and two calls
 * whose GPU work overlaps (different streams, no ordering between them) race on it --
 * serialise them. */
int splash_bwd_fused_static(const SplashParams* p, void* stream);

/* Copies the 4-int status word to the host after synchronising `stream`; returns
 * SPLASH_OK, SPLASH_DEVICE_TIMEOUT or SPLASH_CUDA_ERROR. `host_out` may be NULL. */
int splash_read_status(const int32_t* status, int32_t* host_out, void* stream);

/* Human-readable text for a SplashStatus value (static storage). */
const char* splash_status_string(int status);

/* Text describing the last failing CUDA call on this thread (static storage). */
const char* splash_last_error(void);

/* Single-tile tcgen05 GEMM used to validate operand descriptors on the device:
 * D[128, n] (f32) = A[128, kd] * B[n, kd]^T for bf16/f16 inputs.
 *   a_mode: 0 = A in shared memory, K-major (global A is [128, kd] row-major)
 *           1 = A in shared memory, M-major (global A is [kd, 128] row-major)
 *           2 = A staged through tensor memory (global A is [128, kd] row-major)
 *           3 = no GEMM: the kernel waits on a barrier nothing arrives on, so that its
 *               bounded wait runs out (about a second); it then unwinds and leaves
 *               {1, 102, 0, 7} in `status`.  Checks the report path without a fault.
 *           4 = A in shared memory, K-major, unswizzled 8 x 8 core matrices written by
 *               the kernel's own threads (global A is [128, kd] row-major)
 *   b_mode: 0 = K-major (global B is [n, kd] row-major)
 *           1 = N-major (global B is [kd, n] row-major)
 *           2 = K-major, unswizzled core matrices (global B is [n, kd] row-major)
 * No counterpart in the reference; it exists for the test-suite. */
int splash_selftest_umma(const void* a, const void* b, float* d, int32_t n, int32_t kd, int32_t a_mode,
                         int32_t b_mode, int32_t dtype, int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SPLASH_SM100_H_ */
