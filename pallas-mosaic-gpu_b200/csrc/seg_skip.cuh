// Segment-aware block skipping.
//
// A pre-pass records the smallest and largest segment id of every 64 positions of the q
// and kv segment-id vectors.  A (q block, kv block) pair whose id ranges do not overlap
// holds no equal pair of ids, so it contributes nothing and is left out; a pair where both
// sides carry one single id, the same on both, needs no per-element comparison.  Every
// other pair is compared element by element as before.  For packed documents (ids that
// do not decrease along the sequence) the classification is exact; for arbitrary ids it
// is conservative.
//
// Before its first barrier one warp of a CTA walks the CTA's scheduled steps, classifies
// them and writes the steps that remain to a list in shared memory (16-bit entries: step
// index, top bit set when the ids are uniform); every role then iterates that list, so
// all roles agree on the steps without any of them re-deriving the decision.
#pragma once

#include "ptx.cuh"

namespace splash {

constexpr int kSegChunk = 64;  // positions per recorded (min, max) pair
enum SegKind : int { kSegSkip = 0, kSegMixed = 1, kSegUniform = 2 };
constexpr uint32_t kSegUniformBit = 0x8000u;

struct SegRange {
  int lo, hi;
};

// Range of `chunks` consecutive 64-position chunks starting at `chunk0` of one batch row.
__device__ __forceinline__ SegRange seg_range(const int2* __restrict__ table, int chunk0, int chunks) {
  int2 r = __ldg(table + chunk0);
  for (int i = 1; i < chunks; ++i) {
    const int2 x = __ldg(table + chunk0 + i);
    r.x = min(r.x, x.x);
    r.y = max(r.y, x.y);
  }
  return SegRange{r.x, r.y};
}

__device__ __forceinline__ int seg_classify(SegRange q, SegRange k) {
  if (q.hi < k.lo || k.hi < q.lo) return kSegSkip;
  if (q.lo == q.hi && k.lo == k.hi && q.lo == k.lo) return kSegUniform;
  return kSegMixed;
}

__device__ __forceinline__ void sts16(uint32_t addr, uint32_t v) {
  asm volatile("st.shared.u16 [%0], %1;" ::"r"(addr), "h"(static_cast<uint16_t>(v)) : "memory");
}
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr) : "memory");
  return v;
}

// One warp: keeps the steps i in [0, n) for which classify(i) != kSegSkip, in order.
// Returns their number (the same in every lane).
template <typename F>
__device__ __forceinline__ int build_step_list(uint32_t list_u32, int n, int lane, F classify) {
  int count = 0;
  for (int base = 0; base < n; base += 32) {
    const int i = base + lane;
    const int c = i < n ? classify(i) : static_cast<int>(kSegSkip);
    const uint32_t keep = __ballot_sync(0xffffffffu, c != kSegSkip);
    if (c != kSegSkip) {
      const int pos = count + __popc(keep & ((1u << lane) - 1u));
      sts16(list_u32 + 2u * pos, static_cast<uint32_t>(i) | (c == kSegUniform ? kSegUniformBit : 0u));
    }
    count += __popc(keep);
  }
  return count;
}

}  // namespace splash
