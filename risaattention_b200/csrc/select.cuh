// Retained-mass prefix selection shared by the stand-alone selector (misc.cu) and the attention
// kernel's in-pass pattern construction (attention_tc.cu).
//
// The quantity selected is exact-order dependent: which rank closes the prefix is decided by FP64
// sums whose operation order follows the reference's selector (csrc/kernels/sparse_selection.cu:
// 19-56): the row total is a lane-strided sum finished by a shift-down tree, the running prefix
// advances in chunks of 32 ranks, each chunk scanned with an inclusive Hillis-Steele scan, and a
// rank closes the prefix when (mass before the chunk) + (scan value) >= theta * total.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace risa_b200 {

struct RetainedPrefix {
  uint32_t count;   // ranks kept (at least 1, at most n)
  double selected;  // their mass
  double total;     // mass of the whole row
};

// Whole-warp call.  `sorted` holds the row's n masses in descending order (global or shared
// memory); every lane returns the same result.
__device__ __forceinline__ RetainedPrefix retained_prefix(const float* sorted, uint32_t n,
                                                          double theta) {
  const uint32_t lane = threadIdx.x & 31u;
  double total = 0.0;
  for (uint32_t rank = lane; rank < n; rank += 32) total += static_cast<double>(sorted[rank]);
#pragma unroll
  for (uint32_t off = 16; off > 0; off >>= 1) total += __shfl_down_sync(0xffffffffu, total, off);
  total = __shfl_sync(0xffffffffu, total, 0);
  const double target = theta * total;

  RetainedPrefix result{n, total, total};
  double before = 0.0;  // mass of the chunks already passed
  for (uint32_t chunk = 0; chunk < n; chunk += 32) {
    const uint32_t rank = chunk + lane;
    double scan = rank < n ? static_cast<double>(sorted[rank]) : 0.0;
#pragma unroll
    for (uint32_t off = 1; off < 32; off <<= 1) {
      const double left = __shfl_up_sync(0xffffffffu, scan, off);
      if (lane >= off) scan += left;
    }
    const uint32_t closing = __ballot_sync(0xffffffffu, rank < n && before + scan >= target);
    if (closing != 0) {
      const uint32_t first = __ffs(closing) - 1;
      result.count = chunk + first + 1;
      result.selected = before + __shfl_sync(0xffffffffu, scan, first);
      break;
    }
    before += __shfl_sync(0xffffffffu, scan, 31);
  }
  return result;
}

// Words of the per-row selection bitmap (bit t of word t / 32 = tile t is kept).
__host__ __device__ inline uint32_t bitmap_words(uint32_t key_blocks) {
  return (key_blocks + 31u) / 32u;
}

}  // namespace risa_b200
