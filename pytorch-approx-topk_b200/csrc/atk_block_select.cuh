// Warp-level piece of the exact select (stage 2) shared by its kernels.
//
// Keys are order-preserving 32-bit images of the candidate values.
#pragma once

#include "atk_common.cuh"

namespace atk {

// One warp: given a 256-bin histogram of the digit under inspection (only keys
// that match the prefix found so far are counted) pick the bin that contains
// the need-th largest key.  Bins are walked from 255 downwards.
// `lane` is the caller's lane id within its warp (blocks may be 2-D, so it is
// not derived from threadIdx.x here).
__device__ __forceinline__ void pick_digit(const uint32_t* hist, uint32_t need, int lane, uint32_t* out_digit,
                                           uint32_t* out_need) {
  uint32_t h[8];
  uint32_t total = 0;
#pragma unroll
  for (int t = 0; t < 8; ++t) {
    h[t] = hist[255 - 8 * lane - t];
    total += h[t];
  }
  uint32_t incl = total;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const uint32_t nb = __shfl_up_sync(0xffffffffu, incl, off);
    if (lane >= off) incl += nb;
  }
  uint32_t running = incl - total;
#pragma unroll
  for (int t = 0; t < 8; ++t) {
    if (running < need && running + h[t] >= need) {
      *out_digit = 255 - 8 * lane - t;
      *out_need = need - running;
    }
    running += h[t];
  }
}

}  // namespace atk
