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

// The same choice, made by every warp that calls it (all 32 lanes), with the
// result returned in registers of every lane: no shared-memory hand-off and no
// block barrier after it.  `hist` must be 16-byte aligned.
__device__ __forceinline__ void pick_digit_all(const uint32_t* hist, uint32_t need, int lane, uint32_t& digit,
                                               uint32_t& new_need) {
  // lane l takes bins 255-8l .. 248-8l, i.e. words [248-8l, 256-8l) of the histogram
  const uint4 lo = *reinterpret_cast<const uint4*>(hist + 248 - 8 * lane);
  const uint4 hi = *reinterpret_cast<const uint4*>(hist + 252 - 8 * lane);
  const uint32_t h[8] = {hi.w, hi.z, hi.y, hi.x, lo.w, lo.z, lo.y, lo.x};   // descending bins
  uint32_t total = 0;
#pragma unroll
  for (int t = 0; t < 8; ++t) total += h[t];
  uint32_t incl = total;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const uint32_t nb = __shfl_up_sync(0xffffffffu, incl, off);
    if (lane >= off) incl += nb;
  }
  uint32_t running = incl - total;
  // exactly one lane holds the bin in which the running count crosses `need`
  const bool mine = running < need && incl >= need;
  uint32_t d = 0, nn = 0;
#pragma unroll
  for (int t = 0; t < 8; ++t) {
    if (running < need && running + h[t] >= need) {
      d = 255 - 8 * lane - t;
      nn = need - running;
    }
    running += h[t];
  }
  const int src = __ffs(__ballot_sync(0xffffffffu, mine)) - 1;
  digit = __shfl_sync(0xffffffffu, d, src);
  new_need = __shfl_sync(0xffffffffu, nn, src);
}

}  // namespace atk
