// Warp- and block-level pieces of the exact select (stage 2).
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

// Exclusive block scan of two boolean flags.  Returns this thread's ranks and
// the block totals.  wsum: >= 32 words of shared memory; contains one
// __syncthreads pair, so all threads of the block must call it.  `tid` is the
// linear thread index, `nthreads` the block size (a multiple of 32, <= 1024).
__device__ __forceinline__ void block_rank2(bool f0, bool f1, uint32_t* wsum, int tid, int nthreads,
                                            uint32_t& r0, uint32_t& r1, uint32_t& t0, uint32_t& t1) {
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int nwarps = (nthreads + 31) >> 5;
  const uint32_t m0 = __ballot_sync(0xffffffffu, f0);
  const uint32_t m1 = __ballot_sync(0xffffffffu, f1);
  const uint32_t lt = (1u << lane) - 1u;
  if (lane == 0) wsum[warp] = __popc(m0) | (__popc(m1) << 16);
  __syncthreads();
  uint32_t before = 0, all = 0;
  for (int w = 0; w < nwarps; ++w) {
    const uint32_t s = wsum[w];
    if (w < warp) before += s;
    all += s;
  }
  __syncthreads();
  r0 = (before & 0xffffu) + __popc(m0 & lt);
  r1 = (before >> 16) + __popc(m1 & lt);
  t0 = all & 0xffffu;
  t1 = all >> 16;
}

// Histogram update for a whole (converged) warp: lanes holding the same digit
// elect one of them to add their count, so keys that concentrate on a few
// digits (16-bit floats do) cost one shared-memory atomic per distinct digit
// instead of one per key.
__device__ __forceinline__ void hist_add_warp(uint32_t* hist, uint32_t digit, bool valid, int lane) {
  const uint32_t active = __ballot_sync(0xffffffffu, valid);
  if (!valid) return;
  const uint32_t peers = __match_any_sync(active, digit);
  if (lane == __ffs(peers) - 1) atomicAdd(&hist[digit], static_cast<uint32_t>(__popc(peers)));
}

}  // namespace atk
