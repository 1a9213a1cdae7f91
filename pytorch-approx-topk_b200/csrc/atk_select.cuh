// Launcher interface of the stage-2 exact select kernels.
#pragma once

#include "atk_common.cuh"

namespace atk {

struct SelectLaunch {
  const void* cand_vals;
  const long long* cand_idx;
  long long rows, k0, cand_row_stride, k;
  void* out_vals;
  void* out_idx;             // int64 or int32 positions by out_format (unused for records)
  long long out_row_stride;
  int out_format = ATK_OUT_I64;
  void* workspace;
  size_t workspace_bytes;
  cudaStream_t stream;
};

size_t select_workspace_bytes(int dtype, long long rows, long long k0);
int launch_select(const SelectLaunch& a, int dtype);

// launch_select with the library's built-in static device scratch in place of
// a.workspace (which is ignored).  Returns ATK_ERR_SCRATCH_LIMIT, launching
// nothing, when the problem needs more than that array holds.
int launch_select_static(const SelectLaunch& a, int dtype);

// The select of the two-stage operator when stage 1 handed over its packed queue
// entries (image of the value << shift | stripe; slot s belongs to bucket s / j)
// instead of values and positions: values and positions are rebuilt only for the
// k winners.  `x` is the operator's input (read back for the sign of a zero).
struct SelectPackedLaunch {
  const uint32_t* keys;       // rows x k0, dense
  long long rows, k0, k;
  const void* x;
  long long x_row_stride;     // elements
  long long b;                // buckets per row: position = stripe * b + bucket
  int j;
  void* out_vals;
  void* out_idx;
  long long out_row_stride;
  int out_format = ATK_OUT_I64;
  cudaStream_t stream;
};
// Longest row this select takes (one block per row); longer rows use the plain hand-off.
long long select_packed_max_k0();
int launch_select_packed(const SelectPackedLaunch& a, int dtype);

}  // namespace atk
