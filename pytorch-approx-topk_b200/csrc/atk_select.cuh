// Launcher interface of the stage-2 exact select kernels.
#pragma once

#include "atk_common.cuh"

namespace atk {

struct SelectLaunch {
  const void* cand_vals;
  const long long* cand_idx;
  long long rows, k0, cand_row_stride, k;
  void* out_vals;
  long long* out_idx;
  long long out_row_stride;
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

}  // namespace atk
