// Launcher interface of the contiguous-bucket stage-1 kernel.
#pragma once

#include "atk_common.cuh"

namespace atk {

struct ContigLaunch {
  const void* x;
  void* out_vals;
  long long* out_idx;
  long long rows, n, row_stride, out_row_stride;
  long long b;        // buckets per row
  int j;
  bool first_wins;    // k_b = 1 arg-max conventions (J must be 1)
  bool fixed_chunks;  // fixed ceil(n/b) chunks with tail padding instead of balanced sizes
  cudaStream_t stream;
};

int launch_contig(const ContigLaunch& a, int dtype);

}  // namespace atk
