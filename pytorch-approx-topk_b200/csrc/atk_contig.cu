// Stage 1 for contiguous (non-interleaved) buckets.
//
// A bucket is a contiguous segment of the row.  A group of G lanes (G a power
// of two <= 32, chosen from the bucket length) strides through the segment
// with coalesced scalar loads, every lane keeping its own J-queue; the queues
// are then merged with xor-shuffles under the explicit tie rule and lane 0
// writes the bucket's J slots.  This path exists for API completeness (the
// reference's tests exercise it, its benchmarks never do) and is kept simple.
//
// Two geometries:
//  * balanced (reference CUDA operator, priority_queue_approx_topk.cu:25-56):
//    sizes n/b, the first n%b buckets one longer, laid end to end;
//  * fixed chunks of ceil(n/k) with tail padding (experimental/
//    bucketed_argmax.py:39-41), used by the k_b = 1 arg-max entry.
#include "atk_contig.cuh"

namespace atk {
namespace {

struct ContigParams {
  const void* x;
  void* out_vals;
  long long* out_idx;
  long long rows, n, row_stride, out_row_stride;
  long long b;      // buckets per row
  long long base;   // balanced: n / b;  fixed: chunk length
  long long rem;    // balanced: n % b;  fixed: unused
  int fixed;        // 1: fixed-chunk geometry
  int g;            // lanes per bucket
};

template <typename T, int J, bool FIRST>
__global__ void __launch_bounds__(256) contig_kernel(const ContigParams p) {
  using Tr = ElemTraits<T>;
  using Bits = typename Tr::Bits;
  const int G = p.g;
  const long long gid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) / G;
  const int lane = threadIdx.x % G;
  const bool valid = gid < p.rows * p.b;
  const long long row = valid ? gid / p.b : 0;
  const long long c = valid ? gid - row * p.b : 0;

  long long start, size;
  if (p.fixed) {
    start = c * p.base;
    size = p.n - start;
    if (size > p.base) size = p.base;
    if (size < 0) size = 0;
  } else {
    const long long big = c < p.rem ? c : p.rem;
    const long long normal = c > p.rem ? c - p.rem : 0;
    start = big * (p.base + 1) + normal * p.base;
    size = p.base + (c < p.rem ? 1 : 0);
  }
  if (!valid) size = 0;

  float qv[J];
  int qi[J];
#pragma unroll
  for (int q = 0; q < J; ++q) {
    qv[q] = -INFINITY;
    qi[q] = FIRST ? kSentinelFirst : kSentinelLast;
  }
  const T* seg = static_cast<const T*>(p.x) + row * p.row_stride + start;
  for (long long i = lane; i < size; i += G) {
    float v1[1];
    VecLoad<T, 1>::widen(VecLoad<T, 1>::load(seg + i), v1);
    queue_push_scan<J, FIRST>(qv, qi, v1[0], static_cast<int>(i));
  }
  // Butterfly merge inside the group; all 32 lanes of the warp take part.
  for (int off = G >> 1; off >= 1; off >>= 1) {
    float ov[J];
    int oi[J];
#pragma unroll
    for (int q = 0; q < J; ++q) {
      ov[q] = __shfl_xor_sync(0xffffffffu, qv[q], off);
      oi[q] = __shfl_xor_sync(0xffffffffu, qi[q], off);
    }
#pragma unroll
    for (int q = 0; q < J; ++q) queue_push_ranked<J, FIRST>(qv, qi, ov[q], oi[q]);
  }
  if (!valid || lane != 0) return;
  Bits* vdst = static_cast<Bits*>(p.out_vals) + row * p.out_row_stride + c * J;
  long long* idst = p.out_idx + row * p.out_row_stride + c * J;
#pragma unroll
  for (int q = 0; q < J; ++q) {
    float val = qv[q];
    long long pos = qi[q];
    if (FIRST && qi[q] == kSentinelFirst) {  // empty (all padding) bucket
      val = Tr::lowest();
      pos = 0;
    }
    vdst[q] = Tr::narrow(val);
    idst[q] = start + pos;
  }
}

template <typename T, int J, bool FIRST>
int launch_typed(const ContigLaunch& a) {
  ContigParams p;
  p.x = a.x;
  p.out_vals = a.out_vals;
  p.out_idx = a.out_idx;
  p.rows = a.rows;
  p.n = a.n;
  p.row_stride = a.row_stride;
  p.out_row_stride = a.out_row_stride;
  p.b = a.b;
  p.fixed = a.fixed_chunks ? 1 : 0;
  if (a.fixed_chunks) {
    p.base = (a.n + a.b - 1) / a.b;
    p.rem = 0;
  } else {
    p.base = a.n / a.b;
    p.rem = a.n - p.base * a.b;
  }
  if (p.base + 1 >= (1ll << 31)) return ATK_ERR_TOO_LARGE;
  int g = 1;
  while (g < 32 && static_cast<long long>(g) * 4 < p.base + 1) g *= 2;
  p.g = g;
  const long long threads = a.rows * a.b * g;
  const long long blocks = (threads + 255) / 256;
  if (blocks >= (1ll << 31)) return ATK_ERR_TOO_LARGE;
  contig_kernel<T, J, FIRST><<<static_cast<unsigned>(blocks), 256, 0, a.stream>>>(p);
  note_launch();
  return cudaGetLastError() == cudaSuccess ? ATK_OK : ATK_ERR_CUDA;
}

template <typename T>
int launch_by_j(const ContigLaunch& a) {
  if (a.first_wins) {
    if (a.j != 1) return ATK_ERR_BAD_J;
    return launch_typed<T, 1, true>(a);
  }
  switch (a.j) {
    case 1: return launch_typed<T, 1, false>(a);
    case 2: return launch_typed<T, 2, false>(a);
    case 3: return launch_typed<T, 3, false>(a);
    case 4: return launch_typed<T, 4, false>(a);
    default: return ATK_ERR_BAD_J;
  }
}

}  // namespace

int launch_contig(const ContigLaunch& a, int dtype) {
  if (a.rows <= 0 || a.b <= 0) return ATK_OK;
  switch (dtype) {
    case ATK_F32: return launch_by_j<float>(a);
    case ATK_F16: return launch_by_j<__half>(a);
    case ATK_BF16: return launch_by_j<__nv_bfloat16>(a);
    default: return ATK_ERR_BAD_DTYPE;
  }
}

}  // namespace atk
