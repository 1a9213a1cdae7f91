// Stage 1 for contiguous (non-interleaved) buckets.
//
// A bucket is a contiguous segment of the row.  A group of G lanes (G a power
// of two <= 32, chosen from the bucket length) strides through the segment
// with coalesced (vector where aligned) loads, every lane keeping its own J-queue; the queues
// are then merged with xor-shuffles under the explicit tie rule and lane 0
// writes the bucket's J slots (contig_kernel, used for long buckets).  Short
// buckets go through contig_tile_kernel, which stages a span of 128 buckets in
// shared memory and scans one bucket per thread.  This mode exists for API
// completeness (the reference's tests exercise it, its benchmarks never do).
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

// Scan elements [0, size) of a segment with `nl` cooperating lanes (this is
// lane `l`): scalar head up to the first 16-byte boundary, 16-byte vector body,
// scalar tail.  Each lane sees its elements in increasing position order, so
// the serial insertion rule applies; positions are offsets inside the segment.
template <typename T, int J, bool FIRST>
__device__ __forceinline__ void contig_scan_segment(const T* seg, long long size, int l, int nl,
                                                    typename ElemTraits<T>::Compute (&qv)[J], int (&qi)[J]) {
  using C = typename ElemTraits<T>::Compute;
  constexpr int V = ElemTraits<T>::kVec;
  constexpr int kVecBytes = V * static_cast<int>(sizeof(T));
  const uintptr_t addr0 = reinterpret_cast<uintptr_t>(seg);
  long long head = static_cast<long long>(((kVecBytes - (addr0 & (kVecBytes - 1))) & (kVecBytes - 1)) / sizeof(T));
  if (head > size) head = size;
  const long long body = (size - head) / V;
  for (long long i = l; i < head; i += nl) {
    C f[1];
    VecLoad<T, 1>::widen(VecLoad<T, 1>::load(seg + i), f);
    queue_push_scan<J, FIRST>(qv, qi, f[0], static_cast<int>(i));
  }
  long long v = l;
  for (; v + nl < body; v += 2 * nl) {     // two independent vector loads in flight
    C f0[V], f1[V];
    const typename VecLoad<T, V>::Raw r0 = VecLoad<T, V>::load(seg + head + v * V);
    const typename VecLoad<T, V>::Raw r1 = VecLoad<T, V>::load(seg + head + (v + nl) * V);
    VecLoad<T, V>::widen(r0, f0);
    VecLoad<T, V>::widen(r1, f1);
#pragma unroll
    for (int e = 0; e < V; ++e) queue_push_scan<J, FIRST>(qv, qi, f0[e], static_cast<int>(head + v * V + e));
#pragma unroll
    for (int e = 0; e < V; ++e) queue_push_scan<J, FIRST>(qv, qi, f1[e], static_cast<int>(head + (v + nl) * V + e));
  }
  for (; v < body; v += nl) {
    C f[V];
    VecLoad<T, V>::widen(VecLoad<T, V>::load(seg + head + v * V), f);
#pragma unroll
    for (int e = 0; e < V; ++e) queue_push_scan<J, FIRST>(qv, qi, f[e], static_cast<int>(head + v * V + e));
  }
  for (long long i = head + body * V + l; i < size; i += nl) {
    C f[1];
    VecLoad<T, 1>::widen(VecLoad<T, 1>::load(seg + i), f);
    queue_push_scan<J, FIRST>(qv, qi, f[0], static_cast<int>(i));
  }
}

template <typename T, int J, bool FIRST>
__global__ void __launch_bounds__(256) contig_kernel(const ContigParams p) {
  using Tr = ElemTraits<T>;
  using Bits = typename Tr::Bits;
  using C = typename Tr::Compute;
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

  C qv[J];
  int qi[J];
#pragma unroll
  for (int q = 0; q < J; ++q) {
    qv[q] = Tr::floor();
    qi[q] = FIRST ? kSentinelFirst : kSentinelLast;
  }
  const T* seg = static_cast<const T*>(p.x) + row * p.row_stride + start;
  contig_scan_segment<T, J, FIRST>(seg, size, lane, G, qv, qi);
  // Butterfly merge inside the group; all 32 lanes of the warp take part.
  for (int off = G >> 1; off >= 1; off >>= 1) {
    C ov[J];
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
    C val = qv[q];
    long long pos = qi[q];
    if (FIRST && qi[q] == kSentinelFirst) {  // empty (all padding) bucket
      val = Tr::lowest();
      pos = 0;
    }
    vdst[q] = Tr::narrow(val);
    idst[q] = start + pos;
  }
}

// Very long buckets with too few of them to occupy the GPU with one warp each:
// one block of 256 threads per bucket; warps merge by shuffles, then warp 0
// merges the 8 warp results through shared memory.
template <typename T, int J, bool FIRST>
__global__ void __launch_bounds__(256) contig_block_kernel(const ContigParams p) {
  using Tr = ElemTraits<T>;
  using Bits = typename Tr::Bits;
  using C = typename Tr::Compute;
  __shared__ C sv[8][J];
  __shared__ int si[8][J];
  const long long gid = blockIdx.x;
  const long long row = gid / p.b;
  const long long c = gid - row * p.b;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
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
  C qv[J];
  int qi[J];
#pragma unroll
  for (int q = 0; q < J; ++q) {
    qv[q] = Tr::floor();
    qi[q] = FIRST ? kSentinelFirst : kSentinelLast;
  }
  const T* seg = static_cast<const T*>(p.x) + row * p.row_stride + start;
  contig_scan_segment<T, J, FIRST>(seg, size, threadIdx.x, 256, qv, qi);
  for (int off = 16; off >= 1; off >>= 1) {
    C ov[J];
    int oi[J];
#pragma unroll
    for (int q = 0; q < J; ++q) {
      ov[q] = __shfl_xor_sync(0xffffffffu, qv[q], off);
      oi[q] = __shfl_xor_sync(0xffffffffu, qi[q], off);
    }
#pragma unroll
    for (int q = 0; q < J; ++q) queue_push_ranked<J, FIRST>(qv, qi, ov[q], oi[q]);
  }
  if (lane == 0) {
#pragma unroll
    for (int q = 0; q < J; ++q) {
      sv[warp][q] = qv[q];
      si[warp][q] = qi[q];
    }
  }
  __syncthreads();
  if (threadIdx.x != 0) return;
  for (int w = 1; w < 8; ++w)
#pragma unroll
    for (int q = 0; q < J; ++q) queue_push_ranked<J, FIRST>(qv, qi, sv[w][q], si[w][q]);
  Bits* vdst = static_cast<Bits*>(p.out_vals) + row * p.out_row_stride + c * J;
  long long* idst = p.out_idx + row * p.out_row_stride + c * J;
#pragma unroll
  for (int q = 0; q < J; ++q) {
    C val = qv[q];
    long long pos = qi[q];
    if (FIRST && qi[q] == kSentinelFirst) {
      val = Tr::lowest();
      pos = 0;
    }
    vdst[q] = Tr::narrow(val);
    idst[q] = start + pos;
  }
}

// ---------------------------------------------------------------------------
// Short buckets (at most kTileMaxBucket elements): one block takes kTileBuckets
// consecutive buckets of a row, i.e. one contiguous span of the row.  The span
// is loaded cooperatively with coalesced (16-byte where aligned) loads into
// shared memory in the compute type, then thread t scans bucket t from shared memory with
// the reference's serial insertion rule.  Element i of the span is stored at
// i + i/32, which makes the per-thread strides conflict-free for every bucket
// length.
constexpr int kTileBuckets = 128;    // buckets per block = threads per block
constexpr int kTileMaxBucket = 96;   // longest bucket served by this kernel

__device__ __forceinline__ void bucket_extent(const ContigParams& p, long long c, long long& start,
                                              long long& size) {
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
}

template <typename T, int J, bool FIRST>
__global__ void __launch_bounds__(kTileBuckets) contig_tile_kernel(const ContigParams p, long long tiles) {
  using Tr = ElemTraits<T>;
  using Bits = typename Tr::Bits;
  using C = typename Tr::Compute;
  constexpr int V = Tr::kVec;
  constexpr int kVecBytes = V * static_cast<int>(sizeof(T));
  extern __shared__ __align__(16) unsigned char tile_smem_raw[];
  C* tile_smem = reinterpret_cast<C*>(tile_smem_raw);
  const int t = threadIdx.x;
  const long long row = static_cast<long long>(blockIdx.x) / tiles;
  const long long tile = static_cast<long long>(blockIdx.x) - row * tiles;
  const long long c_begin = tile * kTileBuckets;
  long long c_end = c_begin + kTileBuckets;
  if (c_end > p.b) c_end = p.b;
  long long g0, s0, g1, s1;
  bucket_extent(p, c_begin, g0, s0);
  bucket_extent(p, c_end - 1, g1, s1);
  g1 += s1;                                   // the block's span is [g0, g1) of the row
  if (g0 > p.n) g0 = p.n;
  if (g1 > p.n) g1 = p.n;
  const T* src = static_cast<const T*>(p.x) + row * p.row_stride;
  const long long span = g1 - g0;

  // head up to the first 16-byte boundary, aligned body, tail: all inside [g0, g1)
  const uintptr_t addr0 = reinterpret_cast<uintptr_t>(src + g0);
  long long head = static_cast<long long>(((kVecBytes - (addr0 & (kVecBytes - 1))) & (kVecBytes - 1)) / sizeof(T));
  if (head > span) head = span;
  const long long body = (span - head) / V;    // whole vectors
  for (long long i = t; i < head; i += kTileBuckets) {
    C f[1];
    VecLoad<T, 1>::widen(VecLoad<T, 1>::load(src + g0 + i), f);
    tile_smem[i + (i >> 5)] = f[0];
  }
  for (long long v = t; v < body; v += kTileBuckets) {
    C f[V];
    VecLoad<T, V>::widen(VecLoad<T, V>::load(src + g0 + head + v * V), f);
#pragma unroll
    for (int e = 0; e < V; ++e) {
      const long long i = head + v * V + e;
      tile_smem[i + (i >> 5)] = f[e];
    }
  }
  for (long long i = head + body * V + t; i < span; i += kTileBuckets) {
    C f[1];
    VecLoad<T, 1>::widen(VecLoad<T, 1>::load(src + g0 + i), f);
    tile_smem[i + (i >> 5)] = f[0];
  }
  __syncthreads();

  const long long c = c_begin + t;
  if (c >= c_end) return;
  long long start, size;
  bucket_extent(p, c, start, size);
  C qv[J];
  int qi[J];
#pragma unroll
  for (int q = 0; q < J; ++q) {
    qv[q] = Tr::floor();
    qi[q] = FIRST ? kSentinelFirst : kSentinelLast;
  }
  const long long o = start - g0;
  for (int e = 0; e < static_cast<int>(size); ++e) {
    const long long i = o + e;
    queue_push_scan<J, FIRST>(qv, qi, tile_smem[i + (i >> 5)], e);
  }
  Bits* vdst = static_cast<Bits*>(p.out_vals) + row * p.out_row_stride + c * J;
  long long* idst = p.out_idx + row * p.out_row_stride + c * J;
#pragma unroll
  for (int q = 0; q < J; ++q) {
    C val = qv[q];
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
  p.g = 1;
  if (p.base + 1 <= kTileMaxBucket && p.base >= 2) {
    // short buckets: one block per 128 consecutive buckets, staged through shared memory
    const long long tiles = (a.b + kTileBuckets - 1) / kTileBuckets;
    if (a.rows * tiles >= (1ll << 31)) return ATK_ERR_TOO_LARGE;
    const long long span = static_cast<long long>(kTileBuckets) * (p.base + 1);
    const size_t smem = static_cast<size_t>(span + span / 32 + 2) * sizeof(typename ElemTraits<T>::Compute);
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(contig_tile_kernel<T, J, FIRST>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
      return ATK_ERR_CUDA;
    contig_tile_kernel<T, J, FIRST><<<static_cast<unsigned>(a.rows * tiles), kTileBuckets, smem, a.stream>>>(p, tiles);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? ATK_OK : ATK_ERR_CUDA;
  }
  if (p.base >= 8192 && a.rows * a.b * 32 < static_cast<long long>(sm_count_of_current_device()) * 1024) {
    // few, very long buckets: a block per bucket
    if (a.rows * a.b >= (1ll << 31)) return ATK_ERR_TOO_LARGE;
    contig_block_kernel<T, J, FIRST><<<static_cast<unsigned>(a.rows * a.b), 256, 0, a.stream>>>(p);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? ATK_OK : ATK_ERR_CUDA;
  }
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
    case ATK_F64: return launch_by_j<double>(a);
    case ATK_I32: return launch_by_j<int32_t>(a);
    case ATK_I64: return launch_by_j<long long>(a);
    case ATK_I16: return launch_by_j<int16_t>(a);
    case ATK_I8: return launch_by_j<int8_t>(a);
    case ATK_U8: return launch_by_j<uint8_t>(a);
    default: return ATK_ERR_BAD_DTYPE;
  }
}

}  // namespace atk
