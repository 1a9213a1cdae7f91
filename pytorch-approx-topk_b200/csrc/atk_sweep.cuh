// Stage 1 for interleaved buckets: the "column sweep".
//
// With interleaved buckets a row of n elements is a row-major matrix of
// `stripes x b` (b = number of buckets): element i sits in stripe i / b and
// column (= bucket) i % b, so the per-bucket top-J is a column-wise reduction
// and every stripe is contiguous in memory.  A thread owns V adjacent columns
// (V elements = one 16-byte load per stripe when alignment allows, else V = 1)
// and keeps V queues of J entries in registers; threads with the same
// threadIdx.y walk the same stripes, so a warp always reads contiguous memory
// whatever b is.  When a row offers too few columns to fill the GPU the
// stripes are split S ways inside the block (threadIdx.y) and the partial
// queues are merged through shared memory with the tie rule made explicit.
//
// Semantics follow the reference's thread-per-bucket kernel
// (approx_topk/priority_queue_approx_topk.cu: geometry :25-56, insertion
// :58-79, scan :81-107, index fix-up :109-119, slot layout :190-200).
#pragma once

#include "atk_queue.cuh"

namespace atk {

struct SweepParams {
  const void* x;
  void* out_vals;
  long long* out_idx;
  long long rows;
  long long row_stride;      // elements between rows of x
  long long out_row_stride;  // elements between rows of the outputs
  long long b;               // buckets (= columns) per row
  long long l_full;          // complete stripes: n / b
  long long rem;             // columns present in the ragged last stripe: n % b
  long long stripe_stride;   // elements between consecutive stripes in memory
  long long tiles;           // column tiles (blocks) per row
  long long idx_stride;      // reported position = stripe*idx_stride + idx_offset + column
  long long idx_offset;
  int cw;                    // blockDim.x: threads across columns
  int s;                     // blockDim.y: stripe splits inside the block (power of two)
  int vec_out;               // 16-byte stores are legal for both outputs
};

#ifndef ATK_SWEEP_THREADS
#define ATK_SWEEP_THREADS 128
#endif
#ifndef ATK_SWEEP_MINBLOCKS
#define ATK_SWEEP_MINBLOCKS 1
#endif
constexpr int kSweepMaxThreads = ATK_SWEEP_THREADS;

template <int V, int WORDS> struct SweepUnroll {
  // independent 16-byte loads kept in flight per thread; fewer when the
  // queues themselves take many registers
#ifdef ATK_DEBUG_U
  static constexpr int kU = ATK_DEBUG_U;
#else
  static constexpr int kU = (V * WORDS <= 32) ? 8 : 4;
#endif
};

// Walk this thread's complete stripes (ty, ty+S, ...) of its V columns starting
// at c0, feeding every 16-byte (or scalar) load to QS::consume.  Returns the
// first stripe number not visited (== l_full for the thread that owns the
// ragged last stripe).
template <typename T, typename QS, int V, bool SKIP>
__device__ __forceinline__ long long sweep_walk(QS (&qs)[V / QS::kCols], const SweepParams& p, const T* xrow,
                                                long long c0, int ty, int S) {
  using VL = VecLoad<T, V>;
  constexpr int U = SweepUnroll<V / QS::kCols, QS::kWords>::kU;
  const long long lf = p.l_full;
  const long long step = static_cast<long long>(S) * p.stripe_stride;
  const T* ptr = xrow + c0 + static_cast<long long>(ty) * p.stripe_stride;
  long long l = ty;
  // Main loop: U independent loads in flight, then U insertions, stripes in
  // increasing order so the scan rule resolves ties like the reference.
  for (; l + static_cast<long long>(U - 1) * S < lf; l += static_cast<long long>(U) * S) {
    typename VL::Raw raw[U];
#pragma unroll
    for (int u = 0; u < U; ++u) raw[u] = VL::load(ptr + u * step);
    ptr += U * step;
#pragma unroll
    for (int u = 0; u < U; ++u) QS::template consume<V, SKIP>(qs, raw[u], static_cast<int>(l) + u * S);
  }
  for (; l < lf; l += S) {
    const typename VL::Raw raw = VL::load(ptr);
    ptr += step;
    QS::template consume<V, SKIP>(qs, raw, static_cast<int>(l));
  }
  return l;
}

// Scan into q[V].  With SIMD (16-bit inputs on the vector path) the walk runs
// on two-column SIMD queues that are then converted to packed entries.
template <typename T, typename Q, int V, bool SKIP, bool SIMD>
__device__ __forceinline__ void sweep_scan(Q (&q)[V], const SweepParams& p, const T* xrow, long long c0,
                                           int ty, int S) {
  long long l;
  if constexpr (SIMD) {
    using QS = Simd16Queue<T, Q::kJ, Q::kFirst>;
    QS qs[V / 2];
#pragma unroll
    for (int i = 0; i < V / 2; ++i) qs[i].init();
    l = sweep_walk<T, QS, V, SKIP>(qs, p, xrow, c0, ty, S);
#pragma unroll
    for (int e = 0; e < V; ++e)
#pragma unroll
      for (int j = 0; j < Q::kJ; ++j) q[e].k[j] = qs[e / 2].packed_key(j, e & 1);
  } else {
    l = sweep_walk<T, Q, V, SKIP>(q, p, xrow, c0, ty, S);
  }
  // Ragged last stripe (b does not divide n): only columns < rem exist.  It
  // belongs to the split that would visit stripe l_full, and is that thread's
  // highest stripe, so scan order is preserved.
  if (p.rem > 0 && l == p.l_full) {
    const T* last = xrow + p.l_full * p.stripe_stride + c0;
#pragma unroll
    for (int e = 0; e < V; ++e) {
      if (c0 + e < p.rem) q[e].push_tail(VecLoad<T, 1>::load(last + e), static_cast<int>(p.l_full));
    }
  }
}

// Merge the S partial queues of every column: a binary tree over threadIdx.y.
// Word w of column-thread tx in plane y lives at ((y * V*kWords) + w) * cw + tx,
// so a warp touches consecutive words.  Needs (S/2) * V*kWords * cw words.
template <typename Q, int V>
__device__ __forceinline__ void sweep_merge(Q (&q)[V], uint32_t* smem, int cw, int tx, int ty, int S) {
  constexpr int W = Q::kWords;
  for (int h = S >> 1; h >= 1; h >>= 1) {
    if (ty >= h && ty < 2 * h) {
#pragma unroll
      for (int e = 0; e < V; ++e) q[e].store(smem + (static_cast<size_t>(ty - h) * (V * W) + e * W) * cw + tx, cw);
    }
    __syncthreads();
    if (ty < h) {
#pragma unroll
      for (int e = 0; e < V; ++e) q[e].merge(smem + (static_cast<size_t>(ty) * (V * W) + e * W) * cw + tx, cw);
    }
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------
// Stage 1 only: every block handles one tile of columns of one row and writes
// the J candidates of each bucket (slot = bucket*J + q, ascending).
template <typename T, typename Q, int J, int V, bool SKIP, bool SIMD>
__global__ void __launch_bounds__(kSweepMaxThreads, ATK_SWEEP_MINBLOCKS)
sweep_kernel(const SweepParams p) {
  using Tr = ElemTraits<T>;
  using Bits = typename Tr::Bits;
  extern __shared__ __align__(16) uint32_t sweep_smem[];

  const int tx = threadIdx.x;
  const int ty = threadIdx.y;
  const int S = p.s;
  const long long row = static_cast<long long>(blockIdx.x) / p.tiles;
  const long long tile = static_cast<long long>(blockIdx.x) - row * p.tiles;
  const long long c0 = (tile * p.cw + tx) * V;
  const bool active = c0 < p.b;
  const T* xrow = static_cast<const T*>(p.x) + row * p.row_stride;

  Q q[V];
#pragma unroll
  for (int e = 0; e < V; ++e) q[e].init();

  if (active) sweep_scan<T, Q, V, SKIP, SIMD>(q, p, xrow, c0, ty, S);
  if (S > 1) sweep_merge<Q, V>(q, sweep_smem, p.cw, tx, ty, S);
  if (!active || ty != 0) return;

  // Write-out: bucket c owns slots c*J .. c*J+J-1, ascending queue order.
  __align__(16) Bits ov[V * J];
  __align__(16) long long oi[V * J];
#pragma unroll
  for (int e = 0; e < V; ++e)
#pragma unroll
    for (int j = 0; j < J; ++j) {
      // all-padding bucket of the arg-max entry point (k > n, or the padded tail)
      if (Q::kFirst && p.l_full + (c0 + e < p.rem ? 1 : 0) == 0) {
        ov[e * J + j] = Tr::narrow(Tr::lowest());
        oi[e * J + j] = p.idx_offset + c0 + e;
      } else {
        const long long stripe = q[e].stripe(j);
        ov[e * J + j] = q[e].value_bits(j, xrow + stripe * p.stripe_stride + c0 + e);
        oi[e * J + j] = stripe * p.idx_stride + p.idx_offset + c0 + e;
      }
    }
  const long long out_base = row * p.out_row_stride + c0 * J;
  Bits* vdst = static_cast<Bits*>(p.out_vals) + out_base;
  long long* idst = p.out_idx + out_base;
  constexpr int kValBytes = V * J * static_cast<int>(sizeof(Bits));
  if (kValBytes % 16 == 0 && p.vec_out) {
    const uint4* src = reinterpret_cast<const uint4*>(ov);
#pragma unroll
    for (int i = 0; i < kValBytes / 16; ++i) st_out_16(reinterpret_cast<uint4*>(vdst) + i, src[i]);
    const uint4* isrc = reinterpret_cast<const uint4*>(oi);
#pragma unroll
    for (int i = 0; i < V * J / 2; ++i) st_out_16(reinterpret_cast<uint4*>(idst) + i, isrc[i]);
  } else {
#pragma unroll
    for (int i = 0; i < V * J; ++i) {
      vdst[i] = ov[i];
      idst[i] = oi[i];
    }
  }
}

// Arguments of the typed launchers (one translation unit per element type).
struct SweepLaunch {
  const void* x;
  void* out_vals;
  long long* out_idx;
  long long rows, n, row_stride, out_row_stride;
  long long b;              // buckets per row
  long long stripe_stride;  // == b for a plain row
  long long idx_stride;     // == b for a plain row
  long long idx_offset;
  int j;
  bool first_wins;          // k_b = 1 arg-max conventions (J must be 1)
  int sm_count;
  cudaStream_t stream;
};

int launch_sweep_f32(const SweepLaunch& a);
int launch_sweep_f16(const SweepLaunch& a);
int launch_sweep_bf16(const SweepLaunch& a);

}  // namespace atk
