// Stage 1 for interleaved buckets: the "column sweep".
//
// With interleaved buckets a row of n elements is a row-major matrix of
// `stripes x b` (b = number of buckets): element i sits in stripe i / b and
// column (= bucket) i % b, so the per-bucket top-J is a column-wise reduction
// and every stripe is contiguous in memory.  A thread owns V adjacent columns
// (V elements = one 16-byte load per stripe when alignment allows, else V = 1)
// and keeps V queues of J (value, stripe) pairs in registers; threads with the
// same threadIdx.y walk the same stripes, so a warp always reads contiguous
// memory whatever b is.  When a row offers too few columns to fill the GPU the
// stripes are split S ways inside the block (threadIdx.y) and the partial
// queues are merged through shared memory with the tie rule made explicit.
//
// Semantics follow the reference's thread-per-bucket kernel
// (approx_topk/priority_queue_approx_topk.cu: geometry :25-56, insertion
// :58-79, scan :81-107, index fix-up :109-119, slot layout :190-200).
#pragma once

#include "atk_common.cuh"

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

template <int V, int J> struct SweepUnroll {
  // independent 16-byte loads kept in flight per thread
#ifdef ATK_DEBUG_U
  static constexpr int kU = ATK_DEBUG_U;
#else
  static constexpr int kU = (V * J <= 16) ? 8 : 4;
#endif
};

template <typename T, int J, int V, bool FIRST, bool SKIP>
__device__ __forceinline__ void sweep_consume(float (&qv)[V][J], int (&qi)[V][J],
                                              const typename VecLoad<T, V>::Raw& raw, int stripe) {
  float v[V];
  VecLoad<T, V>::widen(raw, v);
  bool head[V];
#pragma unroll
  for (int e = 0; e < V; ++e) head[e] = !(qv[e][0] > v[e]);
  if (SKIP) {
    // Long columns: almost no element beats the current J-th best, so test
    // the V heads first and only run the insertion network when one does.
    bool any = false;
#pragma unroll
    for (int e = 0; e < V; ++e) any = any || head[e];
    if (any) {
#pragma unroll
      for (int e = 0; e < V; ++e) queue_push_scan<J, FIRST>(qv[e], qi[e], v[e], stripe, head[e]);
    }
  } else {
#pragma unroll
    for (int e = 0; e < V; ++e) queue_push_scan<J, FIRST>(qv[e], qi[e], v[e], stripe, head[e]);
  }
}

template <typename T, int J, int V, bool FIRST, bool SKIP>
__global__ void __launch_bounds__(kSweepMaxThreads, ATK_SWEEP_MINBLOCKS)
sweep_kernel(const SweepParams p) {
  using Tr = ElemTraits<T>;
  using VL = VecLoad<T, V>;
  using Bits = typename Tr::Bits;
  constexpr int U = SweepUnroll<V, J>::kU;
  extern __shared__ __align__(16) unsigned char sweep_smem[];

  const int tx = threadIdx.x;
  const int ty = threadIdx.y;
  const int S = p.s;
  const long long row = static_cast<long long>(blockIdx.x) / p.tiles;
  const long long tile = static_cast<long long>(blockIdx.x) - row * p.tiles;
  const long long c0 = (tile * p.cw + tx) * V;
  const bool active = c0 < p.b;
  const T* xrow = static_cast<const T*>(p.x) + row * p.row_stride;

  float qv[V][J];
  int qi[V][J];
#pragma unroll
  for (int e = 0; e < V; ++e)
#pragma unroll
    for (int q = 0; q < J; ++q) {
      qv[e][q] = -INFINITY;
      qi[e][q] = FIRST ? kSentinelFirst : kSentinelLast;
    }

  if (active) {
    const long long lf = p.l_full;
    const long long step = static_cast<long long>(S) * p.stripe_stride;
    const T* ptr = xrow + c0 + static_cast<long long>(ty) * p.stripe_stride;
    long long l = ty;
    // Main loop: U independent loads in flight, then U insertions, stripes in
    // increasing order so the scan rule resolves ties like the reference.
#if defined(ATK_SWEEP_PIPE)
    // Software-pipelined: the next batch of U loads is issued before the
    // current batch is consumed (two register buffers, ping-pong).
    {
      const long long batch = static_cast<long long>(U) * S;
      typename VL::Raw ra[U], rb[U];
      bool have = l + static_cast<long long>(U - 1) * S < lf;
      if (have) {
#pragma unroll
        for (int u = 0; u < U; ++u) ra[u] = VL::load(ptr + u * step);
        ptr += U * step;
      }
      while (have) {
        const bool have_b = l + batch + static_cast<long long>(U - 1) * S < lf;
        if (have_b) {
#pragma unroll
          for (int u = 0; u < U; ++u) rb[u] = VL::load(ptr + u * step);
          ptr += U * step;
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
          sweep_consume<T, J, V, FIRST, SKIP>(qv, qi, ra[u], static_cast<int>(l) + u * S);
        l += batch;
        if (!have_b) break;
        const bool have_a = l + batch + static_cast<long long>(U - 1) * S < lf;
        if (have_a) {
#pragma unroll
          for (int u = 0; u < U; ++u) ra[u] = VL::load(ptr + u * step);
          ptr += U * step;
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
          sweep_consume<T, J, V, FIRST, SKIP>(qv, qi, rb[u], static_cast<int>(l) + u * S);
        l += batch;
        have = have_a;
      }
    }
#else
    for (; l + static_cast<long long>(U - 1) * S < lf; l += static_cast<long long>(U) * S) {
      typename VL::Raw raw[U];
#pragma unroll
      for (int u = 0; u < U; ++u) raw[u] = VL::load(ptr + u * step);
      ptr += U * step;
#pragma unroll
      for (int u = 0; u < U; ++u)
        sweep_consume<T, J, V, FIRST, SKIP>(qv, qi, raw[u], static_cast<int>(l) + u * S);
    }
#endif
    for (; l < lf; l += S) {
      const typename VL::Raw raw = VL::load(ptr);
      ptr += step;
      sweep_consume<T, J, V, FIRST, SKIP>(qv, qi, raw, static_cast<int>(l));
    }
    // Ragged last stripe (b does not divide n): only columns < rem exist.
    // It belongs to the split that would visit stripe l_full, and is that
    // thread's highest stripe, so scan order is preserved.
    if (p.rem > 0 && l == lf) {
      const T* last = xrow + lf * p.stripe_stride + c0;
#pragma unroll
      for (int e = 0; e < V; ++e) {
        if (c0 + e < p.rem) {
          float v1[1];
          VecLoad<T, 1>::widen(VecLoad<T, 1>::load(last + e), v1);
          queue_push_scan<J, FIRST>(qv[e], qi[e], v1[0], static_cast<int>(lf));
        }
      }
    }
  }

  // Merge the S partial queues of every column: a binary tree over
  // threadIdx.y.  Entry (e, q) of column-thread tx in plane y lives at
  // ((y * V*J) + e*J + q) * cw + tx, so a warp touches consecutive words.
  if (S > 1) {
    const int cw = p.cw;
    float* mv = reinterpret_cast<float*>(sweep_smem);
    int* mi = reinterpret_cast<int*>(mv + static_cast<size_t>(S / 2) * (V * J) * cw);
    for (int h = S >> 1; h >= 1; h >>= 1) {
      if (ty >= h && ty < 2 * h) {
        const int plane = ty - h;
#pragma unroll
        for (int e = 0; e < V; ++e)
#pragma unroll
          for (int q = 0; q < J; ++q) {
            const int off = (plane * (V * J) + e * J + q) * cw + tx;
            mv[off] = qv[e][q];
            mi[off] = qi[e][q];
          }
      }
      __syncthreads();
      if (ty < h) {
#pragma unroll
        for (int e = 0; e < V; ++e)
#pragma unroll
          for (int q = 0; q < J; ++q) {
            const int off = (ty * (V * J) + e * J + q) * cw + tx;
            queue_push_ranked<J, FIRST>(qv[e], qi[e], mv[off], mi[off]);
          }
      }
      __syncthreads();
    }
  }

  if (!active || ty != 0) return;

  // Write-out: bucket c owns slots c*J .. c*J+J-1, ascending queue order.
  __align__(16) Bits ov[V * J];
  __align__(16) long long oi[V * J];
#pragma unroll
  for (int e = 0; e < V; ++e)
#pragma unroll
    for (int q = 0; q < J; ++q) {
      float val = qv[e][q];
      long long stripe = qi[e][q];
      if (FIRST && qi[e][q] == kSentinelFirst) {  // empty (all padding) bucket
        val = Tr::lowest();
        stripe = 0;
      }
      ov[e * J + q] = Tr::narrow(val);
      oi[e * J + q] = stripe * p.idx_stride + p.idx_offset + c0 + e;
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
