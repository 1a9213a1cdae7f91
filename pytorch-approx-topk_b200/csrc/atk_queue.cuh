// Per-column queues of the J best elements, in two register layouts.
//
// FloatQueue  — J (float value, int stripe) pairs; works for every dtype (the
//               16-bit formats widen to float exactly) and follows the
//               reference's insertion rule instruction for instruction,
//               NaN behaviour included.
// PackedQueue — for 16-bit inputs whose columns have at most 65536 stripes:
//               one 32-bit word per entry, (order-preserving image of the
//               value) << 16 | stripe, so that the (value, position) ranking
//               "largest value first, later position wins" is a plain unsigned
//               compare and an insertion is 2J-1 integer min/max operations
//               with the stripe carried for free.  Differences from the
//               reference are confined to inputs it leaves unpinned: NaNs
//               rank by bit pattern (above +inf / below -inf) and -0.0 ties
//               with +0.0 exactly as in a float compare.
//
// Both expose the same interface to the sweep kernels:
//   init(), consume<SKIP>(q[V], raw, stripe), push_tail(elem bits, stripe),
//   store/merge through shared memory words, and accessors for the write-out.
#pragma once

#include "atk_common.cuh"

namespace atk {

// ---------------------------------------------------------------- FloatQueue
template <typename T, int J, bool FIRST>
struct FloatQueue {
  static constexpr int kWords = 2 * J;  // 32-bit words per queue in shared memory
  static constexpr bool kPacked = false;
  float v[J];
  int s[J];

  __device__ __forceinline__ void init() {
#pragma unroll
    for (int q = 0; q < J; ++q) {
      v[q] = -INFINITY;
      s[q] = FIRST ? kSentinelFirst : kSentinelLast;
    }
  }

  template <int V, bool SKIP>
  static __device__ __forceinline__ void consume(FloatQueue (&q)[V], const typename VecLoad<T, V>::Raw& raw,
                                                 int stripe) {
    float x[V];
    VecLoad<T, V>::widen(raw, x);
    bool head[V];
#pragma unroll
    for (int e = 0; e < V; ++e) head[e] = !(q[e].v[0] > x[e]);
    if (SKIP) {
      // Long columns: almost no element beats the current J-th best, so test
      // the V heads first and only run the insertion network when one does.
      bool any = false;
#pragma unroll
      for (int e = 0; e < V; ++e) any = any || head[e];
      if (any) {
#pragma unroll
        for (int e = 0; e < V; ++e) queue_push_scan<J, FIRST>(q[e].v, q[e].s, x[e], stripe, head[e]);
      }
    } else {
#pragma unroll
      for (int e = 0; e < V; ++e) queue_push_scan<J, FIRST>(q[e].v, q[e].s, x[e], stripe, head[e]);
    }
  }

  // one element of the ragged last stripe
  __device__ __forceinline__ void push_tail(typename ElemTraits<T>::Bits bits, int stripe) {
    queue_push_scan<J, FIRST>(v, s, ElemTraits<T>::widen(bits), stripe);
  }

  __device__ __forceinline__ void store(uint32_t* base, int stride) const {
#pragma unroll
    for (int q = 0; q < J; ++q) {
      base[(2 * q) * stride] = __float_as_uint(v[q]);
      base[(2 * q + 1) * stride] = static_cast<uint32_t>(s[q]);
    }
  }
  __device__ __forceinline__ void merge(const uint32_t* base, int stride) {
#pragma unroll
    for (int q = 0; q < J; ++q)
      queue_push_ranked<J, FIRST>(v, s, __uint_as_float(base[(2 * q) * stride]),
                                  static_cast<int>(base[(2 * q + 1) * stride]));
  }

  __device__ __forceinline__ bool empty(int q) const { return FIRST && s[q] == kSentinelFirst; }
  __device__ __forceinline__ long long stripe(int q) const { return s[q]; }
  // value bits for the output; `elem` is only read to restore a zero's sign
  __device__ __forceinline__ typename ElemTraits<T>::Bits value_bits(int q, const T*) const {
    return ElemTraits<T>::narrow(v[q]);
  }
  // order-preserving 32-bit image of the value for the exact select
  __device__ __forceinline__ uint32_t select_key(int q) const {
    const uint32_t u = __float_as_uint(v[q]);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
  }
};

// --------------------------------------------------------------- PackedQueue
// Order-preserving image of two 16-bit floats at once (fp16 or bf16, both are
// sign-magnitude): positive -> 0x8000 + magnitude, negative -> 0x8000 -
// magnitude, so both zeros map to 0x8000 and nothing maps to 0 (the sentinel).
__device__ __forceinline__ uint32_t ord16x2(uint32_t w) {
  const uint32_t sgn = (w >> 15) & 0x00010001u;
  const uint32_t flip = sgn * 0x7fffu + 0x80008000u;  // 0xffff where negative, else 0x8000
  return (w ^ flip) + sgn;
}
__device__ __forceinline__ uint16_t ord16_inverse(uint32_t o) {
  return static_cast<uint16_t>(o >= 0x8000u ? (o ^ 0x8000u) : (0x8000u | (0x8000u - o)));
}

template <typename T, int J, bool FIRST>
struct PackedQueue {
  static_assert(sizeof(T) == 2, "packed queues are for 16-bit element types");
  static constexpr int kWords = J;
  static constexpr bool kPacked = true;
  uint32_t k[J];  // ascending; 0 = never filled

  __device__ __forceinline__ void init() {
#pragma unroll
    for (int q = 0; q < J; ++q) k[q] = 0u;
  }

  // With FIRST the earlier position must win a tie, so the low half holds the
  // complement of the stripe number.
  static __device__ __forceinline__ uint32_t low(int stripe) {
    return FIRST ? (0xffffu - static_cast<uint32_t>(stripe)) : static_cast<uint32_t>(stripe);
  }

  __device__ __forceinline__ void push(uint32_t key) {
    uint32_t n[J];
#pragma unroll
    for (int q = 0; q + 1 < J; ++q) n[q] = min(max(key, k[q]), k[q + 1]);
    n[J - 1] = max(key, k[J - 1]);
#pragma unroll
    for (int q = 0; q < J; ++q) k[q] = n[q];
  }

  template <int V, bool SKIP>
  static __device__ __forceinline__ void consume(PackedQueue (&q)[V], const typename VecLoad<T, V>::Raw& raw,
                                                 int stripe) {
    const uint32_t lo = low(stripe);
    if constexpr (V == 1) {
      const uint32_t key = ((ord16x2(raw) & 0xffffu) << 16) | lo;
      if (!SKIP || key > q[0].k[0]) q[0].push(key);
    } else {
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
      uint32_t key[V];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t o = ord16x2(w[i]);
        key[2 * i] = (o << 16) | lo;
        key[2 * i + 1] = (o & 0xffff0000u) | lo;
      }
      if (SKIP) {
        bool any = false;
#pragma unroll
        for (int e = 0; e < V; ++e) any = any || key[e] > q[e].k[0];
        if (!any) return;
      }
#pragma unroll
      for (int e = 0; e < V; ++e) q[e].push(key[e]);
    }
  }

  __device__ __forceinline__ void push_tail(uint16_t bits, int stripe) {
    push(((ord16x2(bits) & 0xffffu) << 16) | low(stripe));
  }

  __device__ __forceinline__ void store(uint32_t* base, int stride) const {
#pragma unroll
    for (int q = 0; q < J; ++q) base[q * stride] = k[q];
  }
  __device__ __forceinline__ void merge(const uint32_t* base, int stride) {
#pragma unroll
    for (int q = 0; q < J; ++q) push(base[q * stride]);
  }

  __device__ __forceinline__ bool empty(int q) const { return k[q] == 0u; }
  __device__ __forceinline__ long long stripe(int q) const {
    const uint32_t l = k[q] & 0xffffu;
    return FIRST ? (0xffffu - l) : l;
  }
  // Both zeros share one key; the element itself is read back to return the
  // sign the input had (a load that almost never executes).
  __device__ __forceinline__ uint16_t value_bits(int q, const T* elem) const {
    const uint32_t o = k[q] >> 16;
    if (o == 0x8000u) return ld_stream_2(elem);
    return ord16_inverse(o);
  }
  __device__ __forceinline__ uint32_t select_key(int q) const { return k[q] & 0xffff0000u; }
};

}  // namespace atk
