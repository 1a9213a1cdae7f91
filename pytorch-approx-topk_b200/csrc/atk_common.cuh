// Shared device helpers for the approximate top-k kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "atk.h"

namespace atk {

// Thread-local launch counter behind atk_launch_count().
void note_launch(int n = 1);

// Sentinel stripe numbers of never-filled queue slots.  With the "last wins"
// tie rule a real element must outrank the sentinel at equal value (-inf), so
// the sentinel index is below every real index; with "first wins" above.
constexpr int kSentinelLast = -1;
constexpr int kSentinelFirst = 0x7fffffff;

template <typename T> struct ElemTraits;
template <> struct ElemTraits<float> {
  static constexpr int kDtype = ATK_F32;
  static constexpr int kVec = 4;  // elements per 16-byte load
  using Bits = uint32_t;
  static __device__ __forceinline__ float widen(Bits b) { return __uint_as_float(b); }
  static __device__ __forceinline__ Bits narrow(float f) { return __float_as_uint(f); }
  static __device__ __forceinline__ float lowest() { return -3.402823466e+38f; }
};
template <> struct ElemTraits<__half> {
  static constexpr int kDtype = ATK_F16;
  static constexpr int kVec = 8;
  using Bits = uint16_t;
  static __device__ __forceinline__ float widen(Bits b) { return __half2float(__ushort_as_half(b)); }
  static __device__ __forceinline__ Bits narrow(float f) { return __half_as_ushort(__float2half_rn(f)); }
  static __device__ __forceinline__ float lowest() { return -65504.0f; }
};
template <> struct ElemTraits<__nv_bfloat16> {
  static constexpr int kDtype = ATK_BF16;
  static constexpr int kVec = 8;
  using Bits = uint16_t;
  static __device__ __forceinline__ float widen(Bits b) { return __uint_as_float(static_cast<uint32_t>(b) << 16); }
  // The float always originates from a bf16, so the low 16 bits are zero.
  static __device__ __forceinline__ Bits narrow(float f) { return static_cast<Bits>(__float_as_uint(f) >> 16); }
  static __device__ __forceinline__ float lowest() { return -3.3895313892515355e+38f; }
};

// ---- loads of the input, which is read exactly once -------------------------
// Input loads.  Plain cached loads measured 2-6 % faster than ld.global.cs /
// ld.global.nc.L1::no_allocate on the streaming workloads, so that is the
// default; ATK_LD_MODE=0 (evict-first) / 1 (read-only path) remain as build
// knobs for re-measuring on other parts.
#ifndef ATK_LD_MODE
#define ATK_LD_MODE 3
#endif
__device__ __forceinline__ uint4 ld_stream_16(const void* p) {
#if ATK_LD_MODE == 0
  return __ldcs(reinterpret_cast<const uint4*>(p));
#elif ATK_LD_MODE == 1
  return __ldg(reinterpret_cast<const uint4*>(p));
#else
  return *reinterpret_cast<const uint4*>(p);
#endif
}
__device__ __forceinline__ uint2 ld_stream_8(const void* p) {
#if ATK_LD_MODE == 0
  return __ldcs(reinterpret_cast<const uint2*>(p));
#elif ATK_LD_MODE == 1
  return __ldg(reinterpret_cast<const uint2*>(p));
#else
  return *reinterpret_cast<const uint2*>(p);
#endif
}
// Output stores (default caching; streaming variants made no difference).
__device__ __forceinline__ void st_out_16(uint4* p, const uint4& v) { *p = v; }
__device__ __forceinline__ uint32_t ld_stream_4(const void* p) {
  return __ldcs(reinterpret_cast<const unsigned int*>(p));
}
__device__ __forceinline__ uint16_t ld_stream_2(const void* p) {
  return __ldcs(reinterpret_cast<const unsigned short*>(p));
}

// Load V consecutive elements starting at p and widen them to float.
// V == kVec: one aligned 16-byte load.  V == 1: one scalar load.
template <typename T, int V> struct VecLoad;
template <> struct VecLoad<float, 4> {
  using Raw = uint4;
  static __device__ __forceinline__ Raw load(const float* p) { return ld_stream_16(p); }
  static __device__ __forceinline__ void widen(const Raw& r, float (&v)[4]) {
    v[0] = __uint_as_float(r.x); v[1] = __uint_as_float(r.y);
    v[2] = __uint_as_float(r.z); v[3] = __uint_as_float(r.w);
  }
};
template <> struct VecLoad<float, 1> {
  using Raw = uint32_t;
  static __device__ __forceinline__ Raw load(const float* p) { return ld_stream_4(p); }
  static __device__ __forceinline__ void widen(const Raw& r, float (&v)[1]) { v[0] = __uint_as_float(r); }
};
template <> struct VecLoad<__nv_bfloat16, 8> {
  using Raw = uint4;
  static __device__ __forceinline__ Raw load(const __nv_bfloat16* p) { return ld_stream_16(p); }
  static __device__ __forceinline__ void widen(const Raw& r, float (&v)[8]) {
    v[0] = __uint_as_float(r.x << 16); v[1] = __uint_as_float(r.x & 0xffff0000u);
    v[2] = __uint_as_float(r.y << 16); v[3] = __uint_as_float(r.y & 0xffff0000u);
    v[4] = __uint_as_float(r.z << 16); v[5] = __uint_as_float(r.z & 0xffff0000u);
    v[6] = __uint_as_float(r.w << 16); v[7] = __uint_as_float(r.w & 0xffff0000u);
  }
};
template <> struct VecLoad<__nv_bfloat16, 4> {
  using Raw = uint2;
  static __device__ __forceinline__ Raw load(const __nv_bfloat16* p) { return ld_stream_8(p); }
  static __device__ __forceinline__ void widen(const Raw& r, float (&v)[4]) {
    v[0] = __uint_as_float(r.x << 16); v[1] = __uint_as_float(r.x & 0xffff0000u);
    v[2] = __uint_as_float(r.y << 16); v[3] = __uint_as_float(r.y & 0xffff0000u);
  }
};
template <> struct VecLoad<__nv_bfloat16, 1> {
  using Raw = uint16_t;
  static __device__ __forceinline__ Raw load(const __nv_bfloat16* p) { return ld_stream_2(p); }
  static __device__ __forceinline__ void widen(const Raw& r, float (&v)[1]) {
    v[0] = ElemTraits<__nv_bfloat16>::widen(r);
  }
};
template <> struct VecLoad<__half, 8> {
  using Raw = uint4;
  static __device__ __forceinline__ Raw load(const __half* p) { return ld_stream_16(p); }
  static __device__ __forceinline__ void widen(const Raw& r, float (&v)[8]) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
};
template <> struct VecLoad<__half, 4> {
  using Raw = uint2;
  static __device__ __forceinline__ Raw load(const __half* p) { return ld_stream_8(p); }
  static __device__ __forceinline__ void widen(const Raw& r, float (&v)[4]) {
    const uint32_t w[2] = {r.x, r.y};
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
};
template <> struct VecLoad<__half, 1> {
  using Raw = uint16_t;
  static __device__ __forceinline__ Raw load(const __half* p) { return ld_stream_2(p); }
  static __device__ __forceinline__ void widen(const Raw& r, float (&v)[1]) {
    v[0] = ElemTraits<__half>::widen(r);
  }
};

// ---- per-bucket queue of the J best (value, position) pairs -----------------
// Kept ascending: slot 0 is the weakest survivor.  `pos` is whatever integer
// orders elements of one bucket (stripe number or offset inside the bucket).

// Serial-scan insertion: elements arrive in increasing position order.
// LAST wins  (reference operator): enters when !(q > v), passes equal slots.
// FIRST wins (k_b = 1 arg-max entry): needs the explicit position test so a
// real -inf element replaces the sentinel.
//
// `head` is the caller-evaluated test !(qv[0] > v).  It is passed in rather
// than recomputed here on purpose: when this code sits behind a branch on the
// same comparison (the head test of long columns), nvcc 12.9 was seen to fold
// the re-evaluated `head ? v : qv[0]` to qv[0] inside rolled loops, leaving a
// stale value next to the right index.  Reusing the branch predicate itself
// gives the optimiser nothing to "correlate".
template <int J, bool FIRST>
__device__ __forceinline__ void queue_push_scan(float (&qv)[J], int (&qi)[J], float v, int pos, bool head) {
  bool p[J + 1];
#pragma unroll
  for (int i = 0; i < J; ++i) {
    if (FIRST)       p[i] = (v > qv[i]) || (v == qv[i] && pos < qi[i]);
    else if (i == 0) p[i] = head;
    else             p[i] = !(qv[i] > v);
    // The reference loop stops at the first slot that holds; chaining the
    // predicates reproduces that even when NaNs make the queue unordered.
    if (i > 0) p[i] = p[i] && p[i - 1];
  }
  p[J] = false;
#pragma unroll
  for (int i = 0; i < J; ++i) {
    // slot i takes slot i+1's content when the new item moves past i+1, the
    // new item when it stops here, otherwise it keeps its content.
    const float nv = p[i + 1] ? qv[i + 1 < J ? i + 1 : i] : (p[i] ? v : qv[i]);
    const int   ni = p[i + 1] ? qi[i + 1 < J ? i + 1 : i] : (p[i] ? pos : qi[i]);
    qv[i] = nv;
    qi[i] = ni;
  }
}
template <int J, bool FIRST>
__device__ __forceinline__ void queue_push_scan(float (&qv)[J], int (&qi)[J], float v, int pos) {
  queue_push_scan<J, FIRST>(qv, qi, v, pos, !(qv[0] > v));
}

// Order-independent insertion used when partial queues are merged: the rank is
// (value, position) with the tie rule made explicit.
template <int J, bool FIRST>
__device__ __forceinline__ void queue_push_ranked(float (&qv)[J], int (&qi)[J], float v, int pos) {
  bool p[J + 1];
#pragma unroll
  for (int i = 0; i < J; ++i) {
    if (FIRST) p[i] = (v > qv[i]) || (v == qv[i] && pos < qi[i]);
    else       p[i] = (v > qv[i]) || (v == qv[i] && pos > qi[i]);
  }
  p[J] = false;
#pragma unroll
  for (int i = 0; i < J; ++i) {
    const float nv = p[i + 1] ? qv[i + 1 < J ? i + 1 : i] : (p[i] ? v : qv[i]);
    const int   ni = p[i + 1] ? qi[i + 1 < J ? i + 1 : i] : (p[i] ? pos : qi[i]);
    qv[i] = nv;
    qi[i] = ni;
  }
}

}  // namespace atk
