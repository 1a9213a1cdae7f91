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

// Number of SMs of the current device (queried once per device, then cached).
int sm_count_of_current_device();

// Programmatic dependent launch.  The stage-1 kernels announce at their start that the
// kernel after them in the stream may be brought onto the GPU; a consumer launched with
// launch_overlapped() then becomes resident while the producer's last blocks still run,
// does what does not depend on the producer (index arithmetic, clearing shared memory)
// and stops at grid_dependency_wait() until the producer has finished and its writes
// are visible.  Both instructions do nothing in a kernel that was launched the plain way.
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// false when ATK_NO_OVERLAPPED_LAUNCH is set in the environment (read once)
bool overlapped_launch_enabled();

// `overlap` false: a plain launch of the same kernel.
template <typename... Params, typename... Args>
inline cudaError_t launch_overlapped_if(bool overlap, void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem,
                                        cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = overlap && overlapped_launch_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<Params>(args)...);
}

template <typename... Params, typename... Args>
inline cudaError_t launch_overlapped(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem,
                                     cudaStream_t stream, Args&&... args) {
  return launch_overlapped_if(true, kernel, grid, block, smem, stream, static_cast<Args&&>(args)...);
}

// Where the final (value, position) pairs of a row go, in one of the output
// formats of include/atk.h: values + int64 positions (the reference's layout),
// values + int32 positions, or 8-byte records {value bits zero-extended to 32
// bits, int32 position}.  `at(offset)` is the same row advanced by `offset` pairs.
template <typename B>
struct OutRow {
  B* v;
  void* i;      // long long* (ATK_OUT_I64) or int* (ATK_OUT_I32); unused for records
  uint2* rec;   // ATK_OUT_REC32
  int fmt;
  __device__ __forceinline__ OutRow(void* out_vals, void* out_idx, long long row, long long row_stride, int format)
      : v(nullptr), i(nullptr), rec(nullptr), fmt(format) {
    const long long off = row * row_stride;
    if (format == ATK_OUT_REC32) {
      rec = static_cast<uint2*>(out_vals) + off;
    } else {
      v = static_cast<B*>(out_vals) + off;
      i = format == ATK_OUT_I32 ? static_cast<void*>(static_cast<int*>(out_idx) + off)
                                : static_cast<void*>(static_cast<long long*>(out_idx) + off);
    }
  }
  __device__ __forceinline__ OutRow at(long long offset) const {
    OutRow r = *this;
    if (fmt == ATK_OUT_REC32) {
      r.rec += offset;
    } else {
      r.v += offset;
      r.i = fmt == ATK_OUT_I32 ? static_cast<void*>(static_cast<int*>(i) + offset)
                               : static_cast<void*>(static_cast<long long*>(i) + offset);
    }
    return r;
  }
  // both destinations (or the record array) start on a 16-byte boundary
  __device__ __forceinline__ bool aligned16() const {
    if (fmt == ATK_OUT_REC32) return reinterpret_cast<uintptr_t>(rec) % 16 == 0;
    return reinterpret_cast<uintptr_t>(v) % 16 == 0 && reinterpret_cast<uintptr_t>(i) % 16 == 0;
  }
  __device__ __forceinline__ void put(long long slot, B value, long long position) const {
    if (fmt == ATK_OUT_REC32) {
      rec[slot] = make_uint2(static_cast<uint32_t>(value), static_cast<uint32_t>(static_cast<int>(position)));
    } else {
      v[slot] = value;
      if (fmt == ATK_OUT_I32) static_cast<int*>(i)[slot] = static_cast<int>(position);
      else static_cast<long long*>(i)[slot] = position;
    }
  }
};

// Sentinel stripe numbers of never-filled queue slots.  With the "last wins"
// tie rule a real element must outrank the sentinel at equal value (-inf), so
// the sentinel index is below every real index; with "first wins" above.
constexpr int kSentinelLast = -1;
constexpr int kSentinelFirst = 0x7fffffff;

// Per element type: the code in the C ABI, the preferred vector width of the
// sweep (elements per load), the raw storage word (`Bits`), and the type the
// compares run in (`Compute`: float for the three small float types, which
// widen exactly; int for the integer types of 32 bits or fewer; the type itself
// for the 64-bit ones).  `floor()` is the value of a never-filled queue slot:
// it ranks below or equal to every element, and a real element of equal value
// outranks it through the sentinel position.
template <typename T> struct ElemTraits;
template <> struct ElemTraits<float> {
  static constexpr int kDtype = ATK_F32;
  static constexpr int kVec = 4;  // elements per 16-byte load
  static constexpr bool kHalfFloat = false;
  using Bits = uint32_t;
  using Compute = float;
  static __device__ __forceinline__ float widen(Bits b) { return __uint_as_float(b); }
  static __device__ __forceinline__ Bits narrow(float f) { return __float_as_uint(f); }
  static __device__ __forceinline__ float lowest() { return -3.402823466e+38f; }
  static __device__ __forceinline__ float floor() { return -INFINITY; }
};
template <> struct ElemTraits<__half> {
  static constexpr int kDtype = ATK_F16;
  static constexpr int kVec = 8;
  static constexpr bool kHalfFloat = true;
  using Bits = uint16_t;
  using Compute = float;
  static __device__ __forceinline__ float widen(Bits b) { return __half2float(__ushort_as_half(b)); }
  static __device__ __forceinline__ Bits narrow(float f) { return __half_as_ushort(__float2half_rn(f)); }
  static __device__ __forceinline__ float lowest() { return -65504.0f; }
  static __device__ __forceinline__ float floor() { return -INFINITY; }
};
template <> struct ElemTraits<__nv_bfloat16> {
  static constexpr int kDtype = ATK_BF16;
  static constexpr int kVec = 8;
  static constexpr bool kHalfFloat = true;
  using Bits = uint16_t;
  using Compute = float;
  static __device__ __forceinline__ float widen(Bits b) { return __uint_as_float(static_cast<uint32_t>(b) << 16); }
  // The float always originates from a bf16, so the low 16 bits are zero.
  static __device__ __forceinline__ Bits narrow(float f) { return static_cast<Bits>(__float_as_uint(f) >> 16); }
  static __device__ __forceinline__ float lowest() { return -3.3895313892515355e+38f; }
  static __device__ __forceinline__ float floor() { return -INFINITY; }
};
template <> struct ElemTraits<double> {
  static constexpr int kDtype = ATK_F64;
  static constexpr int kVec = 2;
  static constexpr bool kHalfFloat = false;
  using Bits = unsigned long long;
  using Compute = double;
  static __device__ __forceinline__ double widen(Bits b) { return __longlong_as_double(static_cast<long long>(b)); }
  static __device__ __forceinline__ Bits narrow(double f) { return static_cast<Bits>(__double_as_longlong(f)); }
  static __device__ __forceinline__ double lowest() { return -1.7976931348623157e+308; }
  static __device__ __forceinline__ double floor() { return -__longlong_as_double(0x7ff0000000000000ll); }
};
// Integer types: `SIGNED` is the signed type of the same width (or the type
// itself), `lo` the smallest value.
template <typename S, typename BITS, typename COMPUTE, int DTYPE, int VEC, long long LO>
struct IntTraits {
  static constexpr int kDtype = DTYPE;
  static constexpr int kVec = VEC;
  static constexpr bool kHalfFloat = false;
  using Bits = BITS;
  using Compute = COMPUTE;
  static __device__ __forceinline__ COMPUTE widen(BITS b) { return static_cast<COMPUTE>(static_cast<S>(b)); }
  static __device__ __forceinline__ BITS narrow(COMPUTE v) { return static_cast<BITS>(v); }
  static __device__ __forceinline__ COMPUTE lowest() { return static_cast<COMPUTE>(LO); }
  static __device__ __forceinline__ COMPUTE floor() { return static_cast<COMPUTE>(LO); }
};
template <> struct ElemTraits<int32_t> : IntTraits<int32_t, uint32_t, int, ATK_I32, 4, -2147483647ll - 1> {};
template <> struct ElemTraits<long long>
    : IntTraits<long long, unsigned long long, long long, ATK_I64, 2, -9223372036854775807ll - 1> {};
template <> struct ElemTraits<int16_t> : IntTraits<int16_t, uint16_t, int, ATK_I16, 8, -32768> {};
// 8-bit elements: 8 columns per thread (8-byte loads) keep the queues in registers
template <> struct ElemTraits<int8_t> : IntTraits<int8_t, uint8_t, int, ATK_I8, 8, -128> {};
template <> struct ElemTraits<uint8_t> : IntTraits<uint8_t, uint8_t, int, ATK_U8, 8, 0> {};

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
__device__ __forceinline__ uint8_t ld_stream_1(const void* p) {
  return __ldcs(reinterpret_cast<const unsigned char*>(p));
}

// One element as its raw storage word.
template <typename T>
__device__ __forceinline__ typename ElemTraits<T>::Bits load_elem_bits(const T* p) {
  return __ldcs(reinterpret_cast<const typename ElemTraits<T>::Bits*>(p));
}

// A load of BYTES bytes and its view as 32-bit words (low word first).
template <int BYTES> struct RawBytes;
template <> struct RawBytes<16> {
  using Raw = uint4;
  static constexpr int kWords = 4;
  static __device__ __forceinline__ Raw load(const void* p) { return ld_stream_16(p); }
  static __device__ __forceinline__ void words(const Raw& r, uint32_t (&w)[4]) { w[0] = r.x; w[1] = r.y; w[2] = r.z; w[3] = r.w; }
};
template <> struct RawBytes<8> {
  using Raw = uint2;
  static constexpr int kWords = 2;
  static __device__ __forceinline__ Raw load(const void* p) { return ld_stream_8(p); }
  static __device__ __forceinline__ void words(const Raw& r, uint32_t (&w)[2]) { w[0] = r.x; w[1] = r.y; }
};
template <> struct RawBytes<4> {
  using Raw = uint32_t;
  static constexpr int kWords = 1;
  static __device__ __forceinline__ Raw load(const void* p) { return ld_stream_4(p); }
  static __device__ __forceinline__ void words(const Raw& r, uint32_t (&w)[1]) { w[0] = r; }
};
template <> struct RawBytes<2> {
  using Raw = uint16_t;
  static constexpr int kWords = 1;
  static __device__ __forceinline__ Raw load(const void* p) { return ld_stream_2(p); }
  static __device__ __forceinline__ void words(const Raw& r, uint32_t (&w)[1]) { w[0] = r; }
};
template <> struct RawBytes<1> {
  using Raw = uint8_t;
  static constexpr int kWords = 1;
  static __device__ __forceinline__ Raw load(const void* p) { return ld_stream_1(p); }
  static __device__ __forceinline__ void words(const Raw& r, uint32_t (&w)[1]) { w[0] = r; }
};

// Load V consecutive elements starting at p and widen them to the compute type.
// V > 1: one aligned vector load of V * sizeof(T) bytes.  V == 1: one scalar load.
// The primary template serves the integer and 64-bit types (elements are cut
// out of the loaded words); the small float types have their own conversions.
template <typename T, int V> struct VecLoad {
  using Tr = ElemTraits<T>;
  using RB = RawBytes<V * static_cast<int>(sizeof(T))>;
  using Raw = typename RB::Raw;
  static __device__ __forceinline__ Raw load(const T* p) { return RB::load(p); }
  static __device__ __forceinline__ void widen(const Raw& r, typename Tr::Compute (&v)[V]) {
    uint32_t w[RB::kWords];
    RB::words(r, w);
#pragma unroll
    for (int e = 0; e < V; ++e) {
      if constexpr (sizeof(T) == 8) {
        v[e] = Tr::widen(static_cast<typename Tr::Bits>(w[2 * e]) |
                         (static_cast<typename Tr::Bits>(w[2 * e + 1]) << 32));
      } else if constexpr (sizeof(T) == 4) {
        v[e] = Tr::widen(w[e]);
      } else if constexpr (sizeof(T) == 2) {
        v[e] = Tr::widen(static_cast<typename Tr::Bits>((w[e / 2] >> (16 * (e & 1))) & 0xffffu));
      } else {
        v[e] = Tr::widen(static_cast<typename Tr::Bits>((w[e / 4] >> (8 * (e & 3))) & 0xffu));
      }
    }
  }
};
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
template <int J, bool FIRST, typename C>
__device__ __forceinline__ void queue_push_scan(C (&qv)[J], int (&qi)[J], C v, int pos, bool head) {
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
    const C   nv = p[i + 1] ? qv[i + 1 < J ? i + 1 : i] : (p[i] ? v : qv[i]);
    const int ni = p[i + 1] ? qi[i + 1 < J ? i + 1 : i] : (p[i] ? pos : qi[i]);
    qv[i] = nv;
    qi[i] = ni;
  }
}
template <int J, bool FIRST, typename C>
__device__ __forceinline__ void queue_push_scan(C (&qv)[J], int (&qi)[J], C v, int pos) {
  queue_push_scan<J, FIRST, C>(qv, qi, v, pos, !(qv[0] > v));
}

// Order-independent insertion used when partial queues are merged: the rank is
// (value, position) with the tie rule made explicit.
template <int J, bool FIRST, typename C>
__device__ __forceinline__ void queue_push_ranked(C (&qv)[J], int (&qi)[J], C v, int pos) {
  bool p[J + 1];
#pragma unroll
  for (int i = 0; i < J; ++i) {
    if (FIRST) p[i] = (v > qv[i]) || (v == qv[i] && pos < qi[i]);
    else       p[i] = (v > qv[i]) || (v == qv[i] && pos > qi[i]);
  }
  p[J] = false;
#pragma unroll
  for (int i = 0; i < J; ++i) {
    const C   nv = p[i + 1] ? qv[i + 1 < J ? i + 1 : i] : (p[i] ? v : qv[i]);
    const int ni = p[i + 1] ? qi[i + 1 < J ? i + 1 : i] : (p[i] ? pos : qi[i]);
    qv[i] = nv;
    qi[i] = ni;
  }
}

}  // namespace atk
