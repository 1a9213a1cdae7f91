// Per-column queues of the J best elements, in three register layouts.
//
// FloatQueue  — J (value, int stripe) pairs with the value in the element
//               type's compute type (float for the float types of 32 bits or
//               fewer, which widen exactly; int / long long / double for the
//               rest).  Works for every dtype and follows the reference's
//               insertion rule instruction for instruction, NaN behaviour
//               included.
// PackedQueue — for 8- and 16-bit inputs (float or integer) whose stripe numbers
//               fit beside the value (65536 / 2^24 stripes):
//               one 32-bit word per entry, (order-preserving image of the
//               value) << 16 or 24 | stripe, so that the (value, position) ranking
//               "largest value first, later position wins" is a plain unsigned
//               compare and an insertion is 2J-1 integer min/max operations
//               with the stripe carried for free.  Differences from the
//               reference are confined to inputs it leaves unpinned: NaNs
//               rank by bit pattern (above +inf / below -inf) and -0.0 ties
//               with +0.0 exactly as in a float compare.
//
// Simd16Queue — scan-time form of PackedQueue on the vector path, see below.
//
// FloatQueue and PackedQueue expose the same interface to the sweep kernel:
//   init(), consume<V, SKIP>(q[V], raw, stripe), push_tail(elem bits, stripe),
//   store/merge through shared memory words, and accessors for the write-out.
#pragma once

#include "atk_common.cuh"

namespace atk {

// ---------------------------------------------------------------- FloatQueue
// 32-bit words of a compute-type value, for the trip through shared memory.
template <typename C> struct ComputeWords;
template <> struct ComputeWords<float> {
  static constexpr int kN = 1;
  static __device__ __forceinline__ void put(float v, uint32_t* base, int stride) { base[0] = __float_as_uint(v); }
  static __device__ __forceinline__ float get(const uint32_t* base, int stride) { return __uint_as_float(base[0]); }
};
template <> struct ComputeWords<int> {
  static constexpr int kN = 1;
  static __device__ __forceinline__ void put(int v, uint32_t* base, int stride) { base[0] = static_cast<uint32_t>(v); }
  static __device__ __forceinline__ int get(const uint32_t* base, int stride) { return static_cast<int>(base[0]); }
};
template <> struct ComputeWords<long long> {
  static constexpr int kN = 2;
  static __device__ __forceinline__ void put(long long v, uint32_t* base, int stride) {
    base[0] = static_cast<uint32_t>(static_cast<unsigned long long>(v));
    base[stride] = static_cast<uint32_t>(static_cast<unsigned long long>(v) >> 32);
  }
  static __device__ __forceinline__ long long get(const uint32_t* base, int stride) {
    return static_cast<long long>(static_cast<unsigned long long>(base[0]) |
                                  (static_cast<unsigned long long>(base[stride]) << 32));
  }
};
template <> struct ComputeWords<double> {
  static constexpr int kN = 2;
  static __device__ __forceinline__ void put(double v, uint32_t* base, int stride) {
    ComputeWords<long long>::put(__double_as_longlong(v), base, stride);
  }
  static __device__ __forceinline__ double get(const uint32_t* base, int stride) {
    return __longlong_as_double(ComputeWords<long long>::get(base, stride));
  }
};

template <typename T, int J, bool FIRST>
struct FloatQueue {
  using Tr = ElemTraits<T>;
  using C = typename Tr::Compute;
  using CW = ComputeWords<C>;
  static constexpr int kEntryWords = CW::kN + 1;
  static constexpr int kWords = kEntryWords * J;  // 32-bit words per queue in shared memory
  static constexpr bool kPacked = false;
  static constexpr int kCols = 1;       // columns served by one queue object
  static constexpr int kJ = J;
  static constexpr bool kFirst = FIRST;
  C v[J];
  int s[J];

  __device__ __forceinline__ void init() {
#pragma unroll
    for (int q = 0; q < J; ++q) {
      v[q] = Tr::floor();
      s[q] = FIRST ? kSentinelFirst : kSentinelLast;
    }
  }

  template <int V, bool SKIP>
  static __device__ __forceinline__ void consume(FloatQueue (&q)[V], const typename VecLoad<T, V>::Raw& raw,
                                                 int stripe) {
    C x[V];
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
  __device__ __forceinline__ void push_tail(typename Tr::Bits bits, int stripe) {
    queue_push_scan<J, FIRST>(v, s, Tr::widen(bits), stripe);
  }

  __device__ __forceinline__ void store(uint32_t* base, int stride) const {
#pragma unroll
    for (int q = 0; q < J; ++q) {
      CW::put(v[q], base + (kEntryWords * q) * stride, stride);
      base[(kEntryWords * q + CW::kN) * stride] = static_cast<uint32_t>(s[q]);
    }
  }
  __device__ __forceinline__ void merge(const uint32_t* base, int stride) {
#pragma unroll
    for (int q = 0; q < J; ++q)
      queue_push_ranked<J, FIRST>(v, s, CW::get(base + (kEntryWords * q) * stride, stride),
                                  static_cast<int>(base[(kEntryWords * q + CW::kN) * stride]));
  }

  __device__ __forceinline__ long long stripe(int q) const { return s[q]; }
  // value bits for the output (`elem` is unused: the compute value is exact)
  __device__ __forceinline__ typename Tr::Bits value_bits(int q, const T*) const { return Tr::narrow(v[q]); }
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

// The 32-bit words of a vector load of 16-bit elements (two columns per word).
__device__ __forceinline__ void raw_words(const uint4& r, uint32_t (&w)[4]) {
  w[0] = r.x; w[1] = r.y; w[2] = r.z; w[3] = r.w;
}
__device__ __forceinline__ void raw_words(const uint2& r, uint32_t (&w)[2]) {
  w[0] = r.x; w[1] = r.y;
}

__device__ __forceinline__ void raw_words(const uint32_t& r, uint32_t (&w)[1]) { w[0] = r; }

// Order-preserving unsigned image of the elements packed in one 32-bit word
// (two 16-bit or four 8-bit elements), and the way back for one element.
template <typename T> struct PackedImage;
template <> struct PackedImage<__half> {
  static constexpr int kBits = 16;
  static __device__ __forceinline__ uint32_t word(uint32_t w) { return ord16x2(w); }
  // Both zeros share one image; the element itself is read back to return the
  // sign the input had (a load that almost never executes).  `elem` is null when
  // the values were never in memory (fused score producer): +0 is returned then.
  static __device__ __forceinline__ uint16_t inverse(uint32_t o, const __half* elem) {
    if (o == 0x8000u) return elem != nullptr ? ld_stream_2(elem) : uint16_t(0);
    return ord16_inverse(o);
  }
};
template <> struct PackedImage<__nv_bfloat16> {
  static constexpr int kBits = 16;
  static __device__ __forceinline__ uint32_t word(uint32_t w) { return ord16x2(w); }
  static __device__ __forceinline__ uint16_t inverse(uint32_t o, const __nv_bfloat16* elem) {
    if (o == 0x8000u) return elem != nullptr ? ld_stream_2(elem) : uint16_t(0);
    return ord16_inverse(o);
  }
};
template <> struct PackedImage<int16_t> {
  static constexpr int kBits = 16;
  static __device__ __forceinline__ uint32_t word(uint32_t w) { return w ^ 0x80008000u; }
  static __device__ __forceinline__ uint16_t inverse(uint32_t o, const int16_t*) { return static_cast<uint16_t>(o ^ 0x8000u); }
};
template <> struct PackedImage<int8_t> {
  static constexpr int kBits = 8;
  static __device__ __forceinline__ uint32_t word(uint32_t w) { return w ^ 0x80808080u; }
  static __device__ __forceinline__ uint8_t inverse(uint32_t o, const int8_t*) { return static_cast<uint8_t>(o ^ 0x80u); }
};
template <> struct PackedImage<uint8_t> {
  static constexpr int kBits = 8;
  static __device__ __forceinline__ uint32_t word(uint32_t w) { return w; }
  static __device__ __forceinline__ uint8_t inverse(uint32_t o, const uint8_t*) { return static_cast<uint8_t>(o); }
};

// Entry = (image of the value) << kShift | stripe, kShift = 32 - bits of the
// element: 65536 stripes for 16-bit elements, 2^24 for 8-bit ones.  Entry 0
// means "never filled"; for the integer types it is also the entry of the
// lowest value at stripe 0, and an empty slot decodes to exactly that element,
// which is the right answer whenever the slot has to be reported (a bucket
// holds at least J elements).
template <typename T, int J, bool FIRST>
struct PackedQueue {
  static_assert(sizeof(T) <= 2, "packed queues are for 8- and 16-bit element types");
  using Img = PackedImage<T>;
  static constexpr int kBits = Img::kBits;
  static constexpr int kShift = 32 - kBits;
  static constexpr uint32_t kStripeMask = (1u << kShift) - 1u;
  static constexpr long long kMaxStripes = 1ll << kShift;
  static constexpr int kPerWord = 32 / kBits;       // elements per 32-bit word of a vector load
  static constexpr int kWords = J;
  static constexpr bool kPacked = true;
  static constexpr int kCols = 1;
  static constexpr int kJ = J;
  static constexpr bool kFirst = FIRST;
  uint32_t k[J];  // ascending; 0 = never filled

  __device__ __forceinline__ void init() {
#pragma unroll
    for (int q = 0; q < J; ++q) k[q] = 0u;
  }

  // With FIRST the earlier position must win a tie, so the low part holds the
  // complement of the stripe number.
  static __device__ __forceinline__ uint32_t low(int stripe) {
    return FIRST ? (kStripeMask - static_cast<uint32_t>(stripe)) : static_cast<uint32_t>(stripe);
  }

  __device__ __forceinline__ void push(uint32_t key) {
    uint32_t n[J];
#pragma unroll
    for (int q = 0; q + 1 < J; ++q) n[q] = min(max(key, k[q]), k[q + 1]);
    n[J - 1] = max(key, k[J - 1]);
#pragma unroll
    for (int q = 0; q < J; ++q) k[q] = n[q];
  }

  // entry of element `e` (0 = lowest address) of an image word
  static __device__ __forceinline__ uint32_t key_of(uint32_t image_word, int e, uint32_t lo) {
    return ((image_word << (kShift - kBits * e)) & ~kStripeMask) | lo;
  }

  template <int V, bool SKIP>
  static __device__ __forceinline__ void consume(PackedQueue (&q)[V], const typename VecLoad<T, V>::Raw& raw,
                                                 int stripe) {
    const uint32_t lo = low(stripe);
    if constexpr (V == 1) {
      const uint32_t key = key_of(Img::word(raw), 0, lo);
      if (!SKIP || key > q[0].k[0]) q[0].push(key);
    } else {
      uint32_t w[V / kPerWord];
      raw_words(raw, w);
      uint32_t key[V];
#pragma unroll
      for (int i = 0; i < V / kPerWord; ++i) {
        const uint32_t o = Img::word(w[i]);
#pragma unroll
        for (int e = 0; e < kPerWord; ++e) key[kPerWord * i + e] = key_of(o, e, lo);
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

  __device__ __forceinline__ void push_tail(typename ElemTraits<T>::Bits bits, int stripe) {
    push(key_of(Img::word(bits), 0, low(stripe)));
  }

  __device__ __forceinline__ void store(uint32_t* base, int stride) const {
#pragma unroll
    for (int q = 0; q < J; ++q) base[q * stride] = k[q];
  }
  __device__ __forceinline__ void merge(const uint32_t* base, int stride) {
#pragma unroll
    for (int q = 0; q < J; ++q) push(base[q * stride]);
  }

  __device__ __forceinline__ long long stripe(int q) const {
    const uint32_t l = k[q] & kStripeMask;
    return FIRST ? (kStripeMask - l) : l;
  }
  __device__ __forceinline__ typename ElemTraits<T>::Bits value_bits(int q, const T* elem) const {
    return Img::inverse(k[q] >> kShift, elem);
  }
};


// ---------------------------------------------------------------- Simd16Queue
// Scan-time layout for 16-bit inputs on the vector path: one queue serves TWO
// adjacent columns, values kept as raw fp16x2 / bf16x2 words and stripes as
// 16-bit pairs.  The J compares and 2J-1 min/max of an insertion are packed
// half-precision instructions that work on both columns at once (and issue on
// the FMA pipe), the stripe moves are bitwise selects under the compare masks.
// Elements arrive in increasing stripe order, so `>=` lets the later element
// pass equal ones (LAST wins) and `>` keeps the earlier one (FIRST wins), the
// same rule as the reference's scan.  NaNs never enter.  After the scan the
// queues are converted to PackedQueue entries, which carry the merge across
// stripe splits and the write-out.
template <typename T> struct Half2Ops;
template <> struct Half2Ops<__nv_bfloat16> {
  using T2 = __nv_bfloat162;
  static constexpr uint32_t kNegInf2 = 0xff80ff80u;
  static __device__ __forceinline__ T2 as2(uint32_t w) { return *reinterpret_cast<T2*>(&w); }
  static __device__ __forceinline__ uint32_t bits(T2 v) { return *reinterpret_cast<uint32_t*>(&v); }
  static __device__ __forceinline__ uint32_t max2(uint32_t a, uint32_t b) { return bits(__hmax2(as2(a), as2(b))); }
  static __device__ __forceinline__ uint32_t min2(uint32_t a, uint32_t b) { return bits(__hmin2(as2(a), as2(b))); }
  static __device__ __forceinline__ uint32_t ge(uint32_t a, uint32_t b) { return __hge2_mask(as2(a), as2(b)); }
  static __device__ __forceinline__ uint32_t gt(uint32_t a, uint32_t b) { return __hgt2_mask(as2(a), as2(b)); }
};
template <> struct Half2Ops<__half> {
  using T2 = __half2;
  static constexpr uint32_t kNegInf2 = 0xfc00fc00u;
  static __device__ __forceinline__ T2 as2(uint32_t w) { return *reinterpret_cast<T2*>(&w); }
  static __device__ __forceinline__ uint32_t bits(T2 v) { return *reinterpret_cast<uint32_t*>(&v); }
  static __device__ __forceinline__ uint32_t max2(uint32_t a, uint32_t b) { return bits(__hmax2(as2(a), as2(b))); }
  static __device__ __forceinline__ uint32_t min2(uint32_t a, uint32_t b) { return bits(__hmin2(as2(a), as2(b))); }
  static __device__ __forceinline__ uint32_t ge(uint32_t a, uint32_t b) { return __hge2_mask(as2(a), as2(b)); }
  static __device__ __forceinline__ uint32_t gt(uint32_t a, uint32_t b) { return __hgt2_mask(as2(a), as2(b)); }
};

template <typename T, int J, bool FIRST>
struct Simd16Queue {
  static_assert(sizeof(T) == 2, "SIMD queues are for 16-bit element types");
  using Ops = Half2Ops<T>;
  static constexpr int kCols = 2;
  static constexpr int kWords = 2 * J;
  uint32_t v[J];  // value pairs, ascending per half; low half = even column
  uint32_t s[J];  // stripe pairs

  __device__ __forceinline__ void init() {
#pragma unroll
    for (int q = 0; q < J; ++q) {
      v[q] = Ops::kNegInf2;
      s[q] = 0u;
    }
  }

  static __device__ __forceinline__ uint32_t pass_mask(uint32_t x, uint32_t q) {
    return FIRST ? Ops::gt(x, q) : Ops::ge(x, q);
  }
  static __device__ __forceinline__ uint32_t sel(uint32_t m, uint32_t a, uint32_t b) { return (a & m) | (b & ~m); }

  // x: value pair, sp: stripe pair, m0: pass_mask(x, v[0]) already evaluated
  __device__ __forceinline__ void push(uint32_t x, uint32_t sp, uint32_t m0) {
    uint32_t m[J];
    m[0] = m0;
#pragma unroll
    for (int q = 1; q < J; ++q) m[q] = pass_mask(x, v[q]);
    uint32_t nv[J], ns[J];
#pragma unroll
    for (int q = 0; q + 1 < J; ++q) {
      nv[q] = Ops::min2(Ops::max2(x, v[q]), v[q + 1]);
      ns[q] = sel(m[q + 1], s[q + 1], sel(m[q], sp, s[q]));
    }
    nv[J - 1] = Ops::max2(x, v[J - 1]);
    ns[J - 1] = sel(m[J - 1], sp, s[J - 1]);
#pragma unroll
    for (int q = 0; q < J; ++q) {
      v[q] = nv[q];
      s[q] = ns[q];
    }
  }

  // One vector load of V columns feeds V/2 queues.
  template <int V, bool SKIP>
  static __device__ __forceinline__ void consume(Simd16Queue (&q)[V / 2], const typename VecLoad<T, V>::Raw& raw,
                                                 int stripe) {
    static_assert(V == 8 || V == 4, "the SIMD queues need a vector path");
    uint32_t w[V / 2];
    raw_words(raw, w);
    const uint32_t sp = static_cast<uint32_t>(stripe) * 0x00010001u;
    uint32_t m0[V / 2];
    uint32_t any = 0u;
#pragma unroll
    for (int i = 0; i < V / 2; ++i) {
      m0[i] = pass_mask(w[i], q[i].v[0]);
      any |= m0[i];
    }
    if (SKIP) {
      if (any == 0u) return;
    }
#pragma unroll
    for (int i = 0; i < V / 2; ++i) q[i].push(w[i], sp, m0[i]);
  }

  // Entry j of column `half` (0 = even column) as a PackedQueue key.
  __device__ __forceinline__ uint32_t packed_key(int j, int half) const {
    const uint32_t raw = half ? (v[j] >> 16) : (v[j] & 0xffffu);
    const uint32_t st = half ? (s[j] >> 16) : (s[j] & 0xffffu);
    return ((ord16x2(raw) & 0xffffu) << 16) | PackedQueue<T, J, FIRST>::low(static_cast<int>(st));
  }
};

}  // namespace atk
