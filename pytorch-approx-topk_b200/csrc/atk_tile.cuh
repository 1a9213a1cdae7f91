// Stage 1 scan for 16-bit float inputs with short columns: the "two-pass tile".
//
// The insertion queues of atk_queue.cuh cost about nine ALU-pipe operations per
// element at four entries per queue (compares, min/max and the selects that carry
// the stripe numbers), and that pipe issues 64 lanes per clock and SM: short
// columns (no head test to skip insertions) are bound by it, not by memory.
// Here a thread owns two adjacent columns (one 32-bit word per stripe) and sees
// a chunk of CH stripes of them, staged in shared memory by asynchronous copies,
// twice (tile_chunk_shared; holding the chunk in registers instead was measured
// slower: 156 registers leave too few warps to hide the load and the dependent
// min/max chains):
//   pass 1  finds the J-th largest VALUE of either column in the chunk with a
//           values-only network of packed fp16x2 / bf16x2 min/max (sorted batches
//           merged into a running sorted top-J: no stripe numbers are carried);
//   pass 2  compares every word of the chunk with that threshold pair and gathers
//           the outcome as one bit per (column, stripe);
//   then    only the elements at or above the threshold (J of CH unless values
//           tie) are turned into packed queue entries (value image, stripe) and
//           pushed into the exact per-column queues, which rank them by (value,
//           position) like every other path.
// Every element of the true top-J by (value, later position wins) is at or above
// the J-th largest value, so the exact queue receives a superset of the winners
// and the result is identical to the serial scan of the reference
// (approx_topk/priority_queue_approx_topk.cu:58-107), ties included.  NaNs never
// pass the threshold compare (the reference leaves them unspecified).
#pragma once

#include "atk_queue.cuh"

namespace atk {

template <typename Ops>
__device__ __forceinline__ void tile_ce(uint32_t& a, uint32_t& b) {
  const uint32_t lo = Ops::min2(a, b);
  const uint32_t hi = Ops::max2(a, b);
  a = lo;
  b = hi;
}

// Sorted (ascending per half) top-J of a running list and a new batch, J = 2 or 4.
template <typename Ops, int J> struct TileNet;

template <typename Ops> struct TileNet<Ops, 4> {
  static constexpr int kBatch = 4;
  static __device__ __forceinline__ void sort(uint32_t (&a)[4]) {
    tile_ce<Ops>(a[0], a[1]);
    tile_ce<Ops>(a[2], a[3]);
    tile_ce<Ops>(a[0], a[2]);
    tile_ce<Ops>(a[1], a[3]);
    tile_ce<Ops>(a[1], a[2]);
  }
  // t ascending, s ascending: the four largest of the eight form a bitonic list
  static __device__ __forceinline__ void upper(const uint32_t (&t)[4], const uint32_t (&s)[4], uint32_t (&u)[4]) {
    u[0] = Ops::max2(t[0], s[3]);
    u[1] = Ops::max2(t[1], s[2]);
    u[2] = Ops::max2(t[2], s[1]);
    u[3] = Ops::max2(t[3], s[0]);
  }
  static __device__ __forceinline__ void merge(uint32_t (&t)[4], const uint32_t (&s)[4]) {
    uint32_t u[4];
    upper(t, s, u);
    tile_ce<Ops>(u[0], u[2]);
    tile_ce<Ops>(u[1], u[3]);
    tile_ce<Ops>(u[0], u[1]);
    tile_ce<Ops>(u[2], u[3]);
#pragma unroll
    for (int i = 0; i < 4; ++i) t[i] = u[i];
  }
  // smallest of the merged top four = the 4th largest of both lists
  static __device__ __forceinline__ uint32_t merged_min(const uint32_t (&t)[4], const uint32_t (&s)[4]) {
    uint32_t u[4];
    upper(t, s, u);
    return Ops::min2(Ops::min2(u[0], u[1]), Ops::min2(u[2], u[3]));
  }
};

template <typename Ops> struct TileNet<Ops, 2> {
  static constexpr int kBatch = 2;
  static __device__ __forceinline__ void sort(uint32_t (&a)[2]) { tile_ce<Ops>(a[0], a[1]); }
  static __device__ __forceinline__ void merge(uint32_t (&t)[2], const uint32_t (&s)[2]) {
    uint32_t u0 = Ops::max2(t[0], s[1]);
    uint32_t u1 = Ops::max2(t[1], s[0]);
    tile_ce<Ops>(u0, u1);
    t[0] = u0;
    t[1] = u1;
  }
  static __device__ __forceinline__ uint32_t merged_min(const uint32_t (&t)[2], const uint32_t (&s)[2]) {
    return Ops::min2(Ops::max2(t[0], s[1]), Ops::max2(t[1], s[0]));
  }
};

template <typename Ops, int J, int CH>
__device__ __forceinline__ uint32_t tile_threshold_net(const uint32_t (&d)[CH]);

// J-th largest value per half among the CH words of d (values only).  Two
// independent running lists (even and odd batches) give the scheduler two chains
// to interleave; they are combined at the end.
template <typename Ops, int J, int CH>
__device__ __forceinline__ uint32_t tile_threshold(const uint32_t (&d)[CH]) {
  if constexpr (J == 1) {
    // one entry per queue: the largest value, a balanced tree of maxima
    uint32_t m[CH];
#pragma unroll
    for (int i = 0; i < CH; ++i) m[i] = d[i];
#pragma unroll
    for (int w = CH / 2; w >= 1; w /= 2)
#pragma unroll
      for (int i = 0; i < w; ++i) m[i] = Ops::max2(m[i], m[i + w]);
    return m[0];
  } else {
    return tile_threshold_net<Ops, J, CH>(d);
  }
}

template <typename Ops, int J, int CH>
__device__ __forceinline__ uint32_t tile_threshold_net(const uint32_t (&d)[CH]) {
  constexpr int N = (J == 3) ? 4 : J;          // three entries: the four-entry network, third largest
  using Net = TileNet<Ops, N>;
  constexpr int B = Net::kBatch;
  constexpr int NB = CH / B;
  static_assert(CH == B || (CH % (2 * B) == 0 && NB >= 2), "one batch, or an even number of batches");
  if constexpr (NB == 1) {
    uint32_t t[N];
#pragma unroll
    for (int i = 0; i < N; ++i) t[i] = d[i];
    Net::sort(t);
    return t[N - J];
  }
  uint32_t ta[N], tb[N];
#pragma unroll
  for (int i = 0; i < N; ++i) {
    ta[i] = d[i];
    tb[i] = d[(NB > 1 ? B : 0) + i];
  }
  Net::sort(ta);
  Net::sort(tb);
#pragma unroll
  for (int k = 2; k < NB; k += 2) {
    uint32_t sa[N], sb[N];
#pragma unroll
    for (int i = 0; i < N; ++i) {
      sa[i] = d[k * B + i];
      sb[i] = d[(k + 1) * B + i];
    }
    Net::sort(sa);
    Net::sort(sb);
    Net::merge(ta, sa);
    Net::merge(tb, sb);
  }
  if constexpr (J == 3) {
    Net::merge(ta, tb);
    return ta[1];
  } else {
    return Net::merged_min(ta, tb);
  }
}

// The two passes over a chunk that asynchronous copies staged in shared
// memory: `words` points at this thread's word of the chunk's first stripe,
// consecutive stripes are PITCH words apart (a warp reads consecutive words of a
// stripe: no bank conflicts).  `cnt` <= CH stripes exist (FULL: cnt == CH); stripe
// i of the chunk is stripe l_first + i of the column.  Few registers are live (the
// running lists of the network, the bit accumulators, the queues), so many blocks
// fit an SM and their copy, network and extraction phases overlap.
//
// Pass 1 here is cheaper than the full network: the stripes are cut into groups
// of kTileGroup, only the group maxima go through the network, and the J-th
// largest group maximum is the threshold.  It is at most the J-th largest value
// (J different groups each hold an element at or above it), so the elements at or
// above it are still a superset of the winners -- about 4.4 instead of 4 of 64 for
// independent values -- and the exact queues sort it out.
//
// Chunks after the first need no network at all: the queues are full by then and
// the value of their weakest entry -- the J-th largest of everything seen so far
// -- is a tighter threshold than anything local to the chunk.
template <int CH> struct TileGroup {
  // stripes per group: short chunks would let too many elements through with wide groups
  static constexpr int kSize = CH >= 64 ? 4 : (CH >= 32 ? 2 : 1);
};

template <typename T, int J, int CH, int PITCH, bool FULL, bool FIRST_CHUNK>
__device__ __forceinline__ void tile_chunk_shared(PackedQueue<T, J, false> (&q)[2], const uint32_t* words, int cnt,
                                                  int l_first) {
  using Ops = Half2Ops<T>;
  using PQ = PackedQueue<T, J, false>;
  using Img = PackedImage<T>;
  auto word = [&](int i) -> uint32_t { return (FULL || i < cnt) ? words[i * PITCH] : Ops::kNegInf2; };
  uint32_t thr;
  if constexpr (FIRST_CHUNK) {
    // pass 1: maxima of groups of stripes, then the J-th largest of them
    constexpr int kGroup = TileGroup<CH>::kSize;
    constexpr int G = CH / kGroup;
    uint32_t gmax[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      uint32_t m = word(g * kGroup);
#pragma unroll
      for (int e = 1; e < kGroup; ++e) m = Ops::max2(m, word(g * kGroup + e));
      gmax[g] = m;
    }
    thr = tile_threshold<Ops, J, G>(gmax);
  } else {
    // the weakest entries of the two queues, as a value pair (-inf while a queue
    // is not full, which only NaNs in the first chunk can cause)
    uint32_t v[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t k0 = q[h].k[0];
      v[h] = k0 != 0u ? static_cast<uint32_t>(ord16_inverse(k0 >> PQ::kShift)) : (Ops::kNegInf2 & 0xffffu);
    }
    thr = v[0] | (v[1] << 16);
  }
  // pass 2: one bit per (column, stripe)
  constexpr int NA = CH / 16;
  uint32_t acc[NA];
#pragma unroll
  for (int a = 0; a < NA; ++a) acc[a] = 0u;
#pragma unroll
  for (int i = 0; i < CH; ++i) acc[i / 16] |= Ops::ge(word(i), thr) & (0x00010001u << (i % 16));
  constexpr int NW = CH >= 32 ? CH / 32 : 1;
  const uint16_t* halves = reinterpret_cast<const uint16_t*>(words);
#pragma unroll
  for (int h = 0; h < 2; ++h) {
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      uint32_t m;
      if constexpr (CH >= 32) m = __byte_perm(acc[2 * w], acc[2 * w + 1], h ? 0x7632 : 0x5410);
      else m = h ? (acc[0] >> 16) : (acc[0] & 0xffffu);
      if (!FULL) {
        const int live = cnt - 32 * w;
        m = live >= 32 ? m : (live <= 0 ? 0u : (m & ((1u << live) - 1u)));
      }
      while (m != 0u) {
        const int bit = 31 - __clz(m);
        m ^= 1u << bit;
        const int i = 32 * w + bit;
        const uint32_t vb = halves[2 * i * PITCH + h];
        const uint32_t key = PQ::key_of(Img::word(vb), 0, PQ::low(l_first + i));
        if (key > q[h].k[0]) q[h].push(key);
      }
    }
  }
}

// ---- float32 columns ---------------------------------------------------------
// The same two passes for float32, one column per thread (one word per stripe).
// What it buys here is different: long columns that are split over many blocks.
// With insertion queues a warp runs the whole insertion network whenever any of
// its 128 columns takes an element, which is at almost every stripe for the first
// few hundred stripes of every split; here the threshold compare costs the same
// at every stripe and only real candidates reach the queue.
struct FloatWordOps {
  static constexpr uint32_t kNegInf2 = 0xff800000u;
  static __device__ __forceinline__ uint32_t max2(uint32_t a, uint32_t b) {
    return __float_as_uint(fmaxf(__uint_as_float(a), __uint_as_float(b)));
  }
  static __device__ __forceinline__ uint32_t min2(uint32_t a, uint32_t b) {
    return __float_as_uint(fminf(__uint_as_float(a), __uint_as_float(b)));
  }
};

template <int J, int CH, int PITCH, bool FULL, bool FIRST_CHUNK>
__device__ __forceinline__ void tile_chunk_shared_f32(FloatQueue<float, J, false>& q, const uint32_t* words, int cnt,
                                                      int l_first) {
  using Ops = FloatWordOps;
  auto word = [&](int i) -> uint32_t { return (FULL || i < cnt) ? words[i * PITCH] : Ops::kNegInf2; };
  float thr;
  if constexpr (FIRST_CHUNK) {
    constexpr int kGroup = TileGroup<CH>::kSize;
    constexpr int G = CH / kGroup;
    uint32_t gmax[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      uint32_t m = word(g * kGroup);
#pragma unroll
      for (int e = 1; e < kGroup; ++e) m = Ops::max2(m, word(g * kGroup + e));
      gmax[g] = m;
    }
    thr = __uint_as_float(tile_threshold<Ops, J, G>(gmax));
  } else {
    thr = q.v[0];        // the J-th largest value so far (-inf while the queue is not full)
  }
  constexpr int NW = CH / 32 > 0 ? CH / 32 : 1;
  uint32_t acc[NW];
#pragma unroll
  for (int w = 0; w < NW; ++w) acc[w] = 0u;
#pragma unroll
  for (int i = 0; i < CH; ++i) acc[i / 32] |= (__uint_as_float(word(i)) >= thr) ? (1u << (i % 32)) : 0u;
#pragma unroll
  for (int w = 0; w < NW; ++w) {
    uint32_t m = acc[w];
    if (!FULL) {
      const int live = cnt - 32 * w;
      m = live >= 32 ? m : (live <= 0 ? 0u : (m & ((1u << live) - 1u)));
    }
    while (m != 0u) {
      const int bit = 31 - __clz(m);
      m ^= 1u << bit;
      const int i = 32 * w + bit;
      const float v = __uint_as_float(words[i * PITCH]);
      if (v >= q.v[0]) queue_push_ranked<J, false>(q.v, q.s, v, l_first + i);
    }
  }
}

}  // namespace atk
