// Stage 2: exact top-k of the k0 stage-1 candidates of every row, indices
// carried along.  Replaces torch.topk(sorted=False) + gather of the reference
// (approx_topk/priority_queue.py:85-88).
//
// Method: MSB-first radix select on an order-preserving integer image of the
// value finds the k-th largest key T and how many candidates equal to T are
// still needed; an ordered compaction then writes every candidate above T
// followed by the first `need` candidates equal to T, both in candidate-slot
// order, so the result is deterministic.
//
//  * small rows (k0 <= kSmallMaxK0): one block per row, keys live in
//    registers, a single launch;
//  * large rows: several blocks per row; digit histograms, block counts and
//    the running (prefix, need) state live in a caller-provided workspace.
#include <atomic>
#include <type_traits>

#include "atk_select.cuh"
#include "atk_block_select.cuh"
#include "atk_queue.cuh"

namespace atk {
namespace {

constexpr int kSmallMaxK0 = 16384;   // 512 threads x 32 candidates in registers (32-bit keys)
constexpr int kChunk = 2048;         // candidates per block on the large path
constexpr int kLargeThreads = 256;
// Vector loads a thread keeps in flight before it starts computing in the
// histogram kernel of the multi-block path (a build knob; more cost registers
// and with them resident blocks).
// Resident blocks the compiler must allow for in the packed-entry select with at
// most eight entries per thread (2 and 3 measured alike on 1024 rows x 4096 entries,
// 65-66 us for the whole operator; leaving it to the compiler cost 10 us).
#ifndef ATK_SELECT_PACKED_MINBLOCKS
#define ATK_SELECT_PACKED_MINBLOCKS 2
#endif
// Counts of the chunks chained inside the write kernel (1), by a count pass (0), or
// by the shape (-1); a build knob for measurements.
#ifndef ATK_SELECT_CHAINED
#define ATK_SELECT_CHAINED -1
#endif
#ifndef ATK_HIST_BATCH
#define ATK_HIST_BATCH 2
#endif
#ifndef ATK_SELECT_ROW_THREADS
#define ATK_SELECT_ROW_THREADS 512
#endif
constexpr int kSelectRowThreads = ATK_SELECT_ROW_THREADS;
// Resident blocks the compiler must allow for in the variants with at most eight
// candidates per thread (a build knob for measurements).
#ifndef ATK_SELECT_ROW_MINBLOCKS
#define ATK_SELECT_ROW_MINBLOCKS 1
#endif  // preferred block width of the one-block-per-row select

// Order-preserving unsigned image of an element ("key"), its width, and the
// number of 8-bit radix passes, most significant digit first.  Keys of the
// types of 32 bits or fewer sit in the top bits of a 32-bit word; the 64-bit
// types use 64-bit keys.
template <typename T> struct KeyOf;
template <> struct KeyOf<float> {
  using Key = uint32_t;
  static constexpr int kPasses = 4;
  // negative: all bits flipped; positive: sign bit set (shift, then one logic op)
  static __device__ __forceinline__ Key key(uint32_t u) {
    const uint32_t s = static_cast<uint32_t>(static_cast<int32_t>(u) >> 31);
    return u ^ (s | 0x80000000u);
  }
};
template <> struct KeyOf<__half> {
  using Key = uint32_t;
  static constexpr int kPasses = 2;
  // the same on the 16 bits moved to the top half; the low half stays zero
  static __device__ __forceinline__ Key key(uint16_t h) {
    const uint32_t x = static_cast<uint32_t>(h) << 16;
    const uint32_t s = static_cast<uint32_t>(static_cast<int32_t>(x) >> 31);
    return x ^ ((s & 0x7fff0000u) | 0x80000000u);
  }
};
template <> struct KeyOf<__nv_bfloat16> {
  using Key = uint32_t;
  static constexpr int kPasses = 2;
  static __device__ __forceinline__ Key key(uint16_t h) { return KeyOf<__half>::key(h); }
};
template <> struct KeyOf<double> {
  using Key = unsigned long long;
  static constexpr int kPasses = 8;
  static __device__ __forceinline__ Key key(unsigned long long u) {
    const unsigned long long s = static_cast<unsigned long long>(static_cast<long long>(u) >> 63);
    return u ^ (s | 0x8000000000000000ull);
  }
};
template <> struct KeyOf<int32_t> {
  using Key = uint32_t;
  static constexpr int kPasses = 4;
  static __device__ __forceinline__ Key key(uint32_t u) { return u ^ 0x80000000u; }
};
template <> struct KeyOf<long long> {
  using Key = unsigned long long;
  static constexpr int kPasses = 8;
  static __device__ __forceinline__ Key key(unsigned long long u) { return u ^ 0x8000000000000000ull; }
};
template <> struct KeyOf<int16_t> {
  using Key = uint32_t;
  static constexpr int kPasses = 2;
  static __device__ __forceinline__ Key key(uint16_t u) { return (static_cast<uint32_t>(u) ^ 0x8000u) << 16; }
};
template <> struct KeyOf<int8_t> {
  using Key = uint32_t;
  static constexpr int kPasses = 1;
  static __device__ __forceinline__ Key key(uint8_t u) { return (static_cast<uint32_t>(u) ^ 0x80u) << 24; }
};
template <> struct KeyOf<uint8_t> {
  using Key = uint32_t;
  static constexpr int kPasses = 1;
  static __device__ __forceinline__ Key key(uint8_t u) { return static_cast<uint32_t>(u) << 24; }
};
// shift of the digit examined in `pass`
template <typename K> __device__ __forceinline__ int digit_shift(int pass) {
  return static_cast<int>(sizeof(typename K::Key)) * 8 - 8 - 8 * pass;
}

// Digits of the multi-block path.  Elements of 32 bits are cut into digits of
// 11 + 11 + 10 bits (three passes over the candidates instead of four, and 2048
// bins spread the shared-memory atomics of float keys, whose leading bits are
// badly skewed); the other widths keep one pass per byte.
template <typename T> struct LargeDigits {
  using K = KeyOf<T>;
  static constexpr bool kWide = sizeof(T) == 4;
  static constexpr int kPasses = kWide ? 3 : K::kPasses;
  static constexpr int kBins = kWide ? 2048 : 256;
  static __host__ __device__ constexpr int width(int pass) { return kWide ? (pass < 2 ? 11 : 10) : 8; }
  static __host__ __device__ constexpr int shift(int pass) {
    return kWide ? (pass == 0 ? 21 : (pass == 1 ? 10 : 0))
                 : static_cast<int>(sizeof(typename K::Key)) * 8 - 8 - 8 * pass;
  }
};

// ITEMS consecutive raw candidates of one thread, loaded with the widest
// vector loads their size allows (16 bytes at a time).
template <typename B, int ITEMS>
struct alignas((ITEMS * sizeof(B)) % 16 == 0 ? 16 : 8) ItemPack {
  B v[ITEMS];
};
static_assert(sizeof(ItemPack<uint16_t, 8>) == 16 && sizeof(ItemPack<uint8_t, 8>) == 8, "pack layout");

// Loads slots [first, first + ITEMS) of a row into raw[]; slots at or past
// `end` read as zero.  `vec` says the row is aligned for vector loads.
template <typename B, int ITEMS>
__device__ __forceinline__ void load_items(const B* __restrict__ row, long long first, long long end, int vec,
                                           B (&raw)[ITEMS]) {
  if (vec && first + ITEMS <= end) {
    const ItemPack<B, ITEMS> pk = *reinterpret_cast<const ItemPack<B, ITEMS>*>(row + first);
#pragma unroll
    for (int u = 0; u < ITEMS; ++u) raw[u] = pk.v[u];
  } else {
#pragma unroll
    for (int u = 0; u < ITEMS; ++u) raw[u] = first + u < end ? row[first + u] : B(0);
  }
}

template <typename KEY>
struct RowState {
  KEY prefix, mask;
  uint32_t need;
  uint32_t gave_up;   // set when a bounded wait of the write kernel ran out (never seen; the row's output is then invalid)
};

// ---- write-out through shared memory ------------------------------------------
// Winners leave a thread at scattered output positions (a thread owns a run of
// candidate slots, only some of which win), which costs one memory sector per
// element when stored directly.  Instead the block collects a tile of
// kStageTile consecutive output positions in shared memory and then copies the
// tile out with fully coalesced (16-byte where aligned) stores.
constexpr int kStageTile = 2048;
// Staging buffer of a block that writes at most `k` entries: the positions of
// one tile, then (16-byte aligned) its values.
__host__ __device__ inline int stage_tile(long long k) { return k < kStageTile ? static_cast<int>(k) : kStageTile; }
__host__ __device__ inline size_t stage_val_offset(int tile) { return (static_cast<size_t>(tile) * 8 + 15) & ~static_cast<size_t>(15); }
template <typename B> size_t stage_bytes(long long k) {
  return stage_val_offset(stage_tile(k)) + static_cast<size_t>(stage_tile(k)) * sizeof(B);
}
// The packed hand-off stages one (entry, slot) pair of words per output position.
inline size_t packed_stage_bytes(long long k) { return static_cast<size_t>(stage_tile(k)) * sizeof(uint2); }

// Copies staged entries [0, cnt) to the output row `o` (already advanced to the
// first destination slot); all threads of the block take part.  `vec`: the
// destinations start on a 16-byte boundary (used by the int64 layout, whose
// positions are 2/3 of the bytes; the narrow formats store element-wise, which
// is just as coalesced).
template <typename B>
__device__ __forceinline__ void stage_copy_out(const long long* sidx, const B* sval, int cnt, const OutRow<B>& o,
                                               int tid, int nthr, bool vec) {
  if (o.fmt != ATK_OUT_I64) {
    for (int p = tid; p < cnt; p += nthr) o.put(p, sval[p], sidx[p]);
    return;
  }
  B* __restrict__ ov = o.v;
  long long* __restrict__ oi = static_cast<long long*>(o.i);
  if (vec) {
    const int ni = cnt / 2;                                   // 16-byte pieces of positions
    for (int q = tid; q < ni; q += nthr) reinterpret_cast<uint4*>(oi)[q] = reinterpret_cast<const uint4*>(sidx)[q];
    for (int p = 2 * ni + tid; p < cnt; p += nthr) oi[p] = sidx[p];
    constexpr int kPer = 16 / static_cast<int>(sizeof(B));
    const int nv = cnt / kPer;
    for (int q = tid; q < nv; q += nthr) reinterpret_cast<uint4*>(ov)[q] = reinterpret_cast<const uint4*>(sval)[q];
    for (int p = nv * kPer + tid; p < cnt; p += nthr) ov[p] = sval[p];
  } else {
    for (int p = tid; p < cnt; p += nthr) {
      oi[p] = sidx[p];
      ov[p] = sval[p];
    }
  }
}

// ------------------------------------------------------------------ small path
// One block per row.  Thread t owns the ITEMS consecutive candidate slots
// [t*ITEMS, (t+1)*ITEMS): keys stay in registers through the radix passes, and
// because slots are blocked per thread one block-wide scan of the per-thread
// (greater, equal) counts gives every winner its output position in slot order.
// FULL: the row has exactly blockDim.x * ITEMS candidates and is aligned for
// vector loads, so no slot needs a bounds test (the common case: candidate
// counts are powers of two).
template <typename T, int ITEMS, int MAXT, bool FULL>
__global__ void __launch_bounds__(MAXT, (ITEMS <= 8 && MAXT == 512) ? ATK_SELECT_ROW_MINBLOCKS : 1)
select_row_kernel(const typename ElemTraits<T>::Bits* __restrict__ cand_vals,
                  const long long* __restrict__ cand_idx, int k0, long long cand_row_stride, int k,
                  void* __restrict__ out_vals, void* __restrict__ out_idx, long long out_row_stride, int out_fmt,
                  int vec_ok) {
  using K = KeyOf<T>;
  using Key = typename K::Key;
  using Bits = typename ElemTraits<T>::Bits;
  __shared__ __align__(16) uint32_t hist[256 * K::kPasses];
  __shared__ uint32_t misc[2];
  __shared__ uint32_t wsum[32];

  const int tid = threadIdx.x;
  const int nthr = blockDim.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const long long row = blockIdx.x;
  const Bits* vrow = cand_vals + row * cand_row_stride;
  const long long* irow = cand_idx + row * cand_row_stride;
  const int slot0 = tid * ITEMS;
  for (int i = tid; i < 256 * K::kPasses; i += nthr) hist[i] = 0;
  // number of this thread's slots that exist
  int valid = ITEMS;
  if (!FULL) {
    valid = k0 - slot0;
    valid = valid < 0 ? 0 : (valid > ITEMS ? ITEMS : valid);
  }
  const bool vec = FULL || (vec_ok && valid == ITEMS);

  Bits raw[ITEMS];
  load_items<Bits, ITEMS>(vrow, slot0, slot0 + valid, vec, raw);
  // The positions travel with their candidates.  For short per-thread runs
  // they are fetched up front with the values (contiguous, 16-byte loads), so
  // the write-out at the end does not wait on a chain of dependent gathers.
  constexpr bool kPrefetchIdx = ITEMS <= 8;
  long long pidx[kPrefetchIdx ? ITEMS : 1];
  if constexpr (kPrefetchIdx) load_items<long long, ITEMS>(irow, slot0, slot0 + valid, vec, pidx);
  Key key[ITEMS];
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) key[i] = K::key(raw[i]);
  __syncthreads();   // histograms are clear

  Key prefix = 0, mask = 0;
  uint32_t need = static_cast<uint32_t>(k);
  // One histogram per pass, all cleared up front (under the latency of the
  // loads above): two block barriers per pass instead of three.  (Letting every
  // warp pick the digit for itself saves one more barrier but measured slower
  // when the rows fill the GPU.)  Up to four passes are unrolled so that shifts
  // are immediates and the first pass has no prefix test; the eight passes of
  // 64-bit keys stay a loop.
#pragma unroll(K::kPasses <= 4 ? K::kPasses : 1)
  for (int pass = 0; pass < K::kPasses; ++pass) {
    const int shift = digit_shift<K>(pass);
    uint32_t* h = hist + 256 * pass;
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      bool in = FULL || i < valid;
      if (pass > 0) in = in && (key[i] & mask) == prefix;
      if (in) atomicAdd(&h[static_cast<uint32_t>(key[i] >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (warp == 0) {
      uint32_t digit, new_need;
      pick_digit_all(h, need, lane, digit, new_need);
      if (lane == 0) {
        misc[0] = digit;
        misc[1] = new_need;
      }
    }
    __syncthreads();
    prefix |= static_cast<Key>(misc[0]) << shift;
    mask |= static_cast<Key>(255u) << shift;
    need = misc[1];
  }

  // per-thread counts, then one block-wide exclusive scan of (greater | equal << 16)
  uint32_t mine = 0;
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    const bool in = FULL || i < valid;
    mine += (in && key[i] > prefix) ? 1u : 0u;
    mine += (in && key[i] == prefix) ? 0x10000u : 0u;
  }
  uint32_t incl = mine;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const uint32_t nb = __shfl_up_sync(0xffffffffu, incl, off);
    if (lane >= off) incl += nb;
  }
  if (lane == 31) wsum[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    const int nwarps = (nthr + 31) >> 5;
    const uint32_t w = lane < nwarps ? wsum[lane] : 0u;
    uint32_t wi = w;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const uint32_t nb = __shfl_up_sync(0xffffffffu, wi, off);
      if (lane >= off) wi += nb;
    }
    wsum[lane] = wi - w;  // exclusive prefix of the warp totals
  }
  __syncthreads();
  const uint32_t excl = wsum[warp] + incl - mine;
  uint32_t gt_rank = excl & 0xffffu;
  uint32_t eq_rank = excl >> 16;
  const uint32_t n_gt = static_cast<uint32_t>(k) - need;
  const OutRow<Bits> orow(out_vals, out_idx, row, out_row_stride, out_fmt);
  // output position of every item (-1: not selected)
  int pos[ITEMS];
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    pos[i] = -1;
    if (FULL || i < valid) {
      if (key[i] > prefix) {
        pos[i] = static_cast<int>(gt_rank++);
      } else if (key[i] == prefix) {
        if (eq_rank < need) pos[i] = static_cast<int>(n_gt + eq_rank);
        ++eq_rank;
      }
    }
  }
  // Winners go to shared memory at their output position, one tile of output
  // positions at a time, and leave it with coalesced stores.
  extern __shared__ __align__(16) unsigned char stage_smem[];
  long long* sidx = reinterpret_cast<long long*>(stage_smem);
  const int tile = stage_tile(k);
  Bits* sval = reinterpret_cast<Bits*>(stage_smem + stage_val_offset(tile));
  const bool vec_out = orow.aligned16();
  for (int base = 0; base < k; base += tile) {
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      // pos - base in [0, tile) as one unsigned compare; -1 never passes
      const uint32_t rel = static_cast<uint32_t>(pos[i] - base);
      if (pos[i] >= 0 && rel < static_cast<uint32_t>(tile)) {
        sval[rel] = raw[i];
        sidx[rel] = kPrefetchIdx ? pidx[kPrefetchIdx ? i : 0] : irow[slot0 + i];
      }
    }
    __syncthreads();
    const int cnt = k - base < tile ? k - base : tile;
    stage_copy_out<Bits>(sidx, sval, cnt, orow.at(base), tid, nthr, vec_out);
    if (base + tile < k) __syncthreads();
  }
}

// ------------------------------------------------- small path, packed hand-off
// Same selection as select_row_kernel on the packed queue entries of stage 1:
// the top bits of an entry are the order-preserving image of the value (the
// radix digits), the low bits the stripe.  Nothing but the entries is read;
// value bits and positions are rebuilt for the winners only.
// Resident blocks the packed kernel is compiled for: what the register file holds at the
// register count a run of ITEMS entries per thread needs without spilling.
constexpr int packed_min_blocks(int items, int maxt) {
  const int regs = items <= 4 ? 40 : (items <= 8 ? 48 : (items <= 16 ? 64 : 96));
  const int blocks = 65536 / (maxt * regs);
  return blocks < 1 ? 1 : (blocks > 8 ? 8 : blocks);
}

template <typename T, int ITEMS, int MAXT, bool FULL>
__global__ void __launch_bounds__(MAXT, packed_min_blocks(ITEMS, MAXT))
select_row_packed_kernel(const uint32_t* __restrict__ keys, int k0, int k, const T* __restrict__ x,
                         long long x_row_stride, long long b, int j,
                         void* __restrict__ out_vals, void* __restrict__ out_idx, long long out_row_stride,
                         int out_fmt, int vec_ok) {
  using Bits = typename ElemTraits<T>::Bits;
  using PQ = PackedQueue<T, 1, false>;
  using Img = PackedImage<T>;
  constexpr int kPasses = PQ::kBits / 8;
  constexpr uint32_t kValMask = ~PQ::kStripeMask;
  __shared__ __align__(16) uint32_t hist[256 * kPasses];
  __shared__ uint32_t misc[2];
  __shared__ uint32_t wsum[32];

  const int tid = threadIdx.x;
  const int nthr = blockDim.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const long long row = blockIdx.x;
  const uint32_t* krow = keys + row * k0;
  const int slot0 = tid * ITEMS;
  for (int i = tid; i < 256 * kPasses; i += nthr) hist[i] = 0;
  int valid = ITEMS;
  if (!FULL) {
    valid = k0 - slot0;
    valid = valid < 0 ? 0 : (valid > ITEMS ? ITEMS : valid);
  }
  uint32_t key[ITEMS];
  grid_dependency_wait();   // the entries are stage 1's output; everything above overlapped its last blocks
  load_items<uint32_t, ITEMS>(krow, slot0, slot0 + valid, FULL || (vec_ok && valid == ITEMS), key);
  __syncthreads();   // histograms are clear

  uint32_t prefix = 0, mask = 0;
  uint32_t need = static_cast<uint32_t>(k);
#pragma unroll
  for (int pass = 0; pass < kPasses; ++pass) {
    const int shift = 24 - 8 * pass;
    uint32_t* h = hist + 256 * pass;
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      bool in = FULL || i < valid;
      if (pass > 0) in = in && (key[i] & mask) == prefix;
      if (in) atomicAdd(&h[(key[i] >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (warp == 0) {
      uint32_t digit, new_need;
      pick_digit_all(h, need, lane, digit, new_need);
      if (lane == 0) {
        misc[0] = digit;
        misc[1] = new_need;
      }
    }
    __syncthreads();
    prefix |= misc[0] << shift;
    mask |= 255u << shift;
    need = misc[1];
  }

  // Ranking needs no unpacking: an entry is above the threshold value exactly when it
  // is above the threshold's largest entry (all stripe bits set), and on or above it
  // when it is at least the threshold's smallest entry.  Slots past the end of a ragged
  // row hold entry 0; they are the last slots of the row, so even when they tie with the
  // threshold every real tie is ranked before them and takes the places there are.
  const uint32_t top = prefix | PQ::kStripeMask;
  uint32_t n_above = 0, n_from = 0;
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    n_above += key[i] > top ? 1u : 0u;
    n_from += key[i] >= prefix ? 1u : 0u;
  }
  const uint32_t mine = n_above + ((n_from - n_above) << 16);
  uint32_t incl = mine;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const uint32_t nb = __shfl_up_sync(0xffffffffu, incl, off);
    if (lane >= off) incl += nb;
  }
  if (lane == 31) wsum[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    const int nwarps = (nthr + 31) >> 5;
    const uint32_t w = lane < nwarps ? wsum[lane] : 0u;
    uint32_t wi = w;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const uint32_t nb = __shfl_up_sync(0xffffffffu, wi, off);
      if (lane >= off) wi += nb;
    }
    wsum[lane] = wi - w;
  }
  __syncthreads();
  const uint32_t excl = wsum[warp] + incl - mine;
  const uint32_t n_gt = static_cast<uint32_t>(k) - need;
  // Winners go to shared memory as (entry, slot) at their output position, one tile of
  // output positions at a time.  Value bits and positions are rebuilt from there by the
  // thread that stores them, so that work runs once per winner with the warp converged,
  // and every store is coalesced.
  const OutRow<Bits> orow(out_vals, out_idx, row, out_row_stride, out_fmt);
  const T* xrow = x + row * x_row_stride;
  // slot s belongs to bucket s / j: slots are below 2^13 and j is at most 4, so one
  // multiplication by ceil(2^16 / j) and a shift divide exactly (for j = 3 the error
  // of the reciprocal, 1e-5 per slot, stays far below the 1/3 that would change a floor)
  const uint32_t recip_j = (65536u + static_cast<uint32_t>(j) - 1u) / static_cast<uint32_t>(j);
  const uint32_t b32 = static_cast<uint32_t>(b);                       // buckets per row: at most k0
  extern __shared__ __align__(16) unsigned char stage_smem[];
  uint2* staged = reinterpret_cast<uint2*>(stage_smem);
  const uint32_t tile = static_cast<uint32_t>(stage_tile(k));
  auto rebuild = [&](uint2 e, Bits& value, long long& at) {
    const uint32_t bucket = (e.y * recip_j) >> 16;
    at = static_cast<long long>(static_cast<unsigned long long>(e.x & PQ::kStripeMask) * b32 + bucket);
    value = Img::inverse(e.x >> PQ::kShift, xrow + at);
  };
  for (uint32_t base = 0; base < static_cast<uint32_t>(k); base += tile) {
    // output position of every entry of this thread, in slot order (ranked again for
    // every tile: cheaper than keeping the positions in registers)
    uint32_t gt_rank = (excl & 0xffffu) - base;
    uint32_t eq_rank = excl >> 16;
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      const bool above = key[i] > top;
      const bool tie = !above && key[i] >= prefix;
      const uint32_t rel = above ? gt_rank : n_gt - base + eq_rank;   // wraps below the tile: never passes
      if ((above || (tie && eq_rank < need)) && rel < tile)
        staged[rel] = make_uint2(key[i], static_cast<uint32_t>(slot0 + i));
      gt_rank += above ? 1u : 0u;
      eq_rank += tie ? 1u : 0u;
    }
    __syncthreads();
    grid_launch_dependents();   // the next kernel in the stream may come onto the GPU
    const int cnt = static_cast<int>(min(tile, static_cast<uint32_t>(k) - base));
    const OutRow<Bits> o = orow.at(base);
    // two neighbouring outputs per thread: 16 bytes of positions, one word of values
    using Pair = typename std::conditional<sizeof(Bits) == 2, uint32_t, uint16_t>::type;
    const bool pairs = o.fmt == ATK_OUT_I64 && reinterpret_cast<uintptr_t>(o.i) % 16 == 0 &&
                       reinterpret_cast<uintptr_t>(o.v) % sizeof(Pair) == 0;
    int done = 0;
    if (pairs) {
      const int np = cnt >> 1;
      for (int q = tid; q < np; q += nthr) {
        const uint4 e = reinterpret_cast<const uint4*>(staged)[q];
        Bits v0, v1;
        long long a0, a1;
        rebuild(make_uint2(e.x, e.y), v0, a0);
        rebuild(make_uint2(e.z, e.w), v1, a1);
        reinterpret_cast<longlong2*>(o.i)[q] = make_longlong2(a0, a1);
        reinterpret_cast<Pair*>(o.v)[q] = static_cast<Pair>(static_cast<Pair>(v0) | (static_cast<Pair>(v1) << (8 * sizeof(Bits))));
      }
      done = np * 2;
    }
    for (int p = done + tid; p < cnt; p += nthr) {
      Bits v;
      long long at;
      rebuild(staged[p], v, at);
      o.put(p, v, at);
    }
    if (base + tile < static_cast<uint32_t>(k)) __syncthreads();
  }
}

// ------------------------------------------------------------------ large path
// Block-wide choice of the bin that holds the need-th largest key: NB bins in
// shared memory, walked from the top; all kLargeThreads threads take part.
template <int NB>
__device__ __forceinline__ void pick_digit_block(const uint32_t* sh, uint32_t need, uint32_t* res /* [2], shared */,
                                                 uint32_t* wsum /* [kLargeThreads / 32], shared */) {
  constexpr int P = NB / kLargeThreads;
  static_assert(P >= 1 && P * kLargeThreads == NB, "bins divide evenly over the block");
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint32_t h[P];
  uint32_t total = 0;
#pragma unroll
  for (int t = 0; t < P; ++t) {
    h[t] = sh[NB - 1 - (tid * P + t)];
    total += h[t];
  }
  uint32_t incl = total;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const uint32_t nb = __shfl_up_sync(0xffffffffu, incl, off);
    if (lane >= off) incl += nb;
  }
  if (lane == 31) wsum[warp] = incl;
  __syncthreads();
  uint32_t before = 0;
#pragma unroll
  for (int w = 0; w < kLargeThreads / 32; ++w) before += w < warp ? wsum[w] : 0u;
  uint32_t running = before + incl - total;
#pragma unroll
  for (int t = 0; t < P; ++t) {
    if (running < need && running + h[t] >= need) {
      res[0] = static_cast<uint32_t>(NB - 1 - (tid * P + t));
      res[1] = need - running;
    }
    running += h[t];
  }
  __syncthreads();
}

// One radix pass.  Every block histograms its chunks into the row's global
// histogram; the block that finishes last for a row (a ticket counter, no
// waiting) then picks the digit and advances the row's (prefix, mask, need).
// `tickets` and `hist` must be zero on entry (one memset per select call).
template <typename T, int ITEMS>
__global__ void __launch_bounds__(kLargeThreads)
select_hist_kernel(const typename ElemTraits<T>::Bits* __restrict__ cand_vals, long long k0,
                   long long cand_row_stride, int pass, long long k,
                   RowState<typename KeyOf<T>::Key>* __restrict__ state,
                   uint32_t* __restrict__ hist /* [rows][passes][bins] */,
                   uint32_t* __restrict__ tickets /* [rows][passes + 1] */, int cpb /* chunks per block */,
                   int vec /* rows are aligned for vector loads */) {
  using K = KeyOf<T>;
  using Key = typename K::Key;
  using D = LargeDigits<T>;
  constexpr int NB = D::kBins;
  __shared__ uint32_t sh[NB];
  __shared__ uint32_t res[2];
  __shared__ uint32_t wsum[kLargeThreads / 32];
  __shared__ bool last;
  const long long row = blockIdx.y;
  for (int i = threadIdx.x; i < NB; i += blockDim.x) sh[i] = 0;
  // launched overlapped with the end of the kernel before it (the pass before, or the
  // producer of the candidates): nothing of global memory is touched before it has ended
  grid_dependency_wait();
  RowState<Key> st;
  if (pass == 0) {
    st.prefix = 0;
    st.mask = 0;
    st.need = static_cast<uint32_t>(k);
    st.gave_up = 0;
  } else {
    st = state[row];
  }
  const int shift = D::shift(pass);
  const uint32_t digit_mask = (1u << D::width(pass)) - 1u;
  __syncthreads();
  // The block owns cpb consecutive chunks = one contiguous range of the row.
  // Thread t takes packs t, t + 256, ... of ITEMS consecutive candidates, kHistBatch
  // packs (vector loads) in flight before the first histogram update.
  const long long blk_begin = static_cast<long long>(blockIdx.x) * cpb * (kLargeThreads * ITEMS);
  long long blk_len_ll = k0 - blk_begin;
  if (blk_len_ll > static_cast<long long>(cpb) * (kLargeThreads * ITEMS)) blk_len_ll = static_cast<long long>(cpb) * (kLargeThreads * ITEMS);
  const int blk_len = blk_len_ll > 0 ? static_cast<int>(blk_len_ll) : 0;
  const auto* vblk = cand_vals + row * cand_row_stride + blk_begin;
  constexpr int kHistBatch = ATK_HIST_BATCH;
  for (int p0 = threadIdx.x * ITEMS; p0 < blk_len; p0 += kLargeThreads * ITEMS * kHistBatch) {
    typename ElemTraits<T>::Bits raw[kHistBatch][ITEMS];
#pragma unroll
    for (int bb = 0; bb < kHistBatch; ++bb) {
      const int first = p0 + bb * kLargeThreads * ITEMS;
      if (first < blk_len) load_items<typename ElemTraits<T>::Bits, ITEMS>(vblk, first, blk_len, vec, raw[bb]);
    }
#pragma unroll
    for (int bb = 0; bb < kHistBatch; ++bb) {
      const int first = p0 + bb * kLargeThreads * ITEMS;
      const int valid = blk_len - first;       // > 0 exactly for the packs that were loaded
      if (valid <= 0) continue;
      // plain shared-memory atomics: merging runs of equal digits inside a thread
      // first was measured slower in every pass (42 vs 55 us in the first one)
#pragma unroll
      for (int u = 0; u < ITEMS; ++u) {
        const Key key = K::key(raw[bb][u]);
        bool in = (key & st.mask) == st.prefix;
        if (valid < ITEMS) in = in && u < valid;        // only the last pack of a row is short
        if (in) atomicAdd(&sh[static_cast<uint32_t>(key >> shift) & digit_mask], 1u);
      }
    }
  }
  __syncthreads();
  grid_launch_dependents();   // the next pass may come onto the GPU; it waits for this one to end
  uint32_t* gh = hist + (row * D::kPasses + pass) * NB;
  for (int i = threadIdx.x; i < NB; i += blockDim.x)
    if (sh[i]) atomicAdd(&gh[i], sh[i]);
  // publish, then take a ticket; the holder of the last ticket sees every add
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0)
    last = atomicAdd(&tickets[row * (D::kPasses + 1) + pass], 1u) == gridDim.x - 1;
  __syncthreads();
  if (!last) return;
  __threadfence();
  for (int i = threadIdx.x; i < NB; i += blockDim.x) sh[i] = __ldcg(&gh[i]);
  __syncthreads();
  pick_digit_block<NB>(sh, st.need, res, wsum);
  if (threadIdx.x == 0) {
    st.prefix |= static_cast<Key>(res[0]) << shift;
    st.mask |= static_cast<Key>(digit_mask) << shift;
    st.need = res[1];
    state[row] = st;
  }
}

// How many candidates of every chunk lie above / on the threshold.  One warp per
// chunk (no block barriers): lane l takes packs l, l + 32, ... of the chunk,
// several vector loads in flight.  The block that finishes last for a row turns
// the per-chunk counts into exclusive prefixes.
template <typename T, int ITEMS>
__global__ void __launch_bounds__(kLargeThreads)
select_count_kernel(const typename ElemTraits<T>::Bits* __restrict__ cand_vals, long long k0,
                    long long cand_row_stride, const RowState<typename KeyOf<T>::Key>* __restrict__ state,
                    uint2* __restrict__ counts /* [rows][chunks] */, uint32_t* __restrict__ tickets, int chunks,
                    int cpw /* chunks per warp */, int vec) {
  using K = KeyOf<T>;
  using Key = typename K::Key;
  using Bits = typename ElemTraits<T>::Bits;
  using D = LargeDigits<T>;
  __shared__ bool last;
  grid_dependency_wait();   // see select_hist_kernel
  const long long row = blockIdx.y;
  const Key thr = state[row].prefix;
  const int lane = threadIdx.x & 31;
  const long long chunk0 = (static_cast<long long>(blockIdx.x) * (kLargeThreads / 32) + (threadIdx.x >> 5)) * cpw;
  for (long long chunk = chunk0; chunk < chunk0 + cpw && chunk < chunks; ++chunk) {
    const long long begin = chunk * (kLargeThreads * ITEMS);
    long long len_ll = k0 - begin;
    if (len_ll > kLargeThreads * ITEMS) len_ll = kLargeThreads * ITEMS;
    const int len = static_cast<int>(len_ll);
    const Bits* vchunk = cand_vals + row * cand_row_stride + begin;
    constexpr int kPacks = kLargeThreads / 32;                       // packs per lane
    constexpr int kBatch = sizeof(Bits) == 4 ? 4 : 2;   // vector loads in flight per lane (more cost registers)
    uint32_t gt = 0, eq = 0;
#pragma unroll
    for (int b0 = 0; b0 < kPacks; b0 += kBatch) {
      Bits raw[kBatch][ITEMS];
#pragma unroll
      for (int bb = 0; bb < kBatch; ++bb) {
        const int first = ((b0 + bb) * 32 + lane) * ITEMS;
        if (first < len) load_items<Bits, ITEMS>(vchunk, first, len, vec, raw[bb]);
      }
#pragma unroll
      for (int bb = 0; bb < kBatch; ++bb) {
        const int valid = len - ((b0 + bb) * 32 + lane) * ITEMS;
        if (valid >= ITEMS) {
#pragma unroll
          for (int u = 0; u < ITEMS; ++u) {
            const Key key = K::key(raw[bb][u]);
            gt += key > thr ? 1u : 0u;
            eq += key == thr ? 1u : 0u;
          }
        } else {
#pragma unroll
          for (int u = 0; u < ITEMS; ++u) {
            const Key key = K::key(raw[bb][u]);
            gt += (u < valid && key > thr) ? 1u : 0u;
            eq += (u < valid && key == thr) ? 1u : 0u;
          }
        }
      }
    }
    gt = __reduce_add_sync(0xffffffffu, gt);
    eq = __reduce_add_sync(0xffffffffu, eq);
    if (lane == 0) counts[row * chunks + chunk] = make_uint2(gt, eq);
  }
  // The block that finishes last for the row turns the per-chunk counts into
  // exclusive prefixes (one warp).
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0)
    last = atomicAdd(&tickets[row * (D::kPasses + 1) + D::kPasses], 1u) == gridDim.x - 1;
  __syncthreads();
  if (!last || threadIdx.x >= 32) return;
  __threadfence();
  uint2* c = counts + row * chunks;
  uint32_t carry_gt = 0, carry_eq = 0;
  for (int base = 0; base < chunks; base += 32) {
    const int i = base + lane;
    const uint2 v = i < chunks ? __ldcg(&c[i]) : make_uint2(0, 0);
    uint32_t a_gt = v.x, a_eq = v.y;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const uint32_t a = __shfl_up_sync(0xffffffffu, a_gt, off);
      const uint32_t b = __shfl_up_sync(0xffffffffu, a_eq, off);
      if (lane >= off) {
        a_gt += a;
        a_eq += b;
      }
    }
    if (i < chunks) c[i] = make_uint2(carry_gt + a_gt - v.x, carry_eq + a_eq - v.y);
    carry_gt += __shfl_sync(0xffffffffu, a_gt, 31);
    carry_eq += __shfl_sync(0xffffffffu, a_eq, 31);
  }
}

// Status word of a chunk in the write kernel's chained scan: a flag in the top two
// bits (0 nothing yet, 1 the chunk's own counts, 2 the counts of the chunk and all
// chunks before it) over two 31-bit counts (above the threshold, equal to it).
constexpr unsigned long long kScanOwn = 1ull << 62;
constexpr unsigned long long kScanAll = 2ull << 62;
__device__ __forceinline__ unsigned long long scan_pack(unsigned long long gt, unsigned long long eq) {
  return (gt << 31) | eq;
}
// Polls of a predecessor's status word before the write kernel gives up on a row
// (about a quarter of a second; reached only if a started block stops running).
constexpr int kScanMaxPolls = 1 << 22;

// The write pass.  Every block takes the next chunk of its row (a ticket, so that a
// block only ever waits for chunks whose blocks have already started), counts its
// candidates above / on the threshold, learns how many precede it in the row from
// the status words of the earlier chunks (a chained scan with look-back: no
// separate count pass over the candidates), and writes its winners.
// `tickets` (slot kPasses of the row) and `status` must be zero on entry.
// With CHAINED false the counts come from select_count_kernel instead (`status`
// then holds its exclusive prefixes as uint2 per chunk, and chunk = blockIdx.x).
template <typename T, int ITEMS, bool CHAINED>
__global__ void __launch_bounds__(kLargeThreads)
select_write_kernel(const typename ElemTraits<T>::Bits* __restrict__ cand_vals,
                    const long long* __restrict__ cand_idx, long long k0, long long cand_row_stride,
                    long long k, RowState<typename KeyOf<T>::Key>* __restrict__ state,
                    uint32_t* __restrict__ tickets, unsigned long long* __restrict__ status /* [rows][chunks] */,
                    void* __restrict__ out_vals, void* __restrict__ out_idx,
                    long long out_row_stride, int out_fmt, int vec) {
  using K = KeyOf<T>;
  using Key = typename K::Key;
  using D = LargeDigits<T>;
  __shared__ uint32_t wsum[32];
  __shared__ uint32_t block_total;
  __shared__ uint32_t chunk_s;
  __shared__ uint32_t base_s[2];
  __shared__ __align__(16) long long sidx[kLargeThreads * ITEMS];
  __shared__ __align__(16) typename ElemTraits<T>::Bits sval[kLargeThreads * ITEMS];
  grid_dependency_wait();   // see select_hist_kernel
  const long long row = blockIdx.y;
  if (CHAINED) {
    if (threadIdx.x == 0) chunk_s = atomicAdd(&tickets[row * (D::kPasses + 1) + D::kPasses], 1u);
    __syncthreads();
  }
  const long long chunk = CHAINED ? static_cast<long long>(chunk_s) : static_cast<long long>(blockIdx.x);
  const Key thr = state[row].prefix;
  const uint32_t need = state[row].need;
  const long long n_gt = k - need;
  const long long begin = chunk * (kLargeThreads * ITEMS);
  long long end = begin + kLargeThreads * ITEMS;
  if (end > k0) end = k0;
  const auto* vrow = cand_vals + row * cand_row_stride;
  const long long* irow = cand_idx + row * cand_row_stride;
  const OutRow<typename ElemTraits<T>::Bits> orow(out_vals, out_idx, row, out_row_stride, out_fmt);
  // Thread t owns the ITEMS consecutive slots begin + t*ITEMS ...:
  // per-thread counts, one block-wide scan, then every winner knows its place.
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const long long slot0 = begin + static_cast<long long>(threadIdx.x) * ITEMS;
  typename ElemTraits<T>::Bits raws[ITEMS];
  long long idxs[ITEMS];
  Key keys[ITEMS];
  load_items<typename ElemTraits<T>::Bits, ITEMS>(vrow, slot0, end, vec, raws);
  load_items<long long, ITEMS>(irow, slot0, end, vec, idxs);
  // slots of this thread that exist (only the last thread of a row can be short)
  long long valid_ll = end - slot0;
  const int valid = valid_ll >= ITEMS ? ITEMS : (valid_ll > 0 ? static_cast<int>(valid_ll) : 0);
  uint32_t mine = 0;
#pragma unroll
  for (int u = 0; u < ITEMS; ++u) {
    keys[u] = K::key(raws[u]);
    const bool in = valid == ITEMS || u < valid;
    mine += (in && keys[u] > thr) ? 1u : 0u;
    mine += (in && keys[u] == thr) ? 0x10000u : 0u;
  }
  uint32_t incl = mine;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const uint32_t nb = __shfl_up_sync(0xffffffffu, incl, off);
    if (lane >= off) incl += nb;
  }
  if (lane == 31) wsum[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    const uint32_t w = lane < (kLargeThreads >> 5) ? wsum[lane] : 0u;
    uint32_t wi = w;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const uint32_t nb = __shfl_up_sync(0xffffffffu, wi, off);
      if (lane >= off) wi += nb;
    }
    wsum[lane] = wi - w;
    if (lane == 31) block_total = wi;
  }
  __syncthreads();
  const uint32_t excl = wsum[warp] + incl - mine;
  const uint32_t tot_gt = block_total & 0xffffu;
  const uint32_t tot_eq = block_total >> 16;
  // Chained scan over the chunks of the row (warp 0): publish this chunk's counts,
  // look back over the earlier chunks 32 at a time until one of them already knows
  // the total of everything before it, then publish this chunk's total as well.
  if (!CHAINED) {
    if (threadIdx.x == 0) {
      const uint2 b = reinterpret_cast<const uint2*>(status)[row * static_cast<long long>(gridDim.x) + chunk];
      base_s[0] = b.x;
      base_s[1] = b.y;
    }
  } else if (warp == 0) {
    volatile unsigned long long* st = status + row * static_cast<long long>(gridDim.x);
    unsigned long long before_gt = 0, before_eq = 0;
    if (chunk > 0) {
      if (lane == 0) st[chunk] = kScanOwn | scan_pack(tot_gt, tot_eq);
      long long j = chunk - 1;
      int polls = 0;
      bool done = false;
      while (!done) {
        const long long at = j - lane;
        unsigned long long w = 2ull << 62;                               // before the first chunk: nothing
        if (at >= 0) w = st[at];
        const unsigned flag = static_cast<unsigned>(w >> 62);
        const unsigned ready = __ballot_sync(0xffffffffu, flag != 0u);
        const unsigned total_known = __ballot_sync(0xffffffffu, flag == 2u);
        const int stop = total_known ? __ffs(total_known) - 1 : 32;       // nearest chunk that knows its total
        const unsigned wanted = stop >= 31 ? 0xffffffffu : ((2u << stop) - 1u);
        if ((ready & wanted) == wanted) {
          const bool use = lane <= stop;
          unsigned long long g = use ? ((w >> 31) & 0x7fffffffull) : 0ull;
          unsigned long long e = use ? (w & 0x7fffffffull) : 0ull;
#pragma unroll
          for (int off = 16; off >= 1; off >>= 1) {
            g += __shfl_xor_sync(0xffffffffu, g, off);
            e += __shfl_xor_sync(0xffffffffu, e, off);
          }
          before_gt += g;
          before_eq += e;
          if (stop < 32) done = true;
          else j -= 32;
          polls = 0;
        } else if (++polls > kScanMaxPolls) {
          if (lane == 0) state[row].gave_up = 1u;     // never seen; the row's output is invalid then
          done = true;
        } else {
          __nanosleep(40);
        }
      }
    }
    if (lane == 0) {
      st[chunk] = kScanAll | scan_pack(before_gt + tot_gt, before_eq + tot_eq);
      base_s[0] = static_cast<uint32_t>(before_gt);
      base_s[1] = static_cast<uint32_t>(before_eq);
    }
  }
  __syncthreads();
  const uint32_t gt_base = base_s[0], eq_base = base_s[1];
  // The block's winners occupy two contiguous output ranges: those above the
  // threshold at gt_base ..., the selected ones equal to it at n_gt + eq_base ....
  // They are collected in shared memory in that order and copied out coalesced.
  uint32_t sel_eq = need > eq_base ? need - eq_base : 0u;   // equal candidates this block may still take
  if (sel_eq > tot_eq) sel_eq = tot_eq;
  uint32_t lgt = excl & 0xffffu;
  uint32_t leq = excl >> 16;
#pragma unroll
  for (int u = 0; u < ITEMS; ++u) {
    if (valid == ITEMS || u < valid) {
      int at = -1;
      if (keys[u] > thr) {
        at = static_cast<int>(lgt++);
      } else if (keys[u] == thr) {
        if (leq < sel_eq) at = static_cast<int>(tot_gt + leq);
        ++leq;
      }
      if (at >= 0) {
        sval[at] = raws[u];
        sidx[at] = idxs[u];
      }
    }
  }
  __syncthreads();
  const auto gt_row = orow.at(gt_base);
  stage_copy_out<typename ElemTraits<T>::Bits>(sidx, sval, static_cast<int>(tot_gt), gt_row, threadIdx.x,
                                               kLargeThreads, gt_row.aligned16());
  stage_copy_out<typename ElemTraits<T>::Bits>(sidx + tot_gt, sval + tot_gt, static_cast<int>(sel_eq),
                                               orow.at(n_gt + eq_base), threadIdx.x, kLargeThreads, false);
}

// ---- the whole multi-block select in one launch -----------------------------------
// For problems that fit the GPU at once (one long row, a few long rows): every block
// keeps the keys of its CPB chunks in registers through all the digit passes and the
// write, so the candidates are read once instead of once per pass, and the launches of
// the passes (each bound by launch and synchronisation latency at this size) become
// barriers between the blocks of a row.  The kernel is launched cooperatively: the
// launch fails unless every block is resident at once, so the barriers cannot wait for
// a block that has not started.  A barrier is a counter that is zero on entry and
// used once (the `tickets` words of the row); its wait is bounded all the same, and
// gives up with the row's `gave_up` flag set (never seen; the output is invalid then).
constexpr int kCoopMaxPolls = 1 << 22;

__device__ __forceinline__ void row_barrier(uint32_t* counter, uint32_t expected, uint32_t* gave_up) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();                       // this block's histogram / count updates are visible before its arrival
    atomicAdd(counter, 1u);
    int polls = 0;
    while (*reinterpret_cast<volatile uint32_t*>(counter) < expected) {
      if (++polls > kCoopMaxPolls) {
        *gave_up = 1u;
        break;
      }
      __nanosleep(32);
    }
    __threadfence();
  }
  __syncthreads();
}

template <typename T, int ITEMS, int CPB>
__global__ void __launch_bounds__(kLargeThreads, 4)   // four resident blocks per SM: one row of 2^21 fits with CPB = 2
select_coop_kernel(const typename ElemTraits<T>::Bits* __restrict__ cand_vals,
                   const long long* __restrict__ cand_idx, long long k0, long long cand_row_stride, long long k,
                   RowState<typename KeyOf<T>::Key>* __restrict__ state, uint32_t* __restrict__ hist,
                   uint32_t* __restrict__ tickets, unsigned long long* __restrict__ status /* [rows][chunks] */,
                   int chunks, void* __restrict__ out_vals, void* __restrict__ out_idx, long long out_row_stride,
                   int out_fmt, int vec) {
  using K = KeyOf<T>;
  using Key = typename K::Key;
  using Bits = typename ElemTraits<T>::Bits;
  using D = LargeDigits<T>;
  constexpr int NB = D::kBins;
  constexpr int kWarps = kLargeThreads / 32;
  __shared__ uint32_t sh[NB];
  __shared__ uint32_t res[2];
  __shared__ uint32_t wsum[32];
  __shared__ uint32_t block_total;
  __shared__ unsigned long long red[2 * kWarps];
  __shared__ __align__(16) long long sidx[kLargeThreads * ITEMS];
  __shared__ __align__(16) Bits sval[kLargeThreads * ITEMS];
  grid_dependency_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const long long row = blockIdx.y;
  uint32_t* gave_up = &state[row].gave_up;
  if (blockIdx.x == 0 && tid == 0) *gave_up = 0u;      // a barrier could set it a quarter of a second from now at the earliest
  const Bits* vrow = cand_vals + row * cand_row_stride;
  const long long* irow = cand_idx + row * cand_row_stride;
  uint32_t* row_tickets = tickets + row * (D::kPasses + 1);

  // the block's chunks, thread t owning ITEMS consecutive slots of each
  Bits raws[CPB][ITEMS];
  int valid[CPB];
  long long slot0[CPB], end[CPB];
#pragma unroll
  for (int c = 0; c < CPB; ++c) {
    const long long chunk = static_cast<long long>(blockIdx.x) * CPB + c;
    const long long begin = chunk * (kLargeThreads * ITEMS);
    end[c] = begin + kLargeThreads * ITEMS < k0 ? begin + kLargeThreads * ITEMS : k0;
    slot0[c] = begin + static_cast<long long>(tid) * ITEMS;
    const long long v = end[c] - slot0[c];
    valid[c] = v >= ITEMS ? ITEMS : (v > 0 ? static_cast<int>(v) : 0);
    if (valid[c] > 0) load_items<Bits, ITEMS>(vrow, slot0[c], end[c], vec, raws[c]);
  }

  // digit passes
  Key prefix = 0, mask = 0;
  uint32_t need = static_cast<uint32_t>(k);
  for (int pass = 0; pass < D::kPasses; ++pass) {
    const int shift = D::shift(pass);
    const uint32_t digit_mask = (1u << D::width(pass)) - 1u;
    for (int i = tid; i < NB; i += kLargeThreads) sh[i] = 0;
    __syncthreads();
#pragma unroll
    for (int c = 0; c < CPB; ++c) {
#pragma unroll
      for (int u = 0; u < ITEMS; ++u) {
        const Key key = K::key(raws[c][u]);
        if (u < valid[c] && (key & mask) == prefix) atomicAdd(&sh[static_cast<uint32_t>(key >> shift) & digit_mask], 1u);
      }
    }
    __syncthreads();
    uint32_t* gh = hist + (row * D::kPasses + pass) * NB;
    for (int i = tid; i < NB; i += kLargeThreads)
      if (sh[i]) atomicAdd(&gh[i], sh[i]);
    row_barrier(&row_tickets[pass], gridDim.x, gave_up);
    // every block of the row picks the digit for itself from the complete histogram
    for (int i = tid; i < NB; i += kLargeThreads) sh[i] = __ldcg(&gh[i]);
    __syncthreads();
    pick_digit_block<NB>(sh, need, res, wsum);
    prefix |= static_cast<Key>(res[0]) << shift;
    mask |= static_cast<Key>(digit_mask) << shift;
    need = res[1];
    __syncthreads();                       // res has been read before the next pass can write it
  }
  const Key thr = prefix;
  const long long n_gt = k - need;

  // counts of every chunk above / on the threshold, published for the blocks after it
  uint32_t excl[CPB], tot_gt[CPB], tot_eq[CPB];
#pragma unroll
  for (int c = 0; c < CPB; ++c) {
    uint32_t mine = 0;
#pragma unroll
    for (int u = 0; u < ITEMS; ++u) {
      const Key key = K::key(raws[c][u]);
      mine += (u < valid[c] && key > thr) ? 1u : 0u;
      mine += (u < valid[c] && key == thr) ? 0x10000u : 0u;
    }
    uint32_t incl = mine;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const uint32_t nb = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += nb;
    }
    if (lane == 31) wsum[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      const uint32_t w = lane < kWarps ? wsum[lane] : 0u;
      uint32_t wi = w;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const uint32_t nb = __shfl_up_sync(0xffffffffu, wi, off);
        if (lane >= off) wi += nb;
      }
      wsum[lane] = wi - w;
      if (lane == 31) block_total = wi;
    }
    __syncthreads();
    excl[c] = wsum[warp] + incl - mine;
    tot_gt[c] = block_total & 0xffffu;
    tot_eq[c] = block_total >> 16;
    const long long chunk = static_cast<long long>(blockIdx.x) * CPB + c;
    if (tid == 0 && chunk < chunks)
      status[row * chunks + chunk] = (static_cast<unsigned long long>(tot_gt[c]) << 32) | tot_eq[c];
    __syncthreads();                       // wsum and block_total are free for the next chunk
  }
  row_barrier(&row_tickets[D::kPasses], gridDim.x, gave_up);

  // how many candidates above / on the threshold precede this block in the row
  unsigned long long before_gt = 0, before_eq = 0;
  {
    const long long first = static_cast<long long>(blockIdx.x) * CPB;
    for (long long i = tid; i < first; i += kLargeThreads) {
      const unsigned long long w = __ldcg(&status[row * chunks + i]);
      before_gt += w >> 32;
      before_eq += w & 0xffffffffull;
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
      before_gt += __shfl_xor_sync(0xffffffffu, before_gt, off);
      before_eq += __shfl_xor_sync(0xffffffffu, before_eq, off);
    }
    if (lane == 0) {
      red[warp] = before_gt;
      red[kWarps + warp] = before_eq;
    }
    __syncthreads();
    before_gt = 0;
    before_eq = 0;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      before_gt += red[w];
      before_eq += red[kWarps + w];
    }
  }

  // the winners of every chunk: collected in shared memory in output order, copied out coalesced
  const OutRow<Bits> orow(out_vals, out_idx, row, out_row_stride, out_fmt);
  uint32_t gt_base = static_cast<uint32_t>(before_gt), eq_base = static_cast<uint32_t>(before_eq);
#pragma unroll
  for (int c = 0; c < CPB; ++c) {
    if (c > 0) __syncthreads();            // the staging arrays have been copied out
    long long idxs[ITEMS];
    if (valid[c] > 0) load_items<long long, ITEMS>(irow, slot0[c], end[c], vec, idxs);
    uint32_t sel_eq = need > eq_base ? need - eq_base : 0u;   // equal candidates this chunk may still take
    if (sel_eq > tot_eq[c]) sel_eq = tot_eq[c];
    uint32_t lgt = excl[c] & 0xffffu;
    uint32_t leq = excl[c] >> 16;
#pragma unroll
    for (int u = 0; u < ITEMS; ++u) {
      if (u < valid[c]) {
        const Key key = K::key(raws[c][u]);
        int at = -1;
        if (key > thr) {
          at = static_cast<int>(lgt++);
        } else if (key == thr) {
          if (leq < sel_eq) at = static_cast<int>(tot_gt[c] + leq);
          ++leq;
        }
        if (at >= 0) {
          sval[at] = raws[c][u];
          sidx[at] = idxs[u];
        }
      }
    }
    __syncthreads();
    const auto gt_row = orow.at(gt_base);
    stage_copy_out<Bits>(sidx, sval, static_cast<int>(tot_gt[c]), gt_row, tid, kLargeThreads, gt_row.aligned16());
    stage_copy_out<Bits>(sidx + tot_gt[c], sval + tot_gt[c], static_cast<int>(sel_eq), orow.at(n_gt + eq_base), tid,
                         kLargeThreads, false);
    gt_base += tot_gt[c];
    eq_base += tot_eq[c];
  }
}

inline long long chunks_of(long long k0) { return (k0 + kChunk - 1) / kChunk; }
inline size_t align256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

// Largest row the one-block path takes: 512 threads x 32 candidates in
// registers, half that for 64-bit elements.
template <typename T> constexpr int small_max_k0() { return sizeof(T) == 8 ? kSmallMaxK0 / 2 : kSmallMaxK0; }

// Workspace of the multi-block path: [row states][digit histograms | tickets |
// chunk status words], the bracketed part zeroed at the start of every call.
template <typename T>
struct LargeLayout {
  using D = LargeDigits<T>;
  size_t state_bytes, hist_words, ticket_words, status_offset, zero_bytes, total;
  LargeLayout(long long rows, long long k0) {
    state_bytes = align256(sizeof(RowState<typename KeyOf<T>::Key>) * rows);
    hist_words = static_cast<size_t>(D::kBins) * D::kPasses * rows;
    ticket_words = static_cast<size_t>(D::kPasses + 1) * rows;
    status_offset = ((hist_words + ticket_words) * sizeof(uint32_t) + 7) & ~static_cast<size_t>(7);
    zero_bytes = status_offset + sizeof(unsigned long long) * chunks_of(k0) * rows;
    total = state_bytes + align256(zero_bytes);
  }
};

template <typename T>
size_t workspace_typed(long long rows, long long k0) {
  if (k0 <= small_max_k0<T>()) return 0;
  return LargeLayout<T>(rows, k0).total;
}

// Resident blocks of the cooperative select on the current device (0: no cooperative
// launches there), queried once per device and instantiation.
template <typename T, int ITEMS, int CPB>
long long coop_capacity() {
  static std::atomic<long long> cache[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  long long c = cache[dev].load(std::memory_order_relaxed);
  if (c != 0) return c > 0 ? c : 0;
  int coop = 0, per_sm = 0;
  if (cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev) != cudaSuccess) coop = 0;
  if (coop && cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, select_coop_kernel<T, ITEMS, CPB>, kLargeThreads,
                                                            0) != cudaSuccess)
    per_sm = 0;
  cudaGetLastError();
  c = coop ? static_cast<long long>(per_sm) * sm_count_of_current_device() : 0;
  cache[dev].store(c > 0 ? c : -1, std::memory_order_relaxed);
  return c;
}

constexpr int kCoopDeclined = 1;   // nothing launched: the problem does not fit the GPU at once

template <typename T, int ITEMS, int CPB>
int launch_select_coop_cpb(const SelectLaunch& a, const typename ElemTraits<T>::Bits* cv, void* ov,
                           RowState<typename KeyOf<T>::Key>* state, uint32_t* hist, uint32_t* tickets,
                           unsigned long long* status, long long chunks, int vec) {
  const long long per_row = (chunks + CPB - 1) / CPB;
  if (a.rows * per_row > coop_capacity<T, ITEMS, CPB>() || a.rows > 65535) return kCoopDeclined;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(per_row), static_cast<unsigned>(a.rows));
  cfg.blockDim = dim3(kLargeThreads);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = a.stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t rc = cudaLaunchKernelEx(&cfg, select_coop_kernel<T, ITEMS, CPB>, cv,
                                            static_cast<const long long*>(a.cand_idx), static_cast<long long>(a.k0),
                                            static_cast<long long>(a.cand_row_stride), static_cast<long long>(a.k),
                                            state, hist, tickets, status, static_cast<int>(chunks), ov,
                                            static_cast<void*>(a.out_idx), static_cast<long long>(a.out_row_stride),
                                            a.out_format, vec);
  if (rc != cudaSuccess) {
    cudaGetLastError();                   // e.g. the GPU is shared and fewer blocks fit than the occupancy query said
    return kCoopDeclined;
  }
  note_launch();
  return ATK_OK;
}

template <typename T, int ITEMS>
int launch_select_coop(const SelectLaunch& a, const typename ElemTraits<T>::Bits* cv, void* ov,
                       RowState<typename KeyOf<T>::Key>* state, uint32_t* hist, uint32_t* tickets,
                       unsigned long long* status, long long chunks, int vec) {
  if (chunks >= (1ll << 30)) return kCoopDeclined;
  int rc = launch_select_coop_cpb<T, ITEMS, 1>(a, cv, ov, state, hist, tickets, status, chunks, vec);
  if (rc == kCoopDeclined) rc = launch_select_coop_cpb<T, ITEMS, 2>(a, cv, ov, state, hist, tickets, status, chunks, vec);
  return rc;
}

template <typename T>
int select_typed(const SelectLaunch& a) {
  using Bits = typename ElemTraits<T>::Bits;
  using K = KeyOf<T>;
  const Bits* cv = static_cast<const Bits*>(a.cand_vals);
  void* ov = a.out_vals;
  using State = RowState<typename K::Key>;
  if (a.k0 <= small_max_k0<T>()) {
    if (a.rows >= (1ll << 31)) return ATK_ERR_TOO_LARGE;
    const int k0 = static_cast<int>(a.k0);
    const int k = static_cast<int>(a.k);
    const int s = static_cast<int>(sizeof(Bits));
    const int vec_ok = (reinterpret_cast<uintptr_t>(cv) % 16 == 0) && ((a.cand_row_stride * s) % 16 == 0) &&
                       (reinterpret_cast<uintptr_t>(a.cand_idx) % 16 == 0) && ((a.cand_row_stride * 8) % 16 == 0);
    const unsigned rows = static_cast<unsigned>(a.rows);
    auto threads_for = [&](int items) {
      int t = (k0 + items - 1) / items;
      return ((t + 31) / 32) * 32;
    };
    // At least 16 bytes of values per thread; more items per thread until the
    // block is at most kSelectRowThreads wide (512 measured better than 256 on
    // 4096-candidate rows, and equal to 1024), 32 items at most.
    constexpr int kBase = 16 / static_cast<int>(sizeof(Bits));
    constexpr int kMost = sizeof(Bits) == 8 ? 16 : 32;           // per-thread candidates the registers hold
    constexpr int kMid = 4 * kBase <= kMost ? 4 * kBase : kMost;
#define ATK_LAUNCH_SELECT_ROW(ITEMS, MAXT)                                                             \
    do {                                                                                                 \
      if (vec_ok && threads_for(ITEMS) * (ITEMS) == k0)                                                  \
        select_row_kernel<T, ITEMS, MAXT, true><<<rows, threads_for(ITEMS), stage_bytes<Bits>(k), a.stream>>>( \
            cv, a.cand_idx, k0, a.cand_row_stride, k, ov, a.out_idx, a.out_row_stride, a.out_format, vec_ok); \
      else                                                                                               \
        select_row_kernel<T, ITEMS, MAXT, false><<<rows, threads_for(ITEMS), stage_bytes<Bits>(k), a.stream>>>( \
            cv, a.cand_idx, k0, a.cand_row_stride, k, ov, a.out_idx, a.out_row_stride, a.out_format, vec_ok); \
    } while (0)
    if (threads_for(kBase) <= kSelectRowThreads) ATK_LAUNCH_SELECT_ROW(kBase, kSelectRowThreads);
    else if (threads_for(2 * kBase) <= kSelectRowThreads) ATK_LAUNCH_SELECT_ROW(2 * kBase, kSelectRowThreads);
    else if (threads_for(kMid) <= kSelectRowThreads) ATK_LAUNCH_SELECT_ROW(kMid, kSelectRowThreads);
    else ATK_LAUNCH_SELECT_ROW(kMost, 512);
#undef ATK_LAUNCH_SELECT_ROW
    note_launch();
    return cudaGetLastError() == cudaSuccess ? ATK_OK : ATK_ERR_CUDA;
  }

  if (a.k0 >= (1ll << 31) || a.rows > 65535) return ATK_ERR_TOO_LARGE;
  using D = LargeDigits<T>;
  const LargeLayout<T> lay(a.rows, a.k0);
  if (a.workspace == nullptr || a.workspace_bytes < lay.total) return ATK_ERR_WORKSPACE;
  const long long chunks = chunks_of(a.k0);
  unsigned char* ws = static_cast<unsigned char*>(a.workspace);
  State* state = reinterpret_cast<State*>(ws);
  ws += lay.state_bytes;
  uint32_t* hist = reinterpret_cast<uint32_t*>(ws);
  uint32_t* tickets = hist + lay.hist_words;
  unsigned long long* status = reinterpret_cast<unsigned long long*>(ws + lay.status_offset);

  if (cudaMemsetAsync(hist, 0, lay.zero_bytes, a.stream) != cudaSuccess) return ATK_ERR_CUDA;
  // 8 candidates per thread (2048 per block): 32 per thread with wider chunks was
  // measured 40 % slower on 256 rows x 131072 candidates.
  constexpr int kItems = kChunk / kLargeThreads;
  // The histogram blocks loop over several chunks when there are many more chunks
  // than the GPU holds blocks, so that the per-block epilogue (global flush,
  // fence, ticket) is paid once per group of chunks.
  const long long sms = sm_count_of_current_device();
  long long cpb = (a.rows * chunks + sms * 6 - 1) / (sms * 6);
  if (cpb < 1) cpb = 1;
  if (cpb > 64) cpb = 64;
  const long long groups = (chunks + cpb - 1) / cpb;
  const dim3 grid(static_cast<unsigned>(chunks), static_cast<unsigned>(a.rows));
  const dim3 grid_g(static_cast<unsigned>(groups), static_cast<unsigned>(a.rows));
  // vector loads need 16-byte aligned rows of values and of positions
  const int vec = (reinterpret_cast<uintptr_t>(cv) % 16 == 0) && ((a.cand_row_stride * sizeof(Bits)) % 16 == 0) &&
                  (reinterpret_cast<uintptr_t>(a.cand_idx) % 16 == 0) && ((a.cand_row_stride * 8) % 16 == 0);
  // Problems that fit the GPU at once (up to two chunks per resident block): the whole
  // select in ONE cooperative launch, keys in registers from the first pass to the write
  // (select_coop_kernel).  ATK_NO_COOP_SELECT=1 keeps the launch per pass.
  {
    static const bool coop_off = std::getenv("ATK_NO_COOP_SELECT") != nullptr;
    if (!coop_off) {
      const int rc = launch_select_coop<T, kItems>(a, cv, ov, state, hist, tickets, status, chunks, vec);
      if (rc != kCoopDeclined) return rc;
    }
  }
  // Few chunks in all (a long row or two): every launch overlaps the end of the one before
  // it (one row of 2^21: 46.3 -> 45.0 us).  With many blocks per launch the early blocks
  // crowd the SMs that finish first (256 rows x 131072: 259.7 -> 264.4 us): plain launches.
  const bool small = a.rows * chunks <= 4 * sms * 8;
  for (int pass = 0; pass < D::kPasses; ++pass)
    launch_overlapped_if(small, select_hist_kernel<T, kItems>, grid_g, dim3(kLargeThreads), 0, a.stream,
                      cv, a.k0, a.cand_row_stride, pass, a.k, state, hist, tickets, static_cast<int>(cpb), vec);
  // Few chunks in all (a long row or two): the write kernel chains the counts of the
  // chunks itself (one launch and one pass over the values fewer: 57 -> 47 us on one
  // row of 2^21).  Many rows: a separate count pass was measured faster (256 rows x
  // 131072: 290 us against 355 us chained).
  const bool chained = ATK_SELECT_CHAINED < 0 ? small : ATK_SELECT_CHAINED != 0;
  if (chained) {
    launch_overlapped_if(small, select_write_kernel<T, kItems, true>, grid, dim3(kLargeThreads), 0, a.stream,
                      cv, a.cand_idx, a.k0, a.cand_row_stride, a.k, state, tickets, status, ov, a.out_idx,
                      a.out_row_stride, a.out_format, vec);
    note_launch(D::kPasses + 1);
  } else {
    // count: one warp per cpw chunks, about one wave of blocks (every block ends with a fence and a ticket)
    constexpr int kWarps = kLargeThreads / 32;
    long long cpw = (a.rows * chunks + sms * 8 * kWarps - 1) / (sms * 8 * kWarps);
    if (cpw < 1) cpw = 1;
    if (cpw > 16) cpw = 16;
    const dim3 grid_c(static_cast<unsigned>((chunks + kWarps * cpw - 1) / (kWarps * cpw)), static_cast<unsigned>(a.rows));
    launch_overlapped_if(small, select_count_kernel<T, kItems>, grid_c, dim3(kLargeThreads), 0, a.stream,
                      cv, a.k0, a.cand_row_stride, state, reinterpret_cast<uint2*>(status), tickets,
                      static_cast<int>(chunks), static_cast<int>(cpw), vec);
    launch_overlapped_if(small, select_write_kernel<T, kItems, false>, grid, dim3(kLargeThreads), 0, a.stream,
                      cv, a.cand_idx, a.k0, a.cand_row_stride, a.k, state, tickets, status, ov, a.out_idx,
                      a.out_row_stride, a.out_format, vec);
    note_launch(D::kPasses + 2);
  }
  return cudaGetLastError() == cudaSuccess ? ATK_OK : ATK_ERR_CUDA;
}

}  // namespace

size_t select_workspace_bytes(int dtype, long long rows, long long k0) {
  switch (dtype) {
    case ATK_F32: return workspace_typed<float>(rows, k0);
    case ATK_F16: return workspace_typed<__half>(rows, k0);
    case ATK_BF16: return workspace_typed<__nv_bfloat16>(rows, k0);
    case ATK_F64: return workspace_typed<double>(rows, k0);
    case ATK_I32: return workspace_typed<int32_t>(rows, k0);
    case ATK_I64: return workspace_typed<long long>(rows, k0);
    case ATK_I16: return workspace_typed<int16_t>(rows, k0);
    case ATK_I8: return workspace_typed<int8_t>(rows, k0);
    case ATK_U8: return workspace_typed<uint8_t>(rows, k0);
    default: return 0;
  }
}

namespace {
// Rows of up to 8192 entries (16 per thread in a block of 512): with 32 per thread the
// packed form was measured slower than the plain hand-off (88 vs 66 us for 256 rows x 16384).
constexpr long long kPackedMaxK0 = 8192;

template <typename T>
int select_packed_typed(const SelectPackedLaunch& a) {
  using Bits = typename ElemTraits<T>::Bits;
  if (a.k0 > kPackedMaxK0 || a.rows >= (1ll << 31)) return ATK_ERR_TOO_LARGE;
  const int k0 = static_cast<int>(a.k0);
  const int k = static_cast<int>(a.k);
  const int vec_ok = (reinterpret_cast<uintptr_t>(a.keys) % 16 == 0) && ((a.k0 * 4) % 16 == 0);
  const unsigned rows = static_cast<unsigned>(a.rows);
  auto threads_for = [&](int items) {
    int t = (k0 + items - 1) / items;
    return ((t + 31) / 32) * 32;
  };
  const T* x = static_cast<const T*>(a.x);
  void* ov = a.out_vals;
#define ATK_LAUNCH_SELECT_PACKED(ITEMS, MAXT)                                                             \
  do {                                                                                                    \
    if (vec_ok && threads_for(ITEMS) * (ITEMS) == k0)                                                     \
      launch_overlapped(select_row_packed_kernel<T, ITEMS, MAXT, true>, dim3(rows), dim3(threads_for(ITEMS)), \
                        packed_stage_bytes(k), a.stream, a.keys, k0, k, x, a.x_row_stride, a.b, a.j, ov,  \
                        a.out_idx, a.out_row_stride, a.out_format, vec_ok);                               \
    else                                                                                                  \
      launch_overlapped(select_row_packed_kernel<T, ITEMS, MAXT, false>, dim3(rows), dim3(threads_for(ITEMS)), \
                        packed_stage_bytes(k), a.stream, a.keys, k0, k, x, a.x_row_stride, a.b, a.j, ov,  \
                        a.out_idx, a.out_row_stride, a.out_format, vec_ok);                               \
  } while (0)
#define ATK_LAUNCH_SELECT_PACKED_ITEMS(ITEMS)                                 \
  do {                                                                        \
    if (threads_for(ITEMS) <= 128) ATK_LAUNCH_SELECT_PACKED(ITEMS, 128);      \
    else if (threads_for(ITEMS) <= 256) ATK_LAUNCH_SELECT_PACKED(ITEMS, 256); \
    else ATK_LAUNCH_SELECT_PACKED(ITEMS, 512);                                \
  } while (0)
  // Entries per thread: few threads with long runs beat many threads with short ones
  // (the per-thread cost of the scans and barriers is spread over more entries; for
  // bf16 1024 x 4096 -> 2048: 16 per thread 46.4 us for the whole operator, 8 per thread
  // 48.8, 32 per thread 49.8).  ATK_SELECT_PACKED_ITEMS = 4, 8 or 16 overrides the choice.
  static const int forced = [] {
    const char* e = std::getenv("ATK_SELECT_PACKED_ITEMS");
    return e ? std::atoi(e) : 0;
  }();
  int items = k0 >= 4096 ? 16 : (k0 >= 256 ? 8 : 4);
  if ((forced == 4 || forced == 8 || forced == 16) && threads_for(forced) <= kSelectRowThreads) items = forced;
  if (items == 4) ATK_LAUNCH_SELECT_PACKED_ITEMS(4);
  else if (items == 8) ATK_LAUNCH_SELECT_PACKED_ITEMS(8);
  else ATK_LAUNCH_SELECT_PACKED_ITEMS(16);
#undef ATK_LAUNCH_SELECT_PACKED_ITEMS
#undef ATK_LAUNCH_SELECT_PACKED
  note_launch();
  return cudaGetLastError() == cudaSuccess ? ATK_OK : ATK_ERR_CUDA;
}
}  // namespace

long long select_packed_max_k0() { return kPackedMaxK0; }

int launch_select_packed(const SelectPackedLaunch& a, int dtype) {
  if (a.rows <= 0 || a.k <= 0) return ATK_OK;
  switch (dtype) {
    case ATK_F16: return select_packed_typed<__half>(a);
    case ATK_BF16: return select_packed_typed<__nv_bfloat16>(a);
    case ATK_I16: return select_packed_typed<int16_t>(a);
    case ATK_I8: return select_packed_typed<int8_t>(a);
    case ATK_U8: return select_packed_typed<uint8_t>(a);
    default: return ATK_ERR_BAD_DTYPE;
  }
}

// ---- built-in scratch for callers that cannot allocate -----------------------
// Part of the library image: every device that loads the library holds these
// bytes until the process exits.  In host code the name below is only a
// host-side stand-in for the symbol, not a device address; the address that
// kernels may use comes from cudaGetSymbolAddress, looked up once per device.
static __device__ __align__(256) unsigned char g_select_static_scratch[ATK_SELECT_STATIC_SCRATCH_BYTES];

namespace {
// Device address of g_select_static_scratch on the current device, or nullptr
// if the runtime cannot provide it.  The first call on a device does the
// look-up (with that device current) and caches it; later calls only read the
// cache.  Two threads racing on the first call store the same value.
void* static_scratch_of_current_device() {
  static std::atomic<void*> cache[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  if (dev >= 0 && dev < 64) {
    void* known = cache[dev].load(std::memory_order_acquire);
    if (known != nullptr) return known;
  }
  void* ptr = nullptr;
  if (cudaGetSymbolAddress(&ptr, g_select_static_scratch) != cudaSuccess || ptr == nullptr) return nullptr;
  if (dev >= 0 && dev < 64) cache[dev].store(ptr, std::memory_order_release);
  return ptr;
}
}  // namespace

int launch_select_static(const SelectLaunch& a, int dtype) {
  if (a.rows <= 0 || a.k <= 0) return ATK_OK;
  const size_t need = select_workspace_bytes(dtype, a.rows, a.k0);
  if (need > sizeof(g_select_static_scratch)) return ATK_ERR_SCRATCH_LIMIT;
  SelectLaunch b = a;
  b.workspace = nullptr;
  b.workspace_bytes = 0;
  if (need > 0) {
    void* scratch = static_scratch_of_current_device();
    if (scratch == nullptr) return ATK_ERR_CUDA;
    b.workspace = scratch;
    b.workspace_bytes = sizeof(g_select_static_scratch);
  }
  // The select clears the histograms it accumulates into at the start of every
  // call (on the stream); everything else in the scratch is written before it
  // is read, so stale contents of an earlier call are harmless.
  return launch_select(b, dtype);
}

int launch_select(const SelectLaunch& a, int dtype) {
  if (a.rows <= 0 || a.k <= 0) return ATK_OK;
  switch (dtype) {
    case ATK_F32: return select_typed<float>(a);
    case ATK_F16: return select_typed<__half>(a);
    case ATK_BF16: return select_typed<__nv_bfloat16>(a);
    case ATK_F64: return select_typed<double>(a);
    case ATK_I32: return select_typed<int32_t>(a);
    case ATK_I64: return select_typed<long long>(a);
    case ATK_I16: return select_typed<int16_t>(a);
    case ATK_I8: return select_typed<int8_t>(a);
    case ATK_U8: return select_typed<uint8_t>(a);
    default: return ATK_ERR_BAD_DTYPE;
  }
}

}  // namespace atk
