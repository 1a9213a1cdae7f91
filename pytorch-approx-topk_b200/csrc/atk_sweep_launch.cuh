// Host-side launch logic of the column sweep, included
// by one translation unit per element type so the template instantiations
// compile in parallel.
#pragma once

#include <type_traits>

#include "atk_sweep.cuh"

namespace atk {

namespace sweep_detail {

// Stripes per thread from which the head test (skip the insertion when nothing
// enters) pays off; below it 16-bit float inputs take the tile scan.
constexpr long long kSkipStripes = 256;
// Longest columns the shared-memory tile kernel takes (a build knob for measurements).
#ifndef ATK_TILE_MAX_STRIPES
#define ATK_TILE_MAX_STRIPES 65536
#endif
constexpr long long kTileMaxStripes = ATK_TILE_MAX_STRIPES;   // stripe numbers of 16-bit elements: 16 bits
// Shortest float32 columns the tile kernel takes, for queues of two entries and of
// three or four (build knobs for measurements).  Measured on 128 x 2^20 rows: two
// entries 97 us (sweep) against 112 us (tiles) at 32 stripes, even at 128 and 512,
// and 1.1-1.35x for the tiles on columns of 8192 stripes split over blocks; four
// entries 140 against 117 us at 64 stripes, 148 against 104 us at 512.  Queues of
// one entry stay with the sweep for every element type (90 against 118 us).
#ifndef ATK_TILE_FLOAT_MIN_STRIPES_J2
#define ATK_TILE_FLOAT_MIN_STRIPES_J2 1024
#endif
#ifndef ATK_TILE_FLOAT_MIN_STRIPES
#define ATK_TILE_FLOAT_MIN_STRIPES 64
#endif

inline void fill_common(SweepParams& p, const SweepLaunch& a, int elem_size) {
  p.x = a.x;
  p.out_vals = a.out_vals;
  p.out_idx = a.out_idx;
  p.rows = a.rows;
  p.row_stride = a.row_stride;
  p.out_row_stride = a.out_row_stride;
  p.b = a.b;
  p.l_full = a.n / a.b;
  p.rem = a.n - p.l_full * a.b;
  p.stripe_stride = a.stripe_stride;
  p.idx_stride = a.idx_stride;
  p.idx_offset = a.idx_offset;
  p.out_format = a.out_format;
  const uintptr_t ov = reinterpret_cast<uintptr_t>(a.out_vals);
  const uintptr_t oi = reinterpret_cast<uintptr_t>(a.out_idx);
  if (a.out_format == ATK_OUT_REC32)
    p.vec_out = (ov % 16 == 0) && ((a.out_row_stride * 8) % 16 == 0);
  else
    p.vec_out = (ov % 16 == 0) && (oi % 16 == 0) && ((a.out_row_stride * elem_size) % 16 == 0) &&
                ((a.out_row_stride * (a.out_format == ATK_OUT_I32 ? 4 : 8)) % 16 == 0);
}

// ---- stage 1 -----------------------------------------------------------------
// One launch of the sweep kernel for a scan mode (head-test variant by `skip`).
template <typename T, typename Q, int J, int V, int MODE, bool PACKED_OUT>
void launch_sweep_mode(const dim3& grid, const dim3& block, size_t smem, cudaStream_t stream, const SweepParams& p,
                       bool skip) {
  if (skip)
    launch_overlapped(sweep_kernel<T, Q, J, V, true, MODE, PACKED_OUT>, grid, block, smem, stream, p);
  else
    launch_overlapped(sweep_kernel<T, Q, J, V, false, MODE, PACKED_OUT>, grid, block, smem, stream, p);
}

template <typename T, typename Q, int J, int V, int MODE>
int launch_stage1(const SweepLaunch& a) {
  using Bits = typename ElemTraits<T>::Bits;
  SweepParams p;
  fill_common(p, a, static_cast<int>(sizeof(T)));
  if (p.l_full + 1 >= (1ll << 31)) return ATK_ERR_TOO_LARGE;

  SweepPlan pl = plan_sweep(a.rows, a.b, p.l_full, V, a.sm_count);
  const long long k0 = a.b * J;
  constexpr bool kCanPack = Q::kPacked && !Q::kFirst;
  if (a.out_keys != nullptr && (!kCanPack || pl.Z > 1)) return kPackedUnavailable;
  p.out_keys = a.out_keys;
  p.vec_keys = (reinterpret_cast<uintptr_t>(a.out_keys) % 16 == 0) && ((k0 * 4) % 16 == 0);
  if (pl.Z > 1) {
    // use as many planes as the caller's scratch holds (none: no split over blocks)
    const size_t per_z = static_cast<size_t>(a.rows) * k0 * (sizeof(Bits) + 8);
    long long fit = 0;
    if (a.workspace != nullptr && a.workspace_bytes > 256) fit = static_cast<long long>((a.workspace_bytes - 256) / per_z);
    if (fit < pl.Z) pl.Z = fit >= 2 ? fit : 1;
    set_chunks(pl, p.l_full);
  }
  p.tiles = pl.tiles;
  p.cw = static_cast<int>(pl.cw);
  p.s = static_cast<int>(pl.S);
  p.z = static_cast<int>(pl.Z);
  p.z_chunk = pl.z_chunk;
  p.main_units = 0;
  p.z_main = 1;
  p.z_chunk_main = pl.z_chunk;
  p.part_vals = nullptr;
  p.part_idx = nullptr;
  p.vec_part = 0;
  if (pl.Z > 1) {
    // dense planes [z][rows][k0]: all value planes first, then all position planes
    unsigned char* ws = static_cast<unsigned char*>(a.workspace);
    p.part_vals = ws;
    p.part_idx = reinterpret_cast<long long*>(ws + align256(static_cast<size_t>(pl.Z) * a.rows * k0 * sizeof(Bits)));
    p.vec_part = (reinterpret_cast<uintptr_t>(ws) % 16 == 0) && ((k0 * sizeof(Bits)) % 16 == 0) && ((k0 * 8) % 16 == 0);
  }
  if (a.rows * pl.tiles * pl.Z >= (1ll << 31)) return ATK_ERR_TOO_LARGE;

  const size_t smem = pl.S > 1 ? static_cast<size_t>(pl.S / 2) * (V * Q::kWords) * pl.cw * 4 : 0;
  const dim3 grid(static_cast<unsigned>(a.rows * pl.tiles * pl.Z));
  const dim3 block(static_cast<unsigned>(pl.cw), static_cast<unsigned>(pl.S));
  // The head test pays off once a thread walks a long column.
  const bool skip = (pl.z_chunk / pl.S) >= kSkipStripes;
  if constexpr (kCanPack) {
    if (a.out_keys != nullptr) {
      launch_sweep_mode<T, Q, J, V, MODE, true>(grid, block, smem, a.stream, p, skip);
      note_launch();
      return cudaGetLastError() == cudaSuccess ? ATK_OK : ATK_ERR_CUDA;
    }
  }
  launch_sweep_mode<T, Q, J, V, MODE, false>(grid, block, smem, a.stream, p, skip);
  note_launch();
  if (cudaGetLastError() != cudaSuccess) return ATK_ERR_CUDA;
  if (pl.Z > 1) {
    int g = 1;                                   // lanes per bucket: about 8 planes per lane
    while (g < 32 && g * 8 < pl.Z) g *= 2;
    const long long blocks = (a.rows * a.b * g + 255) / 256;
    if (blocks >= (1ll << 31)) return ATK_ERR_TOO_LARGE;
    sweep_merge_planes_kernel<T, J, Q::kFirst><<<static_cast<unsigned>(blocks), 256, 0, a.stream>>>(
        static_cast<const Bits*>(p.part_vals), p.part_idx, p.z, g, a.rows, a.b, 1ll, 1, 0ll, 1, a.out_vals,
        a.out_idx, a.out_row_stride, a.out_format);
    note_launch();
    if (cudaGetLastError() != cudaSuccess) return ATK_ERR_CUDA;
  }
  return ATK_OK;
}

// Queue layout: 8- and 16-bit inputs use packed 32-bit entries whenever the
// stripe number fits beside the value (the float formats scanned with the
// two-column SIMD queues on the vector path); everything else uses (value,
// stripe) pairs.
template <typename T, int J, int V, bool FIRST>
int launch_by_queue(const SweepLaunch& a) {
  if constexpr (sizeof(T) <= 2) {
    // stripes are numbered 0 .. n/b (the last one only when b does not divide n)
    const long long stripes = a.n / a.b + (a.n % a.b != 0 ? 1 : 0);
    if (stripes <= PackedQueue<T, J, FIRST>::kMaxStripes) {
      // the two-column SIMD scan exists for the float formats only
      return launch_stage1<T, PackedQueue<T, J, FIRST>, J, V,
                           (V >= 4 && ElemTraits<T>::kHalfFloat) ? kScanSimd : kScanQueues>(a);
    }
  }
  if (a.out_keys != nullptr) return kPackedUnavailable;
  return launch_stage1<T, FloatQueue<T, J, FIRST>, J, V, kScanQueues>(a);
}

template <typename T, int V>
int launch_by_j(const SweepLaunch& a) {
  if (a.first_wins) {
    if (a.j != 1) return ATK_ERR_BAD_J;
    return launch_by_queue<T, 1, V, true>(a);
  }
  switch (a.j) {
    case 1: return launch_by_queue<T, 1, V, false>(a);
    case 2: return launch_by_queue<T, 2, V, false>(a);
    case 3: return launch_by_queue<T, 3, V, false>(a);
    case 4: return launch_by_queue<T, 4, V, false>(a);
    default: return ATK_ERR_BAD_J;
  }
}

// Returned by the tile launcher (nothing launched) when the shape does not give its
// kernel enough blocks, e.g. because the scratch for a stripe split is missing: the
// caller goes on to the sweep kernel.
constexpr int kTileDeclined = 2;

// The shared-memory tile kernel (tile_kernel): 16-bit floats and float32, 2 <= J <= 4.
template <typename T, int J>
int launch_tile_shared_j(const SweepLaunch& a) {
  using Q = typename TileQueue<T, J>::type;
  using Bits = typename ElemTraits<T>::Bits;
  using Shape = TileShape<T>;
  constexpr bool kCanPack = Q::kPacked;
  if (a.out_keys != nullptr && !kCanPack) return kPackedUnavailable;
  SweepParams p;
  fill_common(p, a, static_cast<int>(sizeof(T)));
  const long long k0 = a.b * J;
  p.out_keys = a.out_keys;
  p.vec_keys = (reinterpret_cast<uintptr_t>(a.out_keys) % 16 == 0) && ((k0 * 4) % 16 == 0);
  p.tiles = (a.b + Shape::kCols - 1) / Shape::kCols;
  p.cw = kTileThreads;
  p.s = 1;
  // stripe split over blocks: as many planes as wanted and as the caller's scratch holds
  TilePlan tp{0, 1, 1};
  if (a.out_keys == nullptr) tp = tile_plan(a.rows, p.tiles, p.l_full, a.sm_count);
  long long Z = tp.z, Zm = tp.z_main;
  if (Z > 1) {
    const size_t per_z = static_cast<size_t>(a.rows) * k0 * (sizeof(Bits) + 8);
    long long fit = 0;
    if (a.workspace != nullptr && a.workspace_bytes > 256) fit = static_cast<long long>((a.workspace_bytes - 256) / per_z);
    if (fit < Z) Z = fit >= 2 ? fit : 1;
    if (fit < Zm) Zm = fit >= 2 ? fit : 1;
  }
  SweepPlan pl, plm;
  pl.S = 1;
  pl.Z = Z;
  set_chunks(pl, p.l_full);
  plm.S = 1;
  plm.Z = Zm;
  set_chunks(plm, p.l_full);
  const long long units = a.rows * p.tiles;
  const long long main_units = pl.Z > plm.Z ? tp.main_units : 0;
  const long long n_blocks = main_units * plm.Z + (units - main_units) * pl.Z;
  // half a wave of blocks at least; below that the sweep with its in-block splits takes over
  if (n_blocks < 3ll * a.sm_count) return a.out_keys != nullptr ? kPackedUnavailable : kTileDeclined;
  p.z = static_cast<int>(pl.Z);
  p.z_chunk = pl.z_chunk;
  p.main_units = main_units;
  p.z_main = static_cast<int>(plm.Z);
  p.z_chunk_main = plm.z_chunk;
  p.part_vals = nullptr;
  p.part_idx = nullptr;
  p.vec_part = 0;
  if (pl.Z > 1) {
    unsigned char* ws = static_cast<unsigned char*>(a.workspace);
    p.part_vals = ws;
    p.part_idx = reinterpret_cast<long long*>(ws + align256(static_cast<size_t>(pl.Z) * a.rows * k0 * sizeof(Bits)));
    p.vec_part = (reinterpret_cast<uintptr_t>(ws) % 16 == 0) && ((k0 * sizeof(Bits)) % 16 == 0) && ((k0 * 8) % 16 == 0);
  }
  if (n_blocks >= (1ll << 31)) return ATK_ERR_TOO_LARGE;
  const dim3 grid(static_cast<unsigned>(n_blocks));
  const bool packed = a.out_keys != nullptr;
  // stripes a block walks (the whole column for the units that are not split)
  const long long longest = main_units > 0 ? plm.z_chunk : pl.z_chunk;
  const long long per_block = longest < p.l_full ? longest : p.l_full;
#define ATK_LAUNCH_TILE(CH, BUFS)                                                                    \
  do {                                                                                               \
    const size_t smem = static_cast<size_t>(BUFS) * (CH) * kTileThreads * 4;                         \
    if constexpr (kCanPack) {                                                                        \
      if (packed) launch_overlapped(tile_kernel<T, J, CH, true, BUFS>, grid, dim3(kTileThreads), smem, a.stream, p); \
      else launch_overlapped(tile_kernel<T, J, CH, false, BUFS>, grid, dim3(kTileThreads), smem, a.stream, p); \
    } else {                                                                                         \
      launch_overlapped(tile_kernel<T, J, CH, false, BUFS>, grid, dim3(kTileThreads), smem, a.stream, p); \
    }                                                                                                \
  } while (0)
  // Up to 256 stripes per block: one buffer of up to 64 stripes, filled and scanned in
  // turns.  Longer columns: two buffers of 32 stripes, the copies of one in flight while
  // the other is scanned (fp16 256 x 2^20, j=4: 512 stripes 100.3 -> 98.0 us, 2048
  // stripes 195.2 -> 190.8; fp32 4 x 2^26 j=4 197 -> 188; at 128 and 256 stripes the
  // shorter chunks cost more than the overlap gives: 114.8 -> 129.5 and 103.0 -> 110.4).
  // ATK_TILE_BUFS = 1 or 2 overrides the choice (an experiment knob).
  static const int forced_bufs = [] {
    const char* e = std::getenv("ATK_TILE_BUFS");
    return e ? std::atoi(e) : 0;
  }();
  int bufs = per_block >= 512 ? 2 : 1;
  if (forced_bufs == 1 || forced_bufs == 2) bufs = forced_bufs;
  if (bufs == 2) ATK_LAUNCH_TILE(32, 2);
  else if (per_block <= 16) ATK_LAUNCH_TILE(16, 1);
  else if (per_block <= 32) ATK_LAUNCH_TILE(32, 1);
  else ATK_LAUNCH_TILE(64, 1);
#undef ATK_LAUNCH_TILE
  note_launch();
  if (cudaGetLastError() != cudaSuccess) return ATK_ERR_CUDA;
  if (pl.Z > 1) {
    int g = 1;                                   // lanes per bucket: about 8 planes per lane
    while (g < 32 && g * 8 < pl.Z) g *= 2;
    const long long blocks = (a.rows * a.b * g + 255) / 256;
    if (blocks >= (1ll << 31)) return ATK_ERR_TOO_LARGE;
    sweep_merge_planes_kernel<T, J, false><<<static_cast<unsigned>(blocks), 256, 0, a.stream>>>(
        static_cast<const Bits*>(p.part_vals), p.part_idx, p.z, g, a.rows, a.b, p.tiles, Shape::kCols, main_units,
        p.z_main, a.out_vals, a.out_idx, a.out_row_stride, a.out_format);
    note_launch();
    if (cudaGetLastError() != cudaSuccess) return ATK_ERR_CUDA;
  }
  return ATK_OK;
}

template <typename T>
int launch_tile_shared(const SweepLaunch& a) {
  switch (a.j) {
    case 2: return launch_tile_shared_j<T, 2>(a);
    case 3: return launch_tile_shared_j<T, 3>(a);
    case 4: return launch_tile_shared_j<T, 4>(a);
    default: return ATK_ERR_BAD_J;
  }
}

// Columns per thread.  A vector of V elements is loaded per stripe, so it must
// be aligned and lie inside one stripe.  The type's preferred vector (16 bytes;
// 8 bytes for 8-bit elements) by default; for elements of 16 bits or fewer,
// queues of three or four entries take half as many columns per thread, which
// halves their register footprint and doubles the number of threads that hide
// each other's latency.
template <typename T>
int launch_sweep(const SweepLaunch& a) {
  constexpr int s = static_cast<int>(sizeof(T));
  constexpr int kVec = ElemTraits<T>::kVec;
  if (a.rows <= 0 || a.b <= 0) return ATK_OK;
  auto fits = [&](int v) {
    const int bytes = v * s;
    return (reinterpret_cast<uintptr_t>(a.x) % bytes == 0) && ((a.row_stride * s) % bytes == 0) &&
           ((a.stripe_stride * s) % bytes == 0) && (a.b % v == 0);
  };
#ifndef ATK_NO_TILE_KERNEL
  if constexpr (ElemTraits<T>::kHalfFloat || std::is_same<T, float>::value) {
    // The shared-memory tile kernel: copies of 16 bytes need 16-byte aligned rows
    // and stripes and whole 16-byte pieces per stripe; with 16-bit elements the
    // stripe numbers must fit the packed entries.  16-bit floats: measured faster
    // than the insertion queues at every column length from 16 to 2048 stripes for
    // two to four entries per queue.  float32: for long columns, where the sweep
    // splits stripes over many threads and every split pays for warps that run the
    // insertion network at almost every stripe until their queues have warmed up.
    using Shape = TileShape<T>;
    const long long l_full = a.n / a.b;
    bool wanted = a.j >= 2 && !a.first_wins && fits(Shape::kPerPiece) && a.b >= Shape::kCols;
    if (sizeof(T) == 2) wanted = wanted && l_full + 1 <= kTileMaxStripes;
    else wanted = wanted && l_full >= (a.j == 2 ? ATK_TILE_FLOAT_MIN_STRIPES_J2 : ATK_TILE_FLOAT_MIN_STRIPES) &&
                    l_full + 1 < (1ll << 31);
    if (wanted) {
      const int rc = launch_tile_shared<T>(a);
      if (rc != kTileDeclined) return rc;
    }
  }
#endif
  if constexpr (sizeof(T) <= 2) {
    constexpr int kHalfVec = kVec / 2;
    if (a.j >= 3 && fits(kHalfVec)) return launch_by_j<T, kHalfVec>(a);
    if (fits(kVec)) return launch_by_j<T, kVec>(a);
    if (fits(kHalfVec)) return launch_by_j<T, kHalfVec>(a);
    return launch_by_j<T, 1>(a);
  } else {
    return fits(kVec) ? launch_by_j<T, kVec>(a) : launch_by_j<T, 1>(a);
  }
}

}  // namespace sweep_detail
}  // namespace atk
