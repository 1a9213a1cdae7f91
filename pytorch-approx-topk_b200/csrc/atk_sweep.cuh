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
#include "atk_tile.cuh"

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
  int vec_out;               // 16-byte stores are legal for the outputs (in their format)
  int out_format;            // ATK_OUT_*: how the final pairs are stored (the scratch planes are always int64)
  int vec_part;              // ... and for the scratch planes of the stripe split
  // Packed hand-off to the select (two-stage operator only): instead of values and
  // positions the kernel writes the queue entries themselves, rows x k0 words.
  uint32_t* out_keys;
  int vec_keys;              // 16-byte stores are legal for out_keys
  // Cross-block stripe split: z blocks share one (row, tile); block z walks
  // stripes [z*z_chunk, (z+1)*z_chunk) and writes its partial candidates to
  // plane z of the scratch buffers (dense [z][rows][k0]); a merge kernel
  // combines the planes.  z == 1: blocks write the outputs directly.
  int z;
  long long z_chunk;
  void* part_vals;
  long long* part_idx;
  // Tile kernel, one row: the first main_units (row, tile) units are split z_main ways
  // (1: scanned whole by one block each and written directly), the units after them z
  // ways; their blocks come last in the grid and fill the last, partial wave of the
  // launch with shorter blocks.  main_units == 0: every unit is split z ways.
  long long main_units;
  int z_main;
  long long z_chunk_main;
};

// Threads per block.  128 measured best on the headline workload (64: +2 %,
// 256: +4 %, 512: +15 % time); kept as a build knob.
#ifndef ATK_SWEEP_THREADS
#define ATK_SWEEP_THREADS 128
#endif
constexpr int kSweepMaxThreads = ATK_SWEEP_THREADS;
// Minimum resident blocks the compiler must allow for.  1 leaves it free to keep
// all loads of an unrolled batch in flight (more registers, fewer blocks).
#ifndef ATK_SWEEP_MINBLOCKS
#define ATK_SWEEP_MINBLOCKS 1
#endif

template <int V, int WORDS> struct SweepUnroll {
  // independent 16-byte loads kept in flight per thread; fewer when the
  // queues themselves take many registers
  static constexpr int kU = (V * WORDS <= 32) ? 8 : 4;
};

// Walk this thread's complete stripes (l_begin+ty, l_begin+ty+S, ... < lf) of its
// V columns starting at c0, feeding every 16-byte (or scalar) load to
// QS::consume.  Returns the first stripe number not visited (== lf for the
// thread that would own stripe lf).
template <typename T, typename QS, int V, bool SKIP>
__device__ __forceinline__ long long sweep_walk(QS (&qs)[V / QS::kCols], const SweepParams& p, const T* xrow,
                                                long long c0, int ty, int S, long long l_begin, long long lf) {
  using VL = VecLoad<T, V>;
  constexpr int U = SweepUnroll<V / QS::kCols, QS::kWords>::kU;
  const long long step = static_cast<long long>(S) * p.stripe_stride;
  long long l = l_begin + ty;
  const T* ptr = xrow + c0 + l * p.stripe_stride;
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

// How a thread scans its columns (template argument MODE of the kernel):
//   kScanQueues   insertion into the queues of Q, element by element;
//   kScanSimd     16-bit float inputs on the vector path: two-column SIMD queues
//                 that are converted to packed entries after the walk.
// (16-bit float inputs with enough columns take tile_kernel below instead.)
constexpr int kScanQueues = 0;
constexpr int kScanSimd = 1;

// Scan into q[V].
template <typename T, typename Q, int V, bool SKIP, int MODE>
__device__ __forceinline__ void sweep_scan(Q (&q)[V], const SweepParams& p, const T* xrow, long long c0,
                                           int ty, int S, int z) {
  // stripe range of this block (the whole column unless stripes are split over blocks)
  const long long l_begin = static_cast<long long>(z) * p.z_chunk;
  long long l_end = l_begin + p.z_chunk;
  if (l_end > p.l_full || z == p.z - 1) l_end = p.l_full;
  long long l;
  if constexpr (MODE == kScanSimd) {
    using QS = Simd16Queue<T, Q::kJ, Q::kFirst>;
    QS qs[V / 2];
#pragma unroll
    for (int i = 0; i < V / 2; ++i) qs[i].init();
    l = sweep_walk<T, QS, V, SKIP>(qs, p, xrow, c0, ty, S, l_begin, l_end);
#pragma unroll
    for (int e = 0; e < V; ++e)
#pragma unroll
      for (int j = 0; j < Q::kJ; ++j) q[e].k[j] = qs[e / 2].packed_key(j, e & 1);
  } else {
    l = sweep_walk<T, Q, V, SKIP>(q, p, xrow, c0, ty, S, l_begin, l_end);
  }
  // Ragged last stripe (b does not divide n): only columns < rem exist.  It
  // belongs to the split that would visit stripe l_full, and is that thread's
  // highest stripe, so scan order is preserved.
  if (p.rem > 0 && l == p.l_full && z == p.z - 1) {
    const T* last = xrow + p.l_full * p.stripe_stride + c0;
#pragma unroll
    for (int e = 0; e < V; ++e) {
      if (c0 + e < p.rem) q[e].push_tail(load_elem_bits<T>(last + e), static_cast<int>(p.l_full));
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

// Stores BYTES bytes from a 16-byte aligned local array to `dst`.  With `vec` the
// destination is known to be aligned to the widest power-of-two store (16, 8 or 4
// bytes) that divides BYTES; otherwise, and for odd sizes, element by element.
template <int BYTES, typename E>
__device__ __forceinline__ void store_run(E* dst, const E* src, bool vec) {
  constexpr int kStore = BYTES % 16 == 0 ? 16 : (BYTES % 8 == 0 ? 8 : (BYTES % 4 == 0 ? 4 : 0));
  if (kStore == 16 && vec) {
#pragma unroll
    for (int i = 0; i < BYTES / 16; ++i) st_out_16(reinterpret_cast<uint4*>(dst) + i, reinterpret_cast<const uint4*>(src)[i]);
  } else if (kStore == 8 && vec) {
#pragma unroll
    for (int i = 0; i < BYTES / 8; ++i) reinterpret_cast<uint2*>(dst)[i] = reinterpret_cast<const uint2*>(src)[i];
  } else if (kStore == 4 && vec) {
#pragma unroll
    for (int i = 0; i < BYTES / 4; ++i) reinterpret_cast<uint32_t*>(dst)[i] = reinterpret_cast<const uint32_t*>(src)[i];
  } else {
#pragma unroll
    for (int i = 0; i < BYTES / static_cast<int>(sizeof(E)); ++i) dst[i] = src[i];
  }
}

// Write-out of a thread's V queues: the J candidates of bucket c go to slots
// c*J .. c*J+J-1 in ascending queue order -- as packed entries for the select, as
// partial candidates of plane z (stripes split over blocks), or as final pairs in
// the output format of the call.
template <typename T, typename Q, int J, int V, bool PACKED_OUT>
__device__ __forceinline__ void sweep_write_out(const SweepParams& p, Q (&q)[V], const T* xrow, long long row,
                                                long long c0, int z, int planes) {
  using Tr = ElemTraits<T>;
  using Bits = typename Tr::Bits;
  if constexpr (PACKED_OUT) {
    // The queue entries go to the select as they are: (image of the value, stripe)
    // words, bucket c in slots c*J .. c*J+J-1, ascending.
    static_assert(Q::kPacked, "only packed queues have entries to hand over");
    __align__(16) uint32_t ok[V * J];
#pragma unroll
    for (int e = 0; e < V; ++e)
#pragma unroll
      for (int j = 0; j < J; ++j) ok[e * J + j] = q[e].k[j];
    uint32_t* kdst = p.out_keys + row * (p.b * J) + c0 * J;
    if ((V * J) % 4 == 0 && p.vec_keys) {
#pragma unroll
      for (int i = 0; i < V * J / 4; ++i)
        st_out_16(reinterpret_cast<uint4*>(kdst) + i, reinterpret_cast<const uint4*>(ok)[i]);
    } else {
#pragma unroll
      for (int i = 0; i < V * J; ++i) kdst[i] = ok[i];
    }
    return;
  }

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
        ov[e * J + j] = q[e].value_bits(j, xrow != nullptr ? xrow + stripe * p.stripe_stride + c0 + e : nullptr);
        oi[e * J + j] = stripe * p.idx_stride + p.idx_offset + c0 + e;
      }
    }
  // direct to the outputs, or to plane z of the scratch when stripes are split over blocks
  const long long k0 = p.b * J;
  // The thread's V*J entries are contiguous in every output array and start at a
  // multiple of their total size there, so the widest store that divides that size
  // is aligned whenever the buffers and their row strides are 16-byte aligned.
  if (planes == 1 && p.out_format != ATK_OUT_I64) {
    const long long out_base = row * p.out_row_stride + c0 * J;
    if (p.out_format == ATK_OUT_REC32) {
      // records {value bits zero-extended to 32 bits, int32 position}
      __align__(16) uint2 rec[V * J];
#pragma unroll
      for (int i = 0; i < V * J; ++i)
        rec[i] = make_uint2(static_cast<uint32_t>(ov[i]), static_cast<uint32_t>(static_cast<int>(oi[i])));
      store_run<V * J * 8>(static_cast<uint2*>(p.out_vals) + out_base, rec, p.vec_out);
    } else {
      __align__(16) int oi32[V * J];
#pragma unroll
      for (int i = 0; i < V * J; ++i) oi32[i] = static_cast<int>(oi[i]);
      store_run<V * J * static_cast<int>(sizeof(Bits))>(static_cast<Bits*>(p.out_vals) + out_base, ov, p.vec_out);
      store_run<V * J * 4>(reinterpret_cast<int*>(p.out_idx) + out_base, oi32, p.vec_out);
    }
    return;
  }
  const long long out_base = planes > 1 ? (static_cast<long long>(z) * p.rows + row) * k0 + c0 * J
                                     : row * p.out_row_stride + c0 * J;
  Bits* vdst = static_cast<Bits*>(planes > 1 ? p.part_vals : p.out_vals) + out_base;
  long long* idst = (planes > 1 ? p.part_idx : p.out_idx) + out_base;
  const bool vec = planes > 1 ? p.vec_part : p.vec_out;
  store_run<V * J * static_cast<int>(sizeof(Bits))>(vdst, ov, vec);
  store_run<V * J * 8>(idst, oi, vec);
}

// ---------------------------------------------------------------------------
// Stage 1 only: every block handles one tile of columns of one row and writes
// the J candidates of each bucket (slot = bucket*J + q, ascending).
template <typename T, typename Q, int J, int V, bool SKIP, int MODE, bool PACKED_OUT>
__global__ void __launch_bounds__(kSweepMaxThreads, ATK_SWEEP_MINBLOCKS)
sweep_kernel(const SweepParams p) {
  using Tr = ElemTraits<T>;
  using Bits = typename Tr::Bits;
  extern __shared__ __align__(16) uint32_t sweep_smem[];
  // Launched overlapped with the end of the kernel before it in the stream: nothing is
  // read or written before that kernel has finished.
  grid_dependency_wait();

  const int tx = threadIdx.x;
  const int ty = threadIdx.y;
  const int S = p.s;
  const long long unit = static_cast<long long>(blockIdx.x) / p.z;        // (row, tile)
  const int z = static_cast<int>(static_cast<long long>(blockIdx.x) - unit * p.z);
  const long long row = unit / p.tiles;
  const long long tile = unit - row * p.tiles;
  const long long c0 = (tile * p.cw + tx) * V;
  const bool active = c0 < p.b;
  const T* xrow = static_cast<const T*>(p.x) + row * p.row_stride;

  Q q[V];
#pragma unroll
  for (int e = 0; e < V; ++e) q[e].init();

  if (active) sweep_scan<T, Q, V, SKIP, MODE>(q, p, xrow, c0, ty, S, z);
  if (S > 1) sweep_merge<Q, V>(q, sweep_smem, p.cw, tx, ty, S);
  if (!active || ty != 0) return;
  // The kernel after this one (the select that reads the packed entries, or the next
  // call's stage 1) may come onto the GPU once every block has finished scanning; it
  // waits for this kernel's end before it touches memory.  (Announcing it at the start of
  // the kernel measured slower: early blocks of the select pile up on the SMs that ran
  // out of stage-1 work first.)
  grid_launch_dependents();
  sweep_write_out<T, Q, J, V, PACKED_OUT>(p, q, xrow, row, c0, z, p.z);
}

// ---------------------------------------------------------------------------
// Stage 1 through shared-memory tiles (16-bit floats and float32): a block of 128
// threads stages a tile of 512 bytes x CH stripes in shared memory with
// asynchronous 16-byte copies (cp.async, global -> shared without passing through
// registers) and every thread runs the two-pass scan of atk_tile.cuh on its
// word of every stripe (two 16-bit columns, or one float32 column).  Longer
// columns take several chunks of CH stripes; the stripes of a column can also be
// split over p.z blocks that write partial candidates to scratch planes (p.s is
// 1).  Needs rows and stripes that are 16-byte aligned and a bucket count that is
// a multiple of 16 bytes' worth of elements.
constexpr int kTileThreads = 128;
template <typename T> struct TileShape {
  static constexpr int kColsPerThread = sizeof(T) == 2 ? 2 : 1;
  static constexpr int kCols = kTileThreads * kColsPerThread;       // columns of a tile: 512 bytes per stripe
  static constexpr int kPerPiece = 16 / static_cast<int>(sizeof(T));  // elements per 16-byte copy
};
// Resident blocks the compiler must allow for (a build knob for measurements).
#ifndef ATK_TILE_MINBLOCKS
#define ATK_TILE_MINBLOCKS 6
#endif

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gmem_src) {
  const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::: "memory"); }
// all groups of this thread but the one committed last have arrived
__device__ __forceinline__ void cp_async_wait_but_one() { asm volatile("cp.async.wait_group 1;\n" ::: "memory"); }

template <typename T, int J> struct TileQueue {
  using type = PackedQueue<T, J, false>;
};
template <int J> struct TileQueue<float, J> {
  using type = FloatQueue<float, J, false>;
};

template <typename T, int J, int CH, bool PACKED_OUT, int BUFS>
__global__ void __launch_bounds__(kTileThreads, ATK_TILE_MINBLOCKS)
tile_kernel(const SweepParams p) {
  using Q = typename TileQueue<T, J>::type;
  using Shape = TileShape<T>;
  constexpr int V = Shape::kColsPerThread;
  extern __shared__ __align__(16) uint32_t tile_smem[];     // BUFS buffers of CH x kTileThreads words
  grid_dependency_wait();   // see sweep_kernel
  const int tx = threadIdx.x;
  // (row, tile) unit and stripe split of this block: the first p.main_units units whole,
  // the units after them in p.z splits each
  long long unit;
  int z, planes;
  long long chunk;
  {
    const long long blk = static_cast<long long>(blockIdx.x);
    const long long main_blocks = p.main_units * p.z_main;
    if (blk < main_blocks) {
      unit = blk / p.z_main;
      z = static_cast<int>(blk - unit * p.z_main);
      planes = p.z_main;
      chunk = p.z_chunk_main;
    } else {
      const long long t = blk - main_blocks;
      unit = p.main_units + t / p.z;
      z = static_cast<int>(t - (unit - p.main_units) * p.z);
      planes = p.z;
      chunk = p.z_chunk;
    }
  }
  const long long row = unit / p.tiles;
  const long long tile = unit - row * p.tiles;
  const long long tile_c0 = tile * Shape::kCols;
  const long long c0 = tile_c0 + V * tx;
  const bool active = c0 < p.b;
  const T* xrow = static_cast<const T*>(p.x) + row * p.row_stride;
  long long wcols = p.b - tile_c0;                           // columns of this tile (whole 16-byte pieces)
  if (wcols > Shape::kCols) wcols = Shape::kCols;
  const int pieces_per_stripe = static_cast<int>(wcols / Shape::kPerPiece);
  // stripe range of this block (the whole column unless stripes are split over blocks)
  const long long l_begin = static_cast<long long>(z) * chunk;
  long long l_end = l_begin + chunk;
  if (l_end > p.l_full || z == planes - 1) l_end = p.l_full;

  Q q[V];
#pragma unroll
  for (int e = 0; e < V; ++e) q[e].init();
  // Long columns (BUFS = 2) go through two buffers of CH stripes in turns: the
  // copies of chunk c + 1 are in flight while chunk c is scanned.  Columns of a few
  // chunks use one buffer of twice the stripes instead (the threshold of a longer first
  // chunk lets fewer elements through, which measured better up to 256 stripes).
  constexpr int bufs = BUFS;
  const int n_chunks = l_end > l_begin ? static_cast<int>((l_end - l_begin + CH - 1) / CH) : 0;
  auto issue = [&](int c) {
    const long long l0 = l_begin + static_cast<long long>(c) * CH;
    const int cnt = l_end - l0 < CH ? static_cast<int>(l_end - l0) : CH;
    uint32_t* buf = tile_smem + (c & (bufs - 1)) * (CH * kTileThreads);
    const int pieces = cnt * pieces_per_stripe;
    const T* src = xrow + l0 * p.stripe_stride + tile_c0;
    if (pieces_per_stripe == kTileThreads / 4) {
      for (int piece = tx; piece < pieces; piece += kTileThreads)
        cp_async_16(buf + (piece >> 5) * kTileThreads + (piece & 31) * 4,
                    src + static_cast<long long>(piece >> 5) * p.stripe_stride + (piece & 31) * Shape::kPerPiece);
    } else {
      for (int piece = tx; piece < pieces; piece += kTileThreads) {
        const int i = piece / pieces_per_stripe;
        const int c4 = piece - i * pieces_per_stripe;
        cp_async_16(buf + i * kTileThreads + c4 * 4,
                    src + static_cast<long long>(i) * p.stripe_stride + c4 * Shape::kPerPiece);
      }
    }
    cp_async_commit();
  };
  if (n_chunks > 0) issue(0);
  for (int c = 0; c < n_chunks; ++c) {
    if (bufs == 2 && c + 1 < n_chunks) {
      issue(c + 1);
      cp_async_wait_but_one();
    } else {
      cp_async_wait_all();
    }
    __syncthreads();                                         // chunk c is in shared memory for every thread
    if (active) {
      const long long l0 = l_begin + static_cast<long long>(c) * CH;
      const int cnt = l_end - l0 < CH ? static_cast<int>(l_end - l0) : CH;
      const uint32_t* words = tile_smem + (c & (bufs - 1)) * (CH * kTileThreads) + tx;
      const int lf = static_cast<int>(l0);
      const bool first = c == 0;
      if constexpr (sizeof(T) == 2) {
        if (first) {
          if (cnt == CH) tile_chunk_shared<T, J, CH, kTileThreads, true, true>(q, words, cnt, lf);
          else tile_chunk_shared<T, J, CH, kTileThreads, false, true>(q, words, cnt, lf);
        } else {
          if (cnt == CH) tile_chunk_shared<T, J, CH, kTileThreads, true, false>(q, words, cnt, lf);
          else tile_chunk_shared<T, J, CH, kTileThreads, false, false>(q, words, cnt, lf);
        }
      } else {
        if (first) {
          if (cnt == CH) tile_chunk_shared_f32<J, CH, kTileThreads, true, true>(q[0], words, cnt, lf);
          else tile_chunk_shared_f32<J, CH, kTileThreads, false, true>(q[0], words, cnt, lf);
        } else {
          if (cnt == CH) tile_chunk_shared_f32<J, CH, kTileThreads, true, false>(q[0], words, cnt, lf);
          else tile_chunk_shared_f32<J, CH, kTileThreads, false, false>(q[0], words, cnt, lf);
        }
      }
    }
    if (c + bufs < n_chunks) __syncthreads();                // chunk c has been read: its buffer is filled again
    if (bufs == 1 && c + 1 < n_chunks) issue(c + 1);
  }
  if (!active) return;
  // ragged last stripe (b does not divide n): only columns < rem exist; it belongs to the last split
  if (p.rem > 0 && z == planes - 1) {
    const T* last = xrow + p.l_full * p.stripe_stride + c0;
#pragma unroll
    for (int e = 0; e < V; ++e)
      if (c0 + e < p.rem) q[e].push_tail(load_elem_bits<T>(last + e), static_cast<int>(p.l_full));
  }
  grid_launch_dependents();   // see sweep_kernel
  sweep_write_out<T, Q, J, V, PACKED_OUT>(p, q, xrow, row, c0, z, planes);
}

// Combine the z partial candidate planes written by a stripe-split sweep: a
// group of g lanes per (row, bucket) (g = 1 for a few planes, up to a whole
// warp for many); lane l ranks the entries of planes l, l+g, ... by value, then
// by position (later wins; earlier with FIRST), the lanes merge by
// xor-shuffles, and lane 0 writes the best J in ascending order — exactly what
// one block walking the whole column would have produced.
template <typename T, int J, bool FIRST>
struct PlaneEntryQueue {
  using Bits = typename ElemTraits<T>::Bits;
  using C = typename ElemTraits<T>::Compute;
  C v[J];
  long long i[J];
  Bits b[J];   // raw bits travel with the entries so NaN payloads survive
  __device__ __forceinline__ void init() {
#pragma unroll
    for (int q = 0; q < J; ++q) {
      v[q] = ElemTraits<T>::floor();
      i[q] = FIRST ? 0x7fffffffffffffffll : -1ll;
      b[q] = ElemTraits<T>::narrow(ElemTraits<T>::floor());
    }
  }
  __device__ __forceinline__ void push(C nv, long long ni, Bits nb) {
    bool p[J + 1];
#pragma unroll
    for (int q = 0; q < J; ++q) p[q] = (nv > v[q]) || (nv == v[q] && (FIRST ? ni < i[q] : ni > i[q]));
    p[J] = false;
#pragma unroll
    for (int q = 0; q < J; ++q) {
      const int up = q + 1 < J ? q + 1 : q;
      const C tv = p[q + 1] ? v[up] : (p[q] ? nv : v[q]);
      const long long ti = p[q + 1] ? i[up] : (p[q] ? ni : i[q]);
      const Bits tb = p[q + 1] ? b[up] : (p[q] ? nb : b[q]);
      v[q] = tv;
      i[q] = ti;
      b[q] = tb;
    }
  }
};

// xor-shuffle of a raw element word of any width
template <typename B>
__device__ __forceinline__ B shfl_xor_bits(B v, int off) {
  if constexpr (sizeof(B) == 8)
    return static_cast<B>(__shfl_xor_sync(0xffffffffu, static_cast<unsigned long long>(v), off));
  else
    return static_cast<B>(__shfl_xor_sync(0xffffffffu, static_cast<uint32_t>(v), off));
}

template <typename T, int J, bool FIRST>
__global__ void __launch_bounds__(256)
sweep_merge_planes_kernel(const typename ElemTraits<T>::Bits* __restrict__ part_vals,
                          const long long* __restrict__ part_idx, int z, int g /* lanes per bucket */,
                          long long rows, long long b, long long tiles, int tile_cols,
                          long long main_units /* (row, tile) units before this one have z_main planes */,
                          int z_main, void* __restrict__ out_vals, void* __restrict__ out_idx,
                          long long out_row_stride, int out_format) {
  using Tr = ElemTraits<T>;
  using Bits = typename Tr::Bits;
  const int lane = threadIdx.x % g;            // g is a power of two <= 32, groups never straddle warps
  const long long unit = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) / g;
  bool valid = unit < rows * b;                // whole warps stay for the shuffles
  const long long row = valid ? unit / b : 0;
  const long long c = valid ? unit - row * b : 0;
  if (row * tiles + c / tile_cols < main_units) z = z_main;
  valid = valid && z > 1;                      // a unit that was not split wrote its buckets itself
  const long long k0 = b * J;
  PlaneEntryQueue<T, J, FIRST> q;
  q.init();
  if (valid) {
    for (int zz = lane; zz < z; zz += g) {
      const long long base = (static_cast<long long>(zz) * rows + row) * k0 + c * J;
#pragma unroll
      for (int j = 0; j < J; ++j) {
        const Bits bits = part_vals[base + j];
        q.push(Tr::widen(bits), part_idx[base + j], bits);
      }
    }
  }
  for (int off = g >> 1; off >= 1; off >>= 1) {
    typename Tr::Compute ov[J];
    long long oi[J];
    Bits ob[J];
#pragma unroll
    for (int j = 0; j < J; ++j) {
      ov[j] = __shfl_xor_sync(0xffffffffu, q.v[j], off);
      oi[j] = __shfl_xor_sync(0xffffffffu, q.i[j], off);
      ob[j] = shfl_xor_bits<Bits>(q.b[j], off);
    }
#pragma unroll
    for (int j = 0; j < J; ++j) q.push(ov[j], oi[j], ob[j]);
  }
  if (!valid || lane != 0) return;
  const OutRow<Bits> orow(out_vals, out_idx, row, out_row_stride, out_format);
#pragma unroll
  for (int j = 0; j < J; ++j) orow.put(c * J + j, q.b[j], q.i[j]);
}

// ---- launch shape (host) -------------------------------------------------------
namespace sweep_detail {
inline long long floor_pow2(long long v) {
  long long r = 1;
  while (r * 2 <= v) r *= 2;
  return r;
}
inline long long ceil_pow2(long long v) {
  long long r = 1;
  while (r < v) r *= 2;
  return r;
}

inline size_t align256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

struct SweepPlan {
  long long cw, tiles, S, Z, z_chunk;
};

// Most entries a queue holds (J <= kMaxJ); every block of a stripe split must
// walk at least that many complete stripes per in-block split, so that no
// never-filled queue slot reaches the scratch planes (a never-filled packed
// entry would decode to a made-up element there).
constexpr long long kMaxJ = 4;

// Equal stripe ranges for Z blocks, with Z lowered so that every range holds at
// least kMaxJ stripes for each of the S in-block splits.  The last block walks
// to the end of the column (and owns the ragged last stripe), so a short
// remainder is folded into it instead of getting a block of its own.
inline void set_chunks(SweepPlan& pl, long long l_full) {
  if (pl.Z < 1) pl.Z = 1;
  const long long least = kMaxJ * (pl.S > 0 ? pl.S : 1);
  pl.z_chunk = (l_full + pl.Z - 1) / pl.Z;
  if (pl.z_chunk < least) pl.z_chunk = least;
  long long used = (l_full + pl.z_chunk - 1) / pl.z_chunk;
  while (used > 1 && l_full - (used - 1) * pl.z_chunk < least) --used;
  pl.Z = used >= 1 ? used : 1;
}

// Columns at least this long are never given narrower tiles for in-block splits
// (a build knob for measurements).
#ifndef ATK_TRADE_MAX_STRIPES
#define ATK_TRADE_MAX_STRIPES 2048
#endif
constexpr long long kTradeMaxStripes = ATK_TRADE_MAX_STRIPES;

// Threads across columns, stripe splits inside a block (S) and over blocks (Z).
// Splitting happens only when the columns alone cannot fill the machine, and
// never beyond what the block size or the stripe count allow.
inline SweepPlan plan_sweep(long long rows, long long b, long long l_full, int V, int sm_count) {
  SweepPlan pl;
  const long long col_threads = (b + V - 1) / V;
  pl.cw = col_threads < kSweepMaxThreads ? col_threads : kSweepMaxThreads;
  pl.tiles = (col_threads + pl.cw - 1) / pl.cw;
  pl.S = 1;
  pl.Z = 1;
  const long long want_threads = static_cast<long long>(sm_count) * 1024;
  long long have_threads = rows * pl.tiles * pl.cw;
  if (have_threads < want_threads && l_full >= 8) {
    const long long by_block = floor_pow2(kSweepMaxThreads / pl.cw);
    const long long by_work = floor_pow2(l_full / 4);
    const long long by_need = ceil_pow2((want_threads + have_threads - 1) / have_threads);
    pl.S = by_block;
    if (by_work < pl.S) pl.S = by_work;
    if (by_need < pl.S) pl.S = by_need;
    if (pl.S < 1) pl.S = 1;
    // A full-width block leaves no room for splits: trade columns for splits
    // (narrower tiles, more of them) while at least a warp of columns remains.
    // Not for long columns: those are split over blocks below, which keeps the
    // blocks reading full-width (2 KiB) pieces of every stripe.
    while (l_full < kTradeMaxStripes && pl.S < by_need && pl.S < by_work && pl.cw >= 64 && pl.cw % 2 == 0) {
      pl.cw /= 2;
      pl.S *= 2;
    }
    pl.tiles = (col_threads + pl.cw - 1) / pl.cw;
  }
  have_threads *= pl.S;
  // Over blocks: only when a thread would otherwise walk a long column (a
  // second launch merges the planes, which costs more than it saves on short
  // ones); every block keeps at least 32 stripes per in-block split.
  if (have_threads * 2 <= want_threads && l_full / pl.S >= 256) {
    long long z = want_threads / have_threads;
    const long long by_work = l_full / (pl.S * 32);
    if (by_work < z) z = by_work;
    if (z > 1024) z = 1024;
    if (z >= 2) pl.Z = z;
  }
  set_chunks(pl, l_full);
  return pl;
}

}  // namespace sweep_detail

// Stripe split of the tile kernel: enough blocks for about two waves of its six
// resident blocks per SM, every split at least 256 stripes long.
inline long long tile_split(long long rows, long long tiles, long long l_full, int sm_count) {
  const long long units = rows * tiles;
  if (units <= 0) return 1;
  long long z = (12ll * sm_count + units - 1) / units;
  const long long by_work = l_full / 256;
  if (z > by_work) z = by_work;
  if (z > 64) z = 64;
  return z < 1 ? 1 : z;
}

// Which (row, tile) units of the tile kernel are split, for columns long enough to split.
// Enough units to fill the GPU at least once: the units of the complete waves are scanned
// whole (no partial candidates, no merge, every queue warms up once), and only the units
// left over for the last, partial wave are split -- as many ways as fit that wave, so that
// it is full and short.  Fewer units: the first wave is units split ceil(capacity / units)
// ways, the rest is split further.  Otherwise every unit is split tile_split() ways.
struct TilePlan {
  long long main_units;   // units split z_main ways, first in the grid
  long long z_main;
  long long z;            // splits of each of the other units
};
inline TilePlan tile_plan(long long rows, long long tiles, long long l_full, int sm_count) {
  TilePlan tp{0, 1, tile_split(rows, tiles, l_full, sm_count)};
  const long long cap = 6ll * sm_count;                      // resident blocks of the tile kernel
  const long long units = rows * tiles;                      // (row, tile) units, row-major
  long long zmax = l_full / 256;
  if (zmax > 64) zmax = 64;
  // columns of 1024 stripes and more: below that the blocks are short anyway and the merge
  // launch costs more than the last wave gains (fp16 256 x 2^20, 512 stripes: 98 -> 105 us)
  if (units <= 0 || cap <= 0 || zmax < 4) return tp;
  // one full wave (or several) of equal blocks first ...
  long long z1 = units >= cap ? 1 : (cap + units - 1) / units;
  if (z1 > zmax) return tp;                                  // few units: every one split as far as it goes
  const long long main_units = units >= cap ? (units / cap) * cap : cap / z1;
  const long long rest = units - main_units;
  if (rest <= 0) {
    tp.z = z1;
    return tp;
  }
  // ... then the units left over, split as many ways as fill one more wave
  long long z2 = cap / rest;
  if (z2 > zmax) z2 = zmax;
  if (z2 <= z1) {
    // The left-over units cannot be split further than the others (short columns): every
    // unit the same number of ways, whichever of "just under one wave" and "just over" needs
    // less time (waves x stripes per block).
    const long long zf = cap / units;                        // 0 when there are more units than blocks
    if (zf >= 1 && zf < z1 && z1 < zf * ((units * z1 + cap - 1) / cap)) tp.z = zf;   // 1 / zf < waves / z1
    else tp.z = z1;
    return tp;
  }
  tp.main_units = main_units;
  tp.z_main = z1;
  tp.z = z2;
  return tp;
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
  int out_format = ATK_OUT_I64;   // format of out_vals / out_idx (out_idx is then an int* for ATK_OUT_I32)
  void* workspace;          // optional scratch for splitting stripes over blocks (may be null)
  size_t workspace_bytes;
  uint32_t* out_keys;       // non-null: hand the packed queue entries to the select instead of out_vals / out_idx
  cudaStream_t stream;
};

// Returned (nothing launched) when packed entries were asked for and this shape or
// element type has none to give: the caller uses the plain outputs instead.
constexpr int kPackedUnavailable = 1;

// Scratch the stripe split over blocks would like for this shape, assuming the
// widest vector path (0 when the shape fills the GPU without it).  The launch
// uses as many planes as the scratch it is given holds.
inline size_t sweep_workspace_bytes(int elem_size, long long rows, long long n, long long b, int j, int sm_count) {
  if (rows <= 0 || b <= 0 || n < b) return 0;
  const int vec = elem_size == 1 ? 8 : 16 / elem_size;   // ElemTraits<T>::kVec by element size
  const sweep_detail::SweepPlan pl = sweep_detail::plan_sweep(rows, b, n / b, (j >= 3 && elem_size <= 2) ? vec / 2 : vec, sm_count);
  long long planes = pl.Z;
  if (elem_size == 2 || elem_size == 4) {
    // the shared-memory tile kernel (16-bit floats, float32) splits long columns too
    const long long tile_cols = elem_size == 2 ? 256 : 128;
    const TilePlan tp = tile_plan(rows, (b + tile_cols - 1) / tile_cols, n / b, sm_count);
    const long long zt = tp.z > tp.z_main ? tp.z : tp.z_main;
    if (zt > planes) planes = zt;
  }
  if (planes <= 1) return 0;
  const size_t k0 = static_cast<size_t>(b) * j;
  return sweep_detail::align256(static_cast<size_t>(planes) * rows * k0 * elem_size) +
         static_cast<size_t>(planes) * rows * k0 * 8 + 256;
}

int launch_sweep_f32(const SweepLaunch& a);
int launch_sweep_f16(const SweepLaunch& a);
int launch_sweep_bf16(const SweepLaunch& a);
int launch_sweep_f64(const SweepLaunch& a);
int launch_sweep_i32(const SweepLaunch& a);
int launch_sweep_i64(const SweepLaunch& a);
int launch_sweep_i16(const SweepLaunch& a);
int launch_sweep_i8(const SweepLaunch& a);
int launch_sweep_u8(const SweepLaunch& a);

}  // namespace atk
