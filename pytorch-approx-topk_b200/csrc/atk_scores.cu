// Fused score producer for the attention-score use case: the scores
// q . K^T * scale of one query per row against the row's n keys are computed on
// the fly and fed to the bucketed stage 1, so the rows x n score matrix is never
// written to or read from memory.  The reference has no counterpart (its users
// run a matrix product first and pass the scores to approx_topk.topk; the
// paper's key-selection experiments, notebooks/20240915-paper-figures.ipynb
// cells 6-7); the result equals the operator applied to the scores rounded to
// the element type, with the accumulation order stated below.
//
// A block of 128 threads owns a tile of 256 buckets (columns) of one row; a warp
// owns 64 of them, i.e. 64 adjacent keys per stripe.  For a chunk of 64 stripes the
// warp computes those scores together (score_stripe: warp-wide matrix instructions
// fed straight from 16-byte loads of K), parks them in shared memory, and then
// every thread runs the two-pass scan of atk_tile.cuh on the words of its own two
// columns as it does on staged input.  Two forms on the FMA pipe were measured
// first and dropped as instruction-bound: every thread reading its own two keys
// (8.5 warp instructions per key, uncoalesced: 4.4 TB/s of key reads) and d/8 lanes
// per key with a shuffle butterfly (16 per key, coalesced: 4.8 TB/s); cuBLAS'
// batched product reads the keys at 7.0 TB/s.
#include "atk_select.cuh"
#include "atk_sweep.cuh"

namespace atk {
namespace {

template <typename T> struct ScoreConv;
template <> struct ScoreConv<__nv_bfloat16> {
  // the two elements of a 32-bit word of K as floats (low address first)
  static __device__ __forceinline__ void widen2(uint32_t w, float& lo, float& hi) {
    lo = __uint_as_float(w << 16);
    hi = __uint_as_float(w & 0xffff0000u);
  }
  static __device__ __forceinline__ float widen1(uint16_t bits) { return __uint_as_float(static_cast<uint32_t>(bits) << 16); }
  static __device__ __forceinline__ uint32_t narrow(float f) {
    return static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(f)));
  }
};
template <> struct ScoreConv<__half> {
  static __device__ __forceinline__ void widen2(uint32_t w, float& lo, float& hi) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
    lo = f.x;
    hi = f.y;
  }
  static __device__ __forceinline__ float widen1(uint16_t bits) { return __half2float(__ushort_as_half(bits)); }
  static __device__ __forceinline__ uint32_t narrow(float f) {
    return static_cast<uint32_t>(__half_as_ushort(__float2half_rn(f)));
  }
};

struct ScoreParams {
  const void* q;        // rows x d
  const void* keys;     // rows x n x d
  long long q_row_stride, keys_row_stride;   // elements
  float scale;
  SweepParams sweep;    // geometry and outputs (x unused)
};

// One warp-wide matrix instruction: D(16x8, f32) += A(16x16) * B(16x8), 16-bit
// float inputs.  The legacy mma.sync form is used on purpose: its operands are
// plain registers, so the keys go from global memory straight into fragment
// registers with 16-byte loads and no staging, and the product is bound by the
// key reads (2 bytes per multiply-add), far from any tensor-core limit.
template <typename T> struct ScoreMma;
template <> struct ScoreMma<__nv_bfloat16> {
  static __device__ __forceinline__ void mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
};
template <> struct ScoreMma<__half> {
  static __device__ __forceinline__ void mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
};

// Scores of the 64 keys a warp owns in one stripe (its 32 threads x 2 columns; the
// keys are 64*D contiguous elements of K), 16 keys at a time.  Lane (g, c) = (lane
// / 4, lane % 4) loads 16 bytes = dimensions 32s + 8c .. +7 of keys g and g + 8
// for every step s of 32 dimensions: a load instruction of the warp covers 64
// contiguous bytes of each of 8 keys.  The four words of such a load are the
// A-fragment registers of two matrix instructions whose 16 "k" positions stand for
// the lane quads' dimensions in that order; B holds the query's words at the same
// dimensions in every one of its 8 columns, so every column of the result is the
// dot product and lane (g, 0) ends up with the scores of keys g and g + 8 (float32
// accumulation inside the instruction).  It scales, rounds to the element type and
// stores the 16-bit scores where the threads that own the columns will read them.
template <typename T, int D>
__device__ __forceinline__ void score_stripe(const T* kstripe /* first key of the warp */, int valid /* keys that exist */,
                                             const uint32_t (&qb)[D / 8], float scale, uint16_t* out /* 64 halves */,
                                             int lane) {
  using C = ScoreConv<T>;
  constexpr int STEPS = D / 32;
  const int g = lane >> 2, c = lane & 3;
  const T* lane_ptr = kstripe + static_cast<long long>(g) * D + c * 8;
#pragma unroll
  for (int m = 0; m < 4; ++m) {                  // 16 keys: 16m + g and 16m + g + 8
    const bool has_x = 16 * m + g < valid, has_y = 16 * m + g + 8 < valid;
    uint4 x[STEPS], y[STEPS];
#pragma unroll
    for (int s = 0; s < STEPS; ++s) {
      x[s] = make_uint4(0u, 0u, 0u, 0u);
      y[s] = make_uint4(0u, 0u, 0u, 0u);
      if (has_x) x[s] = *reinterpret_cast<const uint4*>(lane_ptr + static_cast<long long>(16 * m) * D + 32 * s);
      if (has_y) y[s] = *reinterpret_cast<const uint4*>(lane_ptr + static_cast<long long>(16 * m + 8) * D + 32 * s);
    }
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int s = 0; s < STEPS; ++s) {
      ScoreMma<T>::mma(acc, x[s].x, y[s].x, x[s].y, y[s].y, qb[4 * s + 0], qb[4 * s + 1]);
      ScoreMma<T>::mma(acc, x[s].z, y[s].z, x[s].w, y[s].w, qb[4 * s + 2], qb[4 * s + 3]);
    }
    if (c == 0) {
      const uint16_t none = static_cast<uint16_t>(Half2Ops<T>::kNegInf2 & 0xffffu);
      out[16 * m + g] = has_x ? static_cast<uint16_t>(C::narrow(acc[0] * scale)) : none;
      out[16 * m + g + 8] = has_y ? static_cast<uint16_t>(C::narrow(acc[2] * scale)) : none;
    }
  }
}

constexpr int kScoreChunk = 64;

template <typename T, int J, int D>
__global__ void __launch_bounds__(kTileThreads, 4)
score_tile_kernel(const ScoreParams sp) {
  using Q = PackedQueue<T, J, false>;
  const SweepParams& p = sp.sweep;
  extern __shared__ __align__(16) uint32_t tile_smem[];     // kScoreChunk x kTileThreads words
  const int tx = threadIdx.x;
  const int lane = tx & 31;
  const int warp = tx >> 5;
  const long long row = static_cast<long long>(blockIdx.x) / p.tiles;
  const long long tile = static_cast<long long>(blockIdx.x) - row * p.tiles;
  const long long c0 = tile * (2 * kTileThreads) + 2 * tx;
  const long long warp_c0 = tile * (2 * kTileThreads) + 64 * warp;    // first column of this warp
  if (warp_c0 >= p.b) return;                    // whole warps only: the shuffles below need all lanes
  const bool active = c0 < p.b;
  const bool second = c0 + 1 < p.b;              // an odd bucket count leaves the last thread one column
  const T* qrow = static_cast<const T*>(sp.q) + row * sp.q_row_stride;
  const T* krow = static_cast<const T*>(sp.keys) + row * sp.keys_row_stride;
  // the query's words at this lane's dimensions: B fragments of every step (see score_stripe)
  uint32_t qv[D / 8];
#pragma unroll
  for (int s = 0; s < D / 32; ++s)
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const uint16_t* qh = reinterpret_cast<const uint16_t*>(qrow) + 32 * s + 8 * (lane & 3) + 2 * w;
      qv[4 * s + w] = static_cast<uint32_t>(qh[0]) | (static_cast<uint32_t>(qh[1]) << 16);
    }
  long long cols_left = p.b - warp_c0;
  const int valid = cols_left > 64 ? 64 : static_cast<int>(cols_left);

  Q q[2];
  q[0].init();
  q[1].init();
  uint32_t* words = tile_smem + tx;
  uint16_t* warp_halves = reinterpret_cast<uint16_t*>(tile_smem + 32 * warp);   // + i * 2 * kTileThreads per stripe
  for (long long l0 = 0; l0 < p.l_full; l0 += kScoreChunk) {
    const int cnt = p.l_full - l0 < kScoreChunk ? static_cast<int>(p.l_full - l0) : kScoreChunk;
    __syncwarp();                                 // the previous chunk's words have been read
    for (int i = 0; i < cnt; ++i)
      score_stripe<T, D>(krow + ((l0 + i) * p.b + warp_c0) * D, valid, qv, sp.scale,
                         warp_halves + static_cast<size_t>(i) * 2 * kTileThreads, lane);
    __syncwarp();                                 // scores of the whole warp are in shared memory
    if (active) {
      const int lf = static_cast<int>(l0);
      if (l0 == 0) {
        if (cnt == kScoreChunk) tile_chunk_shared<T, J, kScoreChunk, kTileThreads, true, true>(q, words, cnt, lf);
        else tile_chunk_shared<T, J, kScoreChunk, kTileThreads, false, true>(q, words, cnt, lf);
      } else {
        if (cnt == kScoreChunk) tile_chunk_shared<T, J, kScoreChunk, kTileThreads, true, false>(q, words, cnt, lf);
        else tile_chunk_shared<T, J, kScoreChunk, kTileThreads, false, false>(q, words, cnt, lf);
      }
    }
  }
  // ragged last stripe: the keys l_full*b + c for c < rem (computed by the whole warp, pushed by their owners)
  if (p.rem > warp_c0) {
    long long tail_left = p.rem - warp_c0;
    const int tail_valid = tail_left > 64 ? 64 : static_cast<int>(tail_left);
    __syncwarp();
    score_stripe<T, D>(krow + (p.l_full * p.b + warp_c0) * D, tail_valid, qv, sp.scale, warp_halves, lane);
    __syncwarp();
    const uint32_t w = words[0];
    if (c0 < p.rem) q[0].push_tail(static_cast<uint16_t>(w & 0xffffu), static_cast<int>(p.l_full));
    if (c0 + 1 < p.rem) q[1].push_tail(static_cast<uint16_t>(w >> 16), static_cast<int>(p.l_full));
  }
  if (!active) return;
  if (!second) {
    // the column that does not exist held only -inf scores: nothing of it is written
    Q one[1] = {q[0]};
    sweep_write_out<T, Q, J, 1, false>(p, one, static_cast<const T*>(nullptr), row, c0, 0, 1);
    return;
  }
  sweep_write_out<T, Q, J, 2, false>(p, q, static_cast<const T*>(nullptr), row, c0, 0, 1);
}

// The scores alone, written to memory (the unfused form of the same arithmetic):
// a warp per 64 keys, the same score_stripe as the fused kernel.
template <typename T, int D>
__global__ void __launch_bounds__(kTileThreads)
scores_kernel(const void* __restrict__ q, const void* __restrict__ keys, long long q_row_stride,
              long long keys_row_stride, long long n, float scale, uint16_t* __restrict__ out,
              long long out_row_stride) {
  const int lane = threadIdx.x & 31;
  const long long row = blockIdx.y;
  const long long first = (static_cast<long long>(blockIdx.x) * (kTileThreads / 32) + (threadIdx.x >> 5)) * 64;
  if (first >= n) return;
  const T* qrow = static_cast<const T*>(q) + row * q_row_stride;
  const T* krow = static_cast<const T*>(keys) + row * keys_row_stride;
  uint32_t qv[D / 8];
#pragma unroll
  for (int s = 0; s < D / 32; ++s)
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const uint16_t* qh = reinterpret_cast<const uint16_t*>(qrow) + 32 * s + 8 * (lane & 3) + 2 * w;
      qv[4 * s + w] = static_cast<uint32_t>(qh[0]) | (static_cast<uint32_t>(qh[1]) << 16);
    }
  const long long left = n - first;
  const int valid = left > 64 ? 64 : static_cast<int>(left);
  // keys past the end would be written as -inf: give them a scratch slot past no one's data instead
  __shared__ uint16_t park[kTileThreads / 32][64];
  uint16_t* dst = valid == 64 ? out + row * out_row_stride + first : park[threadIdx.x >> 5];
  score_stripe<T, D>(krow + first * D, valid, qv, scale, dst, lane);
  if (valid < 64) {
    __syncwarp();
    for (int i = lane; i < valid; i += 32) out[row * out_row_stride + first + i] = park[threadIdx.x >> 5][i];
  }
}

template <typename T, int J, int D>
int launch_scores_jd(const ScoreParams& sp, long long rows, cudaStream_t stream) {
  if (rows * sp.sweep.tiles >= (1ll << 31)) return ATK_ERR_TOO_LARGE;
  const size_t smem = static_cast<size_t>(kScoreChunk) * kTileThreads * 4;
  score_tile_kernel<T, J, D><<<static_cast<unsigned>(rows * sp.sweep.tiles), kTileThreads, smem, stream>>>(sp);
  note_launch();
  return cudaGetLastError() == cudaSuccess ? ATK_OK : ATK_ERR_CUDA;
}

template <typename T, int D>
int launch_scores_d(const ScoreParams& sp, long long rows, int j, cudaStream_t stream) {
  switch (j) {
    case 1: return launch_scores_jd<T, 1, D>(sp, rows, stream);
    case 2: return launch_scores_jd<T, 2, D>(sp, rows, stream);
    case 3: return launch_scores_jd<T, 3, D>(sp, rows, stream);
    case 4: return launch_scores_jd<T, 4, D>(sp, rows, stream);
    default: return ATK_ERR_BAD_J;
  }
}

template <typename T>
int launch_scores(const ScoreParams& sp, long long rows, int j, long long d, cudaStream_t stream) {
  if (d == 128) return launch_scores_d<T, 128>(sp, rows, j, stream);
  if (d == 64) return launch_scores_d<T, 64>(sp, rows, j, stream);
  return ATK_ERR_BAD_ARG;
}

size_t align256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

}  // namespace
}  // namespace atk

using namespace atk;

extern "C" {

int atk_scores(const void* q, const void* keys, int dtype, int64_t rows, int64_t n, int64_t d, int64_t q_row_stride,
               int64_t keys_row_stride, float scale, void* out_scores, int64_t out_row_stride, void* stream) {
  if (dtype != ATK_F16 && dtype != ATK_BF16) return ATK_ERR_BAD_DTYPE;
  if (rows < 0 || n < 0 || q_row_stride < 0 || keys_row_stride < 0 || out_row_stride < 0) return ATK_ERR_BAD_ARG;
  if (d != 64 && d != 128) return ATK_ERR_BAD_ARG;
  if (rows == 0 || n == 0) return ATK_OK;
  if (q == nullptr || keys == nullptr || out_scores == nullptr) return ATK_ERR_BAD_ARG;
  if (reinterpret_cast<uintptr_t>(keys) % 16 != 0 || (keys_row_stride * 2) % 16 != 0) return ATK_ERR_BAD_ARG;
  if (rows > 65535) return ATK_ERR_TOO_LARGE;
  const long long groups = (n + 63) / 64;
  const dim3 grid(static_cast<unsigned>((groups + kTileThreads / 32 - 1) / (kTileThreads / 32)), static_cast<unsigned>(rows));
  const cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint16_t* out = static_cast<uint16_t*>(out_scores);
#define ATK_LAUNCH_SCORES(T, D) \
  scores_kernel<T, D><<<grid, kTileThreads, 0, st>>>(q, keys, q_row_stride, keys_row_stride, n, scale, out, out_row_stride)
  if (dtype == ATK_BF16) {
    if (d == 128) ATK_LAUNCH_SCORES(__nv_bfloat16, 128);
    else ATK_LAUNCH_SCORES(__nv_bfloat16, 64);
  } else {
    if (d == 128) ATK_LAUNCH_SCORES(__half, 128);
    else ATK_LAUNCH_SCORES(__half, 64);
  }
#undef ATK_LAUNCH_SCORES
  note_launch();
  return cudaGetLastError() == cudaSuccess ? ATK_OK : ATK_ERR_CUDA;
}

size_t atk_score_topk_workspace_bytes(int dtype, int64_t rows, int64_t n, int64_t k, int j, int64_t k_mult) {
  (void)n;
  (void)j;
  if ((dtype != ATK_F16 && dtype != ATK_BF16) || rows <= 0 || k <= 0 || k_mult < 1) return 0;
  if (k_mult == 1) return 0;
  const int64_t k0 = k * k_mult;
  return align256(static_cast<size_t>(rows) * k0 * 2) + align256(static_cast<size_t>(rows) * k0 * 8) +
         select_workspace_bytes(dtype, rows, k0);
}

int atk_score_topk(const void* q, const void* keys, int dtype, int64_t rows, int64_t n, int64_t d,
                   int64_t q_row_stride, int64_t keys_row_stride, float scale, int64_t k, int j, int64_t k_mult,
                   void* out_vals, int64_t* out_idx, int64_t out_row_stride, void* workspace,
                   size_t workspace_bytes, void* stream) {
  if (dtype != ATK_F16 && dtype != ATK_BF16) return ATK_ERR_BAD_DTYPE;
  if (rows < 0 || n < 0 || k < 0 || k_mult < 1 || q_row_stride < 0 || keys_row_stride < 0 || out_row_stride < 0)
    return ATK_ERR_BAD_ARG;
  if (d != 64 && d != 128) return ATK_ERR_BAD_ARG;
  if (rows == 0 || k == 0) return ATK_OK;
  if (q == nullptr || keys == nullptr || out_vals == nullptr || out_idx == nullptr) return ATK_ERR_BAD_ARG;
  if (j < 1 || j > 4) return ATK_ERR_BAD_J;
  const int64_t k0 = k * k_mult;
  if (k0 % j != 0) return ATK_ERR_J_DIVIDES_K;
  if (k0 > n) return ATK_ERR_K_TOO_LARGE;
  const int64_t b = k0 / j;
  if (n / b + 1 > PackedQueue<__half, 1, false>::kMaxStripes) return ATK_ERR_TOO_LARGE;
  // 16-byte loads of the keys and of q
  if (reinterpret_cast<uintptr_t>(keys) % 16 != 0 || (keys_row_stride * 2) % 16 != 0 ||
      reinterpret_cast<uintptr_t>(q) % 2 != 0)
    return ATK_ERR_BAD_ARG;

  unsigned char* ws = static_cast<unsigned char*>(workspace);
  void* cand_vals = out_vals;
  long long* cand_idx = reinterpret_cast<long long*>(out_idx);
  long long cand_stride = out_row_stride;
  const size_t cand_v = align256(static_cast<size_t>(rows) * k0 * 2);
  const size_t cand_i = align256(static_cast<size_t>(rows) * k0 * 8);
  const size_t sel_ws = k_mult > 1 ? select_workspace_bytes(dtype, rows, k0) : 0;
  if (k_mult > 1) {
    if (ws == nullptr || workspace_bytes < cand_v + cand_i + sel_ws) return ATK_ERR_WORKSPACE;
    cand_vals = ws;
    cand_idx = reinterpret_cast<long long*>(ws + cand_v);
    cand_stride = k0;
  }
  ScoreParams sp;
  sp.q = q;
  sp.keys = keys;
  sp.q_row_stride = q_row_stride;
  sp.keys_row_stride = keys_row_stride;
  sp.scale = scale;
  SweepParams& p = sp.sweep;
  p.x = nullptr;
  p.out_vals = cand_vals;
  p.out_idx = cand_idx;
  p.rows = rows;
  p.row_stride = 0;
  p.out_row_stride = cand_stride;
  p.b = b;
  p.l_full = n / b;
  p.rem = n - p.l_full * b;
  p.stripe_stride = b;
  p.tiles = (b + 2 * kTileThreads - 1) / (2 * kTileThreads);
  p.idx_stride = b;
  p.idx_offset = 0;
  p.cw = kTileThreads;
  p.s = 1;
  p.out_format = ATK_OUT_I64;
  p.vec_out = (reinterpret_cast<uintptr_t>(cand_vals) % 16 == 0) && (reinterpret_cast<uintptr_t>(cand_idx) % 16 == 0) &&
              ((cand_stride * 2) % 16 == 0) && ((cand_stride * 8) % 16 == 0);
  p.vec_part = 0;
  p.out_keys = nullptr;
  p.vec_keys = 0;
  p.z = 1;
  p.z_chunk = p.l_full;
  p.main_units = 0;
  p.z_main = 1;
  p.z_chunk_main = p.l_full;
  p.part_vals = nullptr;
  p.part_idx = nullptr;
  const cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int rc = dtype == ATK_BF16 ? launch_scores<__nv_bfloat16>(sp, rows, j, d, st)
                                   : launch_scores<__half>(sp, rows, j, d, st);
  if (rc != ATK_OK || k_mult == 1) return rc;
  SelectLaunch sel;
  sel.cand_vals = cand_vals;
  sel.cand_idx = cand_idx;
  sel.rows = rows;
  sel.k0 = k0;
  sel.cand_row_stride = k0;
  sel.k = k;
  sel.out_vals = out_vals;
  sel.out_idx = out_idx;
  sel.out_row_stride = out_row_stride;
  sel.out_format = ATK_OUT_I64;
  sel.workspace = sel_ws ? ws + cand_v + cand_i : nullptr;
  sel.workspace_bytes = sel_ws;
  sel.stream = st;
  return launch_select(sel, dtype);
}

}  // extern "C"
