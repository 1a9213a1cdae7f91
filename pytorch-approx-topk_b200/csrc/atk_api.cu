// C ABI of libatk.so: argument validation, dispatch to the kernel launchers and
// the host-buffer pipeline.  See include/atk.h for the contract of every entry
// point and the reference interface each one replaces.
#include <atomic>
#include <mutex>

#include "atk_contig.cuh"
#include "atk_select.cuh"
#include "atk_sweep.cuh"

namespace atk {

static thread_local long long g_launches = 0;
void note_launch(int n) { g_launches += n; }

int stage1_formatted(const void* x, int dtype, int64_t rows, int64_t n, int64_t row_stride, int64_t k0, int j,
                     int interleaved, int mode, int out_format, void* out_vals, void* out_idx,
                     int64_t out_row_stride, void* workspace, size_t workspace_bytes, void* stream);

// Lazily cached SM count per device.  Together with the per-device address cache and
// the built-in scratch array of atk_select_static (atk_select.cu) and the two cached
// pipeline streams per device of atk_topk_host this is all the global state the library has
// (besides the ATK_* environment switches, each read once).
int sm_count_of_current_device() {
  static std::atomic<int> cache[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev >= 0 && dev < 64) {
    const int c = cache[dev].load(std::memory_order_relaxed);
    if (c > 0) return c;
  }
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  if (dev >= 0 && dev < 64) cache[dev].store(n, std::memory_order_relaxed);
  return n;
}

bool overlapped_launch_enabled() {
  static const bool on = std::getenv("ATK_NO_OVERLAPPED_LAUNCH") == nullptr;
  return on;
}

namespace {

int elem_size(int dtype) {
  switch (dtype) {
    case ATK_F32: return 4;
    case ATK_F16: return 2;
    case ATK_BF16: return 2;
    case ATK_F64: return 8;
    case ATK_I32: return 4;
    case ATK_I64: return 8;
    case ATK_I16: return 2;
    case ATK_I8: return 1;
    case ATK_U8: return 1;
    default: return 0;
  }
}

size_t align256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

int sweep_dispatch(const SweepLaunch& a, int dtype) {
  switch (dtype) {
    case ATK_F32: return launch_sweep_f32(a);
    case ATK_F16: return launch_sweep_f16(a);
    case ATK_BF16: return launch_sweep_bf16(a);
    case ATK_F64: return launch_sweep_f64(a);
    case ATK_I32: return launch_sweep_i32(a);
    case ATK_I64: return launch_sweep_i64(a);
    case ATK_I16: return launch_sweep_i16(a);
    case ATK_I8: return launch_sweep_i8(a);
    case ATK_U8: return launch_sweep_u8(a);
    default: return ATK_ERR_BAD_DTYPE;
  }
}

int check_common(const void* x, int dtype, int64_t rows, int64_t n, int64_t row_stride,
                 const void* out_vals, const void* out_idx, int64_t out_row_stride) {
  if (elem_size(dtype) == 0) return ATK_ERR_BAD_DTYPE;
  if (rows < 0 || n < 0 || row_stride < 0 || out_row_stride < 0) return ATK_ERR_BAD_ARG;
  if (rows > 0 && n > 0 && (x == nullptr || out_vals == nullptr || out_idx == nullptr)) return ATK_ERR_BAD_ARG;
  return ATK_OK;
}

}  // namespace
}  // namespace atk

using namespace atk;

extern "C" {

int atk_version(void) { return 10000; }

const char* atk_strerror(int status) {
  switch (status) {
    case ATK_OK: return "ok";
    case ATK_ERR_BAD_J: return "topk: j must 0 < j < 5";
    case ATK_ERR_J_DIVIDES_K: return "topk: j must divide k";
    case ATK_ERR_K_TOO_LARGE: return "topk: k must not be larger than topk size";
    case ATK_ERR_BAD_DTYPE: return "topk: unsupported dtype (float32/16, bfloat16, float64, int8/16/32/64 and uint8 are supported)";
    case ATK_ERR_BAD_ARG: return "topk: invalid argument";
    case ATK_ERR_WORKSPACE: return "topk: workspace missing or too small";
    case ATK_ERR_TOO_LARGE: return "topk: problem size exceeds the kernel's index range";
    case ATK_ERR_CUDA: return "topk: CUDA runtime error";
    case ATK_ERR_SCRATCH_LIMIT:
      return "topk: atk_select_static needs more scratch than its built-in 1 MiB; use atk_select with a workspace";
    default: return "topk: unknown status";
  }
}

int atk_device_supported(void) {
  int dev = 0, major = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return ATK_ERR_CUDA;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return ATK_ERR_CUDA;
  return major == 10 ? ATK_OK : ATK_ERR_CUDA;
}

size_t atk_stage1_workspace_bytes(int dtype, int64_t rows, int64_t n, int64_t k0, int j, int interleaved) {
  const int s = elem_size(dtype);
  if (s == 0 || !interleaved || rows <= 0 || k0 <= 0 || j < 1 || j > 4 || k0 % j != 0 || k0 > n) return 0;
  return sweep_workspace_bytes(s, rows, n, k0 / j, j, sm_count_of_current_device());
}

int atk_stage1(const void* x, int dtype, int64_t rows, int64_t n, int64_t row_stride, int64_t k0,
               int j, int interleaved, int mode, void* out_vals, int64_t* out_idx,
               int64_t out_row_stride, void* workspace, size_t workspace_bytes, void* stream) {
  return stage1_formatted(x, dtype, rows, n, row_stride, k0, j, interleaved, mode, ATK_OUT_I64, out_vals, out_idx,
                          out_row_stride, workspace, workspace_bytes, stream);
}

}  // extern "C"

namespace atk {
// atk_stage1 with the output format of the final pairs as a parameter (the C ABI
// offers the formats through atk_topk_ex only).
int stage1_formatted(const void* x, int dtype, int64_t rows, int64_t n, int64_t row_stride, int64_t k0, int j,
                     int interleaved, int mode, int out_format, void* out_vals, void* out_idx,
                     int64_t out_row_stride, void* workspace, size_t workspace_bytes, void* stream) {
  (void)mode;
  int rc = check_common(x, dtype, rows, n, row_stride, out_vals,
                        out_format == ATK_OUT_REC32 ? out_vals : out_idx, out_row_stride);
  if (rc != ATK_OK) return rc;
  if (k0 < 0) return ATK_ERR_BAD_ARG;
  if (k0 == 0 || rows == 0) return ATK_OK;
  if (j < 1 || j > 4) return ATK_ERR_BAD_J;
  if (k0 % j != 0) return ATK_ERR_J_DIVIDES_K;
  if (k0 > n) return ATK_ERR_K_TOO_LARGE;
  const int64_t b = k0 / j;
  if (interleaved) {
    SweepLaunch a;
    a.x = x;
    a.out_vals = out_vals;
    a.out_idx = reinterpret_cast<long long*>(out_idx);
    a.rows = rows;
    a.n = n;
    a.row_stride = row_stride;
    a.out_row_stride = out_row_stride;
    a.b = b;
    a.stripe_stride = b;
    a.idx_stride = b;
    a.idx_offset = 0;
    a.j = j;
    a.first_wins = false;
    a.sm_count = sm_count_of_current_device();
    a.out_format = out_format;
    a.workspace = workspace;
    a.workspace_bytes = workspace_bytes;
    a.out_keys = nullptr;
    a.stream = static_cast<cudaStream_t>(stream);
    return sweep_dispatch(a, dtype);
  }
  if (out_format != ATK_OUT_I64) return ATK_ERR_BAD_ARG;   // narrow formats: interleaved buckets only
  ContigLaunch c;
  c.x = x;
  c.out_vals = out_vals;
  c.out_idx = reinterpret_cast<long long*>(out_idx);
  c.rows = rows;
  c.n = n;
  c.row_stride = row_stride;
  c.out_row_stride = out_row_stride;
  c.b = b;
  c.j = j;
  c.first_wins = false;
  c.fixed_chunks = false;
  c.stream = static_cast<cudaStream_t>(stream);
  return launch_contig(c, dtype);
}
}  // namespace atk

extern "C" {

size_t atk_stage1_slab_workspace_bytes(int dtype, int64_t stripes, int64_t cols, int j) {
  const int s = elem_size(dtype);
  if (s == 0 || stripes <= 0 || cols <= 0 || j < 1 || j > 4 || j > stripes) return 0;
  return sweep_workspace_bytes(s, 1, stripes * cols, cols, j, sm_count_of_current_device());
}

int atk_stage1_slab(const void* slab, int dtype, int64_t stripes, int64_t cols, int64_t total_buckets,
                    int64_t col_offset, int j, void* out_vals, int64_t* out_idx, void* workspace,
                    size_t workspace_bytes, void* stream) {
  if (elem_size(dtype) == 0) return ATK_ERR_BAD_DTYPE;
  if (stripes < 0 || cols < 0 || total_buckets < cols || col_offset < 0) return ATK_ERR_BAD_ARG;
  if (stripes == 0 || cols == 0) return ATK_OK;
  if (slab == nullptr || out_vals == nullptr || out_idx == nullptr) return ATK_ERR_BAD_ARG;
  if (j < 1 || j > 4) return ATK_ERR_BAD_J;
  if (j > stripes) return ATK_ERR_K_TOO_LARGE;
  SweepLaunch a;
  a.x = slab;
  a.out_vals = out_vals;
  a.out_idx = reinterpret_cast<long long*>(out_idx);
  a.rows = 1;
  a.n = stripes * cols;
  a.row_stride = stripes * cols;
  a.out_row_stride = cols * j;
  a.b = cols;
  a.stripe_stride = cols;
  a.idx_stride = total_buckets;
  a.idx_offset = col_offset;
  a.j = j;
  a.first_wins = false;
  a.sm_count = sm_count_of_current_device();
  a.workspace = workspace;
  a.workspace_bytes = workspace_bytes;
  a.out_keys = nullptr;
  a.stream = static_cast<cudaStream_t>(stream);
  return sweep_dispatch(a, dtype);
}

size_t atk_select_workspace_bytes(int dtype, int64_t rows, int64_t k0, int64_t k) {
  (void)k;
  if (rows <= 0 || k0 <= 0) return 0;
  return select_workspace_bytes(dtype, rows, k0);
}

int atk_select(const void* cand_vals, const int64_t* cand_idx, int dtype, int64_t rows, int64_t k0,
               int64_t cand_row_stride, int64_t k, void* out_vals, int64_t* out_idx,
               int64_t out_row_stride, void* workspace, size_t workspace_bytes, void* stream) {
  if (elem_size(dtype) == 0) return ATK_ERR_BAD_DTYPE;
  if (rows < 0 || k0 < 0 || k < 0 || k > k0 || cand_row_stride < 0 || out_row_stride < 0) return ATK_ERR_BAD_ARG;
  if (rows == 0 || k == 0) return ATK_OK;
  if (cand_vals == nullptr || cand_idx == nullptr || out_vals == nullptr || out_idx == nullptr) return ATK_ERR_BAD_ARG;
  SelectLaunch a;
  a.cand_vals = cand_vals;
  a.cand_idx = reinterpret_cast<const long long*>(cand_idx);
  a.rows = rows;
  a.k0 = k0;
  a.cand_row_stride = cand_row_stride;
  a.k = k;
  a.out_vals = out_vals;
  a.out_idx = out_idx;
  a.out_row_stride = out_row_stride;
  a.workspace = workspace;
  a.workspace_bytes = workspace_bytes;
  a.stream = static_cast<cudaStream_t>(stream);
  return launch_select(a, dtype);
}

int atk_select_static(const void* cand_vals, const int64_t* cand_idx, int dtype, int64_t rows, int64_t k0,
                      int64_t cand_row_stride, int64_t k, void* out_vals, int64_t* out_idx,
                      int64_t out_row_stride, void* stream) {
  if (elem_size(dtype) == 0) return ATK_ERR_BAD_DTYPE;
  if (rows < 0 || k0 < 0 || k < 0 || k > k0 || cand_row_stride < 0 || out_row_stride < 0) return ATK_ERR_BAD_ARG;
  if (rows == 0 || k == 0) return ATK_OK;
  if (cand_vals == nullptr || cand_idx == nullptr || out_vals == nullptr || out_idx == nullptr) return ATK_ERR_BAD_ARG;
  SelectLaunch a;
  a.cand_vals = cand_vals;
  a.cand_idx = reinterpret_cast<const long long*>(cand_idx);
  a.rows = rows;
  a.k0 = k0;
  a.cand_row_stride = cand_row_stride;
  a.k = k;
  a.out_vals = out_vals;
  a.out_idx = out_idx;
  a.out_row_stride = out_row_stride;
  a.workspace = nullptr;
  a.workspace_bytes = 0;
  a.stream = static_cast<cudaStream_t>(stream);
  return launch_select_static(a, dtype);
}

size_t atk_topk_workspace_bytes(int dtype, int64_t rows, int64_t n, int64_t k, int j, int64_t k_mult) {
  const int s = elem_size(dtype);
  if (s == 0 || rows <= 0 || k <= 0 || k_mult < 1) return 0;
  const int64_t k0 = k * k_mult;
  // stage 1 may split stripes over blocks (interleaved buckets; harmless upper bound otherwise)
  size_t total = align256(atk_stage1_workspace_bytes(dtype, rows, n, k0, j, 1));
  if (k_mult > 1)
    total += align256(static_cast<size_t>(rows) * k0 * s) + align256(static_cast<size_t>(rows) * k0 * 8) +
             select_workspace_bytes(dtype, rows, k0);
  return total;
}

int atk_topk(const void* x, int dtype, int64_t rows, int64_t n, int64_t row_stride, int64_t k, int j,
             int64_t k_mult, int interleaved, int mode, void* out_vals, int64_t* out_idx,
             int64_t out_row_stride, void* workspace, size_t workspace_bytes, void* stream) {
  return atk_topk_ex(x, dtype, rows, n, row_stride, k, j, k_mult, interleaved, mode, ATK_OUT_I64, out_vals, out_idx,
                     out_row_stride, workspace, workspace_bytes, stream);
}

int atk_topk_ex(const void* x, int dtype, int64_t rows, int64_t n, int64_t row_stride, int64_t k, int j,
                int64_t k_mult, int interleaved, int mode, int out_format, void* out_vals, void* out_idx,
                int64_t out_row_stride, void* workspace, size_t workspace_bytes, void* stream) {
  if (k_mult < 1 || k < 0) return ATK_ERR_BAD_ARG;
  const int s = elem_size(dtype);
  if (s == 0) return ATK_ERR_BAD_DTYPE;
  if (out_format != ATK_OUT_I64 && out_format != ATK_OUT_I32 && out_format != ATK_OUT_REC32) return ATK_ERR_BAD_ARG;
  if (out_format != ATK_OUT_I64) {
    if (!interleaved) return ATK_ERR_BAD_ARG;
    if (out_format == ATK_OUT_REC32 && s > 4) return ATK_ERR_BAD_DTYPE;
    if (n >= (1ll << 31)) return ATK_ERR_TOO_LARGE;
  }
  if (k == 0 || rows == 0) return ATK_OK;
  const int64_t k0 = k * k_mult;
  // Workspace layout: [stage-1 stripe-split planes][candidate values][candidate positions][select state].
  // The stage-1 part is optional (a smaller or missing workspace only disables the split over blocks);
  // the rest is required when k_mult > 1.
  unsigned char* ws = static_cast<unsigned char*>(workspace);
  size_t split_bytes = align256(atk_stage1_workspace_bytes(dtype, rows, n, k0, j, interleaved));
  if (k_mult == 1) {
    if (ws == nullptr || workspace_bytes < split_bytes) split_bytes = ws == nullptr ? 0 : workspace_bytes;
    return stage1_formatted(x, dtype, rows, n, row_stride, k, j, interleaved, mode, out_format, out_vals, out_idx,
                            out_row_stride, ws, split_bytes, stream);
  }
  const size_t cand_v = align256(static_cast<size_t>(rows) * k0 * s);
  const size_t cand_i = align256(static_cast<size_t>(rows) * k0 * 8);
  const size_t sel_ws = select_workspace_bytes(dtype, rows, k0);
  if (ws == nullptr || workspace_bytes < cand_v + cand_i + sel_ws) return ATK_ERR_WORKSPACE;
  if (workspace_bytes < split_bytes + cand_v + cand_i + sel_ws) split_bytes = 0;
  void* split_ws = split_bytes ? ws : nullptr;
  ws += split_bytes;
  void* cand_vals = ws;
  ws += cand_v;
  int64_t* cand_idx = reinterpret_cast<int64_t*>(ws);
  ws += cand_i;
  // 8- and 16-bit elements, interleaved buckets, rows the one-block select takes:
  // stage 1 hands its packed queue entries (4 bytes per candidate, in the space
  // of the candidate values) straight to a select that works on them; values and
  // positions are rebuilt for the k winners only.  Shapes without packed entries
  // (too many stripes, stripes split over blocks) fall through to the plain form.
  if (interleaved && s <= 2 && k0 <= select_packed_max_k0() && j >= 1 && j <= 4 && k0 % j == 0 && k0 <= n &&
      rows > 0 && n > 0 && x != nullptr && out_vals != nullptr &&
      (out_idx != nullptr || out_format == ATK_OUT_REC32) && row_stride >= 0 &&
      out_row_stride >= 0 && static_cast<size_t>(rows) * k0 * 4 <= cand_v + cand_i) {
    SweepLaunch a;
    a.x = x;
    a.out_vals = nullptr;
    a.out_idx = nullptr;
    a.rows = rows;
    a.n = n;
    a.row_stride = row_stride;
    a.out_row_stride = k0;
    a.b = k0 / j;
    a.stripe_stride = a.b;
    a.idx_stride = a.b;
    a.idx_offset = 0;
    a.j = j;
    a.first_wins = false;
    a.sm_count = sm_count_of_current_device();
    a.workspace = nullptr;
    a.workspace_bytes = 0;
    a.out_keys = static_cast<uint32_t*>(cand_vals);
    a.stream = static_cast<cudaStream_t>(stream);
    const int prc = sweep_dispatch(a, dtype);
    if (prc == ATK_OK) {
      SelectPackedLaunch sp;
      sp.keys = a.out_keys;
      sp.rows = rows;
      sp.k0 = k0;
      sp.k = k;
      sp.x = x;
      sp.x_row_stride = row_stride;
      sp.b = a.b;
      sp.j = j;
      sp.out_vals = out_vals;
      sp.out_idx = out_idx;
      sp.out_row_stride = out_row_stride;
      sp.out_format = out_format;
      sp.stream = a.stream;
      return launch_select_packed(sp, dtype);
    }
    if (prc != kPackedUnavailable) return prc;
  }
  int rc = atk_stage1(x, dtype, rows, n, row_stride, k0, j, interleaved, mode, cand_vals, cand_idx, k0,
                      split_ws, split_bytes, stream);
  if (rc != ATK_OK) return rc;
  if (out_vals == nullptr || (out_idx == nullptr && out_format != ATK_OUT_REC32) || out_row_stride < 0)
    return ATK_ERR_BAD_ARG;
  SelectLaunch sel;
  sel.cand_vals = cand_vals;
  sel.cand_idx = reinterpret_cast<const long long*>(cand_idx);
  sel.rows = rows;
  sel.k0 = k0;
  sel.cand_row_stride = k0;
  sel.k = k;
  sel.out_vals = out_vals;
  sel.out_idx = out_idx;
  sel.out_row_stride = out_row_stride;
  sel.out_format = out_format;
  sel.workspace = sel_ws ? ws : nullptr;
  sel.workspace_bytes = sel_ws;
  sel.stream = static_cast<cudaStream_t>(stream);
  return launch_select(sel, dtype);
}

int atk_bucketed_argmax(const void* x, int dtype, int64_t rows, int64_t n, int64_t row_stride, int64_t k,
                        int interleaved, void* out_vals, int64_t* out_idx, int64_t out_row_stride,
                        void* workspace, size_t workspace_bytes, void* stream) {
  int rc = check_common(x, dtype, rows, n, row_stride, out_vals, out_idx, out_row_stride);
  if (rc != ATK_OK) return rc;
  if (k < 0) return ATK_ERR_BAD_ARG;
  if (k == 0 || rows == 0) return ATK_OK;
  if (n == 0) return ATK_ERR_K_TOO_LARGE;
  if (interleaved) {
    SweepLaunch a;
    a.x = x;
    a.out_vals = out_vals;
    a.out_idx = reinterpret_cast<long long*>(out_idx);
    a.rows = rows;
    a.n = n;
    a.row_stride = row_stride;
    a.out_row_stride = out_row_stride;
    a.b = k;
    a.stripe_stride = k;
    a.idx_stride = k;
    a.idx_offset = 0;
    a.j = 1;
    a.first_wins = true;
    a.sm_count = sm_count_of_current_device();
    a.workspace = workspace;
    a.workspace_bytes = workspace_bytes;
    a.out_keys = nullptr;
    a.stream = static_cast<cudaStream_t>(stream);
    return sweep_dispatch(a, dtype);
  }
  ContigLaunch c;
  c.x = x;
  c.out_vals = out_vals;
  c.out_idx = reinterpret_cast<long long*>(out_idx);
  c.rows = rows;
  c.n = n;
  c.row_stride = row_stride;
  c.out_row_stride = out_row_stride;
  c.b = k;
  c.j = 1;
  c.first_wins = true;
  c.fixed_chunks = true;
  c.stream = static_cast<cudaStream_t>(stream);
  return launch_contig(c, dtype);
}

// ---- host-buffer pipeline ---------------------------------------------------
namespace {
// The two pipeline streams of atk_topk_host, created on the first call on a
// device and kept for the life of the process (creating and destroying two
// streams per call cost tens of microseconds of every step).
bool host_streams_of_current_device(cudaStream_t (&out)[2]) {
  static std::mutex mu;
  static cudaStream_t cache[64][2];
  static bool ready[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
  std::lock_guard<std::mutex> lock(mu);
  if (!ready[dev]) {
    cudaStream_t a = nullptr, b = nullptr;
    if (cudaStreamCreateWithFlags(&a, cudaStreamNonBlocking) != cudaSuccess) return false;
    if (cudaStreamCreateWithFlags(&b, cudaStreamNonBlocking) != cudaSuccess) {
      cudaStreamDestroy(a);
      return false;
    }
    cache[dev][0] = a;
    cache[dev][1] = b;
    ready[dev] = true;
  }
  out[0] = cache[dev][0];
  out[1] = cache[dev][1];
  return true;
}

struct HostPlan {
  int64_t chunk_rows;
  size_t x_bytes, v_bytes, i_bytes, ws_bytes, slot_bytes;
};
HostPlan plan_host(int dtype, int64_t rows, int64_t n, int64_t k, int j, int64_t k_mult, int64_t chunk_rows) {
  HostPlan p{};
  const int s = elem_size(dtype);
  if (chunk_rows <= 0) {
    // about 32 MiB of input per chunk, at least 4 chunks when there are rows to split
    const int64_t row_bytes = n * s > 0 ? n * s : 1;
    chunk_rows = (32ll << 20) / row_bytes;
    if (chunk_rows < 1) chunk_rows = 1;
    if (chunk_rows > (rows + 3) / 4) chunk_rows = (rows + 3) / 4;
    if (chunk_rows < 1) chunk_rows = 1;
  }
  if (chunk_rows > rows) chunk_rows = rows > 0 ? rows : 1;
  p.chunk_rows = chunk_rows;
  p.x_bytes = align256(static_cast<size_t>(chunk_rows) * n * s);
  p.v_bytes = align256(static_cast<size_t>(chunk_rows) * k * s);
  p.i_bytes = align256(static_cast<size_t>(chunk_rows) * k * 8);
  p.ws_bytes = align256(atk_topk_workspace_bytes(dtype, chunk_rows, n, k, j, k_mult));
  p.slot_bytes = p.x_bytes + p.v_bytes + p.i_bytes + p.ws_bytes;
  return p;
}
}  // namespace

size_t atk_topk_host_scratch_bytes(int dtype, int64_t rows, int64_t n, int64_t k, int j, int64_t k_mult,
                                   int64_t chunk_rows) {
  if (elem_size(dtype) == 0 || rows <= 0 || n <= 0 || k < 0 || k_mult < 1) return 0;
  return 2 * plan_host(dtype, rows, n, k, j, k_mult, chunk_rows).slot_bytes;
}

int atk_topk_host(const void* x_host, int dtype, int64_t rows, int64_t n, int64_t row_stride, int64_t k,
                  int j, int64_t k_mult, int interleaved, void* out_vals_host, int64_t* out_idx_host,
                  void* device_scratch, size_t scratch_bytes, int64_t chunk_rows) {
  const int s = elem_size(dtype);
  if (s == 0) return ATK_ERR_BAD_DTYPE;
  if (rows < 0 || n < 0 || k < 0 || k_mult < 1 || row_stride < n) return ATK_ERR_BAD_ARG;
  if (rows == 0 || k == 0) return ATK_OK;
  if (x_host == nullptr || out_vals_host == nullptr || out_idx_host == nullptr) return ATK_ERR_BAD_ARG;
  const HostPlan p = plan_host(dtype, rows, n, k, j, k_mult, chunk_rows);
  if (device_scratch == nullptr || scratch_bytes < 2 * p.slot_bytes) return ATK_ERR_WORKSPACE;

  cudaStream_t st[2] = {nullptr, nullptr};
  if (!host_streams_of_current_device(st)) return ATK_ERR_CUDA;
  int rc = ATK_OK;
  int64_t chunk = 0;
  for (int64_t r0 = 0; r0 < rows && rc == ATK_OK; r0 += p.chunk_rows, ++chunk) {
    const int64_t nr = rows - r0 < p.chunk_rows ? rows - r0 : p.chunk_rows;
    const int slot = static_cast<int>(chunk & 1);
    unsigned char* base = static_cast<unsigned char*>(device_scratch) + slot * p.slot_bytes;
    void* dx = base;
    void* dv = base + p.x_bytes;
    int64_t* di = reinterpret_cast<int64_t*>(base + p.x_bytes + p.v_bytes);
    void* dws = p.ws_bytes ? base + p.x_bytes + p.v_bytes + p.i_bytes : nullptr;
    const unsigned char* hx = static_cast<const unsigned char*>(x_host) + static_cast<size_t>(r0) * row_stride * s;
    // Work queued on a stream runs in order, so a slot is reused only after
    // its previous download has been issued on the same stream.  Dense rows
    // go up as one linear copy, strided rows as a pitched one.
    cudaError_t e;
    if (row_stride == n)
      e = cudaMemcpyAsync(dx, hx, static_cast<size_t>(nr) * n * s, cudaMemcpyHostToDevice, st[slot]);
    else
      e = cudaMemcpy2DAsync(dx, static_cast<size_t>(n) * s, hx, static_cast<size_t>(row_stride) * s,
                            static_cast<size_t>(n) * s, static_cast<size_t>(nr), cudaMemcpyHostToDevice, st[slot]);
    if (e != cudaSuccess) { rc = ATK_ERR_CUDA; break; }
    rc = atk_topk(dx, dtype, nr, n, n, k, j, k_mult, interleaved, -1, dv, di, k, dws, p.ws_bytes, st[slot]);
    if (rc != ATK_OK) break;
    e = cudaMemcpyAsync(static_cast<unsigned char*>(out_vals_host) + static_cast<size_t>(r0) * k * s, dv,
                        static_cast<size_t>(nr) * k * s, cudaMemcpyDeviceToHost, st[slot]);
    if (e == cudaSuccess)
      e = cudaMemcpyAsync(out_idx_host + r0 * k, di, static_cast<size_t>(nr) * k * 8, cudaMemcpyDeviceToHost,
                          st[slot]);
    if (e != cudaSuccess) rc = ATK_ERR_CUDA;
  }
  for (int i = 0; i < 2; ++i)
    if (cudaStreamSynchronize(st[i]) != cudaSuccess && rc == ATK_OK) rc = ATK_ERR_CUDA;
  return rc;
}

int64_t atk_launch_count(void) { return g_launches; }
void atk_reset_launch_count(void) { g_launches = 0; }

}  // extern "C"
