// Gather of the selected records (the step after the operator): out[r][q] =
// src[r][idx[r][q]].  Bandwidth-bound: a group of lanes copies one record in
// 16-byte pieces, records are spread over the grid with a grid-stride loop.
#include "atk_common.cuh"

namespace atk {
namespace {

template <typename P>
__global__ void __launch_bounds__(256)
gather_records_kernel(const unsigned char* __restrict__ src, long long rows, long long n, long long pieces /* per record */,
                      long long src_row_stride_bytes, const long long* __restrict__ idx, long long k,
                      long long idx_row_stride, unsigned char* __restrict__ out, int lanes /* per record, power of two */) {
  const long long total = rows * k;
  const int lane = threadIdx.x % lanes;
  const long long groups_per_block = blockDim.x / lanes;
  const long long record_bytes = pieces * static_cast<long long>(sizeof(P));
  for (long long rec = static_cast<long long>(blockIdx.x) * groups_per_block + threadIdx.x / lanes; rec < total;
       rec += static_cast<long long>(gridDim.x) * groups_per_block) {
    const long long r = rec / k;
    const long long q = rec - r * k;
    const long long pos = idx[r * idx_row_stride + q];
    const bool ok = pos >= 0 && pos < n;
    const P* s = reinterpret_cast<const P*>(src + r * src_row_stride_bytes + (ok ? pos : 0) * record_bytes);
    P* d = reinterpret_cast<P*>(out + rec * record_bytes);
    for (long long i = lane; i < pieces; i += lanes) {
      P v{};
      if (ok) v = s[i];
      d[i] = v;
    }
  }
}

template <typename P>
int launch_gather(const void* src, long long rows, long long n, long long record_bytes, long long src_row_stride_bytes,
                  const long long* idx, long long k, long long idx_row_stride, void* out, cudaStream_t stream) {
  const long long pieces = record_bytes / static_cast<long long>(sizeof(P));
  int lanes = 1;
  while (lanes < 32 && lanes < pieces) lanes *= 2;
  const long long total = rows * k;
  const long long per_block = 256 / lanes;
  long long blocks = (total + per_block - 1) / per_block;
  const long long cap = static_cast<long long>(sm_count_of_current_device()) * 8 * 4;          // a few waves; the loop covers the rest
  if (blocks > cap) blocks = cap;
  gather_records_kernel<P><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
      static_cast<const unsigned char*>(src), rows, n, pieces, src_row_stride_bytes, idx, k, idx_row_stride,
      static_cast<unsigned char*>(out), lanes);
  note_launch();
  return cudaGetLastError() == cudaSuccess ? ATK_OK : ATK_ERR_CUDA;
}

}  // namespace
}  // namespace atk

extern "C" int atk_gather_records(const void* src, int64_t rows, int64_t n, int64_t record_bytes,
                                  int64_t src_row_stride_bytes, const int64_t* idx, int64_t k,
                                  int64_t idx_row_stride, void* out, void* stream) {
  using namespace atk;
  if (rows < 0 || n < 0 || record_bytes < 0 || k < 0 || src_row_stride_bytes < 0 || idx_row_stride < 0) return ATK_ERR_BAD_ARG;
  if (rows == 0 || k == 0 || record_bytes == 0) return ATK_OK;
  if (src == nullptr || idx == nullptr || out == nullptr) return ATK_ERR_BAD_ARG;
  const uintptr_t a = reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(out) |
                      static_cast<uintptr_t>(record_bytes) | static_cast<uintptr_t>(src_row_stride_bytes);
  const long long* i64 = reinterpret_cast<const long long*>(idx);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (a % 16 == 0) return launch_gather<uint4>(src, rows, n, record_bytes, src_row_stride_bytes, i64, k, idx_row_stride, out, st);
  if (a % 4 == 0) return launch_gather<uint32_t>(src, rows, n, record_bytes, src_row_stride_bytes, i64, k, idx_row_stride, out, st);
  if (a % 2 == 0) return launch_gather<uint16_t>(src, rows, n, record_bytes, src_row_stride_bytes, i64, k, idx_row_stride, out, st);
  return launch_gather<uint8_t>(src, rows, n, record_bytes, src_row_stride_bytes, i64, k, idx_row_stride, out, st);
}
