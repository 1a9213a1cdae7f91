// Candidate exchange of the sharded long row without a collective library: a rank
// copies its own block of candidates straight into the candidate buffers of every
// peer (device pointers into the peers' memory, mapped into this process by CUDA IPC)
// with plain stores over NVLink.  One kernel reads every 16-byte piece of the block
// once from this GPU's memory and stores it to all destinations, so all links are
// busy at once.  No loads from peer memory, no switch-side replication, no waiting on peers: the
// ranks synchronise afterwards on the host side of the exchange (a barrier in
// stream order), and only then read what they received.
#include <cstring>

#include "atk_common.cuh"

namespace atk {
namespace {

constexpr int kPushThreads = 256;
constexpr int kPushMaxSegments = ATK_PUSH_MAX_SEGMENTS;
constexpr int kPushMaxDst = ATK_PUSH_MAX_DST;

struct PushParams {
  const unsigned char* src[kPushMaxSegments];
  unsigned long long pieces[kPushMaxSegments];       // 16-byte (VEC) or 4-byte pieces per segment
  unsigned char* dst[kPushMaxSegments][kPushMaxDst];
  int n_seg, n_dst;
};

template <typename Piece>
__global__ void __launch_bounds__(kPushThreads) push_blocks_kernel(const PushParams p) {
  // The blocks of stage 1 that this kernel forwards come from the kernel before it.
  grid_dependency_wait();
  constexpr int kInFlight = 4;                        // independent loads per thread before the stores
  const unsigned long long stride = static_cast<unsigned long long>(gridDim.x) * kPushThreads;
  for (int s = 0; s < p.n_seg; ++s) {
    const Piece* src = reinterpret_cast<const Piece*>(p.src[s]);
    const unsigned long long n = p.pieces[s];
    for (unsigned long long i0 = static_cast<unsigned long long>(blockIdx.x) * kPushThreads + threadIdx.x; i0 < n;
         i0 += stride * kInFlight) {
      Piece v[kInFlight];
#pragma unroll
      for (int u = 0; u < kInFlight; ++u) {
        const unsigned long long i = i0 + u * stride;
        if (i < n) v[u] = src[i];
      }
      for (int d = 0; d < p.n_dst; ++d) {
        Piece* dst = reinterpret_cast<Piece*>(p.dst[s][d]);
#pragma unroll
        for (int u = 0; u < kInFlight; ++u) {
          const unsigned long long i = i0 + u * stride;
          if (i < n) dst[i] = v[u];
        }
      }
    }
  }
}

}  // namespace
}  // namespace atk

extern "C" int atk_push_blocks(int n_seg, const void* const* src, const size_t* bytes, int n_dst,
                               void* const* dst, void* stream) {
  using namespace atk;
  if (n_seg < 0 || n_seg > kPushMaxSegments || n_dst < 0 || n_dst > kPushMaxDst) return ATK_ERR_BAD_ARG;
  if (n_seg == 0 || n_dst == 0) return ATK_OK;
  if (src == nullptr || bytes == nullptr || dst == nullptr) return ATK_ERR_BAD_ARG;
  PushParams p = {};
  p.n_seg = n_seg;
  p.n_dst = n_dst;
  bool vec = true;
  unsigned long long total = 0;
  for (int s = 0; s < n_seg; ++s) {
    if (bytes[s] == 0) continue;
    if (src[s] == nullptr || bytes[s] % 4 != 0 || reinterpret_cast<uintptr_t>(src[s]) % 4 != 0) return ATK_ERR_BAD_ARG;
    vec = vec && bytes[s] % 16 == 0 && reinterpret_cast<uintptr_t>(src[s]) % 16 == 0;
    for (int d = 0; d < n_dst; ++d) {
      void* q = dst[s * n_dst + d];
      if (q == nullptr || reinterpret_cast<uintptr_t>(q) % 4 != 0) return ATK_ERR_BAD_ARG;
      vec = vec && reinterpret_cast<uintptr_t>(q) % 16 == 0;
    }
    total += bytes[s];
  }
  if (total == 0) return ATK_OK;
  const unsigned long long piece = vec ? 16 : 4;
  unsigned long long most = 0;
  for (int s = 0; s < n_seg; ++s) {
    p.src[s] = static_cast<const unsigned char*>(src[s]);
    p.pieces[s] = bytes[s] / piece;
    if (p.pieces[s] > most) most = p.pieces[s];
    for (int d = 0; d < n_dst; ++d) p.dst[s][d] = static_cast<unsigned char*>(dst[s * n_dst + d]);
  }
  // enough blocks to keep every link busy, no more than the longest segment needs
  const unsigned long long want = (most + kPushThreads * 4ull - 1) / (kPushThreads * 4ull);
  const unsigned long long cap = 4ull * sm_count_of_current_device();
  const unsigned blocks = static_cast<unsigned>(want < 1 ? 1 : (want > cap ? cap : want));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t rc;
  if (vec) rc = launch_overlapped(push_blocks_kernel<uint4>, dim3(blocks), dim3(kPushThreads), 0, st, p);
  else rc = launch_overlapped(push_blocks_kernel<uint32_t>, dim3(blocks), dim3(kPushThreads), 0, st, p);
  note_launch();
  return rc == cudaSuccess && cudaGetLastError() == cudaSuccess ? ATK_OK : ATK_ERR_CUDA;
}

// ---- buffers that peers can store to ---------------------------------------------
// A buffer of its own cudaMalloc (the handle of an interprocess mapping names a whole
// allocation), zero-filled, and its 64-byte handle for the other ranks of the node.
extern "C" int atk_peer_alloc(size_t bytes, void** ptr, void* handle64) {
  if (ptr == nullptr || handle64 == nullptr || bytes == 0) return ATK_ERR_BAD_ARG;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle travels as 64 bytes");
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) {
    cudaGetLastError();
    return ATK_ERR_CUDA;
  }
  cudaIpcMemHandle_t h;
  if (cudaMemset(p, 0, bytes) != cudaSuccess || cudaIpcGetMemHandle(&h, p) != cudaSuccess) {
    cudaGetLastError();
    cudaFree(p);
    return ATK_ERR_CUDA;
  }
  memcpy(handle64, &h, sizeof(h));
  *ptr = p;
  return ATK_OK;
}

// Maps a peer's buffer into the address space of the CURRENT device (the one whose
// kernels will store to it) and enables peer access to its GPU if that is still missing.
extern "C" int atk_peer_open(const void* handle64, void** ptr) {
  if (ptr == nullptr || handle64 == nullptr) return ATK_ERR_BAD_ARG;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
    cudaGetLastError();
    return ATK_ERR_CUDA;
  }
  *ptr = p;
  return ATK_OK;
}

extern "C" int atk_peer_close(void* ptr) {
  if (ptr == nullptr) return ATK_OK;
  if (cudaIpcCloseMemHandle(ptr) != cudaSuccess) {
    cudaGetLastError();
    return ATK_ERR_CUDA;
  }
  return ATK_OK;
}

extern "C" int atk_peer_free(void* ptr) {
  if (ptr == nullptr) return ATK_OK;
  if (cudaFree(ptr) != cudaSuccess) {
    cudaGetLastError();
    return ATK_ERR_CUDA;
  }
  return ATK_OK;
}
