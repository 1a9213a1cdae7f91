/*
 * atk.h — C ABI of libatk.so, the sm_100a implementation of bucketed approximate
 * top-k (stage 1: per-bucket top-j; stage 2: exact select over the candidates).
 *
 * This is the boundary a host binding uses in place of the reference's
 * JIT-compiled pybind module.  Every function is plain `extern "C"`, takes raw
 * device (or, where stated, host) pointers and sizes, launches on the stream it
 * is given, never allocates device memory (the caller owns all buffers and the
 * workspace), never synchronises unless stated, never throws and never aborts:
 * it returns ATK_OK (0) or a negative ATK_ERR_* code.  All entry points except
 * atk_select_static are re-entrant and may be called concurrently from several
 * host threads on different streams (atk_select_static shares one built-in
 * scratch array per device: see its description).  The device the pointers
 * live on must be current.
 *
 * NaN inputs are outside the contract for every element type and every entry
 * point, as they are in the reference (its insertion loop makes the result
 * depend on the scan order): nothing crashes or hangs, every returned index is
 * a position of the row, but which elements are returned next to a NaN is
 * unspecified and may depend on the launch shape.
 *
 * Reference interfaces replaced (paths inside the reference project):
 *   approx_topk/priority_queue_approx_topk.cu:378-387,523-525  PriorityQueueTopK (pybind)
 *   approx_topk/priority_queue.py:85-88                        stage 2 (torch.topk + gather)
 *   approx_topk/experimental/bucketed_argmax.py:18-42,145-202  topk_torch / topk_triton
 *   approx_topk/cuda_extensions.py:12-27                       JIT loader (now: dlopen of this library)
 */
#ifndef ATK_H_
#define ATK_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Element types of the input / value output: the nine the reference's native
 * operator dispatches over (AT_DISPATCH_ALL_TYPES_AND2(Half, BFloat16),
 * approx_topk/priority_queue_approx_topk.cu:449-453).  The three float types
 * of 32 bits or fewer are the tuned ones; the others run the same kernels with
 * an exact integer / double compare. */
enum {
  ATK_F32 = 0, ATK_F16 = 1, ATK_BF16 = 2,
  ATK_F64 = 3, ATK_I32 = 4, ATK_I64 = 5, ATK_I16 = 6, ATK_I8 = 7, ATK_U8 = 8
};

/* Status codes.  The Python host maps them to the exception types the
 * reference raises for the same condition. */
enum {
  ATK_OK = 0,
  ATK_ERR_BAD_J = -1,        /* j outside 1..4            (reference .cu:425-435) */
  ATK_ERR_J_DIVIDES_K = -2,  /* k0 % j != 0               (reference .cu:402)     */
  ATK_ERR_K_TOO_LARGE = -3,  /* k0 > n                    (reference .cu:329-330) */
  ATK_ERR_BAD_DTYPE = -4,
  ATK_ERR_BAD_ARG = -5,      /* null pointer, negative size, k_mult < 1, k > k0 ... */
  ATK_ERR_WORKSPACE = -6,    /* workspace missing or smaller than *_workspace_bytes */
  ATK_ERR_TOO_LARGE = -7,    /* a size exceeds what the kernels index (see each function) */
  ATK_ERR_CUDA = -8,         /* a CUDA runtime call failed; see cudaGetLastError */
  ATK_ERR_SCRATCH_LIMIT = -9 /* atk_select_static: the problem needs more than the built-in scratch */
};

/* Formats of the operator's final output (atk_topk_ex).  The reference fixes
 * int64 indices (approx_topk/priority_queue.py:65-67); the narrower ones are
 * opt-in for consumers that do not need 64-bit positions: on the headline
 * workload the int64 indices are two thirds of all bytes written. */
enum {
  ATK_OUT_I64 = 0,   /* out_vals: rows x k of dtype; out_idx: rows x k int64 (the default) */
  ATK_OUT_I32 = 1,   /* out_vals: rows x k of dtype; out_idx: rows x k int32; needs n < 2^31 */
  ATK_OUT_REC32 = 2  /* out_vals: rows x k records of 8 bytes {uint32 value bits (the element's
                        bits zero-extended), int32 position}; out_idx unused (may be NULL);
                        element types of at most 32 bits, n < 2^31 */
};

/* Library version, major*10000 + minor*100 + patch. */
int atk_version(void);

/* Static, human-readable text for a status code. */
const char* atk_strerror(int status);

/* Compute-capability check: returns ATK_OK when the current device can run the
 * kernels in this library (sm_100), ATK_ERR_CUDA otherwise. */
int atk_device_supported(void);

/*
 * Stage 1 — per-bucket top-j.  Replaces PriorityQueueTopK
 * (priority_queue_approx_topk.cu:378-521) with largest = true.
 *
 *   x              rows x n elements of `dtype`, row r at x + r*row_stride (elements)
 *   k0             number of candidates per row, k0 = j * buckets; needs k0 % j == 0, k0 <= n
 *   interleaved    1: bucket c = {c, c+b, c+2b, ...};  0: contiguous segments whose
 *                  sizes differ by at most one, larger ones first (.cu:25-56)
 *   mode           -1 auto / 0 / 1 — the reference's multithread_buckets switch.
 *                  Accepted for signature parity; one kernel family serves all modes.
 *   out_vals       rows x k0 of `dtype`, row r at out_vals + r*out_row_stride
 *   out_idx        rows x k0 int64 positions along the row, same layout
 *
 * Slot layout and tie rule are the reference's thread-per-bucket kernel's:
 * bucket c owns slots c*j .. c*j+j-1 in ascending (value, index) order, and of
 * equal values the later position wins (.cu:58-79,190-200).  Unlike the
 * reference the queue starts at -inf, so -inf inputs are selectable and every
 * output slot is a real element.
 * k0 == 0 is a no-op.  Limits: n / buckets < 2^31.
 *
 * workspace (optional, may be NULL / 0): atk_stage1_workspace_bytes() bytes of
 * device scratch, 256-byte aligned.  Shapes with few rows and few buckets
 * cannot occupy the GPU with one block per group of columns (the weakness of
 * the reference's thread-per-bucket kernel); given scratch, the kernel also
 * splits the stripes of a column over several blocks and merges their partial
 * candidates in a second small launch.  The result does not depend on whether
 * (or how much) scratch is given, only the speed on such shapes does.
 */
size_t atk_stage1_workspace_bytes(int dtype, int64_t rows, int64_t n, int64_t k0, int j, int interleaved);
int atk_stage1(const void* x, int dtype, int64_t rows, int64_t n, int64_t row_stride,
               int64_t k0, int j, int interleaved, int mode,
               void* out_vals, int64_t* out_idx, int64_t out_row_stride,
               void* workspace, size_t workspace_bytes, void* stream);

/*
 * Stage 1 over a column slab of one long interleaved row that is sharded over
 * several GPUs (no counterpart in the reference, which is single-GPU; needed
 * for the bucket-group sharding of a single long row).  `slab` is a dense
 * stripes x cols array holding columns [col_offset, col_offset+cols) of the
 * stripes x total_buckets view of the row; every bucket here has exactly
 * `stripes` elements.  Writes cols*j candidates whose indices are positions in
 * the full row: stripe*total_buckets + col_offset + col.
 * workspace: optional scratch of atk_stage1_slab_workspace_bytes() bytes, same
 * role as in atk_stage1 (a slab of few columns needs it to occupy the GPU).
 */
size_t atk_stage1_slab_workspace_bytes(int dtype, int64_t stripes, int64_t cols, int j);
int atk_stage1_slab(const void* slab, int dtype, int64_t stripes, int64_t cols,
                    int64_t total_buckets, int64_t col_offset, int j,
                    void* out_vals, int64_t* out_idx,
                    void* workspace, size_t workspace_bytes, void* stream);

/*
 * Stage 2 — exact top-k of k0 candidates per row, indices carried along.
 * Replaces torch.topk(sorted=False) + gather (priority_queue.py:85-88).
 * Output order is unspecified but deterministic; of equal values at the k-th
 * boundary the lowest candidate slots are kept.
 * workspace: atk_select_workspace_bytes() bytes of device memory, 256-byte
 * aligned, contents irrelevant on entry (may be NULL when that returns 0).
 */
size_t atk_select_workspace_bytes(int dtype, int64_t rows, int64_t k0, int64_t k);
int atk_select(const void* cand_vals, const int64_t* cand_idx, int dtype, int64_t rows,
               int64_t k0, int64_t cand_row_stride, int64_t k,
               void* out_vals, int64_t* out_idx, int64_t out_row_stride,
               void* workspace, size_t workspace_bytes, void* stream);

/*
 * atk_select without a workspace argument, for callers that cannot allocate
 * device memory.  It has no counterpart in the reference.
 *
 * Who needs it: a plugin loaded into a host process that owns the whole GPU
 * memory budget (an inference server or a database engine that carves up device
 * memory at start-up and gives extensions no allocator), a latency-critical
 * loop in which a cudaMalloc may stall the device, or a caller that only holds
 * raw pointers and a stream from another runtime.  Such callers can still pass
 * their candidate and output buffers, but have nowhere to get the select's
 * scratch (digit histograms, running state, per-block counts) from.
 *
 * Here that scratch is a fixed array of ATK_SELECT_STATIC_SCRATCH_BYTES (1 MiB)
 * of device memory that is part of the library image: every GPU that loads the
 * library holds it until the process exits.  The call is otherwise identical
 * to atk_select and returns the same bits.  It calls no cudaMalloc, cudaFree
 * or any other allocating routine.
 *
 * Limit: when atk_select_workspace_bytes(dtype, rows, k0, k) exceeds the
 * built-in 1 MiB the call is refused with ATK_ERR_SCRATCH_LIMIT and launches
 * nothing (rows of up to 16384 candidates need no scratch at all; one row of
 * 2^21 fp32 candidates needs about 33 KiB; 16 rows of 2^20 about 0.45 MiB).
 *
 * First call on a device: looks up the device address of the array
 * (cudaGetSymbolAddress, with that device current) and caches it per device.
 * Make this first call before starting any stream capture.
 *
 * Sharing: all calls on a device use the same array.  It keeps what the
 * previous call left in it; the parts that must start at zero are cleared on
 * the stream at the start of every call, so back-to-back calls on one stream
 * are safe.  Two calls whose GPU work overlaps in time (different streams or
 * host threads without ordering between them) race on the array and give
 * undefined results: order them, or use atk_select with separate workspaces.
 */
#define ATK_SELECT_STATIC_SCRATCH_BYTES (1u << 20)
int atk_select_static(const void* cand_vals, const int64_t* cand_idx, int dtype, int64_t rows,
                      int64_t k0, int64_t cand_row_stride, int64_t k,
                      void* out_vals, int64_t* out_idx, int64_t out_row_stride, void* stream);

/*
 * The whole operator approx_topk.topk(x, k, dim=-1, j, k_mult, interleaved)
 * (priority_queue.py:14-88): stage 1 with k0 = k*k_mult and, when k_mult > 1,
 * the exact select over the candidates, which pass through the workspace
 * (they are re-read from L2 for the shapes of the reference's configurations).
 * With k_mult == 1 the workspace is optional (see atk_stage1).
 */
size_t atk_topk_workspace_bytes(int dtype, int64_t rows, int64_t n, int64_t k, int j,
                                int64_t k_mult);
int atk_topk(const void* x, int dtype, int64_t rows, int64_t n, int64_t row_stride,
             int64_t k, int j, int64_t k_mult, int interleaved, int mode,
             void* out_vals, int64_t* out_idx, int64_t out_row_stride,
             void* workspace, size_t workspace_bytes, void* stream);

/*
 * atk_topk with a choice of output format (ATK_OUT_*); no counterpart in the
 * reference, whose indices are always int64.  Everything else is atk_topk:
 * the same selection, the same order of the k pairs inside a row, the same
 * workspace (atk_topk_workspace_bytes).  out_row_stride counts pairs (records
 * for ATK_OUT_REC32).  Interleaved buckets only (the layout the narrow formats
 * are meant for); ATK_OUT_I64 is accepted for every layout and is atk_topk.
 */
int atk_topk_ex(const void* x, int dtype, int64_t rows, int64_t n, int64_t row_stride,
                int64_t k, int j, int64_t k_mult, int interleaved, int mode, int out_format,
                void* out_vals, void* out_idx, int64_t out_row_stride,
                void* workspace, size_t workspace_bytes, void* stream);

/*
 * Fused score producer + operator for the attention-score use case (one query
 * per row against that row's n keys of dimension d): computes
 *     score[r][i] = round_to_dtype( (sum over t = 0..d-1 of q[r][t] * keys[r][i][t]) * scale )
 * on the fly -- the products are exact in float32 and accumulated in float32
 * by warp-wide matrix instructions (the order of the additions inside one
 * instruction is the hardware's), the scaled sum is rounded once to `dtype`
 * (nearest even) -- and applies approx_topk.topk(score, k, dim=-1, j, k_mult)
 * with interleaved buckets to it, without the rows x n scores ever being
 * written to memory.  No counterpart in the reference, whose users materialise
 * the scores with a matrix product first (the key-selection experiments behind
 * its paper's figures).  The selection is exactly atk_topk's on the scores that
 * atk_scores writes for the same arguments (same arithmetic, bit for bit); a
 * score of -0.0 is returned as +0.0.
 *   q      rows x d elements of `dtype` (ATK_F16 or ATK_BF16), row r at q + r*q_row_stride
 *   keys   rows x n x d elements, the keys of row r at keys + r*keys_row_stride, key i at + i*d;
 *          16-byte aligned, keys_row_stride a multiple of 8 elements; d = 64 or 128
 *   out_*  rows x k values (`dtype`) and int64 key positions, as for atk_topk
 * workspace: atk_score_topk_workspace_bytes() bytes (candidates and select state when k_mult > 1).
 * Limits: n / (k*k_mult/j) < 65536.
 *
 * atk_scores: the scores alone, rows x n elements of `dtype` at out_scores +
 * r*out_row_stride (the unfused form; also what the fused kernel's selection is
 * checked against).  At most 65535 rows.
 */
int atk_scores(const void* q, const void* keys, int dtype, int64_t rows, int64_t n, int64_t d,
               int64_t q_row_stride, int64_t keys_row_stride, float scale,
               void* out_scores, int64_t out_row_stride, void* stream);
size_t atk_score_topk_workspace_bytes(int dtype, int64_t rows, int64_t n, int64_t k, int j, int64_t k_mult);
int atk_score_topk(const void* q, const void* keys, int dtype, int64_t rows, int64_t n, int64_t d,
                   int64_t q_row_stride, int64_t keys_row_stride, float scale,
                   int64_t k, int j, int64_t k_mult,
                   void* out_vals, int64_t* out_idx, int64_t out_row_stride,
                   void* workspace, size_t workspace_bytes, void* stream);

/*
 * k_b = 1 bucketed arg-max with the conventions of
 * experimental/bucketed_argmax.py (topk_torch :18-42, Triton kernels :70-142):
 * k buckets, rows padded to a multiple of k with the dtype's lowest value,
 * contiguous buckets are fixed chunks of ceil(n/k), the FIRST maximum wins a
 * tie, outputs in bucket order.  k may exceed n (all-padding buckets return
 * the lowest value and the first padded position).
 * workspace: optional, atk_stage1_workspace_bytes(dtype, rows, n, k, 1, interleaved)
 * bytes, same role as in atk_stage1.
 */
int atk_bucketed_argmax(const void* x, int dtype, int64_t rows, int64_t n, int64_t row_stride,
                        int64_t k, int interleaved,
                        void* out_vals, int64_t* out_idx, int64_t out_row_stride,
                        void* workspace, size_t workspace_bytes, void* stream);

/*
 * Host-buffer form of atk_topk: x_host / out_*_host are HOST pointers (pinned
 * memory gives full PCIe speed, pageable memory works).  Rows are processed in
 * chunks so that the upload of chunk i+1, the kernels of chunk i and the
 * download of chunk i-1 overlap.  `device_scratch` is caller-allocated device
 * memory of atk_topk_host_scratch_bytes() bytes.  Works on two internal streams
 * (created on the first call on a device and kept), synchronises before
 * returning.  Calls that overlap on one device from several host threads are
 * correct (each has its own scratch) but share those streams, so their work
 * is serialised.  chunk_rows <= 0 picks a default.
 */
size_t atk_topk_host_scratch_bytes(int dtype, int64_t rows, int64_t n, int64_t k, int j,
                                   int64_t k_mult, int64_t chunk_rows);
int atk_topk_host(const void* x_host, int dtype, int64_t rows, int64_t n, int64_t row_stride,
                  int64_t k, int j, int64_t k_mult, int interleaved,
                  void* out_vals_host, int64_t* out_idx_host,
                  void* device_scratch, size_t scratch_bytes, int64_t chunk_rows);

/*
 * Consumer-side step: gather the records the operator selected.  No counterpart
 * in the reference (its users call torch.gather / index_select on the indices
 * that approx_topk.topk returns, e.g. to fetch the selected keys and values of
 * an attention head).
 *
 *   src   rows x n records of `record_bytes` bytes each; record (r, i) starts at
 *         src + r*src_row_stride_bytes + i*record_bytes
 *   idx   rows x k positions in [0, n), row r at idx + r*idx_row_stride (elements)
 *   out   rows x k records, dense: record (r, q) at out + (r*k + q)*record_bytes
 *
 * Records move in 16-byte pieces when `record_bytes`, the strides and the
 * pointers are multiples of 16, else in pieces of 4, 2 or 1 bytes.  A position
 * outside [0, n) yields a record of zero bytes (nothing is read for it).
 */
int atk_gather_records(const void* src, int64_t rows, int64_t n, int64_t record_bytes,
                       int64_t src_row_stride_bytes, const int64_t* idx, int64_t k,
                       int64_t idx_row_stride, void* out, void* stream);

/*
 * Candidate exchange of the multi-GPU long row over peer memory (no counterpart in
 * the reference, which is single-GPU).  Copies up to ATK_PUSH_MAX_SEGMENTS blocks
 * of this GPU's memory to n_dst <= ATK_PUSH_MAX_DST destinations each, with one
 * kernel that reads every piece once and stores it to every destination.  The
 * destinations are device pointers valid in this process and may lie in other GPUs'
 * memory (CUDA IPC mappings with peer access): that is the use, a rank writes its
 * block of stage-1 candidates into every peer's candidate buffer over NVLink.
 *
 *   src[s], bytes[s]    segment s in this GPU's memory (host arrays of n_seg entries)
 *   dst[s*n_dst + d]    where segment s goes in destination d (host array)
 *
 * Pointers and sizes must be multiples of 4 bytes (ATK_ERR_BAD_ARG otherwise);
 * pieces of 16 bytes are used when everything is a multiple of 16.  Segments of a
 * destination must not overlap one another or a source.  The call only stores:
 * the peers learn that the data has arrived by whatever orders their streams
 * after this kernel (approx_topk.distributed uses a small all-reduce), never by
 * polling memory.
 */
#define ATK_PUSH_MAX_SEGMENTS 4
#define ATK_PUSH_MAX_DST 16
int atk_push_blocks(int n_seg, const void* const* src, const size_t* bytes, int n_dst,
                    void* const* dst, void* stream);

/*
 * Buffers for atk_push_blocks destinations (CUDA interprocess memory handles).
 *   atk_peer_alloc  a zero-filled buffer of its own cudaMalloc on the current device,
 *                   and its 64-byte handle, which the caller sends to the other ranks
 *                   of the node (one process per GPU, all GPUs visible to every process);
 *   atk_peer_open   maps the buffer behind a handle received from another rank into the
 *                   address space of the CURRENT device, i.e. of the GPU whose kernels
 *                   will store to it, and enables peer access to the owner's GPU;
 *   atk_peer_close  unmaps it; every rank closes its mappings of a buffer before the
 *                   owner calls atk_peer_free.
 * These calls synchronise the device like cudaMalloc / cudaFree do: set-up and tear-down
 * only, never inside a CUDA-graph capture.
 */
int atk_peer_alloc(size_t bytes, void** ptr, void* handle64);
int atk_peer_open(const void* handle64, void** ptr);
int atk_peer_close(void* ptr);
int atk_peer_free(void* ptr);

/* Number of kernel launches issued by this library on the calling thread since
 * the last atk_reset_launch_count(); benchmarks use it to report launches. */
int64_t atk_launch_count(void);
void atk_reset_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* ATK_H_ */
