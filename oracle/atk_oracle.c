/*
 * CPU oracle for the bucketed approximate top-k path.  TEST INFRASTRUCTURE ONLY:
 * nothing in the product links, loads or calls this file; only tests/, the
 * smoke check and the CPU-baseline leg of the benchmark may use it, and only as
 * the checker.
 *
 * It is a from-scratch scalar restatement of what the reference's CUDA operator
 * computes, written from the semantics of
 *   approx_topk/priority_queue_approx_topk.cu
 * (bucket geometry :25-56, queue insertion rule :58-79, scan order and sentinel
 * :81-107, index fix-up :109-119, output slot layout :121-147 and :190-200) and
 * of the stage-2 step in approx_topk/priority_queue.py:85-88, plus the k_b = 1
 * "bucketed argmax" of approx_topk/experimental/bucketed_argmax.py:18-42.
 *
 * All arithmetic is done on float: the 16-bit formats convert to float exactly
 * and the reference compares Half/BFloat16 through float as well, so callers
 * widen bf16/fp16 inputs to float, run the oracle and narrow the selected
 * values back (exact round trip).
 *
 * Parity status: pinned.  tests/test_oracle_golden.py checks these functions
 * against every golden vector the reference's tests hold for the path and
 * against fixtures produced by importing the reference's Python modules
 * (tests/golden/make_golden.py); the -m gpu tests additionally compare them
 * with the reference's own CUDA operator compiled by oracle/build_ref.py.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ATK_ORACLE_MAX_J 4

/* Bucket geometry, reference .cu:25-56.
 * size   = n / b (+1 for the first n % b buckets)
 * interleaved: start = bucket, stride = b
 * contiguous : start = prefix sum of sizes, stride = 1                     */
static void bucket_geometry(int64_t bucket, int64_t n, int64_t b, int interleaved,
                            int64_t* size, int64_t* start, int64_t* stride) {
  int64_t base = n / b;
  int64_t rem = n - base * b;
  *size = base + (bucket < rem ? 1 : 0);
  if (interleaved) {
    *start = bucket;
    *stride = b;
  } else {
    int64_t big = bucket < rem ? bucket : rem;
    int64_t normal = bucket > rem ? bucket - rem : 0;
    *start = big * (base + 1) + normal * base;
    *stride = 1;
  }
}

/* Queue insertion, reference .cu:58-79 with largest == true.  The queue is kept
 * ascending; the new item stops at the first slot that is strictly greater,
 * otherwise it shifts that slot one place towards the front and takes its
 * place.  Consequence: a later element outranks an earlier equal one.        */
static void queue_insert(float v, int64_t index, float* qv, int64_t* qi, int j) {
  for (int i = 0; i < j; ++i) {
    if (qv[i] > v) break;
    if (i > 0) {
      qv[i - 1] = qv[i];
      qi[i - 1] = qi[i];
    }
    qv[i] = v;
    qi[i] = index;
  }
}

/*
 * Stage 1 of the operator for `rows` independent rows of length n.
 *   x[row * row_stride + i]            input (float, already widened)
 *   out_vals / out_idx [row * k0 + s]  slot s = bucket * j + q, q ascending
 *                                      (reference .cu:190-200, queue order)
 * `sentinel` is the initial queue value.  The reference uses the dtype's
 * lowest() with an uninitialised index (.cu:95-101); the oracle reports such
 * never-filled slots with index -1.  Passing -INFINITY instead gives the
 * behaviour of the new kernels (every slot is a real element).
 * Returns 0, or -1 on invalid arguments (same conditions the reference checks
 * at .cu:329-330, :402, :425-435).
 */
int atk_oracle_stage1(const float* x, int64_t rows, int64_t n, int64_t row_stride,
                      int64_t k0, int j, int interleaved, float sentinel,
                      float* out_vals, int64_t* out_idx) {
  if (k0 == 0) return 0;
  if (j < 1 || j > ATK_ORACLE_MAX_J || k0 % j != 0 || k0 > n) return -1;
  int64_t b = k0 / j;
  for (int64_t r = 0; r < rows; ++r) {
    const float* row = x + r * row_stride;
    for (int64_t c = 0; c < b; ++c) {
      int64_t size, start, stride;
      bucket_geometry(c, n, b, interleaved, &size, &start, &stride);
      float qv[ATK_ORACLE_MAX_J];
      int64_t qi[ATK_ORACLE_MAX_J];
      for (int q = 0; q < j; ++q) {
        qv[q] = sentinel;
        qi[q] = -1;
      }
      for (int64_t i = 0; i < size; ++i)            /* scan loop, .cu:103-106 */
        queue_insert(row[start + i * stride], i, qv, qi, j);
      for (int q = 0; q < j; ++q) {                 /* index fix-up, .cu:109-119 */
        out_vals[r * k0 + c * j + q] = qv[q];
        out_idx[r * k0 + c * j + q] = qi[q] < 0 ? -1 : start + qi[q] * stride;
      }
    }
  }
  return 0;
}

typedef struct {
  float v;
  int64_t slot;
} cand_t;

static int cand_cmp(const void* pa, const void* pb) {
  const cand_t* a = (const cand_t*)pa;
  const cand_t* b = (const cand_t*)pb;
  /* value descending, NaN first (torch.topk treats NaN as the largest), then
   * candidate slot ascending so the result is deterministic. */
  int an = isnan(a->v), bn = isnan(b->v);
  if (an != bn) return an ? -1 : 1;
  if (!an) {
    if (a->v > b->v) return -1;
    if (a->v < b->v) return 1;
  }
  return (a->slot > b->slot) - (a->slot < b->slot);
}

/*
 * Stage 2: exact top-k of the k0 candidates of every row, indices carried
 * along (reference priority_queue.py:85-88: torch.topk(sorted=False) + gather).
 * The value multiset is unique; which of several equal candidates at the k-th
 * boundary is kept is implementation-defined in torch, here the lowest slot.
 * Output order: value descending.
 */
int atk_oracle_select(const float* cand_vals, const int64_t* cand_idx, int64_t rows,
                      int64_t k0, int64_t k, float* out_vals, int64_t* out_idx) {
  if (k > k0) return -1;
  if (k == 0) return 0;
  cand_t* buf = (cand_t*)malloc(sizeof(cand_t) * (size_t)k0);
  if (!buf) return -2;
  for (int64_t r = 0; r < rows; ++r) {
    for (int64_t s = 0; s < k0; ++s) {
      buf[s].v = cand_vals[r * k0 + s];
      buf[s].slot = s;
    }
    qsort(buf, (size_t)k0, sizeof(cand_t), cand_cmp);
    for (int64_t s = 0; s < k; ++s) {
      out_vals[r * k + s] = buf[s].v;
      out_idx[r * k + s] = cand_idx[r * k0 + buf[s].slot];
    }
  }
  free(buf);
  return 0;
}

/*
 * The whole operator approx_topk.topk(x, k, dim=-1, j, k_mult, interleaved)
 * (reference priority_queue.py:51-88): stage 1 with k0 = k * k_mult, then the
 * exact select when k0 > k.
 */
int atk_oracle_topk(const float* x, int64_t rows, int64_t n, int64_t row_stride,
                    int64_t k, int j, int64_t k_mult, int interleaved, float sentinel,
                    float* out_vals, int64_t* out_idx) {
  if (k_mult < 1) return -1;
  int64_t k0 = k * k_mult;
  if (k0 == k)
    return atk_oracle_stage1(x, rows, n, row_stride, k0, j, interleaved, sentinel,
                             out_vals, out_idx);
  float* cv = (float*)malloc(sizeof(float) * (size_t)(rows * k0));
  int64_t* ci = (int64_t*)malloc(sizeof(int64_t) * (size_t)(rows * k0));
  if (!cv || !ci) {
    free(cv);
    free(ci);
    return -2;
  }
  int rc = atk_oracle_stage1(x, rows, n, row_stride, k0, j, interleaved, sentinel, cv, ci);
  if (rc == 0) rc = atk_oracle_select(cv, ci, rows, k0, k, out_vals, out_idx);
  free(cv);
  free(ci);
  return rc;
}

/*
 * k_b = 1 "bucketed argmax", reference experimental/bucketed_argmax.py:18-42:
 * the row is padded to a multiple of k with `pad_value` (the dtype's minimum),
 * interleaved bucket c = {c, c+k, ...}; contiguous bucket c = the fixed-size
 * chunk [c*m, (c+1)*m) with m = ceil(n/k) (note: a different contiguous
 * geometry from the CUDA operator's).  torch.max returns the FIRST maximum on
 * ties on CPU; the Triton kernels keep the first maximum too (strict '<' at
 * bucketed_argmax.py:101).  Output order = bucket order.
 */
int atk_oracle_bucketed_argmax(const float* x, int64_t rows, int64_t n, int64_t row_stride,
                               int64_t k, int interleaved, float pad_value,
                               float* out_vals, int64_t* out_idx) {
  if (k <= 0) return k == 0 ? 0 : -1;
  int64_t m = (n + k - 1) / k; /* elements per bucket after padding */
  for (int64_t r = 0; r < rows; ++r) {
    const float* row = x + r * row_stride;
    for (int64_t c = 0; c < k; ++c) {
      float best = 0.f;
      int64_t best_i = -1;
      for (int64_t i = 0; i < m; ++i) {
        int64_t pos = interleaved ? c + i * k : c * m + i;
        float v = pos < n ? row[pos] : pad_value;
        if (best_i < 0 || v > best || (isnan(v) && !isnan(best))) {
          best = v;
          best_i = pos;
        }
      }
      out_vals[r * k + c] = best;
      out_idx[r * k + c] = best_i;
    }
  }
  return 0;
}

/*
 * Recall of an approximate result against the exact top-k of the same row, by
 * the reference's tie-robust definition (benchmarks/run_recall.py:27-36): the
 * fraction of returned values that are >= the true k-th largest value.
 */
double atk_oracle_recall(const float* x, int64_t rows, int64_t n, int64_t row_stride,
                         const float* approx_vals, int64_t k) {
  if (k == 0 || rows == 0) return 1.0;
  cand_t* buf = (cand_t*)malloc(sizeof(cand_t) * (size_t)n);
  if (!buf) return -1.0;
  double hits = 0;
  for (int64_t r = 0; r < rows; ++r) {
    for (int64_t i = 0; i < n; ++i) {
      buf[i].v = x[r * row_stride + i];
      buf[i].slot = i;
    }
    qsort(buf, (size_t)n, sizeof(cand_t), cand_cmp);
    float kth = buf[k - 1].v;
    for (int64_t s = 0; s < k; ++s)
      if (approx_vals[r * k + s] >= kth) hits += 1;
  }
  free(buf);
  return hits / ((double)rows * (double)k);
}
