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
 * The functions exist for three carrier types (atk_oracle_body.inc is included
 * once per type): float (plain names), double (suffix _f64) and int64_t
 * (suffix _i64).  The 16-bit float formats convert to float exactly and the
 * reference compares Half/BFloat16 through float as well; the integer types of
 * the reference's dispatch (.cu:449-453) convert to int64_t exactly.  Callers
 * widen the input to its carrier, run the oracle and narrow the selected values
 * back (exact round trip).
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


#define ATK_PASTE(a, b) a##b

#define ATK_T float
#define ATK_NAME(n) n
#define ATK_ISNAN(v) isnan(v)
#include "atk_oracle_body.inc"
#undef ATK_T
#undef ATK_NAME
#undef ATK_ISNAN

#define ATK_T double
#define ATK_NAME(n) ATK_PASTE(n, _f64)
#define ATK_ISNAN(v) isnan(v)
#include "atk_oracle_body.inc"
#undef ATK_T
#undef ATK_NAME
#undef ATK_ISNAN

#define ATK_T int64_t
#define ATK_NAME(n) ATK_PASTE(n, _i64)
#define ATK_ISNAN(v) 0
#include "atk_oracle_body.inc"
#undef ATK_T
#undef ATK_NAME
#undef ATK_ISNAN


/* Reference scores for the fused producer (include/atk.h, atk_score_topk /
 * atk_scores): one query per row against the row's n keys, the dot product formed
 * in double precision (the 16-bit inputs and their products are exact there),
 * rounded to float and multiplied by `scale` in float.  The caller rounds the
 * result to the element type.  The kernels accumulate in float32 inside matrix
 * instructions, so they agree with this to within one unit in the last place of
 * the 16-bit result (a tolerance, stated in the tests); what the fused kernel
 * SELECTS is checked exactly, against the operator's oracle applied to the
 * scores atk_scores wrote.  No counterpart in the reference. */
int atk_oracle_scores(const float* q, const float* keys, int64_t rows, int64_t n, int64_t d, float scale,
                      float* out) {
  if (rows < 0 || n < 0 || d <= 0) return -1;
  for (int64_t r = 0; r < rows; ++r) {
    const float* qr = q + r * d;
    for (int64_t i = 0; i < n; ++i) {
      const float* kr = keys + (r * n + i) * d;
      double a = 0.0;
      for (int64_t t = 0; t < d; ++t) a += (double)kr[t] * (double)qr[t];
      out[r * n + i] = (float)a * scale;
    }
  }
  return 0;
}
