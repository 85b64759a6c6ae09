// What the passes of the tensor-core bucket scan share: the constants of the scheme and the parameter block.
#pragma once

#include "common.cuh"

namespace lsa {

constexpr int kScanRoom = 2048;        // survivors a row can hold over all its lists
constexpr int kScanMinVisible = 1024;  // rows that see fewer buckets take the exact scan (it is cheap there)
constexpr int kScanRetry = 128;        // rows a call can hand to the split exact scan; any more take the plain one
// With both operands rounded to bf16 and fp32 accumulation, the score of a query q against a row of length rho lies
// within |q| * rho * (2^-8 + 2^-16) of the real dot: |q| * (rho * kScanEps + kScanAbsolute) bounds that with room to
// spare, the absolute part covering the rounding of the fixed-order fp32 dots the picks are ranked by. The rows the
// scan multiplies are the centroids LESS A COMMON CENTRE (a query's score against the centre is the same for every
// bucket, so the ranking is the same), and EVERY BUCKET CARRIES ITS OWN rho: where the index vectors lie in a narrow
// cone most rows are short and their scores sharp, and the odd long one only widens its own interval.
constexpr float kScanEps = 1.0f / 240.0f;
constexpr float kScanAbsolute = 1e-5f;

// The slack of a bucket's score, per unit of |q|.
__host__ __device__ __forceinline__ float scan_slack(float rho) { return fmaf(rho, kScanEps, kScanAbsolute); }

struct ScanParams {
  const uint16_t *queries_bf16;    // [rows padded to 128, 64]
  const uint16_t *centroids_bf16;  // [m, 64]
  const int32_t *visible;          // [R]
  const int32_t *row_keep;         // [R] or NULL
  int32_t *flags;                  // [R]: nonzero = the row takes the exact scan (the scan itself flags a row whose
                                   // samples say that more buckets would reach its bar than the pick has room for)
  const float *norms;              // [R] lengths of the query rows
  const float *lengths;            // [m] length of every row of the operand (a bucket's rho), or NULL: all `radius`
  const float *radius;             // [1] the greatest of them, or NULL: 1
  const int32_t *tile_visible;     // [rows / 128] the widest visible count among a tile's unflagged rows
  float *bars;                     // [R] the row's threshold: a bucket is listed when its score plus its slack reaches it
  int32_t *counts;                 // [R, lists] survivors found (past `cap`: the list overflowed)
  int2 *survivors;                 // [R, lists, cap] (bits of the bf16-operand score, bucket); lists = 2 * spans
  int32_t *status;
  int64_t R, m;
  int spans, cap, keep, sample_stride;
  int factor;  // survivors aimed at, in units of top_p
  int room;    // survivors of a row the pick has room for
};

int launch_scan_survivors(const ScanParams &p, int64_t padded_rows, cudaStream_t stream);

}  // namespace lsa
