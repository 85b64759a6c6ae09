// What the passes of the tensor-core bucket scan share: the constants of the scheme and the parameter block.
#pragma once

#include "common.cuh"

namespace lsa {

constexpr int kScanFactor = 4;               // survivors aimed at, in units of top_p
constexpr float kScanMargin = 1.0f / 128.0f;  // bf16 operands move a score of unit vectors by less than 2^-8: twice that
constexpr int kScanMinVisible = 1024;         // rows that see fewer buckets take the exact scan (it is cheap there)

struct ScanParams {
  const uint16_t *queries_bf16;    // [rows padded to 128, 64]
  const uint16_t *centroids_bf16;  // [m, 64]
  const int32_t *visible;          // [R]
  const int32_t *row_keep;         // [R] or NULL
  const int32_t *flags;            // [R]: nonzero = the row takes the exact scan
  const float *norms;              // [R] lengths of the query rows
  const int32_t *tile_visible;     // [rows / 128] the widest visible count among a tile's unflagged rows
  float *thresholds;               // [R]
  int32_t *counts;                 // [R, spans] survivors found (past `cap`: the list overflowed)
  int32_t *survivors;              // [R, spans, cap]
  int32_t *status;
  int64_t R, m;
  int spans, cap, keep, sample_stride;
};

int launch_scan_survivors(const ScanParams &p, int64_t padded_rows, cudaStream_t stream);

}  // namespace lsa
