// What the passes of the bucket-major attention share: the sizes and the parameter block.
#pragma once

#include "common.cuh"

namespace lsa {

constexpr int kBktKeys = 64;     // members a bucket may hold here (the tile of keys a CTA stages)
constexpr int kBktSegment = 128;  // (row, pick) pairs a CTA of the warp-level pass runs through its bucket
constexpr int kBktSegmentTc = 256;  // and of the tcgen05 pass: twice the tiles for one staging of the bucket
constexpr int kBktTile = 16;     // query rows a warp multiplies at once

struct BucketParams {
  const uint16_t *q, *k, *v;
  const int32_t *picked, *members, *row_top_p, *row_top_k;
  const int64_t *positions;
  const float *init_out, *init_lse;
  uint16_t *out_bf16;
  float *lse_out;
  int32_t *status;          // raised when a bounded on-chip wait of the tensor-memory pass gives up, or NULL
  // workspace
  int32_t *starts;         // [R, top_p] selected ids of the row before this pick, -1 = the pick adds nothing
  int32_t *counts;         // [m + 1] pairs of each bucket
  int32_t *offsets;        // [m + 1] exclusive scan of counts
  int32_t *seg_offsets;    // [m + 1] exclusive scan of ceil(counts / segment)
  int32_t *cursors;        // [m]
  int32_t *order;          // [R * top_p] pair ids grouped by bucket
  int32_t *takes;          // [R * top_p] keys of its bucket a pair reads (0 = none), by pair
  int32_t *order_takes;    // [R * top_p] the same beside `order`, so a CTA fetches both with one round of loads
  int4 *segments;          // [segment bound] bucket, first pair in `order`, pairs: what a CTA of the attend pass runs
  uint16_t *part_out;      // [R * top_p, Hq, dh] bf16
  float *part_lse;         // [R * top_p, Hq]
  int64_t R, m, slots, q_row_stride, q_head_stride, kv_row_stride, kv_head_stride;
  int top_p, cap, top_k, sink, window, Hq, Hkv, group;
  int segment;             // pairs a segment, at most: kBktSegment or kBktSegmentTc
  float scale_log2;
};

// The attend pass on the fifth-generation tensor cores (bucket_attend_tc.cu); `variant` picks a descriptor form
// while the kernel is being validated.
int launch_bucket_attend_tc(const BucketParams &p, int64_t segment_bound, cudaStream_t stream);

}  // namespace lsa
