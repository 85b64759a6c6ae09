// What the two forms of the latent (MLA) gather attention share: the parameter block and the tensor-core launcher.
#pragma once

#include "common.cuh"

namespace lsa {

constexpr int kLatHeads = 64;  // query heads a CTA takes (a block of the heads that share the latent rows)

struct LatentParams {
  const uint16_t *q, *latent;
  const int32_t *ids, *lengths;
  uint16_t *out_bf16;
  float *out_f32, *lse, *part_out, *part_lse;
  int32_t *status;  // raised when a bounded on-chip wait of the tensor-memory form gives up, or NULL
  int64_t R, slots, q_row_stride, q_head_stride, latent_row_stride, list_stride;
  int Hq, splits;
  int deal_granule, deal_world, deal_rank;  // ids are positions of a cache dealt over ranks in granules (world <= 1: off)
  int boxes;        // set by the tensor-core launcher: runs of consecutive rows may be staged by tensor-map copies
  float scale_log2;
};

// The tcgen05 form (latent_attend_tc.cu): dk = 576, dv = 512.
int launch_latent_attend_tc(const LatentParams &p, cudaStream_t stream);

}  // namespace lsa
