// Bucket shapes: a bucket's spread about its centroid, kept as `rank` sign directions (one bit a dimension), their
// variances and a floor; a shaped bucket scores as its estimated best key, q.c + z sqrt(q^T Sigma q)
// (src/lsa/core/shape.py:1-18,108-137; the packed layout: shape.py:140-155).
//
// The arithmetic is fixed so that every kernel that scores a shaped bucket, and the CPU oracle, agree bit for bit:
// q.s_j summed over ascending dimensions with the sign as a factor of a fused multiply-add, scaled once by
// 1/sqrt(d); the directions folded in order; no contraction across those steps.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace lsa {

struct ShapeTable {
  const uint32_t *basis;   // [rows, rank, d / 32] words: bit b of word w = dimension 32 w + b, set = positive
  const float *variances;  // [rows, rank]
  const float *floors;     // [rows]; NULL = the buckets are not shaped
  int rank;
  float deviations;  // z
  float scale;       // 1 / sqrt(d), rounded once on the host
};

__device__ __forceinline__ float shape_sign(uint32_t word, int bit) { return ((word >> bit) & 1u) ? 1.0f : -1.0f; }

// Folds one direction's projection into the running variance and the running sum of squared projections.
__device__ __forceinline__ void shape_fold(float along_unscaled, float scale, float variance_j, float &variance,
                                           float &inside) {
  const float along = __fmul_rn(along_unscaled, scale);
  const float squared = __fmul_rn(along, along);
  variance = __fmaf_rn(variance_j, squared, variance);
  inside = __fadd_rn(inside, squared);
}

__device__ __forceinline__ float shape_finish(float centre_score, float variance, float inside, float floor_,
                                              float deviations) {
  variance = __fmaf_rn(floor_, __fsub_rn(1.0f, inside), variance);
  return __fmaf_rn(deviations, __fsqrt_rn(fmaxf(variance, 0.0f)), centre_score);
}

// The shaped score of table row `row` under query q [d] (any memory space), given the centroid's score.
__device__ __forceinline__ float shaped_score(float centre_score, const float *q, int d, const ShapeTable &t,
                                              int64_t row) {
  const int words = d >> 5;
  float variance = 0.0f, inside = 0.0f;
  for (int j = 0; j < t.rank; ++j) {
    const uint32_t *bits = t.basis + (row * t.rank + j) * words;
    float along = 0.0f;
    for (int w = 0; w < words; ++w) {
      const uint32_t word = __ldg(bits + w);
#pragma unroll 8
      for (int b = 0; b < 32; ++b) along = __fmaf_rn(q[w * 32 + b], shape_sign(word, b), along);
    }
    shape_fold(along, t.scale, __ldg(t.variances + row * t.rank + j), variance, inside);
  }
  return shape_finish(centre_score, variance, inside, __ldg(t.floors + row), t.deviations);
}

}  // namespace lsa
