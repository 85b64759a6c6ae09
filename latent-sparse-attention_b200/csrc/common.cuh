// Shared device helpers of the lsa_b200 kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "lsa_b200.h"

#define LSA_API extern "C" __attribute__((visibility("default")))

#define LSA_REQUIRE(cond, code) \
  do {                          \
    if (!(cond)) return (code); \
  } while (0)

#define LSA_LAUNCH_CHECK()                          \
  do {                                              \
    if (cudaPeekAtLastError() != cudaSuccess) {     \
      (void)cudaGetLastError();                     \
      return LSA_ERR_LAUNCH;                        \
    }                                               \
  } while (0)

namespace lsa {

constexpr int kWarp = 32;
constexpr int64_t kEmptyKey = INT64_MIN;

__device__ __forceinline__ int lane_id() { return threadIdx.x & 31; }

// An fp32 score as an int32 of the same order; negatives flip their magnitude bits.
__device__ __forceinline__ int32_t ordered_bits(float score) {
  int32_t bits = __float_as_int(score);
  return bits < 0 ? (bits ^ 0x7FFFFFFF) : bits;
}

// Score in the high word, 2^31-1-id in the low: the greater key is the greater score, then the lower id.
__device__ __forceinline__ int64_t pack_key(float score, int32_t id) {
  return (int64_t)(((uint64_t)(uint32_t)ordered_bits(score)) << 32) | (int64_t)(uint32_t)(0x7FFFFFFF - id);
}

__device__ __forceinline__ int32_t key_id(int64_t key) { return 0x7FFFFFFF - (int32_t)(key & 0xFFFFFFFFll); }

// A packed key as an unsigned number of the same order, for radix passes.
__device__ __forceinline__ uint64_t key_radix(int64_t key) { return (uint64_t)key ^ 0x8000000000000000ull; }

__device__ __forceinline__ float bf16_bits_to_float(uint16_t bits) { return __uint_as_float((uint32_t)bits << 16); }

__device__ __forceinline__ uint16_t float_to_bf16_bits(float x) {
  __nv_bfloat16 h = __float2bfloat16_rn(x);
  return *reinterpret_cast<uint16_t *>(&h);
}

template <typename T>
__device__ __forceinline__ float load_as_float(const T *p, int64_t i);
template <>
__device__ __forceinline__ float load_as_float<float>(const float *p, int64_t i) {
  return p[i];
}
template <>
__device__ __forceinline__ float load_as_float<uint16_t>(const uint16_t *p, int64_t i) {
  return bf16_bits_to_float(p[i]);
}

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

__device__ __forceinline__ int warp_sum_int(int x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

inline int sm_count() {
  int dev = 0, n = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  return n;
}

}  // namespace lsa
