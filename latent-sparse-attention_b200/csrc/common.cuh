// Shared device helpers of the lsa_b200 kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

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

// ---- chained launches of a decode step
// A decode step is a chain of small kernels, each waiting for the one before. Launched as programmatic dependents
// (the attribute below), a kernel's CTAs are placed on the SMs while the kernel before it is still running, do what
// does not depend on it, and wait at `wait_for_earlier_grids()`; the gap between two launches goes. Every kernel that
// may be launched this way calls the wait on every path before it touches memory an earlier kernel wrote (the wait
// ends when the earlier grids have completed and their writes are visible; in a kernel launched the plain way both
// calls do nothing).
__device__ __forceinline__ void dependents_may_launch() { asm volatile("griddepcontrol.launch_dependents;"); }
__device__ __forceinline__ void wait_for_earlier_grids() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

constexpr int64_t kChainedRows = 8;  // calls of at most this many rows are a decode step's: their launches are chained

// Off unless LSA_CHAINED_LAUNCH=1 (read once): a step replayed from a CUDA graph, whose launches are already a
// microsecond apart, measured slower with its whole chain resident and waiting (153 against 130 us for the MLA flat
// step, 84 against 78 for the tree step); only a step launched eagerly from the host gained (196 against 203 us).
inline bool chained_launches() {
  static const bool on = [] {
    const char *set = getenv("LSA_CHAINED_LAUNCH");
    return set && set[0] == '1';
  }();
  return on;
}

// kernel<<<grid, block, smem, stream>>>(args...), as a programmatic dependent of the stream's last kernel when
// `chained`. The error, if any, is left for LSA_LAUNCH_CHECK.
template <typename... Params, typename... Args>
inline void launch(bool chained, void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                   Args &&...args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid, config.blockDim = block, config.dynamicSmemBytes = smem, config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = chained && chained_launches() ? 1 : 0;
  (void)cudaLaunchKernelEx(&config, kernel, Params(args)...);
}

inline int sm_count() {
  int dev = 0, n = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  return n;
}

}  // namespace lsa
