// Index build: pooling, capped Ward bucketing of a cluster block, and the bucket table.
//
// All three reproduce the fp32 evaluation order of the CPU specification (a dot is added in ascending dim
// order with fused multiply-add, everything else is evaluated as written without contraction), so labels,
// member tables and centroids are bit-identical to a CPU replay in that order.
#include "common.cuh"

namespace lsa {

// ------------------------------------------------------------------------------------------------ pooling

template <typename T>
__global__ void pool_keys_kernel(const T *__restrict__ keys, int64_t n_pools, int pool_size, int d,
                                 float *__restrict__ pools) {
  int64_t total = n_pools * d;
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total;
       e += (int64_t)gridDim.x * blockDim.x) {
    int64_t p = e / d;
    int c = (int)(e - p * d);
    float acc = 0.0f;
    for (int j = 0; j < pool_size; ++j) acc = __fadd_rn(acc, load_as_float<T>(keys, (p * pool_size + j) * d + c));
    pools[e] = acc;
  }
}

// ------------------------------------------------------------------------------------------------ Ward

constexpr int kWardThreads = 256;

// Dot of the caller's row (registers when D > 0, shared memory otherwise) with a shared-memory row.
template <int D>
__device__ __forceinline__ float ward_dot(const float *mine, const float *other, int d) {
  float acc = 0.0f;
  if (D > 0) {
#pragma unroll
    for (int k = 0; k < D; k += 4) {
      float4 o = *reinterpret_cast<const float4 *>(other + k);
      acc = fmaf(mine[k], o.x, acc);
      acc = fmaf(mine[k + 1], o.y, acc);
      acc = fmaf(mine[k + 2], o.z, acc);
      acc = fmaf(mine[k + 3], o.w, acc);
    }
  } else {
    for (int k = 0; k < d; ++k) acc = fmaf(mine[k], other[k], acc);
  }
  return acc;
}

// One CTA merges one cluster block. Shared memory: the key sums [P][stride] and a few per-row vectors.
// Rows are stored at a stride of d + 4 floats, which keeps float4 alignment and spreads rows over banks.
template <int D>
__global__ void __launch_bounds__(kWardThreads)
    ward_kernel(const float *__restrict__ pool_keys, const float *__restrict__ pool_sizes, float uniform_size, int P,
                int d, int bucket_count, float bucket_cap, int max_rounds, int64_t *__restrict__ labels,
                uint8_t *__restrict__ reached, int32_t *__restrict__ rounds_out) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int stride = d + 4;
  float *ks = reinterpret_cast<float *>(smem_raw);          // [P][stride]
  float *sz = ks + (size_t)P * stride;                       // [P]
  float *sq = sz + P;                                        // [P]
  float *al = sq + P;                                        // [P]
  float *best_cost = al + P;                                 // [P]
  float *cand_cost = best_cost + P;                          // [kWardThreads]
  int *best = reinterpret_cast<int *>(cand_cost + kWardThreads);  // [P]
  int *cand_j = best + P;                                    // [kWardThreads]
  int *parent = cand_j + kWardThreads;                       // [P]
  int *state = parent + P;                                   // [P] 0 dead, 1 alive; bit 1 = mutual, bit 2 = kept
  __shared__ int n_alive_s, merged_s;

  const int tid = threadIdx.x;
  const int64_t block = blockIdx.x;
  const float *src = pool_keys + block * (int64_t)P * d;
  for (int e = tid; e < P * d; e += kWardThreads) ks[(e / d) * stride + (e % d)] = src[e];
  for (int i = tid; i < P; i += kWardThreads) {
    sz[i] = pool_sizes ? pool_sizes[block * P + i] : uniform_size;
    parent[i] = i;
    state[i] = 1;
  }
  if (tid == 0) n_alive_s = P;
  __syncthreads();

  // Threads a row when the block has fewer rows than the CTA has threads: each takes every tpr-th partner.
  const int tpr = P >= kWardThreads ? 1 : kWardThreads / P;
  int rounds = 0;
  for (int round = 0; round < max_rounds; ++round) {
    const int merges_left = n_alive_s - bucket_count;
    if (merges_left <= 0) break;
    for (int i = tid; i < P; i += kWardThreads) {
      const float *row = ks + (size_t)i * stride;
      float s = 0.0f;
      for (int k = 0; k < d; ++k) s = fmaf(row[k], row[k], s);
      sq[i] = s;
      al[i] = sqrtf(s > 0.0f ? s : 0.0f);
    }
    if (tid == 0) merged_s = 0;
    __syncthreads();

    // Cheapest allowed partner of every row, the first minimum in ascending partner order.
    for (int base = 0; base < P * tpr; base += kWardThreads) {
      const int slot = base + tid;
      const int i = slot / tpr, sub = slot - i * tpr;
      float bc = INFINITY;
      int bj = 0;
      if (i < P && (state[i] & 1)) {
        float mine[D > 0 ? D : 1];
        const float *row = ks + (size_t)i * stride;
        if (D > 0) {
#pragma unroll
          for (int k = 0; k < D; ++k) mine[k] = row[k];
        }
        const float szi = sz[i], sqi = sq[i], ali = al[i];
        for (int j = sub; j < P; j += tpr) {
          if (j == i || !(state[j] & 1) || __fadd_rn(szi, sz[j]) > bucket_cap) continue;
          const float g = ward_dot<D>(D > 0 ? mine : row, ks + (size_t)j * stride, d);
          const float m2 = __fadd_rn(__fadd_rn(sqi, sq[j]), __fmul_rn(2.0f, g));
          const float merged = sqrtf(m2 > 0.0f ? m2 : 0.0f);
          const float cost = __fsub_rn(__fadd_rn(ali, al[j]), merged);
          if (cost < bc) {
            bc = cost;
            bj = j;
          }
        }
      }
      if (tpr == 1) {
        if (i < P) {
          best_cost[i] = bc;
          best[i] = bj;
        }
      } else {
        cand_cost[tid] = bc;
        cand_j[tid] = bj;
        __syncthreads();
        if (i < P && sub == 0) {
          for (int s = 1; s < tpr; ++s) {
            const float c = cand_cost[tid + s];
            const int j = cand_j[tid + s];
            if (c < bc || (c == bc && c < INFINITY && j < bj)) {
              bc = c;
              bj = j;
            }
          }
          best_cost[i] = bc;
          best[i] = bj;
        }
        __syncthreads();
      }
    }
    __syncthreads();

    // Mutual cheapest pairs, held by their lower row.
    for (int i = tid; i < P; i += kWardThreads) {
      const bool mutual = best_cost[i] < INFINITY && best[best[i]] == i && i < best[i];
      state[i] = (state[i] & 1) | (mutual ? 2 : 0);
    }
    __syncthreads();
    // The cheapest merges_left of them merge, a tie to the lower row.
    for (int i = tid; i < P; i += kWardThreads) {
      if (!(state[i] & 2)) continue;
      const float ci = best_cost[i];
      int rank = 0;
      for (int j = 0; j < P; ++j)
        if ((state[j] & 2) && (best_cost[j] < ci || (best_cost[j] == ci && j < i))) ++rank;
      if (rank < merges_left) {
        state[i] |= 4;
        atomicAdd(&merged_s, 1);
      }
    }
    __syncthreads();
    if (merged_s == 0) break;
    for (int e = tid; e < P * d; e += kWardThreads) {
      const int i = e / d, c = e - i * d;
      if (state[i] & 4) ks[(size_t)i * stride + c] = __fadd_rn(ks[(size_t)i * stride + c], ks[(size_t)best[i] * stride + c]);
    }
    __syncthreads();
    for (int i = tid; i < P; i += kWardThreads) {
      if (!(state[i] & 4)) continue;
      const int a = best[i];
      sz[i] = __fadd_rn(sz[i], sz[a]);
      state[a] = 0;
      parent[a] = i;
    }
    if (tid == 0) n_alive_s -= merged_s;
    ++rounds;
    __syncthreads();
    for (int i = tid; i < P; i += kWardThreads) state[i] &= 1;
    __syncthreads();
  }

  // Survivors numbered by their first pool; a merge keeps the lower pool, so a root is its bucket's first pool.
  for (int i = tid; i < P; i += kWardThreads) {
    int r = i;
    while (parent[r] != r) r = parent[r];
    int number = -1;
    for (int j = 0; j <= r; ++j) number += state[j] & 1;
    labels[block * P + i] = number;
  }
  if (tid == 0) {
    reached[block] = n_alive_s <= bucket_count;
    if (rounds_out) rounds_out[block] = rounds;
  }
}

static size_t ward_smem_bytes(int P, int d) {
  return sizeof(float) * ((size_t)P * (d + 4) + 4 * (size_t)P + kWardThreads) +
         sizeof(int) * (3 * (size_t)P + kWardThreads);
}

// ------------------------------------------------------------------------------------------------ bucket table

// One CTA per cluster block. Phase 1: a warp per bucket walks the pools in order, 32 at a time, and lists their
// positions. Phase 2: a thread per (bucket, dim) adds the bucket's keys one by one in position order, eight loads in
// flight at a time (the order of the additions is what the results are pinned to; the loads may run ahead of it).
template <typename T>
__global__ void bucket_table_kernel(const T *__restrict__ index_keys, const int64_t *__restrict__ labels, int P,
                                    int pool_size, int d, int bucket_count, int bucket_cap, int64_t first_position,
                                    int32_t *__restrict__ members, int32_t *__restrict__ sizes,
                                    float *__restrict__ key_sums, float *__restrict__ centroids,
                                    uint16_t *__restrict__ centroids_bf16, int32_t *__restrict__ status) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float *sums = reinterpret_cast<float *>(smem_raw);  // [bucket_count][d]
  const int64_t block = blockIdx.x;
  const int64_t block_keys = (int64_t)P * pool_size;
  const int64_t row0 = block * bucket_count;
  const int64_t *lab = labels + block * P;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  for (int b = warp; b < bucket_count; b += warps) {
    int32_t *row = members + (row0 + b) * bucket_cap;
    int pools = 0;  // pools of the bucket so far
    for (int p0 = 0; p0 < P; p0 += 32) {
      const int p = p0 + lane;
      const bool mine = p < P && lab[p] == b;
      const unsigned votes = __ballot_sync(0xffffffffu, mine);
      if (mine) {
        const int at = (pools + __popc(votes & ((1u << lane) - 1))) * pool_size;
        for (int j = 0; j < pool_size; ++j)
          if (at + j < bucket_cap) row[at + j] = (int32_t)(first_position + block * block_keys + (int64_t)p * pool_size + j);
      }
      pools += __popc(votes);
    }
    const int64_t listed = (int64_t)pools * pool_size;
    const int n = (int)(listed < bucket_cap ? listed : bucket_cap);
    for (int j = n + lane; j < bucket_cap; j += 32) row[j] = LSA_PAD;
    if (lane == 0) {
      sizes[row0 + b] = n;
      if (listed > bucket_cap && status) atomicAdd(status, 1);
    }
  }
  __syncthreads();
  if (!key_sums && !centroids && !centroids_bf16) return;
  for (int e = threadIdx.x; e < bucket_count * d; e += blockDim.x) {
    const int b = e / d, c = e - b * d;
    const int32_t *row = members + (row0 + b) * bucket_cap;
    const int n = sizes[row0 + b];
    float acc = 0.0f;
    for (int j0 = 0; j0 < n; j0 += 8) {
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        v[j] = j0 + j < n ? load_as_float<T>(index_keys, (int64_t)(row[j0 + j] - first_position) * d + c) : 0.0f;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (j0 + j < n) acc = __fadd_rn(acc, v[j]);
    }
    sums[e] = acc;
    if (key_sums) key_sums[(row0 + b) * d + c] = acc;
  }
  __syncthreads();
  if (!centroids && !centroids_bf16) return;
  float *norms = sums + (size_t)bucket_count * d;  // [bucket_count]
  for (int b = threadIdx.x; b < bucket_count; b += blockDim.x) {
    float ss = 0.0f;
    for (int c = 0; c < d; ++c) ss = fmaf(sums[b * d + c], sums[b * d + c], ss);
    const float nrm = sqrtf(ss);
    norms[b] = nrm > 1e-30f ? nrm : 1e-30f;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < bucket_count * d; e += blockDim.x) {
    const int b = e / d;
    const float value = __fdiv_rn(sums[e], norms[b]);
    if (centroids) centroids[row0 * d + e] = value;
    if (centroids_bf16) centroids_bf16[row0 * d + e] = float_to_bf16_bits(value);
  }
}

}  // namespace lsa

// ================================================================================================ C ABI

LSA_API int lsa_pool_keys(const void *index_keys, int key_dtype, int64_t n_pools, int pool_size, int d,
                          float *pools, void *stream) {
  LSA_REQUIRE(index_keys && pools, LSA_ERR_NULL);
  LSA_REQUIRE(n_pools >= 0 && pool_size >= 1 && d >= 1, LSA_ERR_ARGUMENT);
  LSA_REQUIRE(key_dtype == LSA_DTYPE_F32 || key_dtype == LSA_DTYPE_BF16, LSA_ERR_ARGUMENT);
  if (n_pools == 0) return LSA_OK;
  const int threads = 256;
  int64_t want = (n_pools * d + threads - 1) / threads;
  int grid = (int)(want < (int64_t)lsa::sm_count() * 16 ? want : (int64_t)lsa::sm_count() * 16);
  cudaStream_t s = (cudaStream_t)stream;
  if (key_dtype == LSA_DTYPE_F32)
    lsa::pool_keys_kernel<float><<<grid, threads, 0, s>>>((const float *)index_keys, n_pools, pool_size, d, pools);
  else
    lsa::pool_keys_kernel<uint16_t><<<grid, threads, 0, s>>>((const uint16_t *)index_keys, n_pools, pool_size, d, pools);
  LSA_LAUNCH_CHECK();
  return LSA_OK;
}

namespace lsa {
size_t ward_large_workspace_bytes(int64_t G, int P, int d);
int ward_large_run(const float *pool_keys, const float *pool_sizes, float uniform_size, int64_t G, int P, int d,
                   int bucket_count, float bucket_cap, int max_rounds, int64_t *labels, uint8_t *reached,
                   int32_t *rounds, void *workspace, cudaStream_t s);
// Blocks up to this many pools (at 64 dims) are merged by one CTA out of shared memory.
constexpr int kWardOneCtaPools = 512;
}  // namespace lsa

LSA_API size_t lsa_ward_merge_workspace_bytes(int64_t blocks, int P, int d) {
  if (blocks <= 0 || P <= 0 || d <= 0) return 0;
  if (P <= lsa::kWardOneCtaPools && lsa::ward_smem_bytes(P, d) <= 227 * 1024) return 0;
  return lsa::ward_large_workspace_bytes(blocks, P, d);
}

LSA_API int lsa_ward_merge(const float *pool_keys, const float *pool_sizes, float uniform_pool_size, int64_t blocks,
                           int P, int d, int bucket_count, float bucket_cap, int max_rounds, int64_t *labels,
                           uint8_t *reached, int32_t *rounds, void *workspace, size_t workspace_bytes,
                           void *stream) {
  LSA_REQUIRE(pool_keys && labels && reached, LSA_ERR_NULL);
  LSA_REQUIRE(blocks >= 0 && P >= 1 && d >= 4 && d % 4 == 0 && bucket_count >= 1 && max_rounds >= 0,
              LSA_ERR_ARGUMENT);
  LSA_REQUIRE(P <= 4096 && d <= 1024, LSA_ERR_UNSUPPORTED);
  if (blocks == 0) return LSA_OK;
  const size_t need = lsa_ward_merge_workspace_bytes(blocks, P, d);
  if (need > 0) {
    LSA_REQUIRE(d == 16 || d == 32 || d == 64, LSA_ERR_UNSUPPORTED);
    LSA_REQUIRE(workspace, LSA_ERR_NULL);
    LSA_REQUIRE(workspace_bytes >= need, LSA_ERR_WORKSPACE);
    return lsa::ward_large_run(pool_keys, pool_sizes, uniform_pool_size, blocks, P, d, bucket_count, bucket_cap,
                               max_rounds, labels, reached, rounds, workspace, (cudaStream_t)stream);
  }
  const size_t smem = lsa::ward_smem_bytes(P, d);
  cudaStream_t s = (cudaStream_t)stream;
#define LSA_WARD_LAUNCH(DD)                                                                                       \
  do {                                                                                                            \
    if (cudaFuncSetAttribute(lsa::ward_kernel<DD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=     \
        cudaSuccess)                                                                                              \
      return LSA_ERR_LAUNCH;                                                                                      \
    lsa::ward_kernel<DD><<<(unsigned)blocks, lsa::kWardThreads, smem, s>>>(                                       \
        pool_keys, pool_sizes, uniform_pool_size, P, d, bucket_count, bucket_cap, max_rounds, labels, reached,    \
        rounds);                                                                                                  \
  } while (0)
  if (d == 64)
    LSA_WARD_LAUNCH(64);
  else if (d == 32)
    LSA_WARD_LAUNCH(32);
  else if (d == 16)
    LSA_WARD_LAUNCH(16);
  else
    LSA_WARD_LAUNCH(0);
#undef LSA_WARD_LAUNCH
  LSA_LAUNCH_CHECK();
  return LSA_OK;
}

LSA_API int lsa_bucket_table(const void *index_keys, int key_dtype, const int64_t *labels, int64_t blocks, int P,
                             int pool_size, int d, int bucket_count, int bucket_cap, int64_t first_position,
                             int32_t *members, int32_t *sizes, float *key_sums, float *centroids,
                             uint16_t *centroids_bf16, int32_t *status, void *stream) {
  LSA_REQUIRE(labels && members && sizes, LSA_ERR_NULL);
  LSA_REQUIRE(blocks >= 0 && P >= 1 && pool_size >= 1 && d >= 1 && bucket_count >= 1 && bucket_cap >= 1,
              LSA_ERR_ARGUMENT);
  LSA_REQUIRE(key_dtype == LSA_DTYPE_F32 || key_dtype == LSA_DTYPE_BF16, LSA_ERR_ARGUMENT);
  const bool sums = key_sums || centroids || centroids_bf16;
  LSA_REQUIRE(!sums || index_keys, LSA_ERR_NULL);
  if (blocks == 0) return LSA_OK;
  const size_t smem = sums ? sizeof(float) * ((size_t)bucket_count * d + bucket_count) : 0;
  LSA_REQUIRE(smem <= 227 * 1024, LSA_ERR_UNSUPPORTED);
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = 256;
  if (key_dtype == LSA_DTYPE_F32) {
    if (cudaFuncSetAttribute(lsa::bucket_table_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess)
      return LSA_ERR_LAUNCH;
    lsa::bucket_table_kernel<float><<<(unsigned)blocks, threads, smem, s>>>(
        (const float *)index_keys, labels, P, pool_size, d, bucket_count, bucket_cap, first_position, members, sizes,
        key_sums, centroids, centroids_bf16, status);
  } else {
    if (cudaFuncSetAttribute(lsa::bucket_table_kernel<uint16_t>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess)
      return LSA_ERR_LAUNCH;
    lsa::bucket_table_kernel<uint16_t><<<(unsigned)blocks, threads, smem, s>>>(
        (const uint16_t *)index_keys, labels, P, pool_size, d, bucket_count, bucket_cap, first_position, members,
        sizes, key_sums, centroids, centroids_bf16, status);
  }
  LSA_LAUNCH_CHECK();
  return LSA_OK;
}

// ================================================================================================ gathered sums

namespace lsa {

// out[r, :] = sum over c of src[index[r, c] - index_base, :], added one by one in column order; an index < 0 ends
// the row. A thread a (row, dim): reads of a source row are coalesced across the dims.
template <typename TS, typename TI>
__global__ void gather_sum_kernel(const TS *__restrict__ src, const TI *__restrict__ index, int64_t rows, int width,
                                  int d, int64_t index_base, float *__restrict__ out) {
  const int64_t total = rows * d;
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = e / d;
    const int c = (int)(e - r * d);
    float acc = 0.0f;
    for (int j = 0; j < width; ++j) {
      const int64_t id = (int64_t)index[r * width + j];
      if (id < 0) break;
      acc = __fadd_rn(acc, load_as_float<TS>(src, (id - index_base) * d + c));
    }
    out[e] = acc;
  }
}

}  // namespace lsa

LSA_API int lsa_gather_sum(const void *src, int src_dtype, const void *index, int index_is_int64, int64_t rows,
                           int width, int d, int64_t index_base, float *out, void *stream) {
  LSA_REQUIRE(src && index && out, LSA_ERR_NULL);
  LSA_REQUIRE(rows >= 0 && width >= 1 && d >= 1, LSA_ERR_ARGUMENT);
  LSA_REQUIRE(src_dtype == LSA_DTYPE_F32 || src_dtype == LSA_DTYPE_BF16, LSA_ERR_ARGUMENT);
  if (rows == 0) return LSA_OK;
  const int threads = 256;
  const int64_t want = (rows * d + threads - 1) / threads;
  const int grid = (int)(want < (int64_t)lsa::sm_count() * 16 ? want : (int64_t)lsa::sm_count() * 16);
  cudaStream_t s = (cudaStream_t)stream;
  if (src_dtype == LSA_DTYPE_F32) {
    if (index_is_int64)
      lsa::gather_sum_kernel<float, int64_t><<<grid, threads, 0, s>>>((const float *)src, (const int64_t *)index, rows,
                                                                      width, d, index_base, out);
    else
      lsa::gather_sum_kernel<float, int32_t><<<grid, threads, 0, s>>>((const float *)src, (const int32_t *)index, rows,
                                                                      width, d, index_base, out);
  } else {
    if (index_is_int64)
      lsa::gather_sum_kernel<uint16_t, int64_t><<<grid, threads, 0, s>>>((const uint16_t *)src, (const int64_t *)index,
                                                                         rows, width, d, index_base, out);
    else
      lsa::gather_sum_kernel<uint16_t, int32_t><<<grid, threads, 0, s>>>((const uint16_t *)src, (const int32_t *)index,
                                                                         rows, width, d, index_base, out);
  }
  LSA_LAUNCH_CHECK();
  return LSA_OK;
}

// ================================================================================================ k-means update

namespace lsa {

// Update step of the k-means bucketing: cluster j's new centroid is the normalised sum of the pools
// assigned to it, added one by one in pool order (`order` lists the pools cluster by cluster, ascending within a
// cluster; `offsets[j] .. offsets[j + 1]` is cluster j's run). An empty cluster, or one whose sum is zero, keeps its
// centroid. One CTA a cluster; the norm is a single thread's fma chain so that it equals a CPU replay.
__global__ void kmeans_update_kernel(const float *__restrict__ pools, const int64_t *__restrict__ order,
                                     const int64_t *__restrict__ offsets, int d, float *__restrict__ centroids) {
  extern __shared__ float sum[];  // [d]
  __shared__ float norm_s;
  const int64_t j = blockIdx.x;
  const int64_t first = offsets[j], end = offsets[j + 1];
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float acc = 0.0f;
    for (int64_t i = first; i < end; ++i) acc = __fadd_rn(acc, pools[order[i] * d + c]);
    sum[c] = acc;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float ss = 0.0f;
    for (int c = 0; c < d; ++c) ss = fmaf(sum[c], sum[c], ss);
    norm_s = ss > 0.0f ? sqrtf(ss) : 0.0f;
  }
  __syncthreads();
  if (norm_s > 0.0f)
    for (int c = threadIdx.x; c < d; c += blockDim.x) centroids[j * d + c] = __fdiv_rn(sum[c], norm_s);
}

}  // namespace lsa

LSA_API int lsa_kmeans_update(const float *pools, const int64_t *order, const int64_t *offsets, int k, int d,
                              float *centroids, void *stream) {
  LSA_REQUIRE(pools && order && offsets && centroids, LSA_ERR_NULL);
  LSA_REQUIRE(k >= 1 && d >= 1 && d <= 4096, LSA_ERR_ARGUMENT);
  lsa::kmeans_update_kernel<<<(unsigned)k, 64, (size_t)d * sizeof(float), (cudaStream_t)stream>>>(pools, order,
                                                                                                 offsets, d, centroids);
  LSA_LAUNCH_CHECK();
  return LSA_OK;
}
