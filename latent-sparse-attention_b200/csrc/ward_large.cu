// Capped Ward for blocks too large for one CTA's shared memory (up to 4,096 pools): the node-bucket pairings of
// the tree and any big cluster block.
//
// State lives in a caller-provided workspace in global memory (it stays in L2: 1 MB of key sums a block at 4,096 x
// 64). A round is two launches and the host never looks at the device: `ward_nearest` finds every open row's
// cheapest allowed partner with a register-tiled all-pairs pass over the COMPACTED list of open rows (so later
// rounds cost what is left, not P^2), `ward_fix` takes the mutual pairs, merges them, recomputes norms and rebuilds
// the list. Blocks that have reached their count or can merge no further return at once, so launching every
// round up to the cap is cheap. Arithmetic order is the CPU specification's: a dot is an fma chain in ascending
// dim order, costs are evaluated as written, a tie goes to the lower row.
#include "common.cuh"

namespace lsa {

constexpr int kTile = 64;           // rows and partners a CTA of ward_nearest takes at a time
constexpr int kNearestThreads = 256;
constexpr int kFixThreads = 1024;

struct WardState {
  float *ks;        // [G, P, d] key sums
  float *sz;        // [G, P]
  float *sq;        // [G, P] squared norms, fixed-order
  float *al;        // [G, P] norms
  float *best_cost; // [G, P]
  int *best;        // [G, P]
  int *parent;      // [G, P]
  int *alive;       // [G, P]
  int *open;        // [G, P] ascending indices of alive rows
  int *n_alive;     // [G]
  int *done;        // [G] 1 = reached the count or cannot merge further
  int P, d, bucket_count;
  float bucket_cap;
};

__global__ void ward_large_init(WardState w, const float *__restrict__ pool_keys, const float *__restrict__ pool_sizes,
                                float uniform_size) {
  const int64_t g = blockIdx.x;
  const int P = w.P, d = w.d;
  for (int i = threadIdx.x; i < P; i += blockDim.x) {
    const float *row = pool_keys + (g * P + i) * d;
    float *dst = w.ks + (g * P + i) * d;
    float s = 0.0f;
    for (int k = 0; k < d; ++k) {
      dst[k] = row[k];
      s = fmaf(row[k], row[k], s);
    }
    w.sq[g * P + i] = s;
    w.al[g * P + i] = sqrtf(s > 0.0f ? s : 0.0f);
    w.sz[g * P + i] = pool_sizes ? pool_sizes[g * P + i] : uniform_size;
    w.parent[g * P + i] = i;
    w.alive[g * P + i] = 1;
    w.open[g * P + i] = i;
  }
  if (threadIdx.x == 0) {
    w.n_alive[g] = P;
    w.done[g] = P <= w.bucket_count;
  }
}

// grid (ceil(P / 64), G). Each CTA: 64 open rows against every open partner, 4 x 4 dots a thread.
template <int D>
__global__ void __launch_bounds__(kNearestThreads) ward_nearest(WardState w) {
  const int64_t g = blockIdx.y;
  if (w.done[g]) return;
  const int n_open = w.n_alive[g];
  const int row0 = blockIdx.x * kTile;
  if (row0 >= n_open) return;
  const int P = w.P;
  constexpr int LD = kTile + 4;
  __shared__ __align__(16) float a_t[D][LD];  // the CTA's rows, transposed [dim][row]
  __shared__ __align__(16) float b_t[D][LD];  // a tile of partners, transposed
  __shared__ int a_id[kTile], b_id[kTile];
  __shared__ float a_sq[kTile], a_al[kTile], a_sz[kTile], b_sq[kTile], b_al[kTile], b_sz[kTile];

  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int *open = w.open + g * P;
  const float *ks = w.ks + g * P * D;
  for (int r = tid; r < kTile; r += kNearestThreads) {
    const int id = row0 + r < n_open ? open[row0 + r] : -1;
    a_id[r] = id;
    a_sq[r] = id >= 0 ? w.sq[g * P + id] : 0.0f;
    a_al[r] = id >= 0 ? w.al[g * P + id] : 0.0f;
    a_sz[r] = id >= 0 ? w.sz[g * P + id] : 0.0f;
  }
  __syncthreads();
  for (int e = tid; e < kTile * D; e += kNearestThreads) {
    const int r = e / D, k = e - r * D;
    a_t[k][r] = a_id[r] >= 0 ? ks[(int64_t)a_id[r] * D + k] : 0.0f;
  }
  float best_c[4];
  int best_j[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    best_c[i] = INFINITY;
    best_j[i] = 0x7FFFFFFF;
  }
  for (int col0 = 0; col0 < n_open; col0 += kTile) {
    __syncthreads();
    for (int r = tid; r < kTile; r += kNearestThreads) {
      const int id = col0 + r < n_open ? open[col0 + r] : -1;
      b_id[r] = id;
      b_sq[r] = id >= 0 ? w.sq[g * P + id] : 0.0f;
      b_al[r] = id >= 0 ? w.al[g * P + id] : 0.0f;
      b_sz[r] = id >= 0 ? w.sz[g * P + id] : 0.0f;
    }
    __syncthreads();
    for (int e = tid; e < kTile * D; e += kNearestThreads) {
      const int r = e / D, k = e - r * D;
      b_t[k][r] = b_id[r] >= 0 ? ks[(int64_t)b_id[r] * D + k] : 0.0f;
    }
    __syncthreads();
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
#pragma unroll 8
    for (int k = 0; k < D; ++k) {
      const float4 a = *reinterpret_cast<const float4 *>(&a_t[k][ty * 4]);
      const float4 b = *reinterpret_cast<const float4 *>(&b_t[k][tx * 4]);
      const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = ty * 4 + i;
      const int id_i = a_id[r];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c = tx * 4 + j;
        const int id_j = b_id[c];
        if (id_i < 0 || id_j < 0 || id_i == id_j || __fadd_rn(a_sz[r], b_sz[c]) > w.bucket_cap) continue;
        const float m2 = __fadd_rn(__fadd_rn(a_sq[r], b_sq[c]), __fmul_rn(2.0f, acc[i][j]));
        const float merged = sqrtf(m2 > 0.0f ? m2 : 0.0f);
        const float cost = __fsub_rn(__fadd_rn(a_al[r], b_al[c]), merged);
        if (cost < best_c[i] || (cost == best_c[i] && id_j < best_j[i])) {
          best_c[i] = cost;
          best_j[i] = id_j;
        }
      }
    }
  }
  // The 16 threads of a row group are 16 consecutive lanes: fold their minima, a tie to the lower partner.
#pragma unroll
  for (int i = 0; i < 4; ++i) {
#pragma unroll
    for (int o = 1; o < 16; o <<= 1) {
      const float c = __shfl_xor_sync(0xffffffffu, best_c[i], o);
      const int j = __shfl_xor_sync(0xffffffffu, best_j[i], o);
      if (c < best_c[i] || (c == best_c[i] && j < best_j[i])) {
        best_c[i] = c;
        best_j[i] = j;
      }
    }
    const int id_i = a_id[ty * 4 + i];
    if (tx == 0 && id_i >= 0) {
      w.best_cost[g * P + id_i] = best_c[i];
      w.best[g * P + id_i] = best_c[i] < INFINITY ? best_j[i] : 0;
    }
  }
}

// One CTA a block: mutual pairs, the cheapest merges_left of them, the merges, norms, and the new open list.
__global__ void __launch_bounds__(kFixThreads) ward_fix(WardState w, int32_t *__restrict__ rounds_out) {
  const int64_t g = blockIdx.x;
  if (w.done[g]) return;
  const int P = w.P, d = w.d, tid = threadIdx.x;
  extern __shared__ int fix_smem[];
  int *flag = fix_smem;        // [P] 0 none, 1 mutual, 2 merging
  int *scan = fix_smem + P;    // [P] scratch of the compaction
  __shared__ int n_mutual_s, n_merge_s, chunk_base_s;
  float *bc = w.best_cost + g * P;
  int *best = w.best + g * P, *alive = w.alive + g * P, *open = w.open + g * P, *parent = w.parent + g * P;
  const int n_alive = w.n_alive[g];
  const int merges_left = n_alive - w.bucket_count;
  if (tid == 0) n_mutual_s = n_merge_s = 0;
  __syncthreads();
  for (int i = tid; i < P; i += kFixThreads) {
    const bool mutual = alive[i] && bc[i] < INFINITY && best[best[i]] == i && i < best[i];
    flag[i] = mutual;
    if (mutual) atomicAdd(&n_mutual_s, 1);
  }
  __syncthreads();
  const bool cut = n_mutual_s > merges_left;
  for (int i = tid; i < P; i += kFixThreads) {
    if (!flag[i]) continue;
    bool keep = true;
    if (cut) {
      int rank = 0;
      const float ci = bc[i];
      for (int j = 0; j < P; ++j)
        if (flag[j] && (bc[j] < ci || (bc[j] == ci && j < i))) ++rank;
      keep = rank < merges_left;
    }
    if (keep) {
      scan[i] = 1;
      atomicAdd(&n_merge_s, 1);
    } else {
      scan[i] = 0;
    }
  }
  __syncthreads();
  for (int i = tid; i < P; i += kFixThreads) flag[i] = flag[i] && scan[i] ? 2 : 0;
  __syncthreads();
  if (n_merge_s == 0) {
    if (tid == 0) w.done[g] = 1;
    return;
  }
  float *ks = w.ks + g * P * d;
  for (int e = tid; e < P * d; e += kFixThreads) {
    const int i = e / d, c = e - i * d;
    if (flag[i] == 2) ks[(int64_t)i * d + c] = __fadd_rn(ks[(int64_t)i * d + c], ks[(int64_t)best[i] * d + c]);
  }
  __syncthreads();
  for (int i = tid; i < P; i += kFixThreads) {
    if (flag[i] != 2) continue;
    const int a = best[i];
    w.sz[g * P + i] = __fadd_rn(w.sz[g * P + i], w.sz[g * P + a]);
    alive[a] = 0;
    parent[a] = i;
    const float *row = ks + (int64_t)i * d;
    float s = 0.0f;
    for (int k = 0; k < d; ++k) s = fmaf(row[k], row[k], s);
    w.sq[g * P + i] = s;
    w.al[g * P + i] = sqrtf(s > 0.0f ? s : 0.0f);
  }
  __syncthreads();
  // Ordered compaction of the alive rows, 1,024 at a time.
  if (tid == 0) chunk_base_s = 0;
  __syncthreads();
  for (int base = 0; base < P; base += kFixThreads) {
    const int i = base + tid;
    const int a = i < P ? alive[i] : 0;
    // inclusive scan within the CTA: warp scans, then the warp totals
    int v = a;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, v, o);
      if ((tid & 31) >= o) v += n;
    }
    if ((tid & 31) == 31) scan[tid >> 5] = v;
    __syncthreads();
    if (tid < 32) {
      int t = scan[tid];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, t, o);
        if (tid >= o) t += n;
      }
      scan[32 + tid] = t;
    }
    __syncthreads();
    const int before = chunk_base_s + (tid >= 32 ? scan[32 + (tid >> 5) - 1] : 0) + v - a;
    if (a) open[before] = i;
    __syncthreads();
    if (tid == kFixThreads - 1) chunk_base_s = before + a;
    __syncthreads();
  }
  if (tid == 0) {
    const int left = n_alive - n_merge_s;
    w.n_alive[g] = left;
    if (left <= w.bucket_count) w.done[g] = 1;
    if (rounds_out) rounds_out[g] += 1;
  }
}

__global__ void ward_large_labels(WardState w, int64_t *__restrict__ labels, uint8_t *__restrict__ reached) {
  const int64_t g = blockIdx.x;
  const int P = w.P;
  extern __shared__ int number[];  // [P] survivors numbered by first pool
  const int *alive = w.alive + g * P, *parent = w.parent + g * P;
  if (threadIdx.x == 0) {
    int n = -1;
    for (int i = 0; i < P; ++i) {
      n += alive[i];
      number[i] = n;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < P; i += blockDim.x) {
    int r = i;
    while (parent[r] != r) r = parent[r];
    labels[g * P + i] = number[r];
  }
  if (threadIdx.x == 0) reached[g] = w.n_alive[g] <= w.bucket_count;
}

static size_t align_up(size_t n) { return (n + 255) & ~(size_t)255; }

size_t ward_large_workspace_bytes(int64_t G, int P, int d) {
  const size_t rows = (size_t)G * P;
  return align_up(rows * d * 4) + 4 * align_up(rows * 4) + 4 * align_up(rows * 4) + 2 * align_up((size_t)G * 4);
}

int ward_large_run(const float *pool_keys, const float *pool_sizes, float uniform_size, int64_t G, int P, int d,
                   int bucket_count, float bucket_cap, int max_rounds, int64_t *labels, uint8_t *reached,
                   int32_t *rounds, void *workspace, cudaStream_t s) {
  WardState w;
  unsigned char *at = (unsigned char *)workspace;
  const size_t rows = (size_t)G * P;
  auto take = [&](size_t bytes) {
    void *p = at;
    at += align_up(bytes);
    return p;
  };
  w.ks = (float *)take(rows * d * 4);
  w.sz = (float *)take(rows * 4);
  w.sq = (float *)take(rows * 4);
  w.al = (float *)take(rows * 4);
  w.best_cost = (float *)take(rows * 4);
  w.best = (int *)take(rows * 4);
  w.parent = (int *)take(rows * 4);
  w.alive = (int *)take(rows * 4);
  w.open = (int *)take(rows * 4);
  w.n_alive = (int *)take((size_t)G * 4);
  w.done = (int *)take((size_t)G * 4);
  w.P = P;
  w.d = d;
  w.bucket_count = bucket_count;
  w.bucket_cap = bucket_cap;
  if (rounds && cudaMemsetAsync(rounds, 0, (size_t)G * 4, s) != cudaSuccess) return LSA_ERR_LAUNCH;
  ward_large_init<<<(unsigned)G, 256, 0, s>>>(w, pool_keys, pool_sizes, uniform_size);
  const size_t fix_smem = (size_t)P * 2 * sizeof(int) + 64 * sizeof(int);
  if (cudaFuncSetAttribute(ward_fix, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fix_smem) != cudaSuccess)
    return LSA_ERR_LAUNCH;
  dim3 grid((unsigned)((P + kTile - 1) / kTile), (unsigned)G);
  for (int round = 0; round < max_rounds; ++round) {
    if (d == 64)
      ward_nearest<64><<<grid, kNearestThreads, 0, s>>>(w);
    else if (d == 32)
      ward_nearest<32><<<grid, kNearestThreads, 0, s>>>(w);
    else
      ward_nearest<16><<<grid, kNearestThreads, 0, s>>>(w);
    ward_fix<<<(unsigned)G, kFixThreads, fix_smem, s>>>(w, rounds);
  }
  ward_large_labels<<<(unsigned)G, 256, (size_t)P * sizeof(int), s>>>(w, labels, reached);
  LSA_LAUNCH_CHECK();
  return LSA_OK;
}

}  // namespace lsa
