// Bucket search: score candidates with a fixed-order fp32 dot, keep each row's best as packed int64 keys.
//
// One kernel serves the flat prefill scan (eight rows a CTA share every centroid they load), the flat decode
// scan (one row, its buckets split over CTAs, lists merged afterwards) and a beam step of the tree (one row,
// carried children beside a run of open rows). Selection is exact: a streaming top-k over 64-bit keys whose low
// word breaks a score tie toward the lower id, so the result does not depend on the order keys were produced in.
#include "common.cuh"
#include "scan_select.cuh"
#include "shape.cuh"

namespace lsa {

#ifdef LSA_SELECT_TRACE
// Clock stamps of thread 0 of one CTA of a decode row's scan (row 0) and of its merge (row 1), for a build that asks.
__device__ long long lsa_select_trace[2][16];
#define LSA_STAMP(row, at)                                                         \
  do {                                                                             \
    if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0) lsa_select_trace[row][at] = clock64(); \
  } while (0)
#else
#define LSA_STAMP(row, at) \
  do {                     \
  } while (0)
#endif

constexpr int kSelThreads = 256;
constexpr int kSelWarps = kSelThreads / 32;
constexpr int kHistBins = 256;

// ---------------------------------------------------------------------------------------- warp-level top-k

// A threshold t with exactly k keys of buf[0..n) at or above it (n > k >= 1, keys distinct): 8-bit radix passes of
// one warp, most significant byte first, stopped as soon as the chosen bin holds exactly the keys still wanted.
// hist is 256 ints of warp-private shared memory.
__device__ uint64_t warp_kth_greatest(const int64_t *buf, int n, int k, int *hist) {
  const int lane = lane_id();
  uint64_t prefix = 0, mask = 0;
  int remaining = k;
  // The leading bytes every key shares (scores of one row lie close together) need no pass: counting them would
  // send every key to one bin.
  uint64_t every = ~0ull, any = 0;
  for (int i = lane; i < n; i += 32) {
    const uint64_t u = key_radix(buf[i]);
    every &= u, any |= u;
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    every &= __shfl_xor_sync(0xffffffffu, every, o);
    any |= __shfl_xor_sync(0xffffffffu, any, o);
  }
  const uint64_t differ = every ^ any;
  for (int byte = 7; byte >= 0; --byte) {
    const int shift = byte * 8;
    if ((differ >> shift) == 0) {  // (this byte and all above it are shared)
      prefix |= every & ((uint64_t)0xFF << shift);
      mask |= (uint64_t)0xFF << shift;
      continue;
    }
#pragma unroll
    for (int i = 0; i < kHistBins / 32; ++i) hist[lane * (kHistBins / 32) + i] = 0;
    __syncwarp();
    for (int i = lane; i < n; i += 32) {
      const uint64_t u = key_radix(buf[i]);
      if ((u & mask) == prefix) atomicAdd(&hist[(int)((u >> shift) & 0xFF)], 1);
    }
    __syncwarp();
    // Lane l owns bins 8l..8l+7; `above` counts the keys in bins over this lane's.
    int own[kHistBins / 32];
    int own_sum = 0;
#pragma unroll
    for (int i = 0; i < kHistBins / 32; ++i) {
      own[i] = hist[lane * (kHistBins / 32) + i];
      own_sum += own[i];
    }
    int above = own_sum;  // inclusive suffix sum over lanes, then made exclusive
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int other = __shfl_down_sync(0xffffffffu, above, o);
      if (lane + o < 32) above += other;
    }
    above -= own_sum;
    const bool here = above < remaining && above + own_sum >= remaining;
    const unsigned who = __ballot_sync(0xffffffffu, here);
    const int src = __ffs(who) - 1;
    int digit = 0, next_remaining = remaining;
    if (here) {
      int seen = above;
#pragma unroll
      for (int i = kHistBins / 32 - 1; i >= 0; --i) {
        if (seen < remaining && seen + own[i] >= remaining) {
          digit = lane * (kHistBins / 32) + i;
          next_remaining = remaining - seen;
        }
        seen += own[i];
      }
    }
    digit = __shfl_sync(0xffffffffu, digit, src);
    remaining = __shfl_sync(0xffffffffu, next_remaining, src);
    prefix |= (uint64_t)digit << shift;
    mask |= (uint64_t)0xFF << shift;
    // Every key of the chosen bin is wanted: the prefix with zero low bits already separates the k greatest keys.
    const int in_bin = __shfl_sync(0xffffffffu, hist[digit], 0);
    __syncwarp();
    if (in_bin == remaining) break;
  }
  return prefix;
}

// Move the entries of buf[from..to) that pass `keep(key)` down to buf[out..), in order; returns the new end.
template <typename Pred>
__device__ int warp_compact(int64_t *buf, int from, int to, int out, Pred keep) {
  const int lane = lane_id();
  for (int base = from; base < to; base += 32) {
    const int i = base + lane;
    const int64_t key = i < to ? buf[i] : kEmptyKey;
    const bool pass = i < to && keep(key);
    const unsigned votes = __ballot_sync(0xffffffffu, pass);
    __syncwarp();
    if (pass) buf[out + __popc(votes & ((1u << lane) - 1))] = key;
    out += __popc(votes);
    __syncwarp();
  }
  return out;
}

// The same threshold found by a whole CTA of kSelThreads threads (a decode row has the CTA to itself): every
// thread counts into one shared histogram, warp 0 picks the bin, the pick is broadcast through shared memory.
__device__ uint64_t block_kth_greatest(const int64_t *buf, int n, int k, int *hist, int *pick) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint64_t prefix = 0, mask = 0;
  int remaining = k;
  for (int byte = 7; byte >= 0; --byte) {
    const int shift = byte * 8;
    hist[tid] = 0;  // kSelThreads == kHistBins
    __syncthreads();
    for (int i = tid; i < n; i += kSelThreads) {
      const uint64_t u = key_radix(buf[i]);
      if ((u & mask) == prefix) atomicAdd(&hist[(int)((u >> shift) & 0xFF)], 1);
    }
    __syncthreads();
    if (warp == 0) {
      int own[kHistBins / 32];
      int own_sum = 0;
#pragma unroll
      for (int i = 0; i < kHistBins / 32; ++i) {
        own[i] = hist[lane * (kHistBins / 32) + i];
        own_sum += own[i];
      }
      int above = own_sum;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int other = __shfl_down_sync(0xffffffffu, above, o);
        if (lane + o < 32) above += other;
      }
      above -= own_sum;
      if (above < remaining && above + own_sum >= remaining) {
        int seen = above;
#pragma unroll
        for (int i = kHistBins / 32 - 1; i >= 0; --i) {
          if (seen < remaining && seen + own[i] >= remaining) {
            pick[0] = lane * (kHistBins / 32) + i;  // the digit
            pick[1] = remaining - seen;              // keys still wanted inside its bin
            pick[2] = own[i];                        // keys in the bin
          }
          seen += own[i];
        }
      }
    }
    __syncthreads();
    const int digit = pick[0];
    remaining = pick[1];
    const int in_bin = pick[2];
    prefix |= (uint64_t)digit << shift;
    mask |= (uint64_t)0xFF << shift;
    __syncthreads();  // the pick and the histogram are read before the next pass rewrites them
    if (in_bin == remaining) break;
  }
  return prefix;
}

// Keep the entries of buf[from..to) that pass `keep(key)` at buf[out..), in any order, with the whole CTA; returns
// the new end. Every thread first takes its entries into registers, so the source and the target may overlap.
constexpr int kBlockCompactPerThread = 12;  // up to 3,072 entries
template <typename Pred>
__device__ int block_compact(int64_t *buf, int from, int to, int out, int *counter, Pred keep) {
  int64_t mine[kBlockCompactPerThread];
#pragma unroll
  for (int i = 0; i < kBlockCompactPerThread; ++i) {
    const int at = from + (int)threadIdx.x + i * kSelThreads;
    mine[i] = at < to ? buf[at] : kEmptyKey;
    if (at >= to || !keep(mine[i])) mine[i] = kEmptyKey;
  }
  if (threadIdx.x == 0) *counter = out;
  __syncthreads();
#pragma unroll
  for (int i = 0; i < kBlockCompactPerThread; ++i)
    if (mine[i] != kEmptyKey) buf[atomicAdd(counter, 1)] = mine[i];
  __syncthreads();
  const int end = *counter;
  __syncthreads();
  return end;
}

// Sort buf[0..n) descending in place with one warp; buf has room for the next power of two of n.
__device__ void warp_sort_descending(int64_t *buf, int n) {
  const int lane = lane_id();
  int size = 1;
  while (size < n) size <<= 1;
  for (int i = n + lane; i < size; i += 32) buf[i] = kEmptyKey;
  __syncwarp();
  for (int span = 2; span <= size; span <<= 1) {
    for (int stride = span >> 1; stride > 0; stride >>= 1) {
      for (int t = lane; t < (size >> 1); t += 32) {
        const int i = ((t & ~(stride - 1)) << 1) | (t & (stride - 1));
        const int j = i | stride;
        const bool descending = (i & span) == 0;
        const int64_t a = buf[i], b = buf[j];
        if ((a < b) == descending) {
          buf[i] = b;
          buf[j] = a;
        }
      }
      __syncwarp();
    }
  }
}

// ---------------------------------------------------------------------------------------- top 128 in registers

// A decode row's candidates are a thousand or two: cutting them by radix passes costs a dozen barriers and shared
// histograms a pass. Here a warp holds 128 keys in registers, four a lane (key e at register e / 32 of lane e % 32),
// sorts them with a bitonic network whose exchanges are shuffles or register moves - no barrier at all - and the
// warps' lists are folded pairwise: the greater of A[e] and B[127 - e] is the best 128 of both as a bitonic run,
// which seven more stages sort. Keys are distinct (an id in the low word), so the result is the exact top 128.
constexpr int kTopLane = 4;
constexpr int kTopWarp = kTopLane * 32;

// One stage of the network over a warp's 128 keys: exchanges `stride` apart, descending where (e & span) == 0.
__device__ __forceinline__ void warp_exchange(int64_t (&k)[kTopLane], int lane, int span, int stride) {
  if (stride == 64) {  // registers 0-2 and 1-3 of a lane (span is 128 here: descending throughout)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int64_t a = k[j], b = k[j + 2];
      k[j] = a < b ? b : a, k[j + 2] = a < b ? a : b;
    }
  } else if (stride == 32) {  // registers 0-1 and 2-3
#pragma unroll
    for (int j = 0; j < 4; j += 2) {
      const bool descending = ((j * 32) & span) == 0;
      const int64_t a = k[j], b = k[j + 1];
      const bool swap = (a < b) == descending;
      k[j] = swap ? b : a, k[j + 1] = swap ? a : b;
    }
  } else {  // another lane's same register
    const bool lower = (lane & stride) == 0;
#pragma unroll
    for (int j = 0; j < kTopLane; ++j) {
      const bool descending = ((j * 32 + lane) & span) == 0;
      const int64_t mine = k[j], other = __shfl_xor_sync(0xffffffffu, mine, stride);
      const bool greater = lower == descending;  // the lower place of a descending run keeps the greater key
      k[j] = (mine < other) == greater ? other : mine;
    }
  }
}

__device__ __forceinline__ void warp_sort128(int64_t (&k)[kTopLane], int lane) {
  for (int span = 2; span <= kTopWarp; span <<= 1)
    for (int stride = span >> 1; stride > 0; stride >>= 1) warp_exchange(k, lane, span, stride);
}

// A bitonic run of 128 sorted descending.
__device__ __forceinline__ void warp_merge128(int64_t (&k)[kTopLane], int lane) {
  for (int stride = kTopWarp >> 1; stride > 0; stride >>= 1) warp_exchange(k, lane, kTopWarp, stride);
}

// The best 128 of this warp's sorted keys and another sorted list `t` of the same warp, left sorted in k.
__device__ __forceinline__ void warp_fold128(int64_t (&k)[kTopLane], const int64_t (&t)[kTopLane], int lane) {
#pragma unroll
  for (int j = 0; j < kTopLane; ++j) {
    const int64_t other = __shfl_sync(0xffffffffu, t[kTopLane - 1 - j], 31 - lane);  // t[127 - e]
    k[j] = k[j] < other ? other : k[j];
  }
  warp_merge128(k, lane);
}

// The best 128 of what the first `warps` warps of a CTA hold (128 sorted keys each; `warps` a power of two), left
// sorted in warp 0's registers. Every thread of the CTA calls this; `slots` is shared memory for warps / 2 lists that
// nobody reads or writes otherwise from the first barrier here on.
__device__ void block_top128(int64_t (&k)[kTopLane], int64_t *slots, int warps, int warp, int lane) {
  for (int half = warps >> 1; half >= 1; half >>= 1) {
    __syncthreads();
    if (warp >= half && warp < 2 * half) {
#pragma unroll
      for (int j = 0; j < kTopLane; ++j) slots[(warp - half) * kTopWarp + j * 32 + lane] = k[j];
    }
    __syncthreads();
    if (warp < half) {
#pragma unroll
      for (int j = 0; j < kTopLane; ++j) {
        const int64_t other = slots[warp * kTopWarp + kTopWarp - 1 - (j * 32 + lane)];
        k[j] = k[j] < other ? other : k[j];
      }
      warp_merge128(k, lane);
    }
  }
}

// ---------------------------------------------------------------------------------------- the kernel

// Dims whose vectors a single-row scan stages through shared memory: 8 or 16 columns of 16 bytes.
__host__ __device__ inline bool select_stages(int d) { return d == 32 || d == 64; }

// A tile of up to kSelThreads candidate vectors of NV 16-byte columns through shared memory, and this thread's own
// candidate's score out of it (every thread of the CTA calls this). The loads of a thread are all issued before any
// of them is stored: 16 of them wait together, not one after another.
template <int NV>
__device__ __forceinline__ float tile_score(const float *__restrict__ vectors, const int64_t *rowof_s, float4 *tile_s,
                                            const float *qs, int tile_n, int tid, bool scores) {
  float4 v[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int e = tid + i * kSelThreads, cand = e / NV, c4 = e % NV;
    const int64_t row = cand < tile_n ? rowof_s[cand] : -1;
    v[i] = row >= 0 ? __ldg(reinterpret_cast<const float4 *>(vectors + row * (NV * 4)) + c4)
                    : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  }
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int e = tid + i * kSelThreads, cand = e / NV, c4 = e % NV;
    tile_s[cand * NV + (c4 ^ (cand & (NV - 1)))] = v[i];
  }
  __syncthreads();
  float acc = 0.0f;
  if (scores) {
#pragma unroll
    for (int k4 = 0; k4 < NV; ++k4) {
      const float4 w = tile_s[tid * NV + (k4 ^ (tid & (NV - 1)))];
      const float4 q = *reinterpret_cast<const float4 *>(qs + k4 * 4);
      acc = fmaf(q.x, w.x, acc);
      acc = fmaf(q.y, w.y, acc);
      acc = fmaf(q.z, w.z, acc);
      acc = fmaf(q.w, w.w, acc);
    }
  }
  return acc;
}

struct SelectParams {
  const float *queries;         // [R, d]
  const float *vectors;         // [N, d]
  const int64_t *vector_base;   // [R] first row of `vectors` a row's ids are relative to, or NULL
  const int32_t *run_first;     // [R] first id of the contiguous run a row scores, or NULL for 0
  const int32_t *run_end;       // [R] end of that run
  const int32_t *carried;       // [R, n_carried] explicit candidate ids (-1 = none) scored before the run, or NULL
  const int32_t *row_keep;      // [R] a row's own keep (<= keep), or NULL
  const int64_t *children;      // [N, fanout] or NULL
  int64_t *keys_out;            // [splits, R, keep] or NULL
  int32_t *ids_out;             // [splits, R, keep] or NULL
  int32_t *carried_out;         // [R, keep * fanout] or NULL
  int64_t R, N;
  const int32_t *pages;         // [R, max_pages] page of every page_rows ids of a row (-1 = none), or NULL
  int d, n_carried, keep, fanout, id_base, chunk, run_limit, max_pages, page_rows;
  ShapeTable shape;             // the vectors' shapes, row for row (floors NULL: none)
};

// RB rows a CTA. Shared memory: queries [RB][d], per-row key buffers [RB][keep_pow2 + chunk], histograms.
template <int RB, bool SHAPED>
__global__ void __launch_bounds__(kSelThreads) select_kernel(SelectParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  int keep_room = 2;  // even, so the float4 reads of the queries behind the buffers stay 16-byte aligned
  while (keep_room < p.keep) keep_room <<= 1;
  const int row_room = keep_room + p.chunk;
  int64_t *bufs = reinterpret_cast<int64_t *>(smem_raw);               // [RB][row_room]
  float *qs = reinterpret_cast<float *>(bufs + (size_t)RB * row_room);  // [RB][d]
  int *hists = reinterpret_cast<int *>(qs + RB * p.d);                  // [RB][256]
  // (a single row of 32 or 64 dims: a tile of candidate vectors staged for the scoring, and the rows they came from)
  float4 *tile_s = reinterpret_cast<float4 *>(hists + RB * kHistBins);  // [kSelThreads][d / 4], columns swizzled
  int64_t *rowof_s = reinterpret_cast<int64_t *>(tile_s + kSelThreads * (p.d >> 2));  // [kSelThreads]
  const bool staged = RB == 1 && select_stages(p.d);  // (d = 64: 16 columns, d = 32: 8)
  __shared__ int total_s[RB], first_s[RB], end_s[RB];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int64_t row0 = (int64_t)blockIdx.x * RB;
  const int splits = gridDim.y, split = blockIdx.y;
  dependents_may_launch();
  wait_for_earlier_grids();
  LSA_STAMP(0, 0);

  for (int e = tid; e < RB * p.d; e += kSelThreads) {
    const int64_t r = row0 + e / p.d;
    qs[e] = r < p.R ? p.queries[r * p.d + e % p.d] : 0.0f;
  }
  if (tid < RB) {
    const int64_t r = row0 + tid;
    int first = 0, end = 0;
    if (r < p.R) {
      first = p.run_first ? p.run_first[r] : 0;
      end = p.run_end ? p.run_end[r] : 0;
      if (end > p.run_limit) end = p.run_limit;
      if (end < first) end = first;
    }
    first_s[tid] = first;
    end_s[tid] = end;
    total_s[tid] = r < p.R ? p.n_carried + (end - first) : 0;
  }
  __syncthreads();
  LSA_STAMP(0, 1);
  int max_total = 0;
#pragma unroll
  for (int i = 0; i < RB; ++i) max_total = max(max_total, total_s[i]);
  // This CTA's share of the candidate range, the same cut for every row it holds.
  const int per_split = (max_total + splits - 1) / splits;
  const int cand_begin = split * per_split;
  const int cand_end = min(max_total, cand_begin + per_split);

  // Per-row selection state, held by the row's warp.
  int held = 0;                 // keys held at the front of the row's buffer
  int64_t floor_key = kEmptyKey;  // a new key must beat this once the row holds its keep
  const int64_t my_row = row0 + warp;
  const int my_keep = (warp < RB && my_row < p.R) ? (p.row_keep ? min(p.row_keep[my_row], p.keep) : p.keep) : 0;
  // (a single row: every thread of the CTA carries the row's state, which stays the same in all of them)
  const int my_keep_all = (RB == 1 && row0 < p.R) ? (p.row_keep ? min(p.row_keep[row0], p.keep) : p.keep) : 0;
  __shared__ int block_counter, block_pick[3];
  // A single row whose share of the candidates is one chunk of at most 1,024, cut to at most 128: sorted in registers.
  const bool in_registers = RB == 1 && cand_end - cand_begin <= kSelWarps * kTopWarp && cand_end > cand_begin &&
                            cand_end - cand_begin <= p.chunk && p.keep <= kTopWarp &&
                            p.chunk >= kSelWarps / 2 * kTopWarp;  // (the chunk's room holds the lists being folded)
  bool sorted = false;

  for (int chunk_base = cand_begin; chunk_base < cand_end; chunk_base += p.chunk) {
    const int chunk_n = min(p.chunk, cand_end - chunk_base);
    // ---- score, a single row: a tile of candidates at a time. A thread a candidate reading its own vector straight
    // from memory makes every load instruction of a warp touch 32 lines (a vector is 128 or 256 bytes): the loads of
    // a 1,024-candidate share then cost more than everything else the CTA does. Here the tile's vectors come in with
    // every half warp on one vector's 256 contiguous bytes, land in shared memory with their 16-byte columns
    // swizzled by the candidate, and each thread reads its own back without a bank conflict, in the same order.
    for (int t0 = 0; staged && t0 < chunk_n; t0 += kSelThreads) {
      const int t = t0 + tid, c = chunk_base + t;
      int32_t id = -1;
      int64_t vec_row = -1;
      if (t < chunk_n && row0 < p.R && c < total_s[0]) {
        id = c < p.n_carried ? p.carried[row0 * p.n_carried + c] : first_s[0] + (c - p.n_carried);
        vec_row = id >= 0 ? (p.vector_base ? p.vector_base[row0] : 0) + id : -1;
        if (p.pages && id >= 0) {
          const int page = id / p.page_rows < p.max_pages ? p.pages[row0 * p.max_pages + id / p.page_rows] : -1;
          vec_row = page >= 0 ? (int64_t)page * p.page_rows + id % p.page_rows : -1;
          if (page < 0) id = -1;
        }
        if (vec_row >= p.N) vec_row = -1, id = -1;
      }
      rowof_s[tid] = vec_row;
      __syncthreads();
      const int tile_n = min(kSelThreads, chunk_n - t0);
      float acc = p.d == 64 ? tile_score<16>(p.vectors, rowof_s, tile_s, qs, tile_n, tid, vec_row >= 0)
                            : tile_score<8>(p.vectors, rowof_s, tile_s, qs, tile_n, tid, vec_row >= 0);
      if (t < chunk_n) {
        if constexpr (SHAPED) {
          if (vec_row >= 0) acc = shaped_score(acc, qs, p.d, p.shape, vec_row);
        }
        bufs[keep_room + t] = id >= 0 ? pack_key(acc, id + p.id_base) : kEmptyKey;
      }
    }
    // ---- score: a thread a candidate, every row of the CTA against it
    for (int t = tid; !staged && t < chunk_n; t += kSelThreads) {
      const int c = chunk_base + t;
      float acc[RB];
      int64_t vec_row[RB];
      int32_t ids[RB];
      bool same = true;
#pragma unroll
      for (int i = 0; i < RB; ++i) {
        const int64_t r = row0 + i;
        int32_t id = -1;
        if (r < p.R && c < total_s[i])
          id = c < p.n_carried ? p.carried[r * p.n_carried + c] : first_s[i] + (c - p.n_carried);
        ids[i] = id;
        vec_row[i] = id >= 0 ? (p.vector_base ? p.vector_base[r] : 0) + id : -1;
        if (p.pages && id >= 0) {
          // a request's logical bucket id sits at row id % page_rows of its page id / page_rows
          const int page = id / p.page_rows < p.max_pages ? p.pages[r * p.max_pages + id / p.page_rows] : -1;
          vec_row[i] = page >= 0 ? (int64_t)page * p.page_rows + id % p.page_rows : -1;
          if (page < 0) ids[i] = -1;
        }
        if (vec_row[i] >= p.N) vec_row[i] = -1, ids[i] = -1;
        acc[i] = 0.0f;
        same = same && (vec_row[i] == vec_row[0] || vec_row[i] < 0 || vec_row[0] < 0);
      }
      if (RB > 1 && same) {
        // Every row of the CTA scores the same vector: load it once.
        int64_t row = -1;
#pragma unroll
        for (int i = 0; i < RB; ++i)
          if (vec_row[i] >= 0) row = vec_row[i];
        if (row >= 0) {
          const float4 *v4 = reinterpret_cast<const float4 *>(p.vectors + row * p.d);
          for (int k4 = 0; k4 < p.d / 4; ++k4) {
            const float4 v = __ldg(v4 + k4);
#pragma unroll
            for (int i = 0; i < RB; ++i) {
              const float4 q = *reinterpret_cast<const float4 *>(qs + i * p.d + k4 * 4);
              acc[i] = fmaf(q.x, v.x, acc[i]);
              acc[i] = fmaf(q.y, v.y, acc[i]);
              acc[i] = fmaf(q.z, v.z, acc[i]);
              acc[i] = fmaf(q.w, v.w, acc[i]);
            }
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < RB; ++i) {
          if (vec_row[i] < 0) continue;
          const float4 *v4 = reinterpret_cast<const float4 *>(p.vectors + vec_row[i] * p.d);
          for (int k4 = 0; k4 < p.d / 4; ++k4) {
            const float4 v = __ldg(v4 + k4);
            const float4 q = *reinterpret_cast<const float4 *>(qs + i * p.d + k4 * 4);
            acc[i] = fmaf(q.x, v.x, acc[i]);
            acc[i] = fmaf(q.y, v.y, acc[i]);
            acc[i] = fmaf(q.z, v.z, acc[i]);
            acc[i] = fmaf(q.w, v.w, acc[i]);
          }
        }
      }
      if constexpr (SHAPED) {
#pragma unroll
        for (int i = 0; i < RB; ++i)
          if (vec_row[i] >= 0) acc[i] = shaped_score(acc[i], qs + i * p.d, p.d, p.shape, vec_row[i]);
      }
#pragma unroll
      for (int i = 0; i < RB; ++i)
        bufs[(size_t)i * row_room + keep_room + t] = ids[i] >= 0 ? pack_key(acc[i], ids[i] + p.id_base) : kEmptyKey;
    }
    LSA_STAMP(0, 2);
    __syncthreads();
    LSA_STAMP(0, 3);
    if (RB == 1 && in_registers) {
      // ---- select: every warp sorts 128 of the chunk's keys, the warps' lists are folded into warp 0's
      int64_t *chunk = bufs + keep_room;
      int64_t k[kTopLane];
#pragma unroll
      for (int j = 0; j < kTopLane; ++j) {
        const int at = warp * kTopWarp + j * 32 + lane;
        k[j] = at < chunk_n ? chunk[at] : kEmptyKey;
      }
      warp_sort128(k, lane);
      LSA_STAMP(0, 4);
      block_top128(k, chunk, kSelWarps, warp, lane);
      LSA_STAMP(0, 5);
      if (warp == 0) {
        int valid = 0;
#pragma unroll
        for (int j = 0; j < kTopLane; ++j) {
          bufs[j * 32 + lane] = k[j];
          valid += k[j] != kEmptyKey;
        }
        held = min(warp_sum_int(valid), my_keep_all);
        __syncwarp();
      }
      sorted = true;
      continue;
    }
    // ---- select: a row that has the CTA to itself is folded by all of its threads (the keys are distinct and the
    // final sort orders them, so the order they are kept in does not matter)
    if (RB == 1 && row_room <= kBlockCompactPerThread * kSelThreads) {
      if (my_keep_all > 0) {
        int64_t *buf = bufs;
        const int64_t floor_now = floor_key;
        int n = block_compact(buf, keep_room, keep_room + chunk_n, held, &block_counter,
                              [floor_now](int64_t key) { return key > floor_now; });
        if (n > my_keep_all) {
          const uint64_t kth = block_kth_greatest(buf, n, my_keep_all, hists, block_pick);
          n = block_compact(buf, 0, n, 0, &block_counter, [kth](int64_t key) { return key_radix(key) >= kth; });
          floor_key = (int64_t)(kth ^ 0x8000000000000000ull);
        }
        held = n;
      }
      __syncthreads();
      continue;
    }
    // ---- select: the row's warp folds the chunk into what it holds
    if (warp < RB && my_keep > 0) {
      int64_t *buf = bufs + (size_t)warp * row_room;
      const int64_t floor_now = floor_key;
      // Survivors land right after the held keys; room is never short because held <= keep_room.
      int n = warp_compact(buf, keep_room, keep_room + chunk_n, held,
                           [floor_now](int64_t key) { return key > floor_now; });
      if (n > my_keep) {
        const uint64_t kth = warp_kth_greatest(buf, n, my_keep, hists + warp * kHistBins);
        n = warp_compact(buf, 0, n, 0, [kth](int64_t key) { return key_radix(key) >= kth; });
        floor_key = (int64_t)(kth ^ 0x8000000000000000ull);
      }
      held = n;
    }
    __syncthreads();
  }

  if (warp < RB && my_row < p.R) {
    int64_t *buf = bufs + (size_t)warp * row_room;
    if (!sorted) warp_sort_descending(buf, held);
    const int64_t out_row = ((int64_t)split * p.R + my_row) * p.keep;
    for (int i = lane; i < p.keep; i += 32) {
      const int64_t key = i < held ? buf[i] : kEmptyKey;
      if (p.keys_out) p.keys_out[out_row + i] = key;
      if (p.ids_out) p.ids_out[out_row + i] = key == kEmptyKey ? LSA_PAD : key_id(key);
    }
    if (p.carried_out) {
      const int total = p.keep * p.fanout;
      for (int e = lane; e < total; e += 32) {
        const int i = e / p.fanout, c = e - i * p.fanout;
        int32_t child = LSA_PAD;
        if (i < held) child = (int32_t)p.children[(int64_t)(key_id(buf[i]) - p.id_base) * p.fanout + c];
        p.carried_out[my_row * total + e] = child;
      }
    }
  }
  LSA_STAMP(0, 6);
}

// Global top-k of `parts` lists of packed keys, a warp a row.
__global__ void __launch_bounds__(kSelThreads) merge_candidates_kernel(const int64_t *__restrict__ keys_in, int parts,
                                                              int64_t R, int keep, int room,
                                                              int64_t *__restrict__ keys_out,
                                                              int32_t *__restrict__ ids_out,
                                                              const int64_t *__restrict__ children, int fanout,
                                                              int32_t *__restrict__ carried_out, int lists_sorted) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  int64_t *buf = reinterpret_cast<int64_t *>(smem_raw);  // [room]
  int *hist = reinterpret_cast<int *>(buf + room);        // [256]
  const int lane = lane_id();
  const int64_t r = blockIdx.x;
  dependents_may_launch();
  wait_for_earlier_grids();
  LSA_STAMP(1, 0);
  int n = 0;
  bool sorted = false;
  if (keep <= kTopWarp && parts > 1) {
    // lists of at most 128 keys (a decode row split over CTAs, the ranks' candidates): a warp takes a list into its
    // registers, sorts it unless the caller made it and knows it sorted (best first, empty keys last), folds in the
    // lists a stride of warps further on, and the warps' results are folded into warp 0's
    const int warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    int64_t k[kTopLane];
    auto take = [&](int64_t (&into)[kTopLane], int part) {
#pragma unroll
      for (int j = 0; j < kTopLane; ++j) {
        const int e = j * 32 + lane;
        into[j] = part < parts && e < keep ? keys_in[((int64_t)part * R + r) * keep + e] : kEmptyKey;
      }
      if (!lists_sorted) warp_sort128(into, lane);
    };
    take(k, warp);
    LSA_STAMP(1, 1);
    for (int part = warp + warps; part < parts; part += warps) {  // (the same trips for every lane of a warp)
      int64_t t[kTopLane];
      take(t, part);
      warp_fold128(k, t, lane);
    }
    LSA_STAMP(1, 2);
    block_top128(k, buf, warps, warp, lane);
    LSA_STAMP(1, 3);
    if (warp > 0) return;
#pragma unroll
    for (int j = 0; j < kTopLane; ++j) {
      buf[j * 32 + lane] = k[j];
      n += k[j] != kEmptyKey;
    }
    n = warp_sum_int(n);
    if (n > keep) n = keep;
    __syncwarp();
    sorted = true;
  } else if (blockDim.x == kSelThreads) {
    // many candidates (a row split over dozens of CTAs): the whole CTA cuts them to `keep`, warp 0 sorts and writes
    __shared__ int counter, pick[3];
    const int total = parts * keep;
    for (int e = threadIdx.x; e < total; e += kSelThreads)
      buf[e] = keys_in[((int64_t)(e / keep) * R + r) * keep + e % keep];
    __syncthreads();
    n = block_compact(buf, 0, total, 0, &counter, [](int64_t key) { return key != kEmptyKey; });
    if (n > keep) {
      const uint64_t kth = block_kth_greatest(buf, n, keep, hist, pick);
      n = block_compact(buf, 0, n, 0, &counter, [kth](int64_t key) { return key_radix(key) >= kth; });
    }
    if (threadIdx.x >= 32) return;
  } else {
    for (int base = 0; base < parts * keep; base += 32) {
      const int e = base + lane;
      int64_t key = kEmptyKey;
      if (e < parts * keep) key = keys_in[((int64_t)(e / keep) * R + r) * keep + e % keep];
      const bool pass = key != kEmptyKey;
      const unsigned votes = __ballot_sync(0xffffffffu, pass);
      if (pass) buf[n + __popc(votes & ((1u << lane) - 1))] = key;
      n += __popc(votes);
    }
    __syncwarp();
    if (n > keep) {
      const uint64_t kth = warp_kth_greatest(buf, n, keep, hist);
      n = warp_compact(buf, 0, n, 0, [kth](int64_t key) { return key_radix(key) >= kth; });
    }
  }
  if (!sorted) warp_sort_descending(buf, n);
  for (int i = lane; i < keep; i += 32) {
    const int64_t key = i < n ? buf[i] : kEmptyKey;
    if (keys_out) keys_out[r * keep + i] = key;
    if (ids_out) ids_out[r * keep + i] = key == kEmptyKey ? LSA_PAD : key_id(key);
  }
  if (carried_out) {  // the children of the kept rows, best row first
    __syncwarp();
    for (int e = lane; e < keep * fanout; e += 32) {
      const int i = e / fanout, c = e - i * fanout;
      carried_out[r * keep * fanout + e] = i < n ? (int32_t)children[(int64_t)key_id(buf[i]) * fanout + c] : LSA_PAD;
    }
  }
  LSA_STAMP(1, 4);
}

// Threads of a candidate merge: a warp for a few hundred candidates, the whole CTA for what its registers can hold.
static int merge_threads(int parts, int keep) {
  const int64_t total = (int64_t)parts * keep;
  if (keep <= kTopWarp && parts > 1) {  // a warp a list (or several), a power of two of warps
    int warps = 1;
    while (warps < kSelWarps && warps < parts) warps <<= 1;
    return warps * 32;
  }
  return total > 256 && total <= kBlockCompactPerThread * kSelThreads ? kSelThreads : 32;
}

static int pow2_at_least(int n) {
  int v = 2;
  while (v < n) v <<= 1;
  return v;
}

// Chunk of candidates a pass scores: as many as shared memory holds beside the held keys, at most 2048.
static int select_chunk(int rb, int keep, int d, size_t *smem_out) {
  const size_t budget = 200 * 1024;
  const size_t tile = rb == 1 && select_stages(d) ? (size_t)kSelThreads * (d * 4 + 8) : 0;
  const size_t fixed = (size_t)rb * (pow2_at_least(keep) * 8 + d * 4 + kHistBins * 4) + tile;
  int chunk = 2048;
  while (chunk > 256 && fixed + (size_t)rb * chunk * 8 > budget) chunk -= 256;
  if (fixed + (size_t)rb * chunk * 8 > budget) return 0;
  *smem_out = fixed + (size_t)rb * chunk * 8;
  return chunk;
}

template <int RB>
static int launch_select(SelectParams p, int splits, cudaStream_t s) {
  size_t smem = 0;
  p.chunk = select_chunk(RB, p.keep, p.d, &smem);
  if (p.chunk == 0) return LSA_ERR_UNSUPPORTED;
  dim3 grid((unsigned)((p.R + RB - 1) / RB), (unsigned)splits);
  if (p.shape.floors) {
    if (cudaFuncSetAttribute(select_kernel<RB, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return LSA_ERR_LAUNCH;
    launch(p.R <= kChainedRows, select_kernel<RB, true>, grid, dim3(kSelThreads), smem, s, p);
    LSA_LAUNCH_CHECK();
    return LSA_OK;
  }
  if (cudaFuncSetAttribute(select_kernel<RB, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
      cudaSuccess)
    return LSA_ERR_LAUNCH;
  launch(p.R <= kChainedRows, select_kernel<RB, false>, grid, dim3(kSelThreads), smem, s, p);
  LSA_LAUNCH_CHECK();
  return LSA_OK;
}


// ---------------------------------------------------------------------------------------- flat prefill scan

// The prefill form of the flat scan: row r scores the first visible[r] centroids, so every row of a CTA scores the
// SAME centroid for a candidate and it is loaded once for all of them. 16 rows and 16 warps a CTA: all 512 threads
// score a chunk (a thread a centroid, 16 dots), then each warp folds the chunk into its own row's held keys.
constexpr int kFlatRows = 16;
constexpr int kFlatThreads = kFlatRows * 32;

struct FlatParams {
  const float *queries, *centroids;
  const int32_t *visible, *row_keep;
  const int32_t *row_flags;  // [R] or NULL: only rows with a nonzero flag are scanned (the others keep their output)
  int64_t *keys_out;
  int32_t *ids_out;
  int64_t R, m;
  int d, keep, id_base, chunk;
  ShapeTable shape;  // the centroids' shapes, row for row (floors NULL: none)
};

template <int D, bool SHAPED>
__global__ void __launch_bounds__(kFlatThreads) flat_select_kernel(FlatParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  int keep_room = 2;
  while (keep_room < p.keep) keep_room <<= 1;
  const int row_room = keep_room + p.chunk;
  int64_t *bufs = reinterpret_cast<int64_t *>(smem_raw);                     // [16][row_room]
  float *qs = reinterpret_cast<float *>(bufs + (size_t)kFlatRows * row_room);  // [16][D]
  int *hists = reinterpret_cast<int *>(qs + kFlatRows * D);                    // [16][256]
  __shared__ int visible_s[kFlatRows];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int64_t row0 = (int64_t)blockIdx.x * kFlatRows;
  for (int e = tid; e < kFlatRows * D; e += kFlatThreads) {
    const int64_t r = row0 + e / D;
    qs[e] = r < p.R ? p.queries[r * D + e % D] : 0.0f;
  }
  if (tid < kFlatRows) {
    const int64_t r = row0 + tid;
    int v = r < p.R && (!p.row_flags || p.row_flags[r]) ? p.visible[r] : 0;
    visible_s[tid] = v < 0 ? 0 : (v > p.m ? (int)p.m : v);
  }
  __syncthreads();
  int widest = 0;
#pragma unroll
  for (int i = 0; i < kFlatRows; ++i) widest = max(widest, visible_s[i]);

  int held = 0;
  int64_t floor_key = kEmptyKey;
  const int64_t my_row = row0 + warp;
  const int my_visible = visible_s[warp];
  const int my_keep = my_row < p.R ? (p.row_keep ? min(p.row_keep[my_row], p.keep) : p.keep) : 0;

  for (int base = 0; base < widest; base += p.chunk) {
    const int n = min(p.chunk, widest - base);
    for (int c = tid; c < n; c += kFlatThreads) {
      float acc[kFlatRows];
#pragma unroll
      for (int i = 0; i < kFlatRows; ++i) acc[i] = 0.0f;
      const float4 *v4 = reinterpret_cast<const float4 *>(p.centroids + (int64_t)(base + c) * D);
#pragma unroll 4
      for (int k4 = 0; k4 < D / 4; ++k4) {
        const float4 v = __ldg(v4 + k4);
#pragma unroll
        for (int i = 0; i < kFlatRows; ++i) {
          const float4 q = *reinterpret_cast<const float4 *>(qs + i * D + k4 * 4);
          acc[i] = fmaf(q.x, v.x, acc[i]);
          acc[i] = fmaf(q.y, v.y, acc[i]);
          acc[i] = fmaf(q.z, v.z, acc[i]);
          acc[i] = fmaf(q.w, v.w, acc[i]);
        }
      }
      if constexpr (SHAPED) {
        // The spread of this thread's bucket under each of the CTA's rows: a sign is read off its word once and
        // meets all sixteen rows.
        float variance[kFlatRows], inside[kFlatRows];
#pragma unroll
        for (int i = 0; i < kFlatRows; ++i) variance[i] = 0.0f, inside[i] = 0.0f;
        const int64_t bucket = base + c;
        for (int j = 0; j < p.shape.rank; ++j) {
          float along[kFlatRows];
#pragma unroll
          for (int i = 0; i < kFlatRows; ++i) along[i] = 0.0f;
          const uint32_t *bits = p.shape.basis + (bucket * p.shape.rank + j) * (D / 32);
#pragma unroll
          for (int w = 0; w < D / 32; ++w) {
            const uint32_t word = __ldg(bits + w);
#pragma unroll 2
            for (int b4 = 0; b4 < 8; ++b4) {
              const float s0 = shape_sign(word, b4 * 4), s1 = shape_sign(word, b4 * 4 + 1);
              const float s2 = shape_sign(word, b4 * 4 + 2), s3 = shape_sign(word, b4 * 4 + 3);
#pragma unroll
              for (int i = 0; i < kFlatRows; ++i) {
                const float4 q = *reinterpret_cast<const float4 *>(qs + i * D + w * 32 + b4 * 4);
                along[i] = __fmaf_rn(q.x, s0, along[i]);
                along[i] = __fmaf_rn(q.y, s1, along[i]);
                along[i] = __fmaf_rn(q.z, s2, along[i]);
                along[i] = __fmaf_rn(q.w, s3, along[i]);
              }
            }
          }
          const float variance_j = __ldg(p.shape.variances + bucket * p.shape.rank + j);
#pragma unroll
          for (int i = 0; i < kFlatRows; ++i) shape_fold(along[i], p.shape.scale, variance_j, variance[i], inside[i]);
        }
        const float floor_ = __ldg(p.shape.floors + bucket);
#pragma unroll
        for (int i = 0; i < kFlatRows; ++i)
          acc[i] = shape_finish(acc[i], variance[i], inside[i], floor_, p.shape.deviations);
      }
#pragma unroll
      for (int i = 0; i < kFlatRows; ++i)
        bufs[(size_t)i * row_room + keep_room + c] =
            base + c < visible_s[i] ? pack_key(acc[i], base + c + p.id_base) : kEmptyKey;
    }
    __syncthreads();
    if (my_keep > 0 && base < my_visible) {
      int64_t *buf = bufs + (size_t)warp * row_room;
      const int64_t floor_now = floor_key;
      int count = warp_compact(buf, keep_room, keep_room + min(n, my_visible - base), held,
                               [floor_now](int64_t key) { return key > floor_now; });
      if (count > my_keep) {
        const uint64_t kth = warp_kth_greatest(buf, count, my_keep, hists + warp * kHistBins);
        count = warp_compact(buf, 0, count, 0, [kth](int64_t key) { return key_radix(key) >= kth; });
        floor_key = (int64_t)(kth ^ 0x8000000000000000ull);
      }
      held = count;
    }
    __syncthreads();
  }
  if (my_row < p.R && (!p.row_flags || p.row_flags[my_row])) {
    int64_t *buf = bufs + (size_t)warp * row_room;
    warp_sort_descending(buf, held);
    for (int i = lane; i < p.keep; i += 32) {
      const int64_t key = i < held ? buf[i] : kEmptyKey;
      if (p.keys_out) p.keys_out[my_row * p.keep + i] = key;
      if (p.ids_out) p.ids_out[my_row * p.keep + i] = key == kEmptyKey ? LSA_PAD : key_id(key);
    }
  }
}

template <int D>
static int launch_flat(FlatParams p, cudaStream_t s) {
  int keep_room = 2;
  while (keep_room < p.keep) keep_room <<= 1;
  const size_t fixed = (size_t)kFlatRows * (keep_room * 8 + D * 4 + kHistBins * 4);
  p.chunk = 1024;
  while (p.chunk > 256 && fixed + (size_t)kFlatRows * p.chunk * 8 > 200 * 1024) p.chunk -= 256;
  const size_t smem = fixed + (size_t)kFlatRows * p.chunk * 8;
  if (smem > 200 * 1024) return LSA_ERR_UNSUPPORTED;
  const unsigned grid = (unsigned)((p.R + kFlatRows - 1) / kFlatRows);
  if (p.shape.floors) {
    if (cudaFuncSetAttribute(flat_select_kernel<D, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return LSA_ERR_LAUNCH;
    flat_select_kernel<D, true><<<grid, kFlatThreads, smem, s>>>(p);
  } else {
    if (cudaFuncSetAttribute(flat_select_kernel<D, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return LSA_ERR_LAUNCH;
    flat_select_kernel<D, false><<<grid, kFlatThreads, smem, s>>>(p);
  }
  LSA_LAUNCH_CHECK();
  return LSA_OK;
}

}  // namespace lsa

#ifdef LSA_SELECT_TRACE
extern "C" __attribute__((visibility("default"))) int lsa_select_trace_read(long long *host) {
  return (int)cudaMemcpyFromSymbol(host, lsa::lsa_select_trace, sizeof(lsa::lsa_select_trace));
}
#endif

// ================================================================================================ C ABI

// ------------------------------------------------------------------------------------------------ tensor-core scan

namespace lsa {

// Before the scan: a bf16 copy of the query rows (the M operand of the scan's products), their lengths, which rows
// take the exact scan instead (too few visible buckets for a sampled threshold to mean anything), and the widest
// visible count among a tile's other rows.
__global__ void __launch_bounds__(128)
    scan_prepare_kernel(const float *__restrict__ queries, const int32_t *__restrict__ visible, int64_t R, int64_t m,
                        uint16_t *__restrict__ q_bf16, float *__restrict__ norms, int32_t *__restrict__ flags,
                        int32_t *__restrict__ tile_visible, int keep, int min_visible, int32_t *__restrict__ taken,
                        int32_t *__restrict__ retry_visible, int32_t *__restrict__ retry_keep) {
  __shared__ int widest_s;
  const int64_t row = (int64_t)blockIdx.x * 128 + threadIdx.x;
  if (threadIdx.x == 0) widest_s = 0;
  if (blockIdx.x == 0) {  // the split exact scan's row list starts empty, its unused rows seeing nothing
    if (threadIdx.x == 0) *taken = 0;
    if (threadIdx.x < kScanRetry) retry_visible[threadIdx.x] = 0, retry_keep[threadIdx.x] = keep;
  }
  __syncthreads();
  float ss = 0.0f;
  uint32_t packed[32];
#pragma unroll
  for (int k = 0; k < 64; k += 4) {
    const float4 v = row < R ? *reinterpret_cast<const float4 *>(queries + row * 64 + k) : make_float4(0.f, 0.f, 0.f, 0.f);
    ss = fmaf(v.x, v.x, ss), ss = fmaf(v.y, v.y, ss), ss = fmaf(v.z, v.z, ss), ss = fmaf(v.w, v.w, ss);
    packed[k / 2] = (uint32_t)float_to_bf16_bits(v.x) | ((uint32_t)float_to_bf16_bits(v.y) << 16);
    packed[k / 2 + 1] = (uint32_t)float_to_bf16_bits(v.z) | ((uint32_t)float_to_bf16_bits(v.w) << 16);
  }
  uint4 *dst = reinterpret_cast<uint4 *>(q_bf16 + row * 64);
#pragma unroll
  for (int i = 0; i < 8; ++i) dst[i] = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
  if (row < R) {
    const int v = min(max(visible[row], 0), (int)m);
    const bool exact = v < min_visible || !(ss > 0.0f) || !isfinite(ss);
    norms[row] = sqrtf(ss);
    flags[row] = exact ? 1 : 0;
    if (!exact) atomicMax(&widest_s, v);
  }
  __syncthreads();
  if (threadIdx.x == 0) tile_visible[blockIdx.x] = widest_s;
}

// After the scan: a warp a row. A survivor's true score lies within its slack of its bf16-operand score. With s the
// keep-th greatest LOWER bound, at least `keep` buckets truly score s or more, so a bucket whose UPPER bound is under
// s is not among the best `keep`; whatever the scan dropped has an upper bound under the row's threshold. So when s
// reaches the threshold, the survivors whose upper bound reaches s are all that can matter: those are rescored with
// the exact fixed-order fp32 dot and the best `keep` of them are the row's picks, key for key what scoring every
// bucket would give. A row that cannot be proven - a list overflowed, fewer than `keep` survivors, s under the
// threshold - is flagged for an exact scan, which then writes it.
__global__ void __launch_bounds__(kSelThreads)
    scan_pick_kernel(ScanParams p, const float *__restrict__ queries, const float *__restrict__ centroids,
                     int32_t *__restrict__ flags, int id_base, int room, int64_t *__restrict__ keys_out,
                     int32_t *__restrict__ ids_out) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int warp = threadIdx.x >> 5, lane = lane_id();
  int64_t *buf = reinterpret_cast<int64_t *>(smem_raw) + (size_t)warp * room;
  int *hist = reinterpret_cast<int *>(reinterpret_cast<int64_t *>(smem_raw) + (size_t)kSelWarps * room) + warp * kHistBins;
  const int64_t row = (int64_t)blockIdx.x * kSelWarps + warp;
  if (row >= p.R || flags[row]) return;
  const int keep = p.row_keep ? min(p.row_keep[row], p.keep) : p.keep;
  const int lists = 2 * p.spans;
  int total = 0;
  bool proven = true;
  const float norm = p.norms[row];
  const float uniform = scan_slack(p.radius ? *p.radius : 1.0f);
  for (int l = 0; l < lists; ++l) {
    const int found = p.counts[row * lists + l];
    proven &= found <= p.cap && total + found <= room;
    const int n = proven ? found : 0;
    const int2 *list = p.survivors + (row * lists + l) * p.cap;
    for (int j = lane; j < n; j += 32) {
      const int2 e = list[j];
      // keyed by the LEAST its true score can be
      const float slack = norm * (p.lengths ? scan_slack(__ldg(p.lengths + e.y)) : uniform);
      buf[total + j] = pack_key(__int_as_float(e.x) - slack, e.y);
    }
    total += n;
  }
  __syncwarp();
  proven &= total >= keep;
  if (keep == 0) total = 0;  // (a row whose budget is nothing)
  if (proven && keep > 0) {
    // s: the keep-th greatest lower bound - at least `keep` buckets truly score s or more, so a bucket whose upper
    // bound is under s is not among the best `keep`. Whatever the scan dropped has an upper bound under the row's
    // threshold, so with s at or above the threshold everything that can matter is in the lists.
    const uint64_t kth = total > keep ? warp_kth_greatest(buf, total, keep, hist) : 0;
    int64_t least = INT64_MAX;
    for (int j = lane; j < total; j += 32)
      if (key_radix(buf[j]) >= kth) least = min(least, buf[j]);
    for (int off = 16; off; off >>= 1) least = min(least, __shfl_xor_sync(0xffffffffu, least, off));
    const int32_t bits = (int32_t)(least >> 32);
    const float s = __int_as_float(bits < 0 ? (bits ^ 0x7FFFFFFF) : bits);
    proven = s >= p.bars[row];
    if (proven) {
      // keep the buckets whose upper bound (the lower one plus twice the slack) reaches s
      const float *lengths = p.lengths;
      total = warp_compact(buf, 0, total, 0, [s, norm, uniform, lengths](int64_t key) {
        const int32_t b = (int32_t)(key >> 32);
        const float low = __int_as_float(b < 0 ? (b ^ 0x7FFFFFFF) : b);
        const float slack = norm * (lengths ? scan_slack(__ldg(lengths + key_id(key))) : uniform);
        return fmaf(2.0f, slack, low) >= s;
      });
      const float *q = queries + row * 64;
      for (int j = lane; j < total; j += 32) {
        const int32_t id = key_id(buf[j]);
        const float4 *v4 = reinterpret_cast<const float4 *>(centroids + (int64_t)id * 64);
        float acc = 0.0f;
#pragma unroll 4
        for (int k4 = 0; k4 < 16; ++k4) {
          const float4 v = __ldg(v4 + k4);
          const float4 qv = *reinterpret_cast<const float4 *>(q + k4 * 4);
          acc = fmaf(qv.x, v.x, acc), acc = fmaf(qv.y, v.y, acc), acc = fmaf(qv.z, v.z, acc), acc = fmaf(qv.w, v.w, acc);
        }
        buf[j] = pack_key(acc, id + id_base);
      }
      __syncwarp();
      if (total > keep) {
        const uint64_t cut = warp_kth_greatest(buf, total, keep, hist);
        total = warp_compact(buf, 0, total, 0, [cut](int64_t key) { return key_radix(key) >= cut; });
      }
      warp_sort_descending(buf, total);
    }
  }
  if (!proven) {
    if (lane == 0) flags[row] = 1;
    return;
  }
  for (int i = lane; i < p.keep; i += 32) {
    const int64_t key = i < total && i < keep ? buf[i] : kEmptyKey;
    if (keys_out) keys_out[row * p.keep + i] = key;
    if (ids_out) ids_out[row * p.keep + i] = key == kEmptyKey ? LSA_PAD : key_id(key);
  }
}

// The rows still flagged after the pick, gathered side by side for an exact scan that splits each row's buckets over
// many CTAs: at most kScanRetry of them a call (those keep their flag cleared; any more stay flagged for the plain
// exact scan).
__global__ void __launch_bounds__(256)
    scan_collect_kernel(const float *__restrict__ queries, const int32_t *__restrict__ visible,
                        const int32_t *__restrict__ row_keep, int keep, int64_t R, int64_t m, int32_t *__restrict__ flags,
                        int32_t *__restrict__ taken, float *__restrict__ q_out, int32_t *__restrict__ visible_out,
                        int32_t *__restrict__ keep_out, int32_t *__restrict__ row_out) {
  const int64_t row = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= R || !flags[row]) return;
  const int slot = atomicAdd(taken, 1);
  if (slot >= kScanRetry) return;
  flags[row] = 0;
  for (int k = 0; k < 64; k += 4)
    *reinterpret_cast<float4 *>(q_out + slot * 64 + k) = *reinterpret_cast<const float4 *>(queries + row * 64 + k);
  visible_out[slot] = min(max(visible[row], 0), (int)m);
  keep_out[slot] = row_keep ? min(row_keep[row], keep) : keep;
  row_out[slot] = (int32_t)row;
}

// ... and their picks written back where they belong.
__global__ void scan_scatter_kernel(const int64_t *__restrict__ keys_in, const int32_t *__restrict__ row_of,
                                    const int32_t *__restrict__ keep_of, const int32_t *__restrict__ taken, int keep,
                                    int64_t *__restrict__ keys_out, int32_t *__restrict__ ids_out) {
  const int slot = blockIdx.x;
  if (slot >= min(*taken, kScanRetry)) return;
  const int64_t row = row_of[slot];
  const int budget = keep_of[slot];  // (the merge of a row's splits knows the call's top_p, not the row's own)
  for (int i = threadIdx.x; i < keep; i += blockDim.x) {
    const int64_t key = i < budget ? keys_in[(int64_t)slot * keep + i] : kEmptyKey;
    if (keys_out) keys_out[row * keep + i] = key;
    if (ids_out) ids_out[row * keep + i] = key == kEmptyKey ? LSA_PAD : key_id(key);
  }
}

constexpr int kScanRetrySplits = 16;

struct ScanWorkspace {
  size_t q_bf16, norms, flags, tile_visible, thresholds, counts, survivors;
  size_t taken, retry_q, retry_visible, retry_keep, retry_row, retry_parts, retry_keys, total;
};

static int scan_spans(int64_t padded_rows, int64_t m) {
  const int row_tiles = (int)(padded_rows / 128), tiles = (int)((m + 127) / 128);
  // One wave of CTAs (each owns an SM's tensor memory): every span repeats the four sample tiles and the
  // bisection, so the fewest spans that fill the machine, of at least eight tiles each.
  int spans = 148 / row_tiles;
  spans = max(1, min(spans, tiles / 8));
  return min(spans, 16);
}

// Three times top_p survivors are aimed at (twice, from top_p = 512 on, where more would not fit a row's room).
static int scan_factor(int top_p) { return max(2, min(3, kScanRoom / 2 / top_p)); }

// A list holds four times its even share of the survivors aimed at, so a row whose best buckets crowd into a
// quarter of its lists still fits; all of a row's lists together stay within kScanRoom.
static int scan_cap(int top_p, int spans) {
  const int lists = 2 * spans, aimed = scan_factor(top_p) * top_p;
  const int cap = max(32, (4 * aimed / lists + 31) / 32 * 32);
  return min(cap, kScanRoom / lists);
}

// Survivors of a row the pick has room for: twice those aimed at (a row with more is scanned exactly).
static int scan_room(int top_p) { return pow2_at_least(max(256, min(2 * scan_factor(top_p) * top_p, kScanRoom))); }

static ScanWorkspace scan_workspace(int64_t R, int top_p, int64_t m) {
  auto up = [](size_t x) { return (x + 255) & ~(size_t)255; };
  const int64_t padded = (R + 127) / 128 * 128;
  const int spans = scan_spans(padded, m), cap = scan_cap(top_p, spans);
  ScanWorkspace w;
  size_t at = 0;
  w.q_bf16 = at, at += up((size_t)padded * 64 * 2);
  w.norms = at, at += up((size_t)R * 4);
  w.flags = at, at += up((size_t)R * 4);
  w.tile_visible = at, at += up((size_t)(padded / 128) * 4);
  w.thresholds = at, at += up((size_t)R * 4);
  w.counts = at, at += up((size_t)R * 2 * spans * 4);
  w.survivors = at, at += up((size_t)R * 2 * spans * cap * 8);
  w.taken = at, at += 256;
  w.retry_q = at, at += up((size_t)kScanRetry * 64 * 4);
  w.retry_visible = at, at += up((size_t)kScanRetry * 4);
  w.retry_keep = at, at += up((size_t)kScanRetry * 4);
  w.retry_row = at, at += up((size_t)kScanRetry * 4);
  w.retry_parts = at, at += up((size_t)kScanRetrySplits * kScanRetry * top_p * 8);
  w.retry_keys = at, at += up((size_t)kScanRetry * top_p * 8);
  w.total = at;
  return w;
}

}  // namespace lsa

namespace lsa {

// The N operand of the tensor-core scan: the centroids less a common centre, rounded to bf16, and the greatest length
// of such a row (kept as the bits of a non-negative float, which order as integers do).
__global__ void __launch_bounds__(256)
    scan_centre_kernel(const float *__restrict__ centroids, int64_t rows, const float *__restrict__ centre,
                       uint16_t *__restrict__ out, float *__restrict__ lengths, float *__restrict__ radius) {
  const int64_t row = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= rows) return;
  float ss = 0.0f;
#pragma unroll
  for (int k = 0; k < 64; k += 8) {
    uint32_t packed[4];
#pragma unroll
    for (int j = 0; j < 8; j += 2) {
      const float a = centroids[row * 64 + k + j] - (centre ? centre[k + j] : 0.0f);
      const float b = centroids[row * 64 + k + j + 1] - (centre ? centre[k + j + 1] : 0.0f);
      ss = fmaf(a, a, ss), ss = fmaf(b, b, ss);
      packed[j / 2] = (uint32_t)float_to_bf16_bits(a) | ((uint32_t)float_to_bf16_bits(b) << 16);
    }
    *reinterpret_cast<uint4 *>(out + row * 64 + k) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
  }
  const float length = sqrtf(ss) * 1.000001f;
  if (lengths) lengths[row] = length;
  if (radius) atomicMax(reinterpret_cast<int *>(radius), __float_as_int(length));
}

}  // namespace lsa

LSA_API int lsa_scan_centre(const float *centroids, int64_t rows, int d, const float *centre, uint16_t *out_bf16,
                            float *lengths, float *radius, void *stream) {
  LSA_REQUIRE(centroids && out_bf16, LSA_ERR_NULL);
  LSA_REQUIRE(rows >= 0, LSA_ERR_ARGUMENT);
  LSA_REQUIRE(d == 64, LSA_ERR_UNSUPPORTED);
  LSA_REQUIRE(((uintptr_t)out_bf16 % 16) == 0, LSA_ERR_ARGUMENT);
  if (rows == 0) return LSA_OK;
  lsa::scan_centre_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, (cudaStream_t)stream>>>(centroids, rows, centre,
                                                                                            out_bf16, lengths, radius);
  LSA_LAUNCH_CHECK();
  return LSA_OK;
}

LSA_API size_t lsa_scan_select_workspace_bytes(int64_t R, int top_p, int64_t m) {
  if (R <= 0 || top_p <= 0 || m < 0) return 0;
  return lsa::scan_workspace(R, top_p, m).total;
}

LSA_API int lsa_scan_select(const float *queries, int64_t R, int d, const float *centroids,
                            const uint16_t *centroids_bf16, const float *lengths, const float *radius, int64_t m,
                            const int32_t *visible,
                            const int32_t *row_top_p, int top_p, int32_t bucket_id_base, int max_visible,
                            int64_t *keys_out, int32_t *picked_out, int32_t *status, void *workspace,
                            size_t workspace_bytes, void *stream) {
  LSA_REQUIRE(queries && centroids && centroids_bf16 && visible && (keys_out || picked_out) && workspace, LSA_ERR_NULL);
  LSA_REQUIRE(!lengths || radius, LSA_ERR_NULL);
  LSA_REQUIRE(R >= 0 && m >= 0 && m < INT32_MAX && top_p >= 1, LSA_ERR_ARGUMENT);
  LSA_REQUIRE(d == 64 && top_p <= 512, LSA_ERR_UNSUPPORTED);
  LSA_REQUIRE(((uintptr_t)queries % 16) == 0 && ((uintptr_t)centroids % 16) == 0 && ((uintptr_t)centroids_bf16 % 16) == 0 &&
                  ((uintptr_t)workspace % 256) == 0,
              LSA_ERR_ARGUMENT);
  if (R == 0) return LSA_OK;
  const lsa::ScanWorkspace w = lsa::scan_workspace(R, top_p, m);
  LSA_REQUIRE(workspace_bytes >= w.total, LSA_ERR_WORKSPACE);
  cudaStream_t s = (cudaStream_t)stream;
  unsigned char *base = reinterpret_cast<unsigned char *>(workspace);
  const int64_t padded = (R + 127) / 128 * 128;
  lsa::ScanParams p = {};
  p.queries_bf16 = reinterpret_cast<uint16_t *>(base + w.q_bf16);
  p.centroids_bf16 = centroids_bf16;
  p.visible = visible;
  p.row_keep = row_top_p;
  int32_t *flags = reinterpret_cast<int32_t *>(base + w.flags);
  p.flags = flags;
  p.norms = reinterpret_cast<float *>(base + w.norms);
  p.lengths = lengths;
  p.radius = radius;
  p.tile_visible = reinterpret_cast<int32_t *>(base + w.tile_visible);
  p.bars = reinterpret_cast<float *>(base + w.thresholds);
  p.counts = reinterpret_cast<int32_t *>(base + w.counts);
  p.survivors = reinterpret_cast<int2 *>(base + w.survivors);
  p.status = status;
  p.R = R, p.m = m;
  p.spans = lsa::scan_spans(padded, m);
  p.cap = lsa::scan_cap(top_p, p.spans);
  p.keep = top_p;
  p.factor = lsa::scan_factor(top_p);
  p.room = lsa::scan_room(top_p);
  const int64_t widest = max_visible > 0 && max_visible < m ? max_visible : m;
  // (an odd stride: buckets come in blocks of a power of two, and every 32nd bucket would be the same bucket of every
  // fourth block - a sample of one kind of bucket, not of the row's scores)
  p.sample_stride = (int)((widest + 511) / 512 > 1 ? ((widest + 511) / 512) | 1 : 1);
  // The threshold is read off 512 samples of a row's scores: where the buckets a row keeps are too small a share of
  // those it sees for a handful of samples to reach it, the threshold would be noise, and every row is scanned exactly.
  const bool sampled = m >= lsa::kScanMinVisible && (int64_t)p.factor * top_p * 512 >= 8 * widest;
  if (!sampled) {
    lsa::FlatParams f = {};
    f.queries = queries, f.centroids = centroids, f.visible = visible, f.row_keep = row_top_p;
    f.keys_out = keys_out, f.ids_out = picked_out;
    f.R = R, f.m = m, f.d = d, f.keep = top_p, f.id_base = bucket_id_base;
    return lsa::launch_flat<64>(f, s);
  }
  int32_t *taken = reinterpret_cast<int32_t *>(base + w.taken);
  int32_t *retry_visible = reinterpret_cast<int32_t *>(base + w.retry_visible);
  lsa::scan_prepare_kernel<<<(unsigned)(padded / 128), 128, 0, s>>>(
      queries, visible, R, m, const_cast<uint16_t *>(p.queries_bf16), const_cast<float *>(p.norms), flags,
      const_cast<int32_t *>(p.tile_visible), top_p, lsa::kScanMinVisible, taken, retry_visible,
      reinterpret_cast<int32_t *>(base + w.retry_keep));
  LSA_LAUNCH_CHECK();
  {
    int rc = lsa::launch_scan_survivors(p, padded, s);
    if (rc != LSA_OK) return rc;
    const int room = p.room;
    const size_t smem = (size_t)lsa::kSelWarps * ((size_t)room * 8 + lsa::kHistBins * 4);
    LSA_REQUIRE(smem <= 200 * 1024, LSA_ERR_UNSUPPORTED);
    if (cudaFuncSetAttribute(lsa::scan_pick_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return LSA_ERR_LAUNCH;
    lsa::scan_pick_kernel<<<(unsigned)((R + lsa::kSelWarps - 1) / lsa::kSelWarps), lsa::kSelThreads, smem, s>>>(
        p, queries, centroids, flags, bucket_id_base, room, keys_out, picked_out);
    LSA_LAUNCH_CHECK();
    // The rows the pick could not prove (a handful in a thousand): side by side, an exact scan with each row's
    // buckets split over CTAs, and back.
    float *retry_q = reinterpret_cast<float *>(base + w.retry_q);
    int32_t *retry_keep = reinterpret_cast<int32_t *>(base + w.retry_keep);
    int32_t *retry_row = reinterpret_cast<int32_t *>(base + w.retry_row);
    int64_t *retry_parts = reinterpret_cast<int64_t *>(base + w.retry_parts);
    int64_t *retry_keys = reinterpret_cast<int64_t *>(base + w.retry_keys);
    lsa::scan_collect_kernel<<<(unsigned)((R + 255) / 256), 256, 0, s>>>(queries, visible, row_top_p, top_p, R, m, flags,
                                                                        taken, retry_q, retry_visible, retry_keep,
                                                                        retry_row);
    LSA_LAUNCH_CHECK();
    lsa::SelectParams sel = {};
    sel.queries = retry_q;
    sel.vectors = centroids;
    sel.run_end = retry_visible;
    sel.row_keep = retry_keep;
    sel.keys_out = retry_parts;
    sel.R = lsa::kScanRetry;
    sel.N = INT64_MAX;
    sel.d = 64;
    sel.keep = top_p;
    sel.id_base = bucket_id_base;
    sel.run_limit = INT32_MAX;
    rc = lsa::launch_select<1>(sel, lsa::kScanRetrySplits, s);
    if (rc != LSA_OK) return rc;
    rc = lsa_merge_candidates(retry_parts, lsa::kScanRetrySplits, lsa::kScanRetry, top_p, retry_keys, nullptr, stream);
    if (rc != LSA_OK) return rc;
    lsa::scan_scatter_kernel<<<lsa::kScanRetry, 128, 0, s>>>(retry_keys, retry_row, retry_keep, taken, top_p, keys_out,
                                                             picked_out);
    LSA_LAUNCH_CHECK();
  }
  // the plain exact scan of the rows that are still flagged: too few visible buckets, or more unproven rows than
  // the split scan takes
  lsa::FlatParams f = {};
  f.queries = queries;
  f.centroids = centroids;
  f.visible = visible;
  f.row_keep = row_top_p;
  f.row_flags = flags;
  f.keys_out = keys_out;
  f.ids_out = picked_out;
  f.R = R;
  f.m = m;
  f.d = d;
  f.keep = top_p;
  f.id_base = bucket_id_base;
  return lsa::launch_flat<64>(f, s);
}

// ------------------------------------------------------------------------------------------------ dense scores

namespace lsa {

// Every (row, bucket) score written out, each at its own column: the two-pass selection of the reference scores
// first and picks after, and code written against that form asks for the matrix. 8 rows a CTA share a bucket's
// centroid; a thread a bucket, the dot added in ascending dim order.
__global__ void __launch_bounds__(256)
    dense_scores_kernel(const float *__restrict__ queries, const float *__restrict__ centroids,
                        const int32_t *__restrict__ pages, int max_pages, int page_rows,
                        const int32_t *__restrict__ counts, int64_t R, int d, int64_t width, int id_base,
                        float *__restrict__ scores_out, int64_t *__restrict__ keys_out) {
  extern __shared__ __align__(16) float q_s[];  // [8][d]
  const int64_t row0 = (int64_t)blockIdx.y * 8;
  for (int e = threadIdx.x; e < 8 * d; e += blockDim.x) {
    const int64_t r = row0 + e / d;
    q_s[e] = r < R ? queries[r * d + e % d] : 0.0f;
  }
  __syncthreads();
  const int64_t col = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= width) return;
  for (int i = 0; i < 8 && row0 + i < R; ++i) {
    const int64_t r = row0 + i;
    int64_t at = col;
    bool held = col < counts[r];
    if (held && pages) {
      const int page = pages[r * max_pages + col / page_rows];
      held = page >= 0;
      at = (int64_t)page * page_rows + col % page_rows;
    }
    float acc = 0.0f;
    if (held) {
      const float4 *c4 = reinterpret_cast<const float4 *>(centroids + at * d);
      const float *q = q_s + i * d;
      for (int k4 = 0; k4 < d / 4; ++k4) {
        const float4 v = __ldg(c4 + k4);
        acc = fmaf(q[4 * k4], v.x, acc), acc = fmaf(q[4 * k4 + 1], v.y, acc);
        acc = fmaf(q[4 * k4 + 2], v.z, acc), acc = fmaf(q[4 * k4 + 3], v.w, acc);
      }
    }
    if (scores_out) scores_out[r * width + col] = held ? acc : -INFINITY;
    if (keys_out) keys_out[r * width + col] = held ? pack_key(acc, (int32_t)col + id_base) : kEmptyKey;
  }
}

}  // namespace lsa

LSA_API int lsa_dense_scores(const float *queries, int64_t R, int d, const float *centroids, const int32_t *pages,
                             int max_pages, int page_rows, const int32_t *counts, int64_t width,
                             int32_t bucket_id_base, float *scores_out, int64_t *keys_out, void *stream) {
  LSA_REQUIRE(queries && centroids && counts && (scores_out || keys_out), LSA_ERR_NULL);
  LSA_REQUIRE(R >= 0 && width >= 0 && width < INT32_MAX && d >= 4 && d % 4 == 0 && d <= 1024, LSA_ERR_ARGUMENT);
  LSA_REQUIRE(!pages || (max_pages >= 1 && page_rows >= 1), LSA_ERR_ARGUMENT);
  LSA_REQUIRE(((uintptr_t)centroids % 16) == 0, LSA_ERR_ARGUMENT);
  if (R == 0 || width == 0) return LSA_OK;
  const dim3 grid((unsigned)((width + 255) / 256), (unsigned)((R + 7) / 8));
  LSA_REQUIRE(grid.y <= 65535, LSA_ERR_UNSUPPORTED);
  lsa::dense_scores_kernel<<<grid, 256, (size_t)8 * d * 4, (cudaStream_t)stream>>>(
      queries, centroids, pages, max_pages, page_rows, counts, R, d, width, bucket_id_base, scores_out, keys_out);
  LSA_LAUNCH_CHECK();
  return LSA_OK;
}

LSA_API int lsa_flat_select(const float *queries, int64_t R, int d, const float *centroids, int64_t m,
                            const int32_t *visible, const int32_t *row_top_p, int top_p, int32_t bucket_id_base,
                            int64_t *keys_out, int32_t *picked_out, void *stream) {
  LSA_REQUIRE(queries && centroids && visible && (keys_out || picked_out), LSA_ERR_NULL);
  LSA_REQUIRE(R >= 0 && d >= 4 && d % 4 == 0 && m >= 0 && top_p >= 1 && m < INT32_MAX, LSA_ERR_ARGUMENT);
  if (R == 0) return LSA_OK;
  if ((d == 64 || d == 32) && top_p <= 512) {
    lsa::FlatParams f = {};
    f.queries = queries;
    f.centroids = centroids;
    f.visible = visible;
    f.row_keep = row_top_p;
    f.keys_out = keys_out;
    f.ids_out = picked_out;
    f.R = R;
    f.m = m;
    f.d = d;
    f.keep = top_p;
    f.id_base = bucket_id_base;
    return d == 64 ? lsa::launch_flat<64>(f, (cudaStream_t)stream) : lsa::launch_flat<32>(f, (cudaStream_t)stream);
  }
  lsa::SelectParams p = {};
  p.queries = queries;
  p.vectors = centroids;
  p.run_end = visible;
  p.row_keep = row_top_p;
  p.keys_out = keys_out;
  p.ids_out = picked_out;
  p.R = R;
  p.N = m;
  p.d = d;
  p.keep = top_p;
  p.id_base = bucket_id_base;
  p.run_limit = (int)m;
  return lsa::launch_select<8>(p, 1, (cudaStream_t)stream);
}

// ------------------------------------------------------------------------------------------------ shaped buckets

namespace lsa {
static bool shape_table(ShapeTable *t, const uint8_t *basis, const float *variances, const float *floors, int rank,
                        float deviations, int d) {
  if (!floors || rank < 0 || rank > d || d % 32 != 0) return false;
  if (rank > 0 && (!basis || !variances || ((uintptr_t)basis % 4) != 0)) return false;
  t->basis = reinterpret_cast<const uint32_t *>(basis);
  t->variances = variances;
  t->floors = floors;
  t->rank = rank;
  t->deviations = deviations;
  t->scale = 1.0f / sqrtf((float)d);
  return true;
}
}  // namespace lsa

LSA_API int lsa_shaped_select(const float *queries, int64_t R, int d, const float *centroids, int64_t m,
                              const uint8_t *basis, const float *variances, const float *floors, int rank,
                              float deviations, const int32_t *visible, const int32_t *row_top_p, int top_p,
                              int32_t bucket_id_base, int64_t *keys_out, int32_t *picked_out, void *stream) {
  LSA_REQUIRE(queries && centroids && visible && (keys_out || picked_out), LSA_ERR_NULL);
  LSA_REQUIRE(R >= 0 && m >= 0 && top_p >= 1 && m < INT32_MAX, LSA_ERR_ARGUMENT);
  lsa::ShapeTable table;
  LSA_REQUIRE(lsa::shape_table(&table, basis, variances, floors, rank, deviations, d), LSA_ERR_ARGUMENT);
  if (R == 0) return LSA_OK;
  if ((d == 64 || d == 32) && top_p <= 512) {
    lsa::FlatParams f = {};
    f.queries = queries, f.centroids = centroids, f.visible = visible, f.row_keep = row_top_p;
    f.keys_out = keys_out, f.ids_out = picked_out;
    f.R = R, f.m = m, f.d = d, f.keep = top_p, f.id_base = bucket_id_base;
    f.shape = table;
    return d == 64 ? lsa::launch_flat<64>(f, (cudaStream_t)stream) : lsa::launch_flat<32>(f, (cudaStream_t)stream);
  }
  lsa::SelectParams p = {};
  p.queries = queries, p.vectors = centroids, p.run_end = visible, p.row_keep = row_top_p;
  p.keys_out = keys_out, p.ids_out = picked_out;
  p.R = R, p.N = m, p.d = d, p.keep = top_p, p.id_base = bucket_id_base, p.run_limit = (int)m;
  p.shape = table;
  return lsa::launch_select<8>(p, 1, (cudaStream_t)stream);
}

LSA_API size_t lsa_flat_select_decode_workspace_bytes(int64_t R, int top_p, int splits) {
  if (R <= 0 || top_p <= 0 || splits <= 1) return 0;
  return (size_t)R * top_p * splits * sizeof(int64_t);
}

namespace lsa {
// The global top_p of `parts` lists a row; `sorted`: every list arrives best first with its empty keys last (the
// lists this file's own scans write).
static int merge_lists(const int64_t *keys_in, int parts, int64_t R, int top_p, int64_t *keys_out, int32_t *picked_out,
                       const int64_t *children, int fanout, int32_t *carried_out, bool sorted, cudaStream_t stream) {
  // (the lists folded in registers pass through kSelWarps / 2 slots of 128 keys, whatever they hold themselves)
  const int room = max(pow2_at_least(parts * top_p), kSelWarps / 2 * kTopWarp);
  const size_t smem = (size_t)room * 8 + kHistBins * 4;
  LSA_REQUIRE(smem <= 200 * 1024, LSA_ERR_UNSUPPORTED);
  if (cudaFuncSetAttribute(merge_candidates_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
      cudaSuccess)
    return LSA_ERR_LAUNCH;
  launch(R <= kChainedRows, merge_candidates_kernel, dim3((unsigned)R), dim3(merge_threads(parts, top_p)), smem, stream,
         keys_in, parts, R, top_p, room, keys_out, picked_out, children, fanout, carried_out, sorted ? 1 : 0);
  LSA_LAUNCH_CHECK();
  return LSA_OK;
}
}  // namespace lsa

LSA_API int lsa_merge_candidates(const int64_t *keys_in, int parts, int64_t R, int top_p, int64_t *keys_out,
                                 int32_t *picked_out, void *stream) {
  LSA_REQUIRE(keys_in && (keys_out || picked_out), LSA_ERR_NULL);
  LSA_REQUIRE(parts >= 1 && R >= 0 && top_p >= 1, LSA_ERR_ARGUMENT);
  if (R == 0) return LSA_OK;
  return lsa::merge_lists(keys_in, parts, R, top_p, keys_out, picked_out, nullptr, 0, nullptr, false,
                          (cudaStream_t)stream);
}

LSA_API int lsa_flat_select_decode(const float *queries, int64_t R, int d, const float *centroids,
                                   const int64_t *request_first, const int32_t *visible, int top_p, int splits,
                                   int64_t *keys_out, int32_t *picked_out, void *workspace, size_t workspace_bytes,
                                   void *stream) {
  LSA_REQUIRE(queries && centroids && visible && keys_out, LSA_ERR_NULL);
  LSA_REQUIRE(R >= 0 && d >= 4 && d % 4 == 0 && top_p >= 1 && splits >= 1 && splits <= 1024, LSA_ERR_ARGUMENT);
  if (R == 0) return LSA_OK;
  if (splits > 1) {
    LSA_REQUIRE(workspace, LSA_ERR_NULL);
    LSA_REQUIRE(workspace_bytes >= lsa_flat_select_decode_workspace_bytes(R, top_p, splits), LSA_ERR_WORKSPACE);
  }
  lsa::SelectParams p = {};
  p.queries = queries;
  p.vectors = centroids;
  p.vector_base = request_first;
  p.run_end = visible;
  p.R = R;
  p.N = INT64_MAX;
  p.d = d;
  p.keep = top_p;
  p.run_limit = INT32_MAX;
  if (splits == 1) {
    p.keys_out = keys_out;
    p.ids_out = picked_out;
    return lsa::launch_select<1>(p, 1, (cudaStream_t)stream);
  }
  p.keys_out = (int64_t *)workspace;
  int rc = lsa::launch_select<1>(p, splits, (cudaStream_t)stream);
  if (rc != LSA_OK) return rc;
  return lsa::merge_lists((const int64_t *)workspace, splits, R, top_p, keys_out, picked_out, nullptr, 0, nullptr, true,
                          (cudaStream_t)stream);
}

LSA_API int lsa_shaped_select_decode(const float *queries, int64_t R, int d, const float *centroids,
                                     const uint8_t *basis, const float *variances, const float *floors, int rank,
                                     float deviations, const int64_t *request_first, const int32_t *visible,
                                     int top_p, int splits, int64_t *keys_out, int32_t *picked_out, void *workspace,
                                     size_t workspace_bytes, void *stream) {
  LSA_REQUIRE(queries && centroids && visible && keys_out, LSA_ERR_NULL);
  LSA_REQUIRE(R >= 0 && top_p >= 1 && splits >= 1 && splits <= 1024, LSA_ERR_ARGUMENT);
  lsa::ShapeTable table;
  LSA_REQUIRE(lsa::shape_table(&table, basis, variances, floors, rank, deviations, d), LSA_ERR_ARGUMENT);
  if (R == 0) return LSA_OK;
  if (splits > 1) {
    LSA_REQUIRE(workspace, LSA_ERR_NULL);
    LSA_REQUIRE(workspace_bytes >= lsa_flat_select_decode_workspace_bytes(R, top_p, splits), LSA_ERR_WORKSPACE);
  }
  lsa::SelectParams p = {};
  p.queries = queries, p.vectors = centroids, p.vector_base = request_first, p.run_end = visible;
  p.R = R, p.N = INT64_MAX, p.d = d, p.keep = top_p, p.run_limit = INT32_MAX;
  p.shape = table;
  if (splits == 1) {
    p.keys_out = keys_out, p.ids_out = picked_out;
    return lsa::launch_select<1>(p, 1, (cudaStream_t)stream);
  }
  p.keys_out = (int64_t *)workspace;
  int rc = lsa::launch_select<1>(p, splits, (cudaStream_t)stream);
  if (rc != LSA_OK) return rc;
  return lsa::merge_lists((const int64_t *)workspace, splits, R, top_p, keys_out, picked_out, nullptr, 0, nullptr, true,
                          (cudaStream_t)stream);
}

LSA_API int lsa_beam_step(const float *queries, int64_t R, int d, const float *vectors, int64_t N,
                          const int32_t *carried, int n_carried, const int32_t *open_first,
                          const int32_t *open_end, int keep, const int64_t *children, int fanout,
                          int32_t *kept_out, int64_t *keys_out, int32_t *carried_out, void *stream) {
  LSA_REQUIRE(queries && vectors, LSA_ERR_NULL);
  LSA_REQUIRE(R >= 0 && d >= 4 && d % 4 == 0 && N >= 0 && N < INT32_MAX && keep >= 1 && n_carried >= 0,
              LSA_ERR_ARGUMENT);
  LSA_REQUIRE(n_carried == 0 || carried, LSA_ERR_NULL);
  LSA_REQUIRE((children != nullptr) == (carried_out != nullptr), LSA_ERR_ARGUMENT);
  LSA_REQUIRE(!children || fanout >= 1, LSA_ERR_ARGUMENT);
  LSA_REQUIRE(kept_out || keys_out || carried_out, LSA_ERR_NULL);
  if (R == 0) return LSA_OK;
  lsa::SelectParams p = {};
  p.queries = queries;
  p.vectors = vectors;
  p.run_first = open_first;
  p.run_end = open_end;
  p.carried = carried;
  p.children = children;
  p.keys_out = keys_out;
  p.ids_out = kept_out;
  p.carried_out = carried_out;
  p.R = R;
  p.N = N;
  p.d = d;
  p.n_carried = n_carried;
  p.keep = keep;
  p.fanout = fanout;
  p.run_limit = (int)N;
  return lsa::launch_select<1>(p, 1, (cudaStream_t)stream);
}

LSA_API int lsa_flat_select_paged(const float *queries, int64_t R, int d, const float *centroids, int64_t rows,
                                  const int32_t *pages, int max_pages, int page_rows, const int32_t *counts,
                                  int top_p, int splits, int64_t *keys_out, int32_t *picked_out, void *workspace,
                                  size_t workspace_bytes, void *stream) {
  LSA_REQUIRE(queries && centroids && pages && counts && keys_out, LSA_ERR_NULL);
  LSA_REQUIRE(R >= 0 && d >= 4 && d % 4 == 0 && rows >= 0 && max_pages >= 1 && page_rows >= 1 && top_p >= 1 &&
                  splits >= 1 && splits <= 1024,
              LSA_ERR_ARGUMENT);
  if (R == 0) return LSA_OK;
  if (splits > 1) {
    LSA_REQUIRE(workspace, LSA_ERR_NULL);
    LSA_REQUIRE(workspace_bytes >= lsa_flat_select_decode_workspace_bytes(R, top_p, splits), LSA_ERR_WORKSPACE);
  }
  lsa::SelectParams p = {};
  p.queries = queries;
  p.vectors = centroids;
  p.run_end = counts;
  p.pages = pages;
  p.max_pages = max_pages;
  p.page_rows = page_rows;
  p.R = R;
  p.N = rows;
  p.d = d;
  p.keep = top_p;
  p.run_limit = INT32_MAX;
  if (splits == 1) {
    p.keys_out = keys_out;
    p.ids_out = picked_out;
    return lsa::launch_select<1>(p, 1, (cudaStream_t)stream);
  }
  p.keys_out = (int64_t *)workspace;
  int rc = lsa::launch_select<1>(p, splits, (cudaStream_t)stream);
  if (rc != LSA_OK) return rc;
  return lsa::merge_lists((const int64_t *)workspace, splits, R, top_p, keys_out, picked_out, nullptr, 0, nullptr, true,
                          (cudaStream_t)stream);
}

LSA_API int lsa_shaped_select_paged(const float *queries, int64_t R, int d, const float *centroids, int64_t rows,
                                    const uint8_t *basis, const float *variances, const float *floors, int rank,
                                    float deviations, const int32_t *pages, int max_pages, int page_rows,
                                    const int32_t *counts, int top_p, int splits, int64_t *keys_out,
                                    int32_t *picked_out, void *workspace, size_t workspace_bytes, void *stream) {
  LSA_REQUIRE(queries && centroids && pages && counts && keys_out, LSA_ERR_NULL);
  LSA_REQUIRE(R >= 0 && rows >= 0 && max_pages >= 1 && page_rows >= 1 && top_p >= 1 && splits >= 1 && splits <= 1024,
              LSA_ERR_ARGUMENT);
  lsa::ShapeTable table;
  LSA_REQUIRE(lsa::shape_table(&table, basis, variances, floors, rank, deviations, d), LSA_ERR_ARGUMENT);
  if (R == 0) return LSA_OK;
  if (splits > 1) {
    LSA_REQUIRE(workspace, LSA_ERR_NULL);
    LSA_REQUIRE(workspace_bytes >= lsa_flat_select_decode_workspace_bytes(R, top_p, splits), LSA_ERR_WORKSPACE);
  }
  lsa::SelectParams p = {};
  p.queries = queries, p.vectors = centroids, p.run_end = counts;
  p.pages = pages, p.max_pages = max_pages, p.page_rows = page_rows;
  p.R = R, p.N = rows, p.d = d, p.keep = top_p, p.run_limit = INT32_MAX;
  p.shape = table;
  if (splits == 1) {
    p.keys_out = keys_out, p.ids_out = picked_out;
    return lsa::launch_select<1>(p, 1, (cudaStream_t)stream);
  }
  p.keys_out = (int64_t *)workspace;
  int rc = lsa::launch_select<1>(p, splits, (cudaStream_t)stream);
  if (rc != LSA_OK) return rc;
  return lsa::merge_lists((const int64_t *)workspace, splits, R, top_p, keys_out, picked_out, nullptr, 0, nullptr, true,
                          (cudaStream_t)stream);
}

LSA_API size_t lsa_beam_step_workspace_bytes(int64_t R, int keep, int splits) {
  return lsa_flat_select_decode_workspace_bytes(R, keep, splits);
}

LSA_API int lsa_beam_step_split(const float *queries, int64_t R, int d, const float *vectors, int64_t N,
                                const int32_t *carried, int n_carried, const int32_t *open_first,
                                const int32_t *open_end, int keep, const int64_t *children, int fanout, int splits,
                                int32_t *kept_out, int64_t *keys_out, int32_t *carried_out, void *workspace,
                                size_t workspace_bytes, void *stream) {
  if (splits <= 1)
    return lsa_beam_step(queries, R, d, vectors, N, carried, n_carried, open_first, open_end, keep, children, fanout,
                         kept_out, keys_out, carried_out, stream);
  LSA_REQUIRE(queries && vectors && workspace, LSA_ERR_NULL);
  LSA_REQUIRE(R >= 0 && d >= 4 && d % 4 == 0 && N >= 0 && N < INT32_MAX && keep >= 1 && n_carried >= 0 &&
                  splits <= 1024,
              LSA_ERR_ARGUMENT);
  LSA_REQUIRE(n_carried == 0 || carried, LSA_ERR_NULL);
  LSA_REQUIRE((children != nullptr) == (carried_out != nullptr), LSA_ERR_ARGUMENT);
  LSA_REQUIRE(!children || fanout >= 1, LSA_ERR_ARGUMENT);
  LSA_REQUIRE(kept_out || keys_out || carried_out, LSA_ERR_NULL);
  LSA_REQUIRE(workspace_bytes >= lsa_beam_step_workspace_bytes(R, keep, splits), LSA_ERR_WORKSPACE);
  if (R == 0) return LSA_OK;
  lsa::SelectParams p = {};
  p.queries = queries;
  p.vectors = vectors;
  p.run_first = open_first;
  p.run_end = open_end;
  p.carried = carried;
  p.keys_out = (int64_t *)workspace;
  p.R = R;
  p.N = N;
  p.d = d;
  p.n_carried = n_carried;
  p.keep = keep;
  p.run_limit = (int)N;
  int rc = lsa::launch_select<1>(p, splits, (cudaStream_t)stream);
  if (rc != LSA_OK) return rc;
  return lsa::merge_lists((const int64_t *)workspace, splits, R, keep, keys_out, kept_out, children, fanout, carried_out,
                          true, (cudaStream_t)stream);
}
