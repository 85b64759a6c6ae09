// Expansion: a row's picked buckets become its read list - members best bucket first, then the window, then
// the sinks. Pure integer work, one warp a row, ballot-compacted so the order is the table's order.
#include <cooperative_groups.h>

#include "common.cuh"

namespace lsa {

constexpr int kExpandWarps = 8;

struct ExpandParams {
  const int32_t *picked;      // [R, top_p]
  const int64_t *positions;   // [R]
  const int32_t *members;     // [m, cap]
  const int32_t *row_top_p;   // [R] or NULL
  const int32_t *row_top_k;   // [R] or NULL
  const int32_t *page_table;  // [pages] (or [requests, pages] with page_table_stride) or NULL
  const int32_t *row_request;   // [R] request of each row, or NULL for request 0
  const int32_t *bucket_pages;  // [requests, bucket_max_pages] page of every bucket_page_rows logical buckets, or NULL
  int64_t page_table_stride, bucket_pages_stride;
  int bucket_page_rows, bucket_max_pages;
  int32_t *selected;          // [R, width]
  int32_t *lengths;           // [R]
  int32_t *status;
  int64_t R, m, owner_first, owner_end;
  int top_p, cap, top_k, sink, window, page_size, width, granule, world, rank, flags;
};

// Whether this caller keeps an id: inside its contiguous range and, when the cache is dealt out in granules of
// positions round-robin over `world` ranks, in one of its granules.
__device__ __forceinline__ bool owned(const ExpandParams &p, int64_t id) {
  if (id < p.owner_first || id >= p.owner_end) return false;
  if (p.world <= 1) return true;
  const uint32_t u = (uint32_t)id;  // (an id fits 31 bits - the lists are int32 - and 32-bit division is the cheap one)
  return (int)((u / (uint32_t)p.granule) % (uint32_t)p.world) == p.rank;
}

// What is written for an id: the position, its row in the rank's own cache when granules are dealt out, or its KV
// slot through the page table.
__device__ __forceinline__ int32_t stored_id(const ExpandParams &p, const int32_t *table, int64_t id) {
  uint32_t u = (uint32_t)id;
  if (p.world > 1) u = u / ((uint32_t)p.granule * (uint32_t)p.world) * (uint32_t)p.granule + u % (uint32_t)p.granule;
  if (!table) return (int32_t)u;
  return table[u / (uint32_t)p.page_size] * p.page_size + (int32_t)(u % (uint32_t)p.page_size);
}

// Append the owned ids of [first, end) to out[written..], in order; returns the new count.
__device__ __forceinline__ int append_run(const ExpandParams &p, const int32_t *table, int32_t *out, int written,
                                          int64_t first, int64_t end, int lane) {
  const unsigned below = (1u << lane) - 1;
  for (int64_t base = first; base < end; base += 32) {
    const int64_t t = base + lane;
    const bool mine = t < end && owned(p, t);
    const unsigned keeps = __ballot_sync(0xffffffffu, mine);
    if (mine) out[written + __popc(keeps & below)] = stored_id(p, table, t);
    written += __popc(keeps);
  }
  return written;
}

__global__ void __launch_bounds__(kExpandWarps * 32) expand_kernel(ExpandParams p) {
  const int lane = lane_id();
  const int64_t r = (int64_t)blockIdx.x * kExpandWarps + (threadIdx.x >> 5);
  dependents_may_launch();
  wait_for_earlier_grids();
  if (r >= p.R) return;
  const int64_t pos = p.positions[r];
  const int64_t request = p.row_request ? p.row_request[r] : 0;
  const int32_t *table = p.page_table ? p.page_table + request * p.page_table_stride : nullptr;
  const int row_p = p.row_top_p ? min(p.row_top_p[r], p.top_p) : p.top_p;
  const int row_k = p.row_top_k ? min(p.row_top_k[r], p.top_k) : p.top_k;
  const int64_t window_start = max((int64_t)0, pos + 1 - p.window);
  int32_t *out = p.selected + r * p.width;
  const unsigned below = (1u << lane) - 1;
  int counted = 0;  // ids that count toward top_k
  int written = 0;  // ids this owner keeps
  int bad = 0;
  // The picks are read 32 at a time, a lane a pick (so no load waits on the one before), and a bucket's member
  // chunks four at a time: the loads of a group are in flight together, only the counting is in order. A bucket's
  // members ascend and its row ends in padding, so the first chunk that holds padding or a member inside the window
  // is the last one of the bucket that can count: the rest of its row (half of it, on average) is never read.
  for (int i0 = 0; i0 < row_p && counted < row_k; i0 += 32) {
    int64_t my_bucket = -1;
    if (i0 + lane < row_p) {
      my_bucket = p.picked[r * p.top_p + i0 + lane];
      if (my_bucket >= 0 && p.bucket_pages) {
        // a request's logical bucket sits at row bucket % rows of its page bucket / rows
        const int64_t slot = my_bucket / p.bucket_page_rows;
        const int page = slot < p.bucket_max_pages ? p.bucket_pages[request * p.bucket_pages_stride + slot] : -1;
        my_bucket = page >= 0 ? (int64_t)page * p.bucket_page_rows + my_bucket % p.bucket_page_rows : p.m;
      }
      if (my_bucket >= p.m) {
        my_bucket = -1;
        ++bad;
      }
    }
    const int picks = min(32, row_p - i0);
    for (int pick = 0; pick < picks && counted < row_k; ++pick) {
      const int64_t bucket = __shfl_sync(0xffffffffu, my_bucket, pick);
      if (bucket < 0) continue;
      const int32_t *row = p.members + bucket * p.cap;
      bool ended = false;
      for (int at0 = 0; at0 < p.cap && !ended && counted < row_k; at0 += 128) {
        int32_t ids[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int at = at0 + 32 * j + lane;
          ids[j] = at < p.cap ? row[at] : LSA_PAD;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int32_t id = ids[j];
          const bool counts = id >= p.sink && id < window_start;
          const unsigned votes = __ballot_sync(0xffffffffu, counts);
          const bool inside = counts && counted + __popc(votes & below) < row_k;
          const bool mine = inside && owned(p, id);
          const unsigned keeps = __ballot_sync(0xffffffffu, mine);
          if (mine) out[written + __popc(keeps & below)] = stored_id(p, table, id);
          written += __popc(keeps);
          counted += __popc(votes);
          ended |= __any_sync(0xffffffffu, id < 0 || id >= window_start);
        }
      }
    }
  }
  bad = warp_sum_int(bad);
  // The window, ascending, then the sinks.
  if (!(p.flags & LSA_EXPAND_NO_LOCAL)) {
    written = append_run(p, table, out, written, window_start, pos + 1, lane);
    written = append_run(p, table, out, written, 0, min((int64_t)p.sink, min(window_start, pos + 1)), lane);
  }
  if (!(p.flags & LSA_EXPAND_NO_PAD))
    for (int j = written + lane; j < p.width; j += 32) out[j] = LSA_PAD;
  if (lane == 0) {
    p.lengths[r] = written;
    if (bad && p.status) atomicAdd(p.status, bad);
  }
}

// A few rows with long lists (a decode step): a whole CTA a row. The warps count every pick's ids at once, one warp
// scans the counts into write offsets, and the warps write their picks' ids in place - the list is the same as the
// one-warp kernel's, id for id. Only for callers that keep every id (no owner range, no dealt granules), so the ids
// that count toward top_k are the ids written.
constexpr int kWideThreads = 1024;
constexpr int kWideMaxPicks = 1024;

__global__ void __launch_bounds__(kWideThreads) expand_wide_kernel(ExpandParams p) {
  __shared__ int64_t bucket_s[kWideMaxPicks];
  __shared__ int count_s[kWideMaxPicks];
  __shared__ int start_s[kWideMaxPicks + 1];
  __shared__ int bad_s;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr int kWarps = kWideThreads / 32;
  const int64_t r = blockIdx.x;
  dependents_may_launch();
  wait_for_earlier_grids();
  const int64_t pos = p.positions[r];
  const int64_t request = p.row_request ? p.row_request[r] : 0;
  const int32_t *table = p.page_table ? p.page_table + request * p.page_table_stride : nullptr;
  const int row_p = p.row_top_p ? min(p.row_top_p[r], p.top_p) : p.top_p;
  const int row_k = p.row_top_k ? min(p.row_top_k[r], p.top_k) : p.top_k;
  const int64_t window_start = max((int64_t)0, pos + 1 - p.window);
  int32_t *out = p.selected + r * p.width;
  const unsigned below = (1u << lane) - 1;
  if (tid == 0) bad_s = 0;
  __syncthreads();
  for (int i = tid; i < row_p; i += kWideThreads) {
    int64_t bucket = p.picked[r * p.top_p + i];
    if (bucket >= 0 && p.bucket_pages) {
      const int64_t slot = bucket / p.bucket_page_rows;
      const int page = slot < p.bucket_max_pages ? p.bucket_pages[request * p.bucket_pages_stride + slot] : -1;
      bucket = page >= 0 ? (int64_t)page * p.bucket_page_rows + bucket % p.bucket_page_rows : p.m;
    }
    if (bucket >= p.m) {
      bucket = -1;
      atomicAdd(&bad_s, 1);
    }
    bucket_s[i] = bucket;
  }
  __syncthreads();
  for (int pick = warp; pick < row_p; pick += kWarps) {
    const int64_t bucket = bucket_s[pick];
    int n = 0;
    if (bucket >= 0)
      for (int at0 = 0; at0 < p.cap; at0 += 128) {  // four loads in flight
        int32_t ids[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int at = at0 + 32 * j + lane;
          ids[j] = at < p.cap ? p.members[bucket * p.cap + at] : LSA_PAD;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) n += __popc(__ballot_sync(0xffffffffu, ids[j] >= p.sink && ids[j] < window_start));
      }
    if (lane == 0) count_s[pick] = n;
  }
  __syncthreads();
  if (warp == 0) {
    int carry = 0;
    for (int base = 0; base < row_p; base += 32) {
      const int v = base + lane < row_p ? count_s[base + lane] : 0;
      int incl = v;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
      }
      if (base + lane < row_p) start_s[base + lane] = carry + incl - v;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) start_s[row_p] = carry;
  }
  __syncthreads();
  for (int pick = warp; pick < row_p; pick += kWarps) {
    const int64_t bucket = bucket_s[pick];
    int written = start_s[pick];
    if (bucket < 0) continue;
    for (int at0 = 0; at0 < p.cap && written < row_k; at0 += 128) {
      int32_t ids[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int at = at0 + 32 * j + lane;
        ids[j] = at < p.cap ? p.members[bucket * p.cap + at] : LSA_PAD;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const bool counts = ids[j] >= p.sink && ids[j] < window_start;
        const unsigned votes = __ballot_sync(0xffffffffu, counts);
        const int at = written + __popc(votes & below);
        if (counts && at < row_k) out[at] = stored_id(p, table, ids[j]);
        written += __popc(votes);
      }
    }
  }
  int total = min(start_s[row_p], row_k);
  if (!(p.flags & LSA_EXPAND_NO_LOCAL)) {
    const int in_window = (int)(pos + 1 - window_start);
    for (int i = tid; i < in_window; i += kWideThreads) out[total + i] = stored_id(p, table, window_start + i);
    total += in_window;
    const int sinks = (int)min((int64_t)p.sink, min(window_start, pos + 1));
    for (int i = tid; i < sinks; i += kWideThreads) out[total + i] = stored_id(p, table, i);
    total += sinks;
  }
  if (!(p.flags & LSA_EXPAND_NO_PAD))
    for (int j = total + tid; j < p.width; j += kWideThreads) out[j] = LSA_PAD;
  if (tid == 0) {
    p.lengths[r] = total;
    if (bad_s && p.status) atomicAdd(p.status, bad_s);
  }
}

// The same list from a CLUSTER of eight CTAs a row: a decode row of a long context lists hundreds of kilobytes of ids,
// more than one SM moves in the time the rest of the step takes. Each CTA counts and writes an eighth of the picks;
// the CTAs' totals cross through distributed shared memory, which is all the exchange a prefix sum over picks needs.
constexpr int kClusterCtas = 8;
constexpr int kClusterThreads = 512;

__global__ void __cluster_dims__(kClusterCtas, 1, 1) __launch_bounds__(kClusterThreads, 1)
    expand_cluster_kernel(ExpandParams p) {
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  constexpr int kMine = kWideMaxPicks / kClusterCtas;  // picks a CTA takes, at most
  __shared__ int64_t bucket_s[kMine];
  __shared__ int count_s[kMine];
  __shared__ int start_s[kMine];
  __shared__ int total_s, bad_s;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr int kWarps = kClusterThreads / 32;
  const int cta = (int)cluster.block_rank();
  const int64_t r = blockIdx.y;
  dependents_may_launch();
  wait_for_earlier_grids();
  const int64_t pos = p.positions[r];
  const int64_t request = p.row_request ? p.row_request[r] : 0;
  const int32_t *table = p.page_table ? p.page_table + request * p.page_table_stride : nullptr;
  const int row_p = p.row_top_p ? min(p.row_top_p[r], p.top_p) : p.top_p;
  const int row_k = p.row_top_k ? min(p.row_top_k[r], p.top_k) : p.top_k;
  const int64_t window_start = max((int64_t)0, pos + 1 - p.window);
  int32_t *out = p.selected + r * p.width;
  const unsigned below = (1u << lane) - 1;
  const int share = (row_p + kClusterCtas - 1) / kClusterCtas;
  const int first_pick = cta * share;
  const int picks = max(0, min(share, row_p - first_pick));
  if (tid == 0) bad_s = 0;
  __syncthreads();
  for (int i = tid; i < picks; i += kClusterThreads) {
    int64_t bucket = p.picked[r * p.top_p + first_pick + i];
    if (bucket >= 0 && p.bucket_pages) {
      const int64_t slot = bucket / p.bucket_page_rows;
      const int page = slot < p.bucket_max_pages ? p.bucket_pages[request * p.bucket_pages_stride + slot] : -1;
      bucket = page >= 0 ? (int64_t)page * p.bucket_page_rows + bucket % p.bucket_page_rows : p.m;
    }
    if (bucket >= p.m) {
      bucket = -1;
      atomicAdd(&bad_s, 1);
    }
    bucket_s[i] = bucket;
  }
  __syncthreads();
  // A warp's first pick stays in its registers between the count and the write (a row of up to 1,280 members: forty
  // loads a lane, all in flight at once), so the step waits for memory once a pass instead of once a group of four.
  constexpr int kHeld = 40;
  const bool holds = p.cap <= 32 * kHeld && warp < picks;
  int32_t held[kHeld];
  if (holds) {
    const int64_t bucket = bucket_s[warp];
    int n = 0;
#pragma unroll
    for (int j = 0; j < kHeld; ++j) {
      const int at = 32 * j + lane;
      held[j] = bucket >= 0 && at < p.cap ? p.members[bucket * p.cap + at] : LSA_PAD;
    }
#pragma unroll
    for (int j = 0; j < kHeld; ++j) n += __popc(__ballot_sync(0xffffffffu, held[j] >= p.sink && held[j] < window_start));
    if (lane == 0) count_s[warp] = n;
  }
  for (int pick = holds ? warp + kWarps : warp; pick < picks; pick += kWarps) {
    const int64_t bucket = bucket_s[pick];
    int n = 0;
    if (bucket >= 0)
      for (int at0 = 0; at0 < p.cap; at0 += 128) {  // four loads in flight
        int32_t ids[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int at = at0 + 32 * j + lane;
          ids[j] = at < p.cap ? p.members[bucket * p.cap + at] : LSA_PAD;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) n += __popc(__ballot_sync(0xffffffffu, ids[j] >= p.sink && ids[j] < window_start));
      }
    if (lane == 0) count_s[pick] = n;
  }
  __syncthreads();
  if (warp == 0) {  // this CTA's picks, scanned; its total for the others
    int carry = 0;
    for (int base = 0; base < picks; base += 32) {
      const int v = base + lane < picks ? count_s[base + lane] : 0;
      int incl = v;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
      }
      if (base + lane < picks) start_s[base + lane] = carry + incl - v;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) total_s = carry;
  }
  cluster.sync();
  int before = 0, all = 0;  // ids of the CTAs before this one, and of all of them
  for (int c = 0; c < kClusterCtas; ++c) {
    const int t = *cluster.map_shared_rank(&total_s, c);
    if (c < cta) before += t;
    all += t;
  }
  if (holds) {
    int written = before + start_s[warp];
#pragma unroll
    for (int j = 0; j < kHeld; ++j) {
      const bool counts = held[j] >= p.sink && held[j] < window_start;
      const unsigned votes = __ballot_sync(0xffffffffu, counts);
      const int at = written + __popc(votes & below);
      if (counts && at < row_k) out[at] = stored_id(p, table, held[j]);
      written += __popc(votes);
    }
  }
  for (int pick = holds ? warp + kWarps : warp; pick < picks; pick += kWarps) {
    const int64_t bucket = bucket_s[pick];
    int written = before + start_s[pick];
    if (bucket < 0) continue;
    for (int at0 = 0; at0 < p.cap && written < row_k; at0 += 128) {
      int32_t ids[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int at = at0 + 32 * j + lane;
        ids[j] = at < p.cap ? p.members[bucket * p.cap + at] : LSA_PAD;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const bool counts = ids[j] >= p.sink && ids[j] < window_start;
        const unsigned votes = __ballot_sync(0xffffffffu, counts);
        const int at = written + __popc(votes & below);
        if (counts && at < row_k) out[at] = stored_id(p, table, ids[j]);
        written += __popc(votes);
      }
    }
  }
  // the window, the sinks and the padding: an eighth of each a CTA
  int total = min(all, row_k);
  const int gtid = cta * kClusterThreads + tid, gthreads = kClusterCtas * kClusterThreads;
  if (!(p.flags & LSA_EXPAND_NO_LOCAL)) {
    const int in_window = (int)(pos + 1 - window_start);
    for (int i = gtid; i < in_window; i += gthreads) out[total + i] = stored_id(p, table, window_start + i);
    total += in_window;
    const int sinks = (int)min((int64_t)p.sink, min(window_start, pos + 1));
    for (int i = gtid; i < sinks; i += gthreads) out[total + i] = stored_id(p, table, i);
    total += sinks;
  }
  if (!(p.flags & LSA_EXPAND_NO_PAD))
    for (int j = total + gtid; j < p.width; j += gthreads) out[j] = LSA_PAD;
  if (tid == 0) {
    if (cta == 0) p.lengths[r] = total;
    if (bad_s && p.status) atomicAdd(p.status, bad_s);
  }
  cluster.sync();  // nobody leaves while its total may still be read
}

}  // namespace lsa

LSA_API int lsa_expand_batched(const int32_t *picked, int64_t R, int top_p, const int64_t *positions,
                       const int32_t *members, int64_t m, int bucket_cap, const int32_t *row_top_p,
                       const int32_t *row_top_k, int top_k, int sink, int window, const int32_t *page_table,
                       int page_size, int64_t owner_first, int64_t owner_end, int owner_granule, int owner_world,
                       int owner_rank, int flags, const int32_t *row_request, int64_t page_table_stride,
                       const int32_t *bucket_pages, int64_t bucket_pages_stride, int bucket_max_pages,
                       int bucket_page_rows, int32_t *selected, int32_t *lengths,
                       int32_t *status, void *stream) {
  LSA_REQUIRE(picked && positions && selected && lengths, LSA_ERR_NULL);
  LSA_REQUIRE(m == 0 || members, LSA_ERR_NULL);
  LSA_REQUIRE(R >= 0 && top_p >= 1 && m >= 0 && bucket_cap >= 1 && top_k >= 1 && sink >= 0 && window >= 1,
              LSA_ERR_ARGUMENT);
  LSA_REQUIRE(!page_table || page_size >= 1, LSA_ERR_ARGUMENT);
  LSA_REQUIRE(!bucket_pages || (bucket_page_rows >= 1 && bucket_max_pages >= 1), LSA_ERR_ARGUMENT);
  LSA_REQUIRE(owner_world <= 1 || (owner_granule >= 1 && owner_rank >= 0 && owner_rank < owner_world),
              LSA_ERR_ARGUMENT);
  LSA_REQUIRE((int64_t)top_k + window + sink < INT32_MAX, LSA_ERR_ARGUMENT);
  if (R == 0) return LSA_OK;
  lsa::ExpandParams p;
  p.picked = picked;
  p.positions = positions;
  p.members = members;
  p.row_top_p = row_top_p;
  p.row_top_k = row_top_k;
  p.page_table = page_table;
  p.selected = selected;
  p.lengths = lengths;
  p.status = status;
  p.R = R;
  p.m = m;
  p.owner_first = owner_first;
  p.owner_end = owner_end;
  p.granule = owner_granule;
  p.world = owner_world;
  p.rank = owner_rank;
  p.flags = flags;
  p.row_request = row_request;
  p.page_table_stride = page_table_stride;
  p.bucket_pages = bucket_pages;
  p.bucket_pages_stride = bucket_pages_stride;
  p.bucket_max_pages = bucket_max_pages;
  p.bucket_page_rows = bucket_page_rows;
  p.top_p = top_p;
  p.cap = bucket_cap;
  p.top_k = top_k;
  p.sink = sink;
  p.window = window;
  p.page_size = page_size;
  p.width = top_k + window + sink;
  const bool keeps_all = owner_world <= 1 && owner_first <= 0 && owner_end == INT64_MAX;
  if (R <= 8 && keeps_all && top_p <= lsa::kWideMaxPicks && (int64_t)top_p * bucket_cap >= 32768) {
    // a few rows with very long lists: a cluster of CTAs a row
    const dim3 grid(lsa::kClusterCtas, (unsigned)R);
    lsa::launch(true, lsa::expand_cluster_kernel, grid, dim3(lsa::kClusterThreads), 0, (cudaStream_t)stream, p);
    LSA_LAUNCH_CHECK();
    return LSA_OK;
  }
  if (keeps_all && top_p <= lsa::kWideMaxPicks &&
      (int64_t)top_p * bucket_cap + window >= (R <= 8 ? 1024 : (R <= 64 ? 4096 : INT64_MAX))) {
    // a decode step's long lists: one CTA a row
    lsa::launch(R <= lsa::kChainedRows, lsa::expand_wide_kernel, dim3((unsigned)R), dim3(lsa::kWideThreads), 0,
                (cudaStream_t)stream, p);
    LSA_LAUNCH_CHECK();
    return LSA_OK;
  }
  const unsigned grid = (unsigned)((R + lsa::kExpandWarps - 1) / lsa::kExpandWarps);
  lsa::launch(R <= lsa::kChainedRows, lsa::expand_kernel, dim3(grid), dim3(lsa::kExpandWarps * 32), 0,
              (cudaStream_t)stream, p);
  LSA_LAUNCH_CHECK();
  return LSA_OK;
}

LSA_API int lsa_expand(const int32_t *picked, int64_t R, int top_p, const int64_t *positions,
                       const int32_t *members, int64_t m, int bucket_cap, const int32_t *row_top_p,
                       const int32_t *row_top_k, int top_k, int sink, int window, const int32_t *page_table,
                       int page_size, int64_t owner_first, int64_t owner_end, int owner_granule, int owner_world,
                       int owner_rank, int flags, int32_t *selected, int32_t *lengths, int32_t *status,
                       void *stream) {
  return lsa_expand_batched(picked, R, top_p, positions, members, m, bucket_cap, row_top_p, row_top_k, top_k, sink,
                            window, page_table, page_size, owner_first, owner_end, owner_granule, owner_world,
                            owner_rank, flags, nullptr, 0, nullptr, 0, 0, 0, selected, lengths, status, stream);
}
