// Bucket-major attention of a prefill chunk: the selected keys of every row, read bucket by bucket.
//
// The gather kernel reads each listed K/V row once per (query row, KV head); a chunk of 8,192 rows that each pick 64
// of a few thousand buckets reads every bucket a hundred times over. Here the loop is turned inside out:
//
//   starts    a warp a row walks the row's picks in order and records, for each, how many selected ids came before
//             it (the top-k cut needs that) - or -1 when the pick adds nothing
//   invert    the (row, pick) pairs are grouped by bucket: histogram, scan, scatter
//   attend    a CTA owns (bucket, KV head, segment of 128 or 256 pairs): the bucket's K/V rows are staged ONCE in shared
//             memory, each warp takes one query head of the group and runs its pairs through them in tiles of 16
//             query rows (queries as the M side of mma.m16n8k16), writing a normalised bf16 partial output and a
//             log-sum-exp per (pair, head)
//   merge     a warp per (row, head) merges the row's partials with the dense band's partial (window and sinks)
//
// A pair's keys are its bucket's members inside [sink, window_start(row)), cut where the row's running count
// reaches its top-k: with members ascending (as lsa_bucket_table writes them) that is an index range of the bucket.
#include "bucket_attend.cuh"
#include "common.cuh"
#include "mma.cuh"

namespace lsa {

// ---------------------------------------------------------------------------------------------- starts

__global__ void __launch_bounds__(256) bucket_starts_kernel(BucketParams p) {
  const int lane = lane_id();
  const int64_t r = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (r >= p.R) return;
  const int64_t pos = p.positions[r];
  const int row_p = p.row_top_p ? min(p.row_top_p[r], p.top_p) : p.top_p;
  const int row_k = p.row_top_k ? min(p.row_top_k[r], p.top_k) : p.top_k;
  const int64_t window_start = max((int64_t)0, pos + 1 - p.window);
  int running = 0;
  for (int i0 = 0; i0 < p.top_p; i0 += 32) {
    const int i = i0 + lane;
    int64_t bucket = i < row_p ? p.picked[r * p.top_p + i] : -1;
    if (bucket >= p.m) bucket = -1;
    // ids of my pick that count: a lane a pick, the members walked 16 bytes at a time
    int mine = 0;
    if (bucket >= 0) {
      const int32_t *row = p.members + bucket * p.cap;
      auto counts = [&](int32_t id) { return (id >= p.sink && id < window_start) ? 1 : 0; };
      if ((p.cap & 3) == 0 && (reinterpret_cast<uintptr_t>(p.members) & 15) == 0) {
        const int4 *row4 = reinterpret_cast<const int4 *>(row);
#pragma unroll 4
        for (int j = 0; j < p.cap / 4; ++j) {
          const int4 ids = row4[j];
          mine += counts(ids.x) + counts(ids.y) + counts(ids.z) + counts(ids.w);
        }
      } else {
        for (int j = 0; j < p.cap; ++j) mine += counts(row[j]);
      }
    }
    // exclusive scan of the counts over the 32 picks
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    const int before = running + incl - mine;
    const bool adds = bucket >= 0 && mine > 0 && before < row_k;
    if (i < p.top_p) {
      p.starts[r * p.top_p + i] = adds ? before : -1;
      p.takes[r * p.top_p + i] = adds ? min(mine, row_k - before) : 0;  // members ascend: the counted ids are a run
    }
    if (adds) atomicAdd(&p.counts[bucket], 1);
    running += __shfl_sync(0xffffffffu, incl, 31);
  }
}

// ---------------------------------------------------------------------------------------------- invert

// One CTA: exclusive scans of the bucket counts (pairs, and segments of pairs) with a running carry.
__global__ void __launch_bounds__(1024) bucket_scan_kernel(BucketParams p) {
  __shared__ int warp_pairs[32], warp_segs[32];
  __shared__ int carry_pairs, carry_segs;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) carry_pairs = carry_segs = 0;
  __syncthreads();
  for (int64_t base = 0; base < p.m; base += 1024) {
    const int64_t b = base + tid;
    const int c = b < p.m ? p.counts[b] : 0;
    const int s = (c + p.segment - 1) / p.segment;
    int ic = c, is = s;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int uc = __shfl_up_sync(0xffffffffu, ic, o), us = __shfl_up_sync(0xffffffffu, is, o);
      if (lane >= o) ic += uc, is += us;
    }
    if (lane == 31) warp_pairs[warp] = ic, warp_segs[warp] = is;
    __syncthreads();
    if (warp == 0) {
      int wc = warp_pairs[lane], ws = warp_segs[lane];
      const int own_c = wc, own_s = ws;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int uc = __shfl_up_sync(0xffffffffu, wc, o), us = __shfl_up_sync(0xffffffffu, ws, o);
        if (lane >= o) wc += uc, ws += us;
      }
      warp_pairs[lane] = wc - own_c;
      warp_segs[lane] = ws - own_s;
    }
    __syncthreads();
    const int before_c = carry_pairs + warp_pairs[warp] + ic - c;
    const int before_s = carry_segs + warp_segs[warp] + is - s;
    if (b < p.m) {
      p.offsets[b] = before_c;
      p.cursors[b] = before_c;
      p.seg_offsets[b] = before_s;
    }
    __syncthreads();
    if (tid == 1023) {
      carry_pairs = before_c + c;
      carry_segs = before_s + s;
    }
    __syncthreads();
  }
  if (tid == 0) {
    p.offsets[p.m] = carry_pairs;
    p.seg_offsets[p.m] = carry_segs;
  }
}

__global__ void __launch_bounds__(256) bucket_scatter_kernel(BucketParams p) {
  const int64_t pair = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (pair >= p.R * p.top_p) return;
  if (p.starts[pair] < 0) return;
  const int32_t bucket = p.picked[pair];
  const int at = atomicAdd(&p.cursors[bucket], 1);
  p.order[at] = (int32_t)pair;
  p.order_takes[at] = p.takes[pair];
}

// A thread a bucket writes the table of its segments, so a CTA of the attend pass finds its work with one load.
__global__ void __launch_bounds__(256) bucket_segments_kernel(BucketParams p) {
  const int64_t b = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (b >= p.m) return;
  const int count = p.counts[b], first = p.offsets[b], at = p.seg_offsets[b];
  for (int s = 0; s * p.segment < count; ++s)
    p.segments[at + s] = make_int4((int)b, first + s * p.segment, min(p.segment, count - s * p.segment), 0);
}

// ---------------------------------------------------------------------------------------------- attend

// grid (segment bound, Hkv); blockDim = group * 32: warp w serves query head h * group + w.
// Occupancy decides this kernel: at 96 registers and one query buffer a warp, four CTAs of five warps share an SM;
// at 128 registers and two buffers three do, and uncapped one does, each markedly slower.
template <int DH>
__global__ void __maxnreg__(96) bucket_attend_kernel(BucketParams p) {
  constexpr int ROW_BYTES = DH * 2;
  constexpr int CHUNKS = ROW_BYTES / 16;
  constexpr int KV_BYTES = kBktKeys * ROW_BYTES;   // one of K or V
  constexpr int Q_BYTES = kBktTile * ROW_BYTES;    // one warp's tile of query rows
  constexpr int KSTEPS = DH / 16;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ int32_t ids_s[kBktKeys];
  __shared__ int32_t pairs_s[kBktSegment];   // the segment's pairs, -1 past its end
  __shared__ int32_t rows_s[kBktSegment];    // their query rows
  __shared__ int32_t until_s[kBktSegment];   // the position their key range ends before (the window's start)
  __shared__ int32_t allow_s[kBktSegment];   // ids they may still take under the row's top-k
  __shared__ int32_t hi_s[kBktSegment];      // end of their index range of the bucket's members

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int h = blockIdx.y;
  const int seg = blockIdx.x;
  if (seg >= p.seg_offsets[p.m]) return;
  const int4 info = p.segments[seg];  // bucket, first pair of the segment in `order`, pairs of the segment
  const int64_t bucket = info.x;
  const int first = info.y, n_pairs = info.z;
  for (int i = tid; i < kBktKeys; i += blockDim.x) ids_s[i] = i < p.cap ? p.members[bucket * p.cap + i] : LSA_PAD;
  // Everything a pair needs is fetched once for the segment, a thread a pair, not once a tile.
  for (int i = tid; i < kBktSegment; i += blockDim.x) {
    int32_t pair = -1, row = 0, until = 0, allow = 0;
    if (i < n_pairs) {
      pair = p.order[first + i];
      row = pair / p.top_p;
      const int64_t pos = p.positions[row];
      const int row_k = p.row_top_k ? min(p.row_top_k[row], p.top_k) : p.top_k;
      until = (int32_t)max((int64_t)0, pos + 1 - p.window);
      allow = row_k - p.starts[pair];
    }
    pairs_s[i] = pair, rows_s[i] = row, until_s[i] = until, allow_s[i] = allow;
  }
  __syncthreads();

  // The bucket's keys and values of this KV head, staged once (rows of ids outside the cache are zero-filled and
  // never valid: a pair's range only holds ids the starts pass counted).
  const uint32_t k_s = smem_u32(smem_raw), v_s = k_s + KV_BYTES;
  const uint32_t q_s = v_s + KV_BYTES + warp * Q_BYTES;  // a tile a warp: four CTAs share an SM instead of three
  {
    const uint16_t *k_head = p.k + (int64_t)h * p.kv_head_stride, *v_head = p.v + (int64_t)h * p.kv_head_stride;
    for (int e = tid; e < kBktKeys * CHUNKS; e += blockDim.x) {
      const int row = e / CHUNKS, chunk = e - row * CHUNKS;
      const int32_t id = ids_s[row];
      const bool ok = id >= 0 && id < p.slots;
      const int64_t off = ok ? (int64_t)id * p.kv_row_stride + chunk * 8 : 0;
      const uint32_t dst = row * ROW_BYTES + ((chunk ^ (row & 7)) << 4);
      cp_async_16(k_s + dst, k_head + off, ok ? 16 : 0);
      cp_async_16(v_s + dst, v_head + off, ok ? 16 : 0);
    }
    cp_async_commit();
  }
  const int head = h * p.group + warp;
  const int tiles = (n_pairs + kBktTile - 1) / kBktTile;
  // Start the copies of a tile's 16 query rows of this warp's head.
  auto issue_q = [&](int tile) {
    if (tile < tiles) {
      const uint32_t dst0 = q_s;
      for (int e = lane; e < kBktTile * CHUNKS; e += 32) {
        const int row = e / CHUNKS, chunk = e - row * CHUNKS;
        const bool ok = pairs_s[tile * kBktTile + row] >= 0;
        const uint16_t *src = p.q + (int64_t)rows_s[tile * kBktTile + row] * p.q_row_stride +
                              (int64_t)head * p.q_head_stride + chunk * 8;
        cp_async_16(dst0 + row * ROW_BYTES + ((chunk ^ (row & 7)) << 4), src, ok ? 16 : 0);
      }
    }
    cp_async_commit();
  };
  issue_q(0);
  // Index range of the bucket's members below a position: members ascend and their padding comes last.
  int n_members = 0;
  while (n_members < p.cap && n_members < kBktKeys && ids_s[n_members] >= 0) ++n_members;
  auto members_below = [&](int64_t bound) {
    int lo = 0, hi = n_members;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (ids_s[mid] < bound) lo = mid + 1; else hi = mid;
    }
    return lo;
  };
  const int below_sink = members_below(p.sink);
  // members that name a row of the cache handed in (the others are staged as zeros and masked out of the softmax)
  const uint64_t valid_word = (uint64_t)__ballot_sync(0xffffffffu, ids_s[lane] >= 0 && ids_s[lane] < p.slots) |
                              ((uint64_t)__ballot_sync(0xffffffffu, ids_s[lane + 32] >= 0 && ids_s[lane + 32] < p.slots) << 32);
  const int key_steps = (n_members + 15) >> 4;  // 16-key steps that hold members; the rest of the tile is padding
  for (int i = tid; i < kBktSegment; i += blockDim.x)
    hi_s[i] = pairs_s[i] >= 0 ? min(members_below(until_s[i]), below_sink + allow_s[i]) : 0;

  for (int tile = 0; tile < tiles; ++tile) {
    __syncwarp();  // the warp has sent the last tile's outputs, which were staged in this buffer
    if (tile > 0) issue_q(tile);
    cp_async_wait<0>();
    if (tile == 0) __syncthreads(); else __syncwarp();  // the first wait also covers the bucket's K/V and the ranges
    const uint32_t q_tile = q_s;

    // the key range of rows g and g + 8 of the tile
    int lo_key[2], hi_key[2];
    int32_t pair_of[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      pair_of[j] = pairs_s[tile * kBktTile + g + 8 * j];
      lo_key[j] = below_sink;
      hi_key[j] = hi_s[tile * kBktTile + g + 8 * j];
    }

    // S [16 rows x 64 keys]
    float s[kBktKeys / 8][4];
#pragma unroll
    for (int nt = 0; nt < kBktKeys / 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      uint32_t a0, a1, a2, a3;
      {
        const int row = lane & 15, chunk = ks * 2 + (lane >> 4);
        ldmatrix_x4(q_tile + row * ROW_BYTES + ((chunk ^ (row & 7)) << 4), a0, a1, a2, a3);
      }
#pragma unroll
      for (int np = 0; np < kBktKeys / 16; ++np) {
        if (np >= key_steps) continue;
        const int row = np * 16 + ((lane >> 4) & 1) * 8 + (lane & 7), chunk = ks * 2 + ((lane >> 3) & 1);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(k_s + row * ROW_BYTES + ((chunk ^ (row & 7)) << 4), b0, b1, b2, b3);
        mma_bf16(s[2 * np], a0, a1, a2, a3, b0, b1);
        mma_bf16(s[2 * np + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    // softmax over the pair's key range. Most key tiles lie inside every row's range and need no masks: the tile
    // is inside when it starts at or after the warp's greatest range start and ends by its least range end.
    const int lo_max = __reduce_max_sync(0xffffffffu, max(lo_key[0], lo_key[1]));
    const int hi_min = __reduce_min_sync(0xffffffffu, min(hi_key[0], hi_key[1]));
    float m_row[2] = {-INFINITY, -INFINITY}, l_row[2] = {0.0f, 0.0f};
#pragma unroll
    for (int nt = 0; nt < kBktKeys / 8; ++nt) {
      if (nt * 8 >= key_steps * 16) continue;
      if (nt * 8 < lo_max || nt * 8 + 8 > hi_min || ((valid_word >> (nt * 8)) & 0xFFu) != 0xFFu) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int key = nt * 8 + 2 * t + (c & 1), j = c >> 1;
          if (key < lo_key[j] || key >= hi_key[j] || !((valid_word >> key) & 1u)) s[nt][c] = -INFINITY;
        }
      }
      m_row[0] = fmaxf(m_row[0], fmaxf(s[nt][0], s[nt][1]));
      m_row[1] = fmaxf(m_row[1], fmaxf(s[nt][2], s[nt][3]));
    }
    float m_off[2];  // the row maximum in the log2 domain, what the exponent subtracts (0 for a row with no key)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      m_row[j] = fmaxf(m_row[j], __shfl_xor_sync(0xffffffffu, m_row[j], 1));
      m_row[j] = fmaxf(m_row[j], __shfl_xor_sync(0xffffffffu, m_row[j], 2));
      m_row[j] *= p.scale_log2;  // the scale is positive: the maximum of the raw products is the maximum
      m_off[j] = m_row[j] == -INFINITY ? 0.0f : m_row[j];
    }
#pragma unroll
    for (int nt = 0; nt < kBktKeys / 8; ++nt) {
      if (nt * 8 >= key_steps * 16) continue;
      s[nt][0] = fast_exp2(fmaf(s[nt][0], p.scale_log2, -m_off[0]));
      s[nt][1] = fast_exp2(fmaf(s[nt][1], p.scale_log2, -m_off[0]));
      s[nt][2] = fast_exp2(fmaf(s[nt][2], p.scale_log2, -m_off[1]));
      s[nt][3] = fast_exp2(fmaf(s[nt][3], p.scale_log2, -m_off[1]));
      l_row[0] += s[nt][0] + s[nt][1];
      l_row[1] += s[nt][2] + s[nt][3];
    }
    float inv[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      l_row[j] += __shfl_xor_sync(0xffffffffu, l_row[j], 1);
      l_row[j] += __shfl_xor_sync(0xffffffffu, l_row[j], 2);
      inv[j] = l_row[j] > 0.0f ? 1.0f / l_row[j] : 0.0f;
    }
    // P is normalised before it is rounded to bf16 (a row's sum is known by now), so O needs no scaling afterwards.
    // The accumulator of key tiles 2k, 2k + 1 is the A fragment of 16-key step k.
    uint32_t pa[kBktKeys / 16][4];
#pragma unroll
    for (int nt = 0; nt < kBktKeys / 8; ++nt) {
      const bool live = nt * 8 < key_steps * 16;
      pa[nt >> 1][(nt & 1) * 2] = live ? pack_bf16x2(s[nt][0] * inv[0], s[nt][1] * inv[0]) : 0u;
      pa[nt >> 1][(nt & 1) * 2 + 1] = live ? pack_bf16x2(s[nt][2] * inv[1], s[nt][3] * inv[1]) : 0u;
    }
    // O [16 rows x DH] = P V, one half of the head dim at a time: 32 accumulators live instead of 64. Each half is
    // staged in the tile's query buffer (the first product is done with it), so the rows leave in 16-byte pieces.
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      float o[DH / 16][4];
#pragma unroll
      for (int nt = 0; nt < DH / 16; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.0f;
#pragma unroll
      for (int ks = 0; ks < kBktKeys / 16; ++ks) {
        if (ks >= key_steps) continue;
#pragma unroll
        for (int np = 0; np < DH / 32; ++np) {
          const int row = ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
          const int chunk = (half * (DH / 32) + np) * 2 + (lane >> 4);
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4_trans(v_s + row * ROW_BYTES + ((chunk ^ (row & 7)) << 4), b0, b1, b2, b3);
          mma_bf16(o[2 * np], pa[ks][0], pa[ks][1], pa[ks][2], pa[ks][3], b0, b1);
          mma_bf16(o[2 * np + 1], pa[ks][0], pa[ks][1], pa[ks][2], pa[ks][3], b2, b3);
        }
      }
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        if (pair_of[j] < 0) continue;
        const int row = g + 8 * j;
#pragma unroll
        for (int nt = 0; nt < DH / 16; ++nt) {
          const uint32_t at = row * ROW_BYTES + (((half * (DH / 16) + nt) ^ (row & 7)) << 4) + 4 * t;
          asm volatile("st.shared.b32 [%0], %1;" ::"r"(q_tile + at), "r"(pack_bf16x2(o[nt][2 * j], o[nt][2 * j + 1])));
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      if (pair_of[j] < 0 || t != 0) continue;
      p.part_lse[(int64_t)pair_of[j] * p.Hq + head] =
          l_row[j] > 0.0f ? (m_row[j] + log2f(l_row[j])) * 0.6931471805599453f : -INFINITY;
    }
    __syncwarp();
    for (int e = lane; e < kBktTile * CHUNKS; e += 32) {
      const int row = e / CHUNKS, chunk = e - row * CHUNKS;
      const int32_t pair = pairs_s[tile * kBktTile + row];
      if (pair < 0) continue;
      uint4 piece;
      asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                   : "=r"(piece.x), "=r"(piece.y), "=r"(piece.z), "=r"(piece.w)
                   : "r"(q_tile + row * ROW_BYTES + ((chunk ^ (row & 7)) << 4)));
      *reinterpret_cast<uint4 *>(p.part_out + ((int64_t)pair * p.Hq + head) * DH + chunk * 8) = piece;
    }
  }
}

// ---------------------------------------------------------------------------------------------- merge

// A warp per (row, head): the row's partials (one per pick that added keys) and the band's partial, merged by their
// log-sum-exps. A lane holds DH / 32 consecutive dims.
template <int DH>
__global__ void __launch_bounds__(256) bucket_merge_kernel(BucketParams p) {
  constexpr int PER = DH / 32;
  static_assert(PER == 4, "a lane reads four bf16 dims (8 bytes) of a partial");
  const int lane = lane_id();
  const int64_t item = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (item >= p.R * p.Hq) return;
  const int64_t r = item / p.Hq;
  const int head = (int)(item - r * p.Hq);
  const float band_lse = p.init_lse ? p.init_lse[item] : -INFINITY;
  float m = band_lse;
  for (int i = lane; i < p.top_p; i += 32)
    if (p.starts[r * p.top_p + i] >= 0) m = fmaxf(m, p.part_lse[(r * p.top_p + i) * p.Hq + head]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  float acc[PER];
#pragma unroll
  for (int c = 0; c < PER; ++c) acc[c] = 0.0f;
  float l = 0.0f;
  if (m > -INFINITY) {
    if (band_lse > -INFINITY) {
      const float w = expf(band_lse - m);
      l = w;
      const float *src = p.init_out + item * DH + lane * PER;
#pragma unroll
      for (int c = 0; c < PER; ++c) acc[c] = w * src[c];
    }
    for (int i0 = 0; i0 < p.top_p; i0 += 32) {
      const int i = i0 + lane;
      float w_mine = 0.0f;
      if (i < p.top_p && p.starts[r * p.top_p + i] >= 0) {
        const float lse = p.part_lse[(r * p.top_p + i) * p.Hq + head];
        w_mine = lse > -INFINITY ? expf(lse - m) : 0.0f;
      }
      // four partials at a time, their loads in flight together
      unsigned left = __ballot_sync(0xffffffffu, w_mine > 0.0f);
      while (left) {
        float w[4];
        uint2 v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int src_lane = left ? __ffs(left) - 1 : 0;
          w[j] = left ? __shfl_sync(0xffffffffu, w_mine, src_lane) : 0.0f;
          left &= left - 1;
          const uint16_t *src = p.part_out + ((r * p.top_p + i0 + src_lane) * p.Hq + head) * DH + lane * PER;
          v[j] = w[j] > 0.0f ? *reinterpret_cast<const uint2 *>(src) : make_uint2(0u, 0u);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          l += w[j];
          acc[0] = fmaf(w[j], bf16_bits_to_float((uint16_t)(v[j].x & 0xFFFF)), acc[0]);
          acc[1] = fmaf(w[j], bf16_bits_to_float((uint16_t)(v[j].x >> 16)), acc[1]);
          acc[2] = fmaf(w[j], bf16_bits_to_float((uint16_t)(v[j].y & 0xFFFF)), acc[2]);
          acc[3] = fmaf(w[j], bf16_bits_to_float((uint16_t)(v[j].y >> 16)), acc[3]);
        }
      }
    }
  }
  const float inv = l > 0.0f ? 1.0f / l : 0.0f;
  uint16_t *dst = p.out_bf16 + item * DH + lane * PER;
#pragma unroll
  for (int c = 0; c < PER; ++c) dst[c] = float_to_bf16_bits(acc[c] * inv);
  if (lane == 0 && p.lse_out) p.lse_out[item] = l > 0.0f ? m + logf(l) : -INFINITY;
}

struct BucketWorkspace {
  size_t starts, counts, offsets, seg_offsets, cursors, order, takes, order_takes, segments, part_out, part_lse, total;
};

// Every bucket with pairs has at most one ragged segment: segments <= pairs / segment + buckets with pairs.
static int64_t segment_bound(int64_t R, int top_p, int64_t m) {
  const int64_t pairs = R * top_p;
  return pairs / kBktSegment + (m < pairs ? m : pairs) + 1;
}

static BucketWorkspace bucket_workspace(int64_t R, int top_p, int Hq, int dh, int64_t m) {
  auto up = [](size_t x) { return (x + 255) & ~(size_t)255; };
  BucketWorkspace w;
  size_t at = 0;
  const size_t pairs = (size_t)R * top_p;
  w.starts = at, at += up(pairs * 4);
  w.counts = at, at += up((size_t)(m + 1) * 4);
  w.offsets = at, at += up((size_t)(m + 1) * 4);
  w.seg_offsets = at, at += up((size_t)(m + 1) * 4);
  w.cursors = at, at += up((size_t)(m + 1) * 4);
  w.order = at, at += up(pairs * 4);
  w.takes = at, at += up(pairs * 4);
  w.order_takes = at, at += up(pairs * 4);
  w.segments = at, at += up((size_t)segment_bound(R, top_p, m) * 16);
  w.part_out = at, at += up(pairs * Hq * dh * 2);
  w.part_lse = at, at += up(pairs * Hq * 4);
  w.total = at;
  return w;
}

}  // namespace lsa

// ================================================================================================ C ABI

LSA_API size_t lsa_bucket_attend_workspace_bytes(int64_t R, int top_p, int Hq, int dh, int64_t m) {
  if (R <= 0 || top_p <= 0 || Hq <= 0 || dh <= 0 || m < 0) return 0;
  return lsa::bucket_workspace(R, top_p, Hq, dh, m).total;
}

LSA_API int lsa_bucket_attend(const uint16_t *q, int64_t R, int Hq, int dh, int64_t q_row_stride,
                              int64_t q_head_stride, const uint16_t *k, const uint16_t *v, int64_t slots, int Hkv,
                              int64_t kv_row_stride, int64_t kv_head_stride, const int32_t *picked, int top_p,
                              const int64_t *positions, const int32_t *members, int64_t m, int bucket_cap,
                              const int32_t *row_top_p, const int32_t *row_top_k, int top_k, int sink, int window,
                              const float *init_out, const float *init_lse, float scale, uint16_t *out_bf16,
                              float *lse_out, int flags, void *init_ready_event, int32_t *status,
                              void *workspace, size_t workspace_bytes, void *stream) {
  LSA_REQUIRE(q && k && v && picked && positions && out_bf16 && workspace, LSA_ERR_NULL);
  LSA_REQUIRE(m == 0 || members, LSA_ERR_NULL);
  LSA_REQUIRE((init_out == nullptr) == (init_lse == nullptr), LSA_ERR_NULL);
  LSA_REQUIRE(R >= 0 && Hq >= 1 && Hkv >= 1 && Hq % Hkv == 0 && slots >= 0 && slots <= INT32_MAX && top_p >= 1 &&
                  m >= 0 && m < INT32_MAX && bucket_cap >= 1 && top_k >= 1 && sink >= 0 && window >= 1 &&
                  R * top_p < INT32_MAX && scale > 0.0f,
              LSA_ERR_ARGUMENT);
  LSA_REQUIRE(dh == 128 && bucket_cap <= lsa::kBktKeys && Hq / Hkv <= 8, LSA_ERR_UNSUPPORTED);
  LSA_REQUIRE(kv_row_stride % 8 == 0 && kv_head_stride % 8 == 0 && ((uintptr_t)k % 16) == 0 &&
                  ((uintptr_t)v % 16) == 0 && q_row_stride % 8 == 0 && q_head_stride % 8 == 0 &&
                  ((uintptr_t)q % 16) == 0,
              LSA_ERR_ARGUMENT);
  if (R == 0) return LSA_OK;
  const lsa::BucketWorkspace w = lsa::bucket_workspace(R, top_p, Hq, dh, m);
  LSA_REQUIRE(workspace_bytes >= w.total, LSA_ERR_WORKSPACE);
  unsigned char *base = reinterpret_cast<unsigned char *>(workspace);
  lsa::BucketParams p = {};
  p.q = q, p.k = k, p.v = v;
  p.picked = picked, p.members = members, p.row_top_p = row_top_p, p.row_top_k = row_top_k;
  p.positions = positions;
  p.init_out = init_out, p.init_lse = init_lse;
  p.out_bf16 = out_bf16, p.lse_out = lse_out, p.status = status;
  p.starts = reinterpret_cast<int32_t *>(base + w.starts);
  p.counts = reinterpret_cast<int32_t *>(base + w.counts);
  p.offsets = reinterpret_cast<int32_t *>(base + w.offsets);
  p.seg_offsets = reinterpret_cast<int32_t *>(base + w.seg_offsets);
  p.cursors = reinterpret_cast<int32_t *>(base + w.cursors);
  p.order = reinterpret_cast<int32_t *>(base + w.order);
  p.takes = reinterpret_cast<int32_t *>(base + w.takes);
  p.order_takes = reinterpret_cast<int32_t *>(base + w.order_takes);
  p.segments = reinterpret_cast<int4 *>(base + w.segments);
  p.part_out = reinterpret_cast<uint16_t *>(base + w.part_out);
  p.part_lse = reinterpret_cast<float *>(base + w.part_lse);
  p.R = R, p.m = m, p.slots = slots;
  p.q_row_stride = q_row_stride, p.q_head_stride = q_head_stride;
  p.kv_row_stride = kv_row_stride, p.kv_head_stride = kv_head_stride;
  p.top_p = top_p, p.cap = bucket_cap, p.top_k = top_k, p.sink = sink, p.window = window;
  p.Hq = Hq, p.Hkv = Hkv, p.group = Hq / Hkv;
  const bool tensor_memory = !(flags & LSA_BUCKET_WARP_MMA) && R * top_p * Hq < INT32_MAX;
  p.segment = tensor_memory ? lsa::kBktSegmentTc : lsa::kBktSegment;
  p.scale_log2 = scale * 1.4426950408889634f;
  cudaStream_t s = (cudaStream_t)stream;
  if (cudaMemsetAsync(p.counts, 0, (size_t)(m + 1) * 4, s) != cudaSuccess) return LSA_ERR_LAUNCH;
  lsa::bucket_starts_kernel<<<(unsigned)((R + 7) / 8), 256, 0, s>>>(p);
  LSA_LAUNCH_CHECK();
  if (m > 0) {
    lsa::bucket_scan_kernel<<<1, 1024, 0, s>>>(p);
    LSA_LAUNCH_CHECK();
    const int64_t pairs = R * top_p;
    lsa::bucket_scatter_kernel<<<(unsigned)((pairs + 255) / 256), 256, 0, s>>>(p);
    LSA_LAUNCH_CHECK();
    lsa::bucket_segments_kernel<<<(unsigned)((m + 255) / 256), 256, 0, s>>>(p);
    LSA_LAUNCH_CHECK();
    const int64_t bound = lsa::segment_bound(R, top_p, m);
    if (!tensor_memory) {
      const size_t smem = 2 * (size_t)lsa::kBktKeys * dh * 2 + (size_t)p.group * lsa::kBktTile * dh * 2;
      if (cudaFuncSetAttribute(lsa::bucket_attend_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               (int)smem) != cudaSuccess)
        return LSA_ERR_LAUNCH;
      const dim3 grid((unsigned)bound, (unsigned)Hkv);
      lsa::bucket_attend_kernel<128><<<grid, p.group * 32, smem, s>>>(p);
      LSA_LAUNCH_CHECK();
    } else {
      const int rc = lsa::launch_bucket_attend_tc(p, bound, s);
      if (rc != LSA_OK) return rc;
    }
  }
  // init_out / init_lse may be the work of another stream (the dense band running beside the passes above): only
  // the merge reads them, so only the merge waits.
  if (init_ready_event && cudaStreamWaitEvent(s, (cudaEvent_t)init_ready_event, 0) != cudaSuccess) return LSA_ERR_LAUNCH;
  lsa::bucket_merge_kernel<128><<<(unsigned)((R * Hq + 7) / 8), 256, 0, s>>>(p);
  LSA_LAUNCH_CHECK();
  return LSA_OK;
}
