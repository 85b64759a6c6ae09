// The attend pass of the bucket-major attention on the fifth-generation tensor cores.
//
// A CTA owns (bucket, KV head, segment of up to 256 (row, pick) pairs). The M = 128 rows of a tile are (pair, query
// head of the KV head's group) couples, the heads of a pair next to one another, so a ragged segment of n pairs
// costs ceil(n * group / 128) tiles and not `group` of them. A row of S and of O lives in one lane of tensor memory
// and the thread that owns the row does its softmax without talking to anyone:
//
//   S [128 x keys]  = Q [128 x 128] . K^T           tcgen05.mma, A = the tile's query rows, B = the bucket's keys,
//                                                   both K-major planes of 64 dims with the 128-byte swizzle
//   P               = exp2(S - rowmax) / rowsum on the row's key range, bf16, written back to shared memory
//   O [128 x 128]   = P [128 x keys] . V            A = P (K-major), B = the bucket's values AS STORED
//                                                   ([key][dim] planes: an MN-major operand)
//
// Eight warps. Together they gather the query rows of the tile after next (a row of 256 bytes a half warp) and send
// the finished tile's rows out in the same shape. For the softmax and the unloading of O a row has TWO threads, one
// in warp q and one in warp 4 + q (both may read the tensor-memory lanes of quarter q): they take alternate groups
// of 8 keys of S, swap their maxima and sums through shared memory, and take a half of O's columns each. The row's instruction stream is what bounds this kernel, so it
// is cut in two. A lane of warp 0 also issues the MMAs, at the points where the warp would wait for their results
// anyway: a ninth warp for that would cost every thread 32 registers (five warps on a scheduler instead of four).
//
// The tiles of a CTA overlap: the tensor cores multiply S of tile i + 1 while the workers unload O of tile i, and
// the query rows of tile i + 2 are on their way by then. Two CTAs share an SM and fill one another's waits.
//
// Shared-memory operands are written by ordinary and asynchronous copies (the generic proxy), so a proxy fence stands
// before every hand-over to the tensor cores. Every wait on an mbarrier is bounded; a wait that gives up raises the
// CTA's abort flag, the CTA skips its remaining work (but none of its barriers), frees its tensor memory and leaves.
#include "bucket_attend.cuh"
#include "mma.cuh"
#include "umma.cuh"

namespace lsa {

constexpr int kTcThreads = 256;
constexpr int kTcRows = 128;                    // rows of a tile
constexpr int kTcPlane = 64 * 128;              // a plane of 64 rows x 128 bytes (keys or values, 64 dims)
constexpr int kTcQPlane = kTcRows * 128;        // a plane of the query tile or of P
constexpr int kTcKOff = 0;                      // K: 2 planes
constexpr int kTcVOff = 2 * kTcPlane;           // V: 2 planes
constexpr int kTcQOff = 4 * kTcPlane;           // Q: 2 buffers of 2 planes
// P takes the first plane of the tile's own query buffer (the first product is over when P is written), and the
// finished rows of O are staged in the whole of it (the second product is over by then).
constexpr int kTcSmem = kTcQOff + 4 * kTcQPlane + 1024;  // + room to align the base to 1,024 bytes
constexpr int kTcTmemCols = 256;                // S in columns 0-63, O in 64-191
static_assert(kBktSegmentTc == kTcThreads && kBktKeys == 64, "a thread a pair of the segment; 64 keys a bucket");

__device__ __forceinline__ void proxy_fence() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// the two warps of a quarter of the rows
__device__ __forceinline__ void quarter_sync(int quarter) { asm volatile("bar.sync %0, 64;" ::"r"(2 + quarter) : "memory"); }


template <int DH>
__global__ void __launch_bounds__(kTcThreads, 2) bucket_attend_tc_kernel(BucketParams p) {
  static_assert(DH == 128, "two planes of 64 dims");
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ int32_t ids_s[kBktKeys];
  __shared__ int32_t pairs_s[kBktSegmentTc];   // the segment's pairs, -1 past its end
  __shared__ int32_t qrows_s[kBktSegmentTc];   // their query rows
  __shared__ int32_t hi_s[kBktSegmentTc];      // members of the bucket they read
  // of the rows of a tile (a ring of three tiles): where the query row starts in q (-1 past the end), which slot of
  // the partial outputs it fills, and the end of its key range
  __shared__ int64_t src_s[3][kTcRows];
  __shared__ int32_t dst_s[3][kTcRows];  // (the caller has checked that the slots fit 31 bits)
  __shared__ int32_t end_s[3][kTcRows];
  __shared__ float swap_max_s[2][kTcRows], swap_sum_s[2][kTcRows];
  __shared__ __align__(8) uint64_t bars[3];
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int abort_s;
  __shared__ uint32_t valid_s[2];  // which members of the bucket name a row of the cache

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = blockIdx.y;
  const int seg = blockIdx.x;
  // (the table holds a slot for every CTA of the grid: the segment is asked for beside the count, not after it)
  const int4 info = p.segments[seg];
  if (seg >= p.seg_offsets[p.m]) return;
  const int64_t bucket = info.x;
  const int first = info.y, n_pairs = info.z;
  const int n_rows = n_pairs * p.group;
  const int n_tiles = (n_rows + kTcRows - 1) / kTcRows;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  // bar_w: the workers tell the MMA lane that operands are in place; bar_s / bar_o: a product has finished
  const uint32_t bar_w = smem_u32(&bars[0]), bar_s = smem_u32(&bars[1]), bar_o = smem_u32(&bars[2]);

  if (tid == 0) {
    mbar_init(bar_w, kTcThreads);
    mbar_init(bar_s, 1);
    mbar_init(bar_o, 1);
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)),
                 "r"(kTcTmemCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  for (int i = tid; i < kBktKeys; i += kTcThreads) ids_s[i] = i < p.cap ? p.members[bucket * p.cap + i] : LSA_PAD;
  // The segment's pairs, fetched beside the member ids (one round of loads for both). The starts pass has counted the
  // keys a pair takes; its run of members starts where the sinks end, which is added once the ids are in.
  if (tid < kBktSegmentTc) {
    int32_t pair = -1, take = 0;
    if (tid < n_pairs) {
      pair = p.order[first + tid];
      take = p.order_takes[first + tid];
    }
    pairs_s[tid] = pair, qrows_s[tid] = pair >= 0 ? pair / p.top_p : 0, hi_s[tid] = take;
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_s;

  // members of the bucket: the ids before the first pad
  int n_members;
  {
    const unsigned low = __ballot_sync(0xffffffffu, ids_s[lane] >= 0),
                   high = __ballot_sync(0xffffffffu, ids_s[lane + 32] >= 0);
    n_members = low != 0xffffffffu ? __ffs(~low) - 1 : (high != 0xffffffffu ? 32 + __ffs(~high) - 1 : 64);
    n_members = min(n_members, p.cap);
  }
  // members that name a row of the cache handed in: a key outside it is staged as zeros and masked out of the softmax,
  // as the row-by-row read skips such ids
  // (the word stays in shared memory and only a flag in a register: every member is in the cache as a rule, and a
  // 64-bit word held through the tile loop costs this kernel spills)
  bool all_valid;
  {
    const uint32_t v_lo = __ballot_sync(0xffffffffu, ids_s[lane] >= 0 && ids_s[lane] < p.slots),
                   v_hi = __ballot_sync(0xffffffffu, ids_s[lane + 32] >= 0 && ids_s[lane + 32] < p.slots);
    all_valid = __popc(v_lo) + __popc(v_hi) == n_members;
    if (tid == 0) valid_s[0] = v_lo, valid_s[1] = v_hi;
  }
  // which of keys c0 .. c0 + 7 name a row of the cache, a bit each
  auto valid_byte = [&](int c0) { return all_valid ? 0xFFu : (valid_s[c0 >> 5] >> (c0 & 31)) & 0xFFu; };
  const int n_keys = max(16, (n_members + 15) & ~15);  // the N of S and the K of O: whole 16-key steps

  // Step k of the MMAs (warp 0; the whole warp waits so that its lanes stay together, lane 0 issues): once the k-th
  // hand-over of the threads is complete, O of tile k - 1 and S of tile k.
  auto issue_products = [&](int k) {
    if (!__all_sync(0xffffffffu, !abort_s && mbar_wait(bar_w, k & 1))) {
      abort_s = 1;
      return;
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (lane != 0) return;
    if (k >= 1) {  // O = P V: 16 keys are 32 bytes along P's rows, 16 rows (2,048 bytes) down V's planes
      const uint32_t p_buf = base + kTcQOff + ((k - 1) & 1) * 2 * kTcQPlane;
      for (int s = 0; s < n_keys / 16; ++s)
        umma_bf16(tmem_base + 64, smem_desc_sw128(p_buf) + 2 * s, smem_desc_mn_sw128(base + kTcVOff + s * 2048, kTcPlane),
                  umma_idesc(DH, true), s != 0);
      umma_commit(bar_o);
    }
    if (k < n_tiles) {  // S = Q K^T: 16 dims are 32 bytes further inside the swizzle atom
      const uint32_t q_buf = base + kTcQOff + (k & 1) * 2 * kTcQPlane;
#pragma unroll
      for (int plane = 0; plane < 2; ++plane)
#pragma unroll
        for (int s = 0; s < 4; ++s)
          umma_bf16(tmem_base, smem_desc_sw128(q_buf + plane * kTcQPlane) + 2 * s,
                    smem_desc_sw128(base + kTcKOff + plane * kTcPlane) + 2 * s, umma_idesc(n_keys), (plane | s) != 0);
      umma_commit(bar_s);
    }
  };
  {
    const int w = tid;                         // the thread's place in the shared copies
    const int quarter = warp & 3;              // the 32 tensor-memory lanes this warp may read
    const int half = warp >> 2;                // which of the row's two threads
    const int row = quarter * 32 + lane;       // the tile row (= tensor-memory lane)
    auto members_below = [&](int64_t bound) {
      int lo = 0, hi = n_members;
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (ids_s[mid] < bound) lo = mid + 1; else hi = mid;
      }
      return lo;
    };
    const int lo_key = members_below(p.sink);
    // The bucket's keys and values of this KV head: chunk c of member j goes to plane c / 8, row j, 16-byte slot
    // (c % 8) ^ (j % 8) - the layout a tensor-map copy with the 128-byte swizzle would write.
    {
      const uint16_t *k_head = p.k + (int64_t)h * p.kv_head_stride, *v_head = p.v + (int64_t)h * p.kv_head_stride;
#pragma unroll 2
      for (int e = w; e < kBktKeys * 16; e += kTcThreads) {
        const int r = e >> 4, chunk = e & 15;
        const int32_t id = ids_s[r];
        const bool ok = id >= 0 && id < p.slots;
        const int64_t off = ok ? (int64_t)id * p.kv_row_stride + chunk * 8 : 0;
        const uint32_t dst = (chunk >> 3) * kTcPlane + r * 128 + (((chunk & 7) ^ (r & 7)) << 4);
        cp_async_16(base + kTcKOff + dst, k_head + off, ok ? 16 : 0);
        cp_async_16(base + kTcVOff + dst, v_head + off, ok ? 16 : 0);
      }
    }
    // Rows come in, are listed and go out a QUARTER at a time: the two warps that share the tensor-memory lanes of 32
    // rows also copy those rows, so the only barriers inside a tile are between those two warps.
    const int w64 = half * 32 + lane;  // the thread's place among the 64 of its quarter
    auto list_rows = [&](int tile) {
      if (half != 0) return;
      const int flat = tile * kTcRows + row;
      const bool ok = flat < n_rows;
      const int pl = ok ? flat / p.group : 0;
      const int head = h * p.group + (flat - pl * p.group);
      src_s[tile % 3][row] = ok ? (int64_t)qrows_s[pl] * p.q_row_stride + (int64_t)head * p.q_head_stride : -1;
      dst_s[tile % 3][row] = ok ? pairs_s[pl] * p.Hq + head : -1;
      end_s[tile % 3][row] = ok ? lo_key + hi_s[pl] : 0;
    };
    // The query rows of a tile: half a warp copies a row of 256 bytes, in the layout of the keys.
    auto gather_q = [&](int tile) {
      const uint32_t buf = base + kTcQOff + (tile & 1) * 2 * kTcQPlane;
#pragma unroll 4
      for (int j = 0; j < 32 * 16 / 64; ++j) {
        const int e = j * 64 + w64;
        const int r = quarter * 32 + (e >> 4), chunk = e & 15;
        const int64_t from = src_s[tile % 3][r];
        cp_async_16(buf + (chunk >> 3) * kTcQPlane + r * 128 + (((chunk & 7) ^ (r & 7)) << 4),
                    p.q + (from >= 0 ? from + chunk * 8 : 0), from >= 0 ? 16 : 0);
      }
    };
    list_rows(0);
    if (n_tiles > 1) list_rows(1);
    quarter_sync(quarter);  // and the first tiles' rows of this quarter
    gather_q(0);
    cp_async_commit();
    if (n_tiles > 1) gather_q(1);
    cp_async_commit();
    cp_async_wait<1>();
    proxy_fence();
    mbar_arrive(bar_w);  // K, V and the first tile's queries are in place
    if (warp == 0) issue_products(0);

    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    for (int tile = 0; tile < n_tiles; ++tile) {
      const uint32_t parity = tile & 1;
      const uint32_t buf = base + kTcQOff + parity * 2 * kTcQPlane;
      const int hi_key = end_s[tile % 3][row];
      const int64_t slot = dst_s[tile % 3][row];
      // ---- softmax of the row: P, bf16 and already divided by the row's sum, is the A operand of the second product.
      // This thread has the groups of 8 keys 2 j + half. (One decision a warp on the wait: the tensor-memory loads
      // are warp-wide instructions.)
      bool go = __all_sync(0xffffffffu, !abort_s && mbar_wait(bar_s, parity));
      if (!go) abort_s = 1;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      // A group of 8 keys that lies inside the key range of every row of the warp needs no masks: most do.
      uint32_t sv[4][8];
      bool active[4], whole[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c0 = (2 * j + half) * 8;
        active[j] = c0 < n_keys;
        whole[j] = __all_sync(0xffffffffu, c0 >= lo_key && c0 + 8 <= hi_key) && valid_byte(c0) == 0xFFu;
        if (go && active[j]) tmem_load_8(lane_addr + c0, sv[j]);
      }
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      // (four running maxima, and four running sums below: one chain of 32 dependent operations is what a thread
      // with few warps beside it waits on)
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c0 = (2 * j + half) * 8;
        if (!active[j]) continue;
        if (whole[j]) {
#pragma unroll
          for (int c = 0; c < 8; ++c) mx4[c & 3] = fmaxf(mx4[c & 3], __uint_as_float(sv[j][c]));
        } else {
          const uint32_t vb = valid_byte(c0);
#pragma unroll
          for (int c = 0; c < 8; ++c) {  // (bitwise logic and selects: branches here would diverge lane by lane)
            const bool ok = (c0 + c >= lo_key) & (c0 + c < hi_key) & (bool)((vb >> c) & 1u);
            mx4[c & 3] = fmaxf(mx4[c & 3], ok ? __uint_as_float(sv[j][c]) : -INFINITY);
          }
        }
      }
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      swap_max_s[half][row] = mx;
      quarter_sync(quarter);
      mx = fmaxf(mx, swap_max_s[half ^ 1][row]);
      const float m_row = mx == -INFINITY ? 0.0f : mx * p.scale_log2;  // (finite, so that a masked key gives exp2(-inf) = 0)
      float l4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c0 = (2 * j + half) * 8;
        if (!active[j]) continue;
        if (whole[j]) {
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const float e = fast_exp2(fmaf(__uint_as_float(sv[j][c]), p.scale_log2, -m_row));
            l4[c & 3] += e;
            sv[j][c] = __float_as_uint(e);
          }
        } else {
          const uint32_t vb = valid_byte(c0);
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const bool ok = (c0 + c >= lo_key) & (c0 + c < hi_key) & (bool)((vb >> c) & 1u);
            const float e = fast_exp2(fmaf(ok ? __uint_as_float(sv[j][c]) : -INFINITY, p.scale_log2, -m_row));
            l4[c & 3] += e;
            sv[j][c] = __float_as_uint(e);
          }
        }
      }
      float l_row = (l4[0] + l4[1]) + (l4[2] + l4[3]);
      swap_sum_s[half][row] = l_row;
      quarter_sync(quarter);
      l_row += swap_sum_s[half ^ 1][row];
      const float inv = l_row > 0.0f ? 1.0f / l_row : 0.0f;
      const uint32_t p_row = buf + row * 128;  // 16-byte slot (c / 8) ^ (row % 8) of the row
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c8 = 2 * j + half;
        if (!active[j]) continue;
        uint32_t v[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
          v[i] = pack_bf16x2(__uint_as_float(sv[j][2 * i]) * inv, __uint_as_float(sv[j][2 * i + 1]) * inv);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(p_row + ((c8 ^ (row & 7)) << 4)), "r"(v[0]),
                     "r"(v[1]), "r"(v[2]), "r"(v[3])
                     : "memory");
      }
      if (go && half == 0 && slot >= 0)
        p.part_lse[slot] = l_row > 0.0f ? (m_row + log2f(l_row)) * 0.6931471805599453f : -INFINITY;
      cp_async_wait<0>();  // the next tile's queries (sent a tile ago) have landed too
      proxy_fence();
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive(bar_w);
      if (warp == 0) issue_products(tile + 1);
      // ---- O of the tile: out of tensor memory into the tile's (spent) query buffer, this thread's half of the
      // columns, then out in whole rows
      go = __all_sync(0xffffffffu, !abort_s && mbar_wait(bar_o, parity));
      if (!go) abort_s = 1;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (go) {
        uint32_t r[2][32];
        tmem_load_32(lane_addr + 64 + half * (DH / 2), r[0]);
        tmem_load_32(lane_addr + 64 + half * (DH / 2) + 32, r[1]);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t a = pack_bf16x2(__uint_as_float(r[c][8 * i]), __uint_as_float(r[c][8 * i + 1]));
            const uint32_t b = pack_bf16x2(__uint_as_float(r[c][8 * i + 2]), __uint_as_float(r[c][8 * i + 3]));
            const uint32_t d = pack_bf16x2(__uint_as_float(r[c][8 * i + 4]), __uint_as_float(r[c][8 * i + 5]));
            const uint32_t f = pack_bf16x2(__uint_as_float(r[c][8 * i + 6]), __uint_as_float(r[c][8 * i + 7]));
            // (the thread's half of the columns is a plane of the buffer, laid out as the query rows were: a quarter's
            // rows stay inside the bytes that the quarter itself fills again)
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(buf + half * kTcQPlane + row * 128 +
                                                                           (((c * 4 + i) ^ (row & 7)) << 4)),
                         "r"(a), "r"(b), "r"(d), "r"(f)
                         : "memory");
          }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      quarter_sync(quarter);  // the quarter's rows are staged
      if (go) {
#pragma unroll 4
        for (int j = 0; j < 32 * 16 / 64; ++j) {
          const int e = j * 64 + w64;
          const int r = quarter * 32 + (e >> 4), chunk = e & 15;
          const int64_t to = dst_s[tile % 3][r];
          if (to < 0) continue;
          uint4 piece;
          asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(piece.x), "=r"(piece.y), "=r"(piece.z), "=r"(piece.w)
                       : "r"(buf + (chunk >> 3) * kTcQPlane + r * 128 + (((chunk & 7) ^ (r & 7)) << 4)));
          *reinterpret_cast<uint4 *>(p.part_out + to * DH + chunk * 8) = piece;
        }
      }
      if (tile + 2 < n_tiles) list_rows(tile + 2);
      quarter_sync(quarter);  // the quarter's rows have been read out, and those of the tile after next are listed
      if (tile + 2 < n_tiles) gather_q(tile + 2);
      cp_async_commit();
    }
    cp_async_wait<0>();
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTcTmemCols));
  }
  // A CTA that gave up leaves stale partials behind: the status word tells the host that the call's output is void.
  if (tid == 0 && abort_s && p.status) atomicAdd(p.status, 1);
}

int launch_bucket_attend_tc(const BucketParams &p, int64_t segment_bound, cudaStream_t stream) {
  auto kernel = bucket_attend_tc_kernel<128>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmem) != cudaSuccess)
    return LSA_ERR_LAUNCH;
  const dim3 grid((unsigned)segment_bound, (unsigned)p.Hkv);
  kernel<<<grid, kTcThreads, kTcSmem, stream>>>(p);
  LSA_LAUNCH_CHECK();
  return LSA_OK;
}

}  // namespace lsa
