// Gather-sparse attention over a shared latent (the MLA form) on the fifth-generation tensor cores.
//
// A CTA owns a (query row, split of its list, block of 64 heads) item. All heads of a row read the SAME listed latent
// rows, so the heads are the M = 64 side of both products and a gathered row serves 64 heads:
//
//   S [64 heads x 64 keys]  = Q [64 x 576] . K^T      tcgen05.mma, A = the row's heads, B = a tile of gathered
//                                                     latent rows, both K-major planes of 64 dims (128-byte swizzle)
//   P                       = exp2(S - m), bf16       a thread a head; m is the running row maximum, refreshed only
//                                                     when it grows by more than 2^8 (so O is rescaled rarely)
//   O [64 x 512]           += P [64 x 64] . V         A = P (K-major), B = the SAME staged rows read as an MN-major
//                                                     operand: a value is the first 512 dims of its latent row
//
// An M = 64 accumulator fills lanes 0-15 of each 32-lane quarter of tensor memory, and a second one may sit in lanes
// 16-31: O's first 256 value dims live in the lower half-quarters of columns 0-255 and its last 256 in the upper ones,
// S has two buffers in the lower half-quarters of columns 256-319 and 320-383. M = 64 because the shared memory of
// an SM holds the 64 heads' queries (72 KB) beside two stages of 64 gathered rows (72 KB each) and no more.
//
//   warps 0-3   a thread a head (lanes 0-15 of a warp; lanes 16-31 own the upper half of O): S out of tensor memory,
//               masks, P into shared memory, the rare rescale of O, the normalised output
//   warp 4      tensor-memory allocation; one lane issues S = Q K^T of every tile
//   warp 9      one lane issues O += P V of every tile (a lane of its own: the two products belong to tiles in
//               different stages, and one lane for both makes each wait for the other's loads)
//   warps 5-8   staging: a tile is up to 64 listed rows. 64 consecutive rows of the cache - what a bucket's pools
//               and a window are made of - are ONE box of a tensor-map copy per plane, wherever they start;
//               anything else is gathered with 16-byte asynchronous copies into the same swizzled planes
//
// The two stages run as two chains (load, S, softmax, O) that fill one another's waits. Every wait on an mbarrier is bounded; a wait that gives up raises the CTA's
// abort flag and the status word, the roles drain, the tensor memory is freed and the CTA leaves.
#include "latent_attend.cuh"
#include "mma.cuh"
#include "umma.cuh"

namespace lsa {

constexpr int kLtThreads = 320;
constexpr int kLtKeys = 64;                         // gathered rows a tile
constexpr int kLtPlanes = 9;                        // 576 dims = 9 planes of 64
constexpr int kLtPlane = 64 * 128;                  // 64 rows x 64 dims of bf16
constexpr int kLtStage = kLtPlanes * kLtPlane;      // a tile of gathered rows (and the queries: the same shape)
constexpr int kLtStages = 2;
constexpr int kLtKOff = kLtStage;                   // queries first, then the ring
constexpr int kLtPOff = kLtKOff + kLtStages * kLtStage;
constexpr int kLtSmem = kLtPOff + kLtPlane + 1024;  // + room to align the base to 1,024 bytes
constexpr int kLtTmemCols = 512;
constexpr int kLtSCol = 256;                        // S buffers at columns 256 and 320
constexpr int kLtChunks = 72;                       // 16-byte chunks a latent row
constexpr int kLtOutPitch = 516;                    // floats between staged output rows: 16-byte aligned, 4 banks on
constexpr int kLtMinRun = 16;                       // a shorter run of at least this many rows is a tile of its own
constexpr float kLtRescale = 8.0f;                  // the running maximum is refreshed when it grows by 2^8

constexpr uint32_t kLtSpinLimit = 1u << 20;  // polls of one wait (a tile's load or product takes microseconds)
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}
#ifdef LSA_LT_TRACE
// A clock trace of the first CTA's first 64 tiles (a tuning aid, compiled only on request): event e of tile t.
__device__ long long lsa_lt_trace[16 * 64];
#define LT_TRACE(cond, e, t)                                                                     \
  do {                                                                                           \
    if (blockIdx.x == 0 && blockIdx.y == 0 && (cond) && (t) < 64) lsa_lt_trace[(e) * 64 + (t)] = clock64(); \
  } while (0)
#else
#define LT_TRACE(cond, e, t) \
  do {                       \
  } while (0)
#endif
__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap *map, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(map), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void lt_proxy_fence() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void lt_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_store_32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
// Instruction descriptor of an M = 64 product: bf16 x bf16 -> fp32, N = n, A K-major, B K-major or MN-major.
__host__ __device__ constexpr uint32_t lt_idesc(int n, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(64 >> 4) << 24);
}

__global__ void __launch_bounds__(kLtThreads, 1)
    latent_attend_tc_kernel(const __grid_constant__ CUtensorMap map_latent, LatentParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // k_full / k_empty: a ring stage's rows have landed / may be overwritten; s_full / s_empty: an S buffer holds a
  // product / has been read; p_full: P is in place (and O rescaled); pv_done: the second product of a tile is over;
  // drained: every product an issuing lane has issued is complete.
  __shared__ __align__(8) uint64_t bars[3 * kLtStages + 2 * 2 + 4];
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int abort_s;
  __shared__ int32_t ids_s[kLtStages][kLtKeys];
  // what the gather tells the other roles about a staged tile: which of its 64 rows hold a listed key of the cache,
  // and whether it is the item's last; and what its first warp tells the other three about the tile to stage
  __shared__ volatile uint32_t info_s[kLtStages][4];
  __shared__ volatile int32_t plan_s[1];
  // (a stage is given back in two halves: planes 0-3 when the first half of O's product has read them, the rest
  // after the second, so the next box's first planes are already on their way during the second half)
  enum { kFull = 0, kEmpty = kLtStages, kEmptyB = 2 * kLtStages, kSFull = 3 * kLtStages, kSEmpty = 3 * kLtStages + 2 };
  auto bar = [&](int kind, int i) { return smem_u32(&bars[kind + i]); };
  const uint32_t p_full = smem_u32(&bars[3 * kLtStages + 4]), pv_done = smem_u32(&bars[3 * kLtStages + 5]),
                 drained_s = smem_u32(&bars[3 * kLtStages + 6]), drained_o = smem_u32(&bars[3 * kLtStages + 7]);
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int split = (int)(blockIdx.x % p.splits);
  const int64_t r = blockIdx.x / p.splits;
  const int head0 = blockIdx.y * kLatHeads;
  const bool partial = p.splits > 1;
  dependents_may_launch();
  wait_for_earlier_grids();
  LT_TRACE(tid == 0, 10, 0);

  int64_t n_total = p.lengths ? p.lengths[r] : p.list_stride;
  if (n_total > p.list_stride) n_total = p.list_stride;
  if (n_total < 0) n_total = 0;
  int64_t per = (n_total + p.splits - 1) / p.splits;
  per = (per + kLtKeys - 1) / kLtKeys * kLtKeys;
  const int64_t begin = (int64_t)split * per;
  const int64_t end = begin + per < n_total ? begin + per : n_total;
  const int n = end > begin ? (int)(end - begin) : 0;
  const int32_t *list = p.ids + r * p.list_stride + begin;

  // the thread's head and its half of the value dims (threads of the worker warps)
  const int half = lane >> 4;
  const int row = (warp & 3) * 16 + (lane & 15);
  const int64_t out_row = (partial ? (int64_t)split * p.R + r : r) * p.Hq + head0 + row;
  const bool row_ok = warp < 4 && head0 + row < p.Hq;

  if (n == 0) {  // nothing listed for this item: an empty partial
    if (row_ok) {
      if (half == 0) (partial ? p.part_lse : p.lse)[out_row] = -INFINITY;
      for (int c = 0; c < 256; ++c) {
        const int64_t at = out_row * 512 + half * 256 + c;
        if (partial) {
          p.part_out[at] = 0.0f;
        } else {
          if (p.out_f32) p.out_f32[at] = 0.0f;
          if (p.out_bf16) p.out_bf16[at] = 0;
        }
      }
    }
    return;
  }

  if (tid == 0) {
    for (int i = 0; i < kLtStages; ++i) {
      mbar_init(bar(kFull, i), 1);
      mbar_init(bar(kEmpty, i), 1);
      mbar_init(bar(kEmptyB, i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(kSFull, i), 1);
      mbar_init(bar(kSEmpty, i), 128);
    }
    mbar_init(p_full, 128);
    mbar_init(pv_done, 1);
    mbar_init(drained_s, 1);
    mbar_init(drained_o, 1);
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 4) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)),
                 "r"(kLtTmemCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_s;
  LT_TRACE(tid == 0, 10, 1);

  // A wait of one thread: false (and the abort flag) when it gives up or the CTA has already given up elsewhere.
  auto wait_one = [&](uint32_t b, uint32_t parity) {
    bool done = false;
    for (uint32_t spin = 0; spin < kLtSpinLimit && !done && !abort_s; ++spin) done = mbar_try(b, parity);
    if (!done) abort_s = 1;
    return done;
  };
  // The same for a warp whose lanes go on together.
  auto wait = [&](uint32_t b, uint32_t parity) {
    bool done = false;
    for (uint32_t spin = 0; spin < kLtSpinLimit && !done && !abort_s; ++spin) done = mbar_try(b, parity);
    const bool ok = __all_sync(0xffffffffu, done);
    if (!ok) abort_s = 1;
    return ok;
  };
  // An issuing lane leaves only when its products are complete (bounded, but not cut short by the abort flag: the
  // tensor memory must not be freed under a running product).
  auto drain = [&](uint32_t b) {
    umma_commit(b);
    bool done = false;
    for (uint32_t spin = 0; spin < kLtSpinLimit && !done; ++spin) done = mbar_try(b, 0);
  };

  if (warp >= 5 && warp < 9) {
    // ------------------------------------------------------------------------------------------ staging the rows
    const int ptid = tid - 5 * 32;
    auto gather_sync = [] { asm volatile("bar.sync 1, 128;" ::: "memory"); };
    // (the first entries of the list are asked for before the queries, which they do not depend on: a decode step's
    // CTA lives for a few tiles and cannot afford one wait on memory after another)
    int32_t head_a = -1, head_b = -1;
    if (warp == 5) {
      head_a = lane < n ? list[lane] : -1;
      head_b = 32 + lane < n ? list[32 + lane] : -1;
    }
    // the row's query heads
    for (int e = ptid; e < kLatHeads * kLtChunks; e += 128) {
      const int qr = e / kLtChunks, c = e - qr * kLtChunks;
      const bool ok = head0 + qr < p.Hq;
      const uint16_t *src = ok ? p.q + r * p.q_row_stride + (int64_t)(head0 + qr) * p.q_head_stride + c * 8 : p.q;
      cp_async_16(base + (c >> 3) * kLtPlane + qr * 128 + (((c & 7) ^ (qr & 7)) << 4), src, ok ? 16 : 0);
    }
    cp_async_commit();
    cp_async_wait<0>();
    lt_proxy_fence();
    gather_sync();  // the queries are in place before any tile is announced
    // The rows of a tile that is not one box, a quarter of the copies a warp.
    auto gather_rows = [&](int stage) {
      const uint32_t dst0 = base + kLtKOff + stage * kLtStage;
#pragma unroll 4
      for (int i = 0; i < kLtKeys * kLtChunks / 128; ++i) {
        const int e = ptid + i * 128;
        const int kr = e / kLtChunks, c = e - kr * kLtChunks;
        const int32_t id = ids_s[stage][kr];
        const uint16_t *src = p.latent + (id >= 0 ? (int64_t)id * p.latent_row_stride + c * 8 : 0);
        cp_async_16(dst0 + (c >> 3) * kLtPlane + kr * 128 + (((c & 7) ^ (kr & 7)) << 4), src, id >= 0 ? 16 : 0);
      }
      cp_async_commit();
      cp_async_wait<0>();
      lt_proxy_fence();
    };
    if (warp == 5) {
      // The first warp walks the list, 64 entries ahead (two a lane), and stages boxes by itself; the other three
      // wait at the barrier for tiles that must be gathered.
      const bool dealt = p.deal_world > 1;  // ids are positions of a cache dealt over ranks: only this rank's are read
      const int64_t deal_span = (int64_t)p.deal_granule * p.deal_world;
      auto mine = [&](int32_t id) { return !dealt || (int)((id / p.deal_granule) % p.deal_world) == p.deal_rank; };
      auto row_of = [&](int32_t id) {
        return dealt ? (int32_t)(id / deal_span * p.deal_granule + id % p.deal_granule) : id;
      };
      int x = 0, j = 0;
      int32_t id_a = head_a, id_b = head_b;
      bool alive = true;
      while ((x < n || dealt) && alive) {
        const int stage = j & 1;
        const bool closing = x >= n;  // (a dealt list ends with an empty tile: which tile is the last is not known before)
        // 64 consecutive rows of the cache are ONE box of a tensor-map copy per plane, wherever they start. Anything
        // else is gathered row by row (rows that hold no key are zero-filled: a box would bring in rows nobody
        // listed, whose bits need not be finite); a shorter run is a tile of its own, so that the tile after it
        // starts with the next run.
        const int remaining = closing ? 0 : min(kLtKeys, n - x);
        const int32_t first = __shfl_sync(0xffffffffu, id_a, 0);
        const bool ok_a = id_a >= 0 && row_of(id_a) < p.slots && mine(id_a);
        const bool ok_b = id_b >= 0 && row_of(id_b) < p.slots && mine(id_b);
        const uint32_t run_a = __ballot_sync(0xffffffffu, id_a >= 0 && id_a == first + lane);
        const uint32_t run_b = __ballot_sync(0xffffffffu, id_b >= 0 && id_b == first + 32 + lane);
        const int run = closing ? 0 : (run_a != 0xffffffffu ? __ffs(~run_a) - 1
                                                             : 32 + (run_b != 0xffffffffu ? __ffs(~run_b) - 1 : 32));
        const int count = run == kLtKeys ? kLtKeys : (run >= kLtMinRun ? run : remaining);
        const int32_t keep_a = ok_a && lane < count ? row_of(id_a) : -1;
        const int32_t keep_b = ok_b && 32 + lane < count ? row_of(id_b) : -1;
        const uint32_t valid0 = __ballot_sync(0xffffffffu, keep_a >= 0), valid1 = __ballot_sync(0xffffffffu, keep_b >= 0);
        // a box: 64 consecutive rows that this rank holds side by side (under dealing: inside one granule)
        const bool boxed = p.boxes && run == kLtKeys && (valid0 & valid1) == 0xffffffffu &&
                           (!dealt || first % p.deal_granule + kLtKeys <= p.deal_granule);
        const int32_t first_row = __shfl_sync(0xffffffffu, keep_a, 0);
        // the box is asked into the L2 now, a tile's time before its stage is free
        if (boxed && lane < kLtPlanes) tma_prefetch_2d(&map_latent, lane * 64, first_row);
        // the entries after this tile, on their way while it is staged
        const int at = x + count + lane;
        id_a = at < n ? list[at] : -1;
        id_b = at + 32 < n ? list[at + 32] : -1;
        x += count;
        if (dealt && !closing && (valid0 | valid1) == 0u) continue;  // nothing of this tile is stored here
        if (j >= kLtStages) alive = wait(bar(kEmpty, stage), ((j >> 1) - 1) & 1);
        if (!alive) break;
        LT_TRACE(lane == 0, 0, j);
        if (lane == 0) {
          info_s[stage][0] = valid0, info_s[stage][1] = valid1;
          info_s[stage][2] = dealt ? closing : x >= n;  // the last tile
          info_s[stage][3] = closing;                   // nothing staged: the products skip it
        }
        const uint32_t dst0 = base + kLtKOff + stage * kLtStage;
        if (closing) {
          if (j >= kLtStages) alive = wait(bar(kEmptyB, stage), ((j >> 1) - 1) & 1);
          if (!alive) break;
          if (lane == 0) lt_arrive(bar(kFull, stage));
          break;
        }
        if (boxed) {
          // a lane a plane: the copies are issued side by side, the first four planes as soon as they are free
          if (lane == 0) mbar_expect_tx(bar(kFull, stage), kLtStage);
          __syncwarp();
          if (lane < 4) tma_load_2d(dst0 + lane * kLtPlane, &map_latent, bar(kFull, stage), lane * 64, first_row);
          if (j >= kLtStages) alive = wait(bar(kEmptyB, stage), ((j >> 1) - 1) & 1);
          if (!alive) break;
          if (lane >= 4 && lane < kLtPlanes)
            tma_load_2d(dst0 + lane * kLtPlane, &map_latent, bar(kFull, stage), lane * 64, first_row);
          __syncwarp();
          LT_TRACE(lane == 0, 1, j);
        } else {
          if (j >= kLtStages) alive = wait(bar(kEmptyB, stage), ((j >> 1) - 1) & 1);
          if (!alive) break;
          ids_s[stage][lane] = keep_a;
          ids_s[stage][32 + lane] = keep_b;
          if (lane == 0) plan_s[0] = stage;
          gather_sync();  // the other three warps take their quarters
          gather_rows(stage);
          LT_TRACE(lane == 0, 1, j);
          gather_sync();
          if (lane == 0) lt_arrive(bar(kFull, stage));
        }
        LT_TRACE(lane == 0, 2, j);
        ++j;
      }
      if (lane == 0) plan_s[0] = -1;
      gather_sync();  // the other three warps leave
    } else {
      for (;;) {
        gather_sync();
        const int stage = plan_s[0];
        if (stage < 0) break;
        gather_rows(stage);
        gather_sync();
      }
    }
  } else if (warp == 4) {
    // ------------------------------------------------------------------------------------------ S = Q K^T
    if (lane == 0) {
      bool alive = true;
      for (int i = 0; alive; ++i) {
        const int sb = i & 1;
        alive = wait_one(bar(kFull, sb), (i >> 1) & 1);
        if (!alive) break;
        const bool last = info_s[sb][2] != 0, nothing = info_s[sb][3] != 0;
        if (i >= 2) alive = wait_one(bar(kSEmpty, sb), ((i >> 1) - 1) & 1);
        if (!alive) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        LT_TRACE(true, 3, i);
        const uint32_t k_s = base + kLtKOff + sb * kLtStage;
#pragma unroll
        for (int plane = 0; plane < kLtPlanes; ++plane)
#pragma unroll
          for (int s = 0; s < 4; ++s)
            if (!nothing)
              umma_bf16(tmem_base + kLtSCol + sb * kLtKeys, smem_desc_sw128(base + plane * kLtPlane) + 2 * s,
                      smem_desc_sw128(k_s + plane * kLtPlane) + 2 * s, lt_idesc(kLtKeys, false), (plane | s) != 0);
        umma_commit(bar(kSFull, sb));
        LT_TRACE(true, 4, i);
        if (last) break;
      }
      drain(drained_s);
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------------------------------ O += P V
    if (lane == 0) {
      bool alive = true;
      for (int t = 0; alive; ++t) {
        alive = wait_one(p_full, t & 1);
        if (!alive) break;
        const bool last = info_s[t & 1][2] != 0, nothing = info_s[t & 1][3] != 0;  // (read before the stage is given back)
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        LT_TRACE(true, 5, t);
        const uint32_t v_s = base + kLtKOff + (t & 1) * kLtStage;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
          for (int ks = 0; ks < kLtKeys / 16; ++ks)
            if (!nothing)
              umma_bf16(tmem_base + ((uint32_t)(h * 16) << 16), smem_desc_sw128(base + kLtPOff) + 2 * ks,
                      smem_desc_mn_sw128(v_s + h * 4 * kLtPlane + ks * 2048, kLtPlane), lt_idesc(256, true),
                      (t | ks) != 0);
          umma_commit(bar(h == 0 ? kEmpty : kEmptyB, t & 1));
        }
        umma_commit(pv_done);
        LT_TRACE(true, 6, t);
        if (last) break;
      }
      drain(drained_o);
    }
  } else {
    // ------------------------------------------------------------------------------------------ softmax and output
    const uint32_t lane_addr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
    const uint32_t p_row = base + kLtPOff + row * 128;
    float m_used = 0.0f, l_run = 0.0f;
    bool alive = true;
    int tiles = 0;
    for (int i = 0; alive; ++i) {
      const int sb = i & 1;
      // (the stage's own barrier too: it is what publishes the tile's validity masks)
      alive = wait(bar(kFull, sb), (i >> 1) & 1) && wait(bar(kSFull, sb), (i >> 1) & 1);
      if (!alive) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      LT_TRACE(tid == 0, 7, i);
      // The head's 64 products sit in the lane of its first thread; its second thread (lane + 16, which owns the
      // upper half of O) takes the last 32 of them by shuffle, so that both do half of the exponentials.
      uint32_t sv[32];
      {
        uint32_t lo[32], hi[32];
        tmem_load_32(lane_addr + kLtSCol + sb * kLtKeys, lo);
        tmem_load_32(lane_addr + kLtSCol + sb * kLtKeys + 32, hi);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        lt_arrive(bar(kSEmpty, sb));
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const uint32_t other = __shfl_sync(0xffffffffu, hi[c], lane & 15);
          sv[c] = half ? other : lo[c];
        }
      }
      const uint32_t valid = info_s[sb][half];
      const bool last = info_s[sb][2] != 0;
      const bool whole = (info_s[sb][0] & info_s[sb][1]) == 0xffffffffu;
      // the tile's maximum of the row (raw products: the scale is positive)
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (whole) {
#pragma unroll
        for (int c = 0; c < 32; ++c) mx4[c & 3] = fmaxf(mx4[c & 3], __uint_as_float(sv[c]));
      } else {
#pragma unroll
        for (int c = 0; c < 32; ++c)
          mx4[c & 3] = fmaxf(mx4[c & 3], (valid >> c) & 1u ? __uint_as_float(sv[c]) : -INFINITY);
      }
      float m_tile = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
      m_tile = fmaxf(m_tile, __shfl_xor_sync(0xffffffffu, m_tile, 16));
      // The maximum the exponents subtract is refreshed only when the tile's exceeds it by 2^8: P stays below 2^8,
      // and O, which would have to be rescaled in tensor memory, almost never is. (Both threads of a head see the
      // same maxima, so they take the same decisions.)
      float alpha = 1.0f;
      if (i == 0) {
        m_used = m_tile == -INFINITY ? 0.0f : m_tile;
      } else if (m_tile > m_used + kLtRescale) {
        alpha = fast_exp2(m_used - m_tile);
        m_used = m_tile;
      }
      const bool rescale = i > 0 && __any_sync(0xffffffffu, alpha != 1.0f);
      if (i > 0) {  // the last tile's second product is over: O is at rest and P may be overwritten
        alive = wait(pv_done, (i - 1) & 1);
        if (!alive) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      }
      LT_TRACE(tid == 0, 8, i);
      if (rescale) {
#pragma unroll 1
        for (int c = 0; c < 256; c += 32) {
          uint32_t o[32];
          tmem_load_32(lane_addr + c, o);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int k = 0; k < 32; ++k) o[k] = __float_as_uint(__uint_as_float(o[k]) * alpha);
          tmem_store_32(lane_addr + c, o);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      }
      l_run *= alpha;  // (each thread sums its own 32 keys; the two sums meet at the end)
      float l4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int c8 = 0; c8 < 4; ++c8) {
        float e[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const float x = __uint_as_float(sv[c8 * 8 + c]);
          const bool ok = whole || ((valid >> (c8 * 8 + c)) & 1u);
          e[c] = fast_exp2(fmaf(ok ? x : -INFINITY, p.scale_log2, -m_used));
          l4[c & 3] += e[c];
        }
        // 16-byte slot (keys / 8) ^ (row % 8) of the head's row of P
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(p_row + (((half * 4 + c8) ^ (row & 7)) << 4)),
                     "r"(pack_bf16x2(e[0], e[1])), "r"(pack_bf16x2(e[2], e[3])), "r"(pack_bf16x2(e[4], e[5])),
                     "r"(pack_bf16x2(e[6], e[7]))
                     : "memory");
      }
      l_run += (l4[0] + l4[1]) + (l4[2] + l4[3]);
      lt_proxy_fence();
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      lt_arrive(p_full);
      LT_TRACE(tid == 0, 9, i);
      tiles = i + 1;
      if (last) break;
    }
    if (alive) alive = wait(pv_done, (tiles - 1) & 1);
    LT_TRACE(tid == 0, 10, 2);
    if (alive) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      l_run += __shfl_xor_sync(0xffffffffu, l_run, 16);
      const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
      const bool read_any = l_run > 0.0f;  // (else O may never have been written: zeros, not O x 0)
      if (row_ok && half == 0)
        (partial ? p.part_lse : p.lse)[out_row] =
            l_run > 0.0f ? (m_used + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
      // A split's partial output goes out through shared memory (the ring is free by now): a thread holds 128 bytes
      // of ITS head's row, so stores straight from the registers touch 32 lines an instruction; staged, the warp
      // writes its sixteen rows - one contiguous block of the partial outputs - in whole lines. (A decode step, whose
      // CTAs live for a few tiles, spent a quarter of its time in these stores.)
      float *o_s = reinterpret_cast<float *>(smem_raw + (base - smem_u32(smem_raw)) + kLtKOff) +
                   (warp & 3) * (16 * kLtOutPitch);
#pragma unroll 1
      for (int c = 0; c < 256; c += 32) {
        uint32_t o[32];
        tmem_load_32(lane_addr + c, o);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (partial) {
          float *mine = o_s + (lane & 15) * kLtOutPitch + half * 256 + c;
          const float by = read_any ? inv : 0.0f;
#pragma unroll
          for (int k = 0; k < 32; k += 4)
            *reinterpret_cast<float4 *>(mine + k) =
                read_any ? make_float4(__uint_as_float(o[k]) * by, __uint_as_float(o[k + 1]) * by,
                                       __uint_as_float(o[k + 2]) * by, __uint_as_float(o[k + 3]) * by)
                         : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
          continue;
        }
        if (!row_ok) continue;
        if (!read_any) {
#pragma unroll
          for (int k = 0; k < 32; ++k) o[k] = 0u;
        }
        const int64_t at = out_row * 512 + half * 256 + c;
        {
          if (p.out_f32) {
#pragma unroll
            for (int k = 0; k < 32; k += 4)
              *reinterpret_cast<float4 *>(p.out_f32 + at + k) =
                  make_float4(__uint_as_float(o[k]) * inv, __uint_as_float(o[k + 1]) * inv,
                              __uint_as_float(o[k + 2]) * inv, __uint_as_float(o[k + 3]) * inv);
          }
          if (p.out_bf16) {
#pragma unroll
            for (int k = 0; k < 32; k += 8)
              *reinterpret_cast<uint4 *>(p.out_bf16 + at + k) =
                  make_uint4(pack_bf16x2(__uint_as_float(o[k]) * inv, __uint_as_float(o[k + 1]) * inv),
                             pack_bf16x2(__uint_as_float(o[k + 2]) * inv, __uint_as_float(o[k + 3]) * inv),
                             pack_bf16x2(__uint_as_float(o[k + 4]) * inv, __uint_as_float(o[k + 5]) * inv),
                             pack_bf16x2(__uint_as_float(o[k + 6]) * inv, __uint_as_float(o[k + 7]) * inv));
          }
        }
      }
      if (partial) {
        __syncwarp();
        const int first_head = head0 + (warp & 3) * 16;
        float *block = p.part_out + (out_row - (lane & 15)) * 512;  // (the warp's first row)
        for (int i = lane; i < 16 * 128; i += 32) {
          const int local = i >> 7, c4 = i & 127;
          if (first_head + local < p.Hq)
            *reinterpret_cast<float4 *>(block + (int64_t)local * 512 + c4 * 4) =
                *reinterpret_cast<const float4 *>(o_s + local * kLtOutPitch + c4 * 4);
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 4) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kLtTmemCols));
  }
  if (tid == 0 && abort_s && p.status) atomicAdd(p.status, 1);
  LT_TRACE(tid == 0, 10, 3);
}

#ifdef LSA_LT_TRACE
extern "C" __attribute__((visibility("default"))) int lsa_lt_trace_read(long long *host) {
  return (int)cudaMemcpyFromSymbol(host, lsa_lt_trace, sizeof(lsa_lt_trace));
}
#endif

int launch_latent_attend_tc(const LatentParams &p_in, cudaStream_t stream) {
  LatentParams p = p_in;
  // Runs of consecutive rows are staged by tensor-map copies when the cache can be described to one (16-byte aligned
  // base and row pitch); otherwise every tile is gathered row by row.
  CUtensorMap map_latent = {};
  p.boxes = ((uintptr_t)p.latent % 16) == 0 && (p.latent_row_stride * 2) % 16 == 0 && p.slots > 0 &&
                    make_map(&map_latent, p.latent, p.slots, 576, p.latent_row_stride, kLtKeys) == LSA_OK
                ? 1
                : 0;
  if (cudaFuncSetAttribute(latent_attend_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kLtSmem) !=
      cudaSuccess)
    return LSA_ERR_LAUNCH;
  const dim3 grid((unsigned)(p.R * p.splits), (unsigned)((p.Hq + kLatHeads - 1) / kLatHeads));
  launch(p.R <= kChainedRows, latent_attend_tc_kernel, grid, dim3(kLtThreads), kLtSmem, stream, map_latent, p);
  LSA_LAUNCH_CHECK();
  return LSA_OK;
}

}  // namespace lsa
