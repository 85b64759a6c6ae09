// The bucket scan of a prefill chunk on the fifth-generation tensor cores: which buckets of every query row score at
// or above the row's threshold. The scores are never written: they are made in tensor memory, tested there and
// forgotten; what leaves the kernel is, per row, a few short lists of survivors (score, bucket).
//
// A CTA owns 128 query rows and a span of 128-bucket tiles. Its rows are the M side of every product (one shared-memory
// plane: the index space has 64 dims), a tile of bf16 centroids the N side, and a tile's scores S [128 x 128] land in
// one of four accumulators of tensor memory, a row a lane. Two threads own a lane, one for each half of a tile's
// columns; each appends the buckets at or above the row's bar to a list of its own, so nothing is contended.
//
//   warp 0      one lane streams centroid tiles with tensor-map copies through a six-stage ring
//   warp 1      tensor-memory allocation; one lane issues the four products of a tile (K = 64)
//   warps 2-9   two threads a row: threshold, then the tiles' scores out of tensor memory and the test
//
// The threshold comes from the same machinery: the first four tiles a CTA multiplies are SAMPLES - every s-th
// centroid, read through a second tensor map whose rows are s centroids apart - and the row's two threads bisect for
// the value that a chosen number of its 512 sample scores reach, re-reading them from tensor memory at every step.
// The target count is set so that about `factor` x top_p buckets of the whole row survive; the pick that follows
// rescores the best of them in fp32 and proves, row by row, that nothing outside the lists could have been picked.
#include <cuda.h>

#include "scan_select.cuh"
#include "umma.cuh"

namespace lsa {

constexpr int kScanThreads = 320;
constexpr int kScanStages = 6;  // (with the query plane: over half an SM's shared memory, so one CTA an SM owns all 512 columns)
constexpr int kScanTile = 128 * 128;  // bytes of a tile: 128 rows x 64 dims of bf16
constexpr int kScanStaging = 8 * 32 * 32 * 4;  // a consumer warp's 32 x 32 scores, a word a lane a column
constexpr int kScanSmem = (1 + kScanStages) * kScanTile + kScanStaging + 1024;
constexpr int kScanSampleTiles = 4;   // 512 samples a row
constexpr int kScanBisections = 10;  // the threshold to a 1,024th of the score range: the margin is eight times that
constexpr uint32_t kScanSpinLimit = 1u << 22;

__device__ __forceinline__ bool scan_try(uint32_t bar, uint32_t parity) {
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

#ifdef LSA_SCAN_TRACE
// A clock trace of the first CTA's first 64 steps (a tuning aid, compiled only on request): event e of step n.
__device__ long long lsa_scan_trace[8 * 64];
#define SCAN_TRACE(cond, e, n)                                                                                  \
  do {                                                                                                          \
    if (blockIdx.x == 0 && blockIdx.y == 0 && (cond) && (n) < 64) lsa_scan_trace[(e) * 64 + (n)] = clock64(); \
  } while (0)
#else
#define SCAN_TRACE(cond, e, n) \
  do {                         \
  } while (0)
#endif

__device__ __forceinline__ void scan_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__global__ void __launch_bounds__(kScanThreads, 1)
    scan_survivors_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_c,
                          const __grid_constant__ CUtensorMap map_sample, ScanParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // full / empty: a ring stage's tile has landed / has been multiplied; acc_full / acc_empty: an accumulator holds a
  // tile's scores / has been read; q_full: the query rows are in place.
  __shared__ __align__(8) uint64_t bars[2 * kScanStages + 2 * 4 + 1];
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int abort_s, stop_s;  // a wait gave up / no row of the CTA is left to scan
  __shared__ int dead_s;
  __shared__ int count_s[2][2][128];  // [step parity][half][row]: the halves of a row's bisection count
  auto full = [&](int i) { return smem_u32(&bars[i]); };
  auto empty = [&](int i) { return smem_u32(&bars[kScanStages + i]); };
  auto acc_full = [&](int i) { return smem_u32(&bars[2 * kScanStages + i]); };
  auto acc_empty = [&](int i) { return smem_u32(&bars[2 * kScanStages + 4 + i]); };
  const uint32_t q_full = smem_u32(&bars[2 * kScanStages + 8]);
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_s = base, ring = base + kScanTile;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row0 = (int64_t)blockIdx.x * 128;
  const int span = blockIdx.y;
  // the tiles of this span, and of them only those some row of the CTA can see
  const int tiles_all = (int)((p.m + 127) / 128);
  const int per_span = (tiles_all + p.spans - 1) / p.spans;
  const int t0 = span * per_span;
  const int widest = p.tile_visible[blockIdx.x];  // the widest visible count among the CTA's rows that take this path
  int t1 = min(min(tiles_all, t0 + per_span), (widest + 127) / 128);
  if (t1 < t0) t1 = t0;
  const int steps = widest > 0 ? kScanSampleTiles + (t1 - t0) : 0;
  const int stride = p.sample_stride;  // centroids between two samples

  if (threadIdx.x == 0) {
    for (int i = 0; i < kScanStages; ++i) {
      mbar_init(full(i), 1);
      mbar_init(empty(i), 1);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(acc_full(i), 1);
      mbar_init(acc_empty(i), 256);
    }
    mbar_init(q_full, 1);
    abort_s = 0, stop_s = 0, dead_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)),
                 "n"(512));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_s;

  auto wait = [&](uint32_t b, uint32_t parity) {
    bool done = false;
    for (uint32_t spin = 0; spin < kScanSpinLimit && !done && !abort_s && !stop_s; ++spin) done = scan_try(b, parity);
    if (!done && !stop_s) abort_s = 1;
    return done;
  };

  if (warp == 0) {
    if (lane == 0 && steps > 0) {
      mbar_expect_tx(q_full, kScanTile);
      tma_load_2d(q_s, &map_q, q_full, 0, (int)row0);
      int armed = 0;
      for (int n = 0; n < steps; ++n) {
        const int s = n % kScanStages;
        if (n >= kScanStages && !wait(empty(s), ((n / kScanStages) - 1) & 1)) break;
        SCAN_TRACE(true, 0, n);
        mbar_expect_tx(full(s), kScanTile);
        if (n < kScanSampleTiles)  // a row of the sample map is every stride-th centroid
          tma_load_2d(ring + s * kScanTile, &map_sample, full(s), 0, n * 128);
        else
          tma_load_2d(ring + s * kScanTile, &map_c, full(s), 0, (t0 + n - kScanSampleTiles) * 128);
        armed = n + 1;
      }
      if (abort_s || stop_s)  // leave only once the copies in flight have landed (bounded)
        for (int n = max(0, armed - kScanStages); n < armed; ++n) {
          bool done = false;
          for (uint32_t spin = 0; spin < kScanSpinLimit && !done; ++spin)
            done = scan_try(full(n % kScanStages), (n / kScanStages) & 1);
        }
    }
  } else if (warp == 1) {
    if (lane == 0 && steps > 0) {
      constexpr uint32_t idesc = umma_idesc(128);
      bool ok = wait(q_full, 0);
      for (int n = 0; n < steps && ok; ++n) {
        const int s = n % kScanStages, a = n & 3;
        ok = wait(full(s), (n / kScanStages) & 1);
        SCAN_TRACE(true, 1, n);
        if (ok && n >= 4) ok = wait(acc_empty(a), ((n >> 2) - 1) & 1);
        SCAN_TRACE(true, 2, n);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t desc_a = smem_desc_sw128(q_s), desc_b = smem_desc_sw128(ring + s * kScanTile);
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_bf16(tmem_base + a * 128, desc_a + 2 * k, desc_b + 2 * k, idesc, k != 0);
        umma_commit(empty(s));
        umma_commit(acc_full(a));
      }
      // whatever was issued completes before the tensor memory is given back
      umma_commit(q_full);
      bool done = false;
      for (uint32_t spin = 0; spin < kScanSpinLimit && !done; ++spin) done = scan_try(q_full, 1);
    }
  } else if (steps > 0) {
    const int quad = warp & 3, half = (warp - 2) >> 2;
    const int in_tile = quad * 32 + lane;
    const int64_t row = row0 + in_tile;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
    const bool live = row < p.R && p.flags[row] == 0;  // (flagged rows take the exact scan instead)
    const int visible = live ? min(max(p.visible[row], 0), (int)p.m) : 0;
    int visible_now = visible;  // 0 once the row is handed to the exact scan
    const int keep = live ? (p.row_keep ? min(p.row_keep[row], p.keep) : p.keep) : 0;
    const float norm = live ? p.norms[row] : 0.0f;
    const float widest_rho = p.radius ? *p.radius : 1.0f;
    // ---- the threshold: the value that `target` of the row's visible samples reach. Whatever the waits say, every
    // step below is walked by both warps of a quarter, so neither is left at their barrier.
    bool alive = true;
    for (int a = 0; a < kScanSampleTiles && alive; ++a) alive = __all_sync(0xffffffffu, wait(acc_full(a), 0));
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    SCAN_TRACE(warp == 2 && lane == 0, 5, 1);
    const int samples = min(kScanSampleTiles * 128, (visible + stride - 1) / stride);
    const int target = min(samples, max(1, (int)(((int64_t)p.factor * keep * samples + visible - 1) /
                                                   max(visible, 1))));
    const int mine = min(max(samples - half * 256, 0), 256);  // of this thread's 256 sample columns, those that count
    float lo = -1.001f * norm * widest_rho - 1e-30f, hi = 1.001f * norm * widest_rho + 1e-30f;
#pragma unroll 1
    for (int it = 0; it < kScanBisections; ++it) {
      const float mid = 0.5f * (lo + hi);
      int c0 = 0, c1 = 0, c2 = 0, c3 = 0;
#pragma unroll 1
      for (int c = 0; c < 256; c += 32) {
        uint32_t v[32];
        tmem_load_32(lane_addr + half * 256 + c, v);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (c + 32 <= mine) {
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            c0 += __uint_as_float(v[i]) >= mid, c1 += __uint_as_float(v[i + 1]) >= mid;
            c2 += __uint_as_float(v[i + 2]) >= mid, c3 += __uint_as_float(v[i + 3]) >= mid;
          }
        } else if (c < mine) {
#pragma unroll
          for (int i = 0; i < 32; ++i) c0 += (c + i < mine) & (__uint_as_float(v[i]) >= mid);
        }
      }
      count_s[it & 1][half][in_tile] = c0 + c1 + c2 + c3;
      asm volatile("bar.sync %0, 64;" ::"r"(1 + quad) : "memory");
      const int count = count_s[it & 1][0][in_tile] + count_s[it & 1][1][in_tile];
      if (count >= target) lo = mid; else hi = mid;
    }
    SCAN_TRACE(warp == 2 && lane == 0, 5, 2);
    const float threshold = live && samples > 0 ? lo : INFINITY;
    // A bucket is listed when its score PLUS ITS OWN SLACK reaches the threshold: whatever the scan drops has a
    // true score under the threshold.
    const float bar_score = threshold;
    if (span == 0 && half == 0 && row < p.R) p.bars[row] = bar_score;
    // How many buckets would be listed, by the samples (less a typical slack): where the row's scores lie so close
    // together that far more reach the threshold than the pick has room for (half as much again: the estimate is a
    // noisy one), listing them is wasted work and the row is flagged here and now.
    {
      int reach = 0;
#pragma unroll 1
      for (int c = 0; c < 256; c += 32) {  // (every lane walks every step: the loads are the warp's)
        uint32_t v[32];
        tmem_load_32(lane_addr + half * 256 + c, v);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int i = 0; i < 32; ++i) reach += (c + i < mine) & (__uint_as_float(v[i]) >= bar_score - norm * scan_slack(0.5f * widest_rho));
      }
      count_s[0][half][in_tile] = reach;
      asm volatile("bar.sync %0, 64;" ::"r"(1 + quad) : "memory");
      reach = count_s[0][0][in_tile] + count_s[0][1][in_tile];
      const bool crowded = live && (float)reach * (float)visible > 1.5f * (float)p.room * (float)max(samples, 1);
      if (crowded && half == 0) {
        if (span == 0) p.flags[row] = 1;
        atomicAdd(&dead_s, 1);
      }
      if (!live && half == 0) atomicAdd(&dead_s, 1);
      if (crowded) visible_now = 0;
    }
    asm volatile("bar.sync 5, 256;" ::: "memory");
    // With three quarters of its rows gone a CTA's scan is mostly wasted: the rest go to the exact scan too, and the
    // CTA stops (every CTA of these rows counts the same, and every consumer thread writes the same).
    if (dead_s >= 96) {
      stop_s = 1;
      if (live && visible_now && half == 0 && span == 0) p.flags[row] = 1;
      visible_now = 0;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    for (int a = 0; a < kScanSampleTiles; ++a) scan_arrive(acc_empty(a));
    // ---- the scan: this thread's half of every tile's columns
    volatile uint32_t *stage = reinterpret_cast<volatile uint32_t *>(smem_raw + (base - smem_u32(smem_raw)) +
                                                                     (1 + kScanStages) * kScanTile) +
                               (warp - 2) * 1024 + lane;
    const int64_t list_at = (row * p.spans + span) * 2 + half;
    int2 *list = p.survivors + list_at * p.cap;
    int found = 0;
    for (int n = kScanSampleTiles; n < steps && alive && !stop_s; ++n) {
      const int a = n & 3;
      alive = __all_sync(0xffffffffu, wait(acc_full(a), (n >> 2) & 1));
      if (!alive) break;  // (a wait that gave up, or the CTA stopped)
      SCAN_TRACE(warp == 2 && lane == 0, 3, n);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int id0 = (t0 + n - kScanSampleTiles) * 128 + half * 64;
#pragma unroll 1
      for (int c = 0; c < 64; c += 32) {
        uint32_t v[32];
        tmem_load_32(lane_addr + a * 128 + half * 64 + c, v);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        // Which of the 32 scores reach the bar, as a word of bits; the scores themselves go to shared memory (a
        // column a row of 32 lanes, so no two lanes share a bank), where a hit's score can be read by its column.
        // (lane l fetches bucket l's length; every lane then takes each bucket's by shuffle)
        const int mine_id = id0 + c + lane;
        const float rho_l = p.lengths ? (mine_id < p.m ? __ldg(p.lengths + mine_id) : 0.0f) : widest_rho;
        const float slack_l = scan_slack(rho_l);
        uint32_t m0 = 0, m1 = 0, m2 = 0, m3 = 0;
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          stage[(i + 0) * 32] = v[i + 0], stage[(i + 1) * 32] = v[i + 1];
          stage[(i + 2) * 32] = v[i + 2], stage[(i + 3) * 32] = v[i + 3];
          const float s0 = __shfl_sync(0xffffffffu, slack_l, i + 0), s1 = __shfl_sync(0xffffffffu, slack_l, i + 1);
          const float s2 = __shfl_sync(0xffffffffu, slack_l, i + 2), s3 = __shfl_sync(0xffffffffu, slack_l, i + 3);
          m0 |= (fmaf(s0, norm, __uint_as_float(v[i + 0])) >= bar_score ? 1u : 0u) << (i + 0);
          m1 |= (fmaf(s1, norm, __uint_as_float(v[i + 1])) >= bar_score ? 1u : 0u) << (i + 1);
          m2 |= (fmaf(s2, norm, __uint_as_float(v[i + 2])) >= bar_score ? 1u : 0u) << (i + 2);
          m3 |= (fmaf(s3, norm, __uint_as_float(v[i + 3])) >= bar_score ? 1u : 0u) << (i + 3);
        }
        const int seen = visible_now - (id0 + c);  // of these 32 buckets, those the row sees
        uint32_t hits = (m0 | m1) | (m2 | m3);
        hits = seen >= 32 ? hits : (seen <= 0 ? 0u : hits & ((1u << seen) - 1u));
        while (hits) {
          const int i = __ffs(hits) - 1;
          hits &= hits - 1;
          if (found < p.cap) list[found] = make_int2((int)stage[i * 32], id0 + c + i);
          ++found;
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      scan_arrive(acc_empty(a));
      SCAN_TRACE(warp == 2 && lane == 0, 4, n);
    }
    if (row < p.R) p.counts[list_at] = alive || stop_s ? found : p.cap + 1;  // (a cut scan counts as an overflow)
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(512));
  }
  if (threadIdx.x == 0 && abort_s && p.status) atomicAdd(p.status, 1);
  // a CTA with nothing to scan still owes its rows their (empty) counts
  if (steps == 0 && warp >= 2) {
    const int64_t row = row0 + (warp & 3) * 32 + lane;
    const int half = (warp - 2) >> 2;
    if (row < p.R) {
      p.counts[(row * p.spans + span) * 2 + half] = 0;
      if (span == 0 && half == 0) p.bars[row] = INFINITY;
    }
  }
}

#ifdef LSA_SCAN_TRACE
extern "C" __attribute__((visibility("default"))) int lsa_scan_trace_read(long long *host) {
  return (int)cudaMemcpyFromSymbol(host, lsa_scan_trace, sizeof(lsa_scan_trace));
}
#endif

int launch_scan_survivors(const ScanParams &p, int64_t padded_rows, cudaStream_t stream) {
  CUtensorMap map_q, map_c, map_sample;
  int rc = make_map(&map_q, p.queries_bf16, padded_rows, 64, 64, 128);
  if (rc != LSA_OK) return rc;
  rc = make_map(&map_c, p.centroids_bf16, p.m, 64, 64, 128);
  if (rc != LSA_OK) return rc;
  // every stride-th centroid: the same matrix read with rows `stride` centroids apart
  rc = make_map(&map_sample, p.centroids_bf16, (p.m + p.sample_stride - 1) / p.sample_stride, 64,
                (int64_t)64 * p.sample_stride, 128);
  if (rc != LSA_OK) return rc;
  if (cudaFuncSetAttribute(scan_survivors_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kScanSmem) != cudaSuccess)
    return LSA_ERR_LAUNCH;
  const dim3 grid((unsigned)(padded_rows / 128), (unsigned)p.spans);
  scan_survivors_kernel<<<grid, kScanThreads, kScanSmem, stream>>>(map_q, map_c, map_sample, p);
  LSA_LAUNCH_CHECK();
  return LSA_OK;
}

}  // namespace lsa
