// The window and the sinks of a prefill as dense banded attention on the fifth-generation tensor cores.
//
// A CTA owns 128 consecutive query rows of ONE query head and walks the band of keys they see - from the first row's
// window start to the last row, in tiles of 128 keys, plus a tile for the sinks. The rows are the M = 128 side of both
// products, so a row of S and of O lives in one lane of tensor memory and the thread that owns the row does its
// softmax alone. The band is walked TWICE: the first walk only takes every row's maximum, the second computes
// P = exp2(S - max) and accumulates O = sum P V in tensor memory without ever rescaling it (the second product costs
// half a walk more of tensor-core time, which this path has to spare, and saves the read-modify-write of O).
//
//   warp 0      one lane streams the key and value tiles with tensor-map copies (128-byte swizzle) through a ring
//   warp 1      tensor-memory allocation; one lane issues S = Q K^T (both K-major) into one of two S buffers
//   warp 10     one lane issues O += P V with V read as stored (an MN-major operand)
//   warps 2-9   two threads a row (64 of a tile's 128 keys each): S out of tensor memory, masks on the band's edge
//               tiles only, maximum (walk one) or P in bf16 into the consumed key tile's slot (walk two), then the
//               normalised fp32 output
//
// Every wait on an mbarrier is bounded; a wait that gives up raises the CTA's abort flag and the status word, the
// roles drain, the tensor memory is freed and the CTA leaves.
#include "common.cuh"
#include "mma.cuh"
#include "umma.cuh"

namespace lsa {

constexpr int kBtRows = 128;
constexpr int kBtKeys = 128;                        // keys a tile: two planes of 64 for P, N = 128 for S
constexpr int kBtThreads = 352;                      // the copy warp, two MMA warps and eight worker warps
constexpr int kBtWorkers = 256;
constexpr int kBtStages = 3;                        // the ring of key/value tiles: deep enough to hide a tensor-map copy
constexpr int kBtPlane = kBtKeys * 128;             // 128 keys x 64 dims of bf16
constexpr int kBtQPlane = kBtRows * 128;            // 128 rows x 64 dims
constexpr int kBtStage = 4 * kBtPlane;              // K (2 planes; P lands here once S is done) and V (2 planes)
constexpr int kBtSmem = 2 * kBtQPlane + kBtStages * kBtStage + 1024;
constexpr int kBtTmemCols = 512;                    // S buffers in columns 0-127 and 128-255, O in 256-383
constexpr int kBtOCol = 256;

struct BandTcParams {
  float *out, *lse;
  int32_t *status;
  int64_t R, n_keys, first_position;
  int Hq, group, window, sink;
  float scale_log2;
};

__global__ void __launch_bounds__(kBtThreads, 1)
    band_attend_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                          const __grid_constant__ CUtensorMap map_v, BandTcParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // full / empty: a ring stage's tiles have landed / may be overwritten; s_ready / s_free: an S buffer holds a
  // product / has been read; p_ready: a stage holds P; q_full, o_done: once each.
  __shared__ __align__(8) uint64_t bars[3 * kBtStages + 2 * 2 + 2];
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int abort_s;
  __shared__ float swap_s[2][kBtRows];  // where the two threads of a row leave their maximum, then their sum
  auto workers_sync = [] { asm volatile("bar.sync 1, %0;" ::"n"(kBtWorkers) : "memory"); };
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_s = base, ring = base + 2 * kBtQPlane;
  // (kFull, kEmpty, kPReady: one a ring stage; kSReady, kSFree: one an S buffer)
  enum { kFull = 0, kEmpty = kBtStages, kPReady = 2 * kBtStages, kSReady = 3 * kBtStages, kSFree = 3 * kBtStages + 2 };
  auto bar = [&](int kind, int i) { return smem_u32(&bars[kind + i]); };
  const uint32_t q_full = smem_u32(&bars[3 * kBtStages + 4]), o_done = smem_u32(&bars[3 * kBtStages + 5]);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row0 = (int64_t)blockIdx.x * kBtRows;
  const int head = blockIdx.y, kv_head = head / p.group;
  const int64_t pos0 = p.first_position + row0;
  const int64_t pos_last = min(pos0 + kBtRows - 1, p.first_position + p.R - 1);
  const int64_t band_first = max((int64_t)0, pos0 + 1 - p.window) / kBtKeys * kBtKeys;
  const int band_tiles = (int)((pos_last - band_first) / kBtKeys) + 1;
  const bool has_sinks = p.sink > 0 && band_first > 0;
  const int tiles = band_tiles + (has_sinks ? 1 : 0);  // tile 0 is the sinks when there are any
  auto key0_of = [&](int tile) {
    return has_sinks ? (tile == 0 ? (int64_t)0 : band_first + (int64_t)(tile - 1) * kBtKeys)
                     : band_first + (int64_t)tile * kBtKeys;
  };

  if (threadIdx.x == 0) {
    for (int i = 0; i < kBtStages; ++i) {
      mbar_init(bar(kFull, i), 1);
      mbar_init(bar(kEmpty, i), 1);
      mbar_init(bar(kPReady, i), kBtWorkers);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(kSReady, i), 1);
      mbar_init(bar(kSFree, i), kBtWorkers);
    }
    mbar_init(q_full, 1);
    mbar_init(o_done, 1);
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)),
                 "r"(kBtTmemCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_s;

  if (warp == 0) {
    if (lane == 0) {
      // the query tile once, then the ring: keys alone on the first walk, keys and values on the second
      mbar_expect_tx(q_full, 2 * kBtQPlane);
      tma_load_2d(q_s, &map_q, q_full, head * 128, (int)row0);
      tma_load_2d(q_s + kBtQPlane, &map_q, q_full, head * 128 + 64, (int)row0);
      uint32_t phases = 0;  // a parity bit a stage
      for (int n = 0; n < 2 * tiles && !abort_s; ++n) {
        const int stage = n % kBtStages, tile = n % tiles;
        const bool second = n >= tiles;
        if (n >= kBtStages) {
          if (!mbar_wait(bar(kEmpty, stage), (phases >> stage) & 1)) {
            abort_s = 1;
            break;
          }
          phases ^= 1u << stage;
        }
        const uint32_t dst = ring + stage * kBtStage;
        const int y = (int)key0_of(tile), x = kv_head * 128;
        mbar_expect_tx(bar(kFull, stage), second ? 4 * kBtPlane : 2 * kBtPlane);
        tma_load_2d(dst, &map_k, bar(kFull, stage), x, y);
        tma_load_2d(dst + kBtPlane, &map_k, bar(kFull, stage), x + 64, y);
        if (second) {
          tma_load_2d(dst + 2 * kBtPlane, &map_v, bar(kFull, stage), x, y);
          tma_load_2d(dst + 3 * kBtPlane, &map_v, bar(kFull, stage), x + 64, y);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = umma_idesc(kBtKeys);
      uint32_t full_phases = 0, free_phases = 0;  // a parity bit a stage (or S buffer)
      bool ok = mbar_wait(q_full, 0);
      for (int n = 0; n < 2 * tiles && ok && !abort_s; ++n) {
        const int stage = n % kBtStages, sbuf = n & 1;
        const bool second = n >= tiles;
        ok = mbar_wait(bar(kFull, stage), (full_phases >> stage) & 1);
        if (!ok) break;
        full_phases ^= 1u << stage;
        if (n >= 2) {
          ok = mbar_wait(bar(kSFree, sbuf), (free_phases >> sbuf) & 1);
          if (!ok) break;
          free_phases ^= 1u << sbuf;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t k_tile = ring + stage * kBtStage;
#pragma unroll
        for (int plane = 0; plane < 2; ++plane)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16(tmem_base + sbuf * kBtKeys, smem_desc_sw128(q_s + plane * kBtQPlane) + 2 * k,
                      smem_desc_sw128(k_tile + plane * kBtPlane) + 2 * k, idesc_s, (plane | k) != 0);
        umma_commit(bar(kSReady, sbuf));
        if (!second) umma_commit(bar(kEmpty, stage));  // on the first walk the keys are all a stage holds
      }
      if (!ok) abort_s = 1;
    }
  } else if (warp == kBtThreads / 32 - 1) {
    // The second products have an issuing lane of their own: O += P V of tile n once the workers have written its P.
    // (One lane for both products waited for P of tile n - 1 before it could issue S of tile n + 1.) P exists only
    // after S of the tile was read, so the stage's keys are spent too when this product has run.
    if (lane == 0) {
      const uint32_t idesc_o = umma_idesc(128, true);
      uint32_t p_phases = 0;
      bool ok = true;
      for (int n = tiles; n < 2 * tiles && ok && !abort_s; ++n) {
        const int stage = n % kBtStages;
        ok = mbar_wait(bar(kPReady, stage), (p_phases >> stage) & 1);
        if (!ok) break;
        p_phases ^= 1u << stage;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t p_tile = ring + stage * kBtStage, v_tile = p_tile + 2 * kBtPlane;
#pragma unroll
        for (int k = 0; k < kBtKeys / 16; ++k)  // P: two planes of 64 keys; V: 16 keys are 2,048 bytes down a plane
          umma_bf16(tmem_base + kBtOCol, smem_desc_sw128(p_tile + (k >> 2) * kBtQPlane) + 2 * (k & 3),
                    smem_desc_mn_sw128(v_tile + k * 2048, kBtPlane), idesc_o, (n > tiles || k > 0) ? 1u : 0u);
        umma_commit(bar(kEmpty, stage));
      }
      if (!ok) abort_s = 1;
      umma_commit(o_done);
    }
  } else {
    // Workers: TMEM lane 32 * (warp % 4) + lane is this thread's row, and a row has two threads (warps w and w + 4):
    // each takes 64 of a tile's 128 keys and 64 of O's 128 columns. Their maxima and sums meet once a walk, not once
    // a tile. (With one thread a row a step ran some 800 dependent instructions on a scheduler that had nothing
    // else to issue: that, not the tensor pipe or the copies, set the pace.)
    const int half = (warp - 2) >> 2;
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
    const int64_t pos = pos0 + row;
    const bool live = row0 + row < p.R;
    const int64_t start = max((int64_t)0, pos + 1 - p.window);
    const int64_t sink_end = min((int64_t)p.sink, start);
    // a tile inside every row's window, below every row's position and inside the cache needs no masks
    const int64_t inside_from = max((int64_t)0, pos_last + 1 - p.window);
    const bool rows_whole = pos0 + kBtRows <= p.first_position + p.R;
    uint32_t ready_phases = 0;
    float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY}, l4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    float m_row = 0.0f;
    bool go = true;
    for (int n = 0; n < 2 * tiles; ++n) {  // (a warp that gave up still walks on: it owes the others two barriers)
      const int stage = n % kBtStages, sbuf = n & 1, tile = n % tiles;
      const bool second = n >= tiles;
      if (n == tiles) {  // between the walks: the row's maximum is the larger of its two threads'
        float m = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
        swap_s[half][row] = m;
        workers_sync();
        m = fmaxf(m, swap_s[half ^ 1][row]);
        m_row = m == -INFINITY ? 0.0f : m * p.scale_log2;  // the offset of every exponent
        workers_sync();
      }
      go = go && __all_sync(0xffffffffu, mbar_wait(bar(kSReady, sbuf), (ready_phases >> sbuf) & 1) && !abort_s);
      if (!go) continue;
      ready_phases ^= 1u << sbuf;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      uint32_t sv[64];
      tmem_load_32(lane_addr + sbuf * kBtKeys + half * 64, *reinterpret_cast<uint32_t(*)[32]>(&sv[0]));
      tmem_load_32(lane_addr + sbuf * kBtKeys + half * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&sv[32]));
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar(kSFree, sbuf)) : "memory");
      const int64_t key0 = key0_of(tile);
      const bool is_sinks = has_sinks && tile == 0;
      const bool inside = !is_sinks && rows_whole && key0 >= inside_from && key0 + kBtKeys - 1 <= pos0 &&
                          key0 + kBtKeys <= p.n_keys;
      if (!inside) {
        // the row's bounds as columns of this thread's half of the tile
        const int64_t col0 = key0 + half * 64;
        auto rel = [&](int64_t key) { return (int)max((int64_t)-1, min((int64_t)64, key - col0)); };
        const int end = live ? rel(p.n_keys) : 0;                   // columns at or past it are outside the cache
        const int sinks = rel(sink_end);                             // columns below it are the row's sinks
        const int from = is_sinks ? 64 : rel(start), to = is_sinks ? -1 : rel(pos);  // the window: from <= c <= to
        // The row's valid columns as a 64-bit word. A group of 8 columns that every row of the warp sees whole is
        // left alone, and one that none sees is cleared; the others take a bit test and a select a column (no
        // branches on a lane's own bounds: they would diverge lane by lane, 64 times a tile).
        auto below = [](int x) { return x >= 64 ? ~0ull : (x <= 0 ? 0ull : (1ull << x) - 1ull); };
        const unsigned long long valid = ((below(to + 1) & ~below(from)) | below(sinks)) & below(end);
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const uint32_t bits = (uint32_t)(valid >> (8 * g)) & 0xffu;
          if (__all_sync(0xffffffffu, bits == 0xffu)) continue;
          if (__all_sync(0xffffffffu, bits == 0u)) {
#pragma unroll
            for (int c = 0; c < 8; ++c) sv[8 * g + c] = 0xff800000u;  // -inf
          } else {
#pragma unroll
            for (int c = 0; c < 8; ++c) sv[8 * g + c] = (bits & (1u << c)) ? sv[8 * g + c] : 0xff800000u;
          }
        }
      }
      if (!second) {
#pragma unroll
        for (int c = 0; c < 64; ++c) m4[c & 3] = fmaxf(m4[c & 3], __uint_as_float(sv[c]));
      } else {
        const uint32_t p_row = ring + stage * kBtStage + half * kBtQPlane + row * 128;  // the plane of this half's keys
#pragma unroll
        for (int c8 = 0; c8 < 8; ++c8) {
          uint32_t w[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float e0 = fast_exp2(fmaf(__uint_as_float(sv[c8 * 8 + 2 * j]), p.scale_log2, -m_row));
            const float e1 = fast_exp2(fmaf(__uint_as_float(sv[c8 * 8 + 2 * j + 1]), p.scale_log2, -m_row));
            l4[j] += e0 + e1;
            w[j] = pack_bf16x2(e0, e1);
          }
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(p_row + ((c8 ^ (row & 7)) << 4)),
                       "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3])
                       : "memory");
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar(kPReady, stage)) : "memory");
      }
    }
    // the row's sum is the sum of its two threads'
    float l_row = (l4[0] + l4[1]) + (l4[2] + l4[3]);
    swap_s[half][row] = l_row;
    workers_sync();
    l_row += swap_s[half ^ 1][row];
    go = __all_sync(0xffffffffu, go && mbar_wait(o_done, 0) && !abort_s);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (go) {
      const float inv = l_row > 0.0f ? 1.0f / l_row : 0.0f;
      const int64_t out_row = (row0 + row) * p.Hq + head;
#pragma unroll
      for (int c0 = half * 64; c0 < half * 64 + 64; c0 += 32) {
        uint32_t r[32];
        tmem_load_32(lane_addr + kBtOCol + c0, r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (live) {
          float4 *dst = reinterpret_cast<float4 *>(p.out + out_row * 128 + c0);
#pragma unroll
          for (int i = 0; i < 8; ++i)
            dst[i] = make_float4(__uint_as_float(r[4 * i]) * inv, __uint_as_float(r[4 * i + 1]) * inv,
                                 __uint_as_float(r[4 * i + 2]) * inv, __uint_as_float(r[4 * i + 3]) * inv);
        }
      }
      if (live && half == 0) p.lse[out_row] = l_row > 0.0f ? (m_row + log2f(l_row)) * 0.6931471805599453f : -INFINITY;
    } else {
      abort_s = 1;
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kBtTmemCols));
  }
  if (threadIdx.x == 0 && abort_s && p.status) atomicAdd(p.status, 1);
}

// Launches the tensor-core band kernel; the caller has checked dh == 128 and the alignments a tensor map needs.
int launch_band_attend_tc(const uint16_t *q, int64_t R, int Hq, int64_t q_row_stride, const uint16_t *k,
                          const uint16_t *v, int64_t n_keys, int Hkv, int64_t kv_row_stride, int64_t first_position,
                          int window, int sink, float scale, float *out, float *lse, int32_t *status,
                          cudaStream_t stream) {
  CUtensorMap map_q, map_k, map_v;
  int rc = make_map(&map_q, q, R, (int64_t)Hq * 128, q_row_stride, kBtRows);
  if (rc != LSA_OK) return rc;
  rc = make_map(&map_k, k, n_keys, (int64_t)Hkv * 128, kv_row_stride, kBtKeys);
  if (rc != LSA_OK) return rc;
  rc = make_map(&map_v, v, n_keys, (int64_t)Hkv * 128, kv_row_stride, kBtKeys);
  if (rc != LSA_OK) return rc;
  BandTcParams p = {};
  p.out = out, p.lse = lse, p.status = status;
  p.R = R, p.n_keys = n_keys, p.first_position = first_position;
  p.Hq = Hq, p.group = Hq / Hkv, p.window = window, p.sink = sink;
  p.scale_log2 = scale * 1.4426950408889634f;
  if (cudaFuncSetAttribute(band_attend_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kBtSmem) != cudaSuccess)
    return LSA_ERR_LAUNCH;
  const dim3 grid((unsigned)((R + kBtRows - 1) / kBtRows), (unsigned)Hq);
  band_attend_tc_kernel<<<grid, kBtThreads, kBtSmem, stream>>>(map_q, map_k, map_v, p);
  LSA_LAUNCH_CHECK();
  return LSA_OK;
}

}  // namespace lsa
