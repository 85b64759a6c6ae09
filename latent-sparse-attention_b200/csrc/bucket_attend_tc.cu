// The attend pass of the bucket-major attention on the fifth-generation tensor cores.
//
// A CTA owns (bucket, KV head, segment of up to 128 (row, pick) pairs) and takes the query heads of the KV head's
// group one after the other. The pairs are the M = 128 rows of both products, so a row of S and of O lives in one
// lane of tensor memory and the thread that owns the row does its softmax without talking to anyone:
//
//   S [128 x keys]  = Q_head [128 x 128] . K^T      tcgen05.mma, A = the pairs' query rows, B = the bucket's keys,
//                                                   both K-major planes of 64 dims with the 128-byte swizzle
//   P               = exp2(S - rowmax) on the row's key range, bf16, written back to shared memory
//   O [128 x 128]   = P [128 x keys] . V            A = P (K-major), B = the bucket's values AS STORED
//                                                   ([key][dim] planes: an MN-major operand)
//
//   warp 0          tensor-memory allocation; one lane issues the MMAs
//   warps 1-4       thread = row: asynchronous copy of its query row (the next head's while this head computes),
//                   softmax, normalised bf16 partial output and log-sum-exp
//
// Shared-memory operands are written by ordinary and asynchronous copies (the generic proxy), so a proxy fence stands
// before every hand-over to the tensor cores. Every wait on an mbarrier is bounded; a wait that gives up raises the
// CTA's abort flag, the CTA skips its remaining work, frees its tensor memory and leaves.
#include "bucket_attend.cuh"
#include "mma.cuh"
#include "umma.cuh"

namespace lsa {

constexpr int kTcThreads = 160;
constexpr int kTcRows = 128;                    // pairs a CTA holds: kBktSegment
constexpr int kTcPlane = 64 * 128;              // a plane of 64 rows x 128 bytes (keys or values, 64 dims)
constexpr int kTcQPlane = kTcRows * 128;        // a plane of the query tile or of P
constexpr int kTcKOff = 0;                      // K: 2 planes
constexpr int kTcVOff = 2 * kTcPlane;           // V: 2 planes
constexpr int kTcQOff = 4 * kTcPlane;           // Q: 2 buffers of 2 planes
// P takes the first plane of the head's own query buffer: the first product is over when P is written
constexpr int kTcSmem = kTcQOff + 4 * kTcQPlane + 1024;  // + room to align the base to 1,024 bytes
constexpr int kTcTmemCols = 256;                // S in columns 0-63, O in 64-191
static_assert(kBktSegment == kTcRows && kBktKeys == 64, "the tile shapes of the tensor-core attend pass");

__device__ __forceinline__ void proxy_fence() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

template <int DH>
__global__ void __launch_bounds__(kTcThreads, 2) bucket_attend_tc_kernel(BucketParams p) {
  static_assert(DH == 128, "two planes of 64 dims");
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ int32_t ids_s[kBktKeys];
  __shared__ __align__(8) uint64_t bars[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int abort_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = blockIdx.y;
  const int seg = blockIdx.x;
  if (seg >= p.seg_offsets[p.m]) return;
  const int4 info = p.segments[seg];
  const int64_t bucket = info.x;
  const int first = info.y, n_pairs = info.z;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_s = smem_u32(&bars[0]), bar_o = smem_u32(&bars[1]);

  if (tid == 0) {
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
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_s;

  // The bucket's keys and values of this KV head: chunk c of member j goes to plane c / 8, row j, 16-byte slot
  // (c % 8) ^ (j % 8) - the layout a tensor-map copy with the 128-byte swizzle would write.
  {
    const uint16_t *k_head = p.k + (int64_t)h * p.kv_head_stride, *v_head = p.v + (int64_t)h * p.kv_head_stride;
    for (int e = tid; e < kBktKeys * 16; e += kTcThreads) {
      const int row = e >> 4, chunk = e & 15;
      const int32_t id = ids_s[row];
      const bool ok = id >= 0 && id < p.slots;
      const int64_t off = ok ? (int64_t)id * p.kv_row_stride + chunk * 8 : 0;
      const uint32_t dst = (chunk >> 3) * kTcPlane + row * 128 + (((chunk & 7) ^ (row & 7)) << 4);
      cp_async_16(base + kTcKOff + dst, k_head + off, ok ? 16 : 0);
      cp_async_16(base + kTcVOff + dst, v_head + off, ok ? 16 : 0);
    }
  }
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
  const int n_keys = max(16, (n_members + 15) & ~15);  // the N of S and the K of O: whole 16-key steps

  // A worker thread is a row: TMEM lane 32 * (warp % 4) + lane is what its warp may read.
  const bool worker = warp >= 1;
  const int row = (warp & 3) * 32 + lane;
  int32_t pair = -1;
  int64_t q_row = 0;
  int lo_key = 0, hi_key = 0;
  if (worker && row < n_pairs) {
    pair = p.order[first + row];
    q_row = pair / p.top_p;
    const int64_t pos = p.positions[q_row];
    const int row_k = p.row_top_k ? min(p.row_top_k[q_row], p.top_k) : p.top_k;
    lo_key = members_below(p.sink);
    hi_key = min(members_below(max((int64_t)0, pos + 1 - p.window)), lo_key + row_k - p.starts[pair]);
  }
  // Start the copy of this row's query vector of head `hq` into buffer hq % 2 (zero-filled past the segment).
  auto issue_q = [&](int hq) {
    if (worker && hq < p.group) {
      const uint16_t *src = p.q + q_row * p.q_row_stride + (int64_t)(h * p.group + hq) * p.q_head_stride;
      const uint32_t dst0 = base + kTcQOff + (hq & 1) * 2 * kTcQPlane + row * 128;
#pragma unroll
      for (int chunk = 0; chunk < 16; ++chunk)
        cp_async_16(dst0 + (chunk >> 3) * kTcQPlane + (((chunk & 7) ^ (row & 7)) << 4), src + chunk * 8,
                    pair >= 0 ? 16 : 0);
    }
    cp_async_commit();
  };
  issue_q(0);  // (the group also closes the K/V copies above)

  for (int hq = 0; hq < p.group; ++hq) {
    const uint32_t parity = hq & 1;
    issue_q(hq + 1);
    cp_async_wait<1>();
    proxy_fence();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();  // K, V and this head's queries are in shared memory; the last head's reads of S and O are over
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (tid == 0 && !abort_s) {
      const uint32_t q_buf = base + kTcQOff + (hq & 1) * 2 * kTcQPlane;
      const uint32_t idesc = umma_idesc(n_keys);
#pragma unroll
      for (int plane = 0; plane < 2; ++plane)
#pragma unroll
        for (int k = 0; k < 4; ++k)  // 16 dims = 32 bytes further inside the swizzle atom a step
          umma_bf16(tmem_base, smem_desc_sw128(q_buf + plane * kTcQPlane) + 2 * k,
                    smem_desc_sw128(base + kTcKOff + plane * kTcPlane) + 2 * k, idesc, (plane | k) != 0);
      umma_commit(bar_s);
    }
    float m_row = -INFINITY, l_row = 0.0f;
    if (worker) {
      // (one decision a warp: the tensor-memory loads below are warp-wide instructions)
      const bool go = __all_sync(0xffffffffu, mbar_wait(bar_s, parity) && !abort_s);
      if (!go) abort_s = 1;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (go) {
        const uint32_t lane_addr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
        uint32_t r0[32], r1[32];
        tmem_load_32(lane_addr, r0);
        if (n_keys > 32) tmem_load_32(lane_addr + 32, r1);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        float s[64];
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          const float raw = c < 32 ? __uint_as_float(r0[c]) : (n_keys > 32 ? __uint_as_float(r1[c - 32]) : 0.0f);
          s[c] = (c >= lo_key && c < hi_key) ? raw * p.scale_log2 : -INFINITY;
          m_row = fmaxf(m_row, s[c]);
        }
        // P, bf16, as the K-major A operand of the second product: 16-byte slot (c / 8) ^ (row % 8) of the row
        const uint32_t p_row = base + kTcQOff + (hq & 1) * 2 * kTcQPlane + row * 128;
#pragma unroll
        for (int c8 = 0; c8 < 8; ++c8) {
          uint32_t w[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float e0 = m_row == -INFINITY ? 0.0f : fast_exp2(s[c8 * 8 + 2 * j] - m_row);
            const float e1 = m_row == -INFINITY ? 0.0f : fast_exp2(s[c8 * 8 + 2 * j + 1] - m_row);
            l_row += e0 + e1;
            w[j] = pack_bf16x2(e0, e1);
          }
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(p_row + ((c8 ^ (row & 7)) << 4)), "r"(w[0]),
                       "r"(w[1]), "r"(w[2]), "r"(w[3])
                       : "memory");
        }
      }
    }
    proxy_fence();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();  // P is in shared memory and S has been read
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (tid == 0 && !abort_s) {
      const uint32_t idesc = umma_idesc(DH, true);
      for (int k = 0; k < n_keys / 16; ++k)  // 16 keys: 32 bytes along P's rows, 16 rows (2,048 bytes) down V's planes
        umma_bf16(tmem_base + 64, smem_desc_sw128(base + kTcQOff + (hq & 1) * 2 * kTcQPlane) + 2 * k,
                  smem_desc_mn_sw128(base + kTcVOff + k * 2048, kTcPlane), idesc, k != 0);
      umma_commit(bar_o);
    }
    if (worker) {
      const bool go = __all_sync(0xffffffffu, mbar_wait(bar_o, parity) && !abort_s);
      if (!go) abort_s = 1;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (go) {
        const uint32_t lane_addr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + 64;
        const float inv = l_row > 0.0f ? 1.0f / l_row : 0.0f;
        const int64_t slot = (int64_t)pair * p.Hq + h * p.group + hq;
#pragma unroll
        for (int c0 = 0; c0 < DH; c0 += 32) {
          uint32_t r[32];
          tmem_load_32(lane_addr + c0, r);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (pair >= 0) {
            uint4 *dst = reinterpret_cast<uint4 *>(p.part_out + slot * DH + c0);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 piece;
              piece.x = pack_bf16x2(__uint_as_float(r[8 * i]) * inv, __uint_as_float(r[8 * i + 1]) * inv);
              piece.y = pack_bf16x2(__uint_as_float(r[8 * i + 2]) * inv, __uint_as_float(r[8 * i + 3]) * inv);
              piece.z = pack_bf16x2(__uint_as_float(r[8 * i + 4]) * inv, __uint_as_float(r[8 * i + 5]) * inv);
              piece.w = pack_bf16x2(__uint_as_float(r[8 * i + 6]) * inv, __uint_as_float(r[8 * i + 7]) * inv);
              dst[i] = piece;
            }
          }
        }
        if (pair >= 0)
          p.part_lse[slot] = l_row > 0.0f ? (m_row + log2f(l_row)) * 0.6931471805599453f : -INFINITY;
      }
    }
  }
  cp_async_wait<0>();
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTcTmemCols));
  }
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
