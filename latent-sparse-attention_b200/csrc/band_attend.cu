// The local part of a prefill's read - each query's sliding window and the sinks - as dense banded attention.
//
// Consecutive query rows read almost the same recent keys, so unlike the selected keys (one gather a row) the window
// is a shared band: a CTA takes 16 consecutive query rows of one KV head, one warp a query head of the group, and
// streams the band's K/V tiles (64 keys) through shared memory once for all of them. Scores and the weighted sum run
// on mma.m16n8k16 with the queries as M; softmax is online in fp32. The result is a PARTIAL read: normalised output
// and log-sum-exp per (row, head), which lsa_sparse_attend takes as its starting state and extends with the
// gathered keys.
#include "common.cuh"
#include "mma.cuh"

namespace lsa {

constexpr int kBandRows = 16;  // query rows a CTA
constexpr int kBandKeys = 64;  // keys a tile

struct BandParams {
  const uint16_t *q, *k, *v;
  float *out, *lse;
  int64_t R, n_keys, first_position, q_row_stride, q_head_stride, kv_row_stride, kv_head_stride;
  int Hq, Hkv, group, window, sink;
  float scale_log2;
};

// grid (ceil(R / 16), Hkv, ceil(group / 8)); blockDim = min(group, 8) * 32. Row i of the call sits at position first_position + i and KV
// row p holds position p.
template <int DH>
__global__ void band_attend_kernel(BandParams p) {
  constexpr int ROW_BYTES = DH * 2, CHUNKS = ROW_BYTES / 16, KSTEPS = DH / 16;
  constexpr int TILE_BYTES = kBandKeys * ROW_BYTES;
  extern __shared__ __align__(128) unsigned char smem_raw[];  // 2 stages x (K tile, V tile)
  const uint32_t smem_base = smem_u32(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int64_t row0 = (int64_t)blockIdx.x * kBandRows;
  const int h = blockIdx.y;
  // At most eight heads of the group a CTA (blockIdx.z takes the rest); a warp past the group mirrors the last head
  // so that it still takes part in the loads and barriers, and writes nothing.
  const int in_group = blockIdx.z * 8 + warp;
  const bool real_head = in_group < p.group;
  const int head = h * p.group + (real_head ? in_group : p.group - 1);
  const int64_t pos0 = p.first_position + row0;              // position of the tile's first row
  const int64_t pos_last = min(pos0 + kBandRows - 1, p.first_position + p.R - 1);
  // The band of the tile: from the first row's window start to the last row, in whole tiles; tile -1 is the sinks.
  const int64_t band_first = max((int64_t)0, pos0 + 1 - p.window) / kBandKeys * kBandKeys;
  const int tiles = (int)((pos_last - band_first) / kBandKeys) + 1;
  const bool has_sinks = p.sink > 0 && band_first > 0;
  const int first_tile = has_sinks ? -1 : 0;
  const uint16_t *k_head = p.k + (int64_t)h * p.kv_head_stride, *v_head = p.v + (int64_t)h * p.kv_head_stride;

  auto load_tile = [&](int tile, int stage) {
    const int64_t key0 = tile < 0 ? 0 : band_first + (int64_t)tile * kBandKeys;
    const uint32_t dst0 = smem_base + stage * 2 * TILE_BYTES;
    for (int e = threadIdx.x; e < kBandKeys * CHUNKS; e += blockDim.x) {
      const int row = e / CHUNKS, chunk = e - row * CHUNKS;
      const int64_t key = key0 + row;
      const bool ok = key < p.n_keys && (tile >= 0 || row < p.sink);
      const int64_t off = ok ? key * p.kv_row_stride + chunk * 8 : 0;
      const uint32_t dst = dst0 + row * ROW_BYTES + ((chunk ^ (row & 7)) << 4);
      cp_async_16(dst, k_head + off, ok ? 16 : 0);
      cp_async_16(dst + TILE_BYTES, v_head + off, ok ? 16 : 0);
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };

  // Q as the A operand: thread (g, t) holds rows g and g + 8, dims t*2, t*2+1 (+8) of each 16-dim step.
  uint32_t qa[KSTEPS][4];
  {
    const int64_t ra = row0 + g, rb = row0 + g + 8;
    const uint16_t *qa_row = p.q + ra * p.q_row_stride + (int64_t)head * p.q_head_stride;
    const uint16_t *qb_row = p.q + rb * p.q_row_stride + (int64_t)head * p.q_head_stride;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      const int c = ks * 16 + t * 2;
      qa[ks][0] = ra < p.R ? *reinterpret_cast<const uint32_t *>(qa_row + c) : 0u;
      qa[ks][1] = rb < p.R ? *reinterpret_cast<const uint32_t *>(qb_row + c) : 0u;
      qa[ks][2] = ra < p.R ? *reinterpret_cast<const uint32_t *>(qa_row + c + 8) : 0u;
      qa[ks][3] = rb < p.R ? *reinterpret_cast<const uint32_t *>(qb_row + c + 8) : 0u;
    }
  }
  float o[DH / 8][4];
#pragma unroll
  for (int n = 0; n < DH / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
  const int64_t pos_a = pos0 + g, pos_b = pos0 + g + 8;  // positions of this thread's two rows

  load_tile(first_tile, 0);
  for (int tile = first_tile; tile < tiles; ++tile) {
    const int stage = (tile - first_tile) & 1;
    if (tile + 1 < tiles) {
      load_tile(tile + 1, stage ^ 1);
      asm volatile("cp.async.wait_group 1;\n" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    }
    __syncthreads();
    const uint32_t k_src = smem_base + stage * 2 * TILE_BYTES, v_src = k_src + TILE_BYTES;
    const int64_t key0 = tile < 0 ? 0 : band_first + (int64_t)tile * kBandKeys;

    // S [16 rows x 64 keys] = Q K^T
    float s[kBandKeys / 8][4];
#pragma unroll
    for (int n = 0; n < kBandKeys / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.0f;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
      for (int np = 0; np < kBandKeys / 16; ++np) {
        const int row = np * 16 + (lane & 7) + (lane >> 4) * 8;
        const int chunk = ks * 2 + ((lane >> 3) & 1);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(k_src + row * ROW_BYTES + ((chunk ^ (row & 7)) << 4), b0, b1, b2, b3);
        mma_bf16(s[2 * np], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
        mma_bf16(s[2 * np + 1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b2, b3);
      }
    }
    // mask: a key counts for a row if it is inside the row's window (and causal), or one of its sinks. A tile that
    // lies inside every row's window (all but the band's two ends) needs none.
    float mx[2] = {-INFINITY, -INFINITY};
    const bool inside = tile >= 0 && key0 >= max((int64_t)0, pos_last + 1 - p.window) && key0 + kBandKeys - 1 <= pos0 &&
                        key0 + kBandKeys <= p.n_keys && pos0 + kBandRows <= p.first_position + p.R;
    if (inside) {
#pragma unroll
      for (int n = 0; n < kBandKeys / 8; ++n) {
#pragma unroll
        for (int j = 0; j < 4; ++j) mx[j >> 1] = fmaxf(mx[j >> 1], s[n][j]);
      }
    } else {
#pragma unroll
      for (int n = 0; n < kBandKeys / 8; ++n) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int64_t key = key0 + n * 8 + t * 2 + (j & 1);
          const int64_t pos = (j & 2) ? pos_b : pos_a;
          const int64_t start = max((int64_t)0, pos + 1 - p.window);
          const bool ok = pos < p.first_position + p.R && key < p.n_keys &&
                          ((tile >= 0 && key >= start && key <= pos) || key < min((int64_t)p.sink, start));
          s[n][j] = ok ? s[n][j] : -INFINITY;
          mx[j >> 1] = fmaxf(mx[j >> 1], s[n][j]);
        }
      }
    }
    float alpha[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      // the products are raw: the scale is positive, so it is applied to the maximum and inside the exponent
      const float m_new = fmaxf(m_run[r], mx[r] * p.scale_log2);
      const float m_safe = m_new == -INFINITY ? 0.0f : m_new;
      alpha[r] = fast_exp2(m_run[r] - m_safe);
      m_run[r] = m_new;
      mx[r] = m_safe;
      l_run[r] *= alpha[r];
    }
#pragma unroll
    for (int n = 0; n < kBandKeys / 8; ++n) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        s[n][j] = fast_exp2(fmaf(s[n][j], p.scale_log2, -mx[j >> 1]));
        l_run[j >> 1] += s[n][j];
      }
    }
    // (once a row has met its largest keys the maximum stops moving and the rescale is a multiply by one)
    if (__any_sync(0xffffffffu, alpha[0] != 1.0f || alpha[1] != 1.0f)) {
#pragma unroll
      for (int n = 0; n < DH / 8; ++n) {
        o[n][0] *= alpha[0];
        o[n][1] *= alpha[0];
        o[n][2] *= alpha[1];
        o[n][3] *= alpha[1];
      }
    }
    // O [16 rows x DH] += P [16 x 64] V [64 x DH]
#pragma unroll
    for (int kk = 0; kk < kBandKeys / 16; ++kk) {
      const uint32_t a0 = pack_bf16x2(s[2 * kk][0], s[2 * kk][1]), a1 = pack_bf16x2(s[2 * kk][2], s[2 * kk][3]);
      const uint32_t a2 = pack_bf16x2(s[2 * kk + 1][0], s[2 * kk + 1][1]), a3 = pack_bf16x2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int np = 0; np < DH / 16; ++np) {
        const int row = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int chunk = np * 2 + (lane >> 4);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(v_src + row * ROW_BYTES + ((chunk ^ (row & 7)) << 4), b0, b1, b2, b3);
        mma_bf16(o[2 * np], a0, a1, a2, a3, b0, b1);
        mma_bf16(o[2 * np + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    __syncthreads();
  }

  constexpr float kLn2 = 0.6931471805599453f;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    float l = l_run[r];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const int64_t row = row0 + g + r * 8;
    if (row >= p.R || !real_head) continue;
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
    float *dst = p.out + (row * p.Hq + head) * DH;
#pragma unroll
    for (int n = 0; n < DH / 8; ++n)
      *reinterpret_cast<float2 *>(dst + n * 8 + t * 2) = make_float2(o[n][2 * r] * inv, o[n][2 * r + 1] * inv);
    if (t == 0) p.lse[row * p.Hq + head] = l > 0.0f ? (m_run[r] + log2f(l)) * kLn2 : -INFINITY;
  }
}

int launch_band_attend_tc(const uint16_t *q, int64_t R, int Hq, int64_t q_row_stride, const uint16_t *k,
                          const uint16_t *v, int64_t n_keys, int Hkv, int64_t kv_row_stride, int64_t first_position,
                          int window, int sink, float scale, float *out, float *lse, int32_t *status,
                          cudaStream_t stream);

}  // namespace lsa

LSA_API int lsa_band_attend(const uint16_t *q, int64_t R, int Hq, int dh, int64_t q_row_stride,
                            int64_t q_head_stride, const uint16_t *k, const uint16_t *v, int64_t n_keys, int Hkv,
                            int64_t kv_row_stride, int64_t kv_head_stride, int64_t first_position, int window,
                            int sink, float scale, float *out_f32, float *lse, int flags, int32_t *status,
                            void *stream) {
  LSA_REQUIRE(q && k && v && out_f32 && lse, LSA_ERR_NULL);
  LSA_REQUIRE(R >= 0 && Hq >= 1 && Hkv >= 1 && Hq % Hkv == 0 && n_keys >= 0 && first_position >= 0 && window >= 0 &&
                  sink >= 0,
              LSA_ERR_ARGUMENT);
  LSA_REQUIRE(scale > 0.0f, LSA_ERR_ARGUMENT);  // the row maximum is taken before the scale is applied
  LSA_REQUIRE(dh == 64 || dh == 128, LSA_ERR_UNSUPPORTED);
  const int group = Hq / Hkv;
  LSA_REQUIRE(group <= 16 && sink <= lsa::kBandKeys, LSA_ERR_UNSUPPORTED);
  LSA_REQUIRE(kv_row_stride % 8 == 0 && kv_head_stride % 8 == 0 && ((uintptr_t)k % 16) == 0 &&
                  ((uintptr_t)v % 16) == 0 && q_row_stride % 2 == 0 && q_head_stride % 2 == 0 &&
                  ((uintptr_t)q % 4) == 0,
              LSA_ERR_ARGUMENT);
  if (R == 0) return LSA_OK;
  // The tensor-memory form: a head's 128 rows a CTA, operands fetched through tensor maps. It wants heads of 128
  // dims packed densely (a row of heads is a row of the map) and 16-byte aligned rows; a chunk shorter than a tile
  // of rows gains nothing from it.
  const bool dense = q_head_stride == dh && kv_head_stride == dh && q_row_stride % 8 == 0 && ((uintptr_t)q % 16) == 0;
  if (!(flags & LSA_BAND_WARP_MMA) && dh == 128 && dense && R >= 128 && n_keys < INT32_MAX)
    return lsa::launch_band_attend_tc(q, R, Hq, q_row_stride, k, v, n_keys, Hkv, kv_row_stride, first_position,
                                      window, sink, scale, out_f32, lse, status, (cudaStream_t)stream);
  lsa::BandParams p;
  p.q = q;
  p.k = k;
  p.v = v;
  p.out = out_f32;
  p.lse = lse;
  p.R = R;
  p.n_keys = n_keys;
  p.first_position = first_position;
  p.q_row_stride = q_row_stride;
  p.q_head_stride = q_head_stride;
  p.kv_row_stride = kv_row_stride;
  p.kv_head_stride = kv_head_stride;
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.group = group;
  p.window = window;
  p.sink = sink;
  p.scale_log2 = scale * 1.4426950408889634f;
  const size_t smem = (size_t)4 * lsa::kBandKeys * dh * 2;
  dim3 grid((unsigned)((R + lsa::kBandRows - 1) / lsa::kBandRows), (unsigned)Hkv, (unsigned)((group + 7) / 8));
  const int threads = (group < 8 ? group : 8) * 32;
  cudaStream_t s = (cudaStream_t)stream;
  if (dh == 128) {
    // 64 KB of tiles a CTA: ask for the largest shared-memory carve-out so that two or three CTAs share an SM
    if (cudaFuncSetAttribute(lsa::band_attend_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
            cudaSuccess ||
        cudaFuncSetAttribute(lsa::band_attend_kernel<128>, cudaFuncAttributePreferredSharedMemoryCarveout,
                             cudaSharedmemCarveoutMaxShared) != cudaSuccess)
      return LSA_ERR_LAUNCH;
    lsa::band_attend_kernel<128><<<grid, threads, smem, s>>>(p);
  } else {
    // 64 KB of tiles a CTA: ask for the largest shared-memory carve-out so that two or three CTAs share an SM
    if (cudaFuncSetAttribute(lsa::band_attend_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
            cudaSuccess ||
        cudaFuncSetAttribute(lsa::band_attend_kernel<64>, cudaFuncAttributePreferredSharedMemoryCarveout,
                             cudaSharedmemCarveoutMaxShared) != cudaSuccess)
      return LSA_ERR_LAUNCH;
    lsa::band_attend_kernel<64><<<grid, threads, smem, s>>>(p);
  }
  LSA_LAUNCH_CHECK();
  return LSA_OK;
}
