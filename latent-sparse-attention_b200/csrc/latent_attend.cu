// Gather-sparse attention over a shared latent (the MLA form): every query head of a row reads the SAME listed
// latent rows, keys = the whole row (DK dims, rope part included), values = its first DV dims.
//
// One CTA owns a (query row, split, block of 64 heads) item. With all heads sharing the keys, the heads are the M
// side of mma.m16n8k16 (4 tiles of 16) and a gathered row is used by 64 heads: ~121 flops a byte, so this kernel
// is bound by the tensor and shared-memory pipes rather than by the gather.
//
//   stage ring   32 latent rows a stage, 3 stages, 16-byte asynchronous copies (zero-filled for ids outside the
//                cache and past a list's end); rows padded by 16 bytes so ldmatrix reads are conflict-free
//   S phase      warp (head tile, key half) computes a 16 x 16 block of S = Q K^T over all DK dims
//   softmax      online, log2 domain, fp32 statistics; the two key halves exchange row maxima through shared memory
//   PV phase     warp w accumulates O[:, 64 w : 64 w + 64] for all 64 heads from P (bf16, shared memory) and the
//                same staged rows read transposed
//
// The natural-log log-sum-exp is emitted, so splits of a list and ranks of a sharded cache merge exactly.
#include "latent_attend.cuh"
#include "mma.cuh"

namespace lsa {

constexpr int kLatTile = 32;
constexpr int kLatStages = 3;
constexpr int kLatThreads = 256;
constexpr int kLatPPitch = 80;  // bytes a row of P: 32 keys bf16 + 16 of padding

template <int DK, int DV>
struct LatentLayout {
  static constexpr int CHUNKS = DK / 8;        // 16-byte chunks a row
  static constexpr int PITCH = DK * 2 + 16;    // bytes between staged rows
  static constexpr int Q_BYTES = kLatHeads * PITCH;
  static constexpr int STAGE_BYTES = kLatTile * PITCH;
  static constexpr int P_BYTES = kLatHeads * kLatPPitch;
  static constexpr int STATS_BYTES = (2 * kLatHeads + kLatHeads) * 4 + 16;
  static constexpr int TOTAL = Q_BYTES + kLatStages * STAGE_BYTES + P_BYTES + STATS_BYTES;
};

template <int DK, int DV>
__global__ void __launch_bounds__(kLatThreads, 1) latent_attend_kernel(LatentParams p) {
  using L = LatentLayout<DK, DV>;
  static_assert(DK % 16 == 0 && DV % 64 == 0 && DV == 64 * (kLatThreads / 32) && DV <= DK, "shape");
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const uint32_t q_s = smem_u32(smem_raw), k_s = q_s + L::Q_BYTES, p_s = k_s + kLatStages * L::STAGE_BYTES;
  unsigned char *p_ptr = smem_raw + L::Q_BYTES + kLatStages * L::STAGE_BYTES;
  float *smax = reinterpret_cast<float *>(p_ptr + L::P_BYTES);  // [2][64]: row maxima of the two key halves
  float *salpha = smax + 2 * kLatHeads;                          // [64]: this tile's rescale of O
  volatile uint32_t *masks = reinterpret_cast<volatile uint32_t *>(salpha + kLatHeads);  // [stages]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int ht = warp & 3, kh = warp >> 2;
  const int split = (int)(blockIdx.x % p.splits);
  const int64_t r = blockIdx.x / p.splits;
  const int head0 = blockIdx.y * kLatHeads;

  int64_t n_total = p.lengths ? p.lengths[r] : p.list_stride;
  if (n_total > p.list_stride) n_total = p.list_stride;
  if (n_total < 0) n_total = 0;
  int64_t per = (n_total + p.splits - 1) / p.splits;
  per = (per + kLatTile - 1) / kLatTile * kLatTile;
  const int64_t begin = (int64_t)split * per;
  const int64_t end = begin + per < n_total ? begin + per : n_total;
  const int n = end > begin ? (int)(end - begin) : 0;
  const int iters = (n + kLatTile - 1) / kLatTile;
  const int32_t *list = p.ids + r * p.list_stride + begin;

  // The row's query heads, once (they join the first stage's copy group)
  for (int e = tid; e < kLatHeads * L::CHUNKS; e += kLatThreads) {
    const int row = e / L::CHUNKS, c = e - row * L::CHUNKS;
    const bool ok = head0 + row < p.Hq;
    const uint16_t *src = ok ? p.q + r * p.q_row_stride + (int64_t)(head0 + row) * p.q_head_stride + c * 8 : p.q;
    cp_async_16(q_s + row * L::PITCH + c * 16, src, ok ? 16 : 0);
  }

  auto issue = [&](int it) {
    if (it < iters) {
      const int stage = it % kLatStages;
      const int base = it * kLatTile;
      if (warp == 0) {
        const int32_t id = base + lane < n ? list[base + lane] : -1;
        const uint32_t valid = __ballot_sync(0xffffffffu, id >= 0 && id < p.slots);
        if (lane == 0) masks[stage] = valid;
      }
      const uint32_t dst0 = k_s + stage * L::STAGE_BYTES;
#pragma unroll
      for (int i = 0; i < kLatTile * L::CHUNKS / kLatThreads; ++i) {
        const int e = tid + i * kLatThreads;
        const int row = e / L::CHUNKS, c = e - row * L::CHUNKS;
        const int32_t id = base + row < n ? list[base + row] : -1;
        const bool ok = id >= 0 && id < p.slots;
        const uint16_t *src = p.latent + (ok ? (int64_t)id * p.latent_row_stride + c * 8 : 0);
        cp_async_16(dst0 + row * L::PITCH + c * 16, src, ok ? 16 : 0);
      }
    }
    cp_async_commit();
  };
  static_assert((kLatTile * L::CHUNKS) % kLatThreads == 0, "whole passes of copies");

#pragma unroll
  for (int s = 0; s < kLatStages - 1; ++s) issue(s);

  float acc[4][8][4];
#pragma unroll
  for (int mt = 0; mt < 4; ++mt)
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) acc[mt][nt][0] = acc[mt][nt][1] = acc[mt][nt][2] = acc[mt][nt][3] = 0.0f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};

  const uint32_t a_addr = q_s + (ht * 16 + (lane & 15)) * L::PITCH + (lane >> 4) * 16;
  const int b_row = kh * 16 + ((lane >> 4) & 1) * 8 + (lane & 7);
  const int b_col = ((lane >> 3) & 1) * 16;
  const int v_row = ((lane >> 3) & 1) * 8 + (lane & 7);
  const int v_col = (warp * 64 + (lane >> 4) * 8) * 2;

  for (int it = 0; it < iters; ++it) {
    cp_async_wait<kLatStages - 2>();
    __syncthreads();  // tile `it` has landed for everyone; everyone is past the PV of tile it - 1
    issue(it + kLatStages - 1);
    const int stage = it % kLatStages;
    const uint32_t kt = k_s + stage * L::STAGE_BYTES;
    const uint32_t valid = masks[stage];

    // S [16 heads x 16 keys] of this warp
    float s[2][4] = {{0.0f, 0.0f, 0.0f, 0.0f}, {0.0f, 0.0f, 0.0f, 0.0f}};
    {
      const uint32_t b_addr = kt + b_row * L::PITCH + b_col;
#pragma unroll 4
      for (int ks = 0; ks < DK / 16; ++ks) {
        uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
        ldmatrix_x4(a_addr + ks * 32, a0, a1, a2, a3);
        ldmatrix_x4(b_addr + ks * 32, b0, b1, b2, b3);
        mma_bf16(s[0], a0, a1, a2, a3, b0, b1);
        mma_bf16(s[1], a0, a1, a2, a3, b2, b3);
      }
    }
    float x[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const int key = kh * 16 + nt * 8 + 2 * t;
      const bool ok0 = (valid >> key) & 1u, ok1 = (valid >> (key + 1)) & 1u;
      x[nt][0] = ok0 ? s[nt][0] * p.scale_log2 : -INFINITY;
      x[nt][1] = ok1 ? s[nt][1] * p.scale_log2 : -INFINITY;
      x[nt][2] = ok0 ? s[nt][2] * p.scale_log2 : -INFINITY;
      x[nt][3] = ok1 ? s[nt][3] * p.scale_log2 : -INFINITY;
    }
    float mx[2];
    mx[0] = fmaxf(fmaxf(x[0][0], x[0][1]), fmaxf(x[1][0], x[1][1]));
    mx[1] = fmaxf(fmaxf(x[0][2], x[0][3]), fmaxf(x[1][2], x[1][3]));
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      mx[j] = fmaxf(mx[j], __shfl_xor_sync(0xffffffffu, mx[j], 1));
      mx[j] = fmaxf(mx[j], __shfl_xor_sync(0xffffffffu, mx[j], 2));
      if (t == 0) smax[kh * kLatHeads + ht * 16 + g + 8 * j] = mx[j];
    }
    __syncthreads();  // both key halves' maxima are written
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int head = ht * 16 + g + 8 * j;
      const float m_new = fmaxf(m_run[j], fmaxf(smax[head], smax[kLatHeads + head]));
      const float m_safe = m_new == -INFINITY ? 0.0f : m_new;
      const float alpha = exp2f(m_run[j] - m_safe);
      m_run[j] = m_new;
      float sum = 0.0f;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const float p0 = exp2f(x[nt][2 * j] - m_safe), p1 = exp2f(x[nt][2 * j + 1] - m_safe);
        sum += p0 + p1;
        *reinterpret_cast<uint32_t *>(p_ptr + head * kLatPPitch + (kh * 16 + nt * 8 + 2 * t) * 2) = pack_bf16x2(p0, p1);
      }
      l_run[j] = l_run[j] * alpha + sum;
      if (kh == 0 && t == 0) salpha[head] = alpha;
    }
    __syncthreads();  // P and the rescale factors are written

    // O[:, this warp's 64 value dims] = alpha O + P V
#pragma unroll
    for (int mt = 0; mt < 4; ++mt) {
      const float a0 = salpha[mt * 16 + g], a1 = salpha[mt * 16 + g + 8];
      if (a0 != 1.0f || a1 != 1.0f) {
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
          acc[mt][nt][0] *= a0;
          acc[mt][nt][1] *= a0;
          acc[mt][nt][2] *= a1;
          acc[mt][nt][3] *= a1;
        }
      }
    }
#pragma unroll
    for (int ks = 0; ks < kLatTile / 16; ++ks) {
      uint32_t pa[4][4];
#pragma unroll
      for (int mt = 0; mt < 4; ++mt)
        ldmatrix_x4(p_s + (mt * 16 + (lane & 15)) * kLatPPitch + ks * 32 + (lane >> 4) * 16, pa[mt][0], pa[mt][1],
                    pa[mt][2], pa[mt][3]);
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(kt + (ks * 16 + v_row) * L::PITCH + v_col + np * 32, b0, b1, b2, b3);
#pragma unroll
        for (int mt = 0; mt < 4; ++mt) {
          mma_bf16(acc[mt][2 * np], pa[mt][0], pa[mt][1], pa[mt][2], pa[mt][3], b0, b1);
          mma_bf16(acc[mt][2 * np + 1], pa[mt][0], pa[mt][1], pa[mt][2], pa[mt][3], b2, b3);
        }
      }
    }
  }
  cp_async_wait<0>();
  __syncthreads();  // the last PV has read its rescale factors

  // Row sums of the two key halves and the running maxima, through shared memory
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    float l = l_run[j];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    if (t == 0) {
      smax[kh * kLatHeads + ht * 16 + g + 8 * j] = l;
      if (kh == 0) salpha[ht * 16 + g + 8 * j] = m_run[j];
    }
  }
  __syncthreads();

  const bool partial = p.splits > 1;
#pragma unroll
  for (int mt = 0; mt < 4; ++mt) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int head = mt * 16 + g + 8 * j;
      if (head0 + head >= p.Hq) continue;
      const float l = smax[head] + smax[kLatHeads + head];
      const float inv = l > 0.0f ? 1.0f / l : 0.0f;
      const int64_t out_row = (partial ? (int64_t)split * p.R + r : r) * p.Hq + head0 + head;
      if (warp == 0 && t == 0) {
        const float lse = l > 0.0f ? (salpha[head] + log2f(l)) * 0.6931471805599453f : -INFINITY;
        (partial ? p.part_lse : p.lse)[out_row] = lse;
      }
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const int col = warp * 64 + nt * 8 + 2 * t;
        const float v0 = acc[mt][nt][2 * j] * inv, v1 = acc[mt][nt][2 * j + 1] * inv;
        if (partial) {
          *reinterpret_cast<float2 *>(p.part_out + out_row * DV + col) = make_float2(v0, v1);
        } else {
          if (p.out_f32) *reinterpret_cast<float2 *>(p.out_f32 + out_row * DV + col) = make_float2(v0, v1);
          if (p.out_bf16) *reinterpret_cast<uint32_t *>(p.out_bf16 + out_row * DV + col) = pack_bf16x2(v0, v1);
        }
      }
    }
  }
}

}  // namespace lsa

// ================================================================================================ C ABI

LSA_API size_t lsa_latent_attend_workspace_bytes(int64_t R, int Hq, int dv, int splits) {
  if (splits <= 1 || R <= 0 || Hq <= 0 || dv <= 0) return 0;
  return (size_t)splits * (size_t)R * (size_t)Hq * ((size_t)dv + 1) * sizeof(float);
}

LSA_API int lsa_latent_attend(const uint16_t *q, int64_t R, int Hq, int dk, int dv, int64_t q_row_stride,
                              int64_t q_head_stride, const uint16_t *latent, int64_t slots, int64_t latent_row_stride,
                              const int32_t *ids, int64_t list_stride, const int32_t *lengths, float scale,
                              int splits, uint16_t *out_bf16, float *out_f32, float *lse, int flags,
                              int owner_granule, int owner_world, int owner_rank, int32_t *status, void *workspace,
                              size_t workspace_bytes, void *stream) {
  LSA_REQUIRE(q && latent && ids && lse && (out_bf16 || out_f32), LSA_ERR_NULL);
  LSA_REQUIRE(R >= 0 && Hq >= 1 && slots >= 0 && slots <= INT32_MAX && list_stride >= 0 && splits >= 1 &&
                  latent_row_stride >= dk,
              LSA_ERR_ARGUMENT);
  LSA_REQUIRE(dk == 576 && dv == 512, LSA_ERR_UNSUPPORTED);
  LSA_REQUIRE(owner_world <= 1 || (owner_granule >= 64 && owner_granule % 64 == 0 && owner_rank >= 0 &&
                                   owner_rank < owner_world),
              LSA_ERR_ARGUMENT);
  LSA_REQUIRE(owner_world <= 1 || !(flags & LSA_LATENT_WARP_MMA), LSA_ERR_UNSUPPORTED);
  // 16-byte copies of latent rows and query heads need these alignments
  LSA_REQUIRE(latent_row_stride % 8 == 0 && ((uintptr_t)latent % 16) == 0 && q_row_stride % 8 == 0 &&
                  q_head_stride % 8 == 0 && ((uintptr_t)q % 16) == 0,
              LSA_ERR_ARGUMENT);
  LSA_REQUIRE(R * splits <= INT32_MAX, LSA_ERR_ARGUMENT);
  if (R == 0) return LSA_OK;
  lsa::LatentParams p = {};
  p.q = q;
  p.latent = latent;
  p.ids = ids;
  p.lengths = lengths;
  p.out_bf16 = out_bf16;
  p.out_f32 = out_f32;
  p.lse = lse;
  p.R = R;
  p.slots = slots;
  p.q_row_stride = q_row_stride;
  p.q_head_stride = q_head_stride;
  p.latent_row_stride = latent_row_stride;
  p.list_stride = list_stride;
  p.Hq = Hq;
  p.splits = splits;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  p.deal_granule = owner_granule, p.deal_world = owner_world, p.deal_rank = owner_rank;
  if (splits > 1) {
    const size_t need = lsa_latent_attend_workspace_bytes(R, Hq, dv, splits);
    LSA_REQUIRE(workspace && workspace_bytes >= need, LSA_ERR_WORKSPACE);
    p.part_out = reinterpret_cast<float *>(workspace);
    p.part_lse = p.part_out + (size_t)splits * R * Hq * dv;
  }
  if (!(flags & LSA_LATENT_WARP_MMA)) {
    const int rc = lsa::launch_latent_attend_tc(p, (cudaStream_t)stream);
    if (rc != LSA_OK) return rc;
  } else {
    using L = lsa::LatentLayout<576, 512>;
    auto kernel = lsa::latent_attend_kernel<576, 512>;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL) != cudaSuccess)
      return LSA_ERR_LAUNCH;
    const dim3 grid((unsigned)(R * splits), (unsigned)((Hq + lsa::kLatHeads - 1) / lsa::kLatHeads));
    kernel<<<grid, lsa::kLatThreads, L::TOTAL, (cudaStream_t)stream>>>(p);
    LSA_LAUNCH_CHECK();
  }
  if (splits == 1) return LSA_OK;
  return lsa_lse_merge(p.part_out, LSA_DTYPE_F32, p.part_lse, splits, R * Hq, dv, out_bf16, out_f32, lse, stream);
}
