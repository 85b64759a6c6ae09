// Gather-sparse attention: every query row attends over the KV rows its list names.
//
// A warp owns one (query row, KV head, split) item and streams the listed K/V rows through its own
// shared-memory ring with asynchronous 16-byte copies (zero-filled for a list's ragged end), 32 keys a stage. The head group's queries share each gathered row: with the KEYS as the M dimension of the
// tensor-core tile (S^T = K Q^T, O^T = V^T P^T) a group of up to 8 query heads fills the N = 8 side of
// mma.m16n8k16 instead of 5 of 16 M rows, which halves the instructions per key. Softmax is online in the log2
// domain with fp32 statistics; the kernel emits the natural-log log-sum-exp so partial results over disjoint key
// sets (splits of a list here, ranks of a sequence-sharded cache elsewhere) merge exactly.
#include "common.cuh"
#include "mma.cuh"

namespace lsa {

constexpr int kKeysPerStage = 32;  // two 16-key MMA tiles, interleaved for instruction-level parallelism

struct AttendParams {
  const uint16_t *q, *k, *v;
  const int32_t *ids, *lengths;
  uint16_t *out_bf16;
  float *out_f32, *lse, *part_out, *part_lse;
  const float *init_out, *init_lse;  // a partial read to start from ([R,Hq,dh], [R,Hq]), or NULL
  int64_t R, slots, first_slot, q_row_stride, q_head_stride, kv_row_stride, kv_head_stride, list_stride;
  int Hq, Hkv, group, splits;
  float scale_log2;
};

// DH: head dim (64 or 128). NT: 8-head tiles a group needs (1 or 2). W: warps a CTA. STAGES: ring depth.
template <int DH, int NT, int W, int STAGES>
__global__ void __launch_bounds__(W * 32, 1) sparse_attend_kernel(AttendParams p) {
  constexpr int ROW_BYTES = DH * 2;
  constexpr int CHUNKS = ROW_BYTES / 16;                    // 16-byte chunks a row
  constexpr int TILE_BYTES = kKeysPerStage * ROW_BYTES;     // one of K or V
  constexpr int STAGE_BYTES = 2 * TILE_BYTES;
  constexpr int WARP_BYTES = STAGES * STAGE_BYTES + 16;     // + the stages' validity masks
  constexpr int KSTEPS = DH / 16;
  constexpr int ROWS_PER_PASS = 32 / CHUNKS;                // rows one pass of the warp's lanes covers
  constexpr int PASSES = kKeysPerStage / ROWS_PER_PASS;
  static_assert(STAGES >= 2 && STAGES <= 4, "ring depth");

  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int64_t item = (int64_t)blockIdx.x * W + warp;
  dependents_may_launch();
  wait_for_earlier_grids();
  if (item >= p.R * p.splits * p.Hkv) return;
  const int h = (int)(item % p.Hkv);
  const int64_t rs = item / p.Hkv;
  const int split = (int)(rs % p.splits);
  const int64_t r = rs / p.splits;

  unsigned char *mine = smem_raw + (size_t)warp * WARP_BYTES;
  const uint32_t smem_base = smem_u32(mine);
  volatile uint32_t *masks = reinterpret_cast<volatile uint32_t *>(mine + STAGES * STAGE_BYTES);

  int64_t n_total = p.lengths ? p.lengths[r] : p.list_stride;
  if (n_total > p.list_stride) n_total = p.list_stride;
  if (n_total < 0) n_total = 0;
  int64_t per = (n_total + p.splits - 1) / p.splits;
  per = (per + kKeysPerStage - 1) / kKeysPerStage * kKeysPerStage;
  const int64_t begin = (int64_t)split * per;
  const int64_t end = begin + per < n_total ? begin + per : n_total;
  const int n = end > begin ? (int)(end - begin) : 0;
  const int iters = (n + kKeysPerStage - 1) / kKeysPerStage;
  const int32_t *list = p.ids + r * p.list_stride + begin;
  const uint16_t *k_head = p.k + (int64_t)h * p.kv_head_stride;
  const uint16_t *v_head = p.v + (int64_t)h * p.kv_head_stride;

  // Q^T fragments (the B operand of S^T = K Q^T): thread (g, t) holds head g's dims t*2, t*2+1 (+8) of each
  // 16-dim step.
  uint32_t qf[NT][KSTEPS][2];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int head = nt * 8 + g;
    const uint16_t *qrow = p.q + r * p.q_row_stride + (int64_t)(h * p.group + head) * p.q_head_stride;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      if (head < p.group) {
        qf[nt][ks][0] = *reinterpret_cast<const uint32_t *>(qrow + ks * 16 + t * 2);
        qf[nt][ks][1] = *reinterpret_cast<const uint32_t *>(qrow + ks * 16 + t * 2 + 8);
      } else {
        qf[nt][ks][0] = qf[nt][ks][1] = 0u;
      }
    }
  }

  float o[NT][DH / 16][4];
  float m_run[NT][2], l_run[NT][2];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    m_run[nt][0] = m_run[nt][1] = -INFINITY;
    l_run[nt][0] = l_run[nt][1] = 0.0f;
#pragma unroll
    for (int mt = 0; mt < DH / 16; ++mt) o[nt][mt][0] = o[nt][mt][1] = o[nt][mt][2] = o[nt][mt][3] = 0.0f;
  }

  // Start from a partial read over other keys (the dense band of the window): it enters as one more term of the
  // online softmax, weight exp(lse) and value its normalised output. Only the first split carries it.
  if (p.init_out && split == 0) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int head = nt * 8 + t * 2 + j;
        if (head >= p.group) continue;
        const int64_t out_row = r * p.Hq + h * p.group + head;
        const float lse0 = p.init_lse[out_row];
        if (lse0 == -INFINITY) continue;
        m_run[nt][j] = lse0 * 1.4426950408889634f;
        l_run[nt][j] = g == 0 ? 1.0f : 0.0f;
        const float *src = p.init_out + out_row * DH;
#pragma unroll
        for (int mt = 0; mt < DH / 16; ++mt) {
          o[nt][mt][j] = src[mt * 16 + g];
          o[nt][mt][2 + j] = src[mt * 16 + g + 8];
        }
      }
  }

  // A lane's list entry of stage `it`; read a stage ahead of its use so the load never stalls the copies.
  auto entry = [&](int it) -> int32_t {
    const int e = it * kKeysPerStage + lane;
    return e < n ? list[e] : -1;
  };
  // Start the copies of stage `it`, whose list entries the lanes hold in `id`.
  auto issue = [&](int it, int32_t id) {
    if (it < iters) {
      const int stage = it % STAGES;
      id -= (int32_t)p.first_slot;  // k and v point at the row of slot first_slot
      const uint32_t valid = __ballot_sync(0xffffffffu, id >= 0 && id < p.slots);
      if (lane == 0) masks[stage] = valid;
      const uint32_t k_dst = smem_base + stage * STAGE_BYTES;
      const int chunk = lane % CHUNKS;
#pragma unroll
      for (int pass = 0; pass < PASSES; ++pass) {
        const int row = lane / CHUNKS + pass * ROWS_PER_PASS;
        const int32_t row_id = __shfl_sync(0xffffffffu, id, row);
        const bool row_ok = (valid >> row) & 1u;
        const int64_t off = row_ok ? (int64_t)row_id * p.kv_row_stride + chunk * 8 : 0;
        const uint32_t dst = k_dst + row * ROW_BYTES + ((chunk ^ (row & 7)) << 4);
        cp_async_16(dst, k_head + off, row_ok ? 16 : 0);
        cp_async_16(dst + TILE_BYTES, v_head + off, row_ok ? 16 : 0);
      }
    }
    cp_async_commit();
  };

#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) issue(s, entry(s));
  int32_t id_ahead = entry(STAGES - 1);

  for (int it = 0; it < iters; ++it) {
    cp_async_wait<STAGES - 2>();
    __syncwarp();
    issue(it + STAGES - 1, id_ahead);
    id_ahead = entry(it + STAGES);
    const int stage = it % STAGES;
    const uint32_t k_src = smem_base + stage * STAGE_BYTES, v_src = k_src + TILE_BYTES;
    const uint32_t valid = masks[stage];

    // S^T [32 keys x 8 heads] = K [32 x DH] . Q^T, as two independent 16-key accumulations
    float s0[NT][4], s1[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      s0[nt][0] = s0[nt][1] = s0[nt][2] = s0[nt][3] = 0.0f;
      s1[nt][0] = s1[nt][1] = s1[nt][2] = s1[nt][3] = 0.0f;
    }
    {
      const int row = (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
        const int chunk = ks * 2 + (lane >> 4);
        const uint32_t addr = k_src + row * ROW_BYTES + ((chunk ^ (row & 7)) << 4);
        uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
        ldmatrix_x4(addr, a0, a1, a2, a3);
        ldmatrix_x4(addr + 16 * ROW_BYTES, b0, b1, b2, b3);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          mma_bf16(s0[nt], a0, a1, a2, a3, qf[nt][ks][0], qf[nt][ks][1]);
          mma_bf16(s1[nt], b0, b1, b2, b3, qf[nt][ks][0], qf[nt][ks][1]);
        }
      }
    }

    const bool ok0 = (valid >> g) & 1u, ok1 = (valid >> (g + 8)) & 1u;
    const bool ok2 = (valid >> (g + 16)) & 1u, ok3 = (valid >> (g + 24)) & 1u;
    uint32_t pb[NT][4];
    bool rescale = false;
    float alpha[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      float x[8];
      x[0] = ok0 ? s0[nt][0] * p.scale_log2 : -INFINITY;
      x[1] = ok0 ? s0[nt][1] * p.scale_log2 : -INFINITY;
      x[2] = ok1 ? s0[nt][2] * p.scale_log2 : -INFINITY;
      x[3] = ok1 ? s0[nt][3] * p.scale_log2 : -INFINITY;
      x[4] = ok2 ? s1[nt][0] * p.scale_log2 : -INFINITY;
      x[5] = ok2 ? s1[nt][1] * p.scale_log2 : -INFINITY;
      x[6] = ok3 ? s1[nt][2] * p.scale_log2 : -INFINITY;
      x[7] = ok3 ? s1[nt][3] * p.scale_log2 : -INFINITY;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        float mx = fmaxf(fmaxf(x[j], x[2 + j]), fmaxf(x[4 + j], x[6 + j]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
        const float m_new = fmaxf(m_run[nt][j], mx);
        const float m_safe = m_new == -INFINITY ? 0.0f : m_new;
        alpha[nt][j] = exp2f(m_run[nt][j] - m_safe);
        rescale = rescale || (m_new != m_run[nt][j]);
        m_run[nt][j] = m_new;
        x[j] = exp2f(x[j] - m_safe);
        x[2 + j] = exp2f(x[2 + j] - m_safe);
        x[4 + j] = exp2f(x[4 + j] - m_safe);
        x[6 + j] = exp2f(x[6 + j] - m_safe);
        l_run[nt][j] = l_run[nt][j] * alpha[nt][j] + ((x[j] + x[2 + j]) + (x[4 + j] + x[6 + j]));
      }
      pb[nt][0] = movmatrix_trans(pack_bf16x2(x[0], x[1]));
      pb[nt][1] = movmatrix_trans(pack_bf16x2(x[2], x[3]));
      pb[nt][2] = movmatrix_trans(pack_bf16x2(x[4], x[5]));
      pb[nt][3] = movmatrix_trans(pack_bf16x2(x[6], x[7]));
    }
    if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int mt = 0; mt < DH / 16; ++mt) {
          o[nt][mt][0] *= alpha[nt][0];
          o[nt][mt][1] *= alpha[nt][1];
          o[nt][mt][2] *= alpha[nt][0];
          o[nt][mt][3] *= alpha[nt][1];
        }
    }

    // O^T [DH x 8 heads] += V^T [DH x 32 keys] . P^T
    {
      const int row = (lane & 7) + (lane >> 4) * 8;
#pragma unroll
      for (int mt = 0; mt < DH / 16; ++mt) {
        const int chunk = mt * 2 + ((lane >> 3) & 1);
        const uint32_t addr = v_src + row * ROW_BYTES + ((chunk ^ (row & 7)) << 4);
        uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
        ldmatrix_x4_trans(addr, a0, a1, a2, a3);
        ldmatrix_x4_trans(addr + 16 * ROW_BYTES, b0, b1, b2, b3);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          mma_bf16(o[nt][mt], a0, a1, a2, a3, pb[nt][0], pb[nt][1]);
          mma_bf16(o[nt][mt], b0, b1, b2, b3, pb[nt][2], pb[nt][3]);
        }
      }
    }
    __syncwarp();
  }
  cp_async_wait<0>();

  // Finish: the row sums live per thread; add them over the eight key lanes of each head.
  constexpr float kLn2 = 0.6931471805599453f;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      float l = l_run[nt][j];
      l += __shfl_xor_sync(0xffffffffu, l, 4);
      l += __shfl_xor_sync(0xffffffffu, l, 8);
      l += __shfl_xor_sync(0xffffffffu, l, 16);
      const int head = nt * 8 + t * 2 + j;
      if (head >= p.group) continue;
      const float inv = l > 0.0f ? 1.0f / l : 0.0f;
      const float lse = l > 0.0f ? (m_run[nt][j] + log2f(l)) * kLn2 : -INFINITY;
      const int64_t out_row = r * p.Hq + h * p.group + head;
      if (p.splits > 1) {
        float *dst = p.part_out + ((int64_t)split * p.R * p.Hq + out_row) * DH;
#pragma unroll
        for (int mt = 0; mt < DH / 16; ++mt) {
          dst[mt * 16 + g] = o[nt][mt][j] * inv;
          dst[mt * 16 + g + 8] = o[nt][mt][2 + j] * inv;
        }
        if (g == 0) p.part_lse[(int64_t)split * p.R * p.Hq + out_row] = lse;
      } else {
#pragma unroll
        for (int mt = 0; mt < DH / 16; ++mt) {
          const float lo = o[nt][mt][j] * inv, hi = o[nt][mt][2 + j] * inv;
          if (p.out_bf16) {
            p.out_bf16[out_row * DH + mt * 16 + g] = float_to_bf16_bits(lo);
            p.out_bf16[out_row * DH + mt * 16 + g + 8] = float_to_bf16_bits(hi);
          }
          if (p.out_f32) {
            p.out_f32[out_row * DH + mt * 16 + g] = lo;
            p.out_f32[out_row * DH + mt * 16 + g + 8] = hi;
          }
        }
        if (g == 0 && p.lse) p.lse[out_row] = lse;
      }
    }
  }
}

// out = sum_p exp(lse_p - lse) out_p over `n_parts` partial results; a warp a row.
__global__ void lse_merge_kernel(const float *__restrict__ parts, const float *__restrict__ lses, int n_parts,
                                 int64_t rows, int dh, uint16_t *__restrict__ out_bf16, float *__restrict__ out_f32,
                                 float *__restrict__ lse_out) {
  const int lane = lane_id();
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  dependents_may_launch();
  wait_for_earlier_grids();
  if (row >= rows) return;
  float m = -INFINITY;
  for (int i = 0; i < n_parts; ++i) m = fmaxf(m, lses[(int64_t)i * rows + row]);
  float total = -INFINITY;
  if (m > -INFINITY) {
    float l = 0.0f;
    for (int i = 0; i < n_parts; ++i) l += expf(lses[(int64_t)i * rows + row] - m);
    total = m + logf(l);
  }
  for (int c = lane; c < dh; c += 32) {
    float acc = 0.0f;
    if (m > -INFINITY)
      for (int i = 0; i < n_parts; ++i) {
        const float w = expf(lses[(int64_t)i * rows + row] - total);
        acc = fmaf(w, parts[((int64_t)i * rows + row) * dh + c], acc);
      }
    if (out_bf16) out_bf16[row * dh + c] = float_to_bf16_bits(acc);
    if (out_f32) out_f32[row * dh + c] = acc;
  }
  if (lane == 0 && lse_out) lse_out[row] = total;
}

// The same merge for many parts or wide rows (a decode row split over a hundred CTAs): a CTA of 128 threads a row.
// The parts' weights are computed once into shared memory, 256 parts at a time; a thread owns dims tid, tid + 128,
// ... and adds the parts in order, so an output element sees the same sequence of fused multiply-adds either way.
constexpr int kMergeWideDims = 8;  // dims a thread holds: rows of up to 1,024 dims

__global__ void __launch_bounds__(128)
    lse_merge_wide_kernel(const float *__restrict__ parts, const float *__restrict__ lses, int n_parts, int64_t rows,
                          int dh, uint16_t *__restrict__ out_bf16, float *__restrict__ out_f32,
                          float *__restrict__ lse_out) {
  __shared__ float w_s[256];
  __shared__ float red_s[4];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t row = blockIdx.x;
  dependents_may_launch();
  wait_for_earlier_grids();
  float m = -INFINITY;
  for (int i = tid; i < n_parts; i += 128) m = fmaxf(m, lses[(int64_t)i * rows + row]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if (lane == 0) red_s[warp] = m;
  __syncthreads();
  m = fmaxf(fmaxf(red_s[0], red_s[1]), fmaxf(red_s[2], red_s[3]));
  __syncthreads();
  float total = -INFINITY;
  if (m > -INFINITY) {
    float l = 0.0f;
    for (int i = tid; i < n_parts; i += 128) l += expf(lses[(int64_t)i * rows + row] - m);
    l = warp_sum(l);
    if (lane == 0) red_s[warp] = l;
    __syncthreads();
    total = m + logf(red_s[0] + red_s[1] + red_s[2] + red_s[3]);
  }
  float acc[kMergeWideDims];
#pragma unroll
  for (int j = 0; j < kMergeWideDims; ++j) acc[j] = 0.0f;
  for (int i0 = 0; i0 < n_parts; i0 += 256) {
    const int n = min(256, n_parts - i0);
    __syncthreads();
    for (int i = tid; i < n; i += 128)
      w_s[i] = m > -INFINITY ? expf(lses[(int64_t)(i0 + i) * rows + row] - total) : 0.0f;
    __syncthreads();
    const float *src = parts + ((int64_t)i0 * rows + row) * dh;
#pragma unroll 4
    for (int i = 0; i < n; ++i, src += rows * dh) {
      const float w = w_s[i];
#pragma unroll
      for (int j = 0; j < kMergeWideDims; ++j)
        if (tid + 128 * j < dh) acc[j] = fmaf(w, src[tid + 128 * j], acc[j]);
    }
  }
#pragma unroll
  for (int j = 0; j < kMergeWideDims; ++j) {
    const int c = tid + 128 * j;
    if (c >= dh) continue;
    if (out_bf16) out_bf16[row * dh + c] = float_to_bf16_bits(acc[j]);
    if (out_f32) out_f32[row * dh + c] = acc[j];
  }
  if (tid == 0 && lse_out) lse_out[row] = total;
}

template <int DH, int NT, int W, int STAGES>
static int launch_attend(const AttendParams &p, cudaStream_t s) {
  constexpr int WARP_BYTES = STAGES * 2 * kKeysPerStage * DH * 2 + 16;
  const size_t smem = (size_t)W * WARP_BYTES;
  if (cudaFuncSetAttribute(sparse_attend_kernel<DH, NT, W, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)smem) != cudaSuccess)
    return LSA_ERR_LAUNCH;
  const int64_t items = p.R * p.splits * p.Hkv;
  const int64_t grid = (items + W - 1) / W;
  if (grid > INT32_MAX) return LSA_ERR_ARGUMENT;
  launch(p.R <= kChainedRows, sparse_attend_kernel<DH, NT, W, STAGES>, dim3((unsigned)grid), dim3(W * 32), smem, s, p);
  LSA_LAUNCH_CHECK();
  return LSA_OK;
}

// Many parts of wide rows (a decode step split over every SM): a CTA owns (row, 128 dims). Its sixteen warps take
// the parts in turn, a lane four dims of a part (one 16-byte load, ten in flight), and the warps' sums meet in shared
// memory: the partials of a split read are some tens of MB that one pass at the copy bandwidth can merge.
constexpr int kSplitWarps = 16;
constexpr int kSplitThreads = kSplitWarps * 32;
constexpr int kSplitBatch = 10;  // parts a warp asks for at once: 160 parts (a decode row split over every SM) in one go

__global__ void __launch_bounds__(kSplitThreads)
    lse_merge_split_kernel(const float *__restrict__ parts, const float *__restrict__ lses, int n_parts, int64_t rows,
                           int dh, uint16_t *__restrict__ out_bf16, float *__restrict__ out_f32,
                           float *__restrict__ lse_out) {
  __shared__ float w_s[1024];
  __shared__ float max_s[kSplitWarps], sum_l_s[kSplitWarps];
  __shared__ float4 sum_s[kSplitWarps][32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int chunks = dh / 128;
  dependents_may_launch();
  wait_for_earlier_grids();
  const int64_t row = blockIdx.x / chunks;
  const int col = (int)(blockIdx.x % chunks) * 128 + lane * 4;
  const float *src = parts + row * dh + col;
  const int64_t stride = rows * dh;
  // A step is a chain of waits on memory, so everything that can be asked for at once is: this warp's first parts
  // (they do not depend on the weights) and this thread's log-sum-exps, before any of them is used.
  float4 v[kSplitBatch];
#pragma unroll
  for (int j = 0; j < kSplitBatch; ++j) {
    const int i = warp + kSplitWarps * j;
    v[j] = i < n_parts ? *reinterpret_cast<const float4 *>(src + (int64_t)i * stride) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float mine[1024 / kSplitThreads];
#pragma unroll
  for (int j = 0; j < 1024 / kSplitThreads; ++j) {
    const int i = tid + j * kSplitThreads;
    mine[j] = i < n_parts ? lses[(int64_t)i * rows + row] : -INFINITY;
  }
  float m = -INFINITY;
#pragma unroll
  for (int j = 0; j < 1024 / kSplitThreads; ++j) m = fmaxf(m, mine[j]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if (lane == 0) max_s[warp] = m;
  __syncthreads();
  m = -INFINITY;
#pragma unroll
  for (int w = 0; w < kSplitWarps; ++w) m = fmaxf(m, max_s[w]);
  float l = 0.0f;
#pragma unroll
  for (int j = 0; j < 1024 / kSplitThreads; ++j) {
    const int i = tid + j * kSplitThreads;
    if (i < n_parts) {
      const float e = m > -INFINITY ? expf(mine[j] - m) : 0.0f;
      w_s[i] = e;
      l += e;
    }
  }
  l = warp_sum(l);
  if (lane == 0) sum_l_s[warp] = l;
  __syncthreads();
  float denom = 0.0f;
#pragma unroll
  for (int w = 0; w < kSplitWarps; ++w) denom += sum_l_s[w];
  const float inv = denom > 0.0f ? 1.0f / denom : 0.0f;
  float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
  for (int j = 0; j < kSplitBatch; ++j) {
    const int i = warp + kSplitWarps * j;
    const float w = i < n_parts ? w_s[i] : 0.0f;
    acc.x = fmaf(w, v[j].x, acc.x), acc.y = fmaf(w, v[j].y, acc.y);
    acc.z = fmaf(w, v[j].z, acc.z), acc.w = fmaf(w, v[j].w, acc.w);
  }
  for (int i0 = warp + kSplitWarps * kSplitBatch; i0 < n_parts; i0 += kSplitWarps * kSplitBatch) {
#pragma unroll
    for (int j = 0; j < kSplitBatch; ++j) {
      const int i = i0 + kSplitWarps * j;
      v[j] = i < n_parts ? *reinterpret_cast<const float4 *>(src + (int64_t)i * stride) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int j = 0; j < kSplitBatch; ++j) {
      const int i = i0 + kSplitWarps * j;
      const float w = i < n_parts ? w_s[i] : 0.0f;
      acc.x = fmaf(w, v[j].x, acc.x), acc.y = fmaf(w, v[j].y, acc.y);
      acc.z = fmaf(w, v[j].z, acc.z), acc.w = fmaf(w, v[j].w, acc.w);
    }
  }
  sum_s[warp][lane] = acc;
  __syncthreads();
  if (warp == 0) {
    float x = 0.0f, y = 0.0f, z = 0.0f, w = 0.0f;
#pragma unroll
    for (int k = 0; k < kSplitWarps; ++k) {
      const float4 a = sum_s[k][lane];
      x += a.x, y += a.y, z += a.z, w += a.w;
    }
    x *= inv, y *= inv, z *= inv, w *= inv;
    if (out_f32) *reinterpret_cast<float4 *>(out_f32 + row * dh + col) = make_float4(x, y, z, w);
    if (out_bf16) *reinterpret_cast<uint2 *>(out_bf16 + row * dh + col) = make_uint2(pack_bf16x2(x, y), pack_bf16x2(z, w));
    if (lane == 0 && lse_out && blockIdx.x % chunks == 0) lse_out[row] = denom > 0.0f ? m + logf(denom) : -INFINITY;
  }
}

// A few parts of many rows (the ranks' partial reads of a prefill chunk): a warp a row. The parts' weights are
// computed once a row - lane i holds part i's - and a lane carries eight dims of the row through all parts, read 16
// bytes at a time from bf16 or fp32 partials.
template <typename T>
__global__ void __launch_bounds__(256)
    lse_merge_few_kernel(const T *__restrict__ parts, const float *__restrict__ lses, int n_parts, int64_t rows, int dh,
                         uint16_t *__restrict__ out_bf16, float *__restrict__ out_f32, float *__restrict__ lse_out) {
  const int lane = lane_id();
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  dependents_may_launch();
  wait_for_earlier_grids();
  if (row >= rows) return;
  const float mine = lane < n_parts ? lses[(int64_t)lane * rows + row] : -INFINITY;
  float m = mine;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  const float e = m > -INFINITY ? expf(mine - m) : 0.0f;
  const float l = warp_sum(e);
  const float w_mine = l > 0.0f ? e / l : 0.0f;
  for (int c0 = lane * 8; c0 < dh; c0 += 256) {
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.0f;
    for (int i = 0; i < n_parts; ++i) {
      const float w = __shfl_sync(0xffffffffu, w_mine, i);
      const T *src = parts + ((int64_t)i * rows + row) * dh + c0;
      float v[8];
      if constexpr (sizeof(T) == 2) {
        const uint4 raw = *reinterpret_cast<const uint4 *>(src);
        const uint32_t p4[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          v[2 * k] = __uint_as_float(p4[k] << 16);
          v[2 * k + 1] = __uint_as_float(p4[k] & 0xFFFF0000u);
        }
      } else {
        const float4 a = *reinterpret_cast<const float4 *>(src), b = *reinterpret_cast<const float4 *>(src + 4);
        v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] = fmaf(w, v[k], acc[k]);
    }
    if (out_f32) {
      *reinterpret_cast<float4 *>(out_f32 + row * dh + c0) = make_float4(acc[0], acc[1], acc[2], acc[3]);
      *reinterpret_cast<float4 *>(out_f32 + row * dh + c0 + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
    if (out_bf16)
      *reinterpret_cast<uint4 *>(out_bf16 + row * dh + c0) =
          make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]),
                     pack_bf16x2(acc[6], acc[7]));
  }
  if (lane == 0 && lse_out) lse_out[row] = l > 0.0f ? m + logf(l) : -INFINITY;
}

}  // namespace lsa

// ================================================================================================ C ABI

LSA_API size_t lsa_sparse_attend_workspace_bytes(int64_t R, int Hq, int dh, int splits) {
  if (R <= 0 || Hq <= 0 || dh <= 0 || splits <= 1) return 0;
  return (size_t)splits * R * Hq * (dh + 1) * sizeof(float);
}

LSA_API int lsa_lse_merge(const void *parts, int parts_dtype, const float *lses, int n_parts, int64_t rows, int dh,
                          uint16_t *out_bf16, float *out_f32, float *lse_out, void *stream) {
  LSA_REQUIRE(parts && lses && (out_bf16 || out_f32), LSA_ERR_NULL);
  LSA_REQUIRE(n_parts >= 1 && rows >= 0 && dh >= 1, LSA_ERR_ARGUMENT);
  LSA_REQUIRE(parts_dtype == LSA_DTYPE_F32 || parts_dtype == LSA_DTYPE_BF16, LSA_ERR_ARGUMENT);
  if (rows == 0) return LSA_OK;
  // (rows here are (row, head) pairs: a decode step's few query rows of up to 128 heads)
  const bool chained = rows <= lsa::kChainedRows * 128;
  const bool aligned = dh % 8 == 0 && ((uintptr_t)parts % 16) == 0 && (!out_f32 || ((uintptr_t)out_f32 % 16) == 0) &&
                       (!out_bf16 || ((uintptr_t)out_bf16 % 16) == 0);
  if (n_parts < 16 && aligned && (parts_dtype == LSA_DTYPE_BF16 || rows >= 1024)) {
    const unsigned grid = (unsigned)((rows + 7) / 8);
    if (parts_dtype == LSA_DTYPE_BF16)
      lsa::launch(chained, lsa::lse_merge_few_kernel<uint16_t>, dim3(grid), dim3(256), 0, (cudaStream_t)stream,
                  (const uint16_t *)parts, lses, n_parts, rows, dh, out_bf16, out_f32, lse_out);
    else
      lsa::launch(chained, lsa::lse_merge_few_kernel<float>, dim3(grid), dim3(256), 0, (cudaStream_t)stream,
                  (const float *)parts, lses, n_parts, rows, dh, out_bf16, out_f32, lse_out);
    LSA_LAUNCH_CHECK();
    return LSA_OK;
  }
  LSA_REQUIRE(parts_dtype == LSA_DTYPE_F32, LSA_ERR_UNSUPPORTED);
  const float *fparts = (const float *)parts;
  if (n_parts >= 16 && n_parts <= 1024 && dh % 128 == 0 && ((uintptr_t)parts % 16) == 0 &&
      (!out_f32 || ((uintptr_t)out_f32 % 16) == 0) && (!out_bf16 || ((uintptr_t)out_bf16 % 8) == 0)) {
    lsa::launch(chained, lsa::lse_merge_split_kernel, dim3((unsigned)(rows * (dh / 128))), dim3(lsa::kSplitThreads), 0,
                (cudaStream_t)stream, fparts, lses, n_parts, rows, dh, out_bf16, out_f32, lse_out);
    LSA_LAUNCH_CHECK();
    return LSA_OK;
  }
  if ((n_parts >= 16 || dh >= 256) && dh <= 128 * lsa::kMergeWideDims) {
    lsa::launch(chained, lsa::lse_merge_wide_kernel, dim3((unsigned)rows), dim3(128), 0, (cudaStream_t)stream, fparts,
                lses, n_parts, rows, dh, out_bf16, out_f32, lse_out);
    LSA_LAUNCH_CHECK();
    return LSA_OK;
  }
  const int warps = 8;
  lsa::launch(chained, lsa::lse_merge_kernel, dim3((unsigned)((rows + warps - 1) / warps)), dim3(warps * 32), 0,
              (cudaStream_t)stream, fparts, lses, n_parts, rows, dh, out_bf16, out_f32, lse_out);
  LSA_LAUNCH_CHECK();
  return LSA_OK;
}

LSA_API int lsa_sparse_attend(const uint16_t *q, int64_t R, int Hq, int dh, int64_t q_row_stride,
                              int64_t q_head_stride, const uint16_t *k, const uint16_t *v, int64_t slots, int64_t first_slot,
                              int Hkv,
                              int64_t kv_row_stride, int64_t kv_head_stride, const int32_t *ids, int64_t list_stride,
                              const int32_t *lengths, const float *init_out, const float *init_lse, float scale,
                              int splits, uint16_t *out_bf16, float *out_f32, float *lse, void *workspace,
                              size_t workspace_bytes, void *stream) {
  LSA_REQUIRE(q && k && v && ids && (out_bf16 || out_f32), LSA_ERR_NULL);
  LSA_REQUIRE((init_out == nullptr) == (init_lse == nullptr), LSA_ERR_NULL);
  LSA_REQUIRE(R >= 0 && Hq >= 1 && Hkv >= 1 && Hq % Hkv == 0 && slots >= 0 && first_slot >= 0 &&
                  first_slot + slots <= INT32_MAX && list_stride >= 0 && splits >= 1,
              LSA_ERR_ARGUMENT);
  LSA_REQUIRE(dh == 64 || dh == 128, LSA_ERR_UNSUPPORTED);
  const int group = Hq / Hkv;
  LSA_REQUIRE(group <= 16, LSA_ERR_UNSUPPORTED);
  // 16-byte copies of K/V rows and 4-byte reads of Q need these alignments
  LSA_REQUIRE(kv_row_stride % 8 == 0 && kv_head_stride % 8 == 0 && ((uintptr_t)k % 16) == 0 &&
                  ((uintptr_t)v % 16) == 0,
              LSA_ERR_ARGUMENT);
  LSA_REQUIRE(q_row_stride % 2 == 0 && q_head_stride % 2 == 0 && ((uintptr_t)q % 4) == 0, LSA_ERR_ARGUMENT);
  if (R == 0) return LSA_OK;
  lsa::AttendParams p;
  p.q = q;
  p.k = k;
  p.v = v;
  p.ids = ids;
  p.lengths = lengths;
  p.out_bf16 = out_bf16;
  p.out_f32 = out_f32;
  p.lse = lse;
  p.init_out = init_out;
  p.init_lse = init_lse;
  p.part_out = nullptr;
  p.part_lse = nullptr;
  p.R = R;
  p.slots = slots;
  p.first_slot = first_slot;
  p.q_row_stride = q_row_stride;
  p.q_head_stride = q_head_stride;
  p.kv_row_stride = kv_row_stride;
  p.kv_head_stride = kv_head_stride;
  p.list_stride = list_stride;
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.group = group;
  p.splits = splits;
  p.scale_log2 = scale * 1.4426950408889634f;
  if (splits > 1) {
    LSA_REQUIRE(workspace, LSA_ERR_NULL);
    LSA_REQUIRE(workspace_bytes >= lsa_sparse_attend_workspace_bytes(R, Hq, dh, splits), LSA_ERR_WORKSPACE);
    p.part_out = (float *)workspace;
    p.part_lse = p.part_out + (size_t)splits * R * Hq * dh;
  }
  cudaStream_t s = (cudaStream_t)stream;
  int rc;
  // Shared memory a warp: dh 128 -> 2 stages of 16 KB (7 warps fill an SM), dh 64 -> 3 stages of 8 KB (9 warps).
  if (dh == 128)
    rc = group <= 8 ? lsa::launch_attend<128, 1, 7, 2>(p, s) : lsa::launch_attend<128, 2, 7, 2>(p, s);
  else
    rc = group <= 8 ? lsa::launch_attend<64, 1, 9, 3>(p, s) : lsa::launch_attend<64, 2, 9, 3>(p, s);
  if (rc != LSA_OK || splits == 1) return rc;
  return lsa_lse_merge(p.part_out, LSA_DTYPE_F32, p.part_lse, splits, R * Hq, dh, out_bf16, out_f32, lse, stream);
}

// ================================================================================================ no-allocation entry

// Scratch of lsa_sparse_attend_static: the partial outputs and log-sum-exps of a split read. It is part of the
// library image, so every GPU that loads the library holds these bytes until the process exits.
#define LSA_STATIC_SCRATCH_BYTES (8u << 20)
static __device__ __align__(256) unsigned char lsa_static_attend_scratch[LSA_STATIC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
// Device address of the scratch array on each device, resolved on the first call made with that device current.
void *static_scratch_address[kMaxDevices] = {};
}  // namespace

LSA_API size_t lsa_sparse_attend_static_scratch_bytes(void) { return LSA_STATIC_SCRATCH_BYTES; }

LSA_API int lsa_sparse_attend_static(const uint16_t *q, int64_t R, int Hq, int dh, int64_t q_row_stride,
                                     int64_t q_head_stride, const uint16_t *k, const uint16_t *v, int64_t slots,
                                     int64_t first_slot, int Hkv, int64_t kv_row_stride, int64_t kv_head_stride, const int32_t *ids,
                                     int64_t list_stride, const int32_t *lengths, float scale, int splits,
                                     uint16_t *out_bf16, float *out_f32, float *lse, void *stream) {
  LSA_REQUIRE(R >= 0 && Hq >= 1 && dh >= 1 && splits >= 1, LSA_ERR_ARGUMENT);
  const size_t need = lsa_sparse_attend_workspace_bytes(R, Hq, dh, splits);
  if (need > LSA_STATIC_SCRATCH_BYTES) return LSA_ERR_STATIC_SCRATCH;
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return LSA_ERR_DEVICE;
  void *scratch = static_scratch_address[device];
  if (scratch == nullptr) {
    // In host code the array's name is only a handle: the kernels need the address it has on THIS device.
    if (cudaGetSymbolAddress(&scratch, lsa_static_attend_scratch) != cudaSuccess || scratch == nullptr) {
      (void)cudaGetLastError();
      return LSA_ERR_LAUNCH;
    }
    static_scratch_address[device] = scratch;
  }
  return lsa_sparse_attend(q, R, Hq, dh, q_row_stride, q_head_stride, k, v, slots, first_slot, Hkv, kv_row_stride, kv_head_stride,
                           ids, list_stride, lengths, nullptr, nullptr, scale, splits, out_bf16, out_f32, lse, scratch,
                           LSA_STATIC_SCRATCH_BYTES, stream);
}
