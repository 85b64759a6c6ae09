// Dense contractions on the fifth-generation tensor cores: C[M, N] = A[M, K] . B[N, K]^T, bf16 in, fp32 in TMEM.
//
// One CTA computes a 128-row tile. A single thread issues tcgen05.mma (M = 128, N = the tile's width, K = 16 a
// step) on operands that TMA (cp.async.bulk.tensor, 128-byte swizzle) streams through a shared-memory ring; the
// accumulator lives in tensor memory and four epilogue warps read it back with tcgen05.ld, one row a thread, so a
// row-wise epilogue (L2 normalisation, GELU) needs no cross-thread traffic.
//
//   warp 0      TMA producer (one elected lane)
//   warp 1      TMEM allocation, MMA issue (one elected lane), TMEM release
//   warps 2-5   epilogue: TMEM -> registers -> global
//
// Every wait on an mbarrier is bounded; a wait that gives up raises the status word and the CTA drains and leaves.
#include <cuda.h>

#include "common.cuh"
#include "umma.cuh"

namespace lsa {

constexpr int kTileM = 128;
constexpr int kTileK = 64;  // bf16 elements: one 128-byte swizzle atom a row
constexpr int kGemmThreads = 192;

enum GemmEpilogue { kEpilogueRownorm = 0, kEpilogueGelu = 1, kEpiloguePlain = 2 };

struct GemmParams {
  float *out_f32;      // [M, ldc] or NULL
  uint16_t *out_bf16;  // [M, ldc] or NULL
  int32_t *status;     // raised when a bounded wait gives up, or NULL
  int64_t M, ldc;
  int k_blocks;
  int normalize;
};

template <int N_TILE, int STAGES, int EPILOGUE>
__global__ void __launch_bounds__(kGemmThreads)
    umma_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                     GemmParams p) {
  static_assert(N_TILE % 16 == 0 && N_TILE >= 16 && N_TILE <= 256, "UMMA N");
  constexpr int A_BYTES = kTileM * kTileK * 2, B_BYTES = N_TILE * kTileK * 2;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int TMEM_COLS = N_TILE <= 32 ? 32 : (N_TILE <= 64 ? 64 : (N_TILE <= 128 ? 128 : 256));

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // The ring first (1,024-byte aligned tiles, as the swizzle needs), then the barriers.
  const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
  __shared__ __align__(8) uint64_t bars[2 * STAGES + 1];
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int abort_s;
  const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]), done_bar = smem_u32(&bars[2 * STAGES]);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * kTileM, n0 = blockIdx.y * N_TILE;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    mbar_init(done_bar, 1);
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)),
                 "r"(TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_s;

  if (warp == 0) {
    if (lane == 0) {
      int armed = 0;
      for (int kb = 0; kb < p.k_blocks; ++kb) {
        const int s = kb % STAGES;
        if (kb >= STAGES && !mbar_wait(empty0 + 8 * s, ((kb / STAGES) & 1) ^ 1)) {
          abort_s = 1;
          break;
        }
        mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
        tma_load_2d(ring + s * STAGE_BYTES, &map_a, full0 + 8 * s, kb * kTileK, m0);
        tma_load_2d(ring + s * STAGE_BYTES + A_BYTES, &map_b, full0 + 8 * s, kb * kTileK, n0);
        armed = kb + 1;
      }
      if (abort_s) {
        // Leave only once the copies already in flight have landed (bounded), so none writes into a dead CTA.
        for (int kb = max(0, armed - STAGES); kb < armed; ++kb) mbar_wait(full0 + 8 * (kb % STAGES), (kb / STAGES) & 1);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(N_TILE);
      bool ok = true;
      for (int kb = 0; kb < p.k_blocks && ok; ++kb) {
        const int s = kb % STAGES;
        ok = mbar_wait(full0 + 8 * s, (kb / STAGES) & 1);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t desc_a = smem_desc_sw128(ring + s * STAGE_BYTES);
        const uint64_t desc_b = smem_desc_sw128(ring + s * STAGE_BYTES + A_BYTES);
#pragma unroll
        for (int k = 0; k < kTileK / 16; ++k)  // 32 bytes further along K inside the swizzle atom a step
          umma_bf16(tmem_base, desc_a + 2 * k, desc_b + 2 * k, idesc, (kb | k) != 0);
        umma_commit(empty0 + 8 * s);
      }
      if (!ok) abort_s = 1;
      umma_commit(done_bar);
    }
  } else {
    // Epilogue warps: warp w reads the 32 TMEM lanes of its quadrant, w % 4.
    const int quad = warp & 3;
    const int64_t row = (int64_t)m0 + quad * 32 + lane;
    const bool ok = mbar_wait(done_bar, 0);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok && !abort_s) {
      float acc[N_TILE];
#pragma unroll
      for (int c = 0; c < N_TILE; c += 32) {
        uint32_t r[32];
        tmem_load_32(tmem_base + ((uint32_t)(quad * 32) << 16) + c, r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (c + i < N_TILE) acc[c + i] = __uint_as_float(r[i]);
      }
      if (EPILOGUE == kEpilogueRownorm && p.normalize) {
        float ss = 0.0f;
#pragma unroll
        for (int i = 0; i < N_TILE; ++i) ss = fmaf(acc[i], acc[i], ss);
        const float inv = 1.0f / fmaxf(sqrtf(ss), 1e-12f);
#pragma unroll
        for (int i = 0; i < N_TILE; ++i) acc[i] *= inv;
      }
      if (EPILOGUE == kEpilogueGelu) {
#pragma unroll
        for (int i = 0; i < N_TILE; ++i) acc[i] = 0.5f * acc[i] * (1.0f + erff(acc[i] * 0.70710678118654752440f));
      }
      if (row < p.M) {
        if (p.out_f32) {
          float4 *dst = reinterpret_cast<float4 *>(p.out_f32 + row * p.ldc + n0);
#pragma unroll
          for (int i = 0; i < N_TILE / 4; ++i) dst[i] = make_float4(acc[4 * i], acc[4 * i + 1], acc[4 * i + 2], acc[4 * i + 3]);
        }
        if (p.out_bf16) {
          uint4 *dst = reinterpret_cast<uint4 *>(p.out_bf16 + row * p.ldc + n0);
#pragma unroll
          for (int i = 0; i < N_TILE / 8; ++i) {
            uint4 v;
            v.x = (uint32_t)float_to_bf16_bits(acc[8 * i]) | ((uint32_t)float_to_bf16_bits(acc[8 * i + 1]) << 16);
            v.y = (uint32_t)float_to_bf16_bits(acc[8 * i + 2]) | ((uint32_t)float_to_bf16_bits(acc[8 * i + 3]) << 16);
            v.z = (uint32_t)float_to_bf16_bits(acc[8 * i + 4]) | ((uint32_t)float_to_bf16_bits(acc[8 * i + 5]) << 16);
            v.w = (uint32_t)float_to_bf16_bits(acc[8 * i + 6]) | ((uint32_t)float_to_bf16_bits(acc[8 * i + 7]) << 16);
            dst[i] = v;
          }
        }
      }
    } else if (!ok) {
      abort_s = 1;
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS));
  }
  if (threadIdx.x == 0 && abort_s && p.status) atomicAdd(p.status, 1);
}

// ------------------------------------------------------------------------------------------------ host side

template <int N_TILE, int EPILOGUE>
static int launch_gemm(const void *A, int64_t M, int64_t K, int64_t lda, const void *B, int64_t N, int64_t ldb,
                       GemmParams p, cudaStream_t s) {
  constexpr int STAGES = N_TILE <= 64 ? 4 : 3;
  constexpr int STAGE_BYTES = kTileM * kTileK * 2 + N_TILE * kTileK * 2;
  CUtensorMap map_a, map_b;
  int rc = make_map(&map_a, A, M, K, lda, kTileM);
  if (rc != LSA_OK) return rc;
  rc = make_map(&map_b, B, N, K, ldb, N_TILE);
  if (rc != LSA_OK) return rc;
  const size_t smem = (size_t)STAGES * STAGE_BYTES + 1024;
  auto kernel = umma_gemm_kernel<N_TILE, STAGES, EPILOGUE>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return LSA_ERR_LAUNCH;
  p.k_blocks = (int)((K + kTileK - 1) / kTileK);
  dim3 grid((unsigned)((M + kTileM - 1) / kTileM), (unsigned)(N / N_TILE));
  kernel<<<grid, kGemmThreads, smem, s>>>(map_a, map_b, p);
  LSA_LAUNCH_CHECK();
  return LSA_OK;
}

}  // namespace lsa

// ================================================================================================ C ABI

LSA_API int lsa_index_map_tc(const uint16_t *x, int64_t rows, int64_t d_in, int64_t x_row_stride,
                             const uint16_t *Wt, int d_idx, int normalize, float *out_f32, uint16_t *out_bf16,
                             int32_t *status, void *stream) {
  LSA_REQUIRE(x && Wt && (out_f32 || out_bf16), LSA_ERR_NULL);
  LSA_REQUIRE(rows >= 0 && d_in >= 1 && x_row_stride >= d_in, LSA_ERR_ARGUMENT);
  // TMA wants 16-byte aligned bases and row pitches
  LSA_REQUIRE(((uintptr_t)x % 16) == 0 && ((uintptr_t)Wt % 16) == 0 && x_row_stride % 8 == 0 && d_in % 8 == 0,
              LSA_ERR_ARGUMENT);
  LSA_REQUIRE(d_idx == 32 || d_idx == 64 || d_idx == 128, LSA_ERR_UNSUPPORTED);
  if (rows == 0) return LSA_OK;
  lsa::GemmParams p = {};
  p.out_f32 = out_f32;
  p.out_bf16 = out_bf16;
  p.status = status;
  p.M = rows;
  p.ldc = d_idx;
  p.normalize = normalize;
  cudaStream_t s = (cudaStream_t)stream;
  if (d_idx == 32)
    return lsa::launch_gemm<32, lsa::kEpilogueRownorm>(x, rows, d_in, x_row_stride, Wt, d_idx, d_in, p, s);
  if (d_idx == 64)
    return lsa::launch_gemm<64, lsa::kEpilogueRownorm>(x, rows, d_in, x_row_stride, Wt, d_idx, d_in, p, s);
  return lsa::launch_gemm<128, lsa::kEpilogueRownorm>(x, rows, d_in, x_row_stride, Wt, d_idx, d_in, p, s);
}

LSA_API int lsa_gemm_gelu_tc(const uint16_t *x, int64_t rows, int64_t d_in, int64_t x_row_stride, const uint16_t *Wt,
                             int64_t d_out, uint16_t *out_bf16, int32_t *status, void *stream) {
  LSA_REQUIRE(x && Wt && out_bf16, LSA_ERR_NULL);
  LSA_REQUIRE(rows >= 0 && d_in >= 1 && x_row_stride >= d_in && d_out >= 128 && d_out % 128 == 0, LSA_ERR_ARGUMENT);
  LSA_REQUIRE(((uintptr_t)x % 16) == 0 && ((uintptr_t)Wt % 16) == 0 && x_row_stride % 8 == 0 && d_in % 8 == 0,
              LSA_ERR_ARGUMENT);
  if (rows == 0) return LSA_OK;
  lsa::GemmParams p = {};
  p.out_bf16 = out_bf16;
  p.status = status;
  p.M = rows;
  p.ldc = d_out;
  return lsa::launch_gemm<128, lsa::kEpilogueGelu>(x, rows, d_in, x_row_stride, Wt, d_out, d_in, p,
                                                   (cudaStream_t)stream);
}
