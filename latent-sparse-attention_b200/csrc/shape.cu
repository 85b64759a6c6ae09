// Bucket shapes on the device: building them from the keys a bucket holds, and scoring rows of buckets by their
// estimated best key (src/lsa/core/shape.py:36-137; the served builders: src/lsa/core/kernels/triton/shape.py:720-886).
//
// A shape is built exactly: a CTA a bucket sums the [d, d] covariance of its keys about the centroid in shared
// memory (members in stored order) - or, for a bucket of at most 32 keys and fewer than d, the [n, n] Gram matrix of
// the residuals, which carries the same variances and is the smaller matrix (the reference's route for buckets,
// src/lsa/core/kernels/triton/shape.py:849-886) - diagonalises it with cyclic Jacobi rotations and keeps the `rank`
// leading directions as sign bits with their variances; the rest of the trace is the floor. A bucket's few keys
// spread nearly alike along several directions, where a power iteration stops short; the rotations find every
// direction to fp32 rounding whatever the gaps.
#include "common.cuh"
#include "shape.cuh"

namespace lsa {

constexpr int kShapeThreads = 128;
constexpr int kShapeSweeps = 16;
constexpr int kShapeBatch = 8;   // members staged a round of the covariance sum
constexpr int kShapeGram = 32;   // a bucket of at most this many keys goes through its Gram matrix

// Cyclic Jacobi on a symmetric M x M matrix A (row pitch `ld`), M even: a round rotates M / 2 disjoint (p, q) planes
// at once (the circle method's pairing), M - 1 rounds a sweep, until a sweep turns nothing. V (same pitch, the
// identity on entry) collects the rotations: column k = direction k, A's diagonal its variance. Every thread of the
// CTA calls this.
__device__ void jacobi_sweeps(float *A, float *V, int M, int ld, float trace, float *cos_s, float *sin_s, int *p_s,
                              int *q_s, int *moved_s) {
  const int tid = threadIdx.x, half = M >> 1;
  // A plane whose off-diagonal entry is this small against the spread of the whole bucket is left alone: turning it
  // would move a direction by less than fp32 holds. So is a plane of two directions that both carry next to nothing
  // (n keys spread along n - 1 directions at most: the rest is rounding noise that would keep the sweeps going).
  const float tiny = fmaxf(trace, 1e-30f) * (1e-7f / M);
  const float nothing = fmaxf(trace, 1e-30f) * 1e-7f;
  for (int sweep = 0; sweep < kShapeSweeps; ++sweep) {
    if (tid == 0) *moved_s = 0;
    __syncthreads();
    for (int round = 0; round < M - 1; ++round) {
      if (tid < half) {
        int p, q;
        if (tid == 0) {
          p = M - 1, q = round;
        } else {
          p = (round + tid) % (M - 1), q = (round - tid + (M - 1)) % (M - 1);
        }
        if (p > q) {
          const int t = p;
          p = q, q = t;
        }
        const float apq = A[p * ld + q], app = A[p * ld + p], aqq = A[q * ld + q];
        float c = 1.0f, s = 0.0f;
        if (fabsf(apq) > tiny && fmaxf(fabsf(app), fabsf(aqq)) > nothing) {
          const float theta = (aqq - app) / (2.0f * apq);
          const float t = (theta >= 0.0f ? 1.0f : -1.0f) / (fabsf(theta) + sqrtf(theta * theta + 1.0f));
          c = 1.0f / sqrtf(t * t + 1.0f);
          s = t * c;
          *moved_s = 1;
        }
        p_s[tid] = p, q_s[tid] = q, cos_s[tid] = c, sin_s[tid] = s;
      }
      __syncthreads();
      // columns: A <- A J, V <- V J
      for (int e = tid; e < M * half; e += kShapeThreads) {
        const int i = e / half, k = e - i * half;
        const float c = cos_s[k], s = sin_s[k];
        if (s == 0.0f) continue;  // (a plane left alone)
        const int p = p_s[k], q = q_s[k];
        const float aip = A[i * ld + p], aiq = A[i * ld + q];
        A[i * ld + p] = c * aip - s * aiq;
        A[i * ld + q] = s * aip + c * aiq;
        const float vip = V[i * ld + p], viq = V[i * ld + q];
        V[i * ld + p] = c * vip - s * viq;
        V[i * ld + q] = s * vip + c * viq;
      }
      __syncthreads();
      // rows: A <- J^T A
      for (int e = tid; e < M * half; e += kShapeThreads) {
        const int k = e / M, j = e - k * M;
        const float c = cos_s[k], s = sin_s[k];
        if (s == 0.0f) continue;
        const int p = p_s[k], q = q_s[k];
        const float apj = A[p * ld + j], aqj = A[q * ld + j];
        A[p * ld + j] = c * apj - s * aqj;
        A[q * ld + j] = s * apj + c * aqj;
      }
      __syncthreads();
    }
    if (!*moved_s) break;  // (read after the round's last barrier, by every thread alike)
    __syncthreads();
  }
}

template <int D>
__global__ void __launch_bounds__(kShapeThreads)
    shape_build_kernel(const float *__restrict__ index_keys, int64_t key_base, int64_t key_rows,
                       const float *__restrict__ centroids, const int32_t *__restrict__ members, int64_t m, int cap,
                       int rank, uint8_t *__restrict__ basis_out, float *__restrict__ variances_out,
                       float *__restrict__ floors_out) {
  constexpr int LD = D + 1;
  constexpr int kSmall = kShapeGram * (kShapeGram + 1);  // a Gram matrix, and as much again for its rotations
  __shared__ float mat_s[D * LD > 2 * kSmall ? D * LD : 2 * kSmall];  // the matrix that is diagonalised
  __shared__ float vec_s[D * LD];  // the rotations of the covariance, or the residuals a Gram matrix is made of
  __shared__ float res_s[kShapeBatch][D];
  __shared__ float cos_s[D / 2], sin_s[D / 2];
  __shared__ int p_s[D / 2], q_s[D / 2];
  __shared__ float centre_s[D];
  __shared__ float diag_s[D];
  __shared__ int order_s[D];
  __shared__ int32_t held_s[kShapeGram];
  __shared__ int size_s, moved_s;
  __shared__ float trace_s;

  const int tid = threadIdx.x;
  const int64_t bucket = blockIdx.x;
  if (bucket >= m) return;
  if (tid < D) centre_s[tid] = centroids[bucket * D + tid];
  int mine = 0;
  for (int s = tid; s < cap; s += kShapeThreads) mine += members[bucket * cap + s] >= 0;
  if (tid == 0) size_s = 0;
  __syncthreads();
  if (mine) atomicAdd(&size_s, mine);
  __syncthreads();
  const int n = size_s;
  // Fewer keys than dims: the [n, n] Gram matrix of the residuals has the covariance's nonzero variances (times n)
  // and is the smaller matrix to diagonalise; its direction w gives the covariance's as R^T w.
  const bool gram = n <= kShapeGram && n < D;
  const int M = gram ? max(2, (n + 1) & ~1) : D;
  const int ld = gram ? M + 1 : LD;
  float *A = mat_s, *V = gram ? mat_s + kSmall : vec_s;

  if (gram) {
    // ---- the held members in stored order (a bucket's row may hold padding anywhere), their residuals, the Gram matrix
    if (tid == 0) {
      int at = 0;
      for (int s = 0; s < cap && at < n; ++s) {
        const int32_t id = members[bucket * cap + s];
        if (id >= 0) held_s[at++] = id;
      }
    }
    __syncthreads();
    for (int e = tid; e < M * D; e += kShapeThreads) {
      const int s = e / D, i = e - s * D;
      float r = 0.0f;
      if (s < n) {
        const int64_t at = (int64_t)held_s[s] - key_base;
        if (at >= 0 && at < key_rows) r = index_keys[at * D + i] - centre_s[i];
      }
      vec_s[s * LD + i] = r;
    }
    __syncthreads();
    for (int e = tid; e < M * M; e += kShapeThreads) {
      const int a = e / M, b = e - a * M;
      float acc = 0.0f;
#pragma unroll 8
      for (int i = 0; i < D; ++i) acc = fmaf(vec_s[a * LD + i], vec_s[b * LD + i], acc);
      A[a * ld + b] = acc;
      V[a * ld + b] = a == b ? 1.0f : 0.0f;
    }
  } else {
    for (int e = tid; e < D * D; e += kShapeThreads) {
      A[(e / D) * LD + e % D] = 0.0f;
      V[(e / D) * LD + e % D] = e / D == e % D ? 1.0f : 0.0f;
    }
    __syncthreads();
    // ---- covariance: residuals of a few members at a time, every thread adds them into its own entries in slot order
    for (int s0 = 0; s0 < cap; s0 += kShapeBatch) {
      for (int e = tid; e < kShapeBatch * D; e += kShapeThreads) {
        const int s = s0 + e / D;
        const int64_t id = s < cap ? members[bucket * cap + s] : -1;
        const int64_t at = id - key_base;
        res_s[e / D][e % D] = id >= 0 && at >= 0 && at < key_rows ? index_keys[at * D + e % D] - centre_s[e % D] : 0.0f;
      }
      __syncthreads();
      for (int e = tid; e < D * D; e += kShapeThreads) {
        const int i = e / D, j = e % D;
        float acc = A[i * LD + j];
#pragma unroll
        for (int b = 0; b < kShapeBatch; ++b) acc = fmaf(res_s[b][i], res_s[b][j], acc);
        A[i * LD + j] = acc;
      }
      __syncthreads();
    }
  }
  __syncthreads();
  // (both matrices are sums over the keys: the variances come out times n, and are divided at the end)
  if (tid == 0) {
    float trace = 0.0f;
    for (int i = 0; i < M; ++i) trace += A[i * ld + i];
    trace_s = trace;
  }
  __syncthreads();
  if (rank > 0) jacobi_sweeps(A, V, M, ld, trace_s, cos_s, sin_s, p_s, q_s, &moved_s);
  __syncthreads();

  // ---- the leading directions: variances descending, an equal pair by the lower column
  if (tid < M) diag_s[tid] = A[tid * ld + tid];
  __syncthreads();
  if (tid < M) {
    const float own = diag_s[tid];
    int before = 0;
    for (int k = 0; k < M; ++k) before += diag_s[k] > own || (diag_s[k] == own && k < tid);
    order_s[before] = tid;
  }
  __syncthreads();
  for (int e = tid; e < rank * (D / 8); e += kShapeThreads) {
    const int j = e / (D / 8), byte = e % (D / 8);
    unsigned bits = 0;
    if (j < M) {
      const int column = order_s[j];
      for (int b = 0; b < 8; ++b) {
        const int i = byte * 8 + b;
        float along;
        if (gram) {  // the covariance's direction is R^T w (a positive multiple of it: only the signs are kept)
          along = 0.0f;
          for (int s = 0; s < n; ++s) along = fmaf(vec_s[s * LD + i], V[s * ld + column], along);
        } else {
          along = V[i * ld + column];
        }
        bits |= (along > 0.0f ? 1u : 0u) << b;
      }
    }
    basis_out[(bucket * rank + j) * (D / 8) + byte] = (uint8_t)bits;
  }
  if (tid == 0) {
    const float over = 1.0f / (float)max(n, 1);
    float kept = 0.0f;
    for (int j = 0; j < rank; ++j) {
      const float variance = j < M ? fmaxf(diag_s[order_s[j]], 0.0f) * over : 0.0f;
      variances_out[bucket * rank + j] = variance;
      kept += variance;
    }
    floors_out[bucket] = fmaxf((trace_s * over - kept) / (float)max(D - rank, 1), 0.0f);
  }
}

// Scores of rows of buckets: row r against the table rows `rows[r, :]` (-1 = none, scored -inf), or against table rows
// 0..width when `rows` is NULL. 8 query rows a CTA share their staged queries; a thread a (row, column).
__global__ void __launch_bounds__(256)
    shaped_scores_kernel(const float *__restrict__ queries, const float *__restrict__ centroids, int64_t m,
                         ShapeTable table, const int32_t *__restrict__ rows, int64_t R, int d, int64_t width,
                         float *__restrict__ scores_out) {
  extern __shared__ __align__(16) float q_s[];  // [8][d]
  const int64_t row0 = (int64_t)blockIdx.y * 8;
  for (int e = threadIdx.x; e < 8 * d; e += blockDim.x) {
    const int64_t r = row0 + e / d;
    q_s[e] = r < R ? queries[r * d + e % d] : 0.0f;
  }
  __syncthreads();
  const int64_t col = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= width) return;
  for (int i = 0; i < 8 && row0 + i < R; ++i) {
    const int64_t r = row0 + i;
    const int64_t at = rows ? rows[r * width + col] : col;
    float score = -INFINITY;
    if (at >= 0 && at < m) {
      const float4 *c4 = reinterpret_cast<const float4 *>(centroids + at * d);
      const float *q = q_s + i * d;
      float acc = 0.0f;
      for (int k4 = 0; k4 < d / 4; ++k4) {
        const float4 v = __ldg(c4 + k4);
        acc = fmaf(q[4 * k4], v.x, acc), acc = fmaf(q[4 * k4 + 1], v.y, acc);
        acc = fmaf(q[4 * k4 + 2], v.z, acc), acc = fmaf(q[4 * k4 + 3], v.w, acc);
      }
      score = shaped_score(acc, q, d, table, at);
    }
    scores_out[r * width + col] = score;
  }
}

}  // namespace lsa

LSA_API int lsa_shape_build(const float *index_keys, int64_t key_base, int64_t key_rows, const float *centroids,
                            const int32_t *members, int64_t m, int cap, int d, int rank, uint8_t *basis_out,
                            float *variances_out, float *floors_out, void *stream) {
  LSA_REQUIRE(index_keys && centroids && members && floors_out, LSA_ERR_NULL);
  LSA_REQUIRE(m >= 0 && cap >= 1 && key_rows >= 0 && rank >= 0 && rank <= d, LSA_ERR_ARGUMENT);
  LSA_REQUIRE(rank == 0 || (basis_out && variances_out), LSA_ERR_NULL);
  LSA_REQUIRE(d == 32 || d == 64, LSA_ERR_UNSUPPORTED);
  if (m == 0) return LSA_OK;
  LSA_REQUIRE(m <= 0x7fffffff, LSA_ERR_UNSUPPORTED);
  cudaStream_t s = (cudaStream_t)stream;
  if (d == 64)
    lsa::shape_build_kernel<64><<<(unsigned)m, lsa::kShapeThreads, 0, s>>>(
        index_keys, key_base, key_rows, centroids, members, m, cap, rank, basis_out, variances_out, floors_out);
  else
    lsa::shape_build_kernel<32><<<(unsigned)m, lsa::kShapeThreads, 0, s>>>(
        index_keys, key_base, key_rows, centroids, members, m, cap, rank, basis_out, variances_out, floors_out);
  LSA_LAUNCH_CHECK();
  return LSA_OK;
}

LSA_API int lsa_shaped_scores(const float *queries, int64_t R, int d, const float *centroids, int64_t m,
                              const uint8_t *basis, const float *variances, const float *floors, int rank,
                              float deviations, const int32_t *rows, int64_t width, float *scores_out, void *stream) {
  LSA_REQUIRE(queries && centroids && floors && scores_out, LSA_ERR_NULL);
  LSA_REQUIRE(R >= 0 && m >= 0 && width >= 0 && d >= 32 && d % 32 == 0 && d <= 1024 && rank >= 0 && rank <= d,
              LSA_ERR_ARGUMENT);
  LSA_REQUIRE(rank == 0 || (basis && variances && ((uintptr_t)basis % 4) == 0), LSA_ERR_ARGUMENT);
  LSA_REQUIRE(((uintptr_t)centroids % 16) == 0, LSA_ERR_ARGUMENT);
  if (R == 0 || width == 0) return LSA_OK;
  lsa::ShapeTable table;
  table.basis = reinterpret_cast<const uint32_t *>(basis);
  table.variances = variances, table.floors = floors;
  table.rank = rank, table.deviations = deviations, table.scale = 1.0f / sqrtf((float)d);
  const dim3 grid((unsigned)((width + 255) / 256), (unsigned)((R + 7) / 8));
  LSA_REQUIRE(grid.y <= 65535, LSA_ERR_UNSUPPORTED);
  lsa::shaped_scores_kernel<<<grid, 256, (size_t)8 * d * 4, (cudaStream_t)stream>>>(
      queries, centroids, m, table, rows, R, d, width, scores_out);
  LSA_LAUNCH_CHECK();
  return LSA_OK;
}
