// Index space: grouped-query head sum, learned linear map and row normalisation in one pass over the heads.
//
// out[s] = normalize( sum_kv (sum_{g < group} x[s, kv*group + g, off : off + dh_used]) @ W[kv*dh_used : (kv+1)*dh_used] )
// with fp32 accumulation in ascending input-dim order. This is the exact-arithmetic form; rows are read once and
// the head sum never reaches memory.
#include "common.cuh"

namespace lsa {

constexpr int kMapThreads = 256;
constexpr int kMapRows = 64;    // rows a CTA maps, two a thread
constexpr int kMapSlice = 64;   // input dims staged at a time
constexpr int kMapMaxCols = 16; // output dims a thread holds: a CTA writes a slice of up to 128 output dims
constexpr int kMapColSlice = 8 * kMapMaxCols;

template <typename TX, typename TW>
__global__ void __launch_bounds__(kMapThreads)
    index_map_kernel(const TX *__restrict__ x, int64_t rows, int heads, int group, int dh_off, int dh_used,
                     int64_t x_row_stride, int64_t x_head_stride, const TW *__restrict__ W, int d_idx, int normalize,
                     float *__restrict__ out_f32, uint16_t *__restrict__ out_bf16) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float *xs = reinterpret_cast<float *>(smem_raw);       // [kMapRows][kMapSlice + 1]
  float *ws = xs + kMapRows * (kMapSlice + 1);           // [kMapSlice][d_idx]
  const int tid = threadIdx.x;
  const int row_a = tid >> 3, row_b = row_a + 32, cg = tid & 7;
  const int64_t row0 = (int64_t)blockIdx.x * kMapRows;
  const int d_in = heads / group * dh_used;
  // blockIdx.y picks the slice of output dims; a map wider than one slice is normalised by a second kernel
  const int col0 = blockIdx.y * kMapColSlice, width = min(kMapColSlice, d_idx - col0);
  const int cols = (width + 7) / 8;
  float acc_a[kMapMaxCols], acc_b[kMapMaxCols];
#pragma unroll
  for (int i = 0; i < kMapMaxCols; ++i) acc_a[i] = acc_b[i] = 0.0f;

  for (int k0 = 0; k0 < d_in; k0 += kMapSlice) {
    const int kn = min(kMapSlice, d_in - k0);
    for (int e = tid; e < kMapRows * kMapSlice; e += kMapThreads) {
      const int rr = e / kMapSlice, kk = e - rr * kMapSlice;
      float sum = 0.0f;
      const int64_t r = row0 + rr;
      if (r < rows && kk < kn) {
        const int k = k0 + kk, kv = k / dh_used, c = k - kv * dh_used;
        const TX *src = x + r * x_row_stride + (int64_t)kv * group * x_head_stride + dh_off + c;
        for (int g = 0; g < group; ++g) sum = __fadd_rn(sum, load_as_float<TX>(src, (int64_t)g * x_head_stride));
      }
      xs[rr * (kMapSlice + 1) + kk] = sum;
    }
    for (int e = tid; e < kMapSlice * width; e += kMapThreads) {
      const int kk = e / width, j = col0 + e - kk * width;
      float w = 0.0f;
      if (kk < kn) w = W ? load_as_float<TW>(W, (int64_t)(k0 + kk) * d_idx + j) : (k0 + kk == j ? 1.0f : 0.0f);
      ws[e] = w;
    }
    __syncthreads();
    for (int kk = 0; kk < kn; ++kk) {
      const float xa = xs[row_a * (kMapSlice + 1) + kk], xb = xs[row_b * (kMapSlice + 1) + kk];
      const float *wrow = ws + kk * width + cg;
#pragma unroll
      for (int i = 0; i < kMapMaxCols; ++i) {
        if (i < cols) {
          const float w = (cg + 8 * i) < width ? wrow[8 * i] : 0.0f;
          acc_a[i] = fmaf(xa, w, acc_a[i]);
          acc_b[i] = fmaf(xb, w, acc_b[i]);
        }
      }
    }
    __syncthreads();
  }

  float ss_a = 0.0f, ss_b = 0.0f;
#pragma unroll
  for (int i = 0; i < kMapMaxCols; ++i) {
    ss_a = fmaf(acc_a[i], acc_a[i], ss_a);
    ss_b = fmaf(acc_b[i], acc_b[i], ss_b);
  }
#pragma unroll
  for (int o = 1; o < 8; o <<= 1) {
    ss_a += __shfl_xor_sync(0xffffffffu, ss_a, o);
    ss_b += __shfl_xor_sync(0xffffffffu, ss_b, o);
  }
  const float den_a = normalize ? fmaxf(sqrtf(ss_a), 1e-12f) : 1.0f;
  const float den_b = normalize ? fmaxf(sqrtf(ss_b), 1e-12f) : 1.0f;
#pragma unroll
  for (int i = 0; i < kMapMaxCols; ++i) {
    const int j = col0 + cg + 8 * i;
    if (i >= cols || cg + 8 * i >= width) continue;
    if (row0 + row_a < rows) {
      const float v = acc_a[i] / den_a;
      if (out_f32) out_f32[(row0 + row_a) * d_idx + j] = v;
      if (out_bf16) out_bf16[(row0 + row_a) * d_idx + j] = float_to_bf16_bits(v);
    }
    if (row0 + row_b < rows) {
      const float v = acc_b[i] / den_b;
      if (out_f32) out_f32[(row0 + row_b) * d_idx + j] = v;
      if (out_bf16) out_bf16[(row0 + row_b) * d_idx + j] = float_to_bf16_bits(v);
    }
  }
}

// A few rows (a decode step): one CTA a row, its threads splitting the input dims, so the map of a single query
// is not one thread block walking the whole contraction alone.
constexpr int kRowThreads = 256;

template <typename TX, typename TW, int COLS>
__global__ void __launch_bounds__(kRowThreads)
    index_map_rows_kernel(const TX *__restrict__ x, int heads, int group, int dh_off, int dh_used, int64_t x_row_stride,
                          int64_t x_head_stride, const TW *__restrict__ W, int d_idx, int normalize,
                          float *__restrict__ out_f32, uint16_t *__restrict__ out_bf16) {
  __shared__ float partial[kRowThreads / 32][COLS];
  __shared__ float total[COLS];
  __shared__ float norm_s;
  const int64_t row = blockIdx.x;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int d_in = heads / group * dh_used;
  float acc[COLS];
#pragma unroll
  for (int j = 0; j < COLS; ++j) acc[j] = 0.0f;
  for (int k = tid; k < d_in; k += kRowThreads) {
    const int kv = k / dh_used, c = k - kv * dh_used;
    const TX *src = x + row * x_row_stride + (int64_t)kv * group * x_head_stride + dh_off + c;
    float xs = 0.0f;
    for (int g = 0; g < group; ++g) xs = __fadd_rn(xs, load_as_float<TX>(src, (int64_t)g * x_head_stride));
#pragma unroll
    for (int j = 0; j < COLS; ++j)
      if (j < d_idx) acc[j] = fmaf(xs, W ? load_as_float<TW>(W, (int64_t)k * d_idx + j) : (k == j ? 1.0f : 0.0f), acc[j]);
  }
#pragma unroll
  for (int j = 0; j < COLS; ++j) {
    const float v = warp_sum(acc[j]);
    if (lane == 0) partial[warp][j] = v;
  }
  __syncthreads();
  if (tid < COLS) {
    float v = 0.0f;
    for (int w = 0; w < kRowThreads / 32; ++w) v += partial[w][tid];
    total[tid] = tid < d_idx ? v : 0.0f;
  }
  __syncthreads();
  if (tid == 0) {
    float ss = 0.0f;
    for (int j = 0; j < d_idx; ++j) ss = fmaf(total[j], total[j], ss);
    norm_s = normalize ? fmaxf(sqrtf(ss), 1e-12f) : 1.0f;
  }
  __syncthreads();
  if (tid < d_idx) {
    const float v = total[tid] / norm_s;
    if (out_f32) out_f32[row * d_idx + tid] = v;
    if (out_bf16) out_bf16[row * d_idx + tid] = float_to_bf16_bits(v);
  }
}

// Unit rows in place, a warp a row: the second pass of a map wider than one slice.
__global__ void __launch_bounds__(256)
    rownorm_kernel(float *__restrict__ rows, int64_t n, int d, uint16_t *__restrict__ out_bf16) {
  const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= n) return;
  float *r = rows + row * d;
  float ss = 0.0f;
  for (int j = lane; j < d; j += 32) ss = fmaf(r[j], r[j], ss);
  ss = warp_sum(ss);
  const float den = fmaxf(sqrtf(ss), 1e-12f);
  for (int j = lane; j < d; j += 32) {
    const float v = r[j] / den;
    r[j] = v;
    if (out_bf16) out_bf16[row * d + j] = float_to_bf16_bits(v);
  }
}

// The head sum alone (no map, no normalisation): out[r, kv*dh_used + c] = sum_g x[r, kv*group + g, off + c], added in
// head order - what the identity map computes, without walking a contraction.
template <typename TX>
__global__ void __launch_bounds__(256)
    head_sum_kernel(const TX *__restrict__ x, int64_t rows, int d_in, int group, int dh_off, int dh_used,
                    int64_t x_row_stride, int64_t x_head_stride, float *__restrict__ out_f32,
                    uint16_t *__restrict__ out_bf16) {
  const int64_t e = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (e >= rows * d_in) return;
  const int64_t r = e / d_in;
  const int k = (int)(e - r * d_in), kv = k / dh_used, c = k - kv * dh_used;
  const TX *src = x + r * x_row_stride + (int64_t)kv * group * x_head_stride + dh_off + c;
  float sum = 0.0f;
  for (int g = 0; g < group; ++g) sum = __fadd_rn(sum, load_as_float<TX>(src, (int64_t)g * x_head_stride));
  if (out_f32) out_f32[e] = sum;
  if (out_bf16) out_bf16[e] = float_to_bf16_bits(sum);
}

template <typename TX, typename TW>
static int launch_index_map(const void *x, int64_t rows, int heads, int group, int dh_off, int dh_used,
                            int64_t x_row_stride, int64_t x_head_stride, const void *W, int d_idx, int normalize,
                            float *out_f32, uint16_t *out_bf16, cudaStream_t s) {
  if (!W && !normalize) {
    const int64_t total = rows * d_idx;
    head_sum_kernel<TX><<<(unsigned)((total + 255) / 256), 256, 0, s>>>(
        (const TX *)x, rows, d_idx, group, dh_off, dh_used, x_row_stride, x_head_stride, out_f32, out_bf16);
    LSA_LAUNCH_CHECK();
    return LSA_OK;
  }
  if (rows <= 32 && d_idx <= 128) {
    if (d_idx <= 64)
      index_map_rows_kernel<TX, TW, 64><<<(unsigned)rows, kRowThreads, 0, s>>>(
          (const TX *)x, heads, group, dh_off, dh_used, x_row_stride, x_head_stride, (const TW *)W, d_idx, normalize,
          out_f32, out_bf16);
    else
      index_map_rows_kernel<TX, TW, 128><<<(unsigned)rows, kRowThreads, 0, s>>>(
          (const TX *)x, heads, group, dh_off, dh_used, x_row_stride, x_head_stride, (const TW *)W, d_idx, normalize,
          out_f32, out_bf16);
    LSA_LAUNCH_CHECK();
    return LSA_OK;
  }
  const int slices = (d_idx + kMapColSlice - 1) / kMapColSlice;
  const size_t smem =
      sizeof(float) * ((size_t)kMapRows * (kMapSlice + 1) + (size_t)kMapSlice * min(d_idx, kMapColSlice));
  if (cudaFuncSetAttribute(index_map_kernel<TX, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
      cudaSuccess)
    return LSA_ERR_LAUNCH;
  const dim3 grid((unsigned)((rows + kMapRows - 1) / kMapRows), (unsigned)slices);
  // One slice: the CTA holds whole rows and normalises them itself. More: fp32 rows first, then unit rows in place.
  index_map_kernel<TX, TW><<<grid, kMapThreads, smem, s>>>(
      (const TX *)x, rows, heads, group, dh_off, dh_used, x_row_stride, x_head_stride, (const TW *)W, d_idx,
      slices == 1 ? normalize : 0, out_f32, slices == 1 || !normalize ? out_bf16 : nullptr);
  LSA_LAUNCH_CHECK();
  if (slices > 1 && normalize) {
    rownorm_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, s>>>(out_f32, rows, d_idx, out_bf16);
    LSA_LAUNCH_CHECK();
  }
  return LSA_OK;
}

// A linear layer over a FEW rows (a decode step's queries): out[r, n] = act(sum_k xs[r, k] Wt[n, k]), xs = the row's
// heads summed (fp32, rounded once to bf16) or the row itself. A warp owns an output column and walks its weights once
// for all rows; eight columns a CTA, so even a single row's map spreads over N / 8 CTAs instead of one.
constexpr int kLinThreads = 256;
constexpr int kLinMaxRows = 8;
// 16-byte runs of a column's weights a lane takes before anything else: 8 (2,048 weights a column), or 20 (5,120) for
// the widest maps - the kernel is built for both, so that a narrow map does not carry the registers of a wide one.

template <int kLinHeld>
__global__ void __launch_bounds__(kLinThreads)
    rows_linear_kernel(const uint16_t *__restrict__ x, int rows, int heads, int64_t x_row_stride, int64_t x_head_stride,
                       int K, const uint16_t *__restrict__ Wt, int N, int gelu, float *__restrict__ out_f32,
                       uint16_t *__restrict__ out_bf16) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint16_t *xs = reinterpret_cast<uint16_t *>(smem_raw);  // [rows][K] bf16
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  dependents_may_launch();
  // The weights of this warp's column do not depend on the kernel before: up to 5,120 of them are taken first, while
  // that kernel may still be running.
  const int n = blockIdx.x * (kLinThreads / 32) + warp;
  uint4 held[kLinHeld];
#pragma unroll
  for (int i = 0; i < kLinHeld; ++i) {
    const int k = lane * 8 + i * 256;
    held[i] = n < N && k < K ? *reinterpret_cast<const uint4 *>(Wt + (int64_t)n * K + k) : make_uint4(0, 0, 0, 0);
  }
  wait_for_earlier_grids();
  // the head sum: a thread a pair of dims, 32 heads' loads in flight at a time, added in head order
  const bool pairs = (K % 2 == 0) && (x_row_stride % 2 == 0) && (x_head_stride % 2 == 0) && ((uintptr_t)x % 4 == 0);
  if (heads == 1 && x_row_stride % 8 == 0 && ((uintptr_t)x % 16) == 0) {
    // nothing to sum: the rows are copied 16 bytes a thread, four loads in flight (K is a multiple of 8)
    const int per_row = K / 8, total = rows * per_row;
    for (int e0 = tid; e0 < total; e0 += 4 * kLinThreads) {
      uint4 v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int e = e0 + j * kLinThreads, r = e / per_row, c = e - r * per_row;
        if (e < total) v[j] = *reinterpret_cast<const uint4 *>(x + (int64_t)r * x_row_stride + c * 8);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int e = e0 + j * kLinThreads;
        if (e < total) reinterpret_cast<uint4 *>(xs)[e] = v[j];
      }
    }
  } else if (pairs) {
    for (int e = tid; e < rows * (K / 2); e += kLinThreads) {
      const int r = e / (K / 2), k = 2 * (e - r * (K / 2));
      const uint16_t *src = x + (int64_t)r * x_row_stride + k;
      float lo = 0.0f, hi = 0.0f;
      for (int h0 = 0; h0 < heads; h0 += 32) {
        uint32_t v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j)
          v[j] = h0 + j < heads ? *reinterpret_cast<const uint32_t *>(src + (int64_t)(h0 + j) * x_head_stride) : 0u;
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (h0 + j < heads) {
            lo = __fadd_rn(lo, __uint_as_float(v[j] << 16));
            hi = __fadd_rn(hi, __uint_as_float(v[j] & 0xFFFF0000u));
          }
      }
      if (heads > 1) {
        xs[r * K + k] = float_to_bf16_bits(lo), xs[r * K + k + 1] = float_to_bf16_bits(hi);
      } else {
        xs[r * K + k] = src[0], xs[r * K + k + 1] = src[1];
      }
    }
  } else {
    for (int e = tid; e < rows * K; e += kLinThreads) {
      const int r = e / K, k = e - r * K;
      const uint16_t *src = x + (int64_t)r * x_row_stride + k;
      float sum = 0.0f;
      for (int h = 0; h < heads; ++h) sum = __fadd_rn(sum, bf16_bits_to_float(src[(int64_t)h * x_head_stride]));
      xs[e] = heads > 1 ? float_to_bf16_bits(sum) : src[0];
    }
  }
  __syncthreads();
  if (n >= N) return;
  float acc[kLinMaxRows];
#pragma unroll
  for (int r = 0; r < kLinMaxRows; ++r) acc[r] = 0.0f;
  const uint16_t *w = Wt + (int64_t)n * K;
  // (K is a multiple of 8 and the rows are 16-byte aligned; a lane walks its weights in ascending order either way)
  auto fold = [&](const uint4 wv, int k) {
    const uint32_t wp[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
    for (int r = 0; r < kLinMaxRows; ++r) {
      if (r >= rows) break;
      const uint4 xv = *reinterpret_cast<const uint4 *>(xs + r * K + k);
      const uint32_t xp[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc[r] = fmaf(__uint_as_float(xp[i] << 16), __uint_as_float(wp[i] << 16), acc[r]);
        acc[r] = fmaf(__uint_as_float(xp[i] & 0xFFFF0000u), __uint_as_float(wp[i] & 0xFFFF0000u), acc[r]);
      }
    }
  };
#pragma unroll
  for (int i = 0; i < kLinHeld; ++i) {
    const int k = lane * 8 + i * 256;
    if (k < K) fold(held[i], k);
  }
#pragma unroll 4
  for (int k = lane * 8 + kLinHeld * 256; k < K; k += 32 * 8) fold(*reinterpret_cast<const uint4 *>(w + k), k);
#pragma unroll
  for (int r = 0; r < kLinMaxRows; ++r) {
    if (r >= rows) break;
    float v = warp_sum(acc[r]);
    if (gelu) v = 0.5f * v * (1.0f + erff(v * 0.70710678118654752440f));
    if (lane == 0) {
      if (out_f32) out_f32[(int64_t)r * N + n] = v;
      if (out_bf16) out_bf16[(int64_t)r * N + n] = float_to_bf16_bits(v);
    }
  }
}

// rows /= their length (fp32 in place, a warp a row), with an optional bf16 copy
__global__ void rows_unit_kernel(float *__restrict__ rows, int n_rows, int d, uint16_t *__restrict__ out_bf16) {
  dependents_may_launch();
  wait_for_earlier_grids();
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= n_rows) return;
  float ss = 0.0f;
  for (int j = lane; j < d; j += 32) ss = fmaf(rows[(int64_t)r * d + j], rows[(int64_t)r * d + j], ss);
  ss = warp_sum(ss);
  const float den = fmaxf(sqrtf(ss), 1e-12f);
  for (int j = lane; j < d; j += 32) {
    const float v = rows[(int64_t)r * d + j] / den;
    rows[(int64_t)r * d + j] = v;
    if (out_bf16) out_bf16[(int64_t)r * d + j] = float_to_bf16_bits(v);
  }
}

}  // namespace lsa

LSA_API int lsa_rows_linear(const uint16_t *x, int rows, int heads, int64_t x_row_stride, int64_t x_head_stride,
                            int d_in, const uint16_t *Wt, int d_out, int flags, float *out_f32, uint16_t *out_bf16,
                            void *stream) {
  LSA_REQUIRE(x && Wt && (out_f32 || out_bf16), LSA_ERR_NULL);
  LSA_REQUIRE(rows >= 0 && rows <= lsa::kLinMaxRows && heads >= 1 && d_in >= 8 && d_in % 8 == 0 && d_out >= 1,
              LSA_ERR_ARGUMENT);
  LSA_REQUIRE(((uintptr_t)Wt % 16) == 0, LSA_ERR_ARGUMENT);
  LSA_REQUIRE(!(flags & LSA_ROWS_NORMALIZE) || out_f32, LSA_ERR_ARGUMENT);
  const size_t smem = (size_t)rows * d_in * 2;
  LSA_REQUIRE(smem <= 160 * 1024, LSA_ERR_UNSUPPORTED);
  if (rows == 0) return LSA_OK;
  auto kernel = d_in <= 2048 ? lsa::rows_linear_kernel<8> : lsa::rows_linear_kernel<20>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return LSA_ERR_LAUNCH;
  const unsigned grid = (unsigned)((d_out + lsa::kLinThreads / 32 - 1) / (lsa::kLinThreads / 32));
  const bool unit = flags & LSA_ROWS_NORMALIZE;
  lsa::launch(true, kernel, dim3(grid), dim3(lsa::kLinThreads), smem, (cudaStream_t)stream, x, rows,
              heads, x_row_stride, x_head_stride, d_in, Wt, d_out, flags & LSA_ROWS_GELU ? 1 : 0, out_f32,
              unit ? nullptr : out_bf16);
  LSA_LAUNCH_CHECK();
  if (unit) {
    lsa::launch(true, lsa::rows_unit_kernel, dim3((unsigned)((rows + 3) / 4)), dim3(128), 0, (cudaStream_t)stream,
                out_f32, rows, d_out, out_bf16);
    LSA_LAUNCH_CHECK();
  }
  return LSA_OK;
}

LSA_API int lsa_index_map(const void *x, int x_dtype, int64_t rows, int heads, int group, int dh_off, int dh_used,
                          int64_t x_row_stride, int64_t x_head_stride, const void *W, int w_dtype, int d_idx,
                          int normalize, float *out_f32, uint16_t *out_bf16, void *stream) {
  LSA_REQUIRE(x && (out_f32 || out_bf16), LSA_ERR_NULL);
  LSA_REQUIRE(rows >= 0 && heads >= 1 && group >= 1 && heads % group == 0 && dh_off >= 0 && dh_used >= 1 &&
                  d_idx >= 1,
              LSA_ERR_ARGUMENT);
  LSA_REQUIRE(x_dtype == LSA_DTYPE_F32 || x_dtype == LSA_DTYPE_BF16, LSA_ERR_ARGUMENT);
  LSA_REQUIRE(w_dtype == LSA_DTYPE_F32 || w_dtype == LSA_DTYPE_BF16, LSA_ERR_ARGUMENT);
  LSA_REQUIRE(W || d_idx == heads / group * dh_used, LSA_ERR_ARGUMENT);
  // a map wider than one slice of output dims is normalised in place in its fp32 output
  LSA_REQUIRE(d_idx <= lsa::kMapColSlice || !normalize || out_f32, LSA_ERR_UNSUPPORTED);
  if (rows == 0) return LSA_OK;
  cudaStream_t s = (cudaStream_t)stream;
  if (x_dtype == LSA_DTYPE_BF16 && w_dtype == LSA_DTYPE_BF16)
    return lsa::launch_index_map<uint16_t, uint16_t>(x, rows, heads, group, dh_off, dh_used, x_row_stride,
                                                     x_head_stride, W, d_idx, normalize, out_f32, out_bf16, s);
  if (x_dtype == LSA_DTYPE_BF16)
    return lsa::launch_index_map<uint16_t, float>(x, rows, heads, group, dh_off, dh_used, x_row_stride,
                                                  x_head_stride, W, d_idx, normalize, out_f32, out_bf16, s);
  if (w_dtype == LSA_DTYPE_BF16)
    return lsa::launch_index_map<float, uint16_t>(x, rows, heads, group, dh_off, dh_used, x_row_stride,
                                                  x_head_stride, W, d_idx, normalize, out_f32, out_bf16, s);
  return lsa::launch_index_map<float, float>(x, rows, heads, group, dh_off, dh_used, x_row_stride, x_head_stride, W,
                                             d_idx, normalize, out_f32, out_bf16, s);
}
