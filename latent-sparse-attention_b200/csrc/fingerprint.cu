// Page fingerprints for prefix reuse: a fingerprint of each page of what a rank stores for its keys, so a request
// that arrives with a cached prefix can take the index another request built from the same bits
// (src/lsa/sglang/index/layer_index.py:89-137, src/lsa/sglang/index/bucket_cache.py:11-19,257-331).
//
// A row's bits are read as 64-bit words; the fingerprint is a weighted sum, by odd weights a word and a position,
// that wraps instead of rounding - exact whatever order it is added in, so the lanes, warps and ranks may add in any.
// A slot another rank owns adds nothing, and a group's sum of its ranks' fingerprints is the whole page's.
//
// Byte work bound by HBM: a page is read once, a warp a row with the lanes side by side over its words, a page's rows
// dealt over as many CTAs as fill the SMs.
#include "common.cuh"

namespace lsa {

constexpr int kPrintThreads = 256;

__global__ void __launch_bounds__(kPrintThreads)
    page_fingerprints_kernel(const uint64_t *__restrict__ stored, const int64_t *__restrict__ slots,
                             int64_t slot_count, int page_rows, int row_words, int64_t row_stride_words,
                             const uint8_t *__restrict__ owned, const uint64_t *__restrict__ word_weights,
                             const uint64_t *__restrict__ position_weights, int64_t *__restrict__ out) {
  __shared__ uint64_t warp_sums[kPrintThreads / 32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t page = blockIdx.x;
  uint64_t total = 0;
  // (a page's rows are dealt over the CTAs of its grid row: a wrapping sum does not mind who adds what)
  for (int r = blockIdx.y * (kPrintThreads / 32) + warp; r < page_rows; r += gridDim.y * (kPrintThreads / 32)) {
    const int64_t at = page * page_rows + r;
    if (owned && !owned[at]) continue;
    const int64_t row = slots ? slots[at] : at;
    if (row < 0 || (slots && row >= slot_count)) continue;
    const uint64_t *words = stored + row * row_stride_words;
    uint64_t sum = 0;  // (this lane's words of the row; the lanes' shares meet once, at the end)
    for (int w = lane; w < row_words; w += 32) sum += __ldg(words + w) * __ldg(word_weights + w);
    total += sum * __ldg(position_weights + r);
  }
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) total += __shfl_xor_sync(0xffffffffu, total, offset);
  if (lane == 0) warp_sums[warp] = total;
  __syncthreads();
  if (threadIdx.x == 0) {
    uint64_t sum = 0;
    for (int w = 0; w < kPrintThreads / 32; ++w) sum += warp_sums[w];
    atomicAdd(reinterpret_cast<unsigned long long *>(out + page), (unsigned long long)sum);
  }
}

}  // namespace lsa

LSA_API int lsa_page_fingerprints(const void *stored, int64_t row_stride_bytes, int row_bytes, const int64_t *slots,
                                  int64_t slot_count, int64_t pages, int page_rows, const uint8_t *owned,
                                  const int64_t *word_weights, const int64_t *position_weights, int64_t *out,
                                  void *stream) {
  LSA_REQUIRE(stored && word_weights && position_weights && out, LSA_ERR_NULL);
  LSA_REQUIRE(pages >= 0 && page_rows >= 1 && row_bytes >= 8 && row_bytes % 8 == 0 && row_stride_bytes >= row_bytes &&
                  row_stride_bytes % 8 == 0 && ((uintptr_t)stored % 8) == 0 && slot_count >= 0,
              LSA_ERR_ARGUMENT);
  if (pages == 0) return LSA_OK;
  LSA_REQUIRE(pages <= 0x7fffffff, LSA_ERR_UNSUPPORTED);
  // enough CTAs to fill the SMs a few times over, whatever the count of pages: each adds its share into the page's sum
  int shares = (int)((4 * (int64_t)lsa::sm_count() + pages - 1) / pages);
  const int most = (page_rows + lsa::kPrintThreads / 32 - 1) / (lsa::kPrintThreads / 32);
  shares = shares < 1 ? 1 : (shares > most ? most : shares);
  if (cudaMemsetAsync(out, 0, (size_t)pages * sizeof(int64_t), (cudaStream_t)stream) != cudaSuccess) return LSA_ERR_LAUNCH;
  lsa::page_fingerprints_kernel<<<dim3((unsigned)pages, (unsigned)shares), lsa::kPrintThreads, 0, (cudaStream_t)stream>>>(
      (const uint64_t *)stored, slots, slot_count, page_rows, row_bytes / 8, row_stride_bytes / 8, owned,
      (const uint64_t *)word_weights, (const uint64_t *)position_weights, out);
  LSA_LAUNCH_CHECK();
  return LSA_OK;
}
