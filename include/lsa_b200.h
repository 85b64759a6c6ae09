/*
 * lsa_b200 - C ABI of the B200 (sm_100a) kernels for Latent Sparse Attention's selection-plus-attention path.
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer unless its comment says "host".
 *   - Every function returns 0 on success or a negative LSA_ERR_* code decided on the host before any launch.
 *     lsa_error_string() names a code. Nothing here allocates, frees or synchronises unless its comment says so:
 *     scratch memory is passed in by the caller and sized by the matching *_workspace_bytes() query.
 *   - `stream` is a cudaStream_t passed as void*; launches are asynchronous on it.
 *   - Conditions only the device can see (a truncated list, an id out of range) are counted in the int32 word
 *     `status` (may be NULL): the kernel adds one per event and carries on with a safe value; it never traps.
 *   - Strides are in ELEMENTS. bf16 data is passed as uint16_t bit patterns.
 *   - "Reference" citations name files of the Prefrontal-AI/latent-sparse-attention project whose behaviour the
 *     entry point reproduces.
 */
#ifndef LSA_B200_H
#define LSA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LSA_OK 0
#define LSA_ERR_ARGUMENT (-1)    /* a size, stride or combination the kernels do not take */
#define LSA_ERR_NULL (-2)        /* a required pointer is NULL */
#define LSA_ERR_UNSUPPORTED (-3) /* a shape outside what this build was written for */
#define LSA_ERR_WORKSPACE (-4)   /* the workspace passed in is smaller than *_workspace_bytes() asks */
#define LSA_ERR_LAUNCH (-5)      /* the CUDA runtime refused a launch or an attribute */
#define LSA_ERR_DEVICE (-6)      /* not an sm_100 device */
#define LSA_ERR_STATIC_SCRATCH (-7) /* the call needs more scratch than the built-in static array holds */

#define LSA_PAD (-1)                  /* the only padding value an id list carries (src/lsa/constants.py:16-20) */
#define LSA_EMPTY_KEY INT64_MIN       /* the packed key of no bucket (src/lsa/core/kernels/constants.py:29-37) */
/* lsa_expand flag: leave the window and the sinks out of the list (a dense band kernel reads them instead) */
#define LSA_EXPAND_NO_LOCAL 1
#define LSA_EXPAND_NO_PAD 2
#define LSA_DTYPE_F32 0
#define LSA_DTYPE_BF16 1

const char *lsa_error_string(int code);
/* ABI version of this library; bumped when a signature changes. */
int lsa_abi_version(void);

/* ---------------------------------------------------------------------------------------------------------
 * Index space: grouped-query head sum, learned map, row normalisation.
 * Reference: regroup_partial / project_partial / project / rownorm (src/lsa/core/index_space.py:134-187,
 * 378-419, 315-334); served form Projection.__call__ and KeyAndQueryProjection.index_queries / index_keys
 * (src/lsa/sglang/index/layer_index.py:256-267, 331-355).
 *
 * out[s, :] = normalize( sum_kv  ( sum_{g<group} x[s, kv*group+g, off:off+dh_used] ) @ W[kv*dh_used:(kv+1)*dh_used, :] )
 *   x        [rows, heads, *] of x_dtype with element strides (x_row_stride, x_head_stride)
 *   group    query heads added per KV head (1 for keys); heads % group == 0
 *   dh_off   first head dim read (the rotary prefix dropped), dh_used dims read per head
 *   W        [heads/group*dh_used, d_idx] of w_dtype, row-major; NULL = identity (d_idx = heads/group*dh_used)
 *   out_f32  [rows, d_idx] fp32 or NULL; out_bf16 [rows, d_idx] bf16 or NULL (at least one)
 *   normalize 0 = leave the product as it is (the partial form), 1 = unit rows, a zero row stays zero
 * A map wider than 128 output dims (the 512-dim latent space of an MLA layer, regroup_latent at
 * src/lsa/core/index_space.py:271-312) is written in slices and normalised in place by a second launch, so it
 * needs out_f32 when normalize is set.
 * --------------------------------------------------------------------------------------------------------- */
int lsa_index_map(const void *x, int x_dtype, int64_t rows, int heads, int group, int dh_off, int dh_used,
                  int64_t x_row_stride, int64_t x_head_stride, const void *W, int w_dtype, int d_idx,
                  int normalize, float *out_f32, uint16_t *out_bf16, void *stream);

/* The same map on the tensor cores (tcgen05 MMA, TMEM accumulator, TMA-fed operands) for the serving path, where
 * heads and the map are bf16 (src/lsa/sglang/index/layer_index.py:298-300,344,355 does this product in bf16 too).
 *   x    [rows, d_in] bf16 with x_row_stride elements between rows (a [rows, heads, dh] tensor with contiguous
 *        heads IS such a matrix with d_in = heads*dh); base and row pitch 16-byte aligned
 *   Wt   [d_idx, d_in] bf16, the map TRANSPOSED; for grouped queries the caller repeats a KV head's block of the
 *        map under each query head of its group (the head sum then happens inside the product) and zeroes the
 *        columns of dims the index does not read
 *   d_idx 32, 64 or 128. status (may be NULL) is raised if a bounded on-chip wait gives up. */
int lsa_index_map_tc(const uint16_t *x, int64_t rows, int64_t d_in, int64_t x_row_stride, const uint16_t *Wt,
                     int d_idx, int normalize, float *out_f32, uint16_t *out_bf16, int32_t *status, void *stream);

/* out = gelu(x @ Wt^T) in bf16, the hidden layer of the two-layer map (no counterpart in the
 * reference, whose maps are one linear projection); the second layer is lsa_index_map_tc over `out`.
 *   x [rows, d_in] bf16, Wt [d_out, d_in] bf16, out_bf16 [rows, d_out]; d_out a multiple of 128. */
int lsa_gemm_gelu_tc(const uint16_t *x, int64_t rows, int64_t d_in, int64_t x_row_stride, const uint16_t *Wt,
                     int64_t d_out, uint16_t *out_bf16, int32_t *status, void *stream);

/* A linear layer over a few rows (a decode step's queries: the same maps as above when there is one row to map and
 * a tile of 128 rows would be all padding): out[r, n] = act(sum_k xs[r, k] Wt[n, k]).
 * Reference: the map of the decode rows, src/lsa/sglang/index/layer_index.py:906-928 (a torch matmul there).
 *   x     [rows, heads, d_in] bf16 with element strides (x_row_stride, x_head_stride); the heads are summed first
 *         (fp32, rounded once to bf16) - heads = 1 reads the rows as they are; rows <= 8, d_in a multiple of 8
 *   Wt    [d_out, d_in] bf16, 16-byte aligned
 *   flags LSA_ROWS_GELU: act = the exact GELU, else the identity; LSA_ROWS_NORMALIZE: the rows of out_f32 are
 *         divided by their length afterwards (a second small launch), out_bf16 then holds the unit rows */
#define LSA_ROWS_GELU 1
#define LSA_ROWS_NORMALIZE 2
int lsa_rows_linear(const uint16_t *x, int rows, int heads, int64_t x_row_stride, int64_t x_head_stride, int d_in,
                    const uint16_t *Wt, int d_out, int flags, float *out_f32, uint16_t *out_bf16, void *stream);

/* ---------------------------------------------------------------------------------------------------------
 * Pooling. Reference: pool_keys (src/lsa/core/ward.py:15-26).
 * pools[p, :] = sum of index_keys[p*pool_size : (p+1)*pool_size, :] added in position order, fp32.
 * --------------------------------------------------------------------------------------------------------- */
int lsa_pool_keys(const void *index_keys, int key_dtype, int64_t n_pools, int pool_size, int d, float *pools,
                  void *stream);

/* ---------------------------------------------------------------------------------------------------------
 * Capped Ward bucketing of every cluster block. Reference: ward_rounds (src/lsa/core/ward.py:29-90); GPU front
 * door cluster_ward (src/lsa/core/kernels/ward.py:49-81).
 *   pool_keys  [blocks, P, d] fp32, pool_sizes [blocks, P] fp32 (NULL = every pool holds uniform_pool_size)
 *   labels     [blocks, P] int64 out - each pool's bucket, numbered by first pool
 *   reached    [blocks] uint8 out - 1 where the block got down to bucket_count
 *   rounds     [blocks] int32 out or NULL - merge rounds the block ran
 * Blocks of up to 512 pools are merged by one CTA out of shared memory (d % 4 == 0, d <= 1024, the block's
 * P * (d + 4) floats within 227 KB: 64 pools of the 512-dim latent space fit) and need no workspace. Larger blocks (up to 4,096 pools, d 16, 32 or 64: the node-bucket pairings of the tree,
 * src/lsa/core/hierarchy.py:73-98, cluster_node_buckets at src/lsa/core/kernels/ward.py:84-110) keep their state in
 * the caller's workspace and run two launches a round for max_rounds rounds without a host read; a block that is
 * finished returns at once. Costs are fp32 in the reference's evaluation order, the Gram dot added in ascending
 * dim order, so labels equal a CPU replay in that order.
 * --------------------------------------------------------------------------------------------------------- */
size_t lsa_ward_merge_workspace_bytes(int64_t blocks, int P, int d);
int lsa_ward_merge(const float *pool_keys, const float *pool_sizes, float uniform_pool_size, int64_t blocks, int P,
                   int d, int bucket_count, float bucket_cap, int max_rounds, int64_t *labels, uint8_t *reached,
                   int32_t *rounds, void *workspace, size_t workspace_bytes, void *stream);

/* ---------------------------------------------------------------------------------------------------------
 * Bucket table from labels. Reference: build_buckets (src/lsa/core/reference.py:120-144), members_from_labels
 * (src/lsa/core/ward.py:128-143), bucket_members_from_labels (src/lsa/core/kernels/triton/ward.py:551).
 *   index_keys [>= blocks*P*pool_size, d] (key_dtype), labels [blocks, P] int64
 *   members    [blocks*bucket_count, bucket_cap] int32 out, absolute positions ascending, -1 padded; position of
 *              key t of block g is first_position + g*P*pool_size + t
 *   sizes      [blocks*bucket_count] int32 out
 *   key_sums   [blocks*bucket_count, d] fp32 out or NULL - the keys added one by one in position order
 *   centroids  [blocks*bucket_count, d] fp32 out or NULL - key_sum / max(||key_sum||, 1e-30)
 *   centroids_bf16 same, rounded to bf16, or NULL
 * --------------------------------------------------------------------------------------------------------- */
int lsa_bucket_table(const void *index_keys, int key_dtype, const int64_t *labels, int64_t blocks, int P,
                     int pool_size, int d, int bucket_count, int bucket_cap, int64_t first_position,
                     int32_t *members, int32_t *sizes, float *key_sums, float *centroids,
                     uint16_t *centroids_bf16, int32_t *status, void *stream);

/* ---------------------------------------------------------------------------------------------------------
 * Update step of the k-means bucketing (the reference has no k-means: its buckets are Ward's). The
 * assignment step is lsa_flat_select with top_p = 1 over the centroids (first maximum = lower id on a tie); this
 * replaces every non-empty cluster's centroid by the normalised sum of its pools, added in pool order.
 *   pools [n, d] fp32; order [n] int64 - the pools cluster by cluster, ascending inside a cluster;
 *   offsets [k + 1] int64 - cluster j's run of `order`; centroids [k, d] fp32 in and out
 * --------------------------------------------------------------------------------------------------------- */
int lsa_kmeans_update(const float *pools, const int64_t *order, const int64_t *offsets, int k, int d,
                      float *centroids, void *stream);

/* ---------------------------------------------------------------------------------------------------------
 * Sums of gathered rows, in a fixed order: out[r, :] = sum_c src[index[r, c] - index_base, :], added one by one in
 * column order, an index < 0 ending the row. The key sums under buckets and node buckets that the tree build takes
 * (src/lsa/core/hierarchy.py:134-136, 95-97, 157).
 *   src [*, d] of src_dtype; index [rows, width] int32 or int64 (index_is_int64); out [rows, d] fp32
 * --------------------------------------------------------------------------------------------------------- */
int lsa_gather_sum(const void *src, int src_dtype, const void *index, int index_is_int64, int64_t rows, int width,
                   int d, int64_t index_base, float *out, void *stream);

/* ---------------------------------------------------------------------------------------------------------
 * Flat search, prefill form: score every visible bucket, keep the top_p packed keys of each row.
 * Reference: read / _read_row (src/lsa/core/reference.py:228-265); served Selector.read_flat
 * (src/lsa/sglang/index/selector.py:370-423), ScanSelect (src/lsa/core/kernels/scan_select.py:189-385), packed
 * keys (src/lsa/core/kernels/triton/keys.py:18-88).
 *   queries   [R, d] fp32; centroids [m, d] fp32
 *   visible   [R] int32 - buckets the row sees (a prefix of the rows of centroids), clamped to m
 *   row_top_p [R] int32 or NULL - a row's own top_p (an early budget), at most top_p
 *   bucket_id_base  added to the row index of a centroid to give the id packed in the key
 *   keys_out  [R, top_p] int64 - packed keys, best first, LSA_EMPTY_KEY after a row's count
 *   picked_out [R, top_p] int32 or NULL - the ids of keys_out, -1 padded
 * Scores are fp32 dots added in ascending dim order; a tie goes to the lower id.
 * --------------------------------------------------------------------------------------------------------- */
int lsa_flat_select(const float *queries, int64_t R, int d, const float *centroids, int64_t m,
                    const int32_t *visible, const int32_t *row_top_p, int top_p, int32_t bucket_id_base,
                    int64_t *keys_out, int32_t *picked_out, void *stream);

/* The same search with the scan on the tensor cores: the result is lsa_flat_select's, key for key. The bf16
 * scores of every (row, bucket) pair are made in tensor memory by tcgen05 products and never written; a row keeps
 * the buckets whose score, plus the bucket's own bf16 error bound, reaches a threshold bisected from 512 strided
 * samples of its scores; of the few hundred survivors those that can still be among the best top_p by their bounds
 * are rescored with lsa_flat_select's exact fp32 dot and the best top_p kept. A row is accepted only when top_p
 * survivors are sure to score the threshold or more (then no dropped bucket could have displaced one); any other
 * row - and every row that sees fewer than 1,024 buckets - is scanned exactly, so the outcome never depends on the
 * threshold being well chosen.
 * Reference: the Blackwell bucket scan (src/lsa/core/kernels/cutedsl/blackwell/bucket_scan.py:63-836), its
 * sampled thresholds (src/lsa/core/kernels/scan_select.py:228-271) and ScanSelect's exact rescoring
 * (src/lsa/core/kernels/scan_select.py:189-385).
 *   centroids_bf16 [m, 64] the scan's N operand: the centroids LESS A COMMON CENTRE, rounded to bf16 - a query's
 *                score against the centre is the same for every bucket, so the ranking is the centroids' own, and
 *                a bucket's bf16 error shrinks with the length of its row. lsa_scan_centre makes it, a run of rows
 *                at a time as an index grows: centre [64] fp32 or NULL (none); lengths [rows] fp32 out, the length
 *                of each row it wrote; radius [1] fp32, zeroed once by the caller and raised to the greatest of them
 *   lengths      [m] fp32 as lsa_scan_centre wrote them (every bucket's own error bound), with radius [1] fp32 on the
 *                device; both NULL = rows no longer than 1 (the plain bf16 rounding of lsa_bucket_table's centroids).
 *                d = 64, top_p <= 512
 *   max_visible  the host's bound on visible[] (<= 0: m) - it sets how far apart the samples lie
 *   status       (may be NULL) raised if a bounded on-chip wait gives up; the rows it cut are scanned exactly
 *   workspace    lsa_scan_select_workspace_bytes(R, top_p, m), 256-byte aligned */
int lsa_scan_centre(const float *centroids, int64_t rows, int d, const float *centre, uint16_t *out_bf16,
                    float *lengths, float *radius, void *stream);
size_t lsa_scan_select_workspace_bytes(int64_t R, int top_p, int64_t m);
int lsa_scan_select(const float *queries, int64_t R, int d, const float *centroids, const uint16_t *centroids_bf16,
                    const float *lengths, const float *radius, int64_t m, const int32_t *visible, const int32_t *row_top_p, int top_p, int32_t bucket_id_base,
                    int max_visible, int64_t *keys_out, int32_t *picked_out, int32_t *status, void *workspace,
                    size_t workspace_bytes, void *stream);

/* Every (row, bucket) score written out, each at its own column: what the reference's two-pass selection hands from
 * its scoring to its pick (dense_keys, src/lsa/core/kernels/scan_select.py:24-58; scan_paged,
 * src/lsa/core/kernels/triton/paged.py:61-101). The selection entry points above never write this matrix; it is here
 * for callers written against the two-pass form.
 *   queries [R, d] fp32; centroids [*, d] fp32; counts [R] int32 - buckets row r holds (columns past it are empty)
 *   pages [R, max_pages] int32 or NULL - row r's logical bucket i is row i % page_rows of page pages[r, i / page_rows]
 *         (-1 = no page: empty); NULL = bucket i is row i of centroids
 *   scores_out [R, width] fp32 or NULL (-inf where empty); keys_out [R, width] int64 or NULL (packed with the column
 *         + bucket_id_base, LSA_EMPTY_KEY where empty). Scores are fp32 dots added in ascending dim order. */
int lsa_dense_scores(const float *queries, int64_t R, int d, const float *centroids, const int32_t *pages,
                     int max_pages, int page_rows, const int32_t *counts, int64_t width, int32_t bucket_id_base,
                     float *scores_out, int64_t *keys_out, void *stream);

/* Flat search, decode form: few rows, many buckets. The buckets of a row are split over `splits` CTAs whose
 * local top_p lists are merged by a second kernel. Reference: Selector.decode_flat
 * (src/lsa/sglang/index/selector.py:603-660), scan_paged (src/lsa/core/kernels/triton/paged.py:61-101),
 * DecodeSelect.listed (src/lsa/core/kernels/cutedsl/decode.py:1035-1068).
 *   request_first [R] int64 - first row of centroids of each request (requests hold their buckets contiguously)
 *   workspace  lsa_flat_select_decode_workspace_bytes(R, top_p, splits)
 */
size_t lsa_flat_select_decode_workspace_bytes(int64_t R, int top_p, int splits);
int lsa_flat_select_decode(const float *queries, int64_t R, int d, const float *centroids,
                           const int64_t *request_first, const int32_t *visible, int top_p, int splits,
                           int64_t *keys_out, int32_t *picked_out, void *workspace, size_t workspace_bytes,
                           void *stream);

/* The same scan through page tables, as a serving cache holds its buckets: request r's logical bucket i is row
 * i % page_rows of page pages[r, i / page_rows] of `centroids` (-1 = no page: skipped); ids in the keys are the
 * LOGICAL bucket ids. Reference: scan_paged (src/lsa/core/kernels/triton/paged.py:61-101), DecodeSelect.listed
 * (src/lsa/core/kernels/cutedsl/decode.py:1035-1068).
 *   centroids [rows, d] fp32; pages [R, max_pages] int32; counts [R] int32 visible buckets of each request
 *   workspace as lsa_flat_select_decode_workspace_bytes(R, top_p, splits) */
int lsa_flat_select_paged(const float *queries, int64_t R, int d, const float *centroids, int64_t rows,
                          const int32_t *pages, int max_pages, int page_rows, const int32_t *counts, int top_p,
                          int splits, int64_t *keys_out, int32_t *picked_out, void *workspace,
                          size_t workspace_bytes, void *stream);

/* Global top_p of several candidate lists of packed keys (the lists every rank all-gathered, or a row's
 * splits). keys_in [parts, R, top_p] int64; keys_out [R, top_p] best first; picked_out as above or NULL. */
int lsa_merge_candidates(const int64_t *keys_in, int parts, int64_t R, int top_p, int64_t *keys_out,
                         int32_t *picked_out, void *stream);

/* ---------------------------------------------------------------------------------------------------------
 * Bucket shapes: a bucket's spread about its centroid - the covariance of its index keys kept as `rank` leading
 * directions, each rounded to one sign bit a dimension (+-1/sqrt(d)), their variances, and a floor: the rest of the
 * trace spread evenly over the directions left out. A shaped bucket scores as its estimated best key,
 *     q . c + deviations * sqrt( sum_j variance_j (q . s_j)^2 + floor (1 - sum_j (q . s_j)^2) ).
 * Reference: Shapes, build_shapes, spread, shaped_scores, pack_shape_basis (src/lsa/core/shape.py:25-170),
 * shape_buckets and the shaped read (src/lsa/core/reference.py:147-164,229-230), the served builders and scans
 * (src/lsa/core/kernels/triton/shape.py:281-343,659-717,849-886), BucketCache.shape_buckets
 * (src/lsa/sglang/index/bucket_cache.py:603-627).
 *   basis     [rows, rank, d / 8] uint8 - bit b of byte i = dimension 8 i + b, set where the sign is positive;
 *             4-byte aligned (read as words)
 *   variances [rows, rank] fp32 descending;  floors [rows] fp32;  rank 0..d (0: an even spread, basis may be NULL)
 * Every shaped entry point scores in one fixed fp32 order (q . s_j over ascending dimensions with the sign as a
 * factor, scaled once, the directions folded in order), so a bucket scores alike whichever kernel reads it.
 *
 * lsa_shape_build: the shapes of m buckets from the keys they hold, exactly (a CTA a bucket: the [d, d] covariance
 * summed in member order, diagonalised by Jacobi rotations). d = 32 or 64.
 *   index_keys [key_rows, d] fp32 - row i is the key at position key_base + i; members [m, cap] int32 positions,
 *   -1 padded (a position outside the rows given adds nothing); centroids [m, d] fp32 */
int lsa_shape_build(const float *index_keys, int64_t key_base, int64_t key_rows, const float *centroids,
                    const int32_t *members, int64_t m, int cap, int d, int rank, uint8_t *basis_out,
                    float *variances_out, float *floors_out, void *stream);

/* lsa_flat_select over shaped buckets: the same lists, a bucket scored by its estimated best key. */
int lsa_shaped_select(const float *queries, int64_t R, int d, const float *centroids, int64_t m,
                      const uint8_t *basis, const float *variances, const float *floors, int rank, float deviations,
                      const int32_t *visible, const int32_t *row_top_p, int top_p, int32_t bucket_id_base,
                      int64_t *keys_out, int32_t *picked_out, void *stream);

/* lsa_flat_select_decode over shaped buckets (the shape table is indexed like `centroids`: request_first[r] + id). */
int lsa_shaped_select_decode(const float *queries, int64_t R, int d, const float *centroids, const uint8_t *basis,
                             const float *variances, const float *floors, int rank, float deviations,
                             const int64_t *request_first, const int32_t *visible, int top_p, int splits,
                             int64_t *keys_out, int32_t *picked_out, void *workspace, size_t workspace_bytes,
                             void *stream);

/* lsa_flat_select_paged over shaped buckets: the shape table lies row for row beside `centroids` (the pages of a
 * serving cache hold a bucket's shape where they hold its centroid). */
int lsa_shaped_select_paged(const float *queries, int64_t R, int d, const float *centroids, int64_t rows,
                            const uint8_t *basis, const float *variances, const float *floors, int rank,
                            float deviations, const int32_t *pages, int max_pages, int page_rows,
                            const int32_t *counts, int top_p, int splits, int64_t *keys_out, int32_t *picked_out,
                            void *workspace, size_t workspace_bytes, void *stream);

/* Shaped scores written out: row r against the table rows rows[r, :] (int32, -1 = none: -inf), or against table
 * rows 0..width when rows is NULL (score_shaped_rows, add_planes_spread, scan_paged_shaped of the reference).
 *   scores_out [R, width] fp32 */
int lsa_shaped_scores(const float *queries, int64_t R, int d, const float *centroids, int64_t m, const uint8_t *basis,
                      const float *variances, const float *floors, int rank, float deviations, const int32_t *rows,
                      int64_t width, float *scores_out, void *stream);

/* ---------------------------------------------------------------------------------------------------------
 * Prefix reuse: a fingerprint of each page of what a rank stores for a request's keys, by which a request that
 * arrives with a cached prefix takes the index pages another request built from the same bits. Reference:
 * page_fingerprints, fingerprint_weights (src/lsa/sglang/index/layer_index.py:89-122), KeyLookup.fingerprints
 * (layer_index.py:586-610), BucketCache.adopt / fingerprint (src/lsa/sglang/index/bucket_cache.py:257-331).
 * A row's bits are read as int64 words w; out[p] = sum_r position_weights[r] * sum_w word_weights[w] * row(p, r)[w],
 * wrapping as int64 sums do: exact and independent of the order of addition.
 *   stored   the pool's rows: row i at byte i * row_stride_bytes, row_bytes read of each (both multiples of 8)
 *   slots    [pages * page_rows] int64 or NULL - the row of `stored` that holds each position of the pages (a
 *            request table's KV slots; < 0 or >= slot_count adds nothing); NULL = the rows are the positions
 *   owned    [pages * page_rows] uint8 or NULL - 0 where another rank of a decode group owns the slot (adds nothing)
 *   word_weights [>= row_bytes / 8] int64, position_weights [page_rows] int64 (odd);  out [pages] int64 */
int lsa_page_fingerprints(const void *stored, int64_t row_stride_bytes, int row_bytes, const int64_t *slots,
                          int64_t slot_count, int64_t pages, int page_rows, const uint8_t *owned,
                          const int64_t *word_weights, const int64_t *position_weights, int64_t *out, void *stream);

/* ---------------------------------------------------------------------------------------------------------
 * Tree search, one beam step: score the candidate rows of a level (open node buckets first_open..made and the
 * children carried from the level above), keep the best `keep`, a tie to the lower row.
 * Reference: beam_pick / best (src/lsa/core/hierarchy.py:402-451); served Hierarchy.beam_search, pick_buckets
 * (src/lsa/sglang/index/hierarchy.py:494-625, 765-854).
 *   vectors   [N, d] fp32 - the level's node centroids (or the bucket centroids at level 0)
 *   carried   [R, n_carried] int32 candidate rows, -1 = none; may be NULL with n_carried 0
 *   open_first/open_end [R] int32 - the run of rows every query scores besides (open_end <= open_first = none)
 *   children  [N, fanout] int64 or NULL. When given, kept_out is NULL and carried_out [R, keep*fanout] int32
 *             receives the children of the kept rows (-1 padded), best row first.
 *   kept_out  [R, keep] int32 (-1 padded), keys_out [R, keep] int64 or NULL
 * One CTA per row.
 * --------------------------------------------------------------------------------------------------------- */
int lsa_beam_step(const float *queries, int64_t R, int d, const float *vectors, int64_t N, const int32_t *carried,
                  int n_carried, const int32_t *open_first, const int32_t *open_end, int keep,
                  const int64_t *children, int fanout, int32_t *kept_out, int64_t *keys_out, int32_t *carried_out,
                  void *stream);

/* The same step with a row's candidates split over `splits` CTAs and merged by a second launch - the decode form,
 * where one query would otherwise keep one CTA busy. workspace: lsa_beam_step_workspace_bytes(R, keep, splits). */
size_t lsa_beam_step_workspace_bytes(int64_t R, int keep, int splits);
int lsa_beam_step_split(const float *queries, int64_t R, int d, const float *vectors, int64_t N,
                        const int32_t *carried, int n_carried, const int32_t *open_first, const int32_t *open_end,
                        int keep, const int64_t *children, int fanout, int splits, int32_t *kept_out,
                        int64_t *keys_out, int32_t *carried_out, void *workspace, size_t workspace_bytes,
                        void *stream);

/* ---------------------------------------------------------------------------------------------------------
 * Expansion: picked buckets -> the row's read list. Reference: expand_buckets
 * (src/lsa/core/reference.py:268-289), budget_at (src/lsa/budget.py:60-74); served expand_in_order
 * (src/lsa/core/kernels/expansion.py:16-58).
 *   picked     [R, top_p] int32 bucket rows, best first, -1 = none
 *   positions  [R] int64; members [m, bucket_cap] int32, ASCENDING within a bucket and -1 padded at the end (as
 *              lsa_bucket_table writes them): a bucket's row is read up to its first padding or member inside the window
 *   row_top_p / row_top_k [R] int32 or NULL - a row's own budget
 *   page_table [pages] int32 or NULL with page_size - when given every id is stored as the KV slot
 *              page_table[id / page_size] * page_size + id % page_size instead of the position
 *   owner_granule/owner_world/owner_rank - with owner_world > 1 the cache is dealt out round-robin in granules of
 *              owner_granule positions: only ids with (id / granule) % world == rank are written, and each is
 *              stored as its row in that rank's own cache, id / (granule*world) * granule + id % granule
 *   owner_first/owner_end - only ids in [owner_first, owner_end) are written (a rank's share of the sequence);
 *              the top_k cut still counts every id. Pass 0 and INT64_MAX for all.
 *   flags      0, or LSA_EXPAND_NO_LOCAL to write the expansion alone (the cut and the window filter stay), and / or
 *              LSA_EXPAND_NO_PAD to leave the entries past lengths[r] as they were (a caller that reads lists by
 *              their lengths, as the attention entry points do, saves the write of the padding)
 *   selected   [R, top_k + window + sink] int32 out - expansion, window ascending, sinks ascending, -1 padded
 *   lengths    [R] int32 out
 * --------------------------------------------------------------------------------------------------------- */
int lsa_expand(const int32_t *picked, int64_t R, int top_p, const int64_t *positions, const int32_t *members,
               int64_t m, int bucket_cap, const int32_t *row_top_p, const int32_t *row_top_k, int top_k,
               int sink, int window, const int32_t *page_table, int page_size, int64_t owner_first,
               int64_t owner_end, int owner_granule, int owner_world, int owner_rank, int flags,
               int32_t *selected, int32_t *lengths, int32_t *status, void *stream);

/* The same expansion for a batch of requests that share one paged cache (the serving form; reference:
 * expand_in_order / expand_by_threshold with request_blocks, request_rows and slot_table,
 * src/lsa/core/kernels/expansion.py:16-126). Beyond lsa_expand:
 *   row_request   [R] int32 request of each row (NULL = request 0)
 *   page_table    [requests, page_table_stride] KV pages of each request (positions are the request's own)
 *   bucket_pages  [requests, bucket_pages_stride] or NULL - a pick is a request's LOGICAL bucket id, stored at row
 *                 id % bucket_page_rows of page bucket_pages[request, id / bucket_page_rows] of `members` */
int lsa_expand_batched(const int32_t *picked, int64_t R, int top_p, const int64_t *positions, const int32_t *members,
                       int64_t m, int bucket_cap, const int32_t *row_top_p, const int32_t *row_top_k, int top_k,
                       int sink, int window, const int32_t *page_table, int page_size, int64_t owner_first,
                       int64_t owner_end, int owner_granule, int owner_world, int owner_rank, int flags,
                       const int32_t *row_request, int64_t page_table_stride, const int32_t *bucket_pages,
                       int64_t bucket_pages_stride, int bucket_max_pages, int bucket_page_rows, int32_t *selected,
                       int32_t *lengths, int32_t *status, void *stream);

/* ---------------------------------------------------------------------------------------------------------
 * Gather-sparse attention over each row's list, with the log-sum-exp of the scaled logits.
 * Reference: topk_attention / keep_set (src/lsa/core/attention.py:15-146); served sparse_read, partial_read
 * (src/lsa/sglang/models/qwen3_5/backend.py:427-460, 669-721).
 *   q      [R, Hq, dh] bf16 (q_row_stride, q_head_stride); dh = 64 or 128; Hq/Hkv <= 16
 *   k, v   [slots, Hkv, dh] bf16 (kv_row_stride, kv_head_stride), 16-byte aligned rows; they hold the KV rows
 *          first_slot .. first_slot + slots - 1 (a rank's share of a sequence-sharded cache; 0 for a whole one)
 *   ids    [R, list_stride] int32 - the first lengths[r] entries are read, each one once: KV rows (slots) the
 *          caller guarantees causal and distinct, as lsa_expand writes them; an entry outside
 *          [first_slot, first_slot + slots) is skipped
 *   init_out / init_lse  [R, Hq, dh] / [R, Hq] fp32 or both NULL - a partial read over OTHER keys (the dense band
 *          of lsa_band_attend) the read starts from, as one more term of the online softmax
 *   splits CTAs-per-(row, KV head) the list is divided over; > 1 needs the workspace and runs the merge kernel
 *   out    [R, Hq, dh] bf16 (out_bf16) and/or fp32 (out_f32); lse [R, Hq] fp32 or NULL
 * A row that reads nothing gives zeros and lse = -inf.
 * --------------------------------------------------------------------------------------------------------- */
size_t lsa_sparse_attend_workspace_bytes(int64_t R, int Hq, int dh, int splits);
int lsa_sparse_attend(const uint16_t *q, int64_t R, int Hq, int dh, int64_t q_row_stride, int64_t q_head_stride,
                      const uint16_t *k, const uint16_t *v, int64_t slots, int64_t first_slot, int Hkv,
                      int64_t kv_row_stride, int64_t kv_head_stride, const int32_t *ids, int64_t list_stride,
                      const int32_t *lengths, const float *init_out, const float *init_lse, float scale, int splits,
                      uint16_t *out_bf16, float *out_f32, float *lse, void *workspace, size_t workspace_bytes,
                      void *stream);

/* The same read for callers that cannot allocate device memory. This entry point has no counterpart in the
 * reference; it exists for hosts where lsa_sparse_attend's caller-provided workspace is not an option: a serving
 * engine that hands every free byte of the GPU to its KV pool at start-up and forbids later allocations, a
 * plugin thread that is given raw pointers but no allocator, or a latency-critical decode loop that must not
 * risk the implicit device synchronisation of an allocation. The scratch of a split read (the per-split partial
 * outputs and log-sum-exps) lives in an 8 MiB static device array inside the library instead, which every GPU
 * that loads the library holds until the process exits.
 *   - Arguments are those of lsa_sparse_attend without the workspace. A call that needs more than
 *     lsa_sparse_attend_static_scratch_bytes() - that is, splits * R * Hq * (dh + 1) * 4 bytes over 8 MiB -
 *     returns LSA_ERR_STATIC_SCRATCH and launches nothing; lower `splits` or the rows a call.
 *   - It calls no cudaMalloc, cudaFree or other allocating routine. The first call on each device resolves the
 *     array's device address (with that device current); make that first call outside any stream capture.
 *   - Every call on a device uses the same array and leaves its partial results in it. The kernels overwrite all
 *     they later read, so nothing has to be cleared between calls, but two calls whose kernels overlap on the GPU
 *     (different streams) race on it: serialise them. */
size_t lsa_sparse_attend_static_scratch_bytes(void);
int lsa_sparse_attend_static(const uint16_t *q, int64_t R, int Hq, int dh, int64_t q_row_stride,
                             int64_t q_head_stride, const uint16_t *k, const uint16_t *v, int64_t slots,
                             int64_t first_slot, int Hkv, int64_t kv_row_stride, int64_t kv_head_stride,
                             const int32_t *ids, int64_t list_stride,
                             const int32_t *lengths, float scale, int splits, uint16_t *out_bf16, float *out_f32,
                             float *lse, void *stream);

/* The local part of a prefill's read as dense banded attention: rows are consecutive positions (row i sits at
 * first_position + i, KV row p holds position p) and each attends to its window [pos + 1 - window, pos] and its
 * sinks [0, min(sink, window start)). One pass over the band's K/V serves 16 query rows and a whole head group.
 * The result is partial - normalised fp32 output and log-sum-exp - and is meant as lsa_sparse_attend's
 * init_out / init_lse, whose lists then hold only the selected keys (lsa_expand with LSA_EXPAND_NO_LOCAL).
 * Reference: the window and sink terms of keep_set (src/lsa/core/attention.py:49-58). sink <= 64.
 *   flags  0: heads of 128 dims packed densely and at least 128 rows go to the tensor-memory form - 128 rows of one
 *          head a CTA, both products on tcgen05 (the rows as M), K/V tiles streamed by tensor-map copies, the band
 *          walked twice (row maxima, then the sums) so the accumulator in tensor memory is never rescaled;
 *          LSA_BAND_WARP_MMA: always the warp-level form
 *   status (may be NULL) is raised if a bounded on-chip wait of the tensor-memory form gives up */
#define LSA_BAND_WARP_MMA 1
int lsa_band_attend(const uint16_t *q, int64_t R, int Hq, int dh, int64_t q_row_stride, int64_t q_head_stride,
                    const uint16_t *k, const uint16_t *v, int64_t n_keys, int Hkv, int64_t kv_row_stride,
                    int64_t kv_head_stride, int64_t first_position, int window, int sink, float scale, float *out_f32,
                    float *lse, int flags, int32_t *status, void *stream);

/* Gather-sparse attention over a shared latent cache (the MLA form): all Hq heads of a row attend over the SAME
 * listed latent rows; a key is the whole row (dk dims, rope part last), a value its first dv dims, and q holds the
 * absorbed queries (the key up-projection folded into them), so no per-head key is ever materialised.
 * Reference: topk_attention with one KV head (src/lsa/core/attention.py:65-146); the served form is FlashMLA's
 * sparse kernel behind src/lsa/sglang/plugin.py:525-598 and the indexer of
 * src/lsa/sglang/models/glm5_next/indexer.py:83-316.
 *   q       [R, Hq, dk] bf16, element strides (q_row_stride, q_head_stride), 16-byte aligned rows
 *   latent  [slots, dk] bf16 with latent_row_stride elements between rows
 *   ids     [R, list_stride] int32, the first lengths[r] entries read (all when lengths is NULL); ids outside
 *           [0, slots) are skipped. Lists hold each key once and only causal keys (lsa_expand writes such lists).
 *   out     [R, Hq, dv] bf16 and/or fp32; lse [R, Hq] natural-log log-sum-exp (-inf for an empty list)
 *   splits  CTAs a row's list is divided over; > 1 needs lsa_latent_attend_workspace_bytes() of workspace
 *   flags   0: both products run on tcgen05 with a block of 64 heads as the M side, S and O in tensor memory;
 *           LSA_LATENT_WARP_MMA: the same read on warp-level mma.sync tiles
 *   owner_granule / owner_world / owner_rank (world <= 1: off): the cache handed in is one rank's share of a
 *           cache dealt out over owner_world ranks in granules of owner_granule positions (a multiple of 64), the
 *           ids are POSITIONS, and the call reads only the positions its rank holds (position p is row
 *           p / (granule * world) * granule + p % granule of the rank (p / granule) % world) - the lists of
 *           lsa_expand with the same owner arguments hold those rows already and need none of this; tensor-memory
 *           form only
 *   status  (may be NULL) raised if a bounded on-chip wait of the tensor-memory form gives up: the output of a
 *           call that raised it is void
 * dk = 576, dv = 512 in this build. */
#define LSA_LATENT_WARP_MMA 1
size_t lsa_latent_attend_workspace_bytes(int64_t R, int Hq, int dv, int splits);
int lsa_latent_attend(const uint16_t *q, int64_t R, int Hq, int dk, int dv, int64_t q_row_stride,
                      int64_t q_head_stride, const uint16_t *latent, int64_t slots, int64_t latent_row_stride,
                      const int32_t *ids, int64_t list_stride, const int32_t *lengths, float scale, int splits,
                      uint16_t *out_bf16, float *out_f32, float *lse, int flags, int owner_granule, int owner_world,
                      int owner_rank, int32_t *status, void *workspace, size_t workspace_bytes, void *stream);

/* Bucket-major attention of a prefill chunk: expansion and gather attention in one call, the loop over buckets
 * outside the loop over rows. The result is lsa_expand (LSA_EXPAND_NO_LOCAL) followed by lsa_sparse_attend with
 * init_out / init_lse: every row attends over the members of its picked buckets that lie in
 * [sink, position + 1 - window), best bucket first and cut at top_k, merged with the partial read it starts from
 * (lsa_band_attend's window and sinks). A chunk's rows pick the same few thousand buckets a hundred times over:
 * here a bucket's K/V rows are read once per 128 (row, pick) pairs instead of once per pair.
 * Reference: expand_buckets + topk_attention (src/lsa/core/reference.py:268-289, src/lsa/core/attention.py:65-146).
 *   picked   [R, top_p] int32 bucket ids, best first, -1 = none (lsa_flat_select's picked_out)
 *   members  [m, bucket_cap] int32, ASCENDING within a bucket and -1 padded at the end (as lsa_bucket_table writes
 *            them); bucket_cap <= 64
 *   row_top_p / row_top_k [R] or NULL: a row's own budgets (the early budget)
 *   init_out [R, Hq, dh] fp32 + init_lse [R, Hq], or both NULL
 *   out_bf16 [R, Hq, dh]; lse_out [R, Hq] or NULL
 *   workspace: lsa_bucket_attend_workspace_bytes(); it holds a bf16 partial output per (row, pick, head), which is
 *            what trades the gather's repeated reads for one write and one read
 *   init_ready_event  a cudaEvent_t (as void*) or NULL: when init_out / init_lse are written on ANOTHER stream (the
 *            band kernel running beside this call's first passes) the event recorded after that work; only the
 *            merge pass waits for it
 *   status   (may be NULL) raised if a bounded on-chip wait of the tensor-memory pass gives up: the output of a call
 *            that raised it is void
 *   flags    0: the two products of a (bucket, head) run on tcgen05 with the pairs as the M = 128 rows, S and O in
 *            tensor memory; LSA_BUCKET_WARP_MMA: the same pass on warp-level mma.sync tiles of 16 rows
 * dh = 128 and Hq / Hkv <= 8 in this build; other shapes return LSA_ERR_UNSUPPORTED and the caller uses
 * lsa_expand + lsa_sparse_attend. */
#define LSA_BUCKET_WARP_MMA 1
size_t lsa_bucket_attend_workspace_bytes(int64_t R, int top_p, int Hq, int dh, int64_t m);
int lsa_bucket_attend(const uint16_t *q, int64_t R, int Hq, int dh, int64_t q_row_stride, int64_t q_head_stride,
                      const uint16_t *k, const uint16_t *v, int64_t slots, int Hkv, int64_t kv_row_stride,
                      int64_t kv_head_stride, const int32_t *picked, int top_p, const int64_t *positions,
                      const int32_t *members, int64_t m, int bucket_cap, const int32_t *row_top_p,
                      const int32_t *row_top_k, int top_k, int sink, int window, const float *init_out,
                      const float *init_lse, float scale, uint16_t *out_bf16, float *lse_out, int flags,
                      void *init_ready_event, int32_t *status, void *workspace, size_t workspace_bytes,
                      void *stream);

/* Merge of partial attention results over disjoint key sets: lse = logsumexp_p lse_p,
 * out = sum_p exp(lse_p - lse) out_p. The arithmetic of the serving engine's cp_lse_ag_out_rs_mha that the
 * reference calls at src/lsa/sglang/models/qwen3_5/backend.py:724-738.
 *   parts [n_parts, rows, dh] fp32 or bf16 (parts_dtype = LSA_DTYPE_F32 / LSA_DTYPE_BF16; bf16 parts - the ranks'
 *   partial reads of a prefill chunk, which cross NVLink at half the bytes - need n_parts < 16 and dh % 8 == 0),
 *   lses [n_parts, rows] fp32; out_bf16/out_f32 [rows, dh]; lse_out [rows] or NULL */
int lsa_lse_merge(const void *parts, int parts_dtype, const float *lses, int n_parts, int64_t rows, int dh,
                  uint16_t *out_bf16, float *out_f32, float *lse_out, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* LSA_B200_H */
