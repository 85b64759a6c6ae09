"""Tensor-level wrappers of the C-ABI kernels: they check shapes and dtypes, allocate outputs with torch, and
launch on the current CUDA stream. Each names the reference function it stands in for.
"""

from __future__ import annotations

from typing import NamedTuple

import torch

from lsa_b200 import _lib
from lsa_b200._lib import call, ptr, query, stream


def _contig(t: torch.Tensor) -> torch.Tensor:
    return t if t.is_contiguous() else t.contiguous()


def index_map(x: torch.Tensor, index_map_weight: torch.Tensor | None, group: int = 1, dh_off: int = 0,
              dh_used: int | None = None, normalize: bool = True, out_dtype: torch.dtype = torch.float32,
              also_bf16: bool = False, out: torch.Tensor | None = None):
    """Head sum, learned map and normalisation: x [rows, heads, dh] -> [rows, d_idx].

    Stands in for `project(regroup(...))` (src/lsa/core/index_space.py:110-131, 405-419). `x` may be a strided
    view whose last dim is contiguous.
    """
    if x.dim() != 3 or x.stride(2) != 1:
        raise ValueError(f"x must be [rows, heads, dh] with a contiguous last dim - got {tuple(x.shape)}")
    rows, heads, dh = x.shape
    dh_used = dh - dh_off if dh_used is None else dh_used
    if dh_off + dh_used > dh or heads % group:
        raise ValueError("the head dims read must lie inside the head, and the heads must group evenly")
    d_in = heads // group * dh_used
    w = None
    if index_map_weight is not None:
        w = _contig(index_map_weight)
        if w.dim() != 2 or w.shape[0] != d_in:
            raise ValueError(f"rows have {d_in} dims and the map reads {w.shape[0] if w.dim() == 2 else w.shape}")
    d_idx = w.shape[1] if w is not None else d_in
    out_f32 = None
    if out_dtype == torch.float32:
        out_f32 = out if out is not None else torch.empty(rows, d_idx, device=x.device, dtype=torch.float32)
        if out_f32.shape != (rows, d_idx) or out_f32.dtype != torch.float32 or not out_f32.is_contiguous():
            raise ValueError(f"out must be a contiguous float32 [{rows}, {d_idx}]")
    want_bf16 = also_bf16 or out_dtype == torch.bfloat16
    out_bf16 = torch.empty(rows, d_idx, device=x.device, dtype=torch.bfloat16) if want_bf16 else None
    call("lsa_index_map", ptr(x), _lib.dtype_code(x), rows, heads, group, dh_off, dh_used, x.stride(0), x.stride(1),
         ptr(w), _lib.dtype_code(w) if w is not None else 0, d_idx, int(normalize), ptr(out_f32), ptr(out_bf16),
         stream())
    if out_dtype == torch.float32:
        return (out_f32, out_bf16) if also_bf16 else out_f32
    return out_bf16


def expand_map(index_map_weight: torch.Tensor, heads: int, group: int, head_dim: int, dh_off: int = 0,
               dh_used: int | None = None) -> torch.Tensor:
    """The map as `index_map_tc` reads it: transposed, a KV head's block repeated under every query head of its
    group, zero columns for head dims the index drops. [Hkv*dh_used, d_idx] -> [d_idx, heads*head_dim] bf16."""
    dh_used = head_dim - dh_off if dh_used is None else dh_used
    kv_heads = heads // group
    w = index_map_weight.float().view(kv_heads, dh_used, -1)
    full = torch.zeros(heads, head_dim, w.shape[2], device=w.device, dtype=torch.float32)
    full[:, dh_off:dh_off + dh_used] = w.repeat_interleave(group, dim=0)
    return full.view(heads * head_dim, -1).t().contiguous().to(torch.bfloat16)


def index_map_tc(x: torch.Tensor, weight_t: torch.Tensor, normalize: bool = True, out: torch.Tensor | None = None,
                 out_bf16: torch.Tensor | None = None, status: torch.Tensor | None = None):
    """normalize(x @ weight_t^T) on the tensor cores: x [rows, ...] bf16 flattened to [rows, d_in], weight_t
    [d_idx, d_in] bf16 -> fp32 [rows, d_idx] (and/or bf16). Stands in for the serving path's bf16 map product
    (src/lsa/sglang/index/layer_index.py:331-355)."""
    if x.dtype != torch.bfloat16 or weight_t.dtype != torch.bfloat16:
        raise ValueError("the tensor-core map takes bfloat16 rows and a bfloat16 map")
    rows = x.shape[0]
    d_in = x.numel() // max(rows, 1) if rows else weight_t.shape[1]
    inner_ok = x.dim() == 2 or all(x.stride(i) == x.stride(i + 1) * x.shape[i + 1] for i in range(1, x.dim() - 1))
    if x.stride(-1) != 1 or not inner_ok or weight_t.shape[1] != d_in or not weight_t.is_contiguous():
        raise ValueError(f"rows must be contiguous past their first dim and hold {weight_t.shape[1]} dims")
    d_idx = weight_t.shape[0]
    if out is None and out_bf16 is None:
        out = torch.empty(rows, d_idx, device=x.device, dtype=torch.float32)
    call("lsa_index_map_tc", ptr(x), rows, d_in, x.stride(0), ptr(weight_t), d_idx, int(normalize), ptr(out),
         ptr(out_bf16), ptr(status), stream())
    return out if out is not None else out_bf16


def mlp_map(x: torch.Tensor, w1_t: torch.Tensor, w2_t: torch.Tensor, hidden: torch.Tensor | None = None,
            out: torch.Tensor | None = None):
    """The two-layer map (no counterpart in the reference) normalize(gelu(x @ W1) @ W2) on the tensor cores: x [rows, d_in] bf16,
    w1_t [d_hidden, d_in], w2_t [d_idx, d_hidden] bf16 -> fp32 [rows, d_idx]. The hidden layer is held in bf16."""
    rows, d_in = x.shape
    d_hidden = w1_t.shape[0]
    if hidden is None:
        hidden = torch.empty(rows, d_hidden, device=x.device, dtype=torch.bfloat16)
    call("lsa_gemm_gelu_tc", ptr(x), rows, d_in, x.stride(0), ptr(_contig(w1_t)), d_hidden, ptr(hidden), None,
         stream())
    return index_map_tc(hidden, _contig(w2_t), out=out)


def rows_linear(x: torch.Tensor, weight_t: torch.Tensor, sum_heads: bool = False, gelu: bool = False,
                normalize: bool = False, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """A linear layer over a few rows (a decode step): x [rows, d_in] or [rows, heads, d_in] bf16 (`sum_heads` adds
    the heads first), weight_t [d_out, d_in] bf16 -> [rows, d_out] fp32 (unit rows with `normalize`) or bf16. Stands
    in for the map of the decode rows (src/lsa/sglang/index/layer_index.py:906-928)."""
    if x.dtype != torch.bfloat16 or weight_t.dtype != torch.bfloat16 or x.stride(-1) != 1:
        raise ValueError("rows and map must be bfloat16 and the rows contiguous in their last dim")
    heads = x.shape[1] if (sum_heads and x.dim() == 3) else 1
    if x.dim() == 3 and not sum_heads:
        if x.stride(1) != x.shape[2]:
            raise ValueError("heads that are read side by side must be packed")
        d_in = x.shape[1] * x.shape[2]
    else:
        d_in = x.shape[-1]
    w = _contig(weight_t)
    if w.shape[1] != d_in:
        raise ValueError(f"the rows have {d_in} dims and the map reads {w.shape[1]}")
    rows, d_out = x.shape[0], w.shape[0]
    out_f32 = torch.empty(rows, d_out, device=x.device, dtype=torch.float32) \
        if (out_dtype == torch.float32 or normalize) else None
    out_bf16 = torch.empty(rows, d_out, device=x.device, dtype=torch.bfloat16) if out_dtype == torch.bfloat16 else None
    call("lsa_rows_linear", ptr(x), rows, heads, x.stride(0), x.stride(1) if heads > 1 else 0, d_in, ptr(w), d_out,
         (1 if gelu else 0) | (2 if normalize else 0), ptr(out_f32), ptr(out_bf16), stream(),
         launches=2 if normalize else 1)
    return out_f32 if out_dtype == torch.float32 else out_bf16


def pool_keys(index_keys: torch.Tensor, pool_size: int, out: torch.Tensor | None = None) -> torch.Tensor:
    """`pool_keys` (src/lsa/core/ward.py:15-26): [..., T, d] -> [..., T / pool_size, d] fp32."""
    keys = _contig(index_keys)
    T, d = keys.shape[-2], keys.shape[-1]
    if T % pool_size:
        raise ValueError(f"{T} keys do not split into pools of {pool_size}")
    if out is None:
        out = torch.empty(*keys.shape[:-2], T // pool_size, d, device=keys.device, dtype=torch.float32)
    call("lsa_pool_keys", ptr(keys), _lib.dtype_code(keys), out.numel() // d, pool_size, d, ptr(out), stream())
    return out


def ward_rounds(pools: torch.Tensor, pool_sizes: torch.Tensor | float, bucket_count: int, bucket_cap: float,
                max_rounds: int = 256, return_rounds: bool = False, labels: torch.Tensor | None = None,
                reached: torch.Tensor | None = None, workspace: torch.Tensor | None = None):
    """`ward_rounds` (src/lsa/core/ward.py:29-90): labels [G, P] int64 and whether each block reached its count."""
    pools = _contig(pools)
    if pools.dim() != 3 or pools.dtype != torch.float32:
        raise ValueError(f"pool keys must be [G, P, index_dim] float32 - got {tuple(pools.shape)} {pools.dtype}")
    G, P, d = pools.shape
    sizes, uniform = None, 0.0
    if isinstance(pool_sizes, torch.Tensor):
        sizes = _contig(pool_sizes.to(torch.float32))
        if sizes.shape != (G, P):
            raise ValueError(f"pool sizes must be [{G}, {P}] - got {tuple(sizes.shape)}")
    else:
        uniform = float(pool_sizes)
    labels = torch.empty(G, P, device=pools.device, dtype=torch.int64) if labels is None else labels
    raw_reached = torch.empty(G, device=pools.device, dtype=torch.uint8) if reached is None else reached
    rounds = torch.empty(G, device=pools.device, dtype=torch.int32) if return_rounds else None
    need = query("lsa_ward_merge_workspace_bytes", G, P, d)
    if need and (workspace is None or workspace.numel() * workspace.element_size() < need):
        workspace = torch.empty(need, device=pools.device, dtype=torch.uint8)
    call("lsa_ward_merge", ptr(pools), ptr(sizes), uniform, G, P, d, bucket_count, float(bucket_cap), max_rounds,
         ptr(labels), ptr(raw_reached), ptr(rounds), ptr(workspace) if need else None, need, stream(),
         launches=1 if not need else 2 + 2 * max_rounds)
    if reached is not None:
        return labels, raw_reached
    if return_rounds:
        return labels, raw_reached.bool(), rounds
    return labels, raw_reached.bool()


def bucket_table(index_keys: torch.Tensor, labels: torch.Tensor, pool_size: int, bucket_count: int,
                 bucket_cap: int, first_position: int = 0, want_bf16: bool = False, outs: tuple | None = None):
    """Members, sizes, key sums and centroids of every block (src/lsa/core/reference.py:120-144)."""
    keys, labels = _contig(index_keys), _contig(labels)
    G, P = labels.shape
    d = keys.shape[-1]
    rows = G * bucket_count
    if outs is not None:
        members, sizes, key_sums, centroids, centroids_bf16, status = outs
    else:
        members = torch.empty(rows, bucket_cap, device=keys.device, dtype=torch.int32)
        sizes = torch.empty(rows, device=keys.device, dtype=torch.int32)
        key_sums = torch.empty(rows, d, device=keys.device, dtype=torch.float32)
        centroids = torch.empty(rows, d, device=keys.device, dtype=torch.float32)
        centroids_bf16 = torch.empty(rows, d, device=keys.device, dtype=torch.bfloat16) if want_bf16 else None
        status = torch.zeros(1, device=keys.device, dtype=torch.int32)
    call("lsa_bucket_table", ptr(keys), _lib.dtype_code(keys), ptr(labels), G, P, pool_size, d, bucket_count,
         bucket_cap, first_position, ptr(members), ptr(sizes), ptr(key_sums), ptr(centroids), ptr(centroids_bf16),
         ptr(status), stream())
    return members, sizes, key_sums, centroids, centroids_bf16, status


def bucket_members(labels: torch.Tensor, pool_size: int, bucket_count: int, bucket_cap: int,
                   first_position: int = 0):
    """The member table alone (src/lsa/core/ward.py:128-143): (members [G*bucket_count, cap], sizes)."""
    labels = _contig(labels)
    G, P = labels.shape
    members = torch.empty(G * bucket_count, bucket_cap, device=labels.device, dtype=torch.int32)
    sizes = torch.empty(G * bucket_count, device=labels.device, dtype=torch.int32)
    call("lsa_bucket_table", None, 0, ptr(labels), G, P, pool_size, 1, bucket_count, bucket_cap, first_position,
         ptr(members), ptr(sizes), None, None, None, None, stream())
    return members, sizes


def gather_sum(src: torch.Tensor, index: torch.Tensor, index_base: int = 0) -> torch.Tensor:
    """out[r] = the rows src[index[r, c] - index_base] added one by one in column order (an index < 0 ends the row).
    The key sums under buckets and node buckets (src/lsa/core/hierarchy.py:134-136, 157)."""
    src, index = _contig(src), _contig(index)
    if index.dtype not in (torch.int32, torch.int64) or index.dim() != 2:
        raise ValueError("index must be an int32 or int64 matrix")
    out = torch.empty(index.shape[0], src.shape[-1], device=src.device, dtype=torch.float32)
    call("lsa_gather_sum", ptr(src), _lib.dtype_code(src), ptr(index), int(index.dtype == torch.int64),
         index.shape[0], index.shape[1], src.shape[-1], index_base, ptr(out), stream())
    return out


def kmeans(pools: torch.Tensor, init_centroids: torch.Tensor, iters: int):
    """k-means bucketing (no counterpart in the reference): `iters` Lloyd iterations over pool keys
    [n, d] from `init_centroids` [k, d]; returns (centroids [k, d] fp32, assignment [n] int32). Assignment is the
    exact fixed-order argmax of pool . centroid (a tie to the lower cluster)."""
    pools = _contig(pools.float())
    centroids = _contig(init_centroids.float()).clone()
    n, d = pools.shape
    k = centroids.shape[0]
    every = torch.full((n,), k, device=pools.device, dtype=torch.int32)
    assign = None
    for it in range(iters + 1):
        _, picked = flat_select(pools, centroids, every, 1)
        assign = picked[:, 0]
        if it == iters:
            break
        order = torch.argsort(assign, stable=True)
        offsets = torch.zeros(k + 1, device=pools.device, dtype=torch.int64)
        offsets[1:] = torch.cumsum(torch.bincount(assign, minlength=k), 0)
        call("lsa_kmeans_update", ptr(pools), ptr(order), ptr(offsets), k, d, ptr(centroids), stream())
    return centroids, assign


def flat_select(index_queries: torch.Tensor, centroids: torch.Tensor, visible: torch.Tensor, top_p: int,
                row_top_p: torch.Tensor | None = None, bucket_id_base: int = 0, keys: torch.Tensor | None = None,
                picked: torch.Tensor | None = None):
    """Top-p packed keys and bucket ids of every row (src/lsa/core/reference.py:228-265)."""
    q, c = _contig(index_queries.float()), _contig(centroids.float())
    R, d = q.shape
    keys = torch.empty(R, top_p, device=q.device, dtype=torch.int64) if keys is None else keys
    picked = torch.empty(R, top_p, device=q.device, dtype=torch.int32) if picked is None else picked
    call("lsa_flat_select", ptr(q), R, d, ptr(c), c.shape[0], ptr(_contig(visible.to(torch.int32))),
         ptr(row_top_p), top_p, bucket_id_base, ptr(keys), ptr(picked), stream())
    return keys, picked


def dense_scores(index_queries: torch.Tensor, centroids: torch.Tensor, counts: torch.Tensor, width: int | None = None,
                 pages: torch.Tensor | None = None, page_rows: int = 1, bucket_id_base: int = 0, keys: bool = False):
    """Every (row, bucket) score at its own column [R, width] fp32 (-inf past a row's count), or with `keys` the
    packed keys [R, width] int64 (src/lsa/core/kernels/scan_select.py:24-58, triton/paged.py:61-101); through
    `pages` [R, max_pages] where a cache holds its buckets in pages of `page_rows`."""
    q, c = _contig(index_queries.float()), _contig(centroids.float())
    R, d = q.shape
    width = c.shape[0] if width is None else width
    out = torch.empty(R, width, device=q.device, dtype=torch.int64 if keys else torch.float32)
    pages = None if pages is None else _contig(pages.to(torch.int32))
    call("lsa_dense_scores", ptr(q), R, d, ptr(c), ptr(pages), pages.shape[1] if pages is not None else 0, page_rows,
         ptr(_contig(counts.to(torch.int32))), width, bucket_id_base, None if keys else ptr(out),
         ptr(out) if keys else None, stream())
    return out


def scan_centre(centroids: torch.Tensor, centre: torch.Tensor | None = None, out: torch.Tensor | None = None,
                lengths: torch.Tensor | None = None, radius: torch.Tensor | None = None):
    """The tensor-core scan's N operand: `centroids` [rows, 64] fp32 less `centre` [64] (None: no centre), rounded to
    bf16 into `out`; the length of every row into `lengths` [rows] fp32, and `radius` [1] fp32 raised to the greatest
    of them (start it at zero; a run of rows at a time as an index grows). Returns (out, lengths, radius)."""
    c = _contig(centroids.float())
    out = torch.empty(c.shape, device=c.device, dtype=torch.bfloat16) if out is None else out
    lengths = torch.empty(c.shape[0], device=c.device, dtype=torch.float32) if lengths is None else lengths
    radius = torch.zeros(1, device=c.device, dtype=torch.float32) if radius is None else radius
    if out.shape != c.shape or out.dtype != torch.bfloat16 or not out.is_contiguous():
        raise ValueError(f"out must be a contiguous bfloat16 {tuple(c.shape)}")
    if lengths.shape != (c.shape[0],) or lengths.dtype != torch.float32 or not lengths.is_contiguous():
        raise ValueError(f"lengths must be a contiguous float32 [{c.shape[0]}]")
    call("lsa_scan_centre", ptr(c), c.shape[0], c.shape[1], ptr(None if centre is None else _contig(centre.float())),
         ptr(out), ptr(lengths), ptr(radius), stream())
    return out, lengths, radius


def scan_select(index_queries: torch.Tensor, centroids: torch.Tensor, centroids_bf16: torch.Tensor,
                visible: torch.Tensor, top_p: int, row_top_p: torch.Tensor | None = None, bucket_id_base: int = 0,
                max_visible: int = 0, keys: torch.Tensor | None = None, picked: torch.Tensor | None = None,
                status: torch.Tensor | None = None, workspace: torch.Tensor | None = None,
                lengths: torch.Tensor | None = None, radius: torch.Tensor | None = None):
    """`flat_select`'s result with the scan on tcgen05: bf16 scores in tensor memory against a sampled threshold,
    an exact fp32 rescoring of the survivors, and an exact scan of whatever row the survivors cannot prove
    (src/lsa/core/kernels/cutedsl/blackwell/bucket_scan.py:63-836, src/lsa/core/kernels/scan_select.py:189-385).
    `centroids_bf16`, `lengths` and `radius` come from `scan_centre` (without them: the plain bf16 rounding of
    centroids no longer than 1). `max_visible` is the host's bound on `visible` (0: all of the centroids)."""
    q, c, cb = _contig(index_queries.float()), _contig(centroids.float()), _contig(centroids_bf16)
    R, d = q.shape
    if cb.dtype != torch.bfloat16 or cb.shape != c.shape:
        raise ValueError("centroids_bf16 must be a bfloat16 matrix of the centroids' shape")
    keys = torch.empty(R, top_p, device=q.device, dtype=torch.int64) if keys is None else keys
    picked = torch.empty(R, top_p, device=q.device, dtype=torch.int32) if picked is None else picked
    need = query("lsa_scan_select_workspace_bytes", R, top_p, c.shape[0])
    if workspace is None or workspace.numel() * workspace.element_size() < need:
        workspace = torch.empty(max(need, 1), device=q.device, dtype=torch.uint8)
    call("lsa_scan_select", ptr(q), R, d, ptr(c), ptr(cb), ptr(lengths), ptr(radius), c.shape[0],
         ptr(_contig(visible.to(torch.int32))), ptr(row_top_p), top_p, bucket_id_base, int(max_visible), ptr(keys),
         ptr(picked), ptr(status), ptr(workspace), workspace.numel() * workspace.element_size(), stream(),
         launches=8 if _scan_samples(c.shape[0], top_p, int(max_visible)) else 1)
    return keys, picked


def _scan_samples(m: int, top_p: int, max_visible: int) -> bool:
    """Whether `lsa_scan_select` thresholds its rows by sampling (eight launches: operands, scan, pick, the rows left
    over collected, scanned in splits, merged and scattered, the exact scan of the rest) or scans all of them exactly
    (one launch): the gate of csrc/select.cu, restated for the launch count."""
    widest = max_visible if 0 < max_visible < m else m
    factor = max(2, min(3, 1024 // max(top_p, 1)))
    return m >= 1024 and factor * top_p * 512 >= 8 * widest


def flat_select_decode(index_queries: torch.Tensor, centroids: torch.Tensor, request_first: torch.Tensor | None,
                       visible: torch.Tensor, top_p: int, splits: int = 1, workspace: torch.Tensor | None = None):
    """Decode-form flat scan (src/lsa/sglang/index/selector.py:603-660): few rows, their buckets split over CTAs."""
    q, c = _contig(index_queries.float()), _contig(centroids.float())
    R, d = q.shape
    keys = torch.empty(R, top_p, device=q.device, dtype=torch.int64)
    picked = torch.empty(R, top_p, device=q.device, dtype=torch.int32)
    need = query("lsa_flat_select_decode_workspace_bytes", R, top_p, splits)
    if need and (workspace is None or workspace.numel() * workspace.element_size() < need):
        workspace = torch.empty(need, device=q.device, dtype=torch.uint8)
    call("lsa_flat_select_decode", ptr(q), R, d, ptr(c), ptr(request_first), ptr(_contig(visible.to(torch.int32))),
         top_p, splits, ptr(keys), ptr(picked), ptr(workspace),
         workspace.numel() * workspace.element_size() if workspace is not None else 0, stream(),
         launches=1 if splits == 1 else 2)
    return keys, picked


def flat_select_paged(index_queries: torch.Tensor, centroids: torch.Tensor, pages: torch.Tensor,
                      counts: torch.Tensor, page_rows: int, top_p: int, splits: int = 1,
                      workspace: torch.Tensor | None = None):
    """The decode scan through each request's page table (src/lsa/core/kernels/triton/paged.py:61-101): logical
    bucket i of request r is row i % page_rows of page pages[r, i // page_rows]. Returns (keys, logical ids)."""
    q, c = _contig(index_queries.float()), _contig(centroids.float())
    pages = _contig(pages.to(torch.int32))
    R, d = q.shape
    keys = torch.empty(R, top_p, device=q.device, dtype=torch.int64)
    picked = torch.empty(R, top_p, device=q.device, dtype=torch.int32)
    need = query("lsa_flat_select_decode_workspace_bytes", R, top_p, splits)
    if need and (workspace is None or workspace.numel() * workspace.element_size() < need):
        workspace = torch.empty(need, device=q.device, dtype=torch.uint8)
    call("lsa_flat_select_paged", ptr(q), R, d, ptr(c), c.shape[0], ptr(pages), pages.shape[1], page_rows,
         ptr(_contig(counts.to(torch.int32))), top_p, splits, ptr(keys), ptr(picked), ptr(workspace),
         workspace.numel() * workspace.element_size() if workspace is not None else 0, stream(),
         launches=1 if splits == 1 else 2)
    return keys, picked


class ShapeTable(NamedTuple):
    """The shapes of a table of buckets, row for row with their centroids, and the deviations they score with
    (src/lsa/core/kernels/triton/shape.py:42-61)."""

    basis: torch.Tensor  # [m, rank, d / 8] uint8: one sign bit a dimension, bit b of byte i = dimension 8 i + b
    variances: torch.Tensor  # [m, rank] fp32, descending
    floor: torch.Tensor  # [m] fp32
    deviations: float  # z

    def rows(self, rows) -> "ShapeTable":
        """The shapes of some rows (an index tensor or a slice), aligned with them."""
        return ShapeTable(self.basis[rows], self.variances[rows], self.floor[rows], self.deviations)

    @property
    def rank(self) -> int:
        return self.basis.shape[1]


def _shape_args(shapes: ShapeTable, d: int):
    basis, variances, floor = _contig(shapes.basis), _contig(shapes.variances.float()), _contig(shapes.floor.float())
    if basis.dtype != torch.uint8 or basis.dim() != 3 or basis.shape[2] * 8 != d:
        raise ValueError(f"a shape basis is [buckets, rank, {d // 8}] uint8 - got {tuple(basis.shape)} {basis.dtype}")
    if variances.shape != basis.shape[:2] or floor.shape != basis.shape[:1]:
        raise ValueError("a shape's variances are [buckets, rank] and its floor [buckets]")
    return basis, variances, floor


def shape_build(index_keys: torch.Tensor, centroids: torch.Tensor, members: torch.Tensor, rank: int,
                key_base: int = 0, out: ShapeTable | None = None, deviations: float = 0.0) -> ShapeTable:
    """The shapes of buckets from the keys they hold (src/lsa/core/shape.py:88-106; the served builder
    src/lsa/core/kernels/triton/shape.py:849-886): each bucket's covariance about its centroid, diagonalised exactly,
    kept as `rank` packed sign directions, their variances and a floor. `index_keys` [rows, d] fp32 holds the keys at
    positions key_base.. ; `members` [m, cap] are positions, -1 padded. `out`: a table's rows to write into."""
    keys, c, mem = _contig(index_keys.float()), _contig(centroids.float()), _contig(members.to(torch.int32))
    m, d = c.shape
    if out is None:
        out = ShapeTable(torch.empty(m, rank, d // 8, device=c.device, dtype=torch.uint8),
                         torch.empty(m, rank, device=c.device), torch.empty(m, device=c.device), deviations)
    basis, variances, floor = out.basis, out.variances, out.floor
    if not (basis.is_contiguous() and variances.is_contiguous() and floor.is_contiguous()):
        raise ValueError("shapes are written into contiguous rows")
    if basis.shape != (m, rank, d // 8) or variances.shape != (m, rank) or floor.shape != (m,):
        raise ValueError(f"out holds {tuple(basis.shape)} - expected the shapes of {m} buckets of rank {rank}")
    call("lsa_shape_build", ptr(keys), key_base, keys.shape[0], ptr(c), ptr(mem), m, mem.shape[1], d, rank, ptr(basis),
         ptr(variances), ptr(floor), stream())
    return out


def shaped_select(index_queries: torch.Tensor, centroids: torch.Tensor, shapes: ShapeTable, visible: torch.Tensor,
                  top_p: int, row_top_p: torch.Tensor | None = None, bucket_id_base: int = 0,
                  keys: torch.Tensor | None = None, picked: torch.Tensor | None = None):
    """`flat_select` over shaped buckets: a bucket scores as its estimated best key
    (src/lsa/core/reference.py:229-230, src/lsa/core/shape.py:123-137)."""
    q, c = _contig(index_queries.float()), _contig(centroids.float())
    R, d = q.shape
    basis, variances, floor = _shape_args(shapes, d)
    keys = torch.empty(R, top_p, device=q.device, dtype=torch.int64) if keys is None else keys
    picked = torch.empty(R, top_p, device=q.device, dtype=torch.int32) if picked is None else picked
    call("lsa_shaped_select", ptr(q), R, d, ptr(c), c.shape[0], ptr(basis), ptr(variances), ptr(floor),
         basis.shape[1], float(shapes.deviations), ptr(_contig(visible.to(torch.int32))), ptr(row_top_p), top_p,
         bucket_id_base, ptr(keys), ptr(picked), stream())
    return keys, picked


def shaped_select_decode(index_queries: torch.Tensor, centroids: torch.Tensor, shapes: ShapeTable,
                         request_first: torch.Tensor | None, visible: torch.Tensor, top_p: int, splits: int = 1,
                         workspace: torch.Tensor | None = None):
    """`flat_select_decode` over shaped buckets (src/lsa/core/kernels/triton/shape.py:659-717)."""
    q, c = _contig(index_queries.float()), _contig(centroids.float())
    R, d = q.shape
    basis, variances, floor = _shape_args(shapes, d)
    keys = torch.empty(R, top_p, device=q.device, dtype=torch.int64)
    picked = torch.empty(R, top_p, device=q.device, dtype=torch.int32)
    need = query("lsa_flat_select_decode_workspace_bytes", R, top_p, splits)
    if need and (workspace is None or workspace.numel() * workspace.element_size() < need):
        workspace = torch.empty(need, device=q.device, dtype=torch.uint8)
    call("lsa_shaped_select_decode", ptr(q), R, d, ptr(c), ptr(basis), ptr(variances), ptr(floor), basis.shape[1],
         float(shapes.deviations), ptr(request_first), ptr(_contig(visible.to(torch.int32))), top_p, splits, ptr(keys),
         ptr(picked), ptr(workspace), workspace.numel() * workspace.element_size() if workspace is not None else 0,
         stream(), launches=1 if splits == 1 else 2)
    return keys, picked


def shaped_select_paged(index_queries: torch.Tensor, centroids: torch.Tensor, shapes: ShapeTable, pages: torch.Tensor,
                        counts: torch.Tensor, page_rows: int, top_p: int, splits: int = 1,
                        workspace: torch.Tensor | None = None):
    """`flat_select_paged` over shaped buckets, the shapes paged as the centroids are
    (src/lsa/core/kernels/triton/shape.py:573-717). Returns (keys, logical ids)."""
    q, c = _contig(index_queries.float()), _contig(centroids.float())
    pages = _contig(pages.to(torch.int32))
    R, d = q.shape
    basis, variances, floor = _shape_args(shapes, d)
    keys = torch.empty(R, top_p, device=q.device, dtype=torch.int64)
    picked = torch.empty(R, top_p, device=q.device, dtype=torch.int32)
    need = query("lsa_flat_select_decode_workspace_bytes", R, top_p, splits)
    if need and (workspace is None or workspace.numel() * workspace.element_size() < need):
        workspace = torch.empty(need, device=q.device, dtype=torch.uint8)
    call("lsa_shaped_select_paged", ptr(q), R, d, ptr(c), c.shape[0], ptr(basis), ptr(variances), ptr(floor),
         basis.shape[1], float(shapes.deviations), ptr(pages), pages.shape[1], page_rows,
         ptr(_contig(counts.to(torch.int32))), top_p, splits, ptr(keys), ptr(picked), ptr(workspace),
         workspace.numel() * workspace.element_size() if workspace is not None else 0, stream(),
         launches=1 if splits == 1 else 2)
    return keys, picked


def shaped_scores(index_queries: torch.Tensor, centroids: torch.Tensor, shapes: ShapeTable,
                  rows: torch.Tensor | None = None, width: int | None = None) -> torch.Tensor:
    """Shaped scores written out [R, width] fp32: row r against the table rows `rows[r]` (-1: -inf), or against the
    first `width` table rows (src/lsa/core/kernels/triton/shape.py:281-343,407-450)."""
    q, c = _contig(index_queries.float()), _contig(centroids.float())
    R, d = q.shape
    basis, variances, floor = _shape_args(shapes, d)
    rows = None if rows is None else _contig(rows.to(torch.int32))
    width = (c.shape[0] if width is None else width) if rows is None else rows.shape[1]
    out = torch.empty(R, width, device=q.device, dtype=torch.float32)
    call("lsa_shaped_scores", ptr(q), R, d, ptr(c), c.shape[0], ptr(basis), ptr(variances), ptr(floor), basis.shape[1],
         float(shapes.deviations), ptr(rows), width, ptr(out), stream())
    return out


def page_fingerprints(stored: torch.Tensor, page_rows: int, word_weights: torch.Tensor,
                      position_weights: torch.Tensor, slots: torch.Tensor | None = None,
                      owned: torch.Tensor | None = None) -> torch.Tensor:
    """A fingerprint of each page of the bits a pool stores for a run of whole pages [pages] int64
    (src/lsa/sglang/index/layer_index.py:106-122): `stored` [rows, dim] with contiguous rows of a multiple of 8 bytes
    (any stride between rows), read at `slots` [pages * page_rows] int64 (None: rows 0.. in order); `owned`
    [pages * page_rows] bool marks the slots this rank owns (the others add nothing)."""
    if stored.dim() != 2 or stored.stride(1) != 1:
        raise ValueError("stored rows must be contiguous [rows, dim]")
    size = stored.element_size()
    count = stored.shape[0] if slots is None else slots.shape[0]
    if count % page_rows:
        raise ValueError(f"{count} rows are not whole pages of {page_rows}")
    if position_weights.shape[0] != page_rows or word_weights.shape[0] * 8 < stored.shape[1] * size:
        raise ValueError("the weights cover a page's positions and a row's words")
    slots = None if slots is None else _contig(slots.to(torch.int64))
    owned = None if owned is None else _contig(owned.to(torch.uint8))
    out = torch.empty(count // page_rows, device=stored.device, dtype=torch.int64)
    call("lsa_page_fingerprints", ptr(stored), stored.stride(0) * size, stored.shape[1] * size, ptr(slots),
         stored.shape[0], count // page_rows, page_rows, ptr(owned), ptr(_contig(word_weights)),
         ptr(_contig(position_weights)), ptr(out), stream())
    return out


def merge_candidates(keys_in: torch.Tensor):
    """Global top-p of [parts, R, top_p] packed keys: (keys [R, top_p], ids [R, top_p])."""
    keys_in = _contig(keys_in)
    parts, R, top_p = keys_in.shape
    keys = torch.empty(R, top_p, device=keys_in.device, dtype=torch.int64)
    picked = torch.empty(R, top_p, device=keys_in.device, dtype=torch.int32)
    call("lsa_merge_candidates", ptr(keys_in), parts, R, top_p, ptr(keys), ptr(picked), stream())
    return keys, picked


def beam_step(index_queries: torch.Tensor, vectors: torch.Tensor, carried: torch.Tensor | None,
              open_first: torch.Tensor, open_end: torch.Tensor, keep: int, children: torch.Tensor | None = None,
              splits: int = 1, workspace: torch.Tensor | None = None):
    """One level of the beam (src/lsa/core/hierarchy.py:402-451): kept rows, or their children when given."""
    q, v = _contig(index_queries.float()), _contig(vectors.float())
    R, d = q.shape
    n_carried = 0 if carried is None else carried.shape[1]
    carried = None if carried is None else _contig(carried.to(torch.int32))
    kept = keys = carried_out = None
    fanout = 0
    if children is not None:
        children = _contig(children)
        fanout = children.shape[1]
        carried_out = torch.empty(R, keep * fanout, device=q.device, dtype=torch.int32)
    else:
        kept = torch.empty(R, keep, device=q.device, dtype=torch.int32)
        keys = torch.empty(R, keep, device=q.device, dtype=torch.int64)
    need = query("lsa_beam_step_workspace_bytes", R, keep, splits)
    if need and (workspace is None or workspace.numel() * workspace.element_size() < need):
        workspace = torch.empty(need, device=q.device, dtype=torch.uint8)
    call("lsa_beam_step_split", ptr(q), R, d, ptr(v), v.shape[0], ptr(carried), n_carried,
         ptr(_contig(open_first.to(torch.int32))), ptr(_contig(open_end.to(torch.int32))), keep, ptr(children),
         fanout, splits, ptr(kept), ptr(keys), ptr(carried_out), ptr(workspace) if need else None, need, stream(),
         launches=1 if splits <= 1 else 2)
    return carried_out if children is not None else (kept, keys)


def expand(picked: torch.Tensor, positions: torch.Tensor, members: torch.Tensor, top_k: int, sink: int, window: int,
           row_top_p: torch.Tensor | None = None, row_top_k: torch.Tensor | None = None,
           page_table: torch.Tensor | None = None, page_size: int = 0, owner: tuple[int, int] | None = None,
           outs: tuple | None = None, dealt: tuple[int, int, int] | None = None, local: bool = True,
           pad: bool = True):
    """`expand_buckets` for every row (src/lsa/core/reference.py:268-289): (lists, lengths, status). With `pad` off
    the entries past a row's length are left as they were (a reader that goes by the lengths saves their write)."""
    picked, members = _contig(picked), _contig(members)
    R, top_p = picked.shape
    width = top_k + window + sink
    if outs is not None:
        selected, lengths, status = outs
    else:
        selected = torch.empty(R, width, device=picked.device, dtype=torch.int32)
        lengths = torch.empty(R, device=picked.device, dtype=torch.int32)
        status = torch.zeros(1, device=picked.device, dtype=torch.int32)
    first, end = owner if owner is not None else (0, _lib.INT64_MAX)
    # dealt = (granule, world, rank): keep the ids of this rank's granules, stored as rows of its own cache
    granule, world, rank = dealt if dealt is not None else (1, 1, 0)
    call("lsa_expand", ptr(picked), R, top_p, ptr(_contig(positions.to(torch.int64))), ptr(members),
         members.shape[0], members.shape[1], ptr(row_top_p), ptr(row_top_k), top_k, sink, window, ptr(page_table),
         page_size, first, end, granule, world, rank, (0 if local else 1) | (0 if pad else 2), ptr(selected), ptr(lengths),
         ptr(status), stream())
    return selected, lengths, status


def expand_batched(picked: torch.Tensor, positions: torch.Tensor, row_request: torch.Tensor | None,
                   members: torch.Tensor,
                   bucket_pages: torch.Tensor | None, bucket_page_rows: int, kv_pages: torch.Tensor | None,
                   kv_page_size: int, top_k: int, sink: int, window: int, local: bool = True):
    """Expansion for a batch of requests over one paged cache (src/lsa/core/kernels/expansion.py:16-58): row r is a
    query of request row_request[r] (None: request 0) at its own position; picks are the request's logical bucket ids, read through
    `bucket_pages` [requests, pages]; ids are written as KV slots through `kv_pages` [requests, pages]."""
    picked, members = _contig(picked), _contig(members)
    R, top_p = picked.shape
    selected = torch.empty(R, top_k + window + sink, device=picked.device, dtype=torch.int32)
    lengths = torch.empty(R, device=picked.device, dtype=torch.int32)
    status = torch.zeros(1, device=picked.device, dtype=torch.int32)
    bucket_pages = None if bucket_pages is None else _contig(bucket_pages.to(torch.int32))
    kv_pages = None if kv_pages is None else _contig(kv_pages.to(torch.int32))
    call("lsa_expand_batched", ptr(picked), R, top_p, ptr(_contig(positions.to(torch.int64))), ptr(members),
         members.shape[0], members.shape[1], None, None, top_k, sink, window, ptr(kv_pages), kv_page_size, 0,
         _lib.INT64_MAX, 1, 1, 0, 0 if local else 1,
         ptr(None if row_request is None else _contig(row_request.to(torch.int32))),
         kv_pages.shape[1] if kv_pages is not None else 0, ptr(bucket_pages),
         bucket_pages.shape[1] if bucket_pages is not None else 0,
         bucket_pages.shape[1] if bucket_pages is not None else 0, bucket_page_rows, ptr(selected), ptr(lengths),
         ptr(status), stream())
    return selected, lengths, status


def sparse_attend(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, ids: torch.Tensor,
                  lengths: torch.Tensor | None, scale: float, splits: int = 1, out_dtype=torch.bfloat16,
                  workspace: torch.Tensor | None = None, out: torch.Tensor | None = None,
                  lse: torch.Tensor | None = None, first_slot: int = 0, init: tuple | None = None):
    """Attention of q [R, Hq, dh] over the KV rows each list names; returns (out [R, Hq, dh], lse [R, Hq]).
    `k`, `v` hold the KV rows from `first_slot` on (a rank's share of a sharded cache); other ids are skipped."""
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16:
        raise ValueError("q, k and v must be bfloat16")
    if q.stride(2) != 1 or k.stride(2) != 1 or v.stride(2) != 1 or k.stride() != v.stride():
        raise ValueError("head dims must be contiguous and k, v must share their layout")
    ids = _contig(ids)
    R, Hq, dh = q.shape
    slots, Hkv, _ = k.shape
    if out is not None:
        if out.shape != (R, Hq, dh) or not out.is_contiguous() or out.dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"out must be a contiguous bfloat16 or float32 [{R}, {Hq}, {dh}]")
        out_dtype = out.dtype
    else:
        out = torch.empty(R, Hq, dh, device=q.device, dtype=out_dtype)
    out_bf16 = out if out_dtype == torch.bfloat16 else None
    out_f32 = out if out_dtype == torch.float32 else None
    lse = torch.empty(R, Hq, device=q.device, dtype=torch.float32) if lse is None else lse
    need = query("lsa_sparse_attend_workspace_bytes", R, Hq, dh, splits)
    if need and (workspace is None or workspace.numel() * workspace.element_size() < need):
        workspace = torch.empty(need, device=q.device, dtype=torch.uint8)
    call("lsa_sparse_attend", ptr(q), R, Hq, dh, q.stride(0), q.stride(1), ptr(k), ptr(v), slots, first_slot, Hkv,
         k.stride(0),
         k.stride(1), ptr(ids), ids.shape[1], ptr(lengths), ptr(init[0]) if init else None,
         ptr(init[1]) if init else None, float(scale), splits, ptr(out_bf16), ptr(out_f32),
         ptr(lse), ptr(workspace), workspace.numel() * workspace.element_size() if workspace is not None else 0,
         stream(), launches=1 if splits == 1 else 2)
    return (out_bf16 if out_bf16 is not None else out_f32), lse


def latent_attend(q: torch.Tensor, latent: torch.Tensor, ids: torch.Tensor, lengths: torch.Tensor | None,
                  scale: float, value_dim: int = 512, splits: int = 1, out_dtype=torch.bfloat16,
                  workspace: torch.Tensor | None = None, warp_mma: bool = False,
                  status: torch.Tensor | None = None, out: torch.Tensor | None = None,
                  dealt: tuple[int, int, int] | None = None):
    """The MLA read: absorbed queries q [R, Hq, dk] bf16 over the latent rows [slots, dk] bf16 each list names, a
    value being a row's first `value_dim` dims. Returns (out [R, Hq, value_dim], lse [R, Hq]). The products run
    on tcgen05 with tensor-memory accumulators; `warp_mma` takes the warp-level MMA kernel. With `dealt` =
    (granule, world, rank) the lists hold POSITIONS and `latent` is this rank's share of a cache dealt out in
    granules: the call reads the positions its rank holds and skips the rest."""
    if q.dtype != torch.bfloat16 or latent.dtype != torch.bfloat16:
        raise ValueError("q and latent must be bfloat16")
    if q.dim() != 3 or latent.dim() != 2 or q.stride(2) != 1 or latent.stride(1) != 1 or q.shape[2] != latent.shape[1]:
        raise ValueError(f"q must be [R, Hq, dk] and latent [slots, dk] - got {tuple(q.shape)} and {tuple(latent.shape)}")
    ids = _contig(ids)
    R, Hq, dk = q.shape
    if out is None:
        out = torch.empty(R, Hq, value_dim, device=q.device, dtype=out_dtype)
    elif out.shape != (R, Hq, value_dim) or not out.is_contiguous() or out.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError(f"out must be a contiguous bfloat16 or float32 [{R}, {Hq}, {value_dim}]")
    out_dtype = out.dtype
    lse = torch.empty(R, Hq, device=q.device, dtype=torch.float32)
    need = query("lsa_latent_attend_workspace_bytes", R, Hq, value_dim, splits)
    if need and (workspace is None or workspace.numel() * workspace.element_size() < need):
        workspace = torch.empty(need, device=q.device, dtype=torch.uint8)
    call("lsa_latent_attend", ptr(q), R, Hq, dk, value_dim, q.stride(0), q.stride(1), ptr(latent), latent.shape[0],
         latent.stride(0), ptr(ids), ids.shape[1], ptr(lengths), float(scale), splits,
         ptr(out) if out_dtype == torch.bfloat16 else None, ptr(out) if out_dtype == torch.float32 else None, ptr(lse),
         1 if warp_mma else 0, *(dealt if dealt is not None else (0, 1, 0)), ptr(status), ptr(workspace),
         workspace.numel() * workspace.element_size() if workspace is not None else 0, stream(),
         launches=1 if splits == 1 else 2)
    return out, lse


def bucket_attend_supported(q: torch.Tensor, k: torch.Tensor, bucket_cap: int) -> bool:
    """Whether `bucket_attend` takes these shapes (else: `expand` + `sparse_attend`)."""
    return q.shape[2] == 128 and bucket_cap <= 64 and q.shape[1] % k.shape[1] == 0 and q.shape[1] // k.shape[1] <= 8


def bucket_attend(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, picked: torch.Tensor, positions: torch.Tensor,
                  members: torch.Tensor, top_k: int, sink: int, window: int, scale: float, init: tuple | None = None,
                  row_top_p: torch.Tensor | None = None, row_top_k: torch.Tensor | None = None,
                  out: torch.Tensor | None = None, lse: torch.Tensor | None = None,
                  workspace: torch.Tensor | None = None, warp_mma: bool = False,
                  init_ready: torch.cuda.Event | None = None, status: torch.Tensor | None = None):
    """Expansion and attention of a prefill chunk bucket by bucket: q [R, Hq, dh] bf16 over the members of each row's
    picked buckets (picked [R, top_p], members ascending in a bucket) inside [sink, position + 1 - window), cut at
    top_k, merged with the partial read `init` = (out fp32, lse). Returns (out [R, Hq, dh] bf16, lse [R, Hq]).
    The products run on tcgen05 with tensor-memory accumulators; `warp_mma` takes the warp-level MMA kernel."""
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16:
        raise ValueError("q, k and v must be bfloat16")
    if q.stride(2) != 1 or k.stride(2) != 1 or v.stride(2) != 1 or k.stride() != v.stride():
        raise ValueError("head dims must be contiguous and k, v must share their layout")
    picked, members = _contig(picked), _contig(members)
    R, Hq, dh = q.shape
    slots, Hkv, _ = k.shape
    top_p = picked.shape[1]
    out = torch.empty(R, Hq, dh, device=q.device, dtype=torch.bfloat16) if out is None else out
    if out.shape != (R, Hq, dh) or out.dtype != torch.bfloat16 or not out.is_contiguous():
        raise ValueError(f"out must be a contiguous bfloat16 [{R}, {Hq}, {dh}]")
    lse = torch.empty(R, Hq, device=q.device, dtype=torch.float32) if lse is None else lse
    need = query("lsa_bucket_attend_workspace_bytes", R, top_p, Hq, dh, members.shape[0])
    if workspace is None or workspace.numel() * workspace.element_size() < need:
        workspace = torch.empty(max(need, 1), device=q.device, dtype=torch.uint8)
    call("lsa_bucket_attend", ptr(q), R, Hq, dh, q.stride(0), q.stride(1), ptr(k), ptr(v), slots, Hkv, k.stride(0),
         k.stride(1), ptr(picked), top_p, ptr(_contig(positions.to(torch.int64))), ptr(members), members.shape[0],
         members.shape[1], ptr(row_top_p), ptr(row_top_k), top_k, sink, window, ptr(init[0]) if init else None,
         ptr(init[1]) if init else None, float(scale), ptr(out), ptr(lse), 1 if warp_mma else 0,
         init_ready.cuda_event if init_ready is not None else None, ptr(status), ptr(workspace),
         workspace.numel() * workspace.element_size(), stream(), launches=6)
    return out, lse


def band_attend(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, first_position: int, window: int, sink: int,
                scale: float, out: torch.Tensor | None = None, lse: torch.Tensor | None = None,
                warp_mma: bool = False, status: torch.Tensor | None = None):
    """The window and sinks of consecutive query rows as dense banded attention: q [R, Hq, dh] at positions
    first_position.., k/v [n_keys, Hkv, dh] by position. Returns the PARTIAL read (out fp32 [R, Hq, dh], lse [R, Hq])
    that `sparse_attend(..., init=(out, lse))` extends with the selected keys. Dense heads of 128 dims and 128 rows
    or more run on tcgen05 with tensor-memory accumulators unless `warp_mma` asks for the warp-level kernel."""
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16:
        raise ValueError("q, k and v must be bfloat16")
    if q.stride(2) != 1 or k.stride(2) != 1 or v.stride(2) != 1 or k.stride() != v.stride():
        raise ValueError("head dims must be contiguous and k, v must share their layout")
    R, Hq, dh = q.shape
    out = torch.empty(R, Hq, dh, device=q.device, dtype=torch.float32) if out is None else out
    lse = torch.empty(R, Hq, device=q.device, dtype=torch.float32) if lse is None else lse
    call("lsa_band_attend", ptr(q), R, Hq, dh, q.stride(0), q.stride(1), ptr(k), ptr(v), k.shape[0], k.shape[1],
         k.stride(0), k.stride(1), first_position, window, sink, float(scale), ptr(out), ptr(lse),
         1 if warp_mma else 0, ptr(status), stream())
    return out, lse


def lse_merge(parts: torch.Tensor, lses: torch.Tensor, out_dtype=torch.float32):
    """Merge [n, rows..., dh] partial outputs (fp32, or bf16 for fewer than 16 parts) by their [n, rows...]
    log-sum-exps."""
    if parts.dtype != torch.bfloat16 or parts.shape[0] >= 16 or parts.shape[-1] % 8:
        parts = parts.float()
    parts, lses = _contig(parts), _contig(lses.float())
    n, dh = parts.shape[0], parts.shape[-1]
    rows = lses.numel() // n
    out = torch.empty(parts.shape[1:], device=parts.device, dtype=out_dtype)
    lse = torch.empty(lses.shape[1:], device=parts.device, dtype=torch.float32)
    call("lsa_lse_merge", ptr(parts), _lib.dtype_code(parts), ptr(lses), n, rows, dh,
         ptr(out) if out_dtype == torch.bfloat16 else None, ptr(out) if out_dtype == torch.float32 else None, ptr(lse),
         stream())
    return out, lse
