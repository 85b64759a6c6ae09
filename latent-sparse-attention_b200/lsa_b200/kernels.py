"""The device-kernel front doors the serving index calls, by the reference's names (`src/lsa/core/kernels/`):

    pack_keys / unpack_ids / unpack_scores / ordered_int32      triton/keys.py:36-88
    ScanSelect                                                  scan_select.py:189-385
    dense_keys / listed_keys / sample_thresholds                scan_select.py:24-143
    scan_paged                                                  triton/paged.py:61-101
    ShapeTable / build_shapes / build_bucket_shapes / score_shaped_rows / add_spread / add_planes_spread /
    scan_paged_shaped                                           triton/shape.py:42-886
    TopK / top_keys                                             triton/top_k.py:708-997
    DecodeSelect                                                cutedsl/decode.py:1035-1086
    expand_in_order / expand_by_threshold                       expansion.py:16-126
    cluster_ward / cluster_node_buckets                         ward.py:49-110
    bucket_members_from_labels                                  triton/ward.py:551

The reference picks Triton or CuTeDSL per step and may list a row twice or fall back to a dense scoring when its
threshold estimate misses; here one exact kernel answers every row, so `missed_runs` is always False and no call
reads the device on the host. `kernels=` is accepted for signature compatibility and ignored.
"""

from __future__ import annotations

from collections.abc import Sequence
from typing import NamedTuple

import torch

from lsa_b200 import ops
from lsa_b200.budget import EarlyBudget
from lsa_b200.constants import PackedKey, Sentinel


# --------------------------------------------------------------------------------------------- packed keys


def ordered_int32(scores: torch.Tensor) -> torch.Tensor:
    """fp32 scores as int32 of the same order."""
    bits = scores.contiguous().view(torch.int32)
    return torch.where(bits < 0, bits ^ 0x7FFFFFFF, bits)


def pack_keys(scores: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """Score in the high word, 2^31-1-id in the low; the empty key where an id is -1."""
    keys = (ordered_int32(scores).to(torch.int64) << 32) | (0x7FFFFFFF - ids.to(torch.int64))
    return torch.where(ids >= 0, keys, PackedKey.EMPTY)


def unpack_scores(keys: torch.Tensor) -> torch.Tensor:
    ordered = (keys >> 32).to(torch.int32)
    return torch.where(ordered < 0, ordered ^ 0x7FFFFFFF, ordered).view(torch.float32)


def unpack_ids(keys: torch.Tensor) -> torch.Tensor:
    ids = (0x7FFFFFFF - (keys & 0xFFFFFFFF)).to(torch.int32)
    return torch.where(keys == PackedKey.EMPTY, -1, ids)


# --------------------------------------------------------------------------------------------- selection


class Listing(NamedTuple):
    """A chunk's rows with their top-p packed keys, best first."""

    keys: torch.Tensor  # [R, top_p] int64
    visible_counts: torch.Tensor  # [R] int32


class ScanSelect:
    """The top-p buckets of a prefill chunk's centroid scores (scan_select.py:189-385)."""

    def __init__(self, rows: int, top_p: int, device="cuda", kernels: str = "b200") -> None:
        self.top_p, self.kernels = top_p, kernels
        self.keys = torch.empty(rows, top_p, device=device, dtype=torch.int64)
        self.out = torch.empty(rows, top_p, device=device, dtype=torch.int32)

    def __call__(self, index_queries, bucket_centroids, visible_counts, shapes=None) -> torch.Tensor:
        """Buckets [R, top_p] int32, the best score first and a tie to the lower bucket, -1 past a row's count."""
        return self.pick(self.listed(index_queries, bucket_centroids, visible_counts, shapes))

    def listed(self, index_queries, bucket_centroids, visible_counts, shapes=None) -> Listing:
        rows = index_queries.shape[0]
        if shapes is not None:  # (an `ops.ShapeTable`, row for row with the centroids)
            ops.shaped_select(index_queries, bucket_centroids, shapes, visible_counts, self.top_p,
                              keys=self.keys[:rows], picked=self.out[:rows])
        else:
            ops.flat_select(index_queries, bucket_centroids, visible_counts, self.top_p, keys=self.keys[:rows],
                            picked=self.out[:rows])
        return Listing(self.keys[:rows], visible_counts)

    def holds_top_p(self, listing: Listing) -> bool:
        return True

    def missed_runs(self, listing: Listing, runs: Sequence) -> list:
        """No run ever misses: the scan is exact, so nothing is listed again and the host reads nothing."""
        return [False for _ in runs]

    def pick(self, listing: Listing) -> torch.Tensor:
        return self.out[: listing.keys.shape[0]]


# The reference's selection is two passes - scores written out, then a pick over them - and its serving index is
# written against the pieces of that. Here one kernel scores and picks, so these are thin: the dense forms write the
# matrix with the exact fixed-order dot, the picks run the packed-key selection over it.

SAMPLE_TARGET, SAMPLE_RANK, SCAN_MARGIN = 1.5, 64, 1e-4  # (kernels/constants.py:179-186)


def _dense_scores(index_queries, bucket_centroids, visible_counts, width=None, shapes=None) -> torch.Tensor:
    """Every bucket a row sees scored at its own column [R, width] fp32, -inf past a row's count: by its centroid, or
    with `shapes` (an `ops.ShapeTable`) by its estimated best key."""
    if shapes is None:
        return ops.dense_scores(index_queries, bucket_centroids, visible_counts, width)
    scores = ops.shaped_scores(index_queries, bucket_centroids, shapes, width=width)
    columns = torch.arange(scores.shape[1], device=scores.device)
    return torch.where(columns[None] < visible_counts.to(torch.int64)[:, None], scores, float("-inf"))


def dense_keys(index_queries, bucket_centroids, visible_counts, width=None, shapes=None, query_planes=None,
               kernels: str = "b200") -> torch.Tensor:
    """Every bucket a row sees scored and packed with its bucket, at its own column [R, width] int64, the empty key
    past a row's length (scan_select.py:24-58). `shapes`: the buckets' `ShapeTable`; the reference scores a shaped
    bucket against the bit-planes of the query (`query_planes`), here the query itself is read and none are needed."""
    if shapes is None:
        return ops.dense_scores(index_queries, bucket_centroids, visible_counts, width, keys=True)
    scores = _dense_scores(index_queries, bucket_centroids, visible_counts, width, shapes)
    ids = torch.arange(scores.shape[1], device=scores.device, dtype=torch.int32)[None].expand_as(scores)
    return torch.where(scores > float("-inf"), pack_keys(scores, ids), PackedKey.EMPTY)


def scan_paged(index_queries, bucket_centroids, pages, counts, page_size: int, max_rows: int) -> torch.Tensor:
    """Each request's buckets scored through its pages [B, max_rows] fp32, -inf past a request's count or on a page
    it has not got (triton/paged.py:61-101)."""
    return ops.dense_scores(index_queries, bucket_centroids, counts, max_rows, pages=pages, page_rows=page_size)


# --------------------------------------------------------------------------------------------- bucket shapes

ShapeTable = ops.ShapeTable  # (triton/shape.py:42-61)


def build_shapes(index_keys, centroids, members, rank: int):
    """Shape each bucket over every key under it (triton/shape.py:798-846): (packed sign basis [N, rank, d / 8] uint8,
    variances [N, rank] fp32 descending, floor [N] fp32). `index_keys` maps positions [M] int64 to their index keys
    [M, d], as the reference's callers pass it, or is the key matrix itself."""
    if callable(index_keys):
        held = members >= 0
        if not bool(held.any()):
            keys, first = torch.zeros(1, centroids.shape[1], device=centroids.device), 0
        else:
            first, last = int(members[held].min()), int(members[held].max())
            keys = index_keys(torch.arange(first, last + 1, device=members.device))
    else:
        keys, first = index_keys, 0
    built = ops.shape_build(keys, centroids, members, rank, key_base=first)
    return built.basis, built.variances, built.floor


def build_bucket_shapes(index_keys, centroids, members, rank: int):
    """Shape buckets of at most a cap of keys exactly (triton/shape.py:849-886). The device build is exact for any
    bucket, so this is `build_shapes`."""
    return build_shapes(index_keys, centroids, members, rank)


def score_shaped_rows(index_queries, centroids, basis, variances, floor, rows, deviations: float) -> torch.Tensor:
    """Each query against the table rows it names by their estimated best key [S, width] fp32, -inf where a row is
    -1 (triton/shape.py:281-343)."""
    return ops.shaped_scores(index_queries, centroids, ShapeTable(basis, variances, floor, deviations), rows=rows)


def add_spread(scores, index_queries, basis, variances, floor, deviations: float) -> torch.Tensor:
    """`scores` [S, m] plus `deviations` times each bucket's spread under each query (triton/shape.py:523-570)."""
    zero = torch.zeros(floor.shape[0], index_queries.shape[1], device=scores.device)
    return scores + ops.shaped_scores(index_queries, zero, ShapeTable(basis, variances, floor, deviations),
                                      width=scores.shape[1])


def add_planes_spread(scores, index_queries, shapes: ShapeTable) -> torch.Tensor:
    """The same from a table (triton/shape.py:407-450; the reference reads the query's bit-planes there and the bf16
    query in `add_spread`, here both read the fp32 query and agree bit for bit)."""
    return add_spread(scores, index_queries, shapes.basis, shapes.variances, shapes.floor, shapes.deviations)


def scan_paged_shaped(index_queries, bucket_centroids, shapes: ShapeTable, pages, counts, page_size: int,
                      max_rows: int) -> torch.Tensor:
    """Each request's buckets scored by their estimated best key through its pages [B, max_rows] fp32, -inf past a
    request's count or on a page it has not got (triton/shape.py:659-717)."""
    logical = torch.arange(max_rows, device=pages.device)
    page = pages.long()[:, (logical // page_size).clamp_max(pages.shape[1] - 1)]
    held = (logical[None] < counts.to(torch.int64)[:, None]) & (page >= 0) & (logical[None] // page_size < pages.shape[1])
    rows = torch.where(held, page * page_size + logical[None] % page_size, -1).to(torch.int32)
    return ops.shaped_scores(index_queries, bucket_centroids, shapes, rows=rows)


def sample_plan(top_p: int) -> tuple:
    """Buckets between two sampled ones, and the rank in the sample the threshold is read at
    (triton/scan_select.py:687-698)."""
    stride = max(1, round(SAMPLE_TARGET * top_p / SAMPLE_RANK))
    return stride, max(1, round(SAMPLE_TARGET * top_p / stride))


def sample_thresholds(index_queries, bucket_centroids, visible_counts, top_p: int, shapes=None, query_planes=None,
                      kernels: str = "b200") -> torch.Tensor:
    """Each row's score at 1.5 times its top_p, estimated from every stride-th bucket it sees [R] fp32, -inf for a
    row that sees too few to rank (scan_select.py:110-143). The estimate here is the sampled score of that rank
    itself, where the reference takes the lower edge of its histogram bin: both err toward more survivors."""
    stride, rank = sample_plan(top_p)
    sampled = bucket_centroids[::stride]
    counts = (visible_counts.to(torch.int64) + stride - 1) // stride
    scores = _dense_scores(index_queries, sampled, counts.to(torch.int32),
                           shapes=None if shapes is None else shapes.rows(slice(None, None, stride)))
    if scores.shape[1] < rank:
        return torch.full((scores.shape[0],), float("-inf"), device=scores.device)
    ranked = scores.topk(rank, dim=1).values[:, rank - 1]
    return torch.where(counts >= rank, ranked, float("-inf"))


def listed_keys(index_queries, bucket_centroids, visible_counts, thresholds, capacity: int, shapes=None,
                query_planes=None, kernels: str = "b200"):
    """The buckets each row scores near its threshold, scored and packed (scan_select.py:61-107): packed keys
    [R, capacity] int64 of the first `capacity` listed buckets in bucket order, the empty key after; buckets each row
    listed [R] int32 (above capacity: the buffer overflowed); listed buckets at or above the threshold [R] int32."""
    keys = dense_keys(index_queries, bucket_centroids, visible_counts, shapes=shapes)
    scores = unpack_scores(keys)
    shifted = thresholds - SCAN_MARGIN * index_queries.float().norm(dim=1)
    listed = (keys != PackedKey.EMPTY) & (scores >= shifted[:, None])
    slot = listed.cumsum(1) - 1
    out = torch.full((keys.shape[0], capacity + 1), PackedKey.EMPTY, device=keys.device, dtype=torch.int64)
    out.scatter_(1, torch.where(listed & (slot < capacity), slot, capacity), keys)
    reached = (listed & (scores >= thresholds[:, None])).sum(1, dtype=torch.int32)
    return out[:, :capacity].contiguous(), listed.sum(1, dtype=torch.int32), reached


class TopK:
    """The best k columns of each row of a score matrix (triton/top_k.py:708-975). A listing here is always exact:
    each row's best k, which is also a valid superset."""

    def __init__(self, k: int, rows: int | None = None, device="cuda", exact: bool = False) -> None:
        self.k, self.exact = k, exact
        self.keys = torch.empty(0, 0, dtype=torch.int64)
        self.counts = torch.empty(0, dtype=torch.int32)

    def release(self) -> None:
        self.keys = torch.empty(0, 0, dtype=torch.int64)
        self.counts = torch.empty(0, dtype=torch.int32)

    def _best(self, scores: torch.Tensor, lengths: torch.Tensor) -> torch.Tensor:
        """Packed keys [R, k] of each row's best k columns, best first, a tie to the lower column."""
        if scores.dtype != torch.float32:
            raise TypeError(f"a top-k reads fp32 scores, not {scores.dtype}")
        rows, columns = scores.shape
        ids = torch.arange(columns, device=scores.device, dtype=torch.int32)
        keys = torch.where(ids[None] < lengths[:, None], pack_keys(scores, ids.expand(rows, -1)), PackedKey.EMPTY)
        parts = -(-columns // self.k)
        padded = torch.full((rows, parts * self.k), PackedKey.EMPTY, device=scores.device, dtype=torch.int64)
        padded[:, :columns] = keys
        best, _ = ops.merge_candidates(padded.view(rows, parts, self.k).permute(1, 0, 2).contiguous())
        return best

    def listed(self, scores: torch.Tensor, lengths: torch.Tensor):
        """Packed keys [R, W] of each row's best k in column order, W the lesser of k and N, and the keys each row
        listed [R] int32."""
        width = min(self.k, scores.shape[1])
        best = self._best(scores, lengths)[:, :width]
        by_column = torch.where(best != PackedKey.EMPTY, unpack_ids(best).long(), 1 << 40).argsort(dim=1)
        self.keys = best.gather(1, by_column)
        self.counts = torch.clamp(lengths, max=width).to(torch.int32)
        return self.keys, self.counts

    def best(self) -> torch.Tensor:
        """The last listing's best k as packed keys [R, k], the best score first, the empty key past a row's length."""
        rows, width = self.keys.shape
        out = torch.full((rows, self.k), PackedKey.EMPTY, device=self.keys.device, dtype=torch.int64)
        out[:, :width] = self.keys.sort(dim=1, descending=True).values
        return out

    def __call__(self, scores: torch.Tensor, lengths: torch.Tensor) -> torch.Tensor:
        """The k best columns of each row [R, k] int32 in ascending column order, -1 past the last."""
        keys, _ = self.listed(scores, lengths)
        out = torch.full((scores.shape[0], self.k), Sentinel.PAD, device=scores.device, dtype=torch.int32)
        out[:, :keys.shape[1]] = unpack_ids(keys)
        return out


def top_keys(scores: torch.Tensor, lengths: torch.Tensor, k: int) -> torch.Tensor:
    """The best k columns of each row as packed keys [R, k], best first (triton/top_k.py:978-997)."""
    pick = TopK(k)
    pick.listed(scores, lengths)
    return pick.best()


class DecodeSelect:
    """A flat decode step's listing through the requests' page tables (cutedsl/decode.py:1035-1086)."""

    def __init__(self, top_p: int, splits: int = 4) -> None:
        self.top_p, self.splits = top_p, splits

    def listed(self, index_queries, bucket_centroids, pages, counts, page_rows: int, max_rows: int):
        """Packed keys [B, top_p] int64 holding each request's top-p (best first) and the keys each lists [B]."""
        keys, _ = ops.flat_select_paged(index_queries, bucket_centroids, pages, counts, page_rows, self.top_p,
                                        splits=self.splits)
        return keys, (keys != PackedKey.EMPTY).sum(1, dtype=torch.int32)

    def pick(self, listing) -> torch.Tensor:
        """Buckets [B, top_p] int32, best first, -1 past a request's count."""
        return unpack_ids(listing[0])


# --------------------------------------------------------------------------------------------- expansion


def _budgets(positions: torch.Tensor, top_p: int, top_k: int, early: EarlyBudget | None):
    if early is None:
        return None, None
    before = positions < early.position
    return (torch.where(before, early.top_p, top_p).to(torch.int32),
            torch.where(before, early.top_k, top_k).to(torch.int32))


def expand_in_order(selected, bucket_members, positions, window_size, sink_size, top_k, slot_table=None,
                    slot_rows=None, kernels: str = "b200", early: EarlyBudget | None = None):
    """Read lists from picked cache rows, best first until the top-k is full (expansion.py:16-58). With
    `slot_table` [requests, context] every position is stored as its KV slot, `slot_rows` naming each row's
    request."""
    if slot_table is None:
        row_p, row_k = _budgets(positions, selected.shape[1], top_k, early)
        lists, lengths, _ = ops.expand(selected, positions, bucket_members, top_k, sink_size, window_size, row_p, row_k)
        return lists, lengths
    if early is not None:
        raise NotImplementedError("an early budget with a slot table is not built")
    lists, lengths, _ = ops.expand_batched(selected, positions, slot_rows, bucket_members, None, 1, slot_table, 1,
                                           top_k, sink_size, window_size)
    return lists, lengths


def expand_by_threshold(keys, listed, bucket_members, bucket_sizes, request_blocks, request_rows, positions,
                        page_size, cluster_block_size, top_p, window_size, sink_size, top_k, slot_table=None,
                        block_positions=None, kernels: str = "b200", early: EarlyBudget | None = None):
    """Fill each row's read from its listed buckets (expansion.py:59-126): the best `top_p` keys of the listing
    are walked best first until `top_k` members are held. Keys hold a request's logical buckets, read through
    `request_blocks` [requests, pages] of `page_size` cache rows."""
    if block_positions is not None or early is not None:
        raise NotImplementedError("cache-row keys and early budgets are not built for the threshold expansion")
    held = torch.arange(keys.shape[1], device=keys.device)[None] < listed[:, None]
    best = keys.masked_fill(~held, PackedKey.EMPTY).topk(min(top_p, keys.shape[1]), dim=1).values
    picked = unpack_ids(best)
    lists, _, _ = ops.expand_batched(picked, positions, request_rows, bucket_members, request_blocks, page_size,
                                     slot_table, 1, top_k, sink_size, window_size)
    return lists


# --------------------------------------------------------------------------------------------- clustering


def cluster_ward(pool_keys, pool_sizes, bucket_count, bucket_cap, precision: str = "ieee", kernels: str = "b200"):
    """Labels [G, P] int64 and whether each block reached its count (ward.py:49-81). The Gram dot is fp32 in a
    fixed order whatever `precision` says."""
    return ops.ward_rounds(pool_keys, pool_sizes, bucket_count, bucket_cap)


def cluster_node_buckets(key_sums, precision: str = "ieee", rounds_a_check: int = 8, kernels: str = "b200"):
    """Each bucket's pair [G, P] int64, numbered by first bucket (ward.py:84-110)."""
    pairs, _ = ops.ward_rounds(key_sums, 1.0, key_sums.shape[1] // 2, 2.0)
    return pairs


def bucket_members_from_labels(labels, bucket_count: int, bucket_cap: int, pool_size: int = 1):
    """Member table [G * bucket_count, cap] int32 (-1 padded, block-local positions made absolute block after block)."""
    return ops.bucket_members(labels, pool_size, bucket_count, bucket_cap)[0]
