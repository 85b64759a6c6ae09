"""The device-kernel front doors the serving index calls, by the reference's names (`src/lsa/core/kernels/`):

    pack_keys / unpack_ids / unpack_scores / ordered_int32      triton/keys.py:36-88
    ScanSelect                                                  scan_select.py:189-385
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
from lsa_b200.constants import PackedKey


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
        if shapes is not None:
            raise NotImplementedError("bucket shapes are not built in lsa_b200")
        rows = index_queries.shape[0]
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
