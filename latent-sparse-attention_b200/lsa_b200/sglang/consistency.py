"""Whether every rank of a decode context-parallel group holds the same index: a checksum summed across the group
(`src/lsa/sglang/index/consistency.py:1-136`).

Every rank keeps the whole bucket cache and grows it from index keys the group sums. Nothing compares the copies while
serving: a rank whose cache drifted would select other lists without an error. The check folds a request's buckets
into one checksum, sums it across the group and raises on every rank at once when any rank's differs. It costs two
sums and a host read a layer, so a server runs it only when asked to.
"""

from __future__ import annotations

from collections.abc import Callable, Sequence

import torch

CHECKSUM_BYTES = 1 << 24  # bytes folded at once: the int64 copies stay a few hundred MB whatever the context
PIECE_BITS, PIECES = 20, 3  # a checksum crosses the group as exact fp32 pieces: up to 8 ranks sum 20 bits exactly


def checksum(values: torch.Tensor) -> torch.Tensor:
    """An order-sensitive checksum of a tensor's bytes [] int64: every byte times its place, summed in integers, which
    wrap instead of rounding - so the order a reduction adds in does not change it."""
    data = values.clone(memory_format=torch.contiguous_format).view(-1).view(torch.uint8)
    total = torch.zeros((), dtype=torch.int64, device=values.device)
    for first in range(0, len(data), CHECKSUM_BYTES):
        part = data[first:first + CHECKSUM_BYTES].long()
        total += (part * torch.arange(first + 1, first + len(part) + 1, device=values.device)).sum()
    return total


def request_checksum(cache, row: int) -> torch.Tensor:
    """The checksum of one request's index [] int64: the centroids, members and sizes of its buckets in logical
    order, and its counts (keys taken, keys in closed blocks)."""
    held = cache.buckets_of(row)
    rows = cache.rows_of(row, torch.arange(held, device=cache.sizes.device))
    counts = torch.tensor([cache.end(row), cache.closed_keys.get(row, 0), held], dtype=torch.int64,
                          device=cache.sizes.device)
    total = torch.zeros((), dtype=torch.int64, device=cache.sizes.device)
    for place, part in enumerate((cache.centroids[rows], cache.members[rows], cache.sizes[rows], counts)):
        total += checksum(part) * (2 * place + 1)  # an odd factor each: the same bytes in another part check differently
    return total


def check_same_index(cache, rows: Sequence, reduce: Callable[[torch.Tensor], torch.Tensor], size: int) -> None:
    """Raise on every rank unless every rank of the group holds the same buckets for each request. Every rank calls it
    with the same rows, as it holds the same batch.

    Raises:
        RuntimeError: Some rank's index differs from another's.
    """
    if not rows:
        return
    totals = torch.stack([request_checksum(cache, row) for row in rows])
    shifts = PIECE_BITS * torch.arange(PIECES, device=totals.device)
    local = ((totals[:, None] >> shifts) & ((1 << PIECE_BITS) - 1)).float()
    differs = (reduce(local.clone()) != local * size).any().float().reshape(1)
    if float(reduce(differs).item()):
        raise RuntimeError(f"the decode context-parallel group's ranks hold different indexes for request table rows "
                           f"{list(rows)}")
