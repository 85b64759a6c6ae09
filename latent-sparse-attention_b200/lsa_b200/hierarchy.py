"""Fixed and tree: node bucket levels over the buckets, and a beam down them, on B200 kernels.

Same names, argument meaning and results as the reference's specification (`src/lsa/core/hierarchy.py`):
`Hierarchy`, `per_level`, `pair_into_node_buckets`, `build_hierarchy`, `growth_at`, `read_hierarchy`,
`read_hierarchy_counted`. The pairings run in `lsa_ward_merge` (blocks of up to 4,096 children), key sums in
`lsa_gather_sum`, every beam level in `lsa_beam_step`, the expansion in `lsa_expand`. The research options of the
reference (`position` grouping, `lse` scores) are not built and raise `NotImplementedError`.
"""

from __future__ import annotations

from collections.abc import Sequence
from typing import NamedTuple

import torch
import torch.nn.functional as F

from lsa_b200 import ops
from lsa_b200.core import CLUSTER_ALGORITHMS, Buckets, check_read_arguments, check_unit_rows

BUCKET_SCORES = ("centroid", "lse")


class Hierarchy(NamedTuple):
    """The node bucket levels over a cache's buckets (hierarchy.py:37-51), level 1 first."""

    node_centroids: list  # each [N, index_dim] fp32
    children: list  # each [N, node_bucket_size] int64 - bucket rows under level 1, the level below's rows above
    node_means: list  # each [N, index_dim] fp32
    bucket_means: torch.Tensor  # [rows, index_dim] fp32
    node_bucket_size: int
    node_cluster_block_sizes: tuple


class Growth(NamedTuple):
    """The counts of a hierarchy as a query sees it (hierarchy.py:54-62)."""

    covered_buckets: int
    made: list
    closed: list


def per_level(value: int | Sequence[int], top_level: int) -> tuple:
    """A knob's value at each level from 1 to `top_level` - a scalar is every level's (hierarchy.py:65-70)."""
    values = (value,) * top_level if isinstance(value, int) else tuple(value)
    if len(values) != top_level:
        raise ValueError(f"a per-level knob takes one value or {top_level} - got {len(values)}")
    return values


def _rows_of(labels: torch.Tensor, groups: int, width: int) -> torch.Tensor:
    """[G, P] labels -> [G * groups, width] int64: each group's rows ascending, numbered across the blocks."""
    members, _ = ops.bucket_members(labels, 1, groups, width)
    return members.to(torch.int64)


def pair_into_node_buckets(key_sums: torch.Tensor, node_bucket_size: int,
                           node_cluster_algorithm: str = "ward") -> torch.Tensor:
    """Each bucket's node bucket [G, P] int64: paired by the Ward merge, then the pairs, to exactly the size
    (hierarchy.py:73-98)."""
    if node_cluster_algorithm != "ward":
        raise NotImplementedError("only the ward node grouping is built in lsa_b200")
    blocks, buckets, index_dim = key_sums.shape
    labels = torch.arange(buckets, device=key_sums.device).expand(blocks, buckets)
    sums = key_sums.contiguous()
    for _ in range(node_bucket_size.bit_length() - 1):
        count = sums.shape[1]
        pairs, _ = ops.ward_rounds(sums, 1.0, count // 2, 2.0)
        labels = pairs.gather(1, labels)
        # a pair's sum is its lower row plus its higher row
        sums = ops.gather_sum(sums.view(blocks * count, index_dim), _rows_of(pairs, count // 2, 2)).view(
            blocks, count // 2, index_dim)
    return labels


def build_hierarchy(index_keys: torch.Tensor, buckets: Buckets, top_level: int, node_bucket_size: int,
                    node_cluster_block_size: int | Sequence[int], node_cluster_algorithm: str = "ward") -> Hierarchy:
    """Pair every full node cluster block of every level into node buckets (hierarchy.py:101-162)."""
    check_unit_rows("index_keys", index_keys)
    block_sizes = per_level(node_cluster_block_size, top_level)
    if top_level < 1:
        raise ValueError(f"top_level must be 1 or more - got {top_level}")
    if node_bucket_size < 2 or node_bucket_size & (node_bucket_size - 1):
        raise ValueError(f"node_bucket_size must be a power of two from 2 - got {node_bucket_size}")
    if any(block % node_bucket_size for block in block_sizes):
        raise ValueError(f"every node_cluster_block_size must be a multiple of {node_bucket_size} - got {block_sizes}")
    if node_cluster_algorithm not in CLUSTER_ALGORITHMS:
        raise ValueError(f"node_cluster_algorithm must be one of {CLUSTER_ALGORITHMS} - got {node_cluster_algorithm!r}")
    key_sums = ops.gather_sum(index_keys, buckets.bucket_members)
    key_counts = buckets.bucket_sizes.float()
    bucket_means = key_sums / key_counts.clamp_min(1)[:, None]
    node_centroids, children, node_means = [], [], []
    for block in block_sizes:
        blocks = key_sums.shape[0] // block
        if not blocks:
            break
        count = blocks * block
        labels = pair_into_node_buckets(key_sums[:count].view(blocks, block, -1), node_bucket_size,
                                        node_cluster_algorithm)
        kids = _rows_of(labels.contiguous(), block // node_bucket_size, node_bucket_size)
        key_sums = ops.gather_sum(key_sums, kids)
        key_counts = key_counts[kids].sum(1)
        node_centroids.append(F.normalize(key_sums, dim=-1))
        node_means.append(key_sums / key_counts.clamp_min(1)[:, None])
        children.append(kids)
    return Hierarchy(node_centroids, children, node_means, bucket_means, node_bucket_size, block_sizes)


class GrowingHierarchy:
    """A request's hierarchy grown ONLINE, a page end at a time, in tensors whose addresses never move - so a decode
    step captured in a CUDA graph keeps reading the same arrays while the tree grows under it. What the reference
    does with `Hierarchy.grow` / `stage` and the `GraphTree` mirror beside it (src/lsa/sglang/index/hierarchy.py:
    246-476, src/lsa/sglang/index/graph_tree.py:54-330); here the growing tensors are sized once for the longest
    context, so they are their own mirror.

    A growth pairs whole node cluster blocks in the order they fill, and a block's node buckets depend on nothing but
    its own children, so after any number of page ends the levels hold exactly the first `made[level]` node buckets of
    `build_hierarchy` over the full cache (checked in the tests), and `growth_at` counts what each `grow` made.
    Node centroids are fp32 (the reference stores them in bf16 or fp8: not carried).
    """

    def __init__(self, index_dim: int, top_level: int, node_bucket_size: int,
                 node_cluster_block_size: int | Sequence[int], growth_buckets: int, max_buckets: int, device="cuda"):
        self.node_bucket_size, self.growth_buckets = node_bucket_size, growth_buckets
        self.block_sizes = per_level(node_cluster_block_size, top_level)
        if node_bucket_size < 2 or node_bucket_size & (node_bucket_size - 1):
            raise ValueError(f"node_bucket_size must be a power of two from 2 - got {node_bucket_size}")
        if any(block % node_bucket_size for block in self.block_sizes):
            raise ValueError(f"every node_cluster_block_size must be a multiple of {node_bucket_size}")
        self.covered, self.made, self.closed = 0, [0] * top_level, [0] * top_level
        rooms, room = [], max_buckets
        for _ in range(top_level):
            room //= node_bucket_size
            rooms.append(max(room, 1))
        make = lambda rows, cols, dtype: torch.zeros(rows, cols, device=device, dtype=dtype)
        self.node_centroids = [make(room, index_dim, torch.float32) for room in rooms]
        self.node_means = [make(room, index_dim, torch.float32) for room in rooms]
        self.children = [torch.full((room, node_bucket_size), -1, device=device, dtype=torch.int64) for room in rooms]
        self.key_sums = [make(room, index_dim, torch.float32) for room in rooms]
        self.key_counts = [torch.zeros(room, device=device, dtype=torch.float32) for room in rooms]
        self.bucket_means = make(max_buckets, index_dim, torch.float32)
        # the same counts where a captured step can read them: covered, then made and closed a level
        self.counts_device = torch.zeros(1 + 2 * top_level, device=device, dtype=torch.int32)

    def _pair(self, level: int, sums: torch.Tensor, counts: torch.Tensor, first_child: int) -> None:
        """Pair the whole blocks of `sums` [n, d] (children first_child .. of the level below) into node buckets of
        `level`, appended in block order."""
        block, size = self.block_sizes[level - 1], self.node_bucket_size
        blocks = sums.shape[0] // block
        labels = pair_into_node_buckets(sums.view(blocks, block, -1), size)
        kids = _rows_of(labels.contiguous(), block // size, size)
        node_sums = ops.gather_sum(sums.contiguous(), kids)
        node_counts = counts[kids].sum(1)
        at, new = self.made[level - 1], kids.shape[0]
        if at + new > self.children[level - 1].shape[0]:
            raise RuntimeError(f"level {level} holds {self.children[level - 1].shape[0]} node buckets and {at + new} "
                               "were made: the hierarchy was sized for a shorter context")
        self.node_centroids[level - 1][at:at + new] = F.normalize(node_sums, dim=-1)
        self.node_means[level - 1][at:at + new] = node_sums / node_counts.clamp_min(1)[:, None]
        self.children[level - 1][at:at + new] = kids + first_child
        self.key_sums[level - 1][at:at + new] = node_sums
        self.key_counts[level - 1][at:at + new] = node_counts
        self.made[level - 1] = at + new

    def grow(self, closed_buckets: int, index_keys: torch.Tensor, buckets: Buckets) -> int:
        """One page end: with `closed_buckets` buckets of the request closed, pair the full node cluster blocks of
        uncovered buckets (none while fewer than `growth_buckets` wait) and whatever that fills above. Returns the
        level-1 node buckets made."""
        first_block = self.block_sizes[0]
        blocks = (closed_buckets - self.covered) // first_block
        if blocks < max(1, self.growth_buckets // first_block):
            return 0
        count, before = blocks * first_block, self.made[0]
        rows = slice(self.covered, self.covered + count)
        sums = ops.gather_sum(index_keys, buckets.bucket_members[rows])
        counts = buckets.bucket_sizes[rows].float()
        self.bucket_means[rows] = sums / counts.clamp_min(1)[:, None]
        self._pair(1, sums, counts, self.covered)
        self.covered += count
        for level in range(2, len(self.block_sizes) + 1):
            block = self.block_sizes[level - 1]
            taken = (self.made[level - 2] - self.closed[level - 2]) // block * block
            if not taken:
                break
            first = self.closed[level - 2]
            self._pair(level, self.key_sums[level - 2][first:first + taken], self.key_counts[level - 2][first:first + taken],
                       first)
            self.closed[level - 2] = first + taken
        self.counts_device.copy_(torch.tensor([self.covered, *self.made, *self.closed], dtype=torch.int32),
                                 non_blocking=True)
        return self.made[0] - before

    def counts(self) -> Growth:
        return Growth(self.covered, list(self.made), list(self.closed))

    def view(self) -> Hierarchy:
        """The levels as `read_hierarchy` and `TreeDecoder` take them: the whole fixed-address arrays (a read looks at
        the first `made` rows of each, which `growth_at` counts for its position)."""
        return Hierarchy(self.node_centroids, self.children, self.node_means, self.bucket_means, self.node_bucket_size,
                         self.block_sizes)


def growth_at(hierarchy: Hierarchy, closed_buckets: int, page_buckets: int, growth_buckets: int) -> Growth:
    """Replay growing at every page end up to `closed_buckets`, from the counts alone. Integer bookkeeping that must
    match the reference count for count, so it is transcribed from it (src/lsa/core/hierarchy.py:165-196)."""
    sizes = hierarchy.node_cluster_block_sizes
    top_level, size, first_block = len(sizes), hierarchy.node_bucket_size, sizes[0]
    covered, made, closed = 0, [0] * top_level, [0] * top_level
    for end in range(page_buckets, closed_buckets + 1, page_buckets):
        blocks = (end - covered) // first_block
        if blocks < max(1, growth_buckets // first_block):
            continue
        covered += blocks * first_block
        made[0] += blocks * first_block // size
        for level in range(1, top_level):
            taken = (made[level - 1] - closed[level - 1]) // sizes[level] * sizes[level]
            if not taken:
                break
            closed[level - 1] += taken
            made[level] += taken // size
    return Growth(covered, made, closed)


def read_hierarchy(index_queries, positions, buckets, hierarchy, beam_width, start_nodes, top_p, top_k, sink_size,
                   window_size, page_size, growth_buckets, node_bucket_score="centroid", bucket_score="centroid",
                   tau=1.0, index_keys=None):
    """`read_hierarchy_counted` without the count (hierarchy.py:199-260)."""
    selected, lengths, _ = read_hierarchy_counted(index_queries, positions, buckets, hierarchy, beam_width,
                                                  start_nodes, top_p, top_k, sink_size, window_size, page_size,
                                                  growth_buckets, node_bucket_score, bucket_score, tau, index_keys)
    return selected, lengths


def beam_plan(hierarchy: Hierarchy, buckets: Buckets, positions: list, page_size: int, growth_buckets: int,
              start_nodes: int | None):
    """Host arithmetic of a read: for every row its start level and, level by level, the run of open rows it scores.

    Returns `start` [R] and `runs`: runs[level] = (first [R], end [R]) for level 1..top, and runs[0] for the buckets.
    """
    page_buckets = page_size // buckets.cluster_block_size * buckets.block_bucket_count
    top = len(hierarchy.node_cluster_block_sizes)
    total = int(buckets.bucket_sizes.shape[0])
    starts, runs = [], [([], []) for _ in range(top + 1)]
    cache: dict = {}
    for position in positions:
        closed_buckets = position // page_size * page_buckets
        growth = cache.get(closed_buckets)
        if growth is None:
            growth = cache[closed_buckets] = growth_at(hierarchy, closed_buckets, page_buckets, growth_buckets)
        levels = sum(1 for count in growth.made if count)
        start = levels
        if start_nodes is not None:
            start = next((lv for lv in range(1, levels + 1) if growth.made[lv - 1] <= start_nodes), levels)
        starts.append(start)
        for level in range(1, top + 1):
            if level > start:
                first = end = 0
            else:
                first = 0 if level == start and start_nodes is not None else growth.closed[level - 1]
                end = growth.made[level - 1]
            runs[level][0].append(first)
            runs[level][1].append(end)
        visible = min(position // buckets.cluster_block_size * buckets.block_bucket_count, total)
        runs[0][0].append(growth.covered_buckets)
        runs[0][1].append(max(visible, growth.covered_buckets))
    return starts, runs


def read_hierarchy_counted(index_queries, positions, buckets, hierarchy, beam_width, start_nodes, top_p, top_k,
                           sink_size, window_size, page_size, growth_buckets, node_bucket_score="centroid",
                           bucket_score="centroid", tau=1.0, index_keys=None):
    """Select the keys each query reads by a beam down the levels its page saw (hierarchy.py:263-345).

    Returns selected ids [Tq, top_k + window + sink] int32 (-1 padded), lengths [Tq] int32, and the vectors each
    row scored [Tq] int64.
    """
    check_read_arguments(index_queries, positions, buckets, top_p, top_k, sink_size, window_size)
    if page_size % buckets.cluster_block_size:
        raise ValueError(f"page_size {page_size} must be a multiple of cluster_block_size {buckets.cluster_block_size}")
    if node_bucket_score not in BUCKET_SCORES or bucket_score not in BUCKET_SCORES:
        raise ValueError(f"node_bucket_score and bucket_score must be one of {BUCKET_SCORES} - got "
                         f"{node_bucket_score!r}, {bucket_score!r}")
    if tau <= 0:
        raise ValueError(f"tau must be positive - got {tau}")
    if bucket_score == "lse" and index_keys is None:
        raise ValueError("the lse bucket score reads the buckets' keys - pass index_keys")
    if node_bucket_score != "centroid" or bucket_score != "centroid":
        raise NotImplementedError("only centroid scores are built in lsa_b200")
    top = len(hierarchy.node_cluster_block_sizes)
    beam_widths = per_level(beam_width, top)
    device = index_queries.device
    position_list = positions.tolist()
    starts, runs = beam_plan(hierarchy, buckets, position_list, page_size, growth_buckets, start_nodes)
    rows = len(position_list)
    as_tensor = lambda values: torch.tensor(values, dtype=torch.int32, device=device)
    queries = index_queries.float().contiguous()
    picked = torch.full((rows, top_p), -1, dtype=torch.int32, device=device)
    scored = torch.zeros(rows, dtype=torch.int64, device=device)
    built = len(hierarchy.node_centroids)
    # Rows that start at the same level walk the same number of steps: one launch a level for each such group.
    for start in sorted(set(starts)):
        if start > built:
            raise ValueError(f"a query's page saw {start} levels and the hierarchy holds {built}")
        group = torch.tensor([i for i, s in enumerate(starts) if s == start], dtype=torch.int64, device=device)
        q = queries[group]
        carried = None
        for level in range(start, 0, -1):
            first, end = as_tensor(runs[level][0])[group], as_tensor(runs[level][1])[group]
            scored[group] += (end - first).clamp_min(0) + (0 if carried is None else (carried >= 0).sum(1))
            carried = ops.beam_step(q, hierarchy.node_centroids[level - 1], carried, first, end,
                                    beam_widths[level - 1], children=hierarchy.children[level - 1])
        first, end = as_tensor(runs[0][0])[group], as_tensor(runs[0][1])[group]
        scored[group] += (end - first).clamp_min(0) + (0 if carried is None else (carried >= 0).sum(1))
        kept, _ = ops.beam_step(q, buckets.bucket_centroids, carried, first, end, top_p)
        picked[group] = kept
    selected, lengths, _ = ops.expand(picked, positions, buckets.bucket_members, top_k, sink_size, window_size)
    return selected, lengths, scored
