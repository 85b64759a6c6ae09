"""Decode steps with fixed shapes and no host reads, so a step can be captured in a CUDA graph.

`TreeDecoder` is one request's tree read (the reference's captured path: `GraphTree` + `graph_descend.descend`,
`src/lsa/sglang/index/graph_tree.py:1-10`, `src/lsa/sglang/index/graph_descend.py:1-16`, `selector.py:567-601`): the
host replays the tree's growth for the query's page ONCE (`prepare`), which fixes the run of open rows each level
scores; a step is then index map -> one beam step a level -> bucket pick -> expansion -> split attention + merge,
every launch on preallocated shapes.
"""

from __future__ import annotations

import torch

from lsa_b200 import ops, probe
from lsa_b200.core import Buckets
from lsa_b200.hierarchy import Hierarchy, beam_plan, per_level
from lsa_b200.layer import FlatLayer


class TreeDecoder:
    def __init__(self, layer: FlatLayer, buckets: Buckets, hierarchy: Hierarchy, beam_width, start_nodes: int | None,
                 page_size: int, growth_buckets: int, splits: int = 16, select_splits: int = 8):
        self.layer, self.buckets, self.hierarchy = layer, buckets, hierarchy
        self.beam_widths = per_level(beam_width, len(hierarchy.node_cluster_block_sizes))
        self.start_nodes, self.page_size, self.growth_buckets, self.splits = start_nodes, page_size, growth_buckets, splits
        self.select_splits = select_splits
        self.plan = None

    def prepare(self, position: int) -> None:
        """Host work of a step, needed again only when the position crosses a cluster block: the levels the query's
        page saw and the open rows each of them scores."""
        device = self.buckets.bucket_centroids.device
        starts, runs = beam_plan(self.hierarchy, self.buckets, [position], self.page_size, self.growth_buckets,
                                 self.start_nodes)
        as_tensor = lambda values: torch.tensor(values, dtype=torch.int32, device=device)
        fresh = dict(start=starts[0], runs=[(as_tensor(first), as_tensor(end)) for first, end in runs],
                     positions=torch.tensor([position], dtype=torch.int64, device=device))
        if self.plan is not None and self.plan["start"] == fresh["start"]:
            # in place: a step captured in a graph reads these tensors, and follows the position (and a tree that
            # grows in fixed-address arrays, `GrowingHierarchy`) without being captured again
            for (first, end), (new_first, new_end) in zip(self.plan["runs"], fresh["runs"]):
                first.copy_(new_first)
                end.copy_(new_end)
            self.plan["positions"].copy_(fresh["positions"])
        else:  # (a new start level walks another number of beam steps: a graph of the step is captured again)
            self.plan = fresh

    def select(self, q: torch.Tensor):
        """q [1, Hq, dh] bf16 -> (list [1, top_k + window + sink] int32, length [1])."""
        d, plan = self.layer.design, self.plan
        with probe.region("index map"):
            index_query = self.layer.index_queries_rows(q)
        carried = None
        with probe.region("beam"):
            for level in range(plan["start"], 0, -1):
                first, end = plan["runs"][level]
                carried = ops.beam_step(index_query, self.hierarchy.node_centroids[level - 1], carried, first, end,
                                        self.beam_widths[level - 1], children=self.hierarchy.children[level - 1],
                                        splits=self.select_splits)
            first, end = plan["runs"][0]
            picked, _ = ops.beam_step(index_query, self.buckets.bucket_centroids, carried, first, end, d.top_p,
                                      splits=self.select_splits)
        with probe.region("expand"):
            lists, lengths, _ = ops.expand(picked, plan["positions"], self.buckets.bucket_members, d.top_k, d.sink_size,
                                           d.window_size)
        return lists, lengths

    def step(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        """One decode step at the prepared position: out [1, Hq, dh] bf16."""
        lists, lengths = self.select(q)
        with probe.region("attend"):
            out, _ = ops.sparse_attend(q, k, v, lists, lengths, self.layer.scale, splits=self.splits)
        return out
