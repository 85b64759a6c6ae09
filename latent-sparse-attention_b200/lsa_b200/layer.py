"""One LSA global-attention layer, flat design: index build, selection and the sparse read strung together.

This is the call a serving backend makes per layer (the reference's `LayerIndex.extend` followed by
`select_and_read`, src/lsa/sglang/index/layer_index.py:824-882 and src/lsa/sglang/models/qwen3_5/backend.py:784-822),
for a single request whose KV rows sit at their positions.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from lsa_b200 import ops, probe
from lsa_b200.budget import EarlyBudget
from lsa_b200.core import Buckets, RotaryLayout, check_sizes


@dataclass(frozen=True)
class FlatDesign:
    """The sizes of a flat design (the reference's `DesignSettings`, src/lsa/sglang/settings/design.py:163-210)."""

    pool_size: int = 4
    bucket_size: int = 8
    bucket_cap: int = 16
    cluster_block_size: int = 512
    top_p: int = 1024
    top_k: int = 4096
    sink_size: int = 4
    window_size: int = 512
    early_budget: EarlyBudget | None = None

    def __post_init__(self) -> None:
        check_sizes(self.pool_size, self.bucket_size, self.bucket_cap, self.cluster_block_size)
        if min(self.top_p, self.top_k, self.window_size) < 1 or self.sink_size < 0:
            raise ValueError("top_p, top_k and window_size must be positive and sink_size non-negative")
        if self.top_p * self.bucket_cap < self.top_k:
            raise ValueError(f"top_p {self.top_p} buckets of at most {self.bucket_cap} keys cannot fill top_k {self.top_k}")

    @property
    def block_bucket_count(self) -> int:
        return self.cluster_block_size // self.bucket_size

    @property
    def list_width(self) -> int:
        return self.top_k + self.window_size + self.sink_size


class FlatIndex:
    """A request's index: its index keys and the buckets of its closed cluster blocks."""

    def __init__(self, index_keys: torch.Tensor, buckets: Buckets):
        self.index_keys = index_keys
        self.buckets = buckets


class FlatLayer:
    """Prefill and decode of one layer. `query_map` / `key_map` are [Hkv * (dh - rotary), index_dim]."""

    def __init__(self, design: FlatDesign, query_map: torch.Tensor, key_map: torch.Tensor, heads: int, kv_heads: int,
                 head_dim: int, rotary: RotaryLayout = RotaryLayout(), scale: float | None = None):
        if heads % kv_heads:
            raise ValueError(f"query heads must group evenly - {heads} does not divide by {kv_heads}")
        free = head_dim - rotary.dim
        if query_map.shape != key_map.shape or query_map.shape[0] != kv_heads * free:
            raise ValueError(f"the maps must both be [{kv_heads * free}, index_dim] - got {tuple(query_map.shape)} "
                             f"and {tuple(key_map.shape)}")
        self.design = design
        self.query_map, self.key_map = query_map.contiguous(), key_map.contiguous()
        self.heads, self.kv_heads, self.head_dim = heads, kv_heads, head_dim
        self.dh_off = rotary.dim if rotary.end == "prefix" else 0
        self.dh_used = free
        self.scale = head_dim ** -0.5 if scale is None else scale

    # ---- the stages

    def index_queries(self, q: torch.Tensor) -> torch.Tensor:
        """q [T, Hq, dh] bf16 -> unit index queries [T, index_dim] fp32."""
        return ops.index_map(q, self.query_map, group=self.heads // self.kv_heads, dh_off=self.dh_off,
                             dh_used=self.dh_used)

    def index_keys(self, k: torch.Tensor) -> torch.Tensor:
        """k [T, Hkv, dh] bf16 -> unit index keys [T, index_dim] fp32."""
        return ops.index_map(k, self.key_map, group=1, dh_off=self.dh_off, dh_used=self.dh_used)

    def build_index(self, k: torch.Tensor) -> FlatIndex:
        """Index keys, then pools, Ward and the bucket table of every closed cluster block."""
        d = self.design
        with probe.region("index map"):
            keys = self.index_keys(k)
        blocks = keys.shape[0] // d.cluster_block_size
        with probe.region("pool"):
            pools = ops.pool_keys(keys[: blocks * d.cluster_block_size].view(blocks, d.cluster_block_size, -1),
                                  d.pool_size)
        with probe.region("ward"):
            labels, _ = ops.ward_rounds(pools, float(d.pool_size), d.block_bucket_count, d.bucket_cap)
        with probe.region("bucket table"):
            members, sizes, _, centroids, _, _ = ops.bucket_table(keys, labels, d.pool_size, d.block_bucket_count,
                                                                 d.bucket_cap)
        return FlatIndex(keys, Buckets(centroids, members, sizes, d.block_bucket_count, d.cluster_block_size))

    def select(self, index_queries: torch.Tensor, positions: torch.Tensor, index: FlatIndex):
        """Read lists [R, top_k + window + sink] int32 and their lengths for queries at `positions`."""
        d, b = self.design, index.buckets
        positions = positions.to(torch.int64)
        visible = (positions // d.cluster_block_size * d.block_bucket_count).clamp_max(
            b.bucket_centroids.shape[0]).to(torch.int32)
        row_p = row_k = None
        if d.early_budget is not None:
            early = positions < d.early_budget.position
            row_p = torch.where(early, d.early_budget.top_p, d.top_p).to(torch.int32)
            row_k = torch.where(early, d.early_budget.top_k, d.top_k).to(torch.int32)
        with probe.region("select"):
            _, picked = ops.flat_select(index_queries, b.bucket_centroids, visible, d.top_p, row_p)
        with probe.region("expand"):
            lists, lengths, _ = ops.expand(picked, positions, b.bucket_members, d.top_k, d.sink_size, d.window_size,
                                           row_p, row_k)
        return lists, lengths

    def attend(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, lists: torch.Tensor, lengths: torch.Tensor,
               splits: int = 1):
        with probe.region("attend"):
            return ops.sparse_attend(q, k, v, lists, lengths, self.scale, splits=splits)

    # ---- the layer

    def prefill(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, chunk: int = 8192,
                return_index: bool = False):
        """Causal prefill from position 0: q [T,Hq,dh], k/v [T,Hkv,dh] bf16 -> out [T,Hq,dh] bf16."""
        T = q.shape[0]
        index = self.build_index(k)
        out = torch.empty_like(q)
        for start in range(0, T, chunk):
            stop = min(T, start + chunk)
            rows = q[start:stop]
            positions = torch.arange(start, stop, device=q.device)
            with probe.region("index map"):
                index_queries = self.index_queries(rows)
            lists, lengths = self.select(index_queries, positions, index)
            out[start:stop], _ = self.attend(rows, k, v, lists, lengths)
        return (out, index) if return_index else out

    def decode(self, q: torch.Tensor, positions: torch.Tensor, k: torch.Tensor, v: torch.Tensor, index: FlatIndex,
               splits: int = 8):
        """One step for rows at `positions` over a cache whose index is built: out [R,Hq,dh] bf16."""
        lists, lengths = self.select(self.index_queries(q), positions, index)
        out, _ = self.attend(q, k, v, lists, lengths, splits=splits)
        return out
