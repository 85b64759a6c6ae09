"""The settings block `"lsa": {...}` of a model config, parsed into frozen dataclasses that refuse unknown keys and
combinations the kernels cannot run (the reference's `IndexerConfig` / `ServingChoices`,
`src/lsa/sglang/settings/design.py:163-285,586-607`)."""

from __future__ import annotations

from collections.abc import Mapping
from dataclasses import dataclass, fields
from typing import Any

from lsa_b200.budget import EarlyBudget
from lsa_b200.layer import FlatDesign
from lsa_b200.shape import Shape

BLOCK = "lsa"
PAGE_SIZE = 8192  # keys a page of the bucket cache holds: where a prefill segment is cut and a tree grows
TOPK_LIMIT = 2048
KERNELS = ("b200",)
# Longest contexts a decode CUDA graph is captured for, ascending: a batch replays the graph of the first limit its
# longest request fits under, and the full-context graph beyond the last (design.py:46-52: 18 pages times a power of
# two, so that a request at a power of two plus its answer sits high in its range)
DECODE_CONTEXT_LIMITS = tuple(18 * PAGE_SIZE * 2 ** i for i in range(7))
DECODES = ("flat", "descend")


@dataclass(frozen=True)
class IndexerConfig:
    """What a design is (design.py:163-210). The cluster block size is `window_size`."""

    window_size: int = 512
    sink_size: int = 4
    top_k: int = 4096
    top_p: int = 1024
    index_dim: int = 64
    pool_size: int | None = 4
    bucket_size: int = 8
    bucket_cap: int = 16
    top_level: int = 0
    node_bucket_size: int | None = None
    node_cluster_block_size: int | None = None
    beam_width: int | None = None
    start_nodes: int | None = None
    early_budget: EarlyBudget | None = None
    bucket_shape: Shape | None = None  # buckets keep their spread and score as their estimated best key
    node_bucket_shape: Shape | None = None  # the same for the node buckets of a tree

    def __post_init__(self) -> None:
        pool = self.pool_size or 1
        for name in ("window_size", "top_k", "top_p", "index_dim", "bucket_size", "bucket_cap"):
            value = getattr(self, name)
            if isinstance(value, bool) or not isinstance(value, int) or value < 1:
                raise ValueError(f"{name} must be a positive integer - got {value!r}")
        if self.sink_size < 0:
            raise ValueError(f"sink_size must not be negative - got {self.sink_size}")
        if self.bucket_size % pool or self.window_size % self.bucket_size:
            raise ValueError(f"pool_size {pool} must divide bucket_size {self.bucket_size}, which must divide "
                             f"window_size {self.window_size}")
        if self.bucket_cap < 2 * self.bucket_size:
            raise ValueError(f"bucket_cap must be at least twice bucket_size {self.bucket_size} - got {self.bucket_cap}")
        if PAGE_SIZE % self.window_size:
            raise ValueError(f"window_size {self.window_size} must divide the cache page of {PAGE_SIZE} keys")
        if self.top_p > TOPK_LIMIT:
            raise ValueError(f"top_p is at most {TOPK_LIMIT} - got {self.top_p}")
        if self.top_p * self.bucket_cap < self.top_k:
            raise ValueError(f"top_p {self.top_p} buckets of at most {self.bucket_cap} keys cannot fill top_k {self.top_k}")
        tree = (self.node_bucket_size, self.node_cluster_block_size, self.beam_width)
        if (self.top_level >= 1) != all(value is not None for value in tree) or \
                (self.top_level < 1 and any(value is not None for value in tree)):
            raise ValueError("node_bucket_size, node_cluster_block_size and beam_width are set exactly when "
                             "top_level is 1 or more")
        self.check_shapes()
        if self.early_budget is not None:
            if self.top_level:
                raise ValueError("an early budget is flat only")
            if self.early_budget.top_p > self.top_p or self.early_budget.top_k > self.top_k:
                raise ValueError("the early budget is at most the design's top_p and top_k")

    def check_shapes(self) -> None:
        """Build the shape knobs from their mappings and refuse a shape the design cannot hold (design.py:317-345).

        Raises:
            ValueError: A shape is refused, keeps more directions than `index_dim` (or than `bucket_cap`, the most
                keys a bucket holds), `index_dim` is not a multiple of 32 (a basis is read a word at a time), or
                `node_bucket_shape` is set: node buckets are not shaped here.
        """
        for name in ("bucket_shape", "node_bucket_shape"):
            shape = Shape.read(name, getattr(self, name))
            object.__setattr__(self, name, shape)
            if shape is None:
                continue
            if shape.rank > self.index_dim:
                raise ValueError(f"{name} keeps at most index_dim {self.index_dim} directions - got rank {shape.rank}")
            if self.index_dim % 32:
                raise ValueError(f"a shaped design needs index_dim a multiple of 32 - got {self.index_dim}")
        if self.bucket_shape is not None and self.bucket_shape.rank > self.bucket_cap:
            raise ValueError(f"bucket_shape keeps at most bucket_cap {self.bucket_cap} directions - got rank "
                             f"{self.bucket_shape.rank}")
        if self.node_bucket_shape is not None:
            if self.top_level < 1:
                raise ValueError("node_bucket_shape is set with top_level 0, where there are no node buckets")
            raise ValueError("node_bucket_shape is not served: this build shapes the buckets of a flat design only")

    @property
    def width(self) -> int:
        """Columns of a read list."""
        return self.top_k + self.window_size + self.sink_size

    def flat_design(self) -> FlatDesign:
        return FlatDesign(pool_size=self.pool_size or 1, bucket_size=self.bucket_size, bucket_cap=self.bucket_cap,
                          cluster_block_size=self.window_size, top_p=self.top_p, top_k=self.top_k,
                          sink_size=self.sink_size, window_size=self.window_size, early_budget=self.early_budget,
                          bucket_shape=self.bucket_shape)


@dataclass(frozen=True)
class ServingChoices:
    """How a design is served (design.py:586-607)."""

    projections: str | None = None  # the map file: `<layer>.W_Q_idx` / `<layer>.W_K_idx` tensors
    decode: str = "flat"
    kernels: str = "b200"
    # Contexts a flat decode captures a CUDA graph for besides the server's own, ascending - empty captures one
    decode_context_limits: tuple = DECODE_CONTEXT_LIMITS
    # Take a cached prefix's index where the server caches prefixes, rather than build it again - opt-in
    prefix_reuse: bool = False
    # Full contexts the bucket cache holds beyond the KV pool's pages: requests that share a cached prefix in the pool
    # and not in the index are not bounded by the pool's size
    spare_contexts: int = 0

    def __post_init__(self) -> None:
        if self.decode not in DECODES:
            raise ValueError(f"decode must be one of {DECODES} - got {self.decode!r}")
        if self.kernels not in KERNELS:
            raise ValueError(f"kernels must be one of {KERNELS} - got {self.kernels!r}")
        limits = tuple(self.decode_context_limits)
        object.__setattr__(self, "decode_context_limits", limits)
        for limit in limits:
            if isinstance(limit, bool) or not isinstance(limit, int) or limit < PAGE_SIZE:
                raise ValueError(f"decode_context_limits are integers of at least a page of {PAGE_SIZE} keys - got "
                                 f"{limit!r}")
        if list(limits) != sorted(set(limits)):
            raise ValueError(f"decode_context_limits must be ascending and distinct - got {list(limits)}")
        if not isinstance(self.prefix_reuse, bool):
            raise ValueError(f"prefix_reuse is true or false - got {self.prefix_reuse!r}")
        if isinstance(self.spare_contexts, bool) or not isinstance(self.spare_contexts, int) or self.spare_contexts < 0:
            raise ValueError(f"spare_contexts must be a whole number - got {self.spare_contexts!r}")


@dataclass(frozen=True)
class DesignSettings:
    indexer: IndexerConfig
    serving: ServingChoices

    @property
    def width(self) -> int:
        return self.indexer.width

    @property
    def early_width(self) -> int | None:
        early = self.indexer.early_budget
        return None if early is None else early.top_k + self.indexer.window_size + self.indexer.sink_size


def _build(cls, block: Mapping[str, Any] | None, where: str):
    block = dict(block or {})
    known = {item.name for item in fields(cls)}
    unknown = sorted(set(block) - known)
    if unknown:
        raise ValueError(f"{where} has no key {unknown} - it takes {sorted(known)}")
    if "early_budget" in block:
        block["early_budget"] = EarlyBudget.read(block["early_budget"])
    return cls(**block)


def parse(block: Mapping[str, Any]) -> DesignSettings:
    """Parse the `"lsa"` block: `{"indexer": {...}, "serving": {...}}`. Unknown keys are refused."""
    if not isinstance(block, Mapping):
        raise ValueError(f"the {BLOCK!r} block must be a mapping - got {block!r}")
    unknown = sorted(set(block) - {"indexer", "serving"})
    if unknown:
        raise ValueError(f"the {BLOCK!r} block has no key {unknown} - it takes ['indexer', 'serving']")
    design = DesignSettings(_build(IndexerConfig, block.get("indexer"), "lsa.indexer"),
                            _build(ServingChoices, block.get("serving"), "lsa.serving"))
    if design.serving.decode == "descend" and design.indexer.top_level < 1:
        raise ValueError("decode: descend needs a design with top_level 1 or more")
    return design
