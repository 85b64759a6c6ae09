"""The `lsa.core` operator API on B200 kernels.

Same names, argument meaning, return shapes, padding and error behaviour as the reference's pure-PyTorch
specification (`src/lsa/core/__init__.py:36-56`), with CUDA tensors in and out:

    regroup / regroup_partial / rownorm / project / project_partial / position_free   index_space.py
    pool_keys / ward_rounds / ward_merge / members_from_labels                        ward.py
    Buckets / build_buckets / shape_buckets / read                                    reference.py
    topk_attention                                                                    attention.py

Every function raises `ValueError` naming what arrived where the reference does. Bucket shapes live in
`lsa_b200.shape` (the reference's `lsa.core.shape`); `read` given `shapes` scores a bucket by its estimated best key.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import NamedTuple

import torch

from lsa_b200 import constants as const
from lsa_b200 import ops
from lsa_b200.budget import EarlyBudget

NORM_TOLERANCE = {torch.float32: 1e-4, torch.bfloat16: 2e-2}
CLUSTER_ALGORITHMS = ("ward", "position")


# --------------------------------------------------------------------------------------------- index space


@dataclass(frozen=True)
class RotaryLayout:
    """Where the rotation sits in a head vector, and how many dims it covers (index_space.py:44-59)."""

    end: str = const.Rotary.NONE
    dim: int = 0

    def __post_init__(self) -> None:
        if self.end not in const.Rotary.ENDS:
            raise ValueError(f"end must be one of {const.Rotary.ENDS} - got {self.end!r}")
        if self.dim < 0:
            raise ValueError(f"dim must not be negative - got {self.dim}")
        if (self.end == const.Rotary.NONE) != (self.dim == 0):
            raise ValueError(f"end {self.end!r} and dim {self.dim} disagree about whether there is a rotation")


def position_free(q: torch.Tensor, k: torch.Tensor, rotary: RotaryLayout):
    """Views of the heads with the rotated dims dropped (index_space.py:62-107)."""
    head_dim = q.shape[-1]
    if k.shape[-1] != head_dim:
        raise ValueError(f"q and k must share the head dim - {head_dim} != {k.shape[-1]}")
    if rotary.dim >= head_dim:
        raise ValueError(f"rotation covers the whole head - {rotary.dim} dims of {head_dim}, nothing is position-free")
    if rotary.end == const.Rotary.NONE:
        return q, k
    if rotary.end == const.Rotary.PREFIX:
        return q[..., rotary.dim:], k[..., rotary.dim:]
    return q[..., : head_dim - rotary.dim], k[..., : head_dim - rotary.dim]


def _collapse(x: torch.Tensor, group: int, normalize: bool) -> torch.Tensor:
    """[B, H, T, dh] heads -> [B, T, H/group*dh] fp32, the heads of a group added."""
    batch, heads, tokens, _ = x.shape
    if x.stride(3) != 1:
        x = x.contiguous()
    outs = [ops.index_map(x[b].transpose(0, 1), None, group=group, normalize=normalize) for b in range(batch)]
    return torch.stack(outs) if outs else x.new_zeros(0, tokens, heads // group * x.shape[3], dtype=torch.float32)


def _check_heads(q: torch.Tensor, k: torch.Tensor) -> int:
    if k.shape[0] != q.shape[0]:
        raise ValueError(f"q and k must share the batch size - {q.shape[0]} != {k.shape[0]}")
    if k.shape[3] != q.shape[3]:
        raise ValueError(f"q and k must share the head dim - {q.shape[3]} != {k.shape[3]}")
    if q.shape[1] % k.shape[1]:
        raise ValueError(f"query heads must group evenly - {q.shape[1]} does not divide by {k.shape[1]}")
    return q.shape[1] // k.shape[1]


def regroup_partial(q: torch.Tensor, k: torch.Tensor):
    """Head sum and concatenation without the normalisation (index_space.py:134-187)."""
    group = _check_heads(q, k)
    return _collapse(q, group, False), _collapse(k, 1, False)


def regroup(q: torch.Tensor, k: torch.Tensor):
    """q [B,Hq,Tq,dh], k [B,Hkv,Tk,dh] -> unit rows [B,T,Hkv*dh] fp32 each (index_space.py:110-131)."""
    group = _check_heads(q, k)
    return _collapse(q, group, True), _collapse(k, 1, True)


def rownorm(rows: torch.Tensor, eps: float = const.Math.NORM_EPS) -> torch.Tensor:
    """Unit rows in fp32, a zero row left at zero (index_space.py:315-334)."""
    if eps != const.Math.NORM_EPS:
        raise ValueError(f"the kernels normalise with a floor of {const.Math.NORM_EPS} - got {eps}")
    flat = rows.reshape(-1, 1, rows.shape[-1])
    return ops.index_map(flat, None, normalize=True).reshape(rows.shape)


def project_partial(rows: torch.Tensor, index_map: torch.Tensor) -> torch.Tensor:
    """rows @ map in fp32, not normalised (index_space.py:378-402)."""
    if rows.shape[-1] != index_map.shape[0]:
        raise ValueError(f"rows have {rows.shape[-1]} dims and the map reads {index_map.shape[0]}")
    flat = rows.reshape(-1, 1, rows.shape[-1])
    return ops.index_map(flat, index_map, normalize=False).reshape(*rows.shape[:-1], index_map.shape[1])


def project(rows: torch.Tensor, index_map: torch.Tensor) -> torch.Tensor:
    """normalize(rows @ map) (index_space.py:405-419)."""
    if rows.shape[-1] != index_map.shape[0]:
        raise ValueError(f"rows have {rows.shape[-1]} dims and the map reads {index_map.shape[0]}")
    flat = rows.reshape(-1, 1, rows.shape[-1])
    return ops.index_map(flat, index_map, normalize=True).reshape(*rows.shape[:-1], index_map.shape[1])


@dataclass(frozen=True)
class LearnedProjection:
    """The query and key maps of one layer, both [Hkv*dh, index_dim] (index_space.py:337-375)."""

    query_projection: torch.Tensor
    key_projection: torch.Tensor

    def __post_init__(self) -> None:
        if self.query_projection.ndim != 2 or self.key_projection.ndim != 2:
            raise ValueError(f"both projections must be [Hkv * dh, index_dim] - got "
                             f"{tuple(self.query_projection.shape)} and {tuple(self.key_projection.shape)}")
        if self.query_projection.shape != self.key_projection.shape:
            raise ValueError(f"the projections must share their shape - {tuple(self.query_projection.shape)} "
                             f"!= {tuple(self.key_projection.shape)}")

    @property
    def index_dim(self) -> int:
        return int(self.key_projection.shape[1])


@dataclass(frozen=True)
class LatentMetric:
    """An MLA layer's key maps [Hq, dh, r] and the lower Cholesky factor [r, r] fp32 of the metric they impose on the
    latent, `L L^T = sum_h W_h^T W_h` (index_space.py:190-268). `L^T latent` has the lengths and angles the
    concatenated per-head keys have, so a selection made on it is the one made on them, at r dims."""

    key_maps: torch.Tensor
    metric_factor: torch.Tensor

    def __post_init__(self) -> None:
        if self.key_maps.ndim != 3:
            raise ValueError(f"key_maps must be [Hq, dh, r] - got {tuple(self.key_maps.shape)}")
        rank = self.key_maps.shape[2]
        if self.metric_factor.shape != (rank, rank):
            raise ValueError(f"metric_factor must be [{rank}, {rank}] to match the key maps - "
                             f"got {tuple(self.metric_factor.shape)}")

    @property
    def dim(self) -> int:
        return int(self.key_maps.shape[2])

    @classmethod
    def from_key_maps(cls, key_maps: torch.Tensor) -> "LatentMetric":
        """Factor the metric in fp64 (a layer's one-time setup; the factorisation is torch's).

        Raises:
            ValueError: `key_maps` is not `[Hq, dh, r]`, or the maps do not span the latent.
        """
        if key_maps.ndim != 3:
            raise ValueError(f"key_maps must be [Hq, dh, r] - got {tuple(key_maps.shape)}")
        metric = torch.einsum("hdr,hde->re", key_maps.double(), key_maps.double())
        factored = torch.linalg.cholesky_ex(metric)
        if int(factored.info) != 0:
            raise ValueError(f"the key maps do not span the {key_maps.shape[2]}-dim latent - "
                             "the metric they impose on it is singular and cannot be factored")
        return cls(key_maps, factored.L.float())

    def maps(self) -> tuple[torch.Tensor, torch.Tensor]:
        """The two linear maps `regroup_latent` amounts to, fp32 from fp64: queries [Hq*dh] -> r through `W L^-T`
        (every head's key map pulled onto the query side, then `L^-1`), latents r -> r through `L`."""
        wide = self.key_maps.double().reshape(-1, self.dim)
        query_map = torch.linalg.solve_triangular(self.metric_factor.double(), wide.t(), upper=False).t()
        return query_map.float().contiguous(), self.metric_factor.float().contiguous()


def regroup_latent(q: torch.Tensor, latent: torch.Tensor, metric: LatentMetric):
    """q [B,Hq,Tq,dh], latent [B,Tk,r] -> unit rows [B,Tq,r] and [B,Tk,r] fp32 (index_space.py:271-312), the keys
    never expanded: both sides are one pass of the index map kernel, the triangular solve folded into the query map.

    Raises:
        ValueError: `q` or `latent` does not match the key maps.
    """
    head_count, head_dim, rank = metric.key_maps.shape
    if q.ndim != 4 or q.shape[1] != head_count or q.shape[3] != head_dim:
        raise ValueError(f"q must be [B, {head_count}, Tq, {head_dim}] to match the key maps - got {tuple(q.shape)}")
    if latent.ndim != 3 or latent.shape[2] != rank:
        raise ValueError(f"latent must be [B, Tk, {rank}] to match the key maps - got {tuple(latent.shape)}")
    query_map, key_map = metric.maps()
    if q.stride(3) != 1:
        q = q.contiguous()
    queries = [ops.index_map(q[b].transpose(0, 1), query_map) for b in range(q.shape[0])]
    keys = ops.index_map(latent.reshape(-1, 1, rank), key_map).reshape(latent.shape)
    index_queries = torch.stack(queries) if queries else q.new_zeros(0, q.shape[2], rank, dtype=torch.float32)
    return index_queries, keys


# --------------------------------------------------------------------------------------------- Ward


def pool_keys(index_keys: torch.Tensor, pool_size: int) -> torch.Tensor:
    """[G, T, d] -> [G, T/pool_size, d] fp32 (ward.py:15-26)."""
    return ops.pool_keys(index_keys, pool_size)


def ward_rounds(pool_keys: torch.Tensor, pool_sizes: torch.Tensor, bucket_count: int, bucket_cap: int,
                max_rounds: int = 256):
    """Labels [G, P] int64 and whether each block reached its count (ward.py:29-90)."""
    return ops.ward_rounds(pool_keys, pool_sizes, bucket_count, bucket_cap, max_rounds)


def ward_merge(pool_keys: torch.Tensor, pool_sizes: torch.Tensor, bucket_count: int, bucket_cap: int):
    """Merge down to exactly `bucket_count` buckets, or refuse (ward.py:93-125)."""
    bucket_size = pool_sizes.sum(1).max().item() / bucket_count
    if bucket_cap < 2 * bucket_size:
        raise ValueError(
            f"the bucket cap must be at least twice the bucket size, {2 * bucket_size:g} - got {bucket_cap}")
    labels, reached = ward_rounds(pool_keys, pool_sizes, bucket_count, bucket_cap)
    if not reached.all():
        raise ValueError(f"{int((~reached).sum())} blocks stopped short of {bucket_count} buckets under the cap")
    return labels


def members_from_labels(labels: torch.Tensor, bucket_count: int, bucket_cap: int) -> torch.Tensor:
    """Each bucket's keys in position order from the bucket of every key (ward.py:128-143)."""
    members, _ = ops.bucket_members(labels.reshape(1, -1).to(torch.int64), 1, bucket_count, bucket_cap)
    return members


# --------------------------------------------------------------------------------------------- flat


class Buckets(NamedTuple):
    """The buckets of a cache's closed cluster blocks, block after block (reference.py:27-39)."""

    bucket_centroids: torch.Tensor  # [rows, index_dim] fp32
    bucket_members: torch.Tensor  # [rows, bucket_cap] int32, -1 padded
    bucket_sizes: torch.Tensor  # [rows] int32
    block_bucket_count: int
    cluster_block_size: int


def check_unit_rows(name: str, vectors: torch.Tensor) -> None:
    """Refuse vectors that are not a float matrix of unit rows (reference.py:42-60). One host read."""
    if vectors.dim() != 2:
        raise ValueError(f"{name} must be [N, index_dim] - got shape {tuple(vectors.shape)}")
    if vectors.dtype not in NORM_TOLERANCE:
        raise ValueError(f"{name} must be float32 or bfloat16 - got {vectors.dtype}")
    if not vectors.numel():
        return
    norms = vectors.float().norm(dim=1)
    finite, off = torch.stack([vectors.isfinite().all().float(), (norms - 1).abs().max().nan_to_num(0.0)]).tolist()
    if not finite:
        raise ValueError(f"{name} holds a non-finite value")
    if off > NORM_TOLERANCE[vectors.dtype]:
        raise ValueError(f"{name} must be unit rows - a row is {off:.3g} off unit length")


def check_sizes(pool_size: int, bucket_size: int, bucket_cap: int, cluster_block_size: int) -> None:
    """Refuse sizes that do not nest, or a cap under twice the bucket size (reference.py:63-84)."""
    if min(pool_size, bucket_size, bucket_cap, cluster_block_size) < 1:
        raise ValueError("pool_size, bucket_size, bucket_cap and cluster_block_size must be positive")
    if bucket_size % pool_size or cluster_block_size % bucket_size:
        raise ValueError(f"pool_size {pool_size} must divide bucket_size {bucket_size}, which must divide "
                         f"cluster_block_size {cluster_block_size}")
    if bucket_cap < 2 * bucket_size:
        raise ValueError(f"bucket_cap must be at least twice bucket_size {bucket_size} - got {bucket_cap}")


def build_buckets(index_keys: torch.Tensor, pool_size: int, bucket_size: int, bucket_cap: int,
                  cluster_block_size: int, cluster_algorithm: str = "ward") -> Buckets:
    """Cluster every closed cluster block of the index keys into buckets (reference.py:87-144)."""
    check_unit_rows("index_keys", index_keys)
    check_sizes(pool_size, bucket_size, bucket_cap, cluster_block_size)
    if cluster_algorithm not in CLUSTER_ALGORITHMS:
        raise ValueError(f"cluster_algorithm must be one of {CLUSTER_ALGORITHMS} - got {cluster_algorithm!r}")
    keys = index_keys.contiguous()
    blocks = keys.shape[0] // cluster_block_size
    per_block = cluster_block_size // bucket_size
    pools_a_block = cluster_block_size // pool_size
    if cluster_algorithm == "position":
        labels = (torch.arange(pools_a_block, device=keys.device) // (bucket_size // pool_size)).expand(blocks, -1)
        labels = labels.contiguous()
    else:
        pools = ops.pool_keys(keys[: blocks * cluster_block_size].view(blocks, cluster_block_size, -1), pool_size)
        labels, reached = ops.ward_rounds(pools, float(pool_size), per_block, bucket_cap)
        if blocks and not reached.all():
            raise ValueError(f"{int((~reached).sum())} blocks stopped short of {per_block} buckets under the cap")
    members, sizes, _, centroids, _, _ = ops.bucket_table(keys, labels, pool_size, per_block, bucket_cap)
    return Buckets(centroids, members, sizes, per_block, cluster_block_size)


def shape_buckets(index_keys: torch.Tensor, buckets: Buckets, rank: int):
    """Give every bucket its shape: its keys' spread about its centroid, kept as `rank` sign directions
    (reference.py:147-164). Returns `shape.Shapes`, row for row with the buckets."""
    from lsa_b200 import shape

    check_unit_rows("index_keys", index_keys)
    if not 0 <= rank <= index_keys.shape[1]:
        raise ValueError(f"rank must be from 0 to the keys' width {index_keys.shape[1]} - got {rank}")
    return shape.build_shapes(index_keys, buckets.bucket_centroids, buckets.bucket_members, rank)


def check_read_arguments(index_queries, positions, buckets, top_p, top_k, sink_size, window_size,
                         early_budget=None) -> None:
    """The refusals of `read` (reference.py:209-224): unit rows of the buckets' dim, one non-negative integer
    position a query, positive sizes, an early budget within the read's own."""
    check_unit_rows("index_queries", index_queries)
    if index_queries.shape[1] != buckets.bucket_centroids.shape[1]:
        raise ValueError(
            f"index_queries have {index_queries.shape[1]} dims and the buckets {buckets.bucket_centroids.shape[1]}")
    if positions.dtype not in (torch.int32, torch.int64) or positions.shape != (index_queries.shape[0],):
        raise ValueError("positions must be an int32 or int64 vector, one a query")
    if positions.numel() and positions.min() < 0:
        raise ValueError("positions must be non-negative")
    if min(top_p, top_k, window_size) < 1 or sink_size < 0:
        raise ValueError("top_p, top_k and window_size must be positive and sink_size non-negative")
    if early_budget is not None and (early_budget.top_p > top_p or early_budget.top_k > top_k):
        raise ValueError(f"the early budget is at most top_p {top_p} and top_k {top_k} - "
                         f"got top_p {early_budget.top_p} and top_k {early_budget.top_k}")


def read(index_queries: torch.Tensor, positions: torch.Tensor, buckets: Buckets, top_p: int, top_k: int,
         sink_size: int, window_size: int, shapes=None, deviations: float = 0.0,
         early_budget: EarlyBudget | None = None):
    """Select the keys each query reads: score, pick the top_p buckets, expand (reference.py:167-236).

    Returns selected ids [Tq, top_k + window + sink] int32 (-1 padded; expansion, window, sinks) and lengths [Tq].
    """
    check_read_arguments(index_queries, positions, buckets, top_p, top_k, sink_size, window_size, early_budget)
    positions = positions.to(torch.int64)
    visible = (positions // buckets.cluster_block_size * buckets.block_bucket_count).clamp_max(
        buckets.bucket_centroids.shape[0]).to(torch.int32)
    row_p = row_k = None
    if early_budget is not None:
        early = positions < early_budget.position
        row_p = torch.where(early, early_budget.top_p, top_p).to(torch.int32)
        row_k = torch.where(early, early_budget.top_k, top_k).to(torch.int32)
    if shapes is not None:  # a bucket scores as its estimated best key (reference.py:229-230)
        from lsa_b200 import shape

        if shapes.floor.shape[0] != buckets.bucket_centroids.shape[0]:
            raise ValueError(f"shapes hold {shapes.floor.shape[0]} buckets and the table "
                             f"{buckets.bucket_centroids.shape[0]}")
        _, picked = ops.shaped_select(index_queries, buckets.bucket_centroids, shape.table(shapes, deviations),
                                      visible, top_p, row_p)
    else:
        _, picked = ops.flat_select(index_queries, buckets.bucket_centroids, visible, top_p, row_p)
    selected, lengths, _ = ops.expand(picked, positions, buckets.bucket_members, top_k, sink_size, window_size,
                                      row_p, row_k)
    return selected, lengths


# --------------------------------------------------------------------------------------------- attention


def compose_lists(selected: torch.Tensor, positions: torch.Tensor, window: int, sink: int):
    """A row's keep-set as a list of distinct ids, valid entries first: its selected ids that are causal, its
    window and its sinks (the set `keep_set` builds as a mask, attention.py:15-62). The order within a row is
    ascending; attention over a set does not depend on it."""
    rows = selected.shape[0]
    pos = positions.to(torch.int64)[:, None]
    none = 2**40
    ids = selected.to(torch.int64)
    ids = torch.where((ids >= 0) & (ids <= pos), ids, none)
    recent = pos - torch.arange(max(window, 0), device=selected.device)[None, :]
    recent = torch.where(recent >= 0, recent, none)
    first = torch.arange(sink, device=selected.device)[None, :].expand(rows, -1)
    first = torch.where(first <= pos, first, none)
    ids, _ = torch.cat([ids, recent, first], dim=1).sort(dim=1)
    again = torch.zeros_like(ids, dtype=torch.bool)
    again[:, 1:] = ids[:, 1:] == ids[:, :-1]
    ids, _ = torch.where(again, none, ids).sort(dim=1)
    lengths = (ids < none).sum(1)
    return torch.where(ids < none, ids, -1).to(torch.int32), lengths.to(torch.int32)


def topk_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, selected_key_ids: torch.Tensor, window: int,
                   sink: int, scale: float, query_start: int = 0, query_block_size: int = const.Chunk.QUERY):
    """Causal attention over the window, sinks and selected keys (attention.py:65-146).

    q [B,Tq,Hq,Dh], k/v [B,Tk,Hkv,Dh], selected [B,Tq,budget] int32 with -1 padding. Inputs are read as bf16,
    logits and softmax are fp32, the output has q's dtype. `query_block_size` only bounds the rows a launch takes.
    """
    batch, rows, heads, head_dim = q.shape
    out = torch.empty_like(q)
    positions = query_start + torch.arange(rows, device=q.device)
    for b in range(batch):
        kb, vb = k[b].to(torch.bfloat16).contiguous(), v[b].to(torch.bfloat16).contiguous()
        lists, lengths = compose_lists(selected_key_ids[b], positions, window, sink)
        res, _ = ops.sparse_attend(q[b].to(torch.bfloat16).contiguous(), kb, vb, lists, lengths, scale,
                                   out_dtype=torch.float32)
        out[b] = res.to(q.dtype)
    return out


# The hierarchy's half of the operator API lives in its own module; it is re-exported here so that
# `from lsa_b200.core import build_hierarchy, read_hierarchy` reads as the reference's `lsa.core` does.
from lsa_b200.hierarchy import (Hierarchy, build_hierarchy, growth_at, pair_into_node_buckets,  # noqa: E402,F401
                                read_hierarchy, read_hierarchy_counted)
