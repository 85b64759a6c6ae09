"""A flat layer over a sequence-sharded KV cache and index: one process a GPU, `torch.distributed` for the two
small exchanges of a step.

Every rank owns a contiguous run of whole cluster blocks: their KV rows, index keys and bucket centroids. Queries
are replicated. A step on rank r:

  1. scores its own centroids, keeps its local top-p as packed keys whose ids are GLOBAL bucket rows;
  2. all-gathers the candidate lists `[world, R, top_p]` and cuts them to the global top-p with the single-GPU tie
     rule (`lsa_merge_candidates`) - every rank ends with the same picks;
  3. expands the picks against the replicated member table (integers, a few MB) but writes only the ids it owns; the
     top-k cut counts every id, so the union over ranks is the single-GPU list;
  4. attends over its own keys and merges: log-sum-exps are all-gathered, each partial output is weighted by
     exp(lse_r - lse) and a reduce-scatter over query rows leaves rank r with its rows of the final output.

The reference replicates the whole index and interleaves KV slots over ranks instead
(`src/lsa/sglang/context_parallel.py:1-24`, `src/lsa/sglang/models/qwen3_5/backend.py:621-781`); the merged
selection and output are the same single-GPU result either way. Nothing here reads a peer's memory from a kernel.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from lsa_b200 import ops, probe
from lsa_b200.core import Buckets
from lsa_b200.layer import FlatIndex, FlatLayer


def shard_blocks(blocks: int, world: int) -> list:
    """Split `blocks` cluster blocks into `world` contiguous runs, the first ranks one longer: [(first, end)]."""
    base, extra = divmod(blocks, world)
    bounds, first = [], 0
    for rank in range(world):
        end = first + base + (1 if rank < extra else 0)
        bounds.append((first, end))
        first = end
    return bounds


def owned_positions(tokens: int, cluster_block_size: int, rank: int, world: int) -> tuple:
    """The positions [first, end) rank owns: its run of whole blocks; the open tail block goes to the last rank."""
    blocks = tokens // cluster_block_size
    first, end = shard_blocks(blocks, world)[rank]
    lo, hi = first * cluster_block_size, end * cluster_block_size
    if rank == world - 1:
        hi = tokens
    return lo, hi


def _all_gather(out: torch.Tensor, piece: torch.Tensor, group=None) -> None:
    """All-gather equal pieces into out[world, ...]: one fused call on NCCL, the list form elsewhere (gloo)."""
    if dist.get_backend(group) == "nccl":
        dist.all_gather_into_tensor(out, piece.contiguous(), group=group)
    else:
        dist.all_gather(list(out.unbind(0)), piece.contiguous(), group=group)


def gather_candidates(keys: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather every rank's packed candidate keys [R, top_p] int64 into [world, R, top_p]."""
    world = dist.get_world_size(group)
    out = torch.empty(world, *keys.shape, dtype=keys.dtype, device=keys.device)
    _all_gather(out, keys, group)
    return out


def merge_weight(lse: torch.Tensor, group=None) -> tuple:
    """This rank's weight exp(lse - LSE) of every (row, head), and the merged LSE, from an all-gather of the
    log-sum-exps. A row nobody read gives weight 0 and LSE -inf."""
    world = dist.get_world_size(group)
    every = torch.empty(world, *lse.shape, dtype=lse.dtype, device=lse.device)
    _all_gather(every, lse, group)
    total = torch.logsumexp(every, dim=0)
    weight = torch.exp(lse - total)
    return torch.where(torch.isfinite(total), weight, torch.zeros_like(weight)), total


def reduce_rows(weighted: torch.Tensor, group=None) -> torch.Tensor:
    """Sum the weighted partial outputs over ranks and leave this rank its rows: [R, ...] -> [R / world, ...].

    NCCL does this with one reduce-scatter; a backend without one (gloo) sums everywhere and slices.
    """
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    rows = weighted.shape[0]
    if rows % world:
        raise ValueError(f"{rows} rows do not split over {world} ranks")
    if dist.get_backend(group) == "nccl":
        out = torch.empty(rows // world, *weighted.shape[1:], dtype=weighted.dtype, device=weighted.device)
        dist.reduce_scatter_tensor(out, weighted.contiguous(), group=group)
        return out
    total = weighted.clone()
    dist.all_reduce(total, group=group)
    return total[rank * (rows // world):(rank + 1) * (rows // world)]


class ShardedFlatLayer:
    """`FlatLayer.prefill` over a cache whose keys, values and buckets are split by sequence across ranks."""

    def __init__(self, layer: FlatLayer, rank: int, world: int, group=None):
        self.layer, self.rank, self.world, self.group = layer, rank, world, group
        self.design = layer.design

    def build_index(self, k_shard: torch.Tensor, tokens: int) -> tuple:
        """Index this rank's blocks and gather the integer tables: (local FlatIndex with global ids, global members).

        `k_shard` holds the rank's own KV rows [hi - lo, Hkv, dh].
        """
        d = self.design
        lo, hi = owned_positions(tokens, d.cluster_block_size, self.rank, self.world)
        local = self.layer.build_index(k_shard[: hi - lo], reuse_buffers=False)
        members = local.buckets.bucket_members
        members = torch.where(members >= 0, members + lo, members)
        blocks = tokens // d.cluster_block_size
        counts = [(end - first) * d.block_bucket_count for first, end in shard_blocks(blocks, self.world)]
        # ranks may hold one block more or less: gather equal-sized (padded) tables, then drop the padding
        widest = max(counts)
        padded = torch.full((widest, d.bucket_cap), -1, dtype=torch.int32, device=members.device)
        padded[: members.shape[0]] = members
        gathered = torch.empty(self.world, widest, d.bucket_cap, dtype=torch.int32, device=members.device)
        with probe.region("gather members"):
            _all_gather(gathered, padded, self.group)
        every_member = torch.cat([gathered[r, :n] for r, n in enumerate(counts)])
        bucket_base = sum(counts[: self.rank])
        index = FlatIndex(local.index_keys, Buckets(local.buckets.bucket_centroids, members,
                                                    local.buckets.bucket_sizes, d.block_bucket_count,
                                                    d.cluster_block_size))
        return index, every_member, bucket_base, (lo, hi)

    def prefill(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, chunk: int = 8192,
                out: torch.Tensor | None = None):
        """Causal prefill of replicated queries q [T, Hq, dh] over this rank's share of k, v (passed whole or as the
        shard's rows). Returns this rank's rows of the output, [T / world / ..] chunk by chunk: out[c] holds rows
        [c*chunk + rank*chunk/world, ...) of chunk c; shape [T // world, Hq, dh] bf16.
        """
        layer, d = self.layer, self.design
        T = q.shape[0]
        lo, hi = owned_positions(T, d.cluster_block_size, self.rank, self.world)
        k_shard = k[lo:hi] if k.shape[0] == T else k
        v_shard = v[lo:hi] if v.shape[0] == T else v
        index, members, bucket_base, _ = self.build_index(k_shard, T)
        centroids = index.buckets.bucket_centroids
        if T % chunk or chunk % self.world:
            raise ValueError(f"{T} tokens must split into chunks of {chunk} rows, and a chunk over {self.world} ranks")
        share = chunk // self.world
        out = torch.empty(T // self.world, q.shape[1], q.shape[2], dtype=q.dtype, device=q.device) if out is None \
            else out
        for c, start in enumerate(range(0, T, chunk)):
            rows = q[start:start + chunk]
            positions = torch.arange(start, start + chunk, device=q.device)
            with probe.region("index map"):
                index_queries = layer.index_queries(rows)
            visible = (positions // d.cluster_block_size * d.block_bucket_count - bucket_base).clamp(
                0, centroids.shape[0]).to(torch.int32)
            with probe.region("select"):
                keys, _ = ops.flat_select(index_queries, centroids, visible, d.top_p, bucket_id_base=bucket_base)
            with probe.region("exchange candidates"):
                every = gather_candidates(keys, self.group)
            with probe.region("select"):
                _, picked = ops.merge_candidates(every)
            with probe.region("expand"):
                lists, lengths, _ = ops.expand(picked, positions, members, d.top_k, d.sink_size, d.window_size,
                                               owner=(lo, hi))
            with probe.region("attend"):
                partial, lse = ops.sparse_attend(rows, k_shard, v_shard, lists, lengths, layer.scale,
                                                 out_dtype=torch.float32, first_slot=lo)
            with probe.region("merge partials"):
                weight, _ = merge_weight(lse, self.group)
                partial *= weight[..., None]
                out[c * share:(c + 1) * share] = reduce_rows(partial, self.group).to(out.dtype)
        return out
