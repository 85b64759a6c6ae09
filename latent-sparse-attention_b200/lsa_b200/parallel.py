"""A flat layer over a sequence-sharded KV cache and index: one process a GPU, `torch.distributed` for the small
exchanges of a step.

What is split, and how:

  KV rows      dealt out round-robin in granules of `granule` positions (64): position p lives on rank
               (p / granule) % world, at row p / (granule*world) * granule + p % granule of that rank's cache. A
               query's window and the members of its buckets are runs of consecutive positions, so every rank
               holds an even share of every query's keys - a causal prefill stays balanced from the first chunk on.
  buckets      cluster blocks are dealt out round-robin too: rank r clusters and scores blocks r, r + world, ...
  index keys   each rank maps the keys it holds; one all-gather puts all index keys (64 floats a token) on every
               rank, which is what clustering a whole block needs.
  member table integers, a few MB: all-gathered once after the build, so every rank can expand any pick.
  queries      replicated.

A step on rank r: score its own centroids -> local top-p as packed keys with GLOBAL bucket ids -> all-gather the
candidates and cut them to the global top-p with the single-GPU tie rule (`lsa_merge_candidates`), so every rank
holds the same picks -> expand them, writing only the rows this rank holds (the top-k cut counts every id) -> attend
over its own rows -> all-gather the log-sum-exps, weight the partial output by exp(lse_r - lse), reduce-scatter over
query rows. The union of the ranks' lists is the single-GPU list and the merged output the single-GPU output.

That is `prefill`, the context-parallel form, and the only way to split a decode step. A prefill reads almost the
whole cache from every row, so `prefill_by_rows` splits the QUERY ROWS instead: the shares of K, V and the index are
all-gathered once a step and every rank runs the single-GPU read (dense band, bucket-major expansion) over its own
rows of every chunk; nothing is merged.

The reference replicates the whole index and interleaves single KV slots over ranks
(`src/lsa/sglang/context_parallel.py:1-24`, `src/lsa/sglang/models/qwen3_5/backend.py:621-781`). No kernel here reads
a peer's memory; gathered data lands in local memory through the collective first.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from lsa_b200 import ops, probe
from lsa_b200.layer import FlatLayer

GRANULE = 64  # positions a rank holds in a row before the next rank's turn


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
    """The positions [first, end) of a CONTIGUOUS split by whole blocks; the open tail block goes to the last rank."""
    blocks = tokens // cluster_block_size
    first, end = shard_blocks(blocks, world)[rank]
    lo, hi = first * cluster_block_size, end * cluster_block_size
    if rank == world - 1:
        hi = tokens
    return lo, hi


def deal(rows: torch.Tensor, rank: int, world: int, granule: int = GRANULE) -> torch.Tensor:
    """A rank's share of [T, ...] rows dealt out round-robin in granules: [T / world, ...]."""
    T = rows.shape[0]
    if T % (granule * world):
        raise ValueError(f"{T} rows do not deal out in granules of {granule} over {world} ranks")
    return rows.view(T // (granule * world), world, granule, *rows.shape[1:])[:, rank].reshape(
        T // world, *rows.shape[1:])


def undeal(every: torch.Tensor, granule: int = GRANULE) -> torch.Tensor:
    """The inverse for all ranks' shares at once: [world, T / world, ...] -> [T, ...] in position order."""
    world, share = every.shape[0], every.shape[1]
    return every.view(world, share // granule, granule, *every.shape[2:]).transpose(0, 1).reshape(
        world * share, *every.shape[2:])


def _all_gather(out: torch.Tensor, piece: torch.Tensor, group=None) -> None:
    """All-gather equal pieces into out[world, ...]: one fused call on NCCL, the list form elsewhere (gloo)."""
    if dist.get_backend(group) == "nccl":
        dist.all_gather_into_tensor(out, piece.contiguous(), group=group)
    else:
        dist.all_gather(list(out.unbind(0)), piece.contiguous(), group=group)


def gather_pieces(piece: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather one equal-shaped tensor a rank into [world, ...]."""
    out = torch.empty(dist.get_world_size(group), *piece.shape, dtype=piece.dtype, device=piece.device)
    _all_gather(out, piece, group)
    return out


def gather_candidates(keys: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather every rank's packed candidate keys [R, top_p] int64 into [world, R, top_p]."""
    return gather_pieces(keys, group)


def globalise_keys(keys: torch.Tensor, per_block: int, rank: int, world: int) -> torch.Tensor:
    """Packed keys over a rank's OWN bucket rows -> the same keys over global bucket rows, when cluster blocks are
    dealt out round-robin: local row l is global row (l / per_block * world + rank) * per_block + l % per_block.
    The map is increasing, so a tie broken toward the lower local row is broken toward the lower global row."""
    empty = keys == torch.iinfo(torch.int64).min
    local = 0x7FFFFFFF - (keys & 0xFFFFFFFF)
    wide = (local // per_block * world + rank) * per_block + local % per_block
    out = (keys & ~0xFFFFFFFF) | (0x7FFFFFFF - wide)
    return torch.where(empty, keys, out)


def merge_weight(lse: torch.Tensor, group=None) -> tuple:
    """This rank's weight exp(lse - LSE) of every (row, head), and the merged LSE, from an all-gather of the
    log-sum-exps. A row nobody read gives weight 0 and LSE -inf."""
    every = gather_pieces(lse, group)
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
    """`FlatLayer.prefill` over a cache whose keys, values and buckets are dealt out across ranks."""

    def __init__(self, layer: FlatLayer, rank: int, world: int, group=None, granule: int = GRANULE):
        self.layer, self.rank, self.world, self.group, self.granule = layer, rank, world, group, granule
        self.design = layer.design

    def build_index(self, k_share: torch.Tensor, tokens: int):
        """From this rank's dealt keys [tokens / world, Hkv, dh]: its own centroids, the global member table, and
        every index key."""
        d, layer, world, rank = self.design, self.layer, self.world, self.rank
        blocks = tokens // d.cluster_block_size
        if tokens % d.cluster_block_size or blocks % world:
            raise ValueError(f"{tokens} tokens must be whole cluster blocks of {d.cluster_block_size}, a multiple of "
                             f"{world} of them")
        with probe.region("index map"):
            own_keys = layer.index_keys(k_share)
        with probe.region("gather index keys"):
            index_keys = undeal(gather_pieces(own_keys, self.group), self.granule)
        # this rank's blocks: r, r + world, ...
        mine = index_keys.view(blocks // world, world, d.cluster_block_size, -1)[:, rank].contiguous()
        per_block, block = d.block_bucket_count, d.cluster_block_size
        with probe.region("pool"):
            pools = ops.pool_keys(mine, d.pool_size)
        with probe.region("ward"):
            labels, _ = ops.ward_rounds(pools, float(d.pool_size), per_block, d.bucket_cap)
        with probe.region("bucket table"):
            members, _, _, centroids, _, _ = ops.bucket_table(mine.view(-1, mine.shape[-1]), labels, d.pool_size,
                                                              per_block, d.bucket_cap)
            # positions inside this rank's run of blocks -> positions in the sequence
            members = torch.where(members >= 0, members // block * (world * block) + rank * block + members % block,
                                  members)
        with probe.region("gather members"):
            every = gather_pieces(members, self.group)  # [world, blocks / world * per_block, cap]
            table = every.view(world, blocks // world, per_block, d.bucket_cap).transpose(0, 1).reshape(
                blocks * per_block, d.bucket_cap)
        return centroids, table, index_keys

    def rows_of(self, q: torch.Tensor, chunk: int) -> torch.Tensor:
        """This rank's query rows of q [T, ...]: rows [c*chunk + rank*chunk/world, c*chunk + (rank+1)*chunk/world)
        of every chunk c, [T / world, ...] - the rows whose output `prefill` leaves on this rank."""
        share = chunk // self.world
        return q.view(q.shape[0] // chunk, self.world, share, *q.shape[1:])[:, self.rank].reshape(
            q.shape[0] // self.world, *q.shape[1:])

    def prefill_by_rows(self, q: torch.Tensor, k_share: torch.Tensor, v_share: torch.Tensor, tokens: int,
                        chunk: int = 8192, out: torch.Tensor | None = None):
        """Causal prefill with the QUERY ROWS split over the ranks: the cache stays dealt out for storage, but a
        prefill reads almost all of it from every row, so the shares are all-gathered once (K, V and the index - the
        one exchange of the step) and every rank then runs the single-GPU read - dense band, bucket-major expansion -
        over its own rows of every chunk. No partial outputs cross ranks and nothing is merged.

        q holds this rank's rows (`rows_of`), [tokens / world, Hq, dh], or all rows [tokens, Hq, dh]; the result is
        this rank's rows, as `prefill` returns them.
        """
        layer, d, world, rank = self.layer, self.design, self.world, self.rank
        if tokens % chunk or chunk % world:
            raise ValueError(f"{tokens} tokens must split into chunks of {chunk} rows, and a chunk over {world} ranks")
        from lsa_b200.core import Buckets
        from lsa_b200.layer import FlatIndex

        if q.shape[0] == tokens:
            q = self.rows_of(q, chunk)
        own_centroids, members, index_keys = self.build_index(k_share, tokens)
        blocks, per_block = tokens // d.cluster_block_size, d.block_bucket_count
        with probe.region("gather cache"):
            centroids = gather_pieces(own_centroids, self.group).view(world, blocks // world, per_block, -1).transpose(
                0, 1).reshape(blocks * per_block, -1)
            k = undeal(gather_pieces(k_share, self.group), self.granule)
            v = undeal(gather_pieces(v_share, self.group), self.granule)
        index = FlatIndex(index_keys, Buckets(centroids, members, (members >= 0).sum(1, dtype=torch.int32), per_block,
                                              d.cluster_block_size))
        share = chunk // world
        if out is None:
            out = torch.empty(tokens // world, q.shape[1], q.shape[2], dtype=q.dtype, device=q.device)
        for c, start in enumerate(range(0, tokens, chunk)):
            layer.prefill_rows(q[c * share:(c + 1) * share], start + rank * share, k, v, index,
                               out[c * share:(c + 1) * share])
        return out

    def prefill(self, q: torch.Tensor, k_share: torch.Tensor, v_share: torch.Tensor, chunk: int = 8192,
                out: torch.Tensor | None = None):
        """Causal prefill of replicated queries q [T, Hq, dh] over this rank's dealt share of the cache
        (`deal(k, rank, world)`, `deal(v, rank, world)`), every rank reading only the keys it stores and the partial
        outputs merged by their log-sum-exps (context parallel). Returns this rank's rows of the output, chunk by
        chunk: rows [c*chunk + rank*chunk/world, c*chunk + (rank+1)*chunk/world) of every chunk c, [T / world, Hq, dh].
        """
        layer, d, world, rank = self.layer, self.design, self.world, self.rank
        T = q.shape[0]
        if T % chunk or chunk % world:
            raise ValueError(f"{T} tokens must split into chunks of {chunk} rows, and a chunk over {world} ranks")
        centroids, members, _ = self.build_index(k_share, T)
        share = chunk // world
        if out is None:
            out = torch.empty(T // world, q.shape[1], q.shape[2], dtype=q.dtype, device=q.device)
        for c, start in enumerate(range(0, T, chunk)):
            rows = q[start:start + chunk]
            positions = torch.arange(start, start + chunk, device=q.device)
            partial, lse = self._read_rows(rows, positions, centroids, members, k_share, v_share)
            with probe.region("merge partials"):
                weight, _ = merge_weight(lse, self.group)
                partial *= weight[..., None]
                out[c * share:(c + 1) * share] = reduce_rows(partial, self.group).to(out.dtype)
        return out

    def _read_rows(self, rows: torch.Tensor, positions: torch.Tensor, centroids: torch.Tensor, members: torch.Tensor,
                   k_share: torch.Tensor, v_share: torch.Tensor, splits: int = 1) -> tuple:
        """This rank's part of the read of replicated query rows: the buckets are picked together (every rank scores
        the centroids of the blocks it clustered, the candidates are all-gathered and cut), then the rank expands and
        attends over the ids it stores. Returns its partial output (fp32) and log-sum-exp per (row, head)."""
        layer, d, world, rank = self.layer, self.design, self.world, self.rank
        per_block = d.block_bucket_count
        with probe.region("index map"):
            index_queries = layer.index_queries(rows)
        # closed blocks b < n with b % world == rank: ceil((n - rank) / world) of this rank's blocks are visible
        closed = positions // d.cluster_block_size
        visible = (((closed - rank + world - 1) // world).clamp_min(0) * per_block).clamp_max(
            centroids.shape[0]).to(torch.int32)
        with probe.region("select"):
            keys, _ = ops.flat_select(index_queries, centroids, visible, d.top_p)
            keys = globalise_keys(keys, per_block, rank, world)
        with probe.region("exchange candidates"):
            every = gather_candidates(keys, self.group)
        with probe.region("select"):
            _, picked = ops.merge_candidates(every)
        with probe.region("expand"):
            lists, lengths, _ = ops.expand(picked, positions, members, d.top_k, d.sink_size, d.window_size,
                                           dealt=(self.granule, world, rank))
        with probe.region("attend"):
            return ops.sparse_attend(rows, k_share, v_share, lists, lengths, layer.scale, splits=splits,
                                     out_dtype=torch.float32)

    def decode(self, q: torch.Tensor, positions: torch.Tensor, k_share: torch.Tensor, v_share: torch.Tensor,
               index: tuple, splits: int = 8) -> torch.Tensor:
        """One step for replicated rows q [R, Hq, dh] at `positions` over the dealt cache (`index` = what
        `build_index` returned): every rank reads the keys it stores and the partial outputs are merged by their
        log-sum-exps with one all-reduce, so every rank returns the whole [R, Hq, dh] bf16 output. A decode step has
        too few rows to split: context parallel is its only split."""
        centroids, members, _ = index
        partial, lse = self._read_rows(q, positions.to(torch.int64), centroids, members, k_share, v_share, splits)
        with probe.region("merge partials"):
            weight, _ = merge_weight(lse, self.group)
            partial *= weight[..., None]
            dist.all_reduce(partial, group=self.group)
        return partial.to(q.dtype)


def exchange_rows(partial: torch.Tensor, lse: torch.Tensor, group=None) -> tuple:
    """Every rank holds a partial result for ALL rows; rank j needs every rank's partial for ITS rows. One
    all-to-all of the outputs and one of the log-sum-exps: ([world, R / world, ...], [world, R / world, ...]) - the
    parts a local merge kernel reads (what a reduce-scatter of weighted outputs does in the collective, without
    the weighting pass before it)."""
    world = dist.get_world_size(group)
    rows = partial.shape[0]
    if rows % world:
        raise ValueError(f"{rows} rows do not split over {world} ranks")
    parts = torch.empty(world, rows // world, *partial.shape[1:], dtype=partial.dtype, device=partial.device)
    lses = torch.empty(world, rows // world, *lse.shape[1:], dtype=lse.dtype, device=lse.device)
    if dist.get_backend(group) == "nccl":
        dist.all_to_all_single(parts, partial.contiguous(), group=group)
        dist.all_to_all_single(lses, lse.contiguous(), group=group)
    else:  # gloo has no all-to-all: gather everything and keep this rank's rows
        rank, share = dist.get_rank(group), rows // world
        parts.copy_(gather_pieces(partial, group)[:, rank * share:(rank + 1) * share])
        lses.copy_(gather_pieces(lse, group)[:, rank * share:(rank + 1) * share])
    return parts, lses


class ShardedLatentLayer:
    """`LatentLayer` over a latent cache dealt across ranks: rows in granules of 64 positions (a pool of config 4, so
    a bucket's pools and a window stay runs of consecutive rows on every rank), cluster blocks round-robin. A step on
    rank r: map the replicated queries, score the centroids of its own blocks, all-gather the candidates and cut them
    with the single-GPU tie rule, expand the picks into the rows it stores, attend over them, and merge the partial
    outputs by their log-sum-exps - after an all-to-all for a prefill chunk (each rank keeps its share of the rows),
    after an all-gather for a decode step (every rank keeps the row)."""

    def __init__(self, layer, rank: int, world: int, group=None, granule: int = GRANULE):
        self.layer, self.rank, self.world, self.group, self.granule = layer, rank, world, group, granule
        self.design = layer.design
        self.index_keys = self.centroids = self.members = self.members_own = None
        d = self.design
        # A rank's own table of members: every bucket's positions that THIS rank holds (a bucket's pools are dealt
        # round-robin, so a row is an n-th as wide as the global table's and an expansion over it an n-th of the
        # work). Rows count toward top_k only through the global table, so it serves when the cut cannot bite.
        # Room for twice a rank's even share of a full bucket: Ward groups pools by likeness, not by position, so a
        # bucket's pools spread over the ranks. A bucket that does not fit is counted (`check()` raises) - and at
        # build time, where the host may look, it simply turns the own tables off.
        even = -(-d.bucket_cap // (d.pool_size * world)) * d.pool_size
        self.own_cap = min(d.bucket_cap, -(-2 * even // 64) * 64)
        self.own_tables = d.top_k >= d.top_p * d.bucket_cap and self.own_cap < d.bucket_cap
        self.own_overflow = None

    def _own_members(self, members: torch.Tensor) -> torch.Tensor:
        """The positions of `members` [rows, cap] that this rank holds, ascending, -1 padded: [rows, own_cap]."""
        none = torch.iinfo(torch.int32).max
        mine = (members >= 0) & ((members // self.granule) % self.world == self.rank)
        over = (mine.sum(1) > self.own_cap).sum().to(torch.int32).reshape(1)
        self.own_overflow = over if self.own_overflow is None else self.own_overflow + over
        kept, _ = torch.where(mine, members, none).sort(dim=1)
        kept = kept[:, : self.own_cap]
        return torch.where(kept == none, -1, kept).contiguous()

    def check(self) -> None:
        """The layer's deferred checks (`FlatLayer.check`), and that no bucket outgrew this rank's own table since
        the index was built."""
        self.layer.check()
        if self.own_overflow is not None and int(self.own_overflow):
            self.own_overflow.zero_()
            raise ValueError(f"a bucket holds more than {self.own_cap} positions of rank {self.rank}: build the layer "
                             "with own_tables off")

    def _cluster(self, keys: torch.Tensor, first_position: int):
        """Pools, Ward and the bucket table of whole blocks whose index keys are `keys` [blocks * block, d]."""
        d = self.design
        blocks = keys.shape[0] // d.cluster_block_size
        pools = ops.pool_keys(keys.view(blocks, d.cluster_block_size, -1), d.pool_size)
        labels, _ = ops.ward_rounds(pools, float(d.pool_size), d.block_bucket_count, d.bucket_cap)
        members, _, _, centroids, _, _ = ops.bucket_table(keys, labels, d.pool_size, d.block_bucket_count, d.bucket_cap,
                                                          first_position=first_position)
        return members, centroids

    def build_index(self, share: torch.Tensor, tokens: int) -> None:
        """From this rank's dealt rows [tokens / world, latent_dim]: every index key (all-gathered), the centroids of
        its own blocks and the global member table."""
        d, layer, world, rank = self.design, self.layer, self.world, self.rank
        blocks, block, per_block = tokens // d.cluster_block_size, d.cluster_block_size, d.block_bucket_count
        if tokens % block or blocks % world or tokens % (self.granule * world):
            raise ValueError(f"{tokens} tokens must be whole cluster blocks of {block}, a multiple of {world} of them")
        with probe.region("index map"):
            own_keys = layer.index_keys(share)
        with probe.region("gather index keys"):
            self.index_keys = undeal(gather_pieces(own_keys, self.group), self.granule)
        del own_keys
        mine = self.index_keys.view(blocks // world, world, block, -1)[:, rank].reshape(blocks // world * block, -1)
        with probe.region("ward"):
            members, self.centroids = self._cluster(mine, 0)
            members = torch.where(members >= 0, members // block * (world * block) + rank * block + members % block,
                                  members)
        with probe.region("gather members"):
            every = gather_pieces(members, self.group)
            self.members = every.view(world, blocks // world, per_block, d.bucket_cap).transpose(0, 1).reshape(
                blocks * per_block, d.bucket_cap).contiguous()
            if self.own_tables:
                # the widest own row over ALL ranks, in whole pools and with a quarter to spare for the buckets still
                # to come (a one-off host read at build time): every rank keeps tables of the same width
                held = ((self.members >= 0) & ((self.members // self.granule) % world == rank)).sum(1).max().reshape(1)
                dist.all_reduce(held, op=dist.ReduceOp.MAX, group=self.group)
                roomy = -(-int(held) * 5 // 4 // 64) * 64
                self.own_cap = min(d.bucket_cap, max(self.own_cap, roomy))
                self.own_tables = self.own_cap < d.bucket_cap
                self.members_own = self._own_members(self.members) if self.own_tables else None

    def extend_index(self, share: torch.Tensor, first: int, count: int) -> None:
        """The index step of a prefill chunk at positions first .. first + count - 1: every rank maps the rows of
        the chunk it stores, the chunk's index keys are all-gathered, and the cluster blocks that close inside
        (first, first + count] are clustered - by every rank, a fraction of a millisecond that saves an exchange of
        their members; a rank keeps the centroids of its own blocks only."""
        d, layer, world, rank = self.design, self.layer, self.world, self.rank
        block, per_block = d.cluster_block_size, d.block_bucket_count
        if first % (self.granule * world) or count % (self.granule * world):
            raise ValueError("a chunk must deal out in whole granules over the ranks")
        with probe.region("index map"):
            own = layer.index_keys(share[first // world:(first + count) // world])
        with probe.region("gather index keys"):
            self.index_keys[first:first + count] = undeal(gather_pieces(own, self.group), self.granule)
        b0, b1 = first // block, (first + count) // block
        if b1 <= b0:
            return
        with probe.region("ward"):
            members, centroids = self._cluster(self.index_keys[b0 * block:b1 * block], b0 * block)
            self.members[b0 * per_block:b1 * per_block] = members
            if self.own_tables:
                self.members_own[b0 * per_block:b1 * per_block] = self._own_members(members)
            for b in range(b0, b1):
                if b % world == rank:
                    at = (b // world) * per_block
                    self.centroids[at:at + per_block] = centroids[(b - b0) * per_block:(b - b0 + 1) * per_block]

    def adopt_index(self, index_keys: torch.Tensor, centroids: torch.Tensor, members: torch.Tensor) -> None:
        """Take this rank's part of an index that exists whole (every index key, the centroids and the member table
        of ALL buckets, block after block): what `build_index` leaves behind, without its collectives."""
        d, world, rank = self.design, self.world, self.rank
        per_block = d.block_bucket_count
        blocks = members.shape[0] // per_block
        self.index_keys, self.members = index_keys, members.contiguous()
        self.centroids = centroids.view(blocks // world, world, per_block, -1)[:, rank].reshape(
            blocks // world * per_block, -1).contiguous()
        if self.own_tables:
            self.members_own = self._own_members(self.members)
            if int(self.own_overflow):
                self.own_tables, self.members_own, self.own_overflow = False, None, None

    def pick(self, rows: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """Every row's top-p buckets, best first, as GLOBAL bucket ids [R, top_p] - the same on every rank. A
        collective call: each rank scores the centroids of its own blocks, the candidates are all-gathered and cut
        with the single-GPU tie rule."""
        keys = self.local_candidates(rows, positions)
        with probe.region("exchange candidates"):
            every = gather_candidates(keys, self.group)
        with probe.region("select"):
            _, picked = ops.merge_candidates(every)
        return picked

    def local_candidates(self, rows: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """This rank's candidates for every row: the top-p of the buckets it clustered, as packed keys over GLOBAL
        bucket ids [R, top_p]."""
        layer, d, world, rank = self.layer, self.design, self.world, self.rank
        per_block = d.block_bucket_count
        with probe.region("index map"):
            index_queries = layer.index_queries(rows)
        closed = positions // d.cluster_block_size
        visible = (((closed - rank + world - 1) // world).clamp_min(0) * per_block).clamp_max(
            self.centroids.shape[0]).to(torch.int32)
        with probe.region("select"):
            if rows.shape[0] <= 8:
                keys, _ = ops.flat_select_decode(index_queries, self.centroids, None, visible, d.top_p, splits=4)
            else:
                keys, _ = ops.flat_select(index_queries, self.centroids, visible, d.top_p)
            return globalise_keys(keys, per_block, rank, world)

    def select(self, rows: torch.Tensor, positions: torch.Tensor, pad: bool = True) -> tuple:
        """This rank's share of every row's read list, as rows of its own cache: (lists, lengths). A collective call
        (the candidates are exchanged inside). Local row l of rank r is position (l / granule * world + r) * granule
        + l % granule."""
        return self.expand_own(self.pick(rows, positions), positions, pad)

    def expand_own(self, picked: torch.Tensor, positions: torch.Tensor, pad: bool = True) -> tuple:
        """The rows of this rank's cache that the picks (global bucket ids) list for every row: (lists, lengths)."""
        d = self.design
        with probe.region("expand"):
            if self.own_tables:  # (the cut at top_k cannot bite: this rank's members are all there is to list)
                lists, lengths, _ = ops.expand(picked, positions, self.members_own, d.top_p * self.own_cap, d.sink_size,
                                               d.window_size, dealt=(self.granule, self.world, self.rank), pad=pad)
            else:
                lists, lengths, _ = ops.expand(picked, positions, self.members, d.top_k, d.sink_size, d.window_size,
                                               dealt=(self.granule, self.world, self.rank), pad=pad)
        return lists, lengths

    def _read_rows(self, rows: torch.Tensor, positions: torch.Tensor, share: torch.Tensor, splits: int) -> tuple:
        """This rank's partial read of every row: (out bf16, lse). (bf16 partials: they cross NVLink next.)"""
        layer = self.layer
        lists, lengths = self.select(rows, positions, pad=False)  # (read by their lengths just below)
        with probe.region("attend"):
            return ops.latent_attend(rows, share, lists, lengths, layer.scale, value_dim=layer.value_dim,
                                     splits=splits, out_dtype=torch.bfloat16, status=layer._attend_status)

    def prefill_rows(self, rows: torch.Tensor, start: int, share: torch.Tensor, out: torch.Tensor | None = None):
        """The read of replicated query rows [n, heads, latent_dim] at positions start.. : this rank's share of the
        output rows, [n / world, heads, value_dim] bf16 (rows rank * n / world .. of the chunk)."""
        positions = torch.arange(start, start + rows.shape[0], device=rows.device)
        partial, lse = self._read_rows(rows, positions, share, 1)
        with probe.region("merge partials"):
            parts, lses = exchange_rows(partial, lse, self.group)
            merged, _ = ops.lse_merge(parts, lses, out_dtype=torch.bfloat16)
        if out is not None:
            out.copy_(merged)
            return out
        return merged

    def prefill_from_host(self, q_host: torch.Tensor, rows_host: torch.Tensor, start: int, count: int,
                          share: torch.Tensor, out_host: torch.Tensor, pieces: int = 4) -> torch.Tensor:
        """A prefill chunk of `count` rows at positions start.. whose inputs and output live in PINNED host memory,
        the copies beside the work. The host link carries every row once: the chunk is cut into `pieces`, this rank
        brings in the `rank`-th of each piece's query rows (`q_host` [count / world, heads, latent_dim]: its rows of
        piece 0, then of piece 1, ...), the ranks all-gather a piece over NVLink while the piece before is read, and a
        piece's output rows of this rank (`out_host` [count / world, heads, value_dim], in the same order) leave as
        soon as they are merged. `rows_host` holds this rank's dealt rows of the chunk's latent. A collective call; on
        return the current stream has waited for the last output copy."""
        layer, world, dev = self.layer, self.world, share.device
        if count % (pieces * world):
            raise ValueError(f"{count} rows do not cut into {pieces} pieces of {world} shares")
        piece, own = count // pieces, count // pieces // world
        main = torch.cuda.current_stream(dev)
        if layer._copy_in is None:
            layer._copy_in, layer._copy_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        copy_in, copy_out = layer._copy_in, layer._copy_out
        while len(layer._copy_events) < 2 * pieces + 1:
            layer._copy_events.append(torch.cuda.Event())
        rows_in, arrived, done = layer._copy_events[0], layer._copy_events[1::2], layer._copy_events[2::2]
        q_own = layer._buffer("q share from host", tuple(q_host.shape), q_host.dtype, dev)
        q_all = layer._buffer("q pieces", (pieces, piece, *q_host.shape[1:]), q_host.dtype, dev)
        out = layer._buffer("out share to host", tuple(out_host.shape), out_host.dtype, dev)
        copy_in.wait_stream(main)   # the last call's reads of these buffers are over
        copy_out.wait_stream(main)
        with torch.cuda.stream(copy_in):
            share[start // world:(start + count) // world].copy_(rows_host, non_blocking=True)
            rows_in.record(copy_in)
            for i in range(pieces):
                q_own[i * own:(i + 1) * own].copy_(q_host[i * own:(i + 1) * own], non_blocking=True)
                dist.all_gather_into_tensor(q_all[i].view(-1), q_own[i * own:(i + 1) * own].view(-1), group=self.group)
                arrived[i].record(copy_in)
        main.wait_event(rows_in)
        self.extend_index(share, start, count)
        for i in range(pieces):
            main.wait_event(arrived[i])
            self.prefill_rows(q_all[i], start + i * piece, share, out[i * own:(i + 1) * own])
            done[i].record(main)
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(done[i])
                out_host[i * own:(i + 1) * own].copy_(out[i * own:(i + 1) * own], non_blocking=True)
        main.wait_stream(copy_out)
        return out_host

    def decode(self, q: torch.Tensor, positions: torch.Tensor, share: torch.Tensor, splits: int = 32) -> torch.Tensor:
        """One step for replicated rows [R, heads, latent_dim] at `positions`: the whole output on every rank. Every
        rank lists the WHOLE read (a few rows: the clustered expansion, which keeps every id) and its attention
        call skips the positions it does not hold - cheaper than a dealt expansion of so few rows."""
        layer, d = self.layer, self.design
        positions = positions.to(torch.int64)
        picked = self.pick(q, positions)
        with probe.region("expand"):
            lists, lengths, _ = ops.expand(picked, positions, self.members, d.top_k, d.sink_size, d.window_size)
        with probe.region("attend"):
            partial, lse = ops.latent_attend(q, share, lists, lengths, layer.scale, value_dim=layer.value_dim,
                                             splits=splits, out_dtype=torch.float32, status=layer._attend_status,
                                             dealt=(self.granule, self.world, self.rank))
        with probe.region("merge partials"):
            merged, _ = ops.lse_merge(gather_pieces(partial, self.group), gather_pieces(lse, self.group),
                                      out_dtype=torch.bfloat16)
        return merged
