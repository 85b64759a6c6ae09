"""One layer's index read off the key and the heads' queries: the maps, the way to the pool's keys and the selector,
with no engine in sight (`src/lsa/sglang/index/layer_index.py:613-928`).

A model hands in its input (`KeyAndQuery`), the KV slots its tokens were given and the request table, and gets back
lists of KV slots. The keys are in the KV pool already, so the layer keeps no copy of them: an index key is made from
the pool's slot when the cache needs it (`PoolKeys`), and a prefill indexes its chunk from the keys in hand.

What this build serves is the key-and-query input of a grouped-query or latent pool on one rank. The attention
input `x`, a pool split over a decode group (`Shard.size > 1`), key heads split over tensor-parallel ranks (`split`)
and prefix reuse are refused where the reference takes them.
"""

from __future__ import annotations

from collections.abc import Callable, Sequence
from dataclasses import dataclass

import torch

from lsa_b200 import ops
from lsa_b200.serving import BucketCache, Selector
from lsa_b200.sglang.index_space import KeyAndQuery, KeySlot
from lsa_b200.sglang.settings import PAGE_SIZE, DesignSettings


@dataclass(frozen=True)
class Shard:
    """Which KV slots a rank of a decode group owns: slot s lives on rank s % size at row s // size
    (`layer_index.py:65-87`)."""

    rank: int = 0
    size: int = 1

    def __post_init__(self) -> None:
        if not 0 <= self.rank < self.size:
            raise ValueError(f"rank {self.rank} is not in a group of {self.size}")


class KeyAndQueryProjection:
    """A layer's two maps over the key and the heads' queries (`layer_index.py:307-386`): an index key is
    normalize(key @ key map), an index query normalize(sum over heads of query @ query map), fp32 unit rows both.

    Either input form of `KeyAndQuery` is read. The heads attention was handed go through one kernel that sums a
    group's heads, skips the rotated prefix, maps and normalises; the written-out form goes through the same kernel
    with one head of `key_dim` dims.
    """

    def __init__(self, query_projection: torch.Tensor, key_projection: torch.Tensor, key_slot: KeySlot, device) -> None:
        if query_projection.shape != key_projection.shape or key_projection.shape[0] != key_slot.key_dim:
            raise ValueError(f"the pool's key input is {key_slot.key_dim} dims and the maps read "
                             f"{tuple(key_projection.shape)} and {tuple(query_projection.shape)}")
        self.key_slot = key_slot
        self.key_dim, self.index_dim = int(key_projection.shape[0]), int(key_projection.shape[1])
        self.query_projection = query_projection.to(device=device, dtype=torch.bfloat16).contiguous()
        self.key_projection = key_projection.to(device=device, dtype=torch.bfloat16).contiguous()

    def _heads(self, x: torch.Tensor) -> bool:
        """Whether a 3-D input is heads as attention holds them (and not [S, heads, key_dim])."""
        slot = self.key_slot
        return x.dim() == 3 and x.shape[2] == slot.head_dim and x.shape[1] % slot.heads == 0 and \
            (x.shape[2] != self.key_dim or slot.heads == 1 and slot.width == slot.head_dim)

    def index_keys(self, key: torch.Tensor) -> torch.Tensor:
        """key [S, key_dim], or the key heads [S, Hkv, head_dim] -> [S, index_dim] fp32 unit rows."""
        slot = self.key_slot
        if key.dim() == 3 and self._heads(key):
            return ops.index_map(key, self.key_projection, group=1, dh_off=slot.offset, dh_used=slot.width)
        return ops.index_map(key.reshape(key.shape[0], 1, self.key_dim), self.key_projection)

    def index_queries(self, query: torch.Tensor) -> torch.Tensor:
        """query [S, heads, key_dim] (every head is summed), or the query heads [S, Hq, head_dim] (each group is
        summed into its key head's slice) -> [S, index_dim] fp32 unit rows."""
        slot = self.key_slot
        if self._heads(query):
            return ops.index_map(query, self.query_projection, group=query.shape[1] // slot.heads,
                                 dh_off=slot.offset, dh_used=slot.width)
        if query.dim() != 3 or query.shape[2] != self.key_dim:
            raise ValueError(f"queries must be [S, heads, {self.key_dim}] or heads of {slot.head_dim} dims - got "
                             f"{tuple(query.shape)}")
        return ops.index_map(query, self.query_projection, group=query.shape[1])


class PoolKeys:
    """A layer's index keys, made from the keys the KV pool holds when they are read (`layer_index.py:448-527`)."""

    def __init__(self, key_buffer: Callable[[], torch.Tensor], projection: KeyAndQueryProjection) -> None:
        self.key_buffer, self.projection = key_buffer, projection

    def write(self, slots: torch.Tensor, key: torch.Tensor) -> None:
        """Write keys at their KV slots, which attention writes again after the indexer: the key input's dims of
        each head, or whole heads."""
        buffer = self.key_buffer()
        if key.dim() == 3:
            buffer[slots] = key.to(buffer.dtype)
        else:
            self.projection.key_slot.write(buffer, slots, key.to(buffer.dtype))

    def read(self, slots: torch.Tensor) -> torch.Tensor:
        """The index keys at KV slots [S, index_dim] fp32."""
        return self.projection.index_keys(self.key_buffer()[slots])


class KeyLookup:
    """One request's positions to their index keys: the pool's, and a chunk's own where the chunk is in hand
    (`layer_index.py:530-611`)."""

    def __init__(self, buffer: PoolKeys, slot_table: Callable[[], torch.Tensor], row: int,
                 chunk: tuple | None = None) -> None:
        self.buffer, self.slot_table, self.row, self.chunk = buffer, slot_table, row, chunk

    def __call__(self, first: int, stop: int) -> torch.Tensor:
        """The index keys of positions [first, stop) [stop - first, index_dim] fp32, with no device read."""
        table = self.slot_table()
        if self.chunk is not None and first >= self.chunk[0]:
            start, keys = self.chunk
            return keys[first - start:stop - start]
        return self.buffer.read(table[self.row, first:stop].long())


class LayerIndex:
    """The index of one layer: where its index keys come from and how a forward batch reads them."""

    def __init__(self, settings: DesignSettings, projections: tuple, slot_count: int, kv_size: int,
                 slot_table: Callable[[], torch.Tensor], max_context: int, prefill_chunk: int, device,
                 shard: Shard | None = None, check_index: bool = False,
                 key_buffer: Callable[[], torch.Tensor] | None = None, sum_heads=None,
                 key_slot: KeySlot | None = None, prefix_reuse: bool = False, split=None) -> None:
        """Hold the maps and build the selector.

        Args:
            settings: The design.
            projections: The layer's query map and key map, both [key_dim, index_dim].
            slot_count: KV slots the pool holds on this rank, padding included.
            kv_size: Keys the KV pool holds.
            slot_table: Returns the request table, each request's positions to KV slots [requests, context] int32.
            max_context: Longest context a request holds.
            prefill_chunk: Most query rows a prefill call is handed.
            key_buffer: Returns the layer's KV pool buffer [slots, heads, head_dim] bf16.
            key_slot: Where the key input sits in a pool slot; None = a latent at the front of one head.

        Raises:
            ValueError: No way to the KV pool's keys.
            NotImplementedError: A decode group, a tensor-parallel split, a cross-rank head sum or prefix reuse.
        """
        shard = shard or Shard()
        if shard.size > 1 or split is not None or sum_heads is not None or prefix_reuse or check_index:
            raise NotImplementedError("this build serves the key-and-query input on one rank: no decode group, no "
                                      "split of the key heads, no prefix reuse")
        if key_buffer is None:
            raise ValueError("the key and query input reads its keys from the KV pool - it needs the pool's key buffer")
        self.settings, self.shard, self.slot_table = settings, shard, slot_table
        self.index_dim = settings.indexer.index_dim
        key_slot = key_slot or KeySlot.latent(int(projections[1].shape[0]))
        self.projection = KeyAndQueryProjection(*projections, key_slot, device)
        if self.projection.index_dim != self.index_dim:
            raise ValueError(f"the maps write {self.projection.index_dim} dims and the design's index has {self.index_dim}")
        self.buffer = PoolKeys(key_buffer, self.projection)
        design = settings.indexer.flat_design()
        requests = slot_table().shape[0]
        page_buckets = PAGE_SIZE // design.bucket_size
        request_pages = -(-max_context // PAGE_SIZE) + 1
        pages = -(-kv_size // PAGE_SIZE) + requests  # (a request's last page is part full)
        cache = BucketCache(design, self.index_dim, pages, page_buckets, requests, request_pages, device)
        self.selector = Selector(cache, 1, slot_table)
        self.prefill_chunk, self.starts_checked = prefill_chunk, False
        # An attention backend that saves a forward's keys before it selects turns the layer's own write off
        self.writes_pool = True

    # ---- writing

    def project(self, inputs: KeyAndQuery, slots: torch.Tensor) -> tuple:
        """The tokens' index queries [S, index_dim] fp32 and the index keys of the chunk [S, index_dim] fp32; the keys
        themselves are written to the pool at `slots` (attention writes them again, the same)."""
        if not isinstance(inputs, KeyAndQuery):
            raise TypeError("the attention input reached an index built for the key and query")
        if inputs.key.shape[0] != slots.shape[0]:
            raise ValueError(f"the key and query input has {inputs.key.shape[0]} keys for {slots.shape[0]} slots")
        if self.writes_pool:
            self.buffer.write(slots, inputs.key)
        return self.projection.index_queries(inputs.query), self.projection.index_keys(inputs.key)

    def write(self, inputs: KeyAndQuery, slots: torch.Tensor) -> torch.Tensor:
        """Write new tokens' keys at their KV slots and return their index queries."""
        if inputs.key.shape[0] != slots.shape[0]:
            raise ValueError(f"the key and query input has {inputs.key.shape[0]} keys for {slots.shape[0]} slots")
        if self.writes_pool:
            self.buffer.write(slots, inputs.key)
        return self.projection.index_queries(inputs.query)

    def write_chunk(self, inputs: KeyAndQuery, slots: torch.Tensor) -> None:
        """Write a prefill chunk's keys without selecting: a short prompt the dense path prefills. The next
        `maintain` indexes them from the pool."""
        self.buffer.write(slots, inputs.key)

    def keys_of(self, row: int, chunk: tuple | None = None) -> KeyLookup:
        return KeyLookup(self.buffer, self.slot_table, row, chunk)

    # ---- a forward

    def maintain(self, rids: Sequence, rows: Sequence, ends: Sequence) -> int:
        """Bring each request's cache up to the keys already in the pool, eagerly, before a forward."""
        return self.selector.maintain(rids, rows, ends, self.keys_of)

    def extend(self, inputs: KeyAndQuery, positions: torch.Tensor, slots: torch.Tensor, rows: Sequence,
               lengths: Sequence, starts: Sequence) -> torch.Tensor:
        """Write the keys of a prefill batch and select for its queries, request by request.

        Args:
            inputs: The requests' new tokens end to end, as their key and heads' queries.
            positions: Each row's position in its request [S].
            slots: Each new token's KV slot [S] int64.
            rows: The requests' table rows; lengths: new tokens of each; starts: position of each request's first
                new token, from the scheduler - no device read.

        Returns:
            KV slots [S, width] int32, -1 padded, valid entries first.
        """
        index_queries, index_keys = self.project(inputs, slots)
        starts = [int(start) for start in starts]
        self.check_starts(positions, lengths, starts)
        lists, first = [], 0
        for row, count, start in zip(rows, lengths, starts, strict=True):
            stop = first + count
            held = self.selector.cache.end(row)
            if held != start:  # (`maintain` brings a cached prefix's keys in before the forward)
                raise ValueError(f"request {row}'s index holds {held} keys and its chunk starts at {start}")
            lists.append(self.selector.prefill(row, index_queries[first:stop], positions[first:stop],
                                               index_keys[first:stop], start))
            first = stop
        return torch.cat(lists) if lists else torch.empty(0, self.settings.width, device=slots.device,
                                                          dtype=torch.int32)

    def check_starts(self, positions: torch.Tensor, counts: Sequence, starts: Sequence) -> None:
        """Raise unless the scheduler's first positions are the batch's own - once, on the first prefill, as it
        reads the device."""
        if self.starts_checked:
            return
        self.starts_checked = True
        offsets = [sum(counts[:i]) for i, count in enumerate(counts) if count]
        firsts = positions[torch.tensor(offsets, device=positions.device, dtype=torch.long)].tolist()
        wanted = [start for start, count in zip(starts, counts, strict=True) if count]
        if firsts != wanted:
            raise ValueError(f"the batch's first positions {firsts} are not the scheduler's {wanted}")

    def decode(self, inputs: KeyAndQuery, positions: torch.Tensor, slots: torch.Tensor,
               rows: torch.Tensor) -> torch.Tensor:
        """Write a decode step's keys and select for its queries: fixed shapes, no host read.

        Returns:
            KV slots [B, width] int32, -1 padded.
        """
        return self.selector.decode(self.write(inputs, slots), positions, rows)
