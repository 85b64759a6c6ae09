"""One layer's index read off the key and the heads' queries: the maps, the way to the pool's keys and the selector,
with no engine in sight (`src/lsa/sglang/index/layer_index.py:613-928`).

A model hands in its input (`KeyAndQuery`), the KV slots its tokens were given and the request table, and gets back
lists of KV slots. The keys are in the KV pool already, so the layer keeps no copy of them: an index key is made from
the pool's slot when the cache needs it (`PoolKeys`), and a prefill indexes its chunk from the keys in hand.

What this build serves is the key-and-query input of a grouped-query or latent pool: on one rank, with the pool's
slots split over a decode group (`Shard`: a key is mapped on the rank that owns its slot and the group sums), or with
the key heads split over tensor-parallel ranks (`KeySplit`: partial index vectors summed across the group, a token's
index key made once and kept at its KV slot). Under `prefix_reuse` a request that arrives with a cached prefix takes
the index pages another request built from the same pool bits (page fingerprints). The attention input `x` is
refused where the reference takes it.
"""

from __future__ import annotations

from collections.abc import Callable, Sequence
from dataclasses import dataclass

import torch

from lsa_b200 import ops
from lsa_b200.serving import BucketCache, Selector
from lsa_b200.sglang.index_space import KeyAndQuery, KeySlot
from lsa_b200.sglang.settings import PAGE_SIZE, DesignSettings


# Pages fingerprinted a call, which bounds the slots a call reads (`layer_index.py:56`)
FINGERPRINT_PAGES = 8
# Bits a piece of a fingerprint holds while a group sums it: a collective that adds in fp32 is exact on such pieces
FINGERPRINT_PIECE_BITS = 16
FINGERPRINT_SEED = 20261007
FINGERPRINT_WORDS = 4096
_FINGERPRINT_WEIGHTS: dict = {}


def fingerprint_weights(device) -> tuple:
    """The fingerprint's odd int64 weights - one a word of a key's stored bits, one a position of a page - drawn as
    the reference draws them, so a page's fingerprint is the same number (`layer_index.py:89-103`)."""
    key = str(device)
    if key not in _FINGERPRINT_WEIGHTS:
        generator = torch.Generator().manual_seed(FINGERPRINT_SEED)
        words, positions = (torch.randint(-(1 << 62), 1 << 62, (count,), generator=generator) | 1
                            for count in (FINGERPRINT_WORDS, PAGE_SIZE))
        _FINGERPRINT_WEIGHTS[key] = (words.to(device), positions.to(device))
    return _FINGERPRINT_WEIGHTS[key]


def page_fingerprints(stored: torch.Tensor, owned: torch.Tensor | None, slots: torch.Tensor | None = None) -> torch.Tensor:
    """A fingerprint of each page of what a rank stores for its keys [pages] int64 (`layer_index.py:106-122`): a
    weighted sum of the bits that wraps instead of rounding, so it is exact, the order it adds in does not change it,
    and pages that differ in any bit match by chance alone. A slot another rank owns adds nothing, so a group's sum is
    the fingerprint of the whole page. `stored` [rows, dim] is read at `slots` (None: its rows are a run of whole
    pages in order)."""
    words, positions = fingerprint_weights(stored.device)
    return ops.page_fingerprints(stored, PAGE_SIZE, words, positions, slots=slots, owned=owned)


def exact_group_sum(values: torch.Tensor, reduce: Callable[[torch.Tensor], torch.Tensor]) -> torch.Tensor:
    """int64 values summed across a group exactly, wrapping as an int64 sum does, whatever dtype the collective adds
    in: 16-bit pieces as floats, put back together (`layer_index.py:125-137`)."""
    shifts = FINGERPRINT_PIECE_BITS * torch.arange(64 // FINGERPRINT_PIECE_BITS, device=values.device)
    pieces = ((values[:, None] >> shifts) & ((1 << FINGERPRINT_PIECE_BITS) - 1)).float()
    return (reduce(pieces).long() << shifts).sum(1)


@dataclass(frozen=True)
class Shard:
    """Which KV slots a rank of a decode group owns: slot s lives on rank s % size at row s // size
    (`layer_index.py:65-87`)."""

    rank: int = 0
    size: int = 1
    reduce: Callable[[torch.Tensor], torch.Tensor] | None = None  # sums a tensor across the group, the same on every rank

    def __post_init__(self) -> None:
        if not 0 <= self.rank < self.size:
            raise ValueError(f"rank {self.rank} is not in a group of {self.size}")


@dataclass(frozen=True)
class KeySplit:
    """Which dims of the key and query input a tensor-parallel rank holds, and how to sum its share across the group
    (`layer_index.py:296-304`)."""

    start: int
    stop: int
    counts_key: bool  # whether this rank's key heads are added to the sum: one of the ranks that replicate a head is
    reduce: Callable[[torch.Tensor], torch.Tensor]


class KeyBuffer:
    """A layer's index keys held at the KV slots [slots, index_dim] fp32: where a rank's pool holds only some of the
    key heads, a token's index key is made once, as it is written (`layer_index.py:158-232`)."""

    def __init__(self, slot_count: int, index_dim: int, device) -> None:
        self.keys = torch.zeros(slot_count, index_dim, device=device, dtype=torch.float32)

    def write(self, slots: torch.Tensor, keys: torch.Tensor) -> None:
        self.keys[slots] = keys

    def read(self, slots: torch.Tensor) -> torch.Tensor:
        return self.keys[slots]

    def stored(self, slots: torch.Tensor) -> tuple:
        """What this rank stores for KV slots - their index keys - as (table, rows of it, ownership or None), for a
        fingerprint to read in place (`layer_index.py:221-232`)."""
        return self.keys, slots, None


class KeyAndQueryProjection:
    """A layer's two maps over the key and the heads' queries (`layer_index.py:307-386`): an index key is
    normalize(key @ key map), an index query normalize(sum over heads of query @ query map), fp32 unit rows both.

    Either input form of `KeyAndQuery` is read. The heads attention was handed go through one kernel that sums a
    group's heads, skips the rotated prefix, maps and normalises; the written-out form goes through the same kernel
    with one head of `key_dim` dims.
    """

    def __init__(self, query_projection: torch.Tensor, key_projection: torch.Tensor, key_slot: KeySlot, device,
                 split: KeySplit | None = None) -> None:
        """`key_slot` describes the WHOLE input (every key head); under `split` a rank's heads are the rows
        [split.start, split.stop) of both maps."""
        if query_projection.shape != key_projection.shape or key_projection.shape[0] != key_slot.key_dim:
            raise ValueError(f"the pool's key input is {key_slot.key_dim} dims and the maps read "
                             f"{tuple(key_projection.shape)} and {tuple(query_projection.shape)}")
        self.key_slot, self.split = key_slot, split
        self.key_dim, self.index_dim = int(key_projection.shape[0]), int(key_projection.shape[1])
        self.query_projection = query_projection.to(device=device, dtype=torch.bfloat16).contiguous()
        self.key_projection = key_projection.to(device=device, dtype=torch.bfloat16).contiguous()
        if split is not None:
            if not 0 <= split.start < split.stop <= self.key_dim or (split.stop - split.start) % key_slot.width:
                raise ValueError(f"a rank's share [{split.start}, {split.stop}) must be whole heads of {key_slot.width} "
                                 f"dims inside the input's {self.key_dim}")
            self.share_query = self.query_projection[split.start:split.stop].contiguous()
            self.share_key = self.key_projection[split.start:split.stop].contiguous()

    def split_index(self, key: torch.Tensor, query: torch.Tensor) -> tuple:
        """Index queries and index keys from the heads this rank holds, summed across the group (`layer_index.py:
        355-382`): each map is applied to this rank's rows of it (both are linear before the normalise), the two
        [index_dim] partials travel in ONE sum, and the rows are normalised after - the same on every rank. A rank
        that replicates another's key heads adds zeros for its key.

        Args:
            key: This rank's key heads [S, held heads, head_dim] bf16 (or their input [S, share]).
            query: This rank's query heads [S, held query heads, head_dim] bf16 (or [S, heads, share]).

        Returns:
            Index queries [S, index_dim] fp32 unit rows, index keys [S, index_dim] fp32 unit rows.
        """
        split, slot = self.split, self.key_slot
        if split is None:
            raise ValueError("a split index needs the projection's KeySplit")
        held = (split.stop - split.start) // slot.width
        if query.dim() == 3 and query.shape[2] == slot.head_dim and query.shape[2] != split.stop - split.start:
            queries = ops.index_map(query, self.share_query, group=query.shape[1] // held, dh_off=slot.offset,
                                    dh_used=slot.width, normalize=False)
        else:
            queries = ops.index_map(query, self.share_query, group=query.shape[1], normalize=False)
        if not split.counts_key:
            keys = torch.zeros_like(queries)
        elif key.dim() == 3 and key.shape[2] == slot.head_dim:
            keys = ops.index_map(key, self.share_key, group=1, dh_off=slot.offset, dh_used=slot.width, normalize=False)
        else:
            keys = ops.index_map(key.reshape(key.shape[0], 1, -1), self.share_key, normalize=False)
        index_queries, index_keys = split.reduce(torch.cat([queries, keys], dim=1)).split(self.index_dim, dim=1)
        unit = torch.nn.functional.normalize
        return unit(index_queries, dim=-1).contiguous(), unit(index_keys, dim=-1).contiguous()

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

    def __init__(self, key_buffer: Callable[[], torch.Tensor], projection: KeyAndQueryProjection,
                 shard: Shard | None = None) -> None:
        self.key_buffer, self.projection, self.shard = key_buffer, projection, shard or Shard()

    def write(self, slots: torch.Tensor, key: torch.Tensor) -> None:
        """Write keys at their KV slots, which attention writes again after the indexer: the key input's dims of
        each head, or whole heads. Under a decode group nothing is written: attention writes each key to the rank
        that owns it, and the batch being indexed is read from the chunk in hand."""
        if self.shard.size > 1:
            return
        buffer = self.key_buffer()
        if key.dim() == 3:
            buffer[slots] = key.to(buffer.dtype)
        else:
            self.projection.key_slot.write(buffer, slots, key.to(buffer.dtype))

    def read(self, slots: torch.Tensor) -> torch.Tensor:
        """The index keys at KV slots [S, index_dim] fp32, whichever rank holds them: under a decode group slot s is
        row s // size of rank s % size's pool, a key is mapped on the rank that owns it and the group sums - each row
        has one owner and the others add zeros; every rank calls this with the same slots (`layer_index.py:
        497-515`)."""
        if self.shard.size == 1:
            return self.projection.index_keys(self.key_buffer()[slots])
        size, rank = self.shard.size, self.shard.rank
        owned = slots % size == rank
        rows = torch.where(owned, slots // size, 0)  # (another rank's slot reads row 0 here and is zeroed after)
        index_keys = self.projection.index_keys(self.key_buffer()[rows])
        return self.shard.reduce(index_keys * owned[:, None])


    def stored(self, slots: torch.Tensor) -> tuple:
        """What this rank's pool stores for KV slots - their key input - as (table [pool rows, dims], rows of it,
        ownership or None), for a fingerprint to read in place (`layer_index.py:515-527`): the pool's own bits, not
        index keys - a projection rounds by the size of its batch, the pool does not."""
        size, slot = self.shard.size, self.projection.key_slot
        owned = None if size == 1 else slots % size == self.shard.rank
        rows = slots if size == 1 else torch.where(owned, slots // size, 0)
        buffer = self.key_buffer()
        bytes_ = buffer.element_size()
        if slot.heads == 1 and (slot.offset * bytes_) % 8 == 0 and (slot.width * bytes_) % 8 == 0 \
                and (buffer.stride(0) * bytes_) % 8 == 0:
            return buffer[:, 0, slot.offset:slot.offset + slot.width], rows, owned  # (a view: nothing is copied)
        return slot.read(buffer, rows), None, owned


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

    def fingerprints(self, first: int, count: int) -> list:
        """The fingerprints of the request's pages [first, first + count), read from the pool
        (`layer_index.py:586-610`). Under a decode group every rank fingerprints the slots it owns and the group sums
        them, so every rank holds the same numbers."""
        shard = getattr(self.buffer, "shard", None)
        prints = []
        for start in range(first, first + count, FINGERPRINT_PAGES):
            stop = min(first + count, start + FINGERPRINT_PAGES)
            slots = self.slot_table()[self.row, start * PAGE_SIZE:stop * PAGE_SIZE].long()
            stored, rows, owned = self.buffer.stored(slots)
            prints.append(page_fingerprints(stored, owned, rows))
        if not prints:
            return []
        total = torch.cat(prints)
        if shard is not None and shard.reduce is not None:
            total = exact_group_sum(total, shard.reduce)
        return total.tolist()


class LayerIndex:
    """The index of one layer: where its index keys come from and how a forward batch reads them."""

    def __init__(self, settings: DesignSettings, projections: tuple, slot_count: int, kv_size: int,
                 slot_table: Callable[[], torch.Tensor], max_context: int, prefill_chunk: int, device,
                 shard: Shard | None = None, check_index: bool = False,
                 key_buffer: Callable[[], torch.Tensor] | None = None, sum_heads=None,
                 key_slot: KeySlot | None = None, prefix_reuse: bool = False, split=None,
                 spare_contexts: int = 0) -> None:
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
            NotImplementedError: A cross-rank head sum.
        """
        shard = shard or Shard()
        if sum_heads is not None:
            raise NotImplementedError("this build serves no cross-rank head sum for an MLA latent")
        if shard.size > 1 and shard.reduce is None:
            raise ValueError("a decode context-parallel shard needs the sum across its group")
        if split is not None and shard.size > 1:
            raise ValueError("a rank holding some of the key heads keeps the whole context's index keys itself - "
                             "decode context parallel splits the slots as well")
        if split is None and key_buffer is None:
            raise ValueError("the key and query input reads its keys from the KV pool - it needs the pool's key buffer")
        self.settings, self.shard, self.slot_table = settings, shard, slot_table
        self.check_index = check_index and shard.size > 1
        self.index_dim = settings.indexer.index_dim
        key_slot = key_slot or KeySlot.latent(int(projections[1].shape[0]))
        self.projection = KeyAndQueryProjection(*projections, key_slot, device, split)
        if self.projection.index_dim != self.index_dim:
            raise ValueError(f"the maps write {self.projection.index_dim} dims and the design's index has {self.index_dim}")
        # Where a position's index key is found: mapped from the pool's slot when it is read, or - a rank's pool
        # holding only some of the key heads - made once as the token is written and kept at its KV slot.
        self.buffer = KeyBuffer(slot_count, self.index_dim, device) if split is not None else \
            PoolKeys(key_buffer, self.projection, shard)
        design = settings.indexer.flat_design()
        requests = slot_table().shape[0]
        page_buckets = PAGE_SIZE // design.bucket_size
        request_pages = -(-max_context // PAGE_SIZE) + 1
        # (under a decode group every rank indexes each request's whole context: the cache covers `size` pools)
        pages = -(-kv_size * shard.size // PAGE_SIZE) + requests  # (a request's last page is part full)
        # (requests that share a cached prefix hold it once in the KV pool and once each here, unless pages are shared
        # by `prefix_reuse`: `spare_contexts` full contexts of pages on top of what the pool calls for)
        pages += spare_contexts * (request_pages - 1)
        cache = BucketCache(design, self.index_dim, pages, page_buckets, requests, request_pages, device,
                            reuse=prefix_reuse)
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
        if self.projection.split is not None:  # the keys' index keys are made once, here, and kept at their slots
            index_queries, index_keys = self.projection.split_index(inputs.key, inputs.query)
            self.buffer.write(slots, index_keys)
            return index_queries, index_keys
        if self.writes_pool:
            self.buffer.write(slots, inputs.key)
        return self.projection.index_queries(inputs.query), self.projection.index_keys(inputs.key)

    def write(self, inputs: KeyAndQuery, slots: torch.Tensor) -> torch.Tensor:
        """Write new tokens' keys at their KV slots and return their index queries."""
        if inputs.key.shape[0] != slots.shape[0]:
            raise ValueError(f"the key and query input has {inputs.key.shape[0]} keys for {slots.shape[0]} slots")
        if self.projection.split is not None:
            return self.project(inputs, slots)[0]
        if self.writes_pool:
            self.buffer.write(slots, inputs.key)
        return self.projection.index_queries(inputs.query)

    def write_chunk(self, inputs: KeyAndQuery, slots: torch.Tensor) -> None:
        """Write a prefill chunk's keys without selecting: a short prompt the dense path prefills. The next
        `maintain` indexes them from the pool."""
        if self.projection.split is not None:
            self.project(inputs, slots)
        else:
            self.buffer.write(slots, inputs.key)

    def keys_of(self, row: int, chunk: tuple | None = None) -> KeyLookup:
        return KeyLookup(self.buffer, self.slot_table, row, chunk)

    # ---- a forward

    def maintain(self, rids: Sequence, rows: Sequence, ends: Sequence) -> int:
        """Bring each request's cache up to the keys already in the pool, eagerly, before a forward."""
        closed = self.selector.maintain(rids, rows, ends, self.keys_of)
        self.check(rows)
        return closed

    def check(self, rows: Sequence) -> None:
        """Raise unless every rank of the decode group holds the same index for the requests, when asked to check
        (`layer_index.py:776-784`)."""
        if self.check_index and self.shard.reduce is not None:
            from lsa_b200.sglang.consistency import check_same_index
            check_same_index(self.selector.cache, rows, self.shard.reduce, self.shard.size)

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
        self.check(rows)
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
