"""The serving index of a batch of requests over paged memory: a bucket cache and its selector.

A small, engine-free counterpart of the reference's `BucketCache` and `Selector`
(`src/lsa/sglang/index/bucket_cache.py:70-601`, `src/lsa/sglang/index/selector.py:107-700`): a model hands the selector
each request's index keys as they arrive and its page tables, and takes back lists of KV slots.

  - Buckets live in pages of `page_buckets` rows of one device table (centroids, members, sizes). A request owns a
    list of pages; its logical bucket i is row i % page_buckets of its page i / page_buckets. Pages come from a host
    free list and go back when a request is released, so the device tables never move.
  - Positions are a request's own (0 .. length); a KV slot is `kv_pages[request, pos / kv_page] * kv_page + pos % kv_page`
    (the engine's `req_to_token` table in page form). The reference serves with single-token pages only
    (`src/lsa/sglang/models/qwen3_5/backend.py:290-294`); any page size works here because the expansion maps each
    position itself.
  - Decode is fixed-shape and reads no device value on the host: one paged scan, one expansion, one split
    attention with its merge.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from lsa_b200 import ops, probe
from lsa_b200.layer import FlatDesign


@dataclass
class Retained:
    """A finished request's leading full pages and their fingerprints, kept for a request that shares them
    (bucket_cache.py:60-67)."""

    pages: list
    prints: list
    seen: int


def fingerprints_of(lookup, first: int, count: int) -> list:
    """The fingerprints of a request's pages [first, first + count), by the lookup's own read (bucket_cache.py:43-57).

    Raises:
        TypeError: The lookup reads no fingerprints, which prefix reuse needs.
    """
    fingerprints = getattr(lookup, "fingerprints", None)
    if fingerprints is None:
        raise TypeError("prefix reuse fingerprints pages from the pool, and this lookup reads none")
    return fingerprints(first, count) if count > 0 else []


class BucketCache:
    """Paged store of every request's buckets (bucket_cache.py:70-140).

    Under `reuse` - the server's prefix cache on - a request that arrives with a cached prefix takes the index pages of
    that prefix instead of building them again (bucket_cache.py:11-19): a full page's buckets are its own keys' alone
    and never change once full, so a page is shared between requests by a count of its holders. A request fingerprints
    each of its full pages from the pool once its keys are all there; when its row goes to another request, its leading
    fingerprinted pages are kept as a `Retained` prefix rather than freed. A new request fingerprints its own leading
    pages and takes the longest run that matches, from a retained prefix or a running request. Retained prefixes go
    first when pages run short."""

    def __init__(self, design: FlatDesign, index_dim: int, pages: int, page_buckets: int, max_requests: int,
                 max_request_pages: int, device="cuda", reuse: bool = False):
        self.design, self.page_buckets = design, page_buckets
        self.reuse = reuse
        self.holders = [0] * pages          # requests and retained prefixes that hold each page
        self.prints: dict[int, list] = {}   # request -> fingerprints of its leading full pages
        self.retained: list[Retained] = []
        self.clock = 0                      # ticks once a release or a batch: which prefix, which request is oldest
        self.seen: dict[int, int] = {}      # request -> the tick of the last batch that named it
        self.active: set = set()            # the requests of the running batch, whose pages are never reclaimed
        rows = pages * page_buckets
        self.centroids = torch.zeros(rows, index_dim, device=device, dtype=torch.float32)
        self.members = torch.full((rows, design.bucket_cap), -1, device=device, dtype=torch.int32)
        self.sizes = torch.zeros(rows, device=device, dtype=torch.int32)
        self.request_pages = torch.full((max_requests, max_request_pages), -1, device=device, dtype=torch.int32)
        # Buckets each request holds, where a captured decode step can read it
        self.bucket_counts = torch.zeros(max_requests, device=device, dtype=torch.int32)
        # Under `bucket_shape` each bucket also keeps its shape, built as its cluster block closes, in the row that
        # holds its centroid (bucket_cache.py:8-10,108-116)
        self.bucket_shapes: ops.ShapeTable | None = None
        if design.bucket_shape is not None:
            rank = design.bucket_shape.rank
            self.bucket_shapes = ops.ShapeTable(
                torch.zeros(rows, rank, index_dim // 8, device=device, dtype=torch.uint8),
                torch.zeros(rows, rank, device=device), torch.zeros(rows, device=device),
                design.bucket_shape.deviations)
        self.free_pages = list(range(pages - 1, -1, -1))
        self.held: dict[int, list] = {}      # request -> its pages, in order
        self.closed_keys: dict[int, int] = {}  # request -> keys of its closed cluster blocks
        self.pending: dict[int, torch.Tensor] = {}  # request -> index keys of its open block
        self.owner: dict[int, object] = {}   # request table row -> the id of the request that holds it

    def buckets_of(self, request: int) -> int:
        return self.closed_keys.get(request, 0) // self.design.bucket_size

    def end(self, request: int) -> int:
        """Keys of the request the cache has taken: its closed cluster blocks and the open one."""
        held = self.pending.get(request)
        return self.closed_keys.get(request, 0) + (0 if held is None else held.shape[0])

    @property
    def page_keys(self) -> int:
        """Keys whose buckets fill a page."""
        return self.page_buckets * self.design.bucket_size

    def let_go(self, pages: list) -> None:
        """Drop one holder of each page, freeing those no one holds any longer (bucket_cache.py:237-250)."""
        freed = []
        for page in pages:
            self.holders[page] -= 1
            if not self.holders[page]:
                freed.append(page)
        self.free_pages.extend(reversed(freed))

    def release(self, request: int, retain: bool = True) -> None:
        """Give a finished request's pages back - but for its leading fingerprinted pages, under `reuse`, which stay
        as a retained prefix for a request that shares them (bucket_cache.py:196-235)."""
        pages = self.held.pop(request, [])
        prints = self.prints.pop(request, [])
        self.clock += 1
        if self.reuse and retain and prints:
            self.retained.append(Retained(pages[:len(prints)], prints, self.clock))  # (the holder's count goes along)
            pages = pages[len(prints):]
        self.let_go(pages)
        self.seen.pop(request, None)
        self.closed_keys.pop(request, None)
        self.pending.pop(request, None)
        self.owner.pop(request, None)
        self.request_pages[request].fill_(-1)
        self.bucket_counts[request] = 0

    def ensure(self, request: int, rid: object) -> None:
        """Start a row of the request table afresh when another request has taken it (bucket_cache.py:228-262)."""
        if self.owner.get(request, rid) != rid or (request not in self.owner and self.end(request)):
            self.release(request)
        self.owner[request] = rid
        self.seen[request] = self.clock

    def running(self, requests) -> None:
        """Name the requests of the batch about to run: finished requests keep their pages until their row is given
        to another or pages run short, and a running one is never the one to give them up (bucket_cache.py:333-378)."""
        self.clock += 1
        self.active = set(int(request) for request in requests)

    def advance(self, request: int, end: int, index_keys_of) -> int:
        """Bring the request up to `end` keys: the index keys of the positions the cache has not seen come from
        `index_keys_of(first, stop)` [stop - first, index_dim] fp32 (bucket_cache.py:380-441). Returns the cluster
        blocks closed.

        Raises:
            ValueError: The cache already holds keys past `end` (a request cut short keeps no index).
        """
        have = self.end(request)
        if end < have:
            raise ValueError(f"request {request} holds {have} keys in its index and the pool {end}")
        return self.append(request, index_keys_of(have, end)) if end > have else 0

    def adopt(self, request: int, end: int, lookup) -> int:
        """Take the longest run of leading pages another request indexed from the same keys, under `reuse`
        (bucket_cache.py:257-316). Only a request that holds nothing yet takes one - one just admitted with a cached
        prefix of a page or more. The candidates are the retained prefixes and the requests holding fingerprinted
        pages; a page matches when its fingerprint does, every page before it having matched. `lookup.fingerprints(
        first, count)` reads the request's own pages from the pool. Returns the pages taken.

        Raises:
            TypeError: The lookup reads no fingerprints.
        """
        page_keys = self.page_keys
        if not self.reuse or self.end(request) or end < page_keys:
            return 0
        donors = [(entry.pages, entry.prints) for entry in self.retained] + \
            [(self.held[other][:len(found)], found) for other, found in self.prints.items() if other != request and found]
        if not donors:
            return 0
        prints = fingerprints_of(lookup, 0, 1)
        donors = [donor for donor in donors if donor[1][0] == prints[0]]
        if not donors:
            return 0
        longest = min(end // page_keys, max(len(donor[1]) for donor in donors))
        prints += fingerprints_of(lookup, 1, longest - 1)

        def matched(theirs: list) -> int:
            count = 0
            while count < min(len(theirs), longest) and theirs[count] == prints[count]:
                count += 1
            return count

        pages, theirs = max(donors, key=lambda donor: matched(donor[1]))
        count = matched(theirs)
        if count > self.request_pages.shape[1]:
            raise RuntimeError(f"request {request} needs {count} index pages and a request holds at most "
                               f"{self.request_pages.shape[1]}")
        pages = list(pages[:count])
        for page in pages:
            self.holders[page] += 1
        self.held[request] = pages
        self.prints[request] = prints[:count]
        self.request_pages[request, :count] = torch.tensor(pages, dtype=torch.int32, device=self.request_pages.device)
        self.closed_keys[request] = count * page_keys
        self.bucket_counts[request] = count * self.page_buckets
        return count

    def fingerprint(self, request: int, end: int, lookup) -> None:
        """Fingerprint the request's full pages whose keys have all reached the pool, under `reuse`
        (bucket_cache.py:318-331)."""
        if not self.reuse:
            return
        full = min(self.closed_keys.get(request, 0), end) // self.page_keys
        taken = self.prints.setdefault(request, [])
        if full > len(taken):
            taken += fingerprints_of(lookup, len(taken), full - len(taken))

    def reclaim(self, asking: int | None = None) -> None:
        """Drop retained prefixes, oldest first, then release the idle requests seen longest ago, until a page is
        free (bucket_cache.py:252-255,355-378). `asking` is the request that needs the page.

        Raises:
            RuntimeError: Every page belongs to a running request.
        """
        while self.retained and not self.free_pages:
            oldest = min(range(len(self.retained)), key=lambda index: self.retained[index].seen)
            self.let_go(self.retained.pop(oldest).pages)
        idle = [request for request, pages in self.held.items()
                if pages and request != asking and request not in self.active]
        for request in sorted(idle, key=lambda request: self.seen.get(request, 0)):
            if self.free_pages:
                break
            self.release(request, retain=False)
        if not self.free_pages:
            raise RuntimeError("the bucket cache is out of pages - every page belongs to a running request")

    def rows_of(self, request: int, logical: torch.Tensor) -> torch.Tensor:
        """Rows of the device tables that hold a request's logical buckets."""
        return self.request_pages[request][logical // self.page_buckets].long() * self.page_buckets + \
            logical % self.page_buckets

    def gather(self, request: int, buckets: int) -> torch.Tensor:
        """The centroids of a request's first `buckets` buckets, side by side [buckets, index_dim] fp32
        (bucket_cache.py:560-601)."""
        logical = torch.arange(buckets, device=self.centroids.device)
        return self.centroids[self.rows_of(request, logical)]

    def gather_shapes(self, request: int, buckets: int) -> ops.ShapeTable | None:
        """The shapes of the buckets `gather` returns, row for row, or None when buckets are not shaped
        (bucket_cache.py:455-466)."""
        if self.bucket_shapes is None:
            return None
        logical = torch.arange(buckets, device=self.centroids.device)
        return self.bucket_shapes.rows(self.rows_of(request, logical))

    def _grow(self, request: int, buckets: int) -> None:
        pages = self.held.setdefault(request, [])
        need = -(-buckets // self.page_buckets)
        if need > self.request_pages.shape[1]:
            raise RuntimeError(f"request {request} needs {need} index pages and a request holds at most "
                               f"{self.request_pages.shape[1]}")
        fresh = []
        while len(pages) < need:
            if not self.free_pages:
                self.reclaim(request)
            fresh.append(self.free_pages.pop())
            self.holders[fresh[-1]] = 1
            pages.append(fresh[-1])
        if fresh:
            first = len(pages) - len(fresh)
            self.request_pages[request, first:len(pages)] = torch.tensor(fresh, dtype=torch.int32,
                                                                         device=self.request_pages.device)

    def append(self, request: int, index_keys: torch.Tensor) -> int:
        """Take a request's next index keys [n, index_dim] (fp32 unit rows, in position order); cluster every
        cluster block that closes and write its buckets into the request's pages. Returns the blocks closed."""
        d = self.design
        held = self.pending.get(request)
        keys = index_keys if held is None else torch.cat([held, index_keys])
        blocks = keys.shape[0] // d.cluster_block_size
        closed = blocks * d.cluster_block_size
        self.pending[request] = keys[closed:]
        if not blocks:
            return 0
        first_position = self.closed_keys.get(request, 0)
        first_bucket = first_position // d.bucket_size
        per_block = d.block_bucket_count
        self._grow(request, first_bucket + blocks * per_block)
        with probe.region("index k cluster"):
            block_keys = keys[:closed].contiguous()
            pools = ops.pool_keys(block_keys.view(blocks, d.cluster_block_size, -1), d.pool_size)
            labels, _ = ops.ward_rounds(pools, float(d.pool_size), per_block, d.bucket_cap)
            members, sizes, _, centroids, _, _ = ops.bucket_table(block_keys, labels, d.pool_size, per_block,
                                                                  d.bucket_cap, first_position=first_position)
        rows = self.rows_of(request, first_bucket + torch.arange(blocks * per_block, device=members.device))
        self.centroids[rows] = centroids
        self.members[rows] = members
        self.sizes[rows] = sizes
        if self.bucket_shapes is not None:  # (bucket_cache.py:603-627; members are positions from `first_position`)
            with probe.region("bucket shapes"):
                built = ops.shape_build(block_keys, centroids, members, d.bucket_shape.rank, key_base=first_position)
            self.bucket_shapes.basis[rows] = built.basis
            self.bucket_shapes.variances[rows] = built.variances
            self.bucket_shapes.floor[rows] = built.floor
        self.closed_keys[request] = first_position + closed
        self.bucket_counts[request] = first_bucket + blocks * per_block
        return blocks


class Selector:
    """Routes a batch's reads over a `BucketCache` (selector.py:107-700), flat design."""

    scan_rows = 1024  # from this many rows on, a prefill segment's scan runs on the tensor cores

    def __init__(self, cache: BucketCache, kv_page_size: int = 1, slot_table=None):
        """`slot_table()` returns the request table [requests, context / kv_page_size] int32 that maps a request's
        positions to KV slots (an engine's `req_to_token` has pages of one token); `prefill` and `decode` read
        through it, `decode_flat` is handed a batch's own table."""
        self.cache, self.kv_page_size, self.slot_table = cache, kv_page_size, slot_table

    def maintain(self, rids, rows, ends, index_keys_of) -> int:
        """Bring each request's cache up to the keys already in the KV pool - eagerly, before every forward
        (selector.py:162-197). `index_keys_of(row)` returns the row's lookup (first, stop) -> index keys. Returns
        the cluster blocks closed."""
        closed = 0
        self.cache.running(rows)
        for rid, row, end in zip(rids, rows, ends, strict=True):
            self.cache.ensure(row, rid)
            lookup = index_keys_of(row)
            self.cache.adopt(row, end, lookup)
            closed += self.cache.advance(row, end, lookup)
            self.cache.fingerprint(row, end, lookup)
        return closed

    def prefill(self, row: int, index_queries: torch.Tensor, positions: torch.Tensor, index_keys: torch.Tensor,
                query_start: int, local: bool = True) -> torch.Tensor:
        """Read a prefill segment of one request: append its keys, select for its queries (selector.py:199-287).

        The keys go into the cache in one call and every query reads the buckets its own position sees - those of
        the cluster blocks closed before it - which is what it would have seen had the cache grown a page at a time,
        so nothing is cut at page ends.

        Args:
            row: The request table row.
            index_queries: The segment's index queries [S, index_dim] fp32 unit rows.
            positions: Their positions [S], consecutive from `query_start`.
            index_keys: The index keys the cache appends [S', index_dim] fp32, from the cache's end (S' >= S where
                the segment's keys reach back before its first query).
            query_start: Position of the first query, from the scheduler: no device read.

        Returns:
            KV slots [S, width] int32, -1 padded, valid entries first.

        Raises:
            ValueError: The keys do not reach the last query.
        """
        cache, d = self.cache, self.cache.design
        S, dev = index_queries.shape[0], index_queries.device
        cache.append(row, index_keys)
        if cache.end(row) < query_start + S:
            raise ValueError(f"request {row}'s index ends at key {cache.end(row)} and its queries at {query_start + S}")
        if not S:
            return torch.empty(0, d.list_width, device=dev, dtype=torch.int32)
        last = query_start + S - 1
        seen = min(last // d.cluster_block_size * d.block_bucket_count, cache.buckets_of(row))
        positions = positions.to(torch.int64)
        visible = (positions // d.cluster_block_size * d.block_bucket_count).clamp_max(seen).to(torch.int32)
        with probe.region("index q scan"):
            centroids = cache.gather(row, seen)
            if cache.bucket_shapes is not None:
                _, picked = ops.shaped_select(index_queries, centroids, cache.gather_shapes(row, seen), visible,
                                              d.top_p)
            elif S >= self.scan_rows and centroids.shape[1] == 64 and d.top_p <= 512:
                operand, lengths, radius = ops.scan_centre(centroids, centroids.mean(0))
                _, picked = ops.scan_select(index_queries, centroids, operand, visible, d.top_p, max_visible=seen,
                                            lengths=lengths, radius=radius)
            else:
                _, picked = ops.flat_select(index_queries, centroids, visible, d.top_p)
        with probe.region("expand"):
            table = self.slot_table()
            lists, _, _ = ops.expand_batched(picked, positions, None, cache.members, cache.request_pages[row:row + 1],
                                             cache.page_buckets, table[row:row + 1], self.kv_page_size, d.top_k,
                                             d.sink_size, d.window_size, local=local)
        return lists

    def decode(self, index_queries: torch.Tensor, positions: torch.Tensor, rows: torch.Tensor, splits: int = 4,
               local: bool = True) -> torch.Tensor:
        """One query a request, read through the request table: KV slots [B, width] int32 (selector.py:603-700).
        Fixed shapes and no host read, so a step can be captured in a CUDA graph."""
        cache, d = self.cache, self.cache.design
        rows = rows.long()
        positions = positions.to(torch.int64)
        visible = torch.minimum(positions // d.cluster_block_size * d.block_bucket_count,
                                cache.bucket_counts[rows].long())
        pages = cache.request_pages[rows]
        limit = self.captured_limit()
        if limit is not None and -(-limit // cache.page_keys) < pages.shape[1]:
            # A graph captured for contexts up to `limit`: no request of it has a bucket past the range's pages, and
            # a padded row of the graph may name a longer one, so its count is cut to the range (selector.py:620-627)
            held = -(-limit // cache.page_keys)
            pages = pages[:, :held]
            visible = visible.clamp(max=held * cache.page_buckets)
        visible = visible.to(torch.int32)
        with probe.region("index q scan"):
            _, picked = self._scan_paged(index_queries, pages, visible, splits)
        with probe.region("expand"):
            lists, _, _ = ops.expand_batched(picked, positions, rows.to(torch.int32), cache.members,
                                             cache.request_pages, cache.page_buckets, self.slot_table(),
                                             self.kv_page_size, d.top_k, d.sink_size, d.window_size, local=local)
        return lists

    @staticmethod
    def captured_limit() -> int | None:
        """The longest context of the decode graph being captured, when an engine captures one graph a context range
        (`lsa_b200.sglang.context_buckets`); None otherwise."""
        from lsa_b200.sglang import context_buckets

        return context_buckets.captured_limit()

    def _scan_paged(self, index_queries: torch.Tensor, pages: torch.Tensor, visible: torch.Tensor, splits: int):
        """A decode step's scan through the requests' page tables: by centroid, or under `bucket_shape` by each
        bucket's estimated best key (selector.py:603-660)."""
        cache = self.cache
        if cache.bucket_shapes is not None:
            return ops.shaped_select_paged(index_queries, cache.centroids, cache.bucket_shapes, pages, visible,
                                           cache.page_buckets, cache.design.top_p, splits=splits)
        return ops.flat_select_paged(index_queries, cache.centroids, pages, visible, cache.page_buckets,
                                     cache.design.top_p, splits=splits)

    def visible(self, request_rows: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """Buckets each row sees: those of the cluster blocks closed before its own, that the cache holds."""
        d = self.cache.design
        held = torch.tensor([self.cache.buckets_of(int(r)) for r in request_rows.tolist()], device=positions.device)
        return torch.minimum(positions // d.cluster_block_size * d.block_bucket_count, held).to(torch.int32)

    def decode_flat(self, index_queries: torch.Tensor, request_rows: torch.Tensor, positions: torch.Tensor,
                    kv_pages: torch.Tensor, visible: torch.Tensor | None = None, splits: int = 4,
                    local: bool = True):
        """Lists of KV slots [B, top_k + window + sink] int32 (-1 padded, valid first) and their lengths for one
        query a request (selector.py:603-700). `visible` may be passed in to keep the step free of host work."""
        cache, d = self.cache, self.cache.design
        visible = self.visible(request_rows, positions) if visible is None else visible
        pages = cache.request_pages[request_rows.long()]
        with probe.region("index q scan"):
            _, picked = self._scan_paged(index_queries, pages, visible, splits)
        with probe.region("expand"):
            rows = torch.arange(request_rows.shape[0], device=picked.device, dtype=torch.int32)
            lists, lengths, _ = ops.expand_batched(picked, positions, rows, cache.members, pages, cache.page_buckets,
                                                   kv_pages, self.kv_page_size, d.top_k, d.sink_size, d.window_size,
                                                   local=local)
        return lists, lengths
