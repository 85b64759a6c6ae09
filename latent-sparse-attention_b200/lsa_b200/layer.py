"""One LSA global-attention layer, flat design: index build, selection and the sparse read strung together.

This is the call a serving backend makes per layer (the reference's `LayerIndex.extend` followed by
`select_and_read`, src/lsa/sglang/index/layer_index.py:824-882 and src/lsa/sglang/models/qwen3_5/backend.py:784-822),
for a single request whose KV rows sit at their positions.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from lsa_b200 import _lib, ops, probe
from lsa_b200.budget import EarlyBudget
from lsa_b200.core import Buckets, RotaryLayout, check_sizes
from lsa_b200.shape import Shape


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
    bucket_shape: Shape | None = None  # buckets keep their spread and score as their estimated best key

    def __post_init__(self) -> None:
        check_sizes(self.pool_size, self.bucket_size, self.bucket_cap, self.cluster_block_size)
        object.__setattr__(self, "bucket_shape", Shape.read("bucket_shape", self.bucket_shape))
        if self.bucket_shape is not None and self.bucket_shape.rank > self.bucket_cap:
            raise ValueError(f"bucket_shape keeps at most bucket_cap {self.bucket_cap} directions - got rank "
                             f"{self.bucket_shape.rank}")
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
    """A request's index: its index keys and the buckets of its closed cluster blocks (and, where the tensor-core
    scan can use it, its operand: the centroids less a common centre in bf16, and the greatest length of one)."""

    def __init__(self, index_keys: torch.Tensor, buckets: Buckets, centroids_bf16: torch.Tensor | None = None,
                 lengths: torch.Tensor | None = None, radius: torch.Tensor | None = None,
                 shapes: ops.ShapeTable | None = None):
        self.index_keys = index_keys
        self.buckets = buckets
        self.centroids_bf16 = centroids_bf16
        self.lengths, self.radius = lengths, radius
        self.shapes = shapes  # the buckets' shapes, row for row, under a design with `bucket_shape`


class FlatLayer:
    """Prefill and decode of one layer. `query_map` / `key_map` are [Hkv * (dh - rotary), index_dim]."""

    def __init__(self, design: FlatDesign, query_map: torch.Tensor, key_map: torch.Tensor, heads: int, kv_heads: int,
                 head_dim: int, rotary: RotaryLayout = RotaryLayout(), scale: float | None = None,
                 tensor_cores: bool = True):
        if heads % kv_heads:
            raise ValueError(f"query heads must group evenly - {heads} does not divide by {kv_heads}")
        free = head_dim - rotary.dim
        if query_map.shape != key_map.shape or query_map.shape[0] != kv_heads * free:
            raise ValueError(f"the maps must both be [{kv_heads * free}, index_dim] - got {tuple(query_map.shape)} "
                             f"and {tuple(key_map.shape)}")
        self.design = design
        self.index_dim = key_map.shape[1]
        self.query_map, self.key_map = query_map.contiguous(), key_map.contiguous()
        self.heads, self.kv_heads, self.head_dim = heads, kv_heads, head_dim
        self.dh_off = rotary.dim if rotary.end == "prefix" else 0
        self.dh_used = free
        self.scale = head_dim ** -0.5 if scale is None else scale
        self._buffers: dict = {}
        # What the kernels report from the device, read by `check()`: bounded waits of the map kernels that gave up,
        # buckets over their cap in the table, bad picks in the expansion, bounded waits of the attention kernels.
        self._status_slots(query_map.device)
        self._reached: list = []  # per index build: whether each cluster block merged down to its bucket count
        # The bucket-major attend pass has two forms: (pair, head) rows as the M = 128 side of tcgen05 products with S
        # and O in tensor memory (the default), or warp-level MMA tiles of 16 rows.
        self.bucket_tensor_memory = True
        self._band_stream = self._band_done = None  # the side stream the band runs on beside the bucket-major read
        self._copy_in = self._copy_out = self._index_stream = None  # the side streams of `prefill_from_host`
        self._copy_events: list = []
        # bf16 maps run on the tensor cores (the head sum folded into the product); fp32 maps keep the exact form
        self.tensor_cores = tensor_cores and query_map.dtype == torch.bfloat16 and key_map.dtype == torch.bfloat16 \
            and query_map.shape[1] in (32, 64, 128)
        if self.tensor_cores:
            self.query_map_t = ops.expand_map(self.query_map, heads, heads // kv_heads, head_dim, self.dh_off,
                                              self.dh_used)
            self.key_map_t = ops.expand_map(self.key_map, kv_heads, 1, head_dim, self.dh_off, self.dh_used)

    def _status_slots(self, device) -> None:
        """The layer's deferred-status words: index map, bucket table, expansion, attention, bucket scan."""
        self.status = torch.zeros(5, device=device, dtype=torch.int32)
        self._map_status, self._table_status = self.status[0:1], self.status[1:2]
        self._expand_status, self._attend_status = self.status[2:3], self.status[3:4]
        self._scan_status = self.status[4:5]

    def check(self) -> None:
        """The deferred checks of everything launched since the last call: ONE host synchronisation, so a hot path
        calls it once a prefill (or once a benchmark) rather than after every kernel. Raises `ValueError` when a
        cluster block stopped short of its bucket count or a bucket overflowed its cap (what `core.build_buckets`
        raises at once, src/lsa/core/reference.py:131, ward.py:118-122) and `RuntimeError` when a bounded on-chip
        wait gave up, in which case the outputs since the last check are void."""
        counts = self.status.tolist()
        short = sum(int((~r.bool()).sum()) for r in self._reached)
        self.status.zero_()
        self._reached.clear()
        if short or counts[1]:
            raise ValueError(f"{short} cluster blocks stopped short of {self.design.block_bucket_count} buckets under "
                             f"the cap {self.design.bucket_cap}; {counts[1]} buckets overflowed it")
        if counts[2]:
            raise ValueError(f"{counts[2]} picked bucket ids lay outside the member table")
        if counts[0] or counts[3] or counts[4]:
            raise RuntimeError(f"bounded on-chip waits gave up ({counts[0]} in the index map, {counts[3]} in the "
                               f"attention kernels, {counts[4]} in the bucket scan): the outputs since the last "
                               "check are void")

    # ---- buffers

    def _buffer(self, name: str, shape: tuple, dtype: torch.dtype, device) -> torch.Tensor:
        """A tensor that lives as long as the layer: a step allocates nothing once every shape has been seen."""
        key = (name, tuple(shape), dtype, str(device))
        held = self._buffers.get(key)
        if held is None:
            held = self._buffers[key] = torch.empty(shape, device=device, dtype=dtype)
        return held

    def _takes_tensor_cores(self, x: torch.Tensor) -> bool:
        """Heads packed densely in bf16 with a 16-byte aligned row pitch: the layout a TMA descriptor can walk."""
        # (a handful of rows - a decode step - goes to the kernel that splits one row's contraction over a CTA)
        return (self.tensor_cores and x.shape[0] > 32 and x.dtype == torch.bfloat16 and x.stride(2) == 1
                and x.stride(1) == x.shape[2]
                and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0)

    # ---- the stages

    def index_queries(self, q: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """q [T, Hq, dh] bf16 -> unit index queries [T, index_dim] fp32."""
        if self._takes_tensor_cores(q):
            return ops.index_map_tc(q, self.query_map_t, out=out, status=self._map_status)
        return ops.index_map(q, self.query_map, group=self.heads // self.kv_heads, dh_off=self.dh_off,
                             dh_used=self.dh_used, out=out)

    def index_queries_rows(self, q: torch.Tensor) -> torch.Tensor:
        """The same map for the few rows of a decode step, q [R <= 8, Hq, dh] bf16: a kernel that spreads one row's
        contraction over many CTAs (with bf16 maps; other maps take `index_queries`)."""
        if self.tensor_cores and q.shape[0] <= 8 and q.dtype == torch.bfloat16 and q.stride(2) == 1 \
                and q.stride(1) == q.shape[2]:
            return ops.rows_linear(q, self.query_map_t, normalize=True)
        return self.index_queries(q)

    def index_keys(self, k: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """k [T, Hkv, dh] bf16 -> unit index keys [T, index_dim] fp32."""
        if self._takes_tensor_cores(k):
            return ops.index_map_tc(k, self.key_map_t, out=out, status=self._map_status)
        return ops.index_map(k, self.key_map, group=1, dh_off=self.dh_off, dh_used=self.dh_used, out=out)

    def build_index(self, k: torch.Tensor, reuse_buffers: bool = False) -> FlatIndex:
        """Index keys, then pools, Ward and the bucket table of every closed cluster block.

        With `reuse_buffers` the index lives in the layer's own buffers and is overwritten by the next build.
        """
        bufs = self._index_buffers(k.shape[0], k.device, reuse_buffers)
        self._build_blocks(k, 0, bufs)
        return self._index_of(bufs)

    def _index_buffers(self, T: int, dev, reuse_buffers: bool) -> dict:
        """The tensors an index over T keys lives in (the layer's own buffers, or fresh ones)."""
        d, d_idx = self.design, self.index_dim
        blocks = T // d.cluster_block_size
        P, rows = d.cluster_block_size // d.pool_size, blocks * d.block_bucket_count
        make = (lambda name, shape, dtype: self._buffer(name, shape, dtype, dev)) if reuse_buffers else \
            (lambda name, shape, dtype: torch.empty(shape, device=dev, dtype=dtype))
        bufs = {"keys": make("index keys", (T, d_idx), torch.float32),
                "pools": make("pools", (blocks, P, d_idx), torch.float32),
                "labels": make("labels", (blocks, P), torch.int64), "reached": make("reached", (blocks,), torch.uint8),
                "status": self._table_status,
                "members": make("members", (rows, d.bucket_cap), torch.int32), "sizes": make("sizes", (rows,), torch.int32),
                "key sums": make("key sums", (rows, d_idx), torch.float32),
                "centroids": make("centroids", (rows, d_idx), torch.float32)}
        if d_idx == 64:  # (the operand of the tensor-core scan: centroids less the first blocks' mean, in bf16)
            bufs["centroids bf16"] = make("centroids bf16", (rows, d_idx), torch.bfloat16)
            bufs["centre"], bufs["radius"] = make("centre", (d_idx,), torch.float32), make("radius", (1,), torch.float32)
            bufs["lengths"] = make("operand lengths", (rows,), torch.float32)
            bufs["radius"].zero_()
            bufs["centred"] = [False]
        if d.bucket_shape is not None:
            if d_idx not in (32, 64):
                raise ValueError(f"bucket shapes are built over index keys of 32 or 64 dims - got {d_idx}")
            rank = d.bucket_shape.rank
            bufs["shapes"] = ops.ShapeTable(make("shape basis", (rows, rank, d_idx // 8), torch.uint8),
                                            make("shape variances", (rows, rank), torch.float32),
                                            make("shape floor", (rows,), torch.float32), d.bucket_shape.deviations)
        return bufs

    def _index_of(self, bufs: dict) -> FlatIndex:
        d = self.design
        return FlatIndex(bufs["keys"], Buckets(bufs["centroids"], bufs["members"], bufs["sizes"], d.block_bucket_count,
                                               d.cluster_block_size), bufs.get("centroids bf16"), bufs.get("lengths"),
                         bufs.get("radius"), bufs.get("shapes"))

    def _build_blocks(self, k: torch.Tensor, first: int, bufs: dict) -> None:
        """Index keys of k [n, ...] = the keys at positions first.., and the pools, Ward labels and bucket table of
        the cluster blocks they close (first is a multiple of the block size): blocks are independent, so an index
        can be built as its keys arrive."""
        d = self.design
        n = k.shape[0]
        with probe.region("index map"):
            self.index_keys(k, out=bufs["keys"][first:first + n])
        self._cluster_blocks(first // d.cluster_block_size, n // d.cluster_block_size, bufs)

    def _cluster_blocks(self, b0: int, nb: int, bufs: dict) -> None:
        """Pools, Ward labels and the bucket table of cluster blocks b0 .. b0 + nb - 1, whose index keys are in place."""
        d = self.design
        if nb <= 0:
            return
        first = b0 * d.cluster_block_size
        r0, r1 = b0 * d.block_bucket_count, (b0 + nb) * d.block_bucket_count
        keys = bufs["keys"][first:first + nb * d.cluster_block_size]
        with probe.region("pool"):
            pools = ops.pool_keys(keys.view(nb, d.cluster_block_size, -1), d.pool_size, out=bufs["pools"][b0:b0 + nb])
        with probe.region("ward"):
            labels, _ = ops.ward_rounds(pools, float(d.pool_size), d.block_bucket_count, d.bucket_cap,
                                        labels=bufs["labels"][b0:b0 + nb], reached=bufs["reached"][b0:b0 + nb])
            if len(self._reached) < 64:  # (views of the index buffers; `check()` reads and drops them)
                self._reached.append(bufs["reached"][b0:b0 + nb])
        with probe.region("bucket table"):
            outs = (bufs["members"][r0:r1], bufs["sizes"][r0:r1], bufs["key sums"][r0:r1], bufs["centroids"][r0:r1],
                    None, bufs["status"])
            ops.bucket_table(keys, labels, d.pool_size, d.block_bucket_count, d.bucket_cap, first_position=first,
                             outs=outs)
            if "centroids bf16" in bufs:
                # Any centre leaves the ranking as it is; the mean of the first blocks' centroids is where the cone
                # of this layer's index vectors points, and the closer to it the rows lie, the sharper the scan.
                if not bufs["centred"][0]:
                    bufs["centre"].copy_(bufs["centroids"][r0:r1].mean(0))
                    bufs["centred"][0] = True
                ops.scan_centre(bufs["centroids"][r0:r1], bufs["centre"], bufs["centroids bf16"][r0:r1],
                                bufs["lengths"][r0:r1], bufs["radius"])
        if "shapes" in bufs:  # (members are positions: the keys of these blocks start at `first`)
            with probe.region("bucket shapes"):
                ops.shape_build(keys, bufs["centroids"][r0:r1], bufs["members"][r0:r1], d.bucket_shape.rank,
                                key_base=first, out=bufs["shapes"].rows(slice(r0, r1)))

    scan_rows = 1024  # from this many rows on, a pick runs its scan on the tensor cores

    def pick(self, index_queries: torch.Tensor, positions: torch.Tensor, index: FlatIndex,
             reuse_buffers: bool = False, last_position: int | None = None):
        """The top-p buckets of every row, best first: (picked [R, top_p] int32, positions int64, and the rows' own
        budgets under an early budget, else None). `last_position` is the host's bound on `positions`, if it has
        one (it places the samples of the tensor-core scan; the result does not depend on it)."""
        d, b, dev = self.design, index.buckets, index_queries.device
        R = index_queries.shape[0]
        positions = positions.to(torch.int64)
        visible = (positions // d.cluster_block_size * d.block_bucket_count).clamp_max(
            b.bucket_centroids.shape[0]).to(torch.int32)
        row_p = row_k = None
        if d.early_budget is not None:
            early = positions < d.early_budget.position
            row_p = torch.where(early, d.early_budget.top_p, d.top_p).to(torch.int32)
            row_k = torch.where(early, d.early_budget.top_k, d.top_k).to(torch.int32)
        keys = picked = None
        if reuse_buffers:
            keys = self._buffer("keys", (R, d.top_p), torch.int64, dev)
            picked = self._buffer("picked", (R, d.top_p), torch.int32, dev)
        with probe.region("select"):
            bound = 0 if last_position is None else last_position // d.cluster_block_size * d.block_bucket_count
            bound = min(bound or b.bucket_centroids.shape[0], b.bucket_centroids.shape[0])
            # (the scan's threshold rests on 512 samples of a row's scores: it needs a thousand buckets in sight, and
            # the kept ones to be a fair share of them - else the exact scan, at once)
            if index.shapes is not None:  # a bucket scores as its estimated best key: the exact scan, shaped
                _, picked = ops.shaped_select(index_queries, b.bucket_centroids, index.shapes, visible, d.top_p, row_p,
                                              keys=keys, picked=picked)
            elif index.centroids_bf16 is not None and R >= self.scan_rows and d.top_p <= 512 and bound >= 1024 \
                    and 3 * d.top_p * 512 >= 8 * bound:
                need = ops.query("lsa_scan_select_workspace_bytes", R, d.top_p, b.bucket_centroids.shape[0])
                work = self._buffer("scan", (need,), torch.uint8, dev)
                _, picked = ops.scan_select(index_queries, b.bucket_centroids, index.centroids_bf16, visible, d.top_p,
                                            row_p, max_visible=bound, keys=keys, picked=picked,
                                            status=self._scan_status, workspace=work, lengths=index.lengths,
                                            radius=index.radius)
            else:
                _, picked = ops.flat_select(index_queries, b.bucket_centroids, visible, d.top_p, row_p, keys=keys,
                                            picked=picked)
        return picked, positions, row_p, row_k

    def select(self, index_queries: torch.Tensor, positions: torch.Tensor, index: FlatIndex,
               reuse_buffers: bool = False, local: bool = True, last_position: int | None = None):
        """Read lists [R, top_k + window + sink] int32 and their lengths for queries at `positions`; with
        `local=False` the lists hold the expansion alone (a band kernel reads the window and the sinks)."""
        d, b, dev = self.design, index.buckets, index_queries.device
        R = index_queries.shape[0]
        picked, positions, row_p, row_k = self.pick(index_queries, positions, index, reuse_buffers, last_position)
        outs = None
        if reuse_buffers:
            outs = (self._buffer("lists", (R, d.list_width), torch.int32, dev),
                    self._buffer("lengths", (R,), torch.int32, dev), self._expand_status)
        with probe.region("expand"):
            # (the layer's own buffers are read by their lengths: nothing is padded there)
            lists, lengths, _ = ops.expand(picked, positions, b.bucket_members, d.top_k, d.sink_size, d.window_size,
                                           row_p, row_k, outs=outs, local=local, pad=not reuse_buffers)
        return lists, lengths

    def attend(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, lists: torch.Tensor, lengths: torch.Tensor,
               splits: int = 1, out: torch.Tensor | None = None, lse: torch.Tensor | None = None,
               init: tuple | None = None):
        with probe.region("attend"):
            return ops.sparse_attend(q, k, v, lists, lengths, self.scale, splits=splits, out=out, lse=lse, init=init)

    def band(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, first_position: int):
        """The window and sinks of consecutive rows as one dense banded read: a partial (out fp32, lse)."""
        R, dev = q.shape[0], q.device
        with probe.region("band"):
            return ops.band_attend(q, k, v, first_position, self.design.window_size, self.design.sink_size, self.scale,
                                   out=self._buffer("band out", (R, self.heads, self.head_dim), torch.float32, dev),
                                   lse=self._buffer("band lse", (R, self.heads), torch.float32, dev),
                                   status=self._attend_status)

    # ---- the layer

    def prefill(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, chunk: int = 8192,
                return_index: bool = False, out: torch.Tensor | None = None, band: bool = True,
                bucket_major: bool = True):
        """Causal prefill from position 0: q [T,Hq,dh], k/v [T,Hkv,dh] bf16 -> out [T,Hq,dh] bf16.

        Every intermediate lives in buffers the layer keeps, so after the first call a step allocates nothing but
        its output (pass `out` to avoid that too). With `return_index` the index is built in fresh tensors instead.
        `band` reads the window and the sinks as dense tiles; `bucket_major` reads the selected keys bucket by bucket
        where the shapes allow (both off: every row gathers its whole list).
        """
        T = q.shape[0]
        index = self.build_index(k, reuse_buffers=not return_index)
        out = torch.empty_like(q) if out is None else out
        for start in range(0, T, chunk):
            stop = min(T, start + chunk)
            self.prefill_rows(q[start:stop], start, k, v, index, out[start:stop], band, bucket_major)
        return (out, index) if return_index else out

    def prefill_from_host(self, q_host: torch.Tensor, k_host: torch.Tensor, v_host: torch.Tensor,
                          out_host: torch.Tensor, chunk: int = 8192) -> torch.Tensor:
        """`prefill` for inputs and an output that live in PINNED host memory, the copies overlapped with the work.
        A causal chunk needs the keys and values up to its own end and the buckets of the cluster blocks before its
        rows, and blocks are clustered independently: so K, V and Q cross chunk by chunk on a copy stream, each
        chunk's blocks are indexed when its keys have arrived (on a stream of its own: a handful of small launches
        that would otherwise stand between two chunks' reads), and every chunk's output leaves on a second copy
        stream as soon as its merge is done. (`chunk` must hold whole cluster blocks.) On return the current stream
        has waited for the last output copy; synchronise it before reading `out_host`."""
        dev = self.query_map.device
        T = q_host.shape[0]
        if chunk % self.design.cluster_block_size or chunk % 128:
            raise ValueError("a chunk must hold whole cluster blocks (and whole tiles of 128 keys)")
        main = torch.cuda.current_stream(dev)
        if self._copy_in is None:
            self._copy_in, self._copy_out, self._index_stream = (torch.cuda.Stream(dev) for _ in range(3))
        chunks = [(start, min(T, start + chunk)) for start in range(0, T, chunk)]
        while len(self._copy_events) < 3 * len(chunks):
            self._copy_events.append(torch.cuda.Event())
        arrived, done, built = self._copy_events[0::3], self._copy_events[1::3], self._copy_events[2::3]
        q = self._buffer("q from host", tuple(q_host.shape), q_host.dtype, dev)
        k = self._buffer("k from host", tuple(k_host.shape), k_host.dtype, dev)
        v = self._buffer("v from host", tuple(v_host.shape), v_host.dtype, dev)
        out = self._buffer("out to host", tuple(q_host.shape), torch.bfloat16, dev)
        self._copy_in.wait_stream(main)   # the last call's reads of these buffers are over
        self._copy_out.wait_stream(main)
        with torch.cuda.stream(self._copy_in):
            for c, (start, stop) in enumerate(chunks):
                k[start:stop].copy_(k_host[start:stop], non_blocking=True)
                v[start:stop].copy_(v_host[start:stop], non_blocking=True)
                q[start:stop].copy_(q_host[start:stop], non_blocking=True)
                arrived[c].record(self._copy_in)
        bufs = self._index_buffers(T, dev, reuse_buffers=True)
        index = self._index_of(bufs)
        self._index_stream.wait_stream(main)
        with torch.cuda.stream(self._index_stream):
            for c, (start, stop) in enumerate(chunks):
                self._index_stream.wait_event(arrived[c])
                self._build_blocks(k[start:stop], start, bufs)
                built[c].record(self._index_stream)
        for c, (start, stop) in enumerate(chunks):
            main.wait_event(built[c])  # (the chunk's keys, values and queries have arrived, and its blocks are indexed)
            # (the cache as far as it has arrived: no kernel is handed rows that are still on their way)
            self.prefill_rows(q[start:stop], start, k[:stop], v[:stop], index, out[start:stop])
            done[c].record(main)
            with torch.cuda.stream(self._copy_out):
                self._copy_out.wait_event(done[c])
                out_host[start:stop].copy_(out[start:stop], non_blocking=True)
        main.wait_stream(self._copy_out)
        return out_host

    def prefill_rows(self, rows: torch.Tensor, start: int, k: torch.Tensor, v: torch.Tensor, index: FlatIndex,
                     out: torch.Tensor, band: bool = True, bucket_major: bool = True) -> torch.Tensor:
        """The read of consecutive query rows [n, Hq, dh] at positions start.. over a cache whose index is built,
        into `out` [n, Hq, dh] bf16 - one chunk of a prefill, or one rank's rows of a chunk."""
        n, dev = rows.shape[0], rows.device
        stop = start + n
        positions = torch.arange(start, stop, device=dev)
        with probe.region("index map"):
            index_queries = self.index_queries(rows, out=self._buffer("index queries", (n, self.index_dim),
                                                                      torch.float32, dev))
        # The window and the sinks are the same keys for neighbouring rows: one dense band serves them, and the
        # read of the selected keys starts from its partial result.
        banded = band and self.design.sink_size <= 64 and k.shape[0] >= stop
        lse = self._buffer("lse", (n, self.heads), torch.float32, dev)
        # (without the band the window and the sinks are in the lists, which only the gather path reads)
        if banded and bucket_major and ops.bucket_attend_supported(rows, k, self.design.bucket_cap):
            # The band and the read of the selected keys meet only in the merge, and one waits on the tensor pipe
            # while the other is bound by instruction issue: the band runs on a stream of its own beside them.
            main = torch.cuda.current_stream(dev)
            if self._band_stream is None:
                self._band_stream, self._band_done = torch.cuda.Stream(dev), torch.cuda.Event()
            self._band_stream.wait_stream(main)  # the inputs are ready; the last chunk's merge has read the buffers
            with torch.cuda.stream(self._band_stream):
                init = self.band(rows, k, v, start)
                self._band_done.record(self._band_stream)
            # The rows of a chunk pick the same buckets over and over: read each bucket's keys once per 128
            # (row, pick) pairs instead of once per pair.
            picked, positions, row_p, row_k = self.pick(index_queries, positions, index, reuse_buffers=True,
                                                        last_position=stop - 1)
            need = _lib.query("lsa_bucket_attend_workspace_bytes", n, self.design.top_p, self.heads, self.head_dim,
                              index.buckets.bucket_members.shape[0])
            with probe.region("attend"):
                ops.bucket_attend(rows, k, v, picked, positions, index.buckets.bucket_members, self.design.top_k,
                                  self.design.sink_size, self.design.window_size, self.scale, init=init,
                                  row_top_p=row_p, row_top_k=row_k, out=out, lse=lse,
                                  warp_mma=not self.bucket_tensor_memory, init_ready=self._band_done,
                                  status=self._attend_status,
                                  workspace=self._buffer("bucket workspace", (need,), torch.uint8, dev))
            return out
        init = self.band(rows, k, v, start) if banded else None
        lists, lengths = self.select(index_queries, positions, index, reuse_buffers=True, local=not banded,
                                     last_position=stop - 1)
        self.attend(rows, k, v, lists, lengths, out=out, lse=lse, init=init)
        return out

    def decode(self, q: torch.Tensor, positions: torch.Tensor, k: torch.Tensor, v: torch.Tensor, index: FlatIndex,
               splits: int = 8):
        """One step for rows at `positions` over a cache whose index is built: out [R,Hq,dh] bf16."""
        lists, lengths = self.select(self.index_queries(q), positions, index)
        out, _ = self.attend(q, k, v, lists, lengths, splits=splits)
        return out
