"""One LSA global-attention layer over an MLA-style cache, flat design.

Every query head reads the SAME latent rows (512 value dims + 64 rope dims a token), so the index is built from the
latent rows themselves and a query's index vector from the sum of its absorbed heads. This is the layer the reference
serves through its `LSAIndexer` (src/lsa/sglang/models/glm5_next/indexer.py:83-316: index keys from the key latent,
one list of KV slots a token for all heads) with the engine's sparse MLA kernel behind it
(src/lsa/sglang/plugin.py:525-598); the attention arithmetic is `topk_attention` with one KV head
(src/lsa/core/attention.py:65-146).

The maps are either linear ([d_in, index_dim], the reference's `project`, src/lsa/core/index_space.py:405-419) or
two-layer with a GELU between ((w1_t [hidden, d_in], w2_t [index_dim, hidden]); no counterpart in the reference).
"""

from __future__ import annotations

import torch

from lsa_b200 import ops, probe
from lsa_b200.layer import FlatDesign, FlatIndex, FlatLayer


class LatentLayer(FlatLayer):
    """Index build, prefill rows and decode steps over a latent cache [T, latent_dim] bf16; absorbed queries are
    [rows, heads, latent_dim] bf16 and outputs [rows, heads, value_dim]."""

    def __init__(self, design: FlatDesign, query_map, key_map, heads: int, latent_dim: int = 576, value_dim: int = 512,
                 scale: float | None = None, map_piece: int = 1 << 17):
        two_layer = isinstance(key_map, (tuple, list))
        if two_layer != isinstance(query_map, (tuple, list)):
            raise ValueError("the query map and the key map must both be linear or both two-layer")
        if two_layer:
            (q1, q2), (k1, k2) = query_map, key_map
            for w1, w2 in ((q1, q2), (k1, k2)):
                if w1.dim() != 2 or w2.dim() != 2 or w1.shape[1] != latent_dim or w2.shape[1] != w1.shape[0]:
                    raise ValueError(f"a two-layer map is (w1_t [hidden, {latent_dim}], w2_t [index_dim, hidden]) - got "
                                     f"{tuple(w1.shape)} and {tuple(w2.shape)}")
            if q2.shape[0] != k2.shape[0]:
                raise ValueError("the two maps must share their index dim")
            device, index_dim = k1.device, k2.shape[0]
            self.query_map = (q1.contiguous(), q2.contiguous())
            self.key_map = (k1.contiguous(), k2.contiguous())
        else:
            if query_map.shape != key_map.shape or query_map.shape[0] != latent_dim:
                raise ValueError(f"the maps must both be [{latent_dim}, index_dim] - got {tuple(query_map.shape)} and "
                                 f"{tuple(key_map.shape)}")
            device, index_dim = key_map.device, key_map.shape[1]
            # (as the tensor-core map reads them: transposed, bf16)
            self.query_map = query_map.t().contiguous().to(torch.bfloat16)
            self.key_map = key_map.t().contiguous().to(torch.bfloat16)
        self.two_layer = two_layer
        self.design, self.index_dim = design, index_dim
        self.heads, self.kv_heads, self.head_dim, self.value_dim = heads, 1, latent_dim, value_dim
        self.scale = latent_dim ** -0.5 if scale is None else scale
        self.map_piece = map_piece
        self._buffers = {}
        self._status_slots(device)
        self._reached = []
        self._copy_in = self._copy_out = None  # the side streams of `prefill_from_host`
        self._copy_events: list = []

    # ---- the maps

    def _map(self, rows: torch.Tensor, weights, out: torch.Tensor | None) -> torch.Tensor:
        """rows [n, latent_dim] bf16 -> unit index vectors [n, index_dim] fp32, a bounded piece at a time."""
        n = rows.shape[0]
        out = torch.empty(n, self.index_dim, device=rows.device, dtype=torch.float32) if out is None else out
        if not self.two_layer:
            return ops.index_map_tc(rows, weights, out=out, status=self._map_status)
        piece = min(n, self.map_piece)
        hidden = self._buffer("hidden", (piece, weights[0].shape[0]), torch.bfloat16, rows.device)
        for start in range(0, n, piece):
            m = min(piece, n - start)
            ops.mlp_map(rows[start:start + m], weights[0], weights[1], hidden=hidden[:m], out=out[start:start + m])
        return out

    def index_keys(self, latent: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """latent rows [n, latent_dim] bf16 -> unit index keys [n, index_dim] fp32."""
        return self._map(latent, self.key_map, out)

    def index_queries(self, q: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """absorbed queries [n, heads, latent_dim] bf16 -> unit index queries [n, index_dim] fp32: the heads are summed
        (fp32, rounded once to bf16) and the sum is mapped."""
        if q.shape[0] <= 8 and out is None and q.stride(2) == 1:
            return self.index_queries_rows(q)
        summed = ops.index_map(q, None, group=self.heads, normalize=False, out_dtype=torch.bfloat16)
        return self._map(summed, self.query_map, out)

    def index_queries_rows(self, q: torch.Tensor) -> torch.Tensor:
        """The query map for the few rows of a decode step: layers that spread one row's contraction over many CTAs
        instead of padding it to a tile of 128 rows."""
        if not self.two_layer:
            return ops.rows_linear(q, self.query_map, sum_heads=True, normalize=True)
        hidden = ops.rows_linear(q, self.query_map[0], sum_heads=True, gelu=True, out_dtype=torch.bfloat16)
        return ops.rows_linear(hidden, self.query_map[1], normalize=True)

    # ---- the index

    def build_index(self, latent: torch.Tensor, reuse_buffers: bool = False) -> FlatIndex:
        """Index keys of every row, then pools, Ward and the bucket table of every closed cluster block."""
        bufs = self._index_buffers(latent.shape[0], latent.device, reuse_buffers)
        self._build_blocks(latent, 0, bufs)
        self._bufs = bufs
        return self._index_of(bufs)

    def extend_index(self, latent: torch.Tensor, first: int, count: int) -> None:
        """The index step of a prefill chunk: the index keys of rows first .. first + count - 1 of the cache, and the
        buckets of the cluster blocks that close inside (first, first + count] (the index of `build_index`, whose
        buffers it updates in place)."""
        d, bufs = self.design, self._bufs
        with probe.region("index map"):
            self.index_keys(latent[first:first + count], out=bufs["keys"][first:first + count])
        b0 = first // d.cluster_block_size
        b1 = (first + count) // d.cluster_block_size
        self._cluster_blocks(b0, b1 - b0, bufs)

    # ---- the reads

    def prefill_rows(self, rows: torch.Tensor, start: int, latent: torch.Tensor, index: FlatIndex,
                     out: torch.Tensor, warp_mma: bool = False) -> torch.Tensor:
        """The read of consecutive query rows [n, heads, latent_dim] at positions start.. over a cache whose index
        is built, into `out` [n, heads, value_dim] bf16."""
        n, dev = rows.shape[0], rows.device
        positions = torch.arange(start, start + n, device=dev)
        with probe.region("index map"):
            index_queries = self.index_queries(rows, out=self._buffer("index queries", (n, self.index_dim),
                                                                      torch.float32, dev))
        lists, lengths = self.select(index_queries, positions, index, reuse_buffers=True, last_position=start + n - 1)
        with probe.region("attend"):
            ops.latent_attend(rows, latent, lists, lengths, self.scale, value_dim=self.value_dim, out=out,
                              warp_mma=warp_mma, status=self._attend_status)
        return out

    def prefill_from_host(self, q_host: torch.Tensor, rows_host: torch.Tensor, start: int, latent: torch.Tensor,
                          index: FlatIndex, out_host: torch.Tensor, pieces: int = 4) -> torch.Tensor:
        """A prefill chunk whose queries [n, heads, latent_dim], own latent rows [n, latent_dim] and output
        [n, heads, value_dim] live in PINNED host memory, the copies overlapped with the work: the latent rows cross
        first (the chunk's index step needs them all), the queries a piece at a time on a copy stream while the piece
        before is read, and a piece's output leaves on a second copy stream as soon as it is written. `index` is the
        layer's own (`build_index`), which the chunk's closing blocks are added to. On return the current stream has
        waited for the last output copy; synchronise it before reading `out_host`."""
        dev, n = latent.device, q_host.shape[0]
        main = torch.cuda.current_stream(dev)
        if self._copy_in is None:
            self._copy_in, self._copy_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        step = -(-n // max(1, pieces))
        spans = [(first, min(n, first + step)) for first in range(0, n, step)]
        while len(self._copy_events) < 2 * len(spans) + 1:
            self._copy_events.append(torch.cuda.Event())
        rows_in, arrived, done = self._copy_events[0], self._copy_events[1::2], self._copy_events[2::2]
        q = self._buffer("q from host", tuple(q_host.shape), q_host.dtype, dev)
        out = self._buffer("out to host", tuple(out_host.shape), out_host.dtype, dev)
        self._copy_in.wait_stream(main)   # the last call's reads of these buffers are over
        self._copy_out.wait_stream(main)
        with torch.cuda.stream(self._copy_in):
            latent[start:start + n].copy_(rows_host, non_blocking=True)
            rows_in.record(self._copy_in)
            for i, (first, stop) in enumerate(spans):
                q[first:stop].copy_(q_host[first:stop], non_blocking=True)
                arrived[i].record(self._copy_in)
        main.wait_event(rows_in)
        self.extend_index(latent, start, n)
        for i, (first, stop) in enumerate(spans):
            main.wait_event(arrived[i])
            self.prefill_rows(q[first:stop], start + first, latent, index, out[first:stop])
            done[i].record(main)
            with torch.cuda.stream(self._copy_out):
                self._copy_out.wait_event(done[i])
                out_host[first:stop].copy_(out[first:stop], non_blocking=True)
        main.wait_stream(self._copy_out)
        return out_host

    def decode(self, q: torch.Tensor, positions: torch.Tensor, latent: torch.Tensor, index: FlatIndex,
               splits: int = 148, select_splits: int = 32, warp_mma: bool = False) -> torch.Tensor:
        """One step for rows [R, heads, latent_dim] at `positions`: out [R, heads, value_dim] bf16. Fixed shapes and
        no host reads once `visible` is on the device, so a step can be captured in a CUDA graph."""
        d, b = self.design, index.buckets
        with probe.region("index map"):
            index_queries = self.index_queries(q)
        visible = (positions.to(torch.int64) // d.cluster_block_size * d.block_bucket_count).clamp_max(
            b.bucket_centroids.shape[0]).to(torch.int32)
        with probe.region("select"):
            _, picked = ops.flat_select_decode(index_queries, b.bucket_centroids, None, visible, d.top_p,
                                               splits=select_splits)
        with probe.region("expand"):
            lists, lengths, _ = ops.expand(picked, positions, b.bucket_members, d.top_k, d.sink_size, d.window_size)
        with probe.region("attend"):
            out, _ = ops.latent_attend(q, latent, lists, lengths, self.scale, value_dim=self.value_dim, splits=splits,
                                       warp_mma=warp_mma, status=self._attend_status)
        return out
