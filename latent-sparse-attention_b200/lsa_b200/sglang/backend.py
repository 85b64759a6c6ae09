"""The GQA model glue: the attention backend's `forward_extend` / `forward_decode` served from LSA's selection.

Function for function the surface of `src/lsa/sglang/models/qwen3_5/backend.py` - `list_lengths`, `sparse_read`,
`owned_lists`, `partial_read`, `merge_partials`, `group_read`, `select_and_read` - with the engine's attention kernels
replaced by `lsa_sparse_attend` and the engine's LSE merge by `lsa_lse_merge`. The backend, layer and batch objects
are the engine's own; only these attributes are read:

    backend.token_to_kv_pool.get_key_buffer(layer_id) / get_value_buffer(layer_id)   [slots, Hkv, dh] bf16
    layer.layer_id, layer.tp_q_head_num, layer.tp_k_head_num, layer.head_dim, layer.scaling
    forward_batch.forward_mode.is_extend()
"""

from __future__ import annotations

import inspect
from typing import Any, Callable

import torch

from lsa_b200 import ops
from lsa_b200.constants import Sentinel
from lsa_b200.sglang import index_space, weights
from lsa_b200.sglang.layer_index import KeySplit, LayerIndex, Shard
from lsa_b200.sglang.settings import DesignSettings

# Every quadratic layer's indexer, built by the first backend enabled: one index a layer, however many backends read it
ENABLED: dict = {}

# Request table row of each request id, so a decode step finds its rows without a device read
ROWS: dict = {}
ROWS_KEPT = 4096


def list_lengths(lists: torch.Tensor) -> torch.Tensor:
    """Valid entries of each list [T] int32; lists hold their valid entries first (`src/lsa/sglang/index/read.py:29-45`)."""
    return (lists > Sentinel.PAD).sum(1, dtype=torch.int32)


def _pool(backend: Any, layer: Any):
    pool = backend.token_to_kv_pool
    return pool.get_key_buffer(layer.layer_id), pool.get_value_buffer(layer.layer_id)


def sparse_read(backend: Any, q: torch.Tensor, layer: Any, lists: torch.Tensor) -> torch.Tensor:
    """Attend each query over the KV slots its list names (backend.py:427-460): q [T, Hq*dh] or [T, Hq, dh],
    lists [T, width] int32 (-1 padded, valid first) -> [T, Hq*dh]."""
    tokens = lists.shape[0]
    keys, values = _pool(backend, layer)
    out, _ = ops.sparse_attend(q.contiguous().view(tokens, layer.tp_q_head_num, layer.head_dim), keys, values, lists,
                               list_lengths(lists), layer.scaling, splits=_splits(tokens))
    return out.view(tokens, layer.tp_q_head_num * layer.head_dim)


def _splits(tokens: int) -> int:
    """CTAs a row's list is divided over: a prefill chunk fills the GPU by its rows, a decode batch needs the split."""
    return 1 if tokens >= 512 else max(1, min(16, 1024 // max(tokens, 1)))


def owned_lists(lists: torch.Tensor, shard: Shard):
    """The selected slots this rank owns, as rows of its pool, valid entries first (backend.py:621-635)."""
    owned = (lists > Sentinel.PAD) & (lists % shard.size == shard.rank)
    rows = torch.where(owned, lists // shard.size, Sentinel.PAD)
    return rows.sort(dim=1, descending=True).values, owned.sum(1, dtype=torch.int32)


def partial_read(backend: Any, q: torch.Tensor, layer: Any, rows: torch.Tensor, counts: torch.Tensor):
    """Every query head over the selected rows this rank holds: (out [T, Hq, dh] fp32, lse [T, Hq] fp32, minus
    infinity where the rank holds nothing of a query) (backend.py:669-721)."""
    keys, values = _pool(backend, layer)
    out, lse = ops.sparse_attend(q.contiguous(), keys, values, rows, counts, layer.scaling, splits=_splits(rows.shape[0]),
                                 out_dtype=torch.float32)
    return out, lse


def merge_partials(out: torch.Tensor, lse: torch.Tensor, group=None) -> torch.Tensor:
    """Merge a decode group's partial reads into this rank's own heads [T, Hq / size, dh] fp32 (backend.py:724-738):
    the partials and log-sum-exps are all-gathered and merged by `lsa_lse_merge`; a single rank merges nothing."""
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return out
    from lsa_b200.parallel import gather_pieces

    size, rank = dist.get_world_size(group), dist.get_rank(group)
    heads = out.shape[1] // size
    mine = slice(rank * heads, (rank + 1) * heads)
    merged, _ = ops.lse_merge(gather_pieces(out[:, mine].contiguous(), group),
                              gather_pieces(lse[:, mine].contiguous(), group))
    return merged


def gather_heads(q: torch.Tensor, layer: Any, group=None) -> torch.Tensor:
    """Every query head [T, Hq, dh] from this rank's [T, Hq / size, dh] (backend.py:741-755)."""
    import torch.distributed as dist

    local = q.reshape(-1, layer.tp_q_head_num, layer.head_dim).contiguous()
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return local
    from lsa_b200.parallel import gather_pieces

    return gather_pieces(local, group).permute(1, 0, 2, 3).reshape(local.shape[0], -1, layer.head_dim).contiguous()


def group_read(backend: Any, q: torch.Tensor, layer: Any, lists: torch.Tensor, shard: Shard,
               merge: Callable[[torch.Tensor, torch.Tensor], torch.Tensor] = merge_partials) -> torch.Tensor:
    """Each query over the KV slots its list names, the keys spread across a decode group (backend.py:758-781)."""
    rows, counts = owned_lists(lists, shard)
    out, lse = partial_read(backend, q, layer, rows, counts)
    return merge(out, lse).to(q.dtype).reshape(q.shape[0], -1)


class GroupedQueryIndexer:
    """One quadratic layer's index, built on its first use once the model and the KV pool exist
    (`src/lsa/sglang/models/qwen3_5/backend.py:81-217`). Of the backend these are read: `req_to_token`
    [requests, context] int32 and `token_to_kv_pool` (`size`, `page_size`, `get_key_buffer(layer_id)`); of a forward
    batch: `forward_mode`, `positions`, `out_cache_loc`, `req_pool_indices`, `rids`, `seq_lens_cpu`,
    `extend_seq_lens_cpu`, `extend_prefix_lens_cpu`, and `lsa_rows`, which `maintain_all` puts there."""

    is_lsa = True

    def __init__(self, layer_id: int, geometry: index_space.Geometry, design: DesignSettings, backend: Any,
                 shard: Shard | None = None, heads: index_space.HeadShard | None = None,
                 check_index: bool = False, prefill_chunk: int = 8192, maps: tuple | None = None,
                 sum_heads=None) -> None:
        """`shard`: the slots this rank owns under decode context parallel; `heads`: the heads it holds under tensor
        parallel, with `sum_heads` the sum across that group; `maps` = (query map, key map) skips the map file (tests,
        a server that holds the maps already)."""
        if heads is not None and sum_heads is None:
            raise ValueError("a rank holding some of the heads needs the sum across its tensor-parallel group")
        self.layer, self.geometry, self.design, self.backend = layer_id, geometry, design, backend
        self.shard, self.heads, self.prefill_chunk, self.maps = shard or Shard(), heads, prefill_chunk, maps
        self.check_index, self.sum_heads = check_index, sum_heads
        self.index: LayerIndex | None = None

    def request_table(self) -> torch.Tensor:
        return self.backend.req_to_token

    def key_buffer(self) -> torch.Tensor:
        """This layer's key cache [slots, Hkv, dh] bf16.

        Raises:
            NotImplementedError: The KV cache is not bf16, so its keys are not the ones the maps were distilled on.
        """
        buffer = self.backend.token_to_kv_pool.get_key_buffer(self.layer)
        if buffer.dtype != torch.bfloat16:
            raise NotImplementedError(f"the key and query input reads a bf16 KV cache - this one is {buffer.dtype}, "
                                      "serve kv_cache_dtype auto")
        held = self.geometry.kv_head_count if self.heads is None else self.heads.kv_count
        return buffer.view(-1, held, self.geometry.head_dim)

    def ready(self) -> LayerIndex:
        """Build the layer's index once, and return it."""
        if self.index is None:
            table, pool = self.request_table(), self.backend.token_to_kv_pool
            maps = self.maps
            if maps is None:
                maps = weights.read(self.design.serving.projections, self.geometry.key_dim,
                                    self.design.indexer.index_dim, self.geometry.layers)[self.layer]
            split = None
            if self.heads is not None:
                start, stop = self.heads.dims(self.geometry)
                split = KeySplit(start, stop, self.heads.counts_key, self.sum_heads)
            self.index = LayerIndex(self.design, maps, pool.size + pool.page_size, pool.size, self.request_table,
                                    table.shape[1], self.prefill_chunk, table.device, self.shard,
                                    check_index=self.check_index, key_buffer=self.key_buffer,
                                    key_slot=self.geometry.key_slot, split=split,
                                    prefix_reuse=self.design.serving.prefix_reuse,
                                    spare_contexts=self.design.serving.spare_contexts)
            self.index.writes_pool = False  # `select_and_read` saves a forward's keys before it selects
        return self.index

    def maintain(self, forward_batch: Any) -> None:
        """Bring each request's cache up to the tokens already in the KV pool, before every forward."""
        rows = forward_batch.lsa_rows
        self.ready().maintain(forward_batch.rids, rows, ends_of(forward_batch, len(rows)))

    def select(self, q: torch.Tensor, k: torch.Tensor, forward_batch: Any) -> torch.Tensor:
        """Select for every query of a forward, from the heads attention was handed: q [T, Hq * dh] or [T, Hq, dh]
        rotated on the prefix alone, k [T, Hkv, dh] the same, already in the pool at `out_cache_loc`. Returns KV
        slots [T, width] int32, -1 padded, valid entries first."""
        index = self.ready()
        inputs = index_space.key_and_query(q, k, self.geometry, self.heads)
        positions, slots = forward_batch.positions, forward_batch.out_cache_loc.long()
        if forward_batch.forward_mode.is_extend():
            return index.extend(inputs, positions, slots, forward_batch.lsa_rows, forward_batch.extend_seq_lens_cpu,
                                forward_batch.extend_prefix_lens_cpu)
        return index.decode(inputs, positions, slots, forward_batch.req_pool_indices.long())


def rows_of(forward_batch: Any) -> list:
    """Request table rows of the batch: one device read a prefill, none in decode, where they are looked up by
    request id (`src/lsa/sglang/index/registry.py:42-66`)."""
    rids = forward_batch.rids
    if not forward_batch.forward_mode.is_extend() and all(rid in ROWS for rid in rids):
        return [ROWS[rid] for rid in rids]
    rows = forward_batch.req_pool_indices.tolist()
    ROWS.update(zip(rids, rows))
    if len(ROWS) > 4 * len(rows) + ROWS_KEPT:  # finished requests never come back: keep the map small
        for rid in list(ROWS)[: len(ROWS) // 2]:
            del ROWS[rid]
    return rows


def ends_of(forward_batch: Any, request_count: int) -> list:
    """Keys each real request has in the pool before this forward's own (`registry.py:69-86`); a decode batch
    replayed in a CUDA graph is padded, so its length lists run past the requests."""
    seq_lens = forward_batch.seq_lens_cpu.tolist()[:request_count]
    if forward_batch.forward_mode.is_extend():
        lengths = list(forward_batch.extend_seq_lens_cpu)[:request_count]
    else:
        lengths = [1] * request_count
    return [seq_len - length for seq_len, length in zip(seq_lens, lengths, strict=True)]


def maintain_all(backend: Any, forward_batch: Any) -> None:
    """Put the request table rows on the batch and run every indexer's maintenance (`registry.py:89-100`).

    Raises:
        RuntimeError: The batch carries no request ids.
    """
    indexers = getattr(backend, "lsa_indexers", None)
    if not indexers or getattr(forward_batch.forward_mode, "is_idle", lambda: False)():
        return
    if getattr(forward_batch, "rids", None) is None:
        raise RuntimeError("LSA maintenance needs request ids on the forward batch")
    forward_batch.lsa_rows = rows_of(forward_batch)
    for indexer in indexers.values():
        indexer.maintain(forward_batch)


def enable(backend: Any, runner: Any, design: DesignSettings) -> dict:
    """Give a grouped-query server's attention backend an indexer for every quadratic layer
    (`models/qwen3_5/backend.py:305-347`). A backend built for another model or a draft is left as it was; a second
    backend of the same server reads the indexers the first one built, since the pools they index are the runner's."""
    text = runner.model_config.hf_text_config
    if getattr(backend, "is_draft_runner", False) or not index_space.is_grouped_query(text):
        return {}
    if not ENABLED:
        geometry = index_space.geometry_of(text)
        if design.indexer.index_dim not in (16, 32, 64, 128):
            raise NotImplementedError(f"the index kernels take an index of 16, 32, 64 or 128 dims - the design's is "
                                      f"{design.indexer.index_dim}")
        ENABLED.update({layer: GroupedQueryIndexer(layer, geometry, design, backend) for layer in geometry.layers})
    backend.lsa_indexers = ENABLED
    return ENABLED


def bind(original: Any, *args: Any, **kwargs: Any) -> inspect.BoundArguments:
    """The arguments of a wrapped call by name, defaults filled (plugin.py:634-647)."""
    bound = inspect.signature(original).bind(*args, **kwargs)
    bound.apply_defaults()
    return bound


def indexer_of(backend: Any, layer: Any, forward_batch: Any):
    """The layer's indexer, or None for a layer LSA does not serve."""
    indexers = getattr(backend, "lsa_indexers", None)
    if not indexers or forward_batch is None or getattr(forward_batch.forward_mode, "is_idle", lambda: False)():
        return None
    return indexers.get(layer.layer_id)


def save(backend: Any, layer: Any, k: torch.Tensor, v: torch.Tensor, forward_batch: Any, shard: Shard) -> None:
    """Write this step's keys and values into the pool at the slots the batch names (backend.py:395-424). Under a
    decode group a rank keeps the tokens it owns, at row slot // size, as the engine's pools place them (the pool is
    handed the ownership mask, as the reference hands it)."""
    if shard.size > 1:
        loc = forward_batch.out_cache_loc
        backend.token_to_kv_pool.set_kv_buffer(layer, loc // shard.size, k, v, dcp_kv_mask=loc % shard.size == shard.rank)
        return
    backend.token_to_kv_pool.set_kv_buffer(layer, forward_batch.out_cache_loc, k, v)


def select_and_read(original: Any, self: Any, *args: Any, **kwargs: Any) -> Any:
    """Serve a layer's attention from its selection, or hand any other call to the backend as it was
    (backend.py:784-822). `original` is `forward_extend` or `forward_decode`; `self` the attention backend."""
    bound = bind(original, self, *args, **kwargs)
    arguments = bound.arguments
    q, k, v, layer, forward_batch = (arguments[name] for name in ("q", "k", "v", "layer", "forward_batch"))
    indexer = indexer_of(self, layer, forward_batch)
    if indexer is None or k is None:
        return original(*bound.args, **bound.kwargs)
    mode = forward_batch.forward_mode
    if mode.is_extend() and torch.cuda.is_available() and torch.cuda.is_current_stream_capturing():
        raise RuntimeError("LSA builds a prefill's index on the host - serve with --disable-prefill-cuda-graph")
    for refused in ("is_target_verify", "is_draft_extend_v2"):
        if getattr(mode, refused, lambda: False)():
            raise NotImplementedError("LSA reads a plain prefill or decode, without speculative decoding")
    shard = getattr(indexer, "shard", Shard())
    if arguments.get("save_kv_cache", True):
        save(self, layer, k, v, forward_batch, shard)
    if shard.size == 1:
        return sparse_read(self, q, layer, indexer.select(q, k, forward_batch))
    every_head = gather_heads(q, layer)
    return group_read(self, every_head, layer, indexer.select(every_head, k, forward_batch), shard)
