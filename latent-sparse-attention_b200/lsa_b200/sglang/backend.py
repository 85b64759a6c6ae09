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
from dataclasses import dataclass
from typing import Any, Callable

import torch

from lsa_b200 import ops
from lsa_b200.constants import Sentinel


@dataclass(frozen=True)
class Shard:
    """Which KV slots a rank of a decode group owns: slot s lives on rank s % size at row s // size
    (`src/lsa/sglang/index/layer_index.py:65-87`)."""

    rank: int = 0
    size: int = 1


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


def bind(original: Any, *args: Any, **kwargs: Any) -> inspect.BoundArguments:
    """The arguments of a wrapped call by name, defaults filled (plugin.py:634-647)."""
    bound = inspect.signature(original).bind(*args, **kwargs)
    bound.apply_defaults()
    return bound


def indexer_of(backend: Any, layer: Any, forward_batch: Any):
    """The layer's indexer, or None for a layer LSA does not serve."""
    indexers = getattr(backend, "lsa_indexers", None)
    return None if indexers is None else indexers.get(layer.layer_id)


def save(backend: Any, layer: Any, k: torch.Tensor, v: torch.Tensor, forward_batch: Any, shard: Shard) -> None:
    """Write this step's keys and values into the pool at the slots the batch names (backend.py:395-424)."""
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
