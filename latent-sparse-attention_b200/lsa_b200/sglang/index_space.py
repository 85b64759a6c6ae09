"""A grouped-query checkpoint's index geometry, and the key and query input as a server hands it over.

The design's input for a grouped-query model is the position-free part of the logit: every key-value head's dims past
its rotated prefix, side by side, and each group's query heads summed into the slice of the key head they read, so one
selection serves every head (`src/lsa/sglang/models/qwen3_5/index_space.py:1-289`). The names, arguments and refusals
are the reference's; what differs is where the arithmetic runs: `key_and_query` hands back views of the heads
attention was given, and the group sum, the slice past the rotated prefix, the map and the normalisation are one
kernel (`lsa_index_map` with `group` and `dh_off`), so nothing of the input is materialised a token. `materialise`
writes the input out as the reference's tensors for code that wants them.

Nothing here imports an engine.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

FULL_ATTENTION = "full_attention"
TEXT_CONFIG = "text_config"
INTERVAL = "full_attention_interval"


def field_of(config: Any, name: str) -> Any:
    """A field of a config object or of a plain mapping, None when it has none."""
    if isinstance(config, dict):
        return config.get(name)
    return getattr(config, name, None)


@dataclass(frozen=True)
class KeySlot:
    """Where the key input sits in a KV pool slot: the same dims of each of the slot's heads, side by side
    (`src/lsa/sglang/index/layer_index.py:389-445`)."""

    heads: int
    head_dim: int
    offset: int
    width: int

    def __post_init__(self) -> None:
        if self.width <= 0 or self.offset < 0 or self.offset + self.width > self.head_dim:
            raise ValueError(f"a key read of {self.width} dims at {self.offset} does not fit a head of {self.head_dim}")

    @classmethod
    def latent(cls, key_dim: int, rope_dim: int = 0) -> "KeySlot":
        """The slot of an MLA pool: one head, the key latent then its rope dims."""
        return cls(heads=1, head_dim=key_dim + rope_dim, offset=0, width=key_dim)

    @property
    def key_dim(self) -> int:
        return self.heads * self.width

    def read(self, buffer: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
        """The key input [S, key_dim] at some rows of a pool buffer [slots, heads, head_dim]."""
        return buffer[rows, :, self.offset:self.offset + self.width].reshape(len(rows), self.key_dim)

    def write(self, buffer: torch.Tensor, rows: torch.Tensor, key: torch.Tensor) -> None:
        """Write the key input at some rows of a pool buffer, the rest of each slot left as it is."""
        buffer[rows, :, self.offset:self.offset + self.width] = key.view(len(rows), self.heads, self.width)


@dataclass(frozen=True)
class KeyAndQuery:
    """The indexer's input: the new tokens' keys and their heads' queries (`layer_index.py:283-293`).

    Either the reference's tensors - key [S, key_dim] bf16 and query [S, heads, key_dim] (a grouped-query model's:
    one row a token, fp32, each group's queries summed into its key head's slice) - or the heads as attention was
    handed them: key [S, Hkv, head_dim] and query [S, Hq, head_dim] bf16, which the fused map reads in place.
    """

    key: torch.Tensor
    query: torch.Tensor


@dataclass(frozen=True)
class Geometry:
    """One checkpoint's index geometry, read off its config (`index_space.py:42-66`)."""

    query_head_count: int
    kv_head_count: int
    head_dim: int
    rotary_dim: int
    layers: tuple  # the decoder indices that attend quadratically: the ids a server presents as `layer_id`

    @property
    def key_slot(self) -> KeySlot:
        return KeySlot(heads=self.kv_head_count, head_dim=self.head_dim, offset=self.rotary_dim,
                       width=self.head_dim - self.rotary_dim)

    @property
    def key_dim(self) -> int:
        return self.key_slot.key_dim


def text_config_of(config: Any) -> Any:
    """Whichever config holds the text geometry: a server's text config already, or a VL config's nested one."""
    if field_of(config, "head_dim") is None and field_of(config, TEXT_CONFIG) is not None:
        return field_of(config, TEXT_CONFIG)
    return config


def is_grouped_query(config: Any) -> bool:
    """Whether a model is a grouped-query stack this plugin indexes: quadratic layers over per-head keys, no key
    latent (`index_space.py:80-93`)."""
    config = text_config_of(config)
    if field_of(config, "kv_lora_rank") is not None:
        return False
    layer_types = field_of(config, "layer_types") or ()
    return FULL_ATTENTION in layer_types or bool(field_of(config, INTERVAL))


def rotary_dim_of(config: Any) -> int:
    """Leading dims of a head the rotation covers (`index_space.py:96-119`).

    Raises:
        ValueError: The rotation covers every dim of a head, so nothing is position-free.
    """
    factor = field_of(config, "partial_rotary_factor")
    if factor is None:
        factor = field_of(field_of(config, "rope_parameters") or {}, "partial_rotary_factor")
    if factor is None or not 0 <= float(factor) < 1:
        raise ValueError(f"this config's rotation covers every dim of a head (partial_rotary_factor {factor}) - "
                         "nothing is position-free to index")
    return int(int(field_of(config, "head_dim")) * float(factor))


def quadratic_layers(config: Any) -> tuple:
    """The decoder indices that attend quadratically (`index_space.py:122-146`): those `layer_types` names, else
    every `full_attention_interval`-th.

    Raises:
        ValueError: The config names no quadratic layer.
    """
    layer_types = list(field_of(config, "layer_types") or ())
    layers = tuple(index for index, kind in enumerate(layer_types) if kind == FULL_ATTENTION)
    if layers:
        return layers
    interval, depth = field_of(config, INTERVAL), field_of(config, "num_hidden_layers")
    if not interval or not depth:
        raise ValueError(f"this config names no {FULL_ATTENTION} layer among {len(layer_types)} and no {INTERVAL} - "
                         "nothing to index")
    return tuple(range(int(interval) - 1, int(depth), int(interval)))


def geometry_of(config: Any) -> Geometry:
    config = text_config_of(config)
    return Geometry(query_head_count=int(field_of(config, "num_attention_heads")),
                    kv_head_count=int(field_of(config, "num_key_value_heads")),
                    head_dim=int(field_of(config, "head_dim")), rotary_dim=rotary_dim_of(config),
                    layers=quadratic_layers(config))


@dataclass(frozen=True)
class HeadShard:
    """The heads a tensor-parallel rank holds, and the dims of the key and query input they are
    (`index_space.py:169-187`)."""

    kv_first: int
    kv_count: int
    query_count: int
    counts_key: bool  # whether this rank's key heads are added to the group's sum: one of the replicas is

    def dims(self, geometry: Geometry) -> tuple:
        free = geometry.head_dim - geometry.rotary_dim
        return self.kv_first * free, (self.kv_first + self.kv_count) * free


def splits_key_heads(tp_size: int, decode_size: int = 1) -> bool:
    return tp_size // decode_size > 1


def kv_heads_held(geometry: Geometry, tp_size: int) -> int:
    return max(1, geometry.kv_head_count // tp_size)


def head_shard(geometry: Geometry, tp_size: int, tp_rank: int, decode_size: int = 1) -> HeadShard | None:
    """The heads a rank holds when the mesh splits the key-value heads, None where it holds them all
    (`index_space.py:210-257`).

    Raises:
        NotImplementedError: Decode context parallel spans part of the tensor-parallel group; the group splits the
            query heads unevenly; or it neither divides the key-value heads nor holds each on whole ranks.
    """
    if decode_size not in (1, tp_size):
        raise NotImplementedError(f"decode context parallel {decode_size} under tensor parallel {tp_size} splits the "
                                  "pool by slots and the key-value heads by ranks at once, and the index reads one or "
                                  "the other - serve with --dcp-size 1 or equal to --tp")
    if not splits_key_heads(tp_size, decode_size):
        return None
    if geometry.query_head_count % tp_size:
        raise NotImplementedError(f"tensor parallel {tp_size} splits {geometry.query_head_count} query heads unevenly, "
                                  "and an index query sums them across ranks that each hold the same count")
    kv_count = geometry.kv_head_count
    if tp_size <= kv_count and kv_count % tp_size == 0:
        held = kv_count // tp_size
        return HeadShard(tp_rank * held, held, geometry.query_head_count // tp_size, True)
    if tp_size > kv_count and tp_size % kv_count == 0:
        replicas = tp_size // kv_count
        return HeadShard(tp_rank // replicas, 1, geometry.query_head_count // tp_size, tp_rank % replicas == 0)
    raise NotImplementedError(f"tensor parallel {tp_size} neither divides {kv_count} key-value heads nor holds each "
                              "on a whole number of ranks")


def key_and_query(q: torch.Tensor, k: torch.Tensor, geometry: Geometry, heads: HeadShard | None = None) -> KeyAndQuery:
    """The key and query input of a forward's tokens, as views of the heads attention was handed
    (`index_space.py:260-289`): q flat [T, Hq * dh] or [T, Hq, dh], k the same; under `heads` the rank's own."""
    kv_count = geometry.kv_head_count if heads is None else heads.kv_count
    query_count = geometry.query_head_count if heads is None else heads.query_count
    tokens = q.shape[0]
    return KeyAndQuery(k.reshape(tokens, kv_count, geometry.head_dim), q.reshape(tokens, query_count, geometry.head_dim))


def materialise(inputs: KeyAndQuery, geometry: Geometry) -> KeyAndQuery:
    """The same input written out as the reference holds it: keys [T, Hkv * (dh - rotary)] bf16 and the grouped
    queries [T, 1, Hkv * (dh - rotary)] fp32, query head h summed into key head h // G in fp32."""
    tokens, kv_count = inputs.key.shape[0], inputs.key.shape[1]
    free = geometry.head_dim - geometry.rotary_dim
    queries = inputs.query.reshape(tokens, kv_count, -1, geometry.head_dim)[..., geometry.rotary_dim:]
    grouped = queries.sum(2, dtype=torch.float32).reshape(tokens, 1, kv_count * free)
    keys = inputs.key[..., geometry.rotary_dim:].reshape(tokens, -1).to(torch.bfloat16)
    return KeyAndQuery(keys, grouped)
