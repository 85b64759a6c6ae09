"""The maps a server reads index keys and index queries with: one pair a sparse layer, from the flat torch file the
reference's distillation exports (`src/lsa/sglang/index/weights.py:118-162`): `<layer>.W_Q_idx` and `<layer>.W_K_idx`,
each [input_dim, index_dim]. A file may hold more layers than the model indexes; a file whose shapes are not the
input's dims by the design's index dim, or that lacks an indexed layer, is refused with the reason."""

from __future__ import annotations

import re
from collections.abc import Collection
from pathlib import Path
from typing import Any

import torch

from lsa_b200.sglang import index_space

QUERY = "W_Q_idx"
KEY = "W_K_idx"
_ENTRY = re.compile(rf"(?P<layer>\d+)\.(?P<kind>{QUERY}|{KEY})")


def indexed_layers(config: Any) -> list:
    """The layers the design indexes on a grouped-query model: its quadratic ones (weights.py:49-66)."""
    return list(index_space.geometry_of(config).layers)


def input_dim(config: Any) -> int:
    """Dims the maps read: every key head's position-free dims, side by side (weights.py:69-88)."""
    return index_space.geometry_of(config).key_dim


def key_slot(config: Any) -> index_space.KeySlot:
    return index_space.geometry_of(config).key_slot


def read(path: str | Path, input_dim: int, index_dim: int, layers: Collection) -> dict:
    """Each indexed layer's (query map, key map), both [input_dim, index_dim] fp32 on the host.

    Raises:
        ValueError: The file is not a flat dict of `<layer>.W_Q_idx` / `<layer>.W_K_idx` tensors; a map is not
            [input_dim, index_dim]; a layer holds one map of the two; or an indexed layer is missing.
    """
    entries = torch.load(path, map_location="cpu", weights_only=True)
    if not isinstance(entries, dict) or not entries:
        raise ValueError(f"{path} is not a projection file - it holds no '<layer>.{QUERY}' tensors")
    wanted = (input_dim, index_dim)
    maps: dict = {}  # layer -> {W_Q_idx: tensor, W_K_idx: tensor}
    for name, tensor in entries.items():
        match = _ENTRY.fullmatch(str(name))
        if match is None or not torch.is_tensor(tensor):
            raise ValueError(f"{path} holds {name!r} - a projection file holds '<layer>.{QUERY}' and '<layer>.{KEY}'")
        if tuple(tensor.shape) != wanted:
            raise ValueError(f"{path} {name} is {tuple(tensor.shape)} - expected [input_dim, index_dim] = "
                             f"{list(wanted)} for the design's indexer input")
        maps.setdefault(int(match["layer"]), {})[match["kind"]] = tensor.float()
    halves = sorted(layer for layer, pair in maps.items() if len(pair) < 2)
    if halves:
        raise ValueError(f"{path} holds only one of {QUERY} and {KEY} for layers {halves}")
    absent = sorted(set(layers).difference(maps))
    if absent:
        raise ValueError(f"{path} holds layers {sorted(maps)}, and the layers that run an indexer are "
                         f"{sorted(layers)} - missing {absent}")
    return {layer: (maps[layer][QUERY], maps[layer][KEY]) for layer in sorted(set(layers))}
