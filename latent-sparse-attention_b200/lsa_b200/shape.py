"""Bucket shapes: a bucket's spread about its centroid, and the estimated best key it scores by - the reference's
`lsa.core.shape` (src/lsa/core/shape.py:25-170) by the same names, over the device kernels.

A shape is the covariance of a bucket's index keys about its centroid, kept as its `rank` leading directions with
their variances and one floor (the rest of the trace spread evenly over the directions left out). A direction is
served as one sign bit a dimension, `+-1 / sqrt(d)`; a shaped bucket scores `q . c + z sqrt(q^T Sigma q)`.

`Shapes` holds the sign directions as fp32 rows, as the reference's does; the kernels read the packed form
(`ops.ShapeTable`), and `table` converts. Shapes are built on the device by an exact diagonalisation of each
covariance (`ops.shape_build`), where the reference's torch form calls `torch.linalg.eigh`: a direction comes out as
itself or its negation (a score reads only its square), and directions whose variances tie may come out rotated.
"""

from __future__ import annotations

from collections.abc import Mapping
from dataclasses import dataclass, fields
from typing import Any, NamedTuple

import torch

from lsa_b200 import ops
from lsa_b200.ops import ShapeTable


# The most directions a shape keeps (src/lsa/sglang/settings/design.py:54-55)
MAX_SHAPE_RANK = 8


@dataclass(frozen=True)
class Shape:
    """The knob of a design that shapes its buckets: a sketch of rank `rank` that the score adds as `deviations`
    standard deviations (src/lsa/sglang/settings/design.py:111-160)."""

    rank: int = 2  # directions kept; 0 keeps the trace alone, an even spread
    deviations: float = 2.0  # z

    def __post_init__(self) -> None:
        if isinstance(self.rank, bool) or not isinstance(self.rank, int):
            raise ValueError(f"rank must be an integer - got {self.rank!r}")
        if self.rank < 0:
            raise ValueError(f"rank must be at least 0 - got {self.rank}")
        if self.rank > MAX_SHAPE_RANK:
            raise ValueError(f"a shape keeps at most {MAX_SHAPE_RANK} directions - got rank {self.rank}")
        if isinstance(self.deviations, bool) or not isinstance(self.deviations, (int, float)):
            raise ValueError(f"deviations must be a number - got {self.deviations!r}")
        if not self.deviations > 0:
            raise ValueError(f"deviations must be positive - got {self.deviations}")
        object.__setattr__(self, "deviations", float(self.deviations))

    @classmethod
    def read(cls, owner: str, value: "Shape | Mapping[str, Any] | None") -> "Shape | None":
        """A shape knob from what a settings block holds: a mapping of `rank` and `deviations`, or none."""
        if value is None or isinstance(value, Shape):
            return value
        if not isinstance(value, Mapping):
            raise ValueError(f"{owner} is a mapping of rank and deviations, or null - got {value!r}")
        unknown = sorted(set(value) - {item.name for item in fields(cls)})
        if unknown:
            raise ValueError(f"{owner} does not have {unknown} - a shape has rank and deviations")
        return cls(**value)


class Shapes(NamedTuple):
    """The shapes of some buckets, one row each, aligned with their centroids (shape.py:25-33)."""

    basis: torch.Tensor  # sign directions [m, rank, index_dim] fp32, every entry +-1 / sqrt(d), leading first
    variances: torch.Tensor  # variance along each kept direction [m, rank] fp32, descending
    floor: torch.Tensor  # average variance of the index_dim - rank directions left out [m] fp32


def sign_directions(directions: torch.Tensor) -> torch.Tensor:
    """Directions rounded to one sign bit a dimension, `+-1 / sqrt(d)`, a zero entry to the negative side
    (shape.py:76-85)."""
    return ((directions > 0).float() * 2 - 1) / directions.shape[-1] ** 0.5


def pack_shape_basis(basis: torch.Tensor) -> torch.Tensor:
    """A basis [m, rank, index_dim] packed one bit a dimension, set where the entry is positive: bit j of byte i holds
    dimension 8 i + j (shape.py:140-155). [m, rank, index_dim / 8] uint8."""
    index_dim = basis.shape[-1]
    if index_dim % 8:
        raise ValueError(f"a packed basis needs index_dim a multiple of 8 - got {index_dim}")
    weights = 2 ** torch.arange(8, device=basis.device, dtype=torch.int32)
    grouped = (basis > 0).view(*basis.shape[:-1], index_dim // 8, 8).int()
    return (grouped * weights).sum(-1).to(torch.uint8)


def unpack_shape_basis(packed: torch.Tensor) -> torch.Tensor:
    """A packed basis back to its sign directions [m, rank, index_dim] fp32 (shape.py:158-170)."""
    shifts = torch.arange(8, device=packed.device, dtype=torch.int32)
    bits = (packed.int()[..., None] >> shifts) & 1
    signs = bits.flatten(-2).float() * 2 - 1
    return signs / signs.shape[-1] ** 0.5


def table(shapes: Shapes | ShapeTable, deviations: float) -> ShapeTable:
    """The packed table the kernels read, scoring with `deviations`."""
    if isinstance(shapes, ShapeTable):
        return ShapeTable(shapes.basis, shapes.variances, shapes.floor, float(deviations))
    return ShapeTable(pack_shape_basis(shapes.basis), shapes.variances.float().contiguous(),
                      shapes.floor.float().contiguous(), float(deviations))


def build_shapes(index_keys: torch.Tensor, centroids: torch.Tensor, members: torch.Tensor, rank: int) -> Shapes:
    """Shape every bucket of a table: its covariance's leading directions as signs, their variances and a floor
    (shape.py:88-106). `index_keys` [T, index_dim] unit rows, `centroids` [m, index_dim], `members` [m, slots]
    positions with -1 past a bucket's size. An empty bucket's shape is all zero but its signs."""
    built = ops.shape_build(index_keys, centroids, members, rank)
    return Shapes(unpack_shape_basis(built.basis), built.variances, built.floor)


def spread(index_queries: torch.Tensor, shapes: Shapes | ShapeTable) -> torch.Tensor:
    """The estimated standard deviation of each bucket's key scores under each query [R, m] (shape.py:108-120)."""
    packed = table(shapes, 1.0)
    zero = torch.zeros(packed.floor.shape[0], index_queries.shape[1], device=index_queries.device)
    return ops.shaped_scores(index_queries, zero, packed)


def shaped_scores(index_queries: torch.Tensor, centroids: torch.Tensor, shapes: Shapes | ShapeTable,
                  deviations: float) -> torch.Tensor:
    """Each bucket scored by its estimated best key, `q . c + z sqrt(q^T Sigma q)`, [R, m] fp32 (shape.py:123-137)."""
    return ops.shaped_scores(index_queries, centroids, table(shapes, deviations))
