"""A smaller read budget for early queries (the reference's src/lsa/budget.py)."""

from __future__ import annotations

from collections.abc import Mapping
from dataclasses import dataclass
from typing import Any


@dataclass(frozen=True)
class EarlyBudget:
    """`top_k` and `top_p` of a query whose position is below `position`."""

    position: int
    top_k: int
    top_p: int

    def __post_init__(self) -> None:
        for name in ("position", "top_k", "top_p"):
            value = getattr(self, name)
            if isinstance(value, bool) or not isinstance(value, int):
                raise ValueError(f"early_budget {name} must be an integer - got {value!r}")
            if value < 1:
                raise ValueError(f"early_budget {name} must be at least 1 - got {value}")

    @classmethod
    def read(cls, value: "EarlyBudget | Mapping[str, Any] | None") -> "EarlyBudget | None":
        if value is None or isinstance(value, EarlyBudget):
            return value
        if not isinstance(value, Mapping):
            raise ValueError(f"early_budget is a mapping of position, top_k and top_p, or null - got {value!r}")
        names = ["position", "top_k", "top_p"]
        if sorted(value) != sorted(names):
            raise ValueError(f"early_budget has the keys {names} - got {sorted(value)}")
        return cls(**value)


def budget_at(position: int, top_k: int, top_p: int, early: EarlyBudget | None) -> tuple[int, int]:
    """The (top_k, top_p) a query at `position` reads."""
    if early is not None and position < early.position:
        return early.top_k, early.top_p
    return top_k, top_p
