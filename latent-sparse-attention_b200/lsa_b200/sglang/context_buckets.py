"""Decode CUDA graphs keyed by the longest context in the batch (`src/lsa/sglang/context_buckets.py:1-94`).

A captured graph has static shapes, so what a flat decode hands its scan - the columns of a request's page table -
would follow the server's context length however short the requests. A graph per context range trims those columns
to the range, and a replay picks the graph that covers the batch's longest request, as sglang's batch-size graphs
pick the size. SGLang's decode runner keys a graph by an attention variant: a label it reads from an object with
`capture_labels` and `select`. The plugin hands the runner this one, and the selector reads the label being captured.

Here the scan follows each request's own bucket count on the device, so a range changes no launch's work; what it
trims is the page-table slice a step reads and the bound its counts are cut to. The protocol is the reference's.
"""

from __future__ import annotations

import bisect
import sys
from dataclasses import dataclass

from lsa_b200.sglang.settings import PAGE_SIZE

# A label is the prefix and the range's longest context, or `FULL` for the server's own
LABEL_PREFIX = "context_"
FULL = f"{LABEL_PREFIX}full"

# Where sglang keeps the label of the graph being captured
CAPTURE_MODE = "sglang.srt.model_executor.runner_utils.capture_mode"


@dataclass(frozen=True)
class ContextBuckets:
    """The decode graphs of a server, one a context range, in sglang's attention-variant protocol: the runner asks
    `capture_labels` what to capture and `select(forward_batch)` which of them a replay takes."""

    limits: tuple  # longest context of each range below the server's, ascending

    @property
    def capture_labels(self) -> tuple:
        """Widest first - the full graph, then the ranges from the longest down - so that each capture fits in the
        memory of the one before."""
        return tuple([FULL] + [label_of(limit) for limit in sorted(self.limits, reverse=True)])

    def select(self, forward_batch: object) -> str:
        """The narrowest range that holds the batch's longest request; the full graph when none does, or when the
        lengths are not on the host (`seq_lens_cpu` is the mirror a decode step keeps without a sync)."""
        on_host = getattr(forward_batch, "seq_lens_cpu", None)
        if on_host is None or on_host.numel() == 0:
            return FULL
        at = bisect.bisect_left(self.limits, int(on_host.max()))
        return label_of(self.limits[at]) if at < len(self.limits) else FULL

    @classmethod
    def under(cls, limits: tuple, context_length: int) -> "ContextBuckets | None":
        """The design's ranges that are narrower than the server's own context; None when one graph is all there is."""
        kept = tuple(sorted(limit for limit in limits if limit < context_length))
        return cls(kept) if kept else None


def label_of(limit: int) -> str:
    return LABEL_PREFIX + str(limit)


def captured_limit() -> int | None:
    """The longest context of the graph being captured - None in an eager step, in a replay, while the full graph is
    captured, and on a runner that keys no graph by an attention variant (the getter is then absent)."""
    module = sys.modules.get(CAPTURE_MODE)
    read = getattr(module, "get_capture_attention_variant", None) if module is not None else None
    label = read() if read is not None else None
    if not isinstance(label, str) or label == FULL:
        return None
    digits = label[len(LABEL_PREFIX):] if label.startswith(LABEL_PREFIX) else ""
    return int(digits) if digits.isdigit() else None


def pages_of(limit: int) -> int:
    """Pages of cache rows a request of `limit` keys can fill."""
    return (limit + PAGE_SIZE - 1) // PAGE_SIZE
