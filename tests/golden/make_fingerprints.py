"""Generate tests/golden/fingerprints.npz by running the reference's own page fingerprints on inputs a formula makes.

Run where the reference is mounted (it is imported in place, never copied):

    python tests/golden/make_fingerprints.py <checkout of the reference>/src

The stored bits are `pattern(rows, dim)` below, which the tests rebuild, so the fixture holds only the reference's
weights (a sample and a wrapping sum of all of them) and the fingerprints it returned
(src/lsa/sglang/index/layer_index.py:89-137).
"""

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def pattern(rows: int, dim: int) -> np.ndarray:
    """16-bit words [rows, dim] that differ row to row and column to column."""
    i, j = np.arange(rows, dtype=np.int64)[:, None], np.arange(dim, dtype=np.int64)[None]
    return ((i * 40503 + j * 1201 + (i * j) % 251 + 7) & 0xFFFF).astype(np.uint16)


def main(src):
    sys.path.insert(0, src)
    from lsa.sglang.index.layer_index import PAGE_SIZE, exact_group_sum, fingerprint_weights, page_fingerprints

    words, positions = fingerprint_weights("cpu")
    out = {"page_size": np.int64(PAGE_SIZE), "words_head": words[:16].numpy(), "positions_head": positions[:16].numpy(),
           "words_sum": words.sum().numpy(), "positions_sum": positions.sum().numpy(),
           "words_count": np.int64(words.shape[0])}
    for dim in (16, 64, 512):
        bits = pattern(3 * PAGE_SIZE, dim)
        stored = torch.from_numpy(bits.view(np.int16)).view(torch.bfloat16)
        every = torch.ones(3 * PAGE_SIZE, dtype=torch.bool)
        out[f"d{dim}_all"] = page_fingerprints(stored, every).numpy()
        parts = []
        for rank in range(3):  # a decode group of three: each rank adds the slots it owns, the group's sum is the page's
            owned = torch.arange(3 * PAGE_SIZE) % 3 == rank
            parts.append(page_fingerprints(stored, owned))
            out[f"d{dim}_rank{rank}"] = parts[-1].numpy()
        total = exact_group_sum(parts[0], lambda pieces: pieces + exact_pieces(parts[1]) + exact_pieces(parts[2]))
        assert torch.equal(total, page_fingerprints(stored, every))
    np.savez_compressed(os.path.join(HERE, "fingerprints.npz"), **out)
    print({k: v.shape for k, v in out.items()})


def exact_pieces(values: torch.Tensor) -> torch.Tensor:
    """Another rank's 16-bit pieces, as the group's collective would add them."""
    shifts = 16 * torch.arange(4)
    return ((values[:, None] >> shifts) & 0xFFFF).float()


if __name__ == "__main__":
    main(sys.argv[1])
