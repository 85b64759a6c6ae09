"""Generate tests/golden/shapes.npz by running the reference's own `lsa.core.shape` and shaped `read` on seeded inputs.

Run where the reference is mounted (it is imported in place, never copied):

    python tests/golden/make_shapes.py <checkout of the reference>/src

The constructions follow the reference's unit tests (tests/unit/core/test_shape.py: buckets spread along two
directions of their own, padded members, rank 0 to full; a shaped read over built buckets).
"""

import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))


def anisotropic_buckets(count, size, width, generator):
    centres = F.normalize(torch.randn(count, 1, width, generator=generator), dim=-1)
    axes = F.normalize(torch.randn(count, 2, width, generator=generator), dim=-1)
    spreads = torch.randn(count, size, 2, generator=generator) * torch.tensor([0.4, 0.2])
    noise = 0.02 * torch.randn(count, size, width, generator=generator)
    keys = F.normalize(centres + (spreads[..., None] * axes[:, None]).sum(2) + noise, dim=-1)
    return keys.view(-1, width)


def main(src):
    sys.path.insert(0, src)
    from lsa.core import build_buckets, read, shape_buckets
    from lsa.core.shape import build_shapes, covariances, pack_shape_basis, shaped_scores, spread

    torch.set_num_threads(1)
    out = {}

    # ---- shapes of ragged buckets, ranks 0..4 and full (test_shape.py:40-83)
    for width in (32, 64):
        gen = torch.Generator().manual_seed(width)
        count, size = 24, 16
        keys = anisotropic_buckets(count, size, width, gen)
        sizes = torch.randint(1, size + 1, (count,), generator=gen)
        sizes[:3] = torch.tensor([1, 2, size])
        members = torch.arange(count * size).view(count, size)
        members = torch.where(torch.arange(size)[None] < sizes[:, None], members, -1)
        held = members >= 0
        centroids = F.normalize((keys[members.clamp_min(0)] * held[..., None]).sum(1), dim=-1)
        queries = F.normalize(torch.randn(12, width, generator=gen), dim=-1)
        tag = f"w{width}_"
        out[tag + "keys"], out[tag + "centroids"], out[tag + "members"] = keys, centroids, members.int()
        out[tag + "queries"] = queries
        if width == 32:
            out[tag + "covariances"] = covariances(keys, centroids, members)[0]
        for rank in (0, 1, 2, 4, width):
            shapes = build_shapes(keys, centroids, members, rank)
            out[f"{tag}r{rank}_basis"] = pack_shape_basis(shapes.basis)
            out[f"{tag}r{rank}_variances"] = shapes.variances
            out[f"{tag}r{rank}_floor"] = shapes.floor
            out[f"{tag}r{rank}_spread"] = spread(queries, shapes)
            out[f"{tag}r{rank}_scores"] = shaped_scores(queries, centroids, shapes, 2.0)

    # ---- a shaped read over built buckets (test_shape.py:96-111), at two deviations
    gen = torch.Generator().manual_seed(7)
    keys = F.normalize(torch.randn(6 * 64, 32, generator=gen), dim=-1)
    buckets = build_buckets(keys, 4, 8, 16, 64)
    shapes = shape_buckets(keys, buckets, 2)
    queries = F.normalize(torch.randn(20, 32, generator=gen), dim=-1)
    positions = torch.randint(64, 6 * 64, (20,), generator=gen)
    out["read_keys"], out["read_queries"], out["read_positions"] = keys, queries, positions
    out["read_centroids"], out["read_members"] = buckets.bucket_centroids, buckets.bucket_members.int()
    out["read_basis"] = pack_shape_basis(shapes.basis)
    out["read_variances"], out["read_floor"] = shapes.variances, shapes.floor
    for z in (0.0, 2.0):
        selected, lengths = read(queries, positions, buckets, 4, 16, 2, 24, shapes, z)
        out[f"read_z{int(z)}_selected"], out[f"read_z{int(z)}_lengths"] = selected, lengths

    arrays = {k: (v.numpy() if isinstance(v, torch.Tensor) else np.asarray(v)) for k, v in out.items()}
    np.savez_compressed(os.path.join(HERE, "shapes.npz"), **arrays)
    print({k: v.shape for k, v in arrays.items()})


if __name__ == "__main__":
    main(sys.argv[1])
