"""The reference's kernel front doors (`src/lsa/core/kernels/`), by their own names, against the oracle: what a
caller of `ScanSelect`, `expand_in_order`, `expand_by_threshold`, `cluster_ward` and `cluster_node_buckets` gets."""

import numpy as np
import pytest
import torch

from helpers import cuda, mixture, unit_rows

pytestmark = pytest.mark.gpu


def _layer(oracle, tokens=2048, d=32, seed=3):
    raw = mixture(tokens, d, 12, 0.3, seed)
    keys = unit_rows(raw)
    buckets = oracle.build_buckets(keys, 4, 16, 32, 256)
    rng = np.random.default_rng(seed + 1)
    positions = np.sort(rng.choice(np.arange(300, tokens), 96, replace=False))
    queries = unit_rows(raw[positions] + 0.3 * rng.standard_normal((96, d)).astype(np.float32))
    return keys, buckets, queries, positions


def test_packed_keys_round_trip_on_the_device(oracle):
    from lsa_b200 import kernels

    rng = np.random.default_rng(0)
    scores = rng.standard_normal(4096).astype(np.float32)
    scores[:4] = [0.0, -0.0, np.inf, -np.inf]
    ids = rng.integers(-1, 1 << 20, 4096).astype(np.int32)
    keys = kernels.pack_keys(cuda(scores), cuda(ids))
    assert np.array_equal(keys.cpu().numpy(), oracle.pack_keys(scores, ids))
    assert np.array_equal(kernels.unpack_ids(keys).cpu().numpy(), ids)
    held = ids >= 0
    assert np.array_equal(kernels.unpack_scores(keys).cpu().numpy()[held].view(np.int32), scores[held].view(np.int32))


def test_scan_select_then_expand_in_order_is_the_oracles_read(oracle):
    from lsa_b200 import kernels

    keys, buckets, queries, positions = _layer(oracle)
    visible = (positions // 256 * (256 // 16)).astype(np.int32)
    scan = kernels.ScanSelect(128, 6)
    picked = scan(cuda(queries), cuda(buckets.bucket_centroids), cuda(visible))
    listing = scan.listed(cuda(queries), cuda(buckets.bucket_centroids), cuda(visible))
    assert scan.holds_top_p(listing) and scan.missed_runs(listing, [(0, 96)]) == [False]
    want, want_len, want_picked, _ = oracle.read(queries, positions, buckets, 6, 150, 4, 256, return_picked=True)
    assert np.array_equal(picked.cpu().numpy(), want_picked)
    lists, lengths = kernels.expand_in_order(picked, cuda(buckets.bucket_members), cuda(positions), 256, 4, 150)
    assert np.array_equal(lengths.cpu().numpy(), want_len)
    assert np.array_equal(lists.cpu().numpy(), want)

    # a slot table stores every position as its KV slot
    rng = np.random.default_rng(5)
    table = np.stack([rng.permutation(4096).astype(np.int32) for _ in range(3)])
    rows = rng.integers(0, 3, 96).astype(np.int32)
    lists, lengths = kernels.expand_in_order(picked, cuda(buckets.bucket_members), cuda(positions), 256, 4, 150,
                                             slot_table=cuda(table), slot_rows=cuda(rows))
    got = lists.cpu().numpy()
    for r in range(96):
        n = int(want_len[r])
        assert np.array_equal(got[r, :n], table[rows[r], want[r, :n]])
        assert (got[r, n:] == -1).all()


def test_expand_by_threshold_walks_the_best_top_p_of_a_listing(oracle):
    from lsa_b200 import kernels

    keys, buckets, queries, positions = _layer(oracle, seed=9)
    visible = (positions // 256 * (256 // 16)).astype(np.int32)
    # a listing wider than top_p, out of order, as a threshold pass leaves it
    wide, _ = kernels.ScanSelect(128, 16).listed(cuda(queries), cuda(buckets.bucket_centroids), cuda(visible))
    shuffled = wide[:, torch.randperm(16, generator=torch.Generator().manual_seed(0)).cuda()].contiguous()
    listed = torch.full((96,), 16, dtype=torch.int32, device="cuda")
    pages = torch.arange(buckets.bucket_centroids.shape[0] // 16, dtype=torch.int32, device="cuda")[None]
    lists = kernels.expand_by_threshold(shuffled, listed, cuda(buckets.bucket_members), None, pages,
                                        torch.zeros(96, dtype=torch.int32, device="cuda"), cuda(positions), 16, 256,
                                        6, 256, 4, 150)
    want, _ = oracle.read(queries, positions, buckets, 6, 150, 4, 256)
    assert np.array_equal(lists.cpu().numpy(), want)


def test_cluster_front_doors(oracle):
    from lsa_b200 import kernels

    keys = unit_rows(mixture(1024, 32, 8, 0.3, 21))
    pools = oracle.pool_keys(keys.reshape(4, 256, 32), 4)
    labels, reached = kernels.cluster_ward(cuda(pools), 4.0, 16, 32.0)
    want = oracle.ward_rounds(pools, np.full((4, 64), 4.0, dtype=np.float32), 16, 32.0)
    assert np.array_equal(labels.cpu().numpy(), want[0]) and reached.all()
    members = kernels.bucket_members_from_labels(labels, 16, 32, pool_size=4)
    assert np.array_equal(members.cpu().numpy(), oracle.build_buckets(keys, 4, 16, 32, 256).bucket_members)

    buckets = oracle.build_buckets(keys, 4, 16, 32, 256)
    sums = oracle.gather_sum(keys, buckets.bucket_members).reshape(2, 32, 32)
    pairs = kernels.cluster_node_buckets(cuda(sums))
    assert np.array_equal(pairs.cpu().numpy(), oracle.ward_rounds(sums, np.ones((2, 32), dtype=np.float32), 16, 2.0)[0])
