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


def test_the_two_pass_forms_dense_keys_paged_scores_and_the_top_k(oracle):
    from lsa_b200 import kernels

    rng = np.random.default_rng(8)
    R, N, d = 37, 1500, 64
    cents = unit_rows(rng.standard_normal((N, d), dtype=np.float32))
    cents[40:80] = cents[40]  # ties: the lower column wins
    queries = unit_rows(rng.standard_normal((R, d), dtype=np.float32)) * rng.uniform(0.1, 20, (R, 1)).astype(np.float32)
    counts = rng.integers(0, N + 1, R).astype(np.int32)
    counts[:3] = [0, 1, N]
    want = np.full((R, N), oracle.EMPTY_KEY, dtype=np.int64)
    scores = np.full((R, N), -np.inf, dtype=np.float32)
    for r in range(R):
        n = int(counts[r])
        if n:
            scores[r, :n] = oracle.scores(queries[r], cents[:n])
            want[r, :n] = oracle.pack_keys(scores[r, :n], np.arange(n, dtype=np.int32))
    keys = kernels.dense_keys(cuda(queries), cuda(cents), cuda(counts))
    assert np.array_equal(keys.cpu().numpy(), want)
    wide = kernels.dense_keys(cuda(queries), cuda(cents), cuda(counts), width=N + 100)
    assert wide.shape == (R, N + 100) and (wide[:, N:] == oracle.EMPTY_KEY).all()

    # through pages: the same buckets at shuffled rows of a cache, 64 to a page, one request missing a page
    page_rows, pages_each = 64, -(-N // 64)
    order = rng.permutation(R * pages_each + 7).astype(np.int32)
    pages = order[: R * pages_each].reshape(R, pages_each).copy()
    cache = np.zeros(((R * pages_each + 7) * page_rows, d), dtype=np.float32)
    for r in range(R):
        for i in range(pages_each):
            rows = cents[i * page_rows:(i + 1) * page_rows]
            cache[pages[r, i] * page_rows: pages[r, i] * page_rows + len(rows)] = rows
    pages[5, 2] = -1
    got = kernels.scan_paged(cuda(queries), cuda(cache), cuda(pages), cuda(counts), page_rows, N)
    hole = scores.copy()
    hole[5, 2 * page_rows:3 * page_rows] = -np.inf
    assert np.array_equal(got.cpu().numpy().view(np.int32), hole.view(np.int32))

    # the pick over a score matrix: best k with ties to the lower column, as keys and as columns
    k = 48
    pick = kernels.TopK(k, exact=True)
    listed, listed_counts = pick.listed(cuda(scores), cuda(counts))
    best = pick.best().cpu().numpy()
    for r in range(R):
        top = np.sort(want[r])[::-1][:k]
        assert np.array_equal(best[r], top), r
        held = min(k, int(counts[r]))
        assert int(listed_counts[r]) == held
        columns = kernels.unpack_ids(listed[r, :held]).cpu().numpy()
        assert np.array_equal(columns, np.sort(oracle.unpack_ids(top[:held])))
    columns = pick(cuda(scores), cuda(counts)).cpu().numpy()
    assert np.array_equal(columns[2, :k], np.sort(oracle.unpack_ids(np.sort(want[2])[::-1][:k])))
    assert (columns[0] == -1).all() and columns[1, 0] == 0 and (columns[1, 1:] == -1).all()
    assert np.array_equal(kernels.top_keys(cuda(scores), cuda(counts), k).cpu().numpy(), best)

    # thresholds from every stride-th bucket, and the listing they cut
    top_p = 64
    stride, rank = kernels.sample_plan(top_p)
    assert (stride, rank) == (2, 48)
    thresholds = kernels.sample_thresholds(cuda(queries), cuda(cents), cuda(counts), top_p).cpu().numpy()
    for r in (2, 7, 20):
        sampled = scores[r, : counts[r]][::stride]
        want_t = np.sort(sampled)[::-1][rank - 1] if len(sampled) >= rank else -np.inf
        assert thresholds[r] == want_t
    listed_k, listed_n, reached = kernels.listed_keys(cuda(queries), cuda(cents), cuda(counts), cuda(thresholds), 256)
    for r in (2, 7, 20):
        if not np.isfinite(thresholds[r]):
            continue
        shifted = thresholds[r] - 1e-4 * np.linalg.norm(queries[r])
        hit = np.flatnonzero(scores[r] >= np.float32(shifted))
        assert int(listed_n[r]) == len(hit) and int(reached[r]) == int((scores[r] >= thresholds[r]).sum())
        assert np.array_equal(listed_k[r, : min(256, len(hit))].cpu().numpy(), want[r, hit[:256]])
