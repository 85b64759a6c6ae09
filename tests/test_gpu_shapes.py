"""Bucket shapes on the device against the CPU oracle (itself pinned to the reference's shape module by
tests/golden/shapes.npz): the build to the tolerance the reference holds its own device build to
(tests/unit/core/test_shape_kernels.py:95-113), every shaped score bit for bit, the shaped selections key for key."""

import numpy as np
import pytest
import torch

from conftest import golden
from helpers import bf16_round, cuda, layer_inputs, mixture, unit_rows

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from lsa_b200 import ops as module

    return module


@pytest.mark.parametrize("width,size,rank", [(64, 48, 2), (64, 96, 3), (32, 40, 2), (64, 33, 1), (64, 32, 4)])
def test_buckets_of_more_keys_than_a_gram_matrix_takes_go_through_the_covariance(ops, oracle, width, size, rank):
    # (at most 32 keys and fewer than the dims: the Gram matrix; above: the [d, d] covariance - the same shapes)
    keys, centroids, members = anisotropic_buckets(96, size, width, size + rank)
    want = oracle.build_shapes(keys, centroids, members, rank)
    got = ops.shape_build(cuda(keys), cuda(centroids), cuda(members), rank)
    np.testing.assert_allclose(got.variances.cpu().numpy(), want.variances, rtol=1e-3, atol=1e-6)
    np.testing.assert_allclose(got.floor.cpu().numpy(), want.floor, rtol=1e-3, atol=1e-6)
    queries = unit_rows(np.random.default_rng(2).standard_normal((64, width), dtype=np.float32))
    built = oracle.Shapes(got.basis.cpu().numpy(), got.variances.cpu().numpy(), got.floor.cpu().numpy())
    near = np.isclose(oracle.spread(queries, built), oracle.spread(queries, want), rtol=1e-3, atol=1e-5)
    assert near.mean() > 0.99
    full = (members >= 0).sum(1) >= 8
    mine, theirs = got.basis.cpu().numpy()[full, 0], want.basis[full, 0]
    assert ((mine == theirs).all(-1) | (mine == ~theirs).all(-1)).mean() > 0.97


def anisotropic_buckets(count, size, width, seed):
    """Buckets of `size` unit keys spread along two directions of their own (the reference's construction), ragged."""
    rng = np.random.default_rng(seed)
    centres = unit_rows(rng.standard_normal((count, 1, width), dtype=np.float32))
    axes = unit_rows(rng.standard_normal((count, 2, width), dtype=np.float32))
    spreads = rng.standard_normal((count, size, 2), dtype=np.float32) * np.array([0.4, 0.15], np.float32)
    noise = 0.02 * rng.standard_normal((count, size, width), dtype=np.float32)
    keys = unit_rows(centres + (spreads[..., None] * axes[:, None]).sum(2) + noise).reshape(-1, width)
    sizes = rng.integers(size // 2, size + 1, count)
    sizes[:4] = [0, 1, 2, size]
    members = np.arange(count * size, dtype=np.int32).reshape(count, size)
    members = np.where(np.arange(size)[None] < sizes[:, None], members, -1).astype(np.int32)
    held = members >= 0
    centroids = unit_rows((keys[np.maximum(members, 0)] * held[..., None]).sum(1))
    return keys, centroids, members


def table_of(ops, shapes, z):
    return ops.ShapeTable(cuda(shapes.basis), cuda(shapes.variances), cuda(shapes.floor), z)


@pytest.mark.parametrize("width,rank", [(64, 0), (64, 1), (64, 2), (64, 4), (32, 2), (32, 3)])
def test_the_build_is_the_oracles_build(ops, oracle, width, rank):
    keys, centroids, members = anisotropic_buckets(384, 16, width, width + rank)
    want = oracle.build_shapes(keys, centroids, members, rank)
    got = ops.shape_build(cuda(keys), cuda(centroids), cuda(members), rank)
    assert got.basis.shape == (384, rank, width // 8) and got.basis.dtype == torch.uint8
    np.testing.assert_allclose(got.variances.cpu().numpy(), want.variances, rtol=1e-3, atol=1e-6)
    np.testing.assert_allclose(got.floor.cpu().numpy(), want.floor, rtol=1e-3, atol=1e-6)
    assert not got.variances[0].any() and float(got.floor[0]) == 0  # a bucket that holds nothing
    trace = np.trace(oracle.covariances(keys, centroids, members)[0], axis1=1, axis2=2)
    kept = got.variances.sum(1).cpu().numpy() + got.floor.cpu().numpy() * (width - rank)
    np.testing.assert_allclose(kept, trace, rtol=1e-4, atol=1e-6)  # a shape keeps the trace whatever its rank
    queries = unit_rows(np.random.default_rng(1).standard_normal((64, width), dtype=np.float32))
    built = oracle.Shapes(got.basis.cpu().numpy(), got.variances.cpu().numpy(), got.floor.cpu().numpy())
    near = np.isclose(oracle.spread(queries, built), oracle.spread(queries, want), rtol=1e-3, atol=1e-5)
    assert near.mean() > 0.99  # a direction is the same up to its sign, but for a bucket whose variances tie
    if rank:  # the leading direction of a bucket that holds enough keys, bit for bit or its negation
        full = (members >= 0).sum(1) >= 8
        mine, theirs = got.basis.cpu().numpy()[full, 0], want.basis[full, 0]
        same = (mine == theirs).all(-1) | (mine == ~theirs).all(-1)
        assert same.mean() > 0.97


def test_the_build_reads_keys_from_a_base_and_into_rows_of_a_table(ops, oracle):
    keys, centroids, members = anisotropic_buckets(64, 16, 64, 5)
    base = 4096
    shifted = np.where(members >= 0, members + base, -1).astype(np.int32)
    want = ops.shape_build(cuda(keys), cuda(centroids), cuda(members), 2)
    table = ops.ShapeTable(torch.zeros(200, 2, 8, device="cuda", dtype=torch.uint8), torch.zeros(200, 2, device="cuda"),
                           torch.zeros(200, device="cuda"), 2.0)
    ops.shape_build(cuda(keys), cuda(centroids), cuda(shifted), 2, key_base=base, out=table.rows(slice(100, 164)))
    assert torch.equal(table.basis[100:164], want.basis) and torch.equal(table.variances[100:164], want.variances)
    assert torch.equal(table.floor[100:164], want.floor) and not table.floor[:100].any() and not table.floor[164:].any()
    golden_shapes = golden("shapes")  # the reference's own buckets and what it built for them
    got = ops.shape_build(cuda(golden_shapes["w64_keys"]), cuda(golden_shapes["w64_centroids"]),
                          cuda(golden_shapes["w64_members"]), 2)
    np.testing.assert_allclose(got.variances.cpu().numpy(), golden_shapes["w64_r2_variances"], rtol=1e-3, atol=1e-6)
    np.testing.assert_allclose(got.floor.cpu().numpy(), golden_shapes["w64_r2_floor"], rtol=1e-3, atol=1e-6)


@pytest.mark.parametrize("width,rank", [(64, 0), (64, 2), (64, 3), (32, 2), (128, 2), (64, 8)])
def test_shaped_scores_are_the_oracles_bit_for_bit(ops, oracle, width, rank):
    rng = np.random.default_rng(width + rank)
    m, R = 700, 37
    cents = unit_rows(mixture(m, width, 16, 0.4, 2))
    shapes = oracle.Shapes(rng.integers(0, 256, (m, rank, width // 8)).astype(np.uint8),
                           np.sort(rng.uniform(0, 0.05, (m, rank)).astype(np.float32), axis=1)[:, ::-1].copy(),
                           rng.uniform(0, 0.002, m).astype(np.float32))
    queries = unit_rows(rng.standard_normal((R, width), dtype=np.float32))
    table = table_of(ops, shapes, 2.0)
    want = oracle.shaped_scores(queries, cents, shapes, 2.0)
    got = ops.shaped_scores(cuda(queries), cuda(cents), table)
    assert np.array_equal(got.cpu().numpy().view(np.int32), want.view(np.int32))
    rows = rng.integers(-1, m, (R, 200)).astype(np.int32)
    listed = ops.shaped_scores(cuda(queries), cuda(cents), table, rows=cuda(rows)).cpu().numpy()
    expect = np.where(rows >= 0, np.take_along_axis(want, np.maximum(rows, 0), 1), -np.inf).astype(np.float32)
    assert np.array_equal(listed.view(np.int32), expect.view(np.int32))
    # and against the reference's formula in double, to fp32 rounding
    np.testing.assert_allclose(got.cpu().numpy() - queries @ cents.T, 2.0 * oracle.spread(queries, shapes), atol=2e-6)


def _top_keys(oracle, scores, visible, keep, row_keep=None, base=0):
    want = np.full((len(scores), keep), oracle.EMPTY_KEY, dtype=np.int64)
    for r in range(len(scores)):
        n = int(visible[r])
        keys = oracle.pack_keys(scores[r, :n], np.arange(base, base + n, dtype=np.int32))
        top = np.sort(keys)[::-1][: keep if row_keep is None else int(row_keep[r])]
        want[r, : len(top)] = top
    return want


@pytest.mark.parametrize("width,m,keep,rank", [(64, 5000, 64, 2), (32, 3000, 16, 1), (64, 2000, 600, 2), (128, 1500, 32, 2),
                                               (64, 9000, 128, 0)])
def test_a_shaped_selection_is_the_oracles_key_for_key(ops, oracle, width, m, keep, rank):
    rng = np.random.default_rng(m)
    R = 150
    cents = unit_rows(mixture(m, width, 32, 0.4, 3))
    shapes = oracle.Shapes(rng.integers(0, 256, (m, rank, width // 8)).astype(np.uint8),
                           np.sort(rng.uniform(0, 0.08, (m, rank)).astype(np.float32), axis=1)[:, ::-1].copy(),
                           rng.uniform(0, 0.003, m).astype(np.float32))
    queries = unit_rows(cents[rng.integers(0, m, R)] + 0.5 * rng.standard_normal((R, width), dtype=np.float32))
    visible = rng.integers(0, m + 1, R).astype(np.int32)
    visible[:4] = [0, 1, keep, m]
    row_keep = rng.integers(0, keep + 1, R).astype(np.int32)
    table = table_of(ops, shapes, 2.0)
    scores = oracle.shaped_scores(queries, cents, shapes, 2.0)
    got, picked = ops.shaped_select(cuda(queries), cuda(cents), table, cuda(visible), keep)
    assert np.array_equal(got.cpu().numpy(), _top_keys(oracle, scores, visible, keep))
    assert np.array_equal(picked.cpu().numpy(), oracle.unpack_ids(got.cpu().numpy()))
    plain, _ = ops.flat_select(cuda(queries), cuda(cents), cuda(visible), keep)
    assert not torch.equal(plain, got)  # the spread changes what a row picks
    got, _ = ops.shaped_select(cuda(queries), cuda(cents), table, cuda(visible), keep, row_top_p=cuda(row_keep),
                               bucket_id_base=70000)
    assert np.array_equal(got.cpu().numpy(), _top_keys(oracle, scores, visible, keep, row_keep, 70000))
    # no deviations: the centroids' own scores, whatever the shapes
    got, _ = ops.shaped_select(cuda(queries), cuda(cents), table_of(ops, shapes, 0.0), cuda(visible), keep)
    assert torch.equal(got, plain)


def test_a_shaped_decode_scan_is_the_oracles_over_requests_and_splits(ops, oracle):
    rng = np.random.default_rng(9)
    m, R, keep = 6000, 5, 64
    cents = unit_rows(mixture(m, 64, 32, 0.4, 4))
    shapes = oracle.Shapes(rng.integers(0, 256, (m, 2, 8)).astype(np.uint8),
                           np.sort(rng.uniform(0, 0.08, (m, 2)).astype(np.float32), axis=1)[:, ::-1].copy(),
                           rng.uniform(0, 0.003, m).astype(np.float32))
    queries = unit_rows(rng.standard_normal((R, 64), dtype=np.float32))
    first = np.array([0, 1000, 1000, 2500, 5990], dtype=np.int64)
    visible = np.array([1000, 1500, 0, 3400, 10], dtype=np.int32)
    table = table_of(ops, shapes, 1.5)
    want = np.full((R, keep), oracle.EMPTY_KEY, dtype=np.int64)
    for r in range(R):
        part = slice(int(first[r]), int(first[r]) + int(visible[r]))
        own = oracle.Shapes(shapes.basis[part], shapes.variances[part], shapes.floor[part])
        scores = oracle.shaped_scores(queries[r:r + 1], cents[part], own, 1.5)
        want[r] = _top_keys(oracle, scores, visible[r:r + 1], keep)[0]
    for splits in (1, 4, 16):
        got, picked = ops.shaped_select_decode(cuda(queries), cuda(cents), table, cuda(first), cuda(visible), keep,
                                               splits=splits)
        assert np.array_equal(got.cpu().numpy(), want)
        assert np.array_equal(picked.cpu().numpy(), oracle.unpack_ids(want))


def test_the_operator_api_reads_shaped_buckets_as_the_reference_does(oracle):
    from lsa_b200 import core, shape

    g = golden("shapes")
    buckets = core.Buckets(cuda(g["read_centroids"]), cuda(g["read_members"]),
                           cuda((g["read_members"] >= 0).sum(1).astype(np.int32)), 8, 64)
    shapes = shape.Shapes(shape.unpack_shape_basis(cuda(g["read_basis"])), cuda(g["read_variances"]),
                          cuda(g["read_floor"]))
    assert torch.equal(shape.pack_shape_basis(shapes.basis), cuda(g["read_basis"]))
    queries, positions = cuda(g["read_queries"]), cuda(g["read_positions"])
    for z in (0, 2):
        selected, lengths = core.read(queries, positions, buckets, 4, 16, 2, 24, shapes, float(z))
        assert np.array_equal(lengths.cpu().numpy(), g[f"read_z{z}_lengths"])
        assert np.array_equal(selected.cpu().numpy(), g[f"read_z{z}_selected"])
    built = core.shape_buckets(cuda(g["read_keys"]), buckets, 2)
    np.testing.assert_allclose(built.variances.cpu().numpy(), g["read_variances"], rtol=1e-3, atol=1e-6)
    theirs = oracle.spread(g["read_queries"], oracle.Shapes(g["read_basis"], g["read_variances"], g["read_floor"]))
    assert np.isclose(shape.spread(queries, built).cpu().numpy(), theirs, rtol=1e-3, atol=1e-5).mean() > 0.99
    with pytest.raises(ValueError, match="rank must be from 0 to the keys' width 32 - got 33"):
        core.shape_buckets(cuda(g["read_keys"]), buckets, 33)
    want = oracle.shaped_scores(g["read_queries"], g["read_centroids"],
                                oracle.Shapes(g["read_basis"], g["read_variances"], g["read_floor"]), 2.0)
    got = shape.shaped_scores(queries, buckets.bucket_centroids, shapes, 2.0)
    assert np.array_equal(got.cpu().numpy().view(np.int32), want.view(np.int32))


def test_a_layer_of_a_shaped_design_reads_by_estimated_best_keys(oracle):
    from lsa_b200.layer import FlatDesign, FlatLayer

    design = FlatDesign(pool_size=4, bucket_size=16, bucket_cap=32, cluster_block_size=256, top_p=8, top_k=256,
                        sink_size=4, window_size=256, bucket_shape={"rank": 2, "deviations": 2.0})
    T, Hq, Hkv, dh, d_idx = 3000, 16, 4, 128, 64
    rng = np.random.default_rng(12)
    w = bf16_round(rng.standard_normal((2, Hkv * dh, d_idx), dtype=np.float32) / np.sqrt(Hkv * dh))
    layer = FlatLayer(design, cuda(w[0], torch.bfloat16), cuda(w[1], torch.bfloat16), Hq, Hkv, dh)
    q, k, v = layer_inputs(T, Hq, Hkv, dh, 16, 13)
    Q, K, V = (cuda(a, torch.bfloat16) for a in (q, k, v))
    out, index = layer.prefill(Q, K, V, chunk=1024, return_index=True)
    assert index.shapes is not None and index.shapes.deviations == 2.0
    index_q, index_k = layer.index_queries(Q).cpu().numpy(), index.index_keys.cpu().numpy()
    buckets = oracle.build_buckets(index_k, design.pool_size, design.bucket_size, design.bucket_cap,
                                   design.cluster_block_size)
    assert np.array_equal(index.buckets.bucket_members.cpu().numpy(), buckets.bucket_members)
    # the shapes the blocks were given as they closed: the oracle's build of the same buckets
    mine = oracle.Shapes(index.shapes.basis.cpu().numpy(), index.shapes.variances.cpu().numpy(),
                         index.shapes.floor.cpu().numpy())
    theirs = oracle.shape_buckets(index_k, buckets, 2)
    np.testing.assert_allclose(mine.variances, theirs.variances, rtol=1e-3, atol=1e-6)
    np.testing.assert_allclose(mine.floor, theirs.floor, rtol=1e-3, atol=1e-6)
    probe_q = index_q[:: T // 50]
    assert np.isclose(oracle.spread(probe_q, mine), oracle.spread(probe_q, theirs), rtol=1e-3, atol=1e-5).mean() > 0.99
    # from the device's own shapes on, every list is the oracle's shaped read
    positions = np.arange(T)
    lists, lengths = layer.select(cuda(index_q), cuda(positions), index)
    want_lists, want_lengths = oracle.read(index_q, positions, buckets, design.top_p, design.top_k, design.sink_size,
                                           design.window_size, shapes=mine, deviations=2.0)
    assert np.array_equal(lengths.cpu().numpy(), want_lengths)
    assert np.array_equal(lists.cpu().numpy(), want_lists)
    plain, _ = oracle.read(index_q, positions, buckets, design.top_p, design.top_k, design.sink_size,
                           design.window_size)
    assert not np.array_equal(plain, want_lists)
    rows = np.arange(0, T, 41)
    want, _ = oracle.sparse_attend(q[rows], k, v, want_lists[rows], rows, 0, 0, dh ** -0.5, lengths=want_lengths[rows])
    err = np.abs(out.float().cpu().numpy()[rows] - want)
    assert err.max() <= 2e-2 and err.mean() <= 2e-3, (err.max(), err.mean())
    at = torch.tensor([5, 255, 256, 1000, 2999]).cuda()
    step = layer.decode(Q[at], at, K, V, index, splits=4)
    assert (step.float() - out[at].float()).abs().max() <= 1e-2
    with pytest.raises(ValueError, match="bucket_shape keeps at most bucket_cap 4 directions - got rank 5"):
        FlatDesign(pool_size=1, bucket_size=2, bucket_cap=4, cluster_block_size=64, top_p=64, top_k=64,
                   bucket_shape={"rank": 5})


def test_a_serving_cache_pages_the_shapes_with_the_centroids(oracle):
    from lsa_b200.layer import FlatDesign
    from lsa_b200.serving import BucketCache, Selector

    design = FlatDesign(pool_size=4, bucket_size=16, bucket_cap=32, cluster_block_size=256, top_p=6, top_k=150,
                        sink_size=4, window_size=256, bucket_shape={"rank": 2, "deviations": 2.0})
    d_idx, page_buckets = 32, 32
    lengths = [700, 2048, 3000]
    rng = np.random.default_rng(0)
    cache = BucketCache(design, d_idx, pages=16, page_buckets=page_buckets, max_requests=4, max_request_pages=8)
    slots = rng.permutation(4 * 3072).astype(np.int32).reshape(4, 3072)  # a request table of one-token pages
    selector = Selector(cache, 1, slot_table=lambda: cuda(slots))
    raws = [mixture(n, d_idx, 10, 0.3, 100 + r) for r, n in enumerate(lengths)]
    keys = [unit_rows(raw) for raw in raws]
    for r, n in enumerate(lengths):  # in pieces, the requests interleaved: their pages interleave too
        cache.append(r, cuda(keys[r][: n // 3]))
    for r, n in enumerate(lengths):
        cache.append(r, cuda(keys[r][n // 3:]))
    positions = np.array([n - 1 for n in lengths])
    queries = np.stack([unit_rows(raws[r][positions[r]] + 0.3 * rng.standard_normal(d_idx).astype(np.float32))
                        for r in range(len(lengths))])

    def own_shapes(r):
        held = cache.gather_shapes(r, cache.buckets_of(r))
        return oracle.Shapes(held.basis.cpu().numpy(), held.variances.cpu().numpy(), held.floor.cpu().numpy())

    for r in range(len(lengths)):  # what the cache built page by page is the oracle's build of the whole request
        buckets = oracle.build_buckets(keys[r], 4, 16, 32, 256)
        want = oracle.shape_buckets(keys[r], buckets, 2)
        np.testing.assert_allclose(own_shapes(r).variances, want.variances, rtol=1e-3, atol=1e-6)
        np.testing.assert_allclose(own_shapes(r).floor, want.floor, rtol=1e-3, atol=1e-6)
    rows = torch.arange(len(lengths)).cuda()
    for splits in (1, 3):
        lists = selector.decode(cuda(queries), cuda(positions), rows, splits=splits)
        for r in range(len(lengths)):
            buckets = oracle.build_buckets(keys[r], 4, 16, 32, 256)
            want, want_len = oracle.read(queries[r:r + 1], positions[r:r + 1], buckets, 6, 150, 4, 256,
                                         shapes=own_shapes(r), deviations=2.0)
            ids = want[0, : want_len[0]]
            assert np.array_equal(lists[r, : int(want_len[0])].cpu().numpy(), slots[r][ids]), (r, splits)
            assert (lists[r, int(want_len[0]):] == -1).all()
    # a prefill segment of a fourth request: keys appended, every query reads the blocks closed before it, shaped
    raw = mixture(1500, d_idx, 10, 0.3, 7)
    seg_keys, seg_q = unit_rows(raw), unit_rows(raw + 0.3 * rng.standard_normal(raw.shape).astype(np.float32))
    got = selector.prefill(3, cuda(seg_q), cuda(np.arange(1500)), cuda(seg_keys), 0)
    buckets = oracle.build_buckets(seg_keys, 4, 16, 32, 256)
    want, want_len = oracle.read(seg_q, np.arange(1500), buckets, 6, 150, 4, 256, shapes=own_shapes(3), deviations=2.0)
    for r in (0, 255, 256, 700, 1499):
        ids = want[r, : want_len[r]]
        assert np.array_equal(got[r, : int(want_len[r])].cpu().numpy(), slots[3][ids]), r


def test_the_front_doors_by_the_references_names(ops, oracle):
    # (tests/unit/core/test_shape_kernels.py:116-164: rows scored, the dense spread, the decode scan through pages)
    from lsa_b200 import kernels

    keys, centroids, members = anisotropic_buckets(512, 16, 64, 2)
    basis, variances, floor = kernels.build_bucket_shapes(lambda positions: cuda(keys)[positions], cuda(centroids),
                                                          cuda(members), 2)
    again = kernels.build_shapes(cuda(keys), cuda(centroids), cuda(members), 2)
    assert torch.equal(basis, again[0]) and torch.equal(variances, again[1]) and torch.equal(floor, again[2])
    table = kernels.ShapeTable(basis, variances, floor, 2.0)
    mine = oracle.Shapes(basis.cpu().numpy(), variances.cpu().numpy(), floor.cpu().numpy())
    rng = np.random.default_rng(3)
    queries = unit_rows(rng.standard_normal((32, 64), dtype=np.float32))
    want = oracle.shaped_scores(queries, centroids, mine, 2.0)
    rows = rng.integers(-1, 512, (32, 200)).astype(np.int32)
    got = kernels.score_shaped_rows(cuda(queries), cuda(centroids), basis, variances, floor, cuda(rows), 2.0)
    expect = np.where(rows >= 0, np.take_along_axis(want, np.maximum(rows, 0), 1), -np.inf).astype(np.float32)
    assert np.array_equal(got.cpu().numpy().view(np.int32), expect.view(np.int32))
    # the dense spread and the row scoring agree on the spread bit for bit
    zero = torch.zeros(512, 64, device="cuda")
    every = torch.arange(512, device="cuda", dtype=torch.int32).expand(32, -1).contiguous()
    from_rows = kernels.score_shaped_rows(cuda(queries), zero, basis, variances, floor, every, 2.0)
    dense = kernels.add_planes_spread(torch.zeros(32, 512, device="cuda"), cuda(queries), table)
    assert torch.equal(dense, from_rows)
    assert torch.equal(kernels.add_spread(torch.zeros(32, 512, device="cuda"), cuda(queries), basis, variances, floor,
                                          2.0), dense)
    np.testing.assert_allclose(dense.cpu().numpy(), 2.0 * oracle.spread(queries, mine), atol=2e-6)
    # the decode scan scores each page row as the row scoring does
    page_size = 128
    page_table = torch.tensor([[2, 0, 3, -1], [1, 3, -1, -1]], device="cuda", dtype=torch.int32)
    counts = torch.tensor([3 * page_size - 7, page_size + 5], device="cuda", dtype=torch.int32)
    scores = kernels.scan_paged_shaped(cuda(queries[:2]), cuda(centroids), table, page_table, counts, page_size,
                                       4 * page_size)
    logical = torch.arange(4 * page_size, device="cuda")
    for request in range(2):
        page = page_table[request, logical // page_size]
        held = (logical < counts[request]) & (page >= 0)
        at = torch.where(held, page * page_size + logical % page_size, -1).int()[None]
        expect = kernels.score_shaped_rows(cuda(queries[request:request + 1]), cuda(centroids), basis, variances, floor,
                                           at, 2.0)
        assert torch.equal(scores[request:request + 1], expect)
    # the two-pass selection over shaped buckets: dense keys, then the front door's pick
    visible = cuda(rng.integers(0, 513, 32).astype(np.int32))
    dense_keys = kernels.dense_keys(cuda(queries), cuda(centroids), visible, shapes=table)
    select = kernels.ScanSelect(32, 16)
    picked = select(cuda(queries), cuda(centroids), visible, shapes=table)
    top = dense_keys.sort(dim=1, descending=True).values[:, :16]
    assert torch.equal(select.keys, top)
    assert torch.equal(picked, kernels.unpack_ids(top).to(torch.int32))
