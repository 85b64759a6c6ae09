"""The CPU oracle held to the reference: golden vectors the reference itself produced, and the known-answer cases
of its unit tests (tests/unit/core/test_ward.py:42-47,68-74,91-95 and test_attention.py). Integer results must
be equal; floats within the stated tolerance."""

import numpy as np
import pytest

from conftest import golden


def sets(lists):
    return [sorted(row[row >= 0].tolist()) for row in lists]


def test_packed_keys_match_the_reference(oracle):
    g = golden("packed_keys")
    keys = oracle.pack_keys(g["scores"], g["ids"])
    assert np.array_equal(keys, g["keys"])
    assert np.array_equal(oracle.unpack_ids(keys), g["unpacked_ids"])
    assert np.array_equal(oracle.unpack_scores(keys).view(np.int32), g["unpacked_scores"].view(np.int32))
    # greater key = greater score, and the lower id at an equal score
    order = np.argsort(-keys, kind="stable")
    assert g["ids"][order].tolist()[:2] == [6, 2]
    assert keys[9] > keys[8]
    assert oracle.pack_keys([1.0], [-1])[0] == oracle.EMPTY_KEY


def test_regroup_and_project_match_the_reference(oracle):
    g = golden("index_space")
    iq, ik = oracle.regroup(g["q"], g["k"])
    np.testing.assert_allclose(iq, g["index_queries"], rtol=0, atol=2e-7)
    np.testing.assert_allclose(ik, g["index_keys"], rtol=0, atol=2e-7)
    assert not ik[7].any()
    np.testing.assert_allclose(oracle.project(iq, g["w"]), g["projected_queries"], rtol=0, atol=5e-7)
    np.testing.assert_allclose(oracle.project(ik, g["w"]), g["projected_keys"], rtol=0, atol=5e-7)
    assert not oracle.project(ik, g["w"])[7].any()
    with pytest.raises(ValueError, match="dims"):
        oracle.project(iq[:, :8], g["w"])


def test_latent_regroup_matches_the_reference(oracle):
    """The MLA index space (src/lsa/core/index_space.py:240-312): the factor, both sides' unit rows, and the property
    the reference's own test checks - the latent scores rank keys as the expanded keys' scores do."""
    g = golden("latent_space")
    factor = oracle.latent_metric_factor(g["key_maps"])
    assert np.abs(factor - g["metric_factor"]).max() <= 2e-6
    iq, ik = oracle.regroup_latent(g["q"], g["latent"], g["key_maps"], factor)
    assert np.abs(iq - g["index_queries"]).max() <= 5e-6
    assert np.abs(ik - g["index_keys"]).max() <= 5e-6
    assert not ik[5].any()  # a zero latent stays zero
    narrow = iq @ ik.T
    held = np.ones(40, dtype=bool)
    held[5] = False
    assert np.array_equal(np.argsort(narrow[:, held], axis=1), np.argsort(g["wide_scores"][:, held], axis=1))
    degenerate = g["key_maps"].copy()
    degenerate[..., -1] = 0
    with pytest.raises(ValueError, match="do not span"):
        oracle.latent_metric_factor(degenerate)


def test_pooling_matches_the_reference(oracle):
    g = golden("ward")
    np.testing.assert_allclose(oracle.pool_keys(g["c_keys"], 16), g["c_pools"], rtol=0, atol=1e-6)


@pytest.mark.parametrize("tag", ["a", "b", "c", "d", "e"])
def test_ward_labels_match_the_reference(oracle, tag):
    g = golden("ward")
    pool, count, cap = g[f"{tag}_args"].tolist()
    pools = g[f"{tag}_pools"]
    sizes = np.full(pools.shape[:2], float(pool), dtype=np.float32)
    labels = oracle.ward_merge(pools, sizes, count, cap)
    assert np.array_equal(labels, g[f"{tag}_labels"])


@pytest.mark.parametrize("tag", ["near", "rounded"])
def test_ward_on_near_copied_and_rounded_pools(oracle, tag):
    g = golden("ward")
    pool, count, cap = g[f"{tag}_args"].tolist()
    pools = g[f"{tag}_pools"]
    labels, reached = oracle.ward_rounds(pools, np.full(pools.shape[:2], float(pool), np.float32), count, cap)
    assert np.array_equal(reached, g[f"{tag}_reached"])
    # Costs that differ by one rounding can order pairs otherwise: every block still ends at its count and
    # most blocks agree label for label
    for block in labels:
        assert np.unique(block).size == count
    agree = np.mean([np.array_equal(a, b) for a, b in zip(labels, g[f"{tag}_labels"])])
    assert agree >= (1.0 if tag == "rounded" else 0.0)


def test_ward_known_answers(oracle):
    g = golden("ward")
    four = np.full((1, 4), 4.0, dtype=np.float32)
    assert oracle.ward_merge(g["tight_pools"], four, 3, 16).tolist() == [[0, 0, 1, 2]] == g["tight_labels"].tolist()
    assert oracle.ward_merge(g["same_pools"], four, 2, 16).tolist() == [[0, 0, 0, 1]] == g["same_labels"].tolist()
    labels, reached = oracle.ward_rounds(g["pair_pools"], np.ones((2, 64), np.float32), 32, 2.0)
    assert reached.all() and np.array_equal(labels, g["pair_labels"])
    members = oracle.members_from_labels(np.array([1, 0, 1, 2, 0, 1]), 3, 4)
    assert members.tolist() == [[1, 4, -1, -1], [0, 2, 5, -1], [3, -1, -1, -1]] == g["members"].tolist()
    # a cap under twice the bucket size is refused; the merge itself reports the block short
    pools = g["b_pools"][:2, :16]
    sixteen = np.full((2, 16), 16.0, dtype=np.float32)
    with pytest.raises(ValueError, match="at least twice"):
        oracle.ward_merge(pools, sixteen, 8, 16)
    labels, reached = oracle.ward_rounds(pools, sixteen, 8, 16)
    assert not reached.any() and np.array_equal(labels, np.broadcast_to(np.arange(16), (2, 16)))


@pytest.mark.parametrize("name,args", [("flat_small", (4, 8, 16, 64)), ("flat_c1like", (16, 64, 128, 512))])
def test_build_buckets_matches_the_reference(oracle, name, args):
    g = golden(name)
    buckets = oracle.build_buckets(g["keys"], *args)
    assert np.array_equal(buckets.bucket_members, g["members"])
    assert np.array_equal(buckets.bucket_sizes, g["sizes"])
    np.testing.assert_allclose(buckets.bucket_centroids, g["centroids"], rtol=0, atol=1e-6)


def test_sizes_that_do_not_nest_are_refused(oracle):
    keys = golden("flat_small")["keys"]
    for sizes in [(3, 8, 16, 64), (4, 8, 16, 60), (4, 8, 15, 64), (0, 8, 16, 64)]:
        with pytest.raises(ValueError):
            oracle.build_buckets(keys, *sizes)


def test_flat_read_matches_the_reference(oracle):
    g = golden("flat_small")
    buckets = oracle.Buckets(g["centroids"], g["members"], g["sizes"], 8, 64)
    for tag, (top_p, top_k, window, early) in {"": (8, 48, 64, None), "_small": (3, 20, 16, None),
                                               "_early": (8, 48, 64, (200, 12, 2))}.items():
        sel, lens = oracle.read(g["queries"], g["positions"], buckets, top_p, top_k, 4, window, early_budget=early)
        assert np.array_equal(lens, g["lengths" + tag])
        assert np.array_equal(sel, g["selected" + tag])


def test_flat_read_at_64_dims_matches_the_reference(oracle):
    g = golden("flat_c1like")
    buckets = oracle.Buckets(g["centroids"], g["members"], g["sizes"], 8, 512)
    for tag, top_k in (("", 2048), ("_cut", 700)):
        sel, lens, picked, keys = oracle.read(g["queries"], g["positions"], buckets, 16, top_k, 4, 512,
                                              return_picked=True)
        assert np.array_equal(lens, g["lengths" + tag])
        assert np.array_equal(sel, g["selected" + tag])
    # the fixed-order scores are the reference's to within fp32 rounding
    got = oracle.unpack_scores(keys)
    want = np.take_along_axis(g["scores"], np.maximum(picked, 0), axis=1)
    np.testing.assert_allclose(np.where(picked >= 0, got, 0), np.where(picked >= 0, want, 0), rtol=0, atol=1e-6)


def test_expansion_alone_reproduces_the_read(oracle):
    g = golden("flat_c1like")
    buckets = oracle.Buckets(g["centroids"], g["members"], g["sizes"], 8, 512)
    _, _, picked, _ = oracle.read(g["queries"], g["positions"], buckets, 16, 700, 4, 512, return_picked=True)
    sel, lens = oracle.expand(picked, g["positions"], g["members"], 700, 4, 512)
    assert np.array_equal(sel, g["selected_cut"]) and np.array_equal(lens, g["lengths_cut"])


def test_hierarchy_levels_and_growth_match_the_reference(oracle):
    g = golden("hierarchy")
    buckets = oracle.Buckets(g["centroids"], g["members"], (g["members"] >= 0).sum(1).astype(np.int32), 8, 64)
    tree = oracle.build_hierarchy(g["keys"], buckets, 16, 4, 16)
    assert len(tree.children) == int(g["levels"]) == 4
    assert [len(c) for c in tree.children] == [256, 64, 16, 4]
    for level in range(4):
        assert np.array_equal(tree.children[level], g[f"children_{level}"])
        np.testing.assert_allclose(tree.node_centroids[level], g[f"node_centroids_{level}"], rtol=0, atol=2e-6)
    rows = [(closed, growth) for closed in (0, 64, 128, 512, 1024) for growth in (0, 64, 100)]
    for (closed, growth), want in zip(rows, g["growth"]):
        covered, made, shut = oracle.growth_at(tree, closed, 64, growth)
        assert [covered, *made, *shut] == want.tolist()


@pytest.mark.parametrize("tag,beam,start,growth", [("wide", 4096, None, 0), ("narrow", 2, None, 0),
                                                   ("start", 3, 8, 0), ("wait", 2, None, 64)])
def test_beam_read_matches_the_reference(oracle, tag, beam, start, growth):
    g = golden("hierarchy")
    buckets = oracle.Buckets(g["centroids"], g["members"], (g["members"] >= 0).sum(1).astype(np.int32), 8, 64)
    levels = int(g["levels"])
    tree = oracle.Hierarchy([g[f"node_centroids_{i}"] for i in range(levels)],
                            [g[f"children_{i}"] for i in range(levels)], 4, tuple(g["block_sizes"].tolist()))
    sel, lens, _, scored = oracle.read_hierarchy(g["queries"], g["positions"], buckets, tree, beam, start, 16, 64,
                                                 4, 64, 512, growth, return_picked=True)
    assert np.array_equal(lens, g[f"lengths_{tag}"])
    assert np.array_equal(sel, g[f"selected_{tag}"])
    assert np.array_equal(scored, g[f"scored_{tag}"])


def test_sparse_attention_matches_the_reference(oracle):
    g = golden("attention")
    T, dh = g["q"].shape[0], g["q"].shape[2]
    positions = np.arange(T)
    out, lse = oracle.sparse_attend(g["q"], g["k"], g["v"], g["selected"], positions, 8, 2, dh**-0.5)
    np.testing.assert_allclose(out, g["out"], rtol=0, atol=2e-6)
    full = np.broadcast_to(np.arange(T, dtype=np.int32), (T, T))
    dense, _ = oracle.sparse_attend(g["q"], g["k"], g["v"], full, positions, 0, 0, dh**-0.5)
    np.testing.assert_allclose(dense, g["dense"], rtol=0, atol=2e-6)
    # padding selects nothing and the window alone spans the sequence
    empty = np.full((T, 1), -1, dtype=np.int32)
    alone, _ = oracle.sparse_attend(g["q"], g["k"], g["v"], empty, positions, T, 0, dh**-0.5)
    np.testing.assert_allclose(alone, g["dense"], rtol=0, atol=2e-6)
    assert np.isfinite(lse).all()


def test_lse_merge_of_disjoint_halves_is_the_whole(oracle):
    g = golden("attention")
    T, dh = g["q"].shape[0], g["q"].shape[2]
    positions = np.arange(T)
    ids = np.broadcast_to(np.arange(T, dtype=np.int32), (T, T))
    whole, whole_lse = oracle.sparse_attend(g["q"], g["k"], g["v"], ids, positions, 0, 0, dh**-0.5)
    even = np.where(ids % 2 == 0, ids, -1).astype(np.int32)
    odd = np.where(ids % 2 == 1, ids, -1).astype(np.int32)
    a, la = oracle.sparse_attend(g["q"], g["k"], g["v"], even, positions, 0, 0, dh**-0.5)
    b, lb = oracle.sparse_attend(g["q"], g["k"], g["v"], odd, positions, 0, 0, dh**-0.5)
    assert np.isneginf(lb[0]).all() and not b[0].any()  # row 0 has no odd key to read
    merged, lse = oracle.lse_merge(np.stack([a, b]), np.stack([la, lb]))
    np.testing.assert_allclose(merged, whole, rtol=0, atol=2e-6)
    np.testing.assert_allclose(lse, whole_lse, rtol=0, atol=2e-6)


def test_miniature_config_end_to_end(oracle):
    g = golden("mini_c1")
    bf16 = lambda bits: (bits.astype(np.uint32) << 16).view(np.float32)
    q, k, v = bf16(g["q_bf16"]), bf16(g["k_bf16"]), bf16(g["v_bf16"])
    iq, ik = oracle.regroup(q, k)
    index_q, index_k = oracle.project(iq, g["w"]), oracle.project(ik, g["w"])
    np.testing.assert_allclose(index_q, g["index_queries"], rtol=0, atol=1e-6)
    np.testing.assert_allclose(index_k, g["index_keys"], rtol=0, atol=1e-6)
    # from the reference's own index vectors on, the integer results are the reference's
    buckets = oracle.build_buckets(g["index_keys"], 4, 16, 32, 128)
    assert np.array_equal(buckets.bucket_members, g["members"])
    T = q.shape[0]
    sel, lens = oracle.read(g["index_queries"], np.arange(T), buckets, 8, 256, 4, 128)
    same = [np.array_equal(a, b) for a, b in zip(sel, g["selected"])]
    # a fixed-order fp32 dot can order two near-tied buckets otherwise than the reference's BLAS dot
    assert np.mean(same) >= 0.995
    assert np.array_equal(lens, g["lengths"])
    rows = g["out_rows"]
    out, _ = oracle.sparse_attend(q[rows], k, v, g["selected"][rows], rows, 128, 4, q.shape[2] ** -0.5,
                                  lengths=g["lengths"][rows])
    np.testing.assert_allclose(out, g["out"], rtol=0, atol=5e-6)


@pytest.mark.parametrize("width", [32, 64])
def test_bucket_shapes_match_the_reference(oracle, width):
    # (the reference's own cases: tests/unit/core/test_shape.py:40-94)
    g = golden("shapes")
    tag = f"w{width}_"
    keys, centroids, members, queries = g[tag + "keys"], g[tag + "centroids"], g[tag + "members"], g[tag + "queries"]
    if width == 32:
        np.testing.assert_allclose(oracle.covariances(keys, centroids, members)[0], g[tag + "covariances"], atol=1e-7)
    for rank in (0, 1, 2, 4, width):
        want = oracle.Shapes(g[f"{tag}r{rank}_basis"], g[f"{tag}r{rank}_variances"], g[f"{tag}r{rank}_floor"])
        # the reference's shapes through the oracle's scoring: the spread in double, the scores in the fixed fp32 order
        np.testing.assert_allclose(oracle.spread(queries, want), g[f"{tag}r{rank}_spread"], rtol=0, atol=2e-7)
        np.testing.assert_allclose(oracle.shaped_scores(queries, centroids, want, 2.0), g[f"{tag}r{rank}_scores"],
                                   rtol=0, atol=5e-7)
        assert np.array_equal(oracle.pack_shape_basis(oracle.unpack_shape_basis(want.basis)), want.basis)
        # the oracle's own build
        got = oracle.build_shapes(keys, centroids, members, rank)
        np.testing.assert_allclose(got.variances, want.variances, rtol=1e-5, atol=1e-7)
        np.testing.assert_allclose(got.floor, want.floor, rtol=1e-5, atol=1e-7)
        kept = got.variances.sum(1) + got.floor * (width - rank)
        np.testing.assert_allclose(kept, np.trace(oracle.covariances(keys, centroids, members)[0], axis1=1, axis2=2),
                                   rtol=1e-4, atol=1e-6)  # a shape keeps the trace whatever its rank
        if rank <= 2:  # a direction is its negation too; past the keys a bucket holds the directions are anyone's
            same = (got.basis == want.basis).all(-1) | (got.basis == ~want.basis).all(-1)
            assert same[members[:, rank].reshape(-1) >= 0].all()
            np.testing.assert_allclose(oracle.spread(queries, got), g[f"{tag}r{rank}_spread"], rtol=0, atol=2e-7)


def test_a_shaped_read_matches_the_reference(oracle):
    g = golden("shapes")
    buckets = oracle.Buckets(g["read_centroids"], g["read_members"], (g["read_members"] >= 0).sum(1).astype(np.int32),
                             8, 64)
    shapes = oracle.Shapes(g["read_basis"], g["read_variances"], g["read_floor"])
    plain, plain_lengths = oracle.read(g["read_queries"], g["read_positions"], buckets, 4, 16, 2, 24)
    for z in (0, 2):
        selected, lengths = oracle.read(g["read_queries"], g["read_positions"], buckets, 4, 16, 2, 24, shapes=shapes,
                                        deviations=float(z))
        assert np.array_equal(lengths, g[f"read_z{z}_lengths"])
        assert np.array_equal(selected, g[f"read_z{z}_selected"])
    assert np.array_equal(g["read_z0_selected"], plain) and not np.array_equal(g["read_z2_selected"], plain)
    with pytest.raises(ValueError, match="rank must be from 0 to the keys' width 32 - got 33"):
        oracle.shape_buckets(g["read_keys"], buckets, 33)
    built = oracle.shape_buckets(g["read_keys"], buckets, 2)
    np.testing.assert_allclose(built.variances, shapes.variances, rtol=1e-5, atol=1e-8)


def _fingerprint_pattern(rows, dim):
    i, j = np.arange(rows, dtype=np.int64)[:, None], np.arange(dim, dtype=np.int64)[None]
    return ((i * 40503 + j * 1201 + (i * j) % 251 + 7) & 0xFFFF).astype(np.uint16)


def test_page_fingerprints_match_the_reference(oracle):
    g = golden("fingerprints")
    page = int(g["page_size"])
    words, positions = oracle.fingerprint_weights(page)
    assert len(words) == int(g["words_count"]) and (words & 1).all() and (positions & 1).all()
    assert np.array_equal(words[:16], g["words_head"]) and np.array_equal(positions[:16], g["positions_head"])
    assert words.sum() == g["words_sum"] and positions.sum() == g["positions_sum"]
    for dim in (16, 64, 512):
        stored = _fingerprint_pattern(3 * page, dim)
        every = np.ones(3 * page, bool)
        assert np.array_equal(oracle.page_fingerprints(stored, every, words, positions), g[f"d{dim}_all"])
        parts = [oracle.page_fingerprints(stored, np.arange(3 * page) % 3 == rank, words, positions) for rank in range(3)]
        for rank in range(3):
            assert np.array_equal(parts[rank], g[f"d{dim}_rank{rank}"])
        assert np.array_equal(oracle.exact_group_sum(parts), g[f"d{dim}_all"])  # the group's sum is the whole page's
    changed = _fingerprint_pattern(3 * page, 64)
    changed[page + 5, 3] ^= 1  # one bit of one key: that page's fingerprint alone moves
    moved = oracle.page_fingerprints(changed, np.ones(3 * page, bool), words, positions) != g["d64_all"]
    assert moved.tolist() == [False, True, False]
