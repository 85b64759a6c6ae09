"""The tree on the GPU: node bucket levels and the beam read against the reference's golden vectors and the oracle."""

import numpy as np
import pytest
import torch

from conftest import golden
from helpers import cuda, mixture, unit_rows

pytestmark = pytest.mark.gpu


def _golden_store():
    from lsa_b200 import core

    g = golden("hierarchy")
    sizes = (g["members"] >= 0).sum(1).astype(np.int32)
    buckets = core.Buckets(cuda(g["centroids"]), cuda(g["members"]), cuda(sizes), 8, 64)
    return g, buckets


def test_levels_match_the_reference():
    from lsa_b200 import core

    g, buckets = _golden_store()
    tree = core.build_hierarchy(cuda(g["keys"]), buckets, 16, 4, 16)
    assert [len(c) for c in tree.children] == [256, 64, 16, 4]
    for level in range(4):
        assert np.array_equal(tree.children[level].cpu().numpy(), g[f"children_{level}"])
        np.testing.assert_allclose(tree.node_centroids[level].cpu().numpy(), g[f"node_centroids_{level}"], rtol=0,
                                   atol=2e-6)
    rows = [(closed, growth) for closed in (0, 64, 128, 512, 1024) for growth in (0, 64, 100)]
    for (closed, growth), want in zip(rows, g["growth"]):
        grown = core.growth_at(tree, closed, 64, growth)
        assert [grown.covered_buckets, *grown.made, *grown.closed] == want.tolist()
    with pytest.raises(ValueError, match="power of two"):
        core.build_hierarchy(cuda(g["keys"]), buckets, 2, 3, 12)
    with pytest.raises(ValueError, match="multiple"):
        core.build_hierarchy(cuda(g["keys"]), buckets, 2, 4, 18)


@pytest.mark.parametrize("tag,beam,start,growth", [("wide", 4096, None, 0), ("narrow", 2, None, 0),
                                                   ("start", 3, 8, 0), ("wait", 2, None, 64)])
def test_beam_read_matches_the_reference(tag, beam, start, growth):
    from lsa_b200 import core

    g, buckets = _golden_store()
    levels = int(g["levels"])
    tree = core.Hierarchy([cuda(g[f"node_centroids_{i}"]) for i in range(levels)],
                          [cuda(g[f"children_{i}"]) for i in range(levels)], [], None, 4,
                          tuple(g["block_sizes"].tolist()))
    sel, lens, scored = core.read_hierarchy_counted(cuda(g["queries"]), cuda(g["positions"]), buckets, tree, beam,
                                                    start, 16, 64, 4, 64, 512, growth)
    assert np.array_equal(lens.cpu().numpy(), g[f"lengths_{tag}"])
    assert np.array_equal(sel.cpu().numpy(), g[f"selected_{tag}"])
    assert np.array_equal(scored.cpu().numpy(), g[f"scored_{tag}"])
    with pytest.raises(ValueError, match="multiple of cluster_block_size"):
        core.read_hierarchy(cuda(g["queries"]), cuda(g["positions"]), buckets, tree, beam, start, 16, 64, 4, 64, 500,
                            growth)


def test_a_tree_over_large_node_blocks_is_bit_exact_with_the_oracle(oracle):
    """Node cluster blocks of 1,024 buckets (the multi-launch pairing), two levels, then a narrow beam."""
    from lsa_b200 import core

    T, d = 32768 + 300, 64
    raw = mixture(T, d, 48, 0.35, 17)
    keys = unit_rows(raw)
    want_buckets = oracle.build_buckets(keys, 4, 16, 32, 512)
    buckets = core.Buckets(cuda(want_buckets.bucket_centroids), cuda(want_buckets.bucket_members),
                           cuda(want_buckets.bucket_sizes), 32, 512)
    want = oracle.build_hierarchy(keys, want_buckets, 2, 8, (1024, 64))
    tree = core.build_hierarchy(cuda(keys), buckets, 2, 8, (1024, 64))
    assert [len(c) for c in tree.children] == [256, 32] == [len(c) for c in want.children]
    for level in range(2):
        assert np.array_equal(tree.children[level].cpu().numpy(), want.children[level])
        np.testing.assert_allclose(tree.node_centroids[level].cpu().numpy(), want.node_centroids[level], rtol=0,
                                   atol=1e-6)
    rng = np.random.default_rng(3)
    positions = np.sort(rng.integers(0, T, 40))
    queries = unit_rows(raw[positions] + 0.4 * rng.standard_normal((40, d), dtype=np.float32))
    # the read continues from the device's own node centroids, so the picks must be the oracle's
    mine = oracle.Hierarchy([c.cpu().numpy() for c in tree.node_centroids], [c.cpu().numpy() for c in tree.children],
                            8, (1024, 64))
    for beam, start, growth in ((4, None, 0), ((6, 2), 16, 1024)):
        want_sel, want_len, _, want_scored = oracle.read_hierarchy(queries, positions, want_buckets, mine, beam, start,
                                                                   24, 256, 4, 512, 8192, growth, return_picked=True)
        sel, lens, scored = core.read_hierarchy_counted(cuda(queries), cuda(positions), buckets, tree, beam, start, 24,
                                                        256, 4, 512, 8192, growth)
        assert np.array_equal(lens.cpu().numpy(), want_len) and np.array_equal(sel.cpu().numpy(), want_sel)
        assert np.array_equal(scored.cpu().numpy(), want_scored)


def test_a_beam_step_split_over_ctas_keeps_what_one_cta_keeps():
    from lsa_b200 import ops

    g, buckets = _golden_store()
    q = cuda(g["queries"])
    R = q.shape[0]
    nodes, kids = cuda(g["node_centroids_0"]), cuda(g["children_0"])
    zero = torch.zeros(R, dtype=torch.int32).cuda()
    end = torch.full((R,), nodes.shape[0], dtype=torch.int32).cuda()
    want_kept, want_keys = ops.beam_step(q, nodes, None, zero, end, 5)
    want_carried = ops.beam_step(q, nodes, None, zero, end, 5, children=kids)
    for splits in (2, 7, 16):
        kept, keys = ops.beam_step(q, nodes, None, zero, end, 5, splits=splits)
        assert torch.equal(kept, want_kept) and torch.equal(keys, want_keys)
        carried = ops.beam_step(q, nodes, None, zero, end, 5, children=kids, splits=splits)
        assert torch.equal(carried, want_carried)
        first = torch.full((R,), 900, dtype=torch.int32).cuda()
        last = torch.full((R,), 1024, dtype=torch.int32).cuda()
        a, _ = ops.beam_step(q, buckets.bucket_centroids, want_carried, first, last, 16)
        b, _ = ops.beam_step(q, buckets.bucket_centroids, want_carried, first, last, 16, splits=splits)
        assert torch.equal(a, b)


def test_a_tree_grown_a_page_end_at_a_time_is_the_tree_built_at_once_and_a_captured_step_follows_it(oracle):
    """Online growth in fixed-address arrays: after every page end the levels hold the first `made` node buckets of the
    tree built over the whole cache, `growth_at` counts them, reads through the growing tree select what reads through
    the built one select, and a decode step captured in a CUDA graph before the tree grew reads the grown tree."""
    from lsa_b200 import core, hierarchy
    from lsa_b200.decode import TreeDecoder
    from lsa_b200.layer import FlatDesign, FlatLayer

    T, d = 40960, 64
    raw = mixture(T, d, 48, 0.35, 23)
    keys = unit_rows(raw)
    want_buckets = oracle.build_buckets(keys, 4, 16, 32, 512)
    buckets = core.Buckets(cuda(want_buckets.bucket_centroids), cuda(want_buckets.bucket_members),
                           cuda(want_buckets.bucket_sizes), 32, 512)
    m, page_size, page_buckets, growth = T // 16, 4096, 256, 512
    blocks = (512, 32)
    built = core.build_hierarchy(cuda(keys), buckets, 2, 4, blocks)
    grown = hierarchy.GrowingHierarchy(d, 2, 4, blocks, growth, m)
    addresses = [t.data_ptr() for t in (*grown.node_centroids, *grown.children)]
    made_any = False
    for end in range(page_buckets, m + 1, page_buckets):
        new = grown.grow(end, cuda(keys), buckets)
        assert grown.counts() == hierarchy.growth_at(built, end, page_buckets, growth)
        made_any |= new > 0
        for level in range(2):
            n = grown.made[level]
            assert torch.equal(grown.children[level][:n], built.children[level][:n])
            assert torch.equal(grown.node_centroids[level][:n], built.node_centroids[level][:n])
            assert torch.equal(grown.node_means[level][:n], built.node_means[level][:n])
    assert made_any and grown.made[1] > 0 and grown.closed[0] > 0
    assert addresses == [t.data_ptr() for t in (*grown.node_centroids, *grown.children)]
    assert grown.counts_device.tolist() == [grown.covered, *grown.made, *grown.closed]
    assert torch.equal(grown.bucket_means[: grown.covered], built.bucket_means[: grown.covered])
    rng = np.random.default_rng(4)
    positions = np.sort(rng.integers(0, T, 48))
    queries = unit_rows(raw[positions] + 0.4 * rng.standard_normal((48, d), dtype=np.float32))
    for beam, start in ((4, None), ((6, 3), 16)):
        want = core.read_hierarchy_counted(cuda(queries), cuda(positions), buckets, built, beam, start, 24, 256, 4, 512,
                                           page_size, growth)
        got = core.read_hierarchy_counted(cuda(queries), cuda(positions), buckets, grown.view(), beam, start, 24, 256,
                                          4, 512, page_size, growth)
        assert all(torch.equal(a, b) for a, b in zip(got, want))

    # a step captured while the tree covers half the cache keeps reading as the tree grows and the position moves
    Hq, Hkv, dh = 4, 2, 64
    gen = torch.Generator().manual_seed(0)
    k = torch.randn(T, Hkv, dh, generator=gen).bfloat16().cuda()
    v = torch.randn(T, Hkv, dh, generator=gen).bfloat16().cuda()
    wq = (torch.randn(Hkv * dh, d, generator=gen) / 11).bfloat16().cuda()
    wk = (torch.randn(Hkv * dh, d, generator=gen) / 11).bfloat16().cuda()
    design = FlatDesign(pool_size=4, bucket_size=16, bucket_cap=32, cluster_block_size=512, top_p=24, top_k=256,
                        sink_size=4, window_size=512)
    layer = FlatLayer(design, wq, wk, Hq, Hkv, dh)
    half = hierarchy.GrowingHierarchy(d, 2, 4, blocks, growth, m)
    first_half = m // 2 // page_buckets * page_buckets
    for end in range(page_buckets, first_half + 1, page_buckets):
        half.grow(end, cuda(keys), buckets)
    decoder = TreeDecoder(layer, buckets, half.view(), 6, None, page_size, growth, splits=4, select_splits=2)
    q = torch.randn(1, Hq, dh, generator=gen).bfloat16().cuda()
    early, late = first_half * 16 + 700, T - 5
    decoder.prepare(early)
    decoder.step(q, k, v)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = decoder.step(q, k, v)
    graph.replay()
    at_early = out.clone()
    plain = TreeDecoder(layer, buckets, built, 6, None, page_size, growth, splits=4, select_splits=2)
    plain.prepare(early)
    assert torch.equal(at_early, plain.step(q, k, v))
    for end in range(first_half + page_buckets, m + 1, page_buckets):
        half.grow(end, cuda(keys), buckets)
    start_before = decoder.plan["start"]
    decoder.prepare(late)
    assert decoder.plan["start"] == start_before  # (the same levels: the captured step is still the step)
    graph.replay()
    plain.prepare(late)
    assert torch.equal(out, plain.step(q, k, v))
    assert not torch.equal(out, at_early)
