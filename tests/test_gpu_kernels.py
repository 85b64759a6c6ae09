"""Parity of every CUDA kernel with the CPU oracle, called through the C ABI (via the ctypes wrappers).

Integer results (labels, member tables, picked buckets, read lists) must be bit-exact. Floats: index vectors within
2e-6 (fp32 sums in another order), attention within max-abs 2e-2 / mean-abs 2e-3 of the fp32 oracle on bf16 inputs.
"""

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


# ------------------------------------------------------------------------------------------------ index map


@pytest.mark.parametrize("T,Hq,Hkv,dh,d_idx", [(300, 8, 2, 128, 32), (1000, 40, 8, 128, 64), (65, 4, 4, 64, 16)])
def test_index_map_matches_the_oracle(ops, oracle, T, Hq, Hkv, dh, d_idx):
    q, k, _ = layer_inputs(T, Hq, Hkv, dh, 8, 0)
    rng = np.random.default_rng(1)
    w = bf16_round(rng.standard_normal((Hkv * dh, d_idx), dtype=np.float32) / np.sqrt(Hkv * dh))
    want_q = oracle.project(oracle.regroup_queries(q, Hkv), w)
    want_k = oracle.project(k.reshape(T, -1), w)
    got_q, got_q16 = ops.index_map(cuda(q, torch.bfloat16), cuda(w, torch.bfloat16), group=Hq // Hkv, also_bf16=True)
    got_k = ops.index_map(cuda(k, torch.bfloat16), cuda(w), group=1)
    np.testing.assert_allclose(got_q.cpu().numpy(), want_q, rtol=0, atol=2e-6)
    np.testing.assert_allclose(got_k.cpu().numpy(), want_k, rtol=0, atol=2e-6)
    np.testing.assert_allclose(got_q16.float().cpu().numpy(), want_q, rtol=0, atol=4e-3)


@pytest.mark.parametrize("T,Hq,Hkv,dh,d_idx,off", [(1000, 40, 8, 128, 64, 0), (333, 8, 2, 128, 32, 0),
                                                     (4100, 16, 4, 64, 128, 16)])
def test_tensor_core_map_matches_the_oracle(ops, oracle, T, Hq, Hkv, dh, d_idx, off):
    q, k, _ = layer_inputs(T, Hq, Hkv, dh, 8, 5)
    rng = np.random.default_rng(2)
    used = dh - off
    w = bf16_round(rng.standard_normal((Hkv * used, d_idx), dtype=np.float32) / np.sqrt(Hkv * used))
    want_q = oracle.project(oracle.regroup_queries(q[:, :, off:], Hkv), w)
    want_k = oracle.project(np.ascontiguousarray(k[:, :, off:]).reshape(T, -1), w)
    W = cuda(w, torch.bfloat16)
    wq_t = ops.expand_map(W, Hq, Hq // Hkv, dh, off)
    wk_t = ops.expand_map(W, Hkv, 1, dh, off)
    assert wq_t.shape == (d_idx, Hq * dh) and wk_t.shape == (d_idx, Hkv * dh)
    status = torch.zeros(1, dtype=torch.int32).cuda()
    got_q = ops.index_map_tc(cuda(q, torch.bfloat16), wq_t, status=status)
    got_k = ops.index_map_tc(cuda(k, torch.bfloat16), wk_t, status=status)
    assert int(status) == 0
    np.testing.assert_allclose(got_q.cpu().numpy(), want_q, rtol=0, atol=3e-5)
    np.testing.assert_allclose(got_k.cpu().numpy(), want_k, rtol=0, atol=3e-5)
    # it agrees with the exact-order kernel to the same bound, and not normalising leaves the raw product
    exact = ops.index_map(cuda(q, torch.bfloat16), W, group=Hq // Hkv, dh_off=off)
    assert (exact - got_q).abs().max() <= 3e-5
    raw = ops.index_map_tc(cuda(k, torch.bfloat16), wk_t, normalize=False)
    want_raw = oracle.project(np.ascontiguousarray(k[:, :, off:]).reshape(T, -1), w, normalize=False)
    np.testing.assert_allclose(raw.cpu().numpy(), want_raw, rtol=1e-4, atol=1e-4)


def test_two_layer_map_matches_its_restatement(ops, oracle):
    """A variant with no reference code: the oracle restatement is the only pin."""
    from scipy.special import erf

    rng = np.random.default_rng(3)
    T, d_in, d_hidden, d_idx = 700, 128, 2048, 64
    x = bf16_round(rng.standard_normal((T, d_in), dtype=np.float32))
    w1 = bf16_round(rng.standard_normal((d_in, d_hidden), dtype=np.float32) / np.sqrt(d_in))
    w2 = bf16_round(rng.standard_normal((d_hidden, d_idx), dtype=np.float32) / np.sqrt(d_hidden))
    got = ops.mlp_map(cuda(x, torch.bfloat16), cuda(w1.T.copy(), torch.bfloat16), cuda(w2.T.copy(), torch.bfloat16))
    # the kernel keeps the hidden layer in bf16: restate with that rounding, then against the pure fp32 form
    pre = oracle.project(x, w1, normalize=False)
    hidden = bf16_round(0.5 * pre * (1.0 + erf(pre * np.float32(0.7071067811865476))))
    np.testing.assert_allclose(got.cpu().numpy(), oracle.project(hidden, w2), rtol=0, atol=2e-4)
    np.testing.assert_allclose(got.cpu().numpy(), oracle.project_mlp(x, w1, w2), rtol=0, atol=3e-3)


def test_index_map_identity_zero_rows_and_rotary_offsets(ops, oracle):
    g = golden("index_space")
    q, k = cuda(g["q"]), cuda(g["k"])
    iq = ops.index_map(q, None, group=4)
    ik = ops.index_map(k, None, group=1)
    np.testing.assert_allclose(iq.cpu().numpy(), g["index_queries"], rtol=0, atol=2e-6)
    np.testing.assert_allclose(ik.cpu().numpy(), g["index_keys"], rtol=0, atol=2e-6)
    assert not ik[7].any()
    proj = ops.index_map(ik[:, None, :], cuda(g["w"]))
    np.testing.assert_allclose(proj.cpu().numpy(), g["projected_keys"], rtol=0, atol=2e-6)
    # the rotary prefix dropped: dims 8.. of every head
    part = ops.index_map(k, None, group=1, dh_off=8, normalize=False)
    assert torch.equal(part, k[:, :, 8:].reshape(k.shape[0], -1))


# ------------------------------------------------------------------------------------------------ pooling, Ward, table


def test_pooling_is_bit_exact(ops, oracle):
    keys = unit_rows(mixture(4096, 64, 16, 0.3, 3))
    want = oracle.pool_keys(keys.reshape(8, 512, 64), 16)
    got = ops.pool_keys(cuda(keys).view(8, 512, 64), 16)
    assert np.array_equal(got.cpu().numpy().view(np.int32), want.view(np.int32))
    got16 = ops.pool_keys(cuda(keys, torch.bfloat16).view(8, 512, 64), 16)
    want16 = oracle.pool_keys(bf16_round(keys).reshape(8, 512, 64), 16)
    assert np.array_equal(got16.cpu().numpy().view(np.int32), want16.view(np.int32))


@pytest.mark.parametrize("G,P,d,pool,count,cap", [(6, 64, 64, 16, 32, 64), (3, 256, 64, 4, 64, 32),
                                                   (4, 80, 64, 64, 8, 1280), (5, 32, 16, 4, 16, 16),
                                                   (2, 64, 48, 4, 16, 24), (2, 512, 64, 2, 64, 32)])
def test_ward_labels_are_bit_exact(ops, oracle, G, P, d, pool, count, cap):
    keys = unit_rows(mixture(G * P * pool, d, 12, 0.3, P + d))
    pools = oracle.pool_keys(keys.reshape(G, P * pool, d), pool)
    sizes = np.full((G, P), float(pool), dtype=np.float32)
    want, want_reached, want_rounds = oracle.ward_rounds(pools, sizes, count, cap, return_rounds=True)
    got, reached, rounds = ops.ward_rounds(cuda(pools), float(pool), count, cap, return_rounds=True)
    assert np.array_equal(got.cpu().numpy(), want)
    assert np.array_equal(reached.cpu().numpy(), want_reached)
    assert np.array_equal(rounds.cpu().numpy(), want_rounds)
    got2, _ = ops.ward_rounds(cuda(pools), cuda(sizes), count, cap)
    assert torch.equal(got, got2)


@pytest.mark.parametrize("G,P,d,count,cap,sizes", [(3, 1024, 64, 512, 2.0, 1.0), (2, 2048, 16, 1024, 2.0, 1.0),
                                                     (2, 768, 64, 96, 64.0, 4.0), (1, 640, 32, 600, 2.0, 1.0)])
def test_large_block_ward_is_bit_exact(ops, oracle, G, P, d, count, cap, sizes):
    """Blocks past one CTA's shared memory: the multi-launch merge (the tree's pairings at a cap of two, and a
    general cap), against the oracle label for label and round for round."""
    keys = unit_rows(mixture(G * P, d, 40, 0.4, P + d)).reshape(G, P, d) * np.float32(3.0)
    size_rows = np.full((G, P), sizes, dtype=np.float32)
    want, want_reached, want_rounds = oracle.ward_rounds(keys, size_rows, count, cap, return_rounds=True)
    got, reached, rounds = ops.ward_rounds(cuda(keys), sizes, count, cap, return_rounds=True)
    assert np.array_equal(got.cpu().numpy(), want)
    assert np.array_equal(reached.cpu().numpy(), want_reached)
    assert np.array_equal(rounds.cpu().numpy(), want_rounds)


def test_ward_golden_and_adversarial_cases(ops, oracle):
    g = golden("ward")
    for tag in "abcde":
        pool, count, cap = g[f"{tag}_args"].tolist()
        labels, reached = ops.ward_rounds(cuda(g[f"{tag}_pools"]), float(pool), count, cap)
        assert reached.all() and np.array_equal(labels.cpu().numpy(), g[f"{tag}_labels"])
    four = torch.full((1, 4), 4.0).cuda()
    assert ops.ward_rounds(cuda(g["tight_pools"]), four, 3, 16)[0].tolist() == [[0, 0, 1, 2]]
    assert ops.ward_rounds(cuda(g["same_pools"]), four, 2, 16)[0].tolist() == [[0, 0, 0, 1]]
    labels, reached = ops.ward_rounds(cuda(g["pair_pools"]), 1.0, 32, 2)
    assert reached.all() and np.array_equal(labels.cpu().numpy(), g["pair_labels"])
    # near-copied and rounded pools (ties everywhere): bit-exact with the oracle, which runs the same order
    for tag in ("near", "rounded"):
        pools = g[f"{tag}_pools"]
        want, want_reached = oracle.ward_rounds(pools, np.full(pools.shape[:2], 4.0, np.float32), 64, 16)
        got, reached = ops.ward_rounds(cuda(pools), 4.0, 64, 16)
        assert np.array_equal(got.cpu().numpy(), want) and np.array_equal(reached.cpu().numpy(), want_reached)
    # a cap that leaves no pair: every pool stays alone and the block reports short
    sixteen = cuda(g["b_pools"][:2, :16])
    labels, reached = ops.ward_rounds(sixteen, 16.0, 8, 16)
    assert not reached.any() and torch.equal(labels.cpu(), torch.arange(16).expand(2, 16))


def test_linear_layers_over_a_few_rows(ops):
    """The decode-row maps: heads summed or read side by side, GELU or not, unit rows or not, against fp32 torch on
    the same bf16 values (the hidden layer of the two-layer map is rounded to bf16, as the batched map rounds it)."""
    gen = torch.Generator().manual_seed(3)
    for rows in (1, 3, 8):
        x = (0.5 * torch.randn(rows, 64, 576, generator=gen)).bfloat16().cuda()
        w1 = (torch.randn(2048, 576, generator=gen) / 24).bfloat16().cuda()
        w2 = (torch.randn(64, 2048, generator=gen) / 45).bfloat16().cuda()
        summed = x.float().sum(1).bfloat16().float()
        want_hidden = torch.nn.functional.gelu(summed @ w1.float().t())
        hidden = ops.rows_linear(x, w1, sum_heads=True, gelu=True, out_dtype=torch.bfloat16)
        assert (hidden.float() - want_hidden).abs().max() <= 2e-2 * want_hidden.abs().max()
        want = torch.nn.functional.normalize(hidden.float() @ w2.float().t(), dim=1)
        got = ops.rows_linear(hidden, w2, normalize=True)
        assert (got - want).abs().max() <= 1e-5
        # heads side by side under a widened map: [rows, 40, 128] against [64, 5120]
        q = torch.randn(rows, 40, 128, generator=gen).bfloat16().cuda()
        wide = (torch.randn(64, 5120, generator=gen) / 70).bfloat16().cuda()
        got = ops.rows_linear(q, wide, normalize=True)
        want = torch.nn.functional.normalize(q.float().reshape(rows, -1) @ wide.float().t(), dim=1)
        assert (got - want).abs().max() <= 1e-5
        plain = ops.rows_linear(q, wide)
        assert (plain - q.float().reshape(rows, -1) @ wide.float().t()).abs().max() <= 1e-4
    with pytest.raises(ValueError):
        ops.rows_linear(torch.zeros(9, 64, device="cuda", dtype=torch.bfloat16), wide)


def test_kmeans_bucketing_matches_its_restatement(ops, oracle):
    """A variant with no reference code: config 1's shapes - 1,024 pools, 256 centres, 32 dims, 10 rounds."""
    keys = unit_rows(mixture(16384, 32, 64, 0.3, 8))
    pools = oracle.pool_keys(keys[None], 16)[0]
    rng = np.random.default_rng(0)
    init = unit_rows(pools[rng.permutation(len(pools))[:256]])
    want_centroids, want_assign = oracle.kmeans(pools, init, 10)
    centroids, assign = ops.kmeans(cuda(pools), cuda(init), 10)
    assert np.array_equal(assign.cpu().numpy(), want_assign)
    assert np.array_equal(centroids.cpu().numpy().view(np.int32), want_centroids.view(np.int32))


def test_bucket_table_is_bit_exact(ops, oracle):
    for name, (pool, bucket, cap, block) in {"flat_small": (4, 8, 16, 64), "flat_c1like": (16, 64, 128, 512)}.items():
        g = golden(name)
        want = oracle.build_buckets(g["keys"], pool, bucket, cap, block)
        G = g["keys"].shape[0] // block
        pools = oracle.pool_keys(g["keys"][: G * block].reshape(G, block, -1), pool)
        labels, _ = oracle.ward_rounds(pools, np.full(pools.shape[:2], float(pool), np.float32), block // bucket, cap)
        members, sizes, sums, cent, cent16, status = ops.bucket_table(cuda(g["keys"]), cuda(labels), pool,
                                                                       block // bucket, cap, want_bf16=True)
        assert np.array_equal(members.cpu().numpy(), want.bucket_members) and np.array_equal(members.cpu().numpy(), g["members"])
        assert np.array_equal(sizes.cpu().numpy(), want.bucket_sizes)
        assert np.array_equal(cent.cpu().numpy().view(np.int32), want.bucket_centroids.view(np.int32))
        assert torch.equal(cent16, cent.bfloat16()) and int(status) == 0
    from lsa_b200 import core
    members = core.members_from_labels(torch.tensor([1, 0, 1, 2, 0, 1]).cuda(), 3, 4)
    assert members.tolist() == [[1, 4, -1, -1], [0, 2, 5, -1], [3, -1, -1, -1]]


# ------------------------------------------------------------------------------------------------ selection


def _flat_case(T, d, pool, bucket, cap, block, seed, centres=24):
    raw = mixture(T, d, centres, 0.3, seed)
    keys = unit_rows(raw)
    rng = np.random.default_rng(seed + 1)
    return raw, keys, rng


@pytest.mark.parametrize("T,R,top_p,top_k,window,sink", [(4196, 300, 16, 2048, 512, 4), (40000, 257, 64, 700, 1024, 4),
                                                          (9000, 64, 200, 4096, 512, 0)])
def test_flat_read_is_bit_exact(ops, oracle, T, R, top_p, top_k, window, sink):
    raw, keys, rng = _flat_case(T, 64, 16, 64, 128, 512, T)
    buckets = oracle.build_buckets(keys, 16, 64, 128, 512)
    positions = np.sort(rng.integers(0, T, R))
    positions[:4] = [0, 1, 511, 512]
    queries = unit_rows(raw[positions] + 0.5 * rng.standard_normal((R, 64), dtype=np.float32))
    want_sel, want_len, want_picked, want_keys = oracle.read(queries, positions, buckets, top_p, top_k, sink, window,
                                                             return_picked=True)
    m = buckets.bucket_centroids.shape[0]
    visible = np.minimum(positions // 512 * 8, m).astype(np.int32)
    keys_out, picked = ops.flat_select(cuda(queries), cuda(buckets.bucket_centroids), cuda(visible), top_p)
    assert np.array_equal(keys_out.cpu().numpy(), want_keys)
    assert np.array_equal(picked.cpu().numpy(), want_picked)
    sel, lens, status = ops.expand(picked, cuda(positions), cuda(buckets.bucket_members), top_k, sink, window)
    assert np.array_equal(lens.cpu().numpy(), want_len) and np.array_equal(sel.cpu().numpy(), want_sel)
    assert int(status) == 0


def test_flat_read_golden_and_early_budget(oracle):
    from lsa_b200 import core
    from lsa_b200.budget import EarlyBudget
    g = golden("flat_small")
    buckets = core.Buckets(cuda(g["centroids"]), cuda(g["members"]), cuda(g["sizes"]), 8, 64)
    q, pos = cuda(g["queries"]), cuda(g["positions"])
    for tag, (top_p, top_k, window, early) in {"": (8, 48, 64, None), "_small": (3, 20, 16, None),
                                               "_early": (8, 48, 64, EarlyBudget(200, 12, 2))}.items():
        sel, lens = core.read(q, pos, buckets, top_p, top_k, 4, window, early_budget=early)
        assert np.array_equal(sel.cpu().numpy(), g["selected" + tag])
        assert np.array_equal(lens.cpu().numpy(), g["lengths" + tag])
    g = golden("flat_c1like")
    built = core.build_buckets(cuda(g["keys"]), 16, 64, 128, 512)
    assert np.array_equal(built.bucket_members.cpu().numpy(), g["members"])
    sel, lens = core.read(cuda(g["queries"]), cuda(g["positions"]), built, 16, 700, 4, 512)
    assert np.array_equal(sel.cpu().numpy(), g["selected_cut"]) and np.array_equal(lens.cpu().numpy(), g["lengths_cut"])


def test_selection_with_ties_rows_of_every_length_and_query_norms(ops, oracle):
    # thousands of identical centroids tie: the lower bucket wins, run to run the same
    rng = np.random.default_rng(5)
    base = unit_rows(rng.standard_normal((1, 64), dtype=np.float32))
    cents = np.repeat(base, 5000, axis=0)
    cents[::7] = unit_rows(rng.standard_normal((len(cents[::7]), 64), dtype=np.float32))
    queries = unit_rows(base + 0.01 * rng.standard_normal((40, 64), dtype=np.float32))
    queries[1] *= 0.01
    queries[2] *= 500.0
    visible = np.array([0, 1, 300, 1023, 2048, 2049, 4999, 5000] * 5, dtype=np.int32)
    want = np.full((40, 64), oracle.EMPTY_KEY, dtype=np.int64)
    for r in range(40):
        n = int(visible[r])
        keys = oracle.pack_keys(_dots(oracle, queries[r], cents[:n]), np.arange(n, dtype=np.int32))
        top = np.sort(keys)[::-1][:64]
        want[r, : len(top)] = top
    got, picked = ops.flat_select(cuda(queries), cuda(cents), cuda(visible), 64)
    again, _ = ops.flat_select(cuda(queries), cuda(cents), cuda(visible), 64)
    assert np.array_equal(got.cpu().numpy(), want) and torch.equal(got, again)
    assert np.array_equal(picked.cpu().numpy(), oracle.unpack_ids(want))


def _dots(oracle, query, rows):
    return oracle.scores(query, rows) if len(rows) else np.zeros(0, dtype=np.float32)


def test_decode_scan_and_candidate_merge(ops, oracle):
    rng = np.random.default_rng(9)
    lengths = [700, 2048, 5000, 64, 0, 33000]
    first = np.concatenate([[0], np.cumsum(lengths)[:-1]]).astype(np.int64)
    cents = unit_rows(rng.standard_normal((sum(lengths), 64), dtype=np.float32))
    queries = unit_rows(rng.standard_normal((len(lengths), 64), dtype=np.float32))
    want = np.full((len(lengths), 32), oracle.EMPTY_KEY, dtype=np.int64)
    for r, n in enumerate(lengths):
        keys = oracle.pack_keys(_dots(oracle, queries[r], cents[first[r]: first[r] + n]), np.arange(n, dtype=np.int32))
        top = np.sort(keys)[::-1][:32]
        want[r, : len(top)] = top
    for splits in (1, 4, 37):
        got, picked = ops.flat_select_decode(cuda(queries), cuda(cents), cuda(first), cuda(np.array(lengths, np.int32)),
                                             32, splits)
        assert np.array_equal(got.cpu().numpy(), want), splits
        assert np.array_equal(picked.cpu().numpy(), oracle.unpack_ids(want))
    # merging lists that several owners of disjoint bucket ranges produced gives the global list
    parts = []
    for lo, hi in ((0, 11000), (11000, 22000), (22000, 33000)):
        k = oracle.pack_keys(_dots(oracle, queries[5], cents[first[5] + lo: first[5] + hi]), np.arange(lo, hi, dtype=np.int32))
        parts.append(np.sort(k)[::-1][:32])
    merged, ids = ops.merge_candidates(cuda(np.stack(parts)[:, None, :]))
    assert np.array_equal(merged.cpu().numpy()[0], want[5])


def test_beam_step_matches_the_oracle_tree_read(ops, oracle):
    g = golden("hierarchy")
    q = cuda(g["queries"])
    R = q.shape[0]
    nodes, kids = cuda(g["node_centroids_0"]), cuda(g["children_0"])
    # level 1 scored whole, the best 3 kept and their children carried to the buckets
    zero = torch.zeros(R, dtype=torch.int32).cuda()
    end = torch.full((R,), nodes.shape[0], dtype=torch.int32).cuda()
    kept, keys = ops.beam_step(q, nodes, None, zero, end, 3)
    carried = ops.beam_step(q, nodes, None, zero, end, 3, children=kids)
    scores = g["queries"] @ g["node_centroids_0"].T
    for r in range(R):
        order = np.argsort(-scores[r], kind="stable")[:3]
        assert set(kept[r].tolist()) == set(order.tolist())
        assert carried[r].tolist() == g["children_0"][kept[r].cpu().numpy()].reshape(-1).tolist()
    # level 0: carried children beside a run of uncovered buckets, top 16
    first = torch.full((R,), 1000, dtype=torch.int32).cuda()
    last = torch.full((R,), 1024, dtype=torch.int32).cuda()
    picked, _ = ops.beam_step(q, cuda(g["centroids"]), carried, first, last, 16)
    for r in range(R):
        cand = np.concatenate([carried[r].cpu().numpy(), np.arange(1000, 1024)])
        keys = oracle.pack_keys(_dots(oracle, g["queries"][r], g["centroids"])[cand], cand.astype(np.int32))
        want = oracle.unpack_ids(np.sort(keys)[::-1][:16])
        assert picked[r].tolist() == want.tolist()


# ------------------------------------------------------------------------------------------------ expansion


def test_expansion_with_slots_owners_and_bad_ids(ops, oracle):
    g = golden("flat_c1like")
    buckets = oracle.Buckets(g["centroids"], g["members"], g["sizes"], 8, 512)
    _, _, picked, _ = oracle.read(g["queries"], g["positions"], buckets, 16, 700, 4, 512, return_picked=True)
    pos, mem = cuda(g["positions"]), cuda(g["members"])
    want_sel, want_len = oracle.expand(picked, g["positions"], g["members"], 700, 4, 512)
    # KV slots through a permuted page table
    rng = np.random.default_rng(2)
    pages = rng.permutation(70).astype(np.int32)
    sel, lens, _ = ops.expand(cuda(picked), pos, mem, 700, 4, 512, page_table=cuda(pages), page_size=64)
    mapped = np.where(want_sel >= 0, pages[np.maximum(want_sel, 0) // 64] * 64 + np.maximum(want_sel, 0) % 64, -1)
    assert np.array_equal(sel.cpu().numpy(), mapped) and np.array_equal(lens.cpu().numpy(), want_len)
    # two owners of halves of the sequence hold the whole list between them, each id once
    lo, _, _ = ops.expand(cuda(picked), pos, mem, 700, 4, 512, owner=(0, 2048))
    hi, _, _ = ops.expand(cuda(picked), pos, mem, 700, 4, 512, owner=(2048, 1 << 40))
    for a, b, w in zip(lo.cpu().numpy(), hi.cpu().numpy(), want_sel):
        assert sorted(a[a >= 0].tolist() + b[b >= 0].tolist()) == sorted(w[w >= 0].tolist())
        assert (a[a >= 0] < 2048).all() and (b[b >= 0] >= 2048).all()
    # four ranks that hold the cache dealt out in granules of 64 positions: each writes rows of its own share
    seen = [[] for _ in want_sel]
    for rank in range(4):
        part, lens_r, _ = ops.expand(cuda(picked), pos, mem, 700, 4, 512, dealt=(64, 4, rank))
        for r, row in enumerate(part.cpu().numpy()):
            local = row[row >= 0]
            assert len(local) == int(lens_r[r])
            seen[r] += (local // 64 * 256 + rank * 64 + local % 64).tolist()
    for got, w in zip(seen, want_sel):
        assert sorted(got) == sorted(w[w >= 0].tolist())
    # a pick past the table is counted in the status word and skipped
    bad = picked.copy()
    bad[0, 0] = 10**6
    _, _, status = ops.expand(cuda(bad), pos, mem, 700, 4, 512)
    assert int(status) == 1


def test_expansion_of_decode_rows_by_a_cluster(ops, oracle):
    """Eight rows or fewer whose picks hold tens of thousands of ids (a decode step over a long context) go through
    the kernel that gives a row a cluster of CTAs; its lists are the oracle's, id for id: full picks, picks that are
    fewer than the cluster's CTAs, a cut at top_k inside a bucket, holes in the picks, per-row budgets, a page
    table, the window and sinks left out."""
    rng = np.random.default_rng(4)
    cap, buckets_n, T = 1024, 300, 300 * 1024 + 5000
    members = np.full((buckets_n, cap), -1, dtype=np.int32)
    for b in range(buckets_n):  # pools of 64 consecutive positions, 6 to 16 a bucket, ascending
        pools = np.sort(rng.choice(np.arange(b * 16, b * 16 + 16), int(rng.integers(6, 17)), replace=False))
        ids = (pools[:, None] * 64 + np.arange(64)[None]).reshape(-1)
        members[b, : len(ids)] = ids
    positions = np.array([T - 1, T - 700, 200000, 70, 5000], dtype=np.int64)
    for top_p, top_k in ((40, 40 * cap), (40, 9000), (5, 5 * cap + 30000)):
        picked = np.stack([rng.choice(buckets_n, top_p, replace=False) for _ in positions]).astype(np.int32)
        picked[1, 3] = -1
        picked[2, :] = np.sort(picked[2])
        if top_p > 8:
            picked[3, 0] = 0  # the bucket of the sinks, for a row whose window starts at 0
        want_sel, want_len = oracle.expand(picked, positions, members, top_k, 4, 2048)
        sel, lens, _ = ops.expand(cuda(picked), cuda(positions), cuda(members), top_k, 4, 2048)
        assert np.array_equal(lens.cpu().numpy(), want_len), (top_p, top_k)
        assert np.array_equal(sel.cpu().numpy(), want_sel), (top_p, top_k)
    row_p = np.array([40, 7, 40, 1, 12], dtype=np.int32)
    row_k = np.array([40 * cap, 3000, 100, 40 * cap, 5000], dtype=np.int32)
    pages = rng.permutation(T // 64 + 1).astype(np.int32)
    sel, lens, _ = ops.expand(cuda(picked), cuda(positions), cuda(members), 40 * cap, 4, 2048, cuda(row_p), cuda(row_k),
                              page_table=cuda(pages), page_size=64, local=False)
    one, one_len, _ = ops.expand(cuda(picked), cuda(positions), cuda(members), 40 * cap, 4, 2048, cuda(row_p),
                                 cuda(row_k), page_table=cuda(pages), page_size=64, local=False, owner=(0, 1 << 40))
    assert torch.equal(lens, one_len)  # (an owner range takes the one-warp kernel)
    for r in range(len(positions)):
        assert torch.equal(sel[r, : int(lens[r])], one[r, : int(lens[r])])


def test_expansion_of_a_few_rows_with_long_lists(ops, oracle):
    """Up to 64 rows whose picks hold over a thousand ids go through the CTA-a-row kernel; its lists are the
    one-warp kernel's and the oracle's, id for id - cut at top_k, under per-row budgets, through a page table."""
    g = golden("flat_c1like")
    buckets = oracle.Buckets(g["centroids"], g["members"], g["sizes"], 8, 512)
    rows = slice(40, 88)
    positions = g["positions"][rows]
    _, _, picked, _ = oracle.read(g["queries"][rows], positions, buckets, 16, 700, 4, 512, return_picked=True)
    pos, mem = cuda(positions), cuda(g["members"])
    for top_k in (700, 150, 4000):
        want_sel, want_len = oracle.expand(picked, positions, g["members"], top_k, 4, 512)
        sel, lens, _ = ops.expand(cuda(picked), pos, mem, top_k, 4, 512)
        assert np.array_equal(sel.cpu().numpy(), want_sel) and np.array_equal(lens.cpu().numpy(), want_len), top_k
    # the early budget of the first rows
    cut = int(positions[20])
    want_sel, want_len = oracle.expand(picked, positions, g["members"], 700, 4, 512, early_budget=(cut, 90, 5))
    early = positions < cut
    row_p = cuda(np.where(early, 5, 16).astype(np.int32))
    row_k = cuda(np.where(early, 90, 700).astype(np.int32))
    sel, lens, _ = ops.expand(cuda(picked), pos, mem, 700, 4, 512, row_p, row_k)
    assert np.array_equal(sel.cpu().numpy(), want_sel) and np.array_equal(lens.cpu().numpy(), want_len)
    # KV slots through a page table, the window and sinks left out, a pick past the table
    pages = np.random.default_rng(3).permutation(70).astype(np.int32)
    want_sel, want_len = oracle.expand(picked, positions, g["members"], 700, 4, 512)
    sel, lens, _ = ops.expand(cuda(picked), pos, mem, 700, 4, 512, page_table=cuda(pages), page_size=64)
    mapped = np.where(want_sel >= 0, pages[np.maximum(want_sel, 0) // 64] * 64 + np.maximum(want_sel, 0) % 64, -1)
    assert np.array_equal(sel.cpu().numpy(), mapped) and np.array_equal(lens.cpu().numpy(), want_len)
    bare, bare_len, _ = ops.expand(cuda(picked), pos, mem, 700, 4, 512, local=False)
    for r in range(len(positions)):
        n = int(bare_len[r])
        assert np.array_equal(bare[r, :n].cpu().numpy(), want_sel[r, :n]) and (bare[r, n:] == -1).all()
        assert n == int(want_len[r]) - min(512, int(positions[r]) + 1) - min(4, max(0, int(positions[r]) + 1 - 512))
    bad = picked.copy()
    bad[3, 1] = 10**6
    sel, _, status = ops.expand(cuda(bad), pos, mem, 700, 4, 512)
    assert int(status) == 1
    keep = np.delete(bad[3], 1)[None]
    want_row, _ = oracle.expand(np.concatenate([keep, np.full((1, 1), -1, np.int32)], 1), positions[3:4],
                                g["members"], 700, 4, 512)
    assert np.array_equal(sel[3].cpu().numpy(), want_row[0])


# ------------------------------------------------------------------------------------------------ attention


def _attend_case(T, Hq, Hkv, dh, R, L, seed):
    q, k, v = layer_inputs(T, Hq, Hkv, dh, 16, seed)
    rng = np.random.default_rng(seed)
    rows = np.sort(rng.choice(T, R, replace=False))
    ids = np.full((R, L), -1, dtype=np.int32)
    lens = np.zeros(R, dtype=np.int32)
    for i, pos in enumerate(rows):
        n = min(L, pos + 1, int(rng.integers(0, L + 1)))
        ids[i, :n] = rng.choice(pos + 1, n, replace=False)
        lens[i] = n
    return q, k, v, rows, ids, lens


@pytest.mark.parametrize("T,Hq,Hkv,dh,R,L,splits", [(3000, 40, 8, 128, 24, 700, 1), (3000, 8, 2, 128, 40, 333, 1),
                                                    (2000, 16, 1, 64, 16, 500, 1), (5000, 40, 8, 128, 6, 3000, 5),
                                                    (1500, 4, 4, 64, 10, 100, 3)])
def test_sparse_attention_within_bf16_tolerance(ops, oracle, T, Hq, Hkv, dh, R, L, splits):
    q, k, v, rows, ids, lens = _attend_case(T, Hq, Hkv, dh, R, L, T + L)
    lens[0] = 0  # a row that reads nothing
    scale = dh ** -0.5
    want, want_lse = oracle.sparse_attend(q[rows], k, v, ids, rows, 0, 0, scale, lengths=lens)
    out, lse = ops.sparse_attend(cuda(q[rows], torch.bfloat16), cuda(k, torch.bfloat16), cuda(v, torch.bfloat16),
                                 cuda(ids), cuda(lens), scale, splits=splits, out_dtype=torch.float32)
    err = np.abs(out.cpu().numpy() - want)
    assert err.max() <= 2e-2 and err.mean() <= 2e-3, (err.max(), err.mean())
    got_lse = lse.cpu().numpy()
    assert np.isneginf(got_lse[0]).all() and not out[0].any()
    np.testing.assert_allclose(got_lse[1:], want_lse[1:], rtol=0, atol=2e-3)
    out16, _ = ops.sparse_attend(cuda(q[rows], torch.bfloat16), cuda(k, torch.bfloat16), cuda(v, torch.bfloat16),
                                 cuda(ids), cuda(lens), scale, splits=splits)
    assert np.abs(out16.float().cpu().numpy() - want).max() <= 2e-2


@pytest.mark.parametrize("T,Hq,Hkv,dh,window,sink,first,R", [(3000, 40, 8, 128, 1024, 4, 1500, 700),
                                                             (700, 8, 2, 128, 512, 4, 0, 700),
                                                             (2000, 16, 1, 64, 300, 0, 90, 333),
                                                             (2500, 8, 8, 64, 64, 7, 1000, 61)])
def test_band_attention_and_its_hand_over_to_the_gather(ops, oracle, T, Hq, Hkv, dh, window, sink, first, R):
    q, k, v = layer_inputs(T, Hq, Hkv, dh, 16, T + window)
    rows = np.arange(first, first + R)
    scale = dh ** -0.5
    empty = np.full((R, 1), -1, dtype=np.int32)
    want, want_lse = oracle.sparse_attend(q[rows], k, v, empty, rows, window, sink, scale)
    Q, K, V = cuda(q[rows], torch.bfloat16), cuda(k, torch.bfloat16), cuda(v, torch.bfloat16)
    # both forms: tensor memory (dense heads of 128 dims, 128 rows or more) and warp-level tiles
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for warp_mma in (True, False):
        out, lse = ops.band_attend(Q, K, V, first, window, sink, scale, warp_mma=warp_mma, status=status)
        err = np.abs(out.cpu().numpy() - want)
        assert err.max() <= 2e-2 and err.mean() <= 2e-3, (warp_mma, err.max(), err.mean())
        np.testing.assert_allclose(lse.cpu().numpy(), want_lse, rtol=0, atol=2e-3)
    assert int(status) == 0
    # the gather continues from the band's partial result over keys outside the window and the sinks
    rng = np.random.default_rng(1)
    ids = np.full((R, 200), -1, dtype=np.int32)
    lens = np.zeros(R, dtype=np.int32)
    for i, pos in enumerate(rows):
        lo, hi = sink, max(sink, pos + 1 - window)
        n = min(200, hi - lo)
        if n > 0:
            ids[i, :n] = rng.choice(np.arange(lo, hi), n, replace=False)
        lens[i] = max(n, 0)
    whole, whole_lse = oracle.sparse_attend(q[rows], k, v, ids, rows, window, sink, scale, lengths=lens)
    for splits in (1, 3):
        got, got_lse = ops.sparse_attend(Q, K, V, cuda(ids), cuda(lens), scale, splits=splits, out_dtype=torch.float32,
                                         init=(out, lse))
        err = np.abs(got.cpu().numpy() - whole)
        assert err.max() <= 2e-2 and err.mean() <= 2e-3, (splits, err.max(), err.mean())
        np.testing.assert_allclose(got_lse.cpu().numpy(), whole_lse, rtol=0, atol=2e-3)


def test_attention_skips_bad_ids_and_merges_partials(ops, oracle):
    q, k, v, rows, ids, lens = _attend_case(2000, 8, 2, 128, 12, 400, 4)
    scale = 128 ** -0.5
    want, want_lse = oracle.sparse_attend(q[rows], k, v, ids, rows, 0, 0, scale, lengths=lens)
    spoiled = ids.copy()
    spoiled = np.concatenate([spoiled, np.full((12, 8), 10**7, np.int32)], axis=1)
    for r in range(12):  # ids past the cache and negative ids inside the list are skipped
        spoiled[r, lens[r]: lens[r] + 4] = [-5, 10**7, -1, 2000]
    Q, K, V = cuda(q[rows], torch.bfloat16), cuda(k, torch.bfloat16), cuda(v, torch.bfloat16)
    out, lse = ops.sparse_attend(Q, K, V, cuda(spoiled), cuda(lens + 4), scale, out_dtype=torch.float32)
    assert np.abs(out.cpu().numpy() - want).max() <= 2e-2
    # halves of every list attended apart, merged by their log-sum-exps
    a = np.where(np.arange(400)[None, :] % 2 == 0, ids, -1)
    b = np.where(np.arange(400)[None, :] % 2 == 1, ids, -1)
    oa, la = ops.sparse_attend(Q, K, V, cuda(a), cuda(lens), scale, out_dtype=torch.float32)
    ob, lb = ops.sparse_attend(Q, K, V, cuda(b), cuda(lens), scale, out_dtype=torch.float32)
    merged, mlse = ops.lse_merge(torch.stack([oa, ob]), torch.stack([la, lb]))
    assert np.abs(merged.cpu().numpy() - want).max() <= 2e-2
    ok = np.isfinite(want_lse)
    np.testing.assert_allclose(mlse.cpu().numpy()[ok], want_lse[ok], rtol=0, atol=2e-3)
    cpu_merge, _ = oracle.lse_merge(torch.stack([oa, ob]).cpu().numpy(), torch.stack([la, lb]).cpu().numpy())
    np.testing.assert_allclose(merged.cpu().numpy(), cpu_merge, rtol=0, atol=1e-5)


def test_topk_attention_reproduces_the_reference(oracle):
    from lsa_b200 import core
    g = golden("attention")
    q, k, v = (cuda(bf16_round(g[n]))[None] for n in "qkv")
    T, dh = g["q"].shape[0], g["q"].shape[2]
    # dh 16 is below what the tensor-core kernel takes: the call is refused, not rerouted
    with pytest.raises(ValueError, match="shape outside"):
        core.topk_attention(q, k, v, cuda(g["selected"])[None], 8, 2, dh ** -0.5)
    m = golden("mini_c1")
    bf = lambda bits: (torch.from_numpy(bits.astype(np.int32)) << 16).view(torch.float32)
    Q, K, V = bf(m["q_bf16"]).cuda(), bf(m["k_bf16"]).cuda(), bf(m["v_bf16"]).cuda()
    out = core.topk_attention(Q[None], K[None], V[None], cuda(m["selected"])[None], 128, 4, 64 ** -0.5)
    err = np.abs(out[0].cpu().numpy()[m["out_rows"]] - m["out"])
    assert err.max() <= 2e-2 and err.mean() <= 2e-3
    # full budget is dense causal attention; future keys in the selection are dropped
    full = torch.arange(1024, dtype=torch.int32).expand(1, 1024, 1024).contiguous().cuda()
    dense = core.topk_attention(Q[None], K[None], V[None], full, 0, 0, 64 ** -0.5)
    window = core.topk_attention(Q[None], K[None], V[None], torch.full((1, 1024, 1), -1, dtype=torch.int32).cuda(),
                                 1024, 0, 64 ** -0.5)
    assert (dense - window).abs().max() <= 2e-2


def test_cpu_tensors_are_refused(ops):
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.pool_keys(torch.zeros(1, 16, 8), 4)
