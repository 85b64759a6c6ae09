"""Bucket-major attention of a prefill chunk (`lsa_bucket_attend`): the same read as expansion + gather attention
(`expand_buckets` then `topk_attention`, src/lsa/core/reference.py:268-289, src/lsa/core/attention.py:65-146), with
the loop over buckets outside the loop over rows. Held to the oracle's read and to the gather path."""

import numpy as np
import pytest
import torch

from helpers import cuda, layer_inputs, mixture, unit_rows

pytestmark = pytest.mark.gpu


def _case(oracle, seed=5, Hq=10, Hkv=2):
    T, dh, d = 3072, 128, 32
    q, k, v = layer_inputs(T, Hq, Hkv, dh, 16, seed)
    raw = mixture(T, d, 24, 0.3, seed + 1)
    buckets = oracle.build_buckets(unit_rows(raw), 4, 16, 32, 256)
    first, rows = 1500, 600
    positions = np.arange(first, first + rows)
    rng = np.random.default_rng(seed + 2)
    index_q = unit_rows(raw[positions] + 0.3 * rng.standard_normal((rows, d)).astype(np.float32))
    return q, k, v, buckets, positions, index_q, first


def _close(got, want, what):
    gap = np.abs(got - want)
    assert gap.max() <= 2e-2 and gap.mean() <= 2e-3, (what, gap.max(), gap.mean())


@pytest.mark.parametrize("warp_mma", [False, True])
@pytest.mark.parametrize("top_p,top_k", [(12, 400), (12, 150), (3, 400)])
def test_bucket_major_read_matches_the_oracle_and_the_gather_path(oracle, top_p, top_k, warp_mma):
    from lsa_b200 import ops

    q, k, v, buckets, positions, index_q, first = _case(oracle)
    sink, window, scale = 4, 128, 128 ** -0.5
    want_lists, want_len, picked, _ = oracle.read(index_q, positions, buckets, top_p, top_k, sink, window,
                                                  return_picked=True)
    Q, K, V = (cuda(a, torch.bfloat16) for a in (q, k, v))
    rows = Q[first:first + len(positions)]
    pos, mem, pk = cuda(positions), cuda(buckets.bucket_members), cuda(picked)
    band = ops.band_attend(rows, K, V, first, window, sink, scale)
    out, lse = ops.bucket_attend(rows, K, V, pk, pos, mem, top_k, sink, window, scale, init=band, warp_mma=warp_mma)
    want, want_lse = oracle.sparse_attend(q[positions], k, v, want_lists, positions, 0, 0, scale, lengths=want_len)
    _close(out.float().cpu().numpy(), want, "oracle")
    assert np.abs(lse.cpu().numpy() - want_lse).max() <= 2e-2
    lists, lens, _ = ops.expand(pk, pos, mem, top_k, sink, window, local=False)
    gathered, _ = ops.sparse_attend(rows, K, V, lists, lens, scale, init=band)
    _close(out.float().cpu().numpy(), gathered.float().cpu().numpy(), "gather path")


@pytest.mark.parametrize("warp_mma", [False, True])
@pytest.mark.parametrize("Hq,Hkv", [(2, 2), (6, 2), (8, 2), (7, 1), (8, 1)])
def test_bucket_major_read_over_head_groups(oracle, Hq, Hkv, warp_mma):
    """Groups of 1, 3, 4, 7 and 8 query heads a KV head: a tile of the tcgen05 pass holds (pair, head) rows, so the
    group decides where a pair's rows sit and which tile they fall in."""
    from lsa_b200 import ops

    q, k, v, buckets, positions, index_q, first = _case(oracle, seed=7, Hq=Hq, Hkv=Hkv)
    sink, window, scale, top_p, top_k = 4, 128, 128 ** -0.5, 12, 300
    want_lists, want_len, picked, _ = oracle.read(index_q, positions, buckets, top_p, top_k, sink, window,
                                                  return_picked=True)
    Q, K, V = (cuda(a, torch.bfloat16) for a in (q, k, v))
    rows = Q[first:first + len(positions)]
    pos, mem, pk = cuda(positions), cuda(buckets.bucket_members), cuda(picked)
    band = ops.band_attend(rows, K, V, first, window, sink, scale)
    out, lse = ops.bucket_attend(rows, K, V, pk, pos, mem, top_k, sink, window, scale, init=band, warp_mma=warp_mma)
    want, want_lse = oracle.sparse_attend(q[positions], k, v, want_lists, positions, 0, 0, scale, lengths=want_len)
    _close(out.float().cpu().numpy(), want, "oracle")
    assert np.abs(lse.cpu().numpy() - want_lse).max() <= 2e-2


@pytest.mark.parametrize("warp_mma", [False, True])
def test_bucket_major_read_alone_under_row_budgets_and_missing_picks(oracle, warp_mma):
    from lsa_b200 import ops

    q, k, v, buckets, positions, index_q, first = _case(oracle, seed=11)
    sink, window, scale, top_p, top_k = 4, 128, 128 ** -0.5, 12, 400
    _, _, picked, _ = oracle.read(index_q, positions, buckets, top_p, top_k, sink, window, return_picked=True)
    picked = picked.copy()
    picked[::7, 2] = -1       # a hole in a row's picks
    picked[5] = -1            # a row that picked nothing
    early = positions < first + 200
    row_p = np.where(early, 5, top_p).astype(np.int32)
    row_k = np.where(early, 90, top_k).astype(np.int32)
    Q, K, V = (cuda(a, torch.bfloat16) for a in (q, k, v))
    rows = Q[first:first + len(positions)]
    pos, mem, pk = cuda(positions), cuda(buckets.bucket_members), cuda(picked)
    # no band: the read is over the expansion alone, which the one-warp expansion lists for the oracle
    lists, lens, _ = ops.expand(pk, pos, mem, top_k, sink, window, cuda(row_p), cuda(row_k), local=False)
    want, want_lse = oracle.sparse_attend(q[positions], k, v, lists.cpu().numpy(), positions, 0, 0, scale,
                                          lengths=lens.cpu().numpy())
    out, lse = ops.bucket_attend(rows, K, V, pk, pos, mem, top_k, sink, window, scale, row_top_p=cuda(row_p),
                                 row_top_k=cuda(row_k), warp_mma=warp_mma)
    _close(out.float().cpu().numpy(), want, "oracle")
    got_lse = lse.cpu().numpy()
    assert int(lens[5]) == 0 and not out[5].any() and np.isneginf(got_lse[5]).all()
    held = lens.cpu().numpy() > 0
    assert np.abs(got_lse[held] - want_lse[held]).max() <= 2e-2
    # cut lists: some row's running count must have stopped inside a bucket for the budget to have been exercised
    assert (lens.cpu().numpy()[early] == 90).any()


@pytest.mark.parametrize("warp_mma", [False, True])
def test_full_buckets_a_bucket_across_the_sinks_and_a_bucket_with_many_pairs(oracle, warp_mma):
    """The edges of the bucket-major pass that clustered data seldom meets: every bucket full to the cap of 64, a
    bucket whose members straddle the sink boundary (its first ids belong to the sinks and are not read as
    expansion), one bucket picked by every row (far more than the 256 pairs a CTA takes, so it is cut into
    segments), and members past the cache handed in (skipped, as the gather path skips them)."""
    from lsa_b200 import ops

    rng = np.random.default_rng(3)
    T, Hq, Hkv, dh, cap = 4096, 10, 2, 128, 64
    q, k, v = layer_inputs(T, Hq, Hkv, dh, 16, 13)
    buckets_n = T // cap
    members = np.arange(T, dtype=np.int32).reshape(buckets_n, cap)  # bucket b = positions 64 b .. 64 b + 63, all full
    first, rows, top_p, top_k, sink, window, scale = 3000, 700, 6, 384, 4, 256, 128 ** -0.5
    positions = np.arange(first, first + rows)
    picked = np.empty((rows, top_p), dtype=np.int32)
    for r in range(rows):
        # everybody reads bucket 0 (sinks inside) and bucket 7; the rest at random among the buckets before the window
        free = np.setdiff1d(np.arange(1, (first - window) // cap), [7])  # (a bucket is picked once a row)
        others = rng.choice(free, top_p - 2, replace=False)
        picked[r] = np.concatenate([[7, 0], others])
        rng.shuffle(picked[r])
    want_lists, want_len = oracle.expand(picked, positions, members, top_k, sink, window)
    assert (want_len == want_len[0]).all() and want_len[0] == (top_p * cap - sink) + window + sink
    Q, K, V = (cuda(a, torch.bfloat16) for a in (q, k, v))
    rows_q = Q[first:first + rows]
    pos, mem, pk = cuda(positions), cuda(members), cuda(picked)
    band = ops.band_attend(rows_q, K, V, first, window, sink, scale)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out, lse = ops.bucket_attend(rows_q, K, V, pk, pos, mem, top_k, sink, window, scale, init=band, warp_mma=warp_mma,
                                 status=status)
    want, want_lse = oracle.sparse_attend(q[positions], k, v, want_lists, positions, 0, 0, scale, lengths=want_len)
    assert int(status) == 0
    _close(out.float().cpu().numpy(), want, "oracle")
    assert np.abs(lse.cpu().numpy() - want_lse).max() <= 2e-2

    # the same picks over a cache that ends before some members: those ids are skipped
    short = 2000
    lists, lens, _ = ops.expand(pk, pos, mem, top_k, sink, window, local=False)
    want_s, _ = ops.sparse_attend(rows_q, K[:short], V[:short], lists, lens, scale)
    got_s, _ = ops.bucket_attend(rows_q, K[:short], V[:short], pk, pos, mem, top_k, sink, window, scale,
                                 warp_mma=warp_mma)
    _close(got_s.float().cpu().numpy(), want_s.float().cpu().numpy(), "short cache")
