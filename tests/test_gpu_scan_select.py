"""The tensor-core bucket scan must return the exact scan's packed keys, key for key: its bf16 scores only ever choose
which buckets are rescored, and a row it cannot prove is scanned exactly. The cases below lean on the places a
thresholded scan goes wrong: ties at the threshold, rows that see nothing or almost nothing, wild query lengths, lists
that overflow, samples that say nothing about the row."""

import numpy as np
import pytest
import torch

from helpers import cuda, mixture, unit_rows

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from lsa_b200 import ops as module

    return module


def _oracle_keys(oracle, queries, cents, visible, keep, row_keep=None, base=0):
    want = np.full((len(queries), keep), oracle.EMPTY_KEY, dtype=np.int64)
    for r in range(len(queries)):
        n = int(visible[r])
        if n == 0:
            continue
        keys = oracle.pack_keys(oracle.scores(queries[r], cents[:n]), np.arange(base, base + n, dtype=np.int32))
        top = np.sort(keys)[::-1][: keep if row_keep is None else int(row_keep[r])]
        want[r, : len(top)] = top
    return want


def _both(ops, queries, cents, visible, keep, **kw):
    q, c, v = cuda(queries), cuda(cents), cuda(visible)
    status = torch.zeros(1, device="cuda", dtype=torch.int32)
    got, picked = ops.scan_select(q, c, c.bfloat16(), v, keep, status=status, **kw)
    flat = {k: kw[k] for k in ("row_top_p", "bucket_id_base") if k in kw}
    want, want_picked = ops.flat_select(q, c, v, keep, **flat)
    assert int(status) == 0
    assert torch.equal(got, want) and torch.equal(picked, want_picked)
    return got


@pytest.mark.parametrize("R,m,keep,hint", [(300, 5000, 64, 0), (128, 1024, 16, 1024), (1000, 40000, 128, 0),
                                             (257, 20000, 512, 9000), (5, 3000, 8, 0)])
def test_scan_matches_the_oracle_and_the_exact_scan(ops, oracle, R, m, keep, hint):
    raw = mixture(m, 64, 48, 0.4, R + m)
    cents = unit_rows(raw) * np.random.default_rng(0).uniform(0.5, 1.0, (m, 1)).astype(np.float32)
    rng = np.random.default_rng(R)
    queries = unit_rows(raw[rng.integers(0, m, R)] + 0.5 * rng.standard_normal((R, 64), dtype=np.float32))
    visible = rng.integers(0, (hint or m) + 1, R).astype(np.int32)
    visible[:5] = [0, 1, min(1023, hint or m), min(1024, hint or m), hint or m]
    got = _both(ops, queries, cents, visible, keep, max_visible=hint)
    rows = np.r_[0:5, rng.integers(0, R, 12)]
    want = _oracle_keys(oracle, queries[rows], cents, visible[rows], keep)
    assert np.array_equal(got.cpu().numpy()[rows], want)


def test_ties_at_the_threshold_and_lists_that_overflow(ops, oracle):
    rng = np.random.default_rng(5)
    base = unit_rows(rng.standard_normal((1, 64), dtype=np.float32))
    cents = np.repeat(base, 6000, axis=0)  # thousands of identical centroids: every sample ties, every list overflows
    cents[::7] = unit_rows(rng.standard_normal((len(cents[::7]), 64), dtype=np.float32))
    queries = unit_rows(base + 0.01 * rng.standard_normal((200, 64), dtype=np.float32))
    queries[1] *= 0.01
    queries[2] *= 500.0
    queries[3] = 0.0
    visible = np.array([0, 1, 300, 1023, 1024, 2049, 5999, 6000] * 25, dtype=np.int32)
    got = _both(ops, queries, cents, visible, 64)
    want = _oracle_keys(oracle, queries[:16], cents, visible[:16], 64)
    assert np.array_equal(got.cpu().numpy()[:16], want)
    # scores that differ in the last bits only: the bf16 scan cannot rank them, the rescoring must
    close = unit_rows(base + 1e-4 * rng.standard_normal((4096, 64), dtype=np.float32))
    _both(ops, queries, close, np.full(200, 4096, np.int32), 32)


def test_samples_that_mislead(ops):
    # every sampled centroid (a stride of 4 apart) scores low, the best buckets lie between the samples; and the
    # other way round: only the samples score high
    rng = np.random.default_rng(11)
    m = 2048
    axis = unit_rows(rng.standard_normal((1, 64), dtype=np.float32))
    noise = unit_rows(rng.standard_normal((m, 64), dtype=np.float32))
    queries = unit_rows(axis + 0.05 * rng.standard_normal((130, 64), dtype=np.float32))
    visible = np.full(130, m, np.int32)
    for sampled_high in (False, True):
        cents = noise.copy()
        on = np.arange(m) % 4 == 0
        hot = on if sampled_high else ~on
        cents[hot] = unit_rows(axis + 0.3 * rng.standard_normal((int(hot.sum()), 64), dtype=np.float32))
        _both(ops, queries, cents, visible, 64)


def test_row_budgets_id_base_and_ragged_rows(ops, oracle):
    rng = np.random.default_rng(3)
    m, R = 9000, 391
    cents = unit_rows(mixture(m, 64, 16, 0.3, 1))
    queries = unit_rows(rng.standard_normal((R, 64), dtype=np.float32)) * rng.uniform(0.01, 500, (R, 1)).astype(np.float32)
    visible = rng.integers(0, m + 1, R).astype(np.int32)
    row_keep = rng.integers(0, 33, R).astype(np.int32)
    got = _both(ops, queries, cents, visible, 32, row_top_p=cuda(row_keep), bucket_id_base=70000)
    want = _oracle_keys(oracle, queries[:24], cents, visible[:24], 32, row_keep[:24], base=70000)
    assert np.array_equal(got.cpu().numpy()[:24], want)


def test_a_chunk_of_the_long_context_shape(ops):
    # the shape of a prefill chunk deep in a 10M-token context: 8,192 rows over 16,384 buckets, top 128
    gen = torch.Generator(device="cuda").manual_seed(0)
    m, R = 16384, 8192
    mu = torch.randn(256, 64, generator=gen, device="cuda")
    cents = torch.nn.functional.normalize(mu[torch.randint(0, 256, (m,), generator=gen, device="cuda")] +
                                          0.5 * torch.randn(m, 64, generator=gen, device="cuda"), dim=1)
    queries = torch.nn.functional.normalize(cents[torch.randint(0, m, (R,), generator=gen, device="cuda")] +
                                            0.5 * torch.randn(R, 64, generator=gen, device="cuda"), dim=1)
    visible = torch.full((R,), m - 8, device="cuda", dtype=torch.int32)
    status = torch.zeros(1, device="cuda", dtype=torch.int32)
    got, _ = ops.scan_select(queries, cents, cents.bfloat16(), visible, 128, max_visible=m, status=status)
    want, _ = ops.flat_select(queries, cents, visible, 128)
    assert int(status) == 0 and torch.equal(got, want)


def test_index_vectors_in_a_narrow_cone_are_told_apart_about_their_centre(ops):
    # every centroid within 0.1 of one axis: a row's scores differ in the third digit, under what bf16 can rank - until
    # the common centre is taken out of the operand
    rng = np.random.default_rng(21)
    m, R = 8192, 1500
    axis = unit_rows(rng.standard_normal((1, 64), dtype=np.float32))
    cents = unit_rows(axis + 0.012 * rng.standard_normal((m, 64), dtype=np.float32))
    queries = unit_rows(axis + 0.012 * rng.standard_normal((R, 64), dtype=np.float32))
    visible = rng.integers(1024, m + 1, R).astype(np.int32)
    q, c, v = cuda(queries), cuda(cents), cuda(visible)
    cents[::97] = unit_rows(axis + 0.06 * rng.standard_normal((len(cents[::97]), 64), dtype=np.float32))  # a few stray far
    c = cuda(cents)
    operand, lengths, radius = ops.scan_centre(c[:4096], c[:64].mean(0))
    later = ops.scan_centre(c[4096:], c[:64].mean(0), radius=radius)  # as an index grows
    operand, lengths = torch.cat([operand, later[0]]), torch.cat([lengths, later[1]])
    assert 0.3 < float(radius) < 0.7 and float(lengths.median()) < 0.15
    assert torch.allclose(lengths, (c - c[:64].mean(0)).norm(dim=1), rtol=1e-4)
    want, _ = ops.flat_select(q, c, v, 64)
    got, _ = ops.scan_select(q, c, operand, v, 64, lengths=lengths, radius=radius)
    assert torch.equal(got, want)
    plain, ones, unit = ops.scan_centre(c)
    assert 0.99 < float(unit) < 1.01 and torch.equal(plain, c.bfloat16())
    got, _ = ops.scan_select(q, c, plain, v, 64, lengths=ones, radius=unit)  # (the rows are crowded: scanned exactly)
    assert torch.equal(got, want)
