"""The paged serving index on the GPU: requests of different lengths share one bucket cache and one KV pool whose
pages are not in order, and every decode list must be the oracle's read of that request, as KV slots."""

import numpy as np
import pytest
import torch

from helpers import bf16_round, cuda, mixture, unit_rows

pytestmark = pytest.mark.gpu


def test_batched_decode_over_paged_buckets_and_kv(oracle):
    from lsa_b200 import ops
    from lsa_b200.layer import FlatDesign
    from lsa_b200.serving import BucketCache, Selector

    design = FlatDesign(pool_size=4, bucket_size=16, bucket_cap=32, cluster_block_size=256, top_p=6, top_k=150,
                        sink_size=4, window_size=256)
    d_idx, kv_page, page_buckets = 32, 64, 32
    lengths = [700, 2048, 5000, 300, 1333]
    rng = np.random.default_rng(0)
    cache = BucketCache(design, d_idx, pages=24, page_buckets=page_buckets, max_requests=8, max_request_pages=16)
    selector = Selector(cache, kv_page)
    # KV pool pages dealt to requests in a shuffled order
    total_pages = sum(-(-n // kv_page) for n in lengths)
    order = rng.permutation(total_pages + 5).astype(np.int32)
    kv_pages = np.full((len(lengths), max(-(-n // kv_page) for n in lengths)), -1, dtype=np.int32)
    taken = 0
    keys, raws = [], []
    for r, n in enumerate(lengths):
        count = -(-n // kv_page)
        kv_pages[r, :count] = order[taken:taken + count]
        taken += count
        raw = mixture(n, d_idx, 10, 0.3, 100 + r)
        raws.append(raw)
        keys.append(unit_rows(raw))
    # prefill arrives in pieces, the requests interleaved, so pages of the bucket cache interleave too
    cut = [n // 3 for n in lengths]
    for r, n in enumerate(lengths):
        cache.append(r, cuda(keys[r][: cut[r]]))
    for r, n in enumerate(lengths):
        cache.append(r, cuda(keys[r][cut[r]:]))
    assert [cache.closed_keys.get(r, 0) for r in range(len(lengths))] == [n // 256 * 256 for n in lengths]

    positions = np.array([n - 1 for n in lengths])
    queries = np.stack([unit_rows(raws[r][positions[r]] + 0.3 * rng.standard_normal(d_idx).astype(np.float32))
                        for r in range(len(lengths))])
    rows = torch.arange(len(lengths)).cuda()
    for splits in (1, 3):
        lists, lens = selector.decode_flat(cuda(queries), rows, cuda(positions), cuda(kv_pages), splits=splits)
        for r, n in enumerate(lengths):
            buckets = oracle.build_buckets(keys[r], 4, 16, 32, 256)
            want, want_len = oracle.read(queries[r:r + 1], positions[r:r + 1], buckets, 6, 150, 4, 256)
            ids = want[0, : want_len[0]]
            slots = kv_pages[r][ids // kv_page] * kv_page + ids % kv_page
            assert int(lens[r]) == int(want_len[0])
            assert np.array_equal(lists[r, : int(lens[r])].cpu().numpy(), slots), (r, splits)
            assert (lists[r, int(lens[r]):] == -1).all()

    # the read over the pool: slots in, the oracle reads the same keys through the same table
    Hq, Hkv, dh = 8, 2, 128
    pool_rows = (total_pages + 5) * kv_page
    k = bf16_round(rng.standard_normal((pool_rows, Hkv, dh), dtype=np.float32))
    v = bf16_round(rng.standard_normal((pool_rows, Hkv, dh), dtype=np.float32))
    q = bf16_round(rng.standard_normal((len(lengths), Hq, dh), dtype=np.float32))
    out, _ = ops.sparse_attend(cuda(q, torch.bfloat16), cuda(k, torch.bfloat16), cuda(v, torch.bfloat16), lists, lens,
                               dh ** -0.5, splits=4, out_dtype=torch.float32)
    listed = lists.cpu().numpy()
    want, _ = oracle.sparse_attend(q, k, v, listed, np.full(len(lengths), pool_rows), 0, 0, dh ** -0.5,
                                   lengths=lens.cpu().numpy())
    assert np.abs(out.cpu().numpy() - want).max() <= 2e-2

    # releasing a request gives its pages back, and a new request can take them
    free_before = len(cache.free_pages)
    cache.release(2)
    assert len(cache.free_pages) > free_before and (cache.request_pages[2] == -1).all()
    cache.append(5, cuda(keys[1]))
    assert cache.buckets_of(5) == 2048 // 16
    # pages run short: a request of the running batch never gives its pages up ...
    cache.running(range(8))
    with pytest.raises(RuntimeError, match="out of pages"):
        for r in (6, 7):
            cache.append(r, cuda(keys[2]))
    # ... an idle one does, and the cache goes on
    cache.running([6, 7])
    for r in (6, 7):
        cache.release(r, retain=False)
        cache.append(r, cuda(keys[2]))
    assert cache.buckets_of(6) == cache.buckets_of(7) == 5000 // 256 * 256 // 16


def test_a_decode_graph_captured_for_a_context_range_reads_the_same_lists(oracle, monkeypatch):
    # (an engine that captures one decode graph a context range says which through its capture module; the selector
    # then reads no page past the range and cuts the counts to it - for requests inside the range, nothing changes)
    import sys
    import types

    from lsa_b200.layer import FlatDesign
    from lsa_b200.serving import BucketCache, Selector
    from lsa_b200.sglang import context_buckets

    design = FlatDesign(pool_size=4, bucket_size=16, bucket_cap=32, cluster_block_size=256, top_p=6, top_k=150,
                        sink_size=4, window_size=256)
    d_idx, page_buckets = 32, 32
    lengths = [700, 2048, 3000]
    rng = np.random.default_rng(1)
    cache = BucketCache(design, d_idx, pages=16, page_buckets=page_buckets, max_requests=4, max_request_pages=8)
    slots = rng.permutation(4 * 3072).astype(np.int32).reshape(4, 3072)
    selector = Selector(cache, 1, slot_table=lambda: cuda(slots))
    raws = [mixture(n, d_idx, 10, 0.3, 200 + r) for r, n in enumerate(lengths)]
    for r, n in enumerate(lengths):
        cache.append(r, cuda(unit_rows(raws[r])))
    positions = np.array([n - 1 for n in lengths])
    queries = np.stack([unit_rows(raws[r][positions[r]] + 0.3 * rng.standard_normal(d_idx).astype(np.float32))
                        for r in range(len(lengths))])
    rows = torch.arange(len(lengths)).cuda()
    want = selector.decode(cuda(queries), cuda(positions), rows)
    for r, n in enumerate(lengths):  # (and the oracle's read, as slots)
        buckets = oracle.build_buckets(unit_rows(raws[r]), 4, 16, 32, 256)
        lists, lens = oracle.read(queries[r:r + 1], positions[r:r + 1], buckets, 6, 150, 4, 256)
        assert np.array_equal(want[r, : int(lens[0])].cpu().numpy(), slots[r][lists[0, : int(lens[0])]])
    capture = types.ModuleType(context_buckets.CAPTURE_MODE)
    label = {"now": None}
    capture.get_capture_attention_variant = lambda: label["now"]
    monkeypatch.setitem(sys.modules, context_buckets.CAPTURE_MODE, capture)
    page_keys = cache.page_keys
    assert page_keys == 512
    for limit in (6 * page_keys, 7 * page_keys, 64 * page_keys):  # ranges that hold every request here
        label["now"] = f"context_{limit}"
        assert torch.equal(selector.decode(cuda(queries), cuda(positions), rows), want)
    # a range shorter than a request cuts what that padded row may count to the range's pages; the others are as before
    label["now"] = f"context_{4 * page_keys}"
    cut = selector.decode(cuda(queries), cuda(positions), rows)
    assert torch.equal(cut[:2], want[:2]) and not torch.equal(cut[2], want[2])
