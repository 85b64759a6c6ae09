"""The host side of the sequence-sharded layer with two gloo ranks on CPU: shard bounds, the candidate exchange,
the log-sum-exp weights and the row reduction, checked against what one rank holding everything computes. The CUDA
kernels of a step are replaced by the oracle (local scores, local attention)."""

import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import PACKAGE_DIR, ROOT


def test_shard_bounds_cover_every_block_once():
    from lsa_b200.parallel import owned_positions, shard_blocks

    for blocks, world in [(128, 8), (10, 4), (3, 8), (1, 1), (0, 2)]:
        bounds = shard_blocks(blocks, world)
        assert bounds[0][0] == 0 and bounds[-1][1] == blocks
        assert all(a[1] == b[0] for a, b in zip(bounds, bounds[1:]))
        sizes = [end - first for first, end in bounds]
        assert max(sizes) - min(sizes) <= 1
    # the open tail block belongs to the last rank
    assert owned_positions(1000, 64, 0, 2) == (0, 512)
    assert owned_positions(1000, 64, 1, 2) == (512, 1000)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, result_dir):
    for path in (ROOT, PACKAGE_DIR, os.path.join(ROOT, "tests")):
        if path not in sys.path:
            sys.path.insert(0, path)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle
        from helpers import mixture, unit_rows
        from lsa_b200.parallel import gather_candidates, merge_weight, owned_positions, reduce_rows, shard_blocks

        # ---- the same seeded cache on every rank
        T, d, block, bucket, cap, pool = 4096, 32, 256, 16, 32, 4
        top_p, top_k, sink, window = 8, 100, 4, 256
        raw = mixture(T, d, 12, 0.3, 5)
        keys = unit_rows(raw)
        buckets = oracle.build_buckets(keys, pool, bucket, cap, block)
        rng = np.random.default_rng(6)
        positions = np.sort(rng.integers(0, T, 32))
        queries = unit_rows(raw[positions] + 0.4 * rng.standard_normal((32, d), dtype=np.float32))
        want_lists, want_len, want_picked, want_keys = oracle.read(queries, positions, buckets, top_p, top_k, sink,
                                                                   window, return_picked=True)
        # ---- this rank's buckets: local top-p with global ids
        per_block = block // bucket
        first, end = shard_blocks(T // block, world)[rank]
        base, stop = first * per_block, end * per_block
        local = np.full((32, top_p), oracle.EMPTY_KEY, dtype=np.int64)
        for r in range(32):
            visible = min(positions[r] // block * per_block, len(buckets.bucket_sizes))
            n = int(np.clip(visible - base, 0, stop - base))
            scores = oracle.scores(queries[r], buckets.bucket_centroids[base:base + n]) if n else np.zeros(0, np.float32)
            packed = np.sort(oracle.pack_keys(scores, np.arange(base, base + n, dtype=np.int32)))[::-1][:top_p]
            local[r, : len(packed)] = packed
        every = gather_candidates(torch.from_numpy(local))
        assert every.shape == (world, 32, top_p)
        merged = np.sort(every.numpy().transpose(1, 0, 2).reshape(32, -1), axis=1)[:, ::-1][:, :top_p]
        assert np.array_equal(merged, want_keys), "the merged candidates are not the single-rank top-p"
        picked = oracle.unpack_ids(merged)
        # ---- owned share of the expansion: the union over ranks is the single-rank list
        lo, hi = owned_positions(T, block, rank, world)
        lists, lens = oracle.expand(picked, positions, buckets.bucket_members, top_k, sink, window)
        assert np.array_equal(lists, want_lists)
        mine = np.where((lists >= lo) & (lists < hi), lists, -1)
        # ---- partial attention over the owned keys, merged by log-sum-exp and reduced to this rank's rows
        Hq, Hkv, dh = 4, 2, 16
        q = rng.standard_normal((32, Hq, dh), dtype=np.float32)
        k = rng.standard_normal((T, Hkv, dh), dtype=np.float32)
        v = rng.standard_normal((T, Hkv, dh), dtype=np.float32)
        whole, whole_lse = oracle.sparse_attend(q, k, v, lists, positions, 0, 0, 0.25, lengths=lens)
        part, lse = oracle.sparse_attend(q, k, v, mine, positions, 0, 0, 0.25)
        weight, total = merge_weight(torch.from_numpy(lse))
        np.testing.assert_allclose(total.numpy(), whole_lse, rtol=0, atol=2e-6)
        out = reduce_rows(torch.from_numpy(part) * weight[..., None])
        share = 32 // world
        np.testing.assert_allclose(out.numpy(), whole[rank * share:(rank + 1) * share], rtol=0, atol=5e-6)
        # the all-to-all form: every rank receives all ranks' parts of ITS rows and merges them locally
        from lsa_b200.parallel import exchange_rows
        parts, lses = exchange_rows(torch.from_numpy(part), torch.from_numpy(lse))
        assert parts.shape == (world, share, Hq, dh) and lses.shape == (world, share, Hq)
        merged, merged_lse = oracle.lse_merge(parts.numpy(), lses.numpy())
        np.testing.assert_allclose(merged, whole[rank * share:(rank + 1) * share], rtol=0, atol=5e-6)
        np.testing.assert_allclose(merged_lse, whole_lse[rank * share:(rank + 1) * share], rtol=0, atol=2e-6)
        # a row nobody reads has weight zero everywhere, not NaN
        weight, total = merge_weight(torch.full((3, 2), float("-inf")))
        assert not weight.any() and torch.isinf(total).all()
        # page fingerprints of a decode group: each rank prints the slots it owns (slot s lives on rank s % world),
        # the group adds the 16-bit pieces with a float all-reduce, and every rank holds the whole page's number
        from lsa_b200.sglang.layer_index import exact_group_sum
        page_rows, pages = 64, 3
        bits = rng.integers(0, 1 << 16, (pages * page_rows, 32), dtype=np.uint16)
        words, places = oracle.fingerprint_weights(page_rows)
        slots = np.arange(pages * page_rows)
        own = oracle.page_fingerprints(bits, slots % world == rank, words, places)

        def group_sum(pieces):
            dist.all_reduce(pieces)
            return pieces

        total = exact_group_sum(torch.from_numpy(own), group_sum)
        whole_pages = oracle.page_fingerprints(bits, np.ones(len(slots), bool), words, places)
        assert np.array_equal(total.numpy(), whole_pages), "the group's sum is not the whole page's fingerprint"
        open(os.path.join(result_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def test_two_ranks_reproduce_the_single_rank_read(tmp_path):
    world = 2
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert sorted(os.listdir(tmp_path)) == ["ok0", "ok1"]
