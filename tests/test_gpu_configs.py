"""The benchmark configurations at their stated sizes, against the oracle: config 1 whole (16,384 tokens, a PCA map
256 -> 32, Ward buckets and the k-means variant), config 2's index parameters (top 64 buckets of at most 64 keys) over
32,768 tokens, and the MLA layer of config 4 end to end on a cut of its context."""

import numpy as np
import pytest
import torch

from helpers import cuda

pytestmark = pytest.mark.gpu


def _close(got, want, what):
    gap = np.abs(got - want)
    assert gap.max() <= 2e-2 and gap.mean() <= 2e-3, (what, gap.max(), gap.mean())


def test_config_1_whole(oracle):
    from lsa_b200 import ops
    from lsa_b200 import workloads as W
    from lsa_b200.layer import FlatLayer

    cfg = W.C1
    q, k, v, index_map = W.c1_inputs(cfg)
    T, Hq, Hkv, dh = cfg["tokens"], cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    layer = FlatLayer(W.design_of(cfg), index_map.cuda(), index_map.cuda(), Hq, Hkv, dh)  # fp32 maps: the exact form
    Q, K, V = q.cuda().bfloat16(), k.cuda().bfloat16(), v.cuda().bfloat16()
    out, index = layer.prefill(Q, K, V, chunk=cfg["chunk"], return_index=True)
    torch.cuda.synchronize()
    layer.check()
    # the index vectors are the oracle's (fp32 in a fixed order on both sides); the integer stages then continue from
    # the device's own vectors, so every one of them must be equal
    want_keys = oracle.project(k.numpy().reshape(T, -1), index_map.numpy())
    want_queries = oracle.project(oracle.regroup_queries(q.numpy(), Hkv), index_map.numpy())
    got_keys = index.index_keys.cpu().numpy()
    assert np.abs(got_keys - want_keys).max() <= 5e-6
    buckets = oracle.build_buckets(got_keys, cfg["pool_size"], cfg["bucket_size"], cfg["bucket_cap"],
                                   cfg["cluster_block_size"])
    assert np.array_equal(index.buckets.bucket_members.cpu().numpy(), buckets.bucket_members)
    assert index.buckets.bucket_members.shape == (256, cfg["bucket_cap"])
    positions = np.arange(T)
    index_q = layer.index_queries(Q)
    got_queries = index_q.cpu().numpy()
    assert np.abs(got_queries - want_queries).max() <= 5e-6
    lists, lens = layer.select(index_q, cuda(positions), index)
    want_lists, want_lens = oracle.read(got_queries, positions, buckets, cfg["top_p"], cfg["top_k"], cfg["sink_size"],
                                        cfg["window_size"])
    assert np.array_equal(lists.cpu().numpy(), want_lists) and np.array_equal(lens.cpu().numpy(), want_lens)
    rows = np.arange(0, T, 61)
    want, _ = oracle.sparse_attend(q.numpy()[rows], k.numpy(), v.numpy(), want_lists[rows], rows, 0, 0, dh ** -0.5,
                                   lengths=want_lens[rows])
    _close(out.float().cpu().numpy()[rows], want, "config 1 attention")

    # the k-means variant of the bucketing (no counterpart in the reference): 10 iterations over the 1,024 pools
    # from 256 seeded pools, against the oracle's restatement
    pools = ops.pool_keys(index.index_keys, cfg["pool_size"])
    init = pools[torch.randperm(pools.shape[0], generator=torch.Generator().manual_seed(cfg["seed"]))[:256].cuda()]
    centroids, assign = ops.kmeans(pools, init, 10)
    want_centroids, want_assign = oracle.kmeans(pools.cpu().numpy(), init.cpu().numpy(), 10)
    assert np.array_equal(assign.cpu().numpy(), want_assign)
    assert np.array_equal(centroids.cpu().numpy().view(np.int32), want_centroids.view(np.int32))


def test_config_2_parameters_over_32768_tokens(oracle):
    from lsa_b200 import workloads as W
    from lsa_b200.layer import FlatLayer

    cfg = W.cut(W.C2, 32768)
    q, k, v, wq, wk = W.gqa_inputs(cfg)
    T, Hq, Hkv, dh = cfg["tokens"], cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    layer = FlatLayer(W.design_of(cfg), wq.cuda(), wk.cuda(), Hq, Hkv, dh)
    Q, K, V = q.cuda(), k.cuda(), v.cuda()
    out, index = layer.prefill(Q, K, V, chunk=cfg["chunk"], return_index=True)
    torch.cuda.synchronize()
    layer.check()
    b = index.buckets
    buckets = oracle.Buckets(b.bucket_centroids.cpu().numpy(), b.bucket_members.cpu().numpy(),
                             b.bucket_sizes.cpu().numpy(), b.block_bucket_count, b.cluster_block_size)
    # the device's own index keys through the oracle's clustering: the same members
    rebuilt = oracle.build_buckets(index.index_keys.cpu().numpy(), cfg["pool_size"], cfg["bucket_size"],
                                   cfg["bucket_cap"], cfg["cluster_block_size"])
    assert np.array_equal(rebuilt.bucket_members, buckets.bucket_members)
    rows = np.unique(np.concatenate([np.arange(0, T, 509), [1023, 1024, 8191, 8192, T - 1]]))
    rows_d = cuda(rows)
    index_q = layer.index_queries(Q)
    lists, lens = layer.select(index_q[rows_d], rows_d, index)
    want_lists, want_lens = oracle.read(index_q[rows_d].cpu().numpy(), rows, buckets, cfg["top_p"], cfg["top_k"],
                                        cfg["sink_size"], cfg["window_size"])
    assert np.array_equal(lists.cpu().numpy(), want_lists) and np.array_equal(lens.cpu().numpy(), want_lens)
    assert want_lens.max() > 3000  # the top 64 buckets are really read
    want, _ = oracle.sparse_attend(q[rows].float().numpy(), k.float().numpy(), v.float().numpy(), want_lists, rows, 0, 0,
                                   dh ** -0.5, lengths=want_lens)
    _close(out[rows_d].float().cpu().numpy(), want, "config 2 attention")
    # the same prefill from pinned host memory, streamed: bit-equal
    out_h = torch.empty(T, Hq, dh, dtype=torch.bfloat16).pin_memory()
    layer.prefill_from_host(q.pin_memory(), k.pin_memory(), v.pin_memory(), out_h, chunk=cfg["chunk"])
    torch.cuda.synchronize()
    assert torch.equal(out_h, out.cpu())


def test_config_4_layer_on_a_cut_of_its_context(oracle):
    """The MLA layer as the benchmark steps it - index build, the chunk's own index step, prefill rows and a decode
    row - over 40 cluster blocks of config 4's shape."""
    from lsa_b200 import workloads as W
    from lsa_b200.latent import LatentLayer

    cfg = W.cut(W.C4, 40 * 5120)
    T, chunk, Hq, dk, dv = cfg["tokens"], 2048, cfg["heads"], cfg["latent_dim"], cfg["value_dim"]
    gen = torch.Generator(device="cuda").manual_seed(1)
    cache, tail = W.latent_cache(cfg, gen, keep_tail=chunk)
    qmap, kmap = W.latent_maps(cfg, gen)
    q = W.latent_queries(cfg, tail, gen)
    layer = LatentLayer(W.design_of(cfg), qmap, kmap, Hq, dk, dv, scale=W.latent_scale(cfg))
    index = layer.build_index(cache)
    before = index.buckets.bucket_members.clone()
    first = T - chunk
    layer.extend_index(cache, first, chunk)  # the same keys again: the same buckets
    out = torch.empty(chunk, Hq, dv, dtype=torch.bfloat16, device="cuda")
    layer.prefill_rows(q, first, cache, index, out)
    out1 = layer.decode(q[-1:].contiguous(), torch.tensor([T - 1], device="cuda"), cache, index, splits=37)
    torch.cuda.synchronize()
    layer.check()
    assert torch.equal(before, index.buckets.bucket_members)
    b = index.buckets
    buckets = oracle.Buckets(b.bucket_centroids.cpu().numpy(), b.bucket_members.cpu().numpy(),
                             b.bucket_sizes.cpu().numpy(), b.block_bucket_count, b.cluster_block_size)
    rebuilt = oracle.build_buckets(index.index_keys.cpu().numpy(), cfg["pool_size"], cfg["bucket_size"],
                                   cfg["bucket_cap"], cfg["cluster_block_size"])
    assert np.array_equal(rebuilt.bucket_members, buckets.bucket_members)
    rows = np.array([0, 1, 777, chunk - 2, chunk - 1])
    positions = first + rows
    index_q = layer.index_queries(q)
    lists, lens = layer.select(index_q[cuda(rows)], cuda(positions), index)
    want_lists, want_lens = oracle.read(index_q[cuda(rows)].cpu().numpy(), positions, buckets, cfg["top_p"],
                                        cfg["top_k"], cfg["sink_size"], cfg["window_size"])
    assert np.array_equal(lens.cpu().numpy(), want_lens)
    assert all(np.array_equal(lists[i, : want_lens[i]].cpu().numpy(), want_lists[i, : want_lens[i]]) for i in range(5))
    latent = cache.float().cpu().numpy()
    for i in (2, 4):
        ids = want_lists[i, : want_lens[i]]
        gathered = latent[ids]
        want, _ = oracle.sparse_attend(q[rows[i]:rows[i] + 1].float().cpu().numpy(), gathered[:, None, :],
                                       gathered[:, None, :], np.arange(len(ids), dtype=np.int32)[None],
                                       np.array([len(ids)]), 0, 0, W.latent_scale(cfg))
        _close(out[rows[i]].float().cpu().numpy(), want[0, :, :dv], f"row {rows[i]}")
    # the decode row maps its query through the few-rows kernels: its own index vector, its own list
    iq1 = layer.index_queries(q[-1:].contiguous())
    assert (iq1 - index_q[-1:]).abs().max() <= 2e-3
    list1, len1 = oracle.read(iq1.cpu().numpy(), np.array([T - 1]), buckets, cfg["top_p"], cfg["top_k"],
                              cfg["sink_size"], cfg["window_size"])
    ids = list1[0, : len1[0]]
    gathered = latent[ids]
    want, _ = oracle.sparse_attend(q[-1:].float().cpu().numpy(), gathered[:, None, :], gathered[:, None, :],
                                   np.arange(len(ids), dtype=np.int32)[None], np.array([len(ids)]), 0, 0,
                                   W.latent_scale(cfg))
    _close(out1[0].float().cpu().numpy(), want[0, :, :dv], "decode row")
    # the same chunk from pinned host buffers, a piece at a time with the copies beside the work: the same bits
    q_h, rows_h = q.cpu().pin_memory(), cache[first:].cpu().pin_memory()
    out_h = torch.empty(chunk, Hq, dv, dtype=torch.bfloat16).pin_memory()
    cache[first:].zero_()
    layer.prefill_from_host(q_h, rows_h, first, cache, index, out_h, pieces=3)
    torch.cuda.synchronize()
    layer.check()
    assert torch.equal(cache[first:].cpu(), rows_h) and torch.equal(out_h, out.cpu())
