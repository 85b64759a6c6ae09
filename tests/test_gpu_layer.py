"""One flat layer end to end on the GPU against the oracle: config 1's shapes cut to a few thousand tokens, the
served GQA shapes, and decode rows against their prefill rows."""

import numpy as np
import pytest
import torch

from helpers import bf16_round, cuda, layer_inputs

pytestmark = pytest.mark.gpu


def _layer(Hq, Hkv, dh, d_idx, design, seed):
    from lsa_b200.layer import FlatLayer

    rng = np.random.default_rng(seed)
    w = bf16_round(rng.standard_normal((2, Hkv * dh, d_idx), dtype=np.float32) / np.sqrt(Hkv * dh))
    return FlatLayer(design, cuda(w[0], torch.bfloat16), cuda(w[1], torch.bfloat16), Hq, Hkv, dh), w


@pytest.mark.parametrize("T,Hq,Hkv,dh,d_idx,sizes", [
    (4096 + 200, 8, 2, 128, 32, dict(pool_size=16, bucket_size=64, bucket_cap=128, cluster_block_size=512, top_p=4,
                                     top_k=512, sink_size=4, window_size=512)),
    (6144, 40, 8, 128, 64, dict(pool_size=16, bucket_size=32, bucket_cap=64, cluster_block_size=1024, top_p=16,
                                top_k=1024, sink_size=4, window_size=1024)),
])
def test_prefill_matches_the_oracle_stage_by_stage(oracle, T, Hq, Hkv, dh, d_idx, sizes):
    from lsa_b200.layer import FlatDesign

    design = FlatDesign(**sizes)
    layer, w = _layer(Hq, Hkv, dh, d_idx, design, T)
    q, k, v = layer_inputs(T, Hq, Hkv, dh, 32, T + 1)
    Q, K, V = (cuda(a, torch.bfloat16) for a in (q, k, v))
    out, index = layer.prefill(Q, K, V, chunk=2048, return_index=True)
    # index vectors: float, within rounding of the fixed-order oracle
    want_q = oracle.project(oracle.regroup_queries(q, Hkv), w[0])
    want_k = oracle.project(k.reshape(T, -1), w[1])
    index_q = layer.index_queries(Q).cpu().numpy()
    index_k = index.index_keys.cpu().numpy()
    # (tensor-core accumulation order differs from the oracle's: a few 1e-6 on unit rows)
    assert np.abs(index_q - want_q).max() < 3e-5 and np.abs(index_k - want_k).max() < 3e-5
    # from the device's own index vectors on, every integer result is the oracle's
    buckets = oracle.build_buckets(index_k, design.pool_size, design.bucket_size, design.bucket_cap,
                                   design.cluster_block_size)
    assert np.array_equal(index.buckets.bucket_members.cpu().numpy(), buckets.bucket_members)
    assert np.array_equal(index.buckets.bucket_centroids.cpu().numpy().view(np.int32),
                          buckets.bucket_centroids.view(np.int32))
    positions = np.arange(T)
    lists, lengths = layer.select(cuda(index_q), cuda(positions), index)
    want_lists, want_lengths = oracle.read(index_q, positions, buckets, design.top_p, design.top_k, design.sink_size,
                                           design.window_size)
    assert np.array_equal(lengths.cpu().numpy(), want_lengths)
    assert np.array_equal(lists.cpu().numpy(), want_lists)
    # and against the oracle's own index vectors the selection is the same except where two scores nearly tie
    own = oracle.build_buckets(want_k, design.pool_size, design.bucket_size, design.bucket_cap,
                               design.cluster_block_size)
    own_lists, _ = oracle.read(want_q, positions, own, design.top_p, design.top_k, design.sink_size,
                               design.window_size)
    same = np.mean([np.array_equal(a, b) for a, b in zip(own_lists, want_lists)])
    assert same >= 0.98, same
    rows = np.arange(0, T, 37)
    want, _ = oracle.sparse_attend(q[rows], k, v, want_lists[rows], rows, 0, 0, dh ** -0.5, lengths=want_lengths[rows])
    err = np.abs(out.float().cpu().numpy()[rows] - want)
    assert err.max() <= 2e-2 and err.mean() <= 2e-3, (err.max(), err.mean())


def test_a_decode_step_matches_its_prefill_row(oracle):
    from lsa_b200.layer import FlatDesign

    design = FlatDesign(pool_size=4, bucket_size=16, bucket_cap=32, cluster_block_size=256, top_p=8, top_k=256,
                        sink_size=4, window_size=256)
    T, Hq, Hkv, dh = 3000, 40, 8, 128
    layer, _ = _layer(Hq, Hkv, dh, 64, design, 3)
    q, k, v = layer_inputs(T, Hq, Hkv, dh, 16, 4)
    Q, K, V = (cuda(a, torch.bfloat16) for a in (q, k, v))
    out, index = layer.prefill(Q, K, V, chunk=1024, return_index=True)
    rows = torch.tensor([5, 255, 256, 1000, 2999]).cuda()
    for splits in (1, 4):
        step = layer.decode(Q[rows], rows, K, V, index, splits=splits)
        assert (step.float() - out[rows].float()).abs().max() <= 1e-2


def test_prefill_from_pinned_host_memory_is_the_resident_prefill():
    from lsa_b200.layer import FlatDesign

    design = FlatDesign(pool_size=16, bucket_size=32, bucket_cap=64, cluster_block_size=1024, top_p=16, top_k=1024,
                        sink_size=4, window_size=1024)
    T, Hq, Hkv, dh = 6144 + 300, 40, 8, 128
    layer, _ = _layer(Hq, Hkv, dh, 64, design, 9)
    q, k, v = (torch.from_numpy(a).bfloat16().pin_memory() for a in layer_inputs(T, Hq, Hkv, dh, 32, 10))
    want = layer.prefill(q.cuda(), k.cuda(), v.cuda(), chunk=2048)
    out = torch.empty(T, Hq, dh, dtype=torch.bfloat16).pin_memory()
    for _ in range(2):  # the second call reuses the buffers, streams and events of the first
        out.zero_()
        layer.prefill_from_host(q, k, v, out, chunk=2048)
        torch.cuda.current_stream().synchronize()
        assert torch.equal(out, want.cpu())
