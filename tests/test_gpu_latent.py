"""The MLA form of the path: the latent index space (`regroup_latent`, `LatentMetric`,
src/lsa/core/index_space.py:190-312) and gather attention over a shared latent cache (`topk_attention` with one KV
head whose values are the first 512 dims of the key, src/lsa/core/attention.py:65-146)."""

import numpy as np
import pytest
import torch

from conftest import golden
from helpers import bf16_round, cuda, mixture

pytestmark = pytest.mark.gpu


def test_latent_regroup_matches_the_reference_vectors():
    from lsa_b200 import core

    g = golden("latent_space")
    metric = core.LatentMetric.from_key_maps(cuda(g["key_maps"]))
    assert metric.dim == 12
    assert np.abs(metric.metric_factor.cpu().numpy() - g["metric_factor"]).max() <= 2e-6
    q = cuda(g["q"]).transpose(0, 1)[None]  # [1, Hq, T, dh]
    iq, ik = core.regroup_latent(q, cuda(g["latent"])[None], metric)
    assert iq.shape == (1, 40, 12) and ik.shape == (1, 40, 12)
    assert np.abs(iq[0].cpu().numpy() - g["index_queries"]).max() <= 5e-6
    assert np.abs(ik[0].cpu().numpy() - g["index_keys"]).max() <= 5e-6
    assert not ik[0, 5].any()

    degenerate = cuda(g["key_maps"]).clone()
    degenerate[..., -1] = 0
    with pytest.raises(ValueError, match="do not span"):
        core.LatentMetric.from_key_maps(degenerate)
    with pytest.raises(ValueError, match=r"\[Hq, dh, r\]"):
        core.LatentMetric.from_key_maps(torch.randn(16, 12, device="cuda"))
    with pytest.raises(ValueError, match="metric_factor must be"):
        core.LatentMetric(key_maps=cuda(g["key_maps"]), metric_factor=torch.eye(13, device="cuda"))
    with pytest.raises(ValueError, match="to match the key maps"):
        core.regroup_latent(q[:, :4], cuda(g["latent"])[None], metric)
    with pytest.raises(ValueError, match="to match the key maps"):
        core.regroup_latent(q, cuda(g["latent"])[None, :, :8], metric)


def test_latent_regroup_at_the_served_width(oracle):
    """r = 512, 16 heads of 64 dims: the map is wider than one slice of output dims, so the second-pass
    normalisation runs. Both sides against the oracle's fixed-order product."""
    from lsa_b200 import core

    rng = np.random.default_rng(0)
    heads, dh, r, tokens = 16, 64, 512, 300
    key_maps = (rng.standard_normal((heads, dh, r)) / dh ** 0.5).astype(np.float32)
    q = rng.standard_normal((tokens, heads, dh)).astype(np.float32)
    latent = mixture(tokens, r, 8, 0.3, 1)
    latent[17] = 0
    factor = oracle.latent_metric_factor(key_maps)
    want_q, want_k = oracle.regroup_latent(q, latent, key_maps, factor)
    metric = core.LatentMetric.from_key_maps(cuda(key_maps))
    assert np.abs(metric.metric_factor.cpu().numpy() - factor).max() <= 1e-5
    iq, ik = core.regroup_latent(cuda(q).transpose(0, 1)[None], cuda(latent)[None], metric)
    assert np.abs(iq[0].cpu().numpy() - want_q).max() <= 2e-5
    assert np.abs(ik[0].cpu().numpy() - want_k).max() <= 2e-5
    assert not ik[0, 17].any()
    norms = ik[0].norm(dim=-1).cpu().numpy()
    assert np.abs(np.delete(norms, 17) - 1).max() <= 1e-5


def _latent_case(seed, rows, heads, slots, width, ragged=True):
    rng = np.random.default_rng(seed)
    latent = bf16_round(np.concatenate([mixture(slots, 512, 16, 0.5, seed), rng.standard_normal((slots, 64),
                                                                                                 dtype=np.float32)], 1))
    q = bf16_round(0.3 * rng.standard_normal((rows, heads, 576), dtype=np.float32))
    ids = np.full((rows, width), -1, dtype=np.int32)
    lengths = np.zeros(rows, dtype=np.int32)
    for r in range(rows):
        n = int(rng.integers(0, width + 1)) if ragged else width
        if r == 0:
            n = 0  # an empty list: zeros and a log-sum-exp of minus infinity
        if r == 1:
            n = min(width, 33)  # one key past a tile
        ids[r, :n] = rng.choice(slots, n, replace=False)
        lengths[r] = n
    return q, latent, ids, lengths


@pytest.mark.parametrize("heads,splits,warp_mma", [(64, 1, False), (64, 4, False), (16, 1, False), (128, 3, False),
                                                   (64, 1, True), (128, 3, True)])
def test_latent_attend_matches_the_oracle(oracle, heads, splits, warp_mma):
    """Both forms of the kernel (tcgen05 with tensor-memory accumulators, the default, and warp-level MMA)."""
    from lsa_b200 import ops

    rows, slots, width = 12, 3000, 700
    q, latent, ids, lengths = _latent_case(heads + splits, rows, heads, slots, width)
    scale = 576 ** -0.5
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out, lse = ops.latent_attend(cuda(q, torch.bfloat16), cuda(latent, torch.bfloat16), cuda(ids), cuda(lengths), scale,
                                 splits=splits, out_dtype=torch.float32, warp_mma=warp_mma, status=status)
    assert int(status) == 0
    want, want_lse = oracle.sparse_attend(q, latent[:, None, :], latent[:, None, :], ids,
                                          np.full(rows, slots, dtype=np.int64), 0, 0, scale, lengths=lengths)
    got, got_lse = out.cpu().numpy(), lse.cpu().numpy()
    assert not got[0].any() and np.isneginf(got_lse[0]).all()
    gap = np.abs(got - want[:, :, :512])
    assert gap.max() <= 2e-2 and gap.mean() <= 2e-3, (gap.max(), gap.mean())
    held = lengths > 0
    assert np.abs(got_lse[held] - want_lse[held]).max() <= 2e-2

    # bf16 output, ids outside the cache skipped, lengths left out (the -1 padding is skipped like any bad id)
    ids_bad = ids.copy()
    ids_bad[2, : lengths[2] // 2] = slots + 5
    out16, _ = ops.latent_attend(cuda(q, torch.bfloat16), cuda(latent, torch.bfloat16), cuda(ids_bad), None, scale,
                                 splits=splits, warp_mma=warp_mma)
    keep = ids.copy()
    keep[2, : lengths[2] // 2] = -1
    want2, _ = oracle.sparse_attend(q, latent[:, None, :], latent[:, None, :], keep,
                                    np.full(rows, slots, dtype=np.int64), 0, 0, scale)
    assert np.abs(out16.float().cpu().numpy() - want2[:, :, :512]).max() <= 3e-2


@pytest.mark.parametrize("splits", [1, 3])
def test_latent_attend_with_a_growing_maximum(oracle, splits):
    """Keys whose logits grow along the list: the running maximum of the tensor-memory form jumps by far more than
    the 2^8 it tolerates, so the accumulated output is rescaled in tensor memory, several times a row."""
    from lsa_b200 import ops

    rows, heads, slots, width = 6, 64, 4000, 1500
    q, latent, ids, lengths = _latent_case(11, rows, heads, slots, width, ragged=False)
    rng = np.random.default_rng(5)
    lengths[:] = width
    for r in range(rows):
        ids[r] = rng.choice(slots, width, replace=False)
    # the rows a list names late are scaled up, the same factor for every list that names them
    gain = np.ones(slots, dtype=np.float32)
    for r in range(rows):
        gain[ids[r, width // 3:]] = 3.0
        gain[ids[r, 2 * width // 3:]] = 9.0
    latent = bf16_round(latent * gain[:, None])
    scale = 0.15
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out, lse = ops.latent_attend(cuda(q, torch.bfloat16), cuda(latent, torch.bfloat16), cuda(ids), cuda(lengths), scale,
                                 splits=splits, out_dtype=torch.float32, status=status)
    want, want_lse = oracle.sparse_attend(q, latent[:, None, :], latent[:, None, :], ids,
                                          np.full(rows, slots, dtype=np.int64), 0, 0, scale, lengths=lengths)
    assert int(status) == 0
    gap = np.abs(out.cpu().numpy() - want[:, :, :512])
    assert gap.max() <= 2e-2 * max(1.0, np.abs(want).max()) and gap.mean() <= 2e-3 * max(1.0, np.abs(want).mean() * 10)
    assert np.abs(lse.cpu().numpy() - want_lse).max() <= 2e-2


@pytest.mark.parametrize("splits", [1, 4])
def test_latent_attend_over_runs_of_consecutive_rows(oracle, splits):
    """Lists as an expansion writes them: pools of 64 consecutive rows starting anywhere, a run cut short, a long
    window, sinks, a run that ends with the cache, and scattered ids between them. Whole runs of 64 are staged by
    tensor-map copies and everything else row by row; both must see exactly the listed rows."""
    from lsa_b200 import ops

    rng = np.random.default_rng(21)
    rows, heads, slots, width = 7, 64, 9000, 2600
    q, latent, _, _ = _latent_case(9, rows, heads, slots, 8, ragged=False)
    ids = np.full((rows, width), -1, dtype=np.int32)
    lengths = np.zeros(rows, dtype=np.int32)
    for r in range(rows):
        pieces = []
        taken = np.zeros(slots, dtype=bool)
        for _ in range(int(rng.integers(8, 24))):
            n = int(rng.choice([64, 64, 64, 128, 40, 17, 5, 1]))
            first = int(rng.integers(4, slots - 700 - n))
            if taken[first:first + n].any():
                continue
            taken[first:first + n] = True
            pieces.append(np.arange(first, first + n))
        if r % 2:
            pieces.append(np.arange(slots - 64, slots))            # a run that ends with the cache
        pieces.append(np.arange(slots - 700, slots - 700 + 517))   # the window
        pieces.append(np.arange(0, 4))                             # the sinks
        row = np.concatenate(pieces).astype(np.int32)
        ids[r, : len(row)] = row
        lengths[r] = len(row)
    scale = 576 ** -0.5
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out, lse = ops.latent_attend(cuda(q, torch.bfloat16), cuda(latent, torch.bfloat16), cuda(ids), cuda(lengths), scale,
                                 splits=splits, out_dtype=torch.float32, status=status)
    want, want_lse = oracle.sparse_attend(q, latent[:, None, :], latent[:, None, :], ids,
                                          np.full(rows, slots, dtype=np.int64), 0, 0, scale, lengths=lengths)
    assert int(status) == 0
    gap = np.abs(out.cpu().numpy() - want[:, :, :512])
    assert gap.max() <= 2e-2 and gap.mean() <= 2e-3, (gap.max(), gap.mean())
    assert np.abs(lse.cpu().numpy() - want_lse).max() <= 2e-2
    # a cache that is a strided view (rows 1,200 bytes apart) and ids past its end
    wide = torch.zeros(slots - 100, 600, dtype=torch.bfloat16, device="cuda")
    wide[:, :576] = cuda(latent[: slots - 100], torch.bfloat16)
    out2, _ = ops.latent_attend(cuda(q, torch.bfloat16), wide[:, :576], cuda(ids), cuda(lengths), scale, splits=splits,
                                out_dtype=torch.float32)
    keep = np.where(ids < slots - 100, ids, -1)
    want2, _ = oracle.sparse_attend(q, latent[:, None, :], latent[:, None, :], keep,
                                    np.full(rows, slots, dtype=np.int64), 0, 0, scale, lengths=lengths)
    assert np.abs(out2.cpu().numpy() - want2[:, :, :512]).max() <= 2e-2


@pytest.mark.parametrize("splits", [1, 5])
def test_latent_attend_over_a_dealt_cache(oracle, splits):
    """Four ranks' shares of one cache, dealt out in granules of 64 positions: every rank is handed the WHOLE list of
    positions and reads the ones it holds; the four partial reads merged by their log-sum-exps are the read of the
    whole cache. (One GPU plays the four ranks in turn; lists hold whole pools, cut pools and scattered ids, and one
    row lists nothing that the last rank holds.)"""
    from lsa_b200 import ops
    from lsa_b200.parallel import deal

    rng = np.random.default_rng(8)
    rows, heads, slots, width, world = 5, 64, 64 * 4 * 30, 2400, 4
    q, latent, _, _ = _latent_case(12, rows, heads, slots, 8, ragged=False)
    ids = np.full((rows, width), -1, dtype=np.int32)
    lengths = np.zeros(rows, dtype=np.int32)
    for r in range(rows):
        pieces, taken = [], np.zeros(slots, dtype=bool)
        for _ in range(int(rng.integers(10, 25))):
            n = int(rng.choice([64, 64, 64, 128, 40, 17, 3]))
            first = int(rng.integers(0, slots - 800)) // 64 * 64 + int(rng.choice([0, 0, 0, 5]))
            if r == 1:
                first = first // 256 * 256  # granules of rank 0 only, and what spills over into rank 1's
            if taken[first:first + n].any():  # (a list names a row once)
                continue
            taken[first:first + n] = True
            pieces.append(np.arange(first, first + n))
        pieces.append(np.arange(slots - 600, slots - 600 + 300 + r))
        row = np.concatenate(pieces).astype(np.int32)
        ids[r, : len(row)] = row
        lengths[r] = len(row)
    scale = 576 ** -0.5
    Q, L, I, N = cuda(q, torch.bfloat16), cuda(latent, torch.bfloat16), cuda(ids), cuda(lengths)
    parts, lses = [], []
    for rank in range(world):
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        out, lse = ops.latent_attend(Q, deal(L, rank, world).contiguous(), I, N, scale, splits=splits,
                                     out_dtype=torch.float32, status=status, dealt=(64, world, rank))
        assert int(status) == 0
        parts.append(out)
        lses.append(lse)
    merged, merged_lse = ops.lse_merge(torch.stack(parts), torch.stack(lses))
    want, want_lse = oracle.sparse_attend(q, latent[:, None, :], latent[:, None, :], ids,
                                          np.full(rows, slots, dtype=np.int64), 0, 0, scale, lengths=lengths)
    gap = np.abs(merged.cpu().numpy() - want[:, :, :512])
    assert gap.max() <= 2e-2 and gap.mean() <= 2e-3, (gap.max(), gap.mean())
    assert np.abs(merged_lse.cpu().numpy() - want_lse).max() <= 2e-2
    # a rank that holds nothing of a list returns an empty partial, not garbage
    only0 = np.full((1, 128), -1, dtype=np.int32)
    only0[0, :64] = np.arange(0, 64)
    out, lse = ops.latent_attend(Q[:1], deal(L, 3, world).contiguous(), cuda(only0), None, scale, out_dtype=torch.float32,
                                 dealt=(64, world, 3))
    assert not out.any() and torch.isinf(lse).all()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_the_ranks_of_a_sharded_layer_played_on_one_gpu(world):
    """Every step a rank of the sharded MLA layer takes except the collectives themselves, for 2, 4 and 8 ranks in
    turn on one GPU: the candidates of the ranks' own buckets cut together are the single-GPU picks, bit for bit;
    the rows the ranks list (through their own member tables where the layer keeps them) are, united, the
    single-GPU list; and the ranks' partial reads merged by their log-sum-exps are the single-GPU output."""
    from lsa_b200 import ops
    from lsa_b200 import workloads as W
    from lsa_b200.latent import LatentLayer
    from lsa_b200.parallel import ShardedLatentLayer, deal

    cfg = W.cut(W.C4, 64 * 5120)
    T, chunk, Hq, dk, dv = cfg["tokens"], 256, cfg["heads"], cfg["latent_dim"], cfg["value_dim"]
    gen = torch.Generator(device="cuda").manual_seed(4)
    cache, tail = W.latent_cache(cfg, gen, keep_tail=chunk)
    qmap, kmap = W.latent_maps(cfg, gen)
    q = W.latent_queries(cfg, tail, gen)
    layer = LatentLayer(W.design_of(cfg), qmap, kmap, Hq, dk, dv, scale=W.latent_scale(cfg))
    index = layer.build_index(cache)
    positions = torch.arange(T - chunk, T, device="cuda")
    index_q = layer.index_queries(q)
    want_picked = layer.pick(index_q, positions, index)[0]
    want_lists, want_lens = layer.select(index_q, positions, index)
    want = torch.empty(chunk, Hq, dv, dtype=torch.bfloat16, device="cuda")
    layer.prefill_rows(q, T - chunk, cache, index, want)

    ranks = [ShardedLatentLayer(layer, r, world) for r in range(world)]
    for s in ranks:
        s.adopt_index(index.index_keys, index.buckets.bucket_centroids, index.buckets.bucket_members)
    assert [s.own_tables for s in ranks] == [world >= 4] * world
    every = torch.stack([s.local_candidates(q, positions) for s in ranks])
    _, picked = ops.merge_candidates(every)
    assert torch.equal(picked, want_picked)
    parts, lses, union = [], [], [[] for _ in range(chunk)]
    for r, s in enumerate(ranks):
        lists, lens = s.expand_own(picked, positions)
        local = lists.cpu().numpy().astype(np.int64)
        for i in range(0, chunk, 17):
            row = local[i, : int(lens[i])]
            assert (row >= 0).all()
            union[i] += ((row // 64 * world + r) * 64 + row % 64).tolist()
        out, lse = ops.latent_attend(q, deal(cache, r, world).contiguous(), lists, lens, layer.scale,
                                     out_dtype=torch.bfloat16)
        parts.append(out)
        lses.append(lse)
    for i in range(0, chunk, 17):
        assert sorted(union[i]) == sorted(want_lists[i, : int(want_lens[i])].tolist()), i
    merged, _ = ops.lse_merge(torch.stack(parts), torch.stack(lses), out_dtype=torch.bfloat16)
    gap = (merged.float() - want.float()).abs()
    assert gap.max().item() <= 2e-2 and gap.mean().item() <= 2e-3, (gap.max().item(), gap.mean().item())
    # the decode row: every rank is handed the whole list and reads the positions it holds
    parts, lses = [], []
    for r in range(world):
        out, lse = ops.latent_attend(q[-1:], deal(cache, r, world).contiguous(), want_lists[-1:], want_lens[-1:],
                                     layer.scale, splits=5, out_dtype=torch.float32, dealt=(64, world, r))
        parts.append(out)
        lses.append(lse)
    merged, _ = ops.lse_merge(torch.stack(parts), torch.stack(lses), out_dtype=torch.bfloat16)
    assert (merged.float() - want[-1:].float()).abs().max().item() <= 2e-2


def test_latent_attend_long_lists_in_bf16(oracle):
    """Lists of thousands of keys (a hundred tiles a row), ragged ends, bf16 output: the size a served row has."""
    from lsa_b200 import ops

    rows, heads, slots, width = 5, 64, 20000, 9000
    q, latent, ids, lengths = _latent_case(3, rows, heads, slots, width, ragged=True)
    lengths[2], lengths[3], lengths[4] = width, width - 1, 64 * 17
    for r in (2, 3, 4):
        ids[r, : lengths[r]] = np.random.default_rng(r).choice(slots, lengths[r], replace=False)
    scale = 576 ** -0.5
    out, lse = ops.latent_attend(cuda(q, torch.bfloat16), cuda(latent, torch.bfloat16), cuda(ids), cuda(lengths), scale)
    want, want_lse = oracle.sparse_attend(q, latent[:, None, :], latent[:, None, :], ids,
                                          np.full(rows, slots, dtype=np.int64), 0, 0, scale, lengths=lengths)
    gap = np.abs(out.float().cpu().numpy() - want[:, :, :512])
    assert gap.max() <= 2e-2 and gap.mean() <= 2e-3, (gap.max(), gap.mean())
    held = lengths > 0
    assert np.abs(lse.cpu().numpy()[held] - want_lse[held]).max() <= 2e-2


def test_latent_layer_end_to_end(oracle):
    """Index space -> buckets -> read -> attention for an MLA layer, against the oracle stage by stage."""
    from lsa_b200 import core, ops

    rng = np.random.default_rng(7)
    heads, dh, r, tokens = 16, 64, 512, 2048
    key_maps = (rng.standard_normal((heads, dh, r)) / dh ** 0.5).astype(np.float32)
    latent_nope = bf16_round(mixture(tokens, r, 12, 0.3, 3))
    rope = bf16_round(rng.standard_normal((tokens, 64), dtype=np.float32))
    # pre-index queries whose absorbed form points at their own latent
    q_heads = bf16_round(np.einsum("tr,hdr->thd", latent_nope + 0.3 * rng.standard_normal((tokens, r), dtype=np.float32),
                                   key_maps))
    factor = oracle.latent_metric_factor(key_maps)
    want_q, want_k = oracle.regroup_latent(q_heads, latent_nope, key_maps, factor)
    metric = core.LatentMetric.from_key_maps(cuda(key_maps))
    iq, ik = core.regroup_latent(cuda(q_heads).transpose(0, 1)[None], cuda(latent_nope)[None], metric)
    assert np.abs(ik[0].cpu().numpy() - want_k).max() <= 2e-5

    # buckets and lists from the oracle's keys on both sides, so the integer stages compare bit for bit
    buckets = core.build_buckets(cuda(want_k), 4, 16, 32, 256)
    want_buckets = oracle.build_buckets(want_k, 4, 16, 32, 256)
    assert np.array_equal(buckets.bucket_members.cpu().numpy(), want_buckets.bucket_members)
    positions = np.arange(tokens - 64, tokens)
    lists, lens = core.read(cuda(want_q[positions]), cuda(positions), buckets, 8, 200, 4, 256)
    want_lists, want_lens = oracle.read(want_q[positions], positions, want_buckets, 8, 200, 4, 256)
    assert np.array_equal(lists.cpu().numpy(), want_lists) and np.array_equal(lens.cpu().numpy(), want_lens)

    # the read: absorbed queries (W_h^T q_h, rope part appended) over the latent cache
    absorbed = np.einsum("thd,hdr->thr", q_heads[positions], key_maps)
    q_full = bf16_round(np.concatenate([absorbed, rng.standard_normal((64, heads, 64), dtype=np.float32)], 2))
    cache = np.concatenate([latent_nope, rope], 1)
    scale = (dh + 64) ** -0.5
    out, _ = ops.latent_attend(cuda(q_full, torch.bfloat16), cuda(cache, torch.bfloat16), lists, lens, scale, splits=2,
                               out_dtype=torch.float32)
    want, _ = oracle.sparse_attend(q_full, cache[:, None, :], cache[:, None, :], want_lists, positions, 0, 0, scale,
                                   lengths=want_lens)
    gap = np.abs(out.cpu().numpy() - want[:, :, :512])
    assert gap.max() <= 2e-2 and gap.mean() <= 2e-3, (gap.max(), gap.mean())
