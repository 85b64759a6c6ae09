"""The sequence-sharded layer on real GPUs over NCCL: every rank's rows of the output against the single-GPU layer.
Needs two or more GPUs in the box; one process a GPU, spawned as children."""

import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import PACKAGE_DIR, ROOT

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, result_dir):
    for path in (ROOT, PACKAGE_DIR, os.path.join(ROOT, "tests")):
        if path not in sys.path:
            sys.path.insert(0, path)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from helpers import bf16_round, cuda, layer_inputs
        from lsa_b200.layer import FlatDesign, FlatLayer
        from lsa_b200.parallel import ShardedFlatLayer, deal

        T, Hq, Hkv, dh, chunk = 8192, 40, 8, 128, 1024
        design = FlatDesign(pool_size=16, bucket_size=32, bucket_cap=64, cluster_block_size=512, top_p=8, top_k=300,
                            sink_size=4, window_size=512)
        rng = np.random.default_rng(0)
        w = bf16_round(rng.standard_normal((2, Hkv * dh, 64), dtype=np.float32) / np.sqrt(Hkv * dh))
        layer = FlatLayer(design, cuda(w[0], torch.bfloat16), cuda(w[1], torch.bfloat16), Hq, Hkv, dh)
        q, k, v = (cuda(a, torch.bfloat16) for a in layer_inputs(T, Hq, Hkv, dh, 32, 1))
        want = layer.prefill(q, k, v, chunk=chunk)
        sharded = ShardedFlatLayer(layer, rank, world)
        got = sharded.prefill(q, deal(k, rank, world).contiguous(), deal(v, rank, world).contiguous(), chunk=chunk)
        share = chunk // world
        mine = torch.cat([want[c * chunk + rank * share: c * chunk + (rank + 1) * share] for c in range(T // chunk)])
        err = (got.float() - mine.float()).abs()
        assert got.shape == mine.shape
        assert err.max().item() <= 2e-2 and err.mean().item() <= 2e-3, (err.max().item(), err.mean().item())
        # the query rows split over the ranks instead: the same rows from the gathered cache, all queries or its own
        for rows in (q, sharded.rows_of(q, chunk).contiguous()):
            split = sharded.prefill_by_rows(rows, deal(k, rank, world).contiguous(), deal(v, rank, world).contiguous(),
                                            T, chunk=chunk)
            err = (split.float() - mine.float()).abs()
            assert split.shape == mine.shape
            assert err.max().item() <= 2e-2 and err.mean().item() <= 2e-3, (err.max().item(), err.mean().item())
        # a decode step over the dealt cache: replicated rows, every rank returns the whole output
        k_share, v_share = deal(k, rank, world).contiguous(), deal(v, rank, world).contiguous()
        index = sharded.build_index(k_share, T)
        _, single = layer.prefill(q, k, v, chunk=chunk, return_index=True)
        rows = torch.tensor([5, 511, 512, 4000, T - 1], device="cuda")
        for splits in (1, 4):
            step = sharded.decode(q[rows], rows, k_share, v_share, index, splits=splits)
            alone = layer.decode(q[rows], rows, k, v, single, splits=splits)
            err = (step.float() - alone.float()).abs()
            assert step.shape == alone.shape and err.max().item() <= 2e-2, err.max().item()
        open(os.path.join(result_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def _latent_rank_main(rank, world, port, result_dir):
    for path in (ROOT, PACKAGE_DIR, os.path.join(ROOT, "tests")):
        if path not in sys.path:
            sys.path.insert(0, path)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from lsa_b200 import workloads as W
        from lsa_b200.latent import LatentLayer
        from lsa_b200.parallel import ShardedLatentLayer, deal

        # config 4's shape over 32 cluster blocks: every rank builds the whole cache and keeps its dealt share
        cfg = W.cut(W.C4, 32 * 5120)
        T, chunk, Hq, dk, dv = cfg["tokens"], 2048, cfg["heads"], cfg["latent_dim"], cfg["value_dim"]
        gen = torch.Generator(device="cuda").manual_seed(2)
        cache, tail = W.latent_cache(cfg, gen, keep_tail=chunk)
        qmap, kmap = W.latent_maps(cfg, gen)
        q = W.latent_queries(cfg, tail, gen)
        first = T - chunk
        single = LatentLayer(W.design_of(cfg), qmap, kmap, Hq, dk, dv, scale=W.latent_scale(cfg))
        index = single.build_index(cache)
        want = torch.empty(chunk, Hq, dv, dtype=torch.bfloat16, device="cuda")
        single.prefill_rows(q, first, cache, index, want)
        want1 = single.decode(q[-1:].contiguous(), torch.tensor([T - 1], device="cuda"), cache, index, splits=8)

        layer = LatentLayer(W.design_of(cfg), qmap, kmap, Hq, dk, dv, scale=W.latent_scale(cfg))
        sharded = ShardedLatentLayer(layer, rank, world)
        share = deal(cache, rank, world).contiguous()
        sharded.build_index(share, T)
        # the global member table is the single-GPU one; this rank's centroids are those of its own blocks
        assert torch.equal(sharded.members, index.buckets.bucket_members)
        per_block, blocks = 8, T // 5120
        mine = index.buckets.bucket_centroids.view(blocks // world, world, per_block, -1)[:, rank].reshape(-1, 64)
        assert torch.equal(sharded.centroids, mine)
        sharded.extend_index(share, first, chunk)  # the same keys again: the same index
        assert torch.equal(sharded.members, index.buckets.bucket_members) and torch.equal(sharded.centroids, mine)
        got = sharded.prefill_rows(q, first, share)
        rows = chunk // world
        err = (got.float() - want[rank * rows:(rank + 1) * rows].float()).abs()
        assert got.shape == (rows, Hq, dv)
        assert err.max().item() <= 2e-2 and err.mean().item() <= 2e-3, (err.max().item(), err.mean().item())
        got1 = sharded.decode(q[-1:].contiguous(), torch.tensor([T - 1], device="cuda"), share, splits=4)
        assert (got1.float() - want1.float()).abs().max().item() <= 2e-2
        # the same chunk from pinned host buffers, two pieces: this rank brings in and takes out its rows of each
        pieces, own = 2, chunk // 2 // world
        q_h = q.view(pieces, world, own, Hq, dk)[:, rank].reshape(pieces * own, Hq, dk).cpu().pin_memory()
        rows_h = share[first // world:].cpu().pin_memory()
        out_h = torch.empty(pieces * own, Hq, dv, dtype=torch.bfloat16).pin_memory()
        share[first // world:].zero_()
        sharded.prefill_from_host(q_h, rows_h, first, chunk, share, out_h, pieces=pieces)
        torch.cuda.synchronize()
        want_h = want.view(pieces, world, own, Hq, dv)[:, rank].reshape(pieces * own, Hq, dv)
        err = (out_h.cuda().float() - want_h.float()).abs()
        assert err.max().item() <= 2e-2 and err.mean().item() <= 2e-3, (err.max().item(), err.mean().item())
        assert torch.equal(share[first // world:].cpu(), rows_h)
        layer.check()
        open(os.path.join(result_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def test_sharded_latent_layer_matches_the_single_gpu_layer(tmp_path):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs two or more GPUs")
    mp.spawn(_latent_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert sorted(os.listdir(tmp_path)) == [f"ok{r}" for r in range(world)]


def test_sharded_prefill_matches_the_single_gpu_layer(tmp_path):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs two or more GPUs")
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert sorted(os.listdir(tmp_path)) == [f"ok{r}" for r in range(world)]
