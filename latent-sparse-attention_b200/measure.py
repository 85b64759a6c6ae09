"""Measurements of the configurations the main benchmark does not time: the tree decode over a 1M-token cache, the
batched paged decode of 64 requests, and the flat design over an MLA-style latent cache. Each prints one JSON line (device time from CUDA events, the CPU oracle timed
beside it on a stated sample, and a parity check of the measured path against the oracle).

    python latent-sparse-attention_b200/measure.py tree-decode   [--tokens 1048576] [--steps 256]
    python latent-sparse-attention_b200/measure.py batched-decode [--requests 64] [--steps 64]
    python latent-sparse-attention_b200/measure.py latent-layer   [--tokens 10485760] [--chunk 8192] [--splits 148]
    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        latent-sparse-attention_b200/measure.py sharded-decode [--tokens 1048576] [--steps 256]

Inputs are seeded synthetic tensors with the shapes of the benchmark configurations.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
for _path in (HERE, os.path.dirname(HERE)):
    if _path not in sys.path:
        sys.path.insert(0, _path)

import numpy as np  # noqa: E402
import torch  # noqa: E402

from lsa_b200 import ops  # noqa: E402
from lsa_b200.layer import FlatDesign, FlatLayer  # noqa: E402


def clustered_cache(tokens: int, kv_heads: int, head_dim: int, centres: int, gen: torch.Generator, chunk: int = 1 << 17):
    """K, V [tokens, Hkv, dh] bf16 on the device, keys around `centres` centres, built in chunks."""
    k = torch.empty(tokens, kv_heads, head_dim, dtype=torch.bfloat16, device="cuda")
    v = torch.empty_like(k)
    mu = torch.randn(centres, kv_heads, head_dim, generator=gen, device="cuda")
    for start in range(0, tokens, chunk):
        n = min(chunk, tokens - start)
        label = torch.randint(0, centres, (n,), generator=gen, device="cuda")
        k[start:start + n] = (0.7071 * mu[label] + 0.7071 * torch.randn(n, kv_heads, head_dim, generator=gen,
                                                                        device="cuda")).bfloat16()
        v[start:start + n] = torch.randn(n, kv_heads, head_dim, generator=gen, device="cuda").bfloat16()
    return k, v


def timed_graph(step, warmup: int, steps: int) -> float:
    """Microseconds a step, the step captured in a CUDA graph and replayed (falls back to eager launches if capture
    is refused)."""
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    run = step
    try:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        run = graph.replay
    except Exception as failure:  # capture is an optimisation of the measurement, not of the result
        print(f"graph capture refused ({failure}); timing eager launches", file=sys.stderr)
    for _ in range(warmup):
        run()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(steps):
        run()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) * 1e3 / steps


def tree_decode(args) -> dict:
    """Config 3: one query a step over a 1M-token cache, a two-level tree of 64-child node buckets."""
    import oracle
    from lsa_b200.core import Buckets
    from lsa_b200.decode import TreeDecoder
    from lsa_b200.hierarchy import build_hierarchy

    gen = torch.Generator(device="cuda").manual_seed(0)
    T, Hq, Hkv, dh = args.tokens, 40, 8, 128
    design = FlatDesign(pool_size=4, bucket_size=16, bucket_cap=32, cluster_block_size=1024, top_p=64, top_k=2048,
                        sink_size=4, window_size=1024)
    k, v = clustered_cache(T, Hkv, dh, 256, gen)
    w = (torch.randn(2, Hkv * dh, 64, generator=gen, device="cuda") / (Hkv * dh) ** 0.5).bfloat16()
    layer = FlatLayer(design, w[0], w[1], Hq, Hkv, dh)
    t0 = time.perf_counter()
    index = layer.build_index(k)
    torch.cuda.synchronize()
    t_buckets = time.perf_counter() - t0
    t0 = time.perf_counter()
    tree = build_hierarchy(index.index_keys, index.buckets, 1, 64, 4096)
    torch.cuda.synchronize()
    t_tree = time.perf_counter() - t0
    position = T - 1
    decoder = TreeDecoder(layer, index.buckets, tree, 32, None, 8192, 4096, splits=args.splits)
    decoder.prepare(position)
    q = (0.7071 * k[position].repeat_interleave(Hq // Hkv, dim=0) + 0.7071 * torch.randn(
        Hq, dh, generator=gen, device="cuda").bfloat16())[None].contiguous()
    out = decoder.step(q, k, v)
    us = timed_graph(lambda: decoder.step(q, k, v), 5, args.steps)
    lists, lengths = decoder.select(q)
    from lsa_b200 import probe
    recorder = probe.CudaEventRecorder()
    probe.install(recorder)
    for _ in range(20):
        decoder.step(q, k, v)
    stages = {name: total * 1e3 / 20 for name, (total, _) in recorder.totals_ms().items()}
    probe.uninstall()

    # parity and the CPU baseline: the oracle reads the same step from the device's own index
    b = index.buckets
    buckets_np = oracle.Buckets(b.bucket_centroids.cpu().numpy(), b.bucket_members.cpu().numpy(),
                                b.bucket_sizes.cpu().numpy(), b.block_bucket_count, b.cluster_block_size)
    tree_np = oracle.Hierarchy([c.cpu().numpy() for c in tree.node_centroids], [c.cpu().numpy() for c in tree.children],
                               64, (4096,))
    index_q = layer.index_queries(q).cpu().numpy()
    kf, vf = None, None
    t0 = time.perf_counter()
    want_lists, want_len = oracle.read_hierarchy(index_q, np.array([position]), buckets_np, tree_np, 32, None, 64,
                                                 2048, 4, 1024, 8192, 4096)
    t_read = time.perf_counter() - t0
    same = bool(np.array_equal(lists.cpu().numpy(), want_lists) and int(lengths[0]) == int(want_len[0]))
    ids = want_lists[0, : want_len[0]]
    # gather the listed rows so the oracle need not hold a 2 GB fp32 copy of the cache
    rows = torch.from_numpy(np.sort(ids)).cuda().long()
    remap = {int(p): i for i, p in enumerate(np.sort(ids))}
    local = np.array([[remap[int(p)] for p in ids]], dtype=np.int32)
    kf, vf = k[rows].float().cpu().numpy(), v[rows].float().cpu().numpy()
    t0 = time.perf_counter()
    want, _ = oracle.sparse_attend(q.float().cpu().numpy(), kf, vf, local, np.array([len(ids)]), 0, 0, dh ** -0.5)
    t_attend = time.perf_counter() - t0
    err = float(np.abs(out.float().cpu().numpy() - want).max())
    node_bytes = (960 + 32 * 64 + (int(want_len[0]) and 4032)) * 64 * 4
    kv_bytes = int(want_len[0]) * Hkv * dh * 2 * 2
    return {"metric": "tree decode us/step", "value": us, "unit": "us", "higher_is_better": False, "n_gpus": 1,
            "config": {"workload": "C3", "tokens": T, "buckets": int(b.bucket_sizes.shape[0]),
                       "nodes": int(tree.children[0].shape[0]), "beam": 32, "top_p": 64, "list": int(want_len[0]),
                       "splits": args.splits},
            "build": {"buckets_s": t_buckets, "tree_s": t_tree}, "stages_us_eager": stages,
            "parity": {"lists_equal": same, "attention_max_abs": err},
            "algorithmic_bytes_per_step": node_bytes + kv_bytes,
            "hbm_floor_us": (node_bytes + kv_bytes) / 6536.4e3,
            "cpu_baseline": {"value": (t_read + t_attend) * 1e6, "unit": "us", "kind": "port",
                             "cores": len(os.sched_getaffinity(0)), "sample": "one step: tree read + attend"}}


def batched_decode(args) -> dict:
    """Config 5: one decode step of 64 requests of 32k-512k tokens over a paged bf16 KV pool (page 64) and a paged
    bucket cache, flat design."""
    import oracle
    from lsa_b200.serving import BucketCache, Selector

    gen = torch.Generator(device="cuda").manual_seed(0)
    rng = np.random.default_rng(0)
    B, Hq, Hkv, dh, kv_page = args.requests, 40, 8, 128, 64
    design = FlatDesign(pool_size=16, bucket_size=256, bucket_cap=512, cluster_block_size=1024, top_p=32, top_k=16384,
                        sink_size=4, window_size=1024)
    lengths = (np.exp(rng.uniform(math.log(args.min_len), math.log(args.max_len), B)) // 1024 * 1024).astype(np.int64)
    total = int(lengths.sum())
    pool_pages = total // kv_page + B
    k, v = clustered_cache(pool_pages * kv_page, Hkv, dh, 256, gen)
    w = (torch.randn(2, Hkv * dh, 64, generator=gen, device="cuda") / (Hkv * dh) ** 0.5).bfloat16()
    layer = FlatLayer(design, w[0], w[1], Hq, Hkv, dh)
    # KV pages dealt to the requests in a shuffled order; a request's position p is slot pages[p / 64] * 64 + p % 64
    order = torch.from_numpy(rng.permutation(pool_pages).astype(np.int32)).cuda()
    max_kv_pages = int(lengths.max()) // kv_page
    kv_pages = torch.full((B, max_kv_pages), -1, dtype=torch.int32, device="cuda")
    page_buckets = 32  # buckets of 8,192 keys a page of the bucket cache
    cache = BucketCache(design, 64, pages=total // 8192 + 2 * B, page_buckets=page_buckets, max_requests=B,
                        max_request_pages=int(lengths.max()) // 8192 + 1)
    taken = 0
    t0 = time.perf_counter()
    for r, n in enumerate(lengths.tolist()):
        count = n // kv_page
        kv_pages[r, :count] = order[taken:taken + count]
        taken += count
        slots = (kv_pages[r, :count].long()[:, None] * kv_page + torch.arange(kv_page, device="cuda")[None]).reshape(-1)
        for start in range(0, n, 1 << 17):  # index keys of the request, in position order, a piece at a time
            piece = slots[start:start + (1 << 17)]
            cache.append(r, layer.index_keys(k[piece]))
    torch.cuda.synchronize()
    t_build = time.perf_counter() - t0
    selector = Selector(cache, kv_page)
    rows = torch.arange(B, device="cuda")
    positions = torch.from_numpy(lengths - 1).cuda()
    last_slot = kv_pages[rows, (positions // kv_page)].long() * kv_page + positions % kv_page
    q = (0.7071 * k[last_slot].repeat_interleave(Hq // Hkv, dim=1) + 0.7071 * torch.randn(
        B, Hq, dh, generator=gen, device="cuda")).bfloat16().contiguous()
    visible = selector.visible(rows, positions)

    def step():
        lists, lens = selector.decode_flat(layer.index_queries(q), rows, positions, kv_pages, visible=visible,
                                           splits=args.select_splits)
        return ops.sparse_attend(q, k, v, lists, lens, layer.scale, splits=args.splits)[0], lists, lens

    out, lists, lens = step()
    us = timed_graph(lambda: step(), 3, args.steps)

    # parity on a few requests, the oracle reading each from the device's own index vectors
    index_q = layer.index_queries(q).cpu().numpy()
    checked, worst, t_cpu = 0, 0.0, 0.0
    for r in rng.choice(B, min(B, args.check), replace=False).tolist():
        n = int(lengths[r])
        slots = (kv_pages[r, : n // kv_page].long()[:, None] * kv_page + torch.arange(kv_page, device="cuda")[None]).reshape(-1)
        index_k = torch.cat([layer.index_keys(k[slots[s:s + (1 << 17)]]) for s in range(0, n, 1 << 17)]).cpu().numpy()
        t0 = time.perf_counter()
        buckets = oracle.build_buckets(index_k, 16, 256, 512, 1024)
        t_index = time.perf_counter() - t0
        t0 = time.perf_counter()
        want, want_len = oracle.read(index_q[r:r + 1], np.array([n - 1]), buckets, 32, 16384, 4, 1024)
        ids = want[0, : want_len[0]]
        mine = lists[r, : int(lens[r])].cpu().numpy()
        want_slots = slots[torch.from_numpy(ids.astype(np.int64)).cuda()].cpu().numpy()
        assert int(lens[r]) == int(want_len[0]) and np.array_equal(mine, want_slots), f"request {r}: lists differ"
        gathered = torch.from_numpy(want_slots).cuda().long()
        ref, _ = oracle.sparse_attend(q[r:r + 1].float().cpu().numpy(), k[gathered].float().cpu().numpy(),
                                      v[gathered].float().cpu().numpy(), np.arange(len(ids), dtype=np.int32)[None],
                                      np.array([len(ids)]), 0, 0, dh ** -0.5)
        t_cpu += time.perf_counter() - t0
        worst = max(worst, float(np.abs(out[r].float().cpu().numpy() - ref[0]).max()))
        checked += 1
        del t_index
    listed = int(lens.sum())
    centroid_bytes = int(visible.sum()) * 64 * 4
    kv_bytes = listed * Hkv * dh * 2 * 2
    return {"metric": "batched decode steps/s", "value": 1e6 / us, "unit": "steps/s", "us_per_step": us,
            "higher_is_better": True, "n_gpus": 1,
            "config": {"workload": "C5", "requests": B, "tokens_total": total, "min_len": int(lengths.min()),
                       "max_len": int(lengths.max()), "kv_page": kv_page, "top_p": 32, "listed_keys": listed,
                       "splits": args.splits, "select_splits": args.select_splits},
            "build": {"index_s": t_build},
            "parity": {"requests_checked": checked, "lists_equal": True, "attention_max_abs": worst},
            "algorithmic_bytes_per_step": centroid_bytes + kv_bytes,
            "hbm_floor_us": (centroid_bytes + kv_bytes) / 6536.4e3,
            "cpu_baseline": {"value": 1.0 / (t_cpu / max(checked, 1) * B), "unit": "steps/s", "kind": "port",
                             "cores": len(os.sched_getaffinity(0)),
                             "sample": f"read + attend of {checked} requests, scaled to {B}"}}


def latent_layer(args) -> dict:
    """Config 4: the flat design over an MLA-style layer - 64 query heads over a shared latent of 512 + 64 rope dims,
    two-layer maps 576 -> 2048 -> 64, keys pooled by 64 into buckets of 640 (cap 1,280, 8 a cluster block), the top
    128 buckets plus 4 sinks and a 5,120-key window; one prefill chunk of 8,192 queries at the end of the context,
    then decode steps at the last position."""
    import oracle
    from lsa_b200 import core

    gen = torch.Generator(device="cuda").manual_seed(0)
    T, Hq, dk, dv, d_idx, hidden_dim = args.tokens, 64, 576, 512, 64, 2048
    chunk = min(args.chunk, T)
    top_p, cap = 128, 1280
    top_k = top_p * cap
    sink, window = 4, 5120
    # the latent cache: a clustered 512-dim part (256 centres) and N(0,1) rope dims, built a piece at a time
    cache = torch.empty(T, dk, dtype=torch.bfloat16, device="cuda")
    mu = torch.randn(256, dv, generator=gen, device="cuda")
    for start in range(0, T, 1 << 18):
        n = min(1 << 18, T - start)
        label = torch.randint(0, 256, (n,), generator=gen, device="cuda")
        cache[start:start + n, :dv] = (0.7071 * mu[label] + 0.7071 * torch.randn(n, dv, generator=gen,
                                                                                 device="cuda")).bfloat16()
        cache[start:start + n, dv:] = torch.randn(n, dk - dv, generator=gen, device="cuda").bfloat16()
    w1 = [(torch.randn(hidden_dim, dk, generator=gen, device="cuda") / dk ** 0.5).bfloat16() for _ in range(2)]
    w2 = [(torch.randn(d_idx, hidden_dim, generator=gen, device="cuda") / hidden_dim ** 0.5).bfloat16() for _ in range(2)]
    # absorbed queries of the chunk: every head points at its token's latent, plus noise
    positions = torch.arange(T - chunk, T, device="cuda")
    q = (0.7071 * cache[T - chunk:, None, :].float() + 0.7071 * torch.randn(chunk, Hq, dk, generator=gen,
                                                                            device="cuda")).bfloat16().contiguous()
    scale = (128 + 64) ** -0.5 / 4  # keeps the logits of unit-variance 576-dim vectors in a softmax's working range

    start_ev, stop_ev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed(fn):
        torch.cuda.synchronize()
        start_ev.record()
        result = fn()
        stop_ev.record()
        torch.cuda.synchronize()
        return result, start_ev.elapsed_time(stop_ev)

    def key_map():
        index_keys = torch.empty(T, d_idx, dtype=torch.float32, device="cuda")
        piece = 1 << 19
        hidden = torch.empty(min(piece, T), hidden_dim, dtype=torch.bfloat16, device="cuda")
        for start in range(0, T, piece):
            n = min(piece, T - start)
            ops.mlp_map(cache[start:start + n], w1[1], w2[1], hidden=hidden[:n], out=index_keys[start:start + n])
        return index_keys

    def query_map(rows):
        summed = ops.index_map(rows, None, group=Hq, normalize=False, out_dtype=torch.bfloat16)
        return ops.mlp_map(summed, w1[0], w2[0])

    index_keys, ms_key_map = timed(key_map)
    buckets, ms_buckets = timed(lambda: core.build_buckets(index_keys, 64, 640, cap, 5120))

    def prefill():
        index_q = query_map(q)
        lists, lens = core.read(index_q, positions, buckets, top_p, top_k, sink, window)
        out, _ = ops.latent_attend(q, cache, lists, lens, scale)
        return index_q, lists, lens, out

    prefill()  # warm-up
    (index_q, lists, lens, out), ms_prefill = timed(prefill)
    _, ms_attend = timed(lambda: ops.latent_attend(q, cache, lists, lens, scale))

    # decode at the last position
    q1, pos1 = q[-1:].contiguous(), positions[-1:]
    visible1 = torch.full((1,), (T - 1) // 5120 * 8, dtype=torch.int32, device="cuda")

    from lsa_b200 import probe

    def decode():
        with probe.region("index map"):
            index_q1 = query_map(q1)
        with probe.region("select"):
            _, picked = ops.flat_select_decode(index_q1, buckets.bucket_centroids, None, visible1, top_p,
                                               splits=args.select_splits)
        with probe.region("expand"):
            l1, n1, _ = ops.expand(picked, pos1, buckets.bucket_members, top_k, sink, window)
        with probe.region("attend"):
            return ops.latent_attend(q1, cache, l1, n1, scale, splits=args.splits)[0], l1, n1

    out1, l1, n1 = decode()
    us_decode = timed_graph(lambda: decode(), 3, args.steps)
    recorder = probe.CudaEventRecorder()
    probe.install(recorder)
    for _ in range(20):
        decode()
    decode_stages = {name: total * 1e3 / 20 for name, (total, _) in recorder.totals_ms().items()}
    probe.uninstall()

    # parity on sample rows of the chunk and the decode row, the oracle reading the device's own index vectors
    b_np = oracle.Buckets(buckets.bucket_centroids.cpu().numpy(), buckets.bucket_members.cpu().numpy(),
                          buckets.bucket_sizes.cpu().numpy(), buckets.block_bucket_count, buckets.cluster_block_size)
    rows = sorted({0, chunk - 1} | set(np.random.default_rng(0).choice(chunk, min(args.check, chunk), replace=False).tolist()))
    iq_np, pos_np = index_q.cpu().numpy(), positions.cpu().numpy()
    t0 = time.perf_counter()
    want_lists, want_lens = oracle.read(iq_np[rows], pos_np[rows], b_np, top_p, top_k, sink, window)
    t_read = time.perf_counter() - t0
    same = all(int(lens[r]) == int(want_lens[i]) and np.array_equal(lists[r, : int(lens[r])].cpu().numpy(),
                                                                  want_lists[i, : want_lens[i]])
               for i, r in enumerate(rows))
    same = same and np.array_equal(l1[0, : int(n1[0])].cpu().numpy(), want_lists[-1, : want_lens[-1]])
    worst, t_attend = 0.0, 0.0
    for i, r in list(enumerate(rows))[-2:]:
        ids = np.sort(want_lists[i, : want_lens[i]])
        gathered = cache[torch.from_numpy(ids.astype(np.int64)).cuda()].float().cpu().numpy()
        t0 = time.perf_counter()
        ref, _ = oracle.sparse_attend(q[r:r + 1].float().cpu().numpy(), gathered[:, None, :], gathered[:, None, :],
                                      np.arange(len(ids), dtype=np.int32)[None], np.array([len(ids)]), 0, 0, scale)
        t_attend += time.perf_counter() - t0
        worst = max(worst, float(np.abs(out[r].float().cpu().numpy() - ref[0, :, :dv]).max()))
        if r == chunk - 1:
            worst = max(worst, float(np.abs(out1[0].float().cpu().numpy() - ref[0, :, :dv]).max()))
    gathered_total = int(lens.sum())
    flops = 2.0 * gathered_total * Hq * (dk + dv)
    cpu_row_s = t_read / len(rows) + t_attend / 2
    return {"metric": "MLA flat prefill tokens/s", "value": chunk / (ms_prefill * 1e-3), "unit": "tokens/s",
            "higher_is_better": True, "n_gpus": 1, "decode_us_per_step": us_decode,
            "config": {"workload": "C4", "tokens": T, "chunk": chunk, "heads": Hq, "latent": dk, "value_dim": dv,
                       "buckets": int(buckets.bucket_sizes.shape[0]), "top_p": top_p, "window": window,
                       "keys_listed_per_row": gathered_total / chunk, "decode_splits": args.splits},
            "build_ms": {"key_map": ms_key_map, "buckets": ms_buckets},
            "stages_ms": {"prefill_chunk": ms_prefill, "attend": ms_attend}, "decode_stages_us_eager": decode_stages,
            "attend": {"tflops": flops / (ms_attend * 1e-3) / 1e12, "gathered_GBps": gathered_total * dk * 2 / (
                ms_attend * 1e-3) / 1e9},
            "parity": {"rows_checked": len(rows), "lists_equal": bool(same), "attention_max_abs": worst},
            "hbm_floor_decode_us": (int(n1[0]) * dk * 2 + int(visible1[0]) * d_idx * 4) / 6536.4e3,
            "cpu_baseline": {"value": 1.0 / cpu_row_s, "unit": "tokens/s", "kind": "port",
                             "cores": len(os.sched_getaffinity(0)),
                             "sample": f"read of {len(rows)} rows and attend of 2 rows, per-row times summed"}}


def sharded_decode(args) -> dict:
    """One decode row of the flat design (config 2's index parameters) over a cache dealt across the ranks of a
    torchrun launch (`ShardedFlatLayer.decode`: every rank scores the centroids of its blocks, the candidates are
    all-gathered and cut, each rank reads the keys it stores, the partial outputs merge with one all-reduce).
    Eager launches (the step holds NCCL calls), device time from CUDA events, max over ranks; at one rank the
    single-GPU step is timed beside it and the outputs are compared."""
    import torch.distributed as dist

    from lsa_b200.parallel import ShardedFlatLayer, deal

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    heads, kv_heads, dh = 40, 8, 128
    design = FlatDesign(pool_size=16, bucket_size=32, bucket_cap=64, cluster_block_size=1024, top_p=64, top_k=4096,
                        sink_size=4, window_size=1024)
    gen = torch.Generator(device="cuda").manual_seed(0)
    k, v = clustered_cache(args.tokens, kv_heads, dh, 256, gen)
    maps = torch.randn(2, kv_heads * dh, 64, generator=gen, device="cuda") / math.sqrt(kv_heads * dh)
    layer = FlatLayer(design, maps[0].bfloat16(), maps[1].bfloat16(), heads, kv_heads, dh)
    sharded = ShardedFlatLayer(layer, rank, world)
    k_share, v_share = deal(k, rank, world).contiguous(), deal(v, rank, world).contiguous()
    index = sharded.build_index(k_share, args.tokens)
    position = torch.tensor([args.tokens - 1], device="cuda")
    q = (k[-1:].repeat_interleave(heads // kv_heads, dim=1).float() +
         0.5 * torch.randn(1, heads, dh, generator=gen, device="cuda")).bfloat16()
    single = layer.build_index(k) if world == 1 else None
    del k, v

    def timed(step) -> float:
        for _ in range(8):
            step()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dist.barrier()
        torch.cuda.synchronize()
        start.record()
        for _ in range(args.steps):
            step()
        stop.record()
        torch.cuda.synchronize()
        us = torch.tensor([start.elapsed_time(stop) * 1e3 / args.steps], device="cuda")
        dist.all_reduce(us, op=dist.ReduceOp.MAX)
        return float(us)

    us = timed(lambda: sharded.decode(q, position, k_share, v_share, index, splits=args.splits))
    result = {"metric": "flat decode us/step over a dealt cache", "value": us, "unit": "us", "n_gpus": world,
              "steps": args.steps, "config": {"workload": "C2 index parameters, one row at the end of the context",
                                              "tokens": args.tokens, "splits": args.splits}}
    if world == 1:
        out = sharded.decode(q, position, k_share, v_share, index, splits=args.splits)
        alone = layer.decode(q, position, k_share, v_share, single, splits=args.splits)
        result["single_gpu_us"] = timed(lambda: layer.decode(q, position, k_share, v_share, single, splits=args.splits))
        result["gap_to_single_gpu_step"] = float((out.float() - alone.float()).abs().max())
    dist.destroy_process_group()
    return result if rank == 0 else {}


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("what", choices=["tree-decode", "batched-decode", "latent-layer", "sharded-decode"])
    parser.add_argument("--chunk", type=int, default=8192)
    parser.add_argument("--tokens", type=int, default=1 << 20)
    parser.add_argument("--steps", type=int, default=256)
    parser.add_argument("--splits", type=int, default=16)
    parser.add_argument("--select-splits", type=int, default=4)
    parser.add_argument("--requests", type=int, default=64)
    parser.add_argument("--min-len", type=int, default=32768)
    parser.add_argument("--max-len", type=int, default=524288)
    parser.add_argument("--check", type=int, default=4)
    args = parser.parse_args()
    if args.what == "sharded-decode":  # under torchrun, one rank a GPU
        result = sharded_decode(args)
        if result:
            print(json.dumps(result))
        return
    torch.cuda.set_device(0)
    result = {"tree-decode": tree_decode, "batched-decode": batched_decode, "latent-layer": latent_layer}[args.what](args)
    print(json.dumps(result))


if __name__ == "__main__":
    main()
