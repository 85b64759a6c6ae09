"""The five benchmark configurations as seeded synthetic workloads: shapes, index parameters and input generators.

The reference times this path on real checkpoints, distilled map files and a tokenised book, none of which travel
with it; these generators take the shapes of its benchmark configurations and the value recipe of its own synthetic
roofline workload (clustered keys, queries = a key plus noise: src/lsa/evaluation/performance/roofline/workloads.py:
148-183) and stand in for them. The benchmark, the full-size parity tests and the profiling runs all draw from here,
so they time and check the same bits.
"""

from __future__ import annotations

import math

import numpy as np
import torch

from lsa_b200.layer import FlatDesign

# C1: the CPU-sized config - one GQA layer, 16,384 tokens, a 256 -> 32 PCA map, 256 buckets.
C1 = dict(workload="C1", tokens=16384, heads=8, kv_heads=2, head_dim=128, index_dim=32, pool_size=16, bucket_size=64,
          bucket_cap=128, cluster_block_size=512, top_p=16, top_k=2048, sink_size=4, window_size=512, chunk=4096,
          centres=64, sigma=0.3, query_noise=0.5, seed=0)
# C2: flat prefill of 128k tokens, 40 query heads over 8 KV heads.
C2 = dict(workload="C2", tokens=131072, heads=40, kv_heads=8, head_dim=128, index_dim=64, pool_size=16,
          bucket_size=32, bucket_cap=64, cluster_block_size=1024, top_p=64, top_k=4096, sink_size=4,
          window_size=1024, chunk=8192, centres=256, seed=0)
# C3: tree decode over a 1M-token cache: 65,536 buckets under 1,024 node buckets of 64.
C3 = dict(workload="C3", tokens=1 << 20, heads=40, kv_heads=8, head_dim=128, index_dim=64, pool_size=4, bucket_size=16,
          bucket_cap=32, cluster_block_size=1024, top_p=64, top_k=2048, sink_size=4, window_size=1024, centres=256,
          top_level=1, node_bucket_size=64, node_cluster_block_size=4096, beam_width=32, page_size=8192,
          growth_buckets=4096, seed=0)
# C4: the flat design over an MLA-style latent cache of 10M tokens: 64 heads, 512 + 64 dims, two-layer maps.
C4 = dict(workload="C4", tokens=10485760, heads=64, latent_dim=576, value_dim=512, index_dim=64, hidden_dim=2048,
          pool_size=64, bucket_size=640, bucket_cap=1280, cluster_block_size=5120, top_p=128, top_k=128 * 1280,
          sink_size=4, window_size=5120, chunk=8192, centres=256, seed=0)
# C5: batched serving decode: 64 requests of 32k-512k tokens over a paged KV pool (page 64) and a paged bucket cache.
C5 = dict(workload="C5", requests=64, min_len=32768, max_len=524288, heads=40, kv_heads=8, head_dim=128, index_dim=64,
          pool_size=16, bucket_size=256, bucket_cap=512, cluster_block_size=1024, top_p=32, top_k=16384, sink_size=4,
          window_size=1024, kv_page=64, page_buckets=32, centres=256, seed=0)

CONFIGS = {"C1": C1, "C2": C2, "C3": C3, "C4": C4, "C5": C5}


def cut(cfg: dict, tokens: int) -> dict:
    """The same workload over a shorter context (profiling, tests)."""
    out = dict(cfg)
    out["tokens"] = tokens
    return out


def design_of(cfg: dict) -> FlatDesign:
    return FlatDesign(pool_size=cfg["pool_size"], bucket_size=cfg["bucket_size"], bucket_cap=cfg["bucket_cap"],
                      cluster_block_size=cfg["cluster_block_size"], top_p=cfg["top_p"], top_k=cfg["top_k"],
                      sink_size=cfg["sink_size"], window_size=cfg["window_size"])


def gqa_inputs(cfg: dict, pin: bool = False):
    """Seeded q [T,Hq,dh], k, v [T,Hkv,dh] bf16 on the HOST and the two linear maps [Hkv*dh, index_dim] bf16: keys
    around `centres` centres, every query head = its key head plus noise (unit variance throughout)."""
    gen = torch.Generator().manual_seed(cfg["seed"])
    T, Hq, Hkv, dh = cfg["tokens"], cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    mu = torch.randn(cfg["centres"], Hkv, dh, generator=gen)
    label = torch.randint(0, cfg["centres"], (T,), generator=gen)
    half = 0.5 ** 0.5
    k = half * mu[label] + half * torch.randn(T, Hkv, dh, generator=gen)
    q = torch.empty(T, Hq, dh, dtype=torch.bfloat16)
    group = Hq // Hkv
    grouped = q.view(T, Hkv, group, dh)  # head h reads KV head h // group
    for g in range(group):  # one query head of every group at a time keeps the fp32 scratch small
        grouped[:, :, g] = (half * k + half * torch.randn(T, Hkv, dh, generator=gen)).bfloat16()
    v = torch.randn(T, Hkv, dh, generator=gen).bfloat16()
    k = k.bfloat16()
    d_in = Hkv * dh
    wq = (torch.randn(d_in, cfg["index_dim"], generator=gen) / d_in ** 0.5).bfloat16()
    wk = (torch.randn(d_in, cfg["index_dim"], generator=gen) / d_in ** 0.5).bfloat16()
    if pin:
        q, k, v = q.pin_memory(), k.pin_memory(), v.pin_memory()
    return q, k, v, wq, wk


def c1_inputs(cfg: dict = C1):
    """Config 1 on the host, fp32 values that are exact in bf16: keys = a centre + 0.3 N(0,1), queries = their key
    head + 0.5 N(0,1), values N(0,1), and the index map = the top right-singular vectors of the centred pooled keys
    (how the reference initialises a map: src/lsa/training/distillation/model.py:289-304)."""
    gen = torch.Generator().manual_seed(cfg["seed"])
    T, Hq, Hkv, dh = cfg["tokens"], cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    mu = torch.randn(cfg["centres"], Hkv, dh, generator=gen)
    label = torch.randint(0, cfg["centres"], (T,), generator=gen)
    k = (mu[label] + cfg["sigma"] * torch.randn(T, Hkv, dh, generator=gen)).bfloat16().float()
    q = (k.repeat_interleave(Hq // Hkv, dim=1) + cfg["query_noise"] * torch.randn(T, Hq, dh, generator=gen)
         ).bfloat16().float()
    v = torch.randn(T, Hkv, dh, generator=gen).bfloat16().float()
    pooled = k.reshape(T // cfg["pool_size"], cfg["pool_size"], Hkv * dh).mean(1)
    _, _, vt = torch.linalg.svd(pooled - pooled.mean(0, keepdim=True), full_matrices=False)
    index_map = vt[: cfg["index_dim"]].t().contiguous()
    return q, k, v, index_map


def clustered_cache(tokens: int, kv_heads: int, head_dim: int, centres: int, gen: torch.Generator,
                    chunk: int = 1 << 17):
    """K, V [tokens, Hkv, dh] bf16 built ON THE DEVICE a piece at a time (the long-context configs: a host copy of a
    1M-10M token cache would take longer to make than the benchmark to run)."""
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


def latent_cache(cfg: dict, gen: torch.Generator, world: int = 1, rank: int = 0, granule: int = 64,
                 keep_tail: int = 0):
    """The latent cache [tokens, latent_dim] bf16 on the device: a clustered value part (256 centres in 512 dims) and
    N(0,1) rope dims. Rows are generated in position order from one generator, a piece at a time; with `world` > 1
    only the granules dealt to `rank` are kept (every rank walks the same generator, so the shares are shares of
    ONE cache). Returns (cache or share, the last `keep_tail` rows in full)."""
    T, dk, dv = cfg["tokens"], cfg["latent_dim"], cfg["value_dim"]
    piece = min(1 << 18, T)
    if T % (granule * world) or keep_tail > min(piece, T % piece or piece):
        raise ValueError(f"{T} tokens do not deal out in granules of {granule} over {world} ranks")
    share = T // world
    tail = None
    cache = torch.empty(share, dk, dtype=torch.bfloat16, device="cuda")
    mu = torch.randn(cfg["centres"], dv, generator=gen, device="cuda")
    for start in range(0, T, piece):
        n = min(piece, T - start)
        label = torch.randint(0, cfg["centres"], (n,), generator=gen, device="cuda")
        rows = torch.empty(n, dk, dtype=torch.bfloat16, device="cuda")
        rows[:, :dv] = (0.7071 * mu[label] + 0.7071 * torch.randn(n, dv, generator=gen, device="cuda")).bfloat16()
        rows[:, dv:] = torch.randn(n, dk - dv, generator=gen, device="cuda").bfloat16()
        if world == 1:
            cache[start:start + n] = rows
        else:
            mine = rows.view(n // (granule * world), world, granule, dk)[:, rank].reshape(n // world, dk)
            cache[start // world:start // world + n // world] = mine
        if keep_tail and start + n == T:
            tail = rows[n - keep_tail:].clone()
    return cache, tail


def latent_maps(cfg: dict, gen: torch.Generator):
    """Random two-layer maps of config 4: ((w1_t, w2_t) for the queries, (w1_t, w2_t) for the keys), N(0, 1/fan_in)."""
    dk, hidden, d_idx = cfg["latent_dim"], cfg["hidden_dim"], cfg["index_dim"]
    w1 = [(torch.randn(hidden, dk, generator=gen, device="cuda") / dk ** 0.5).bfloat16() for _ in range(2)]
    w2 = [(torch.randn(d_idx, hidden, generator=gen, device="cuda") / hidden ** 0.5).bfloat16() for _ in range(2)]
    return (w1[0], w2[0]), (w1[1], w2[1])


def latent_queries(cfg: dict, own_rows: torch.Tensor, gen: torch.Generator) -> torch.Tensor:
    """Absorbed queries [n, heads, latent_dim] bf16 of tokens whose latent rows are `own_rows`: every head points at
    its own token's latent, plus noise."""
    n, dk = own_rows.shape
    return (0.7071 * own_rows[:, None, :].float() + 0.7071 * torch.randn(n, cfg["heads"], dk, generator=gen,
                                                                         device="cuda")).bfloat16().contiguous()


def latent_scale(cfg: dict) -> float:
    """(128 + 64)^-0.5 / 4: keeps the logits of unit-variance 576-dim vectors in a softmax's working range."""
    return (128 + 64) ** -0.5 / 4


def request_lengths(cfg: dict) -> np.ndarray:
    """Config 5's request lengths: log-uniform in [min_len, max_len], rounded down to whole cluster blocks."""
    rng = np.random.default_rng(cfg["seed"])
    raw = np.exp(rng.uniform(math.log(cfg["min_len"]), math.log(cfg["max_len"]), cfg["requests"]))
    return (raw // cfg["cluster_block_size"] * cfg["cluster_block_size"]).astype(np.int64)
