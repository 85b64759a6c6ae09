"""Generate the golden vectors under tests/golden/ by running the reference's own `lsa.core` on seeded inputs.

Run where the reference is mounted (it is imported in place, never copied):

    python tests/golden/make_golden.py <checkout of the reference>/src

Each `.npz` holds the inputs and what the reference returned for them, so the tests need neither the reference
nor torch's random streams. The constructions follow the reference's own unit tests
(tests/unit/core/test_ward.py, test_reference.py, test_hierarchy.py, test_attention.py, test_index_space.py).
"""

import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))


def unit(count, dim, seed):
    gen = torch.Generator().manual_seed(seed)
    return F.normalize(torch.randn(count, dim, generator=gen), dim=-1)


def clustered(count, dim, centres, sigma, seed):
    gen = torch.Generator().manual_seed(seed)
    mu = torch.randn(centres, dim, generator=gen)
    label = torch.randint(0, centres, (count,), generator=gen)
    return mu[label] + sigma * torch.randn(count, dim, generator=gen)


def save(name, **arrays):
    out = {}
    for key, value in arrays.items():
        if isinstance(value, torch.Tensor):
            value = value.numpy()
        out[key] = np.asarray(value)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    print(name, {k: v.shape for k, v in out.items()})


def main(src):
    sys.path.insert(0, src)
    from lsa.budget import EarlyBudget
    from lsa.core import (build_buckets, build_hierarchy, project, read, read_hierarchy_counted, regroup,
                          topk_attention)
    from lsa.core.hierarchy import growth_at
    from lsa.core.kernels.triton.keys import pack_keys, unpack_ids, unpack_scores
    from lsa.core.ward import members_from_labels, pool_keys, ward_merge, ward_rounds

    torch.set_num_threads(1)

    # ---- index space: regroup and project (tests/unit/core/test_index_space.py)
    gen = torch.Generator().manual_seed(0)
    q = torch.randn(1, 8, 40, 32, generator=gen)
    k = torch.randn(1, 2, 40, 32, generator=gen)
    k[0, :, 7] = 0  # a zero key row stays zero
    iq, ik = regroup(q, k)
    w = torch.randn(64, 16, generator=gen) / 8
    save("index_space", q=q[0].transpose(0, 1), k=k[0].transpose(0, 1), index_queries=iq[0], index_keys=ik[0],
         w=w, projected_queries=project(iq[0], w), projected_keys=project(ik[0], w))

    # ---- the MLA index space: latent keys under the metric their key maps impose (test_index_space.py:169-232)
    from lsa.core import LatentMetric, regroup_latent
    gen = torch.Generator().manual_seed(4)
    ql = torch.randn(1, 8, 40, 16, generator=gen)
    latent = torch.randn(1, 40, 12, generator=gen)
    latent[0, 5] = 0
    key_maps = torch.randn(8, 16, 12, generator=gen) / 4
    metric = LatentMetric.from_key_maps(key_maps)
    lq, lk = regroup_latent(ql, latent, metric)
    wide_q, wide_k = regroup(ql, torch.einsum("btr,hdr->bhtd", latent, key_maps))
    save("latent_space", q=ql[0].transpose(0, 1), latent=latent[0], key_maps=key_maps,
         metric_factor=metric.metric_factor, index_queries=lq[0], index_keys=lk[0],
         wide_scores=wide_q[0] @ wide_k[0].T)

    # ---- packed keys (src/lsa/core/kernels/triton/keys.py)
    scores = torch.tensor([0.0, -0.0, 1.5, -1.5, 1e-30, -1e-30, 3.0e38, -3.0e38, 0.25, 0.25])
    ids = torch.tensor([0, 1, 2, 3, 4, 5, 6, 7, 9, 8], dtype=torch.int32)
    keys = pack_keys(scores, ids)
    save("packed_keys", scores=scores, ids=ids, keys=keys, unpacked_ids=unpack_ids(keys),
         unpacked_scores=unpack_scores(keys))

    # ---- Ward (tests/unit/core/test_ward.py)
    ward = {}
    for tag, (blocks, pools, dim, pool, count, cap, seed) in {
        "a": (3, 64, 16, 4, 32, 16, 0),
        "b": (4, 32, 16, 4, 16, 16, 3),
        "c": (2, 64, 64, 16, 32, 64, 5),
        "d": (2, 256, 64, 4, 64, 32, 6),
        "e": (2, 80, 64, 8, 8, 160, 7),
    }.items():
        keys_ = unit(blocks * pools * pool, dim, seed).view(blocks, pools * pool, dim)
        sums = pool_keys(keys_, pool)
        sizes = torch.full((blocks, pools), float(pool))
        labels = ward_merge(sums, sizes, count, cap)
        ward.update({f"{tag}_pools": sums, f"{tag}_labels": labels, f"{tag}_args": np.array([pool, count, cap])})
        if tag == "c":
            ward["c_keys"] = keys_
    # near-copied and rounded pools, the reference's own adversarial constructions (test_ward.py:98-110)
    for tag, seed in (("near", 1), ("rounded", 2)):
        keys_ = unit(8 * 128 * 4, 16, seed).view(8, 512, 16)
        sums = pool_keys(keys_, 4)
        sums = sums[:, :1].expand_as(sums) + 1e-3 * sums if tag == "near" else sums.round()
        labels, reached = ward_rounds(sums.contiguous(), torch.full((8, 128), 4.0), 64, 16)
        ward.update({f"{tag}_pools": sums, f"{tag}_labels": labels, f"{tag}_reached": reached,
                     f"{tag}_args": np.array([4, 64, 16])})
    # pairings at a cap of two, as the hierarchy uses the merge (hierarchy.py:92)
    sums = unit(2 * 64, 16, 9).view(2, 64, 16) * 3
    labels, reached = ward_rounds(sums, torch.ones(2, 64), 32, 2)
    ward.update({"pair_pools": sums, "pair_labels": labels, "pair_reached": reached})
    base = F.normalize(torch.randn(4, 8, generator=torch.Generator().manual_seed(1)), dim=-1)
    near = F.normalize(base[0] + 0.01 * base[1], dim=-1)
    tight = torch.stack([base[0], near, base[2], base[3]])[None] * 4
    ward.update({"tight_pools": tight, "tight_labels": ward_merge(tight, torch.full((1, 4), 4.0), 3, 16)})
    same = (torch.eye(8)[:1].expand(1, 4, 8) * 4).contiguous()
    ward.update({"same_pools": same, "same_labels": ward_merge(same, torch.full((1, 4), 4.0), 2, 16)})
    ward["members"] = members_from_labels(torch.tensor([1, 0, 1, 2, 0, 1]), 3, 4)
    save("ward", **ward)

    # ---- flat: build_buckets and read (tests/unit/core/test_reference.py fixture, and a 64-dim case)
    keys_ = unit(4 * 64 + 20, 16, 0)
    buckets = build_buckets(keys_, 4, 8, 16, 64)
    positions = torch.tensor([0, 3, 63, 64, 65, 127, 128, 191, 200, 255, 256, 270, 275])
    queries = F.normalize(keys_[positions.clamp_max(len(keys_) - 1)] + 0.3 * unit(len(positions), 16, 1), dim=-1)
    sel, lens = read(queries, positions, buckets, 8, 48, 4, 64)
    sel_small, lens_small = read(queries, positions, buckets, 3, 20, 4, 16)
    early = EarlyBudget(position=200, top_k=12, top_p=2)
    sel_early, lens_early = read(queries, positions, buckets, 8, 48, 4, 64, early_budget=early)
    save("flat_small", keys=keys_, centroids=buckets.bucket_centroids, members=buckets.bucket_members,
         sizes=buckets.bucket_sizes, positions=positions, queries=queries, selected=sel, lengths=lens,
         selected_small=sel_small, lengths_small=lens_small, selected_early=sel_early, lengths_early=lens_early)

    raw = clustered(4096 + 100, 64, 24, 0.3, 11)
    keys_ = F.normalize(raw, dim=-1)
    buckets = build_buckets(keys_, 16, 64, 128, 512)
    gen = torch.Generator().manual_seed(12)
    positions = torch.randint(0, len(keys_), (96,), generator=gen).sort().values
    queries = F.normalize(raw[positions] + 0.5 * torch.randn(96, 64, generator=gen), dim=-1)
    sel, lens = read(queries, positions, buckets, 16, 2048, 4, 512)
    sel_cut, lens_cut = read(queries, positions, buckets, 16, 700, 4, 512)
    scores = queries @ buckets.bucket_centroids.T
    save("flat_c1like", keys=keys_, centroids=buckets.bucket_centroids, members=buckets.bucket_members,
         sizes=buckets.bucket_sizes, positions=positions, queries=queries, selected=sel, lengths=lens,
         selected_cut=sel_cut, lengths_cut=lens_cut, scores=scores)

    # ---- hierarchy (tests/unit/core/test_hierarchy.py store)
    gen = torch.Generator().manual_seed(0)
    count = 8192
    anchors = torch.randn(count // 12 + 1, 16, generator=gen)
    keys_ = F.normalize(anchors[torch.arange(count) // 12] + 0.5 * torch.randn(count, 16, generator=gen), dim=-1)
    buckets = build_buckets(keys_, 4, 8, 16, 64)
    hierarchy = build_hierarchy(keys_, buckets, 16, 4, 16)
    positions = torch.tensor([100, 511, 512, 1023, 1024, 2047, 2048, 3000, 4095, 4096, 5000, 6143, 7000, 8191])
    gen = torch.Generator().manual_seed(1)
    earlier = (torch.rand(len(positions), generator=gen) * positions).long()
    queries = F.normalize(keys_[earlier] + 0.1 * torch.randn(len(positions), 16, generator=gen), dim=-1)
    tree = {"keys": keys_, "centroids": buckets.bucket_centroids, "members": buckets.bucket_members,
            "positions": positions, "queries": queries, "levels": np.array(len(hierarchy.children)),
            "block_sizes": np.array(hierarchy.node_cluster_block_sizes)}
    for level, (cent, kids) in enumerate(zip(hierarchy.node_centroids, hierarchy.children)):
        tree[f"node_centroids_{level}"] = cent
        tree[f"children_{level}"] = kids
    for tag, (beam, start, growth) in {"wide": (4096, None, 0), "narrow": (2, None, 0), "start": (3, 8, 0),
                                        "wait": (2, None, 64)}.items():
        sel, lens, scored = read_hierarchy_counted(queries, positions, buckets, hierarchy, beam, start, 16, 64, 4,
                                                   64, 512, growth)
        tree.update({f"selected_{tag}": sel, f"lengths_{tag}": lens, f"scored_{tag}": scored})
    grown = [growth_at(hierarchy, closed, 64, g) for closed in (0, 64, 128, 512, 1024) for g in (0, 64, 100)]
    tree["growth"] = np.array([[g.covered_buckets, *g.made, *g.closed] for g in grown])
    save("hierarchy", **tree)

    # ---- attention (tests/unit/core/test_attention.py)
    gen = torch.Generator().manual_seed(0)
    T, Hq, Hkv, dh = 96, 8, 2, 16
    q = torch.randn(1, T, Hq, dh, generator=gen)
    k = torch.randn(1, T, Hkv, dh, generator=gen)
    v = torch.randn(1, T, Hkv, dh, generator=gen)
    sel = torch.full((1, T, 12), -1, dtype=torch.int32)
    for row in range(T):
        pick = torch.randperm(T, generator=gen)[:9]
        sel[0, row, : len(pick)] = pick.to(torch.int32)  # some are in the future: causality drops them
    out = topk_attention(q, k, v, sel, window=8, sink=2, scale=dh**-0.5)
    full = torch.arange(T, dtype=torch.int32).expand(1, T, T).contiguous()
    dense = topk_attention(q, k, v, full, window=0, sink=0, scale=dh**-0.5)
    save("attention", q=q[0], k=k[0], v=v[0], selected=sel[0], out=out[0], dense=dense[0])

    # ---- a miniature of config 1 end to end: map, buckets, read, attend
    gen = torch.Generator().manual_seed(21)
    T, Hq, Hkv, dh = 1024, 8, 2, 64
    mu = torch.randn(16, Hkv, dh, generator=gen)
    label = torch.randint(0, 16, (T,), generator=gen)
    kk = mu[label] + 0.3 * torch.randn(T, Hkv, dh, generator=gen)
    qq = kk.repeat_interleave(Hq // Hkv, dim=1) + 0.5 * torch.randn(T, Hq, dh, generator=gen)
    vv = torch.randn(T, Hkv, dh, generator=gen)
    kk, qq, vv = (t.bfloat16().float() for t in (kk, qq, vv))
    iq, ik = regroup(qq.transpose(0, 1)[None], kk.transpose(0, 1)[None])
    w = (torch.randn(Hkv * dh, 32, generator=gen) / (Hkv * dh) ** 0.5).bfloat16().float()
    index_q, index_k = project(iq[0], w), project(ik[0], w)
    buckets = build_buckets(index_k, 4, 16, 32, 128)
    positions = torch.arange(T)
    sel, lens = read(index_q, positions, buckets, 8, 256, 4, 128)
    out = topk_attention(qq[None], kk[None], vv[None], sel[None], window=128, sink=4, scale=dh**-0.5)
    # q, k, v hold bf16 values: stored as their 16-bit patterns; the output is kept for every fourth row
    bits = lambda t: t.bfloat16().view(torch.int16).numpy().view(np.uint16)
    save("mini_c1", q_bf16=bits(qq), k_bf16=bits(kk), v_bf16=bits(vv), w=w, index_queries=index_q,
         index_keys=index_k, centroids=buckets.bucket_centroids, members=buckets.bucket_members, selected=sel,
         lengths=lens, out_rows=np.arange(0, T, 4), out=out[0][::4])


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py <checkout of the reference>/src")
    main(sys.argv[1])
