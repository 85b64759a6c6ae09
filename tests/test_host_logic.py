"""Host-side logic that needs no GPU: budgets, design checks, validation errors, list composition, the probe."""

import pytest
import torch

from lsa_b200 import core, probe
from lsa_b200.budget import EarlyBudget, budget_at
from lsa_b200.layer import FlatDesign


def test_early_budget_is_validated_and_applied():
    early = EarlyBudget(position=100, top_k=8, top_p=2)
    assert budget_at(99, 64, 16, early) == (8, 2) and budget_at(100, 64, 16, early) == (64, 16)
    assert budget_at(5, 64, 16, None) == (64, 16)
    assert EarlyBudget.read({"position": 3, "top_k": 2, "top_p": 1}) == EarlyBudget(3, 2, 1)
    assert EarlyBudget.read(None) is None
    for bad in ({"position": 0, "top_k": 1, "top_p": 1}, {"position": True, "top_k": 1, "top_p": 1},
                {"position": 1, "top_k": 1}, [1, 2, 3]):
        with pytest.raises(ValueError):
            EarlyBudget.read(bad)


def test_design_sizes_must_nest():
    FlatDesign(16, 32, 64, 1024, 64, 4096, 4, 1024)
    for bad in [(3, 8, 16, 64), (4, 8, 16, 60), (4, 8, 15, 64), (0, 8, 16, 64)]:
        with pytest.raises(ValueError):
            core.check_sizes(*bad)
    with pytest.raises(ValueError, match="cannot fill"):
        FlatDesign(4, 8, 16, 64, top_p=2, top_k=64)


def test_rows_that_are_not_unit_length_are_refused_before_any_kernel():
    with pytest.raises(ValueError, match="unit rows"):
        core.check_unit_rows("index_keys", torch.ones(4, 8))
    with pytest.raises(ValueError, match="float32 or bfloat16"):
        core.check_unit_rows("index_keys", torch.ones(4, 8, dtype=torch.float64))
    with pytest.raises(ValueError, match="non-finite"):
        core.check_unit_rows("index_keys", torch.full((2, 2), float("nan")))
    with pytest.raises(ValueError, match=r"\[N, index_dim\]"):
        core.check_unit_rows("index_keys", torch.ones(4))
    core.check_unit_rows("index_keys", torch.nn.functional.normalize(torch.randn(5, 8), dim=-1).bfloat16())


def test_rotary_layout_and_position_free_views():
    q, k = torch.randn(2, 4, 3, 16), torch.randn(2, 2, 3, 16)
    a, b = core.position_free(q, k, core.RotaryLayout("prefix", 4))
    assert a.shape[-1] == 12 and torch.equal(b, k[..., 4:])
    a, _ = core.position_free(q, k, core.RotaryLayout("suffix", 4))
    assert torch.equal(a, q[..., :12])
    assert core.position_free(q, k, core.RotaryLayout())[0] is q
    with pytest.raises(ValueError):
        core.RotaryLayout("prefix", 0)
    with pytest.raises(ValueError, match="whole head"):
        core.position_free(q, k, core.RotaryLayout("prefix", 16))


def test_a_keep_set_list_is_the_union_with_every_key_once():
    # tests/unit/core/test_attention.py:60-65 of the reference: keep-set {0,1,40,47,48,49,50} at position 50
    selected = torch.tensor([[40, 49, 60, -1, 40]], dtype=torch.int32)
    lists, lengths = core.compose_lists(selected, torch.tensor([50]), 4, 2)
    assert lists[0, : int(lengths[0])].tolist() == [0, 1, 40, 47, 48, 49, 50]
    assert (lists[0, int(lengths[0]):] == -1).all()
    # padding selects nothing; no window and no sinks leaves only causal picks
    lists, lengths = core.compose_lists(torch.tensor([[-1, 7, 2]], dtype=torch.int32), torch.tensor([5]), 0, 0)
    assert lists[0, : int(lengths[0])].tolist() == [2]


def test_regions_cost_nothing_until_a_recorder_listens():
    seen = []

    class Recorder:
        def region(self, name):
            import contextlib

            seen.append(name)
            return contextlib.nullcontext()

    with probe.region("select"):
        pass
    assert not seen
    probe.install(Recorder())
    with probe.region("select"):
        pass
    probe.uninstall()
    assert seen == ["select"]


def test_the_rows_a_rank_keeps_partition_every_chunk():
    from types import SimpleNamespace

    from lsa_b200.parallel import ShardedFlatLayer, deal, undeal

    tokens, chunk, world = 4096, 1024, 4
    rows = torch.arange(tokens)[:, None].expand(tokens, 3)
    kept = []
    for rank in range(world):
        sharded = ShardedFlatLayer(SimpleNamespace(design=None), rank, world)
        mine = sharded.rows_of(rows, chunk)
        assert mine.shape == (tokens // world, 3)
        share = chunk // world
        want = torch.cat([torch.arange(c * chunk + rank * share, c * chunk + (rank + 1) * share)
                          for c in range(tokens // chunk)])
        assert torch.equal(mine[:, 0], want)
        kept.append(mine[:, 0])
    assert torch.equal(torch.cat(kept).sort().values, torch.arange(tokens))
    # the dealt cache and its inverse: granules of 64 positions round-robin over the ranks
    dealt = torch.stack([deal(rows, rank, world) for rank in range(world)])
    assert dealt[1, :64, 0].tolist() == list(range(64, 128)) and dealt[1, 64, 0] == 64 + 64 * world
    assert torch.equal(undeal(dealt), rows)


def test_a_layer_raises_what_its_kernels_reported():
    """`FlatLayer.check()` reads the status words the kernels raise and the per-block `reached` flags of the last
    index builds; here they are set by hand, on the host, as a kernel would have set them."""
    from lsa_b200.layer import FlatDesign, FlatLayer

    maps = torch.randn(2 * 128, 32)
    layer = FlatLayer(FlatDesign(pool_size=4, bucket_size=8, bucket_cap=16, cluster_block_size=64, top_p=8, top_k=64,
                                 window_size=64), maps, maps, 4, 2, 128)
    layer.check()  # nothing was reported
    layer._reached.append(torch.tensor([1, 0, 1], dtype=torch.uint8))
    with pytest.raises(ValueError, match="1 cluster blocks stopped short"):
        layer.check()
    layer.check()  # the report was consumed
    layer._table_status += 2
    with pytest.raises(ValueError, match="2 buckets overflowed"):
        layer.check()
    layer._attend_status += 1
    with pytest.raises(RuntimeError, match="bounded on-chip waits gave up"):
        layer.check()
    layer._expand_status += 3
    with pytest.raises(ValueError, match="3 picked bucket ids"):
        layer.check()
    assert not layer.status.any()


def test_an_address_keeps_its_tensor_alive():
    import ctypes
    import gc
    import weakref

    from lsa_b200._lib import Address

    tensor = torch.zeros(8)
    address = Address(tensor)
    alive = weakref.ref(tensor)
    del tensor
    gc.collect()
    assert alive() is not None and int(address) == address.tensor.data_ptr()
    assert ctypes.c_void_p.from_param(address) is not None  # ctypes takes it where it takes an int


def test_workload_generators_are_seeded_and_shaped():
    from lsa_b200 import workloads as W

    cfg = W.cut(W.C2, 2048)
    a, b = W.gqa_inputs(cfg), W.gqa_inputs(cfg)
    assert all(torch.equal(x, y) for x, y in zip(a, b))
    q, k, v, wq, wk = a
    assert q.shape == (2048, 40, 128) and k.shape == (2048, 8, 128) and wq.shape == (1024, 64)
    lengths = W.request_lengths(W.C5)
    assert len(lengths) == 64 and lengths.min() >= 32768 and lengths.max() <= 524288 and not (lengths % 1024).any()
    small = dict(W.C1, tokens=2048)
    q1, k1, v1, index_map = W.c1_inputs(small)
    assert index_map.shape == (256, 32) and torch.allclose(index_map.t() @ index_map, torch.eye(32), atol=1e-4)
    for name, cfg in W.CONFIGS.items():
        W.design_of(cfg)  # the sizes of every config nest and fill their top_k


class _Lookup:
    """A request's pages as a list of fingerprints: what `KeyLookup.fingerprints` would read from the pool."""

    def __init__(self, prints):
        self.prints, self.reads = prints, 0

    def fingerprints(self, first, count):
        self.reads += count
        return self.prints[first:first + count]


def test_prefix_reuse_shares_full_pages_by_fingerprint_and_keeps_a_finished_prefix():
    from lsa_b200.serving import BucketCache

    design = FlatDesign(pool_size=1, bucket_size=2, bucket_cap=4, cluster_block_size=8, top_p=8, top_k=16)
    cache = BucketCache(design, 32, pages=6, page_buckets=4, max_requests=4, max_request_pages=4, device="cpu",
                        reuse=True)
    page = cache.page_keys
    assert page == 8

    def filled(request, pages):  # (what `append` leaves once `pages` pages of keys were clustered)
        cache._grow(request, pages * cache.page_buckets)
        cache.closed_keys[request] = pages * page
        cache.bucket_counts[request] = pages * cache.page_buckets

    filled(0, 3)
    cache.fingerprint(0, 3 * page, _Lookup([11, 12, 13]))
    assert cache.prints[0] == [11, 12, 13] and cache.adopt(0, 3 * page, _Lookup([11, 12, 13])) == 0  # (it holds keys)
    # a request sharing two pages takes them by reference; a third print it has not got keys for is never read
    second = _Lookup([11, 12, 99])
    assert cache.adopt(1, 2 * page + 3, second) == 2 and second.reads == 2
    assert cache.held[1] == cache.held[0][:2] and cache.end(1) == 2 * page and int(cache.bucket_counts[1]) == 8
    assert cache.request_pages[1, :2].tolist() == cache.held[0][:2] and cache.request_pages[1, 2] == -1
    assert [cache.holders[p] for p in cache.held[0]] == [2, 2, 1] and len(cache.free_pages) == 3
    assert cache.adopt(2, page - 1, _Lookup([11])) == 0            # less than a page in the pool
    assert cache.adopt(2, 3 * page, _Lookup([77, 12, 13])) == 0     # the first page differs: nothing after it counts
    # the first request ends: its fingerprinted pages stay as a retained prefix, nothing is freed
    kept = list(cache.held[0])
    cache.release(0)
    assert len(cache.retained) == 1 and cache.retained[0].pages == kept and len(cache.free_pages) == 3
    assert cache.adopt(2, 3 * page + 1, _Lookup([11, 12, 13, 14])) == 3 and cache.held[2] == kept
    assert [cache.holders[p] for p in kept] == [3, 3, 2]
    # a request that holds shared pages and ends keeps the prefix alive: each holder is counted
    cache.release(2, retain=False)
    cache.release(1, retain=False)
    assert [cache.holders[p] for p in kept] == [1, 1, 1] and len(cache.free_pages) == 3
    # pages run short: the retained prefix goes first, and its pages come back as no one else holds them
    filled(3, 3)
    assert not cache.free_pages
    cache._grow(2, cache.page_buckets)
    assert not cache.retained and len(cache.free_pages) == 2 and cache.holders[cache.held[2][0]] == 1
    cache.running([1, 2, 3])
    with pytest.raises(RuntimeError, match="out of pages"):
        cache._grow(1, 3 * cache.page_buckets)
    for request in (1, 2, 3):
        cache.release(request, retain=False)
    assert sorted(cache.free_pages) == list(range(6)) and not any(cache.holders)
    # idle requests give their pages up, the one seen longest ago first; a request of the running batch never does
    for request, rid in ((0, "a"), (1, "b"), (2, "c")):
        cache.running([request])
        cache.ensure(request, rid)
        filled(request, 2)
    assert not cache.free_pages
    cache.running([1, 3])
    cache.ensure(3, "d")
    filled(3, 1)                      # request 0, seen first, goes; its pages come back
    assert 0 not in cache.held and cache.held[1] and cache.held[2] and len(cache.free_pages) == 1
    filled(3, 3)                      # one free page, then request 2 goes (1 is running)
    assert 2 not in cache.held and len(cache.held[1]) == 2 and len(cache.held[3]) == 3 and len(cache.free_pages) == 1
    with pytest.raises(RuntimeError, match="every page belongs to a running request"):
        filled(3, 4), filled(1, 4)
    for request in (1, 3):
        cache.release(request, retain=False)
    assert sorted(cache.free_pages) == list(range(6)) and not any(cache.holders)
    with pytest.raises(TypeError, match="this lookup reads none"):
        filled(0, 1)
        cache.fingerprint(0, page, object())
    plain = BucketCache(design, 32, pages=2, page_buckets=4, max_requests=2, max_request_pages=2, device="cpu")
    assert plain.adopt(0, 4 * page, object()) == 0 and plain.fingerprint(0, page, object()) is None
