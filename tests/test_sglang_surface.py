"""The SGLang plugin surface without SGLang (as the reference tests it, tests/integ/sglang/test_plugin.py:1-7 and
tests/unit/sglang/test_qwen3_5.py:1-9): settings parsing, hook registration against a fake registry, the call
routing of `select_and_read` with fake backend objects; on a GPU, that a read attends over exactly the slots a list
names and that a decode group's partial reads merge to the whole."""

import enum
import types

import numpy as np
import pytest
import torch

from lsa_b200.sglang import backend, plugin, settings


class FakeRegistry:
    class HookType(enum.Enum):
        BEFORE = 1
        AFTER = 2
        AROUND = 3
        REPLACE = 4

    def __init__(self):
        self.hooks, self.applied = [], 0

    def register(self, target, hook, kind):
        self.hooks.append((target, hook, kind))

    def apply_hooks(self):
        self.applied += 1


def test_settings_block_is_parsed_and_unknown_keys_are_refused():
    design = settings.parse({"indexer": {"window_size": 1024, "top_p": 64, "top_k": 4096, "pool_size": 16,
                                         "bucket_size": 32, "bucket_cap": 64},
                             "serving": {"projections": "maps.safetensors"}})
    assert design.width == 4096 + 1024 + 4 and design.early_width is None
    flat = design.indexer.flat_design()
    assert (flat.cluster_block_size, flat.block_bucket_count) == (1024, 32)
    assert settings.parse({}).indexer.top_p == 1024  # the reference's defaults
    early = settings.parse({"indexer": {"early_budget": {"position": 4096, "top_k": 512, "top_p": 64}}})
    assert early.early_width == 512 + 512 + 4
    shaped = settings.parse({"indexer": {"bucket_shape": {"rank": 2, "deviations": 1.5}}})
    assert shaped.indexer.bucket_shape.rank == 2 and shaped.indexer.flat_design().bucket_shape.deviations == 1.5
    assert settings.parse({"indexer": {"bucket_shape": {}}}).indexer.bucket_shape.deviations == 2.0  # (the defaults)
    for refused, why in (({"bucket_shape": {"rank": 9}}, "at most 8 directions"),
                         ({"bucket_shape": {"rank": 2, "deviations": 0}}, "deviations must be positive"),
                         ({"bucket_shape": {"spread": 1}}, "rank and deviations"),
                         ({"bucket_shape": 2}, "a mapping of rank and deviations"),
                         ({"bucket_shape": {"rank": 2}, "index_dim": 48}, "multiple of 32"),
                         ({"node_bucket_shape": {"rank": 1}}, "top_level 0")):
        with pytest.raises(ValueError, match=why):
            settings.parse({"indexer": refused})
    for bad in ({"indexer": {"windows": 3}}, {"serving": {"kernels": "triton"}}, {"extra": 1},
                {"indexer": {"bucket_cap": 8}}, {"indexer": {"window_size": 500}}, {"indexer": {"top_level": 1}},
                {"serving": {"decode": "descend"}}, {"indexer": {"top_p": 4096}},
                {"indexer": {"top_p": 2, "top_k": 4096}}, []):
        with pytest.raises(ValueError):
            settings.parse(bad)


def test_every_target_is_resolved_before_any_hook_is_registered(monkeypatch):
    design = settings.parse({"serving": {"projections": "maps.safetensors"}})
    registry = FakeRegistry()
    # sglang is not installed: nothing resolves, so nothing may be registered
    with pytest.raises(RuntimeError, match="no longer resolve"):
        plugin.enable_lsa(design, registry=registry)
    assert not registry.hooks and not registry.applied
    with pytest.raises(RuntimeError, match="no serving.projections"):
        plugin.enable_lsa(settings.parse({}), registry=registry)
    # against targets that do resolve the whole table goes in, then the hooks are applied once
    fake = types.ModuleType("fake_engine")

    class Attention:
        def __init__(self): ...
        def init_forward_metadata(self, forward_batch): ...
        def init_forward_metadata_out_graph(self, forward_batch): ...
        def forward_extend(self, q, k, v, layer, forward_batch, save_kv_cache=True): ...
        def forward_decode(self, q, k, v, layer, forward_batch, save_kv_cache=True): ...

    fake.Attention = Attention
    monkeypatch.setitem(__import__("sys").modules, "fake_engine", fake)
    targets = tuple(f"fake_engine.Attention.{m}" for m in plugin.GROUPED_QUERY_METHODS)
    monkeypatch.setattr(plugin, "ENABLED", {})
    assert plugin.enable_lsa(design, registry=registry, targets=targets) == 5
    kinds = {target.rpartition(".")[2]: kind for target, _, kind in registry.hooks}
    assert kinds["forward_extend"] == kinds["forward_decode"] == FakeRegistry.HookType.AROUND
    assert kinds["__init__"] == FakeRegistry.HookType.AFTER and registry.applied == 1
    assert plugin.ENABLED["design"] is design


def test_the_standing_hook_enables_a_design_only_when_a_config_names_one(monkeypatch):
    registry = FakeRegistry()
    plugin.register(registry=registry)
    assert [(t, h.__name__) for t, h, _ in registry.hooks] == [(plugin.MODEL_CONFIG, "configure")]
    monkeypatch.setattr(plugin, "ENABLED", {})
    plugin.configure(None, types.SimpleNamespace(hf_config=types.SimpleNamespace()), registry=registry)  # no block
    assert "design" not in plugin.ENABLED
    with pytest.raises(RuntimeError):  # a block is found and enabling it needs an engine that is not here
        config = types.SimpleNamespace(hf_config=types.SimpleNamespace(lsa={"serving": {"projections": "m"}}))
        plugin.configure(None, config, registry=registry)
    with pytest.raises(RuntimeError, match="cannot read its settings"):
        plugin.register()


def test_select_and_read_hands_unserved_calls_back_untouched():
    calls = []

    def forward_decode(self, q, k, v, layer, forward_batch, save_kv_cache=True):
        calls.append((q, save_kv_cache))
        return "original"

    engine = types.SimpleNamespace()  # no indexers: not an LSA layer
    layer = types.SimpleNamespace(layer_id=3)
    assert backend.select_and_read(forward_decode, engine, 1, 2, 3, layer, None) == "original"
    engine.lsa_indexers = {3: object()}
    assert backend.select_and_read(forward_decode, engine, 1, None, None, layer, None, save_kv_cache=False) == "original"
    assert calls == [(1, True), (1, False)]
    mode = types.SimpleNamespace(is_extend=lambda: False, is_target_verify=lambda: True)
    with pytest.raises(NotImplementedError, match="speculative"):
        backend.select_and_read(forward_decode, engine, 1, 2, 3, layer, types.SimpleNamespace(forward_mode=mode))


def test_the_map_file_reader_refuses_what_is_not_the_models(tmp_path):
    from lsa_b200.sglang import weights

    good = {f"{layer}.{kind}": torch.randn(192, 64) for layer in (3, 7, 9) for kind in (weights.QUERY, weights.KEY)}
    path = tmp_path / "maps.pt"
    torch.save(good, path)
    maps = weights.read(path, 192, 64, [3, 7])
    assert sorted(maps) == [3, 7] and maps[3][0].dtype == torch.float32 and torch.equal(maps[7][1], good["7.W_K_idx"])
    for bad, match in (({**good, "extra": torch.zeros(1)}, "projection file holds"),
                       ({k: v for k, v in good.items() if k != "7.W_K_idx"}, "only one of"),
                       ({k: v for k, v in good.items() if not k.startswith("7.")}, "missing"),
                       ({**good, "3.W_Q_idx": torch.randn(64, 192)}, "expected"), ({}, "not a projection file")):
        torch.save(bad, path)
        with pytest.raises(ValueError, match=match):
            weights.read(path, 192, 64, [3, 7])


def test_a_grouped_query_checkpoints_geometry_and_the_heads_a_rank_holds():
    from lsa_b200.sglang import index_space as space

    published = types.SimpleNamespace(text_config=types.SimpleNamespace(
        num_attention_heads=24, num_key_value_heads=4, head_dim=256, rope_parameters={"partial_rotary_factor": 0.25},
        layer_types=["linear_attention"] * 3 + ["full_attention"], num_hidden_layers=4))
    served = types.SimpleNamespace(num_attention_heads=24, num_key_value_heads=4, head_dim=256,
                                   partial_rotary_factor=0.25, num_hidden_layers=8, full_attention_interval=4)
    geometry = space.geometry_of(published)
    assert (geometry.rotary_dim, geometry.key_dim, geometry.layers) == (64, 768, (3,))
    assert space.geometry_of(served).layers == (3, 7) and space.is_grouped_query(served)
    assert not space.is_grouped_query(types.SimpleNamespace(kv_lora_rank=512, layer_types=["full_attention"]))
    with pytest.raises(ValueError, match="nothing is position-free"):
        space.rotary_dim_of(types.SimpleNamespace(head_dim=128, partial_rotary_factor=1.0))
    with pytest.raises(ValueError, match="nothing to index"):
        space.quadratic_layers(types.SimpleNamespace(layer_types=["linear_attention"]))
    slot = geometry.key_slot
    assert (slot.heads, slot.offset, slot.width) == (4, 64, 192)
    with pytest.raises(ValueError, match="does not fit"):
        space.KeySlot(heads=1, head_dim=64, offset=32, width=48)
    pool = torch.arange(5 * 4 * 256, dtype=torch.float32).view(5, 4, 256)
    read = slot.read(pool, torch.tensor([1, 3]))
    assert read.shape == (2, 768) and torch.equal(read[0, 192:384], pool[1, 1, 64:])
    slot.write(pool, torch.tensor([0]), torch.zeros(1, 768))
    assert not pool[0, :, 64:].any() and pool[0, :, :64].any()
    # tensor parallel: the key heads dealt in order, a head replicated once the ranks outnumber them
    assert space.head_shard(geometry, 1, 0) is None and space.head_shard(geometry, 4, 1, decode_size=4) is None
    assert space.head_shard(geometry, 2, 1) == space.HeadShard(2, 2, 12, True)
    eight = [space.head_shard(geometry, 8, rank) for rank in range(8)]
    assert [(s.kv_first, s.counts_key) for s in eight[:4]] == [(0, True), (0, False), (1, True), (1, False)]
    assert sum(s.counts_key for s in eight) == 4 and eight[5].dims(geometry) == (384, 576)
    for size, decode in ((3, 1), (5, 1), (16, 1), (8, 2)):
        with pytest.raises(NotImplementedError):
            space.head_shard(geometry, size, 0, decode)
    q, k = torch.randn(6, 24 * 256), torch.randn(6, 4, 256)
    written = space.materialise(space.key_and_query(q, k, geometry), geometry)
    assert written.key.shape == (6, 768) and written.query.shape == (6, 1, 768) and written.query.dtype == torch.float32
    want = q.view(6, 4, 6, 256)[..., 64:].sum(2).reshape(6, 768)
    assert torch.allclose(written.query[:, 0], want, atol=1e-5)


def test_a_group_whose_ranks_hold_different_indexes_is_told_so_on_every_rank():
    from lsa_b200.sglang import consistency

    a = torch.arange(12, dtype=torch.float32).view(3, 4)
    assert int(consistency.checksum(a)) != int(consistency.checksum(a.flip(0)))  # order-sensitive
    assert int(consistency.checksum(a)) == int(consistency.checksum(a.t().contiguous().t()))  # by value, not by stride

    class Cache:  # what the check reads of a bucket cache
        def __init__(self, seed):
            g = torch.Generator().manual_seed(seed)
            self.centroids, self.members = torch.randn(40, 8, generator=g), torch.randint(0, 999, (40, 6), generator=g)
            self.sizes, self.closed_keys = torch.randint(1, 6, (40,), generator=g).int(), {2: 64, 5: 32}

        def buckets_of(self, row):
            return self.closed_keys.get(row, 0) // 8

        def end(self, row):
            return self.closed_keys.get(row, 0) + 3

        def rows_of(self, row, logical):
            return logical + 4 * row

    def run(caches):
        # each rank's two collective calls answered with the true sums of what every rank would send
        locals_, flags = [], []
        for cache in caches:
            sent = []
            try:
                consistency.check_same_index(cache, [2, 5], lambda t: (sent.append(t.clone()), t)[1], len(caches))
            except RuntimeError:
                pass
            locals_.append(sent[0])
        total = sum(locals_[1:], locals_[0])
        outcomes = []
        for cache, local in zip(caches, locals_):
            differs = (total != local * len(caches)).any().float().reshape(1)
            flags.append(differs)
        any_differs = sum(flags[1:], flags[0])
        for cache in caches:
            answers = iter([total, any_differs])
            try:
                consistency.check_same_index(cache, [2, 5], lambda t: next(answers), len(caches))
                outcomes.append("same")
            except RuntimeError as failure:
                assert "different indexes" in str(failure)
                outcomes.append("differ")
        return outcomes

    assert run([Cache(0), Cache(0), Cache(0)]) == ["same"] * 3
    drifted = Cache(0)
    drifted.members[21, 2] += 1  # one member of one bucket of request 5
    assert run([Cache(0), drifted, Cache(0)]) == ["differ"] * 3
    consistency.check_same_index(Cache(0), [], None, 3)  # an empty batch checks nothing


def test_lists_split_over_a_decode_group_hold_every_slot_once():
    lists = torch.tensor([[5, 2, 9, 4, -1, -1], [7, -1, -1, -1, -1, -1]], dtype=torch.int32)
    assert backend.list_lengths(lists).tolist() == [4, 1]
    seen = [[], []]
    for rank in range(3):
        rows, counts = backend.owned_lists(lists, backend.Shard(rank, 3))
        for r in range(2):
            held = rows[r, : int(counts[r])]
            assert (rows[r, int(counts[r]):] == -1).all()
            seen[r] += (held * 3 + rank).tolist()
    assert sorted(seen[0]) == [2, 4, 5, 9] and seen[1] == [7]


class _Pool:
    def __init__(self, k, v):
        self.k, self.v, self.saved = k, v, []

    def get_key_buffer(self, layer_id):
        return self.k

    def get_value_buffer(self, layer_id):
        return self.v

    def set_kv_buffer(self, layer, loc, k, v):
        self.saved.append(loc)
        self.k[loc.long()] = k
        self.v[loc.long()] = v


@pytest.mark.gpu
def test_a_read_attends_over_exactly_the_slots_a_list_names(oracle):
    from helpers import bf16_round, cuda

    rng = np.random.default_rng(0)
    slots, Hq, Hkv, dh, T, width = 3000, 8, 2, 128, 6, 700
    k = bf16_round(rng.standard_normal((slots, Hkv, dh), dtype=np.float32))
    v = bf16_round(rng.standard_normal((slots, Hkv, dh), dtype=np.float32))
    q = bf16_round(rng.standard_normal((T, Hq, dh), dtype=np.float32))
    lists = np.full((T, width), -1, dtype=np.int32)
    for r in range(T):
        n = int(rng.integers(1, width))
        lists[r, :n] = rng.choice(slots - 10, n, replace=False)
    pool = _Pool(cuda(k, torch.bfloat16), cuda(v, torch.bfloat16))
    engine = types.SimpleNamespace(token_to_kv_pool=pool)
    layer = types.SimpleNamespace(layer_id=0, tp_q_head_num=Hq, tp_k_head_num=Hkv, head_dim=dh, scaling=dh ** -0.5)
    want, _ = oracle.sparse_attend(q, k, v, lists, np.full(T, slots), 0, 0, dh ** -0.5)
    out = backend.sparse_read(engine, cuda(q, torch.bfloat16).view(T, Hq * dh), layer, cuda(lists))
    assert out.shape == (T, Hq * dh)
    assert np.abs(out.float().cpu().numpy().reshape(T, Hq, dh) - want).max() <= 2e-2
    # a decode group of two: each rank's pool holds every other slot, partial reads merged by hand
    parts, lses = [], []
    for rank in range(2):
        shard = backend.Shard(rank, 2)
        mine = types.SimpleNamespace(token_to_kv_pool=_Pool(pool.k[rank::2].contiguous(), pool.v[rank::2].contiguous()))
        rows, counts = backend.owned_lists(cuda(lists), shard)
        part, lse = backend.partial_read(mine, cuda(q, torch.bfloat16), layer, rows, counts)
        parts.append(part)
        lses.append(lse)
    from lsa_b200 import ops
    merged, _ = ops.lse_merge(torch.stack(parts), torch.stack(lses))
    assert np.abs(merged.cpu().numpy() - want).max() <= 2e-2
    # the full hook: save this step's keys, select, read
    step_k, step_v = cuda(k[-T:], torch.bfloat16), cuda(v[-T:], torch.bfloat16)
    indexer = types.SimpleNamespace(shard=backend.Shard(), select=lambda q_, k_, fb: cuda(lists))
    engine.lsa_indexers = {0: indexer}
    batch = types.SimpleNamespace(forward_mode=types.SimpleNamespace(is_extend=lambda: False),
                                  out_cache_loc=torch.arange(slots - T, slots).cuda())

    def forward_decode(self, q, k, v, layer, forward_batch, save_kv_cache=True):
        raise AssertionError("a served layer must not reach the engine's own attention")

    got = backend.select_and_read(forward_decode, engine, cuda(q, torch.bfloat16).view(T, Hq * dh), step_k, step_v, layer,
                                  batch)
    assert len(pool.saved) == 1 and np.abs(got.float().cpu().numpy().reshape(T, Hq, dh) - want).max() <= 2e-2


def test_decode_graphs_are_keyed_by_context_ranges(monkeypatch):
    import sys

    import torch

    from lsa_b200.sglang import context_buckets

    page = settings.PAGE_SIZE
    # the knobs: ascending whole pages, and the reference's default ranges
    defaults = settings.parse({}).serving
    assert defaults.decode_context_limits == tuple(18 * page * 2 ** i for i in range(7))
    assert defaults.prefix_reuse is False and defaults.spare_contexts == 0
    chosen = settings.parse({"serving": {"decode_context_limits": [2 * page, 8 * page], "prefix_reuse": True,
                                         "spare_contexts": 2}}).serving
    assert chosen.decode_context_limits == (2 * page, 8 * page) and chosen.prefix_reuse and chosen.spare_contexts == 2
    for refused in ({"decode_context_limits": [page - 1]}, {"decode_context_limits": [4 * page, 2 * page]},
                    {"decode_context_limits": [2 * page, 2 * page]}, {"prefix_reuse": "yes"}, {"spare_contexts": -1}):
        with pytest.raises(ValueError):
            settings.parse({"serving": refused})
    # the ranges narrower than the server's context; the widest graph is captured first
    ranges = context_buckets.ContextBuckets.under(chosen.decode_context_limits + (64 * page,), 32 * page)
    assert ranges.limits == (2 * page, 8 * page)
    assert ranges.capture_labels == ("context_full", f"context_{8 * page}", f"context_{2 * page}")
    assert context_buckets.ContextBuckets.under((8 * page,), 4 * page) is None

    def batch(*lengths):
        return types.SimpleNamespace(seq_lens_cpu=torch.tensor(lengths))

    assert ranges.select(batch(5, 2 * page)) == f"context_{2 * page}"          # the longest request decides
    assert ranges.select(batch(2 * page + 1, 9)) == f"context_{8 * page}"
    assert ranges.select(batch(8 * page + 1)) == "context_full"
    assert ranges.select(types.SimpleNamespace()) == "context_full"           # lengths not on the host
    assert ranges.select(types.SimpleNamespace(seq_lens_cpu=torch.tensor([], dtype=torch.int64))) == "context_full"
    assert context_buckets.pages_of(page) == 1 and context_buckets.pages_of(page + 1) == 2
    # the label being captured, where an engine's capture module says one
    assert context_buckets.captured_limit() is None
    capture = types.ModuleType(context_buckets.CAPTURE_MODE)
    label = {"now": None}
    capture.get_capture_attention_variant = lambda: label["now"]
    monkeypatch.setitem(sys.modules, context_buckets.CAPTURE_MODE, capture)
    for said, limit in ((None, None), ("context_full", None), (f"context_{2 * page}", 2 * page), ("other", None)):
        label["now"] = said
        assert context_buckets.captured_limit() == limit
    # the capture hook hands a decode runner the ranges once, and leaves a runner with variants of its own alone
    design = settings.parse({"serving": {"projections": "m", "decode_context_limits": [2 * page, 8 * page]}})
    monkeypatch.setattr(plugin, "ENABLED", {"design": design})
    seen = []

    def capture_one_stream(self, *args):
        seen.append(self.attention_graph_variants)
        return "captured"

    def runner(variants=None, decode=True):
        config = types.SimpleNamespace(context_len=32 * page)
        return types.SimpleNamespace(attention_graph_variants=variants, model_runner=types.SimpleNamespace(model_config=config),
                                     capture_forward_mode=types.SimpleNamespace(is_decode=lambda: decode))

    assert plugin.capture_context_graphs(capture_one_stream, runner()) == "captured"
    assert seen[-1].limits == (2 * page, 8 * page)
    plugin.capture_context_graphs(capture_one_stream, runner(variants="theirs"))
    plugin.capture_context_graphs(capture_one_stream, runner(decode=False))
    assert seen[-2] == "theirs" and seen[-1] is None
    # the hook is registered only where both the capture and the getter resolve
    registry = FakeRegistry()
    assert not plugin.context_graphs(registry, registry.HookType) and not registry.hooks
    fake = types.ModuleType("fake_runner")
    fake.Runner = type("Runner", (), {"_capture_one_stream": capture_one_stream})
    fake.get_capture_attention_variant = capture.get_capture_attention_variant
    monkeypatch.setitem(sys.modules, "fake_runner", fake)
    targets = ("fake_runner.Runner._capture_one_stream", "fake_runner.get_capture_attention_variant")
    assert plugin.context_graphs(registry, registry.HookType, targets)
    assert [(t, h.__name__, k) for t, h, k in registry.hooks] == [(targets[0], "capture_context_graphs",
                                                                   FakeRegistry.HookType.AROUND)]
