"""The SGLang glue end to end on the GPU, with no engine: a fake attention backend that holds a real KV pool and a
request table that is not the identity (so a list of KV slots is told apart from a list of positions) is enabled
through the plugin's hooks, and one prefill batch and one decode batch go through `select_and_read`. Lists must be the
oracle's read of each request, slot for slot; the attention within max-abs 2e-2 / mean-abs 2e-3 of the fp32 oracle."""

import types

import numpy as np
import pytest
import torch

from helpers import bf16_round, cuda

pytestmark = pytest.mark.gpu

HQ, HKV, DH, ROTARY, D_IDX = 8, 2, 128, 32, 64
BLOCK = {"indexer": {"window_size": 256, "sink_size": 4, "top_k": 512, "top_p": 32, "index_dim": D_IDX, "pool_size": 4,
                     "bucket_size": 16, "bucket_cap": 32}, "serving": {"projections": "maps.pt"}}
TEXT = types.SimpleNamespace(num_attention_heads=HQ, num_key_value_heads=HKV, head_dim=DH,
                             partial_rotary_factor=ROTARY / DH, num_hidden_layers=8, full_attention_interval=4)


class Mode:
    def __init__(self, extend):
        self.extend = extend

    def is_extend(self):
        return self.extend

    def is_idle(self):
        return False


class Pool:
    page_size = 1

    def __init__(self, slots):
        self.size = slots - 1
        self.k = torch.zeros(slots, HKV, DH, device="cuda", dtype=torch.bfloat16)
        self.v = torch.zeros(slots, HKV, DH, device="cuda", dtype=torch.bfloat16)

    def get_key_buffer(self, layer_id):
        return self.k

    def get_value_buffer(self, layer_id):
        return self.v

    def set_kv_buffer(self, layer, loc, k, v):
        self.k[loc.long()] = k.view(-1, HKV, DH)
        self.v[loc.long()] = v.view(-1, HKV, DH)


class Engine:
    """What an attention backend is to the hooks: a request table, a pool, and the methods they wrap."""

    def __init__(self, model_runner):
        self.req_to_token = model_runner.req_to_token
        self.token_to_kv_pool = model_runner.pool

    def forward_extend(self, q, k, v, layer, forward_batch, save_kv_cache=True):
        raise AssertionError("a served layer must not reach the backend's own attention")

    forward_decode = forward_extend


def _requests(lengths, rng):
    """Clustered keys, queries near their own key, values; and a request table of shuffled slots."""
    total = max(lengths) + 8
    table = np.full((4, total), 0, dtype=np.int32)
    rows = [0, 2, 3][: len(lengths)]
    data = []
    for i, (row, n) in enumerate(zip(rows, lengths)):
        table[row] = rng.permutation(total) + i * total + 1
        centres = rng.standard_normal((12, HKV, DH), dtype=np.float32)
        k = bf16_round(centres[rng.integers(0, 12, n + 1)] + 0.4 * rng.standard_normal((n + 1, HKV, DH), dtype=np.float32))
        q = bf16_round(np.repeat(k, HQ // HKV, axis=1) + 0.5 * rng.standard_normal((n + 1, HQ, DH), dtype=np.float32))
        v = bf16_round(rng.standard_normal((n + 1, HKV, DH), dtype=np.float32))
        data.append((q, k, v))
    return rows, table, data, len(lengths) * total + 1


def _batch(extend, rows, rids, positions, slots, seq_lens, new):
    return types.SimpleNamespace(
        forward_mode=Mode(extend), positions=cuda(np.asarray(positions, np.int64)),
        out_cache_loc=cuda(np.asarray(slots, np.int64)), req_pool_indices=cuda(np.asarray(rows, np.int64)), rids=rids,
        seq_lens_cpu=torch.tensor(seq_lens), extend_seq_lens_cpu=list(new),
        extend_prefix_lens_cpu=[s - n for s, n in zip(seq_lens, new)])


def _oracle_lists(oracle, index_keys, index_queries, positions, table_row):
    design = BLOCK["indexer"]
    buckets = oracle.build_buckets(index_keys, design["pool_size"], design["bucket_size"], design["bucket_cap"],
                                   design["window_size"])
    want, lens = oracle.read(index_queries, positions, buckets, design["top_p"], design["top_k"], design["sink_size"],
                             design["window_size"])
    return np.where(want >= 0, table_row[np.maximum(want, 0)], -1), lens


def test_prefill_and_decode_through_the_hooks(oracle, monkeypatch, tmp_path):
    from lsa_b200.sglang import backend, index_space, plugin, settings, weights

    rng = np.random.default_rng(0)
    lengths = [3000, 1800, 2100]
    rows, table, data, slots_total = _requests(lengths, rng)
    wq = bf16_round(rng.standard_normal((HKV * (DH - ROTARY), D_IDX), dtype=np.float32) / 14)
    wk = bf16_round(rng.standard_normal((HKV * (DH - ROTARY), D_IDX), dtype=np.float32) / 14)
    path = tmp_path / "maps.pt"
    layers = index_space.quadratic_layers(TEXT)
    assert layers == (3, 7)
    torch.save({f"{layer}.{kind}": torch.from_numpy(w) for layer in (*layers, 5)
                for kind, w in ((weights.QUERY, wq), (weights.KEY, wk))}, path)
    block = {**BLOCK, "serving": {"projections": str(path)}}

    # ---- the plugin's hooks, as a server's start applies them
    monkeypatch.setattr(plugin, "ENABLED", {"design": settings.parse(block)})
    monkeypatch.setattr(backend, "ENABLED", {})
    monkeypatch.setattr(backend, "ROWS", {})
    runner = types.SimpleNamespace(model_config=types.SimpleNamespace(hf_text_config=TEXT), pool=Pool(slots_total),
                                   req_to_token=cuda(table))
    engine = Engine(runner)
    plugin.enable(None, engine, runner)
    assert sorted(engine.lsa_indexers) == [3, 7]
    layer = types.SimpleNamespace(layer_id=3, tp_q_head_num=HQ, tp_k_head_num=HKV, head_dim=DH, scaling=DH ** -0.5)
    other = types.SimpleNamespace(layer_id=4)

    def gpu(x):
        return cuda(x, torch.bfloat16)

    # ---- one prefill batch of two requests, end to end (the third request's keys reach the pool with no indexer call)
    two = [0, 1]
    q = np.concatenate([data[i][0][: lengths[i]] for i in two])
    k = np.concatenate([data[i][1][: lengths[i]] for i in two])
    v = np.concatenate([data[i][2][: lengths[i]] for i in two])
    positions = np.concatenate([np.arange(lengths[i]) for i in two])
    slots = np.concatenate([table[rows[i], : lengths[i]] for i in two])
    batch = _batch(True, [rows[i] for i in two], ["a", "b"], positions, slots, [lengths[i] for i in two],
                   [lengths[i] for i in two])
    plugin.maintain(engine, batch)
    assert batch.lsa_rows == [rows[0], rows[1]]
    with pytest.raises(AssertionError):  # a layer outside the design reaches the backend as it was
        backend.select_and_read(Engine.forward_extend, engine, gpu(q), gpu(k), gpu(v), other, batch)
    T = len(q)
    out = backend.select_and_read(Engine.forward_extend, engine, gpu(q).view(T, HQ * DH), gpu(k), gpu(v), layer, batch)
    assert out.shape == (T, HQ * DH)
    assert torch.equal(runner.pool.k[cuda(slots).long()], gpu(k))  # the step's keys were saved at their slots

    indexer = engine.lsa_indexers[3]
    projection = indexer.index.projection
    # the maps: the fused read of the heads is the oracle's map of the written-out input
    index_keys = projection.index_keys(gpu(k)).cpu().numpy()
    index_queries = projection.index_queries(gpu(q)).cpu().numpy()
    want_keys = oracle.project(k[..., ROTARY:].reshape(T, -1), wk)
    want_queries = oracle.project(oracle.regroup_queries(np.ascontiguousarray(q[..., ROTARY:]), HKV), wq)
    np.testing.assert_allclose(index_keys, want_keys, rtol=0, atol=2e-6)
    np.testing.assert_allclose(index_queries, want_queries, rtol=0, atol=2e-6)
    written = index_space.materialise(index_space.key_and_query(gpu(q), gpu(k), indexer.geometry), indexer.geometry)
    assert written.key.shape == (T, HKV * (DH - ROTARY)) and written.query.shape == (T, 1, HKV * (DH - ROTARY))
    np.testing.assert_allclose(projection.index_keys(written.key).cpu().numpy(), index_keys, rtol=0, atol=2e-6)
    np.testing.assert_allclose(projection.index_queries(written.query).cpu().numpy(), index_queries, rtol=0, atol=2e-6)

    # the lists: each request read as the oracle reads its own keys, as KV slots through its row of the table
    first = 0
    kpool, vpool = runner.pool.k.float().cpu().numpy(), runner.pool.v.float().cpu().numpy()
    for i in two:
        n = lengths[i]
        span = slice(first, first + n)
        want, lens = _oracle_lists(oracle, index_keys[span], index_queries[span], np.arange(n), table[rows[i]])
        sample = np.r_[0:6, rng.integers(0, n, 40), n - 3:n]
        want_out, _ = oracle.sparse_attend(q[span][sample], kpool, vpool, want[sample].astype(np.int32),
                                           np.full(len(sample), len(kpool)), 0, 0, DH ** -0.5, lengths=lens[sample])
        err = np.abs(out.float().cpu().numpy().reshape(T, HQ, DH)[span][sample] - want_out)
        assert err.max() <= 2e-2 and err.mean() <= 2e-3, (i, err.max(), err.mean())
        first += n
    cache = indexer.index.selector.cache
    assert [cache.end(rows[i]) for i in two] == [lengths[i] for i in two]

    # ---- the lists themselves, on a fresh index over the same pool (a second layer's indexer)
    second = engine.lsa_indexers[7]
    second.maintain(batch)
    got = second.select(gpu(q), gpu(k), batch).cpu().numpy()
    first = 0
    for i in two:
        n = lengths[i]
        want, lens = _oracle_lists(oracle, index_keys[first:first + n], index_queries[first:first + n], np.arange(n),
                                   table[rows[i]])
        assert got.shape[1] == 512 + 256 + 4
        assert np.array_equal(got[first:first + n], want), i
        assert np.array_equal((got[first:first + n] >= 0).sum(1), lens)
        first += n

    # ---- one decode batch of all three; the third request's keys were written by the engine alone
    q3, k3, v3 = data[2]
    runner.pool.set_kv_buffer(None, cuda(table[rows[2], : lengths[2]].astype(np.int64)), gpu(k3[: lengths[2]]),
                              gpu(v3[: lengths[2]]))
    step_q = np.stack([data[i][0][lengths[i]] for i in range(3)])
    step_k = np.stack([data[i][1][lengths[i]] for i in range(3)])
    step_v = np.stack([data[i][2][lengths[i]] for i in range(3)])
    step_slots = [table[rows[i], lengths[i]] for i in range(3)]
    batch = _batch(False, rows, ["a", "b", "c"], lengths, step_slots, [n + 1 for n in lengths], [1, 1, 1])
    batch.req_pool_indices = cuda(np.asarray(rows, np.int64))
    plugin.maintain(engine, batch)  # request c enters here: its 2,100 keys are indexed from the pool
    assert cache.end(rows[2]) == lengths[2] and cache.buckets_of(rows[2]) == lengths[2] // 256 * 16
    out = backend.select_and_read(Engine.forward_decode, engine, gpu(step_q).view(3, HQ * DH), gpu(step_k), gpu(step_v),
                                  layer, batch)
    got = indexer.index.decode(index_space.key_and_query(gpu(step_q), gpu(step_k), indexer.geometry), batch.positions,
                               batch.out_cache_loc, batch.req_pool_indices).cpu().numpy()
    kpool, vpool = runner.pool.k.float().cpu().numpy(), runner.pool.v.float().cpu().numpy()
    for i in range(3):
        n = lengths[i]
        keys_i = projection.index_keys(gpu(data[i][1][: n + 1])).cpu().numpy()
        query_i = projection.index_queries(gpu(step_q[i:i + 1])).cpu().numpy()
        want, lens = _oracle_lists(oracle, keys_i, query_i, np.array([n]), table[rows[i]])
        assert np.array_equal(got[i:i + 1], want), i
        want_out, _ = oracle.sparse_attend(step_q[i:i + 1], kpool, vpool, want.astype(np.int32),
                                           np.full(1, len(kpool)), 0, 0, DH ** -0.5, lengths=lens)
        err = np.abs(out.float().cpu().numpy().reshape(3, HQ, DH)[i:i + 1] - want_out)
        assert err.max() <= 2e-2 and err.mean() <= 2e-3, (i, err.max())

    # a request table row taken over by another request starts afresh
    batch = _batch(True, [rows[1]], ["d"], np.arange(300), table[rows[1], :300], [300], [300])
    plugin.maintain(engine, batch)
    assert cache.end(rows[1]) == 0 and (cache.request_pages[rows[1]] == -1).all()


class Fabric:
    """The ranks of a group in one process: a first pass over the ranks records each one's term, `close` adds them in
    rank order, and every later call returns that sum - what a collective hands each rank."""

    def __init__(self):
        self.terms, self.total = [], None

    def reduce(self, term):
        if self.total is not None:
            return self.total
        self.terms.append(term)
        return term

    def close(self):
        self.total = self.terms[0]
        for term in self.terms[1:]:
            self.total = self.total + term


@pytest.mark.parametrize("tp", [2, 4])
def test_key_heads_split_over_a_tensor_parallel_group_give_the_index_of_one_rank(tp):
    from lsa_b200.sglang import index_space, settings
    from lsa_b200.sglang.layer_index import KeyAndQueryProjection, KeySplit, LayerIndex

    geometry = index_space.geometry_of(TEXT)
    rng = np.random.default_rng(tp)
    n = 2300
    rows, table, data, slots_total = _requests([n], rng)
    q, k = cuda(data[0][0][:n], torch.bfloat16), cuda(data[0][1][:n], torch.bfloat16)
    wq = torch.from_numpy(bf16_round(rng.standard_normal((geometry.key_dim, D_IDX), dtype=np.float32) / 14))
    wk = torch.from_numpy(bf16_round(rng.standard_normal((geometry.key_dim, D_IDX), dtype=np.float32) / 14))
    whole = KeyAndQueryProjection(wq, wk, geometry.key_slot, "cuda")
    want_q, want_k = whole.index_queries(q), whole.index_keys(k)
    shards = [index_space.head_shard(geometry, tp, rank) for rank in range(tp)]
    assert sum(s.counts_key for s in shards) == HKV and sum(s.query_count for s in shards) == HQ

    def inputs_of(rank):
        s = shards[rank]
        local_q = q[:, rank * s.query_count:(rank + 1) * s.query_count]
        return index_space.key_and_query(local_q, k[:, s.kv_first:s.kv_first + s.kv_count], geometry, s)

    fabric = Fabric()
    projections = [KeyAndQueryProjection(wq, wk, geometry.key_slot, "cuda",
                                         KeySplit(*s.dims(geometry), s.counts_key, fabric.reduce)) for s in shards]
    for _ in range(2):
        index = [p.split_index(inputs_of(r).key, inputs_of(r).query) for r, p in enumerate(projections)]
        fabric.close()
    for got_q, got_k in index:  # the same bits on every rank, and the unsplit vectors to rounding
        assert torch.equal(got_q, index[0][0]) and torch.equal(got_k, index[0][1])
    assert (index[0][0] - want_q).abs().max() <= 2e-6 and (index[0][1] - want_k).abs().max() <= 2e-6
    # a layer on such a rank keeps each token's index key at its KV slot, and selects what one rank selects
    design = settings.parse({**BLOCK, "serving": {"projections": "unused"}})
    table_d = cuda(table)
    positions = torch.arange(n, device="cuda")
    slots = table_d[rows[0], :n].long()
    pool = torch.zeros(slots_total, HKV, DH, device="cuda", dtype=torch.bfloat16)
    pool[slots] = k
    one = LayerIndex(design, (wq, wk), slots_total, slots_total, lambda: table_d, table.shape[1], 8192, "cuda",
                     key_buffer=lambda: pool, key_slot=geometry.key_slot)
    want = one.extend(index_space.key_and_query(q, k, geometry), positions, slots, [rows[0]], [n], [0])
    rank = tp - 1
    layer = LayerIndex(design, (wq, wk), slots_total, slots_total, lambda: table_d, table.shape[1], 8192, "cuda",
                       key_slot=geometry.key_slot, split=KeySplit(*shards[rank].dims(geometry),
                                                                  shards[rank].counts_key, fabric.reduce))
    got = layer.extend(inputs_of(rank), positions, slots, [rows[0]], [n], [0])
    assert torch.equal(layer.buffer.read(slots), index[0][1])
    agree = (got == want).all(1).float().mean().item()
    assert agree >= 0.995  # (index vectors equal to 2e-6: a near-tie may fall the other way in a row or two)


def test_a_decode_group_reads_each_key_on_the_rank_that_owns_its_slot():
    from lsa_b200.sglang import index_space, settings
    from lsa_b200.sglang.layer_index import LayerIndex, Shard

    geometry = index_space.geometry_of(TEXT)
    rng = np.random.default_rng(9)
    n, size = 2100, 2
    rows, table, data, slots_total = _requests([n], rng)
    slots_total += slots_total % size
    q, k = cuda(data[0][0][: n + 1], torch.bfloat16), cuda(data[0][1][: n + 1], torch.bfloat16)
    wq = torch.from_numpy(bf16_round(rng.standard_normal((geometry.key_dim, D_IDX), dtype=np.float32) / 14))
    wk = torch.from_numpy(bf16_round(rng.standard_normal((geometry.key_dim, D_IDX), dtype=np.float32) / 14))
    design = settings.parse({**BLOCK, "serving": {"projections": "unused"}})
    table_d = cuda(table)
    slots = table_d[rows[0], : n + 1].long()
    pool = torch.zeros(slots_total, HKV, DH, device="cuda", dtype=torch.bfloat16)
    pool[slots] = k
    pools = [pool[rank::size].contiguous() for rank in range(size)]  # slot s is row s // size of rank s % size
    one = LayerIndex(design, (wq, wk), slots_total, slots_total, lambda: table_d, table.shape[1], 8192, "cuda",
                     key_buffer=lambda: pool, key_slot=geometry.key_slot)
    group = [LayerIndex(design, (wq, wk), slots_total // size, slots_total // size, lambda: table_d, table.shape[1],
                        8192, "cuda", Shard(rank, size, lambda term: term), key_buffer=lambda rank=rank: pools[rank],
                        key_slot=geometry.key_slot) for rank in range(size)]

    def read(at):  # the group's sum, every rank's owned term added in rank order
        terms = []
        for rank, layer in enumerate(group):
            owned = at % size == rank
            keys = layer.projection.index_keys(pools[rank][torch.where(owned, at // size, 0)])
            terms.append(keys * owned[:, None])
        return terms[0] + terms[1]

    assert torch.equal(read(slots[:64]), one.buffer.read(slots[:64]))
    for layer in group:
        layer.buffer.read = read
    with pytest.raises(ValueError, match="needs the sum"):
        LayerIndex(design, (wq, wk), 8, 8, lambda: table_d, 8, 8, "cuda", Shard(1, 2), key_buffer=lambda: pool)
    # the keys reach the pools with no indexer call (a cached prefix): every rank indexes them through the group's reads
    step = index_space.key_and_query(q[n:], k[n:], geometry)
    position, row = torch.tensor([n], device="cuda"), torch.tensor([rows[0]], device="cuda")
    one.maintain(["a"], [rows[0]], [n])
    want = one.decode(step, position, slots[n:], row)
    for layer in group:
        layer.maintain(["a"], [rows[0]], [n])
        assert torch.equal(layer.decode(step, position, slots[n:], row), want)
        assert layer.selector.cache.buckets_of(rows[0]) == n // 256 * 16
