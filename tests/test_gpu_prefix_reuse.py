"""Prefix reuse on the GPU: page fingerprints of the pool's bits against the oracle (itself pinned to the reference's
`page_fingerprints` by tests/golden/fingerprints.npz), and a layer index under `prefix_reuse` whose second request
takes the first one's index pages and reads exactly what it would have read from pages of its own."""

import types

import numpy as np
import pytest
import torch

from conftest import golden
from helpers import bf16_round, cuda

pytestmark = pytest.mark.gpu

HQ, HKV, DH, ROTARY, D_IDX = 8, 2, 128, 32, 64
BLOCK = {"indexer": {"window_size": 256, "sink_size": 4, "top_k": 512, "top_p": 32, "index_dim": D_IDX, "pool_size": 4,
                     "bucket_size": 16, "bucket_cap": 32}, "serving": {"projections": "unused"}}
TEXT = types.SimpleNamespace(num_attention_heads=HQ, num_key_value_heads=HKV, head_dim=DH,
                             partial_rotary_factor=ROTARY / DH, num_hidden_layers=8, full_attention_interval=4)


def pattern(rows, dim):
    i, j = np.arange(rows, dtype=np.int64)[:, None], np.arange(dim, dtype=np.int64)[None]
    return ((i * 40503 + j * 1201 + (i * j) % 251 + 7) & 0xFFFF).astype(np.uint16)


def test_page_fingerprints_are_the_references_bit_for_bit(oracle):
    from lsa_b200 import ops
    from lsa_b200.sglang import layer_index

    g = golden("fingerprints")
    page = int(g["page_size"])
    assert page == layer_index.PAGE_SIZE
    words, positions = layer_index.fingerprint_weights("cuda")
    assert np.array_equal(words[:16].cpu().numpy(), g["words_head"]) and int(words.sum()) == int(g["words_sum"])
    assert np.array_equal(positions[:16].cpu().numpy(), g["positions_head"])
    for dim in (16, 64, 512):
        bits = pattern(3 * page, dim)
        stored = cuda(bits.view(np.int16)).view(torch.bfloat16)
        got = layer_index.page_fingerprints(stored, None)
        assert np.array_equal(got.cpu().numpy(), g[f"d{dim}_all"])
        parts = []
        for rank in range(3):
            owned = torch.arange(3 * page, device="cuda") % 3 == rank
            parts.append(layer_index.page_fingerprints(stored, owned))
            assert np.array_equal(parts[-1].cpu().numpy(), g[f"d{dim}_rank{rank}"])
        # the group's sum through 16-bit pieces a collective may add in fp32: the whole page's fingerprint
        def reduce(pieces):
            others = [((p[:, None] >> (16 * torch.arange(4, device="cuda"))) & 0xFFFF).float() for p in parts[1:]]
            return pieces + others[0] + others[1]

        assert torch.equal(layer_index.exact_group_sum(parts[0], reduce), got)
    # read in place out of a pool: rows of a strided view, named by slots in any order; slots out of range add nothing
    rng = np.random.default_rng(0)
    pool_bits = rng.integers(0, 1 << 16, (40000, 2, 96), dtype=np.uint16)
    pool = cuda(pool_bits.view(np.int16)).view(torch.bfloat16)
    slots = rng.permutation(40000)[: 2 * page].astype(np.int64)
    w, p = oracle.fingerprint_weights(page)
    want = oracle.page_fingerprints(pool_bits[slots, 0, 32:96], np.ones(2 * page, bool), w, p)
    got = ops.page_fingerprints(pool[:, 0, 32:96], page, words, positions, slots=cuda(slots))
    assert np.array_equal(got.cpu().numpy(), want)
    owned = rng.integers(0, 2, 2 * page).astype(bool)
    gone = slots.copy()
    gone[7], gone[page + 9] = -1, 40000
    owned_gone = owned.copy()
    owned_gone[[7, page + 9]] = False
    want = oracle.page_fingerprints(pool_bits[slots, 0, 32:96], owned_gone, w, p)
    got = ops.page_fingerprints(pool[:, 0, 32:96], page, words, positions, slots=cuda(gone), owned=cuda(owned))
    assert np.array_equal(got.cpu().numpy(), want)
    with pytest.raises(ValueError, match="whole pages"):
        ops.page_fingerprints(pool[:, 0, 32:96], page, words, positions, slots=cuda(slots[:-1]))


def test_a_request_with_a_cached_prefix_takes_the_index_pages_built_from_the_same_bits(oracle):
    from lsa_b200.sglang import index_space, settings
    from lsa_b200.sglang.layer_index import PAGE_SIZE, LayerIndex

    geometry = index_space.geometry_of(TEXT)
    rng = np.random.default_rng(4)
    shared, n_a, n_b = 2 * PAGE_SIZE, 2 * PAGE_SIZE + 900, 2 * PAGE_SIZE + 1500
    total = n_a + (n_b - shared) + PAGE_SIZE + 64
    free = rng.permutation(total).astype(np.int32) + 1
    table = np.zeros((4, n_b + 8), dtype=np.int32)
    table[0, :n_a] = free[:n_a]
    table[2, :shared] = table[0, :shared]                     # the prefix cache hands the same slots to both
    table[2, shared:n_b] = free[n_a:n_a + n_b - shared]
    table[3, :PAGE_SIZE] = free[n_a + n_b - shared:n_a + n_b - shared + PAGE_SIZE]  # a copy of page 0, one bit off
    centres = rng.standard_normal((12, HKV, DH), dtype=np.float32)
    pool = torch.zeros(total + 1, HKV, DH, device="cuda", dtype=torch.bfloat16)
    keys = bf16_round(centres[rng.integers(0, 12, total + 1)] + 0.4 * rng.standard_normal((total + 1, HKV, DH),
                                                                                         dtype=np.float32))
    pool.copy_(cuda(keys, torch.bfloat16))
    pool[table[3, :PAGE_SIZE]] = pool[table[0, :PAGE_SIZE]]
    wq = torch.from_numpy(bf16_round(rng.standard_normal((geometry.key_dim, D_IDX), dtype=np.float32) / 14))
    wk = torch.from_numpy(bf16_round(rng.standard_normal((geometry.key_dim, D_IDX), dtype=np.float32) / 14))
    design = settings.parse(BLOCK)
    table_d = cuda(table)

    def layer(reuse):
        return LayerIndex(design, (wq, wk), total + 1, total + 1, lambda: table_d, table.shape[1], 8192, "cuda",
                          key_buffer=lambda: pool, key_slot=geometry.key_slot, prefix_reuse=reuse)

    reuse, plain = layer(True), layer(False)
    reuse.writes_pool = plain.writes_pool = False  # (the keys are in the pool: a step here writes nothing over them)
    cache = reuse.selector.cache
    reuse.maintain(["a"], [0], [n_a])
    # a page's fingerprint is the oracle's over the pool's own bits at the request's slots
    slot = geometry.key_slot
    stored = pool[table[0, :shared]][:, :, slot.offset:slot.offset + slot.width].reshape(shared, -1)
    w, p = oracle.fingerprint_weights(PAGE_SIZE)
    want = oracle.page_fingerprints(stored.view(torch.int16).cpu().numpy(), np.ones(shared, bool), w, p)
    assert cache.prints[0] == want.tolist()
    before = len(cache.free_pages)
    reuse.maintain(["a", "b"], [0, 2], [n_a, n_b])
    assert cache.held[2][:2] == cache.held[0][:2] and cache.holders[cache.held[0][0]] == 2
    assert len(cache.free_pages) == before - 1 and cache.end(2) == n_b  # (one page of its own, for what follows)
    plain.maintain(["b"], [2], [n_b])
    assert len(plain.selector.cache.held[2]) == 3 and not plain.selector.cache.prints
    # what it reads is what it would have read from pages of its own
    q = cuda(bf16_round(rng.standard_normal((1, HQ, DH), dtype=np.float32)), torch.bfloat16)
    k = pool[int(table[2, n_b - 1])][None]
    step = index_space.key_and_query(q, k, geometry)
    for at in (n_b - 1, shared + 5, shared - 1, 700):
        position, row = torch.tensor([at], device="cuda"), torch.tensor([2], device="cuda")
        slots = table_d[2, at:at + 1].long()
        assert torch.equal(reuse.decode(step, position, slots, row), plain.decode(step, position, slots, row))
    # the same keys with one bit rewritten match nothing: a match compares the pool's bits
    pool.view(torch.int16)[int(table[3, 100]), 1, 40] ^= 1
    reuse.maintain(["c"], [3], [PAGE_SIZE])
    assert cache.held[3][0] not in cache.held[0] and cache.prints[3] != cache.prints[0][:1]
    # request a ends and its row goes to another: the prefix stays, and the newcomer takes it
    reuse.maintain(["d"], [0], [shared + 40])
    assert cache.held[0][:2] == cache.held[2][:2] and cache.holders[cache.held[2][0]] == 3 and len(cache.retained) == 1
