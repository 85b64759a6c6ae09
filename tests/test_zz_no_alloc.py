"""The allocation-free attention entry point, `lsa_sparse_attend_static`, against `lsa_sparse_attend`.

Some hosts of this library cannot allocate device memory when they call it (an engine that gave every free byte
to its KV pool, a plugin thread with pointers but no allocator), so the split read's scratch sits in a static
device array inside the library. Both entry points run the same kernels, so through the C ABI their outputs must
agree (the suite's bf16 tolerance is the bound; equality is what is expected), on two calls in a row whose second
has other inputs, which also shows that nothing the first call left in the shared array leaks into the second.
This file is named to be collected last.
"""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(seed, R, T, Hq, Hkv, dh, L):
    gen = torch.Generator().manual_seed(seed)
    q = torch.randn(R, Hq, dh, generator=gen).bfloat16().cuda()
    k = torch.randn(T, Hkv, dh, generator=gen).bfloat16().cuda()
    v = torch.randn(T, Hkv, dh, generator=gen).bfloat16().cuda()
    ids = torch.stack([torch.randperm(T, generator=gen)[:L] for _ in range(R)]).to(torch.int32).cuda()
    lengths = torch.randint(L // 2, L + 1, (R,), generator=gen).to(torch.int32).cuda()
    lengths[0] = 0
    return q, k, v, ids, lengths


def _static(q, k, v, ids, lengths, scale, splits):
    from lsa_b200._lib import call, ptr, stream

    R, Hq, dh = q.shape
    out = torch.empty(R, Hq, dh, device=q.device, dtype=torch.float32)
    lse = torch.empty(R, Hq, device=q.device, dtype=torch.float32)
    call("lsa_sparse_attend_static", ptr(q), R, Hq, dh, q.stride(0), q.stride(1), ptr(k), ptr(v), k.shape[0],
         0, k.shape[1], k.stride(0), k.stride(1), ptr(ids), ids.shape[1], ptr(lengths), scale, splits, None, ptr(out),
         ptr(lse), stream(), launches=2 if splits > 1 else 1)
    return out, lse


def test_the_static_scratch_entry_point_matches_the_workspace_one_twice_in_a_row():
    from lsa_b200 import _lib, ops

    assert _lib.query("lsa_sparse_attend_static_scratch_bytes") == 8 << 20
    for seed, (R, T, Hq, Hkv, dh, L, splits) in enumerate([(4, 6000, 40, 8, 128, 3000, 8),
                                                           (3, 2500, 8, 2, 64, 700, 5)]):
        q, k, v, ids, lengths = _case(seed, R, T, Hq, Hkv, dh, L)
        scale = dh ** -0.5
        want, want_lse = ops.sparse_attend(q, k, v, ids, lengths, scale, splits=splits, out_dtype=torch.float32)
        got, got_lse = _static(q, k, v, ids, lengths, scale, splits)
        torch.cuda.synchronize()
        assert (got - want).abs().max().item() <= 2e-2
        assert torch.equal(got, want) and torch.equal(got_lse, want_lse)
        assert not got[0].any() and torch.isinf(got_lse[0]).all()


def test_a_call_past_the_static_scratch_is_refused_with_its_own_error():
    q, k, v, ids, lengths = _case(7, 64, 512, 40, 8, 128, 64)
    # 64 rows x 40 heads x 129 floats x 32 splits = 42 MB of partial results: more than the array holds
    with pytest.raises(ValueError, match="static array"):
        _static(q, k, v, ids, lengths, 0.1, 32)
