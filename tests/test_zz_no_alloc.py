"""The allocation-free attention entry point against the regular one.

This file sorts last on purpose: if it fails under `-x`, every other test has already run.  The
entry point exists for hosts that may not allocate device memory while running (their memory pool
is owned by another allocator, or cudaMalloc's hidden synchronisation is not acceptable in their
loop); it works out of a fixed array inside the library, so it is called twice in a row here, with
different sizes, to show that what the first call leaves in that array does not leak into the second.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _reference(l2j, q, k_dev, v_dev, pos, heads, kv_heads, head, seq):
    """The existing entry point: host arrays, caches in the reference's (position, kv_dim) layout."""
    k_ref = np.ascontiguousarray(k_dev[:, :pos + 1, :].transpose(1, 0, 2)).reshape(-1)
    v_ref = np.ascontiguousarray(v_dev[:, :pos + 1, :].transpose(1, 0, 2)).reshape(-1)
    out = np.empty(heads * head, dtype=np.float32)
    l2j.check(l2j.load().l2j_k_attention(0, q.ctypes.data, k_ref.ctypes.data, v_ref.ctypes.data, pos, heads, kv_heads, head,
                                         seq, out.ctypes.data))
    return out


def _no_alloc(l2j, torch, q, k_dev, v_dev, pos, heads, kv_heads, head, seq):
    dq = torch.from_numpy(q).cuda()
    dk = torch.from_numpy(k_dev).cuda()
    dv = torch.from_numpy(v_dev).cuda()
    dout = torch.full((heads * head,), float("nan"), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    rc = l2j.load().l2j_k_attention_noalloc(0, dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), pos, heads, kv_heads, head, seq,
                                            dout.data_ptr(), None)
    assert rc == 0, l2j.load().l2j_noalloc_last_error()
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    return dout.cpu().numpy()


def test_no_alloc_attention_matches_regular_entry_point_twice(l2j):
    import torch
    rng = np.random.default_rng(77)
    # two calls in a row: many splits first, then a short one that uses a single block per head
    for (heads, kv_heads, head, seq, pos) in [(32, 8, 128, 4096, 1500), (12, 12, 64, 1024, 37), (32, 8, 128, 4096, 1500)]:
        q = rng.normal(0, 1.0, heads * head).astype(np.float32)
        k = rng.normal(0, 0.5, (kv_heads, seq, head)).astype(np.float32)
        v = rng.normal(0, 1.0, (kv_heads, seq, head)).astype(np.float32)
        want = _reference(l2j, q, k, v, pos, heads, kv_heads, head, seq)
        got = _no_alloc(l2j, torch, q, k, v, pos, heads, kv_heads, head, seq)
        assert np.isfinite(got).all()
        assert np.abs(got - want).max() < 1e-5          # the tolerance of the attention parity tests
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))   # same kernel, same split: same bits


def test_no_alloc_attention_rejects_what_the_fixed_scratch_cannot_hold(l2j):
    import torch
    lib = l2j.load()
    x = torch.zeros(1 << 16, dtype=torch.float32, device="cuda")
    p = x.data_ptr()
    assert lib.l2j_k_attention_noalloc(0, p, p, p, 3, 256, 256, 64, 64, p, None) == l2j.E_INVALID   # too many heads
    assert b"at most 128 heads" in lib.l2j_noalloc_last_error()
    assert lib.l2j_k_attention_noalloc(0, p, p, p, 3, 4, 4, 256, 64, p, None) == l2j.E_INVALID      # head too wide
    assert lib.l2j_k_attention_noalloc(0, p, p, p, 64, 4, 4, 64, 64, p, None) == l2j.E_INVALID      # position outside the cache
    assert lib.l2j_k_attention_noalloc(0, None, p, p, 3, 4, 4, 64, 64, p, None) == l2j.E_INVALID
