"""Kernel-by-kernel comparison with the oracle, with the absolute thresholds of the reference's
TEST mode (Run.java:186-303): matMulI8 1e-3 (kernel/MatMul.java:275-276), matMulFP32 1e-4 (:253-254),
weight-normalise 1e-5 (kernel/WeightNormalizeAndScale.java:100), RoPE 1e-5 (kernel/ApplyRope.java:110-111),
softmax / weighted values 1e-5 (kernel/ExpSumNormalize.java:55-56, kernel/AccumWeightedValue.java:110),
SiLU 1e-5 (kernel/Silu.java:94).  Tighter relative bounds are added where the data allow."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _matvec_i8(l2j, groups, total, widx, n, d, x, flags=0):
    out = np.empty(d, dtype=np.float32)
    rc = l2j.load().l2j_k_matvec_i8(0, flags, groups.ctypes.data, total, widx, n, d, x.ctypes.data, out.ctypes.data)
    l2j.check(rc)
    return out


# (n, d, layer): the row lengths of all benchmark shapes; 288 makes rows straddle groups.
MATVEC_SHAPES = [(288, 288, 1), (288, 768, 2), (768, 288, 1), (768, 768, 0), (768, 2048, 1), (2048, 768, 1),
                 (4096, 600, 1), (11008, 300, 0), (5120, 333, 1), (13824, 130, 0), (4096, 2, 0), (4096, 3, 0), (256, 1, 0)]


@pytest.mark.parametrize("n,d,layer", MATVEC_SHAPES)
def test_matvec_i8_ring_and_plain(oracle, l2j, n, d, layer):
    rng = np.random.default_rng(n * 7 + d)
    total = (layer + 1) * n * d + 40                                # an odd tail after the matrix
    w = rng.normal(0, 0.02, total).astype(np.float32)
    groups = oracle.quant_encode(w)
    x = rng.normal(0, 1.0, n).astype(np.float32)
    ref = oracle.matmul_i8(groups, layer * n * d, n, d, x)
    for flags in (0, l2j.F_SIMPLE):
        got = _matvec_i8(l2j, groups, total, layer * n * d, n, d, x, flags)
        err = np.abs(got - ref).max()
        assert err < 1e-3, (flags, err)
        assert err < 2e-5 * np.abs(ref).max() + 1e-6, (flags, err, np.abs(ref).max())


def test_matvec_i8_unsupported_row_length_uses_plain_kernel(oracle, l2j):
    n, d = 100, 37                                                   # not a multiple of 16
    rng = np.random.default_rng(2)
    w = rng.normal(0, 0.02, n * d).astype(np.float32)
    groups = oracle.quant_encode(w)
    x = rng.normal(0, 1.0, n).astype(np.float32)
    got = _matvec_i8(l2j, groups, n * d, 0, n, d, x, 0)
    assert np.abs(got - oracle.matmul_i8(groups, 0, n, d, x)).max() < 1e-5


@pytest.mark.parametrize("n,d", [(288, 32000), (768, 32000), (4096, 3000), (5120, 1001), (4096, 1)])
def test_matvec_f32_and_argmax(oracle, l2j, n, d):
    rng = np.random.default_rng(n + d)
    w = rng.normal(0, 0.02, n * d).astype(np.float32)
    x = rng.normal(0, 1.0, n).astype(np.float32)
    if d > 10:
        w.reshape(d, n)[d // 2] = w.reshape(d, n)[d // 3]            # an exact tie: the lower index must win
    ref = oracle.matmul_f32(w, n, d, x)
    for flags in (0, l2j.F_SIMPLE):
        out = np.empty(d, dtype=np.float32)
        am = C.c_int(-1)
        l2j.check(l2j.load().l2j_k_matvec_f32(0, flags, w.ctypes.data, n, d, x.ctypes.data, out.ctypes.data, C.byref(am)))
        assert np.abs(out - ref).max() < 1e-4
        assert am.value == int(np.argmax(out))                        # first maximum of the device's own logits
        out2 = np.empty(d, dtype=np.float32)
        l2j.check(l2j.load().l2j_k_matvec_f32(0, flags, w.ctypes.data, n, d, x.ctypes.data, out2.ctypes.data, None))
        assert np.array_equal(out, out2)


def test_argmax_tie_lowest_index(l2j):
    n, d = 64, 4000
    w = np.zeros((d, n), dtype=np.float32)
    w[[700, 1500, 3999]] = 1.0
    x = np.ones(n, dtype=np.float32)
    out = np.empty(d, dtype=np.float32)
    am = C.c_int(-1)
    l2j.check(l2j.load().l2j_k_matvec_f32(0, 0, w.ctypes.data, n, d, x.ctypes.data, out.ctypes.data, C.byref(am)))
    assert am.value == 700


@pytest.mark.parametrize("n,layer", [(288, 3), (768, 1), (4096, 2)])
def test_rmsnorm(oracle, l2j, n, layer):
    rng = np.random.default_rng(n)
    total = (layer + 2) * n
    w = rng.uniform(0.5, 1.5, total).astype(np.float32)
    groups = oracle.quant_encode(w)
    x = rng.normal(0, 0.7, n).astype(np.float32)
    out = np.empty(n, dtype=np.float32)
    l2j.check(l2j.load().l2j_k_rmsnorm(0, groups.ctypes.data, total, layer * n, n, x.ctypes.data, out.ctypes.data))
    ref = oracle.rmsnorm_i8(groups, layer * n, x)
    assert np.abs(out - ref).max() < 1e-5


@pytest.mark.parametrize("dim,kv_dim,head,pos", [(288, 288, 48, 0), (288, 288, 48, 255), (768, 768, 64, 1023),
                                                  (4096, 4096, 128, 4095), (4096, 1024, 128, 77)])
def test_rope(oracle, l2j, dim, kv_dim, head, pos):
    rng = np.random.default_rng(pos + dim)
    q = rng.normal(0, 1, dim).astype(np.float32)
    k = rng.normal(0, 1, kv_dim).astype(np.float32)
    rq, rk = oracle.rope(q, k, pos, head)
    l2j.check(l2j.load().l2j_k_rope(0, q.ctypes.data, k.ctypes.data, pos, dim, kv_dim, head))
    assert np.abs(q - rq).max() < 1e-5 and np.abs(k - rk).max() < 1e-5


@pytest.mark.parametrize("heads,kv_heads,head,seq,pos", [
    (6, 6, 48, 256, 0), (6, 6, 48, 256, 1), (6, 6, 48, 256, 255), (12, 12, 64, 1024, 17), (12, 12, 64, 1024, 1023),
    (32, 32, 128, 4096, 300), (32, 8, 128, 4096, 2049), (8, 2, 32, 64, 63), (4, 4, 128, 4096, 4095)])
def test_attention(oracle, l2j, heads, kv_heads, head, seq, pos):
    rng = np.random.default_rng(heads * 1000 + pos)
    kv_dim = kv_heads * head
    q = rng.normal(0, 1.0, heads * head).astype(np.float32)
    kc = rng.normal(0, 0.5, (pos + 1) * kv_dim).astype(np.float32)
    vc = rng.normal(0, 1.0, (pos + 1) * kv_dim).astype(np.float32)
    out = np.empty(heads * head, dtype=np.float32)
    l2j.check(l2j.load().l2j_k_attention(0, q.ctypes.data, kc.ctypes.data, vc.ctypes.data, pos, heads, kv_heads, head, seq,
                                         out.ctypes.data))
    for mode in (oracle.SOFTMAX_TRUE, oracle.SOFTMAX_REFERENCE):
        ref = oracle.attention(q, kc, vc, pos, heads, kv_heads, head, mode)
        assert np.abs(out - ref).max() < 1e-5, mode


def test_swiglu(oracle, l2j):
    rng = np.random.default_rng(9)
    n = 11008
    hb = rng.normal(0, 2.0, n).astype(np.float32)
    hb[:8] = [0.0, -0.0, 30.0, -30.0, 88.0, -88.0, 1e-20, -100.0]
    hb2 = rng.normal(0, 1.0, n).astype(np.float32)
    ref = oracle.silu(hb, hb2, oracle.SILU_EXACT)
    got = hb.copy()
    l2j.check(l2j.load().l2j_k_swiglu(0, got.ctypes.data, hb2.ctypes.data, n))
    assert np.abs(got - ref).max() < 1e-5
    assert np.abs(got - ref).max() <= 4e-7 * np.abs(ref).max()
    lookup = oracle.silu(hb, hb2, oracle.SILU_LOOKUP)               # the CPU path's table: reported, looser
    assert np.abs(got - lookup).max() < 5e-3


def test_bad_arguments_are_rejected_on_the_host(l2j):
    lib = l2j.load()
    x = np.zeros(16, dtype=np.float32)
    assert lib.l2j_k_swiglu(0, None, x.ctypes.data, 16) == l2j.E_INVALID
    assert lib.l2j_k_rope(0, x.ctypes.data, x.ctypes.data, -1, 16, 16, 8) == l2j.E_INVALID
    assert lib.l2j_k_attention(0, x.ctypes.data, x.ctypes.data, x.ctypes.data, 70, 1, 1, 16, 64, x.ctypes.data) == l2j.E_INVALID
    assert lib.l2j_k_matvec_i8(5000, 0, x.ctypes.data, 16, 0, 16, 1, x.ctypes.data, x.ctypes.data) == l2j.E_INVALID
