"""CPU checks of the oracle itself: the reference's own quantiser check, hand-derived known answers,
an independent float64 model, and the committed regression vectors."""
import os
from fractions import Fraction

import numpy as np
import pytest

from llama2j_b200.model_files import ModelConfig
from tests.np_model import NumpyModel, dequant

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "oracle_golden.npz")
TINY = ModelConfig(dim=64, hidden_dim=176, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=96, seq_len=32,
                   shared_classifier=False)


def test_quant_main_vector(oracle):
    """Quant.main (Quant.java:69-77) encodes the floats 0..99; every byte has a closed form."""
    x = np.arange(100, dtype=np.float32)
    enc = oracle.quant_encode(x)
    assert enc.size == 264
    assert bytes(enc[0:4]) == b"\x00\x00\x00\x00"            # min 0.0, big-endian
    assert bytes(enc[4:8]) == b"\x42\xc6\x00\x00"            # max 99.0 = 0x42C60000, big-endian
    for i in range(100):
        exact = Fraction(i, 99) * 255
        lo, hi = int(exact), int(exact) + 1
        assert enc[8 + i] in (lo, hi)                         # float rounding may move a .5 case by one
        t = np.float32(np.float32(np.float32(i) / np.float32(99.0)) * np.float32(255.0))
        assert enc[8 + i] == int(np.floor(np.float64(t) + 0.5))
    assert not enc[108:].any()                                # padding of the partial group is zero
    # The reference's own acceptance rule flags the coarse small values of this ramp (its main()
    # logs them); the count must agree with the rule evaluated independently in float64.
    dec = enc[8:108].astype(np.float64) / 255.0 * 99.0
    diff = np.abs(dec - x)
    with np.errstate(divide="ignore", invalid="ignore"):
        expected = int(np.sum((diff / np.abs(x) > 0.01) & (diff > 1e-2)))
    assert oracle.load().l2jo_quant_roundtrip_violations(x.ctypes.data, 100) == expected


def test_quant_roundtrip_rule_random(oracle):
    """The acceptance rule of Quant.testEncode (Quant.java:118-154) on N(0, 0.02) data."""
    x = np.random.default_rng(3).normal(0, 0.02, 50_000).astype(np.float32)
    assert oracle.load().l2jo_quant_roundtrip_violations(x.ctypes.data, x.size) == 0
    dec = oracle.quant_decode(oracle.quant_encode(x), x.size)
    step = (x.reshape(-1, 250)[:1].max() - x.min())   # loose bound: half a quantisation step of the widest group
    assert np.abs(dec - x).max() <= 0.5 * (x.max() - x.min()) / 255 * 1.001 + 1e-9
    assert step > 0


def test_quant_edge_cases(oracle):
    const = np.full(300, 1.0, dtype=np.float32)              # RMSNorm weights of the synthetic checkpoints
    enc = oracle.quant_encode(const)
    assert enc.size == 528
    assert bytes(enc[0:8]) == b"\x3f\x80\x00\x00\x3f\x80\x00\x00"
    assert not enc[8:264].any() and not enc[272:].any()      # 0/0 = NaN -> Math.round(NaN) = 0
    assert np.all(oracle.quant_decode(enc, 300) == 1.0)      # 0/255*0 + min
    x = np.array([0.0, -0.0, 0.0], dtype=np.float32)         # first occurrence wins ties: +0 stays
    assert bytes(oracle.quant_encode(x)[0:8]) == b"\x00" * 8
    x = np.array([-0.0, 0.0], dtype=np.float32)
    assert bytes(oracle.quant_encode(x)[0:8]) == b"\x80\x00\x00\x00\x80\x00\x00\x00"
    ramp = np.linspace(-1, 1, 256, dtype=np.float32)
    e = oracle.quant_encode(ramp)
    assert e[8] == 0 and e[8 + 255] == 255
    assert np.all(np.diff(e[8:].astype(int)) >= 0)


def test_matmul_i8_matches_float64_and_straddles_groups(oracle):
    rng = np.random.default_rng(5)
    for (n, d, layer) in [(288, 288, 1), (768, 40, 2), (256, 16, 0), (304, 7, 3)]:
        total = (layer + 1) * n * d
        w = rng.normal(0, 0.02, total).astype(np.float32)
        enc = oracle.quant_encode(w)
        x = rng.normal(0, 1, n).astype(np.float32)
        got = oracle.matmul_i8(enc, layer * n * d, n, d, x)
        wd = dequant(enc, total)[layer * n * d:].reshape(d, n)
        ref = wd @ x.astype(np.float64)
        assert np.abs(got - ref).max() < 2e-5 * np.abs(ref).max() + 1e-6


def test_forward_matches_independent_float64_model(oracle):
    tensors = oracle.synthetic_tensors(TINY, seed=7)
    tensors[oracle.T_RMS_ATT] = oracle.quant_encode(np.random.default_rng(1).uniform(0.5, 1.5, TINY.n_layers * TINY.dim))
    tensors[oracle.T_RMS_FFN] = oracle.quant_encode(np.random.default_rng(2).uniform(0.5, 1.5, TINY.n_layers * TINY.dim))
    om = oracle.OracleModel(TINY, tensors, oracle.SILU_EXACT, oracle.SOFTMAX_REFERENCE)
    nm = NumpyModel(TINY, tensors)
    toks = [1, 17, 3, 90, 45, 45, 8, 2, 60, 33]
    for pos, tok in enumerate(toks):
        a = om.forward(tok, pos).astype(np.float64)
        b = nm.forward(tok, pos)
        assert np.abs(a - b).max() < 2e-5 * (b.max() - b.min())


def test_mode_switches_are_small(oracle):
    """Lookup-table SiLU (CPU path) vs exact (CUDA order) and reference vs true softmax shift differ
    only at the levels the reference's two paths differ from each other."""
    tensors = oracle.synthetic_tensors(TINY, seed=7)
    base = oracle.OracleModel(TINY, tensors, oracle.SILU_EXACT, oracle.SOFTMAX_REFERENCE)
    lookup = oracle.OracleModel(TINY, tensors, oracle.SILU_LOOKUP, oracle.SOFTMAX_REFERENCE)
    true_max = oracle.OracleModel(TINY, tensors, oracle.SILU_EXACT, oracle.SOFTMAX_TRUE)
    for pos, tok in enumerate([1, 5, 9, 70, 12]):
        a, b, c = base.forward(tok, pos).copy(), lookup.forward(tok, pos).copy(), true_max.forward(tok, pos).copy()
        rng_ = a.max() - a.min()
        assert np.abs(a - b).max() < 1e-3 * rng_
        assert np.abs(a - c).max() < 1e-5 * rng_
    h = np.linspace(-6, 6, 1001, dtype=np.float32)
    one = np.ones_like(h)
    assert np.abs(oracle.silu(h, one, oracle.SILU_LOOKUP) - oracle.silu(h, one, oracle.SILU_EXACT)).max() < 4e-4 * 6


def test_argmax_first_maximum(oracle):
    assert oracle.argmax(np.array([1, 3, 3, 2], dtype=np.float32)) == 1
    assert oracle.argmax(np.array([5, 5, 5], dtype=np.float32)) == 0


def test_synthetic_generator_is_normal_and_counter_based(oracle):
    a = oracle.synth_normal(400_000, seed=0, stream=2, scale=1.0)
    assert abs(a.mean()) < 0.01 and abs(a.std() - 1.0) < 0.01
    kurt = ((a - a.mean()) ** 4).mean() / a.var() ** 2
    assert abs(kurt - 3.0) < 0.05
    b = oracle.synth_normal(1000, seed=0, stream=2, start=1234, scale=1.0)
    assert np.array_equal(a[1234:2234], b)                   # any slice can be regenerated on its own
    assert not np.array_equal(a[:1000], oracle.synth_normal(1000, seed=0, stream=3, scale=1.0))
    q = oracle.synth_quant(256 * 9 + 40, seed=0, stream=2)
    assert np.array_equal(q, oracle.quant_encode(oracle.synth_normal(256 * 9 + 40, seed=0, stream=2)))


def test_golden_regression(oracle):
    """Committed vectors made by tests/golden/make_golden.py from this oracle (the reference ships
    none): they pin the oracle against accidental change, not against the reference."""
    g = np.load(GOLDEN)
    assert np.array_equal(oracle.quant_encode(g["quant_in"]), g["quant_out"])
    assert np.array_equal(oracle.synth_normal(64, seed=0, stream=2), g["synth"])
    tensors = oracle.synthetic_tensors(TINY, seed=11)
    m = oracle.OracleModel(TINY, tensors, oracle.SILU_EXACT, oracle.SOFTMAX_REFERENCE)
    toks, lgs = oracle.greedy_run(m, g["prompt"], int(g["steps"]))
    assert np.array_equal(toks, g["tokens"])
    assert np.abs(lgs - g["logits"]).max() <= 1e-6


# ---- Sampler.java + java.util.Random restated (token choice for --temp > 0) ------------------------------

def test_java_random_known_answers(oracle):
    """java.util.Random is specified bit for bit (48-bit LCG, seed scrambled with 0x5DEECE66D); these are the
    values every JDK prints for new Random(42).nextInt() twice and new Random(0).nextInt()."""
    s = oracle.Sampler(42, 4)
    assert s.next_int() == -1170105035
    assert s.next_int() == 234785527
    s.close()
    s = oracle.Sampler(0, 4)
    assert s.next_int() == -1155484576
    s.close()
    s = oracle.Sampler(42, 4)
    assert abs(s.next_float() - 0.7275637) < 5e-8     # new Random(42).nextFloat()
    s.close()


def _python_java_random(seed):
    state = (seed ^ 0x5DEECE66D) & ((1 << 48) - 1)
    while True:
        state = (state * 0x5DEECE66D + 0xB) & ((1 << 48) - 1)
        yield np.float32(state >> 24) / np.float32(1 << 24)


def test_sampler_plain_follows_the_cumulative_walk(oracle):
    """Sampler.sample (Sampler.java:33-44) from an independent restatement in numpy float32."""
    rng = np.random.default_rng(0)
    n = 500
    s = oracle.Sampler(2024, n)
    draws = _python_java_random(2024)
    for _ in range(50):
        logits = rng.standard_normal(n).astype(np.float32) * np.float32(3)
        t = np.float32(0.8)
        x = logits / t
        e = np.exp((x - x.max()).astype(np.float64)).astype(np.float32)
        tot = np.float32(0)
        for v in e:
            tot = np.float32(tot + v)
        p = e / tot
        r = next(draws)
        cdf, want = np.float32(0), n - 1
        for i, v in enumerate(p):
            cdf = np.float32(cdf + v)
            if r < cdf:
                want = i
                break
        assert s.sample(logits.copy(), 0.8, 1.0) == want
    s.close()


def test_sampler_top_p_keeps_the_nucleus(oracle):
    """Sampler.sample_topp (Sampler.java:76-120): only tokens of the smallest prefix (by descending probability)
    whose mass exceeds topp can be chosen; a one-hot distribution always returns its token."""
    n = 64
    s = oracle.Sampler(5, n)
    logits = np.full(n, -30.0, dtype=np.float32)
    logits[17] = 10.0
    for _ in range(20):
        assert s.sample(logits.copy(), 1.0, 0.9) == 17
    base = np.linspace(0.0, 6.0, n).astype(np.float32)
    p = np.exp(base - base.max())
    p /= p.sum()
    order = np.argsort(-p, kind="stable")
    k = int(np.searchsorted(np.cumsum(p[order]), 0.5)) + 1
    allowed = set(int(i) for i in order[:k + 1])
    seen = set()
    for _ in range(300):
        t = s.sample(base.copy(), 1.0, 0.5)
        assert t in allowed
        seen.add(t)
    assert len(seen) > 1
    s.close()
