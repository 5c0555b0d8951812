"""Load-time device code against the oracle, bit for bit: the quantiser (Quant.encode) and the
synthetic-checkpoint generator."""
import numpy as np
import pytest

from llama2j_b200 import synthetic as syn

pytestmark = pytest.mark.gpu


def test_quant_encode_bit_exact_random(oracle, l2j):
    rng = np.random.default_rng(0)
    for n in (256, 256 * 33 + 17, 1, 255, 257, 288 * 6, 1_000_003):
        x = rng.normal(0, 0.02, n).astype(np.float32)
        assert np.array_equal(syn.quant_encode(x), oracle.quant_encode(x)), n


def test_quant_encode_bit_exact_edge_cases(oracle, l2j):
    cases = [
        np.ones(300, dtype=np.float32),                                  # constant group: 0/0 -> byte 0
        np.arange(100, dtype=np.float32),                                # the vector of Quant.main
        np.array([0.0, -0.0, 0.0, -0.0] * 64, dtype=np.float32),         # signed zeros: first occurrence wins
        np.array([-0.0, 0.0] * 128, dtype=np.float32),
        np.linspace(-1, 1, 256, dtype=np.float32),
        np.concatenate([np.full(255, 0.25, np.float32), [0.75]]).astype(np.float32),
        (np.arange(512) % 2).astype(np.float32) * 1e-30,                 # tiny range
        np.array([3.0e38, -3.0e38] + [0.0] * 254, dtype=np.float32),     # range overflows to inf
        np.array([1.0, np.nan, 2.0, 0.5] + [1.5] * 252, dtype=np.float32),   # NaN after the first element is skipped
        np.array([np.nan, 1.0, 2.0] + [1.5] * 253, dtype=np.float32),    # NaN first poisons min and max
        np.array([np.inf, 1.0] + [2.0] * 254, dtype=np.float32),
    ]
    rng = np.random.default_rng(1)
    halves = np.concatenate([[0.0, 255.0], rng.integers(0, 255, 254) + 0.5]).astype(np.float32)
    cases.append(halves)                                                 # values on the .5 rounding boundary
    for i, x in enumerate(cases):
        got, ref = syn.quant_encode(x), oracle.quant_encode(x)
        assert np.array_equal(got, ref), f"case {i}: first diff at {np.flatnonzero(got != ref)[:5]}"


def test_synthetic_generator_bit_exact(oracle, l2j):
    for (n, seed, stream, start) in [(100_000, 0, 2, 0), (4097, 0, 7, 123_456_789), (1000, 5, 0, 6_000_000_000), (1 << 20, 0, 11, 0)]:
        got = syn.synth_f32(n, seed, stream, start=start)
        ref = oracle.synth_normal(n, seed, stream, start=start)
        assert np.array_equal(got.view(np.uint32), ref.view(np.uint32)), (n, seed, stream, start)


def test_synth_quant_equals_oracle(oracle, l2j):
    n = 256 * 1000 + 40
    assert np.array_equal(syn.synth_quant(n, 0, 3), oracle.synth_quant(n, 0, 3))


def test_synthetic_checkpoint_equals_oracle_checkpoint(oracle, l2j):
    cfg = syn.SHAPES["stories15M"]
    a = syn.synthetic_tensors(cfg, seed=0)
    b = oracle.synthetic_tensors(cfg, seed=0)
    assert sorted(a) == sorted(b)
    for t in a:
        assert np.array_equal(a[t].view(np.uint8), b[t].view(np.uint8)), t
