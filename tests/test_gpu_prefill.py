"""Batched prompt processing (l2j_prefill) against the decode path it replaces and against the CPU checker.

The reference pushes every prompt token through the decode step (Run.java:623-637); l2j_prefill runs 64
positions per sweep over the weights on the tensor cores.  Per position it computes the decode step's
arithmetic with the row sums added in another order, so the gates are tolerances, written here: the K/V
cache rows the prompt leaves behind within 1e-4 of the row's largest magnitude, and the logits of the decode
step after the prompt within 1e-4 of the logit range of the decode-only path (and within the 1e-3 of the
north star against the CPU checker), same arg-max.
"""
import numpy as np
import pytest

from llama2j_b200 import lib as L
from llama2j_b200 import synthetic as syn
from llama2j_b200.model_files import ModelConfig
from llama2j_b200.transformer import Transformer

pytestmark = pytest.mark.gpu

CACHE_TOL = 1e-4     # of the row's largest magnitude
LOGIT_TOL = 1e-4     # of the logit range, prefill + decode step against decode only
ORACLE_TOL = 1e-3    # of the logit range, against the CPU checker (north star)


def _tensors(cfg, seed):
    tensors = syn.synthetic_tensors(cfg, seed)
    rng = np.random.default_rng(seed + 100)
    for t in (L.T_RMS_ATT, L.T_RMS_FFN, L.T_RMS_FINAL):
        tensors[t] = syn.quant_encode(rng.uniform(0.5, 1.5, cfg.tensor_floats(t)).astype(np.float32))
    return tensors


def _build(cfg, tensors, flags=0):
    m = Transformer(cfg, 0, 0, None, flags)
    m.upload_all(tensors)
    m.finalize()
    return m


def _inputs(cfg, n, seed=3):
    """BOS and then the prompt: the token fed at each of the first n positions (Run.java:614,635-637)."""
    return np.concatenate([[1], syn.synthetic_prompt(n - 1, seed, cfg.vocab_size)]).astype(np.int32)


def _compare_with_decode(cfg, tensors, n, positions, layers, next_token=7):
    toks = _inputs(cfg, n)
    dec = _build(cfg, tensors)
    for i in range(n):
        dec.forward(int(toks[i]), i, want_logits=False)
    pre = _build(cfg, tensors)
    pre.prefill(toks, 0)
    assert pre.prefill_launches() > 0, "the tensor-core path did not run"
    worst = 0.0
    for layer in layers:
        for pos in positions:
            for which in (5, 6):
                a = dec.read_buffer(which, cfg.kv_dim, layer, pos)
                b = pre.read_buffer(which, cfg.kv_dim, layer, pos)
                worst = max(worst, float(np.abs(a - b).max()) / float(np.abs(a).max()))
    ref = dec.forward(next_token, n)[0].copy()
    got = pre.forward(next_token, n)[0].copy()
    status = (dec.stats().device_status, pre.stats().device_status)
    dec.close()
    pre.close()
    assert status == (0, 0)
    assert worst < CACHE_TOL, worst
    span = float(ref.max() - ref.min())
    assert float(np.abs(got - ref).max()) / span < LOGIT_TOL
    assert int(got.argmax()) == int(ref.argmax())
    return got


def test_prefill_512_tokens_110m_shape():
    cfg = syn.SHAPES["stories110M"]      # head size 64, K/V rows of 768, three groups per row
    _compare_with_decode(cfg, _tensors(cfg, 1), 512, (0, 1, 63, 64, 300, 511), (0, 5, 11))


def test_prefill_512_tokens_7b_shape():
    cfg = syn.SHAPES["llama2-7b"]
    _compare_with_decode(cfg, _tensors(cfg, 2), 512, (0, 63, 64, 511), (0, 31))


def test_prefill_ragged_lengths_and_continuation():
    """Lengths that are not multiples of 64, a second call that continues at pos0 > 0, grouped-query heads."""
    cfg = ModelConfig(512, 1280, 3, 8, 2, 1000, 512, True)      # 8 query heads on 2 K/V heads of 64
    tensors = _tensors(cfg, 4)
    toks = _inputs(cfg, 203)
    dec = _build(cfg, tensors)
    for i in range(203):
        dec.forward(int(toks[i]), i, want_logits=False)
    ref = dec.forward(9, 203)[0].copy()
    for first in (1, 63, 65, 130):
        pre = _build(cfg, tensors)
        pre.prefill(toks[:first], 0)
        pre.prefill(toks[first:], first)
        got = pre.forward(9, 203)[0].copy()
        for pos in (0, first - 1, first, 202):
            a, b = dec.read_buffer(5, cfg.kv_dim, 2, pos), pre.read_buffer(5, cfg.kv_dim, 2, pos)
            assert float(np.abs(a - b).max()) / float(np.abs(a).max()) < CACHE_TOL, (first, pos)
        assert pre.stats().device_status == 0
        pre.close()
        assert float(np.abs(got - ref).max()) / float(ref.max() - ref.min()) < LOGIT_TOL, first
    dec.close()


def test_prefill_then_decode_against_the_checker(oracle):
    """A 100-token prompt through l2j_prefill, then greedy decoding: logits of every decoded position within
    the north star's 1e-3 of range of the CPU checker that ran the whole sequence token by token."""
    cfg = ModelConfig(256, 768, 4, 4, 4, 2000, 256, True)
    tensors = _tensors(cfg, 5)
    toks = _inputs(cfg, 100)
    pre = _build(cfg, tensors)
    pre.prefill(toks, 0)
    om = oracle.OracleModel(cfg, tensors, oracle.SILU_EXACT, oracle.SOFTMAX_REFERENCE)
    for i in range(100):
        om.forward(int(toks[i]), i)
    token = 11
    for pos in range(100, 132):
        got = pre.forward(token, pos)[0].copy()
        ref = om.forward(token, pos).copy()
        span = float(ref.max() - ref.min())
        assert float(np.abs(got - ref).max()) / span < ORACLE_TOL, pos
        assert int(got.argmax()) == int(ref.argmax()), pos
        token = int(ref.argmax())
    om.close()
    pre.close()


def test_shapes_outside_the_tensor_core_path_use_the_decode_step():
    """Rows that straddle quantisation groups (15M shape): the prompt goes through the decode step, bitwise."""
    cfg = syn.SHAPES["stories15M"]
    tensors = _tensors(cfg, 6)
    toks = _inputs(cfg, 40)
    dec = _build(cfg, tensors)
    for i in range(40):
        dec.forward(int(toks[i]), i, want_logits=False)
    ref = dec.forward(5, 40)[0].copy()
    dec.close()
    pre = _build(cfg, tensors)
    pre.prefill(toks, 0)
    assert pre.prefill_launches() == 0
    got = pre.forward(5, 40)[0].copy()
    pre.close()
    assert np.array_equal(got, ref)


def test_prefill_argument_checks():
    cfg = ModelConfig(256, 768, 2, 4, 4, 500, 128, True)
    m = _build(cfg, _tensors(cfg, 7))
    with pytest.raises(L.L2jError):
        m.prefill(np.arange(3, 133, dtype=np.int32), 0)          # 130 positions in a sequence of 128
    with pytest.raises(L.L2jError):
        m.prefill(np.array([1, 500], dtype=np.int32), 0)          # token outside the vocabulary
    m.prefill(np.array([], dtype=np.int32), 0)
    m.close()
