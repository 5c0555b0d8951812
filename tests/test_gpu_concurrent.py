"""Concurrent sequences on one sweep over the weights (l2j_batch_create / l2j_batch_forward) against the
single-sequence decode path: every sequence of a batch must see exactly its own history.

Gates (the batched path adds the row sums in another order than the decode kernels, so tolerances, written
here): logits within 1e-4 of the logit range of a decode-only context that ran the same sequence alone, same
arg-max; and within the north star's 1e-3 of the CPU checker.
"""
import numpy as np
import pytest

from llama2j_b200 import lib as L
from llama2j_b200 import synthetic as syn
from llama2j_b200.model_files import ModelConfig
from llama2j_b200.transformer import Transformer

pytestmark = pytest.mark.gpu

LOGIT_TOL = 1e-4
ORACLE_TOL = 1e-3


def _tensors(cfg, seed):
    tensors = syn.synthetic_tensors(cfg, seed)
    rng = np.random.default_rng(seed + 100)
    for t in (L.T_RMS_ATT, L.T_RMS_FFN, L.T_RMS_FINAL):
        tensors[t] = syn.quant_encode(rng.uniform(0.5, 1.5, cfg.tensor_floats(t)).astype(np.float32))
    return tensors


def _build(cfg, tensors):
    m = Transformer(cfg, 0, 0, None, 0)
    m.upload_all(tensors)
    m.finalize()
    return m


def _alone(cfg, tensors, stream):
    """Logits of every position of one forced token stream through the decode path."""
    m = _build(cfg, tensors)
    out = [m.forward(int(t), p)[0].copy() for p, t in enumerate(stream)]
    m.close()
    return out


def _check(got, ref):
    span = float(ref.max() - ref.min())
    assert float(np.abs(got - ref).max()) / span < LOGIT_TOL
    assert int(got.argmax()) == int(ref.argmax())


@pytest.mark.parametrize("cfg", [ModelConfig(256, 768, 3, 4, 4, 1000, 128, True),
                                 ModelConfig(512, 1280, 2, 8, 2, 1500, 128, False)], ids=["heads64", "grouped-query"])
def test_sequences_of_different_lengths_step_together(cfg):
    """Five sequences that start at different steps and have different tokens; one batch step per round."""
    tensors = _tensors(cfg, 11)
    rng = np.random.default_rng(12)
    n_seq, rounds = 5, 40
    starts = [0, 0, 3, 7, 20]                      # the round in which a sequence joins
    streams = [np.concatenate([[1], rng.integers(3, cfg.vocab_size, rounds)]).astype(np.int32) for _ in range(n_seq)]
    refs = [_alone(cfg, tensors, streams[s][:rounds - starts[s]]) for s in range(n_seq)]
    m = _build(cfg, tensors)
    m.batch_create(n_seq, 64)
    for r in range(rounds):
        live = [s for s in range(n_seq) if r >= starts[s]]
        pos = [r - starts[s] for s in live]
        toks = [int(streams[s][p]) for s, p in zip(live, pos)]
        logits, am = m.batch_forward(live, pos, toks)
        for i, (s, p) in enumerate(zip(live, pos)):
            _check(logits[i], refs[s][p])
            assert int(am[i]) == int(logits[i].argmax())
    assert m.stats().device_status == 0
    m.close()


def test_full_batch_of_64_at_the_110m_shape():
    cfg = syn.SHAPES["stories110M"]
    tensors = _tensors(cfg, 13)
    rng = np.random.default_rng(14)
    steps = 6
    streams = [np.concatenate([[1], rng.integers(3, cfg.vocab_size, steps)]).astype(np.int32) for _ in range(64)]
    m = _build(cfg, tensors)
    m.batch_create(64, 16)
    last = None
    for p in range(steps):
        last, _ = m.batch_forward(np.arange(64), np.full(64, p), [int(s[p]) for s in streams])
    m.close()
    for s in (0, 17, 63):
        _check(last[s], _alone(cfg, tensors, streams[s][:steps])[-1])


def test_a_prompt_in_slices_beside_decoding_sequences(oracle):
    """One call carries 40 positions of a new sequence's prompt and one position each of two running
    sequences; the checker runs every sequence alone."""
    cfg = ModelConfig(256, 768, 2, 4, 4, 800, 128, True)
    tensors = _tensors(cfg, 15)
    rng = np.random.default_rng(16)
    a = np.concatenate([[1], rng.integers(3, 800, 10)]).astype(np.int32)
    b = np.concatenate([[1], rng.integers(3, 800, 10)]).astype(np.int32)
    c = np.concatenate([[1], rng.integers(3, 800, 45)]).astype(np.int32)
    m = _build(cfg, tensors)
    m.batch_create(3, 64)
    for p in range(9):
        m.batch_forward([0, 1], [p, p], [int(a[p]), int(b[p])], want_logits=False)
    seq = [0, 1] + [2] * 40
    pos = [9, 9] + list(range(40))
    tok = [int(a[9]), int(b[9])] + [int(t) for t in c[:40]]
    logits, _ = m.batch_forward(seq, pos, tok)
    nxt, _ = m.batch_forward([2], [40], [int(c[40])])
    m.close()

    def checker(stream):
        om = oracle.OracleModel(cfg, tensors, oracle.SILU_EXACT, oracle.SOFTMAX_REFERENCE)
        out = [om.forward(int(t), p).copy() for p, t in enumerate(stream)]
        om.close()
        return out

    for got, ref in ((logits[0], checker(a[:10])[-1]), (logits[1], checker(b[:10])[-1]), (logits[41], checker(c[:40])[-1]),
                     (nxt[0], checker(c[:41])[-1])):
        span = float(ref.max() - ref.min())
        assert float(np.abs(got - ref).max()) / span < ORACLE_TOL
        assert int(got.argmax()) == int(ref.argmax())


def test_batch_argument_checks():
    cfg = ModelConfig(256, 768, 2, 4, 4, 500, 64, True)
    m = _build(cfg, _tensors(cfg, 17))
    with pytest.raises(L.L2jError):
        m.batch_forward([0], [0], [1])                       # before batch_create
    m.batch_create(2, 32)
    for seq, pos, tok in (([2], [0], [1]), ([0], [32], [1]), ([0], [0], [500]), ([0, 0], [3, 3], [1, 1])):
        with pytest.raises(L.L2jError):
            m.batch_forward(seq, pos, tok)
    m.batch_forward([], [], [])
    m.close()
    small = syn.SHAPES["stories15M"]
    s = _build(small, _tensors(small, 18))
    with pytest.raises(L.L2jError):
        s.batch_create(2, 32)                                 # rows that straddle quantisation groups
    s.close()
