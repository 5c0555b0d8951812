"""Failure detection without a GPU fault: a device-side wait that runs out is reported, not hung on.

The failure is injected on the host (l2j_debug_desync advances the context's forward counter as if a
partner had run a forward that this context missed), so the hand-over counters of the next forward never
reach their targets.  Every wait in the kernels is bounded: the forward ends by its limit, the call
returns L2J_E_DEVICE with L2J_DS_WAIT_TIMEOUT in the status word, the status stays raised until
l2j_reset, and after the reset the context computes the same logits as before.  The reference has no
counterpart beyond the exception of ContextCUDA.java:296-304."""
import time

import numpy as np
import pytest

from llama2j_b200 import lib as L
from llama2j_b200 import synthetic as syn
from llama2j_b200.model_files import ModelConfig
from llama2j_b200.transformer import LinkedStages, Transformer

pytestmark = pytest.mark.gpu


def _build(cfg, tensors, flags=0, first=0, last=None, limit_us=None):
    m = Transformer(cfg, 0, first, last, flags)
    if limit_us is not None:
        m.set_wait_limit_us(limit_us)
    m.upload_all(tensors)
    m.finalize()
    return m


@pytest.mark.parametrize("flags,kernels", [(L.F_PERSISTENT, "persistent"), (L.F_STEP_KERNELS, "per-step")])
def test_wait_runs_out_is_reported_and_reset_recovers(flags, kernels):
    cfg = ModelConfig(dim=512, hidden_dim=1536, n_layers=3, n_heads=8, n_kv_heads=8, vocab_size=2048, seq_len=64,
                      shared_classifier=False)
    tensors = syn.synthetic_tensors(cfg, 2)
    m = _build(cfg, tensors, flags, limit_us=500)
    assert m.stats().kernels_per_forward == (3 if kernels == "persistent" else 2 + 5 * cfg.n_layers)
    good = [m.forward(t, p)[0].copy() for p, t in enumerate((1, 17, 400))]

    m.debug_desync()
    t0 = time.perf_counter()
    with pytest.raises(L.L2jError) as e:
        m.forward(1, 0)
    assert time.perf_counter() - t0 < 5.0                       # ended by the wait limit, not by a watchdog
    assert e.value.code == L.E_DEVICE
    assert m.stats().device_status & L.DS_WAIT_TIMEOUT
    with pytest.raises(L.L2jError) as e:                         # sticky until the reset
        m.forward(17, 1)
    assert e.value.code == L.E_DEVICE

    m.reset()
    assert m.stats().device_status == 0
    again = [m.forward(t, p)[0].copy() for p, t in enumerate((1, 17, 400))]
    for a, b in zip(good, again):
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    m.close()


def test_wait_limit_is_fixed_at_finalize():
    cfg = ModelConfig(dim=256, hidden_dim=512, n_layers=1, n_heads=4, n_kv_heads=4, vocab_size=256, seq_len=16,
                      shared_classifier=True)
    m = _build(cfg, syn.synthetic_tensors(cfg, 1))
    with pytest.raises(L.L2jError) as e:
        m.set_wait_limit_us(100)
    assert e.value.code == L.E_STATE
    m.close()
    m = Transformer(cfg)
    with pytest.raises(L.L2jError) as e:
        m.set_wait_limit_us(1)
    assert e.value.code == L.E_INVALID
    m.close()


def test_layer_split_needs_the_link():
    """l2j_pipeline_forward on stages that were never linked (or whose partner is gone) answers L2J_E_STATE
    instead of handing the begin kernel a null peer pointer."""
    cfg = ModelConfig(dim=256, hidden_dim=512, n_layers=2, n_heads=4, n_kv_heads=4, vocab_size=256, seq_len=16,
                      shared_classifier=False)
    tensors = syn.synthetic_tensors(cfg, 1)
    a = _build(cfg, tensors, first=0, last=0)
    b = _build(cfg, tensors, first=1, last=1)
    stages = LinkedStages([a, b], link=False)
    with pytest.raises(L.L2jError) as e:
        stages.forward(1, 0)
    assert e.value.code == L.E_STATE
    with pytest.raises(L.L2jError) as e:
        stages.generate_greedy([5, 6], 4)
    assert e.value.code == L.E_STATE
    stages.link()
    lg, _ = stages.forward(1, 0)
    assert np.isfinite(lg).all()
    # a third context takes stage b's place: the old link no longer holds for (a, c)
    c = _build(cfg, tensors, first=1, last=1)
    other = LinkedStages([a, c], link=False)
    with pytest.raises(L.L2jError) as e:
        other.forward(1, 0)
    assert e.value.code == L.E_STATE
    c.close()
    b.close()                                                   # destroying a member unlinks its partner
    rest = LinkedStages([a], link=False)                        # `a` alone does not tile the layers either
    with pytest.raises(L.L2jError):
        rest.forward(1, 0)
    a.close()


def test_duplicate_part_cannot_stand_in_for_a_missing_one():
    """A tensor uploaded in parts (the multi-part .quant cache): a part sent twice is refused, and the hole the
    missing part leaves is seen at finalize (the parts have equal sizes, so a count of groups would not see it)."""
    cfg = ModelConfig(dim=256, hidden_dim=512, n_layers=2, n_heads=4, n_kv_heads=4, vocab_size=256, seq_len=16,
                      shared_classifier=True)
    tensors = syn.synthetic_tensors(cfg, 1)
    m = Transformer(cfg)
    for t in L.QUANT_TENSORS:
        if t != L.T_W1:
            m.upload_quant(t, tensors[t])
    m.upload_f32(L.T_TOKEN_EMBEDDING, tensors[L.T_TOKEN_EMBEDDING])
    per_layer = cfg.hidden_dim * cfg.dim                       # floats of one layer of W1: a multiple of 256
    part_bytes = per_layer // 256 * 264
    first = tensors[L.T_W1][:part_bytes]
    m.upload_quant(L.T_W1, first, n_floats=per_layer, float_offset=0)
    with pytest.raises(L.L2jError) as e:
        m.upload_quant(L.T_W1, first, n_floats=per_layer, float_offset=0)      # the same part again
    assert e.value.code == L.E_INVALID
    with pytest.raises(L.L2jError) as e:
        m.finalize()                                                           # layer 1 never came
    assert e.value.code == L.E_STATE
    m.upload_quant(L.T_W1, tensors[L.T_W1][part_bytes:], n_floats=per_layer, float_offset=per_layer)
    m.finalize()
    lg, _ = m.forward(1, 0)
    assert np.isfinite(lg).all()
    m.close()
