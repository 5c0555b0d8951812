"""Tensor-parallel group (l2j_create_tp / l2j_tp_*): every output element is computed by one rank in the
order of the single device's per-step kernels, so logits and greedy tokens must be bitwise those of one device
running those kernels (the persistent kernel sums the attention partials in another order: close, not bitwise).  Ranks wait for each
other inside their kernels (with a time limit) and therefore need a GPU each: the tests with more than
one rank are skipped on a single GPU."""
import numpy as np
import pytest

from llama2j_b200 import lib as L
from llama2j_b200 import synthetic as syn
from llama2j_b200.model_files import ModelConfig
from llama2j_b200.transformer import TensorParallel, Transformer

pytestmark = pytest.mark.gpu


def _device_count() -> int:
    import torch
    return torch.cuda.device_count()


def _whole(cfg, tensors):
    m = Transformer(cfg, flags=L.F_STEP_KERNELS)
    m.upload_all(tensors)
    m.finalize()
    return m


def _check_group(cfg, tensors, n_ranks, steps, n_prompt, flags=0):
    prompt = syn.synthetic_prompt(n_prompt, 1, cfg.vocab_size)
    whole = _whole(cfg, tensors)
    ref_tokens = whole.generate_greedy(prompt, steps)
    whole.reset()
    group = TensorParallel.from_devices(cfg, tensors, list(range(n_ranks)), flags=flags)
    token = 1
    for pos in range(12):
        lg, am = whole.forward(token, pos)
        lg2, am2 = group.forward(token, pos)
        assert np.array_equal(lg.view(np.uint32), lg2.view(np.uint32)), pos
        assert am == am2
        token = int(prompt[pos]) if pos < n_prompt else am
    toks = group.generate_greedy(prompt, steps)
    assert np.array_equal(toks, ref_tokens)
    assert np.array_equal(group.generate_greedy(prompt, steps), ref_tokens)
    whole.close()
    group.close()


def test_group_of_one_is_the_plain_context():
    cfg = syn.SHAPES["stories15M"]
    tensors = syn.synthetic_tensors(cfg, 0)
    _check_group(cfg, tensors, 1, steps=48, n_prompt=8)


def test_two_ranks_stories15m_unaligned_rows():
    if _device_count() < 2:
        pytest.skip("needs two GPUs")
    cfg = syn.SHAPES["stories15M"]          # dim 288: rows straddle quantisation groups
    tensors = syn.synthetic_tensors(cfg, 0)
    _check_group(cfg, tensors, 2, steps=200, n_prompt=16)


def test_ranks_stories110m():
    n = min(_device_count(), 4)
    if n < 2:
        pytest.skip("needs two GPUs")
    cfg = syn.SHAPES["stories110M"]         # 12 heads: 2 or 4 ranks
    tensors = syn.synthetic_tensors(cfg, 0)
    _check_group(cfg, tensors, n, steps=900, n_prompt=16)   # crosses into the long-context attention launch


def test_two_ranks_grouped_query_attention():
    if _device_count() < 2:
        pytest.skip("needs two GPUs")
    cfg = ModelConfig(dim=256, hidden_dim=704, n_layers=3, n_heads=8, n_kv_heads=4, vocab_size=512, seq_len=128,
                      shared_classifier=False)       # two query heads per kv head; hidden_dim not a multiple of 256
    tensors = syn.synthetic_tensors(cfg, 3)
    _check_group(cfg, tensors, 2, steps=128, n_prompt=8)


def test_two_ranks_split_classifier():
    """Opt-in mode: the classifier's rows are split too and the ranks exchange their best candidates."""
    if _device_count() < 2:
        pytest.skip("needs two GPUs")
    cfg = syn.SHAPES["stories110M"]
    tensors = syn.synthetic_tensors(cfg, 0)
    _check_group(cfg, tensors, 2, steps=96, n_prompt=16, flags=L.F_TP_SPLIT_CLASSIFIER)


def test_two_ranks_lost_partner_is_reported_and_group_reset_recovers():
    """One rank misses a forward (host-side injection): its partners' results never carry the sequence numbers
    it polls for, every poll gives up by the wait limit, the call answers L2J_E_DEVICE, and after
    l2j_tp_reset the group is bitwise right again.  No kernel faults or hangs: all waits are bounded."""
    if _device_count() < 2:
        pytest.skip("needs two GPUs")
    cfg = ModelConfig(dim=512, hidden_dim=1536, n_layers=2, n_heads=8, n_kv_heads=8, vocab_size=1024, seq_len=64,
                      shared_classifier=False)
    tensors = syn.synthetic_tensors(cfg, 5)
    ranks = []
    for r in range(2):
        t = Transformer(cfg, device=r, tp_rank=r, tp_size=2)
        t.set_wait_limit_us(500)
        t.upload_all(tensors)
        t.finalize()
        ranks.append(t)
    group = TensorParallel(ranks)
    good = [group.forward(t, p)[0].copy() for p, t in enumerate((1, 9, 77))]
    ranks[0].debug_desync()
    with pytest.raises(L.L2jError) as e:
        group.forward(1, 0)
    assert e.value.code == L.E_DEVICE
    assert ranks[0].stats().device_status & L.DS_WAIT_TIMEOUT
    group.reset()
    again = [group.forward(t, p)[0].copy() for p, t in enumerate((1, 9, 77))]
    for a, b in zip(good, again):
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    group.close()


def test_rejects_bad_groups():
    cfg = syn.SHAPES["stories15M"]          # 6 heads
    with pytest.raises(L.L2jError) as e:
        Transformer(cfg, tp_rank=0, tp_size=4)          # 6 heads do not divide by 4
    assert e.value.code == L.E_INVALID
    with pytest.raises(L.L2jError):
        Transformer(cfg, tp_rank=2, tp_size=2)
    tensors = syn.synthetic_tensors(cfg, 0)
    a = Transformer(cfg, device=0, tp_rank=0, tp_size=2)
    b = Transformer(cfg, device=0, tp_rank=1, tp_size=2)
    for m in (a, b):
        m.upload_all(tensors)
        m.finalize()
    with pytest.raises(L.L2jError) as e:
        TensorParallel([a, b])                           # two ranks on one device are refused
    assert e.value.code == L.E_INVALID
    with pytest.raises(L.L2jError) as e:
        a.forward(1, 0)                                  # a rank does not run alone
    assert e.value.code == L.E_STATE
    a.close()
    b.close()
