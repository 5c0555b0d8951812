"""Layer split over linked stages (l2j_pipeline_*): the reference's multi-GPU mode, Run.java:368-413.

A split must give bitwise the logits and the greedy sequence of the single context: the stages run
the same kernels on the same data, only the hand-over of x differs.  With one GPU both stages sit on
device 0 (ordered by events, no kernel waits for another); with two or more GPUs every stage gets its
own device and x crosses the peer link.
"""
import ctypes as C

import numpy as np
import pytest

from llama2j_b200 import lib as L
from llama2j_b200 import synthetic as syn
from llama2j_b200.layer_allocation import LayerAllocation
from llama2j_b200.transformer import LinkedStages, Transformer

pytestmark = pytest.mark.gpu


def _device_count() -> int:
    import torch
    return torch.cuda.device_count()


def _whole(cfg, tensors):
    m = Transformer(cfg)
    m.upload_all(tensors)
    m.finalize()
    return m


def _check_split(cfg, tensors, firsts, lasts, devices, steps, n_prompt):
    prompt = syn.synthetic_prompt(n_prompt, 1, cfg.vocab_size)
    whole = _whole(cfg, tensors)
    ref_tokens = whole.generate_greedy(prompt, steps)
    whole.reset()
    split = LinkedStages.from_allocation(cfg, firsts, lasts, tensors, devices)
    token = 1
    for pos in range(12):
        lg, am = whole.forward(token, pos)
        lg2, am2 = split.forward(token, pos)
        assert np.array_equal(lg.view(np.uint32), lg2.view(np.uint32)), pos
        assert am == am2
        token = int(prompt[pos]) if pos < n_prompt else am
    toks = split.generate_greedy(prompt, steps)
    assert np.array_equal(toks, ref_tokens)
    toks2 = split.generate_greedy(prompt, steps)          # a second sequence on the same stages
    assert np.array_equal(toks2, ref_tokens)
    assert split.last_generate_us() > 0
    whole.close()
    split.close()


def test_two_stages_on_one_device():
    cfg = syn.SHAPES["stories15M"]
    tensors = syn.synthetic_tensors(cfg, 0)
    _check_split(cfg, tensors, [0, 3], [2, 5], [0, 0], steps=96, n_prompt=16)


def test_three_uneven_stages_on_one_device():
    cfg = syn.SHAPES["stories15M"]
    tensors = syn.synthetic_tensors(cfg, 0)
    _check_split(cfg, tensors, [0, 1, 4], [0, 3, 5], [0, 0, 0], steps=40, n_prompt=8)


def test_stages_on_separate_devices():
    n = _device_count()
    if n < 2:
        pytest.skip("needs two GPUs")
    cfg = syn.SHAPES["stories110M"]
    tensors = syn.synthetic_tensors(cfg, 0)
    n = min(n, 4)
    per = cfg.n_layers // n
    firsts = [i * per for i in range(n)]
    lasts = [(i + 1) * per - 1 for i in range(n - 1)] + [cfg.n_layers - 1]
    _check_split(cfg, tensors, firsts, lasts, list(range(n)), steps=128, n_prompt=16)


def test_link_rejects_gaps_and_wrong_order():
    cfg = syn.SHAPES["stories15M"]
    tensors = syn.synthetic_tensors(cfg, 0)
    a = Transformer(cfg, first_layer=0, last_layer=1)
    b = Transformer(cfg, first_layer=3, last_layer=5)
    for m in (a, b):
        m.upload_all(tensors)
        m.finalize()
    with pytest.raises(L.L2jError) as e:
        LinkedStages([a, b])                      # layer 2 is missing
    assert e.value.code == L.E_INVALID
    with pytest.raises(L.L2jError):
        LinkedStages([b, a])
    a.close()
    b.close()
