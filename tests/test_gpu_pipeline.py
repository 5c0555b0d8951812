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


def test_command_line_loop_over_two_devices(tmp_path, monkeypatch, capsys):
    """`--gpuMem a,b` (LayerAllocation.java:54-95) splits the layers over two devices; the command-line loop links
    the stages and must print the tokens of the single-device run."""
    if _device_count() < 2:
        pytest.skip("needs two GPUs")
    import numpy as np

    from llama2j_b200 import model_files as mf
    from llama2j_b200 import run as cli
    from llama2j_b200.model_files import ModelConfig
    cfg = ModelConfig(dim=256, hidden_dim=768, n_layers=6, n_heads=4, n_kv_heads=4, vocab_size=400, seq_len=64,
                      shared_classifier=True)
    rng = np.random.default_rng(21)
    fp32 = {t: rng.normal(0, 0.05, cfg.tensor_floats(t)).astype(np.float32) for t in range(11)}
    for t in (L.T_RMS_ATT, L.T_RMS_FFN, L.T_RMS_FINAL):
        fp32[t] = rng.uniform(0.5, 1.5, cfg.tensor_floats(t)).astype(np.float32)
    (tmp_path / "models").mkdir()
    mf.write_checkpoint(str(tmp_path / "models" / "tiny.bin"), cfg, fp32)
    monkeypatch.chdir(tmp_path)
    base = ["--checkpoint", "tiny.bin", "--temp", "0.0", "--steps", "40", "--promptTokens", "5,17,200,3",
            "--mode", "CUDA"]
    assert cli.main(base) == 0
    one = capsys.readouterr().out.strip().splitlines()
    assert cli.main(base + ["--gpuMem", "1,1"]) == 0      # equal budgets: three layers on each device
    two = capsys.readouterr().out.strip().splitlines()
    tokens = lambda lines: [ln for ln in lines if ln and ln[0].isdigit()][0]
    assert tokens(two) == tokens(one)
    assert not any("not linked" in ln for ln in two)
