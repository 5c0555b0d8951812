"""Token selection on the device for --temp > 0 against the checker's restatement of Sampler.java.

Both sides get the same logits (the device's own, read back once) and the same seed; the ids must be
identical at every step, which needs the same java.util.Random stream, the same float rounding in the
softmax and the cumulative sums, and the same stable descending sort of the whole candidate array,
stale entries of earlier calls included.  The temperature changes during a run so that the number of
nucleus candidates shrinks and grows.
"""
import numpy as np
import pytest

from llama2j_b200 import lib as L
from llama2j_b200 import synthetic as syn
from llama2j_b200.model_files import ModelConfig
from llama2j_b200.transformer import Transformer

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def model():
    s = syn.SHAPES["stories15M"]
    cfg = ModelConfig(s.dim, s.hidden_dim, s.n_layers, s.n_heads, s.n_kv_heads, s.vocab_size, s.seq_len, False)
    tensors = syn.synthetic_tensors(cfg, 3)
    # a wide logit distribution: the prescribed N(0, 0.02) classifier gives almost flat probabilities
    wcls = np.asarray(tensors[L.T_WCLS], dtype=np.float32)
    tensors[L.T_WCLS] = (wcls * np.float32(9.0)).astype(np.float32)
    m = Transformer(cfg, 0, 0, None, 0)
    m.upload_all(tensors)
    m.finalize()
    yield m
    m.close()


def _run(model, oracle, seed, schedule, steps=64):
    """schedule(step) -> (temperature, topp); returns (device ids, checker ids)."""
    vocab = model.cfg.vocab_size
    ref = oracle.Sampler(seed, vocab)
    model.sampler_seed(seed)
    token, got, want = 1, [], []
    for pos in range(steps):
        logits, _ = model.forward(token, pos)
        temperature, topp = schedule(pos)
        dev = model.sample(temperature, topp)
        cpu = ref.sample(logits.copy(), temperature, topp)
        got.append(dev)
        want.append(cpu)
        token = cpu
    ref.close()
    assert model.stats().device_status == 0
    return got, want


def test_top_p_default_flags(model, oracle):
    """The reference's defaults: --temp 0.9 --topp 0.9."""
    got, want = _run(model, oracle, 12345, lambda s: (0.9, 0.9))
    assert got == want
    assert len(set(want)) > 8


def test_plain_sampling(model, oracle):
    """topp > 0.999 walks the whole distribution (Sampler.sample)."""
    got, want = _run(model, oracle, 7, lambda s: (1.0, 1.0))
    assert got == want
    assert len(set(want)) > 8


def test_changing_candidate_counts(model, oracle):
    """A sharp step leaves few candidates, the next flat one many: the array the reference keeps across calls
    is sorted whole, so what earlier calls left beyond the candidates takes part."""
    temps = (0.9, 0.05, 2.0, 0.3, 0.01, 1.3)
    tops = (0.9, 0.5, 0.95, 0.1)
    got, want = _run(model, oracle, -99, lambda s: (temps[s % len(temps)], tops[s % len(tops)]), steps=96)
    assert got == want


def test_probabilities_replace_logits(model, oracle):
    """The reference turns the logits into probabilities in place; so does the device (Run.java:645-656)."""
    model.sampler_seed(1)
    logits, _ = model.forward(5, 0)
    want = logits.copy()
    oracle.Sampler(1, model.cfg.vocab_size).sample(want, 0.7, 0.9)
    model.sample(0.7, 0.9)
    import ctypes as C

    import torch   # noqa: F401  (loads the CUDA runtime the next line binds to)
    cudart = C.CDLL("libcudart.so.12")
    _, ptr = model.device_buffers()
    got = np.empty(model.cfg.vocab_size, dtype=np.float32)
    rc = cudart.cudaMemcpy(C.c_void_p(got.ctypes.data), C.c_void_p(ptr), C.c_size_t(got.nbytes), 2)   # device to host
    assert rc == 0
    assert np.array_equal(got, want)


def test_temperature_zero_is_argmax(model):
    logits, _ = model.forward(9, 0)
    assert model.sample(0.0, 0.9) == int(np.argmax(logits))


def test_sampler_needs_seed(oracle):
    cfg = syn.SHAPES["stories15M"]
    m = Transformer(cfg, 0, 0, None, 0)
    m.upload_all(syn.synthetic_tensors(cfg, 3))
    m.finalize()
    m.forward(1, 0)
    with pytest.raises(L.L2jError):
        m.sample(0.9, 0.9)
    m.close()


def test_command_line_loop_with_temperature(oracle, tmp_path, monkeypatch, capsys):
    """`--temp 0.9 --topp 0.9 --seed 42` through the command-line loop: the ids of the checker's run loop with
    its restatement of the Sampler, fed the device's logits."""
    from llama2j_b200 import model_files as mf
    from llama2j_b200 import run as cli
    cfg = ModelConfig(dim=128, hidden_dim=352, n_layers=2, n_heads=4, n_kv_heads=4, vocab_size=300, seq_len=48,
                      shared_classifier=True)
    rng = np.random.default_rng(12)
    fp32 = {t: rng.normal(0, 0.05, cfg.tensor_floats(t)).astype(np.float32) for t in range(11)}
    for t in (L.T_RMS_ATT, L.T_RMS_FFN, L.T_RMS_FINAL):
        fp32[t] = rng.uniform(0.5, 1.5, cfg.tensor_floats(t)).astype(np.float32)
    (tmp_path / "models").mkdir()
    path = str(tmp_path / "models" / "tiny.bin")
    mf.write_checkpoint(path, cfg, fp32)
    monkeypatch.chdir(tmp_path)
    argv = ["--checkpoint", "tiny.bin", "--temp", "0.9", "--topp", "0.9", "--seed", "42", "--steps", "40",
            "--promptTokens", "5,17,200,3"]
    assert cli.main(argv) == 0
    got = [int(t) for t in capsys.readouterr().out.strip().splitlines()[1].split()]

    tensors = {L.T_TOKEN_EMBEDDING: fp32[L.T_TOKEN_EMBEDDING]}
    for t in L.QUANT_TENSORS:
        tensors[t] = oracle.quant_encode(fp32[t])
    m = Transformer(cfg, 0, 0, None, 0)
    m.upload_all(tensors)
    m.finalize()
    ref = oracle.Sampler(42, cfg.vocab_size)
    prompt, token, want = [5, 17, 200, 3], 1, []
    for pos in range(40):
        logits, _ = m.forward(token, pos)
        nxt = prompt[pos] if pos < len(prompt) else ref.sample(logits.copy(), 0.9, 0.9)
        if nxt == 1:
            break
        want.append(nxt)
        token = nxt
    ref.close()
    m.close()
    assert got == want
    assert len(set(want)) > 4
