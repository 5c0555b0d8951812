"""End-to-end parity of the decode path with the oracle through the C ABI.

Gates (the north-star criteria): per-token logits within 1e-3 of the logit range, identical greedy
token sequence.  The oracle runs in its CUDA-faithful arithmetic (exact sigmoid); the difference to
its CPU-faithful lookup-table SiLU is measured and bounded separately, as the reference's two paths
differ from each other by that much.  The oracle is teacher-forced with the GPU's tokens so that every
position is compared even if a near-tie flips an arg-max."""
import os

import numpy as np
import pytest

from llama2j_b200 import lib as L
from llama2j_b200 import synthetic as syn
from llama2j_b200.model_files import ModelConfig
from llama2j_b200.transformer import Transformer, run_greedy_host_loop

pytestmark = pytest.mark.gpu

TOL = 1e-3


def _build(cfg, tensors, flags=0, first=0, last=None):
    m = Transformer(cfg, 0, first, last, flags)
    m.upload_all(tensors)
    m.finalize()
    return m


def _compare_run(oracle, cfg, tensors, prompt, steps, flags=0):
    gpu = _build(cfg, tensors, flags)
    toks, logits = run_greedy_host_loop(gpu, prompt, steps, stop_on_bos=False)
    om = oracle.OracleModel(cfg, tensors, oracle.SILU_EXACT, oracle.SOFTMAX_REFERENCE)
    ref_toks, ref_logits = oracle.greedy_run(om, prompt, steps, forced=toks)
    worst = 0.0
    flips = []
    for p in range(steps):
        rng_ = float(ref_logits[p].max() - ref_logits[p].min())
        err = float(np.abs(logits[p] - ref_logits[p]).max()) / rng_
        worst = max(worst, err)
        if toks[p] != ref_toks[p]:
            top2 = np.sort(ref_logits[p])[-2:]
            flips.append((p, int(toks[p]), int(ref_toks[p]), float(top2[1] - top2[0]) / rng_))
    mode = gpu.launch_mode()
    stats = gpu.stats()
    gpu.close()
    om.close()
    return toks, worst, flips, mode, stats


def test_config1_stories15m_256_steps(oracle):
    """dim 288: every row straddles quantisation groups; seq_len 256; 16-token prompt, 240 greedy tokens."""
    cfg = syn.SHAPES["stories15M"]
    tensors = syn.synthetic_tensors(cfg, 0)
    prompt = syn.synthetic_prompt(16, 1)
    toks, worst, flips, mode, stats = _compare_run(oracle, cfg, tensors, prompt, 256)
    assert mode["ring"], "the bulk-copy ring kernels must be the path that runs"
    assert worst < TOL, worst
    assert not flips, flips
    assert stats.kernels_per_forward == 2 + 5 * cfg.n_layers


def test_config1_varied_tokens_and_rms_weights(oracle):
    """The prescribed weights make greedy decoding collapse onto one token; force a varied token stream
    and non-trivial RMSNorm weights through the same comparison."""
    cfg = syn.SHAPES["stories15M"]
    tensors = syn.synthetic_tensors(cfg, 3)
    rng = np.random.default_rng(4)
    for t in (L.T_RMS_ATT, L.T_RMS_FFN, L.T_RMS_FINAL):
        tensors[t] = syn.quant_encode(rng.uniform(0.3, 2.0, cfg.tensor_floats(t)).astype(np.float32))
    prompt = syn.synthetic_prompt(255, 9)
    toks, worst, flips, _, _ = _compare_run(oracle, cfg, tensors, prompt, 256)
    assert worst < TOL, worst
    assert not flips, flips


def test_paths_agree_and_are_deterministic(oracle):
    """Graph replay, direct launches, no-PDL and the plain kernels all produce the same tokens; the
    fused paths are bitwise repeatable (no atomics on floats anywhere)."""
    cfg = syn.SHAPES["stories15M"]
    tensors = syn.synthetic_tensors(cfg, 0)
    prompt = syn.synthetic_prompt(16, 1)
    runs = {}
    for name, flags in (("graph+pdl", 0), ("graph", L.F_NO_PDL), ("direct+pdl", L.F_NO_GRAPH),
                        ("direct", L.F_NO_GRAPH | L.F_NO_PDL), ("plain", L.F_SIMPLE)):
        m = _build(cfg, tensors, flags)
        toks, logits = run_greedy_host_loop(m, prompt, 64, stop_on_bos=False)
        toks2, logits2 = run_greedy_host_loop(m, prompt, 64, stop_on_bos=False)
        assert np.array_equal(logits.view(np.uint32), logits2.view(np.uint32)), name
        runs[name] = (toks, logits)
        m.close()
    base_t, base_l = runs["graph+pdl"]
    for name in ("graph", "direct+pdl", "direct"):
        assert np.array_equal(runs[name][1].view(np.uint32), base_l.view(np.uint32)), name
    rng_ = base_l.max() - base_l.min()
    assert np.abs(runs["plain"][1] - base_l).max() < 2e-4 * rng_
    assert np.array_equal(runs["plain"][0], base_t)


def test_device_greedy_loop_equals_host_loop(oracle):
    cfg = syn.SHAPES["stories15M"]
    tensors = syn.synthetic_tensors(cfg, 0)
    prompt = syn.synthetic_prompt(16, 1)
    m = _build(cfg, tensors)
    host_toks, _ = run_greedy_host_loop(m, prompt, 256, stop_on_bos=False)
    dev_toks = m.generate_greedy(prompt, 256)
    assert np.array_equal(dev_toks, host_toks)
    assert np.array_equal(dev_toks[:16], prompt)
    assert m.last_generate_us() > 0
    st = m.stats()
    assert st.device_status == 0
    m.close()


def test_stage_buffers_follow_the_oracle(oracle):
    """TEST-mode style: after one forward, the run-state buffers agree with the CPU run state."""
    cfg = ModelConfig(dim=256, hidden_dim=688, n_layers=1, n_heads=4, n_kv_heads=2, vocab_size=512, seq_len=64,
                      shared_classifier=False)
    tensors = syn.synthetic_tensors(cfg, 2)
    m = _build(cfg, tensors)
    om = oracle.OracleModel(cfg, tensors, oracle.SILU_EXACT, oracle.SOFTMAX_REFERENCE)
    for pos, tok in enumerate([1, 40, 300, 7]):
        lg, am = m.forward(tok, pos)
        ref = om.forward(tok, pos)
        assert np.abs(m.read_buffer(2, cfg.dim) - om.buffer(2, cfg.dim)).max() < 1e-5            # q after RoPE
        krow = m.read_buffer(5, cfg.kv_dim, layer=0, pos=pos)
        vrow = m.read_buffer(6, cfg.kv_dim, layer=0, pos=pos)
        assert np.abs(krow - om.buffer(6, cfg.kv_dim, pos * cfg.kv_dim)).max() < 1e-5               # K row of the cache
        assert np.abs(vrow - om.buffer(7, cfg.kv_dim, pos * cfg.kv_dim)).max() < 1e-5
        assert np.abs(m.read_buffer(3, cfg.hidden_dim) - om.buffer(5, cfg.hidden_dim)).max() < 1e-5  # SwiGLU output
        assert np.abs(lg - ref).max() < 1e-4
        assert am == int(np.argmax(lg))
    m.close()


def test_grouped_query_heads(oracle):
    cfg = ModelConfig(dim=512, hidden_dim=1376, n_layers=2, n_heads=8, n_kv_heads=2, vocab_size=1000, seq_len=128,
                      shared_classifier=True)
    tensors = syn.synthetic_tensors(cfg, 5)
    prompt = syn.synthetic_prompt(100, 2, vocab=1000)
    toks, worst, flips, _, _ = _compare_run(oracle, cfg, tensors, prompt, 128)
    assert worst < TOL and not flips


def test_layer_split_two_stages_equal_one(oracle):
    """The reference's multi-GPU layer split (Run.java:368-413), here as two contexts with the activation
    handed over between them: bitwise the same logits as the single context."""
    cfg = syn.SHAPES["stories15M"]
    tensors = syn.synthetic_tensors(cfg, 0)
    whole = _build(cfg, tensors)
    s0 = _build(cfg, tensors, 0, 0, 2)
    s1 = _build(cfg, tensors, 0, 3, 5)
    token = 1
    for pos in range(24):
        lg, am = whole.forward(token, pos)
        x = s0.forward_stage(token, pos)
        lg2, am2 = s1.forward_stage(0, pos, x_in=x)
        assert np.array_equal(lg.view(np.uint32), lg2.view(np.uint32)), pos
        assert am == am2
        token = am
    for m in (whole, s0, s1):
        m.close()


@pytest.mark.parametrize("flags,persistent", [(0, False), (L.F_PERSISTENT, True)])
def test_config2_stories110m_to_position_1024(oracle, flags, persistent):
    """dim 768 (group-aligned rows), 32-token prompt, greedy decode to position 1024: with the per-step kernels
    (the default at this width) and with all layers in one persistent launch."""
    cfg = syn.SHAPES["stories110M"]
    tensors = syn.synthetic_tensors(cfg, 0)
    prompt = syn.synthetic_prompt(32, 1)
    toks, worst, flips, mode, stats = _compare_run(oracle, cfg, tensors, prompt, 1024, flags)
    assert mode["ring"] and mode["persistent"] == persistent
    assert stats.kernels_per_forward == (3 if persistent else 2 + 5 * cfg.n_layers)
    assert worst < TOL, worst
    assert not flips, flips


def test_long_context_positions_to_4096(oracle):
    """The long-context workload at a small width: a 3840-token forced prompt through the decode path, then
    greedy decode to position 4095 (the sequence length).  Every position is compared with the oracle; past
    position 768 the forward runs the long-context attention launch (no cluster, pipelined loop, partial
    results merged by the last block of a head), with up to 512 positions per block at the end."""
    cfg = ModelConfig(dim=256, hidden_dim=704, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=2048, seq_len=4096,
                      shared_classifier=False)
    tensors = syn.synthetic_tensors(cfg, 5)
    prompt = syn.synthetic_prompt(3840, 7, cfg.vocab_size)
    toks, worst, flips, mode, _ = _compare_run(oracle, cfg, tensors, prompt, 4096)
    assert mode["ring"]
    assert worst < TOL, worst
    assert not flips, flips
    assert np.array_equal(toks[:3840], prompt)


def test_host_side_faults(oracle):
    cfg = ModelConfig(dim=64, hidden_dim=176, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=96, seq_len=32,
                      shared_classifier=False)
    tensors = syn.synthetic_tensors(cfg, 1)
    m = Transformer(cfg)
    with pytest.raises(L.L2jError) as e:
        m.forward(1, 0)
    assert e.value.code == L.E_STATE                                   # forward before finalize
    m.upload_quant(L.T_WQ, tensors[L.T_WQ])
    with pytest.raises(ValueError):
        m.upload_quant(L.T_WK, tensors[L.T_WK][:-264])                 # wrong byte count for the tensor
    with pytest.raises(L.L2jError) as e:
        m.finalize()
    assert e.value.code == L.E_STATE                                   # tensors missing
    for t in L.QUANT_TENSORS:
        if t != L.T_WQ:
            m.upload_quant(t, tensors[t])
    m.upload_f32(L.T_TOKEN_EMBEDDING, tensors[L.T_TOKEN_EMBEDDING])
    m.upload_f32(L.T_WCLS, tensors[L.T_WCLS])
    m.finalize()
    for bad in ((1, -1), (1, 32), (-5, 0), (96, 0)):
        with pytest.raises(L.L2jError) as e:
            m.forward(*bad)
        assert e.value.code == L.E_INVALID
    lg, am = m.forward(1, 0)                                           # the context is still usable
    assert np.isfinite(lg).all()
    m.close()
    with pytest.raises(L.L2jError):
        Transformer(ModelConfig(100, 64, 1, 3, 3, 10, 8))              # dim not divisible by heads


def test_llama2_7b_shape_first_positions(oracle):
    """Full-size check: the Llama-2-7B-shaped synthetic checkpoint, a handful of positions against the
    oracle (each oracle token streams 7.2 GB on the host), then the device loop's size-independent
    properties over the whole 288-step workload."""
    cfg = syn.SHAPES["llama2-7b"]
    tensors = syn.synthetic_tensors(cfg, 0)
    m = _build(cfg, tensors)
    prompt = syn.synthetic_prompt(32, 1)
    om = oracle.OracleModel(cfg, tensors, oracle.SILU_EXACT, oracle.SOFTMAX_REFERENCE)
    token = 1
    for pos in range(4):
        lg, am = m.forward(token, pos)
        ref = om.forward(token, pos)
        rng_ = float(ref.max() - ref.min())
        assert np.abs(lg - ref).max() < TOL * rng_, pos
        assert am == int(np.argmax(ref))
        token = int(prompt[pos])
    om.close()
    a = m.generate_greedy(prompt, 288)
    b = m.generate_greedy(prompt, 288)
    assert np.array_equal(a, b)                                        # repeatable
    assert np.array_equal(a[:32], prompt)                              # forced prompt echoed
    host, _ = run_greedy_host_loop(m, prompt, 48, stop_on_bos=False)
    assert np.array_equal(host, a[:48])                                # host-driven loop = device loop
    assert m.stats().device_status == 0
    m.close()


def test_cli_run_loop_with_checkpoint_and_quant_cache(oracle, tmp_path, monkeypatch, capsys):
    """The reference's flow end to end: llama2.c checkpoint under models/, quant cache files written beside
    it on the first run (bit-identical to the oracle's Quant.encode) and read back on the second, greedy
    tokens equal to the oracle's run loop."""
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
    argv = ["--checkpoint", "tiny.bin", "--mode", "CUDA", "--temp", "0.0", "--steps", "40", "--promptTokens", "5,17,200,3"]
    assert cli.main(argv) == 0
    first = capsys.readouterr().out.strip().splitlines()
    tensors = {L.T_TOKEN_EMBEDDING: fp32[L.T_TOKEN_EMBEDDING]}
    for t in L.QUANT_TENSORS:
        cache = mf.quant_cache_path(path, t)
        assert os.path.exists(cache)
        tensors[t] = oracle.quant_encode(fp32[t])
        assert np.array_equal(mf.read_quant_cache(cache, cfg.tensor_floats(t)), tensors[t])
    om = oracle.OracleModel(cfg, tensors, oracle.SILU_EXACT, oracle.SOFTMAX_REFERENCE)
    ref, _ = oracle.greedy_run(om, [5, 17, 200, 3], 40)
    ref = ref.tolist()
    if 1 in ref:
        ref = ref[:ref.index(1)]                                      # the loop stops on a sampled BOS
    got = [int(t) for t in first[1].split()]
    assert got == ref
    assert cli.main(argv) == 0                                         # second run: from the cache files
    second = capsys.readouterr().out.strip().splitlines()
    assert second[1] == first[1]
    with pytest.raises(SystemExit):
        cli.main(["--checkpoint", "tiny.bin", "--mode", "CPU"])
