"""Host-side file formats and the layer split, checked on the CPU."""
import os
import struct

import numpy as np
import pytest

from llama2j_b200 import lib as L
from llama2j_b200 import model_files as mf
from llama2j_b200.layer_allocation import GIGA, LayerAllocation, parse_gpu_mem
from llama2j_b200.synthetic import SHAPES

TINY = mf.ModelConfig(dim=64, hidden_dim=176, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=96, seq_len=32,
                      shared_classifier=False)


def test_checkpoint_sizes_of_the_benchmark_shapes():
    """File sizes of llama2.c legacy checkpoints (28-byte header, FP32 tensors, two skipped RoPE tables)."""
    expect = {
        ("stories15M", True): 60_816_028, ("stories15M", False): 97_680_028,
        ("stories110M", True): 438_381_596, ("stories110M", False): 536_685_596,
        ("llama2-7b", True): 26_431_471_644, ("llama2-7b", False): 26_955_759_644,
        ("llama2-13b", True): 51_410_194_460, ("llama2-13b", False): 52_065_554_460,
    }
    for (name, shared), size in expect.items():
        c = SHAPES[name]
        cfg = mf.ModelConfig(c.dim, c.hidden_dim, c.n_layers, c.n_heads, c.n_kv_heads, c.vocab_size, c.seq_len, shared)
        assert mf.checkpoint_offsets(cfg)["end"] == size


def test_quant_sizes_match_the_bytes_per_token_model():
    """Encoded bytes of all matrices / RMSNorm weights per shape (groups of 264 bytes)."""
    expect = {"stories15M": (6_158_592, 4_224), "stories110M": (87_588_864, 19_800),
              "llama2-7b": (6_678_380_544, 274_560), "llama2-13b": (13_084_262_400, 427_680)}
    for name, (q_mat, q_rms) in expect.items():
        cfg = SHAPES[name]
        mats = sum(mf.quant_bytes(cfg.tensor_floats(t)) for t in (L.T_WQ, L.T_WK, L.T_WV, L.T_WO, L.T_W1, L.T_W2, L.T_W3))
        rms = sum(mf.quant_bytes(cfg.tensor_floats(t)) for t in (L.T_RMS_ATT, L.T_RMS_FFN, L.T_RMS_FINAL))
        assert (mats, rms) == (q_mat, q_rms)


def test_checkpoint_round_trip(tmp_path, oracle):
    rng = np.random.default_rng(0)
    tensors = {t: rng.normal(0, 0.02, TINY.tensor_floats(t)).astype(np.float32) for t in range(12)}
    path = str(tmp_path / "tiny.bin")
    mf.write_checkpoint(path, TINY, tensors)
    assert os.path.getsize(path) == mf.checkpoint_offsets(TINY)["end"]
    cfg = mf.read_checkpoint_header(path)
    assert cfg == TINY
    for t in range(12):
        assert np.array_equal(mf.read_checkpoint_tensor(path, cfg, t), tensors[t])
    shared = mf.ModelConfig(**{**TINY.__dict__, "shared_classifier": True})
    mf.write_checkpoint(path, shared, tensors)
    with open(path, "rb") as f:
        assert struct.unpack("<7i", f.read(28))[5] == 96          # positive vocab: shared classifier
    assert mf.read_checkpoint_header(path).shared_classifier
    with pytest.raises(KeyError):
        mf.read_checkpoint_tensor(path, shared, L.T_WCLS)


def test_quant_cache_round_trip_and_faults(tmp_path, oracle):
    n = TINY.tensor_floats(L.T_WQ)
    groups = oracle.quant_encode(np.random.default_rng(1).normal(0, 0.02, n).astype(np.float32))
    ckpt = str(tmp_path / "model.v2.bin")
    path = mf.quant_cache_path(ckpt, L.T_WQ)
    assert os.path.basename(path) == "model.v2_l_wq_256_8.quant"
    mf.write_quant_cache(path, groups)
    with open(path, "rb") as f:
        assert struct.unpack("<i", f.read(4))[0] == groups.size   # little-endian int32 byte count
    assert np.array_equal(mf.read_quant_cache(path, n), groups)
    with pytest.raises(ValueError):
        mf.read_quant_cache(path, n + 256)                         # size does not fit the tensor
    with open(path, "r+b") as f:
        f.truncate(100)
    with pytest.raises(ValueError):
        mf.read_quant_cache(path, n)                               # truncated payload
    with open(path, "wb") as f:
        f.write(b"\x01")
    with pytest.raises(ValueError):
        mf.read_quant_cache(path, n)                               # truncated length field


def test_layer_allocation_equal_budgets():
    """Equal --gpuMem budgets give equal contiguous ranges (LayerAllocation.java:84-95)."""
    c7, c13 = SHAPES["llama2-7b"], SHAPES["llama2-13b"]
    a = LayerAllocation.from_gpu_mem([24 * GIGA] * 8, c7)
    assert a.first_layer == tuple(range(0, 32, 4)) and a.last_layer == tuple(range(3, 32, 4))
    for n, per in ((2, 20), (4, 10), (8, 5)):
        a = LayerAllocation.from_gpu_mem([80 * GIGA] * n, c13)
        assert a.covers_model()
        assert all(l - f + 1 == per for f, l in zip(a.first_layer, a.last_layer))
        assert a == LayerAllocation.equal_split(n, c13)
    one = LayerAllocation.from_gpu_mem([180 * GIGA], c7)
    assert one.first_layer == (0,) and one.last_layer == (31,)


def test_layer_allocation_uneven_budgets_and_parsing():
    """The IDE run configuration of the reference uses --gpuMem "17,24,24,24" for the 7B model."""
    mem = parse_gpu_mem("17,24,24,24")
    assert mem == [17 * GIGA, 24 * GIGA, 24 * GIGA, 24 * GIGA]
    a = LayerAllocation.from_gpu_mem(mem, SHAPES["llama2-7b"])
    assert a.device_count == 4 and a.covers_model()
    sizes = [l - f + 1 for f, l in zip(a.first_layer, a.last_layer)]
    assert sizes[0] < sizes[1] and sum(sizes) == 32
    for f, l, m in zip(a.first_layer, a.last_layer, mem):
        assert a.static_bytes + (l - f + 1) * a.bytes_per_layer <= m
    with pytest.raises(ValueError):
        LayerAllocation.from_gpu_mem([], SHAPES["llama2-7b"])


def test_quant_cache_parts_for_tensors_beyond_one_file(tmp_path):
    """Tensors whose encoding exceeds the cache format's 2^31-1 bytes (every matrix of the 13B shape) are kept
    as numbered parts, each a file in the reference's own format, split on layer boundaries."""
    cfg13 = SHAPES["llama2-13b"]
    n = cfg13.tensor_floats(L.T_W1)                                  # 40 x 13824 x 5120 floats
    parts = mf.quant_cache_parts(n, cfg13.n_layers)
    assert len(parts) > 1 and sum(c for _, c in parts) == n
    per_layer = n // cfg13.n_layers
    assert all(first % per_layer == 0 and count % per_layer == 0 for first, count in parts)
    assert all(mf.quant_bytes(count) <= mf.MAX_CACHE_BYTES for _, count in parts)
    assert mf.quant_cache_parts(cfg13.tensor_floats(L.T_RMS_ATT), cfg13.n_layers) == [(0, cfg13.tensor_floats(L.T_RMS_ATT))]
    n7 = SHAPES["llama2-7b"].tensor_floats(L.T_W1)               # 1.49 GB encoded: one file, as in the reference
    assert mf.quant_cache_parts(n7, 32) == [(0, n7)]

    # round trip at a small size with a small limit: 6 layers of 3 groups, at most 2 layers per part
    layers, per = 6, 3 * 256
    rng = np.random.default_rng(0)
    data = rng.integers(0, 256, mf.quant_bytes(layers * per), dtype=np.uint8)
    ckpt = str(tmp_path / "model.bin")
    limit = 2 * mf.quant_bytes(per) + 100
    paths = mf.write_quant_cache_parts(ckpt, L.T_WQ, data, layers * per, layers, max_bytes=limit)
    assert [os.path.basename(p) for p in paths] == [f"model_l_wq.part{k}_256_8.quant" for k in range(3)]
    back = mf.read_quant_cache_parts(ckpt, L.T_WQ, layers * per, layers, max_bytes=limit)
    assert np.array_equal(back, data)
    assert np.array_equal(mf.read_quant_cache(paths[1], 2 * per), data[2 * mf.quant_bytes(per): 4 * mf.quant_bytes(per)])
    os.remove(paths[2])
    assert mf.read_quant_cache_parts(ckpt, L.T_WQ, layers * per, layers, max_bytes=limit) is None
    # layers that are not whole groups: parts end on group boundaries instead
    odd = mf.quant_cache_parts(6 * 288, 6, max_bytes=3 * 264)
    assert sum(c for _, c in odd) == 6 * 288 and all(f % 256 == 0 for f, _ in odd)
    # a tensor that fits keeps the reference's single file name
    one = mf.write_quant_cache_parts(ckpt, L.T_WK, data[: mf.quant_bytes(per)], per, 1)
    assert [os.path.basename(p) for p in one] == ["model_l_wk_256_8.quant"]
