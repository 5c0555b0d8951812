"""Synthetic checkpoints of the benchmark configurations, generated and quantised on the GPU.

The reference loads real Llama-2 / tinyllamas checkpoints that are not available offline; the
benchmark configurations prescribe random stand-ins of the same shapes: matrices and the embedding
N(0, 0.02^2) from seed 0, RMSNorm weights exactly 1.0.  Every tensor is a counter-based stream
(stream id = tensor id, element index = position in the flattened tensor), so any part of any tensor
can be regenerated independently and the CPU checker can reproduce the same bits.

Quantisation runs through l2j_quant_encode / l2j_synth_quant, the device restatement of
Quant.encode (src/main/java/com/lastbot/llama2j/Quant.java:156-193).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import lib as _lib
from .model_files import ModelConfig, quant_bytes

WEIGHT_SCALE = 0.02

# The shapes of the benchmark configurations (dim, hidden, layers, heads, kv heads, vocab, seq_len, shared classifier).
SHAPES = {
    "stories15M": ModelConfig(288, 768, 6, 6, 6, 32000, 256, True),
    "stories110M": ModelConfig(768, 2048, 12, 12, 12, 32000, 1024, True),
    "llama2-7b": ModelConfig(4096, 11008, 32, 32, 32, 32000, 4096, False),
    "llama2-13b": ModelConfig(5120, 13824, 40, 40, 40, 32000, 4096, False),
}


def synthetic_prompt(n: int, seed: int = 1, vocab: int = 32000) -> np.ndarray:
    """Token ids uniform in [3, vocab) from the given seed."""
    return np.random.default_rng(seed).integers(3, vocab, n).astype(np.int32)


def quant_encode(values: np.ndarray, device: int = 0) -> np.ndarray:
    """Quant.encode on the device: float32 array -> group-format bytes."""
    lib = _lib.load()
    data = np.ascontiguousarray(values, dtype=np.float32).reshape(-1)
    out = np.empty(quant_bytes(data.size), dtype=np.uint8)
    _lib.check(lib.l2j_quant_encode(device, data.ctypes.data, data.size, out.ctypes.data))
    return out


def synth_f32(n: int, seed: int, stream: int, device: int = 0, start: int = 0, scale: float = WEIGHT_SCALE) -> np.ndarray:
    lib = _lib.load()
    out = np.empty(n, dtype=np.float32)
    _lib.check(lib.l2j_synth_f32(device, seed, stream, start, n, C.c_float(scale), out.ctypes.data))
    return out


def synth_quant(n: int, seed: int, stream: int, device: int = 0, scale: float = WEIGHT_SCALE) -> np.ndarray:
    lib = _lib.load()
    out = np.empty(quant_bytes(n), dtype=np.uint8)
    _lib.check(lib.l2j_synth_quant(device, seed, stream, n, C.c_float(scale), out.ctypes.data))
    return out


def synthetic_tensors(cfg: ModelConfig, seed: int = 0, device: int = 0) -> dict:
    """{tensor id: host array}: quantised tensors in group format, embedding / classifier as float32."""
    out = {}
    for t in _lib.QUANT_TENSORS:
        n = cfg.tensor_floats(t)
        if t in (_lib.T_RMS_ATT, _lib.T_RMS_FFN, _lib.T_RMS_FINAL):
            out[t] = quant_encode(np.ones(n, dtype=np.float32), device)
        else:
            out[t] = synth_quant(n, seed, t, device)
    out[_lib.T_TOKEN_EMBEDDING] = synth_f32(cfg.tensor_floats(_lib.T_TOKEN_EMBEDDING), seed, _lib.T_TOKEN_EMBEDDING, device)
    if not cfg.shared_classifier:
        out[_lib.T_WCLS] = synth_f32(cfg.tensor_floats(_lib.T_WCLS), seed, _lib.T_WCLS, device)
    return out
