"""File formats of the reference, read and written bit for bit: the llama2.c legacy checkpoint and
the quant-cache files.

References (paths relative to src/main/java/com/lastbot/llama2j/):
  checkpoint header and tensor order   Run.java:563-573, TransformerWeights.java:50-122
  quant cache file                     BinFileWriter.java:20-34, TransformerWeights.java:191-232
  group format and size arithmetic     Quant.java:30-63
"""
from __future__ import annotations

import os
import struct
from dataclasses import dataclass

import numpy as np

from . import lib as _lib

QUANT_GROUP_SIZE = 256   # Run.java:27
QUANT_BITS = 8           # Run.java:28
GROUP_BYTES = 264        # Quant.encodedBytesPerGroup, Quant.java:35-37


@dataclass(frozen=True)
class ModelConfig:
    """Config.java:6-13 plus the shared-classifier flag carried by the sign of vocab_size."""

    dim: int
    hidden_dim: int
    n_layers: int
    n_heads: int
    n_kv_heads: int
    vocab_size: int
    seq_len: int
    shared_classifier: bool = True

    @property
    def head_size(self) -> int:
        return self.dim // self.n_heads

    @property
    def kv_dim(self) -> int:
        return self.dim * self.n_kv_heads // self.n_heads

    def to_c(self) -> _lib.Config:
        return _lib.Config(self.dim, self.hidden_dim, self.n_layers, self.n_heads, self.n_kv_heads, self.vocab_size,
                           self.seq_len, 1 if self.shared_classifier else 0)

    def tensor_floats(self, tensor: int) -> int:
        """Element count of a whole tensor (all layers), TransformerWeights.java:54-122."""
        d, h, L, kv, v = self.dim, self.hidden_dim, self.n_layers, self.kv_dim, self.vocab_size
        return {
            _lib.T_TOKEN_EMBEDDING: v * d, _lib.T_RMS_ATT: L * d, _lib.T_WQ: L * d * d, _lib.T_WK: L * d * kv,
            _lib.T_WV: L * d * kv, _lib.T_WO: L * d * d, _lib.T_RMS_FFN: L * d, _lib.T_W1: L * d * h,
            _lib.T_W2: L * h * d, _lib.T_W3: L * d * h, _lib.T_RMS_FINAL: d, _lib.T_WCLS: v * d,
        }[tensor]


# Order of the tensors in a checkpoint after the header; None marks the two skipped RoPE tables.
CHECKPOINT_ORDER = (_lib.T_TOKEN_EMBEDDING, _lib.T_RMS_ATT, _lib.T_WQ, _lib.T_WK, _lib.T_WV, _lib.T_WO,
                    _lib.T_RMS_FFN, _lib.T_W1, _lib.T_W2, _lib.T_W3, _lib.T_RMS_FINAL, None, None, _lib.T_WCLS)


def quant_groups(n_floats: int) -> int:
    """Quant.numberOfGroupsByFloatSize, Quant.java:39-42."""
    return -(-n_floats // QUANT_GROUP_SIZE)


def quant_bytes(n_floats: int) -> int:
    """Quant.numberOfBytesByFloatSize, Quant.java:44-48."""
    return quant_groups(n_floats) * GROUP_BYTES


def quant_cache_path(checkpoint_path: str, tensor: int) -> str:
    """<dir>/<basename>_<tensor>_<group>_<bits>.quant, TransformerWeights.java:194 and Quant.java:195-197."""
    directory = os.path.dirname(checkpoint_path)
    base = os.path.basename(checkpoint_path)
    dot = base.rfind(".")
    if dot > 0:
        base = base[:dot]
    name = f"{base}_{_lib.TENSOR_NAMES[tensor]}_{QUANT_GROUP_SIZE}_{QUANT_BITS}.quant"
    return os.path.join(directory, name)


def write_quant_cache(path: str, groups: np.ndarray) -> None:
    """int32 little-endian byte count, then the encoded groups (BinFileWriter.java:20-34)."""
    data = np.ascontiguousarray(groups, dtype=np.uint8)
    if data.size > 0x7FFFFFFF:
        raise ValueError("the reference's cache format holds at most 2^31-1 bytes per tensor")
    with open(path, "wb") as f:
        f.write(struct.pack("<i", int(data.size)))
        data.tofile(f)


def read_quant_cache(path: str, expected_floats: int) -> np.ndarray:
    """Reads a cache file and checks its length field as TransformerWeights.java:219-223 does."""
    with open(path, "rb") as f:
        head = f.read(4)
        if len(head) != 4:
            raise ValueError(f"{path}: truncated length field")
        (size,) = struct.unpack("<i", head)
        data = np.fromfile(f, dtype=np.uint8, count=size)
    if data.size != size:
        raise ValueError(f"{path}: length field says {size} bytes, file holds {data.size}")
    if size != quant_bytes(expected_floats):
        raise ValueError(f"{path}: {size} bytes, expected {quant_bytes(expected_floats)} for {expected_floats} floats")
    return data


MAX_CACHE_BYTES = 0x7FFFFFFF   # the length field is a Java int (BinFileWriter.java:26)


def quant_cache_part_path(checkpoint_path: str, tensor: int, part: int) -> str:
    """<dir>/<basename>_<tensor>.part<K>_<group>_<bits>.quant: one part of a tensor whose encoding does not fit
    the reference's single cache file (every quantised matrix of the 13B shape: 3.4-7.4 GB encoded).  Each
    part is a file in the reference's own format."""
    single = quant_cache_path(checkpoint_path, tensor)
    stem = single[: -len(f"_{QUANT_GROUP_SIZE}_{QUANT_BITS}.quant")]
    return f"{stem}.part{part}_{QUANT_GROUP_SIZE}_{QUANT_BITS}.quant"


def quant_cache_parts(n_floats: int, n_layers: int = 1, max_bytes: int = MAX_CACHE_BYTES):
    """Splits a tensor of n_floats into parts of at most max_bytes encoded bytes: [(first_float, floats), ...].
    Parts end on layer boundaries when the layers are whole groups (so a stage of a layer split needs whole
    files only), else on group boundaries; one part if the tensor fits."""
    if quant_bytes(n_floats) <= max_bytes:
        return [(0, n_floats)]
    max_groups = max_bytes // GROUP_BYTES
    if max_groups <= 0:
        raise ValueError("max_bytes is smaller than one group")
    per_layer = n_floats // n_layers if n_layers > 0 and n_floats % n_layers == 0 else 0
    unit = per_layer if per_layer and per_layer % QUANT_GROUP_SIZE == 0 and per_layer // QUANT_GROUP_SIZE <= max_groups \
        else QUANT_GROUP_SIZE
    units_per_part = (max_groups * QUANT_GROUP_SIZE) // unit
    parts, start = [], 0
    while start < n_floats:
        count = min(units_per_part * unit, n_floats - start)
        parts.append((start, count))
        start += count
    return parts


def write_quant_cache_parts(checkpoint_path: str, tensor: int, groups: np.ndarray, n_floats: int, n_layers: int = 1,
                            max_bytes: int = MAX_CACHE_BYTES) -> list:
    """Writes the cache of one tensor: the reference's single file if it fits, else numbered parts."""
    data = np.ascontiguousarray(groups, dtype=np.uint8).reshape(-1)
    if data.size != quant_bytes(n_floats):
        raise ValueError(f"{data.size} bytes for {n_floats} floats, expected {quant_bytes(n_floats)}")
    parts = quant_cache_parts(n_floats, n_layers, max_bytes)
    if len(parts) == 1:
        path = quant_cache_path(checkpoint_path, tensor)
        write_quant_cache(path, data)
        return [path]
    paths = []
    for k, (first, count) in enumerate(parts):
        g0 = first // QUANT_GROUP_SIZE
        path = quant_cache_part_path(checkpoint_path, tensor, k)
        write_quant_cache(path, data[g0 * GROUP_BYTES: g0 * GROUP_BYTES + quant_bytes(count)])
        paths.append(path)
    return paths


def read_quant_cache_parts(checkpoint_path: str, tensor: int, n_floats: int, n_layers: int = 1,
                           max_bytes: int = MAX_CACHE_BYTES):
    """Reads the cache of one tensor, single file or parts; None if (any part of) it is missing."""
    parts = quant_cache_parts(n_floats, n_layers, max_bytes)
    if len(parts) == 1:
        path = quant_cache_path(checkpoint_path, tensor)
        return read_quant_cache(path, n_floats) if os.path.exists(path) else None
    paths = [quant_cache_part_path(checkpoint_path, tensor, k) for k in range(len(parts))]
    if not all(os.path.exists(p) for p in paths):
        return None
    return np.concatenate([read_quant_cache(p, count) for p, (_, count) in zip(paths, parts)])


def read_checkpoint_header(path: str) -> ModelConfig:
    """Seven little-endian int32; a negative vocab size signals an unshared classifier (Run.java:563-573)."""
    with open(path, "rb") as f:
        raw = f.read(28)
    if len(raw) != 28:
        raise ValueError(f"{path}: truncated header")
    dim, hidden, layers, heads, kv_heads, vocab, seq = struct.unpack("<7i", raw)
    return ModelConfig(dim, hidden, layers, heads, kv_heads, abs(vocab), seq, shared_classifier=vocab > 0)


def checkpoint_offsets(cfg: ModelConfig) -> dict:
    """Byte offset of every tensor in a checkpoint file of this configuration."""
    off = 28
    out = {}
    rope = cfg.seq_len * cfg.head_size // 2
    for t in CHECKPOINT_ORDER:
        if t is None:
            off += 4 * rope
            continue
        if t == _lib.T_WCLS and cfg.shared_classifier:
            continue
        out[t] = off
        off += 4 * cfg.tensor_floats(t)
    out["end"] = off
    return out


def read_checkpoint_tensor(path: str, cfg: ModelConfig, tensor: int) -> np.ndarray:
    """One FP32 tensor of the checkpoint as a read-only memory map."""
    offs = checkpoint_offsets(cfg)
    if tensor not in offs:
        raise KeyError(f"tensor {tensor} is not stored in this checkpoint")
    return np.memmap(path, dtype="<f4", mode="r", offset=offs[tensor], shape=(cfg.tensor_floats(tensor),))


def write_checkpoint(path: str, cfg: ModelConfig, tensors: dict) -> None:
    """Writes a llama2.c legacy checkpoint; the two RoPE tables the reader skips are written as zeros."""
    rope = np.zeros(cfg.seq_len * cfg.head_size // 2, dtype="<f4")
    vocab = cfg.vocab_size if cfg.shared_classifier else -cfg.vocab_size
    with open(path, "wb") as f:
        f.write(struct.pack("<7i", cfg.dim, cfg.hidden_dim, cfg.n_layers, cfg.n_heads, cfg.n_kv_heads, vocab, cfg.seq_len))
        for t in CHECKPOINT_ORDER:
            if t is None:
                rope.tofile(f)
                continue
            if t == _lib.T_WCLS and cfg.shared_classifier:
                continue
            arr = np.ascontiguousarray(tensors[t], dtype="<f4").reshape(-1)
            if arr.size != cfg.tensor_floats(t):
                raise ValueError(f"tensor {t}: {arr.size} floats, expected {cfg.tensor_floats(t)}")
            arr.tofile(f)
