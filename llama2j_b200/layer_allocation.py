"""Contiguous layer ranges per GPU from a list of memory budgets.

Mirror of LayerAllocation.java:54-95 (paths relative to src/main/java/com/lastbot/llama2j/): the
number of devices is the length of the --gpuMem list, every device first pays the static bytes
(FP32 embedding, classifier, activations), the rest of its budget is filled with layers in
proportion to the overall utilisation, rounded, then lowered until it fits.
"""
from __future__ import annotations

from dataclasses import dataclass

from .model_files import ModelConfig

GIGA = 1024 ** 3   # CommandLine.java:29


def weights_bytes_static(cfg: ModelConfig) -> int:
    """TransformerWeights.bytesStatic, TransformerWeights.java:146-155."""
    head = cfg.dim // cfg.n_heads
    floats = cfg.vocab_size * cfg.dim + cfg.dim + 2 * (cfg.seq_len * head // 2)
    if not cfg.shared_classifier:
        floats += cfg.vocab_size * cfg.dim
    return 4 * floats


def weights_bytes_per_layer(cfg: ModelConfig) -> int:
    """TransformerWeights.bytesPerLayer, TransformerWeights.java:157-172 (the reference's own
    estimate: each term is truncated to a long after scaling by the compression ratio)."""
    c = 264.0 / 1024.0
    d, h = cfg.dim, cfg.hidden_dim
    floats = d + 4 * int(d * d * c) + int(d * c) + 3 * int(d * h * c)
    return 4 * floats


def state_bytes_static(cfg: ModelConfig) -> int:
    """RunState.bytesStatic, RunState.java:52-69 (tmp1 is counted as max(dim, vocab)*4 elements)."""
    kv_dim = cfg.kv_dim
    tmp = max(cfg.dim, cfg.vocab_size) * 4
    floats = 4 * cfg.dim + 2 * cfg.hidden_dim + 2 * kv_dim + cfg.n_heads * cfg.seq_len + cfg.vocab_size + tmp
    return 4 * floats


def state_bytes_per_layer(cfg: ModelConfig) -> int:
    """RunState.bytesPerLayer, RunState.java:71-77: the two KV-cache slices."""
    return 4 * 2 * cfg.seq_len * cfg.kv_dim


def _java_round(x: float) -> int:
    import math
    return int(math.floor(x + 0.5))


@dataclass(frozen=True)
class LayerAllocation:
    n_layers: int
    device_count: int
    static_bytes: int
    bytes_per_layer: int
    first_layer: tuple
    last_layer: tuple

    @staticmethod
    def from_gpu_mem(gpu_mem_bytes, cfg: ModelConfig) -> "LayerAllocation":
        if not gpu_mem_bytes:
            raise ValueError("mode CUDA needs at least one --gpuMem entry")   # LayerAllocation.java:50-52
        static = weights_bytes_static(cfg) + state_bytes_static(cfg)
        per_layer = weights_bytes_per_layer(cfg) + state_bytes_per_layer(cfg)
        layer_size = cfg.n_layers * per_layer
        layer_bytes = [m - static for m in gpu_mem_bytes]
        capacity = sum(layer_bytes)
        utilisation = layer_size / capacity
        first, last = [], []
        nxt = 0
        for dev, mem in enumerate(gpu_mem_bytes):
            n = _java_round(layer_bytes[dev] * utilisation / per_layer)
            while static + n * per_layer > mem:
                n -= 1
            first.append(nxt)
            last.append(min(nxt + n - 1, cfg.n_layers - 1))
            nxt += n
        return LayerAllocation(cfg.n_layers, len(gpu_mem_bytes), static, per_layer, tuple(first), tuple(last))

    @staticmethod
    def equal_split(n_devices: int, cfg: ModelConfig) -> "LayerAllocation":
        """What equal --gpuMem budgets give: n_layers / n_devices contiguous layers each."""
        if n_devices <= 0 or cfg.n_layers % n_devices != 0:
            raise ValueError("equal_split needs a device count that divides the layer count")
        per = cfg.n_layers // n_devices
        first = tuple(i * per for i in range(n_devices))
        last = tuple((i + 1) * per - 1 for i in range(n_devices))
        static = weights_bytes_static(cfg) + state_bytes_static(cfg)
        per_layer = weights_bytes_per_layer(cfg) + state_bytes_per_layer(cfg)
        return LayerAllocation(cfg.n_layers, n_devices, static, per_layer, first, last)

    def covers_model(self) -> bool:
        """True when the ranges tile [0, n_layers) without gaps (the reference does not check)."""
        nxt = 0
        for f, l in zip(self.first_layer, self.last_layer):
            if f != nxt or l < f:
                return False
            nxt = l + 1
        return nxt == self.n_layers


def parse_gpu_mem(arg: str):
    """--gpuMem "17,24,24,24": whole gigabytes per device (CommandLine.java:108-114)."""
    return [int(part.strip()) * GIGA for part in arg.split(",")]
