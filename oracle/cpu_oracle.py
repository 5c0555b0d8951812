"""ctypes wrapper of oracle/libl2j_oracle.so, the CPU restatement of llama2j's CPU forward.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the CPU-baseline legs of the
benchmark.  PARITY UNPINNED: the reference holds no golden vectors for this path and cannot be run
without a JVM; see the header of l2j_oracle.c for what the restatement is anchored on.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libl2j_oracle.so")

GROUP, GROUP_BYTES = 256, 264
(T_EMB, T_RMS_ATT, T_WQ, T_WK, T_WV, T_WO, T_RMS_FFN, T_W1, T_W2, T_W3, T_RMS_FINAL, T_WCLS) = range(12)
QUANT_TENSORS = (T_RMS_ATT, T_WQ, T_WK, T_WV, T_WO, T_RMS_FFN, T_W1, T_W2, T_W3, T_RMS_FINAL)
SILU_LOOKUP, SILU_EXACT = 0, 1
SOFTMAX_REFERENCE, SOFTMAX_TRUE = 0, 1

_lib = None


def build(force: bool = False) -> str:
    src = os.path.join(HERE, "l2j_oracle.c")
    if force or not os.path.exists(LIB_PATH) or os.path.getmtime(src) > os.path.getmtime(LIB_PATH):
        subprocess.run(["make", "-C", HERE, "-B" if force else "-s", "libl2j_oracle.so"], check=True,
                       capture_output=True)
    return LIB_PATH


def load():
    global _lib
    if _lib is not None:
        return _lib
    build()
    lib = C.CDLL(LIB_PATH)
    P, I64, I = C.c_void_p, C.c_int64, C.c_int
    sig = {
        "l2jo_num_threads": (I, []),
        "l2jo_set_num_threads": (None, [I]),
        "l2jo_quant_bytes": (I64, [I64]),
        "l2jo_quant_encode": (None, [P, I64, P]),
        "l2jo_quant_decode": (None, [P, I64, I64, P]),
        "l2jo_quant_roundtrip_violations": (I64, [P, I64]),
        "l2jo_rms": (None, [P, P, I]),
        "l2jo_weight_normalize_i8": (None, [P, P, P, I64, P, I]),
        "l2jo_matmul_i8": (None, [P, P, P, I64, I, I]),
        "l2jo_matmul_f32": (None, [P, P, P, I64, I, I]),
        "l2jo_rope": (None, [P, P, I, I, I, I]),
        "l2jo_attention_scores": (None, [P, P, P, P, I64, I, I, I]),
        "l2jo_exp_sum_normalize": (None, [P, C.c_float, I]),
        "l2jo_accum_weighted_value": (None, [P, P, P, I, I64, I, I]),
        "l2jo_accum": (None, [P, P, I]),
        "l2jo_silu": (None, [P, P, I, I]),
        "l2jo_argmax": (I, [P, I]),
        "l2jo_model_create": (P, [I, I, I, I, I, I, I, I, I]),
        "l2jo_model_set_tensor": (None, [P, I, P]),
        "l2jo_model_reset": (None, [P]),
        "l2jo_model_destroy": (None, [P]),
        "l2jo_model_buffer": (P, [P, I]),
        "l2jo_model_forward": (None, [P, I, I, P]),
        "l2jo_sampler_create": (P, [I64, I]),
        "l2jo_sampler_destroy": (None, [P]),
        "l2jo_sampler_next_int": (C.c_int32, [P]),
        "l2jo_sampler_next_float": (C.c_float, [P]),
        "l2jo_sampler_sample": (I, [P, P, I, C.c_float, C.c_float]),
        "l2jo_synth_normal": (None, [P, I64, C.c_uint64, C.c_uint32, I64, C.c_float]),
        "l2jo_synth_quant": (None, [P, I64, C.c_uint64, C.c_uint32, C.c_float]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def quant_bytes(n: int) -> int:
    return -(-n // GROUP) * GROUP_BYTES


def quant_encode(values) -> np.ndarray:
    v = _f32(values).reshape(-1)
    out = np.empty(quant_bytes(v.size), dtype=np.uint8)
    load().l2jo_quant_encode(v.ctypes.data, v.size, out.ctypes.data)
    return out


def quant_decode(groups: np.ndarray, n: int, start: int = 0) -> np.ndarray:
    g = np.ascontiguousarray(groups, dtype=np.uint8)
    out = np.empty(n, dtype=np.float32)
    load().l2jo_quant_decode(g.ctypes.data, start, n, out.ctypes.data)
    return out


def synth_normal(n: int, seed: int, stream: int, start: int = 0, scale: float = 0.02) -> np.ndarray:
    out = np.empty(n, dtype=np.float32)
    load().l2jo_synth_normal(out.ctypes.data, n, seed, stream, start, C.c_float(scale))
    return out


def synth_quant(n: int, seed: int, stream: int, scale: float = 0.02) -> np.ndarray:
    out = np.empty(quant_bytes(n), dtype=np.uint8)
    load().l2jo_synth_quant(out.ctypes.data, n, seed, stream, C.c_float(scale))
    return out


def matmul_i8(groups, weight_index: int, n: int, d: int, x) -> np.ndarray:
    g = np.ascontiguousarray(groups, dtype=np.uint8)
    xv = _f32(x)
    out = np.empty(d, dtype=np.float32)
    load().l2jo_matmul_i8(out.ctypes.data, xv.ctypes.data, g.ctypes.data, weight_index, n, d)
    return out


def matmul_f32(w, n: int, d: int, x) -> np.ndarray:
    wv, xv = _f32(w), _f32(x)
    out = np.empty(d, dtype=np.float32)
    load().l2jo_matmul_f32(out.ctypes.data, xv.ctypes.data, wv.ctypes.data, 0, n, d)
    return out


def rmsnorm_i8(groups, weight_index: int, x) -> np.ndarray:
    g = np.ascontiguousarray(groups, dtype=np.uint8)
    xv = _f32(x)
    ss = np.zeros(1, dtype=np.float32)
    out = np.empty(xv.size, dtype=np.float32)
    lib = load()
    lib.l2jo_rms(ss.ctypes.data, xv.ctypes.data, xv.size)
    lib.l2jo_weight_normalize_i8(out.ctypes.data, xv.ctypes.data, g.ctypes.data, weight_index, ss.ctypes.data, xv.size)
    return out


def rope(q, k, pos: int, head_size: int):
    qv, kv = _f32(q).copy(), _f32(k).copy()
    load().l2jo_rope(qv.ctypes.data, kv.ctypes.data, pos, qv.size, kv.size, head_size)
    return qv, kv


def attention(q, key_cache, value_cache, pos: int, n_heads: int, n_kv_heads: int, head_size: int,
              softmax_mode: int = SOFTMAX_TRUE) -> np.ndarray:
    """All heads of one layer; caches in the reference layout (seq, kv_dim)."""
    lib = load()
    qv, kc, vc = _f32(q), _f32(key_cache), _f32(value_cache)
    kv_dim = n_kv_heads * head_size
    kv_mul = n_heads // n_kv_heads
    out = np.zeros(n_heads * head_size, dtype=np.float32)
    att = np.zeros(pos + 1, dtype=np.float32)
    for h in range(n_heads):
        base = (h // kv_mul) * head_size
        slot = np.zeros(1, dtype=np.float32)
        qh = qv[h * head_size:(h + 1) * head_size].copy()
        lib.l2jo_attention_scores(qh.ctypes.data, kc.ctypes.data, att.ctypes.data, slot.ctypes.data, base, kv_dim, pos, head_size)
        shift = float(slot[0]) if softmax_mode == SOFTMAX_REFERENCE else float(att.max())
        lib.l2jo_exp_sum_normalize(att.ctypes.data, C.c_float(shift), pos + 1)
        oh = np.zeros(head_size, dtype=np.float32)
        lib.l2jo_accum_weighted_value(oh.ctypes.data, att.ctypes.data, vc.ctypes.data, pos, base, head_size, kv_dim)
        out[h * head_size:(h + 1) * head_size] = oh
    return out


def silu(hb, hb2, mode: int = SILU_EXACT) -> np.ndarray:
    a, b = _f32(hb).copy(), _f32(hb2)
    load().l2jo_silu(a.ctypes.data, b.ctypes.data, a.size, mode)
    return a


def argmax(logits) -> int:
    v = _f32(logits)
    return int(load().l2jo_argmax(v.ctypes.data, v.size))


class OracleModel:
    """The CPU forward (Run.transformerCPU) over host tensors; keeps the arrays alive."""

    def __init__(self, cfg, tensors: dict, silu_mode: int = SILU_EXACT, softmax_mode: int = SOFTMAX_REFERENCE):
        self.cfg = cfg
        self.lib = load()
        self._keep = {}
        self.h = self.lib.l2jo_model_create(cfg.dim, cfg.hidden_dim, cfg.n_layers, cfg.n_heads, cfg.n_kv_heads,
                                            cfg.vocab_size, cfg.seq_len, silu_mode, softmax_mode)
        for t, arr in tensors.items():
            a = np.ascontiguousarray(arr)
            self._keep[t] = a
            self.lib.l2jo_model_set_tensor(self.h, int(t), a.ctypes.data)
        self.logits = np.zeros(cfg.vocab_size, dtype=np.float32)

    def forward(self, token: int, pos: int) -> np.ndarray:
        self.lib.l2jo_model_forward(self.h, int(token), int(pos), self.logits.ctypes.data)
        return self.logits

    def buffer(self, which: int, n: int, offset: int = 0) -> np.ndarray:
        ptr = self.lib.l2jo_model_buffer(self.h, which)
        arr = np.ctypeslib.as_array(C.cast(ptr, C.POINTER(C.c_float)), shape=(offset + n,))
        return arr[offset:offset + n].copy()

    def close(self):
        if self.h:
            self.lib.l2jo_model_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Sampler:
    """Sampler.java + java.util.Random restated: temperature / top-p token choice from logits."""

    def __init__(self, seed: int, vocab: int):
        self.lib = load()
        self.vocab = vocab
        self.h = self.lib.l2jo_sampler_create(int(seed), int(vocab))

    def next_int(self) -> int:
        return int(self.lib.l2jo_sampler_next_int(self.h))

    def next_float(self) -> float:
        return float(self.lib.l2jo_sampler_next_float(self.h))

    def sample(self, logits: np.ndarray, temperature: float, topp: float) -> int:
        """Run.java:643-665: the logits are consumed (turned into probabilities in place)."""
        a = np.ascontiguousarray(logits, dtype=np.float32)
        return int(self.lib.l2jo_sampler_sample(self.h, a.ctypes.data, a.size, C.c_float(temperature), C.c_float(topp)))

    def close(self):
        if self.h:
            self.lib.l2jo_sampler_destroy(self.h)
            self.h = None


def synthetic_tensors(cfg, seed: int = 0) -> dict:
    """The same synthetic checkpoint the product's GPU generator makes, computed on the CPU:
    stream id = tensor id, scale 0.02, RMSNorm weights 1.0."""
    def floats(t):
        d, h, L, v = cfg.dim, cfg.hidden_dim, cfg.n_layers, cfg.vocab_size
        kv = cfg.dim * cfg.n_kv_heads // cfg.n_heads
        return {T_EMB: v * d, T_RMS_ATT: L * d, T_WQ: L * d * d, T_WK: L * d * kv, T_WV: L * d * kv, T_WO: L * d * d,
                T_RMS_FFN: L * d, T_W1: L * d * h, T_W2: L * h * d, T_W3: L * d * h, T_RMS_FINAL: d, T_WCLS: v * d}[t]
    out = {}
    for t in QUANT_TENSORS:
        if t in (T_RMS_ATT, T_RMS_FFN, T_RMS_FINAL):
            out[t] = quant_encode(np.ones(floats(t), dtype=np.float32))
        else:
            out[t] = synth_quant(floats(t), seed, t)
    out[T_EMB] = synth_normal(floats(T_EMB), seed, T_EMB)
    if not cfg.shared_classifier:
        out[T_WCLS] = synth_normal(floats(T_WCLS), seed, T_WCLS)
    return out


def greedy_run(model: OracleModel, prompt, steps: int, forced=None):
    """Run.java:609-685 with --temp 0.0 on the CPU forward.  `forced`, if given, replaces the
    sampled tokens (teacher forcing) so that every position can be compared after a tie-break flip."""
    prompt = [int(t) for t in prompt]
    token, pos = 1, 0
    chosen, logits_all = [], []
    while pos < steps:
        lg = model.forward(token, pos)
        nxt = prompt[pos] if pos < len(prompt) else argmax(lg)
        logits_all.append(lg.copy())
        chosen.append(nxt)
        if forced is not None:
            nxt = int(forced[pos])
        pos += 1
        token = nxt
    return np.asarray(chosen, dtype=np.int32), np.stack(logits_all)
