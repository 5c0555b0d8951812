"""Host-side mirror of the reference's CUDA-mode objects over the C ABI.

`Transformer` plays the part of TransformerWeights + RunState + Run.transformerCUDA for one device
and one contiguous layer range (paths relative to src/main/java/com/lastbot/llama2j/):

  Transformer.upload_quant / upload_f32   TransformerWeights.readAsQuant upload half, :238-350
  Transformer.forward(token, pos)         Run.transformer(token, pos, Mode.CUDA, ...), Run.java:44-51,315-519
                                          plus the logits read-back of Run.java:628-632
  Transformer.generate_greedy             the token loop of Run.java:609-685 with --temp 0.0
  argmax                                  Sampler.argmax, Sampler.java:46-57

Everything numerical happens in libl2j_b200.so; this module only moves host buffers across the ABI.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import lib as _lib
from .model_files import ModelConfig, quant_bytes


def argmax(logits: np.ndarray) -> int:
    """First index of the maximum, as Sampler.argmax (Sampler.java:46-57)."""
    return int(np.argmax(logits))


class Transformer:
    """One device, layers [first_layer, last_layer] of the model (LayerAllocation.java:67-95)."""

    def __init__(self, cfg: ModelConfig, device: int = 0, first_layer: int = 0, last_layer: int | None = None,
                 flags: int = 0, tp_rank: int = 0, tp_size: int = 1):
        self.cfg = cfg
        self.device = device
        self.first_layer = first_layer
        self.last_layer = cfg.n_layers - 1 if last_layer is None else last_layer
        self._lib = _lib.load()
        self._ctx = C.c_void_p()
        ccfg = cfg.to_c()
        if tp_size > 1:
            rc = self._lib.l2j_create_tp(C.byref(ccfg), device, tp_rank, tp_size, flags, C.byref(self._ctx))
        else:
            rc = self._lib.l2j_create(C.byref(ccfg), device, self.first_layer, self.last_layer, flags, C.byref(self._ctx))
        _lib.check(rc, None)
        self._logits = np.zeros(cfg.vocab_size, dtype=np.float32)

    # ---- lifetime -----------------------------------------------------------------------------
    def close(self) -> None:
        if self._ctx:
            self._lib.l2j_destroy(self._ctx)
            self._ctx = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def is_first(self) -> bool:
        return self.first_layer == 0

    @property
    def is_last(self) -> bool:
        return self.last_layer == self.cfg.n_layers - 1

    # ---- weights ------------------------------------------------------------------------------
    def upload_quant(self, tensor: int, groups: np.ndarray, n_floats: int | None = None, float_offset: int = 0) -> None:
        """`groups`: bytes of the tensor (or of a part starting at `float_offset`) in the group format."""
        data = np.ascontiguousarray(groups, dtype=np.uint8).reshape(-1)
        if n_floats is None:
            n_floats = self.cfg.tensor_floats(tensor) - float_offset
        if data.size != quant_bytes(n_floats):
            raise ValueError(f"tensor {tensor}: {data.size} bytes for {n_floats} floats, expected {quant_bytes(n_floats)}")
        rc = self._lib.l2j_upload_quant(self._ctx, tensor, float_offset, data.ctypes.data, data.size, n_floats)
        _lib.check(rc, self._ctx)

    def upload_f32(self, tensor: int, values: np.ndarray, float_offset: int = 0) -> None:
        data = np.ascontiguousarray(values, dtype=np.float32).reshape(-1)
        rc = self._lib.l2j_upload_f32(self._ctx, tensor, float_offset, data.ctypes.data, data.size)
        _lib.check(rc, self._ctx)

    def upload_all(self, tensors: dict) -> None:
        """Uploads a {tensor id: host array} checkpoint (quantised tensors in group format)."""
        for t in _lib.QUANT_TENSORS:
            self.upload_quant(t, tensors[t])
        self.upload_f32(_lib.T_TOKEN_EMBEDDING, tensors[_lib.T_TOKEN_EMBEDDING])
        if not self.cfg.shared_classifier and self.is_last:
            self.upload_f32(_lib.T_WCLS, tensors[_lib.T_WCLS])

    def finalize(self) -> None:
        _lib.check(self._lib.l2j_finalize(self._ctx), self._ctx)

    # ---- forward ------------------------------------------------------------------------------
    def forward(self, token: int, pos: int, want_logits: bool = True):
        """One decode step of a whole-model context; returns (logits or None, device argmax)."""
        am = C.c_int(-1)
        ptr = self._logits.ctypes.data if want_logits else None
        rc = self._lib.l2j_forward(self._ctx, int(token), int(pos), ptr, C.byref(am))
        _lib.check(rc, self._ctx)
        return (self._logits if want_logits else None), am.value

    def forward_stage(self, token: int, pos: int, x_in: np.ndarray | None = None, want_logits: bool = True):
        """One step of a pipeline stage; returns x (not last stage) or (logits, argmax) (last stage)."""
        xin = None
        if x_in is not None:
            x_in = np.ascontiguousarray(x_in, dtype=np.float32)
            xin = x_in.ctypes.data
        am = C.c_int(-1)
        if self.is_last:
            ptr = self._logits.ctypes.data if want_logits else None
            rc = self._lib.l2j_forward_stage(self._ctx, int(token), int(pos), xin, None, ptr, C.byref(am))
            _lib.check(rc, self._ctx)
            return (self._logits if want_logits else None), am.value
        x_out = np.empty(self.cfg.dim, dtype=np.float32)
        rc = self._lib.l2j_forward_stage(self._ctx, int(token), int(pos), xin, x_out.ctypes.data, None, None)
        _lib.check(rc, self._ctx)
        return x_out

    def prefill(self, tokens, pos0: int = 0) -> None:
        """Positions pos0 .. pos0 + len(tokens) - 1 in batches of 64 on the tensor cores; tokens[i] is the input
        token of position pos0 + i (BOS, then the prompt: Run.java:614,635-637).  No logits."""
        t = np.ascontiguousarray(tokens, dtype=np.int32).reshape(-1)
        ptr = t.ctypes.data_as(C.POINTER(C.c_int32)) if t.size else None
        _lib.check(self._lib.l2j_prefill(self._ctx, ptr, int(t.size), int(pos0)), self._ctx)

    def prefill_launches(self) -> int:
        return int(self._lib.l2j_prefill_launches(self._ctx))

    def batch_create(self, n_seq: int, seq_len: int) -> None:
        """K/V caches for n_seq concurrent sequences of seq_len positions."""
        _lib.check(self._lib.l2j_batch_create(self._ctx, int(n_seq), int(seq_len)), self._ctx)

    def batch_forward(self, seq, pos, tokens, want_logits: bool = True):
        """One decode step for up to 64 (sequence, position, token) entries on one sweep over the weights;
        returns (logits [n, vocab] or None, arg-max [n])."""
        sq = np.ascontiguousarray(seq, dtype=np.int32).reshape(-1)
        ps = np.ascontiguousarray(pos, dtype=np.int32).reshape(-1)
        tk = np.ascontiguousarray(tokens, dtype=np.int32).reshape(-1)
        n = int(sq.size)
        assert ps.size == n and tk.size == n
        logits = np.empty((n, self.cfg.vocab_size), dtype=np.float32) if want_logits else None
        am = np.zeros(n, dtype=np.int32)
        ip = C.POINTER(C.c_int32)
        rc = self._lib.l2j_batch_forward(self._ctx, n, sq.ctypes.data_as(ip), ps.ctypes.data_as(ip), tk.ctypes.data_as(ip),
                                         logits.ctypes.data if want_logits else None, am.ctypes.data_as(ip))
        _lib.check(rc, self._ctx)
        return logits, am

    def sampler_seed(self, seed: int) -> None:
        """new Sampler(seed, vocab) on the device (Sampler.java:24-31)."""
        _lib.check(self._lib.l2j_sampler_seed(self._ctx, int(seed)), self._ctx)

    def sample(self, temperature: float, topp: float) -> int:
        """The token the reference's Sampler would choose from the logits of the last forward (Run.java:639-665)."""
        tok = C.c_int(-1)
        _lib.check(self._lib.l2j_sample(self._ctx, C.c_float(temperature), C.c_float(topp), C.byref(tok)), self._ctx)
        return tok.value

    def generate_greedy(self, prompt, steps: int) -> np.ndarray:
        """Greedy run loop on the device; element p is the token chosen after position p."""
        prompt = np.ascontiguousarray(prompt, dtype=np.int32).reshape(-1)
        out = np.zeros(steps, dtype=np.int32)
        rc = self._lib.l2j_generate_greedy(self._ctx, prompt.ctypes.data if prompt.size else None, int(prompt.size),
                                           int(steps), out.ctypes.data)
        _lib.check(rc, self._ctx)
        return out

    def last_generate_us(self) -> float:
        v = C.c_double(0.0)
        _lib.check(self._lib.l2j_last_generate_us(self._ctx, C.byref(v)), self._ctx)
        return v.value

    def time_kernels(self, pos: int, reps: int = 3) -> dict:
        """Average device microseconds per launch of each kernel of a layer at position `pos`."""
        arr = (C.c_double * 6)()
        _lib.check(self._lib.l2j_time_kernels(self._ctx, int(pos), int(reps), arr), self._ctx)
        return dict(zip(("qkv_rope", "attention", "wo_residual", "w13_swiglu", "w2_residual", "classifier_argmax"), arr))

    def time_layers_kernel(self, pos: int, reps: int = 3) -> float:
        """Average device microseconds of one launch of the persistent all-layers kernel at position `pos`."""
        us = C.c_double(0.0)
        _lib.check(self._lib.l2j_time_layers_kernel(self._ctx, int(pos), int(reps), C.byref(us)), self._ctx)
        return us.value

    def trace_kernel(self, kind: int, layer: int = 0, pos: int = 0) -> np.ndarray:
        """In-kernel timeline of one ring-kernel launch: array (blocks, 8), see l2j_trace_kernel."""
        nb = self.launch_mode()["ring_blocks"]
        out = np.zeros((nb, 16), dtype=np.uint64)
        _lib.check(self._lib.l2j_trace_kernel(self._ctx, kind, layer, pos, out.ctypes.data, nb), self._ctx)
        return out

    def read_trace(self) -> np.ndarray:
        """Timelines of every launch of the last forward: (launches, blocks, 16); the ring kernels of the
        layers first (4 per layer), the classifier, then the attention kernels (one per layer)."""
        launches = 5 * (self.last_layer - self.first_layer + 1) + 1
        nb = self.launch_mode()["ring_blocks"]
        out = np.zeros((launches, nb, 16), dtype=np.uint64)
        _lib.check(self._lib.l2j_read_trace(self._ctx, out.ctypes.data, out.size), self._ctx)
        return out

    def kv_write(self, layer: int, pos0: int, k_rows: np.ndarray, v_rows: np.ndarray) -> None:
        """Restores rows [pos0, pos0 + len) of a layer's KV cache from (position, kv_dim) float arrays, the
        layout the reference keeps them in (RunState.java:141-151)."""
        k = np.ascontiguousarray(k_rows, dtype=np.float32)
        v = np.ascontiguousarray(v_rows, dtype=np.float32)
        if k.shape != v.shape or k.ndim != 2 or k.shape[1] != self.cfg.kv_dim:
            raise ValueError("k_rows and v_rows must both be (positions, kv_dim)")
        _lib.check(self._lib.l2j_kv_write(self._ctx, int(layer), int(pos0), int(k.shape[0]), k.ctypes.data, v.ctypes.data),
                   self._ctx)

    def reset(self) -> None:
        _lib.check(self._lib.l2j_reset(self._ctx), self._ctx)

    def set_wait_limit_us(self, limit_us: int) -> None:
        """Bound of every device-side wait (before finalize); see l2j_set_wait_limit_us."""
        _lib.check(self._lib.l2j_set_wait_limit_us(self._ctx, int(limit_us)), self._ctx)

    def debug_desync(self) -> None:
        """Host-side failure injection: the next forward waits for hand-overs that never come."""
        _lib.check(self._lib.l2j_debug_desync(self._ctx), self._ctx)

    def stats(self) -> _lib.Stats:
        st = _lib.Stats()
        _lib.check(self._lib.l2j_get_stats(self._ctx, C.byref(st)), self._ctx)
        return st

    def launch_mode(self) -> dict:
        m = self._lib.l2j_launch_mode(self._ctx)
        return {"graph": bool(m & 1), "pdl": bool(m & 2), "ring": bool(m & 4), "persistent": bool(m & 8),
                "ring_blocks": m >> 8}

    def read_buffer(self, which: int, n: int, layer: int = 0, pos: int = 0) -> np.ndarray:
        out = np.empty(n, dtype=np.float32)
        _lib.check(self._lib.l2j_read_buffer(self._ctx, which, layer, pos, out.ctypes.data, n), self._ctx)
        return out

    def device_buffers(self):
        x, lg = C.c_void_p(), C.c_void_p()
        _lib.check(self._lib.l2j_device_buffers(self._ctx, C.byref(x), C.byref(lg)), self._ctx)
        return x.value, lg.value


def run_greedy_host_loop(model: Transformer, prompt, steps: int, stop_on_bos: bool = True):
    """The reference's run loop (Run.java:609-685) with --temp 0.0, one blocking forward per token and
    the arg-max on the host, exactly what the Java host does through the ABI.  Returns the chosen
    tokens (forced ones included) and the logits of every step."""
    prompt = [int(t) for t in prompt]
    token, pos = 1, 0   # BOS, Run.java:614
    chosen, all_logits = [], []
    while pos < steps:
        logits, _ = model.forward(token, pos)
        if pos < len(prompt):
            nxt = prompt[pos]          # Run.java:635-637
        else:
            nxt = argmax(logits)       # Run.java:640-642
        all_logits.append(logits.copy())
        chosen.append(nxt)
        pos += 1
        if stop_on_bos and nxt == 1:   # Run.java:670-672
            break
        token = nxt
    return np.asarray(chosen, dtype=np.int32), np.stack(all_logits) if all_logits else np.zeros((0, model.cfg.vocab_size))


class LinkedStages:
    """A layer split driven by one host thread, the reference's multi-GPU mode (Run.java:368-413,
    Context.java:16-23): stage i is a Transformer on its own device holding a contiguous layer range,
    and each stage reads x from the device of the stage in front over the peer link."""

    def __init__(self, stages, link: bool = True):
        self.stages = list(stages)
        if not self.stages:
            raise ValueError("no stages")
        self._lib = _lib.load()
        self._arr = (C.c_void_p * len(self.stages))(*[s._ctx for s in self.stages])
        self._logits = np.zeros(self.stages[0].cfg.vocab_size, dtype=np.float32)
        if link:
            self.link()

    def link(self) -> None:
        """l2j_pipeline_link: every stage learns where its neighbour's x (and the chosen token) lives."""
        _lib.check(self._lib.l2j_pipeline_link(self._arr, len(self.stages)), self.stages[0]._ctx)

    def reset(self) -> None:
        _lib.check(self._lib.l2j_pipeline_reset(self._arr, len(self.stages)), self.stages[0]._ctx)

    @classmethod
    def from_allocation(cls, cfg: ModelConfig, first_layers, last_layers, tensors: dict, devices=None, flags: int = 0):
        """One stage per (first, last) layer range, e.g. the ranges LayerAllocation computes from --gpuMem."""
        devices = list(range(len(first_layers))) if devices is None else list(devices)
        stages = []
        for dev, a, b in zip(devices, first_layers, last_layers):
            t = Transformer(cfg, device=dev, first_layer=a, last_layer=b, flags=flags)
            t.upload_all(tensors)
            t.finalize()
            stages.append(t)
        return cls(stages)

    def forward(self, token: int, pos: int, want_logits: bool = True):
        am = C.c_int(-1)
        ptr = self._logits.ctypes.data if want_logits else None
        rc = self._lib.l2j_pipeline_forward(self._arr, len(self.stages), int(token), int(pos), ptr, C.byref(am))
        _lib.check(rc, self.stages[0]._ctx)
        return (self._logits if want_logits else None), am.value

    def generate_greedy(self, prompt, steps: int) -> np.ndarray:
        prompt = np.ascontiguousarray(prompt, dtype=np.int32).reshape(-1)
        out = np.zeros(steps, dtype=np.int32)
        rc = self._lib.l2j_pipeline_generate_greedy(self._arr, len(self.stages), prompt.ctypes.data if prompt.size else None,
                                                    int(prompt.size), int(steps), out.ctypes.data)
        _lib.check(rc, self.stages[0]._ctx)
        return out

    def last_generate_us(self) -> float:
        return self.stages[0].last_generate_us()

    def close(self) -> None:
        for s in self.stages:
            s.close()


class TensorParallel:
    """A tensor-parallel group driven by one host thread: rank r (a Transformer created with tp_rank=r on a
    device of its own) computes a block of rows of every matrix and stores its results into all ranks'
    vectors over the peer links.  The reference has no such mode; results are bitwise those of one device."""

    def __init__(self, ranks):
        self.ranks = list(ranks)
        self._lib = _lib.load()
        self._arr = (C.c_void_p * len(self.ranks))(*[r._ctx for r in self.ranks])
        _lib.check(self._lib.l2j_tp_link(self._arr, len(self.ranks)), self.ranks[0]._ctx)
        self._logits = np.zeros(self.ranks[0].cfg.vocab_size, dtype=np.float32)

    @classmethod
    def from_devices(cls, cfg: ModelConfig, tensors: dict, devices, flags: int = 0):
        devices = list(devices)
        ranks = []
        for r, dev in enumerate(devices):
            t = Transformer(cfg, device=dev, flags=flags, tp_rank=r, tp_size=len(devices))
            t.upload_all(tensors)
            t.finalize()
            ranks.append(t)
        return cls(ranks)

    def forward(self, token: int, pos: int, want_logits: bool = True):
        am = C.c_int(-1)
        ptr = self._logits.ctypes.data if want_logits else None
        rc = self._lib.l2j_tp_forward(self._arr, len(self.ranks), int(token), int(pos), ptr, C.byref(am))
        _lib.check(rc, self.ranks[0]._ctx)
        return (self._logits if want_logits else None), am.value

    def generate_greedy(self, prompt, steps: int) -> np.ndarray:
        prompt = np.ascontiguousarray(prompt, dtype=np.int32).reshape(-1)
        out = np.zeros(steps, dtype=np.int32)
        rc = self._lib.l2j_tp_generate_greedy(self._arr, len(self.ranks), prompt.ctypes.data if prompt.size else None,
                                              int(prompt.size), int(steps), out.ctypes.data)
        _lib.check(rc, self.ranks[0]._ctx)
        return out

    def last_generate_us(self) -> float:
        return self.ranks[0].last_generate_us()

    def reset(self) -> None:
        """l2j_tp_reset: every rank starts a new sequence (their hand-over counters must agree)."""
        _lib.check(self._lib.l2j_tp_reset(self._arr, len(self.ranks)), self.ranks[0]._ctx)

    def close(self) -> None:
        for r in self.ranks:
            r.close()
