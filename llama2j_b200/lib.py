"""ctypes binding of libl2j_b200.so, the C ABI declared in include/l2j_b200.h.

There is no fallback: if the shared object has not been built, or no CUDA device is present when a
compute call is made, the call raises.  Every function of the header is bound here with the same
name minus the ``l2j_`` prefix.
"""
from __future__ import annotations

import ctypes as C
import os

from . import build as _build

E_INVALID, E_CUDA, E_STATE, E_DEVICE, E_NOMEM = -1, -2, -3, -4, -5
DS_WAIT_TIMEOUT, DS_BAD_POS, DS_BAD_TOKEN, DS_BAD_LINK = 0x1, 0x2, 0x4, 0x8
F_NO_GRAPH, F_NO_PDL, F_SIMPLE, F_STEP_KERNELS, F_TP_SPLIT_CLASSIFIER, F_PERSISTENT = 0x1, 0x2, 0x4, 0x8, 0x10, 0x20
F_NO_TENSOR_PREFILL = 0x40
QUANT_GROUP, QUANT_GROUP_BYTES = 256, 264

(T_TOKEN_EMBEDDING, T_RMS_ATT, T_WQ, T_WK, T_WV, T_WO, T_RMS_FFN, T_W1, T_W2, T_W3, T_RMS_FINAL, T_WCLS) = range(12)
QUANT_TENSORS = (T_RMS_ATT, T_WQ, T_WK, T_WV, T_WO, T_RMS_FFN, T_W1, T_W2, T_W3, T_RMS_FINAL)
TENSOR_NAMES = {
    T_TOKEN_EMBEDDING: "token_embedding_table", T_RMS_ATT: "l_rms_att_weight", T_WQ: "l_wq", T_WK: "l_wk",
    T_WV: "l_wv", T_WO: "l_wo", T_RMS_FFN: "l_rms_ffn_weight", T_W1: "l_w1", T_W2: "l_w2", T_W3: "l_w3",
    T_RMS_FINAL: "rms_final_weight", T_WCLS: "wcls",
}


class L2jError(RuntimeError):
    """A call into libl2j_b200 returned a non-zero status."""

    def __init__(self, code: int, message: str):
        super().__init__(f"l2j error {code}: {message}")
        self.code = code


class Config(C.Structure):
    """l2j_config: the seven header ints of a llama2.c checkpoint plus the shared-classifier flag."""

    _fields_ = [(n, C.c_int32) for n in ("dim", "hidden_dim", "n_layers", "n_heads", "n_kv_heads", "vocab_size",
                                         "seq_len", "shared_classifier")]


class Stats(C.Structure):
    _fields_ = [("forwards", C.c_int64), ("kernels_per_forward", C.c_int64), ("device_bytes", C.c_int64),
                ("device_status", C.c_int32), ("last_pos", C.c_int32), ("last_token", C.c_int32), ("sm_count", C.c_int32)]


_P = C.c_void_p
_SIGNATURES = {
    "l2j_create": (C.c_int, [C.POINTER(Config), C.c_int, C.c_int, C.c_int, C.c_uint32, C.POINTER(_P)]),
    "l2j_destroy": (None, [_P]),
    "l2j_last_error": (C.c_char_p, [_P]),
    "l2j_upload_quant": (C.c_int, [_P, C.c_int, C.c_int64, _P, C.c_int64, C.c_int64]),
    "l2j_upload_f32": (C.c_int, [_P, C.c_int, C.c_int64, _P, C.c_int64]),
    "l2j_finalize": (C.c_int, [_P]),
    "l2j_forward": (C.c_int, [_P, C.c_int, C.c_int, _P, C.POINTER(C.c_int)]),
    "l2j_forward_stage": (C.c_int, [_P, C.c_int, C.c_int, _P, _P, _P, C.POINTER(C.c_int)]),
    "l2j_prefill": (C.c_int, [_P, C.POINTER(C.c_int32), C.c_int, C.c_int]),
    "l2j_prefill_launches": (C.c_uint64, [_P]),
    "l2j_batch_create": (C.c_int, [_P, C.c_int, C.c_int]),
    "l2j_batch_forward": (C.c_int, [_P, C.c_int, C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.c_void_p,
                                   C.POINTER(C.c_int32)]),
    "l2j_sampler_seed": (C.c_int, [_P, C.c_int64]),
    "l2j_sample": (C.c_int, [_P, C.c_float, C.c_float, C.POINTER(C.c_int)]),
    "l2j_device_buffers": (C.c_int, [_P, C.POINTER(_P), C.POINTER(_P)]),
    "l2j_forward_stage_async": (C.c_int, [_P, C.c_int, C.c_int]),
    "l2j_sync": (C.c_int, [_P]),
    "l2j_generate_greedy": (C.c_int, [_P, _P, C.c_int, C.c_int, _P]),
    "l2j_pipeline_link": (C.c_int, [C.POINTER(_P), C.c_int]),
    "l2j_pipeline_forward": (C.c_int, [C.POINTER(_P), C.c_int, C.c_int, C.c_int, _P, C.POINTER(C.c_int)]),
    "l2j_pipeline_generate_greedy": (C.c_int, [C.POINTER(_P), C.c_int, _P, C.c_int, C.c_int, _P]),
    "l2j_create_tp": (C.c_int, [C.POINTER(Config), C.c_int, C.c_int, C.c_int, C.c_uint32, C.POINTER(_P)]),
    "l2j_tp_link": (C.c_int, [C.POINTER(_P), C.c_int]),
    "l2j_tp_forward": (C.c_int, [C.POINTER(_P), C.c_int, C.c_int, C.c_int, _P, C.POINTER(C.c_int)]),
    "l2j_tp_generate_greedy": (C.c_int, [C.POINTER(_P), C.c_int, _P, C.c_int, C.c_int, _P]),
    "l2j_reset": (C.c_int, [_P]),
    "l2j_tp_reset": (C.c_int, [C.POINTER(_P), C.c_int]),
    "l2j_pipeline_reset": (C.c_int, [C.POINTER(_P), C.c_int]),
    "l2j_set_wait_limit_us": (C.c_int, [_P, C.c_int]),
    "l2j_debug_desync": (C.c_int, [_P]),
    "l2j_get_stats": (C.c_int, [_P, C.POINTER(Stats)]),
    "l2j_launch_mode": (C.c_int, [_P]),
    "l2j_read_buffer": (C.c_int, [_P, C.c_int, C.c_int, C.c_int, _P, C.c_int]),
    "l2j_kv_write": (C.c_int, [_P, C.c_int, C.c_int, C.c_int, _P, _P]),
    "l2j_last_generate_us": (C.c_int, [_P, C.POINTER(C.c_double)]),
    "l2j_time_kernels": (C.c_int, [_P, C.c_int, C.c_int, C.POINTER(C.c_double)]),
    "l2j_time_layers_kernel": (C.c_int, [_P, C.c_int, C.c_int, C.POINTER(C.c_double)]),
    "l2j_trace_kernel": (C.c_int, [_P, C.c_int, C.c_int, C.c_int, _P, C.c_int]),
    "l2j_read_trace": (C.c_int, [_P, _P, C.c_int64]),
    "l2j_quant_encode": (C.c_int, [C.c_int, _P, C.c_int64, _P]),
    "l2j_synth_f32": (C.c_int, [C.c_int, C.c_uint64, C.c_uint32, C.c_int64, C.c_int64, C.c_float, _P]),
    "l2j_synth_quant": (C.c_int, [C.c_int, C.c_uint64, C.c_uint32, C.c_int64, C.c_float, _P]),
    "l2j_k_matvec_i8": (C.c_int, [C.c_int, C.c_uint32, _P, C.c_int64, C.c_int64, C.c_int, C.c_int, _P, _P]),
    "l2j_k_matvec_f32": (C.c_int, [C.c_int, C.c_uint32, _P, C.c_int, C.c_int, _P, _P, C.POINTER(C.c_int)]),
    "l2j_k_rmsnorm": (C.c_int, [C.c_int, _P, C.c_int64, C.c_int64, C.c_int, _P, _P]),
    "l2j_k_rope": (C.c_int, [C.c_int, _P, _P, C.c_int, C.c_int, C.c_int, C.c_int]),
    "l2j_k_attention": (C.c_int, [C.c_int, _P, _P, _P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _P]),
    "l2j_k_swiglu": (C.c_int, [C.c_int, _P, _P, C.c_int]),
    "l2j_k_attention_noalloc": (C.c_int, [C.c_int, _P, _P, _P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _P, _P]),
    "l2j_noalloc_last_error": (C.c_char_p, []),
}

EXPORTED_SYMBOLS = tuple(_SIGNATURES)

_lib = None


def library_path() -> str:
    return _build.LIB_PATH


def load(build_if_missing: bool = False):
    """Loads the shared object (once) and returns the ctypes handle.

    Raises FileNotFoundError when the library has not been built; pass build_if_missing=True to run
    nvcc first."""
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if not os.path.exists(path):
        if not build_if_missing:
            raise FileNotFoundError(
                f"{path} is missing: build it with `python -m llama2j_b200.build` (there is no CPU fallback)")
        _build.build()
    lib = C.CDLL(path)
    for name, (restype, argtypes) in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(rc: int, ctx=None) -> None:
    """Raises L2jError for a non-zero status, with the library's message."""
    if rc != 0:
        msg = load().l2j_last_error(ctx)
        raise L2jError(rc, msg.decode("utf-8", "replace") if msg else "")
