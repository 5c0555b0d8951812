"""The C-ABI library builds for sm_100a, loads, and exports every symbol the header declares.
No compute call is made here (no GPU on the CPU test box)."""
import os
import re

from llama2j_b200 import lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "l2j_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(l2j_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(l2j):
    lib = l2j.load()
    declared = _declared_symbols()
    assert len(declared) >= 25
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/l2j_b200.h but not exported"
    assert sorted(L.EXPORTED_SYMBOLS) == declared          # the Python binding covers the whole header


def test_header_constants_match_binding():
    text = open(os.path.join(ROOT, "include", "l2j_b200.h")).read()
    assert "#define L2J_QUANT_GROUP 256" in text and "#define L2J_QUANT_GROUP_BYTES 264" in text
    ids = re.findall(r"L2J_T_[A-Z0-9_]+ = (\d+)", text)
    assert [int(i) for i in ids] == list(range(13))
    assert (L.F_NO_GRAPH, L.F_NO_PDL, L.F_SIMPLE) == (1, 2, 4)


def test_missing_device_fails_loudly(l2j):
    """Without a CUDA device the library refuses to create a context: there is no CPU path."""
    import ctypes as C
    import torch
    if torch.cuda.is_available():
        return
    lib = l2j.load()
    cfg = l2j.Config(64, 176, 2, 4, 2, 96, 32, 0)
    ctx = C.c_void_p()
    rc = lib.l2j_create(C.byref(cfg), 0, 0, 1, 0, C.byref(ctx))
    assert rc == l2j.E_CUDA and not ctx.value
    assert b"no CPU path" in lib.l2j_last_error(None)
