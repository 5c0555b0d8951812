"""Writes tests/golden/oracle_golden.npz from the CPU oracle.

The reference project has no golden vectors and cannot be executed without a JVM, so these vectors
are regression pins of the oracle (oracle/l2j_oracle.c), not outputs of the reference.
Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from llama2j_b200.model_files import ModelConfig  # noqa: E402
from oracle import cpu_oracle as o  # noqa: E402

TINY = ModelConfig(dim=64, hidden_dim=176, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=96, seq_len=32,
                   shared_classifier=False)


def main():
    rng = np.random.default_rng(42)
    quant_in = rng.normal(0, 0.02, 256 * 3 + 17).astype(np.float32)
    tensors = o.synthetic_tensors(TINY, seed=11)
    m = o.OracleModel(TINY, tensors, o.SILU_EXACT, o.SOFTMAX_REFERENCE)
    prompt = np.array([5, 77, 31, 8], dtype=np.int32)
    steps = 16
    toks, lgs = o.greedy_run(m, prompt, steps)
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "oracle_golden.npz"),
                        quant_in=quant_in, quant_out=o.quant_encode(quant_in), synth=o.synth_normal(64, 0, 2),
                        prompt=prompt, steps=steps, tokens=toks, logits=lgs)


if __name__ == "__main__":
    main()
