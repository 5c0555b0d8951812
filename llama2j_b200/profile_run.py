"""A short, fixed decode run for profilers: builds a synthetic checkpoint of a benchmark shape
(optionally with fewer layers, so that a full-metric capture holds only a few GB on the device),
decodes a few tokens on the device and prints per-kernel event timings.

  python -m llama2j_b200.profile_run --shape llama2-7b --layers 4 --forwards 4
  python -m llama2j_b200.profile_run --shape llama2-7b --layers 4 --forwards 0 --prefill 128 --pos0 1024
  python -m llama2j_b200.profile_run --shape llama2-7b --layers 4 --forwards 0 --concurrent 64 --steps 3
  python -m llama2j_b200.profile_run --shape llama2-7b --layers 2 --forwards 0 --flags 8 --prefill 3840 --decode 3

Meant to be run plainly first and then under `ncu --clock-control none ...`.
"""
from __future__ import annotations

import argparse
import json

import numpy as np

from . import synthetic as syn
from .model_files import ModelConfig
from .transformer import Transformer


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="llama2-7b")
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (0: the shape's own)")
    ap.add_argument("--forwards", type=int, default=4)
    ap.add_argument("--flags", type=int, default=0)
    ap.add_argument("--time-kernels", type=int, default=0, help="position for the per-kernel event timing (0: skip)")
    ap.add_argument("--prefill", type=int, default=0, help="tokens to push through l2j_prefill, twice (0: skip)")
    ap.add_argument("--pos0", type=int, default=0, help="first position of the prefill")
    ap.add_argument("--decode", type=int, default=0, help="decode steps after the prefill, from the position behind it (0: skip)")
    ap.add_argument("--concurrent", type=int, default=0, help="sequences to decode together with l2j_batch_forward (0: skip)")
    ap.add_argument("--steps", type=int, default=3, help="steps of the concurrent run")
    args = ap.parse_args()
    base = syn.SHAPES[args.shape]
    cfg = base if args.layers <= 0 else ModelConfig(base.dim, base.hidden_dim, args.layers, base.n_heads, base.n_kv_heads,
                                                     base.vocab_size, base.seq_len, base.shared_classifier)
    tensors = syn.synthetic_tensors(cfg, 0)
    prompt = syn.synthetic_prompt(32, 1, cfg.vocab_size)
    with Transformer(cfg, flags=args.flags) as m:
        m.upload_all(tensors)
        m.finalize()
        out = {"shape": args.shape, "layers": cfg.n_layers, "forwards": args.forwards, "mode": m.launch_mode()}
        if args.forwards > 0:
            toks = m.generate_greedy(prompt, args.forwards)
            out.update({"us_per_forward": m.last_generate_us() / args.forwards, "tokens": [int(t) for t in toks[:8]],
                        "kernels_per_forward": int(m.stats().kernels_per_forward)})
        if args.prefill > 0:
            inputs = np.concatenate([[1], syn.synthetic_prompt(args.prefill - 1, 3, cfg.vocab_size)]).astype(np.int32)
            m.prefill(inputs, args.pos0)
            m.prefill(inputs, args.pos0)
            out["prefill_launches"] = m.prefill_launches()
            tok = 7
            for i in range(args.decode):          # long-context decode steps over the cache the prefill left
                _, tok = m.forward(tok, args.pos0 + args.prefill + i, want_logits=False)
        if args.concurrent > 0:
            m.batch_create(args.concurrent, 64)
            toks = np.ones(args.concurrent, dtype=np.int32)
            for p in range(args.steps):
                _, toks = m.batch_forward(np.arange(args.concurrent), np.full(args.concurrent, p), toks, want_logits=False)
            out["concurrent_tokens"] = [int(t) for t in toks[:4]]
        out["device_status"] = int(m.stats().device_status)
        if args.time_kernels > 0:
            out["kernel_us"] = m.time_kernels(args.time_kernels, reps=2)
        print(json.dumps(out))


if __name__ == "__main__":
    main()
