"""A short, fixed decode run for profilers: builds a synthetic checkpoint of a benchmark shape
(optionally with fewer layers, so that a full-metric capture holds only a few GB on the device),
decodes a few tokens on the device and prints per-kernel event timings.

  python -m llama2j_b200.profile_run --shape llama2-7b --layers 4 --forwards 4

Meant to be run plainly first and then under `ncu --clock-control none ...`.
"""
from __future__ import annotations

import argparse
import json

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
    args = ap.parse_args()
    base = syn.SHAPES[args.shape]
    cfg = base if args.layers <= 0 else ModelConfig(base.dim, base.hidden_dim, args.layers, base.n_heads, base.n_kv_heads,
                                                     base.vocab_size, base.seq_len, base.shared_classifier)
    tensors = syn.synthetic_tensors(cfg, 0)
    prompt = syn.synthetic_prompt(32, 1, cfg.vocab_size)
    with Transformer(cfg, flags=args.flags) as m:
        m.upload_all(tensors)
        m.finalize()
        toks = m.generate_greedy(prompt, args.forwards)
        out = {"shape": args.shape, "layers": cfg.n_layers, "forwards": args.forwards, "mode": m.launch_mode(),
               "us_per_forward": m.last_generate_us() / args.forwards, "tokens": [int(t) for t in toks[:8]],
               "kernels_per_forward": int(m.stats().kernels_per_forward)}
        if args.time_kernels > 0:
            out["kernel_us"] = m.time_kernels(args.time_kernels, reps=2)
        print(json.dumps(out))


if __name__ == "__main__":
    main()
