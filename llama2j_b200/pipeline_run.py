"""Times the layer split on linked stages: the reference's `--gpuMem a,b,...` mode (Run.java:368-413)
with equal budgets, greedy decode kept on the devices.

  python -m llama2j_b200.pipeline_run --shape llama2-13b --stages 2 [--check]

Prints one JSON line: tok/s over `--forwards` positions (BOS + 32 forced prompt tokens, then greedy),
the layer ranges, and with --check whether the tokens equal those of a single-device run.
"""
from __future__ import annotations

import argparse
import json

import numpy as np

from . import synthetic as syn
from .layer_allocation import LayerAllocation
from .transformer import LinkedStages, Transformer


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="llama2-13b")
    ap.add_argument("--stages", type=int, default=2)
    ap.add_argument("--forwards", type=int, default=288)
    ap.add_argument("--repeats", type=int, default=3)
    ap.add_argument("--check", action="store_true", help="compare with a single-device run of the same checkpoint")
    ap.add_argument("--same-device", action="store_true", help="all stages on device 0 (hand-over logic without a peer link)")
    args = ap.parse_args()
    cfg = syn.SHAPES[args.shape]
    alloc = LayerAllocation.equal_split(args.stages, cfg)
    tensors = syn.synthetic_tensors(cfg, 0)
    prompt = syn.synthetic_prompt(32, 1, cfg.vocab_size)
    devices = [0] * args.stages if args.same_device else list(range(args.stages))
    out = {"shape": args.shape, "stages": args.stages, "devices": devices, "first_layer": list(alloc.first_layer),
           "last_layer": list(alloc.last_layer), "forwards": args.forwards}
    ref = None
    if args.check:
        with Transformer(cfg) as whole:
            whole.upload_all(tensors)
            whole.finalize()
            whole.generate_greedy(prompt, args.forwards)
            ref = whole.generate_greedy(prompt, args.forwards)
            out["single_device_tok_s"] = args.forwards / (whole.last_generate_us() * 1e-6)
    split = LinkedStages.from_allocation(cfg, alloc.first_layer, alloc.last_layer, tensors, devices)
    toks = split.generate_greedy(prompt, args.forwards)   # warm-up
    us = []
    for _ in range(args.repeats):
        toks = split.generate_greedy(prompt, args.forwards)
        us.append(split.last_generate_us())
    out["tok_s"] = args.forwards / (float(np.median(us)) * 1e-6)
    out["us_per_forward"] = float(np.median(us)) / args.forwards
    if ref is not None:
        out["tokens_equal_single_device"] = bool(np.array_equal(ref, toks))
    split.close()
    print(json.dumps(out))


if __name__ == "__main__":
    main()
