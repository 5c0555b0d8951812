"""Times the two multi-GPU modes on the devices of one box, driven by one host thread:

  --mode pipeline   the reference's `--gpuMem a,b,...` layer split (Run.java:368-413) with equal budgets,
                    stages linked over the peer links
  --mode tp         the tensor-parallel group (no counterpart in the reference)

  python -m llama2j_b200.multi_gpu_run --mode tp --shape llama2-13b --gpus 2 [--check] [--long]

Prints one JSON line: tok/s of greedy decode kept on the devices (BOS + 32 forced prompt tokens, then
greedy, `--forwards` positions; with --long a 3840-token prompt and the rate over positions 3840-4095),
and with --check whether the tokens equal those of a single-device run of the same checkpoint.
"""
from __future__ import annotations

import argparse
import json

import numpy as np

from . import synthetic as syn
from .layer_allocation import LayerAllocation
from .transformer import LinkedStages, TensorParallel, Transformer


def _timed(model, prompt, forwards: int, repeats: int):
    toks = model.generate_greedy(prompt, forwards)   # warm-up
    us = []
    for _ in range(repeats):
        toks = model.generate_greedy(prompt, forwards)
        us.append(model.last_generate_us())
    return toks, float(np.median(us))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", choices=["pipeline", "tp"], default="pipeline")
    ap.add_argument("--shape", default="llama2-13b")
    ap.add_argument("--gpus", type=int, default=2)
    ap.add_argument("--forwards", type=int, default=288)
    ap.add_argument("--repeats", type=int, default=3)
    ap.add_argument("--long", action="store_true", help="3840-token prompt, rate over positions 3840..seq_len-1")
    ap.add_argument("--check", action="store_true", help="compare with a single-device run of the same checkpoint")
    args = ap.parse_args()
    cfg = syn.SHAPES[args.shape]
    tensors = syn.synthetic_tensors(cfg, 0)
    n_prompt = min(3840, cfg.seq_len - 2) if args.long else 32
    forwards = cfg.seq_len if args.long else args.forwards
    prompt = syn.synthetic_prompt(n_prompt, 1, cfg.vocab_size)
    devices = list(range(args.gpus))
    out = {"mode": args.mode, "shape": args.shape, "devices": devices, "forwards": forwards, "prompt": n_prompt}

    def rate(model):
        toks, us_full = _timed(model, prompt, forwards, args.repeats)
        if not args.long:
            return toks, forwards / (us_full * 1e-6), us_full / forwards
        _, us_head = _timed(model, prompt, n_prompt, args.repeats)
        n = forwards - n_prompt
        return toks, n / ((us_full - us_head) * 1e-6), (us_full - us_head) / n

    ref = None
    if args.check:
        with Transformer(cfg) as whole:
            whole.upload_all(tensors)
            whole.finalize()
            ref, out["single_device_tok_s"], _ = rate(whole)
    if args.mode == "pipeline":
        alloc = LayerAllocation.equal_split(args.gpus, cfg)
        out["first_layer"], out["last_layer"] = list(alloc.first_layer), list(alloc.last_layer)
        model = LinkedStages.from_allocation(cfg, alloc.first_layer, alloc.last_layer, tensors, devices)
    else:
        model = TensorParallel.from_devices(cfg, tensors, devices)
    toks, out["tok_s"], out["us_per_forward"] = rate(model)
    if ref is not None:
        out["tokens_equal_single_device"] = bool(np.array_equal(ref, toks))
    model.close()
    print(json.dumps(out))


if __name__ == "__main__":
    main()
