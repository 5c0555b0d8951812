"""Command-line run loop with the reference's flags, CUDA mode only.

Mirror of Run.main (Run.java:528-707) and CommandLine (CommandLine.java:12-133) for the decode path:
`--checkpoint X --mode CUDA --gpuMem a,b --temp T --topp P --seed S --steps N`, checkpoint resolved under
`models/`, quant cache files beside it (TransformerWeights.java:191-232).  With --temp > 0 the token is
chosen on the device by the restatement of Sampler.java (same java.util.Random stream for the same seed),
and only its id comes back.  The tokenizer stays outside this
repository, so prompts are token ids (`--promptTokens 5,17,...`, an addition) and the output is ids.
There is no CPU mode here: `--mode CPU` is refused.

  python -m llama2j_b200.run --checkpoint stories15M.bin --temp 0.0 --steps 64 --promptTokens 5,9
"""
from __future__ import annotations

import os
import sys
import time

import numpy as np

from . import lib as _lib
from . import model_files as mf
from . import synthetic as syn
from .layer_allocation import LayerAllocation, parse_gpu_mem
from .transformer import LinkedStages, Transformer, argmax

MODELS_DIRECTORY = "models"   # Run.java:34

FLAGS = ("--checkpoint", "--mode", "--temp", "--topp", "--seed", "--steps", "--gpuMem", "--prompt", "--tokenizer",
         "--promptTokens")


def parse_args(argv):
    """`--flag value` pairs (CommandLine.java:35-39) with the reference's defaults (CommandLine.java:22-29)."""
    args = {"--mode": "CUDA", "--temp": "0.9", "--topp": "0.9", "--steps": "256", "--gpuMem": None,
            "--promptTokens": ""}
    for i in range(0, len(argv) - 1, 2):
        args[argv[i]] = argv[i + 1]
    if "--checkpoint" not in args:
        raise SystemExit("Usage: --checkpoint <file> [--mode CUDA] [--temp 0.0] [--steps N] [--gpuMem a,b,...] "
                         "[--promptTokens id,id,...]")
    return args


def load_quant_tensor(path: str, cfg: mf.ModelConfig, tensor: int, device: int) -> np.ndarray:
    """readAsQuant (TransformerWeights.java:191-232): use the cache file if present, otherwise quantise the
    checkpoint tensor (on the GPU, bit-exact Quant.encode) and write the cache."""
    n = cfg.tensor_floats(tensor)
    layers = 1 if tensor == _lib.T_RMS_FINAL else cfg.n_layers
    cached = mf.read_quant_cache_parts(path, tensor, n, layers)
    if cached is not None:
        return cached
    groups = syn.quant_encode(np.asarray(mf.read_checkpoint_tensor(path, cfg, tensor)), device)
    mf.write_quant_cache_parts(path, tensor, groups, n, layers)   # numbered parts when one file cannot hold it
    return groups


def main(argv=None) -> int:
    args = parse_args(sys.argv[1:] if argv is None else argv)
    if args["--mode"].upper() != "CUDA":
        raise SystemExit("only --mode CUDA exists in this implementation (no CPU path)")
    temperature, topp = float(args["--temp"]), float(args["--topp"])
    seed = int(args["--seed"]) if "--seed" in args else int(time.time())   # Run.java:542-545
    path = os.path.join(MODELS_DIRECTORY, args["--checkpoint"])
    cfg = mf.read_checkpoint_header(path)
    gpu_mem = parse_gpu_mem(args["--gpuMem"]) if args["--gpuMem"] else [180 * 1024 ** 3]
    alloc = LayerAllocation.from_gpu_mem(gpu_mem, cfg)
    t0 = time.time()
    stages = [Transformer(cfg, dev, alloc.first_layer[dev], alloc.last_layer[dev]) for dev in range(alloc.device_count)]
    for t in _lib.QUANT_TENSORS:
        groups = load_quant_tensor(path, cfg, t, 0)
        for st in stages:
            st.upload_quant(t, groups)
    emb = np.asarray(mf.read_checkpoint_tensor(path, cfg, _lib.T_TOKEN_EMBEDDING))
    for st in stages:
        st.upload_f32(_lib.T_TOKEN_EMBEDDING, emb)
    if not cfg.shared_classifier:
        stages[-1].upload_f32(_lib.T_WCLS, np.asarray(mf.read_checkpoint_tensor(path, cfg, _lib.T_WCLS)))
    for st in stages:
        st.finalize()
    print(f"INFO: Initialized transformer in {time.time() - t0:.2f} s")
    steps = int(args["--steps"])
    if steps <= 0 or steps > cfg.seq_len:
        steps = cfg.seq_len                                  # Run.java:599-602
    prompt = [int(t) for t in args["--promptTokens"].split(",") if t.strip()]
    if temperature != 0.0:
        stages[-1].sampler_seed(seed)                        # Run.java:620
    # several devices: the stages hand x over the peer links (l2j_pipeline_*), the host sees one forward per token;
    # without peer access between the devices the link is refused and x travels through the host array, as in the
    # reference (Run.java:368-413)
    linked = None
    if len(stages) > 1:
        try:
            linked = LinkedStages(stages)
        except _lib.L2jError as e:
            print(f"INFO: stages not linked ({e}); hand-over through the host")
    token, pos, start, out = 1, 0, 0.0, []
    if len(stages) == 1 and 1 < len(prompt) < steps and 1 not in prompt:
        # positions 0 .. len(prompt) - 1 (fed BOS, then the prompt) in one batched call instead of one decode step
        # per token (Run.java:623-637 takes the steps); their forced results are the prompt itself
        stages[0].prefill([1] + prompt[:-1], 0)
        out, token, pos, start = list(prompt), prompt[-1], len(prompt), time.time()
    while pos < steps:                                       # Run.java:623-685
        want = temperature == 0.0 and pos >= len(prompt)
        if linked is not None:
            logits, _ = linked.forward(token, pos, want)
        elif len(stages) > 1:
            x = None
            for st in stages[:-1]:
                x = st.forward_stage(token, pos, x)
            logits, _ = stages[-1].forward_stage(token, pos, x, want)
        else:
            logits, _ = stages[0].forward(token, pos, want)
        if pos < len(prompt):
            nxt = prompt[pos]                                # Run.java:635-637
        elif temperature == 0.0:
            nxt = argmax(logits)
        else:
            nxt = stages[-1].sample(temperature, topp)       # Run.java:643-665, on the device
        pos += 1
        if nxt == 1:
            break
        out.append(nxt)
        token = nxt
        if start == 0.0:
            start = time.time()
    end = time.time()
    print(" ".join(str(t) for t in out))
    if pos > 1:
        print(f"DEBUG: achieved tok/s: {(pos - 1) / max(end - start, 1e-9):.2f}")   # Run.java:703-706
    for st in stages:
        st.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
