"""Benchmark of the decode path: batch-1 greedy decode tok/s at the Llama-2-7B shape, W8A32.

One step = one pass over the workload of the headline configuration: BOS + 32 forced prompt tokens,
then greedy tokens up to 288 forwards in total.  Every forward is the same batch-1 decode pass (the
reference pushes prompt tokens through the decode path too, and its own tok/s counts them,
Run.java:682-706), so the metric is forwards per second.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--shape llama2-7b|llama2-13b] [--impl reference]

N = 1: one device, all layers of a token in one persistent launch.  N > 1 (launched by
torch.distributed.run, one rank per GPU): the ONE sequence is decoded by a tensor-parallel group over the
N devices, driven by rank 0 the way the reference drives several GPUs from one host thread
(Context.java:16-23); the other ranks hold their GPU and wait at the barriers.  The value is the
single-sequence tok/s (strong scaling); `accounts` adds the reference's own multi-GPU mode, the layer split
(Run.java:368-413), and the single device measured in the same run.  --impl reference times the CPU
restatement of the reference's CPU mode on the host cores (the reference is a Java program and no JVM is
present).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

PROMPT_LEN = 32
FORWARDS_PER_STEP = 288
PUBLISHED_TOK_S = 20.9      # llama2j --mode CUDA, Llama-2-7B-chat, one RTX 4090 (reference README.md:46,63)
FALLBACK_HBM_GBS = 6650.0

# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the persistent all-layers kernel, measured with
# ncu on the same shape with 4 layers (a full-metric capture of 32 layers would hold too much on the device)
# and scaled by the layer count: the traffic of a launch is the layers' weights, in proportion.  None for
# other shapes.
NCU_TRAFFIC_BYTES_PER_LAYER = {"llama2-7b": (835265280 + 23664640) // 4}


def bytes_per_token(cfg, pos: int) -> dict:
    """Algorithmic bytes of one forward at position pos, from the file formats: quantised matrices with
    their group headers, quantised RMSNorm weights, FP32 classifier, one embedding row, KV read for
    positions 0..pos, KV write, logits write."""
    def q(n):
        return -(-n // 256) * 264
    d, h, L, kv, v = cfg.dim, cfg.hidden_dim, cfg.n_layers, cfg.kv_dim, cfg.vocab_size
    per_layer = {
        "qkv_rope": q(d * d) + 2 * q(kv * d) + q(d) + 2 * kv * 4,
        "attention": 2 * kv * 4 * (pos + 1),
        "wo_residual": q(d * d),
        "w13_swiglu": 2 * q(h * d) + q(d),
        "w2_residual": q(d * h),
    }
    out = {k: val for k, val in per_layer.items()}
    out["classifier_argmax"] = 4 * v * d + q(d) + 4 * v
    out["total"] = L * sum(per_layer.values()) + out["classifier_argmax"] + 4 * d
    return out


def peak_hbm_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-i", str(self.gpu), "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        def reader():
            for line in self.proc.stdout:
                self.rows.append(line.strip())
        self.thread = threading.Thread(target=reader, daemon=True)
        self.thread.start()

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, power, reasons = [], [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for row in self.rows:
            parts = [p.strip() for p in row.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
                power.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def cpu_baseline_sample(cfg, tensors, budget_s: float = 15.0, max_forwards: int = 8) -> dict:
    """Times the CPU checker (restatement of the reference's CPU mode) on the host cores for a bounded
    sample: the first forwards of the workload."""
    from oracle import cpu_oracle
    om = cpu_oracle.OracleModel(cfg, tensors, cpu_oracle.SILU_LOOKUP, cpu_oracle.SOFTMAX_REFERENCE)
    prompt = [1] + list(range(3, 3 + max_forwards))
    om.forward(prompt[0], 0)   # touch the weights once (page-in), untimed
    n, t0 = 0, time.perf_counter()
    while n < max_forwards and (time.perf_counter() - t0 < budget_s or n == 0):
        om.forward(prompt[n], n)
        n += 1
    dt = time.perf_counter() - t0
    om.close()
    return {"value": n / dt, "unit": "tok/s", "cores": cpu_oracle.load().l2jo_num_threads(), "kind": "port",
            "sample": f"{n} forwards at positions 0..{n - 1} of the same checkpoint, CPU-faithful arithmetic (lookup SiLU)"}


def run_reference(args, cfg, rank: int, world: int) -> None:
    if rank != 0:
        return
    from oracle import cpu_oracle
    # a launcher may pin OMP_NUM_THREADS=1 for its ranks: the CPU arm uses every host core, said in `cores`
    cpu_oracle.load().l2jo_set_num_threads(os.cpu_count() or 1)
    t_setup = time.perf_counter()
    tensors = cpu_oracle.synthetic_tensors(cfg, 0)
    om = cpu_oracle.OracleModel(cfg, tensors, cpu_oracle.SILU_LOOKUP, cpu_oracle.SOFTMAX_REFERENCE)
    setup_s = time.perf_counter() - t_setup
    from llama2j_b200.synthetic import synthetic_prompt
    prompt = [1] + [int(t) for t in synthetic_prompt(PROMPT_LEN, 1, cfg.vocab_size)]
    # one step = a bounded sample of the workload: the next `sample` positions of the same sequence
    sample = 2 if cfg.dim >= 2048 else 16
    pos = 0
    token = prompt[0]

    def step():
        nonlocal pos, token
        for _ in range(sample):
            lg = om.forward(token, pos % cfg.seq_len)
            pos += 1
            token = prompt[pos] if pos < len(prompt) else cpu_oracle.argmax(lg)
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    value = args.steps * sample / dt
    cores = cpu_oracle.load().l2jo_num_threads()
    line = {
        "impl": "reference", "metric": "batch-1 decode tok/s (forwards per second)", "value": value, "unit": "tok/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak" if args.gpus == 1 else "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": workload_name(args.shape), "sample_per_step": f"{sample} consecutive forwards",
                   "note": "the reference is Java (JDK 20 + JCuda) and cannot run without a JVM; this is the C restatement "
                           "of its CPU mode (Run.transformerCPU) on all host cores", "setup_s": round(setup_s, 1)},
        "cpu_baseline": {"value": value, "unit": "tok/s", "cores": cores, "kind": "port",
                         "sample": f"{args.steps} steps of {sample} consecutive forwards from position {args.warmup * sample}"},
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_name(shape: str) -> str:
    return (f"{shape}-shaped W8A32 batch-1 decode: BOS + {PROMPT_LEN} forced prompt tokens + greedy to "
            f"{FORWARDS_PER_STEP} forwards per step; N(0,0.02) weights seed 0, prompt seed 1")


PHASES = ("qkv_rope", "attention", "wo_residual", "w13_swiglu", "w2_residual")


def in_situ_split(cfg, tensors, device: int, prompt, pos: int) -> dict:
    """Per-phase times of the persistent kernel inside a real forward at position `pos`, from the kernel's own
    timeline (global-timer marks written by one thread per block): a second context of the same checkpoint is
    created with the timeline switched on, decodes up to `pos`, and the last launch is read back.  A phase
    lasts from the moment the last block reported the phase in front to the moment the last block reports
    this one; `stall` is the part of it before the median block has its input vector ready (hand-over,
    load, RMSNorm, fixed-point conversion), `tail` the part after the median block's last stage."""
    from llama2j_b200.transformer import Transformer
    os.environ["L2J_TRACE"] = "1"
    try:
        m = Transformer(cfg, device=device)
    finally:
        del os.environ["L2J_TRACE"]
    m.upload_all(tensors)
    m.finalize()
    if not m.launch_mode().get("persistent"):
        m.close()
        return {}
    m.generate_greedy(prompt, pos + 1)
    nb, L = m.launch_mode()["ring_blocks"], cfg.n_layers
    t = m.read_trace().reshape(-1)[: nb * 5 * L * 8].reshape(nb, 5 * L, 8).astype(np.int64)
    m.close()
    out = {"pos": pos, "us_per_layer": float((t[:, 5 * L - 1, 3].max() - t[:, 4, 3].max()) / 1e3 / (L - 1))}
    bpt = bytes_per_token(cfg, pos)
    for ph, name in enumerate(PHASES):
        total, stall, tail = [], [], []
        for l in range(1, L):
            i = 5 * l + ph
            act = t[:, i, 0] > 0
            if not act.any():
                continue
            prev_done, done = t[:, i - 1, 3].max(), t[:, i, 3].max()
            total.append(done - prev_done)
            ready = np.median(t[act, i, 1]) if ph != 1 else np.median(t[act, i, 0])
            stall.append(ready - prev_done)
            tail.append(done - np.median(t[act, i, 2]))
        us = float(np.mean(total)) / 1e3
        out[name] = {"us": us, "stall_us": float(np.mean(stall)) / 1e3, "tail_us": float(np.mean(tail)) / 1e3,
                     "bytes": bpt[name], "gbs": bpt[name] / (us * 1e3)}
    return out


def long_context_account(cfg, model, tensors, device: int, peak: float) -> dict:
    """Positions 3840..seq_len-1 after a 3840-token seeded prompt pushed through the decode path (the reference has no
    batched prefill): tok/s over that span as the difference of two device-timed runs, and the attention phase of
    the persistent kernel at the middle position from its own timeline."""
    from llama2j_b200 import synthetic as syn
    n_prompt = min(3840, cfg.seq_len - 2)
    prompt = syn.synthetic_prompt(n_prompt, 1, cfg.vocab_size)
    full = cfg.seq_len
    model.generate_greedy(prompt, full)                     # warm-up, fills the KV cache
    model.generate_greedy(prompt, full)
    t_full = model.last_generate_us()
    model.generate_greedy(prompt, n_prompt)
    t_head = model.last_generate_us()
    n_dec = full - n_prompt
    span_us = t_full - t_head
    pos_mid = n_prompt + n_dec // 2
    tok_bytes = float(np.mean([bytes_per_token(cfg, p)["total"] for p in range(n_prompt, full)]))
    out = {"positions": [n_prompt, full - 1], "tok_s": n_dec / (span_us * 1e-6), "us_per_token": span_us / n_dec,
           "token_gbs": tok_bytes / (span_us / n_dec * 1e3), "token_frac": tok_bytes / (span_us / n_dec * 1e3) / peak}
    split = in_situ_split(cfg, tensors, device, prompt, pos_mid)
    if split:
        a = split["attention"]
        out["attention"] = {"pos": pos_mid, "us_per_layer": a["us"], "bytes_per_layer": a["bytes"], "gbs": a["gbs"],
                            "frac": a["gbs"] / peak, "where": "attention phase of the persistent kernel, in situ"}
        out["us_per_layer"] = split["us_per_layer"]
    # the same prompt through l2j_prefill (64 positions per weight sweep on the tensor cores) beside the decode path
    inputs = np.concatenate([[1], prompt[:n_prompt - 1]]).astype(np.int32)   # BOS, then the prompt: what each position is fed
    model.prefill(inputs, 0)
    import torch
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    model.prefill(inputs, 0)
    pf_s = time.perf_counter() - t0
    out["prefill"] = {"tokens": int(n_prompt), "batched_s": pf_s, "batched_tok_s": n_prompt / pf_s,
                      "decode_path_s": t_head * 1e-6, "speedup": t_head * 1e-6 / pf_s,
                      "tensor_core_path": model.prefill_launches() > 0,
                      "timing": "host wall clock around one blocking l2j_prefill call, tokens copied from host memory"}
    return out


def concurrent_account(cfg, model, single_tok_s: float) -> dict:
    """64 sequences decoded together (l2j_batch_forward): one sweep over the weights per step for all of them.
    Greedy from BOS, every sequence fed its own arg-max; host wall clock per blocking step (ids in, ids out)."""
    n_seq, seq_len, steps, skip = 64, 256, 72, 8
    model.batch_create(n_seq, seq_len)
    toks = np.ones(n_seq, dtype=np.int32)
    seq = np.arange(n_seq, dtype=np.int32)
    times = []
    for p in range(steps):
        t0 = time.perf_counter()
        _, toks = model.batch_forward(seq, np.full(n_seq, p, dtype=np.int32), toks, want_logits=False)
        times.append(time.perf_counter() - t0)
    per = float(np.mean(times[skip:]))
    return {"sequences": n_seq, "positions": [skip, steps - 1], "ms_per_step": per * 1e3, "aggregate_tok_s": n_seq / per,
            "vs_one_sequence": n_seq / per / single_tok_s,
            "note": "each step reads every weight once for 64 sequences; attention and K/V traffic grow with the positions"}


def host_loop(model, prompt, forwards: int) -> np.ndarray:
    """The run loop of Run.java:609-685 with --temp 0.0 as a host makes it through the C ABI: one blocking
    l2j_forward per token, the token from pinned host memory to the device, the 128 KB of logits back into a host
    buffer, the next token = forced prompt token or the first maximum (the call returns the device's arg-max of
    the same logits; the parity tests check that it is the host's)."""
    prompt = [int(t) for t in prompt]
    token, out = 1, np.empty(forwards, dtype=np.int32)
    for pos in range(forwards):
        _, am = model.forward(token, pos)
        token = prompt[pos] if pos < len(prompt) else am
        out[pos] = token
    return out


def run_single(args, cfg, local_rank: int) -> dict:
    from llama2j_b200 import synthetic as syn
    from llama2j_b200.transformer import Transformer, run_greedy_host_loop
    import torch
    forwards = min(FORWARDS_PER_STEP, cfg.seq_len)
    tensors = syn.synthetic_tensors(cfg, 0, device=local_rank)
    t_load = time.perf_counter()
    model = Transformer(cfg, device=local_rank)
    model.upload_all(tensors)
    model.finalize()
    load_s = time.perf_counter() - t_load
    prompt = syn.synthetic_prompt(PROMPT_LEN, 1, cfg.vocab_size)
    mode = model.launch_mode()
    if not mode["ring"]:
        raise SystemExit("the sm_100a ring kernels are not active; refusing to time a fallback")

    # ---- device-resident arm: inputs in HBM, the whole greedy loop queued on the device -----------
    for _ in range(args.warmup):
        tokens = model.generate_greedy(prompt, forwards)
    sampler = ClockSampler(local_rank)
    torch.cuda.synchronize()
    sampler.start()
    wall0 = time.perf_counter()
    dev_us = 0.0
    for _ in range(args.steps):
        tokens = model.generate_greedy(prompt, forwards)
        dev_us += model.last_generate_us()
    torch.cuda.synchronize()
    wall = time.perf_counter() - wall0
    clocks = sampler.stop()
    stats = model.stats()
    value = args.steps * forwards / (dev_us * 1e-6)
    launches = int(stats.kernels_per_forward) * args.steps * forwards

    # ---- the same loop by the reference's two other accounts (outside the timed region) -------------
    model.generate_greedy(prompt, PROMPT_LEN + 1)
    head_us = model.last_generate_us()
    model.generate_greedy(prompt, 1)
    first_us = model.last_generate_us()
    step_us = dev_us / args.steps
    decode_only = (forwards - PROMPT_LEN - 1) / ((step_us - head_us) * 1e-6) if step_us > head_us else None
    reference_style = (forwards - 1) / ((step_us - first_us) * 1e-6) if step_us > first_us else None

    # ---- end-to-end arm: the call the Java host makes, once per token, logits back to the host ----
    host_loop(model, prompt, min(forwards, 64))
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        host_tokens = host_loop(model, prompt, forwards)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    e2e_value = args.steps * forwards / e2e_s
    tokens_agree = bool(np.array_equal(host_tokens, tokens))

    # ---- the dominant kernel against the HBM roofline ---------------------------------------------
    peak, peak_kind = peak_hbm_gbs()
    mid_pos = (PROMPT_LEN + forwards) // 2
    bpt = bytes_per_token(cfg, mid_pos)
    layer_bytes = sum(bpt[k] for k in PHASES)
    mean_bytes = float(np.mean([bytes_per_token(cfg, p)["total"] for p in range(forwards)]))
    token_gbs = mean_bytes * args.steps * forwards / (dev_us * 1e-6) / 1e9
    if mode.get("persistent"):
        us_launch = model.time_layers_kernel(mid_pos, reps=5)
        model.reset()
        launch_bytes = cfg.n_layers * layer_bytes
        traffic = NCU_TRAFFIC_BYTES_PER_LAYER.get(args.shape)
        roofline = {
            "bound": "hbm", "kernel": "fused_layers_kernel (all layers of a token in one persistent launch)",
            "achieved": launch_bytes / (us_launch * 1e3), "peak": peak, "unit": "GB/s",
            "frac": launch_bytes / (us_launch * 1e3) / peak, "peak_kind": f"of {peak_kind}",
            "traffic": traffic * cfg.n_layers if traffic else None,
            "traffic_note": "ncu capture of the same kernel at 4 layers, scaled by the layer count",
            "bytes_per_launch": launch_bytes, "us_per_launch": us_launch, "pos": mid_pos,
        }
    else:
        kt = model.time_kernels(mid_pos, reps=3)
        model.reset()
        u8 = ("qkv_rope", "wo_residual", "w13_swiglu", "w2_residual")
        u8_bytes = sum(bpt[k] for k in u8) / len(u8)
        u8_us = sum(kt[k] for k in u8) / len(u8)
        roofline = {"bound": "hbm", "kernel": "matvec_ring_kernel<u8> (QKV, Wo, W1/W3, W2 launches of a layer, averaged)",
                    "achieved": u8_bytes / (u8_us * 1e3), "peak": peak, "unit": "GB/s", "frac": u8_bytes / (u8_us * 1e3) / peak,
                    "peak_kind": f"of {peak_kind}", "traffic": None, "bytes_per_launch": u8_bytes, "us_per_launch": u8_us}
    roofline["token"] = {"bytes": mean_bytes, "gbs": token_gbs, "frac": token_gbs / peak}
    accounts = {"all_forwards_tok_s": value, "decode_only_tok_s": decode_only, "reference_style_tok_s": reference_style,
                "note": "decode only = the forwards after the forced prompt; reference style = (positions - 1) / time "
                        "from the end of the first iteration (Run.java:682-706)"}
    if not args.quick:
        roofline["in_situ"] = in_situ_split(cfg, tensors, local_rank, prompt, mid_pos)
        if cfg.seq_len >= 4096:
            accounts["long_context"] = long_context_account(cfg, model, tensors, local_rank, peak)
            model.reset()
        if model.prefill_launches() > 0:
            accounts["concurrent_sequences"] = concurrent_account(cfg, model, value)
        # loading (TransformerWeights.java:191-232 quantises on first use and caches; the reference publishes 15.3 s for
        # the first load and 0.8 s from the cache at 7B): no checkpoint file exists here, so the two device-side parts
        # are timed on arrays in host memory -- context creation + upload of the quantised tensors + finalize, and the
        # device quantiser (FP32 in, groups out, both through host memory) on one W1 matrix, scaled to all matrices
        sample = np.asarray(syn.synth_f32(cfg.hidden_dim * cfg.dim, 0, 99, local_rank), dtype=np.float32)
        syn.quant_encode(sample[:1 << 20], local_rank)
        t0 = time.perf_counter()
        syn.quant_encode(sample, local_rank)
        q_s = time.perf_counter() - t0
        from llama2j_b200 import lib as _l2j
        n_mat = sum(cfg.tensor_floats(t) for t in _l2j.QUANT_TENSORS)
        accounts["load"] = {"upload_quantised_s": load_s, "device_quantiser_floats_per_s": sample.size / q_s,
                            "quantise_all_matrices_s": n_mat / (sample.size / q_s),
                            "note": "host arrays in memory, no file I/O: create + upload + finalize of the quantised model; "
                                    "first-load analogue = quantise_all_matrices_s + upload_quantised_s"}

    line = {
        "metric": "batch-1 decode tok/s (forwards per second)", "value": value, "unit": "tok/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_us * 1e-3 / args.steps,
        "wall_ms_per_step": wall / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": value / PUBLISHED_TOK_S, "dtype": "f32 activations x u8 group-quantised weights",
        "data": "synthetic",
        "config": {"workload": workload_name(args.shape), "parallelism": "one device",
                   "l2": "inputs larger than L2: %.1f GB of weights are streamed per forward" % (bytes_per_token(cfg, 0)["total"] / 1e9),
                   "baseline_note": "vs_baseline divides by the reference's published 20.9 tok/s per RTX 4090 (README.md:46)",
                   "launch": mode, "tokens_agree_host_vs_device_loop": tokens_agree},
        "clocks": clocks, "roofline": roofline,
        "e2e": {"value": e2e_value, "unit": "tok/s", "h2d_bytes_per_step": 16 * forwards,
                "d2h_bytes_per_step": (4 * cfg.vocab_size + 32) * forwards},
        "gpu_launches": launches, "accounts": accounts,
    }
    model.close()
    if not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline_sample(cfg, tensors)
    return line


def run_group(args, cfg, world: int) -> dict:
    """Rank 0's part at N > 1: one sequence over a tensor-parallel group of the N devices."""
    from llama2j_b200 import synthetic as syn
    from llama2j_b200.layer_allocation import LayerAllocation
    from llama2j_b200.transformer import LinkedStages, TensorParallel, Transformer, run_greedy_host_loop
    forwards = min(FORWARDS_PER_STEP, cfg.seq_len)
    tensors = syn.synthetic_tensors(cfg, 0, device=0)
    prompt = syn.synthetic_prompt(PROMPT_LEN, 1, cfg.vocab_size)
    devices = list(range(world))

    def device_rate(model, repeats=3):
        model.generate_greedy(prompt, forwards)
        us = []
        for _ in range(repeats):
            toks = model.generate_greedy(prompt, forwards)
            us.append(model.last_generate_us())
        return toks, forwards / (float(np.median(us)) * 1e-6)

    # one device, the same checkpoint: the logits the group has to reproduce bit for bit, and its tok/s
    check_positions = 12
    with Transformer(cfg, device=0) as whole:
        whole.upload_all(tensors)
        whole.finalize()
        ref_tokens, ref_logits = run_greedy_host_loop(whole, prompt, check_positions, stop_on_bos=False)
        single_tokens, single_tok_s = device_rate(whole)
        single_mode = whole.launch_mode()
    with Transformer(cfg, device=0, flags=0x8) as steps_ctx:    # the per-step kernels the group is built from
        steps_ctx.upload_all(tensors)
        steps_ctx.finalize()
        step_tokens, step_logits = run_greedy_host_loop(steps_ctx, prompt, check_positions, stop_on_bos=False)

    group = TensorParallel.from_devices(cfg, tensors, devices)
    tp_tokens, tp_logits = run_greedy_host_loop(group, prompt, check_positions, stop_on_bos=False)
    bitwise = bool(np.array_equal(tp_logits.view(np.uint32), step_logits.view(np.uint32)))
    span = float(ref_logits.max() - ref_logits.min())
    close = float(np.abs(tp_logits - ref_logits).max()) / span

    for _ in range(args.warmup):
        tokens = group.generate_greedy(prompt, forwards)
    sampler = ClockSampler(0)
    sampler.start()
    wall0 = time.perf_counter()
    dev_us = 0.0
    for _ in range(args.steps):
        tokens = group.generate_greedy(prompt, forwards)
        dev_us += group.last_generate_us()
    wall = time.perf_counter() - wall0
    clocks = sampler.stop()
    value = args.steps * forwards / (dev_us * 1e-6)
    kpf = int(group.ranks[0].stats().kernels_per_forward)

    host_loop(group, prompt, min(forwards, 64))
    t0 = time.perf_counter()
    for _ in range(args.steps):
        host_tokens = host_loop(group, prompt, forwards)
    e2e_value = args.steps * forwards / (time.perf_counter() - t0)
    group.close()

    alloc = LayerAllocation.equal_split(world, cfg)
    split = LinkedStages.from_allocation(cfg, alloc.first_layer, alloc.last_layer, tensors, devices)
    split_tokens, split_tok_s = device_rate(split)
    split_logits = run_greedy_host_loop(split, prompt, check_positions, stop_on_bos=False)[1]
    split.close()

    peak, peak_kind = peak_hbm_gbs()
    mean_bytes = float(np.mean([bytes_per_token(cfg, p)["total"] for p in range(forwards)]))
    token_gbs = mean_bytes * value / 1e9
    return {
        "metric": "batch-1 decode tok/s (forwards per second)", "value": value, "unit": "tok/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_us * 1e-3 / args.steps,
        "wall_ms_per_step": wall / args.steps * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": value / PUBLISHED_TOK_S, "dtype": "f32 activations x u8 group-quantised weights", "data": "synthetic",
        "config": {"workload": workload_name(args.shape), "parallelism": f"tensor-parallel x{world}",
                   "driver": "rank 0 drives all devices of the group from one host thread; the other ranks hold their GPU",
                   "l2": "inputs larger than L2: %.1f GB of weights are streamed per forward" % (bytes_per_token(cfg, 0)["total"] / 1e9),
                   "logits_bitwise_equal_to_one_device_per_step_kernels": bitwise,
                   "logits_vs_one_device_persistent_kernel_of_range": close,
                   "tokens_equal_one_device": bool(np.array_equal(tokens, single_tokens)),
                   "tokens_agree_host_vs_device_loop": bool(np.array_equal(host_tokens, tokens)),
                   "checked_positions": check_positions, "one_device_launch": single_mode},
        "clocks": clocks,
        "roofline": {"bound": "hbm", "kernel": "whole token over the group (matvec_ring_kernel<u8> per rank, rows split)",
                     "achieved": token_gbs, "peak": peak * world, "unit": "GB/s", "frac": token_gbs / (peak * world),
                     "peak_kind": f"of {peak_kind} x {world} devices", "traffic": None,
                     "token": {"bytes": mean_bytes, "gbs": token_gbs, "frac": token_gbs / (peak * world)}},
        "e2e": {"value": e2e_value, "unit": "tok/s", "h2d_bytes_per_step": 16 * forwards * world,
                "d2h_bytes_per_step": (4 * cfg.vocab_size + 32 * world) * forwards},
        "gpu_launches": kpf * world * args.steps * forwards,
        "accounts": {"tensor_parallel_tok_s": value, "one_device_tok_s": single_tok_s, "layer_split_tok_s": split_tok_s,
                     "layer_split_first_last": [list(alloc.first_layer), list(alloc.last_layer)],
                     "layer_split_tokens_equal_one_device": bool(np.array_equal(split_tokens, single_tokens)),
                     "layer_split_logits_vs_one_device_of_range":
                         float(np.abs(split_logits - ref_logits).max()) / span,
                     "note": "one sequence in every account; the layer split is the reference's multi-GPU mode "
                             "(Run.java:368-413, stages run one after the other at batch 1)"},
    }


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--shape", default="llama2-7b")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--quick", action="store_true", help="skip the in-kernel timeline and the long-context account")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    from llama2j_b200 import synthetic as syn
    cfg = syn.SHAPES[args.shape]

    if args.impl == "reference":
        run_reference(args, cfg, rank, world)
        return

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the decode path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world == 1:
        print(json.dumps(run_single(args, cfg, local_rank)), flush=True)
        return

    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    # The ranks that hold a GPU for rank 0 wait on the host: a NCCL barrier would park a kernel on their SMs
    # while the group's kernels want all of them.
    host = dist.new_group(backend="gloo")

    def barrier():
        dist.barrier(group=host)
        torch.cuda.synchronize(local_rank)

    barrier()
    line = run_group(args, cfg, world) if rank == 0 else None
    barrier()
    # device time of the timed steps, maximum over the ranks (only rank 0 ran kernels of the group)
    torch.cuda.set_device(local_rank)   # the group's calls moved rank 0's current device around
    t = torch.tensor([line["ms_per_step"] if line else 0.0], dtype=torch.float64, device=torch.device("cuda", local_rank))
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        line["ms_per_step"] = float(t.item())
        print(json.dumps(line), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
