"""Benchmark of the decode path: batch-1 greedy decode tok/s at the Llama-2-7B shape, W8A32.

One step = one pass over the workload of the headline configuration: BOS + 32 forced prompt tokens,
then greedy tokens up to 288 forwards in total.  Every forward is the same batch-1 decode pass (the
reference pushes prompt tokens through the decode path too, and its own tok/s counts them,
Run.java:682-706), so the metric is forwards per second.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--shape llama2-7b] [--impl reference]

N > 1 (launched by torch.distributed.run, one rank per GPU) runs N independent replicas, the way
the reference uses several GPUs for throughput (README.md:369-370): weak scaling, no collective on
the data path.  --impl reference times the CPU restatement of the reference's CPU mode on the host
cores (the reference is a Java program and no JVM is present).
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

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel (mean of the QKV, Wo, W1/W3 and
# W2 launches of a layer), from the ncu capture summarised in profiles/matvec_ring_u8_llama2-7b-4layer_full.md,
# taken with the cross-launch L2 prefetch switched off: ncu flushes the caches between kernels, so what a
# launch prefetches for the next one would be counted here and read again there.  None for other shapes.
NCU_TRAFFIC_BYTES = {"llama2-7b": 52351360}


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
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(args.shape), "sample_per_step": f"{sample} consecutive forwards",
                   "note": "the reference is Java (JDK 20 + JCuda) and cannot run without a JVM; this is the C restatement "
                           "of its CPU mode (Run.transformerCPU) on all host cores", "setup_s": round(setup_s, 1)},
        "cpu_baseline": {"value": value, "unit": "tok/s", "cores": cores, "kind": "port",
                         "sample": f"{args.steps} steps of {sample} consecutive forwards from position {args.warmup * sample}"},
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_long_context(args, cfg, model, rank, world, max_over_ranks, barrier) -> None:
    """Long-context attention stress: a 3840-token seeded prompt pushed through the decode path (the
    reference has no batched prefill), then greedy decode of positions 3840..seq_len-1.  The decode span is
    timed as the difference of two device-timed runs (to seq_len and to 3840 positions)."""
    from llama2j_b200 import synthetic as syn
    n_prompt = min(3840, cfg.seq_len - 2)
    prompt = syn.synthetic_prompt(n_prompt, 1, cfg.vocab_size)
    full, head = cfg.seq_len, n_prompt
    model.generate_greedy(prompt, full)                     # warm-up, fills the KV cache
    t_full, t_head = [], []
    for _ in range(max(1, args.steps)):
        barrier()
        model.generate_greedy(prompt, full)
        t_full.append(model.last_generate_us())
        model.generate_greedy(prompt, head)
        t_head.append(model.last_generate_us())
    span_us = max_over_ranks(float(np.median(t_full) - np.median(t_head)))
    n_dec = full - head
    pos_mid = head + n_dec // 2
    kt = model.time_kernels(pos_mid, reps=2)
    model.reset()
    peak, peak_kind = peak_hbm_gbs()
    attn_bytes = 2 * cfg.kv_dim * 4 * (pos_mid + 1)
    tok_bytes = float(np.mean([bytes_per_token(cfg, p)["total"] for p in range(head, full)]))
    value = world * n_dec / (span_us * 1e-6)
    line = {
        "metric": "batch-1 decode tok/s at positions %d-%d" % (head, full - 1), "value": value, "unit": "tok/s",
        "n_gpus": world, "steps": args.steps, "warmup": 1, "ms_per_step": span_us * 1e-3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32 activations x u8 group-quantised weights", "data": "synthetic",
        "config": {"workload": f"{args.shape}-shaped, KV cache prefilled by a {n_prompt}-token seeded prompt, greedy decode of "
                               f"positions {head}-{full - 1}", "parallelism": f"replicas x{world}"},
        "attention_kernel": {"pos": pos_mid, "us_per_layer": kt["attention"], "bytes_per_layer": attn_bytes,
                             "gbs": attn_bytes / (kt["attention"] * 1e3), "frac": attn_bytes / (kt["attention"] * 1e3) / peak},
        "roofline": {"bound": "hbm", "achieved": tok_bytes / (span_us / n_dec * 1e3), "peak": peak, "unit": "GB/s",
                     "frac": tok_bytes / (span_us / n_dec * 1e3) / peak, "peak_kind": f"of {peak_kind}", "traffic": None,
                     "bytes_per_token": tok_bytes},
        "gpu_launches": int(model.stats().kernels_per_forward) * (full + head) * max(1, args.steps),
    }
    if rank == 0:
        print(json.dumps(line), flush=True)


def workload_name(shape: str) -> str:
    return (f"{shape}-shaped W8A32 batch-1 decode: BOS + {PROMPT_LEN} forced prompt tokens + greedy to "
            f"{FORWARDS_PER_STEP} forwards per step; N(0,0.02) weights seed 0, prompt seed 1")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--shape", default="llama2-7b")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", default="decode", choices=["decode", "long"],
                    help="decode: the headline 288-forward workload; long: positions 3840-4095 after a 3840-token prompt")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    from llama2j_b200 import synthetic as syn
    cfg = syn.SHAPES[args.shape]
    forwards = min(FORWARDS_PER_STEP, cfg.seq_len)

    if args.impl == "reference":
        run_reference(args, cfg, rank, world)
        return

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the decode path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    from llama2j_b200.transformer import Transformer, run_greedy_host_loop
    tensors = syn.synthetic_tensors(cfg, 0, device=local_rank)
    model = Transformer(cfg, device=local_rank)
    model.upload_all(tensors)
    model.finalize()
    prompt = syn.synthetic_prompt(PROMPT_LEN, 1, cfg.vocab_size)
    mode = model.launch_mode()
    if not mode["ring"]:
        raise SystemExit("the sm_100a ring kernels are not active; refusing to time a fallback")

    if args.workload == "long":
        run_long_context(args, cfg, model, rank, world, max_over_ranks, barrier)
        model.close()
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- device-resident arm: inputs in HBM, the whole greedy loop queued on the device -----------
    for _ in range(args.warmup):
        tokens = model.generate_greedy(prompt, forwards)
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    wall0 = time.perf_counter()
    dev_us = 0.0
    for _ in range(args.steps):
        tokens = model.generate_greedy(prompt, forwards)
        dev_us += model.last_generate_us()
    barrier()
    wall = time.perf_counter() - wall0
    clocks = sampler.stop()
    dev_s = max_over_ranks(dev_us * 1e-6)
    wall = max_over_ranks(wall)
    stats = model.stats()
    value = world * args.steps * forwards / dev_s
    launches = int(stats.kernels_per_forward) * args.steps * forwards

    # ---- the same loop by the reference's two other accounts (outside the timed region) -------------
    # decode only: the sampled forwards after the prompt, by difference of two device-timed runs;
    # reference style: (positions - 1) / time from the end of the first iteration (Run.java:682-706).
    model.generate_greedy(prompt, PROMPT_LEN + 1)
    head_us = model.last_generate_us()
    model.generate_greedy(prompt, 1)
    first_us = model.last_generate_us()
    step_us = dev_us / args.steps
    decode_only = (forwards - PROMPT_LEN - 1) / ((step_us - head_us) * 1e-6) if step_us > head_us else None
    reference_style = (forwards - 1) / ((step_us - first_us) * 1e-6) if step_us > first_us else None

    # ---- end-to-end arm: the call the Java host makes, once per token, logits back to the host ----
    run_greedy_host_loop(model, prompt, min(forwards, 64), stop_on_bos=False)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        host_tokens, _ = run_greedy_host_loop(model, prompt, forwards, stop_on_bos=False)
    barrier()
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    e2e_value = world * args.steps * forwards / e2e_s
    tokens_agree = bool(np.array_equal(host_tokens, tokens))

    # ---- per-kernel times and the roofline of the dominant kernel --------------------------------
    peak, peak_kind = peak_hbm_gbs()
    mid_pos = (PROMPT_LEN + forwards) // 2
    kt = model.time_kernels(mid_pos, reps=3)
    model.reset()
    bpt = bytes_per_token(cfg, mid_pos)
    kernels = {k: {"us": kt[k], "bytes": bpt[k], "gbs": bpt[k] / (kt[k] * 1e3) if kt[k] > 0 else None} for k in kt}
    u8 = ("qkv_rope", "wo_residual", "w13_swiglu", "w2_residual")
    u8_bytes = sum(bpt[k] for k in u8) / len(u8)
    u8_us = sum(kt[k] for k in u8) / len(u8)
    achieved = u8_bytes / (u8_us * 1e3)
    mean_bytes = float(np.mean([bytes_per_token(cfg, p)["total"] for p in range(forwards)]))
    token_gbs = mean_bytes * args.steps * forwards / (dev_us * 1e-6) / 1e9
    roofline = {
        "bound": "hbm", "kernel": "matvec_ring_kernel<u8> (QKV, Wo, W1/W3, W2 launches of a layer, averaged)",
        "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_kind": f"of {peak_kind}",
        "traffic": NCU_TRAFFIC_BYTES.get(args.shape), "bytes_per_launch": u8_bytes, "us_per_launch": u8_us,
        "kernels": kernels,
        "token": {"bytes": mean_bytes, "gbs": token_gbs, "frac": token_gbs / peak},
    }

    line = {
        "metric": "batch-1 decode tok/s (forwards per second)", "value": value, "unit": "tok/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_s / args.steps * 1e3,
        "wall_ms_per_step": wall / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": value / (PUBLISHED_TOK_S * world), "dtype": "f32 activations x u8 group-quantised weights",
        "data": "synthetic",
        "config": {"workload": workload_name(args.shape), "parallelism": f"replicas x{world}",
                   "l2": "inputs larger than L2: %.1f GB of weights are streamed per forward" % (bytes_per_token(cfg, 0)["total"] / 1e9),
                   "baseline_note": "vs_baseline divides by the reference's published 20.9 tok/s per RTX 4090 (README.md:46)",
                   "launch": mode, "tokens_agree_host_vs_device_loop": tokens_agree},
        "clocks": clocks, "roofline": roofline,
        "e2e": {"value": e2e_value, "unit": "tok/s", "h2d_bytes_per_step": 16 * forwards,
                "d2h_bytes_per_step": (4 * cfg.vocab_size + 32) * forwards},
        "gpu_launches": launches,
        "accounts": {"all_forwards_tok_s": value / world, "decode_only_tok_s": decode_only,
                     "reference_style_tok_s": reference_style,
                     "note": "per GPU; decode only = the forwards after the forced prompt; reference style = "
                             "(positions - 1) / time from the end of the first iteration (Run.java:682-706)"},
    }
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        model.close()
        line["cpu_baseline"] = cpu_baseline_sample(cfg, tensors)
    else:
        model.close()
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
