#!/usr/bin/env python
"""Benchmark of the GPT-2 decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload: GPT-2 medium (24 layers, d_model 1024, 16 heads, d_ff 4096, vocab 50257), FP32
random-init N(0, 0.02) weights (seed 0), 64 independent sequences per GPU with 128-token seeded
uniform prompts, greedy decode. A step is one batched decode step: every sequence of the rank
advances by one token. Weights and KV cache (> 1.4 GB per step) are far larger than L2, so no
explicit L2 flush is needed between steps. For N > 1 (launched by torchrun, one rank per GPU)
every rank holds a full weight replica and its own 64 sequences; there is no collective on the
token path (weak scaling).

One JSON line is printed by rank 0; see the keys `value`, `e2e`, `roofline`, `cpu_baseline`.
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
sys.path.insert(0, ROOT)

METRIC = "gpt2_decode_tokens_per_sec"
UNIT = "tokens/s"
MODEL = "medium"
SEQS_PER_GPU = 64
PROMPT_LEN = 128
WEIGHT_SEED = 0


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device: int):
        self.device, self.proc, self.lines = device, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.device)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower() == "active":
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def make_prompts(cfg, rank):
    from puppygrad_b200 import synthetic
    base = rank * SEQS_PER_GPU
    return [synthetic.uniform_prompt(base + i + 1, PROMPT_LEN, cfg["vocab_size"]) for i in range(SEQS_PER_GPU)]


def kv_bytes_per_step(cfg, lens):
    # each sequence reads K and V of all cached positions (plus the new one) in every layer, and
    # writes one K row and one V row per layer
    c, L = cfg["n_embd"], cfg["n_layer"]
    return sum(2 * L * (t + 1) * c * 4 + 2 * L * c * 4 for t in lens)


# ---------------------------------------------------------------------------------------------
def cpu_baseline_sample(cfg, weights, tokens: int, prompt_len: int, threads: int):
    """Times the CPU oracle (the port of the reference path) on one sequence of the workload:
    prefill `prompt_len` tokens untimed, then `tokens` greedy decode steps timed."""
    from oracle import oracle
    from puppygrad_b200 import synthetic
    model = oracle.Model(cfg, weights, threads=threads)
    cache = model.new_kv_cache()
    prompt = synthetic.uniform_prompt(1, prompt_len, cfg["vocab_size"])
    logits = model.prefill(prompt, cache)
    t0 = time.perf_counter()
    for _ in range(tokens):
        logits = model.forward_one(oracle.argmax_logits(logits), cache)
    dt = time.perf_counter() - t0
    return tokens / dt, dt


def run_reference(args):
    """The reference's CPU implementation of the path (its C++ port: the reference is Rust and no
    Rust toolchain exists on these machines), all host threads, one sequence at a time as the
    reference serves them. A step is one decode token of one sequence of the workload."""
    rank, world, local = dist_env()
    if rank != 0:
        return
    from oracle import oracle
    from puppygrad_b200 import synthetic
    cfg = synthetic.preset(MODEL)
    weights = synthetic.random_init_weights(cfg, WEIGHT_SEED)
    threads = os.cpu_count() or 1
    model = oracle.Model(cfg, weights, threads=threads)
    cache = model.new_kv_cache()
    # a short prompt keeps the untimed prefill bounded; decode cost is dominated by the weights
    prompt = synthetic.uniform_prompt(1, PROMPT_LEN, cfg["vocab_size"])[:16]
    logits = model.prefill(prompt, cache)
    for _ in range(args.warmup):
        logits = model.forward_one(oracle.argmax_logits(logits), cache)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        if cache.seq_len >= cfg["n_positions"]:
            cache.clear()
            logits = model.prefill(prompt, cache)
        logits = model.forward_one(oracle.argmax_logits(logits), cache)
    dt = time.perf_counter() - t0
    value = args.steps / dt
    sample = (f"1 sequence, {args.steps} greedy decode tokens after a 16-token prompt, {threads} threads, "
              "C++ port of the reference CPU path")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"gpt2-{MODEL} fp32 greedy decode, one sequence at a time on host cores"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0}))


def small_batch1(pg, synthetic, device):
    """GPT-2 small, one sequence, 32-token prompt, 64 greedy tokens: the latency-bound case."""
    cfg = synthetic.preset("small")
    model = pg.Gpt2Model(cfg, synthetic.random_init_weights(cfg, 0), pg.Gpt2CudaConfig(device=device))
    cache = model.new_kv_cache()
    prompt = synthetic.uniform_prompt(1, 32, cfg["vocab_size"])
    best = None
    for _ in range(3):
        _, first = model.prefill_batch([prompt], cache)
        first = model.decode_greedy(first, cache, 4)[-1]
        cache.time_begin()
        model.decode_greedy(first, cache, 60)
        sec = cache.time_end()
        best = sec if best is None else min(best, sec)
    _, cur = model.prefill_batch([prompt], cache)
    t0 = time.perf_counter()
    for _ in range(60):
        _, cur, _, _ = model.forward_one_batch(cur, cache)
    e2e = time.perf_counter() - t0
    peak, _ = measured_peaks()
    step_bytes = model.weight_bytes_per_step() + kv_bytes_per_step(cfg, [66])
    us = best / 60 * 1e6
    return {"tokens_per_s": 60 / best, "us_per_token": us, "e2e_tokens_per_s": 60 / e2e,
            "bytes_per_token": step_bytes, "hbm_frac": step_bytes / (best / 60) / 1e9 / peak}


def xl_sampling(pg, synthetic, device, seqs=32, prompt_len=512, steps=48):
    """GPT-2 XL with temperature 0.8 / top-k 40 sampling and one RNG seed per sequence (the
    256-sequence sampling workload, one GPU's share of it: 256 sequences over 8 GPUs = 32 per GPU,
    512-token prompts).
    Every step runs the persistent step kernel, the device top-k, and the host draw of the reference
    sampler; timed on the host clock through the public API (token ids in, top-k rows out)."""
    from puppygrad_b200.generation import LogitsSampler
    cfg = synthetic.preset("xl")
    model = pg.Gpt2Model(cfg, synthetic.random_init_weights(cfg, 0), pg.Gpt2CudaConfig(device=device, math_mode="tf32x3"))
    cache = model.new_kv_cache(max_batch=seqs)
    prompts = [synthetic.uniform_prompt(5000 + i, prompt_len, cfg["vocab_size"]) for i in range(seqs)]
    conf = pg.TextGenerationConfig(steps, temperature=0.8, top_k=40, seed=1234)
    samplers = [LogitsSampler(conf.seed + i) for i in range(seqs)]
    t0 = time.perf_counter()
    _, cur = model.prefill_batch(prompts, cache)
    prefill_s = time.perf_counter() - t0
    _, _, tv, ti = model.forward_one_batch(cur, cache, top_k=40)  # warm-up step: graph capture
    launches0 = cache.kernel_launches()
    t0 = time.perf_counter()
    for _ in range(steps):
        nxt = [samplers[i].select_from_topk(tv[i], ti[i], conf) for i in range(seqs)]
        _, _, tv, ti = model.forward_one_batch(nxt, cache, top_k=40)
    sec = time.perf_counter() - t0
    return {"tokens_per_s": seqs * steps / sec, "ms_per_step": sec / steps * 1e3, "seqs": seqs, "prompt_len": prompt_len,
            "steps": steps, "prefill_s": prefill_s, "kernel_launches_per_step": (cache.kernel_launches() - launches0) / steps,
            "bytes_per_step": model.weight_bytes_per_step() + kv_bytes_per_step(cfg, [prompt_len + steps // 2] * seqs)}


def prefill_small(pg, synthetic, device):
    """GPT-2 small prefill, 8 prompts of 1024 tokens (the prefill-only workload): FP32 FMA path and the
    single-pass TF32 tensor-core path. flops = linear GEMMs only (2*B*T*L*12*C^2), over the whole
    prefill time (attention, LayerNorm and the KV scatter included), so the rate is a lower bound."""
    cfg = synthetic.preset("small")
    weights = synthetic.random_init_weights(cfg, 0)
    prompts = [synthetic.uniform_prompt(s + 1, 1024, cfg["vocab_size"]) for s in range(8)]
    flops = 2 * 8 * 1024 * cfg["n_layer"] * 12 * cfg["n_embd"] ** 2
    out = {}
    for mode in ("fp32", "tf32"):
        model = pg.Gpt2Model(cfg, weights, pg.Gpt2CudaConfig(device=device, math_mode=mode))
        cache = model.new_kv_cache(max_batch=8)
        model.prefill_batch(prompts, cache)
        best = None
        for _ in range(3):
            cache.time_begin()
            model.prefill_batch(prompts, cache)
            sec = cache.time_end()
            best = sec if best is None else min(best, sec)
        out[mode] = {"ms": best * 1e3, "prompt_tokens_per_s": 8 * 1024 / best, "linear_tflops": flops / best / 1e12}
        del cache, model
    return out


# ---------------------------------------------------------------------------------------------
def run_ours(args):
    rank, world, local = dist_env()
    import torch
    import torch.distributed as dist

    import puppygrad_b200 as pg
    from puppygrad_b200 import sharding, synthetic

    if world > 1:
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    cfg = synthetic.preset(MODEL)
    weights = synthetic.random_init_weights(cfg, WEIGHT_SEED)
    model = pg.Gpt2Model(cfg, weights, pg.Gpt2CudaConfig(device=local, math_mode=args.math))
    cache = model.new_kv_cache(max_batch=args.seqs)
    prompts = make_prompts(cfg, rank)[:args.seqs]
    B, K, W = args.seqs, args.steps, args.warmup
    if PROMPT_LEN + W + K + 1 > cfg["n_positions"]:
        raise SystemExit("steps + warmup exceed the context window")

    # ---- device-resident throughput: tokens fed back on the device, timed with CUDA events on
    # the library's stream
    _, first = model.prefill_batch(prompts, cache)
    if W:
        warm = model.decode_greedy(first, cache, W)
        first = warm[-1]
    clocks = ClockSampler(local)
    launches0 = cache.kernel_launches()
    barrier()
    clocks.start()
    cache.time_begin()
    toks = model.decode_greedy(first, cache, K)
    sec = cache.time_end()
    barrier()
    clock_info = clocks.stop()
    launches = cache.kernel_launches() - launches0
    lens_mid = [PROMPT_LEN + W + K // 2] * B

    sec_max = sharding.max_over_ranks(sec, device=f"cuda:{local}")
    value = world * B * K / sec_max
    if args.skip_extras:  # profiling runs: only the timed decode loop
        if rank == 0:
            print(json.dumps({"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K,
                              "warmup": W, "ms_per_step": sec_max / K * 1e3, "seqs_per_gpu": B,
                              "gpu_launches": int(launches)}))
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- end to end through the public API: host token ids in, host argmax out, every step
    _, cur = model.prefill_batch(prompts, cache)
    for _ in range(W):
        _, cur, _, _ = model.forward_one_batch(cur, cache)
    barrier()
    t0 = time.perf_counter()
    for _ in range(K):
        _, cur, _, _ = model.forward_one_batch(cur, cache)
    e2e_sec = time.perf_counter() - t0
    barrier()
    e2e_value = world * B * K / sharding.max_over_ranks(e2e_sec, device=f"cuda:{local}")

    # ---- per-operation device time of one step (kernel by kernel), for the roofline line
    _, cur = model.prefill_batch(prompts, cache)
    for _ in range(max(W, 3)):
        _, cur, _, _ = model.forward_one_batch(cur, cache)
    prof = {}
    reps = 3
    for _ in range(reps):
        p = model.profile_forward_one(cur, cache)
        for k, (s, n) in p.items():
            prof[k] = (prof.get(k, (0.0, 0))[0] + s / reps, n)
        _, cur, _, _ = model.forward_one_batch(cur, cache)
    t_prof = cache.seq_len_of(0) - 1

    weight_bytes_step = model.weight_bytes_per_step()
    small = small_batch1(pg, synthetic, local) if rank == 0 else None
    prefill = prefill_small(pg, synthetic, local) if rank == 0 else None
    xl = None
    if rank == 0 and not args.no_xl:
        del model, cache  # free the medium model before the 6 GB one comes in
        try:
            xl = xl_sampling(pg, synthetic, local)
        except Exception as exc:  # reported, not fatal: the headline numbers above stand
            xl = {"error": f"{type(exc).__name__}: {exc}"[:300]}
    if rank == 0:
        peak, peak_src = measured_peaks()
        c, f, L = cfg["n_embd"], cfg["n_inner"], cfg["n_layer"]
        # Kernel families of the step and their algorithmic bytes per step. The four linears of a
        # layer (and the lm_head) run the same kernel; its time is the sum of their buckets.
        V = cfg["vocab_size"]
        lin_bytes = L * 4 * (3 * c * c + c * c + 2 * c * f + 4 * c + f) + 4 * V * c  # weights + biases, once
        lin_bytes += L * 4 * B * (2 * c + 3 * c + 2 * c + c + 2 * c + 2 * f + 2 * f + c) + 4 * B * (2 * c + V)
        lin_keys = ("qkv_projection", "attention_projection", "mlp_fc_projection", "mlp_projection", "final_logits")
        attn_bytes = kv_bytes_per_step(cfg, [t_prof] * B) + 4 * B * 4 * c * L
        fam = {
            "linears": (lin_bytes, sum(prof[k][0] for k in lin_keys), sum(prof[k][1] for k in lin_keys)),
            "decode_attention_kernel": (attn_bytes, prof["attention"][0], prof["attention"][1]),
        }
        fused = prof.get("fused_step_kernel")
        phase_roofline = None
        if fused:
            # The whole step is one persistent kernel: it is the dominant kernel, its algorithmic
            # bytes are the step's (weights once + KV cache once), its duration comes from CUDA
            # events around the launch. The kernel's own phase time stamps give the split below.
            dom, dom_bytes, dom_sec, dom_n = "chain_kernel", lin_bytes + attn_bytes, fused[0], 1
            phase_roofline = {
                "gemm_phases": {"bytes": lin_bytes, "us": fam["linears"][1] * 1e6,
                                "GB/s": lin_bytes / fam["linears"][1] / 1e9, "phases": fam["linears"][2]},
                "attention_phases": {"bytes": attn_bytes, "us": prof["attention"][0] * 1e6,
                                     "GB/s": attn_bytes / prof["attention"][0] / 1e9, "phases": prof["attention"][1]},
                "bias_residual_layernorm_phases": {"us": prof["layer_norm"][0] * 1e6, "phases": prof["layer_norm"][1]},
            }
        else:
            dom = max(fam, key=lambda k: fam[k][1])
            dom_bytes, dom_sec, dom_n = fam[dom]
        per_launch = dom_sec / max(dom_n, 1)
        achieved = dom_bytes / dom_sec / 1e9
        kernel_name = dom
        if dom == "linears":
            kernel_name = "tc_gemm_x3_kernel" if args.math == "tf32x3" and 8 < B <= 64 else "linear_decode_kernel"
        # DRAM traffic of the captured launches equals the algorithmic bytes within 4 %
        # (profiles/tc_gemm_x3_kernel_m64_4096x1024.md, profiles/decode_attention_kernel_b64_h16_kv256.md)
        traffic = dom_bytes / max(dom_n, 1) * (1.035 if dom == "linears" else 1.004)
        if fused:
            # ncu capture at 16 sequences: 1.823 GB read vs 1.825 GB algorithmic, writes 0.8 %
            # (profiles/chain_kernel_medium_seqs16.md); both terms scale with the sequences
            traffic = dom_bytes * 1.008
        step_bytes = weight_bytes_step + kv_bytes_per_step(cfg, lens_mid)
        step_achieved = step_bytes / (sec_max / K) / 1e9

        cpu_tokens = 24
        cpu_val, cpu_dt = cpu_baseline_sample(cfg, weights, cpu_tokens, 16, os.cpu_count() or 1)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": sec_max / K * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"gpt2-{MODEL} fp32, {B} sequences per GPU, {PROMPT_LEN}-token prompts, "
                                   f"greedy decode; step = one batched decode step ({B} tokens per GPU)",
                       "linears": ("fp32 weights and activations; products as 3xTF32 on tcgen05 tensor cores, "
                                   "FP32 accumulate" if args.math == "tf32x3" else "fp32 CUDA-core FMA"),
                       "step_kernels": ("ONE persistent kernel per step: embedding, all layers, lm_head, arg-max, "
                                        "token feedback" if fused else "one kernel per operation"),
                       "l2": "inputs larger than L2 (1.4 GB weights + KV per step)", "parallelism": f"replicas x{world}"},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": 4 * B, "d2h_bytes_per_step": 4 * B},
            "gpu_launches": int(launches),
            "clocks": clock_info,
            "roofline": {"bound": "hbm", "kernel": kernel_name, "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": traffic, "peak_source": peak_src,
                         "launches_per_step": dom_n, "per_launch_us": per_launch * 1e6,
                         "algorithmic_bytes_per_launch": dom_bytes / max(dom_n, 1)},
            "step_roofline": {"bound": "hbm", "bytes_per_step": step_bytes, "achieved": step_achieved,
                              "peak": peak, "frac": step_achieved / peak},
            "profile_us": {k: round(v[0] * 1e6, 1) for k, v in prof.items()},
            "phase_roofline": phase_roofline,
            "cpu_baseline": {"value": cpu_val, "unit": UNIT, "cores": os.cpu_count() or 1, "kind": "port",
                             "sample": f"1 sequence, {cpu_tokens} greedy decode tokens after a 16-token prompt "
                                       f"({cpu_dt:.1f} s)"},
            "check": {"tokens_last_step": [int(x) for x in toks[-1][:4]]},
            "also": {"gpt2_small_batch1": small, "gpt2_small_prefill_8x1024": prefill,
                     "gpt2_xl_sampling_32x512_per_gpu": xl},
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--seqs", type=int, default=SEQS_PER_GPU,
                    help="sequences per GPU (default 64, the benchmark workload; smaller for profiler captures)")
    ap.add_argument("--math", default="tf32x3", choices=["fp32", "tf32x3"],
                    help="arithmetic of the batched decode linears: fp32 = CUDA-core FMA, tf32x3 = three TF32 "
                         "tensor-core products with FP32 accumulation (FP32-grade, token-exact against the oracle)")
    ap.add_argument("--no-xl", action="store_true", help="skip the GPT-2 XL sampling line under `also`")
    ap.add_argument("--skip-extras", action="store_true",
                    help="only the device-timed decode loop (no e2e, per-op profile, CPU baseline)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
