#!/usr/bin/env python
"""Benchmark of the GPT-2 decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline workload: GPT-2 medium (24 layers, d_model 1024, 16 heads, d_ff 4096, vocab 50257), FP32
random-init N(0, 0.02) weights (seed 0), 64 independent sequences IN TOTAL with 128-token seeded
uniform prompts, greedy decode. Sequence i runs on GPU i mod N (N = 1, 2, 4, 8; launched by torchrun,
one rank per GPU); every rank holds a full weight replica and there is no collective on the token
path, so the total work is fixed as N grows ("strong" scaling). A step is one decode step of every
sequence (64 tokens). Weights and KV cache (> 1.4 GB per step and GPU) are far larger than L2, so no
explicit L2 flush is needed between steps. Every rank compares the streams it produced with the
committed oracle streams of its sequences (`check.ranks_ok`).

One JSON line is printed by rank 0; see the keys `value`, `e2e`, `roofline`, `cpu_baseline`, `also`.
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
TOTAL_SEQS = 64
PROMPT_LEN = 128
WEIGHT_SEED = 0
GOLDEN = os.path.join(ROOT, "tests", "golden")
NEAR_TIE = 1e-4  # top-2 logit gap below which a greedy choice may legitimately differ (the FP32 logit tolerance)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p.get("bf16_tflops", 1590.0)), "measured"
    return 6650.0, 1590.0, "fallback"


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


def kv_bytes_per_step(cfg, lens):
    # each sequence reads K and V of all cached positions (plus the new one) in every layer, and
    # writes one K row and one V row per layer
    c, L = cfg["n_embd"], cfg["n_layer"]
    return sum(2 * L * (t + 1) * c * 4 + 2 * L * c * 4 for t in lens)


def load_golden(name):
    with open(os.path.join(GOLDEN, name)) as f:
        return json.load(f)


def stream_check(got, gold_tokens, gold_gaps):
    """got: [seq][step] tokens of a free-running greedy decode; a stream is right when it equals the oracle's
    up to its first near-tie (where the oracle's own top-2 gap is below the FP32 logit tolerance)."""
    exact = ok = 0
    for g, t, gap in zip(got, gold_tokens, gold_gaps):
        n = min(len(g), len(t))
        diff = [i for i in range(n) if g[i] != t[i]]
        exact += not diff
        ok += (not diff) or gap[diff[0]] < NEAR_TIE
    return exact, ok


# ---------------------------------------------------------------------------------------------
def cpu_decode_rate(cfg, weights, tokens: int, prompt_len: int, threads: int, warmup: int = 0):
    """Times the CPU oracle (the port of the reference path) on one sequence of the workload:
    prefill `prompt_len` tokens and `warmup` decode steps untimed, then `tokens` greedy decode steps timed."""
    from oracle import oracle
    from puppygrad_b200 import synthetic
    model = oracle.Model(cfg, weights, threads=threads)
    cache = model.new_kv_cache()
    prompt = synthetic.uniform_prompt(1, prompt_len, cfg["vocab_size"])
    logits = model.prefill(prompt, cache)
    for _ in range(warmup):
        logits = model.forward_one(oracle.argmax_logits(logits), cache)
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
    from puppygrad_b200 import synthetic
    cfg = synthetic.preset(MODEL)
    weights = synthetic.random_init_weights(cfg, WEIGHT_SEED)
    threads = os.cpu_count() or 1
    value, dt = cpu_decode_rate(cfg, weights, args.steps, PROMPT_LEN, threads, args.warmup)
    sample = (f"1 of the {TOTAL_SEQS} sequences, {args.steps} greedy decode tokens after its {PROMPT_LEN}-token prompt, "
              f"{threads} threads, C++ port of the reference CPU path")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"gpt2-{MODEL} fp32 greedy decode, one sequence at a time on host cores"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0}))


# --------------------------------------------------------------------------------------------- `also` entries
def small_batch1(pg, synthetic, device):
    """GPT-2 small, one sequence, 32-token prompt, 64 greedy tokens (the first benchmark config): the
    latency-bound case, with FP32, BF16 and int8 weights. FP32 is checked against the committed oracle stream."""
    gold = load_golden("gpt2_small_b1.json")
    cfg = gold["config"]
    weights = synthetic.random_init_weights(cfg, gold["weight_seed"])
    prompt = synthetic.uniform_prompt(gold["prompt_seed"], 32, cfg["vocab_size"])
    peak, _, _ = measured_peaks()
    out = {}
    for name, conf in (("fp32", pg.Gpt2CudaConfig(device=device)),
                       ("bf16_weights", pg.Gpt2CudaConfig(device=device, math_mode="bf16")),
                       ("int8_weights", pg.Gpt2CudaConfig(device=device, quantized_weights=True))):
        model = pg.Gpt2Model(cfg, weights, conf)
        cache = model.new_kv_cache()
        best, toks, first, launches = None, None, None, 0
        for _ in range(3):
            _, first = model.prefill_batch([prompt], cache)
            warm = model.decode_greedy(first, cache, 3)
            n0 = cache.kernel_launches()
            cache.time_begin()
            toks = model.decode_greedy(warm[-1], cache, 60)
            sec = cache.time_end()
            launches = cache.kernel_launches() - n0
            best = sec if best is None else min(best, sec)
        stream = [int(first[0])] + [int(t) for t in warm[:, 0]] + [int(t) for t in toks[:, 0]]
        _, cur = model.prefill_batch([prompt], cache)
        t0 = time.perf_counter()
        for _ in range(60):
            _, cur, _, _ = model.forward_one_batch(cur, cache)
        e2e = time.perf_counter() - t0
        step_bytes = model.weight_bytes_per_step() + kv_bytes_per_step(cfg, [66])
        entry = {"tokens_per_s": 60 / best, "us_per_token": best / 60 * 1e6, "e2e_tokens_per_s": 60 / e2e,
                 "bytes_per_token": step_bytes, "hbm_frac": step_bytes / (best / 60) / 1e9 / peak,
                 "kernel_launches_per_token": launches / 60}
        if name == "fp32":
            entry["check"] = {"tokens_equal_oracle_stream": stream == gold["tokens"][:64]}
        else:
            entry["check"] = {"stream_agrees_with_fp32_for_tokens": int(next(
                (i for i, (a, b) in enumerate(zip(stream, gold["tokens"])) if a != b), 64)),
                "note": "a narrow-weight model is another model: its own parity tests compare it with the oracle run on the same narrow weights"}
        out[name] = entry
        del cache, model
    return out


def prefill_small(pg, synthetic, device):
    """GPT-2 small prefill, 8 prompts of 1024 tokens (the prefill-only config). flops = linear GEMMs only
    (2*B*T*L*12*C^2), over the whole prefill time (attention, LayerNorm and the KV scatter included), so the rate
    is a lower bound. Every mode's final-position logits are compared with the committed oracle rows."""
    gold = load_golden("gpt2_small_prefill_8x1024.json")
    cfg = gold["config"]
    weights = synthetic.random_init_weights(cfg, gold["weight_seed"])
    prompts = [synthetic.uniform_prompt(s, gold["prompt_len"], cfg["vocab_size"]) for s in gold["prompt_seeds"]]
    flops = 2 * 8 * 1024 * cfg["n_layer"] * 12 * cfg["n_embd"] ** 2
    stride = gold["logit_stride"]
    out = {}
    for mode in ("fp32", "tf32x3", "tf32", "bf16"):
        model = pg.Gpt2Model(cfg, weights, pg.Gpt2CudaConfig(device=device, math_mode=mode))
        cache = model.new_kv_cache(max_batch=8)
        logits, _ = model.prefill_batch(prompts, cache, want_logits=True)
        err_abs, err_span = 0.0, 0.0
        for i, rec in enumerate(gold["final_logits"]):
            got = np.concatenate([logits[i, ::stride], logits[i, rec["top_idx"]]])
            want = np.array(rec["strided"] + rec["top_val"], np.float32)
            e = float(np.abs(got - want).max())
            err_abs, err_span = max(err_abs, e), max(err_span, e / gold["logit_span"][i])
        best = None
        for _ in range(3):
            cache.time_begin()
            model.prefill_batch(prompts, cache)
            sec = cache.time_end()
            best = sec if best is None else min(best, sec)
        out[mode] = {"ms": best * 1e3, "prompt_tokens_per_s": 8 * 1024 / best, "linear_tflops": flops / best / 1e12,
                     "check": {"max_abs_logit_error_vs_oracle": err_abs, "as_fraction_of_logit_span": err_span,
                               "bound": "1e-4 + 1e-3*|logit|" if mode in ("fp32", "tf32x3") else
                               ("5e-3 of span" if mode == "tf32" else "3e-2 of span")}}
        del cache, model
    return out


def xl_sampling(pg, synthetic, device, seqs=32, steps=32):
    """GPT-2 XL with temperature 0.8 / top-k 40 sampling and one RNG seed per sequence: one GPU's share (32
    sequences) of the 256-sequence config, 512-token prompts. Every step runs the persistent step kernel, the
    device top-k, and the host draw of the reference sampler; timed on the host clock through the public API
    (token ids in, top-k rows out). The 32 sequences are the 4 sequences of the committed oracle run, eight
    times over, so every drawn token can be compared with the oracle's."""
    from puppygrad_b200.generation import LogitsSampler
    gold = load_golden("gpt2_xl_sampling_4x512.json")
    cfg = gold["config"]
    steps = min(steps, len(gold["steps"]))
    model = pg.Gpt2Model(cfg, synthetic.random_init_weights(cfg, gold["weight_seed"]),
                         pg.Gpt2CudaConfig(device=device, math_mode="tf32x3"))
    base = [synthetic.uniform_prompt(s, gold["prompt_len"], cfg["vocab_size"]) for s in gold["prompt_seeds"]]
    n0 = len(base)
    prompts = [base[i % n0] for i in range(seqs)]
    conf = pg.TextGenerationConfig(steps, temperature=gold["temperature"], top_k=gold["top_k"], seed=gold["sampler_seed"])
    samplers = [LogitsSampler(conf.seed + (i % n0)) for i in range(seqs)]
    cache = model.new_kv_cache(max_batch=seqs)
    t0 = time.perf_counter()
    model.prefill_batch([p[:-1] for p in prompts], cache)
    prefill_s = time.perf_counter() - t0
    _, _, tv, ti = model.forward_one_batch([int(p[-1]) for p in prompts], cache, top_k=40)  # also captures the graph
    launches0 = cache.kernel_launches()
    equal = total = 0
    t0 = time.perf_counter()
    for s in range(steps):
        nxt = LogitsSampler.select_from_topk_batch(samplers, tv, ti, conf)  # one native call for the 32 draws
        want = gold["steps"][s]["tokens"]
        equal += sum(int(nxt[i] == want[i % n0]) for i in range(seqs))
        total += seqs
        if s + 1 < steps:  # teacher-forced, so that one boundary draw does not void the rest of the comparison
            _, _, tv, ti = model.forward_one_batch([want[i % n0] for i in range(seqs)], cache, top_k=40)
    sec = time.perf_counter() - t0
    n_fwd = steps - 1
    return {"tokens_per_s": seqs * n_fwd / sec, "ms_per_step": sec / n_fwd * 1e3, "seqs": seqs,
            "prompt_len": gold["prompt_len"], "steps": n_fwd, "prefill_s": prefill_s,
            "kernel_launches_per_step": (cache.kernel_launches() - launches0) / n_fwd,
            "bytes_per_step": model.weight_bytes_per_step() + kv_bytes_per_step(cfg, [gold["prompt_len"] + steps // 2] * seqs),
            "check": {"drawn_tokens_equal_oracle": equal, "of": total}}


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

    def gather(obj):
        if world == 1:
            return [obj]
        parts = [None] * world
        dist.all_gather_object(parts, obj)
        return parts

    dev = f"cuda:{local}"
    gold = load_golden("gpt2_medium_b64.json")
    cfg = gold["config"]
    weights = synthetic.random_init_weights(cfg, gold["weight_seed"])
    model = pg.Gpt2Model(cfg, weights, pg.Gpt2CudaConfig(device=local, math_mode=args.math))
    total = args.seqs
    mine = sharding.partition(total, world, rank)  # sequence i on GPU i mod N
    prompts = [synthetic.uniform_prompt(gold["prompt_seeds"][i], PROMPT_LEN, cfg["vocab_size"]) for i in mine]
    B, K, W = len(mine), args.steps, args.warmup
    if PROMPT_LEN + W + K + 1 > cfg["n_positions"]:
        raise SystemExit("steps + warmup exceed the context window")
    cache = model.new_kv_cache(max_batch=max(B, 1))

    def decode_block():
        """prefill, W warm-up steps, then K timed steps fed back on the device; device seconds and the streams"""
        _, first = model.prefill_batch(prompts, cache)
        warm = model.decode_greedy(first, cache, W) if W else np.zeros((0, B), np.int32)
        start = warm[-1] if W else first
        n0 = cache.kernel_launches()
        barrier()
        cache.time_begin()
        toks = model.decode_greedy(start, cache, K)
        sec = cache.time_end()
        barrier()
        streams = np.concatenate([first[None, :], warm, toks], axis=0).T  # [seq][step]
        return sec, streams, cache.kernel_launches() - n0

    # ---- device-resident throughput: tokens fed back on the device, CUDA events on the library's stream
    decode_block()  # graph capture, allocator and clock warm-up: untimed
    clocks = ClockSampler(local)
    clocks.start()
    # The same prefill + W warm-up + K-step block again and again until the clock sampler has seen about a second
    # of it (a K-step region alone is tens of milliseconds); the MEDIAN block is the one reported as `value`.
    repeats = []
    if not args.skip_extras:
        while sum(repeats) < 1.0 and len(repeats) < 64:
            repeats.append(sharding.max_over_ranks(decode_block()[0], device=dev))
    sec, streams, launches = decode_block()
    repeats.append(sharding.max_over_ranks(sec, device=dev))
    # every block is W untimed warm-up steps and exactly K timed steps (max over ranks); the reported region is the
    # median block: single blocks of a few tens of milliseconds scatter by several per cent with the power state
    sec_max = float(np.median(repeats)) if not args.skip_extras else repeats[-1]
    value = total * K / sec_max
    exact, ok = stream_check(streams.tolist(), [gold["tokens"][i] for i in mine], [gold["top2_gap"][i] for i in mine])
    checks = gather({"rank": rank, "seqs": B, "exact": int(exact), "ok": int(ok)})
    if args.skip_extras:  # profiling runs: only the timed decode loop
        clocks.stop()
        if rank == 0:
            print(json.dumps({"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K,
                              "warmup": W, "ms_per_step": sec_max / K * 1e3, "seqs_per_gpu": B,
                              "gpu_launches": int(launches),
                              "streams_ok": sum(ch["ok"] for ch in checks), "streams_exact": sum(ch["exact"] for ch in checks)}))
        if world > 1:
            dist.destroy_process_group()
        return
    clock_info = clocks.stop()

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
    e2e_value = total * K / sharding.max_over_ranks(e2e_sec, device=dev)

    # ---- per-operation device time of one step (kernel by kernel), for the roofline line
    prof = {}
    reps = 3
    for _ in range(reps):
        p = model.profile_forward_one(cur, cache)
        for k, (s, n) in p.items():
            prof[k] = (prof.get(k, (0.0, 0))[0] + s / reps, n)
        _, cur, _, _ = model.forward_one_batch(cur, cache)
    t_prof = cache.seq_len_of(0) - 1
    weight_bytes_step = model.weight_bytes_per_step()

    # ---- 64 sequences on EVERY GPU (replicas, weak scaling): what the previous revision of this bench printed
    weak = None
    if world > 1:
        del cache
        wprompts = [synthetic.uniform_prompt(rank * TOTAL_SEQS + i + 1, PROMPT_LEN, cfg["vocab_size"]) for i in range(TOTAL_SEQS)]
        wcache = model.new_kv_cache(max_batch=TOTAL_SEQS)
        _, first = model.prefill_batch(wprompts, wcache)
        first = model.decode_greedy(first, wcache, max(W, 1))[-1]
        barrier()
        wcache.time_begin()
        model.decode_greedy(first, wcache, K)
        wsec = sharding.max_over_ranks(wcache.time_end(), device=dev)
        barrier()
        weak = {"tokens_per_s": world * TOTAL_SEQS * K / wsec, "ms_per_step": wsec / K * 1e3, "seqs_per_gpu": TOTAL_SEQS,
                "scaling": "weak", "check": "rank 0 decodes the oracle's 64 prompts here as well; ranks > 0 use other seeds"}
        del wcache
        cache = None

    small = prefill = xl = None
    if rank == 0 and not args.no_also and world == 1:  # single-GPU measurements: the same at every N
        del cache
        small = small_batch1(pg, synthetic, local)
        prefill = prefill_small(pg, synthetic, local)
        if not args.no_xl:
            del model  # free the medium model before the 6 GB one comes in
            try:
                xl = xl_sampling(pg, synthetic, local)
            except Exception as exc:  # reported, not fatal: the headline numbers above stand
                xl = {"error": f"{type(exc).__name__}: {exc}"[:300]}
    if rank == 0:
        peak, _, peak_src = measured_peaks()
        c, f, L, V = cfg["n_embd"], cfg["n_inner"], cfg["n_layer"], cfg["vocab_size"]
        # algorithmic bytes of a step on one GPU: every weight once, the KV cache of its sequences once
        kv_prof = kv_bytes_per_step(cfg, [t_prof] * B)
        lin_keys = ("qkv_projection", "attention_projection", "mlp_fc_projection", "mlp_projection", "final_logits")
        fused = prof.get("fused_step_kernel")
        phase_roofline = None
        if fused and fused[0] > 0:
            # The whole step is one persistent kernel: it is the dominant kernel, its algorithmic bytes are the step's,
            # its duration comes from CUDA events around one launch in the profiling entry point (which also makes the
            # kernel write per-phase time stamps; the timed steps above run without them and are a little faster).
            kernel_name, dom_bytes, dom_sec, dom_n = "chain_kernel", weight_bytes_step + kv_prof, fused[0], 1
            lin_sec = sum(prof[k][0] for k in lin_keys)
            phase_roofline = {
                "gemm_phases": {"bytes": weight_bytes_step, "us": lin_sec * 1e6, "GB/s": weight_bytes_step / lin_sec / 1e9,
                                "phases": sum(prof[k][1] for k in lin_keys)},
                "attention_phases": {"bytes": kv_prof, "us": prof["attention"][0] * 1e6,
                                     "GB/s": kv_prof / prof["attention"][0] / 1e9, "phases": prof["attention"][1]},
                "bias_residual_layernorm_phases": {"us": prof["layer_norm"][0] * 1e6, "phases": prof["layer_norm"][1]},
            }
        else:
            lin_sec, lin_n = sum(prof[k][0] for k in lin_keys), sum(prof[k][1] for k in lin_keys)
            if lin_sec >= prof["attention"][0]:
                kernel_name = "linear_decode_kernel" if B <= 1 else "linear_rows_smem_kernel" if B <= 8 else "tc_gemm_x3_kernel"
                dom_bytes, dom_sec, dom_n = weight_bytes_step, lin_sec, lin_n
            else:
                kernel_name, dom_bytes, dom_sec, dom_n = "decode_attention_kernel", kv_prof, prof["attention"][0], prof["attention"][1]
        achieved = dom_bytes / dom_sec / 1e9
        # DRAM traffic of the captured launches is within 1 % of the algorithmic bytes (ncu, smaller captures of the same
        # kernels: traffic grows in proportion to the weights and sequences read); scaled, not measured at this size
        traffic = dom_bytes / max(dom_n, 1) * 1.008
        lens_mid = [PROMPT_LEN + W + K // 2] * B
        step_bytes = weight_bytes_step + kv_bytes_per_step(cfg, lens_mid)
        step_achieved = step_bytes / (sec_max / K) / 1e9

        cpu_tokens = 400  # about ten seconds of host work on 16 threads
        cpu_val, cpu_dt = cpu_decode_rate(cfg, weights, cpu_tokens, PROMPT_LEN, os.cpu_count() or 1)
        ranks_ok = [bool(ch["ok"] == ch["seqs"]) for ch in sorted(checks, key=lambda ch: ch["rank"])]
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": sec_max / K * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"gpt2-{MODEL} fp32, {total} sequences in total ({B} per GPU, sequence i on GPU i mod {world}), "
                                   f"{PROMPT_LEN}-token prompts, greedy decode; step = one decode step of every sequence "
                                   f"({total} tokens)",
                       "linears": ("fp32 weights and activations; products as 3xTF32 on tcgen05 tensor cores, "
                                   "FP32 accumulate" if args.math == "tf32x3" and B > 8 else "fp32 CUDA-core FMA"),
                       "step_kernels": ("ONE persistent kernel per step: embedding, all layers, lm_head, arg-max, "
                                        "token feedback" if launches == K else f"{launches // K} kernels per step in a CUDA graph"),
                       "l2": "inputs larger than L2 (1.4 GB weights + KV per step and GPU)", "parallelism": f"replicas x{world}, batch-sharded"},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": 4 * total, "d2h_bytes_per_step": 4 * total},
            "gpu_launches": int(launches) * world,
            "clocks": clock_info,
            "repeat": {"blocks": len(repeats), "seconds": sum(repeats),
                       "ms_per_step": {"min": min(repeats) / K * 1e3, "median": float(np.median(repeats)) / K * 1e3,
                                       "max": max(repeats) / K * 1e3},
                       "what": "the same prefill + warm-up + K-step block repeated under the clock sampler; `value` is the median block"},
            "roofline": {"bound": "hbm", "kernel": kernel_name, "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": traffic, "peak_source": peak_src,
                         "launches_per_step": dom_n, "per_launch_us": dom_sec / max(dom_n, 1) * 1e6,
                         "per_launch_us_is": "CUDA events around the launch(es) of one step in the per-operation profiling call",
                         "algorithmic_bytes_per_launch": dom_bytes / max(dom_n, 1),
                         "algorithmic_bytes_are": "every weight once + K and V of the GPU's sequences once, at the profiled context"},
            "step_roofline": {"bound": "hbm", "bytes_per_step": step_bytes, "achieved": step_achieved,
                              "peak": peak, "frac": step_achieved / peak},
            "profile_us": {k: round(v[0] * 1e6, 1) for k, v in prof.items()},
            "phase_roofline": phase_roofline,
            "cpu_baseline": {"value": cpu_val, "unit": UNIT, "cores": os.cpu_count() or 1, "kind": "port",
                             "sample": f"1 of the {total} sequences, {cpu_tokens} greedy decode tokens after its "
                                       f"{PROMPT_LEN}-token prompt ({cpu_dt:.1f} s timed, prompt not counted)"},
            "check": {"ranks_ok": ranks_ok, "streams_exact": sum(ch["exact"] for ch in checks),
                      "streams_equal_up_to_first_near_tie": sum(ch["ok"] for ch in checks), "of": total,
                      "against": "tests/golden/gpt2_medium_b64.json (oracle streams and top-2 gaps)",
                      "tokens_compared_per_stream": min(W + K + 1, len(gold["tokens"][0]))},
            "also": {"weak_scaling_64_per_gpu": weak, "gpt2_small_batch1": small, "gpt2_small_prefill_8x1024": prefill,
                     "gpt2_xl_sampling_32x512_per_gpu": xl},
        }
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--seqs", type=int, default=TOTAL_SEQS,
                    help="sequences in total (default 64, the benchmark workload; smaller for profiler captures)")
    ap.add_argument("--math", default="tf32x3", choices=["fp32", "tf32x3"],
                    help="arithmetic of decode linears of 9..64 sequences per GPU: fp32 = CUDA-core FMA, tf32x3 = three TF32 "
                         "tensor-core products with FP32 accumulation (FP32-grade, token-exact against the oracle)")
    ap.add_argument("--no-xl", action="store_true", help="skip the GPT-2 XL sampling line under `also`")
    ap.add_argument("--no-also", action="store_true", help="skip every line under `also` but the weak-scaling one")
    ap.add_argument("--skip-extras", action="store_true",
                    help="only the device-timed decode loop (no e2e, per-op profile, CPU baseline)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
