"""Generates the committed golden fixtures from the CPU oracle.

    python tests/golden/make_golden.py [small] [medium] [small_prefill] [xl]

`small`  -> gpt2_small_b1.json : GPT-2 small, seeded random-init weights (seed 0), one 32-token
            prompt (seed 1), greedy decode of 64 tokens with the KV cache; the token stream plus,
            for a few steps, the top-5 logits and a strided sample of the logits row.
`medium` -> gpt2_medium_b64.json: GPT-2 medium, 64 prompts of 128 tokens (seeds 1..64), greedy
            decode of 256 tokens each (batched-loop oracle mode: bit-identical to per-sequence).
`small_prefill` -> gpt2_small_prefill_8x1024.json: GPT-2 small, 8 prompts of 1024 tokens (seeds 1..8),
            prefill token by token as the reference does (rust.rs:906-927; the lm_head of positions
            nobody reads is skipped); per sequence the final-position logits: top-40 and a strided sample.
`xl`     -> gpt2_xl_sampling_4x512.json: GPT-2 XL, 4 prompts of 512 tokens (seeds 5000..5003), 32 tokens
            sampled at temperature 0.8 / top-k 40 with sampler seed 1234 + i (generation.rs:221-362);
            per step the drawn token and the top-40 list the draw was made from, so that a run whose
            draw lands on the other side of a cumulative-weight boundary can still be verified
            teacher-forced.
The fixtures record the host architecture: the oracle follows the reference's x86-64 AVX dot.
"""
import json
import os
import platform
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import oracle  # noqa: E402
from puppygrad_b200 import synthetic  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
STRIDE = 997


def logits_record(logits):
    order = sorted(range(logits.size), key=lambda i: (-float(logits[i]), i))[:5]
    return {"top_idx": [int(i) for i in order], "top_val": [float(logits[i]) for i in order],
            "strided": [float(v) for v in logits[::STRIDE]]}


def make_small():
    cfg = synthetic.preset("small")
    w = synthetic.random_init_weights(cfg, seed=0)
    prompt = synthetic.uniform_prompt(1, 32, cfg["vocab_size"])
    model = oracle.Model(cfg, w, threads=os.cpu_count())
    cache = model.new_kv_cache()
    t0 = time.time()
    logits = model.prefill(prompt, cache)
    tokens, records, gaps = [], {}, []
    for step in range(64):
        top2 = np.partition(logits, -2)[-2:]
        gaps.append(float(top2[1] - top2[0]))
        if step in (0, 1, 31, 63):
            records[str(step)] = logits_record(logits)
        nxt = oracle.argmax_logits(logits)
        tokens.append(nxt)
        logits = model.forward_one(nxt, cache)
    out = {"config": cfg, "weight_seed": 0, "prompt_seed": 1, "prompt": [int(t) for t in prompt],
           "tokens": tokens, "logits": records, "logit_stride": STRIDE, "top2_gap_min": min(gaps),
           "host_arch": platform.machine(), "oracle_seconds": round(time.time() - t0, 2)}
    with open(os.path.join(HERE, "gpt2_small_b1.json"), "w") as f:
        json.dump(out, f)
    print("small: tokens", tokens[:8], "... min top-2 gap", min(gaps), "in", out["oracle_seconds"], "s")


def make_medium(n_seq=64, prompt_len=128, new_tokens=256):
    cfg = synthetic.preset("medium")
    w = synthetic.random_init_weights(cfg, seed=0)
    model = oracle.Model(cfg, w, threads=os.cpu_count())
    prompts = [synthetic.uniform_prompt(s + 1, prompt_len, cfg["vocab_size"]) for s in range(n_seq)]
    caches = [model.new_kv_cache() for _ in range(n_seq)]
    t0 = time.time()
    for p, c in zip(prompts, caches):
        c.clear()
    # prefill token by token through the batched loop (same arithmetic as prefill)
    am = None
    for t in range(prompt_len):
        logits, am = model.forward_one_batch([int(p[t]) for p in prompts], caches, want_logits=(t == prompt_len - 1))
    gaps = np.full((new_tokens, n_seq), np.inf, np.float32)
    tokens = np.zeros((new_tokens, n_seq), np.int64)
    for step in range(new_tokens):
        top2 = np.partition(logits, -2, axis=1)[:, -2:]
        gaps[step] = top2[:, 1] - top2[:, 0]
        tokens[step] = am
        if step + 1 < new_tokens:
            logits, am = model.forward_one_batch(am, caches, want_logits=True)
        if step % 16 == 0:
            print("medium step", step, round(time.time() - t0, 1), "s", flush=True)
    out = {"config": cfg, "weight_seed": 0, "prompt_seeds": list(range(1, n_seq + 1)), "prompt_len": prompt_len,
           "tokens": tokens.T.tolist(), "top2_gap": [[round(float(g), 7) for g in row] for row in gaps.T],
           "host_arch": platform.machine(), "oracle_seconds": round(time.time() - t0, 1)}
    with open(os.path.join(HERE, "gpt2_medium_b64.json"), "w") as f:
        json.dump(out, f)
    print("medium done in", out["oracle_seconds"], "s; min gap", float(gaps.min()))


def top_record(logits, k=40, stride=97):
    order = np.lexsort((np.arange(logits.size), -logits.astype(np.float64)))[:k]
    return {"top_idx": [int(i) for i in order], "top_val": [float(logits[i]) for i in order],
            "strided": [float(v) for v in logits[::stride]]}


def make_small_prefill(n_seq=8, prompt_len=1024):
    cfg = synthetic.preset("small")
    w = synthetic.random_init_weights(cfg, seed=0)
    model = oracle.Model(cfg, w, threads=os.cpu_count())
    prompts = [synthetic.uniform_prompt(s + 1, prompt_len, cfg["vocab_size"]) for s in range(n_seq)]
    caches = [model.new_kv_cache() for _ in range(n_seq)]
    t0 = time.time()
    logits = None
    for t in range(prompt_len):
        last = t == prompt_len - 1
        logits, _ = model.forward_one_batch([int(p[t]) for p in prompts], caches, want_logits=last,
                                            want_argmax=last)
        if t % 128 == 0:
            print("small_prefill position", t, round(time.time() - t0, 1), "s", flush=True)
    out = {"config": cfg, "weight_seed": 0, "prompt_seeds": list(range(1, n_seq + 1)), "prompt_len": prompt_len,
           "logit_stride": 97, "final_logits": [top_record(row) for row in logits],
           "logit_span": [float(row.max() - row.min()) for row in logits],
           "host_arch": platform.machine(), "oracle_seconds": round(time.time() - t0, 1)}
    with open(os.path.join(HERE, "gpt2_small_prefill_8x1024.json"), "w") as f:
        json.dump(out, f)
    print("small_prefill done in", out["oracle_seconds"], "s")


def make_xl(n_seq=4, prompt_len=512, new_tokens=32, prompt_seed0=5000, sampler_seed=1234):
    cfg = synthetic.preset("xl")
    w = synthetic.random_init_weights(cfg, seed=0)
    model = oracle.Model(cfg, w, threads=os.cpu_count())
    del w
    prompts = [synthetic.uniform_prompt(prompt_seed0 + s, prompt_len, cfg["vocab_size"]) for s in range(n_seq)]
    caches = [model.new_kv_cache() for _ in range(n_seq)]
    conf = oracle.generation_config(new_tokens, temperature=0.8, top_k=40, seed=sampler_seed)
    samplers = [oracle.LogitsSampler(sampler_seed + i) for i in range(n_seq)]
    t0 = time.time()
    logits = None
    for t in range(prompt_len):
        last = t == prompt_len - 1
        logits, _ = model.forward_one_batch([int(p[t]) for p in prompts], caches, want_logits=last,
                                            want_argmax=last)
        if t % 64 == 0:
            print("xl prompt position", t, round(time.time() - t0, 1), "s", flush=True)
    steps = []
    history = [[int(t) for t in p] for p in prompts]
    for step in range(new_tokens):
        nxt = [samplers[i].select_next_token(logits[i], history[i], conf) for i in range(n_seq)]
        rec = {"tokens": nxt, "top": [top_record(logits[i], 40, 997) for i in range(n_seq)]}
        steps.append(rec)
        for i in range(n_seq):
            history[i].append(nxt[i])
        if step + 1 < new_tokens:
            logits, _ = model.forward_one_batch(nxt, caches, want_logits=True)
        print("xl step", step, round(time.time() - t0, 1), "s", flush=True)
    out = {"config": cfg, "weight_seed": 0, "prompt_seeds": [prompt_seed0 + s for s in range(n_seq)],
           "prompt_len": prompt_len, "temperature": 0.8, "top_k": 40, "sampler_seed": sampler_seed,
           "logit_stride": 997, "steps": steps, "host_arch": platform.machine(),
           "oracle_seconds": round(time.time() - t0, 1)}
    with open(os.path.join(HERE, "gpt2_xl_sampling_4x512.json"), "w") as f:
        json.dump(out, f)
    print("xl done in", out["oracle_seconds"], "s")


if __name__ == "__main__":
    what = sys.argv[1:] or ["small"]
    if "small" in what:
        make_small()
    if "medium" in what:
        make_medium()
    if "small_prefill" in what:
        make_small_prefill()
    if "xl" in what:
        make_xl()
