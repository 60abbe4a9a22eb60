"""Kernel sweep on single operators (device-timed, L2 flushed before every launch).

    python -m puppygrad_b200.sweep linear --m 1 8 64 --n 4800 1600 6400 --k 1600 --math fp32 tf32x3
    python -m puppygrad_b200.sweep linear --preset xl
    python -m puppygrad_b200.sweep linear_q8 --m 1 8 --n 4800 6400 --k 1600
    python -m puppygrad_b200.sweep prefill --model small --seqs 8 --prompt-len 1024 --math fp32 tf32
    python -m puppygrad_b200.sweep layernorm --m 1 64 4096 --k 1600
    python -m puppygrad_b200.sweep lm_head --m 1 8 --k 1600
    python -m puppygrad_b200.sweep xl_table        # every case of the GPT-2 XL kernel sweep as one markdown table
    python -m puppygrad_b200.sweep decode --model small --batch 1 --prompt-len 32 --steps 60 [--weights fp32 bf16 int8]

Prints one JSON line per case: seconds per launch, algorithmic GB/s (4*(k*n + m*k + m*n + n) bytes)
and TFLOP/s (2*m*n*k), plus the largest deviation from a float64 product of the same inputs.
Inputs are N(0, 1) float32 from a per-case seed.
"""
from __future__ import annotations

import argparse
import json

import numpy as np

from . import ops

XL = dict(c=1600, f=6400)


def linear_case(m, n, k, math, epilogue, reps, seed=0):
    rng = np.random.default_rng(seed + 7 * m + 13 * n + 17 * k)
    x = rng.standard_normal((m, k), dtype=np.float32)
    w = rng.standard_normal((n, k), dtype=np.float32)
    b = rng.standard_normal(n, dtype=np.float32)
    r = rng.standard_normal((m, n), dtype=np.float32) if epilogue == "resid" else None
    out, sec = ops.linear(x, w, b, r, epilogue, math, reps=reps)
    rows = min(m, 4)  # float64 check on a few rows keeps the host cost bounded
    want = x[:rows].astype(np.float64) @ w.astype(np.float64).T + b
    if epilogue == "gelu":
        want = 0.5 * want * (1 + np.tanh(0.7978845608028654 * (want + 0.044715 * want ** 3)))
    if epilogue == "resid":
        want = want + r[:rows]
    err = float(np.abs(out[:rows] - want).max() / max(np.abs(want).max(), 1e-30))
    bytes_ = 4 * (k * n + m * k + m * n + n)
    return {"op": "linear", "m": m, "n": n, "k": k, "math": math, "epilogue": epilogue, "us": sec * 1e6,
            "gbps": bytes_ / sec / 1e9, "tflops": 2 * m * n * k / sec / 1e12, "max_rel_err_vs_f64": err}


def attention_case(batch, n_head, kv_len, splits, reps, seed=0):
    """Decode attention, head_dim 64. Algorithmic bytes: 4 * batch * (2 * kv_len * c + 4 * c)."""
    rng = np.random.default_rng(seed + batch + 3 * kv_len)
    d = 64
    c = n_head * d
    qkv = rng.standard_normal((batch, 3 * c), dtype=np.float32)
    keys = rng.standard_normal((batch, n_head, kv_len, d), dtype=np.float32)
    values = rng.standard_normal((batch, n_head, kv_len, d), dtype=np.float32)
    out, sec = ops.decode_attention(qkv, keys, values, page_tokens=32, splits=splits, reps=reps)
    # float64 check on the first sequence and head
    k_all = np.concatenate([keys[0, 0], qkv[0, c:c + d][None]], 0).astype(np.float64)
    v_all = np.concatenate([values[0, 0], qkv[0, 2 * c:2 * c + d][None]], 0).astype(np.float64)
    sc = k_all @ qkv[0, :d].astype(np.float64) / 8.0
    p = np.exp(sc - sc.max())
    want = (p / p.sum()) @ v_all
    err = float(np.abs(out[0, :d] - want).max() / max(np.abs(want).max(), 1e-30))
    bytes_ = 4 * batch * (2 * kv_len * c + 4 * c)
    return {"op": "decode_attention", "batch": batch, "n_head": n_head, "kv_len": kv_len, "splits": splits,
            "us": sec * 1e6, "gbps": bytes_ / sec / 1e9, "max_rel_err_vs_f64": err}


def linear_q8_case(m, n, k, reps, seed=0):
    """Decode-sized projection over int8 row-quantised weights. Algorithmic bytes: n*k weights +
    4*(n scales + n bias + m*k + m*n)."""
    rng = np.random.default_rng(seed + 7 * m + 13 * n + 17 * k)
    x = rng.standard_normal((m, k), dtype=np.float32)
    w = rng.standard_normal((n, k), dtype=np.float32)
    b = rng.standard_normal(n, dtype=np.float32)
    q, scales = ops.quantize_rows(w)
    out, sec = ops.linear_q8(x, q, scales, b, reps=reps)
    deq = q[:4].astype(np.float64) * scales[:4, None].astype(np.float64)
    want = x.astype(np.float64) @ deq.T + b[:4]
    err = float(np.abs(out[:, :4] - want).max() / max(np.abs(want).max(), 1e-30))
    bytes_ = n * k + 4 * (2 * n + m * k + m * n)
    return {"op": "linear_q8", "m": m, "n": n, "k": k, "us": sec * 1e6, "gbps": bytes_ / sec / 1e9,
            "fp32_equivalent_gbps": 4 * n * k / sec / 1e9, "max_rel_err_vs_f64": err}


def layernorm_case(rows, d, reps, seed=0):
    """LayerNorm of `rows` rows of width d. Algorithmic bytes: 4 * (2 * rows * d + 2 * d)."""
    rng = np.random.default_rng(seed + rows + 3 * d)
    x = rng.standard_normal((rows, d), dtype=np.float32)
    g = rng.standard_normal(d, dtype=np.float32)
    b = rng.standard_normal(d, dtype=np.float32)
    out, sec = ops.layernorm(x, g, b, 1e-5, reps=reps)
    x64 = x[:4].astype(np.float64)
    want = (x64 - x64.mean(1, keepdims=True)) / np.sqrt(x64.var(1, keepdims=True) + 1e-5) * g + b
    err = float(np.abs(out[:4] - want).max() / max(np.abs(want).max(), 1e-30))
    bytes_ = 4 * (2 * rows * d + 2 * d)
    return {"op": "layernorm", "rows": rows, "d": d, "us": sec * 1e6, "gbps": bytes_ / sec / 1e9, "max_rel_err_vs_f64": err}


def lm_head_case(m, k, vocab, reps, seed=0):
    """Tied lm_head GEMV with the arg-max fused. Algorithmic bytes: 4 * (vocab * k + m * k + m * vocab)."""
    rng = np.random.default_rng(seed + m + 3 * k)
    h = rng.standard_normal((m, k), dtype=np.float32)
    w = rng.standard_normal((vocab, k), dtype=np.float32)
    logits, am, sec = ops.lm_head_argmax(h, w, reps=reps)
    want = h.astype(np.float64) @ w.astype(np.float64).T
    err = float(np.abs(logits - want).max() / max(np.abs(want).max(), 1e-30))
    bytes_ = 4 * (vocab * k + m * k + m * vocab)
    return {"op": "lm_head_argmax", "m": m, "k": k, "vocab": vocab, "us": sec * 1e6, "gbps": bytes_ / sec / 1e9,
            "argmax_equal_f64": bool((am == want.argmax(1)).all()), "max_rel_err_vs_f64": err}


def xl_table(reps, hbm_gbs, tf32_tflops, fp32_tflops=74.5):
    """Every case of the kernel sweep on GPT-2 XL shapes, one markdown row each: time, algorithmic GB/s or
    TFLOP/s, the fraction of the given peak that bounds the case, error against a float64 product."""
    c, f, v = XL["c"], XL["f"], 50257
    rows = ["| operator | shape | path | us | GB/s | TFLOP/s | bound | fraction of peak | max rel. error vs float64 |",
            "|---|---|---|---|---|---|---|---|---|"]
    print("\n".join(rows), flush=True)

    def add(name, shape, path, r, bound):
        frac = (r["gbps"] / hbm_gbs if bound == "hbm" else
                r.get("tflops", 0.0) / (fp32_tflops if bound == "fp32 fma" else tf32_tflops))
        rows.append(f"| {name} | {shape} | {path} | {r['us']:.1f} | {r['gbps']:.0f} | {r.get('tflops', 0.0):.1f} | {bound} | "
                    f"{frac:.3f} | {r['max_rel_err_vs_f64']:.1e} |")
        print(rows[-1], flush=True)

    for m in (1, 8, 64, 512, 4096):
        for (n, k) in ((3 * c, c), (c, c), (f, c), (c, f)):
            maths = ["fp32"] + (["tf32x3"] if m > 8 else []) + (["tf32"] if m >= 128 else [])
            for math in maths:
                r = linear_case(m, n, k, math, "none", reps)
                add("linear", f"{m} x {k} -> {n}", math, r, "hbm" if m <= 64 else ("fp32 fma" if math == "fp32" else "tensor"))
    for b in (1, 32, 256):
        for kv in (128, 256, 512, 1024):
            sp = max(1, min(8, (2 * 148 + b * 25 - 1) // (b * 25), (kv + 128) // 128))
            add("decode attention", f"batch {b}, 25 heads, {kv} keys", f"{sp} splits", attention_case(b, 25, kv, sp, reps), "hbm")
    for rws in (1, 64, 4096):
        add("layernorm", f"{rws} x {c}", "fp32", layernorm_case(rws, c, reps), "hbm")
    for m in (1, 8):
        add("lm_head + arg-max", f"{m} x {c} -> {v}", "fp32", lm_head_case(m, c, v, reps), "hbm")
    return rows


def decode_case(preset, batch, prompt_len, steps, math, weights, persistent, reps):
    """Greedy decode fed back on the device: `steps` steps of `batch` sequences after seeded prompts; best of `reps`.
    Algorithmic bytes per step: every weight once (at its stored width) + K and V of every sequence once."""
    from . import synthetic
    from .gpt2 import Gpt2CudaConfig, Gpt2Model
    cfg = synthetic.preset(preset)
    conf = Gpt2CudaConfig(math_mode="bf16" if weights == "bf16" else math, quantized_weights=weights == "int8",
                          persistent_step=persistent)
    model = Gpt2Model(cfg, synthetic.random_init_weights(cfg, 0), conf)
    cache = model.new_kv_cache(max_batch=batch)
    prompts = [synthetic.uniform_prompt(i + 1, prompt_len, cfg["vocab_size"]) for i in range(batch)]
    best, launches = None, 0
    for _ in range(reps):
        _, first = model.prefill_batch(prompts, cache)
        first = model.decode_greedy(first, cache, 4)[-1]
        n0 = cache.kernel_launches()
        cache.time_begin()
        model.decode_greedy(first, cache, steps)
        sec = cache.time_end()
        launches = cache.kernel_launches() - n0
        best = sec if best is None else min(best, sec)
    mid = prompt_len + 4 + steps // 2
    kv = batch * (2 * cfg["n_layer"] * (mid + 1) * cfg["n_embd"] * 4 + 2 * cfg["n_layer"] * cfg["n_embd"] * 4)
    bytes_ = model.weight_bytes_per_step() + kv
    return {"op": "decode", "preset": preset, "batch": batch, "prompt_len": prompt_len, "steps": steps, "math": math,
            "weights": weights, "persistent_step": persistent, "us_per_step": best / steps * 1e6,
            "tokens_per_s": batch * steps / best, "kernel_launches_per_step": launches / steps,
            "bytes_per_step": bytes_, "gbps": bytes_ / (best / steps) / 1e9}


def prefill_case(preset, seqs, prompt_len, math, reps):
    """Whole prefill of `seqs` prompts of `prompt_len` tokens (seeded random weights and ids),
    device-timed; the best of `reps` runs after one warm-up."""
    from . import synthetic
    from .gpt2 import Gpt2CudaConfig, Gpt2Model
    cfg = synthetic.preset(preset)
    model = Gpt2Model(cfg, synthetic.random_init_weights(cfg, 0), Gpt2CudaConfig(math_mode=math))
    prompts = [synthetic.uniform_prompt(s + 1, prompt_len, cfg["vocab_size"]) for s in range(seqs)]
    cache = model.new_kv_cache(max_batch=seqs)
    model.prefill_batch(prompts, cache)
    best = None
    for _ in range(reps):
        cache.time_begin()
        model.prefill_batch(prompts, cache)
        sec = cache.time_end()
        best = sec if best is None else min(best, sec)
    c, layers, t = cfg["n_embd"], cfg["n_layer"], seqs * prompt_len
    attn_flops = 4 * seqs * cfg["n_head"] * (c // cfg["n_head"]) * prompt_len * (prompt_len + 1) // 2 * layers
    return {"op": "prefill", "preset": preset, "seqs": seqs, "prompt_len": prompt_len, "math": math,
            "ms": best * 1e3, "prompt_tokens_per_s": t / best,
            "linear_tflops": 2 * t * layers * 12 * c * c / best / 1e12,
            "linear_plus_attention_tflops": (2 * t * layers * 12 * c * c + attn_flops) / best / 1e12}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("op", choices=["linear", "linear_q8", "attention", "prefill", "layernorm", "lm_head", "xl_table", "decode"])
    ap.add_argument("--steps", type=int, default=60, help="decode: timed steps")
    ap.add_argument("--weights", nargs="+", default=["fp32"], choices=["fp32", "bf16", "int8"])
    ap.add_argument("--persistent", default="auto", choices=["auto", "on", "off"],
                    help="decode: the single-kernel step of small batches")
    ap.add_argument("--hbm-gbs", type=float, default=6534.5, help="xl_table: HBM peak the fractions are taken of")
    ap.add_argument("--tf32-tflops", type=float, default=725.0, help="xl_table: TF32 tensor peak (library GEMM at 8192^3 on B200)")
    ap.add_argument("--vocab", type=int, default=50257)
    ap.add_argument("--model", default="small", help="prefill: model preset")
    ap.add_argument("--seqs", type=int, default=8, help="prefill: prompts per call")
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--batch", type=int, nargs="+", default=[1, 32, 256])
    ap.add_argument("--kv", type=int, nargs="+", default=[128, 256, 512, 1024])
    ap.add_argument("--heads", type=int, default=25)
    ap.add_argument("--splits", type=int, default=0, help="0 = as the model would choose")
    ap.add_argument("--preset", choices=["xl"], default=None)
    ap.add_argument("--m", type=int, nargs="+", default=[64])
    ap.add_argument("--n", type=int, nargs="+", default=[4096])
    ap.add_argument("--k", type=int, nargs="+", default=[1024])
    ap.add_argument("--math", nargs="+", default=["fp32"])
    ap.add_argument("--epilogue", default="none")
    ap.add_argument("--reps", type=int, default=10)
    a = ap.parse_args()
    if a.op == "decode":
        pers = {"auto": None, "on": True, "off": False}[a.persistent]
        for b in a.batch:
            for wt in a.weights:
                print(json.dumps(decode_case(a.model, b, a.prompt_len, a.steps, a.math[0], wt, pers, a.reps)), flush=True)
        return
    if a.op == "xl_table":
        xl_table(a.reps, a.hbm_gbs, a.tf32_tflops)
        return
    if a.op == "layernorm":
        for m in a.m:
            for k in a.k:
                print(json.dumps(layernorm_case(m, k, a.reps)), flush=True)
        return
    if a.op == "lm_head":
        for m in a.m:
            for k in a.k:
                print(json.dumps(lm_head_case(m, k, a.vocab, a.reps)), flush=True)
        return
    if a.op == "prefill":
        for math in a.math:
            print(json.dumps(prefill_case(a.model, a.seqs, a.prompt_len, math, a.reps)), flush=True)
        return
    if a.op == "linear_q8":
        for m in a.m:
            for n in a.n:
                for k in a.k:
                    print(json.dumps(linear_q8_case(m, n, k, a.reps)), flush=True)
        return
    if a.op == "attention":
        for b in a.batch:
            for kv in a.kv:
                sp = a.splits or max(1, min(8, (2 * 148 + b * a.heads - 1) // (b * a.heads), (kv + 128) // 128))
                print(json.dumps(attention_case(b, a.heads, kv, sp, a.reps)), flush=True)
        return
    shapes = []
    if a.preset == "xl":
        c, f = XL["c"], XL["f"]
        for m in (1, 8, 64, 512, 4096):
            shapes += [(m, 3 * c, c), (m, c, c), (m, f, c), (m, c, f)]
    else:
        shapes = [(m, n, k) for m in a.m for n in a.n for k in a.k]
    for (m, n, k) in shapes:
        for math in a.math:
            if math != "fp32" and k % 32:
                continue
            print(json.dumps(linear_case(m, n, k, math, a.epilogue, a.reps)), flush=True)


if __name__ == "__main__":
    main()
