"""Kernel sweep on single operators (device-timed, L2 flushed before every launch).

    python -m puppygrad_b200.sweep linear --m 1 8 64 --n 4800 1600 6400 --k 1600 --math fp32 tf32x3
    python -m puppygrad_b200.sweep linear --preset xl

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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("op", choices=["linear"])
    ap.add_argument("--preset", choices=["xl"], default=None)
    ap.add_argument("--m", type=int, nargs="+", default=[64])
    ap.add_argument("--n", type=int, nargs="+", default=[4096])
    ap.add_argument("--k", type=int, nargs="+", default=[1024])
    ap.add_argument("--math", nargs="+", default=["fp32"])
    ap.add_argument("--epilogue", default="none")
    ap.add_argument("--reps", type=int, default=10)
    a = ap.parse_args()
    shapes = []
    if a.preset == "xl":
        c, f = XL["c"], XL["f"]
        for m in (1, 8, 64, 512, 4096):
            shapes += [(m, 3 * c, c), (m, c, c), (m, f, c), (m, c, f)]
    else:
        shapes = [(m, n, k) for m in a.m for n in a.n for k in a.k]
    for (m, n, k) in shapes:
        for math in a.math:
            if math == "tf32x3" and m > 64:
                continue
            if math != "fp32" and k % 32:
                continue
            print(json.dumps(linear_case(m, n, k, math, a.epilogue, a.reps)), flush=True)


if __name__ == "__main__":
    main()
