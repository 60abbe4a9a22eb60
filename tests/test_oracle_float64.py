"""Pin the oracle's absolute numbers against an independent float64 forward."""
import numpy as np
import pytest

from puppygrad_b200 import synthetic
from tests.f64_model import forward_f64


@pytest.mark.parametrize("name,seed,t", [("tiny", 0, 5), ("mini", 1, 24), ("midi", 2, 40)])
def test_full_forward_matches_float64(oracle, name, seed, t):
    cfg = synthetic.preset(name)
    w = synthetic.tiny_weights(cfg) if name == "tiny" else synthetic.perturbed_weights(cfg, seed)
    ids = synthetic.uniform_prompt(seed + 10, t, cfg["vocab_size"])
    got = oracle.Model(cfg, w, threads=2).forward(ids)
    want = forward_f64(cfg, w, ids)
    np.testing.assert_allclose(got, want, rtol=1e-4, atol=2e-5)


def test_cached_path_matches_float64(oracle):
    cfg = synthetic.preset("midi")
    w = synthetic.perturbed_weights(cfg, 4)
    ids = synthetic.uniform_prompt(3, 33, cfg["vocab_size"])
    model = oracle.Model(cfg, w, threads=2)
    cache = model.new_kv_cache()
    want = forward_f64(cfg, w, ids)
    got = model.prefill(ids[:20], cache)
    np.testing.assert_allclose(got, want[19], rtol=1e-4, atol=2e-5)
    for i in range(20, 33):
        got = model.forward_one(ids[i], cache)
        np.testing.assert_allclose(got, want[i], rtol=1e-4, atol=2e-5)


def test_kv_cache_layout_is_head_major(oracle):
    """rust.rs:1851-1855: (head * max_seq_len + pos) * head_dim + dim."""
    cfg = synthetic.preset("mini")
    w = synthetic.perturbed_weights(cfg, 5)
    ids = synthetic.uniform_prompt(4, 6, cfg["vocab_size"])
    model = oracle.Model(cfg, w)
    cache = model.new_kv_cache()
    model.prefill(ids, cache)
    k, v = cache.read_layer(0)
    W = {n: np.asarray(a, np.float64) for n, a in w.items()}
    x = W["wte.weight"][ids] + W["wpe.weight"][:6]
    mu = x.mean(-1, keepdims=True)
    n = (x - mu) / np.sqrt(((x - mu) ** 2).mean(-1, keepdims=True) + 1e-5) * W["h.0.ln_1.weight"] + W["h.0.ln_1.bias"]
    qkv = n @ W["h.0.attn.c_attn.weight"] + W["h.0.attn.c_attn.bias"]
    c, h = cfg["n_embd"], cfg["n_head"]
    d = c // h
    np.testing.assert_allclose(k[:, :6], qkv[:, c:2 * c].reshape(6, h, d).transpose(1, 0, 2), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(v[:, :6], qkv[:, 2 * c:].reshape(6, h, d).transpose(1, 0, 2), rtol=1e-4, atol=1e-5)
    assert not k[:, 6:].any()
