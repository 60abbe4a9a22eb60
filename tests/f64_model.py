"""An independent float64 GPT-2 forward in vectorised numpy (no shared code with the oracle).

It follows the published GPT-2 architecture (pre-LN blocks, tanh-GELU, learned positions, tied
lm_head) rather than the reference's loops, so agreement with the oracle checks the oracle's
structure, and its float64 logits classify a token mismatch as a near-tie or a bug.
"""
import numpy as np


def _ln(x, g, b, eps):
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * g + b


def forward_f64(cfg, w, ids):
    """Logits [T, V] in float64 for one sequence."""
    W = {k: np.asarray(v, np.float64) for k, v in w.items()}
    t, c, h = len(ids), cfg["n_embd"], cfg["n_head"]
    d = c // h
    eps = float(np.float32(cfg.get("layer_norm_epsilon", 1e-5)))
    x = W["wte.weight"][np.asarray(ids)] + W["wpe.weight"][:t]
    mask = np.tril(np.ones((t, t), bool))
    for i in range(cfg["n_layer"]):
        p = f"h.{i}."
        n = _ln(x, W[p + "ln_1.weight"], W[p + "ln_1.bias"], eps)
        qkv = n @ W[p + "attn.c_attn.weight"] + W[p + "attn.c_attn.bias"]
        q, k, v = (qkv[:, j * c:(j + 1) * c].reshape(t, h, d).transpose(1, 0, 2) for j in range(3))
        s = q @ k.transpose(0, 2, 1) / np.sqrt(float(d))
        s = np.where(mask, s, -np.inf)
        s = np.exp(s - s.max(-1, keepdims=True))
        s /= s.sum(-1, keepdims=True)
        a = (s @ v).transpose(1, 0, 2).reshape(t, c)
        x = x + a @ W[p + "attn.c_proj.weight"] + W[p + "attn.c_proj.bias"]
        n = _ln(x, W[p + "ln_2.weight"], W[p + "ln_2.bias"], eps)
        m = n @ W[p + "mlp.c_fc.weight"] + W[p + "mlp.c_fc.bias"]
        m = 0.5 * m * (1.0 + np.tanh(0.7978845608028654 * (m + 0.044715 * m ** 3)))
        x = x + m @ W[p + "mlp.c_proj.weight"] + W[p + "mlp.c_proj.bias"]
    x = _ln(x, W["ln_f.weight"], W["ln_f.bias"], eps)
    return x @ W["wte.weight"].T
