"""Seeded synthetic GPT-2 assets: shape presets, random-init weights, model directories, prompts.

The weights follow the Hugging Face GPT-2 key names and Conv1D `[in, out]` layout that the
reference loader reads (puppygrad src/models/gpt2/rust.rs:713-772). Values: one
`numpy.random.Generator(PCG64(seed))`, `standard_normal(float32) * 0.02`, drawn in the order
wte, wpe, then per layer c_attn, attn.c_proj, c_fc, mlp.c_proj; every bias and LayerNorm beta
is 0 and every LayerNorm gamma is 1.
"""
from __future__ import annotations

import json
import os

import numpy as np

PRESETS = {
    # reference unit-test shape (rust.rs:2082-2092)
    "tiny": dict(vocab_size=8, n_positions=5, n_embd=4, n_layer=1, n_head=2, n_inner=8),
    # small shapes for fast CPU/GPU parity runs; head_dim 64 like every real GPT-2
    "mini": dict(vocab_size=1000, n_positions=128, n_embd=128, n_layer=2, n_head=2, n_inner=512),
    "midi": dict(vocab_size=5003, n_positions=256, n_embd=256, n_layer=3, n_head=4, n_inner=1024),
    "small": dict(vocab_size=50257, n_positions=1024, n_embd=768, n_layer=12, n_head=12, n_inner=3072),
    "medium": dict(vocab_size=50257, n_positions=1024, n_embd=1024, n_layer=24, n_head=16, n_inner=4096),
    "xl": dict(vocab_size=50257, n_positions=1024, n_embd=1600, n_layer=48, n_head=25, n_inner=6400),
}


def preset(name: str) -> dict:
    cfg = dict(PRESETS[name])
    cfg["layer_norm_epsilon"] = 1e-5
    return cfg


def tensor_names(cfg: dict) -> list[str]:
    names = ["wte.weight", "wpe.weight", "ln_f.weight", "ln_f.bias"]
    for i in range(cfg["n_layer"]):
        p = f"h.{i}."
        names += [p + s for s in ("ln_1.weight", "ln_1.bias", "attn.c_attn.weight", "attn.c_attn.bias",
                                  "attn.c_proj.weight", "attn.c_proj.bias", "ln_2.weight", "ln_2.bias",
                                  "mlp.c_fc.weight", "mlp.c_fc.bias", "mlp.c_proj.weight",
                                  "mlp.c_proj.bias")]
    return names


def random_init_weights(cfg: dict, seed: int = 0, std: float = 0.02) -> dict[str, np.ndarray]:
    rng = np.random.Generator(np.random.PCG64(seed))
    c, f, v, p = cfg["n_embd"], cfg["n_inner"], cfg["vocab_size"], cfg["n_positions"]

    def normal(*shape):
        a = rng.standard_normal(shape, dtype=np.float32)
        a *= np.float32(std)
        return a

    w = {"wte.weight": normal(v, c), "wpe.weight": normal(p, c),
         "ln_f.weight": np.ones(c, np.float32), "ln_f.bias": np.zeros(c, np.float32)}
    for i in range(cfg["n_layer"]):
        q = f"h.{i}."
        w[q + "ln_1.weight"] = np.ones(c, np.float32)
        w[q + "ln_1.bias"] = np.zeros(c, np.float32)
        w[q + "attn.c_attn.weight"] = normal(c, 3 * c)
        w[q + "attn.c_attn.bias"] = np.zeros(3 * c, np.float32)
        w[q + "attn.c_proj.weight"] = normal(c, c)
        w[q + "attn.c_proj.bias"] = np.zeros(c, np.float32)
        w[q + "ln_2.weight"] = np.ones(c, np.float32)
        w[q + "ln_2.bias"] = np.zeros(c, np.float32)
        w[q + "mlp.c_fc.weight"] = normal(c, f)
        w[q + "mlp.c_fc.bias"] = np.zeros(f, np.float32)
        w[q + "mlp.c_proj.weight"] = normal(f, c)
        w[q + "mlp.c_proj.bias"] = np.zeros(c, np.float32)
    return w


def perturbed_weights(cfg: dict, seed: int = 0) -> dict[str, np.ndarray]:
    """Like `random_init_weights`, but with non-trivial biases, gammas and betas so that tests
    exercise every term of LayerNorm and of the bias adds."""
    w = random_init_weights(cfg, seed)
    rng = np.random.Generator(np.random.PCG64(seed + 7919))
    for k in w:
        if k.endswith(".bias"):
            w[k] = (rng.standard_normal(w[k].shape, dtype=np.float32) * np.float32(0.05))
        elif "ln_" in k and k.endswith(".weight"):
            w[k] = (1.0 + rng.standard_normal(w[k].shape, dtype=np.float32) * np.float32(0.1)).astype(np.float32)
    return w


def round_bf16(a: np.ndarray) -> np.ndarray:
    """float32 values rounded to the nearest BF16 (ties to even), returned as float32."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32)
    r = ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)) << np.uint32(16)
    return r.view(np.float32).reshape(a.shape)


def bf16_rounded_weights(w: dict[str, np.ndarray]) -> dict[str, np.ndarray]:
    """What math_mode "bf16" computes with: the four dense matrices of every block and the tied embedding rounded
    to BF16, everything else (biases, LayerNorm, position embedding) unchanged."""
    out = dict(w)
    for name, a in w.items():
        if name == "wte.weight" or (a.ndim == 2 and name.startswith("h.")):
            out[name] = round_bf16(a)
    return out


def patterned(n: int, scale: float) -> np.ndarray:
    """The reference tests' deterministic fill (rust.rs:2117-2121, cpu.rs:348-352)."""
    i = np.arange(n, dtype=np.int64)
    return (((i * 17 + 11) % 23).astype(np.float32) - np.float32(11.0)) * np.float32(scale)


def tiny_weights(cfg: dict | None = None) -> dict[str, np.ndarray]:
    """The reference tests' tiny model (rust.rs:2094-2115), in HF `[in,out]` layout."""
    cfg = cfg or preset("tiny")
    c, f = cfg["n_embd"], cfg["n_inner"]
    assert cfg["n_layer"] == 1
    return {
        "wte.weight": patterned(cfg["vocab_size"] * c, 0.03).reshape(cfg["vocab_size"], c),
        "wpe.weight": patterned(cfg["n_positions"] * c, 0.02).reshape(cfg["n_positions"], c),
        "ln_f.weight": np.ones(c, np.float32), "ln_f.bias": np.zeros(c, np.float32),
        "h.0.ln_1.weight": np.ones(c, np.float32), "h.0.ln_1.bias": np.zeros(c, np.float32),
        "h.0.attn.c_attn.weight": patterned(c * 3 * c, 0.01).reshape(c, 3 * c),
        "h.0.attn.c_attn.bias": np.zeros(3 * c, np.float32),
        "h.0.attn.c_proj.weight": patterned(c * c, 0.015).reshape(c, c),
        "h.0.attn.c_proj.bias": np.zeros(c, np.float32),
        "h.0.ln_2.weight": np.ones(c, np.float32), "h.0.ln_2.bias": np.zeros(c, np.float32),
        "h.0.mlp.c_fc.weight": patterned(c * f, 0.01).reshape(c, f),
        "h.0.mlp.c_fc.bias": np.zeros(f, np.float32),
        "h.0.mlp.c_proj.weight": patterned(f * c, 0.012).reshape(f, c),
        "h.0.mlp.c_proj.bias": np.zeros(c, np.float32),
    }


def uniform_prompt(seed: int, length: int, vocab_size: int) -> np.ndarray:
    rng = np.random.Generator(np.random.PCG64(seed))
    return rng.integers(0, vocab_size, size=length, dtype=np.int64)


def write_safetensors(path: str, tensors: dict[str, np.ndarray], prefix: str = "") -> None:
    """Minimal safetensors writer: u64 LE header length, JSON header, raw little-endian data."""
    header, offset = {}, 0
    order = list(tensors)
    for name in order:
        a = tensors[name]
        assert a.dtype == np.float32
        header[prefix + name] = {"dtype": "F32", "shape": list(a.shape),
                                 "data_offsets": [offset, offset + a.nbytes]}
        offset += a.nbytes
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(len(blob).to_bytes(8, "little"))
        f.write(blob)
        for name in order:
            f.write(np.ascontiguousarray(tensors[name]).astype("<f4", copy=False).tobytes())


def read_safetensors(path: str) -> dict[str, np.ndarray]:
    """Reads the F32 tensors of a safetensors file by name (an optional "transformer." prefix is dropped)."""
    with open(path, "rb") as f:
        n = int.from_bytes(f.read(8), "little")
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        if e["dtype"] != "F32":
            raise ValueError(f"tensor {name} has dtype {e['dtype']}, expected F32")
        b, e_ = e["data_offsets"]
        key = name[len("transformer."):] if name.startswith("transformer.") else name
        out[key] = np.frombuffer(data[b:e_], "<f4").reshape(e["shape"]).copy()
    return out


def write_model_dir(path: str, cfg: dict, weights: dict[str, np.ndarray], prefix: str = "") -> str:
    """`config.json` + `model.safetensors`, the two files the loader needs
    (puppygrad src/models/gpt2/assets.rs:6-30)."""
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump({k: cfg[k] for k in ("vocab_size", "n_positions", "n_embd", "n_layer", "n_head",
                                       "n_inner", "layer_norm_epsilon") if k in cfg}, f)
    write_safetensors(os.path.join(path, "model.safetensors"), weights, prefix)
    return path
