"""ctypes binding of the CPU oracle (`libpg_oracle.so`). TEST INFRASTRUCTURE ONLY.

Only the tests, the smoke check and the benchmark's CPU-baseline leg import this module; the
product package never does. Build the library with `make -C oracle` (or `build()` below).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libpg_oracle.so")

TENSORS_PER_LAYER = 12


class PoConfig(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in
                ("vocab_size", "n_positions", "n_embd", "n_layer", "n_head", "n_inner")] + \
               [("layer_norm_epsilon", C.c_float)]


class PoRustConfig(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in
                ("threads", "dense_parallel_threshold", "qkv_chunk_size",
                 "attention_projection_chunk_size", "mlp_fc_chunk_size",
                 "mlp_projection_chunk_size", "logits_chunk_size",
                 "attention_head_parallel_threshold")]


class PoGenerationConfig(C.Structure):
    _fields_ = [("max_new_tokens", C.c_uint64), ("eos_token_id", C.c_int64),
                ("temperature", C.c_float), ("top_p", C.c_float), ("top_k", C.c_int64),
                ("seed", C.c_uint64), ("repeat_penalty", C.c_float), ("repeat_last_n", C.c_uint64)]


class OracleError(Exception):
    def __init__(self, code: int, message: str):
        super().__init__(message)
        self.code = code
        self.message = message


def build(force: bool = False) -> str:
    src = [os.path.join(_HERE, f) for f in ("pg_oracle.cpp", "pg_oracle.h")]
    stale = force or not os.path.exists(_LIB_PATH) or any(
        os.path.getmtime(s) > os.path.getmtime(_LIB_PATH) for s in src)
    if stale:
        subprocess.run(["make", "-C", _HERE, "-B", "libpg_oracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        L = C.CDLL(_LIB_PATH)
        fp, u64p, vp = C.POINTER(C.c_float), C.POINTER(C.c_uint64), C.c_void_p
        L.po_last_error.restype = C.c_char_p
        L.po_dot.restype = C.c_float
        L.po_dot.argtypes = [fp, fp, C.c_size_t]
        L.po_dot_scalar.restype = C.c_float
        L.po_dot_scalar.argtypes = [fp, fp, C.c_size_t]
        L.po_transposed_dense_projection.argtypes = [fp, C.c_size_t, C.c_size_t, C.c_size_t, fp, fp, fp]
        L.po_dense_projection.argtypes = [fp, C.c_size_t, C.c_size_t, C.c_size_t, fp, fp, fp]
        i8p = C.POINTER(C.c_int8)
        L.po_quantize_rows.argtypes = [fp, C.c_size_t, C.c_size_t, i8p, fp]
        L.po_quantized_projection.argtypes = [fp, C.c_size_t, C.c_size_t, C.c_size_t, i8p, fp, fp, fp]
        L.po_layer_norm_in_place.argtypes = [fp, C.c_size_t, C.c_size_t, fp, fp, C.c_float]
        L.po_gelu_in_place.argtypes = [fp, C.c_size_t]
        L.po_softmax_in_place.argtypes = [fp, C.c_size_t]
        L.po_add_in_place.argtypes = [fp, fp, C.c_size_t]
        L.po_transpose_in_out.argtypes = [fp, C.c_size_t, C.c_size_t, fp]
        L.po_model_new.argtypes = [C.POINTER(PoConfig), C.POINTER(fp), u64p, C.c_uint64,
                                   C.POINTER(PoRustConfig), C.POINTER(vp)]
        L.po_model_free.argtypes = [vp]
        L.po_model_quantize_weights.argtypes = [vp]
        L.po_config_validate.argtypes = [C.POINTER(PoConfig)]
        L.po_cache_new.argtypes = [vp, C.POINTER(vp)]
        L.po_cache_free.argtypes = [vp]
        L.po_cache_seq_len.restype = C.c_uint64
        L.po_cache_seq_len.argtypes = [vp]
        L.po_cache_max_seq_len.restype = C.c_uint64
        L.po_cache_max_seq_len.argtypes = [vp]
        L.po_cache_clear.argtypes = [vp]
        L.po_cache_set_seq_len.argtypes = [vp, C.c_uint64]
        L.po_cache_read_layer.argtypes = [vp, C.c_uint64, fp, fp]
        L.po_forward.argtypes = [vp, u64p, C.c_uint64, fp]
        L.po_prefill.argtypes = [vp, u64p, C.c_uint64, vp, fp]
        L.po_forward_one.argtypes = [vp, C.c_uint64, vp, fp]
        L.po_generate_greedy.argtypes = [vp, u64p, C.c_uint64, C.c_uint64, u64p, u64p]
        L.po_generate_greedy_cached.argtypes = [vp, u64p, C.c_uint64, C.c_uint64, vp, vp, u64p, u64p]
        L.po_forward_one_batch.argtypes = [vp, u64p, C.POINTER(vp), C.c_uint64, fp, u64p]
        L.po_argmax_logits.restype = C.c_uint64
        L.po_argmax_logits.argtypes = [fp, C.c_size_t]
        L.po_generation_config_validate.argtypes = [C.POINTER(PoGenerationConfig)]
        L.po_default_generation_config.argtypes = [C.c_uint64, C.POINTER(PoGenerationConfig)]
        L.po_default_rust_config.argtypes = [C.POINTER(PoRustConfig)]
        L.po_sampler_new.restype = vp
        L.po_sampler_new.argtypes = [C.c_uint64]
        L.po_sampler_free.argtypes = [vp]
        L.po_sampler_next_u64.restype = C.c_uint64
        L.po_sampler_next_u64.argtypes = [vp]
        L.po_sampler_select_next_token.argtypes = [vp, fp, C.c_size_t, u64p, C.c_size_t,
                                                   C.POINTER(PoGenerationConfig), u64p]
        L.po_pool_worker_chunks.restype = C.c_uint64
        L.po_pool_worker_chunks.argtypes = [C.c_uint64] * 4 + [u64p, C.c_uint64]
        _lib = L
    return _lib


def _fp(a: np.ndarray):
    assert a.dtype == np.float32 and a.flags.c_contiguous
    return a.ctypes.data_as(C.POINTER(C.c_float))


def _u64(a: np.ndarray):
    assert a.dtype == np.uint64 and a.flags.c_contiguous
    return a.ctypes.data_as(C.POINTER(C.c_uint64))


def _check(rc: int):
    if rc != 0:
        raise OracleError(rc, lib().po_last_error().decode())


# ------------------------------------------------------------------ cpu.rs kernels
def dot(a, b):
    a = np.ascontiguousarray(a, np.float32); b = np.ascontiguousarray(b, np.float32)
    return float(lib().po_dot(_fp(a), _fp(b), a.size))


def dot_scalar(a, b):
    a = np.ascontiguousarray(a, np.float32); b = np.ascontiguousarray(b, np.float32)
    return float(lib().po_dot_scalar(_fp(a), _fp(b), a.size))


def transposed_dense_projection(x, rows, in_f, out_f, w, bias):
    x = np.ascontiguousarray(x, np.float32); w = np.ascontiguousarray(w, np.float32)
    bias = np.ascontiguousarray(bias, np.float32)
    out = np.empty(rows * out_f, np.float32)
    lib().po_transposed_dense_projection(_fp(x), rows, in_f, out_f, _fp(w), _fp(bias), _fp(out))
    return out


def quantize_rows(w, rows, cols):
    """QuantizedRows::from_f32 (cpu.rs:33-57): returns (int8 values [rows, cols], f32 scales [rows])."""
    w = np.ascontiguousarray(w, np.float32)
    q = np.empty((rows, cols), np.int8)
    scales = np.empty(rows, np.float32)
    lib().po_quantize_rows(_fp(w), rows, cols, q.ctypes.data_as(C.POINTER(C.c_int8)), _fp(scales))
    return q, scales


def quantized_projection(x, rows, in_f, out_f, q, scales, bias):
    """quantized_transposed_dense_projection_into (cpu.rs:99-117)."""
    x = np.ascontiguousarray(x, np.float32); q = np.ascontiguousarray(q, np.int8)
    scales = np.ascontiguousarray(scales, np.float32); bias = np.ascontiguousarray(bias, np.float32)
    out = np.empty(rows * out_f, np.float32)
    lib().po_quantized_projection(_fp(x), rows, in_f, out_f, q.ctypes.data_as(C.POINTER(C.c_int8)), _fp(scales),
                                  _fp(bias), _fp(out))
    return out


def dense_projection(x, rows, in_f, out_f, w, bias):
    x = np.ascontiguousarray(x, np.float32); w = np.ascontiguousarray(w, np.float32)
    bias = np.ascontiguousarray(bias, np.float32)
    out = np.empty(rows * out_f, np.float32)
    lib().po_dense_projection(_fp(x), rows, in_f, out_f, _fp(w), _fp(bias), _fp(out))
    return out


def layer_norm(x, rows, cols, gamma, beta, eps):
    y = np.array(x, np.float32, copy=True).reshape(-1)
    g = np.ascontiguousarray(gamma, np.float32); b = np.ascontiguousarray(beta, np.float32)
    lib().po_layer_norm_in_place(_fp(y), rows, cols, _fp(g), _fp(b), eps)
    return y


def gelu(x):
    y = np.array(x, np.float32, copy=True).reshape(-1)
    lib().po_gelu_in_place(_fp(y), y.size)
    return y


def softmax(x):
    y = np.array(x, np.float32, copy=True).reshape(-1)
    lib().po_softmax_in_place(_fp(y), y.size)
    return y


def transpose_in_out(w, in_f, out_f):
    w = np.ascontiguousarray(w, np.float32).reshape(-1)
    out = np.empty_like(w)
    lib().po_transpose_in_out(_fp(w), in_f, out_f, _fp(out))
    return out


def argmax_logits(v):
    v = np.ascontiguousarray(v, np.float32)
    return int(lib().po_argmax_logits(_fp(v), v.size))


def pool_worker_chunks(threads, length, chunk_size, worker):
    buf = np.zeros(max(1, (length + max(chunk_size, 1) - 1) // max(chunk_size, 1)), np.uint64)
    n = lib().po_pool_worker_chunks(threads, length, chunk_size, worker, _u64(buf), buf.size)
    return [int(v) for v in buf[:n]]


# ------------------------------------------------------------------ model
def tensor_list(cfg: dict, weights: dict):
    """Order the HF-named tensors the way `po_model_new` (and the product ABI) expects them."""
    names = ["wte.weight", "wpe.weight", "ln_f.weight", "ln_f.bias"]
    for i in range(int(cfg["n_layer"])):
        p = f"h.{i}."
        names += [p + s for s in ("ln_1.weight", "ln_1.bias", "attn.c_attn.weight", "attn.c_attn.bias",
                                  "attn.c_proj.weight", "attn.c_proj.bias", "ln_2.weight", "ln_2.bias",
                                  "mlp.c_fc.weight", "mlp.c_fc.bias", "mlp.c_proj.weight", "mlp.c_proj.bias")]
    return [np.ascontiguousarray(weights[n], np.float32) for n in names]


def make_config(cfg: dict) -> PoConfig:
    return PoConfig(cfg["vocab_size"], cfg["n_positions"], cfg["n_embd"], cfg["n_layer"], cfg["n_head"],
                    cfg.get("n_inner") or 4 * cfg["n_embd"], cfg.get("layer_norm_epsilon", 1e-5))


class Cache:
    def __init__(self, model: "Model"):
        self._h = C.c_void_p()
        _check(lib().po_cache_new(model._h, C.byref(self._h)))
        self.model = model

    def __del__(self):
        if getattr(self, "_h", None):
            lib().po_cache_free(self._h)
            self._h = None

    @property
    def seq_len(self):
        return int(lib().po_cache_seq_len(self._h))

    @seq_len.setter
    def seq_len(self, n):
        lib().po_cache_set_seq_len(self._h, n)

    @property
    def max_seq_len(self):
        return int(lib().po_cache_max_seq_len(self._h))

    def clear(self):
        lib().po_cache_clear(self._h)

    def read_layer(self, layer):
        cfg = self.model.cfg
        n = cfg["n_positions"] * cfg["n_embd"]
        k = np.empty(n, np.float32); v = np.empty(n, np.float32)
        _check(lib().po_cache_read_layer(self._h, layer, _fp(k), _fp(v)))
        shape = (cfg["n_head"], cfg["n_positions"], cfg["n_embd"] // cfg["n_head"])
        return k.reshape(shape), v.reshape(shape)


class Model:
    """Mirror of the reference `Gpt2Model` (rust.rs:798-1027) over the C++ restatement."""

    def __init__(self, cfg: dict, weights, threads: int = 1, rust_config: dict | None = None,
                 quantized_weights: bool = False):
        self.cfg = dict(cfg)
        self.cfg.setdefault("n_inner", 4 * cfg["n_embd"])
        self.cfg.setdefault("layer_norm_epsilon", 1e-5)
        tensors = weights if isinstance(weights, list) else tensor_list(self.cfg, weights)
        tensors = [np.ascontiguousarray(t, np.float32).reshape(-1) for t in tensors]
        n = len(tensors)
        ptrs = (C.POINTER(C.c_float) * n)(*[_fp(t) for t in tensors])
        lens = np.array([t.size for t in tensors], np.uint64)
        rc = PoRustConfig()
        lib().po_default_rust_config(C.byref(rc))
        rc.threads = threads
        for k, v in (rust_config or {}).items():
            setattr(rc, k, v)
        pc = make_config(self.cfg)
        self._h = C.c_void_p()
        _check(lib().po_model_new(C.byref(pc), ptrs, _u64(lens), n, C.byref(rc), C.byref(self._h)))
        self.vocab_size = int(self.cfg["vocab_size"])
        if quantized_weights:  # Gpt2RustConfig::quantized_weights (options.rs:62-104)
            lib().po_model_quantize_weights(self._h)

    def __del__(self):
        if getattr(self, "_h", None):
            lib().po_model_free(self._h)
            self._h = None

    def new_kv_cache(self) -> Cache:
        return Cache(self)

    def forward(self, ids):
        ids = np.ascontiguousarray(ids, np.uint64)
        out = np.empty((max(ids.size, 1), self.vocab_size), np.float32)
        _check(lib().po_forward(self._h, _u64(ids), ids.size, _fp(out)))
        return out

    def prefill(self, ids, cache: Cache):
        ids = np.ascontiguousarray(ids, np.uint64)
        out = np.empty(self.vocab_size, np.float32)
        _check(lib().po_prefill(self._h, _u64(ids), ids.size, cache._h, _fp(out)))
        return out

    def forward_one(self, token: int, cache: Cache):
        out = np.empty(self.vocab_size, np.float32)
        _check(lib().po_forward_one(self._h, int(token), cache._h, _fp(out)))
        return out

    def generate_greedy(self, ids, max_new_tokens: int):
        ids = np.ascontiguousarray(ids, np.uint64)
        out = np.empty(ids.size + max_new_tokens + 1, np.uint64)
        n = C.c_uint64()
        _check(lib().po_generate_greedy(self._h, _u64(ids), ids.size, max_new_tokens, _u64(out), C.byref(n)))
        return [int(t) for t in out[:n.value]]

    def generate_greedy_cached(self, ids, max_new_tokens: int, on_token=None):
        ids = np.ascontiguousarray(ids, np.uint64)
        out = np.empty(ids.size + max_new_tokens + 1, np.uint64)
        n = C.c_uint64()
        cb_t = C.CFUNCTYPE(C.c_int, C.c_uint64, C.c_void_p)
        cb = cb_t(lambda tok, _u: int(bool(on_token(int(tok))))) if on_token else None
        _check(lib().po_generate_greedy_cached(self._h, _u64(ids), ids.size, max_new_tokens,
                                               C.cast(cb, C.c_void_p) if cb else None, None,
                                               _u64(out), C.byref(n)))
        return [int(t) for t in out[:n.value]]

    def forward_one_batch(self, tokens, caches, want_logits=False, want_argmax=True):
        """One position for every sequence. With neither output asked for (prompt positions whose
        logits nobody reads) the lm_head is skipped; the caches receive the same K and V."""
        tokens = np.ascontiguousarray(tokens, np.uint64)
        b = tokens.size
        handles = (C.c_void_p * b)(*[c._h for c in caches])
        logits = np.empty((b, self.vocab_size), np.float32) if want_logits else None
        am = np.empty(b, np.uint64) if (want_argmax or want_logits) else None
        _check(lib().po_forward_one_batch(self._h, _u64(tokens), handles, b,
                                          _fp(logits) if want_logits else None,
                                          _u64(am) if am is not None else None))
        return (logits if want_logits else None), (am.astype(np.int64) if am is not None else None)


# ------------------------------------------------------------------ sampling
def generation_config(max_new_tokens=32, eos_token_id=None, temperature=0.0, top_p=None, top_k=None,
                      seed=299_792_458, repeat_penalty=1.0, repeat_last_n=128) -> PoGenerationConfig:
    return PoGenerationConfig(max_new_tokens, -1 if eos_token_id is None else eos_token_id, temperature,
                              -1.0 if top_p is None else top_p, -1 if top_k is None else top_k, seed,
                              repeat_penalty, repeat_last_n)


def validate_generation_config(g: PoGenerationConfig):
    _check(lib().po_generation_config_validate(C.byref(g)))


class LogitsSampler:
    """generation.rs:209-241"""

    def __init__(self, seed: int):
        self._h = C.c_void_p(lib().po_sampler_new(seed))

    def __del__(self):
        if getattr(self, "_h", None):
            lib().po_sampler_free(self._h)
            self._h = None

    def next_u64(self):
        return int(lib().po_sampler_next_u64(self._h))

    def select_next_token(self, logits, history, config: PoGenerationConfig) -> int:
        logits = np.ascontiguousarray(logits, np.float32)
        hist = np.ascontiguousarray(history, np.uint64)
        out = C.c_uint64()
        _check(lib().po_sampler_select_next_token(self._h, _fp(logits), logits.size, _u64(hist), hist.size,
                                                  C.byref(config), C.byref(out)))
        return int(out.value)
