"""Host-side mirror of the reference's GPT-2 model API over the CUDA library.

Names, argument meaning and error behaviour follow puppygrad src/models/gpt2/rust.rs:
`Gpt2Config` (31-100), `Gpt2Model` (798-1027), `Gpt2KvCache` (178-249), `Gpt2Output` (150-175) and
the `AutoregressiveDecoder` impl (1253-1277). Batched calls (`*_batch`, `decode_greedy`) are
additions; with one sequence they reduce to the reference calls.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

import numpy as np

from . import _native as N
from .errors import Gpt2Error, check
from .generation import GenerationStats, TextGenerationConfig

_MATH = {"fp32": 0, "tf32x3": 1, "tf32": 2, "bf16": 3}


@dataclass
class Gpt2Config:
    vocab_size: int
    n_positions: int
    n_embd: int
    n_layer: int
    n_head: int
    n_inner: int = 0
    layer_norm_epsilon: float = 1e-5

    def __post_init__(self):
        if not self.n_inner:
            self.n_inner = 4 * self.n_embd

    @classmethod
    def from_dict(cls, d: dict) -> "Gpt2Config":
        return cls(d["vocab_size"], d["n_positions"], d["n_embd"], d["n_layer"], d["n_head"],
                   d.get("n_inner") or 0, d.get("layer_norm_epsilon", 1e-5))

    @classmethod
    def from_json(cls, path: str) -> "Gpt2Config":
        """load_config, rust.rs:696-711"""
        c = N.PgConfig()
        check(N.lib.pg_config_load_json(str(path).encode(), C.byref(c)))
        return cls._from_native(c)

    @classmethod
    def _from_native(cls, c: N.PgConfig) -> "Gpt2Config":
        return cls(c.vocab_size, c.n_positions, c.n_embd, c.n_layer, c.n_head, c.n_inner, c.layer_norm_epsilon)

    def to_native(self) -> N.PgConfig:
        return N.PgConfig(self.vocab_size, self.n_positions, self.n_embd, self.n_layer, self.n_head,
                          self.n_inner, self.layer_norm_epsilon)

    def validate(self) -> None:
        c = self.to_native()
        check(N.lib.pg_config_validate(C.byref(c)))

    def head_dim(self) -> int:
        return self.n_embd // self.n_head


@dataclass
class Gpt2CudaConfig:
    """Knobs of this backend; stands where `Gpt2RustConfig` stands in the reference
    (src/models/gpt2/options.rs:52-96)."""
    device: int = 0
    math_mode: str = "fp32"
    page_tokens: int = 32
    use_graphs: bool = True
    attn_splits: int = 0
    # one cooperative kernel per decode step of <= 8 sequences: None = where it is the faster path, True = whenever
    # the shapes allow, False = never (a CUDA graph of one kernel per operation)
    persistent_step: Optional[bool] = None
    quantized_weights: bool = False  # Gpt2RustConfig::quantized_weights: row-wise int8 dense matrices and lm_head

    def describe(self) -> str:
        """Gpt2BackendConfig::describe (options.rs:36-50), the `backend:` line of run-gpt2."""
        weights = "int8" if self.quantized_weights else "bf16" if self.math_mode == "bf16" else "f32"
        return f"cuda (device={self.device}, math={self.math_mode}, page_tokens={self.page_tokens}, weights={weights})"

    def to_native(self) -> N.PgBackendConfig:
        if self.math_mode not in _MATH:
            raise Gpt2Error("InvalidConfig", f"cuda math_mode {self.math_mode!r} must be one of {sorted(_MATH)}")
        b = N.PgBackendConfig()
        b.device, b.math_mode, b.page_tokens = self.device, _MATH[self.math_mode], self.page_tokens
        b.use_graphs, b.attn_splits = (1 if self.use_graphs else 2), self.attn_splits
        b.persistent_step = 0 if self.persistent_step is None else (1 if self.persistent_step else 2)
        b.quantized_weights = 1 if self.quantized_weights else 0
        return b


@dataclass
class Gpt2Output:
    logits: np.ndarray  # [seq_len, vocab_size]
    seq_len: int
    vocab_size: int

    def logits_for_position(self, pos: int) -> np.ndarray:
        if pos >= self.seq_len:
            raise Gpt2Error("InvalidInput", f"position {pos} out of range for seq_len {self.seq_len}")
        return self.logits[pos]

    def last_logits(self) -> np.ndarray:
        if self.seq_len == 0:
            raise Gpt2Error("InvalidInput", "empty sequence")
        return self.logits_for_position(self.seq_len - 1)


def _i32(a) -> np.ndarray:
    arr = np.asarray(a)
    if arr.size and (arr.min() < -2**31 or arr.max() >= 2**31):
        # keep the id visible to the range check in the library's message
        arr = np.clip(arr, -1, 2**31 - 1)
    return np.ascontiguousarray(arr, np.int32)


def _ip(a: np.ndarray):
    return a.ctypes.data_as(C.POINTER(C.c_int32))


def _fp(a: Optional[np.ndarray]):
    return a.ctypes.data_as(C.POINTER(C.c_float)) if a is not None else None


class Gpt2KvCache:
    """Paged device-resident KV cache for `max_batch` independent sequences."""

    def __init__(self, model: "Gpt2Model", max_batch: int = 1):
        self._h = C.c_void_p()
        self.model = model
        check(N.lib.pg_cache_new(model._h, max_batch, C.byref(self._h)))
        self.max_batch = max_batch

    def __del__(self):
        if getattr(self, "_h", None):
            N.lib.pg_cache_free(self._h)
            self._h = None

    def seq_len_of(self, slot: int) -> int:
        out = C.c_uint64()
        check(N.lib.pg_cache_seq_len(self._h, slot, C.byref(out)))
        return int(out.value)

    @property
    def seq_len(self) -> int:
        return self.seq_len_of(0)

    @property
    def max_seq_len(self) -> int:
        return int(N.lib.pg_cache_max_seq_len(self._h))

    def clear(self) -> None:
        check(N.lib.pg_cache_clear(self._h))

    def clear_slot(self, slot: int) -> None:
        check(N.lib.pg_cache_clear_slot(self._h, slot))

    def time_begin(self) -> None:
        """Starts the device-side stopwatch on this cache's stream."""
        check(N.lib.pg_cache_time_begin(self._h))

    def time_end(self) -> float:
        """Seconds of device time since `time_begin` (waits for the queued work)."""
        out = C.c_double()
        check(N.lib.pg_cache_time_end(self._h, C.byref(out)))
        return float(out.value)

    def kernel_launches(self) -> int:
        return int(N.lib.pg_cache_kernel_launches(self._h))

    def debug_expire_next_wait(self, spin_limit: int = 4096) -> None:
        """Test hook: one bounded device-side wait of the next decode step runs out by its limit."""
        check(N.lib.pg_cache_debug_expire_next_wait(self._h, spin_limit))

    def read_layer(self, layer: int, slot: int = 0):
        """Keys and values in the reference layout [head][max_seq_len][head_dim]."""
        cfg = self.model.config
        n = cfg.n_positions * cfg.n_embd
        k = np.empty(n, np.float32)
        v = np.empty(n, np.float32)
        check(N.lib.pg_cache_read_layer(self._h, slot, layer, _fp(k), _fp(v)))
        shape = (cfg.n_head, cfg.n_positions, cfg.head_dim())
        return k.reshape(shape), v.reshape(shape)


class Gpt2Model:
    def __init__(self, config, weights, cuda_config: Optional[Gpt2CudaConfig] = None):
        """Gpt2Model::new_with_rust_config (rust.rs:803-825). `weights` maps Hugging Face tensor
        names to float32 arrays (dense matrices `[in, out]`), or is the flat list in ABI order."""
        from .synthetic import tensor_names
        self.config = config if isinstance(config, Gpt2Config) else Gpt2Config.from_dict(config)
        self.cuda_config = cuda_config or Gpt2CudaConfig()
        if isinstance(weights, dict):
            names = tensor_names({"n_layer": self.config.n_layer})
            missing = [n for n in names if n not in weights]
            if missing:
                raise Gpt2Error("Asset", f"tensor {missing[0]} not found")
            weights = [weights[n] for n in names]
        tensors = [np.ascontiguousarray(t, np.float32).reshape(-1) for t in weights]
        n = len(tensors)
        ptrs = (C.POINTER(C.c_float) * n)(*[_fp(t) for t in tensors])
        lens = np.array([t.size for t in tensors], np.uint64)
        c, b = self.config.to_native(), self.cuda_config.to_native()
        self._h = C.c_void_p()
        check(N.lib.pg_model_from_host_weights(C.byref(c), ptrs, lens.ctypes.data_as(C.POINTER(C.c_uint64)), n,
                                               C.byref(b), C.byref(self._h)))

    @classmethod
    def from_dir(cls, model_dir: str, cuda_config: Optional[Gpt2CudaConfig] = None, use_tuning: bool = True,
                 tuning_file: Optional[str] = None) -> "Gpt2Model":
        """The model half of Gpt2Runtime::from_dir_with_backend (rust.rs:382-396). Without an explicit
        configuration the tuning file of the model directory is used when it exists (the reference's
        `puppygrad-tune.json` behaviour, main.rs:1333-1342, 2564-2585; `use_tuning=False` is its --no-tuning)."""
        self = cls.__new__(cls)
        if cuda_config is None and use_tuning:
            from .autotune import load_tuning
            cuda_config = load_tuning(str(model_dir), tuning_file)
        self.cuda_config = cuda_config or Gpt2CudaConfig()
        b = self.cuda_config.to_native()
        self._h = C.c_void_p()
        check(N.lib.pg_model_load_dir(str(model_dir).encode(), C.byref(b), C.byref(self._h)))
        c = N.PgConfig()
        check(N.lib.pg_model_config(self._h, C.byref(c)))
        self.config = Gpt2Config._from_native(c)
        return self

    def __del__(self):
        if getattr(self, "_h", None):
            N.lib.pg_model_free(self._h)
            self._h = None

    # ---- AutoregressiveDecoder (rust.rs:1253-1277)
    def max_context_len(self) -> int:
        return int(N.lib.pg_model_max_context_len(self._h))

    def new_cache(self) -> Gpt2KvCache:
        return self.new_kv_cache()

    def select_next_token(self, logits) -> int:
        from .generation import argmax_logits
        return argmax_logits(logits)

    def weight_bytes_per_step(self) -> int:
        return int(N.lib.pg_model_weight_bytes_per_step(self._h))

    # ---- reference single-sequence API
    def new_kv_cache(self, max_batch: int = 1) -> Gpt2KvCache:
        return Gpt2KvCache(self, max_batch)

    def forward(self, input_ids: Sequence[int]) -> Gpt2Output:
        ids = _i32(input_ids)
        v = self.config.vocab_size
        out = np.empty((max(ids.size, 1), v), np.float32)
        check(N.lib.pg_forward(self._h, _ip(ids), ids.size, _fp(out)))
        return Gpt2Output(out, ids.size, v)

    def generate_greedy(self, input_ids: Sequence[int], max_new_tokens: int) -> List[int]:
        ids = _i32(input_ids)
        out = np.empty(ids.size + max_new_tokens + 1, np.int32)
        n = C.c_uint64()
        check(N.lib.pg_generate_greedy(self._h, _ip(ids), ids.size, max_new_tokens, _ip(out), C.byref(n)))
        return [int(t) for t in out[:n.value]]

    def prefill(self, input_ids: Sequence[int], cache: Gpt2KvCache) -> np.ndarray:
        ids = _i32(input_ids)
        lens = np.array([ids.size], np.int32)
        out = np.empty(self.config.vocab_size, np.float32)
        check(N.lib.pg_prefill(self._h, cache._h, _ip(ids), _ip(lens), 1, _fp(out), None))
        return out

    def forward_one(self, token_id: int, cache: Gpt2KvCache) -> np.ndarray:
        ids = _i32([token_id])
        out = np.empty(self.config.vocab_size, np.float32)
        check(N.lib.pg_forward_one(self._h, cache._h, _ip(ids), 1, _fp(out), None, None, None, 0))
        return out

    def generate_greedy_cached(self, input_ids: Sequence[int], max_new_tokens: int) -> List[int]:
        return self.stream_greedy_tokens(input_ids, max_new_tokens, None)

    def stream_greedy_tokens(self, input_ids: Sequence[int], max_new_tokens: int,
                             on_token: Optional[Callable[[int], Optional[bool]]] = None) -> List[int]:
        """rust.rs:1016-1027. `on_token` may return True to abort (the closure returning Err)."""
        ids = _i32(input_ids)
        out = np.empty(ids.size + max_new_tokens + 1, np.int32)
        n = C.c_uint64()
        cb = N.TOKEN_CALLBACK(lambda tok, _u: int(bool(on_token(int(tok))))) if on_token else N.TOKEN_CALLBACK()
        check(N.lib.pg_stream_greedy_tokens(self._h, _ip(ids), ids.size, max_new_tokens, cb, None, _ip(out),
                                            C.byref(n)))
        return [int(t) for t in out[:n.value]]

    def generate_with_config(self, input_ids: Sequence[int], config: TextGenerationConfig,
                             on_token: Optional[Callable[[int], Optional[bool]]] = None):
        """The token-id loop of Gpt2Runtime::stream_token_ids_with_stats (rust.rs:548-635).
        Returns (generated ids, GenerationStats)."""
        ids = _i32(input_ids)
        g = config.to_native()
        out = np.empty(max(config.max_new_tokens, 1), np.int32)
        n = C.c_uint64()
        st = N.PgGenerationStats()
        cb = N.TOKEN_CALLBACK(lambda tok, _u: int(bool(on_token(int(tok))))) if on_token else N.TOKEN_CALLBACK()
        check(N.lib.pg_generate_with_config(self._h, _ip(ids), ids.size, C.byref(g), cb, None, _ip(out),
                                            C.byref(n), C.byref(st)))
        stats = GenerationStats(st.prompt_tokens, st.generated_tokens, st.tokenize_time, st.prefill_time,
                                st.decode_time, st.total_generation_time,
                                None if st.first_token_time < 0 else st.first_token_time)
        return [int(t) for t in out[:n.value]], stats

    # ---- batched additions
    def prefill_batch(self, prompts: Sequence[Sequence[int]], cache: Gpt2KvCache, want_logits: bool = False):
        lens = np.array([len(p) for p in prompts], np.int32)
        ids = _i32(np.concatenate([np.asarray(p, np.int64) for p in prompts]) if len(prompts) else [])
        b = len(prompts)
        logits = np.empty((b, self.config.vocab_size), np.float32) if want_logits else None
        am = np.empty(b, np.int32)
        check(N.lib.pg_prefill(self._h, cache._h, _ip(ids), _ip(lens), b, _fp(logits), _ip(am)))
        return logits, am

    def forward_one_batch(self, token_ids: Sequence[int], cache: Gpt2KvCache, want_logits: bool = False,
                          top_k: int = 0):
        ids = _i32(token_ids)
        b = ids.size
        logits = np.empty((b, self.config.vocab_size), np.float32) if want_logits else None
        am = np.empty(b, np.int32)
        tv = np.empty((b, top_k), np.float32) if top_k else None
        ti = np.empty((b, top_k), np.int32) if top_k else None
        check(N.lib.pg_forward_one(self._h, cache._h, _ip(ids), b, _fp(logits), _ip(am), _fp(tv),
                                   _ip(ti) if top_k else None, top_k))
        return logits, am, tv, ti

    def profile_forward_one(self, token_ids: Sequence[int], cache: Gpt2KvCache) -> dict:
        """One decode step timed per operation class (Gpt2OperationProfile, rust.rs:336-347).
        Returns {bucket: (seconds, kernel launches)}; when the step ran as one persistent kernel the
        counts are phases of that kernel and "fused_step_kernel" holds (its duration, phases)."""
        ids = _i32(token_ids)
        p = N.PgOperationProfile()
        check(N.lib.pg_profile_forward_one(self._h, cache._h, _ip(ids), ids.size, C.byref(p)))
        names = ("layer_norm", "qkv_projection", "attention", "attention_projection", "mlp_fc_projection",
                 "mlp_projection", "final_logits", "other")
        out = {n: (getattr(p, n), int(p.launches[i])) for i, n in enumerate(names)}
        if p.fused_phases:
            out["fused_step_kernel"] = (p.fused_step_kernel, int(p.fused_phases))
        return out

    def generate_batch(self, prompts: Sequence[Sequence[int]], config: TextGenerationConfig,
                       seeds: Optional[Sequence[int]] = None, cache: Optional[Gpt2KvCache] = None) -> List[List[int]]:
        """The token-id loop of Gpt2Runtime::stream_token_ids_with_stats (rust.rs:577-617) for a
        batch of independent sequences, each with its own LogitsSampler seeded `seeds[i]`
        (default config.seed + i). Greedy without repeat penalty uses the device arg-max;
        temperature with top_k <= 64 and no repeat penalty uses the device top-k and the host
        draw of sample_logits; anything else brings the logits rows back to the host sampler.
        A sequence that emits EOS stops; the others continue. Returns the generated ids."""
        from .generation import LogitsSampler
        config.validate()
        n = len(prompts)
        seeds = list(seeds) if seeds is not None else [config.seed + i for i in range(n)]
        samplers = [LogitsSampler(s) for s in seeds]
        cache = cache or self.new_kv_cache(max_batch=n)
        penalty = not (config.repeat_penalty == 1.0 or config.repeat_last_n == 0)
        greedy = config.temperature <= 0.0
        use_argmax = greedy and not penalty
        use_topk = (not greedy) and (not penalty) and config.top_k is not None and 0 < config.top_k <= 64
        k = config.top_k if use_topk else 0
        history = [[int(t) for t in p] for p in prompts]
        out: List[List[int]] = [[] for _ in range(n)]
        done = [False] * n
        logits, am = self.prefill_batch(prompts, cache, want_logits=not use_argmax)
        tv = ti = None
        if use_topk:  # prefill returns whole rows: order them on the host like the device top-k does
            tv = np.empty((n, k), np.float32)
            ti = np.empty((n, k), np.int32)
            idx = np.arange(logits.shape[1])
            for i in range(n):
                order = np.lexsort((idx, -logits[i]))[:k]  # descending value, ties by lower index
                tv[i], ti[i] = logits[i, order], order
        for step in range(config.max_new_tokens):
            nxt = np.zeros(n, np.int32)
            # all draws of the step in one native call when every sequence is still running
            drawn = LogitsSampler.select_from_topk_batch(samplers, tv, ti, config) if use_topk and not any(done) else None
            for i in range(n):
                if done[i]:
                    nxt[i] = history[i][-1]
                    continue
                if len(history[i]) >= self.config.n_positions:
                    done[i] = True
                    nxt[i] = history[i][-1]
                    continue
                if use_argmax:
                    tok = int(am[i])
                elif use_topk:
                    tok = int(drawn[i]) if drawn is not None else samplers[i].select_from_topk(tv[i], ti[i], config)
                else:
                    tok = samplers[i].select_next_token(logits[i], history[i], config)
                if config.eos_token_id is not None and tok == config.eos_token_id:
                    done[i] = True
                    nxt[i] = history[i][-1]
                    continue
                history[i].append(tok)
                out[i].append(tok)
                nxt[i] = tok
            if all(done) or step + 1 == config.max_new_tokens:
                break
            if any(len(h) >= self.config.n_positions for h, d in zip(history, done) if not d):
                for i in range(n):
                    if len(history[i]) >= self.config.n_positions:
                        done[i] = True
                if all(done):
                    break
            # finished sequences keep stepping on their last token: their slots are independent
            # and their outputs are ignored; a full slot would raise, so stop feeding those
            if any(cache.seq_len_of(i) >= self.config.n_positions for i in range(n)):
                break
            logits, am, tv, ti = self.forward_one_batch(nxt, cache, want_logits=not (use_argmax or use_topk), top_k=k)
        return out

    def decode_greedy(self, first_ids: Sequence[int], cache: Gpt2KvCache, steps: int) -> np.ndarray:
        """`steps` greedy steps with the token fed back on the device; returns [steps, batch]."""
        ids = _i32(first_ids)
        out = np.empty((steps, ids.size), np.int32)
        check(N.lib.pg_decode_greedy(self._h, cache._h, _ip(ids), ids.size, steps, _ip(out)))
        return out
