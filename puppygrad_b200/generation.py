"""Sampling configuration and the logits sampler, mirroring puppygrad src/models/generation.rs.
The arithmetic runs in the native library (csrc/sampler.cpp); nothing here touches the GPU."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np

from . import _native as N
from .errors import Gpt2Error, check

GPT2_EOS_TOKEN_ID = 50_256  # src/models/gpt2/options.rs:8


@dataclass
class TextGenerationConfig:
    """generation.rs:60-116; defaults of TextGenerationConfig::new."""
    max_new_tokens: int = 32
    eos_token_id: Optional[int] = None
    temperature: float = 0.0
    top_p: Optional[float] = None
    top_k: Optional[int] = None
    seed: int = 299_792_458
    repeat_penalty: float = 1.0
    repeat_last_n: int = 128

    def with_eos_token_id(self, eos_token_id: Optional[int]) -> "TextGenerationConfig":
        self.eos_token_id = eos_token_id
        return self

    def to_native(self) -> N.PgGenerationConfig:
        return N.PgGenerationConfig(self.max_new_tokens, -1 if self.eos_token_id is None else self.eos_token_id,
                                    self.temperature, -1.0 if self.top_p is None else self.top_p,
                                    -1 if self.top_k is None else self.top_k, self.seed, self.repeat_penalty,
                                    self.repeat_last_n)

    def validate(self) -> None:
        g = self.to_native()
        check(N.lib.pg_generation_config_validate(C.byref(g)))


def gpt2_generation_config(max_new_tokens: int) -> TextGenerationConfig:
    """Gpt2GenerationConfig::new (options.rs:156-162): EOS 50256."""
    return TextGenerationConfig(max_new_tokens).with_eos_token_id(GPT2_EOS_TOKEN_ID)


@dataclass
class GenerationStats:
    """generation.rs:129-180"""
    prompt_tokens: int = 0
    generated_tokens: int = 0
    tokenize_time: float = 0.0
    prefill_time: float = 0.0
    decode_time: float = 0.0
    total_generation_time: float = 0.0
    first_token_time: Optional[float] = None

    def to_native(self) -> "N.PgGenerationStats":
        return N.PgGenerationStats(self.prompt_tokens, self.generated_tokens, self.tokenize_time, self.prefill_time,
                                   self.decode_time, self.total_generation_time,
                                   -1.0 if self.first_token_time is None else self.first_token_time)

    def with_profile(self, profile) -> "ProfiledGenerationStats":
        """generation.rs:141-146"""
        return ProfiledGenerationStats(self, profile)

    def total_model_tokens(self) -> int:
        return int(N.lib.pg_generation_stats_total_model_tokens(C.byref(self.to_native())))

    def prefill_tokens_per_second(self) -> float:
        return float(N.lib.pg_generation_stats_prefill_tokens_per_second(C.byref(self.to_native())))

    def decode_tokens_per_second(self) -> float:
        return float(N.lib.pg_generation_stats_decode_tokens_per_second(C.byref(self.to_native())))

    def total_tokens_per_second(self) -> float:
        return float(N.lib.pg_generation_stats_total_tokens_per_second(C.byref(self.to_native())))

    def average_decode_token_time(self) -> Optional[float]:
        t = float(N.lib.pg_generation_stats_average_decode_token_time(C.byref(self.to_native())))
        return None if t < 0 else t


@dataclass
class ProfiledGenerationStats:
    """generation.rs:182-196: the common statistics with a model's own profile beside them."""
    common: GenerationStats
    profile: object

    def split(self):
        return self.common, self.profile


def argmax_logits(values: Sequence[float]) -> int:
    """generation.rs:269-279"""
    v = np.ascontiguousarray(values, np.float32)
    return int(N.lib.pg_argmax_logits(v.ctypes.data_as(C.POINTER(C.c_float)), v.size))


class LogitsSampler:
    """generation.rs:209-241"""

    def __init__(self, seed: int):
        self._h = C.c_void_p()
        check(N.lib.pg_sampler_new(seed, C.byref(self._h)))

    def __del__(self):
        if getattr(self, "_h", None):
            N.lib.pg_sampler_free(self._h)
            self._h = None

    def select_next_token(self, logits, history, config: TextGenerationConfig) -> int:
        v = np.ascontiguousarray(logits, np.float32)
        h = np.ascontiguousarray(history, np.uint64)
        g = config.to_native()
        out = C.c_uint64()
        check(N.lib.pg_sampler_select_next_token(self._h, v.ctypes.data_as(C.POINTER(C.c_float)), v.size,
                                                 h.ctypes.data_as(C.POINTER(C.c_uint64)), h.size, C.byref(g),
                                                 C.byref(out)))
        return int(out.value)

    def select_from_topk(self, vals, idx, config: TextGenerationConfig) -> int:
        v = np.ascontiguousarray(vals, np.float32)
        i = np.ascontiguousarray(idx, np.int32)
        g = config.to_native()
        out = C.c_uint64()
        check(N.lib.pg_sampler_select_from_topk(self._h, v.ctypes.data_as(C.POINTER(C.c_float)),
                                                i.ctypes.data_as(C.POINTER(C.c_int32)), v.size, C.byref(g),
                                                C.byref(out)))
        return int(out.value)

    @staticmethod
    def select_from_topk_batch(samplers, vals, idx, config: TextGenerationConfig) -> np.ndarray:
        """One draw per sampler from row i of the [batch, k] top-k arrays, in one native call."""
        v = np.ascontiguousarray(vals, np.float32)
        i = np.ascontiguousarray(idx, np.int32)
        n, k = v.shape
        if len(samplers) != n:
            raise ValueError("one sampler per row")
        handles = (C.c_void_p * n)(*[s_._h for s_ in samplers])
        g = config.to_native()
        out = np.empty(n, np.uint64)
        check(N.lib.pg_sampler_select_from_topk_batch(handles, v.ctypes.data_as(C.POINTER(C.c_float)),
                                                      i.ctypes.data_as(C.POINTER(C.c_int32)), n, k, C.byref(g),
                                                      out.ctypes.data_as(C.POINTER(C.c_uint64))))
        return out


__all__ = ["TextGenerationConfig", "GenerationStats", "LogitsSampler", "argmax_logits", "Gpt2Error",
           "gpt2_generation_config", "GPT2_EOS_TOKEN_ID"]
