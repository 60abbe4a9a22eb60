"""B200-native (sm_100a) GPT-2 inference path behind the puppygrad generation API.

`Gpt2Model`, `Gpt2KvCache`, `Gpt2Config`, `generate`, `TextGenerationConfig`, `LogitsSampler`
mirror the reference's Rust types of the same names; the compute runs in
`libpuppygrad_b200.so` (hand-written CUDA behind the C ABI of include/puppygrad_b200.h).
"""
from .autoregressive import generate
from .errors import Gpt2Error
from .generation import (GPT2_EOS_TOKEN_ID, GenerationStats, LogitsSampler, ProfiledGenerationStats,
                         TextGenerationConfig, argmax_logits, gpt2_generation_config)
from .gpt2 import Gpt2Config, Gpt2CudaConfig, Gpt2KvCache, Gpt2Model, Gpt2Output
from .runtime import (Gpt2AssetPaths, Gpt2GenerationStats, Gpt2OperationProfile, Gpt2Runtime, Gpt2Tokenizer,
                      write_raw_token_event)
from .streaming import IncrementalTextStreamer, escape_raw_token, is_incremental_decode_safe

__all__ = ["generate", "Gpt2Error", "GPT2_EOS_TOKEN_ID", "GenerationStats", "LogitsSampler",
           "TextGenerationConfig", "argmax_logits", "gpt2_generation_config", "Gpt2Config",
           "Gpt2CudaConfig", "Gpt2KvCache", "Gpt2Model", "Gpt2Output", "IncrementalTextStreamer", "escape_raw_token",
           "is_incremental_decode_safe", "Gpt2AssetPaths", "Gpt2GenerationStats", "Gpt2OperationProfile", "Gpt2Runtime",
           "Gpt2Tokenizer", "write_raw_token_event", "ProfiledGenerationStats"]
