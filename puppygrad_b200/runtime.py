"""Text-level runtime of the GPT-2 path: prompt text in, generated text (or raw tokens) out.

Mirrors `Gpt2Tokenizer`, `Gpt2Runtime`, `Gpt2OperationProfile` and `Gpt2GenerationStats`
(puppygrad src/models/gpt2/rust.rs:269-653), `Gpt2AssetPaths` (src/models/gpt2/assets.rs:12-30) and the
output of `run-gpt2` (src/main.rs:1305-1388, 2462-2485, 3169-3261).

The reference reads `tokenizer.json` with the `tokenizers` crate; this module uses the same library through
its Python package, so text <-> ids is the reference's own code. Everything between the ids is the CUDA
library: prefill, decode steps and sampling run in `pg_generate_with_config`, and the callback it calls per
token does the incremental text decoding here.

    python -m puppygrad_b200.run_gpt2 --model-dir DIR --prompt "..." [--max-new-tokens N] [--stats]
                                      [--stream-raw-tokens] [--temperature T --top-k K --top-p P --seed S]
"""
from __future__ import annotations

import argparse
import os
import sys
import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence, TextIO, Tuple

from .errors import Gpt2Error
from .generation import GenerationStats, ProfiledGenerationStats, TextGenerationConfig, gpt2_generation_config
from .gpt2 import Gpt2CudaConfig, Gpt2Model
from .streaming import IncrementalTextStreamer, escape_raw_token


@dataclass(frozen=True)
class Gpt2AssetPaths:
    """assets.rs:12-30: the three files of a Hugging Face GPT-2 directory."""
    model_dir: str
    config: str
    tokenizer: str
    weights: str

    @classmethod
    def new(cls, model_dir: str) -> "Gpt2AssetPaths":
        d = str(model_dir)
        return cls(d, os.path.join(d, "config.json"), os.path.join(d, "tokenizer.json"),
                   os.path.join(d, "model.safetensors"))


class Gpt2Tokenizer:
    """rust.rs:269-323. Also a `TokenDecoder` and a `RawTokenDecoder` (streaming.rs:1-15)."""

    def __init__(self, tokenizer):
        self._tok = tokenizer

    @classmethod
    def from_file(cls, path: str) -> "Gpt2Tokenizer":
        try:
            from tokenizers import Tokenizer
            return cls(Tokenizer.from_file(str(path)))
        except Exception as err:  # missing package, missing file, malformed JSON
            raise Gpt2Error("Asset", f"failed to load tokenizer {path}: {err}") from err

    def encode(self, text: str) -> List[int]:
        try:
            return [int(i) for i in self._tok.encode(text, add_special_tokens=True).ids]
        except Exception as err:
            raise Gpt2Error("Asset", f"failed to encode prompt: {err}") from err

    def decode(self, token_ids: Sequence[int]) -> str:
        ids = [int(t) for t in token_ids]
        if any(t < 0 or t > 0xFFFFFFFF for t in ids):
            raise Gpt2Error("InvalidInput", "token id does not fit in u32")
        try:
            return self._tok.decode(ids, skip_special_tokens=True)
        except Exception as err:
            raise Gpt2Error("Asset", f"failed to decode tokens: {err}") from err

    def decode_tokens(self, token_ids: Sequence[int]) -> str:
        return self.decode(token_ids)

    def decode_token(self, token_id: int) -> str:
        return self.decode([token_id])

    def raw_token(self, token_id: int) -> str:
        t = int(token_id)
        if t < 0 or t > 0xFFFFFFFF:
            raise Gpt2Error("InvalidInput", "token id does not fit in u32")
        token = self._tok.id_to_token(t)
        if token is None:
            raise Gpt2Error("InvalidInput", f"unknown token id {t}")
        return token


@dataclass
class Gpt2OperationProfile:
    """rust.rs:335-347, in seconds. `tokenization` and `decoding` (token ids -> text while streaming) are
    measured here. The per-operation times of the model are left at zero by the generation calls: on the
    device a decode step is one kernel, and `Gpt2Model.profile_forward_one` is the call that times its
    operation classes."""
    tokenization: float = 0.0
    layer_norm: float = 0.0
    qkv_projection: float = 0.0
    attention: float = 0.0
    attention_projection: float = 0.0
    mlp_fc_projection: float = 0.0
    mlp_projection: float = 0.0
    final_logits: float = 0.0
    decoding: float = 0.0


@dataclass
class Gpt2GenerationStats:
    """rust.rs:329-374: the common statistics plus the operation profile; attributes of `common` read through."""
    common: GenerationStats = field(default_factory=GenerationStats)
    operation_profile: Gpt2OperationProfile = field(default_factory=Gpt2OperationProfile)

    @classmethod
    def new(cls, common: GenerationStats, operation_profile: Gpt2OperationProfile) -> "Gpt2GenerationStats":
        common, operation_profile = common.with_profile(operation_profile).split()
        return cls(common, operation_profile)

    def as_profiled(self) -> ProfiledGenerationStats:
        return ProfiledGenerationStats(self.common, self.operation_profile)

    def __getattr__(self, name):  # Deref<Target = GenerationStats>
        return getattr(object.__getattribute__(self, "common"), name)


class Gpt2Runtime:
    """rust.rs:324-327, 377-635."""

    def __init__(self, model: Gpt2Model, tokenizer: Gpt2Tokenizer):
        self.model = model
        self.tokenizer = tokenizer

    @classmethod
    def from_dir(cls, model_dir: str) -> "Gpt2Runtime":
        return cls.from_dir_with_backend(model_dir, None)

    @classmethod
    def from_dir_with_backend(cls, model_dir: str, backend: Optional[Gpt2CudaConfig], use_tuning: bool = True,
                              tuning_file: Optional[str] = None) -> "Gpt2Runtime":
        paths = Gpt2AssetPaths.new(model_dir)
        model = Gpt2Model.from_dir(paths.model_dir, backend, use_tuning=use_tuning, tuning_file=tuning_file)
        return cls(model, Gpt2Tokenizer.from_file(paths.tokenizer))

    def generate_greedy_text(self, prompt: str, max_new_tokens: int) -> str:
        input_ids = self.tokenizer.encode(prompt)
        return self.tokenizer.decode(self.model.generate_greedy_cached(input_ids, max_new_tokens))

    def stream_greedy_text(self, prompt: str, max_new_tokens: int, on_text: Callable[[str], None]) -> str:
        """rust.rs:406-432: the decoded prompt first, then one piece of text per generated token."""
        input_ids = self.tokenizer.encode(prompt)
        output_ids = list(input_ids)
        streamer = IncrementalTextStreamer(self.tokenizer.decode(output_ids))
        on_text(streamer.decoded())
        failure: List[BaseException] = []

        def on_token(token_id: int) -> bool:
            output_ids.append(token_id)
            try:
                streamer.stream_token(self.tokenizer, output_ids, token_id, on_text)
            except BaseException as exc:  # the closure's error ends the generation and is raised below
                failure.append(exc)
                return True
            return False

        self._run(failure, self.model.stream_greedy_tokens, input_ids, max_new_tokens, on_token)
        return streamer.decoded()

    def stream_greedy_text_with_stats(self, prompt: str, max_new_tokens: int, on_text: Callable[[str], None]
                                      ) -> Tuple[str, Gpt2GenerationStats]:
        return self.stream_text_with_stats(prompt, gpt2_generation_config(max_new_tokens), on_text)

    @staticmethod
    def _run(failure: List[BaseException], call, *args):
        """A callback that raised has stopped the generation (the library reports an aborted callback): what the
        caller sees is the callback's own exception, as the closure's error is in the reference."""
        try:
            result = call(*args)
        except Gpt2Error:
            if failure:
                raise failure[0]
            raise
        if failure:
            raise failure[0]
        return result

    def _check_generation(self, generation: TextGenerationConfig) -> None:
        generation.validate()
        eos, v = generation.eos_token_id, self.model.config.vocab_size
        if eos is not None and eos >= v:
            raise Gpt2Error("InvalidConfig", f"generation eos_token_id {eos} is outside vocab_size {v}")

    def stream_text_with_stats(self, prompt: str, generation: TextGenerationConfig, on_text: Callable[[str], None]
                               ) -> Tuple[str, Gpt2GenerationStats]:
        """rust.rs:446-546."""
        self._check_generation(generation)
        profile = Gpt2OperationProfile()
        t0 = time.perf_counter()
        input_ids = self.tokenizer.encode(prompt)
        tokenize_time = time.perf_counter() - t0
        profile.tokenization += tokenize_time
        output_ids = list(input_ids)
        t0 = time.perf_counter()
        decoded = self.tokenizer.decode(output_ids)
        profile.decoding += time.perf_counter() - t0
        streamer = IncrementalTextStreamer(decoded)
        on_text(streamer.decoded())
        failure: List[BaseException] = []

        def on_token(token_id: int) -> bool:
            output_ids.append(token_id)
            t = time.perf_counter()
            try:
                streamer.stream_token(self.tokenizer, output_ids, token_id, on_text)
            except BaseException as exc:
                failure.append(exc)
                return True
            finally:
                profile.decoding += time.perf_counter() - t
            return False

        _, common = self._run(failure, self.model.generate_with_config, input_ids, generation, on_token)
        common.tokenize_time = tokenize_time
        return streamer.decoded(), Gpt2GenerationStats(common, profile)

    def stream_token_ids_with_stats(self, prompt: str, generation: TextGenerationConfig,
                                    on_token: Callable[[int], None]) -> Tuple[List[int], Gpt2GenerationStats]:
        """rust.rs:548-635: returns prompt ids + generated ids."""
        self._check_generation(generation)
        profile = Gpt2OperationProfile()
        t0 = time.perf_counter()
        input_ids = self.tokenizer.encode(prompt)
        tokenize_time = time.perf_counter() - t0
        profile.tokenization += tokenize_time
        failure: List[BaseException] = []

        def relay(token_id: int) -> bool:
            try:
                on_token(token_id)
            except BaseException as exc:
                failure.append(exc)
                return True
            return False

        generated, common = self._run(failure, self.model.generate_with_config, input_ids, generation, relay)
        common.tokenize_time = tokenize_time
        return list(input_ids) + generated, Gpt2GenerationStats(common, profile)


# ------------------------------------------------------------------ what run-gpt2 prints
def write_raw_token_event(writer: TextIO, segment_index: Optional[int], phase: str, token_id: int, decoder) -> None:
    """main.rs:2462-2485: `[segment TAB] phase TAB id TAB escaped token`."""
    token = escape_raw_token(decoder.raw_token(token_id))
    if segment_index is not None:
        writer.write(f"{segment_index}\t{phase}\t{token_id}\t{token}\n")
    else:
        writer.write(f"{phase}\t{token_id}\t{token}\n")


def format_duration(seconds: float) -> str:
    """main.rs:3250-3261"""
    if seconds >= 1.0:
        return f"{seconds:.3f}s"
    if seconds * 1e3 >= 1.0:
        return f"{seconds * 1e3:.2f}ms"
    return f"{seconds * 1e6:.2f}us"


def format_gpt2_speed(stats: Gpt2GenerationStats) -> str:
    """main.rs:3169-3175"""
    return f"\ntokens/sec: {stats.decode_tokens_per_second():.2f} tok/s ({stats.generated_tokens} generated tokens)"


def format_gpt2_stats(load_time: float, stats: Gpt2GenerationStats) -> str:
    """main.rs:3177-3248"""
    p = stats.operation_profile
    lines = ["", "stats:", f"  load: {format_duration(load_time)}", f"  tokenize: {format_duration(stats.tokenize_time)}",
             f"  prefill: {format_duration(stats.prefill_time)} ({stats.prompt_tokens} prompt tokens, "
             f"{stats.prefill_tokens_per_second():.2f} tok/s)"]
    if stats.first_token_time is not None:
        lines.append(f"  time to first token: {format_duration(stats.first_token_time)}")
    lines.append(f"  decode: {format_duration(stats.decode_time)} ({stats.generated_tokens} generated tokens, "
                 f"{stats.decode_tokens_per_second():.2f} tok/s)")
    avg = stats.average_decode_token_time()
    if avg is not None:
        lines.append(f"  avg decode token: {format_duration(avg)}")
    lines.append(f"  generation total: {format_duration(stats.total_generation_time)} ({stats.total_model_tokens()} "
                 f"model tokens, {stats.total_tokens_per_second():.2f} tok/s)")
    lines.append("  profile:")
    for label, value in (("layernorm", p.layer_norm), ("qkv projection", p.qkv_projection), ("attention", p.attention),
                         ("attention projection", p.attention_projection), ("mlp fc projection", p.mlp_fc_projection),
                         ("mlp projection", p.mlp_projection), ("final logits", p.final_logits),
                         ("tokenization", p.tokenization), ("decoding", p.decoding)):
        lines.append(f"    {label}: {format_duration(value)}")
    return "\n".join(lines)


def run_gpt2(argv: Optional[Sequence[str]] = None, stdout: TextIO = sys.stdout, stderr: TextIO = sys.stderr) -> int:
    """The generation part of `run-gpt2` (main.rs:1305-1388): no download, the model directory must exist."""
    ap = argparse.ArgumentParser(prog="python -m puppygrad_b200.run_gpt2")
    ap.add_argument("--model-dir", required=True)
    ap.add_argument("--prompt", required=True)
    ap.add_argument("--max-new-tokens", type=int, default=32)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-p", type=float, default=None)
    ap.add_argument("--top-k", type=int, default=None)
    ap.add_argument("--seed", type=int, default=299_792_458)
    ap.add_argument("--repeat-penalty", type=float, default=1.0)
    ap.add_argument("--repeat-last-n", type=int, default=128)
    ap.add_argument("--eos-token-id", type=int, default=None)
    ap.add_argument("--no-eos-stop", action="store_true")
    ap.add_argument("--stream-raw-tokens", action="store_true")
    ap.add_argument("--stats", action="store_true")
    ap.add_argument("--no-tuning", action="store_true")
    ap.add_argument("--tuning-file", default=None)
    ap.add_argument("--math-mode", default=None, help="fp32, tf32x3, tf32 or bf16 (default: the tuning file's, else fp32)")
    ap.add_argument("--quantized-weights", action="store_true")
    a = ap.parse_args(argv)
    generation = gpt2_generation_config(a.max_new_tokens)
    generation.temperature, generation.top_p, generation.top_k = a.temperature, a.top_p, a.top_k
    generation.seed, generation.repeat_penalty, generation.repeat_last_n = a.seed, a.repeat_penalty, a.repeat_last_n
    if a.no_eos_stop:
        generation.eos_token_id = None
    elif a.eos_token_id is not None:
        generation.eos_token_id = a.eos_token_id
    generation.validate()
    backend = None
    if a.math_mode is not None or a.quantized_weights:
        backend = Gpt2CudaConfig(math_mode=a.math_mode or "fp32", quantized_weights=a.quantized_weights)
    stderr.write(f"loading GPT-2 from {a.model_dir}\n")
    t0 = time.perf_counter()
    runtime = Gpt2Runtime.from_dir_with_backend(a.model_dir, backend, use_tuning=not a.no_tuning, tuning_file=a.tuning_file)
    load_time = time.perf_counter() - t0
    used = getattr(runtime.model, "cuda_config", None)  # the tuning file's when no backend was given
    stderr.write(f"backend: {used.describe() if used is not None else 'cuda'}\n")
    if a.stream_raw_tokens:
        for token_id in runtime.tokenizer.encode(a.prompt):
            write_raw_token_event(stdout, None, "prompt", token_id, runtime.tokenizer)
        stdout.flush()

        def on_token(token_id: int) -> None:
            write_raw_token_event(stdout, None, "generated", token_id, runtime.tokenizer)
            stdout.flush()

        _, stats = runtime.stream_token_ids_with_stats(a.prompt, generation, on_token)
    else:
        def on_text(text: str) -> None:
            stdout.write(text)
            stdout.flush()

        _, stats = runtime.stream_text_with_stats(a.prompt, generation, on_text)
        stdout.write("\n")
    stdout.flush()
    stderr.write((format_gpt2_stats(load_time, stats) if a.stats else format_gpt2_speed(stats)) + "\n")
    return 0
