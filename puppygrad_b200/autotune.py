"""Exhaustive tuning of this backend's knobs, after the reference's autotune harness.

`autotune` is the reference's generic loop (puppygrad src/models/autotune.rs:32-85): every candidate
configuration is evaluated, scored, and the best one kept together with all trials. The GPT-2 target
(src/main.rs:2588-2985 for the CPU backend's chunk sizes) here searches what the CUDA backend exposes:
KV page size, split-K factor of decode attention, and whether small-batch steps run as the single
persistent kernel. The score is the median decode tokens/s (`median_decode_tokens_per_second`, as in
main.rs:2927-2958). The result is saved next to the model as `puppygrad-b200-tune.json` and loaded by
`Gpt2Model.from_dir` when no configuration is passed (main.rs:2564-2585 does the same with
`puppygrad-tune.json`).

    python -m puppygrad_b200.autotune --model-dir DIR [--batch 1] [--prompt-len 32] [--new-tokens 64] [--no-save]
"""
from __future__ import annotations

import argparse
import itertools
import json
import os
import statistics
import sys
from dataclasses import asdict, dataclass, field
from typing import Any, Callable, Generic, List, Optional, TypeVar

TUNING_FILE = "puppygrad-b200-tune.json"
SCORE_NAME = "median_decode_tokens_per_second"

C = TypeVar("C")
M = TypeVar("M")


@dataclass
class AutoTuneOptions:
    """autotune.rs:1-17"""
    warmup_runs: int = 1
    measured_runs: int = 3
    max_trials: Optional[int] = None


@dataclass
class AutoTuneTrial(Generic[C, M]):
    config: C
    measurement: M
    score: float


@dataclass
class AutoTuneResult(Generic[C, M]):
    best_config: C
    best_score: float
    trials: List[AutoTuneTrial] = field(default_factory=list)


def autotune(target, options: AutoTuneOptions) -> AutoTuneResult:
    """autotune.rs:47-85. `target` has candidate_configs(), evaluate_config(config, options) and
    score(measurement); the first best score wins ties."""
    candidates = list(target.candidate_configs())
    if options.max_trials is not None:
        candidates = candidates[:options.max_trials]
    if not candidates:
        raise ValueError("autotune requires at least one candidate")
    trials, best_index, best_score = [], None, float("-inf")
    for config in candidates:
        measurement = target.evaluate_config(config, options)
        score = float(target.score(measurement))
        if score > best_score:
            best_score, best_index = score, len(trials)
        trials.append(AutoTuneTrial(config, measurement, score))
    return AutoTuneResult(trials[best_index].config, best_score, trials)


@dataclass
class DecodeMeasurement:
    decode_tokens_per_second: List[float]
    decode_tokens_per_second_median: float


class Gpt2CudaAutoTuneTarget:
    """Decode throughput of one model at one batch size over the backend's knobs."""

    def __init__(self, config, weights, prompts, new_tokens: int, base=None,
                 page_tokens=(16, 32, 64), attn_splits=(0, 1, 2, 4, 8), persistent_step=(None, True, False)):
        from .gpt2 import Gpt2CudaConfig
        self.config, self.weights, self.prompts, self.new_tokens = config, weights, prompts, new_tokens
        self.base = base or Gpt2CudaConfig()
        self.space = (page_tokens, attn_splits, persistent_step)

    def candidate_configs(self):
        from dataclasses import replace
        return [replace(self.base, page_tokens=p, attn_splits=s, persistent_step=k)
                for p, s, k in itertools.product(*self.space)]

    def evaluate_config(self, cuda_config, options: AutoTuneOptions) -> DecodeMeasurement:
        from .gpt2 import Gpt2Model
        model = Gpt2Model(self.config, self.weights, cuda_config)
        cache = model.new_kv_cache(max_batch=len(self.prompts))
        rates = []
        for run in range(options.warmup_runs + options.measured_runs):
            _, first = model.prefill_batch(self.prompts, cache)
            cache.time_begin()
            model.decode_greedy(first, cache, self.new_tokens)
            sec = cache.time_end()
            if run >= options.warmup_runs:
                rates.append(len(self.prompts) * self.new_tokens / sec)
        return DecodeMeasurement(rates, statistics.median(rates))

    def score(self, measurement: DecodeMeasurement) -> float:
        return measurement.decode_tokens_per_second_median


def tuning_path(model_dir: str) -> str:
    return os.path.join(model_dir, TUNING_FILE)


def save_tuning(path: str, result: AutoTuneResult, new_tokens: int, batch: int, options: AutoTuneOptions) -> None:
    """main.rs:2927-2958"""
    saved = {"model": "gpt2", "backend": "cuda", "score_name": SCORE_NAME, "score": result.best_score,
             "max_new_tokens": new_tokens, "batch": batch, "warmup_runs": options.warmup_runs,
             "measured_runs": options.measured_runs, "cuda": asdict(result.best_config),
             "trials": [{"cuda": asdict(t.config), "score": t.score} for t in result.trials]}
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "w") as f:
        f.write(json.dumps(saved, indent=2) + "\n")


def load_tuning(model_dir: str, tuning_file: Optional[str] = None):
    """main.rs:2564-2585: the named file must exist; the default file may be absent (then None)."""
    from .errors import Gpt2Error
    from .gpt2 import Gpt2CudaConfig
    path = tuning_file or tuning_path(model_dir)
    if not os.path.exists(path):
        if tuning_file:
            raise Gpt2Error("Asset", f"tuning file {path} does not exist")
        return None
    try:
        with open(path) as f:
            saved = json.load(f)
        cfg = Gpt2CudaConfig(**saved["cuda"])
        cfg.to_native()  # validates the names it carries
    except (OSError, ValueError, KeyError, TypeError) as exc:
        raise Gpt2Error("Asset", f"failed to parse tuning file {path}: {exc}") from exc
    print(f"loaded tuning config from {path}", file=sys.stderr)
    return cfg


def main(argv=None):
    from . import synthetic
    from .gpt2 import Gpt2Config
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model-dir", required=True, help="directory with config.json and model.safetensors")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--prompt-len", type=int, default=32)
    ap.add_argument("--new-tokens", type=int, default=64)
    ap.add_argument("--warmup-runs", type=int, default=1)
    ap.add_argument("--measured-runs", type=int, default=3)
    ap.add_argument("--max-trials", type=int, default=None)
    ap.add_argument("--no-save", action="store_true")
    a = ap.parse_args(argv)
    config = Gpt2Config.from_json(os.path.join(a.model_dir, "config.json"))
    weights = synthetic.read_safetensors(os.path.join(a.model_dir, "model.safetensors"))
    prompts = [synthetic.uniform_prompt(i + 1, a.prompt_len, config.vocab_size) for i in range(a.batch)]
    options = AutoTuneOptions(a.warmup_runs, a.measured_runs, a.max_trials)
    result = autotune(Gpt2CudaAutoTuneTarget(config, weights, prompts, a.new_tokens), options)
    for t in sorted(result.trials, key=lambda t: -t.score)[:10]:
        print(f"{t.score:12.1f} tokens/s  page_tokens={t.config.page_tokens} attn_splits={t.config.attn_splits} "
              f"persistent_step={t.config.persistent_step}")
    if not a.no_save:
        save_tuning(tuning_path(a.model_dir), result, a.new_tokens, a.batch, options)
        print("saved", tuning_path(a.model_dir))


if __name__ == "__main__":
    main()
