"""The tuning harness (reference: src/models/autotune.rs:32-85, tuning file of src/main.rs:2564-2585, 2927-2958)."""
import json
import os

import pytest

import puppygrad_b200 as pg
from puppygrad_b200 import autotune, synthetic


class FakeTarget:
    def __init__(self, scores):
        self.scores, self.seen = scores, []

    def candidate_configs(self):
        return list(range(len(self.scores)))

    def evaluate_config(self, config, options):
        self.seen.append(config)
        return {"tps": self.scores[config], "runs": options.measured_runs}

    def score(self, m):
        return m["tps"]


def test_autotune_keeps_the_first_best_candidate_and_every_trial():
    t = FakeTarget([3.0, 9.0, 9.0, 1.0])
    r = autotune.autotune(t, autotune.AutoTuneOptions())
    assert r.best_config == 1 and r.best_score == 9.0 and [x.score for x in r.trials] == [3.0, 9.0, 9.0, 1.0]
    assert r.trials[0].measurement["runs"] == 3
    t = FakeTarget([3.0, 9.0, 9.0, 1.0])
    r = autotune.autotune(t, autotune.AutoTuneOptions(max_trials=1))
    assert r.best_config == 0 and t.seen == [0]
    with pytest.raises(ValueError):
        autotune.autotune(FakeTarget([]), autotune.AutoTuneOptions())


def test_tuning_file_round_trip(tmp_path):
    best = pg.Gpt2CudaConfig(page_tokens=64, attn_splits=4, persistent_step=True)
    result = autotune.AutoTuneResult(best, 123.0, [autotune.AutoTuneTrial(best, None, 123.0)])
    path = autotune.tuning_path(str(tmp_path))
    autotune.save_tuning(path, result, 64, 1, autotune.AutoTuneOptions())
    saved = json.load(open(path))
    assert saved["backend"] == "cuda" and saved["score_name"] == "median_decode_tokens_per_second" and saved["score"] == 123.0
    assert autotune.load_tuning(str(tmp_path)) == best
    assert autotune.load_tuning(str(tmp_path / "nowhere")) is None  # the default file may be absent
    with pytest.raises(pg.Gpt2Error, match="does not exist"):
        autotune.load_tuning(str(tmp_path), str(tmp_path / "missing.json"))
    open(path, "w").write("{ not json")
    with pytest.raises(pg.Gpt2Error, match="failed to parse tuning file"):
        autotune.load_tuning(str(tmp_path))


def test_safetensors_reader_round_trip(tmp_path):
    cfg = synthetic.preset("tiny")
    w = synthetic.tiny_weights(cfg)
    synthetic.write_model_dir(str(tmp_path), cfg, w, prefix="transformer.")
    back = synthetic.read_safetensors(os.path.join(str(tmp_path), "model.safetensors"))
    assert set(back) == set(w) and all((back[k] == w[k]).all() for k in w)


@pytest.mark.gpu
def test_autotune_on_a_small_model_saves_a_configuration_that_from_dir_loads(tmp_path, oracle):
    cfg = synthetic.preset("midi")
    w = synthetic.perturbed_weights(cfg, 61)
    synthetic.write_model_dir(str(tmp_path), cfg, w)
    prompts = [synthetic.uniform_prompt(70, 40, cfg["vocab_size"])]
    target = autotune.Gpt2CudaAutoTuneTarget(cfg, w, prompts, 16, page_tokens=(16, 64), attn_splits=(0, 2),
                                             persistent_step=(True, False))
    options = autotune.AutoTuneOptions(warmup_runs=1, measured_runs=2)
    result = autotune.autotune(target, options)
    assert len(result.trials) == 8 and result.best_score == max(t.score for t in result.trials) > 0
    autotune.save_tuning(autotune.tuning_path(str(tmp_path)), result, 16, 1, options)
    model = pg.Gpt2Model.from_dir(str(tmp_path))
    assert model.cuda_config == result.best_config
    want = oracle.Model(cfg, w, threads=4).generate_greedy_cached(prompts[0], 8)
    assert model.generate_greedy_cached(prompts[0], 8) == want
    assert pg.Gpt2Model.from_dir(str(tmp_path), use_tuning=False).cuda_config == pg.Gpt2CudaConfig()
