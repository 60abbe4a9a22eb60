"""CPU-only checks of the product library: it loads, exports every symbol the header declares,
and its host-side logic (config, safetensors, sampler, validation) matches the reference rules.
No compute entry point can succeed here: there is no CPU fallback."""
import ctypes as C
import json
import os
import re

import numpy as np
import pytest

import puppygrad_b200 as pg
from puppygrad_b200 import _native as N
from puppygrad_b200 import synthetic

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "puppygrad_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pg_[a-z0-9_]+)\s*\(", text)) - {"pg_token_callback"})


def test_library_exports_every_declared_symbol():
    names = declared_functions()
    assert len(names) >= 30
    lib = C.CDLL(N.LIB_PATH)
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in the header but not exported"
    assert sorted(N.SIGNATURES) == names


def test_version_and_device_count_do_not_need_a_gpu():
    assert b"sm_100a" in N.lib.pg_version()
    assert N.lib.pg_device_count() >= 0


def test_config_validation_messages():
    """rust.rs:59-94"""
    ok = pg.Gpt2Config(8, 5, 4, 1, 2)
    ok.validate()
    assert ok.n_inner == 16 and ok.head_dim() == 2
    for field, msg in [("vocab_size", "vocab_size must be > 0"), ("n_positions", "n_positions must be > 0"),
                       ("n_embd", "n_embd must be > 0"), ("n_layer", "n_layer must be > 0"),
                       ("n_head", "n_head must be > 0")]:
        c = pg.Gpt2Config(8, 5, 4, 1, 2)
        setattr(c, field, 0)
        with pytest.raises(pg.Gpt2Error, match=msg) as e:
            c.validate()
        assert e.value.kind == "InvalidConfig"
    with pytest.raises(pg.Gpt2Error, match="n_embd 6 must be divisible by n_head 4"):
        pg.Gpt2Config(8, 5, 6, 1, 4).validate()
    with pytest.raises(pg.Gpt2Error, match="layer_norm_epsilon must be > 0"):
        pg.Gpt2Config(8, 5, 4, 1, 2, layer_norm_epsilon=0.0).validate()


def test_config_json_loading(tmp_path):
    """rust.rs:684-711: n_ctx fallback, n_inner and epsilon defaults, missing keys."""
    p = tmp_path / "config.json"
    p.write_text(json.dumps({"vocab_size": 50257, "n_ctx": 1024, "n_embd": 768, "n_layer": 12, "n_head": 12,
                             "model_type": "gpt2", "nested": {"a": [1, 2, {"b": None}]}, "s": "q\\u00e9\\n"}))
    c = pg.Gpt2Config.from_json(p)
    assert (c.n_positions, c.n_inner, c.n_embd) == (1024, 3072, 768)
    assert abs(c.layer_norm_epsilon - 1e-5) < 1e-12
    p.write_text(json.dumps({"vocab_size": 10, "n_positions": 7, "n_ctx": 9, "n_embd": 8, "n_layer": 1,
                             "n_head": 2, "n_inner": 20, "layer_norm_epsilon": 1e-6}))
    c = pg.Gpt2Config.from_json(p)
    assert (c.n_positions, c.n_inner) == (7, 20) and abs(c.layer_norm_epsilon - 1e-6) < 1e-12
    p.write_text(json.dumps({"vocab_size": 10, "n_embd": 8, "n_layer": 1, "n_head": 2}))
    with pytest.raises(pg.Gpt2Error, match="config must contain n_positions or n_ctx") as e:
        pg.Gpt2Config.from_json(p)
    assert e.value.kind == "InvalidConfig"
    p.write_text(json.dumps({"n_positions": 4, "n_embd": 8, "n_layer": 1, "n_head": 2}))
    with pytest.raises(pg.Gpt2Error, match="vocab_size") as e:
        pg.Gpt2Config.from_json(p)
    assert e.value.kind == "Asset"
    p.write_text("{not json")
    with pytest.raises(pg.Gpt2Error) as e:
        pg.Gpt2Config.from_json(p)
    assert e.value.kind == "Asset"
    with pytest.raises(pg.Gpt2Error) as e:
        pg.Gpt2Config.from_json(tmp_path / "absent.json")
    assert e.value.kind == "Asset"


def test_weight_length_validation_precedes_any_device_work():
    """validate_weights, rust.rs:1279-1343 (the reference test asserts 'wte len', rust.rs:1872)."""
    cfg = synthetic.preset("tiny")
    w = synthetic.tiny_weights(cfg)
    w["wte.weight"] = w["wte.weight"].reshape(-1)[:-1]
    with pytest.raises(pg.Gpt2Error, match="wte len 31 does not match expected 32") as e:
        pg.Gpt2Model(cfg, w)
    assert e.value.kind == "InvalidWeights"
    w = synthetic.tiny_weights(cfg)
    w["h.0.mlp.c_fc.bias"] = np.zeros(3, np.float32)
    with pytest.raises(pg.Gpt2Error, match=r"blocks\[0\]\.c_fc_b len 3 does not match expected 8"):
        pg.Gpt2Model(cfg, w)
    flat = [w2 for w2 in synthetic.tiny_weights(cfg).values()]
    with pytest.raises(pg.Gpt2Error, match="blocks len 0 does not match n_layer 1"):
        pg.Gpt2Model(cfg, flat[:4])


def test_safetensors_loader_errors(tmp_path):
    """load_weights / tensor_f32, rust.rs:713-795; validate_tensor, safetensors.rs:149-170."""
    cfg = synthetic.preset("tiny")
    w = synthetic.tiny_weights(cfg)
    d = tmp_path / "m"
    with pytest.raises(pg.Gpt2Error) as e:
        pg.Gpt2Model.from_dir(d)
    assert e.value.kind == "Asset"
    synthetic.write_model_dir(str(d), cfg, w)
    os.remove(d / "model.safetensors")
    with pytest.raises(pg.Gpt2Error, match="model.safetensors") as e:
        pg.Gpt2Model.from_dir(d)
    assert e.value.kind == "Asset"
    bad = dict(w)
    bad["h.0.attn.c_attn.weight"] = bad["h.0.attn.c_attn.weight"].T.copy()
    synthetic.write_model_dir(str(d), cfg, bad)
    with pytest.raises(pg.Gpt2Error, match=r"tensor h\.0\.attn\.c_attn\.weight shape \[12, 4\] does not match expected \[4, 12\]") as e:
        pg.Gpt2Model.from_dir(d)
    assert e.value.kind == "InvalidWeights"
    missing = {k: v for k, v in w.items() if k != "ln_f.bias"}
    synthetic.write_model_dir(str(d), cfg, missing)
    with pytest.raises(pg.Gpt2Error, match="transformer.ln_f.bias") as e:
        pg.Gpt2Model.from_dir(d)
    assert e.value.kind == "Asset"
    # F32 only (safetensors.rs:126-130)
    synthetic.write_model_dir(str(d), cfg, w)
    path = d / "model.safetensors"
    raw = path.read_bytes()
    n = int.from_bytes(raw[:8], "little")
    hdr = raw[8:8 + n].replace(b'"wpe.weight":{"dtype":"F32"', b'"wpe.weight":{"dtype":"I32"')
    path.write_bytes(raw[:8] + hdr + raw[8 + n:])
    with pytest.raises(pg.Gpt2Error, match="dtype I32") as e:
        pg.Gpt2Model.from_dir(d)
    assert e.value.kind == "Asset"
    path.write_bytes(raw[:20])
    with pytest.raises(pg.Gpt2Error) as e:
        pg.Gpt2Model.from_dir(d)
    assert e.value.kind == "Asset"


def test_no_cpu_fallback(tmp_path):
    """A valid model on a machine without an sm_100 device must fail loudly, not compute."""
    if N.lib.pg_device_count() > 0:
        pytest.skip("a CUDA device is present")
    cfg = synthetic.preset("tiny")
    with pytest.raises(pg.Gpt2Error) as e:
        pg.Gpt2Model(cfg, synthetic.tiny_weights(cfg))
    assert e.value.kind == "Cuda"
    d = synthetic.write_model_dir(str(tmp_path / "ok"), cfg, synthetic.tiny_weights(cfg), prefix="transformer.")
    with pytest.raises(pg.Gpt2Error) as e:
        pg.Gpt2Model.from_dir(d)
    assert e.value.kind == "Cuda"


def test_backend_config_validation():
    cfg = synthetic.preset("tiny")
    w = synthetic.tiny_weights(cfg)
    with pytest.raises(pg.Gpt2Error, match="page_tokens"):
        pg.Gpt2Model(cfg, w, pg.Gpt2CudaConfig(page_tokens=7))
    with pytest.raises(pg.Gpt2Error, match="math_mode"):
        pg.Gpt2Model(cfg, w, pg.Gpt2CudaConfig(math_mode="int4"))


# ---- sampler: the product's host code against the reference's tests and the oracle
def test_reference_sampler_tests():
    """generation.rs:364-404"""
    g = pg.TextGenerationConfig(1, repeat_penalty=2.0)
    assert pg.LogitsSampler(g.seed).select_next_token([1.0, 3.0, 2.0], [1], g) == 2
    g = pg.TextGenerationConfig(1, temperature=1.0, top_k=1)
    assert pg.LogitsSampler(g.seed).select_next_token([0.0, 10.0, 9.0], [], g) == 1
    with pytest.raises(pg.Gpt2Error):
        pg.TextGenerationConfig(1, top_p=2.0).validate()
    with pytest.raises(pg.Gpt2Error, match="top_k must be > 0"):
        pg.TextGenerationConfig(1, top_k=0).validate()
    pg.TextGenerationConfig(1).validate()
    assert pg.gpt2_generation_config(5).eos_token_id == 50256


@pytest.mark.parametrize("kw", [dict(temperature=0.8, top_k=40), dict(temperature=1.3),
                                dict(temperature=0.7, top_p=0.9), dict(temperature=1.0, top_k=50, top_p=0.5),
                                dict(temperature=0.9, top_k=40, repeat_penalty=1.3, repeat_last_n=4),
                                dict(repeat_penalty=1.5)])
def test_sampler_matches_oracle_draw_for_draw(oracle, kw):
    rng = np.random.default_rng(7)
    cfg = pg.TextGenerationConfig(1, seed=4242, **kw)
    og = oracle.generation_config(1, seed=4242, **kw)
    a, b = pg.LogitsSampler(cfg.seed), oracle.LogitsSampler(og.seed)
    history = []
    for step in range(60):
        logits = rng.standard_normal(500).astype(np.float32) * 3
        logits[rng.integers(0, 500, 5)] = logits[3]  # ties
        if step % 7 == 0:
            logits[rng.integers(0, 500, 3)] = np.float32("nan")
            logits[11] = np.float32("-inf")
        ta = a.select_next_token(logits, history, cfg)
        tb = b.select_next_token(logits, history, og)
        assert ta == tb
        history.append(ta)


def test_topk_shortcut_equals_full_sampler(oracle):
    rng = np.random.default_rng(9)
    cfg = pg.TextGenerationConfig(1, temperature=0.8, top_k=40, seed=99)
    a, b = pg.LogitsSampler(cfg.seed), pg.LogitsSampler(cfg.seed)
    for _ in range(40):
        logits = rng.standard_normal(3000).astype(np.float32)
        logits[100] = logits[200] = logits.max()  # tie at the top: lower index first
        order = sorted(range(3000), key=lambda i: (-float(logits[i]), i))[:40]
        vals = logits[order]
        assert a.select_from_topk(vals, order, cfg) == b.select_next_token(logits, [], cfg)


def test_argmax_rule():
    assert pg.argmax_logits([1.0, 5.0, 5.0, 2.0]) == 1
    assert pg.argmax_logits([float("nan"), 1.0, float("nan")]) == 1
    assert pg.argmax_logits([float("-inf")] * 3) == 0


def test_generation_stats_report_token_rates():
    """rust.rs:2037-2059"""
    s = pg.GenerationStats(4, 6, 0.005, 0.020, 0.030, 0.050, 0.022)
    assert s.total_model_tokens() == 10
    assert s.prefill_tokens_per_second() == pytest.approx(200.0)
    assert s.decode_tokens_per_second() == pytest.approx(200.0)
    assert s.total_tokens_per_second() == pytest.approx(200.0)
    assert s.average_decode_token_time() == pytest.approx(0.005)
    assert pg.GenerationStats().decode_tokens_per_second() == 0.0


# ------------------------------------------------------------------ text streaming (streaming.rs:80-146) and stats
class MockDecoder:
    """streaming.rs:84-100"""

    def decode_tokens(self, token_ids):
        return "".join({0: "hello", 1: " world", 2: ""}.get(t, "�") for t in token_ids)


def test_streams_safe_token_text_incrementally():
    from puppygrad_b200.streaming import IncrementalTextStreamer
    s = IncrementalTextStreamer("hello")
    chunks = []
    s.stream_token(MockDecoder(), [0, 1], 1, chunks.append)
    assert chunks == [" world"] and s.decoded() == "hello world"


def test_falls_back_to_full_decode_for_unsafe_token_text():
    from puppygrad_b200.streaming import IncrementalTextStreamer
    s = IncrementalTextStreamer("hello")
    chunks = []
    s.stream_token(MockDecoder(), [0, 1, 2], 2, chunks.append)
    assert chunks == [" world"] and s.decoded() == "hello world"
    # a decode that does not extend what was streamed emits the token's own text (streaming.rs:66-70)
    s2 = IncrementalTextStreamer("other")
    chunks = []
    s2.stream_token(MockDecoder(), [0, 3], 3, chunks.append)
    assert chunks == ["�"] and s2.decoded() == "hello�"
    # long texts take the decoder's second call with a larger buffer
    class Long:
        def decode_tokens(self, ids):
            return "x" * 1000 * len(ids)
    s3 = IncrementalTextStreamer("")
    chunks = []
    s3.stream_token(Long(), [7], 7, chunks.append)
    assert chunks == ["x" * 1000] and s3.decoded() == "x" * 1000
    # errors of the decoder and of the text callback come back to the caller
    class Broken:
        def decode_tokens(self, ids):
            raise KeyError("no such token")
    with pytest.raises(KeyError):
        IncrementalTextStreamer("").stream_token(Broken(), [1], 1, chunks.append)


def test_incremental_decode_rejects_empty_and_replacement_text():
    from puppygrad_b200.streaming import is_incremental_decode_safe
    assert is_incremental_decode_safe(" hello")
    assert not is_incremental_decode_safe("")
    assert not is_incremental_decode_safe("�")
    assert not is_incremental_decode_safe("a�")


def test_escapes_raw_tokens_for_line_streams():
    from puppygrad_b200.streaming import escape_raw_token
    assert escape_raw_token("<|en|>") == "<|en|>"
    assert escape_raw_token("ĠI") == "ĠI"
    assert escape_raw_token("a\tb\nc") == "a\\tb\\nc"
    assert escape_raw_token("back\\slash\r") == "back\\\\slash\\r"
    assert escape_raw_token("\x01\x7f\u0085é😀") == "\\u{1}\\u{7f}\\u{85}é😀"


def test_generation_stats_rates():
    """generation.rs:129-181"""
    s = pg.GenerationStats(prompt_tokens=10, generated_tokens=5, prefill_time=2.0, decode_time=0.5, total_generation_time=3.0)
    assert s.total_model_tokens() == 15
    assert s.prefill_tokens_per_second() == 5.0 and s.decode_tokens_per_second() == 10.0
    assert s.total_tokens_per_second() == 5.0 and s.average_decode_token_time() == 0.1
    z = pg.GenerationStats()
    assert z.decode_tokens_per_second() == 0.0 and z.average_decode_token_time() is None


def test_struct_layouts_of_the_binding_match_the_header(tmp_path):
    """The ctypes structures (and with them the `#[repr(C)]` structs of the Rust binding, which list the
    same fields in the same order and types) are pinned to the header: a C program compiled against
    include/puppygrad_b200.h prints the size and every field offset of each struct."""
    import shutil
    import subprocess
    if shutil.which("gcc") is None:
        pytest.skip("no C compiler")
    structs = {
        "pg_gpt2_config": N.PgConfig, "pg_backend_config": N.PgBackendConfig,
        "pg_generation_config": N.PgGenerationConfig, "pg_generation_stats": N.PgGenerationStats,
        "pg_operation_profile": N.PgOperationProfile,
    }
    lines = ['#include <stddef.h>', '#include <stdio.h>', '#include "puppygrad_b200.h"', "int main(void) {"]
    for cname, st in structs.items():
        lines.append(f'  printf("{cname} size %zu\\n", sizeof({cname}));')
        for field, _ in st._fields_:
            lines.append(f'  printf("{cname} {field} %zu\\n", offsetof({cname}, {field}));')
    lines += ["  return 0;", "}"]
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    include = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include")
    subprocess.run(["gcc", "-std=c11", "-I", include, str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split("\n")
    seen = 0
    for line in out:
        if not line:
            continue
        cname, field, value = line.split()
        st = structs[cname]
        if field == "size":
            assert C.sizeof(st) == int(value), cname
        else:
            assert getattr(st, field).offset == int(value), (cname, field)
        seen += 1
    assert seen == sum(len(st._fields_) + 1 for st in structs.values())


def test_batch_draw_from_topk_rows_equals_one_call_per_sampler():
    """pg_sampler_select_from_topk_batch: sampler i draws from row i exactly as a call of its own would
    (sample_logits over a pre-sorted top-k list, src/models/generation.rs:300-362), one RNG draw each."""
    from puppygrad_b200.generation import LogitsSampler
    rng = np.random.default_rng(3)
    n, k = 7, 40
    vals = -np.sort(-rng.standard_normal((n, k)).astype(np.float32), axis=1)
    idx = np.stack([rng.permutation(5000)[:k] for _ in range(n)]).astype(np.int32)
    conf = pg.TextGenerationConfig(4, temperature=0.8, top_k=40, seed=11)
    a = [LogitsSampler(100 + i) for i in range(n)]
    b = [LogitsSampler(100 + i) for i in range(n)]
    for _ in range(5):
        want = [a[i].select_from_topk(vals[i], idx[i], conf) for i in range(n)]
        got = LogitsSampler.select_from_topk_batch(b, vals, idx, conf)
        assert [int(t) for t in got] == want
    with pytest.raises(ValueError):
        LogitsSampler.select_from_topk_batch(b[:3], vals, idx, conf)
