"""Text-level runtime (Gpt2Tokenizer, Gpt2Runtime, raw-token events, the statistics printout): host logic on the
CPU with a small byte-level BPE tokenizer made here and a stand-in for the model; one GPU test end to end.

puppygrad src/models/gpt2/rust.rs:269-653, src/models/streaming.rs, src/main.rs:1305-1388, 2462-2485, 3169-3261.
"""
import io

import pytest

import puppygrad_b200 as pg
from puppygrad_b200 import runtime as rt
from puppygrad_b200 import synthetic

tokenizers = pytest.importorskip("tokenizers")

CORPUS = ["the quick brown fox jumps over the lazy dog", "a naïve café in Zürich — déjà vu", "日本語のテキスト 日本",
          "emoji 🙂🙂 and tabs\tand\nnewlines", "hello world hello there", "tokens and more tokens"] * 4


def make_tokenizer_json(path, vocab_size=320):
    """A GPT-2 style tokenizer: byte-level pre-tokenizer and decoder, BPE merges learnt from a few lines."""
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers
    tok = Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = decoders.ByteLevel()
    trainer = trainers.BpeTrainer(vocab_size=vocab_size, special_tokens=["<|endoftext|>"],
                                  initial_alphabet=pre_tokenizers.ByteLevel.alphabet(), show_progress=False)
    tok.train_from_iterator(CORPUS, trainer)
    tok.save(str(path))
    return tok.get_vocab_size()


@pytest.fixture(scope="module")
def tok_path(tmp_path_factory):
    p = tmp_path_factory.mktemp("tok") / "tokenizer.json"
    make_tokenizer_json(p)
    return str(p)


@pytest.fixture(scope="module")
def tokenizer(tok_path):
    return pg.Gpt2Tokenizer.from_file(tok_path)


def test_asset_paths():
    p = pg.Gpt2AssetPaths.new("/models/gpt2")
    assert (p.model_dir, p.config, p.tokenizer, p.weights) == (
        "/models/gpt2", "/models/gpt2/config.json", "/models/gpt2/tokenizer.json", "/models/gpt2/model.safetensors")


def test_tokenizer_round_trip_and_raw_tokens(tokenizer):
    text = "the quick café 日本 🙂"
    ids = tokenizer.encode(text)
    assert ids and all(isinstance(i, int) for i in ids)
    assert tokenizer.decode(ids) == text
    assert tokenizer.decode_tokens(ids) == text
    assert tokenizer.decode_token(ids[0]) == tokenizer.decode(ids[:1])
    # the end-of-text token is special: decode skips it (decode(.., true) in the reference), raw_token names it
    assert tokenizer.raw_token(0) == "<|endoftext|>"
    assert tokenizer.decode([0] + ids) == text
    # byte-level tokens keep their marker for a leading space
    space_word = tokenizer.encode(" the")
    assert tokenizer.raw_token(space_word[0]).startswith("Ġ")


def test_tokenizer_errors(tokenizer, tmp_path):
    with pytest.raises(pg.Gpt2Error) as e:
        tokenizer.raw_token(10 ** 6)
    assert str(e.value) == "invalid GPT-2 input: unknown token id 1000000"
    with pytest.raises(pg.Gpt2Error) as e:
        tokenizer.decode([1 << 32])
    assert str(e.value) == "invalid GPT-2 input: token id does not fit in u32"
    missing = tmp_path / "nope" / "tokenizer.json"
    with pytest.raises(pg.Gpt2Error) as e:
        pg.Gpt2Tokenizer.from_file(str(missing))
    assert e.value.kind == "Asset" and str(e.value).startswith(f"GPT-2 asset error: failed to load tokenizer {missing}: ")
    bad = tmp_path / "tokenizer.json"
    bad.write_text("{not json")
    with pytest.raises(pg.Gpt2Error) as e:
        pg.Gpt2Tokenizer.from_file(str(bad))
    assert e.value.kind == "Asset"


def test_incremental_streaming_over_split_characters(tokenizer):
    """Characters of several bytes are split over tokens by a byte-level vocabulary: such a token decodes to
    U+FFFD by itself, the streamer then decodes the whole sequence and emits the new suffix
    (streaming.rs:46-74). What the streamer holds at the end is the decoding of everything."""
    text = "naïve 日本語 🙂 done"
    ids = tokenizer.encode(text)
    unsafe = [t for t in ids if not pg.is_incremental_decode_safe(tokenizer.decode_token(t))]
    assert unsafe, "the test text must split a character over tokens"
    streamer = pg.IncrementalTextStreamer("")
    pieces, out = [], []
    for t in ids:
        out.append(t)
        streamer.stream_token(tokenizer, out, t, pieces.append)
    assert streamer.decoded() == text == tokenizer.decode(ids)
    assert len(pieces) == len(ids)  # one piece per token, whichever way it was decoded
    # with single-byte characters every token is safe and the pieces are the text
    plain, pieces, out = tokenizer.encode("the quick brown fox"), [], []
    streamer = pg.IncrementalTextStreamer("")
    for t in plain:
        out.append(t)
        streamer.stream_token(tokenizer, out, t, pieces.append)
    assert "".join(pieces) == "the quick brown fox" == streamer.decoded()


def test_raw_token_events_and_durations(tokenizer):
    w = io.StringIO()
    ids = tokenizer.encode("a\tb\n")
    for t in ids:
        rt.write_raw_token_event(w, None, "prompt", t, tokenizer)
    rt.write_raw_token_event(w, 3, "generated", ids[0], tokenizer)
    lines = w.getvalue().splitlines()
    assert len(lines) == len(ids) + 1
    for line, t in zip(lines, ids):
        phase, tid, token = line.split("\t")
        assert (phase, int(tid)) == ("prompt", t) and token == pg.escape_raw_token(tokenizer.raw_token(t))
    assert lines[-1].split("\t")[:3] == ["3", "generated", str(ids[0])]
    assert rt.format_duration(1.5) == "1.500s"
    assert rt.format_duration(0.0025) == "2.50ms"
    assert rt.format_duration(3e-6) == "3.00us"


def test_generic_generation_stats_report_token_rates():
    """rust.rs:2040-2060"""
    stats = pg.GenerationStats(prompt_tokens=4, generated_tokens=6, tokenize_time=0.005, prefill_time=0.020,
                               decode_time=0.030, total_generation_time=0.050, first_token_time=0.022)
    assert stats.total_model_tokens() == 10
    assert stats.prefill_tokens_per_second() == pytest.approx(200.0)
    assert stats.decode_tokens_per_second() == pytest.approx(200.0)
    assert stats.total_tokens_per_second() == pytest.approx(200.0)
    assert stats.average_decode_token_time() == pytest.approx(0.005)


def test_gpt2_operation_profile_attaches_to_generic_stats():
    """rust.rs:2062-2080"""
    stats = pg.Gpt2GenerationStats.new(pg.GenerationStats(prompt_tokens=2, generated_tokens=3),
                                       pg.Gpt2OperationProfile(qkv_projection=0.007))
    profiled = stats.as_profiled()
    assert profiled.common.total_model_tokens() == 5
    assert profiled.profile.qkv_projection == 0.007
    common, profile = profiled.split()
    assert common is stats.common and profile is stats.operation_profile
    assert stats.generated_tokens == 3 and stats.total_model_tokens() == 5  # reads through to the common part


class StandInModel:
    """Emits a fixed continuation the way the library's calls do: callback per token, abort when it returns True."""

    def __init__(self, vocab_size, continuation):
        self.config = type("Cfg", (), {"vocab_size": vocab_size, "n_positions": 1024})()
        self.continuation = list(continuation)

    def generate_greedy_cached(self, ids, n):
        return list(ids) + self.continuation[:n]

    def stream_greedy_tokens(self, ids, n, on_token=None):
        out = list(ids)
        for t in self.continuation[:n]:
            if on_token and on_token(t):
                raise pg.Gpt2Error("InvalidInput", "token callback aborted generation")
            out.append(t)
        return out

    def generate_with_config(self, ids, cfg, on_token=None):
        out = []
        for t in self.continuation[:cfg.max_new_tokens]:
            if cfg.eos_token_id == t:
                break
            if on_token and on_token(t):
                raise pg.Gpt2Error("InvalidInput", "token callback aborted generation")
            out.append(t)
        return out, pg.GenerationStats(len(ids), len(out), 0.0, 0.25, 0.5, 0.75, 0.3 if out else None)


def test_runtime_text_calls_with_a_stand_in_model(tokenizer):
    cont = tokenizer.encode(" jumps over 日本 🙂 dog")
    r = pg.Gpt2Runtime(StandInModel(320, cont), tokenizer)
    prompt = "the quick brown fox"
    full = prompt + " jumps over 日本 🙂 dog"
    assert r.generate_greedy_text(prompt, len(cont)) == full
    pieces = []
    assert r.stream_greedy_text(prompt, len(cont), pieces.append) == full
    assert pieces[0] == prompt and len(pieces) == 1 + len(cont)

    pieces = []
    text, stats = r.stream_text_with_stats(prompt, pg.TextGenerationConfig(len(cont)), pieces.append)
    assert text == full and pieces[0] == prompt
    assert stats.prompt_tokens == len(tokenizer.encode(prompt)) and stats.generated_tokens == len(cont)
    assert stats.tokenize_time > 0 and stats.operation_profile.tokenization == stats.tokenize_time
    assert stats.operation_profile.decoding > 0 and stats.operation_profile.attention == 0.0
    assert stats.decode_tokens_per_second() == pytest.approx(len(cont) / 0.5)  # methods of the common part read through
    printed = rt.format_gpt2_stats(1.25, stats)
    assert "  load: 1.250s" in printed and f"({len(cont)} generated tokens, " in printed and "    decoding: " in printed
    assert rt.format_gpt2_speed(stats).startswith("\ntokens/sec: ")

    seen = []
    ids, stats = r.stream_token_ids_with_stats(prompt, pg.TextGenerationConfig(3), seen.append)
    assert ids == tokenizer.encode(prompt) + cont[:3] and seen == cont[:3] and stats.generated_tokens == 3
    # the end-of-sequence token stops the run before it is emitted
    ids, stats = r.stream_token_ids_with_stats(prompt, pg.TextGenerationConfig(8, eos_token_id=cont[2]), seen.append)
    assert ids == tokenizer.encode(prompt) + cont[:2]


def test_runtime_errors_with_a_stand_in_model(tokenizer):
    cont = tokenizer.encode(" jumps over")
    r = pg.Gpt2Runtime(StandInModel(320, cont), tokenizer)
    with pytest.raises(pg.Gpt2Error) as e:
        r.stream_text_with_stats("x", pg.TextGenerationConfig(4, eos_token_id=320), lambda s: None)
    assert str(e.value) == "invalid GPT-2 config: generation eos_token_id 320 is outside vocab_size 320"
    with pytest.raises(pg.Gpt2Error):
        r.stream_token_ids_with_stats("x", pg.TextGenerationConfig(4, top_p=0.0), lambda t: None)

    class Stop(Exception):
        pass

    def on_text(piece, n=[0]):
        n[0] += 1
        if n[0] == 3:
            raise Stop("enough")

    with pytest.raises(Stop):  # the callback's own error, not the library's "aborted" status
        r.stream_greedy_text("the quick", len(cont), on_text)

    def on_token(t):
        raise Stop("no tokens")

    with pytest.raises(Stop):
        r.stream_token_ids_with_stats("the quick", pg.TextGenerationConfig(4), on_token)


def test_command_output_with_a_stand_in_model(tokenizer, monkeypatch):
    """run-gpt2 (main.rs:1305-1388): text to stdout and the speed line to stderr; with --stream-raw-tokens one
    `phase TAB id TAB token` line per prompt and generated token; --stats prints the statistics block;
    --no-eos-stop and --eos-token-id set the end-of-sequence token of the generation."""
    cont = tokenizer.encode(" jumps over the lazy dog")
    seen = {}

    def from_dir_with_backend(model_dir, backend, use_tuning=True, tuning_file=None):
        seen.update(model_dir=model_dir, backend=backend, use_tuning=use_tuning)
        return pg.Gpt2Runtime(StandInModel(50257, cont), tokenizer)  # room for the default end-of-sequence id

    monkeypatch.setattr(rt.Gpt2Runtime, "from_dir_with_backend", staticmethod(from_dir_with_backend))
    prompt = "the quick brown fox"
    out, err = io.StringIO(), io.StringIO()
    assert rt.run_gpt2(["--model-dir", "/m", "--prompt", prompt, "--max-new-tokens", "4", "--no-tuning"], out, err) == 0
    assert out.getvalue() == prompt + tokenizer.decode(cont[:4]) + "\n"
    assert "loading GPT-2 from /m" in err.getvalue() and "tokens/sec: " in err.getvalue() and "stats:" not in err.getvalue()
    assert seen == {"model_dir": "/m", "backend": None, "use_tuning": False}

    out, err = io.StringIO(), io.StringIO()
    assert rt.run_gpt2(["--model-dir", "/m", "--prompt", prompt, "--max-new-tokens", "3", "--stream-raw-tokens", "--stats",
                        "--math-mode", "tf32x3", "--quantized-weights"], out, err) == 0
    rows = [l.split("\t") for l in out.getvalue().splitlines()]
    ids = tokenizer.encode(prompt)
    assert [(r[0], int(r[1])) for r in rows] == [("prompt", t) for t in ids] + [("generated", t) for t in cont[:3]]
    assert all(r[2] == pg.escape_raw_token(tokenizer.raw_token(int(r[1]))) for r in rows)
    assert "stats:" in err.getvalue() and "    tokenization: " in err.getvalue()
    assert seen["backend"].math_mode == "tf32x3" and seen["backend"].quantized_weights and seen["use_tuning"]
    assert seen["backend"].describe() == "cuda (device=0, math=tf32x3, page_tokens=32, weights=int8)"
    assert pg.Gpt2CudaConfig().describe() == "cuda (device=0, math=fp32, page_tokens=32, weights=f32)"

    out, err = io.StringIO(), io.StringIO()  # the third token of the continuation as end-of-sequence token
    assert rt.run_gpt2(["--model-dir", "/m", "--prompt", prompt, "--max-new-tokens", "8", "--eos-token-id", str(cont[2])],
                       out, err) == 0
    assert out.getvalue() == prompt + tokenizer.decode(cont[:2]) + "\n"
    with pytest.raises(pg.Gpt2Error):  # validated before anything is loaded
        rt.run_gpt2(["--model-dir", "/m", "--prompt", prompt, "--top-p", "0"], io.StringIO(), io.StringIO())


@pytest.mark.gpu
def test_runtime_from_dir_generates_text_end_to_end(tmp_path):

    vocab = make_tokenizer_json(tmp_path / "tokenizer.json")
    cfg = dict(vocab_size=vocab, n_positions=64, n_embd=64, n_layer=2, n_head=1, n_inner=256, layer_norm_epsilon=1e-5)
    w = synthetic.perturbed_weights(cfg, 77)
    d = synthetic.write_model_dir(str(tmp_path), cfg, w)
    r = pg.Gpt2Runtime.from_dir(d)
    tok = r.tokenizer
    prompt = "the quick brown"
    ids = tok.encode(prompt)
    want_ids = r.model.generate_greedy_cached(ids, 12)
    assert r.generate_greedy_text(prompt, 12) == tok.decode(want_ids)

    pieces = []
    text = r.stream_greedy_text(prompt, 12, pieces.append)
    assert text == tok.decode(want_ids) and pieces[0] == tok.decode(ids) and len(pieces) == 13

    gen = pg.TextGenerationConfig(12)  # greedy, no end-of-sequence token: the same 12 tokens
    pieces = []
    text2, stats = r.stream_text_with_stats(prompt, gen, pieces.append)
    assert text2 == text and stats.prompt_tokens == len(ids) and stats.generated_tokens == 12
    assert stats.prefill_time > 0 and stats.decode_time > 0 and stats.first_token_time is not None
    seen = []
    out_ids, stats = r.stream_token_ids_with_stats(prompt, gen, seen.append)
    assert out_ids == want_ids and seen == want_ids[len(ids):]

    out, err = io.StringIO(), io.StringIO()
    assert rt.run_gpt2(["--model-dir", d, "--prompt", prompt, "--max-new-tokens", "5", "--no-eos-stop",
                        "--stream-raw-tokens", "--stats"], out, err) == 0
    lines = [l.split("\t") for l in out.getvalue().splitlines()]
    assert [l[0] for l in lines] == ["prompt"] * len(ids) + ["generated"] * 5
    assert [int(l[1]) for l in lines] == want_ids[:len(ids) + 5]
    assert "stats:" in err.getvalue() and "  prefill: " in err.getvalue()
    out, err = io.StringIO(), io.StringIO()
    assert rt.run_gpt2(["--model-dir", d, "--prompt", prompt, "--max-new-tokens", "5", "--no-eos-stop"], out, err) == 0
    assert out.getvalue() == tok.decode(want_ids[:len(ids) + 5]) + "\n" and "tokens/sec: " in err.getvalue()
