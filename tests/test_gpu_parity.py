"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle.

Tolerance for FP32 logits: |gpu - oracle| <= 1e-4 + 1e-3 * |oracle| (the bound the task states
for the FP32 path); greedy token streams must be identical.
"""
import json
import os

import numpy as np
import pytest

import puppygrad_b200 as pg
from puppygrad_b200 import synthetic

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-3, 1e-4
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def assert_logits_close(got, want):
    np.testing.assert_allclose(got, want, rtol=RTOL, atol=ATOL)


def tiny():
    cfg = synthetic.preset("tiny")
    return cfg, synthetic.tiny_weights(cfg)


def assert_greedy_within_tolerance(tokens, n_prompt, o):
    """Every generated token must be an arg-max of the oracle's logits for the same prefix up to
    the logit tolerance. The reference's tiny test model (patterned weights of period 23) has
    logits that tie to 1e-10, so its greedy choice is decided by the last ulp of whichever
    summation order runs; identical streams are only required where the oracle's own top-2 gap
    exceeds the tolerance."""
    for i in range(n_prompt, len(tokens)):
        lo = o.forward(tokens[:i])[-1]
        assert lo[tokens[i]] >= lo.max() - (ATOL + RTOL * abs(float(lo.max()))), (i, tokens)


@pytest.fixture(scope="module")
def midi(oracle):
    cfg = synthetic.preset("midi")
    w = synthetic.perturbed_weights(cfg, 11)
    return cfg, w, pg.Gpt2Model(cfg, w), oracle.Model(cfg, w, threads=4)


# ------------------------------------------------------------------ the reference's tests (rust.rs:1861-1994)
def test_forward_returns_logits_for_each_position():
    cfg, w = tiny()
    out = pg.Gpt2Model(cfg, w).forward([1, 2, 3])
    assert out.seq_len == 3 and out.vocab_size == cfg["vocab_size"]
    assert out.logits.shape == (3, cfg["vocab_size"]) and np.isfinite(out.logits).all()


def test_greedy_generation_appends_tokens_until_context_limit():
    cfg, w = tiny()
    tokens = pg.Gpt2Model(cfg, w).generate_greedy([0, 1], 10)
    assert len(tokens) == cfg["n_positions"] and tokens[:2] == [0, 1]
    assert all(t < cfg["vocab_size"] for t in tokens)


def test_cached_prefill_matches_full_forward_last_logits():
    cfg, w = tiny()
    model = pg.Gpt2Model(cfg, w)
    full = model.forward([1, 2, 3])
    cache = model.new_kv_cache()
    cached = model.prefill([1, 2, 3], cache)
    assert cache.seq_len == 3
    assert np.all(np.abs(full.last_logits() - cached) <= 1e-5)


def test_cached_greedy_generation_matches_full_generation(oracle):
    # on a model without exact logit ties the two GPU paths must give the same stream
    cfg = synthetic.preset("mini")
    w = synthetic.perturbed_weights(cfg, 3)
    model = pg.Gpt2Model(cfg, w)
    prompt = synthetic.uniform_prompt(2, 6, cfg["vocab_size"])
    assert model.generate_greedy_cached(prompt, 12) == model.generate_greedy(prompt, 12)
    # the reference's tiny model ties to 1e-10: both paths must stay within tolerance of the oracle
    cfg, w = tiny()
    model, o = pg.Gpt2Model(cfg, w), oracle.Model(cfg, w)
    for toks in (model.generate_greedy_cached([0, 1], 3), model.generate_greedy([0, 1], 3)):
        assert len(toks) == 5 and toks[:2] == [0, 1]
        assert_greedy_within_tolerance(toks, 2, o)


def test_streams_generated_tokens_in_order():
    cfg, w = tiny()
    streamed = []
    tokens = pg.Gpt2Model(cfg, w).stream_greedy_tokens([0, 1], 3, lambda t: streamed.append(t))
    assert tokens[:2] == [0, 1] and streamed == tokens[2:]


def test_implements_generic_autoregressive_decoder():
    cfg, w = tiny()
    model = pg.Gpt2Model(cfg, w)
    assert pg.generate(model, [0, 1], 3) == model.generate_greedy_cached([0, 1], 3)


def test_gpt2_cache_exposes_generic_kv_cache_contract():
    cfg, w = tiny()
    model = pg.Gpt2Model(cfg, w)
    cache = model.new_kv_cache()
    model.prefill([0, 1], cache)
    assert cache.seq_len == 2 and cache.max_seq_len == cfg["n_positions"]
    cache.clear()
    assert cache.seq_len == 0


def test_tiny_model_matches_oracle_everywhere(oracle):
    cfg, w = tiny()
    g, o = pg.Gpt2Model(cfg, w), oracle.Model(cfg, w)
    assert_logits_close(g.forward([1, 2, 3, 4, 5]).logits, o.forward([1, 2, 3, 4, 5]))
    assert_greedy_within_tolerance(g.generate_greedy_cached([0, 1], 3), 2, o)
    assert_greedy_within_tolerance(g.generate_greedy([3], 10), 1, o)
    gc, oc = g.new_kv_cache(), o.new_kv_cache()
    assert_logits_close(g.prefill([1, 2, 3], gc), o.prefill([1, 2, 3], oc))
    assert_logits_close(g.forward_one(4, gc), o.forward_one(4, oc))


def test_input_validation_messages():
    """rust.rs:1029-1051, 950-962: same classes and texts as the reference."""
    cfg, w = tiny()
    model = pg.Gpt2Model(cfg, w)
    with pytest.raises(pg.Gpt2Error, match="input_ids must not be empty") as e:
        model.forward([])
    assert e.value.kind == "InvalidInput"
    with pytest.raises(pg.Gpt2Error, match="sequence length 6 exceeds n_positions 5"):
        model.forward([0] * 6)
    with pytest.raises(pg.Gpt2Error, match="token id 8 at index 1 exceeds vocab_size 8"):
        model.forward([0, 8])
    cache = model.new_kv_cache()
    with pytest.raises(pg.Gpt2Error, match="token id 9 exceeds vocab_size 8"):
        model.forward_one(9, cache)
    model.prefill([0, 1, 2, 3, 4], cache)
    with pytest.raises(pg.Gpt2Error, match="cache is full at seq_len 5"):
        model.forward_one(1, cache)
    other = pg.Gpt2Model(synthetic.preset("mini"), synthetic.random_init_weights(synthetic.preset("mini")))
    with pytest.raises(pg.Gpt2Error, match="cache layer count 1 does not match n_layer 2"):
        other.forward_one(1, cache)
    with pytest.raises(pg.Gpt2Error, match="max_batch"):
        model.prefill_batch([[1], [2]], cache)


# ------------------------------------------------------------------ numeric parity on larger shapes
def test_full_forward_matches_oracle(midi):
    cfg, w, g, o = midi
    ids = synthetic.uniform_prompt(5, 70, cfg["vocab_size"])
    assert_logits_close(g.forward(ids).logits, o.forward(ids))


def test_prefill_and_forward_one_match_oracle(midi):
    cfg, w, g, o = midi
    ids = synthetic.uniform_prompt(6, 50, cfg["vocab_size"])
    gc, oc = g.new_kv_cache(), o.new_kv_cache()
    assert_logits_close(g.prefill(ids[:33], gc), o.prefill(ids[:33], oc))
    for t in ids[33:]:
        assert_logits_close(g.forward_one(int(t), gc), o.forward_one(int(t), oc))
    assert gc.seq_len == oc.seq_len == 50


def test_kv_cache_contents_match_oracle(midi):
    cfg, w, g, o = midi
    ids = synthetic.uniform_prompt(7, 40, cfg["vocab_size"])
    gc, oc = g.new_kv_cache(), o.new_kv_cache()
    g.prefill(ids[:37], gc)
    o.prefill(ids[:37], oc)
    for t in ids[37:]:
        g.forward_one(int(t), gc)
        o.forward_one(int(t), oc)
    for layer in (0, cfg["n_layer"] - 1):
        gk, gv = gc.read_layer(layer)
        ok, ov = oc.read_layer(layer)
        np.testing.assert_allclose(gk, ok, rtol=1e-4, atol=1e-5)
        np.testing.assert_allclose(gv, ov, rtol=1e-4, atol=1e-5)
        assert not gk[:, 40:].any()


def test_token_by_token_prefill_equals_batched_prefill(midi):
    """The reference prefills token by token (rust.rs:920-926); the GEMM prefill must agree."""
    cfg, w, g, o = midi
    ids = synthetic.uniform_prompt(8, 45, cfg["vocab_size"])
    a, b = g.new_kv_cache(), g.new_kv_cache()
    la = g.prefill(ids, a)
    g.prefill(ids[:1], b)
    for t in ids[1:]:
        lb = g.forward_one(int(t), b)
    assert_logits_close(la, lb)
    np.testing.assert_allclose(a.read_layer(1)[0], b.read_layer(1)[0], rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("batch,math_mode", [(2, "fp32"), (5, "fp32"), (8, "fp32"), (12, "fp32"),
                                             (5, "tf32x3"), (8, "tf32x3"), (12, "tf32x3"), (20, "tf32x3"),
                                             (33, "tf32x3"), (64, "tf32x3"), (70, "tf32x3"), (130, "tf32x3")])
def test_ragged_batches_match_single_sequences(midi, oracle, batch, math_mode):
    cfg, w, g, o = midi
    if math_mode != "fp32":  # linears as three TF32 tensor-core products with FP32 accumulation
        g = pg.Gpt2Model(cfg, w, pg.Gpt2CudaConfig(math_mode=math_mode))
    prompts = [synthetic.uniform_prompt(100 + i, 3 + 7 * i % 40 + i, cfg["vocab_size"]) for i in range(batch)]
    cache = g.new_kv_cache(max_batch=batch)
    logits, am = g.prefill_batch(prompts, cache, want_logits=True)
    ocaches, olog = [], []
    for p in prompts:
        c = o.new_kv_cache()
        olog.append(o.prefill(p, c))
        ocaches.append(c)
    assert_logits_close(logits, np.stack(olog))
    assert [cache.seq_len_of(i) for i in range(batch)] == [len(p) for p in prompts]
    cur = am.copy()
    assert list(cur) == [oracle.argmax_logits(l) for l in olog]
    for step in range(6):
        n0 = cache.kernel_launches()
        logits, am, _, _ = g.forward_one_batch(cur, cache, want_logits=True)
        if math_mode != "fp32" and batch >= 9:  # one persistent kernel per 64 sequences
            assert cache.kernel_launches() - n0 == (batch + 63) // 64
        ol = np.stack([o.forward_one(int(cur[i]), ocaches[i]) for i in range(batch)])
        assert_logits_close(logits, ol)
        assert list(am) == [oracle.argmax_logits(l) for l in ol]
        cur = am.copy()
    if batch > 64:  # the device-fed loop over several launches per step
        toks = g.decode_greedy(cur, cache, 3)
        for step in range(3):
            ol = [o.forward_one(int(cur[i]), ocaches[i]) for i in range(batch)]
            cur = np.array([oracle.argmax_logits(l) for l in ol], dtype=np.int32)
            assert list(toks[step]) == list(cur)


def test_device_fed_greedy_equals_oracle_stream(midi):
    cfg, w, g, o = midi
    prompts = [synthetic.uniform_prompt(200 + i, 20 + i, cfg["vocab_size"]) for i in range(4)]
    cache = g.new_kv_cache(max_batch=4)
    _, first = g.prefill_batch(prompts, cache)
    toks = g.decode_greedy(first, cache, 40)  # [steps, batch]; step s returns the token after first
    for i, p in enumerate(prompts):
        want = o.generate_greedy_cached(p, 41)[len(p):]
        got = [int(first[i])] + [int(t) for t in toks[:40, i]]
        assert got[:41] == want


def test_paging_survives_clear_and_reuse(midi):
    cfg, w, g, o = midi
    cache = g.new_kv_cache(max_batch=3)
    p1 = [synthetic.uniform_prompt(300 + i, 70 + 13 * i, cfg["vocab_size"]) for i in range(3)]
    g.prefill_batch(p1, cache)
    cache.clear_slot(1)
    assert cache.seq_len_of(1) == 0 and cache.seq_len_of(0) == 70
    p2 = [synthetic.uniform_prompt(400 + i, 33 + 5 * i, cfg["vocab_size"]) for i in range(3)]
    logits, _ = g.prefill_batch(p2, cache, want_logits=True)
    for i, p in enumerate(p2):
        assert_logits_close(logits[i], o.prefill(p, o.new_kv_cache()))


@pytest.mark.parametrize("page_tokens,splits", [(16, 1), (32, 4), (64, 8)])
def test_page_sizes_and_attention_splits(oracle, page_tokens, splits):
    cfg = synthetic.preset("midi")
    w = synthetic.perturbed_weights(cfg, 12)
    g = pg.Gpt2Model(cfg, w, pg.Gpt2CudaConfig(page_tokens=page_tokens, attn_splits=splits))
    o = oracle.Model(cfg, w, threads=4)
    ids = synthetic.uniform_prompt(9, 150, cfg["vocab_size"])
    gc, oc = g.new_kv_cache(), o.new_kv_cache()
    assert_logits_close(g.prefill(ids[:140], gc), o.prefill(ids[:140], oc))
    for t in ids[140:]:
        assert_logits_close(g.forward_one(int(t), gc), o.forward_one(int(t), oc))


def test_greedy_steps_store_no_logits_and_later_steps_return_fresh_ones(midi, oracle):
    """decode_greedy and arg-max-only forward_one calls run the persistent step with an lm_head reduce
    phase that keeps the row arg-max but writes no logits; a later call that asks for logits must get
    that step's logits, not a stale buffer, and the token streams must be the oracle's."""
    cfg, w, _, o = midi
    g = pg.Gpt2Model(cfg, w, pg.Gpt2CudaConfig(math_mode="tf32x3"))
    batch = 10
    prompts = [synthetic.uniform_prompt(700 + i, 9 + 5 * i, cfg["vocab_size"]) for i in range(batch)]
    cache = g.new_kv_cache(max_batch=batch)
    _, first = g.prefill_batch(prompts, cache)
    steps = g.decode_greedy(first, cache, 4)                # [step, sequence]; steps without logits
    _, am, _, _ = g.forward_one_batch(steps[-1], cache)     # arg-max only
    logits, am2, _, _ = g.forward_one_batch(am, cache, want_logits=True)
    for i, p in enumerate(prompts):
        oc = o.new_kv_cache()
        cur = oracle.argmax_logits(o.prefill(p, oc))
        assert int(first[i]) == cur
        want = []
        for _ in range(5):
            lo = o.forward_one(cur, oc)
            cur = oracle.argmax_logits(lo)
            want.append(cur)
        assert [int(t) for t in steps[:, i]] + [int(am[i])] == want, i
        lo = o.forward_one(cur, oc)
        assert_logits_close(logits[i], lo)
        assert int(am2[i]) == oracle.argmax_logits(lo)


@pytest.mark.parametrize("page_tokens", [16, 32, 64])
def test_batched_tensor_core_step_is_one_persistent_kernel(oracle, monkeypatch, page_tokens):
    """9..64 sequences in the tensor-core modes: the layers and the lm_head of a decode step run as
    ONE persistent kernel, from the embedding to the token fed back: one launch per step. Checked against the oracle for every page size, for sequences of very different
    lengths up to the last position of the context, and against the kernel-per-operation path."""
    cfg = synthetic.preset("midi")
    w = synthetic.perturbed_weights(cfg, 21)
    o = oracle.Model(cfg, w, threads=4)
    batch = 12
    lens = [1, 2, 15, 16, 17, 31, 33, 64, 100, 200, cfg["n_positions"] - 4, cfg["n_positions"] - 3]
    prompts = [synthetic.uniform_prompt(500 + i, n, cfg["vocab_size"]) for i, n in enumerate(lens)]

    def run(no_chain):
        if no_chain:
            monkeypatch.setenv("PG_NO_CHAIN", "1")
        else:
            monkeypatch.delenv("PG_NO_CHAIN", raising=False)
        g = pg.Gpt2Model(cfg, w, pg.Gpt2CudaConfig(math_mode="tf32x3", page_tokens=page_tokens))
        cache = g.new_kv_cache(max_batch=batch)
        _, cur = g.prefill_batch(prompts, cache)
        out, launches = [], []
        for _ in range(3):
            n0 = cache.kernel_launches()
            logits, am, _, _ = g.forward_one_batch(cur, cache, want_logits=True)
            launches.append(cache.kernel_launches() - n0)
            out.append(logits)
            cur = am.copy()
        return out, launches, cache, g

    fused, fused_launches, cache, g = run(False)
    assert fused_launches == [1, 1, 1]
    split, split_launches, _, _ = run(True)
    assert min(split_launches) > 5 * cfg["n_layer"]
    ocaches = [o.new_kv_cache() for _ in prompts]
    cur = [oracle.argmax_logits(o.prefill(p, c)) for p, c in zip(prompts, ocaches)]
    for step in range(3):
        ol = np.stack([o.forward_one(int(cur[i]), ocaches[i]) for i in range(batch)])
        assert_logits_close(fused[step], ol)
        assert_logits_close(split[step], ol)
        cur = [oracle.argmax_logits(l) for l in ol]
    # the keys and values the persistent kernel appended are the oracle's
    k, v = cache.read_layer(cfg["n_layer"] - 1, slot=3)
    ok_, ov_ = ocaches[3].read_layer(cfg["n_layer"] - 1)
    np.testing.assert_allclose(k, ok_, rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(v, ov_, rtol=1e-4, atol=1e-5)


def test_graphs_and_plain_launches_agree_bitwise(oracle):
    cfg = synthetic.preset("mini")
    w = synthetic.perturbed_weights(cfg, 13)
    ids = synthetic.uniform_prompt(10, 30, cfg["vocab_size"])
    outs = []
    for graphs in (True, False):
        g = pg.Gpt2Model(cfg, w, pg.Gpt2CudaConfig(use_graphs=graphs))
        c = g.new_kv_cache()
        g.prefill(ids[:20], c)
        outs.append(np.stack([g.forward_one(int(t), c) for t in ids[20:]]))
    assert np.array_equal(outs[0], outs[1])


@pytest.mark.parametrize("persistent", [True, False])
@pytest.mark.parametrize("batch", [1, 2, 3, 5, 8])
def test_small_batch_step_matches_oracle(midi, oracle, batch, persistent):
    """A decode step of at most 8 sequences: as ONE persistent kernel (the default: weight stream through a
    shared-memory ring, tagged hand-over of activations between CTAs) and as a graph of one kernel per
    operation."""
    cfg, w, _, o = midi
    g = pg.Gpt2Model(cfg, w, pg.Gpt2CudaConfig(persistent_step=persistent, attn_splits=2 if batch == 3 else 0))
    prompts = [synthetic.uniform_prompt(800 + i, 40 + 9 * i, cfg["vocab_size"]) for i in range(batch)]
    cache = g.new_kv_cache(max_batch=batch)
    _, cur = g.prefill_batch(prompts, cache)
    ocaches = []
    for p in prompts:
        c = o.new_kv_cache()
        o.prefill(p, c)
        ocaches.append(c)
    for step in range(5):
        n0 = cache.kernel_launches()
        logits, am, _, _ = g.forward_one_batch(cur, cache, want_logits=True)
        assert (cache.kernel_launches() - n0 == 1) == persistent
        ol = np.stack([o.forward_one(int(cur[i]), ocaches[i]) for i in range(batch)])
        assert_logits_close(logits, ol)
        assert list(am) == [oracle.argmax_logits(l) for l in ol]
        cur = am.copy()
    np.testing.assert_allclose(cache.read_layer(1, batch - 1)[0], ocaches[-1].read_layer(1)[0], rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("splits", [0, 1, 3, 8])
def test_small_batch_step_over_long_and_ragged_contexts(oracle, splits):
    """Contexts of 5, 130 and 700 cached positions in one batch of the persistent step: attention over one
    and several 128-key rounds, split over CTAs with the partial results merged by the first split's CTA,
    keys and values of pages that another sequence used before."""
    cfg = dict(vocab_size=3001, n_positions=1024, n_embd=256, n_layer=2, n_head=4, n_inner=1024,
               layer_norm_epsilon=1e-5)
    w = synthetic.perturbed_weights(cfg, 77)
    g = pg.Gpt2Model(cfg, w, pg.Gpt2CudaConfig(attn_splits=splits, page_tokens=16))
    o = oracle.Model(cfg, w, threads=8)
    lens = [700, 130, 5]
    prompts = [synthetic.uniform_prompt(900 + i, n, cfg["vocab_size"]) for i, n in enumerate(lens)]
    cache = g.new_kv_cache(max_batch=3)
    g.prefill_batch(prompts[::-1], cache)  # scatter the pages
    cache.clear()
    _, cur = g.prefill_batch(prompts, cache)
    ocaches = [o.new_kv_cache() for _ in prompts]
    ocur = [oracle.argmax_logits(o.prefill(p, c)) for p, c in zip(prompts, ocaches)]
    assert list(cur) == ocur
    for step in range(4):
        n0 = cache.kernel_launches()
        logits, am, _, _ = g.forward_one_batch(cur, cache, want_logits=True)
        assert cache.kernel_launches() - n0 == 1
        ol = np.stack([o.forward_one(int(cur[i]), ocaches[i]) for i in range(3)])
        assert_logits_close(logits, ol)
        assert list(am) == [oracle.argmax_logits(l) for l in ol]
        cur = am.copy()
    for layer in range(2):
        k, v = cache.read_layer(layer, 0)
        ok, ov = ocaches[0].read_layer(layer)
        np.testing.assert_allclose(k, ok, rtol=1e-4, atol=1e-5)
        np.testing.assert_allclose(v, ov, rtol=1e-4, atol=1e-5)


def test_small_batch_step_fills_the_context_to_its_last_position(midi, oracle):
    """Greedy decode fed back on the device until the cache is full (ragged starts: only one sequence reaches
    n_positions), then the error of the reference for a full cache (rust.rs:957-962)."""
    cfg, w, g, o = midi
    P = cfg["n_positions"]
    prompts = [synthetic.uniform_prompt(950, P - 6, cfg["vocab_size"]), synthetic.uniform_prompt(951, 10, cfg["vocab_size"])]
    cache = g.new_kv_cache(max_batch=2)
    _, first = g.prefill_batch(prompts[::-1], cache)  # slot 0 is the short one
    toks = g.decode_greedy(first, cache, 6)
    assert (toks >= 0).all()
    for i, p in enumerate(prompts[::-1]):
        oc = o.new_kv_cache()
        want = [oracle.argmax_logits(o.prefill(p, oc))]
        for _ in range(6):
            want.append(oracle.argmax_logits(o.forward_one(want[-1], oc)))
        assert [int(first[i])] + [int(t) for t in toks[:, i]] == want
    assert cache.seq_len_of(1) == P
    with pytest.raises(pg.Gpt2Error, match=f"cache is full at seq_len {P}"):
        g.forward_one_batch([1, 1], cache)


def test_a_wait_that_runs_out_returns_timeout_and_the_cache_recovers(midi, oracle):
    """Every device-side wait has a limit. The test hook gives the next step a limit of a few thousand polls
    and makes it wait for a hand-over that never comes: every CTA gives up, the call returns PG_TIMEOUT
    (nothing faults, nothing hangs), and after a clear the same cache decodes correctly again."""
    cfg, w, g, o = midi
    for batch in (1, 4):
        prompts = [synthetic.uniform_prompt(960 + i, 20 + i, cfg["vocab_size"]) for i in range(batch)]
        cache = g.new_kv_cache(max_batch=batch)
        _, cur = g.prefill_batch(prompts, cache)
        cache.debug_expire_next_wait(2000)
        with pytest.raises(pg.Gpt2Error, match="bounded wait") as e:
            g.forward_one_batch(cur, cache)
        assert e.value.kind == "Timeout"
        cache.debug_expire_next_wait(2000)
        with pytest.raises(pg.Gpt2Error, match="bounded wait"):
            g.decode_greedy(cur, cache, 3)
        cache.clear()
        _, cur = g.prefill_batch(prompts, cache)
        toks = g.decode_greedy(cur, cache, 8)
        for i, p in enumerate(prompts):
            want = o.generate_greedy_cached(p, 9)[len(p):]
            assert [int(cur[i])] + [int(t) for t in toks[:, i]] == want


def test_odd_inner_dimension_takes_the_generic_path(oracle):
    """n_embd = 6 is not a multiple of 4: no vector loads, no fusion; head_dim 3."""
    cfg = dict(vocab_size=11, n_positions=9, n_embd=6, n_layer=2, n_head=2, n_inner=10, layer_norm_epsilon=1e-5)
    w = synthetic.perturbed_weights(cfg, 14)
    g, o = pg.Gpt2Model(cfg, w), oracle.Model(cfg, w)
    ids = [1, 10, 3, 7, 0, 2]
    assert_logits_close(g.forward(ids).logits, o.forward(ids))
    gc, oc = g.new_kv_cache(), o.new_kv_cache()
    assert_logits_close(g.prefill(ids[:4], gc), o.prefill(ids[:4], oc))
    assert_logits_close(g.forward_one(ids[4], gc), o.forward_one(ids[4], oc))


def test_model_dir_loader_matches_host_weights(tmp_path, oracle):
    cfg = synthetic.preset("mini")
    w = synthetic.perturbed_weights(cfg, 15)
    d = synthetic.write_model_dir(str(tmp_path / "m"), cfg, w, prefix="transformer.")
    a, b = pg.Gpt2Model.from_dir(d), pg.Gpt2Model(cfg, w)
    assert a.config.layer_norm_epsilon == pytest.approx(b.config.layer_norm_epsilon)
    a.config.layer_norm_epsilon = b.config.layer_norm_epsilon
    assert a.config == b.config
    ids = synthetic.uniform_prompt(11, 12, cfg["vocab_size"])
    assert np.array_equal(a.forward(ids).logits, b.forward(ids).logits)


# ------------------------------------------------------------------ sampling
def test_device_topk_order(midi):
    cfg, w, g, o = midi
    cache = g.new_kv_cache(max_batch=3)
    prompts = [synthetic.uniform_prompt(500 + i, 9, cfg["vocab_size"]) for i in range(3)]
    _, am = g.prefill_batch(prompts, cache)
    logits, am2, tv, ti = g.forward_one_batch(am, cache, want_logits=True, top_k=40)
    for r in range(3):
        order = sorted(range(cfg["vocab_size"]), key=lambda i: (-float(logits[r, i]), i))[:40]
        assert list(ti[r]) == order
        assert np.array_equal(tv[r], logits[r, order])
        assert am2[r] == order[0]


@pytest.mark.parametrize("kw", [dict(temperature=0.8, top_k=40), dict(temperature=0.9, top_p=0.95),
                                dict(temperature=0.0, repeat_penalty=1.4), dict(temperature=0.0)])
def test_generate_with_config_matches_oracle_loop(midi, oracle, kw):
    """Gpt2Runtime::stream_token_ids_with_stats (rust.rs:548-635) restated over the oracle."""
    cfg, w, g, o = midi
    prompt = synthetic.uniform_prompt(600, 17, cfg["vocab_size"])
    conf = pg.TextGenerationConfig(24, seed=77, **kw)
    got, stats = g.generate_with_config(prompt, conf)
    og = oracle.generation_config(24, seed=77, **kw)
    sampler = oracle.LogitsSampler(og.seed)
    cache = o.new_kv_cache()
    logits = o.prefill(prompt, cache)
    hist, want = [int(t) for t in prompt], []
    for i in range(24):
        nxt = sampler.select_next_token(logits, hist, og)
        hist.append(nxt)
        want.append(nxt)
        if i + 1 < 24:
            logits = o.forward_one(nxt, cache)
    assert got == want
    assert stats.prompt_tokens == 17 and stats.generated_tokens == 24
    assert stats.decode_tokens_per_second() > 0 and stats.first_token_time is not None


def test_eos_stops_generation(midi):
    cfg, w, g, o = midi
    prompt = synthetic.uniform_prompt(601, 10, cfg["vocab_size"])
    full, _ = g.generate_with_config(prompt, pg.TextGenerationConfig(12))
    eos = full[5]
    cut, stats = g.generate_with_config(prompt, pg.TextGenerationConfig(12, eos_token_id=eos))
    assert cut == full[:full.index(eos)]
    assert stats.generated_tokens == len(cut)


# ------------------------------------------------------------------ GPT-2 small, batch 1 (first benchmark config)
def test_gpt2_small_greedy_stream_is_token_exact_against_golden(oracle):
    gold = json.load(open(os.path.join(GOLDEN, "gpt2_small_b1.json")))
    cfg = gold["config"]
    w = synthetic.random_init_weights(cfg, seed=gold["weight_seed"])
    prompt = synthetic.uniform_prompt(gold["prompt_seed"], 32, cfg["vocab_size"])
    assert [int(t) for t in prompt] == gold["prompt"]
    g = pg.Gpt2Model(cfg, w)
    cache = g.new_kv_cache()
    logits = g.prefill(prompt, cache)
    tokens = []
    stride = gold["logit_stride"]
    for step in range(64):
        rec = gold["logits"].get(str(step))
        if rec:
            assert_logits_close(logits[::stride], np.array(rec["strided"], np.float32))
            assert_logits_close(logits[rec["top_idx"]], np.array(rec["top_val"], np.float32))
        nxt = pg.argmax_logits(logits)
        tokens.append(nxt)
        logits = g.forward_one(nxt, cache)
    assert tokens == gold["tokens"]
    # the same stream through the generic loop and the device-fed loop
    assert g.generate_greedy_cached(prompt, 64)[32:] == gold["tokens"]
    c2 = g.new_kv_cache()
    _, first = g.prefill_batch([prompt], c2)
    dev = g.decode_greedy(first, c2, 63)
    assert [int(first[0])] + [int(t) for t in dev[:, 0]] == gold["tokens"]
    # and live against the oracle on this host for the first steps
    o = oracle.Model(cfg, w, threads=os.cpu_count())
    oc = o.new_kv_cache()
    c3 = g.new_kv_cache()
    assert_logits_close(g.prefill(prompt, c3), o.prefill(prompt, oc))
    for t in gold["tokens"][:4]:
        assert_logits_close(g.forward_one(t, c3), o.forward_one(t, oc))


# ------------------------------------------------------------------ GPT-2 medium, 64 sequences (benchmark config)
@pytest.mark.parametrize("math_mode", ["fp32", "tf32x3"])
def test_gpt2_medium_64_sequences_against_golden_streams(math_mode):
    """64 prompts of 128 tokens, 256 greedy tokens each, against the oracle's committed streams.
    Teacher-forced: every step is fed the golden token, so all 64 x 256 arg-max decisions are
    checked even after a near-tie. A GPU arg-max may differ from the golden one only where the
    oracle's own top-2 logit gap is below 1e-4 (the FP32 logit tolerance); over 16384 decisions
    the smallest golden gap is 1.3e-5. The free-running device-fed decode must reproduce each
    golden stream exactly up to that sequence's first such near-tie."""
    gold = json.load(open(os.path.join(GOLDEN, "gpt2_medium_b64.json")))
    cfg = gold["config"]
    w = synthetic.random_init_weights(cfg, seed=gold["weight_seed"])
    prompts = [synthetic.uniform_prompt(s, gold["prompt_len"], cfg["vocab_size"]) for s in gold["prompt_seeds"]]
    tokens = np.array(gold["tokens"], np.int64)  # [seq, step]
    gaps = np.array(gold["top2_gap"], np.float32)
    n_seq, n_new = tokens.shape
    g = pg.Gpt2Model(cfg, w, pg.Gpt2CudaConfig(math_mode=math_mode))
    cache = g.new_kv_cache(max_batch=n_seq)
    _, am = g.prefill_batch(prompts, cache)
    near_tie = 1e-4
    mismatches = []
    for step in range(n_new):
        bad = np.nonzero(am != tokens[:, step])[0]
        for i in bad:
            assert gaps[i, step] < near_tie, (int(i), step, float(gaps[i, step]))
            mismatches.append((int(i), step))
        if step + 1 < n_new:
            _, am, _, _ = g.forward_one_batch(tokens[:, step], cache)
    assert len(mismatches) <= 4, mismatches
    # free-running, token fed back on the device
    _, first = g.prefill_batch(prompts, cache)
    dev = g.decode_greedy(first, cache, n_new - 1)
    got = np.concatenate([first[None, :], dev], axis=0).T  # [seq, step]
    for i in range(n_seq):
        diff = np.nonzero(got[i] != tokens[i])[0]
        if diff.size:
            assert gaps[i, diff[0]] < near_tie, (i, int(diff[0]), float(gaps[i, diff[0]]))
    exact = sum(int(np.array_equal(got[i], tokens[i])) for i in range(n_seq))
    assert exact >= n_seq - 4


def test_sharding_over_two_gpus_gives_the_single_gpu_streams(midi):
    """Sequence i on GPU i mod G: every sequence's stream is independent of G."""
    from puppygrad_b200 import _native, sharding
    if _native.lib.pg_device_count() < 2:
        pytest.skip("needs two GPUs")
    cfg, w, g0, o = midi
    prompts = [synthetic.uniform_prompt(700 + i, 10 + i, cfg["vocab_size"]) for i in range(6)]

    def run(model, idx):
        cache = model.new_kv_cache(max_batch=len(idx))
        _, first = model.prefill_batch([prompts[i] for i in idx], cache)
        toks = model.decode_greedy(first, cache, 20)
        return {i: [int(first[j])] + [int(t) for t in toks[:, j]] for j, i in enumerate(idx)}

    single = run(g0, list(range(6)))
    merged = {}
    for rank in range(2):
        model = pg.Gpt2Model(cfg, w, pg.Gpt2CudaConfig(device=rank))
        merged.update(run(model, sharding.partition(6, 2, rank)))
    assert sharding.gather_streams(merged, 6) == [single[i] for i in range(6)]


def test_tf32_prefill_is_within_its_stated_bound(oracle):
    """math_mode tf32: prefill GEMMs as one TF32 tensor-core pass. Stated bound for the final-position
    logits against the FP32 oracle: 5e-3 of the logit range (the FP32 path holds 1e-3 / 1e-4)."""
    cfg = synthetic.preset("midi")
    cfg["n_positions"] = 512
    w = synthetic.random_init_weights(cfg, 5)
    prompts = [synthetic.uniform_prompt(900 + i, 300, cfg["vocab_size"]) for i in range(2)]
    g = pg.Gpt2Model(cfg, w, pg.Gpt2CudaConfig(math_mode="tf32"))
    o = oracle.Model(cfg, w, threads=os.cpu_count())
    cache = g.new_kv_cache(max_batch=2)
    logits, _ = g.prefill_batch(prompts, cache, want_logits=True)
    for i, p in enumerate(prompts):
        want = o.prefill(p, o.new_kv_cache())
        span = float(want.max() - want.min())
        assert np.abs(logits[i] - want).max() <= 5e-3 * span


@pytest.mark.parametrize("math_mode", ["tf32", "tf32x3", "bf16"])
def test_prefill_attention_on_tensor_cores_with_ragged_prompts(oracle, math_mode):
    """Prefill runs causal attention on the tensor cores (128-query x 128-key tiles, head_dim 64): as single
    TF32 products in the tf32 mode, as three TF32 products per term (FP32 grade) in the tf32x3 and bf16
    modes. Prompt lengths on, just past and far from the tile edges, several sequences in one call:
    final-position logits stay within the mode's stated bound (tf32: 5e-3 of the logit span; the others:
    the FP32 tolerance, bf16 against the oracle on the same rounded weights), the first greedy token is
    the oracle's wherever the oracle's own top-2 gap is clear of that bound, and the keys and values that
    went into the cache are the oracle's."""
    cfg = synthetic.preset("midi")
    cfg["n_positions"] = 512
    w = synthetic.random_init_weights(cfg, 6)
    lens = [300, 129, 128, 1, 257, 512, 127]
    prompts = [synthetic.uniform_prompt(950 + i, n, cfg["vocab_size"]) for i, n in enumerate(lens)]
    g = pg.Gpt2Model(cfg, w, pg.Gpt2CudaConfig(math_mode=math_mode))
    o = oracle.Model(cfg, synthetic.bf16_rounded_weights(w) if math_mode == "bf16" else w, threads=os.cpu_count())
    cache = g.new_kv_cache(max_batch=len(lens))
    logits, first = g.prefill_batch(prompts, cache, want_logits=True)
    assert np.isfinite(logits).all()
    for i, p in enumerate(prompts):
        want = o.prefill(p, o.new_kv_cache())
        span = float(want.max() - want.min())
        if math_mode == "tf32":
            assert np.abs(logits[i] - want).max() <= 5e-3 * span, (i, lens[i])
            clear = 1e-2 * span
        else:
            assert_logits_close(logits[i], want)
            clear = 1e-4
        top2 = np.sort(want)[-2:]
        if top2[1] - top2[0] > clear:
            assert int(first[i]) == int(want.argmax()), i


@pytest.mark.parametrize("kw", [dict(temperature=0.8, top_k=40), dict(temperature=0.0),
                                dict(temperature=0.7, top_p=0.9, repeat_penalty=1.2)])
def test_batched_sampling_with_per_sequence_seeds_matches_oracle(midi, oracle, kw):
    """Temperature / top-k / top-p sampling for a batch, one RNG per sequence (seed base + i): the
    sequences reproduce the oracle's single-sequence sampler loop draw for draw. A draw that falls within
    rounding distance of a cumulative-probability boundary (the logits agree to 1e-6, not bitwise) may
    legitimately go the other way and changes the rest of that sequence, so one of the 6 may differ."""
    cfg, w, g, o = midi
    n, new = 6, 20
    differing = 0
    prompts = [synthetic.uniform_prompt(1000 + i, 12 + 3 * i, cfg["vocab_size"]) for i in range(n)]
    conf = pg.TextGenerationConfig(new, seed=500, **kw)
    got = g.generate_batch(prompts, conf)
    for i, p in enumerate(prompts):
        og = oracle.generation_config(new, seed=500 + i, **kw)
        sampler = oracle.LogitsSampler(og.seed)
        cache = o.new_kv_cache()
        logits = o.prefill(p, cache)
        hist, want = [int(t) for t in p], []
        for s in range(new):
            nxt = sampler.select_next_token(logits, hist, og)
            hist.append(nxt)
            want.append(nxt)
            if s + 1 < new:
                logits = o.forward_one(nxt, cache)
        differing += got[i] != want
    assert differing <= 1


def test_batched_sampling_on_the_persistent_step_kernel(oracle):
    """configs of the XL run in small: temperature 0.8 / top-k 40 with a fixed seed per sequence, 12
    sequences on the tensor-core path (device top-k after the persistent step kernel, host draw).
    A draw that falls within rounding distance of a cumulative-probability boundary may legitimately
    go the other way and changes the rest of that sequence, so one of the 12 may differ."""
    cfg = synthetic.preset("midi")
    w = synthetic.perturbed_weights(cfg, 31)
    g = pg.Gpt2Model(cfg, w, pg.Gpt2CudaConfig(math_mode="tf32x3"))
    o = oracle.Model(cfg, w, threads=4)
    n, new = 12, 24
    kw = dict(temperature=0.8, top_k=40)
    prompts = [synthetic.uniform_prompt(2000 + i, 10 + 5 * i, cfg["vocab_size"]) for i in range(n)]
    got = g.generate_batch(prompts, pg.TextGenerationConfig(new, seed=900, **kw))
    differing = 0
    for i, p in enumerate(prompts):
        og = oracle.generation_config(new, seed=900 + i, **kw)
        sampler = oracle.LogitsSampler(og.seed)
        cache = o.new_kv_cache()
        logits = o.prefill(p, cache)
        hist, want = [int(t) for t in p], []
        for s in range(new):
            nxt = sampler.select_next_token(logits, hist, og)
            hist.append(nxt)
            want.append(nxt)
            if s + 1 < new:
                logits = o.forward_one(nxt, cache)
        differing += got[i] != want
    assert differing <= 1


def test_persistent_step_when_shares_straddle_row_tiles(oracle):
    """A width whose GEMMs do not divide evenly over the SMs (17 units of 64 per 1088-wide row, as
    25 for GPT-2 XL's 1600): every CTA's share of the QKV, both projections, the MLP and the lm_head
    then crosses row-tile boundaries, the reduce and attention phases add a varying number of
    partial tiles per output, and rows need two float4 per worker thread."""
    cfg = dict(vocab_size=2003, n_positions=96, n_embd=1088, n_layer=2, n_head=17, n_inner=4352,
               layer_norm_epsilon=1e-5)
    w = synthetic.perturbed_weights(cfg, 41)
    g = pg.Gpt2Model(cfg, w, pg.Gpt2CudaConfig(math_mode="tf32x3"))
    o = oracle.Model(cfg, w, threads=8)
    batch = 10
    prompts = [synthetic.uniform_prompt(700 + i, 1 + 9 * i, cfg["vocab_size"]) for i in range(batch)]
    cache = g.new_kv_cache(max_batch=batch)
    _, cur = g.prefill_batch(prompts, cache)
    ocaches = [o.new_kv_cache() for _ in prompts]
    ocur = [oracle.argmax_logits(o.prefill(p, c)) for p, c in zip(prompts, ocaches)]
    assert list(cur) == ocur
    for _ in range(3):
        n0 = cache.kernel_launches()
        logits, am, _, _ = g.forward_one_batch(cur, cache, want_logits=True)
        assert cache.kernel_launches() - n0 == 1
        ol = np.stack([o.forward_one(int(cur[i]), ocaches[i]) for i in range(batch)])
        assert_logits_close(logits, ol)
        assert list(am) == [oracle.argmax_logits(l) for l in ol]
        cur = am.copy()


def test_persistent_step_breaks_logit_ties_towards_the_lowest_index(oracle):
    """argmax_logits (generation.rs:269-279) keeps the first strict maximum. With a tied embedding whose rows
    repeat (row v = row v + 1 for even v, and again 400 and 800 rows further on), every logit occurs six times:
    in neighbouring lanes of one warp, in other warps and in other row tiles of the lm_head. Every row tile sums
    in the same order, so the six are equal bit for bit and the answer must be the even index below 400."""
    cfg = dict(vocab_size=1200, n_positions=64, n_embd=256, n_layer=2, n_head=4, n_inner=1024,
               layer_norm_epsilon=1e-5)
    w = synthetic.perturbed_weights(cfg, 43)
    base = w["wte.weight"][:200].copy()
    w["wte.weight"] = np.ascontiguousarray(base[(np.arange(1200) % 400) // 2])
    g = pg.Gpt2Model(cfg, w, pg.Gpt2CudaConfig(math_mode="tf32x3"))
    o = oracle.Model(cfg, w, threads=4)
    batch = 12
    prompts = [synthetic.uniform_prompt(900 + i, 2 + 3 * i, cfg["vocab_size"]) for i in range(batch)]
    cache = g.new_kv_cache(max_batch=batch)
    _, cur = g.prefill_batch(prompts, cache)
    ocaches = [o.new_kv_cache() for _ in prompts]
    ocur = [oracle.argmax_logits(o.prefill(p, c)) for p, c in zip(prompts, ocaches)]
    assert list(cur) == ocur
    for step in range(4):
        n0 = cache.kernel_launches()
        logits, am, _, _ = g.forward_one_batch(cur, cache, want_logits=step % 2 == 0)
        assert cache.kernel_launches() - n0 == 1
        ol = np.stack([o.forward_one(int(cur[i]), ocaches[i]) for i in range(batch)])
        if logits is not None:
            assert_logits_close(logits, ol)
            assert np.array_equal(logits[:, :400], logits[:, 400:800]) and np.array_equal(logits[:, :400], logits[:, 800:])
        assert all(int(t) < 400 and int(t) % 2 == 0 for t in am)
        assert list(am) == [oracle.argmax_logits(l) for l in ol]
        cur = am.copy()


# ------------------------------------------------------------------ narrow weights: int8 rows (the reference's variant), BF16
@pytest.mark.parametrize("batch,math_mode", [(1, "fp32"), (3, "fp32"), (8, "fp32"), (12, "tf32x3")])
def test_quantized_weights_model_matches_the_quantized_oracle(oracle, batch, math_mode):
    """Gpt2RustConfig::quantized_weights (options.rs:62-104): int8 rows for the four linears and the lm_head,
    FP32 embedding lookup. Prefill runs the FP32 kernels on q * scale, decode steps of up to 8 sequences stream
    the int8 rows, larger batches run the tensor-core step on q * scale; all against the oracle's quantised model
    (quantized_linear_into, rust.rs:1535-1578; quantized_logits_from_hidden_into, rust.rs:1815-1849)."""
    cfg = synthetic.preset("midi")
    w = synthetic.perturbed_weights(cfg, 51)
    g = pg.Gpt2Model(cfg, w, pg.Gpt2CudaConfig(quantized_weights=True, math_mode=math_mode))
    o = oracle.Model(cfg, w, threads=4, quantized_weights=True)
    prompts = [synthetic.uniform_prompt(1100 + i, 9 + 11 * i, cfg["vocab_size"]) for i in range(batch)]
    cache = g.new_kv_cache(max_batch=batch)
    logits, cur = g.prefill_batch(prompts, cache, want_logits=True)
    ocaches = [o.new_kv_cache() for _ in prompts]
    ol = np.stack([o.prefill(p, c) for p, c in zip(prompts, ocaches)])
    assert_logits_close(logits, ol)
    assert list(cur) == [oracle.argmax_logits(l) for l in ol]
    for step in range(4):
        n0 = cache.kernel_launches()
        logits, am, _, _ = g.forward_one_batch(cur, cache, want_logits=True)
        assert cache.kernel_launches() - n0 == 1  # the persistent step kernels
        ol = np.stack([o.forward_one(int(cur[i]), ocaches[i]) for i in range(batch)])
        assert_logits_close(logits, ol)
        assert list(am) == [oracle.argmax_logits(l) for l in ol]
        cur = am.copy()
    # the reference's own test (rust.rs:1996-2013) on its tiny model
    tcfg, tw = tiny()
    out = pg.Gpt2Model(tcfg, tw, pg.Gpt2CudaConfig(quantized_weights=True)).forward([1, 2, 3])
    assert out.logits.shape == (3, tcfg["vocab_size"]) and np.isfinite(out.logits).all()
    assert_logits_close(out.logits, oracle.Model(tcfg, tw, quantized_weights=True).forward([1, 2, 3]))


@pytest.mark.parametrize("batch", [1, 4, 8, 12])
def test_bf16_weights_model_is_fp32_math_on_rounded_weights(oracle, batch):
    """math_mode "bf16": the dense matrices and the tied embedding rounded to BF16, FP32 activations and sums.
    Against the oracle run on the same rounded weights the FP32 tolerance holds (1e-3 relative / 1e-4 absolute);
    against the FP32 model the stated, looser bound of this variant is 3 % of the logit span."""
    cfg = synthetic.preset("midi")
    w = synthetic.perturbed_weights(cfg, 52)
    g = pg.Gpt2Model(cfg, w, pg.Gpt2CudaConfig(math_mode="bf16"))
    o = oracle.Model(cfg, synthetic.bf16_rounded_weights(w), threads=4)
    o32 = oracle.Model(cfg, w, threads=4)
    prompts = [synthetic.uniform_prompt(1200 + i, 7 + 13 * i, cfg["vocab_size"]) for i in range(batch)]
    cache = g.new_kv_cache(max_batch=batch)
    logits, cur = g.prefill_batch(prompts, cache, want_logits=True)
    ocaches = [o.new_kv_cache() for _ in prompts]
    ol = np.stack([o.prefill(p, c) for p, c in zip(prompts, ocaches)])
    assert_logits_close(logits, ol)
    l32 = np.stack([o32.prefill(p, o32.new_kv_cache()) for p in prompts])
    assert np.abs(logits - l32).max() <= 0.03 * (l32.max() - l32.min())
    for step in range(4):
        logits, am, _, _ = g.forward_one_batch(cur, cache, want_logits=True)
        ol = np.stack([o.forward_one(int(cur[i]), ocaches[i]) for i in range(batch)])
        assert_logits_close(logits, ol)
        assert list(am) == [oracle.argmax_logits(l) for l in ol]
        cur = am.copy()


def test_narrow_weight_modes_exclude_each_other():
    cfg, w = tiny()
    with pytest.raises(pg.Gpt2Error, match="exclude each other"):
        pg.Gpt2Model(cfg, w, pg.Gpt2CudaConfig(math_mode="bf16", quantized_weights=True))


# ------------------------------------------------------------------ GPT-2 small prefill, 8 x 1024 (second benchmark config)
@pytest.mark.parametrize("math_mode,span_bound", [("fp32", None), ("tf32x3", None), ("tf32", 5e-3), ("bf16", 3e-2)])
def test_gpt2_small_prefill_8x1024_against_golden(math_mode, span_bound):
    """Eight prompts of 1024 tokens through the batched prefill, final-position logits against the oracle's
    committed rows (prefill token by token, rust.rs:906-927): the FP32 modes at 1e-3 relative / 1e-4 absolute,
    the single-pass TF32 mode within 5e-3 of the logit span, BF16 weights within 3e-2 of it."""
    gold = json.load(open(os.path.join(GOLDEN, "gpt2_small_prefill_8x1024.json")))
    cfg = gold["config"]
    w = synthetic.random_init_weights(cfg, seed=gold["weight_seed"])
    prompts = [synthetic.uniform_prompt(s, gold["prompt_len"], cfg["vocab_size"]) for s in gold["prompt_seeds"]]
    g = pg.Gpt2Model(cfg, w, pg.Gpt2CudaConfig(math_mode=math_mode))
    cache = g.new_kv_cache(max_batch=len(prompts))
    logits, am = g.prefill_batch(prompts, cache, want_logits=True)
    stride = gold["logit_stride"]
    for i, rec in enumerate(gold["final_logits"]):
        got = np.concatenate([logits[i, ::stride], logits[i, rec["top_idx"]]])
        want = np.array(rec["strided"] + rec["top_val"], np.float32)
        if span_bound is None:
            assert_logits_close(got, want)
            assert int(am[i]) == rec["top_idx"][0]
        else:
            assert np.abs(got - want).max() <= span_bound * gold["logit_span"][i], (i, float(np.abs(got - want).max()))


# ------------------------------------------------------------------ GPT-2 XL, sampled decode (fourth benchmark config, a subset)
@pytest.mark.parametrize("copies", [1, 3])
def test_gpt2_xl_sampling_against_golden(copies):
    """GPT-2 XL (48 layers, 1600 wide, 25 heads), 512-token prompts, 32 tokens drawn at temperature 0.8 / top-k 40
    with one seed per sequence, against the oracle's committed run of four sequences. Teacher-forced: every step
    is fed the golden token, its 40 largest logits must equal the golden list (values at the FP32 tolerance, the
    same indices wherever neighbouring values differ by more than it), and the library's sampler, drawing from the
    device's list with the golden seed, must pick the golden token (a draw within rounding of a cumulative-weight
    boundary may go the other way: at most one of the 128 draws). copies = 1: four sequences on the single-kernel
    step of small batches; copies = 3: twelve on the tensor-core step kernel."""
    gold = json.load(open(os.path.join(GOLDEN, "gpt2_xl_sampling_4x512.json")))
    cfg = gold["config"]
    w = synthetic.random_init_weights(cfg, seed=gold["weight_seed"])
    base = [synthetic.uniform_prompt(s, gold["prompt_len"], cfg["vocab_size"]) for s in gold["prompt_seeds"]]
    n0 = len(base)
    prompts = base * copies
    g = pg.Gpt2Model(cfg, w, pg.Gpt2CudaConfig(math_mode="tf32x3"))
    del w
    conf = pg.TextGenerationConfig(len(gold["steps"]), temperature=gold["temperature"], top_k=gold["top_k"],
                                   seed=gold["sampler_seed"])
    from puppygrad_b200.generation import LogitsSampler
    samplers = [LogitsSampler(conf.seed + (i % n0)) for i in range(len(prompts))]
    cache = g.new_kv_cache(max_batch=len(prompts))
    g.prefill_batch([p[:-1] for p in prompts], cache)
    cur = [int(p[-1]) for p in prompts]
    wrong_draws = 0
    for step, rec in enumerate(gold["steps"]):
        n_before = cache.kernel_launches()
        _, _, tv, ti = g.forward_one_batch(cur, cache, top_k=40)
        assert cache.kernel_launches() - n_before == 1
        for i in range(len(prompts)):
            want = rec["top"][i % n0]
            wv, wi = np.array(want["top_val"], np.float32), np.array(want["top_idx"])
            assert_logits_close(tv[i], wv)
            gaps = np.minimum(np.abs(np.diff(wv, prepend=np.inf)), np.abs(np.diff(wv, append=-np.inf)))
            clear = gaps > 2 * (ATOL + RTOL * np.abs(wv))
            clear[-1] = False  # its lower neighbour, the 41st value, is not in the fixture
            assert np.array_equal(ti[i][clear], wi[clear])
            wrong_draws += int(samplers[i].select_from_topk(tv[i], ti[i], conf) != rec["tokens"][i % n0])
        cur = [rec["tokens"][i % n0] for i in range(len(prompts))]
    assert wrong_draws <= copies
