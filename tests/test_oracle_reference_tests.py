"""The reference's own unit tests for the GPT-2 path, restated against the CPU oracle.

Each test names the reference test it follows. These are the only known-answer and relation
tests the reference holds for this path; passing them is what pins the oracle.
"""
import numpy as np
import pytest

from puppygrad_b200 import synthetic


def tiny():
    cfg = synthetic.preset("tiny")
    return cfg, synthetic.tiny_weights(cfg)


# ---- src/models/cpu.rs:299-346
def test_dot_matches_scalar_reference(oracle):
    a = synthetic.patterned(37, 0.013)
    b = synthetic.patterned(37, -0.021)
    assert abs(oracle.dot(a, b) - oracle.dot_scalar(a, b)) <= 1e-6


def test_transposed_dense_projection_matches_dense_projection(oracle):
    x = synthetic.patterned(6, 0.2)
    weight = synthetic.patterned(12, 0.1)
    bias = np.array([0.5, -0.25, 0.125, 0.0], np.float32)
    transposed = oracle.transpose_in_out(weight, 3, 4)
    dense = oracle.dense_projection(x, 2, 3, 4, weight, bias)
    tdense = oracle.transposed_dense_projection(x, 2, 3, 4, transposed, bias)
    assert np.all(np.abs(dense - tdense) <= 1e-6)


def test_quantized_projection_returns_finite_values(oracle):
    """cpu.rs:327-343, plus what the reference's quantiser implies for the same inputs: the bytes and
    scales equal an independent float32 restatement, and the projection equals the FP32 projection
    over the dequantised weights."""
    x = synthetic.patterned(6, 0.2)
    weight = synthetic.patterned(12, 0.1)
    bias = np.array([0.5, -0.25, 0.125, 0.0], np.float32)
    wt = oracle.transpose_in_out(weight, 3, 4)
    q, scales = oracle.quantize_rows(wt, 4, 3)
    out = oracle.quantized_projection(x, 2, 3, 4, q, scales, bias)
    assert out.shape == (8,) and np.isfinite(out).all()
    rows = wt.reshape(4, 3)
    want_scales = (np.abs(rows).max(axis=1) / np.float32(127.0)).astype(np.float32)
    assert np.array_equal(scales, want_scales)
    t = (rows / want_scales[:, None]).astype(np.float32).astype(np.float64)
    want_q = np.clip(np.where(t >= 0, np.floor(t + 0.5), np.ceil(t - 0.5)), -127, 127).astype(np.int8)
    assert np.array_equal(q, want_q)
    deq = (q.astype(np.float32) * scales[:, None]).astype(np.float32)
    assert np.all(np.abs(out - oracle.transposed_dense_projection(x, 2, 3, 4, deq, bias)) <= 1e-6)


def test_quantized_rows_edge_cases(oracle):
    """QuantizedRows::from_f32 (cpu.rs:33-57): an all-zero row gets scale 1 and zeros, the largest
    magnitude of a row maps to +-127, every weight is reproduced within half a step, NaN does not
    take part in the row maximum and becomes 0."""
    rng = np.random.default_rng(3)
    w = rng.standard_normal((5, 64)).astype(np.float32)
    w[2] = 0.0
    w[3, 7] = np.nan
    q, scales = oracle.quantize_rows(w, 5, 64)
    assert scales[2] == 1.0 and not q[2].any()
    assert q[3, 7] == 0 and np.isfinite(scales[3])
    for r in (0, 1, 4):
        assert np.abs(q[r]).max() == 127
        assert np.all(np.abs(q[r].astype(np.float32) * scales[r] - w[r]) <= 0.5 * scales[r] * (1 + 1e-6))


def test_dot_lane_order_is_the_avx_one(oracle):
    """cpu.rs:231-254: lane j sums elements i = j (mod 8) unfused; lanes added 0..7; scalar tail."""
    rng = np.random.default_rng(5)
    for n in (8, 37, 768, 1600):
        a = rng.standard_normal(n).astype(np.float32)
        b = rng.standard_normal(n).astype(np.float32)
        lanes = np.zeros(8, np.float32)
        m = n // 8 * 8
        for i in range(0, m, 8):
            lanes = (lanes + (a[i:i + 8] * b[i:i + 8]).astype(np.float32)).astype(np.float32)
        s = np.float32(0.0)
        for j in range(8):
            s = np.float32(s + lanes[j])
        for i in range(m, n):
            s = np.float32(s + np.float32(a[i] * b[i]))
        assert oracle.dot(a, b) == float(s)


# ---- src/models/gpt2/rust.rs:1861-2013
def test_validates_weight_shapes(oracle):
    cfg, w = tiny()
    w["wte.weight"] = w["wte.weight"].reshape(-1)[:-1]
    with pytest.raises(oracle.OracleError) as e:
        oracle.Model(cfg, w)
    assert "wte len" in str(e.value)
    assert e.value.code == 4


def test_forward_returns_logits_for_each_position(oracle):
    cfg, w = tiny()
    out = oracle.Model(cfg, w).forward([1, 2, 3])
    assert out.shape == (3, cfg["vocab_size"])
    assert np.isfinite(out).all()


def test_greedy_generation_appends_tokens_until_context_limit(oracle):
    cfg, w = tiny()
    tokens = oracle.Model(cfg, w).generate_greedy([0, 1], 10)
    assert len(tokens) == cfg["n_positions"]
    assert tokens[:2] == [0, 1]
    assert all(t < cfg["vocab_size"] for t in tokens)


def test_cached_prefill_matches_full_forward_last_logits(oracle):
    cfg, w = tiny()
    model = oracle.Model(cfg, w)
    full = model.forward([1, 2, 3])
    cache = model.new_kv_cache()
    cached = model.prefill([1, 2, 3], cache)
    assert cache.seq_len == 3
    assert np.all(np.abs(full[-1] - cached) <= 1e-5)


def test_cached_greedy_generation_matches_full_generation(oracle):
    cfg, w = tiny()
    model = oracle.Model(cfg, w)
    assert model.generate_greedy_cached([0, 1], 3) == model.generate_greedy([0, 1], 3)


def test_streams_generated_tokens_in_order(oracle):
    cfg, w = tiny()
    streamed = []
    tokens = oracle.Model(cfg, w).generate_greedy_cached([0, 1], 3, on_token=lambda t: streamed.append(t))
    assert tokens[:2] == [0, 1]
    assert streamed == tokens[2:]


def test_gpt2_cache_exposes_generic_kv_cache_contract(oracle):
    cfg, w = tiny()
    cache = oracle.Model(cfg, w).new_kv_cache()
    cache.seq_len = 2
    assert cache.seq_len == 2
    assert cache.max_seq_len == cfg["n_positions"]
    cache.clear()
    assert cache.seq_len == 0


def test_threaded_rust_generation_matches_single_threaded(oracle):
    cfg, w = tiny()
    single = oracle.Model(cfg, w, threads=1).generate_greedy_cached([0, 1], 3)
    threaded = oracle.Model(cfg, w, threads=3).generate_greedy_cached([0, 1], 3)
    assert threaded == single


def test_threaded_logits_are_bit_identical_on_a_larger_model(oracle):
    """rust.rs:1511-1531: threads only re-assemble chunks; every element uses the same dot()."""
    cfg = synthetic.preset("midi")
    w = synthetic.perturbed_weights(cfg, 3)
    ids = synthetic.uniform_prompt(1, 9, cfg["vocab_size"])
    a = oracle.Model(cfg, w, threads=1)
    b = oracle.Model(cfg, w, threads=4, rust_config=dict(dense_parallel_threshold=1))
    la = a.prefill(ids, a.new_kv_cache())
    lb = b.prefill(ids, b.new_kv_cache())
    assert np.array_equal(la, lb)
    assert np.array_equal(a.forward(ids), b.forward(ids))


def test_quantized_rust_forward_returns_finite_logits(oracle):
    """rust.rs:1996-2013, plus what the reference's code implies for the quantised model: threads do not
    matter, cached == full, the batched loop is the same arithmetic, and the result stays close to FP32."""
    cfg = synthetic.preset("tiny")
    w = synthetic.tiny_weights(cfg)
    q = oracle.Model(cfg, w, quantized_weights=True)
    out = q.forward([1, 2, 3])
    assert out.shape == (3, cfg["vocab_size"]) and np.isfinite(out).all()
    assert np.array_equal(out, oracle.Model(cfg, w, threads=3, quantized_weights=True).forward([1, 2, 3]))
    cache = q.new_kv_cache()
    assert np.all(np.abs(q.prefill([1, 2, 3], cache) - out[-1]) <= 1e-5)

    cfg = synthetic.preset("mini")
    w = synthetic.perturbed_weights(cfg, 5)
    ids = synthetic.uniform_prompt(4, 9, cfg["vocab_size"])
    qm = oracle.Model(cfg, w, quantized_weights=True)
    c1, c2 = qm.new_kv_cache(), qm.new_kv_cache()
    qm.prefill(ids[:5], c1)
    qm.prefill(ids[:5], c2)
    one = np.stack([qm.forward_one(int(t), c) for t, c in ((ids[5], c1), (ids[6], c2))])
    c1.seq_len = c2.seq_len = 5
    both, am = qm.forward_one_batch([int(ids[5]), int(ids[6])], [c1, c2], want_logits=True)
    assert np.array_equal(one, both) and list(am) == [oracle.argmax_logits(r) for r in one]
    fp32 = oracle.Model(cfg, w).forward(ids)
    assert np.abs(qm.forward(ids) - fp32).max() < 0.05 * np.abs(fp32).max() + 0.05


def test_input_validation_messages(oracle):
    """rust.rs:1029-1051, 950-962"""
    cfg, w = tiny()
    model = oracle.Model(cfg, w)
    with pytest.raises(oracle.OracleError, match="input_ids must not be empty"):
        model.forward([])
    with pytest.raises(oracle.OracleError, match="sequence length 6 exceeds n_positions 5"):
        model.forward([0] * 6)
    with pytest.raises(oracle.OracleError, match="token id 8 at index 1 exceeds vocab_size 8"):
        model.forward([0, 8])
    cache = model.new_kv_cache()
    with pytest.raises(oracle.OracleError, match="token id 9 exceeds vocab_size 8"):
        model.forward_one(9, cache)
    model.prefill([0, 1, 2, 3, 4], cache)
    with pytest.raises(oracle.OracleError, match="cache is full at seq_len 5"):
        model.forward_one(1, cache)


def test_batched_loop_order_is_bit_identical(oracle):
    cfg = synthetic.preset("mini")
    w = synthetic.perturbed_weights(cfg, 1)
    model = oracle.Model(cfg, w, threads=2)
    prompts = [synthetic.uniform_prompt(s, 5 + s, cfg["vocab_size"]) for s in range(3)]
    singles, caches = [], []
    for p in prompts:
        c = model.new_kv_cache()
        model.prefill(p, c)
        caches.append(c)
        c2 = model.new_kv_cache()
        model.prefill(p, c2)
        singles.append(model.forward_one(7, c2))
    logits, am = model.forward_one_batch([7, 7, 7], caches, want_logits=True)
    for i in range(3):
        assert np.array_equal(logits[i], singles[i])
        assert am[i] == oracle.argmax_logits(singles[i])
        assert caches[i].seq_len == len(prompts[i]) + 1


# ---- src/models/generation.rs:364-404
def test_repeat_penalty_can_change_greedy_selection(oracle):
    g = oracle.generation_config(1, repeat_penalty=2.0)
    s = oracle.LogitsSampler(g.seed)
    assert s.select_next_token([1.0, 3.0, 2.0], [1], g) == 2


def test_top_k_one_samples_best_candidate(oracle):
    g = oracle.generation_config(1, temperature=1.0, top_k=1)
    s = oracle.LogitsSampler(g.seed)
    assert s.select_next_token([0.0, 10.0, 9.0], [], g) == 1


def test_validates_sampling_config(oracle):
    g = oracle.generation_config(1, top_p=2.0)
    with pytest.raises(oracle.OracleError):
        oracle.validate_generation_config(g)
    with pytest.raises(oracle.OracleError, match="top_k must be > 0"):
        oracle.validate_generation_config(oracle.generation_config(1, top_k=0))
    oracle.validate_generation_config(oracle.generation_config(1))


def test_argmax_ties_go_to_the_lowest_index(oracle):
    """generation.rs:269-279: strict > from -inf; NaN never wins."""
    assert oracle.argmax_logits([1.0, 5.0, 5.0, 2.0]) == 1
    assert oracle.argmax_logits([float("nan"), 1.0, float("nan")]) == 1
    assert oracle.argmax_logits([float("-inf")] * 3) == 0


def test_splitmix64_known_answers(oracle):
    """generation.rs:243-267 is SplitMix64 started at seed ^ golden-gamma. With seed = gamma the
    state starts at 0, and the published SplitMix64 sequence for state 0 is the known answer."""
    s = oracle.LogitsSampler(0x9E3779B97F4A7C15)
    assert [s.next_u64() for _ in range(3)] == [0xE220A8397B1DCDAF, 0x6E789E6AA1B965F4, 0x06C45D188009454F]


def test_sampler_draw_follows_the_cdf_walk(oracle):
    """generation.rs:300-362 re-derived in Python floats (f64) for one seeded draw sequence."""
    rng = np.random.default_rng(0)
    logits = rng.standard_normal(200).astype(np.float32)
    logits[5] = logits[9]  # a tie: the stable sort keeps index 5 first
    g = oracle.generation_config(1, temperature=0.8, top_k=40, seed=1234)
    s = oracle.LogitsSampler(g.seed)
    shadow = oracle.LogitsSampler(g.seed)
    order = sorted(range(200), key=lambda i: (-float(logits[i]), i))[:40]
    t = float(np.float32(0.8))
    mx = float(logits[order[0]]) / t
    import math
    w = [math.exp(float(logits[i]) / t - mx) for i in order]
    total = 0.0
    for x in w:
        total += x
    for _ in range(50):
        u = (shadow.next_u64() >> 11) * (1.0 / (1 << 53))
        target = u * total
        want = order[-1]
        for i, x in zip(order, w):
            target -= x
            if target <= 0.0:
                want = i
                break
        assert s.select_next_token(logits, [], g) == want


# ---- src/runtime/thread_pool.rs:107-170, 226-257
def test_pool_chunk_to_worker_mapping(oracle):
    assert oracle.pool_worker_chunks(4, 10, 3, 0) == [0]
    assert oracle.pool_worker_chunks(4, 10, 3, 3) == [3]
    assert oracle.pool_worker_chunks(2, 10, 3, 0) == [0, 2]
    assert oracle.pool_worker_chunks(2, 10, 3, 1) == [1, 3]
    assert oracle.pool_worker_chunks(1, 10, 3, 0) == [0, 1, 2, 3]
    assert oracle.pool_worker_chunks(4, 0, 3, 0) == []


def _pool_chunks(oracle, threads, length, chunk_size):
    """What parallel_chunks returns, in chunk order: the (start, end) every worker was given, merged by chunk index."""
    owned = sorted(c for w in range(threads) for c in oracle.pool_worker_chunks(threads, length, chunk_size, w))
    return [(c * chunk_size, min(length, (c + 1) * chunk_size)) for c in owned]


def test_parallel_chunks_preserves_order(oracle):
    """thread_pool.rs:230-237"""
    chunks = _pool_chunks(oracle, 4, 10, 3)
    assert [v for a, b in chunks for v in range(a, b)] == list(range(10))


def test_single_thread_chunks_preserve_order(oracle):
    """thread_pool.rs:239-245"""
    assert [sum(range(a, b)) for a, b in _pool_chunks(oracle, 1, 7, 2)] == [1, 5, 9, 6]


def test_cloned_pool_reuses_workers(oracle):
    """thread_pool.rs:247-256: chunk sizes of (4, 1) on two workers; a clone is the same pool, so the same mapping."""
    assert [b - a for a, b in _pool_chunks(oracle, 2, 4, 1)] == [1, 1, 1, 1]
    assert _pool_chunks(oracle, 2, 4, 1) == _pool_chunks(oracle, 2, 4, 1)
