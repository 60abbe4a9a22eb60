"""Operator-level GPU parity: single kernels through the C ABI against the CPU oracle's kernels
(shapes of the GPT-2 XL kernel sweep, reduced where the oracle would take long)."""
import numpy as np
import pytest

import puppygrad_b200 as pg
from puppygrad_b200 import ops

pytestmark = pytest.mark.gpu


def oracle_linear(oracle, x, w, b, epilogue, resid):
    m, k = x.shape
    n = w.shape[0]
    out = oracle.transposed_dense_projection(x.reshape(-1), m, k, n, w.reshape(-1), b).reshape(m, n)
    if epilogue == "gelu":
        out = oracle.gelu(out).reshape(m, n)
    if epilogue == "resid":
        out = (resid + out).astype(np.float32)  # add_in_place: dst += src
    return out


# FP32 path: 1e-3 relative / 1e-4 absolute on values of magnitude sqrt(k).
@pytest.mark.parametrize("m,n,k", [(1, 4800, 1600), (8, 1600, 1600), (64, 6400, 1600), (3, 1600, 6400),
                                   (5, 50257, 768), (2, 7, 37), (300, 200, 96)])
@pytest.mark.parametrize("epilogue", ["none", "gelu", "resid"])
def test_linear_fp32_matches_oracle(oracle, m, n, k, epilogue):
    rng = np.random.default_rng(m * 31 + n * 7 + k)
    x = rng.standard_normal((m, k), dtype=np.float32)
    w = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.05)
    b = rng.standard_normal(n, dtype=np.float32)
    r = rng.standard_normal((m, n), dtype=np.float32)
    got, _ = ops.linear(x, w, b, r if epilogue == "resid" else None, epilogue, "fp32")
    np.testing.assert_allclose(got, oracle_linear(oracle, x, w, b, epilogue, r), rtol=1e-3, atol=1e-4)


@pytest.mark.parametrize("m,n,k", [(9, 4800, 1600), (16, 1600, 1600), (64, 6400, 1600), (33, 1600, 6400),
                                   (64, 50257, 1024), (40, 1000, 256)])
@pytest.mark.parametrize("epilogue", ["none", "gelu", "resid"])
def test_linear_tf32x3_matches_oracle(oracle, m, n, k, epilogue):
    """Three TF32 tensor-core products with FP32 accumulation: the same bound as the FP32 path."""
    rng = np.random.default_rng(m * 31 + n * 7 + k + 1)
    x = rng.standard_normal((m, k), dtype=np.float32)
    w = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.05)
    b = rng.standard_normal(n, dtype=np.float32)
    r = rng.standard_normal((m, n), dtype=np.float32)
    got, _ = ops.linear(x, w, b, r if epilogue == "resid" else None, epilogue, "tf32x3")
    np.testing.assert_allclose(got, oracle_linear(oracle, x, w, b, epilogue, r), rtol=1e-3, atol=1e-4)


@pytest.mark.parametrize("m,n,k", [(128, 1600, 1600), (512, 4800, 1600), (300, 1600, 6400), (1000, 777, 256)])
@pytest.mark.parametrize("epilogue", ["none", "gelu", "resid"])
def test_linear_tf32x3_prefill_sized_matches_oracle(oracle, m, n, k, epilogue):
    """More than 64 rows: hi and lo parts of both operands from shared memory, three TF32 MMAs per k step into
    two accumulators (the hi.hi products and the small terms). Same bound as the FP32 path; row and column
    counts that are not multiples of the 128 x 128 tile included."""
    rng = np.random.default_rng(m * 13 + n * 5 + k + 2)
    x = rng.standard_normal((m, k), dtype=np.float32)
    w = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.05)
    b = rng.standard_normal(n, dtype=np.float32)
    r = rng.standard_normal((m, n), dtype=np.float32)
    got, _ = ops.linear(x, w, b, r if epilogue == "resid" else None, epilogue, "tf32x3")
    np.testing.assert_allclose(got, oracle_linear(oracle, x, w, b, epilogue, r), rtol=1e-3, atol=1e-4)


@pytest.mark.parametrize("m,n,k", [(16, 1600, 1600), (64, 6400, 1600), (33, 1600, 6400), (40, 1000, 256)])
@pytest.mark.parametrize("epilogue", ["none", "gelu", "resid"])
def test_linear_tf32x3_one_launch_per_gemm_kernel_matches_oracle(oracle, monkeypatch, m, n, k, epilogue):
    """The same product on the kernel that is launched once per GEMM (split-K over a thread-block
    cluster), which the model keeps for shapes the persistent chain kernel does not take."""
    monkeypatch.setenv("PG_NO_CHAIN", "1")
    rng = np.random.default_rng(m * 31 + n * 7 + k + 2)
    x = rng.standard_normal((m, k), dtype=np.float32)
    w = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.05)
    b = rng.standard_normal(n, dtype=np.float32)
    r = rng.standard_normal((m, n), dtype=np.float32)
    got, _ = ops.linear(x, w, b, r if epilogue == "resid" else None, epilogue, "tf32x3")
    np.testing.assert_allclose(got, oracle_linear(oracle, x, w, b, epilogue, r), rtol=1e-3, atol=1e-4)


@pytest.mark.parametrize("m,n,k,epilogue", [(128, 128, 32, "none"), (512, 4800, 1600, "none"), (1000, 770, 768, "none"),
                                            (4096, 1600, 6400, "none"), (1000, 770, 768, "gelu"),
                                            (2300, 768, 3072, "resid"), (300, 771, 64, "resid"), (129, 515, 96, "gelu")])
def test_linear_tf32_single_pass_is_within_its_stated_bound(oracle, m, n, k, epilogue):
    """One TF32 pass (10-bit mantissas, truncated): error <= 2e-3 of the output scale
    sqrt(k) * |x| * |w|, the looser bound of the TF32 prefill variant. Ragged row and column
    counts (odd n takes the scalar store path of the epilogue), all three epilogues."""
    rng = np.random.default_rng(m + n + k)
    x = rng.standard_normal((m, k), dtype=np.float32)
    w = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.05)
    b = rng.standard_normal(n, dtype=np.float32)
    r = rng.standard_normal((m, n), dtype=np.float32) if epilogue == "resid" else None
    got, _ = ops.linear(x, w, b, r, epilogue, "tf32")
    rows = slice(0, min(m, 64))
    want = oracle_linear(oracle, x[rows], w, b, epilogue, None if r is None else r[rows])
    scale = float(np.abs(want).max())
    assert np.abs(got[rows] - want).max() <= 2e-3 * scale
    full = x.astype(np.float64) @ w.astype(np.float64).T + b
    if epilogue == "gelu":
        full = 0.5 * full * (1 + np.tanh(0.7978845608028654 * (full + 0.044715 * full ** 3)))
    if epilogue == "resid":
        full = full + r
    assert np.abs(got - full).max() <= 2e-3 * np.abs(full).max()


# ---- int8 row-quantised weights (the reference's --quantized-weights variant)
@pytest.mark.parametrize("rows,cols", [(4, 3), (37, 768), (300, 1600), (5, 6400)])
def test_quantize_rows_is_bit_identical_to_oracle(oracle, rows, cols):
    """QuantizedRows::from_f32 (cpu.rs:33-57) on the device: integer / byte work, so the bytes and the
    scales must equal the oracle's exactly, including an all-zero row and a NaN entry."""
    rng = np.random.default_rng(rows + cols)
    w = (rng.standard_normal((rows, cols)) * 0.02).astype(np.float32)
    w[rows // 2] = 0.0
    w[0, cols - 1] = np.nan
    w[rows - 1, 0] = 3.0   # one dominant value: the rest of the row quantises to small integers
    q, scales = ops.quantize_rows(w)
    oq, oscales = oracle.quantize_rows(w, rows, cols)
    assert np.array_equal(scales, oscales)
    assert np.array_equal(q, oq)


@pytest.mark.parametrize("m,n,k,with_bias", [(1, 4800, 1600, True), (8, 1600, 6400, True), (3, 50257, 768, False),
                                             (2, 7, 48, True), (5, 3072, 768, True)])
def test_linear_q8_matches_oracle(oracle, m, n, k, with_bias):
    """quantized_transposed_dense_projection_into (cpu.rs:99-117): FP32 activations against int8 rows
    dequantised on the fly. Same tolerance as the FP32 linears (1e-3 relative, 1e-4 absolute): the
    kernel sums in a different order and applies the row scale after the sum."""
    rng = np.random.default_rng(m + n + k)
    x = rng.standard_normal((m, k), dtype=np.float32)
    w = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.05)
    b = rng.standard_normal(n, dtype=np.float32) if with_bias else None
    q, scales = oracle.quantize_rows(w, n, k)
    got, _ = ops.linear_q8(x, q, scales, b)
    want = oracle.quantized_projection(x, m, k, n, q, scales, b if with_bias else np.zeros(n, np.float32)).reshape(m, n)
    np.testing.assert_allclose(got, want, rtol=1e-3, atol=1e-4)


def test_linear_q8_rejects_prefill_sized_inputs():
    x = np.zeros((9, 32), np.float32)
    q = np.zeros((4, 32), np.int8)
    with pytest.raises(pg.Gpt2Error, match="m <= 8"):
        ops.linear_q8(x, q, np.ones(4, np.float32))
    with pytest.raises(pg.Gpt2Error, match="multiple of 16"):
        ops.linear_q8(np.zeros((1, 24), np.float32), np.zeros((4, 24), np.int8), np.ones(4, np.float32))


def oracle_attention(oracle, qkv, keys, values):
    """cached_self_attention_into (rust.rs:1662-1741) restated with the oracle's kernels: scalar
    sequential score sums, oracle softmax, value accumulation in key order."""
    batch, n_head, kv_len, d = keys.shape
    c = n_head * d
    out = np.zeros((batch, c), np.float32)
    scale = np.float32(1.0) / np.sqrt(np.float32(d))
    for b in range(batch):
        for h in range(n_head):
            q = qkv[b, h * d:(h + 1) * d]
            k_all = np.concatenate([keys[b, h], qkv[b, c + h * d:c + (h + 1) * d][None]], 0)
            v_all = np.concatenate([values[b, h], qkv[b, 2 * c + h * d:2 * c + (h + 1) * d][None]], 0)
            scores = np.array([np.float32(oracle.dot_scalar(q, k_all[i])) * scale for i in range(kv_len + 1)],
                              np.float32)
            p = oracle.softmax(scores)
            acc = np.zeros(d, np.float32)
            for i in range(kv_len + 1):
                acc = (acc + p[i] * v_all[i]).astype(np.float32)
            out[b, h * d:(h + 1) * d] = acc
    return out


@pytest.mark.parametrize("batch,n_head,d,kv_len,page,splits", [
    (1, 25, 64, 128, 32, 1), (3, 25, 64, 255, 16, 4), (2, 12, 64, 1023, 64, 8), (32, 4, 64, 300, 32, 2),
    (2, 3, 8, 17, 16, 1), (1, 2, 64, 0, 32, 1), (4, 16, 64, 31, 32, 16)])
def test_decode_attention_matches_oracle(oracle, batch, n_head, d, kv_len, page, splits):
    rng = np.random.default_rng(batch + n_head + kv_len)
    qkv = rng.standard_normal((batch, 3 * n_head * d), dtype=np.float32)
    keys = rng.standard_normal((batch, n_head, kv_len, d), dtype=np.float32)
    values = rng.standard_normal((batch, n_head, kv_len, d), dtype=np.float32)
    got, _ = ops.decode_attention(qkv, keys, values, page_tokens=page, splits=splits)
    np.testing.assert_allclose(got, oracle_attention(oracle, qkv, keys, values), rtol=1e-3, atol=1e-4)


@pytest.mark.parametrize("rows", [1, 7, 300])
def test_layernorm_operator_matches_oracle(oracle, rows):
    """layer_norm_in_place (cpu.rs:119-143) at the width of GPT-2 XL."""
    rng = np.random.default_rng(rows)
    d = 1600
    x = rng.standard_normal((rows, d), dtype=np.float32) * 3 + 0.5
    g = rng.standard_normal(d, dtype=np.float32)
    b = rng.standard_normal(d, dtype=np.float32)
    got, _ = ops.layernorm(x, g, b, 1e-5)
    want = oracle.layer_norm(x, rows, d, g, b, 1e-5).reshape(rows, d)
    np.testing.assert_allclose(got, want, rtol=1e-3, atol=1e-4)


@pytest.mark.parametrize("m", [1, 3, 8])
def test_lm_head_with_fused_argmax_matches_oracle(oracle, m):
    """logits_from_hidden_into (rust.rs:1767-1813) + argmax_logits (generation.rs:269-279), 1600 -> 50257."""
    rng = np.random.default_rng(m)
    k, v = 1600, 50257
    h = rng.standard_normal((m, k), dtype=np.float32)
    w = rng.standard_normal((v, k), dtype=np.float32) * 0.02
    w[4321] = w[1234]  # an exact tie must go to the lower index
    h[0] = w[1234] * 40  # ... and be the row maximum of the first row
    logits, am, _ = ops.lm_head_argmax(h, w)
    want = oracle.transposed_dense_projection(h, m, k, v, w, np.zeros(v, np.float32)).reshape(m, v)
    np.testing.assert_allclose(logits, want, rtol=1e-3, atol=1e-4)
    assert list(am) == [oracle.argmax_logits(r) for r in want] and am[0] == 1234
    _, am2, _ = ops.lm_head_argmax(h, w, want_logits=False)
    assert list(am2) == list(am)
