"""Single operators of the path on host arrays (kernel sweeps and operator-level parity tests)."""
from __future__ import annotations

import ctypes as C
from typing import Optional

import numpy as np

from . import _native as N
from .errors import check
from .gpt2 import _MATH

EPILOGUES = {"none": 0, "gelu": 1, "resid": 2}


def linear(x, w, bias=None, resid=None, epilogue: str = "none", math_mode: str = "fp32", device: int = 0,
           reps: int = 0):
    """out = x @ w.T (+ bias) with the epilogue fused; `w` is [out, in] like the reference keeps it
    after transpose_dense_weights. Returns (out, seconds_per_launch or None)."""
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(w, np.float32)
    m, k = x.shape
    n = w.shape[0]
    assert w.shape[1] == k
    out = np.empty((m, n), np.float32)
    fp = lambda a: a.ctypes.data_as(C.POINTER(C.c_float)) if a is not None else None
    bias = None if bias is None else np.ascontiguousarray(bias, np.float32)
    resid = None if resid is None else np.ascontiguousarray(resid, np.float32)
    sec = C.c_double(0.0)
    check(N.lib.pg_op_linear(fp(x), fp(w), fp(bias), fp(resid), m, n, k, EPILOGUES[epilogue], _MATH[math_mode],
                             device, reps, fp(out), C.byref(sec)))
    return out, (float(sec.value) if reps > 0 else None)


def layernorm(x, gamma, beta, eps: float = 1e-5, device: int = 0, reps: int = 0):
    """LayerNorm of every row of x [rows, cols] (layer_norm_in_place of the reference). Returns (out, seconds)."""
    x = np.ascontiguousarray(x, np.float32)
    gamma = np.ascontiguousarray(gamma, np.float32)
    beta = np.ascontiguousarray(beta, np.float32)
    rows, cols = x.shape
    out = np.empty_like(x)
    fp = lambda a: a.ctypes.data_as(C.POINTER(C.c_float))
    sec = C.c_double(0.0)
    check(N.lib.pg_op_layernorm(fp(x), fp(gamma), fp(beta), eps, rows, cols, device, reps, fp(out), C.byref(sec)))
    return out, (float(sec.value) if reps > 0 else None)


def lm_head_argmax(hidden, wte, want_logits: bool = True, device: int = 0, reps: int = 0):
    """logits = hidden @ wte.T (no bias) with the row arg-max found in the same pass; at most 8 rows.
    Returns (logits or None, argmax [m], seconds)."""
    hidden = np.ascontiguousarray(hidden, np.float32)
    wte = np.ascontiguousarray(wte, np.float32)
    m, k = hidden.shape
    v = wte.shape[0]
    assert wte.shape[1] == k
    logits = np.empty((m, v), np.float32) if want_logits else None
    am = np.empty(m, np.int32)
    fp = lambda a: a.ctypes.data_as(C.POINTER(C.c_float)) if a is not None else None
    sec = C.c_double(0.0)
    check(N.lib.pg_op_lm_head_argmax(fp(hidden), fp(wte), m, v, k, device, reps, fp(logits),
                                     am.ctypes.data_as(C.POINTER(C.c_int32)), C.byref(sec)))
    return logits, am, (float(sec.value) if reps > 0 else None)


def quantize_rows(w, device: int = 0):
    """Row-wise symmetric int8 quantisation on the device (QuantizedRows::from_f32 of the reference).
    w [rows, cols] -> (int8 [rows, cols], float32 scales [rows])."""
    w = np.ascontiguousarray(w, np.float32)
    rows, cols = w.shape
    q = np.empty((rows, cols), np.int8)
    scales = np.empty(rows, np.float32)
    check(N.lib.pg_op_quantize_rows(w.ctypes.data_as(C.POINTER(C.c_float)), rows, cols, device,
                                    q.ctypes.data_as(C.POINTER(C.c_int8)),
                                    scales.ctypes.data_as(C.POINTER(C.c_float))))
    return q, scales


def linear_q8(x, q, scales, bias=None, device: int = 0, reps: int = 0):
    """out = x @ dequant(q).T (+ bias) over int8 weights with one scale per output row (the
    reference's quantized projection); at most 8 rows of x. Returns (out, seconds_per_launch or None)."""
    x = np.ascontiguousarray(x, np.float32)
    q = np.ascontiguousarray(q, np.int8)
    scales = np.ascontiguousarray(scales, np.float32)
    m, k = x.shape
    n = q.shape[0]
    assert q.shape[1] == k and scales.shape == (n,)
    out = np.empty((m, n), np.float32)
    fp = lambda a: a.ctypes.data_as(C.POINTER(C.c_float)) if a is not None else None
    bias = None if bias is None else np.ascontiguousarray(bias, np.float32)
    sec = C.c_double(0.0)
    check(N.lib.pg_op_linear_q8(fp(x), q.ctypes.data_as(C.POINTER(C.c_int8)), fp(scales), fp(bias), m, n, k, device,
                                reps, fp(out), C.byref(sec)))
    return out, (float(sec.value) if reps > 0 else None)


def decode_attention(qkv, keys, values, page_tokens: int = 32, splits: int = 1, device: int = 0, reps: int = 0):
    """One new token per sequence against `kv_len` cached positions.
    qkv [batch, 3*c]; keys, values [batch, n_head, kv_len, head_dim]. Returns (out [batch, c], seconds)."""
    keys = np.ascontiguousarray(keys, np.float32)
    values = np.ascontiguousarray(values, np.float32)
    qkv = np.ascontiguousarray(qkv, np.float32)
    batch, n_head, kv_len, head_dim = keys.shape
    assert qkv.shape == (batch, 3 * n_head * head_dim)
    out = np.empty((batch, n_head * head_dim), np.float32)
    fp = lambda a: a.ctypes.data_as(C.POINTER(C.c_float))
    sec = C.c_double(0.0)
    check(N.lib.pg_op_decode_attention(fp(qkv), fp(keys), fp(values), batch, n_head, head_dim, kv_len, page_tokens,
                                       splits, device, reps, fp(out), C.byref(sec)))
    return out, (float(sec.value) if reps > 0 else None)


def decode_attention_noalloc(d_qkv: int, d_out: int, d_kv_pool: int, d_page_table: int, d_pos: int, batch: int,
                             n_head: int, head_dim: int, page_tokens: int, pages_per_seq: int, splits: int = 1,
                             device: int = 0, stream: int = 0) -> None:
    """Decode attention on device buffers the caller owns (arguments are raw device addresses),
    for callers that may not allocate device memory when they call: the kernel's split-K scratch
    is an array built into the library. Enqueues on `stream` and returns without waiting. Limits:
    batch * n_head <= 2048, splits <= 8. Calls on one device must not overlap on the GPU."""
    check(N.lib.pg_decode_attention_noalloc(d_qkv, d_out, d_kv_pool, d_page_table, d_pos, batch, n_head, head_dim,
                                            page_tokens, pages_per_seq, splits, device, stream or None))
