"""ctypes binding of `libpuppygrad_b200.so` (the C ABI in include/puppygrad_b200.h).

There is no fallback: if the library is missing, importing this module raises, and every compute
call fails with `Gpt2Error` when no sm_100 device is present.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libpuppygrad_b200.so")

PG_OK, PG_ASSET, PG_INVALID_CONFIG, PG_INVALID_INPUT, PG_INVALID_WEIGHTS, PG_CUDA, PG_TIMEOUT = range(7)


class PgConfig(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in
                ("vocab_size", "n_positions", "n_embd", "n_layer", "n_head", "n_inner")] + \
               [("layer_norm_epsilon", C.c_float)]


class PgBackendConfig(C.Structure):
    _fields_ = [("device", C.c_int32), ("math_mode", C.c_int32), ("page_tokens", C.c_int32),
                ("use_graphs", C.c_int32), ("attn_splits", C.c_int32), ("persistent_step", C.c_int32),
                ("quantized_weights", C.c_int32), ("reserved", C.c_int32 * 1)]


class PgGenerationConfig(C.Structure):
    _fields_ = [("max_new_tokens", C.c_uint64), ("eos_token_id", C.c_int64),
                ("temperature", C.c_float), ("top_p", C.c_float), ("top_k", C.c_int64),
                ("seed", C.c_uint64), ("repeat_penalty", C.c_float), ("repeat_last_n", C.c_uint64)]


class PgGenerationStats(C.Structure):
    _fields_ = [("prompt_tokens", C.c_uint64), ("generated_tokens", C.c_uint64),
                ("tokenize_time", C.c_double), ("prefill_time", C.c_double),
                ("decode_time", C.c_double), ("total_generation_time", C.c_double),
                ("first_token_time", C.c_double)]


class PgOperationProfile(C.Structure):
    _fields_ = [(n, C.c_double) for n in
                ("tokenization", "layer_norm", "qkv_projection", "attention", "attention_projection",
                 "mlp_fc_projection", "mlp_projection", "final_logits", "decoding", "other")] + \
               [("launches", C.c_uint64 * 8), ("fused_step_kernel", C.c_double), ("fused_phases", C.c_uint64)]


TOKEN_CALLBACK = C.CFUNCTYPE(C.c_int, C.c_uint64, C.c_void_p)
DECODE_TOKENS_FN = C.CFUNCTYPE(C.c_int, C.POINTER(C.c_uint64), C.c_size_t, C.POINTER(C.c_char), C.c_size_t,
                               C.POINTER(C.c_size_t), C.c_void_p)
TEXT_CALLBACK = C.CFUNCTYPE(C.c_int, C.POINTER(C.c_char), C.c_size_t, C.c_void_p)

_fp, _ip = C.POINTER(C.c_float), C.POINTER(C.c_int32)
_u64p, _vp = C.POINTER(C.c_uint64), C.c_void_p

# name -> (restype, argtypes); one entry per declaration in include/puppygrad_b200.h
SIGNATURES = {
    "pg_last_error_message": (C.c_char_p, []),
    "pg_version": (C.c_char_p, []),
    "pg_device_count": (C.c_int, []),
    "pg_config_validate": (C.c_int, [C.POINTER(PgConfig)]),
    "pg_config_load_json": (C.c_int, [C.c_char_p, C.POINTER(PgConfig)]),
    "pg_generation_config_default": (None, [C.c_uint64, C.POINTER(PgGenerationConfig)]),
    "pg_generation_config_validate": (C.c_int, [C.POINTER(PgGenerationConfig)]),
    "pg_backend_config_default": (None, [C.POINTER(PgBackendConfig)]),
    "pg_model_load_dir": (C.c_int, [C.c_char_p, C.POINTER(PgBackendConfig), C.POINTER(_vp)]),
    "pg_model_from_host_weights": (C.c_int, [C.POINTER(PgConfig), C.POINTER(_fp), _u64p, C.c_uint64,
                                             C.POINTER(PgBackendConfig), C.POINTER(_vp)]),
    "pg_model_config": (C.c_int, [_vp, C.POINTER(PgConfig)]),
    "pg_model_max_context_len": (C.c_uint64, [_vp]),
    "pg_model_weight_bytes_per_step": (C.c_uint64, [_vp]),
    "pg_model_free": (None, [_vp]),
    "pg_cache_new": (C.c_int, [_vp, C.c_int32, C.POINTER(_vp)]),
    "pg_cache_clear": (C.c_int, [_vp]),
    "pg_cache_clear_slot": (C.c_int, [_vp, C.c_int32]),
    "pg_cache_seq_len": (C.c_int, [_vp, C.c_int32, _u64p]),
    "pg_cache_max_seq_len": (C.c_uint64, [_vp]),
    "pg_cache_max_batch": (C.c_int32, [_vp]),
    "pg_cache_read_layer": (C.c_int, [_vp, C.c_int32, C.c_uint64, _fp, _fp]),
    "pg_cache_free": (None, [_vp]),
    "pg_prefill": (C.c_int, [_vp, _vp, _ip, _ip, C.c_int32, _fp, _ip]),
    "pg_forward_one": (C.c_int, [_vp, _vp, _ip, C.c_int32, _fp, _ip, _fp, _ip, C.c_int32]),
    "pg_forward": (C.c_int, [_vp, _ip, C.c_int32, _fp]),
    "pg_decode_greedy": (C.c_int, [_vp, _vp, _ip, C.c_int32, C.c_int32, _ip]),
    "pg_profile_forward_one": (C.c_int, [_vp, _vp, _ip, C.c_int32, C.POINTER(PgOperationProfile)]),
    "pg_cache_time_begin": (C.c_int, [_vp]),
    "pg_cache_time_end": (C.c_int, [_vp, C.POINTER(C.c_double)]),
    "pg_cache_kernel_launches": (C.c_uint64, [_vp]),
    "pg_cache_debug_expire_next_wait": (C.c_int, [_vp, C.c_uint32]),
    "pg_op_linear": (C.c_int, [_fp, _fp, _fp, _fp, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                               C.c_int32, C.c_int32, _fp, C.POINTER(C.c_double)]),
    "pg_op_decode_attention": (C.c_int, [_fp, _fp, _fp, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                         C.c_int32, C.c_int32, C.c_int32, _fp, C.POINTER(C.c_double)]),
    "pg_op_layernorm": (C.c_int, [_fp, _fp, _fp, C.c_float, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _fp,
                                  C.POINTER(C.c_double)]),
    "pg_op_lm_head_argmax": (C.c_int, [_fp, _fp, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _fp, _ip,
                                       C.POINTER(C.c_double)]),
    "pg_op_quantize_rows": (C.c_int, [_fp, C.c_int32, C.c_int32, C.c_int32, C.POINTER(C.c_int8), _fp]),
    "pg_op_linear_q8": (C.c_int, [_fp, C.POINTER(C.c_int8), _fp, _fp, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                  C.c_int32, _fp, C.POINTER(C.c_double)]),
    "pg_decode_attention_noalloc": (C.c_int, [_vp, _vp, _vp, _vp, _vp, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                              C.c_int32, C.c_int32, C.c_int32, _vp]),
    "pg_generate_greedy": (C.c_int, [_vp, _ip, C.c_int32, C.c_uint64, _ip, _u64p]),
    "pg_stream_greedy_tokens": (C.c_int, [_vp, _ip, C.c_int32, C.c_uint64, TOKEN_CALLBACK, _vp, _ip, _u64p]),
    "pg_generate_with_config": (C.c_int, [_vp, _ip, C.c_int32, C.POINTER(PgGenerationConfig), TOKEN_CALLBACK,
                                          _vp, _ip, _u64p, C.POINTER(PgGenerationStats)]),
    "pg_text_streamer_new": (C.c_int, [C.c_char_p, C.c_size_t, C.POINTER(_vp)]),
    "pg_text_streamer_free": (None, [_vp]),
    "pg_text_streamer_decoded": (C.c_int, [_vp, C.POINTER(C.c_char_p), C.POINTER(C.c_size_t)]),
    "pg_text_streamer_stream_token": (C.c_int, [_vp, DECODE_TOKENS_FN, _vp, _u64p, C.c_size_t, C.c_uint64,
                                                TEXT_CALLBACK, _vp]),
    "pg_is_incremental_decode_safe": (C.c_int, [C.c_char_p, C.c_size_t]),
    "pg_escape_raw_token": (C.c_int, [C.c_char_p, C.c_size_t, C.c_char_p, C.c_size_t, C.POINTER(C.c_size_t)]),
    "pg_generation_stats_total_model_tokens": (C.c_uint64, [C.POINTER(PgGenerationStats)]),
    "pg_generation_stats_prefill_tokens_per_second": (C.c_double, [C.POINTER(PgGenerationStats)]),
    "pg_generation_stats_decode_tokens_per_second": (C.c_double, [C.POINTER(PgGenerationStats)]),
    "pg_generation_stats_total_tokens_per_second": (C.c_double, [C.POINTER(PgGenerationStats)]),
    "pg_generation_stats_average_decode_token_time": (C.c_double, [C.POINTER(PgGenerationStats)]),
    "pg_argmax_logits": (C.c_uint64, [_fp, C.c_size_t]),
    "pg_sampler_new": (C.c_int, [C.c_uint64, C.POINTER(_vp)]),
    "pg_sampler_free": (None, [_vp]),
    "pg_sampler_select_next_token": (C.c_int, [_vp, _fp, C.c_size_t, _u64p, C.c_size_t,
                                               C.POINTER(PgGenerationConfig), _u64p]),
    "pg_sampler_select_from_topk": (C.c_int, [_vp, _fp, _ip, C.c_size_t, C.POINTER(PgGenerationConfig), _u64p]),
    "pg_sampler_select_from_topk_batch": (C.c_int, [C.POINTER(C.c_void_p), _fp, _ip, C.c_size_t, C.c_size_t,
                                                      C.POINTER(PgGenerationConfig), _u64p]),
}


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m puppygrad_b200.build` "
            "(needs nvcc); there is no CPU fallback")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


class _Library:
    """Loads the shared library on first use, so that `python -m puppygrad_b200.build` can run
    before the library exists. Any call without the library raises ImportError."""
    _lib = None

    def __getattr__(self, name):
        if _Library._lib is None:
            _Library._lib = _load()
        return getattr(_Library._lib, name)


lib = _Library()
