"""Host-side mirror of the reference's text streaming helpers (puppygrad src/models/streaming.rs) over the C ABI.

A `TokenDecoder` here is any object with `decode_tokens(token_ids) -> str` (the reference's trait,
streaming.rs:1-9; its `decode_token` default decodes a one-element list). The tokenizer itself is the
caller's: GPT-2's needs a `tokenizer.json`, which this library neither ships nor reads.
"""
from __future__ import annotations

import ctypes as C
from typing import Callable, Sequence

import numpy as np

from . import _native as N
from .errors import check


def is_incremental_decode_safe(token_text: str) -> bool:
    """streaming.rs:76-78"""
    b = token_text.encode("utf-8", "surrogatepass")
    return bool(N.lib.pg_is_incremental_decode_safe(b, len(b)))


def escape_raw_token(token: str) -> str:
    """streaming.rs:17-30"""
    b = token.encode("utf-8")
    n = C.c_size_t()
    buf = C.create_string_buffer(6 * len(b) + 16)
    check(N.lib.pg_escape_raw_token(b, len(b), buf, len(buf), C.byref(n)))
    return buf.raw[:n.value].decode("utf-8")


class IncrementalTextStreamer:
    """streaming.rs:32-74"""

    def __init__(self, decoded: str = ""):
        b = decoded.encode("utf-8")
        self._h = C.c_void_p()
        check(N.lib.pg_text_streamer_new(b, len(b), C.byref(self._h)))

    def __del__(self):
        if getattr(self, "_h", None):
            N.lib.pg_text_streamer_free(self._h)
            self._h = None

    def decoded(self) -> str:
        text, n = C.c_char_p(), C.c_size_t()
        check(N.lib.pg_text_streamer_decoded(self._h, C.byref(text), C.byref(n)))
        return C.string_at(text, n.value).decode("utf-8", "replace")

    def stream_token(self, decoder, output_ids: Sequence[int], token_id: int, on_text: Callable[[str], None]) -> None:
        errors = []

        def decode(ids, n, out, cap, out_len, _user):
            try:
                b = decoder.decode_tokens([int(ids[i]) for i in range(n)]).encode("utf-8")
            except Exception as exc:  # the decoder's error becomes the call's error
                errors.append(exc)
                return 1
            out_len[0] = len(b)
            if len(b) <= cap:
                C.memmove(out, b, len(b))
            return 0

        def text(ptr, n, _user):
            try:
                on_text(C.string_at(ptr, n).decode("utf-8", "replace"))
            except Exception as exc:
                errors.append(exc)
                return 1
            return 0

        ids = np.ascontiguousarray(output_ids, np.uint64)
        rc = N.lib.pg_text_streamer_stream_token(self._h, N.DECODE_TOKENS_FN(decode), None,
                                                 ids.ctypes.data_as(C.POINTER(C.c_uint64)), ids.size, int(token_id),
                                                 N.TEXT_CALLBACK(text), None)
        if errors:
            raise errors[0]
        check(rc)
