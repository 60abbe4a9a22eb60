"""The reference's error type for this path (puppygrad src/models/gpt2/error.rs:4-25)."""
from __future__ import annotations

from . import _native as N


class Gpt2Error(Exception):
    """One of Asset / InvalidConfig / InvalidInput / InvalidWeights, plus Cuda and Timeout, which
    only this backend can raise. `str()` gives the same text as the reference's Display impl."""

    KINDS = {N.PG_ASSET: "Asset", N.PG_INVALID_CONFIG: "InvalidConfig", N.PG_INVALID_INPUT: "InvalidInput",
             N.PG_INVALID_WEIGHTS: "InvalidWeights", N.PG_CUDA: "Cuda", N.PG_TIMEOUT: "Timeout"}
    _PREFIX = {"Asset": "GPT-2 asset error: ", "InvalidConfig": "invalid GPT-2 config: ",
               "InvalidInput": "invalid GPT-2 input: ", "InvalidWeights": "invalid GPT-2 weights: ",
               "Cuda": "GPT-2 CUDA error: ", "Timeout": "GPT-2 device timeout: "}

    def __init__(self, kind: str, message: str):
        super().__init__(self._PREFIX.get(kind, "") + message)
        self.kind = kind
        self.message = message


def check(status: int) -> None:
    if status != N.PG_OK:
        raise Gpt2Error(Gpt2Error.KINDS.get(status, "Cuda"), N.lib.pg_last_error_message().decode())
