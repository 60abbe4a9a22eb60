"""The generic decoding loop of puppygrad src/models/autoregressive.rs:61-87 over any object with
the AutoregressiveDecoder surface (max_context_len, new_cache, prefill, forward_one,
select_next_token)."""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence


def generate(model, input_ids: Sequence[int], max_new_tokens: int,
             on_token: Optional[Callable[[int], None]] = None) -> List[int]:
    cache = model.new_cache()
    logits = model.prefill(input_ids, cache)
    tokens = [int(t) for t in input_ids]
    for _ in range(max_new_tokens):
        if len(tokens) >= model.max_context_len():
            break
        nxt = model.select_next_token(logits)
        tokens.append(nxt)
        if on_token is not None:
            on_token(nxt)
        logits = model.forward_one(nxt, cache)
    return tokens
