"""The allocation-free decode attention entry point against the ordinary one.

Some callers cannot call cudaMalloc at the moment they need a decode step (their own pool owns all
device memory, or their embedder forbids allocation there). `pg_decode_attention_noalloc` serves
them: inputs and outputs are the caller's device buffers and the kernel's split-K scratch is an
array inside the library. This file is collected last on purpose, so that a run that stops at the
first failure has already run every other test.
"""
import numpy as np
import pytest

from puppygrad_b200 import ops

pytestmark = pytest.mark.gpu


def paged_pool(keys, values, page_tokens, pages_per_seq):
    """[page][2][head][page_tokens][head_dim] with the identity page table."""
    batch, n_head, kv_len, d = keys.shape
    pool = np.zeros((batch * pages_per_seq, 2, n_head, page_tokens, d), np.float32)
    table = np.arange(batch * pages_per_seq, dtype=np.int32).reshape(batch, pages_per_seq)
    for b in range(batch):
        for p in range(kv_len):
            pool[table[b, p // page_tokens], 0, :, p % page_tokens] = keys[b, :, p]
            pool[table[b, p // page_tokens], 1, :, p % page_tokens] = values[b, :, p]
    return pool, table


def attention_f64(qkv, keys, values):
    """cached_self_attention_into (rust.rs:1662-1741) in float64: the new token's q against the cached keys and
    its own key, softmax, weighted values."""
    batch, n_head, kv_len, d = keys.shape
    c = n_head * d
    out = np.zeros((batch, c))
    for b in range(batch):
        for h in range(n_head):
            q = qkv[b, h * d:(h + 1) * d].astype(np.float64)
            k_all = np.concatenate([keys[b, h], qkv[b, c + h * d:c + (h + 1) * d][None]], 0).astype(np.float64)
            v_all = np.concatenate([values[b, h], qkv[b, 2 * c + h * d:2 * c + (h + 1) * d][None]], 0).astype(np.float64)
            s = k_all @ q / np.sqrt(d)
            p = np.exp(s - s.max())
            out[b, h * d:(h + 1) * d] = (p / p.sum()) @ v_all
    return out


@pytest.mark.parametrize("batch,n_head,d,kv_len,page,splits,own_stream",
                         [(3, 25, 64, 200, 32, 4, False), (64, 16, 64, 129, 16, 2, True), (5, 6, 32, 70, 32, 3, False),
                          (2, 12, 64, 1000, 64, 8, True)])
def test_noalloc_entry_point_matches_the_allocating_one_twice_in_a_row(batch, n_head, d, kv_len, page, splits, own_stream):
    """Against the allocating entry point (same kernel, scratch from cudaMalloc) and against a float64 restatement
    of the reference's attention; twice in a row, because the built-in scratch keeps the last call's contents.
    head_dim 32 takes the generic kernel (one split, no scratch); own_stream runs the call on a stream of the
    caller's instead of the default stream."""
    import torch
    rng = np.random.default_rng(kv_len)
    qkv = rng.standard_normal((batch, 3 * n_head * d), dtype=np.float32)
    keys = rng.standard_normal((batch, n_head, kv_len, d), dtype=np.float32)
    values = rng.standard_normal((batch, n_head, kv_len, d), dtype=np.float32)
    want, _ = ops.decode_attention(qkv, keys, values, page_tokens=page, splits=splits)
    np.testing.assert_allclose(want, attention_f64(qkv, keys, values), rtol=1e-3, atol=1e-4)

    pages_per_seq = (kv_len + 1 + page - 1) // page
    pool, table = paged_pool(keys, values, page, pages_per_seq)
    dev = torch.device("cuda", 0)
    t_qkv = torch.from_numpy(qkv).to(dev)
    t_pool = torch.from_numpy(pool).to(dev)
    t_table = torch.from_numpy(table).to(dev)
    t_pos = torch.full((batch,), kv_len, dtype=torch.int32, device=dev)
    stream = torch.cuda.Stream(device=dev) if own_stream else None
    torch.cuda.synchronize()
    for call in range(2):  # the built-in scratch keeps the last call's contents: call twice
        t_out = torch.full((batch, n_head * d), float("nan"), device=dev)
        torch.cuda.synchronize()
        ops.decode_attention_noalloc(t_qkv.data_ptr(), t_out.data_ptr(), t_pool.data_ptr(), t_table.data_ptr(),
                                     t_pos.data_ptr(), batch, n_head, d, page, pages_per_seq, splits,
                                     stream=stream.cuda_stream if stream else 0)
        torch.cuda.synchronize()
        got = t_out.cpu().numpy()
        np.testing.assert_allclose(got, want, rtol=1e-3, atol=1e-4, err_msg=f"call {call}")
    # the new token's K and V were appended to the caller's pool
    c = n_head * d
    new_page = table[0, kv_len // page]
    k_new = t_pool[new_page, 0, :, kv_len % page].cpu().numpy().reshape(-1)
    np.testing.assert_array_equal(k_new, qkv[0, c:2 * c])


def test_noalloc_entry_point_rejects_sizes_beyond_its_scratch():
    import torch
    from puppygrad_b200 import Gpt2Error
    z = torch.zeros(16, device="cuda")
    zi = torch.zeros(16, dtype=torch.int32, device="cuda")
    with pytest.raises(Gpt2Error, match="exceeds the built-in scratch limit of 2048"):
        ops.decode_attention_noalloc(z.data_ptr(), z.data_ptr(), z.data_ptr(), zi.data_ptr(), zi.data_ptr(),
                                     100, 25, 64, 32, 4, 1)
    with pytest.raises(Gpt2Error, match="exceeds the built-in scratch limit of 8"):
        ops.decode_attention_noalloc(z.data_ptr(), z.data_ptr(), z.data_ptr(), zi.data_ptr(), zi.data_ptr(),
                                     1, 2, 64, 32, 4, 16)
