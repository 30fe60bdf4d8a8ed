"""GPU: the allocation-free decode-attention entry point.

Some callers of this library cannot allocate device memory when they need attention (a control
loop with a fixed memory footprint, a plugin inside another runtime's pool).  For them
efm_b200_op_decode_attention_noalloc keeps the split-KV scratch in an array built into the
library.  Here it is called through the C ABI twice in a row, on different inputs, and each
result is compared with the allocating entry point on the same inputs and with fp32 torch; shapes
beyond the built-in scratch must be refused.  Slots of more than 2048 rows take the split-KV form
whose partial outputs, softmax statistics and tickets really live in the built-in array (shorter
slots merge through distributed shared memory and only clear the tickets).  Collected last so that
a failure here cannot hide another test."""
import ctypes as C
import math

import pytest
import torch

import cabi

pytestmark = pytest.mark.gpu


def P(t):
    return C.c_void_p(t.data_ptr())


def bf16(*shape, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn(*shape, generator=g, device="cuda").to(torch.bfloat16)


def attention_fp32(q, k, v, kv_len):
    """softmax(q K^T / sqrt(D)) V over the first kv_len cache rows, fp32; q [qh, D], k / v [T, kvh, D]."""
    qh, D = q.shape
    g = qh // k.shape[1]
    K = k[:kv_len].float().repeat_interleave(g, dim=1)
    V = v[:kv_len].float().repeat_interleave(g, dim=1)
    s = torch.einsum("hd,thd->ht", q.float(), K) / math.sqrt(D)
    return torch.einsum("ht,thd->hd", torch.softmax(s, dim=-1), V)


# the last three slots are longer than 2048 rows: split-KV through the built-in scratch (up to 64 chunks)
@pytest.mark.parametrize("qh,kvh,D,max_tokens,lens", [(12, 2, 128, 1024, (769, 770)), (14, 2, 64, 256, (193, 7)),
                                                      (28, 4, 128, 1580, (1325, 1580)), (8, 1, 64, 5000, (100, 4999)),
                                                      (12, 2, 128, 4096, (4096, 2049)), (32, 16, 128, 2304, (2304, 1))])
def test_noalloc_matches_allocating_entry_point_twice(qh, kvh, D, max_tokens, lens):
    L = cabi.lib()
    for call, kv_len in enumerate(lens):               # two calls in a row share the built-in scratch
        q = bf16(qh, D, seed=100 + call)
        k, v = bf16(max_tokens, kvh, D, seed=200 + call), bf16(max_tokens, kvh, D, seed=300 + call)
        want = torch.zeros(qh, D, device="cuda", dtype=torch.bfloat16)
        got = torch.full((qh, D), float("nan"), device="cuda", dtype=torch.bfloat16)
        assert L.efm_b200_op_decode_attention(P(q), P(k), P(v), P(want), qh, kvh, D, kv_len, max_tokens) == 0
        st = L.efm_b200_op_decode_attention_noalloc(P(q), P(k), P(v), P(got), qh, kvh, D, kv_len, max_tokens)
        assert st == 0, L.efm_b200_last_error(None).decode()
        assert torch.allclose(got.float(), want.float(), atol=1e-2, rtol=2e-2)
        assert torch.equal(got, want)                   # same kernel, same split plan: bit-identical
        ref = attention_fp32(q, k, v, kv_len)
        assert torch.allclose(got.float(), ref, atol=1e-2, rtol=2e-2)


def test_noalloc_refuses_shapes_beyond_its_scratch():
    L = cabi.lib()
    qh, kvh, D, T = 40, 5, 128, 64                      # 40 * 128 = 5120 > 4096
    q, k, v = bf16(qh, D, seed=1), bf16(T, kvh, D, seed=2), bf16(T, kvh, D, seed=3)
    out = torch.zeros(qh, D, device="cuda", dtype=torch.bfloat16)
    st = L.efm_b200_op_decode_attention_noalloc(P(q), P(k), P(v), P(out), qh, kvh, D, T, T)
    assert st == 5                                      # EFM_ERR_UNSUPPORTED
    assert b"built-in scratch" in L.efm_b200_last_error(None)
    assert L.efm_b200_op_decode_attention(P(q), P(k), P(v), P(out), qh, kvh, D, T, T) == 0
