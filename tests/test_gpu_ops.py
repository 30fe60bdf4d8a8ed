"""GPU: every kernel on its own, through the C ABI, against fp32 torch on the same inputs.
Shapes are those of the benchmark configurations (0.5B / 1.5B / 3B / 7B) plus ragged cases."""
import ctypes as C
import math

import numpy as np
import pytest
import torch

import cabi
from oracle import sampling

pytestmark = pytest.mark.gpu


def P(t):
    return C.c_void_p(t.data_ptr())


def ok(st):
    assert st == 0, cabi.lib().efm_b200_last_error(None).decode()


def bf16(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


# n, k of: 0.5B qkv / o / down, 1.5B qkv / down, 7B o_proj, tiny ragged
GEMV_SHAPES = [(1152, 896), (896, 896), (896, 4864), (2048, 1536), (1536, 8960), (3584, 3584), (256, 128), (10, 72)]


@pytest.mark.parametrize("n,k", GEMV_SHAPES)
def test_gemv_plain(n, k):
    L = cabi.lib()
    w, x = bf16(n, k, scale=0.02, seed=1), bf16(k, seed=2)
    y = torch.zeros(n, device="cuda", dtype=torch.bfloat16)
    ok(L.efm_b200_op_gemv(P(w), P(x), None, 0.0, P(y), None, n, k))
    ref = (w.double() @ x.double()).float()
    assert torch.allclose(y.float(), ref, atol=2e-3, rtol=1e-2)
    # bf16 rounding of the exact fp32 result: at most one ulp off
    assert (y.float() - ref.to(torch.bfloat16).float()).abs().max() <= ref.abs().max() * 2 ** -7


@pytest.mark.parametrize("n,k", [(1152, 896), (2048, 1536), (4608, 3584), (256, 128)])
def test_gemv_rmsnorm_prologue_and_residual_epilogue(n, k):
    L = cabi.lib()
    w, x, g = bf16(n, k, scale=0.02, seed=3), bf16(k, seed=4), (1 + 0.02 * torch.randn(k, device="cuda")).to(torch.bfloat16)
    eps = 1e-6
    xf = x.float()                        # the norm prologue reads the residual stream in fp32 and keeps it fp32
    xn = xf * torch.rsqrt(xf.pow(2).mean() + eps) * g.float()
    y = torch.zeros(n, device="cuda", dtype=torch.bfloat16)
    ok(L.efm_b200_op_gemv(P(w), P(xf), P(g), eps, P(y), None, n, k))
    ref = (w.double() @ xn.double()).float()
    assert (y.float() - ref.to(torch.bfloat16).float()).abs().max() <= ref.abs().max() * 2 ** -7      # one bf16 ulp of the output
    # residual epilogue: r (fp32) += W x
    xb = xn.to(torch.bfloat16)
    refb = (w.double() @ xb.double()).float()
    r0 = torch.randn(n, device="cuda")
    r = r0.clone()
    ok(L.efm_b200_op_gemv(P(w), P(xb), None, 0.0, None, P(r), n, k))
    assert torch.allclose(r, r0 + refb, atol=1e-4, rtol=1e-4)


# the last three have a few more output tiles than a multiple of the SM count: their tail tiles are split along K
@pytest.mark.parametrize("m,n,k", [(64, 1152, 896), (256, 2048, 1536), (320, 2048, 2048), (1324, 4608, 3584),
                                   (200, 896, 4864), (1, 256, 128), (131, 130, 96),
                                   (1324, 3584, 3584), (1300, 3600, 4096), (1323, 3584, 18944)])
def test_prefill_gemm(m, n, k):
    L = cabi.lib()
    x, w, b = bf16(m, k, seed=6), bf16(n, k, scale=0.02, seed=7), bf16(n, scale=0.02, seed=8)
    y = torch.zeros(m, n, device="cuda", dtype=torch.bfloat16)
    ok(L.efm_b200_op_gemm(P(x), P(w), P(b), P(y), m, n, k))
    ref = x.float() @ w.float().T + b.float()
    assert torch.allclose(y.float(), ref, atol=1e-2, rtol=2e-2)
    y2 = torch.zeros_like(y)
    ok(L.efm_b200_op_gemm(P(x), P(w), None, P(y2), m, n, k))
    assert torch.allclose(y2.float(), x.float() @ w.float().T, atol=1e-2, rtol=2e-2)


def attention_ref(q, k, v, kv_len):
    """q [S, qh, D]; k, v [T, kvh, D]; query i sees rows [0, kv_len - S + i]."""
    S, qh, D = q.shape
    g = qh // k.shape[1]
    K = k[:kv_len].float().repeat_interleave(g, dim=1)
    V = v[:kv_len].float().repeat_interleave(g, dim=1)
    s = torch.einsum("shd,thd->hst", q.float(), K) / math.sqrt(D)
    qpos = torch.arange(kv_len - S, kv_len, device=q.device)[:, None]
    mask = torch.arange(kv_len, device=q.device)[None, :] <= qpos
    s = s.masked_fill(~mask[None], float("-inf"))
    return torch.einsum("hst,thd->shd", torch.softmax(s, dim=-1), V)


# (q heads, kv heads, D, kv_len, max_tokens): 0.5B, 1.5B, 3B, 7B geometries + edge lengths
@pytest.mark.parametrize("qh,kvh,D,kv_len,max_tokens", [
    (14, 2, 64, 193, 256), (12, 2, 128, 769, 1024), (16, 2, 128, 321, 448), (28, 4, 128, 1325, 1580),
    (2, 1, 64, 1, 64), (2, 1, 64, 33, 64), (4, 2, 128, 64, 64), (8, 1, 64, 100, 5000)])
def test_decode_attention(qh, kvh, D, kv_len, max_tokens):
    L = cabi.lib()
    q = bf16(qh, D, seed=9)
    k, v = bf16(max_tokens, kvh, D, seed=10), bf16(max_tokens, kvh, D, seed=11)
    k[kv_len:] = float("nan")        # rows past kv_len must never be read
    v[kv_len:] = float("nan")
    out = torch.zeros(qh, D, device="cuda", dtype=torch.bfloat16)
    for _ in range(2):               # twice: the split counters must come back to zero
        ok(L.efm_b200_op_decode_attention(P(q), P(k), P(v), P(out), qh, kvh, D, kv_len, max_tokens))
        ref = attention_ref(q[None], k, v, kv_len)[0]
        assert torch.allclose(out.float(), ref, atol=1e-2, rtol=2e-2)


@pytest.mark.parametrize("qh,kvh,D,S,off", [(14, 2, 64, 64, 128), (12, 2, 128, 256, 512), (28, 4, 128, 200, 0),
                                            (2, 1, 64, 1, 0), (2, 1, 64, 7, 3), (28, 4, 128, 1324, 0), (4, 2, 64, 300, 131)])
def test_prefill_attention(qh, kvh, D, S, off):
    L = cabi.lib()
    T = off + S
    q = bf16(S, qh, D, seed=12)
    k, v = bf16(T, kvh, D, seed=13), bf16(T, kvh, D, seed=14)
    out = torch.zeros(S, qh, D, device="cuda", dtype=torch.bfloat16)
    ok(L.efm_b200_op_prefill_attention(P(q), P(k), P(v), P(out), S, off, qh, kvh, D))
    ref = attention_ref(q, k, v, T)
    assert torch.allclose(out.float(), ref, atol=1e-2, rtol=2e-2)


def run_sampler(logits, temperature, top_p, seed, step):
    L = cabi.lib()
    s = cabi.Sampling(temperature, top_p, 1, 0, seed)
    tok = torch.zeros(1, device="cuda", dtype=torch.int32)
    ok(L.efm_b200_op_sample(C.cast(logits.data_ptr(), C.POINTER(C.c_float)), logits.numel(), C.byref(s), step,
                            C.cast(tok.data_ptr(), C.POINTER(C.c_int32))))
    return int(tok.item())


def test_sampler_greedy_ties_and_argmax():
    g = torch.Generator(device="cuda").manual_seed(0)
    for vocab in (151936, 1000, 2):
        l = torch.randn(vocab, generator=g, device="cuda")
        assert run_sampler(l, 0.0, 1.0, 0, 0) == int(torch.argmax(l))
    l = torch.zeros(151936, device="cuda")
    l[[77, 4000, 150000]] = 5.0
    assert run_sampler(l, 0.0, 1.0, 0, 0) == 77


@pytest.mark.parametrize("vocab,temperature,top_p", [(151936, 0.7, 0.9), (151936, 1.0, 1.0), (1000, 0.7, 0.9),
                                                     (2000, 0.3, 0.5), (151936, 0.7, 0.05)])
def test_sampler_top_p_equals_oracle(vocab, temperature, top_p):
    """Bit-equal ids with the CPU statement of the sampling rule, over many RNG steps."""
    rng = np.random.default_rng(vocab)
    l = (rng.standard_normal(vocab) * 0.8).astype(np.float32)
    ld = torch.from_numpy(l).cuda()
    multi = 0
    for step in range(24):
        want, rounds = sampling.sample_top_p(l, temperature, top_p, 1234, step, return_rounds=True)
        multi += rounds > 1
        assert run_sampler(ld, temperature, top_p, 1234, step) == want
    if top_p <= 0.5:
        assert multi > 0             # the rejection path was exercised


def test_sampler_ties_at_the_nucleus_edge():
    l = np.zeros(64, dtype=np.float32)        # all equal: nucleus = the first ceil(0.5 * 64) ids
    ld = torch.from_numpy(l).cuda()
    seen = set()
    for step in range(200):
        want = sampling.sample_top_p(l, 1.0, 0.5, 7, step)
        got = run_sampler(ld, 1.0, 0.5, 7, step)
        assert got == want
        seen.add(got)
    assert max(seen) < 32


def peer_words(vals, count):
    """[n_parts, k] fp32 -> the exchange's 8-byte words {fp32 value (low half), count (high half)}."""
    w = torch.empty(vals.shape + (2,), dtype=torch.int32, device="cuda")
    w[..., 0] = vals.view(torch.int32)
    w[..., 1] = count
    return w.contiguous()


@pytest.mark.parametrize("n,k,parts", [(512, 896, 2), (1024, 3584, 8)])
def test_peer_consumer_sums_the_partials_in_rank_order(n, k, parts):
    """Consumer side of the tensor-parallel decode exchange on one GPU: x = resid + p0 + p1 + ..., then norm + GEMV."""
    L = cabi.lib()
    g = torch.Generator(device="cuda").manual_seed(21)
    w, nw = bf16(n, k, scale=0.02, seed=22), (1 + 0.02 * torch.randn(k, device="cuda", generator=g)).to(torch.bfloat16)
    resid = torch.randn(k, device="cuda", generator=g)
    vals = torch.randn(parts, k, device="cuda", generator=g)
    words = peer_words(vals, 7)
    y = torch.zeros(n, device="cuda", dtype=torch.bfloat16)
    rout = torch.zeros(k, device="cuda")
    ok(L.efm_b200_op_gemv_peer_consume(P(w), P(resid), P(nw), 1e-6, P(words), parts, 7, 200_000, P(y), P(rout), n, k))
    acc = torch.zeros(k, device="cuda")
    for r in range(parts):
        acc = acc + vals[r]
    x = resid + acc
    assert torch.equal(rout, x)                       # same order of additions: bit-identical
    xn = x * torch.rsqrt(x.pow(2).mean() + 1e-6) * nw.float()
    ref = (w.double() @ xn.double()).float()
    assert (y.float() - ref.to(torch.bfloat16).float()).abs().max() <= ref.abs().max() * 2 ** -7


def test_peer_wait_runs_out_and_the_device_stays_usable():
    """Failure detection without a fault: one word of one partial never receives the awaited count (as if its rank
    were lost).  The kernel's wait is bounded in TIME and in total, so the call must come back promptly with
    EFM_ERR_DEVICE_WAIT, and the next call on the same device must work."""
    import time
    L = cabi.lib()
    n, k, parts = 512, 1536, 4
    g = torch.Generator(device="cuda").manual_seed(23)
    w, nw = bf16(n, k, scale=0.02, seed=24), torch.ones(k, device="cuda", dtype=torch.bfloat16)
    resid = torch.randn(k, device="cuda", generator=g)
    vals = torch.randn(parts, k, device="cuda", generator=g)
    words = peer_words(vals, 5)
    words[2, 100, 1] = 4                              # rank 2 is one exchange behind on one value, forever
    y = torch.zeros(n, device="cuda", dtype=torch.bfloat16)
    rout = torch.zeros(k, device="cuda")
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    st = L.efm_b200_op_gemv_peer_consume(P(w), P(resid), P(nw), 1e-6, P(words), parts, 5, 20_000, P(y), P(rout), n, k)
    waited = time.perf_counter() - t0
    assert st == 6 and b"ran out" in L.efm_b200_last_error(None)          # EFM_ERR_DEVICE_WAIT
    assert waited < 2.0, waited                       # 20 ms budget for the whole kernel, not per wait
    words[2, 100, 1] = 5                              # the word arrives: same call succeeds, device still usable
    ok(L.efm_b200_op_gemv_peer_consume(P(w), P(resid), P(nw), 1e-6, P(words), parts, 5, 20_000, P(y), P(rout), n, k))
    assert torch.equal(rout, resid + (((vals[0] + vals[1]) + vals[2]) + vals[3]))
