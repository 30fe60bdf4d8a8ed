"""GPU: INT8 ("SageAttention"-style) prefill attention through the C ABI against its CPU statement
(oracle/sage.py) and against exact attention."""
import ctypes as C

import numpy as np
import pytest
import torch

import cabi
from oracle import sage, synth

pytestmark = pytest.mark.gpu


def P(t):
    return C.c_void_p(t.data_ptr())


def make(S, off, qh, kvh, D, seed, k_bias=0.5):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(S, qh, D, generator=g).to(torch.bfloat16)
    k = (torch.randn(off + S, kvh, D, generator=g) + k_bias).to(torch.bfloat16)     # a common offset: what the centring removes
    v = torch.randn(off + S, kvh, D, generator=g).to(torch.bfloat16)
    return q, k, v


# 7B geometry (28 q / 4 kv heads, D 128) at ragged lengths, the 1.5B one with a resident prefix, D 64, tiny
@pytest.mark.parametrize("qh,kvh,D,S,off", [(28, 4, 128, 300, 0), (12, 2, 128, 256, 512), (14, 2, 64, 130, 61),
                                            (2, 1, 128, 1, 0), (4, 2, 64, 129, 0)])
def test_sage_attention_matches_its_cpu_statement(qh, kvh, D, S, off):
    L = cabi.lib()
    q, k, v = make(S, off, qh, kvh, D, seed=S + off)
    out = torch.zeros(S, qh, D, device="cuda", dtype=torch.bfloat16)
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    st = L.efm_b200_op_sage_prefill_attention(P(qd), P(kd), P(vd), P(out), S, off, qh, kvh, D)
    assert st == 0, L.efm_b200_last_error(None).decode()
    want = sage.sage_prefill_attention(q, k, v, off)
    exact = sage.exact_prefill_attention(q, k, v, off)
    got = out.float().cpu()
    scale = exact.abs().max().item()
    # same rule on both sides: bf16 output rounding plus the rare INT8 step that flips with the summation order of
    # the key mean
    assert (got - want).abs().max().item() <= 1.5e-2 * scale
    assert (got - want).abs().mean().item() <= 1e-3 * scale
    # the scheme itself against exact attention
    assert (got - exact).abs().max().item() <= 5e-2 * scale


def test_int8_prefill_inside_the_model_stays_inside_the_logit_bar():
    """Same prompt through the bf16 and the INT8 prefill attention: logits within the 2e-2 bar of each other and the
    first greedy token equal to the oracle's."""
    cfg = synth.tiny_config(num_layers=4, hidden=256, q_heads=4, kv_heads=2, intermediate=512, vocab=2000)
    w = synth.make_weights(cfg, seed=5)
    ids = synth.make_token_ids(200, seed=5, vocab=cfg.vocab)
    logits = {}
    for kind in (0, 1):
        be = cabi.Backend(cfg, max_prefill_tokens=256, max_response_tokens=8)
        be.load_weights(w)
        be.alloc_slot(0, 256)
        be.set_prefill_attention(kind)
        be.set_sampling(0.0, 1.0, 0)
        be.prefill(0, ids, sample=True)
        logits[kind] = be.read_logits()
        be.close()
    a, b = logits[0], logits[1]
    assert np.abs(a - b).max() / np.abs(a).max() < 2e-2
    from oracle import qwen_text
    o = qwen_text.QwenTextOracle(cfg, w, "exact_fp32")
    ref = o.forward(ids).numpy()
    assert np.abs(b - ref).max() / np.abs(ref).max() < 2e-2


def test_int8_prefill_needs_a_slot_first():
    cfg = synth.tiny_config()
    be = cabi.Backend(cfg, max_prefill_tokens=64, max_response_tokens=8)
    with pytest.raises(cabi.BackendError, match="KV slots"):
        be.set_prefill_attention(1)
    with pytest.raises(cabi.BackendError, match="kind"):
        be.set_prefill_attention(7)
    be.close()
