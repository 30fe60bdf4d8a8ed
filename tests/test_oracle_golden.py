"""CPU: the oracle against the committed Hugging Face golden vectors and known-answer vectors."""
import os

import numpy as np
import pytest
import torch

from oracle import qwen_text, sampling, synth

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
CASES = {
    "qwen2_tiny_tied": (dict(num_layers=2, hidden=128, q_heads=2, kv_heads=1, intermediate=256, vocab=1000, tied=True), 0),
    "qwen2_small_untied": (dict(num_layers=3, hidden=256, q_heads=4, kv_heads=2, intermediate=512, vocab=2000,
                                tied=False, rope_theta=1e4), 1),
}


def load_case(name):
    kw, seed = CASES[name]
    g = np.load(os.path.join(GOLDEN, name + ".npz"))
    cfg = synth.tiny_config(**kw)
    return cfg, synth.make_weights(cfg, seed=seed), g


@pytest.mark.parametrize("name", sorted(CASES))
def test_exact_fp32_oracle_reproduces_hf(name):
    cfg, w, g = load_case(name)
    o = qwen_text.QwenTextOracle(cfg, w, "exact_fp32")
    r = qwen_text.generate(o, g["prompt"].tolist(), len(g["tokens"]))
    assert r.tokens == g["tokens"].tolist()            # the reference's own bar: exact greedy ids vs HF
    lg = torch.stack(r.logits).numpy()
    rel = np.abs(lg - g["logits"]).max(axis=1) / np.abs(g["logits"]).max(axis=1)
    assert rel.max() < 1e-5


@pytest.mark.parametrize("name", sorted(CASES))
def test_bf16_points_oracle_within_tolerance_of_hf(name):
    cfg, w, g = load_case(name)
    o = qwen_text.QwenTextOracle(cfg, w, "bf16_points")
    r = qwen_text.generate(o, g["prompt"].tolist(), len(g["tokens"]), forced=g["tokens"].tolist())
    lg = torch.stack(r.logits).numpy()
    rel = np.abs(lg - g["logits"]).max(axis=1) / np.abs(g["logits"]).max(axis=1)
    assert rel.max() < 2e-2                            # logits tolerance of the workload definition


def test_prefix_then_suffix_equals_one_prefill():
    cfg, w, g = load_case("qwen2_tiny_tied")
    prompt = g["prompt"].tolist()
    a = qwen_text.QwenTextOracle(cfg, w, "exact_fp32")
    la = a.forward(prompt)
    b = qwen_text.QwenTextOracle(cfg, w, "exact_fp32")
    b.forward(prompt[:5])
    lb = b.forward(prompt[5:])
    assert torch.allclose(la, lb, atol=1e-5)


def test_decode_equals_prefill_of_longer_sequence():
    cfg, w, g = load_case("qwen2_small_untied")
    prompt = g["prompt"].tolist()
    a = qwen_text.QwenTextOracle(cfg, w, "exact_fp32")
    a.forward(prompt[:-1])
    la = a.forward(prompt[-1:])
    b = qwen_text.QwenTextOracle(cfg, w, "exact_fp32")
    lb = b.forward(prompt)
    assert torch.allclose(la, lb, atol=1e-5)


def test_mrope_with_equal_rows_is_plain_rope():
    kw = dict(num_layers=2, hidden=128, q_heads=2, kv_heads=1, intermediate=256, vocab=1000, tied=True)
    cfg_t = synth.tiny_config(**kw)
    cfg_m = synth.tiny_config(**kw, mrope_section=[8, 12, 12])
    w = synth.make_weights(cfg_t, seed=3)
    ids = synth.make_token_ids(9, seed=3, vocab=1000)
    pos = torch.arange(9).repeat(3, 1)
    lt = qwen_text.QwenTextOracle(cfg_t, w, "exact_fp32").forward(ids)
    lm = qwen_text.QwenTextOracle(cfg_m, w, "exact_fp32").forward(ids, position_ids=pos)
    assert torch.allclose(lt, lm, atol=1e-6)


def test_embedding_injection_rule():
    cfg, w, _ = load_case("qwen2_tiny_tied")
    o = qwen_text.QwenTextOracle(cfg, w, "exact_fp32")
    emb = torch.randn(3, cfg.hidden).to(torch.bfloat16)
    rows = o.embed_tokens([5, 2000, 2002, 2003, -1], emb, 2000)
    assert torch.equal(rows[0], o.embed[5])
    assert torch.equal(rows[1], emb[0].float()) and torch.equal(rows[2], emb[2].float())
    assert rows[3].abs().sum() == 0 and rows[4].abs().sum() == 0      # outside both ranges -> zeros


def test_philox_known_answers():
    # Random123 known-answer vectors for philox4x32-10
    assert sampling.philox4x32_10([0, 0, 0, 0], [0, 0]) == [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]
    assert sampling.philox4x32_10([0xffffffff] * 4, [0xffffffff] * 2) == [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]
    assert sampling.philox4x32_10([0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344], [0xa4093822, 0x299f31d0]) == \
        [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1]


def test_greedy_tie_rule_lowest_index():
    l = np.zeros(50, dtype=np.float32)
    l[[7, 19]] = 3.0
    assert sampling.sample_top_p(l, 0.0, 1.0, 0, 0) == 7
    assert qwen_text.greedy(torch.from_numpy(l)) == 7


def test_top_p_distribution_is_the_renormalised_nucleus():
    l = np.array([2.0, 1.0, 0.5, 0.0, -1.0, 1.0], dtype=np.float32)
    counts = np.zeros(6)
    n = 6000
    for s in range(n):
        counts[sampling.sample_top_p(l, 1.0, 0.8, 1, s)] += 1
    p = np.exp(l - l.max())
    p /= p.sum()
    nucleus = [0, 1, 5]                                  # 0.466 + 0.172 + 0.172 >= 0.8; ties by lower id
    assert counts[[2, 3, 4]].sum() == 0
    expect = p[nucleus] / p[nucleus].sum()
    assert np.abs(counts[nucleus] / n - expect).max() < 0.02


def test_top_p_one_keeps_every_token_with_weight():
    rng = np.random.default_rng(0)
    l = rng.standard_normal(300).astype(np.float32)
    seen = {sampling.sample_top_p(l, 1.5, 1.0, 5, s) for s in range(3000)}
    assert len(seen) > 250


def test_synthetic_checkpoint_roundtrip(tmp_path):
    from safetensors.torch import load_file
    cfg = synth.tiny_config()
    w = synth.make_weights(cfg, seed=0)
    d = synth.write_checkpoint(str(tmp_path / "m"), cfg, w)
    back = load_file(os.path.join(d, "model.safetensors"))
    assert set(back) == set(w) and all(torch.equal(back[k], w[k]) for k in w)
    w2 = synth.make_weights(cfg, seed=0)
    assert all(torch.equal(w[k], w2[k]) for k in w)      # seeded: identical on every machine


# ---- vision tower: pinned to transformers' Qwen2_5_VisionTransformerPretrainedModel ---------------------
@pytest.mark.parametrize("case", ["one_window", "ragged", "frames_and_image"])
def test_vit_oracle_reproduces_hf_outputs(case):
    from oracle import qwen_vit
    z = np.load(os.path.join(os.path.dirname(__file__), "golden", "qwen_vit_tiny.npz"))
    cfg = qwen_vit.VitConfig(**eval(str(z["cfg"])))
    w = qwen_vit.make_weights(cfg, seed=int(z["seed"]))
    grids = [tuple(g) for g in z[case + "_grids"].tolist()]
    px = qwen_vit.make_pixels(cfg, grids, seed=int(z["seed"]))
    want = z[case + "_out"]
    got = qwen_vit.VitOracle(cfg, w, "exact_fp32").forward(px, grids).numpy()
    assert np.abs(got - want).max() < 2e-5
    got_b = qwen_vit.VitOracle(cfg, w, "bf16_points").forward(px, grids).numpy()
    assert np.abs(got_b - want).max() < 1e-2             # bf16 rounding points only


def test_vit_plan_windows_of_the_benchmark_images():
    from oracle import qwen_vit
    cfg = qwen_vit.CONFIGS[2]
    p = qwen_vit.make_plan(cfg, [qwen_vit.GRIDS[2]])      # 448x448: 16 windows of 64 patches
    lens = np.diff(p.cu_window)
    assert len(lens) == 16 and set(lens) == {64} and sorted(p.order) == list(range(256))
    p = qwen_vit.make_plan(cfg, [qwen_vit.GRIDS[3]])      # 1288x728: 92x52 patches, 84 windows
    lens = np.diff(p.cu_window)
    assert len(lens) == 84 and set(lens) == {64, 32, 16} and lens.sum() == 4784
    assert sorted(p.order) == list(range(1196)) and p.cu_full == [0, 4784]
    assert max(p.pos_h) == 51 and max(p.pos_w) == 91


# ---- INT8 prefill attention: properties of the CPU statement (no reference vectors exist for it) -------------
def test_sage_statement_properties():
    from oracle import sage
    g = torch.Generator().manual_seed(11)
    S, off, qh, kvh, D = 150, 40, 4, 2, 128
    q = torch.randn(S, qh, D, generator=g).to(torch.bfloat16)
    k = (torch.randn(off + S, kvh, D, generator=g) + 2.0).to(torch.bfloat16)      # large common offset
    v = torch.randn(off + S, kvh, D, generator=g).to(torch.bfloat16)
    exact = sage.exact_prefill_attention(q, k, v, off)
    got = sage.sage_prefill_attention(q, k, v, off)
    assert (got - exact).abs().max() < 5e-2 * exact.abs().max()
    # quantisation: |x - q * scale| <= scale / 2, scale = max|x| / 127 per 128-token block and head
    x = torch.randn(300, 3, 64, generator=g)
    qi, sc = sage.quantize_blocks(x)
    assert qi.abs().max() == 127 and sc.shape == (3, 3)
    err = (x - qi.float() * sc[torch.arange(300) // 128][:, :, None]).abs()
    assert (err <= sc[torch.arange(300) // 128][:, :, None] * 0.5 + 1e-7).all()
    # the first query sees exactly keys [0, off]: row 0 equals plain softmax attention over them to INT8 accuracy
    one = sage.sage_prefill_attention(q[:1], k[:off + 1], v[:off + 1], off)
    assert (one - exact[:1]).abs().max() < 5e-2 * exact.abs().max()
