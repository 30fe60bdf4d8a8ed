"""GPU: group-wise INT4 (W4A16) decode weights.  Prefill (and the first sampled token) runs on the bf16 checkpoint,
every decode step on the INT4 copy of the linears (two checkpoints, the reference's prefill_model_path /
decode_model_path).  Oracle: the fp32 text oracle with the de-quantised weights for the decode steps, sharing the KV
cache the bf16 oracle prefilled.  Tolerances: logits within 2e-2 relative of that oracle (the kernel keeps fp16
products inside a 16-column chunk, as the reference's kernel keeps its whole row sum in fp16); a differing greedy id
must sit inside twice the observed logit error."""
import numpy as np
import pytest
import torch

import cabi
from oracle import int4, qwen_text, synth

pytestmark = pytest.mark.gpu


def oracle_run(cfg, w, deq, prompt, steps, forced, pos=None, last=None):
    """Prefill on the bf16 weights, decode on the de-quantised ones, one KV cache."""
    a = qwen_text.QwenTextOracle(cfg, w, "exact_fp32")
    b = qwen_text.QwenTextOracle(cfg, deq, "exact_fp32")
    pt = None if pos is None else torch.tensor(pos)
    logits = [a.forward(prompt, position_ids=pt)]
    b.k_cache, b.v_cache = a.k_cache, a.v_cache
    for s in range(steps - 1):
        p3 = None if pos is None else torch.full((3, 1), last + 1 + s)
        logits.append(b.forward([forced[s]], position_ids=p3))
    return logits


@pytest.mark.parametrize("kw,lm_head", [
    (dict(num_layers=2, hidden=256, q_heads=4, kv_heads=2, intermediate=512, vocab=1500, tied=True), True),
    (dict(num_layers=3, hidden=384, q_heads=6, kv_heads=2, intermediate=1152, vocab=2000, tied=False), True),
    (dict(num_layers=2, hidden=512, q_heads=4, kv_heads=2, intermediate=640, vocab=1200, tied=True,
          mrope_section=[16, 24, 24], model_type="qwen2_5_vl"), False),
    # one layer at the 7B shape's widths (K = 3584 / 18944, head_dim 128): the sizes at which the kernel is bandwidth-relevant
    (dict(num_layers=1, hidden=3584, q_heads=28, kv_heads=4, intermediate=18944, vocab=2048, tied=False), True),
], ids=["h256", "h384-untied", "h512-mrope", "layer_7b_width"])
def test_int4_decode_against_the_oracle(kw, lm_head):
    cfg = synth.tiny_config(**kw)
    w = synth.make_weights(cfg, seed=12)
    packed, deq = int4.quantize_checkpoint(w, cfg.num_layers, lm_head=lm_head)
    be = cabi.Backend(cfg)
    be.load_weights_partial(w)
    be.load_decode_weights_int4(packed)
    be.finalize()
    be.alloc_slot(0, 128)
    be.set_sampling(0.0, 1.0, 0)
    n, steps = 19, 10
    prompt = synth.make_token_ids(n, seed=13, vocab=cfg.vocab)
    pos = [list(range(n))] * 3 if cfg.mrope_section is not None else None
    toks, logits = cabi.generate(be, 0, prompt, steps, pos3=pos, collect_logits=True)
    graph, _ = cabi.generate(be, 0, prompt, steps, pos3=pos, use_graph=True)
    assert graph == toks                                        # captured decode graph == plain launches
    int4_bytes, bf16_bytes = be.decode_step_bytes(n + 1), None
    ref = oracle_run(cfg, w, deq, prompt, steps, toks, pos, n - 1)
    for s in range(steps):
        r = ref[s].numpy()
        err = np.abs(logits[s] - r).max()
        assert err / np.abs(r).max() < 2e-2, (s, err / np.abs(r).max())
        if toks[s] != qwen_text.greedy(ref[s]):
            assert qwen_text.top2_margin(ref[s]) <= 2 * err, s
    be.close()
    # the step streams about a quarter of the bf16 linear bytes
    bf = cabi.Backend(cfg)
    bf.load_weights(w)
    bf.alloc_slot(0, 128)
    bf16_bytes = bf.decode_step_bytes(n + 1)
    bf.close()
    assert int4_bytes < 0.45 * bf16_bytes if lm_head else int4_bytes < bf16_bytes


def test_int4_weights_are_all_or_nothing():
    cfg = synth.tiny_config(num_layers=2, hidden=256, q_heads=4, kv_heads=2, intermediate=512, vocab=1500)
    w = synth.make_weights(cfg, seed=12)
    packed, _ = int4.quantize_checkpoint(w, cfg.num_layers)
    del packed["model.layers.1.mlp.down_proj.qweight"], packed["model.layers.1.mlp.down_proj.scaling_factors"]
    be = cabi.Backend(cfg)
    be.load_weights_partial(w)
    be.load_decode_weights_int4(packed)
    with pytest.raises(cabi.BackendError, match="every layer"):
        be.finalize()
    be.close()


def test_int4_decode_checkpoint_through_the_public_api(tmp_path, built):
    """decode_model_path names a second checkpoint directory holding the INT4 tensors: the engine prefills with the
    bf16 checkpoint and decodes with the INT4 one; same tokens as the C-ABI path with the same two weight sets."""
    import json
    import edge_fm
    from safetensors.torch import save_file
    cfg = synth.tiny_config(num_layers=2, hidden=256, q_heads=4, kv_heads=2, intermediate=512, vocab=1500)
    w = synth.make_weights(cfg, seed=14)
    packed, _ = int4.quantize_checkpoint(w, cfg.num_layers)
    model_dir = synth.write_checkpoint(str(tmp_path / "bf16"), cfg, w)
    dec_dir = tmp_path / "int4"
    dec_dir.mkdir()
    json.dump(cfg.hf_config(), open(dec_dir / "config.json", "w"))
    save_file({k: v.contiguous() for k, v in packed.items()}, str(dec_dir / "model.safetensors"))
    prompt = synth.make_token_ids(17, seed=15, vocab=cfg.vocab)
    path = synth.write_engine_config(str(tmp_path / "engine.json"), model_dir, max_tokens=64, max_new_tokens=9)
    ej = json.load(open(path))
    ej["decode_model_path"] = str(dec_dir)
    json.dump(ej, open(path, "w"))
    eng = edge_fm.EdgeFM(path)
    req = edge_fm.Request(0, prompt)
    req.set_ignore_stop_tokens(True)
    got = list(eng.generate(req).token_ids())
    del eng
    be = cabi.Backend(cfg)
    be.load_weights_partial(w)
    be.load_decode_weights_int4(packed)
    be.finalize()
    be.alloc_slot(0, 64)
    be.set_sampling(0.0, 1.0, 0)
    want, _ = cabi.generate(be, 0, prompt, 9)
    be.close()
    assert got == want
    plain = cabi.Backend(cfg)
    plain.load_weights(w)
    plain.alloc_slot(0, 64)
    plain.set_sampling(0.0, 1.0, 0)
    bf, _ = cabi.generate(plain, 0, prompt, 9)
    plain.close()
    assert got[0] == bf[0]                                      # the first token comes from the bf16 prefill
