"""GPU: the generate() path end to end against the CPU oracle and the HF golden vectors.
Through the C ABI (tests/cabi.py) and through the public `edge_fm` module."""
import os

import numpy as np
import pytest
import torch

import cabi
from oracle import qwen_text, sampling, synth

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
LOGIT_TOL = 2e-2          # relative (max-norm) logits tolerance of the workload definition


def rel_err(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def make_backend(cfg, weights, max_tokens=256, slots=(0,), **kw):
    be = cabi.Backend(cfg, **kw)
    be.load_weights(weights)
    for s in slots:
        be.alloc_slot(s, max_tokens)
    be.set_sampling(0.0, 1.0, 0)
    return be


def check_against_oracle(cfg, weights, prompt, steps, tokens, logits, **okw):
    """Greedy ids vs the bf16_points oracle (teacher-forced with the GPU's ids, so one near-tie
    cannot cascade); logits vs exact_fp32.  A differing id is accepted only when the oracle's own
    top-1/top-2 margin is below the logit error observed at that step (a tie within tolerance)."""
    ob = qwen_text.QwenTextOracle(cfg, weights, "bf16_points")
    rb = qwen_text.generate(ob, prompt, steps, forced=tokens, **okw)
    oe = qwen_text.QwenTextOracle(cfg, weights, "exact_fp32")
    re = qwen_text.generate(oe, prompt, steps, forced=tokens, **okw)
    ties = 0
    for s in range(steps):
        eb = np.abs(logits[s] - rb.logits[s].numpy()).max()
        assert rel_err(logits[s], re.logits[s].numpy()) < LOGIT_TOL, f"step {s}"
        assert rel_err(logits[s], rb.logits[s].numpy()) < LOGIT_TOL / 2, f"step {s}"
        if tokens[s] != rb.tokens[s]:
            assert rb.margins[s] <= 2 * eb, f"step {s}: id {tokens[s]} vs oracle {rb.tokens[s]}, margin {rb.margins[s]}, err {eb}"
            ties += 1
    return ties


@pytest.mark.parametrize("name,kw,seed", [
    ("qwen2_tiny_tied", dict(num_layers=2, hidden=128, q_heads=2, kv_heads=1, intermediate=256, vocab=1000, tied=True), 0),
    ("qwen2_small_untied", dict(num_layers=3, hidden=256, q_heads=4, kv_heads=2, intermediate=512, vocab=2000,
                                tied=False, rope_theta=1e4), 1)])
def test_golden_hf_vectors(name, kw, seed):
    g = np.load(os.path.join(GOLDEN, name + ".npz"))
    cfg = synth.tiny_config(**kw)
    w = synth.make_weights(cfg, seed=seed)
    be = make_backend(cfg, w)
    prompt, want = g["prompt"].tolist(), g["tokens"].tolist()
    toks, logits = cabi.generate(be, 0, prompt, len(want), forced=want, collect_logits=True)
    for s in range(len(want)):
        assert rel_err(logits[s], g["logits"][s]) < LOGIT_TOL
        if toks[s] != want[s]:
            srt = np.sort(g["logits"][s])
            assert srt[-1] - srt[-2] <= 2 * np.abs(logits[s] - g["logits"][s]).max()
    be.close()


@pytest.mark.parametrize("kw", [
    dict(num_layers=2, hidden=128, q_heads=2, kv_heads=1, intermediate=256, vocab=1000),
    dict(num_layers=2, hidden=896, q_heads=14, kv_heads=2, intermediate=4864 // 19, vocab=3000),        # 0.5B head geometry (D 64, group 7)
    dict(num_layers=2, hidden=1536, q_heads=12, kv_heads=2, intermediate=512, vocab=3000, tied=False),  # 1.5B geometry (D 128, group 6)
    dict(num_layers=2, hidden=1024, q_heads=8, kv_heads=1, intermediate=320, vocab=2002)])               # group 8
def test_generate_matches_oracle(kw):
    cfg = synth.tiny_config(**kw)
    w = synth.make_weights(cfg, seed=11)
    be = make_backend(cfg, w)
    prompt = synth.make_token_ids(37, seed=5, vocab=cfg.vocab)
    steps = 32
    toks, logits = cabi.generate(be, 0, prompt, steps, collect_logits=True)
    ties = check_against_oracle(cfg, w, prompt, steps, toks, logits)
    assert ties <= 2
    # the captured graph, plain launches and step-by-step replay give identical ids
    t_graph, _ = cabi.generate(be, 0, prompt, steps, use_graph=True)
    t_eager, _ = cabi.generate(be, 0, prompt, steps, use_graph=False)
    assert t_graph == toks and t_eager == toks
    be.close()


def test_fixed_prefix_equals_full_prefill_and_survives_requests():
    cfg = synth.tiny_config(num_layers=2, hidden=256, q_heads=4, kv_heads=2, intermediate=256, vocab=1500)
    w = synth.make_weights(cfg, seed=2)
    be = make_backend(cfg, w, slots=(0, 3))
    prefix = synth.make_token_ids(20, seed=1, vocab=cfg.vocab)
    a = prefix + synth.make_token_ids(9, seed=2, vocab=cfg.vocab)
    b = prefix + synth.make_token_ids(14, seed=3, vocab=cfg.vocab)
    be.prefill(3, prefix, kv_offset=0, sample=False)              # what warmup() does for a slot with a prefix
    full_a, la = cabi.generate(be, 0, a, 12, collect_logits=True)
    pre_a, lpa = cabi.generate(be, 3, a, 12, prefix_len=len(prefix), collect_logits=True)
    assert pre_a == full_a
    assert rel_err(lpa[0], la[0]) < 1e-2
    full_b, _ = cabi.generate(be, 0, b, 12)
    pre_b, _ = cabi.generate(be, 3, b, 12, prefix_len=len(prefix))  # the prefix rows were not disturbed by request a
    assert pre_b == full_b
    pre_a2, _ = cabi.generate(be, 3, a, 12, prefix_len=len(prefix))
    assert pre_a2 == pre_a
    be.close()


def test_chunked_prefill_equals_single_pass():
    cfg = synth.tiny_config(num_layers=2, hidden=128, q_heads=2, kv_heads=1, intermediate=128, vocab=1000)
    w = synth.make_weights(cfg, seed=4)
    prompt = synth.make_token_ids(150, seed=9, vocab=cfg.vocab)
    one = make_backend(cfg, w, max_prefill_tokens=256)
    t1, l1 = cabi.generate(one, 0, prompt, 8, collect_logits=True)
    many = make_backend(cfg, w, max_prefill_tokens=64)              # 150 tokens -> chunks of 64, 64, 22
    t2, l2 = cabi.generate(many, 0, prompt, 8, collect_logits=True)
    assert t1 == t2 and rel_err(l2[0], l1[0]) < 1e-2
    one.close()
    many.close()


def test_mrope_and_embedding_injection():
    cfg = synth.tiny_config(num_layers=2, hidden=256, q_heads=2, kv_heads=1, intermediate=256, vocab=1200,
                            mrope_section=[16, 24, 24], model_type="qwen2_5_vl")          # head_dim 128
    w = synth.make_weights(cfg, seed=6)
    be = make_backend(cfg, w)
    n_img, grid = 16, 4                                          # a 4x4 merged image block first, then text
    embed_id = cfg.vocab + 10
    g = torch.Generator().manual_seed(0)
    embeds = (torch.randn(n_img, cfg.hidden, generator=g) * 0.05).to(torch.bfloat16)
    text = synth.make_token_ids(11, seed=8, vocab=cfg.vocab)
    ids = [embed_id + i for i in range(n_img)] + text
    pos = torch.zeros(3, len(ids), dtype=torch.int64)
    for i in range(n_img):
        pos[:, i] = torch.tensor([0, i // grid, i % grid])
    for j in range(len(text)):
        pos[:, n_img + j] = grid + j
    last = [int(pos.max())] * 3
    steps = 16
    for dev_embeds in (embeds, embeds.cuda()):
        toks, logits = cabi.generate(be, 0, ids, steps, embeds=dev_embeds, embed_token_id=embed_id, pos3=pos.tolist(),
                                     mrope_last_pos=last, collect_logits=True)
        ties = check_against_oracle(cfg, w, ids, steps, toks, logits, embeds=embeds, embed_token_id=embed_id,
                                    position_ids=pos, mrope_last_pos=last)
        assert ties <= 1
    be.close()


def test_top_p_decode_teacher_forced_and_sampler_on_oracle_logits():
    cfg = synth.tiny_config(num_layers=2, hidden=256, q_heads=4, kv_heads=2, intermediate=256, vocab=3000)
    w = synth.make_weights(cfg, seed=7)
    be = make_backend(cfg, w)
    T, top_p, seed = 0.7, 0.9, 42
    be.set_sampling(T, top_p, seed)
    prompt = synth.make_token_ids(25, seed=3, vocab=cfg.vocab)
    steps = 24
    free, _ = cabi.generate(be, 0, prompt, steps)
    again, _ = cabi.generate(be, 0, prompt, steps, use_graph=False)
    assert free == again                                         # seeded: reproducible, graph or not
    assert len(set(free)) > 4
    # teacher-force the oracle's own sampled trajectory; the GPU's logits must stay within tolerance and
    # its sampler, fed its own logits, must agree with the CPU sampling rule on those same logits
    o = qwen_text.QwenTextOracle(cfg, w, "bf16_points")
    ro = qwen_text.generate(o, prompt, steps, sampler=sampling.make_sampler(T, top_p, seed))
    toks, logits = cabi.generate(be, 0, prompt, steps, forced=ro.tokens, collect_logits=True)
    for s in range(steps):
        assert rel_err(logits[s], ro.logits[s].numpy()) < LOGIT_TOL / 2
        assert toks[s] == sampling.sample_top_p(logits[s], T, top_p, seed, s)
    be.close()


def test_backend_argument_errors_are_reported_not_fatal():
    cfg = synth.tiny_config()
    w = synth.make_weights(cfg, seed=0)
    be = cabi.Backend(cfg)
    with pytest.raises(cabi.BackendError, match="not finalized"):
        be.prefill(0, [1, 2, 3])
    be.load_weights(w)
    be.alloc_slot(0, 16)
    with pytest.raises(cabi.BackendError, match="unknown KV slot"):
        be.prefill(5, [1, 2, 3])
    with pytest.raises(cabi.BackendError, match="max_tokens"):
        be.prefill(0, list(range(17)))
    with pytest.raises(cabi.BackendError, match="already allocated"):
        be.alloc_slot(0, 16)
    be.prefill(0, [1, 2, 3])
    with pytest.raises(cabi.BackendError, match="no room"):
        be.decode_begin(0, 16)
    be.decode_begin(0, 3)
    be.decode_steps(2)
    assert len(be.read_tokens(0, 3)) == 3                         # still usable after the refused calls
    missing = cabi.Backend(cfg)
    part = dict(w)
    part.pop("model.layers.1.mlp.down_proj.weight")
    with pytest.raises(cabi.BackendError, match="layer 1"):
        missing.load_weights(part)
    be.close()
    missing.close()


# ------------------------------------------------------------------------------------------------
# public API: edge_fm.EdgeFM(config).generate(Request)
# ------------------------------------------------------------------------------------------------
def test_edge_fm_module_generate(tmp_path, built):
    import edge_fm
    cfg = synth.tiny_config(num_layers=2, hidden=256, q_heads=4, kv_heads=2, intermediate=256, vocab=1500)
    w = synth.make_weights(cfg, seed=2)
    model_dir = synth.write_checkpoint(str(tmp_path / "model"), cfg, w)
    prefix = synth.make_token_ids(20, seed=1, vocab=cfg.vocab)
    prompt = prefix + synth.make_token_ids(9, seed=2, vocab=cfg.vocab)
    o = qwen_text.QwenTextOracle(cfg, w, "bf16_points")
    want = qwen_text.generate(o, prompt, 16)
    outs = {}
    for graph in (True, False):
        path = synth.write_engine_config(str(tmp_path / f"engine_{graph}.json"), model_dir, prefix_ids=prefix,
                                         max_tokens=64, max_new_tokens=16, temperature=0.0, use_cuda_graph=graph,
                                         extra_requests=[{"request_id": 7, "prefix_token_ids": [], "max_tokens": 40}])
        eng = edge_fm.EdgeFM(path)
        req = edge_fm.Request(0, prompt)
        req.set_ignore_stop_tokens(True)
        outs[graph] = list(eng.generate(req).token_ids())
        m = eng.last_generate_metrics()
        for key in ("prefill_ms", "decode_ms", "total_stage_ms", "decode_step_avg_ms", "generated_tokens_total",
                    "decode_steps", "tokens_per_second", "decode_tokens_per_second", "cuda_graph_enabled",
                    "executed_generated_tokens_total", "returned_generated_tokens_total", "response_tokens_capacity"):
            assert key in m
        assert m["generated_tokens_total"] == 16 and m["decode_steps"] == 15 and m["cuda_graph_enabled"] == float(graph)
        # no-prefix slot, same tokens -> same ids; capacity caps generation: 40 - 29 + 1 = 12
        r7 = edge_fm.Request(7, prompt)
        r7.set_ignore_stop_tokens(True)
        assert list(eng.generate(r7).token_ids()) == outs[graph][:12]
        # stop token: cut after (and including) its first occurrence
        stop = outs[graph][3]
        rs = edge_fm.Request(0, prompt)
        rs.set_stop_token_ids([stop])
        got = list(eng.generate(rs).token_ids())
        assert got == outs[graph][:outs[graph].index(stop) + 1]
        assert eng.last_generate_metrics()["executed_generated_tokens_total"] == 16
        # the engine's device backend is reachable for C-ABI companions (vision encoder on the same stream / communicator)
        handle = eng.backend_handle()
        assert handle != 0
        L = cabi.lib()
        assert L.efm_b200_synchronize(cabi.P(handle)) == 0
        n_launch = cabi.C.c_int64(0)
        assert L.efm_b200_launch_count(cabi.P(handle), cabi.C.byref(n_launch)) == 0 and n_launch.value > 0
        # request errors surface as ValueError, like the reference's binding
        with pytest.raises(ValueError, match="prefix"):
            eng.generate(edge_fm.Request(0, [1, 2, 3] + prompt))
        with pytest.raises(ValueError, match="request_id"):
            eng.generate(edge_fm.Request(99, prompt))
        del eng
    assert outs[True] == outs[False]
    mism = [s for s in range(16) if outs[True][s] != want.tokens[s]]
    assert not mism or want.margins[mism[0]] < 1e-2


def test_edge_fm_module_configuration_errors(tmp_path, built):
    import edge_fm
    cfg = synth.tiny_config()
    w = synth.make_weights(cfg)
    model_dir = synth.write_checkpoint(str(tmp_path / "model"), cfg, w)
    with pytest.raises(ValueError):
        edge_fm.EdgeFM(str(tmp_path / "missing.json"))
    bad = synth.write_engine_config(str(tmp_path / "bad.json"), str(tmp_path / "nowhere"))
    with pytest.raises(ValueError, match="prefill_model_path"):
        edge_fm.EdgeFM(bad)
    unk = synth.write_engine_config(str(tmp_path / "unk.json"), model_dir, model_name="Llama")
    with pytest.raises(ValueError, match="model_name"):
        edge_fm.EdgeFM(unk)
    # truncated checkpoint -> RuntimeError (ModelNotLoadedError), no crash
    st = os.path.join(model_dir, "model.safetensors")
    data = open(st, "rb").read()
    open(st, "wb").write(data[: len(data) // 2])
    ok_cfg = synth.write_engine_config(str(tmp_path / "trunc.json"), model_dir)
    with pytest.raises(RuntimeError, match="truncated|outside"):
        edge_fm.EdgeFM(ok_cfg)
    # a record whose byte range disagrees with its shape (mis-sharded header) is refused, not read past its end
    import json
    import struct
    n = struct.unpack("<Q", data[:8])[0]
    header = json.loads(data[8:8 + n])
    name = next(k for k in header if k.endswith("q_proj.weight"))
    header[name]["shape"][0] *= 2
    hb = json.dumps(header).encode()
    open(st, "wb").write(struct.pack("<Q", len(hb)) + hb + data[8 + n:])
    with pytest.raises(RuntimeError, match="shape and dtype need"):
        edge_fm.EdgeFM(ok_cfg)


def test_edge_fm_compact_vocab_and_int8_prefill_through_the_public_api(tmp_path, built):
    """Non-identity compact vocabulary: requests and responses stay in tokenizer ids while the model runs on a
    pre-pruned checkpoint (the reference's test_generate_compact_vocab_non_identity_remaps_request_response_and_stop).
    The same engine also runs with runtime.prefill_attention = "int8"."""
    import json
    import edge_fm
    full = synth.tiny_config(num_layers=2, hidden=256, q_heads=4, kv_heads=2, intermediate=256, vocab=1500)
    w_full = synth.make_weights(full, seed=4)
    g = torch.Generator().manual_seed(9)
    keep = torch.randperm(full.vocab, generator=g)[:900].sort().values            # new -> old, increasing
    old_to_new = torch.full((full.vocab,), -1, dtype=torch.int64)
    old_to_new[keep] = torch.arange(keep.numel())
    pruned = synth.tiny_config(num_layers=2, hidden=256, q_heads=4, kv_heads=2, intermediate=256, vocab=int(keep.numel()))
    w = dict(w_full)
    w["model.embed_tokens.weight"] = w_full["model.embed_tokens.weight"][keep].contiguous()
    model_dir = synth.write_checkpoint(str(tmp_path / "model"), pruned, w)
    hf = json.load(open(os.path.join(model_dir, "config.json")))
    hf["eos_token_id"] = int(keep[1])                      # tokenizer id space, and kept
    hf.pop("bos_token_id", None)
    json.dump(hf, open(os.path.join(model_dir, "config.json"), "w"))
    prompt_new = synth.make_token_ids(24, seed=3, vocab=pruned.vocab)
    prompt_old = [int(keep[i]) for i in prompt_new]
    (tmp_path / "map.json").write_text(json.dumps(dict(
        format="edgefm.compact_vocab.v1", original_vocab_size=full.vocab, compact_vocab_size=pruned.vocab,
        old_to_new=old_to_new.tolist(), new_to_old=keep.tolist(), special_token_ids=[int(keep[0])])))

    # what the model itself produces on compact ids, straight through the C ABI
    be = cabi.Backend(pruned, max_prefill_tokens=64, max_response_tokens=16)
    be.load_weights(w)
    be.alloc_slot(0, 64)
    be.set_sampling(0.0, 1.0, 0)
    compact_tokens, _ = cabi.generate(be, 0, prompt_new, 12)
    be.close()

    for attention in ("bf16", "int8"):
        path = synth.write_engine_config(str(tmp_path / f"engine_{attention}.json"), model_dir, max_tokens=64, max_new_tokens=12)
        cfg = json.load(open(path))
        cfg["compact_vocab"] = {"enabled": True, "mapping_path": "map.json", "reject_unknown_input_ids": True}
        cfg["runtime"]["prefill_attention"] = attention
        json.dump(cfg, open(path, "w"))
        eng = edge_fm.EdgeFM(path)
        req = edge_fm.Request(0, prompt_old)
        req.set_ignore_stop_tokens(True)
        got = list(eng.generate(req).token_ids())
        if attention == "bf16":
            assert got == [int(keep[t]) for t in compact_tokens]             # restored to tokenizer ids
        else:
            assert got[0] == int(keep[compact_tokens[0]]) and all(int(old_to_new[t]) >= 0 for t in got)
        # a stop id given in tokenizer ids cuts the restored response
        rs = edge_fm.Request(0, prompt_old)
        rs.set_stop_token_ids([got[2]])
        assert list(eng.generate(rs).token_ids()) == got[:got.index(got[2]) + 1]
        # a pruned id in the request (or as a request stop id) is refused, not remapped
        pruned_id = int((old_to_new < 0).nonzero()[0])
        with pytest.raises(ValueError, match="compact_vocab"):
            eng.generate(edge_fm.Request(0, prompt_old[:5] + [pruned_id]))
        bad_stop = edge_fm.Request(0, prompt_old)
        bad_stop.set_stop_token_ids([pruned_id])
        with pytest.raises(ValueError, match="compact_vocab"):
            eng.generate(bad_stop)
        del eng
    # an unpruned checkpoint behind an enabled mapping is a configuration error
    other = synth.write_checkpoint(str(tmp_path / "full"), full, w_full)
    hf = json.load(open(os.path.join(other, "config.json")))
    hf["eos_token_id"] = int(keep[1])
    json.dump(hf, open(os.path.join(other, "config.json"), "w"))
    path = synth.write_engine_config(str(tmp_path / "engine_bad.json"), other, max_tokens=64)
    cfg = json.load(open(path))
    cfg["compact_vocab"] = {"enabled": True, "mapping_path": "map.json"}
    json.dump(cfg, open(path, "w"))
    with pytest.raises(Exception, match="pre-pruned"):
        edge_fm.EdgeFM(path)


def test_edge_fm_stage_api_prefill_and_decode(tmp_path, built):
    """Tensor-in / tensor-out stage calls (EdgeFM.prefill / decode / run_stage): the prefill stage over a request whose
    prefix is resident returns the logits and the first token generate() returns; decode stages, one token each, walk
    the same greedy sequence and accept a fed token; both kinds of M-RoPE input travel as tensors."""
    import edge_fm
    for kw in (dict(), dict(mrope_section=[8, 12, 12], model_type="qwen2_5_vl")):
        cfg = synth.tiny_config(num_layers=2, hidden=256, q_heads=4, kv_heads=2, intermediate=256, vocab=1500, **kw)
        tag = "vl" if kw else "text"
        w = synth.make_weights(cfg, seed=11)
        model_dir = synth.write_checkpoint(str(tmp_path / f"model_{tag}"), cfg, w)
        prefix = synth.make_token_ids(9, seed=3, vocab=cfg.vocab) if not kw else []
        prompt = prefix + synth.make_token_ids(14, seed=4, vocab=cfg.vocab)
        path = synth.write_engine_config(str(tmp_path / f"engine_{tag}.json"), model_dir, model_name="Qwen2.5-VL" if kw else "Qwen2.5",
                                         prefix_ids=prefix, max_tokens=64, max_new_tokens=8)
        eng = edge_fm.EdgeFM(path)
        ids_t = torch.tensor(prompt, dtype=torch.int32)
        inputs = {"token_ids": edge_fm.Tensor(ids_t.data_ptr(), [len(prompt)], edge_fm.DType.Int32, edge_fm.Device.CPU)}
        if kw:
            emb = (torch.randn(3, cfg.hidden) * 0.02).to(torch.bfloat16)
            ids_v = [cfg.vocab, cfg.vocab + 1, cfg.vocab + 2] + prompt
            pos = torch.tensor([[0, 0, 0] + list(range(2, 2 + len(prompt))), [0, 0, 1] + list(range(2, 2 + len(prompt))),
                                [0, 1, 0] + list(range(2, 2 + len(prompt)))], dtype=torch.int32)
            req = edge_fm.Request(0, ids_v, edge_fm.Tensor(emb.data_ptr(), [3, cfg.hidden], edge_fm.DType.BFloat16, edge_fm.Device.CPU),
                                  cfg.vocab, edge_fm.Tensor(pos.data_ptr(), [3, len(ids_v)], edge_fm.DType.Int32, edge_fm.Device.CPU))
            ids_t = torch.tensor(ids_v, dtype=torch.int64)                 # int64 ids are accepted too
            eid = torch.tensor([cfg.vocab], dtype=torch.int32)
            inputs = {"token_ids": edge_fm.Tensor(ids_t.data_ptr(), [1, len(ids_v)], edge_fm.DType.Int64, edge_fm.Device.CPU),
                      "embedding": edge_fm.Tensor(emb.data_ptr(), [3, cfg.hidden], edge_fm.DType.BFloat16, edge_fm.Device.CPU),
                      "embed_token_id": edge_fm.Tensor(eid.data_ptr(), [1], edge_fm.DType.Int32, edge_fm.Device.CPU),
                      "position_ids": edge_fm.Tensor(pos.data_ptr(), [3, len(ids_v)], edge_fm.DType.Int32, edge_fm.Device.CPU)}
        else:
            req = edge_fm.Request(0, prompt)
        req.set_ignore_stop_tokens(True)
        want = list(eng.generate(req).token_ids())
        assert len(want) == 8

        def unpack(out):
            lg = torch.from_dlpack(out["logits"].to_dlpack()).clone()
            tk = int(torch.from_dlpack(out["next_token"].to_dlpack())[0])
            assert lg.shape == (1, cfg.vocab) and lg.dtype == torch.float32
            assert int(lg.argmax()) == tk
            return lg, tk

        _, t0 = unpack(eng.prefill(0, inputs))
        got = [t0]
        assert eng.last_stage_metrics()["kv_len"] == len(ids_t.flatten())
        for _ in range(7):
            _, t = unpack(eng.decode(0, {}))
            got.append(t)
        assert got == want
        # the same walk with every token fed explicitly (run_stage by name), restarting from the prefill stage
        _, t0 = unpack(eng.run_stage(0, "prefill", inputs))
        again = [t0]
        for s in range(7):
            feed = torch.tensor([want[s]], dtype=torch.int32)
            _, t = unpack(eng.run_stage(0, "decode", {"token_ids": edge_fm.Tensor(feed.data_ptr(), [1], edge_fm.DType.Int32, edge_fm.Device.CPU)}))
            again.append(t)
        assert again == want
        with pytest.raises(ValueError, match="prefill"):
            eng.run_stage(0, "context", {})
        with pytest.raises(ValueError, match="before a prefill"):
            eng.decode(1, {}) if False else edge_fm.EdgeFM.decode(eng, 7, {})
        assert edge_fm.ModelStage.Prefill != edge_fm.ModelStage.Decode
        del eng


def test_prefill_cuda_graph_buckets():
    """Prefill graphs: the first prefill of a shape runs kernel by kernel, the second is captured, later ones replay;
    every form must return the tokens and logits of the plain launch sequence, for fresh token ids each time, with and
    without a resident prefix, with injected embeddings, and after the sampling parameters change."""
    cfg = synth.tiny_config(num_layers=3, hidden=256, q_heads=4, kv_heads=2, intermediate=512, vocab=1500,
                            mrope_section=[8, 12, 12], model_type="qwen2_5_vl")
    w = synth.make_weights(cfg, seed=8)
    plain, graph = cabi.Backend(cfg), cabi.Backend(cfg)
    for be in (plain, graph):
        be.load_weights(w)
        be.alloc_slot(0, 128)
        be.alloc_slot(1, 128)
        be.set_sampling(0.0, 1.0, 0)
    graph.set_prefill_graph(True)
    prefix = synth.make_token_ids(12, seed=1, vocab=cfg.vocab)
    for be in (plain, graph):
        be.prefill(1, prefix, kv_offset=0, pos3=[list(range(12))] * 3, sample=False)
    emb = (torch.randn(4, cfg.hidden, generator=torch.Generator().manual_seed(3)) * 0.02).to(torch.bfloat16).cuda()
    for trial in range(4):
        ids = synth.make_token_ids(20, seed=10 + trial, vocab=cfg.vocab)
        pos = [list(range(20))] * 3
        a, la = cabi.generate(plain, 0, ids, 6, pos3=pos, collect_logits=True)
        b, lb = cabi.generate(graph, 0, ids, 6, pos3=pos, collect_logits=True)
        assert a == b and np.array_equal(la[0], lb[0]), trial
        full = prefix + ids                                   # slot 1: resident prefix, prefill at kv_offset 12
        pos = [list(range(32))] * 3
        a, la = cabi.generate(plain, 1, full, 5, prefix_len=12, pos3=pos, collect_logits=True)
        b, lb = cabi.generate(graph, 1, full, 5, prefix_len=12, pos3=pos, collect_logits=True)
        assert a == b and np.array_equal(la[0], lb[0]), trial
        vis = [cfg.vocab + i for i in range(4)] + ids[:10]     # injected embedding rows
        pos = [list(range(14))] * 3
        a, la = cabi.generate(plain, 0, vis, 4, embeds=emb, embed_token_id=cfg.vocab, pos3=pos, collect_logits=True)
        b, lb = cabi.generate(graph, 0, vis, 4, embeds=emb, embed_token_id=cfg.vocab, pos3=pos, collect_logits=True)
        assert a == b and np.array_equal(la[0], lb[0]), trial
    captured, replays = graph.prefill_graph_stats()
    assert captured == 3 and replays == 9                     # three shapes, each: eager, capture + launch, replay, replay
    for be in (plain, graph):
        be.set_sampling(0.8, 0.9, 5)                          # baked into the graphs: they must be dropped
    ids = synth.make_token_ids(20, seed=40, vocab=cfg.vocab)
    for _ in range(3):
        a, _ = cabi.generate(plain, 0, ids, 6, pos3=[list(range(20))] * 3)
        b, _ = cabi.generate(graph, 0, ids, 6, pos3=[list(range(20))] * 3)
        assert a == b
    assert graph.prefill_graph_stats()[0] == 1
    plain.close()
    graph.close()
