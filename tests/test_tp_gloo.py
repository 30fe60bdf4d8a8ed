"""CPU, world_size 2 and 4 over gloo: the tensor-parallel partition (head shards, paired ranks that
split o_proj's input, MLP columns, vocabulary rows) reproduces the unpartitioned oracle."""
import socket

import pytest
import torch
import torch.multiprocessing as mp

import tp_worker
from oracle import qwen_text, synth, tp as tp_oracle


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


CFG = dict(num_layers=2, hidden=256, q_heads=4, kv_heads=2, intermediate=512, vocab=1200, tied=False)


@pytest.mark.parametrize("world", [2, 4])           # 4 ranks on 2 kv heads: ranks pair up on a head shard
def test_tp_oracle_matches_single_rank(tmp_path, world):
    steps, n_prompt, seed = 6, 19, 5
    mp.spawn(tp_worker.cpu_rank, args=(world, free_port(), CFG, seed, n_prompt, steps, str(tmp_path)), nprocs=world, join=True)
    cfg = synth.tiny_config(**CFG)
    w = synth.make_weights(cfg, seed=seed)
    o = qwen_text.QwenTextOracle(cfg, w, "exact_fp32")
    ref = qwen_text.generate(o, synth.make_token_ids(n_prompt, seed=seed, vocab=cfg.vocab), steps)
    for rank in range(world):
        got = torch.load(tmp_path / f"rank{rank}.pt")
        assert got["tokens"] == ref.tokens                         # every rank samples the same ids
        assert torch.allclose(got["logits"], torch.stack(ref.logits), atol=2e-4, rtol=1e-4)


def test_tp_layout_covers_every_weight_exactly_once():
    cfg = synth.CONFIGS[3]                                          # 28 q / 4 kv heads, MLP 18944, vocab 152064
    for tp in (1, 2, 4, 8):
        cols, rows_i, rows_v = [], [], []
        for r in range(tp):
            lay = tp_oracle.tp_layout(cfg, r, tp)
            cols += list(range(lay["o_cols"].start, lay["o_cols"].stop))
            rows_i += list(range(lay["i_rows"].start, lay["i_rows"].stop))
            rows_v += list(range(lay["v_rows"].start, lay["v_rows"].stop))
            assert lay["q_l"] * lay["att_shards"] == cfg.q_heads and lay["kv_l"] * lay["att_shards"] == cfg.kv_heads
        assert sorted(cols) == list(range(cfg.q_heads * cfg.head_dim))
        assert sorted(rows_i) == list(range(cfg.intermediate)) and sorted(rows_v) == list(range(cfg.vocab))
    with pytest.raises(AssertionError):
        tp_oracle.tp_layout(cfg, 0, 3)
