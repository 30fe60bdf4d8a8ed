"""GPU parity of the SmolVLA-shaped action chunk (efm_b200_vla_*) against oracle/smolvla.py.

Floating point: bf16 tensor-core GEMMs with fp32 accumulation against an fp32 restatement that rounds to bf16
at the same points; tolerance 3e-2 absolute on actions of unit scale (ten Euler steps through 16 expert layers)."""
import pytest
import torch

import cabi
from oracle import smolvla

pytestmark = pytest.mark.gpu

TOL = 3e-2


def _run(cfg, seed):
    w = smolvla.make_weights(cfg, seed=seed)
    inp = smolvla.make_inputs(cfg, seed=seed)
    pol = cabi.VlaPolicy(cfg)
    try:
        pol.load_weights(w)
        first = pol.chunk(*inp)            # kernel by kernel
        second = pol.chunk(*inp)           # captures the graph
        third = pol.chunk(*inp)            # replays it
        launches = pol.launch_count()
    finally:
        pol.close()
    return w, inp, first, second, third, launches


def test_tiny_chunk_equals_oracle_and_graph_replay_is_identical():
    cfg = smolvla.VlaConfig.tiny()
    w, inp, first, second, third, launches = _run(cfg, seed=21)
    want = smolvla.VlaOracle(cfg, w, mode="bf16_points").chunk(*inp)
    assert torch.isfinite(first).all()
    err = (first - want).abs().max().item()
    assert err < TOL, err
    assert torch.equal(first, second) and torch.equal(first, third)      # same kernels, same order: bit-identical
    assert launches[1] > 0 and launches[0] == 3 * launches[1]
    assert (first - inp[3]).abs().max().item() > 0.1                      # the chunk moved away from the noise


def test_odd_sizes_chunk_equals_oracle():
    # widths that are not multiples of the GEMM tile (K = 720-like remainders, N below one tile), 3 images
    cfg = smolvla.VlaConfig(image_size=128, patch=16, vit_layers=2, vit_hidden=192, vit_heads=3, vit_mlp=328, shuffle=2,
                            n_images=3, hidden=320, layers=2, q_heads=5, kv_heads=5, head_dim=64, mlp=448, vocab=1000,
                            lang_tokens=5, expert_hidden=200, expert_mlp=320, chunk=7, steps=3)
    w, inp, first, second, third, _ = _run(cfg, seed=22)
    want = smolvla.VlaOracle(cfg, w, mode="bf16_points").chunk(*inp)
    err = (first - want).abs().max().item()
    assert err < TOL, err
    assert torch.equal(first, third)


def test_new_inputs_give_new_actions_through_the_graph():
    cfg = smolvla.VlaConfig.tiny()
    w = smolvla.make_weights(cfg, seed=23)
    a = smolvla.make_inputs(cfg, seed=23)
    b = smolvla.make_inputs(cfg, seed=24)
    pol = cabi.VlaPolicy(cfg)
    try:
        pol.load_weights(w)
        pol.chunk(*a)
        pol.chunk(*a)
        got_b = pol.chunk(*b)              # graph replay on different inputs
        got_a = pol.chunk(*a)
    finally:
        pol.close()
    o = smolvla.VlaOracle(cfg, w, mode="bf16_points")
    assert (got_b - o.chunk(*b)).abs().max().item() < TOL
    assert (got_a - o.chunk(*a)).abs().max().item() < TOL


def test_missing_weight_and_bad_shape_are_reported():
    cfg = smolvla.VlaConfig.tiny()
    w = smolvla.make_weights(cfg, seed=25)
    pol = cabi.VlaPolicy(cfg)
    try:
        partial = dict(w)
        partial.pop("expert.norm")
        with pytest.raises(RuntimeError, match="missing tensor: expert.norm"):
            pol.load_weights(partial)
        with pytest.raises(RuntimeError, match="unexpected shape"):
            pol.load_weights({"embed": torch.zeros(3, 3, dtype=torch.bfloat16)})
        with pytest.raises(RuntimeError, match="unknown tensor"):
            pol.load_weights({"nope": torch.zeros(3, dtype=torch.bfloat16)})
    finally:
        pol.close()


def test_benchmark_size_chunk_equals_oracle():
    # the configuration the chunks/s number is quoted on (3 x 512 px, 241-token prefix, 10 steps x 50 actions)
    cfg = smolvla.VlaConfig()
    w, inp, first, second, third, launches = _run(cfg, seed=0)
    with torch.no_grad():
        want = smolvla.VlaOracle(cfg, w, mode="bf16_points").chunk(*inp)
    err = (first - want).abs().max().item()
    assert err < TOL, err
    assert torch.equal(first, third)
    assert cfg.prefix == 241 and tuple(first.shape) == (50, 32)


def test_chunk_wider_than_64_rows_takes_the_tensor_core_products():
    # more than 64 action rows: the expert's products go through the tcgen05 GEMM with separate norm / rope kernels
    cfg = smolvla.VlaConfig(image_size=128, patch=16, vit_layers=1, vit_hidden=128, vit_heads=2, vit_mlp=256, shuffle=4,
                            n_images=1, hidden=192, layers=2, q_heads=3, kv_heads=1, head_dim=64, mlp=256, vocab=300,
                            lang_tokens=6, expert_hidden=128, expert_mlp=256, chunk=70, steps=3)
    w, inp, first, second, third, _ = _run(cfg, seed=26)
    want = smolvla.VlaOracle(cfg, w, mode="bf16_points").chunk(*inp)
    err = (first - want).abs().max().item()
    assert err < TOL, err
    assert torch.equal(first, third)
