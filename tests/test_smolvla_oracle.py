"""CPU checks of the SmolVLA-shaped oracle: the vision tower + connector against the fixture made from the public
SmolVLM implementation, and structural properties of the chunk (mask rule, step plumbing, determinism)."""
import os

import numpy as np
import pytest
import torch

from oracle import smolvla

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "smolvla_vision_tiny.npz")


def test_vision_and_connector_match_the_public_implementation():
    g = np.load(GOLDEN)
    c = smolvla.VlaConfig.tiny()
    seed = int(g["seed"])
    images, _, _, _ = smolvla.make_inputs(c, seed=seed)
    out = smolvla.VlaOracle(c, smolvla.make_weights(c, seed=seed), mode="exact_fp32").vision(images)
    want = torch.from_numpy(g["expected"])
    assert out.shape == want.shape == (c.n_images * c.image_tokens, c.hidden)
    assert (out - want).abs().max().item() < 1e-4 * max(1.0, want.abs().max().item())


def test_pixel_shuffle_index_rule():
    side, s, d = 8, 4, 3
    x = torch.arange(side * side * d, dtype=torch.float32).reshape(side * side, d)
    y = smolvla.pixel_shuffle(x, side, s)
    assert y.shape == (4, s * s * d)
    for R in range(2):
        for Cc in range(2):
            for ry in range(s):
                for cx in range(s):
                    src = x[(R * s + ry) * side + (Cc * s + cx)]
                    got = y[R * 2 + Cc, (ry * s + cx) * d:(ry * s + cx + 1) * d]
                    assert torch.equal(src, got)


def test_geometry_of_the_benchmark_configuration():
    c = smolvla.VlaConfig()
    assert c.patches == 1024 and c.image_tokens == 64 and c.prefix == 3 * 64 + 48 + 1 == 241
    assert c.expert_mlp == 256 * ((4 * int(2 * c.expert_hidden / 3) + 255) // 256) == 2048
    names = dict((n, s) for n, s, _ in smolvla.weight_names(c))
    assert names["expert.0.k.weight"] == (320, 720) and names["expert.1.k.weight"] == (320, 320)
    assert names["connector.weight"] == (960, 768 * 16)


def test_state_token_is_invisible_to_the_rest_of_the_prefix():
    c = smolvla.VlaConfig.tiny()
    w = smolvla.make_weights(c, seed=5)
    o = smolvla.VlaOracle(c, w, mode="exact_fp32")
    images, ids, state, _ = smolvla.make_inputs(c, seed=5)
    x1, cache1 = o.prefix(images, ids, state)
    x2, cache2 = o.prefix(images, ids, -state)
    assert torch.allclose(x1[:-1], x2[:-1], atol=1e-6)          # image and prompt rows do not see the state
    assert not torch.allclose(x1[-1], x2[-1], atol=1e-3)
    assert torch.allclose(cache1[-1][0][:-1], cache2[-1][0][:-1], atol=1e-6)


def test_chunk_is_the_euler_sum_of_velocities_and_bf16_points_stay_close():
    c = smolvla.VlaConfig.tiny()
    w = smolvla.make_weights(c, seed=6)
    inp = smolvla.make_inputs(c, seed=6)
    o = smolvla.VlaOracle(c, w, mode="exact_fp32")
    _, cache = o.prefix(*inp[:3])
    x = inp[3].clone()
    for s in range(c.steps):
        x = x - o.velocity(x, 1.0 - s / c.steps, cache) / c.steps
    full = o.chunk(*inp)
    assert torch.allclose(full, x, atol=1e-6)
    again = o.chunk(*inp)
    assert torch.equal(full, again)
    b = smolvla.VlaOracle(c, w, mode="bf16_points").chunk(*inp)
    assert (b - full).abs().max().item() < 5e-2


def test_time_embedding_endpoints():
    e = smolvla.time_embedding(1.0, 8)
    # periods 4e-3 .. 4.0 geometric; last sine is sin(2*pi*1/4) = 1
    assert abs(e[3].item() - 1.0) < 1e-6 and e.shape == (8,)
