"""GPU: the Qwen2.5-VL vision encoder through the C ABI against the CPU oracle (oracle/qwen_vit.py,
itself pinned to transformers' implementation by tests/golden/qwen_vit_tiny.npz)."""
import ctypes as C
import math
import os

import numpy as np
import pytest
import torch

import cabi
from oracle import qwen_vit, synth

pytestmark = pytest.mark.gpu


def P(t):
    return C.c_void_p(t.data_ptr())


def segment_ref(q, k, v, lo, hi):
    """q, k, v [S, h, D] fp32; row i sees keys [lo[i], hi[i])."""
    S, h, D = q.shape
    s = torch.einsum("shd,thd->hst", q, k) / math.sqrt(D)
    j = torch.arange(S, device=q.device)[None, :]
    mask = (j >= lo[:, None]) & (j < hi[:, None])
    s = s.masked_fill(~mask[None], float("-inf"))
    return torch.einsum("hst,thd->shd", torch.softmax(s, dim=-1), v)


def make_segments(S, lens, device):
    lo = torch.empty(S, dtype=torch.int32)
    hi = torch.empty(S, dtype=torch.int32)
    a, i = 0, 0
    while a < S:
        b = min(S, a + lens[i % len(lens)])
        lo[a:b], hi[a:b] = a, b
        a, i = b, i + 1
    return lo.to(device), hi.to(device)


# (heads, D, S, segment lengths): ViT windows (64 / 32 / 16 patches), one whole frame, ragged tails
@pytest.mark.parametrize("heads,D,S,lens", [(16, 80, 1024, [64]), (16, 80, 400, [64, 32, 16, 64]), (4, 80, 777, [777]),
                                            (2, 64, 130, [100, 30]), (3, 128, 257, [5, 252]), (2, 80, 8, [4])])
def test_segment_attention(heads, D, S, lens):
    L = cabi.lib()
    g = torch.Generator(device="cuda").manual_seed(S)
    qkv = torch.randn(S, 3, heads, D, generator=g, device="cuda").to(torch.bfloat16)
    lo, hi = make_segments(S, lens, "cuda")
    out = torch.zeros(S, heads, D, device="cuda", dtype=torch.bfloat16)
    flat = qkv.view(S, 3 * heads * D)
    st = L.efm_b200_op_segment_attention(P(flat), C.c_void_p(flat.data_ptr() + heads * D * 2),
                                         C.c_void_p(flat.data_ptr() + 2 * heads * D * 2), P(out), P(lo), P(hi), S, heads, D,
                                         3 * heads * D)
    assert st == 0
    ref = segment_ref(qkv[:, 0].float(), qkv[:, 1].float(), qkv[:, 2].float(), lo, hi)
    assert torch.allclose(out.float(), ref, atol=1e-2, rtol=2e-2)


def tiny_backend():
    cfg = synth.tiny_config()
    be = cabi.Backend(cfg, max_prefill_tokens=64, max_response_tokens=8)
    return be


def run_encoder(vcfg, weights, pixels, grids, device_io):
    be = tiny_backend()
    n = pixels.shape[0]
    enc = cabi.VitEncoder(be, vcfg, max_patches=(n + 3) // 4 * 4)
    try:
        enc.load_weights(weights)
        if device_io:
            out = torch.zeros(n // 4, vcfg.out_hidden, device="cuda", dtype=torch.bfloat16)
            enc.encode(pixels.cuda(), grids, out)
            be.synchronize()
            out = out.cpu()
        else:
            out = torch.zeros(n // 4, vcfg.out_hidden, dtype=torch.bfloat16)
            enc.encode(pixels, grids, out)
        return out.float()
    finally:
        enc.close()
        be.close()


@pytest.mark.parametrize("case,device_io", [("one_window", False), ("ragged", True), ("frames_and_image", False)])
def test_tiny_encoder_matches_oracle_and_hf(case, device_io):
    z = np.load(os.path.join(os.path.dirname(__file__), "golden", "qwen_vit_tiny.npz"))
    vcfg = qwen_vit.VitConfig(**eval(str(z["cfg"])))
    w = qwen_vit.make_weights(vcfg, seed=int(z["seed"]))
    grids = [tuple(g) for g in z[case + "_grids"].tolist()]
    px = qwen_vit.make_pixels(vcfg, grids, seed=int(z["seed"]))
    got = run_encoder(vcfg, w, px, grids, device_io)
    want = qwen_vit.VitOracle(vcfg, w, "bf16_points").forward(px, grids)
    hf = torch.from_numpy(z[case + "_out"])
    scale = hf.abs().max().item()
    assert (got - want).abs().max().item() <= 0.02 * scale      # same rounding points: a few bf16 ulps
    assert (got - hf).abs().max().item() <= 0.03 * scale        # vs transformers in fp32


def test_encoder_rejects_bad_input():
    be = tiny_backend()
    vcfg = qwen_vit.VitConfig(depth=1, hidden=160, heads=2, intermediate=344, out_hidden=96, fullatt=(0,))
    enc = cabi.VitEncoder(be, vcfg, max_patches=64)
    try:
        out = torch.zeros(16, 96, dtype=torch.bfloat16)
        px = torch.zeros(64, vcfg.patch_dim, dtype=torch.bfloat16)
        with pytest.raises(cabi.BackendError, match="not finalized"):
            enc.encode(px, [(1, 8, 8)], out)
        enc.load_weights(qwen_vit.make_weights(vcfg, seed=0))
        with pytest.raises(cabi.BackendError, match="max_patches"):
            enc.encode(torch.zeros(128, vcfg.patch_dim, dtype=torch.bfloat16), [(2, 8, 8)], torch.zeros(32, 96, dtype=torch.bfloat16))
        with pytest.raises(cabi.BackendError, match="merge size"):
            enc.encode(px, [(1, 7, 8)], out)
        enc.encode(px, [(1, 8, 8)], out)                        # still usable after the refusals
    finally:
        enc.close()
        be.close()


@pytest.mark.parametrize("idx", [2, 3])
def test_full_size_encoder_against_oracle(idx):
    """The benchmark images (448x448 -> 1024 patches; 1288x728 -> 4784 patches) through all 32 layers."""
    vcfg, grids = qwen_vit.CONFIGS[idx], [qwen_vit.GRIDS[idx]]
    w = qwen_vit.make_weights(vcfg, seed=idx)
    px = qwen_vit.make_pixels(vcfg, grids, seed=idx)
    got = run_encoder(vcfg, w, px, grids, device_io=True)
    want = qwen_vit.VitOracle(vcfg, w, "bf16_points").forward(px, grids)
    exact = qwen_vit.VitOracle(vcfg, w, "exact_fp32").forward(px, grids)
    scale = exact.abs().max().item()
    assert torch.isfinite(got).all()
    assert (got - want).abs().max().item() <= 0.03 * scale
    assert (got - exact).abs().max().item() <= 0.05 * scale
    # cosine similarity per produced token against the exact oracle
    cos = torch.nn.functional.cosine_similarity(got, exact, dim=1)
    assert cos.min().item() > 0.995
