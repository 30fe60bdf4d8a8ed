"""CPU restatement of the Qwen2.5-VL vision encoder (fp32 torch).  Test infrastructure only:
the product never imports this file.

The reference project has no vision tower (image embeddings are computed outside and injected
through Request.embedding, examples/qwen2.5-vl-3b-instruct/generate.py:3); the algorithm is the
published Qwen2.5-VL one, whose public implementation is
transformers.models.qwen2_5_vl.modeling_qwen2_5_vl.Qwen2_5_VisionTransformerPretrainedModel.
This file states it independently and is pinned to that implementation by
tests/golden/qwen_vit_tiny.npz (made by tests/golden/make_golden_vit.py, checked by
tests/test_oracle_golden.py).

Shapes: pixel rows [N, C*T*P*P] in merge-block-major order (every 4 consecutive rows are one 2x2
block of patches; blocks row-major over the merged grid, frames outermost); output [N/4, out].

Two numeric modes as in oracle/qwen_text.py: "exact_fp32" (no rounding) and "bf16_points"
(activations rounded to bf16 where the CUDA path stores bf16; the residual stream stays fp32).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Sequence, Tuple

import torch


@dataclass
class VitConfig:
    depth: int = 32
    hidden: int = 1280
    heads: int = 16
    intermediate: int = 3420
    out_hidden: int = 2048
    patch: int = 14
    temporal_patch: int = 2
    in_channels: int = 3
    merge: int = 2
    window: int = 112
    fullatt: Tuple[int, ...] = (7, 15, 23, 31)
    rms_eps: float = 1e-6
    rope_theta: float = 10000.0

    @property
    def head_dim(self) -> int:
        return self.hidden // self.heads

    @property
    def patch_dim(self) -> int:
        return self.in_channels * self.temporal_patch * self.patch * self.patch

    def hf_config(self) -> dict:
        return dict(depth=self.depth, hidden_size=self.hidden, num_heads=self.heads,
                    intermediate_size=self.intermediate, out_hidden_size=self.out_hidden,
                    patch_size=self.patch, temporal_patch_size=self.temporal_patch,
                    in_channels=self.in_channels, spatial_merge_size=self.merge, window_size=self.window,
                    fullatt_block_indexes=list(self.fullatt), hidden_act="silu")


CONFIGS = {2: VitConfig(out_hidden=2048), 3: VitConfig(out_hidden=3584)}
# patch grids (t, h, w) of the benchmark images: 448x448 and 1288x728 (h = 728/14, w = 1288/14)
GRIDS = {2: (1, 32, 32), 3: (1, 52, 92)}


def _bf16_round(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.bfloat16).to(torch.float32)


@dataclass
class VitPlan:
    """Everything the encoder derives from the patch grid alone."""
    order: List[int]            # merged-token permutation: position i holds merged token order[i]
    cu_window: List[int]        # patch offsets of the attention windows (in permuted order)
    cu_full: List[int]          # patch offsets of the frames (full-attention layers)
    pos_h: List[int]            # per patch, permuted order: patch row / column inside its frame
    pos_w: List[int] = field(default_factory=list)


def make_plan(cfg: VitConfig, grids: Sequence[Tuple[int, int, int]]) -> VitPlan:
    """Window-major token order, window/frame boundaries and 2-D positions.

    A window covers window/patch/merge merged tokens per side (4 for the released models); windows
    tile each frame row-major and edge windows are partial."""
    m = cfg.merge
    win = cfg.window // cfg.patch // m
    order, cu_window, cu_full, rows, cols = [], [0], [0], [], []
    base = 0
    for (t, H, W) in grids:
        assert H % m == 0 and W % m == 0
        h, w = H // m, W // m
        for f in range(t):
            for wr in range((h + win - 1) // win):
                for wc in range((w + win - 1) // win):
                    n = 0
                    for r in range(wr * win, min(h, (wr + 1) * win)):
                        for c in range(wc * win, min(w, (wc + 1) * win)):
                            order.append(base + (f * h + r) * w + c)
                            for dy in range(m):
                                for dx in range(m):
                                    rows.append(r * m + dy)
                                    cols.append(c * m + dx)
                            n += 1
                    cu_window.append(cu_window[-1] + n * m * m)
            cu_full.append(cu_full[-1] + H * W)
        base += t * h * w
    return VitPlan(order, cu_window, cu_full, rows, cols)


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return x * torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps) * w


def gelu_erf(x: torch.Tensor) -> torch.Tensor:
    return 0.5 * x * (1.0 + torch.erf(x / math.sqrt(2.0)))


def rope_2d(x: torch.Tensor, pos_h: torch.Tensor, pos_w: torch.Tensor, theta: float) -> torch.Tensor:
    """x [S, heads, D].  D/4 angles from the row index, D/4 from the column index; the D/2 angles
    are used twice (pair d <-> d + D/2), rotate-half over the whole head."""
    D = x.shape[-1]
    q = D // 4
    inv = 1.0 / (theta ** (torch.arange(0, q, dtype=torch.float32) * 2.0 / (D // 2)))
    ang = torch.cat([pos_h[:, None].float() * inv[None], pos_w[:, None].float() * inv[None]], dim=1)   # [S, D/2]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., : D // 2], x[..., D // 2:]
    return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)


def segment_attention(q, k, v, cu: Sequence[int]) -> torch.Tensor:
    """Bidirectional softmax attention inside each [cu[i], cu[i+1]) row range.  q, k, v [S, h, D]."""
    out = torch.empty_like(q)
    scale = 1.0 / math.sqrt(q.shape[-1])
    for a, b in zip(cu[:-1], cu[1:]):
        if b == a:
            continue
        s = torch.einsum("shd,thd->hst", q[a:b], k[a:b]) * scale
        out[a:b] = torch.einsum("hst,thd->shd", torch.softmax(s, dim=-1), v[a:b])
    return out


class VitOracle:
    def __init__(self, cfg: VitConfig, weights: Dict[str, torch.Tensor], mode: str = "bf16_points",
                 prefix: str = "visual."):
        assert mode in ("exact_fp32", "bf16_points")
        self.cfg = cfg
        self.r = _bf16_round if mode == "bf16_points" else (lambda t: t)
        f = lambda n: weights[prefix + n].to(torch.float32)
        self.w_patch = f("patch_embed.proj.weight").reshape(cfg.hidden, cfg.patch_dim)
        self.blocks = []
        for l in range(cfg.depth):
            p = f"blocks.{l}."
            self.blocks.append({k: f(p + k) for k in (
                "norm1.weight", "norm2.weight", "attn.qkv.weight", "attn.qkv.bias", "attn.proj.weight",
                "attn.proj.bias", "mlp.gate_proj.weight", "mlp.gate_proj.bias", "mlp.up_proj.weight",
                "mlp.up_proj.bias", "mlp.down_proj.weight", "mlp.down_proj.bias")})
        self.ln_q = f("merger.ln_q.weight")
        self.m0w, self.m0b = f("merger.mlp.0.weight"), f("merger.mlp.0.bias")
        self.m2w, self.m2b = f("merger.mlp.2.weight"), f("merger.mlp.2.bias")

    def forward(self, pixels: torch.Tensor, grids: Sequence[Tuple[int, int, int]]) -> torch.Tensor:
        c, r = self.cfg, self.r
        unit = c.merge * c.merge
        plan = make_plan(c, grids)
        N = pixels.shape[0]
        assert N == plan.cu_full[-1] and pixels.shape[1] == c.patch_dim
        order = torch.tensor(plan.order)
        x = r(pixels.to(torch.float32)) @ self.w_patch.T                       # [N, hidden], fp32 stream
        x = x.reshape(N // unit, unit, c.hidden)[order].reshape(N, c.hidden)   # window-major order
        ph, pw = torch.tensor(plan.pos_h), torch.tensor(plan.pos_w)
        H, D = c.heads, c.head_dim
        for l, w in enumerate(self.blocks):
            n = r(rmsnorm(x, w["norm1.weight"], c.rms_eps))
            qkv = r(n @ w["attn.qkv.weight"].T + w["attn.qkv.bias"]).reshape(N, 3, H, D)
            q = r(rope_2d(qkv[:, 0], ph, pw, c.rope_theta))
            k = r(rope_2d(qkv[:, 1], ph, pw, c.rope_theta))
            cu = plan.cu_full if l in c.fullatt else plan.cu_window
            a = r(segment_attention(q, k, qkv[:, 2], cu).reshape(N, c.hidden))
            x = x + (a @ w["attn.proj.weight"].T + w["attn.proj.bias"])
            n2 = r(rmsnorm(x, w["norm2.weight"], c.rms_eps))
            g = n2 @ w["mlp.gate_proj.weight"].T + w["mlp.gate_proj.bias"]
            u = n2 @ w["mlp.up_proj.weight"].T + w["mlp.up_proj.bias"]
            act = r(g * torch.sigmoid(g) * u)
            x = x + (act @ w["mlp.down_proj.weight"].T + w["mlp.down_proj.bias"])
        n = r(rmsnorm(x, self.ln_q, c.rms_eps)).reshape(N // unit, unit * c.hidden)
        h1 = r(gelu_erf(n @ self.m0w.T + self.m0b))
        out = r(h1 @ self.m2w.T + self.m2b)
        inv = torch.empty_like(order)
        inv[order] = torch.arange(order.numel())
        return out[inv]


def weight_names(cfg: VitConfig, prefix: str = "visual.") -> List[tuple]:
    Hd, I = cfg.hidden, cfg.intermediate
    out = [(prefix + "patch_embed.proj.weight",
            (Hd, cfg.in_channels, cfg.temporal_patch, cfg.patch, cfg.patch), "w")]
    for l in range(cfg.depth):
        p = f"{prefix}blocks.{l}."
        out += [(p + "norm1.weight", (Hd,), "n"), (p + "norm2.weight", (Hd,), "n"),
                (p + "attn.qkv.weight", (3 * Hd, Hd), "w"), (p + "attn.qkv.bias", (3 * Hd,), "w"),
                (p + "attn.proj.weight", (Hd, Hd), "w"), (p + "attn.proj.bias", (Hd,), "w"),
                (p + "mlp.gate_proj.weight", (I, Hd), "w"), (p + "mlp.gate_proj.bias", (I,), "w"),
                (p + "mlp.up_proj.weight", (I, Hd), "w"), (p + "mlp.up_proj.bias", (I,), "w"),
                (p + "mlp.down_proj.weight", (Hd, I), "w"), (p + "mlp.down_proj.bias", (Hd,), "w")]
    M = Hd * cfg.merge * cfg.merge
    out += [(prefix + "merger.ln_q.weight", (Hd,), "n"),
            (prefix + "merger.mlp.0.weight", (M, M), "w"), (prefix + "merger.mlp.0.bias", (M,), "w"),
            (prefix + "merger.mlp.2.weight", (cfg.out_hidden, M), "w"),
            (prefix + "merger.mlp.2.bias", (cfg.out_hidden,), "w")]
    return out


def make_weights(cfg: VitConfig, seed: int = 0, device: str = "cpu", prefix: str = "visual.") -> Dict[str, torch.Tensor]:
    """bf16 N(0, 0.02) weights (norm weights 1 + N(0, 0.02)) in a fixed order from one generator."""
    g = torch.Generator(device=device).manual_seed(seed)
    out = {}
    for name, shape, kind in weight_names(cfg, prefix):
        t = torch.randn(*shape, generator=g, device=device) * 0.02
        out[name] = (1.0 + t if kind == "n" else t).to(torch.bfloat16)
    return out


def image_mean_std():
    """Per-channel normalisation constants of the Qwen2-VL image processor, read from transformers at run time."""
    from transformers.image_utils import OPENAI_CLIP_MEAN, OPENAI_CLIP_STD
    return list(OPENAI_CLIP_MEAN), list(OPENAI_CLIP_STD)


def make_pixels(cfg: VitConfig, grids: Sequence[Tuple[int, int, int]], seed: int = 0, device: str = "cpu") -> torch.Tensor:
    """Synthetic images as the benchmark describes them: RGB uniform in [0, 1], mean/std normalised, already in the
    processor's patch-row layout [n_patches, C*T*P*P] (channel-major inside a row), bf16."""
    n = sum(t * h * w for t, h, w in grids)
    g = torch.Generator(device=device).manual_seed(seed + 7919)
    px = torch.rand(n, cfg.in_channels, cfg.temporal_patch * cfg.patch * cfg.patch, generator=g, device=device)
    mean, std = image_mean_std()
    if len(mean) == cfg.in_channels:
        m = torch.tensor(mean, device=device)[None, :, None]
        s = torch.tensor(std, device=device)[None, :, None]
        px = (px - m) / s
    return px.reshape(n, cfg.patch_dim).to(torch.bfloat16)
