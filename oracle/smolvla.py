"""CPU restatement of the SmolVLA-shaped action chunk (fp32 torch).  Test infrastructure only:
the product never imports this file.

The reference project ships no code for this model, only a description:
doc/smolvla_architecture.md (vision tower and connector :155-259, Llama backbone :264-409, action
expert :411-517, flow-matching head and suffix embedding :519-617, mask rule :619-656, the two
inference phases :776-1150).  The timestep plumbing follows the reference's Euler loop
(src/engine/tasks/trajectory_planning/trajectory_planner_engine.cpp:70-78,298-318).

Pinning: the vision tower and the connector (pixel shuffle + projection) are checked against
transformers.models.smolvlm.modeling_smolvlm (SmolVLMVisionTransformer, SmolVLMConnector) through
tests/golden/smolvla_vision_tiny.npz (made by tests/golden/make_golden_smolvla.py).  The backbone /
expert glue has no runnable public implementation in this environment (lerobot is not installed):
PARITY UNPINNED for that part; it restates the description above, with these choices where the
description is silent or inconsistent:
  * expert MLP width = the description's own formula (round 4 * int(2 * 720 / 3) up to 256) = 2048;
  * RoPE base 1e5 (rotate-half) for backbone and expert; prefix positions 0..P-1, suffix positions
    P..P+n-1 in the self-attention layers and 0..n-1 in the cross-attention layers;
  * image tokens and language embeddings are multiplied by sqrt(hidden); the state token is not;
  * prefix mask: image and language tokens see each other, the state token sees everything, nothing
    sees the state token; suffix mask: every prefix token visible, causal among action tokens;
  * time embedding: sin/cos of 2*pi*t / period, periods geometric between 4e-3 and 4.0, computed in
    fp64 and rounded to fp32;
  * t runs 1.0, 0.9, ... and x += dt * v with dt = -1/steps.

Numeric modes as in oracle/qwen_text.py: "exact_fp32" and "bf16_points" (activations rounded to
bf16 where the CUDA path stores bf16; residual streams and the action state stay fp32).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List

import torch


@dataclass
class VlaConfig:
    image_size: int = 512
    patch: int = 16
    vit_layers: int = 12
    vit_hidden: int = 768
    vit_heads: int = 12
    vit_mlp: int = 3072
    shuffle: int = 4
    n_images: int = 3
    hidden: int = 960
    layers: int = 16
    q_heads: int = 15
    kv_heads: int = 5
    head_dim: int = 64
    mlp: int = 2560
    vocab: int = 49152
    lang_tokens: int = 48
    expert_hidden: int = 720
    expert_mlp: int = 2048
    state_dim: int = 32
    action_dim: int = 32
    chunk: int = 50
    steps: int = 10
    rope_theta: float = 1e5
    rms_eps: float = 1e-5
    ln_eps: float = 1e-6

    @property
    def side(self) -> int:
        return self.image_size // self.patch

    @property
    def patches(self) -> int:
        return self.side * self.side

    @property
    def image_tokens(self) -> int:
        return self.patches // (self.shuffle * self.shuffle)

    @property
    def prefix(self) -> int:
        return self.n_images * self.image_tokens + self.lang_tokens + 1

    @property
    def patch_dim(self) -> int:
        return 3 * self.patch * self.patch

    @staticmethod
    def tiny() -> "VlaConfig":
        return VlaConfig(image_size=128, patch=16, vit_layers=2, vit_hidden=128, vit_heads=2, vit_mlp=256, shuffle=4,
                         n_images=2, hidden=192, layers=4, q_heads=3, kv_heads=1, head_dim=64, mlp=256, vocab=512,
                         lang_tokens=8, expert_hidden=128, expert_mlp=256, chunk=10, steps=4)


def _bf16_round(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.bfloat16).to(torch.float32)


def weight_names(c: VlaConfig) -> List[tuple]:
    """(name, shape, kind) in a fixed order; kind 'n' = norm weight (1 + noise), 'w' = plain."""
    Hv, H, He = c.vit_hidden, c.hidden, c.expert_hidden
    QD, KD = c.q_heads * c.head_dim, c.kv_heads * c.head_dim
    out = [("vit.patch.weight", (Hv, c.patch_dim), "w"), ("vit.patch.bias", (Hv,), "w"), ("vit.pos", (c.patches, Hv), "w")]
    for l in range(c.vit_layers):
        p = f"vit.{l}."
        out += [(p + "ln1.weight", (Hv,), "n"), (p + "ln1.bias", (Hv,), "w")]
        for n in ("q", "k", "v", "o"):
            out += [(p + n + ".weight", (Hv, Hv), "w"), (p + n + ".bias", (Hv,), "w")]
        out += [(p + "ln2.weight", (Hv,), "n"), (p + "ln2.bias", (Hv,), "w"),
                (p + "fc1.weight", (c.vit_mlp, Hv), "w"), (p + "fc1.bias", (c.vit_mlp,), "w"),
                (p + "fc2.weight", (Hv, c.vit_mlp), "w"), (p + "fc2.bias", (Hv,), "w")]
    out += [("vit.post_ln.weight", (Hv,), "n"), ("vit.post_ln.bias", (Hv,), "w"),
            ("connector.weight", (H, Hv * c.shuffle * c.shuffle), "w"),
            ("embed", (c.vocab, H), "w"), ("state_proj.weight", (H, c.state_dim), "w"), ("state_proj.bias", (H,), "w")]
    for l in range(c.layers):
        p = f"vlm.{l}."
        out += [(p + "norm1", (H,), "n"), (p + "q.weight", (QD, H), "w"), (p + "k.weight", (KD, H), "w"),
                (p + "v.weight", (KD, H), "w"), (p + "o.weight", (H, QD), "w"), (p + "norm2", (H,), "n"),
                (p + "gate.weight", (c.mlp, H), "w"), (p + "up.weight", (c.mlp, H), "w"), (p + "down.weight", (H, c.mlp), "w")]
    for l in range(c.layers):
        p = f"expert.{l}."
        kin = He if l % 2 == 0 else KD          # cross-attention layers re-project the backbone's K / V rows
        out += [(p + "norm1", (He,), "n"), (p + "q.weight", (QD, He), "w"), (p + "k.weight", (KD, kin), "w"),
                (p + "v.weight", (KD, kin), "w"), (p + "o.weight", (He, QD), "w"), (p + "norm2", (He,), "n"),
                (p + "gate.weight", (c.expert_mlp, He), "w"), (p + "up.weight", (c.expert_mlp, He), "w"),
                (p + "down.weight", (He, c.expert_mlp), "w")]
    out += [("expert.norm", (He,), "n"),
            ("action_in.weight", (He, c.action_dim), "w"), ("action_in.bias", (He,), "w"),
            ("time_in.weight", (He, 2 * He), "w"), ("time_in.bias", (He,), "w"),
            ("time_out.weight", (He, He), "w"), ("time_out.bias", (He,), "w"),
            ("action_out.weight", (c.action_dim, He), "w"), ("action_out.bias", (c.action_dim,), "w")]
    return out


def make_weights(c: VlaConfig, seed: int = 0) -> Dict[str, torch.Tensor]:
    """bf16 weights from one generator: N(0, 1/sqrt(fan_in)) matrices (so that activations keep unit scale through
    the 16-layer stacks), N(0, 0.02) vectors, norm weights 1 + N(0, 0.02)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape, kind in weight_names(c):
        if len(shape) == 2 and name not in ("vit.pos", "embed"):
            t = torch.randn(*shape, generator=g) * (0.5 / math.sqrt(shape[1]))
        else:
            t = torch.randn(*shape, generator=g) * 0.02
        out[name] = (1.0 + t if kind == "n" else t).to(torch.bfloat16)
    return out


def make_inputs(c: VlaConfig, seed: int = 0):
    """Synthetic request as the benchmark describes it: images uniform in [0, 1] mapped to [-1, 1], random prompt
    ids, state uniform in [-1, 1], N(0, 1) noise."""
    g = torch.Generator().manual_seed(seed + 4242)
    images = torch.rand(c.n_images, 3, c.image_size, c.image_size, generator=g) * 2.0 - 1.0
    ids = torch.randint(0, c.vocab, (c.lang_tokens,), generator=g, dtype=torch.int32)
    state = torch.rand(c.state_dim, generator=g) * 2.0 - 1.0
    noise = torch.randn(c.chunk, c.action_dim, generator=g)
    return images, ids, state, noise


def layernorm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) * torch.rsqrt(var + eps) * w + b


def rmsnorm(x, w, eps):
    return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w


def gelu_tanh(x):
    return 0.5 * x * (1.0 + torch.tanh(0.7978845608028654 * (x + 0.044715 * x ** 3)))


def rope_half(x: torch.Tensor, pos: torch.Tensor, theta: float) -> torch.Tensor:
    """x [n, heads, D]; rotate-half with inverse frequencies theta^(-2i/D)."""
    D = x.shape[-1]
    inv = theta ** (-torch.arange(0, D, 2, dtype=torch.float32) / D)
    ang = pos.to(torch.float32)[:, None] * inv[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    x1, x2 = x[..., : D // 2], x[..., D // 2:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)


def attention(q, k, v, visible: torch.Tensor) -> torch.Tensor:
    """q [n, Hq, D], k/v [m, Hkv, D], visible [n, m] bool -> [n, Hq*D] (grouped-query, fp32 softmax)."""
    n, Hq, D = q.shape
    rep = Hq // k.shape[1]
    kk, vv = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    s = torch.einsum("nhd,mhd->hnm", q, kk) / math.sqrt(D)
    s = s.masked_fill(~visible[None], float("-inf"))
    return torch.einsum("hnm,mhd->nhd", torch.softmax(s, dim=-1), vv).reshape(n, Hq * D)


def pixel_shuffle(x: torch.Tensor, side: int, s: int) -> torch.Tensor:
    """[side*side, d] -> [(side/s)^2, d*s*s]: output token (R, C) holds, at channel (ry*s + cx)*d + e, the value of
    patch (R*s + ry, C*s + cx) channel e."""
    d = x.shape[-1]
    x = x.reshape(side // s, s, side // s, s, d)          # R, ry, C, cx, e
    return x.permute(0, 2, 1, 3, 4).reshape((side // s) ** 2, s * s * d)


def time_embedding(t: float, dim: int, min_period: float = 4e-3, max_period: float = 4.0) -> torch.Tensor:
    frac = torch.linspace(0.0, 1.0, dim // 2, dtype=torch.float64)
    period = min_period * (max_period / min_period) ** frac
    ang = (2.0 * math.pi / period) * t
    return torch.cat([ang.sin(), ang.cos()]).to(torch.float32)


class VlaOracle:
    def __init__(self, cfg: VlaConfig, weights: Dict[str, torch.Tensor], mode: str = "bf16_points"):
        assert mode in ("exact_fp32", "bf16_points")
        self.c = cfg
        self.r = _bf16_round if mode == "bf16_points" else (lambda t: t)
        self.w = {k: v.to(torch.float32) for k, v in weights.items()}

    # ---- vision tower + connector: [n_images, 3, S, S] -> [n_images * image_tokens, hidden] ----
    def vision(self, images: torch.Tensor) -> torch.Tensor:
        c, r, w = self.c, self.r, self.w
        p, side, Hv = c.patch, c.side, c.vit_hidden
        n = images.shape[0]
        # patch rows, (channel, ky, kx) inside a row as in the convolution weight
        rows = images.to(torch.float32).reshape(n, 3, side, p, side, p).permute(0, 2, 4, 1, 3, 5).reshape(n * c.patches, c.patch_dim)
        x = r(rows) @ w["vit.patch.weight"].T + w["vit.patch.bias"] + w["vit.pos"].repeat(n, 1)
        vis = torch.zeros(n * c.patches, n * c.patches, dtype=torch.bool)
        for i in range(n):
            vis[i * c.patches:(i + 1) * c.patches, i * c.patches:(i + 1) * c.patches] = True
        D = Hv // c.vit_heads
        for l in range(c.vit_layers):
            q_ = f"vit.{l}."
            h = r(layernorm(x, w[q_ + "ln1.weight"], w[q_ + "ln1.bias"], c.ln_eps))
            q = r(h @ w[q_ + "q.weight"].T + w[q_ + "q.bias"]).reshape(-1, c.vit_heads, D)
            k = r(h @ w[q_ + "k.weight"].T + w[q_ + "k.bias"]).reshape(-1, c.vit_heads, D)
            v = r(h @ w[q_ + "v.weight"].T + w[q_ + "v.bias"]).reshape(-1, c.vit_heads, D)
            a = r(attention(q, k, v, vis))
            x = x + (a @ w[q_ + "o.weight"].T + w[q_ + "o.bias"])
            h = r(layernorm(x, w[q_ + "ln2.weight"], w[q_ + "ln2.bias"], c.ln_eps))
            f = r(gelu_tanh(h @ w[q_ + "fc1.weight"].T + w[q_ + "fc1.bias"]))
            x = x + (f @ w[q_ + "fc2.weight"].T + w[q_ + "fc2.bias"])
        x = r(layernorm(x, w["vit.post_ln.weight"], w["vit.post_ln.bias"], c.ln_eps))
        toks = torch.cat([pixel_shuffle(x[i * c.patches:(i + 1) * c.patches], side, c.shuffle) for i in range(n)])
        return toks @ w["connector.weight"].T

    # ---- prefix: embeddings, backbone layers, per-layer rotated K and V ----
    def prefix(self, images, ids, state):
        c, r, w = self.c, self.r, self.w
        H, P = c.hidden, c.prefix
        x = torch.cat([self.vision(images) * math.sqrt(H),
                       w["embed"][ids.long()] * math.sqrt(H),
                       (state.to(torch.float32) @ w["state_proj.weight"].T + w["state_proj.bias"])[None, :]])
        assert x.shape == (P, H)
        vis = torch.ones(P, P, dtype=torch.bool)
        vis[: P - 1, P - 1] = False
        pos = torch.arange(P)
        cache = []
        for l in range(c.layers):
            p = f"vlm.{l}."
            h = r(rmsnorm(x, w[p + "norm1"], c.rms_eps))
            q = r(rope_half(r(h @ w[p + "q.weight"].T).reshape(P, c.q_heads, c.head_dim), pos, c.rope_theta))
            k = r(rope_half(r(h @ w[p + "k.weight"].T).reshape(P, c.kv_heads, c.head_dim), pos, c.rope_theta))
            v = r(h @ w[p + "v.weight"].T).reshape(P, c.kv_heads, c.head_dim)
            cache.append((k, v))
            a = r(attention(q, k, v, vis))
            x = x + a @ w[p + "o.weight"].T
            h = r(rmsnorm(x, w[p + "norm2"], c.rms_eps))
            g, u = h @ w[p + "gate.weight"].T, h @ w[p + "up.weight"].T
            x = x + r(g * torch.sigmoid(g) * u) @ w[p + "down.weight"].T
        return x, cache

    # ---- one denoising step: velocity [chunk, action_dim] ----
    def velocity(self, x_t: torch.Tensor, t: float, cache) -> torch.Tensor:
        c, r, w = self.c, self.r, self.w
        n, P, He = c.chunk, c.prefix, c.expert_hidden
        a_emb = x_t @ w["action_in.weight"].T + w["action_in.bias"]
        cat = r(torch.cat([a_emb, time_embedding(t, He)[None, :].expand(n, He)], dim=1))
        h = cat @ w["time_in.weight"].T + w["time_in.bias"]
        x = r(h * torch.sigmoid(h)) @ w["time_out.weight"].T + w["time_out.bias"]
        vis_self = torch.cat([torch.ones(n, P, dtype=torch.bool), torch.tril(torch.ones(n, n, dtype=torch.bool))], dim=1)
        vis_cross = torch.ones(n, P, dtype=torch.bool)
        for l in range(c.layers):
            p = f"expert.{l}."
            kc, vc = cache[l]
            h = r(rmsnorm(x, w[p + "norm1"], c.rms_eps))
            q = r(h @ w[p + "q.weight"].T).reshape(n, c.q_heads, c.head_dim)
            if l % 2 == 0:
                pos = torch.arange(P, P + n)
                q = r(rope_half(q, pos, c.rope_theta))
                k = r(rope_half(r(h @ w[p + "k.weight"].T).reshape(n, c.kv_heads, c.head_dim), pos, c.rope_theta))
                v = r(h @ w[p + "v.weight"].T).reshape(n, c.kv_heads, c.head_dim)
                a = attention(q, torch.cat([kc, k]), torch.cat([vc, v]), vis_self)
            else:
                q = r(rope_half(q, torch.arange(n), c.rope_theta))
                k = r(kc.reshape(P, -1) @ w[p + "k.weight"].T).reshape(P, c.kv_heads, c.head_dim)
                v = r(vc.reshape(P, -1) @ w[p + "v.weight"].T).reshape(P, c.kv_heads, c.head_dim)
                a = attention(q, k, v, vis_cross)
            x = x + r(a) @ w[p + "o.weight"].T
            h = r(rmsnorm(x, w[p + "norm2"], c.rms_eps))
            g, u = h @ w[p + "gate.weight"].T, h @ w[p + "up.weight"].T
            x = x + r(g * torch.sigmoid(g) * u) @ w[p + "down.weight"].T
        h = r(rmsnorm(x, w["expert.norm"], c.rms_eps))
        return h @ w["action_out.weight"].T + w["action_out.bias"]

    def chunk(self, images, ids, state, noise) -> torch.Tensor:
        c = self.c
        _, cache = self.prefix(images, ids, state)
        x_t = noise.to(torch.float32).clone()
        dt = -1.0 / c.steps
        for s in range(c.steps):
            x_t = x_t + dt * self.velocity(x_t, 1.0 + s * dt, cache)
        return x_t
