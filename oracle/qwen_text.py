"""fp32 torch-CPU oracle of the Qwen2.5 / Qwen2.5-VL text tower.  Test infrastructure only.

Three modes:

* ``exact_fp32``  — every intermediate stays fp32 (weights are the bf16 checkpoint
  values upcast).  Logit tolerance (2e-2 relative) is graded against this mode.
* ``kv_bf16``     — fp32 everywhere except the K / V rows, which are rounded to bf16
  when they enter the cache: the storage format the engine configuration prescribes
  (``kvcache.dtype: bf16``).  Separates what the cache format costs from what the
  kernels cost: on the 1.5B shape at 768 tokens of context the cache rounding alone
  moves the logits by 0.7e-2 (max-norm, relative) against ``exact_fp32``.
* ``bf16_points`` — same math, but every value the CUDA path stores as bf16 is
  rounded to bf16 at that point.  Rows that go through the prefill GEMMs round
  the norm output, the QKV outputs, rotated q/k, the attention output and the
  SiLU-gated activation.  A row that goes through the decode kernels (every
  decode step, and the LAST row of a sampled prefill, which the CUDA path runs
  as a decode step so that all logits come from one arithmetic) keeps fp32
  activations and rounds only the K row (once, after the rotation) and the V row
  it appends to the cache.  The residual stream is fp32 on the GPU and here.
  Greedy-token identity is graded against this mode.

Dataflow follows src/models/qwen2_5/qwen2_5.cpp:534-930 of the reference:
embedding -> per layer [RMSNorm -> fused QKV (+bias) -> RoPE -> attention over the
cache -> o_proj -> residual add -> RMSNorm -> SiLU-gated MLP -> residual add]
-> final RMSNorm -> lm_head (fp32 logits of the last row).

Two deliberate differences from the reference.  (1) The reference stores the
residual stream in bf16 after every add (tests/operators/test_norm_sampler.py:82-86);
here it stays fp32: on 24-36 layer stacks the bf16 stream alone costs about as much
logit error as the whole 2e-2 budget.

(2) The reference's text path keeps K
unrotated in the cache and lets the attention kernel rotate every cached key each
step (src/operators/attention_op.cu:1428-1466, kRoPELlama).  Here K is rotated
once, when it is appended (what the reference itself does for M-RoPE models,
src/engine/tasks/token_generation/cuda/kernels/decode_runtime_kernels.cu:152-225).
In exact arithmetic the two are identical; in ``bf16_points`` mode the rotated
key is rounded to bf16 once.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch


@dataclass
class QwenConfig:
    num_layers: int
    hidden: int
    q_heads: int
    kv_heads: int
    intermediate: int
    vocab: int
    rms_eps: float = 1e-6
    rope_theta: float = 1e6
    tied: bool = True
    mrope_section: Optional[List[int]] = None   # e.g. [16, 24, 24] for Qwen2.5-VL
    model_type: str = "qwen2"
    eos_token_id: int = 151645

    @property
    def head_dim(self) -> int:          # reference: kv_manager.cpp:80 (hidden / q heads)
        return self.hidden // self.q_heads

    def hf_config(self) -> dict:
        cfg = {
            "architectures": ["Qwen2ForCausalLM"],
            "model_type": self.model_type,
            "num_hidden_layers": self.num_layers,
            "hidden_size": self.hidden,
            "num_attention_heads": self.q_heads,
            "num_key_value_heads": self.kv_heads,
            "intermediate_size": self.intermediate,
            "vocab_size": self.vocab,
            "rms_norm_eps": self.rms_eps,
            "rope_theta": self.rope_theta,
            "hidden_act": "silu",
            "torch_dtype": "bfloat16",
            "tie_word_embeddings": self.tied,
            "eos_token_id": self.eos_token_id,
            "max_position_embeddings": 32768,
        }
        if self.mrope_section is not None:
            cfg["rope_scaling"] = {"type": "mrope", "mrope_section": list(self.mrope_section)}
        return cfg


def _bf16_round(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).to(torch.float32)


def rope_inv_freq(head_dim: int, theta: float) -> torch.Tensor:
    """inv_freq[d] = theta^(-2d/D), d in [0, D/2)   (attention_op.cu:362-363)."""
    d = torch.arange(head_dim // 2, dtype=torch.float64)
    return torch.pow(torch.tensor(theta, dtype=torch.float64), -2.0 * d / head_dim).to(torch.float32)


def mrope_pair_section(head_dim: int, section: Sequence[int]) -> torch.Tensor:
    """Which of the three position rows drives rotary pair d (layers/attention.cu:36-55)."""
    c0, c1 = section[0], section[0] + section[1]
    d = torch.arange(head_dim // 2)
    return (d >= c0).long() + (d >= c1).long()


def apply_rope(x: torch.Tensor, pos: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """Rotate-half RoPE.  x: [S, heads, D] fp32; pos: [S, D/2] (per-pair positions, fp32).

    o[d] = x0*cos - x1*sin ; o[d+D/2] = x1*cos + x0*sin   (attention_op.cu:359-369)
    """
    half = x.shape[-1] // 2
    ang = pos.to(torch.float32) * inv_freq[None, :]            # [S, D/2] fp32 product
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    x0, x1 = x[..., :half], x[..., half:]
    return torch.cat([x0 * c - x1 * s, x1 * c + x0 * s], dim=-1)


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """x * rsqrt(mean(x^2) + eps) * w in fp32 (test_norm_sampler.py:62-64)."""
    inv = torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)
    return x * inv * w


def silu(x: torch.Tensor) -> torch.Tensor:
    return x / (1.0 + torch.exp(-x))       # activation_op.cu:18-20


class QwenTextOracle:
    """Keeps one KV cache (one request slot).  Weights: dict of HF-named bf16 tensors."""

    def __init__(self, cfg: QwenConfig, weights: Dict[str, torch.Tensor], mode: str = "bf16_points"):
        assert mode in ("bf16_points", "exact_fp32", "kv_bf16")
        self.cfg, self.mode = cfg, mode
        self.r = _bf16_round if mode == "bf16_points" else (lambda t: t)
        self.r_kv = (lambda t: t) if mode == "exact_fp32" else _bf16_round
        f = lambda n: weights[n].to(torch.float32)
        self.embed = f("model.embed_tokens.weight")
        self.lm_head = self.embed if "lm_head.weight" not in weights else f("lm_head.weight")
        self.final_norm = f("model.norm.weight")
        self.layers = []
        for l in range(cfg.num_layers):
            p = f"model.layers.{l}."
            self.layers.append({
                "in_norm": f(p + "input_layernorm.weight"),
                "post_norm": f(p + "post_attention_layernorm.weight"),
                "wqkv": torch.cat([f(p + "self_attn.q_proj.weight"), f(p + "self_attn.k_proj.weight"),
                                   f(p + "self_attn.v_proj.weight")], dim=0),
                "bqkv": torch.cat([f(p + "self_attn.q_proj.bias"), f(p + "self_attn.k_proj.bias"),
                                   f(p + "self_attn.v_proj.bias")], dim=0),
                "wo": f(p + "self_attn.o_proj.weight"),
                "wg": f(p + "mlp.gate_proj.weight"),
                "wu": f(p + "mlp.up_proj.weight"),
                "wd": f(p + "mlp.down_proj.weight"),
            })
        self.inv_freq = rope_inv_freq(cfg.head_dim, cfg.rope_theta)
        self.pair_section = (mrope_pair_section(cfg.head_dim, cfg.mrope_section)
                             if cfg.mrope_section is not None else None)
        self.reset()

    # ------------------------------------------------------------------ cache
    def reset(self) -> None:
        c = self.cfg
        self.k_cache = [torch.zeros(0, c.kv_heads, c.head_dim) for _ in range(c.num_layers)]
        self.v_cache = [torch.zeros(0, c.kv_heads, c.head_dim) for _ in range(c.num_layers)]

    @property
    def kv_len(self) -> int:
        return self.k_cache[0].shape[0]

    def truncate(self, n: int) -> None:
        self.k_cache = [k[:n] for k in self.k_cache]
        self.v_cache = [v[:n] for v in self.v_cache]

    # ---------------------------------------------------------------- forward
    def embed_tokens(self, ids: Sequence[int], embeds: Optional[torch.Tensor] = None,
                     embed_token_id: int = -1) -> torch.Tensor:
        """Row gather with custom-embedding injection (embed_head.cu:93-116)."""
        c = self.cfg
        out = torch.zeros(len(ids), c.hidden)
        n_custom = 0 if embeds is None else embeds.shape[0]
        for t, tok in enumerate(ids):
            if embeds is not None and embed_token_id >= 0 and embed_token_id <= tok < embed_token_id + n_custom:
                out[t] = embeds[tok - embed_token_id].to(torch.float32)
            elif 0 <= tok < c.vocab:
                out[t] = self.embed[tok]
        return out

    def forward(self, ids: Sequence[int], embeds: Optional[torch.Tensor] = None, embed_token_id: int = -1,
                position_ids: Optional[torch.Tensor] = None, all_logits: bool = False, tail: bool = True) -> torch.Tensor:
        """Append len(ids) tokens to the cache; return fp32 logits of the last row ([V]),
        or of every row ([S, V]) when all_logits.  position_ids: [3, S] for M-RoPE models;
        text models use the cache index as position (attention_op.cu: q at kv_len-1).
        tail (bf16_points mode only): the last row is computed with the decode kernels' rounding
        points (a sampled prefill or a decode step); False: every row takes the prefill GEMMs'
        (a prefix prefill without sampling)."""
        c = self.cfg
        S, P, D = len(ids), self.kv_len, c.head_dim
        r_all = self.r
        last_custom = embeds is not None and embed_token_id >= 0 and embed_token_id <= ids[-1] < embed_token_id + embeds.shape[0]
        if self.mode == "bf16_points" and tail and not last_custom and 0 <= ids[-1] < c.vocab:
            keep = torch.zeros(S, dtype=torch.bool)
            keep[-1] = True                                  # rows that keep fp32 activations

            def r(t):                                        # [S, ...]: round every row but the kept ones
                k = keep.view(S, *([1] * (t.dim() - 1)))
                return torch.where(k, t, _bf16_round(t))
        else:
            keep = None
            r = r_all
        if self.pair_section is not None:
            assert position_ids is not None and tuple(position_ids.shape) == (3, S)
            pos = position_ids.to(torch.float32)[self.pair_section, :].T.contiguous()      # [S, D/2]
        else:
            pos = torch.arange(P, P + S, dtype=torch.float32)[:, None].expand(S, D // 2)
        R = self.embed_tokens(ids, embeds, embed_token_id)
        qd, kd = c.q_heads * D, c.kv_heads * D
        group = c.q_heads // c.kv_heads
        # causal mask with the query offset = tokens already cached (qwen2_5.cpp:812-814)
        kpos = torch.arange(P + S)[None, :]
        qpos = torch.arange(P, P + S)[:, None]
        mask = kpos <= qpos                                                     # [S, P+S]
        for l, w in enumerate(self.layers):
            n = r(rmsnorm(R, w["in_norm"], c.rms_eps))
            qkv = r(n @ w["wqkv"].T + w["bqkv"])
            q = r(apply_rope(qkv[:, :qd].reshape(S, c.q_heads, D), pos, self.inv_freq))
            # the cache holds bf16 for every row: kept rows round K once (after the rotation) and V once
            k = self.r_kv(apply_rope(qkv[:, qd:qd + kd].reshape(S, c.kv_heads, D), pos, self.inv_freq))
            v = self.r_kv(qkv[:, qd + kd:].reshape(S, c.kv_heads, D))
            self.k_cache[l] = torch.cat([self.k_cache[l], k], dim=0)
            self.v_cache[l] = torch.cat([self.v_cache[l], v], dim=0)
            K = self.k_cache[l].repeat_interleave(group, dim=1)                 # [T, q_heads, D]
            V = self.v_cache[l].repeat_interleave(group, dim=1)
            s = torch.einsum("shd,thd->hst", q, K) / math.sqrt(D)
            s = s.masked_fill(~mask[None], float("-inf"))
            p = torch.softmax(s, dim=-1)
            attn = r(torch.einsum("hst,thd->shd", p, V).reshape(S, qd))
            R = R + attn @ w["wo"].T                # residual stream stays fp32 in both modes
            n2 = r(rmsnorm(R, w["post_norm"], c.rms_eps))
            act = r(silu(n2 @ w["wg"].T) * (n2 @ w["wu"].T))
            R = R + act @ w["wd"].T
        rows = R if all_logits else R[-1:]
        hn = rmsnorm(rows, self.final_norm, c.rms_eps)
        if keep is None or all_logits:
            hn = r_all(hn) if keep is None else r(hn)
        logits = hn @ self.lm_head.T
        return logits if all_logits else logits[0]


def greedy(logits: torch.Tensor) -> int:
    """argmax, ties -> lowest index (sampler.cu:17-35)."""
    m = logits.max()
    return int(torch.nonzero(logits == m)[0, 0])


def top2_margin(logits: torch.Tensor) -> float:
    v = torch.topk(logits, 2).values
    return float(v[0] - v[1])


@dataclass
class GenerateResult:
    tokens: List[int] = field(default_factory=list)
    logits: List[torch.Tensor] = field(default_factory=list)
    margins: List[float] = field(default_factory=list)


def generate(oracle: QwenTextOracle, prompt: Sequence[int], max_new_tokens: int, *, sampler=None,
             embeds=None, embed_token_id=-1, position_ids=None, mrope_last_pos=None,
             forced: Optional[Sequence[int]] = None, keep_logits: bool = True) -> GenerateResult:
    """generate() semantics of the reference (standard_engine.cpp:925-1035): one prefill over
    the not-yet-cached part of ``prompt`` (the oracle's cache already holds any fixed prefix),
    a sample, then one decode step per further token.  ``forced`` teacher-forces the token fed
    back at each step (the returned tokens are still this oracle's own choices).
    sampler(logits, step) -> id; default greedy."""
    res = GenerateResult()
    P = oracle.kv_len
    todo = list(prompt[P:])
    pid = position_ids[:, P:] if position_ids is not None else None
    logits = oracle.forward(todo, embeds, embed_token_id, pid)
    mr = None
    if oracle.pair_section is not None:
        if mrope_last_pos is None:
            mrope_last_pos = [int(position_ids.max())] * 3
        mr = list(mrope_last_pos)
    for step in range(max_new_tokens):
        tok = greedy(logits) if sampler is None else sampler(logits, step)
        res.tokens.append(tok)
        res.margins.append(top2_margin(logits))
        if keep_logits:
            res.logits.append(logits.clone())
        if step + 1 == max_new_tokens:
            break
        feed = tok if forced is None else int(forced[step])
        if mr is not None:          # decode positions: mrope_last_pos + generated (qwen2_5.cpp:932-955)
            p3 = torch.tensor([[m + step + 1] for m in mr], dtype=torch.int64)
            logits = oracle.forward([feed], position_ids=p3)
        else:
            logits = oracle.forward([feed])
    return res
