"""Tensor-parallel restatement of the text tower on CPU (torch.distributed, any backend).
Test infrastructure only.

The reference is single-GPU; tensor parallelism is this repository's addition for the 7B-class
shapes.  This file states the partition the CUDA backend uses (efm_b200_set_weight) so that it can be
checked on CPU with gloo ranks against the unpartitioned oracle:

* attention: heads are sharded ``att_shards = min(tp, kv_heads)`` ways; when tp exceeds the number
  of kv heads, ``att_rep = tp / att_shards`` ranks hold the same head shard and split the o_proj
  INPUT columns of that shard between them, so that the all-reduce over all ranks is still the sum;
* MLP: gate/up rows and down columns in tp equal parts;
* lm_head: vocabulary rows in tp equal parts, logits all-gathered;
* embedding and norms replicated; o_proj / down outputs are summed in fp32 across ranks, then the
  residual add happens in fp32 exactly as on one GPU: r += sum.
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Sequence

import torch
import torch.distributed as dist

from .qwen_text import QwenConfig, _bf16_round, apply_rope, mrope_pair_section, rmsnorm, rope_inv_freq, silu


def tp_layout(cfg: QwenConfig, rank: int, tp: int) -> dict:
    att_shards = min(tp, cfg.kv_heads)
    assert tp % att_shards == 0 and cfg.kv_heads % att_shards == 0 and cfg.q_heads % att_shards == 0
    att_rep = tp // att_shards
    q_l, kv_l = cfg.q_heads // att_shards, cfg.kv_heads // att_shards
    D = cfg.head_dim
    assert cfg.intermediate % (64 * tp) == 0 and cfg.vocab % (2 * tp) == 0 and (q_l * D) % (32 * att_rep) == 0
    shard, rep = rank // att_rep, rank % att_rep
    o_k = q_l * D // att_rep
    return dict(att_shards=att_shards, att_rep=att_rep, shard=shard, rep=rep, q_l=q_l, kv_l=kv_l, o_k=o_k,
                q_rows=slice(shard * q_l * D, (shard + 1) * q_l * D),
                kv_rows=slice(shard * kv_l * D, (shard + 1) * kv_l * D),
                o_cols=slice(shard * q_l * D + rep * o_k, shard * q_l * D + (rep + 1) * o_k),
                i_rows=slice(rank * cfg.intermediate // tp, (rank + 1) * cfg.intermediate // tp),
                v_rows=slice(rank * cfg.vocab // tp, (rank + 1) * cfg.vocab // tp))


class TpOracle:
    """One rank of the tensor-parallel model.  `weights` is the WHOLE checkpoint."""

    def __init__(self, cfg: QwenConfig, weights: Dict[str, torch.Tensor], rank: int, tp: int, mode: str = "bf16_points"):
        self.cfg, self.rank, self.tp = cfg, rank, tp
        self.lay = lay = tp_layout(cfg, rank, tp)
        self.r = _bf16_round if mode == "bf16_points" else (lambda t: t)
        f = lambda n: weights[n].to(torch.float32)
        self.embed = f("model.embed_tokens.weight")
        head = self.embed if "lm_head.weight" not in weights else f("lm_head.weight")
        self.lm_head = head[lay["v_rows"]]
        self.final_norm = f("model.norm.weight")
        self.layers = []
        for l in range(cfg.num_layers):
            p = f"model.layers.{l}."
            self.layers.append({
                "in_norm": f(p + "input_layernorm.weight"), "post_norm": f(p + "post_attention_layernorm.weight"),
                "wq": f(p + "self_attn.q_proj.weight")[lay["q_rows"]], "bq": f(p + "self_attn.q_proj.bias")[lay["q_rows"]],
                "wk": f(p + "self_attn.k_proj.weight")[lay["kv_rows"]], "bk": f(p + "self_attn.k_proj.bias")[lay["kv_rows"]],
                "wv": f(p + "self_attn.v_proj.weight")[lay["kv_rows"]], "bv": f(p + "self_attn.v_proj.bias")[lay["kv_rows"]],
                "wo": f(p + "self_attn.o_proj.weight")[:, lay["o_cols"]],
                "wg": f(p + "mlp.gate_proj.weight")[lay["i_rows"]], "wu": f(p + "mlp.up_proj.weight")[lay["i_rows"]],
                "wd": f(p + "mlp.down_proj.weight")[:, lay["i_rows"]],
            })
        self.inv_freq = rope_inv_freq(cfg.head_dim, cfg.rope_theta)
        self.pair_section = mrope_pair_section(cfg.head_dim, cfg.mrope_section) if cfg.mrope_section is not None else None
        self.k_cache = [torch.zeros(0, lay["kv_l"], cfg.head_dim) for _ in range(cfg.num_layers)]
        self.v_cache = [torch.zeros(0, lay["kv_l"], cfg.head_dim) for _ in range(cfg.num_layers)]

    def _sum(self, t: torch.Tensor) -> torch.Tensor:
        t = t.contiguous()
        if self.tp > 1:
            dist.all_reduce(t)
        return t

    def forward(self, ids: Sequence[int], position_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
        c, r, lay = self.cfg, self.r, self.lay
        S, P, D = len(ids), self.k_cache[0].shape[0], c.head_dim
        if self.pair_section is not None:
            pos = position_ids.to(torch.float32)[self.pair_section, :].T.contiguous()
        else:
            pos = torch.arange(P, P + S, dtype=torch.float32)[:, None].expand(S, D // 2)
        R = self.embed[torch.tensor(list(ids))]
        q_l, kv_l = lay["q_l"], lay["kv_l"]
        group = q_l // kv_l
        mask = torch.arange(P + S)[None, :] <= torch.arange(P, P + S)[:, None]
        for l, w in enumerate(self.layers):
            n = r(rmsnorm(R, w["in_norm"], c.rms_eps))
            q = r(apply_rope(r(n @ w["wq"].T + w["bq"]).reshape(S, q_l, D), pos, self.inv_freq))
            k = r(apply_rope(r(n @ w["wk"].T + w["bk"]).reshape(S, kv_l, D), pos, self.inv_freq))
            v = r(n @ w["wv"].T + w["bv"]).reshape(S, kv_l, D)
            self.k_cache[l] = torch.cat([self.k_cache[l], k])
            self.v_cache[l] = torch.cat([self.v_cache[l], v])
            K = self.k_cache[l].repeat_interleave(group, dim=1)
            V = self.v_cache[l].repeat_interleave(group, dim=1)
            s = torch.einsum("shd,thd->hst", q, K) / math.sqrt(D)
            s = s.masked_fill(~mask[None], float("-inf"))
            attn = r(torch.einsum("hst,thd->shd", torch.softmax(s, dim=-1), V).reshape(S, q_l * D))
            mine = attn[:, lay["rep"] * lay["o_k"]:(lay["rep"] + 1) * lay["o_k"]]
            R = R + self._sum(mine @ w["wo"].T)
            n2 = r(rmsnorm(R, w["post_norm"], c.rms_eps))
            act = r(silu(n2 @ w["wg"].T) * (n2 @ w["wu"].T))
            R = R + self._sum(act @ w["wd"].T)
        hn = r(rmsnorm(R[-1:], self.final_norm, c.rms_eps))
        local = (hn @ self.lm_head.T)[0].contiguous()
        if self.tp == 1:
            return local
        parts = [torch.empty_like(local) for _ in range(self.tp)]
        dist.all_gather(parts, local)
        return torch.cat(parts)


def greedy_by_exchange(local: torch.Tensor, rank: int, tp: int) -> int:
    """Greedy sampling as the tensor-parallel decode step does it (sample kernel, tensor-parallel branch): every rank
    reduces its own vocabulary rows to (maximum, lowest local id), the ranks exchange those pairs -- one 8-byte word
    {fp32 maximum, global id} each on the GPU -- and every rank picks the largest value, the lowest global id on ties:
    the id a greedy pass over the gathered logits returns (reference tie rule: src/layers/sampler.cu, lowest index)."""
    v = local.max()
    i = int((local == v).nonzero()[0])
    pair = torch.tensor([float(v), float(rank * local.numel() + i)], dtype=torch.float64)
    if tp == 1:
        return int(pair[1])
    pairs = [torch.empty_like(pair) for _ in range(tp)]
    dist.all_gather(pairs, pair)
    best = max(float(q[0]) for q in pairs)
    return int(min(float(q[1]) for q in pairs if float(q[0]) == best))

