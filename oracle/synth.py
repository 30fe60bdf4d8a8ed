"""Seeded synthetic checkpoints, inputs and engine configs.  Test / benchmark infrastructure.

Real Qwen2.5 checkpoints and tokenizers are not available offline, so every workload is a
random-initialised model of the named architecture: each weight N(0, 0.02) rounded to bf16
(RMSNorm weights 1 + N(0, 0.02), so that the normalised activations keep unit scale),
drawn in a fixed tensor order from one torch.Generator(seed).  Token ids are uniform in
[0, 151643) (below the special-token range of the Qwen2.5 vocabulary).  The on-disk layout
is what the reference loads: an HF directory with config.json + model.safetensors
(src/engine/engine_factory.cpp:27-49), plus an engine JSON with the keys of
examples/config/base/engine_default.json.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional

import torch

from .qwen_text import QwenConfig

# Architectures named by the benchmark configurations (index = configuration number).
CONFIGS = {
    0: QwenConfig(24, 896, 14, 2, 4864, 151936, tied=True),                      # Qwen2.5-0.5B
    1: QwenConfig(28, 1536, 12, 2, 8960, 151936, tied=True),                     # Qwen2.5-1.5B
    2: QwenConfig(36, 2048, 16, 2, 11008, 151936, tied=True, mrope_section=[16, 24, 24],
                  model_type="qwen2_5_vl"),                                      # Qwen2.5-VL-3B LLM
    3: QwenConfig(28, 3584, 28, 4, 18944, 152064, tied=False, mrope_section=[16, 24, 24],
                  model_type="qwen2_5_vl"),                                      # Qwen2.5-VL-7B LLM
}
# (fixed prefix tokens, prompt tokens, decode steps, temperature, top_p)
WORKLOADS = {0: (128, 64, 64, 0.0, 1.0), 1: (512, 256, 256, 0.7, 0.9),
             2: (0, 320, 128, 0.0, 1.0), 3: (0, 1324, 256, 0.0, 1.0)}

TOKEN_ID_RANGE = 151643


def tiny_config(**kw) -> QwenConfig:
    """Small model with the real head_dim (64) for fast oracle-vs-CUDA comparisons."""
    base = dict(num_layers=2, hidden=128, q_heads=2, kv_heads=1, intermediate=256, vocab=1000, tied=True)
    base.update(kw)
    return QwenConfig(**base)


def weight_names(cfg: QwenConfig) -> List[tuple]:
    D, H, I = cfg.head_dim, cfg.hidden, cfg.intermediate
    out = [("model.embed_tokens.weight", (cfg.vocab, H), "w")]
    for l in range(cfg.num_layers):
        p = f"model.layers.{l}."
        out += [
            (p + "input_layernorm.weight", (H,), "n"),
            (p + "self_attn.q_proj.weight", (cfg.q_heads * D, H), "w"),
            (p + "self_attn.q_proj.bias", (cfg.q_heads * D,), "w"),
            (p + "self_attn.k_proj.weight", (cfg.kv_heads * D, H), "w"),
            (p + "self_attn.k_proj.bias", (cfg.kv_heads * D,), "w"),
            (p + "self_attn.v_proj.weight", (cfg.kv_heads * D, H), "w"),
            (p + "self_attn.v_proj.bias", (cfg.kv_heads * D,), "w"),
            (p + "self_attn.o_proj.weight", (H, cfg.q_heads * D), "w"),
            (p + "post_attention_layernorm.weight", (H,), "n"),
            (p + "mlp.gate_proj.weight", (I, H), "w"),
            (p + "mlp.up_proj.weight", (I, H), "w"),
            (p + "mlp.down_proj.weight", (H, I), "w"),
        ]
    out.append(("model.norm.weight", (H,), "n"))
    if not cfg.tied:
        out.append(("lm_head.weight", (cfg.vocab, H), "w"))
    return out


def make_weights(cfg: QwenConfig, seed: int = 0, device: str = "cpu", std: float = 0.02) -> Dict[str, torch.Tensor]:
    """bf16 tensors keyed by HF names.  device='cuda' draws on the GPU (used only where no
    CPU oracle run needs the same values, e.g. the 7B-shaped property tests)."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    w = {}
    for name, shape, kind in weight_names(cfg):
        t = torch.randn(shape, generator=g, device=device, dtype=torch.float32) * std
        if kind == "n":
            t += 1.0
        w[name] = t.to(torch.bfloat16)
    return w


def make_token_ids(n: int, seed: int = 0, vocab: Optional[int] = None) -> List[int]:
    g = torch.Generator()
    g.manual_seed(seed)
    hi = TOKEN_ID_RANGE if vocab is None else min(TOKEN_ID_RANGE, vocab)
    return torch.randint(0, hi, (n,), generator=g).tolist()


def vlm_request(cfg_id: int) -> dict:
    """Image-first multimodal prompt of configurations 2 / 3: the image's merged tokens (ids >= vocab select rows of
    the injected embeddings), then text.  M-RoPE positions: image t = 0, h = merged row, w = merged column; text
    continues from max(rows, columns) on all three axes."""
    from . import qwen_vit
    cfg = CONFIGS[cfg_id]
    vcfg = qwen_vit.CONFIGS[cfg_id]
    t, h, w = qwen_vit.GRIDS[cfg_id]
    hm, wm = h // vcfg.merge, w // vcfg.merge
    n_img = t * hm * wm
    n_text = WORKLOADS[cfg_id][1] - n_img
    ids = [cfg.vocab + k for k in range(n_img)] + make_token_ids(n_text, seed=0)
    start = max(hm, wm)
    text_pos = [start + i for i in range(n_text)]
    pos = [[0] * n_img + text_pos,
           [r for r in range(hm) for _ in range(wm)] * t + text_pos,
           [c for _ in range(hm) for c in range(wm)] * t + text_pos]
    return {"vcfg": vcfg, "grids": [(t, h, w)], "ids": ids, "pos": pos, "n_img": n_img, "embed_id": cfg.vocab,
            "last": start + n_text - 1}


def write_checkpoint(dirname: str, cfg: QwenConfig, weights: Dict[str, torch.Tensor]) -> str:
    from safetensors.torch import save_file
    os.makedirs(dirname, exist_ok=True)
    with open(os.path.join(dirname, "config.json"), "w") as f:
        json.dump(cfg.hf_config(), f, indent=1)
    save_file({k: v.contiguous().cpu() for k, v in weights.items()}, os.path.join(dirname, "model.safetensors"))
    return dirname


def write_engine_config(path: str, model_dir: str, *, model_name: str = "Qwen2.5", prefix_ids=(),
                        max_tokens: int = 4096, max_new_tokens: int = 64, temperature: float = 0.0,
                        top_p: float = 1.0, seed: int = 0, use_cuda_graph: bool = True, device_id: int = 0,
                        extra_requests=(), stop_token_ids=()) -> str:
    """Engine JSON with the key set of the reference's engine_default.json.  The user file is
    shallow-merged over defaults (src/engine/engine.cpp:212), so whole sections are given."""
    reqs = [{"request_id": 0, "prefix_token_ids": list(prefix_ids), "max_tokens": max_tokens}]
    reqs += list(extra_requests)
    cfg = {
        "model_name": model_name,
        "runtime": {"device": "cuda", "device_id": device_id, "use_cuda_graph": use_cuda_graph,
                    "hw_profile": "cuda_sm100"},
        "prefill_model_path": model_dir,
        "kvcache": {"dtype": "bf16", "attention_type": "gqa", "requests": reqs},
        "sampling": {"temperature": temperature, "top_p": top_p, "top_k": 1, "seed": seed,
                     "max_new_tokens": max_new_tokens, "stop_token_ids": list(stop_token_ids)},
    }
    with open(path, "w") as f:
        json.dump(cfg, f)
    return path
