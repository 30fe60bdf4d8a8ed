"""Generates the committed golden vectors in this directory.

The reference's own acceptance test demands exact greedy-token equality with Hugging Face
Transformers (tests/engine/test_qwen2_generate.py:758-1227 of windog-labs/edge-fm-x).  Real
checkpoints are unavailable offline, so the same check is made on seeded tiny checkpoints:
transformers' Qwen2ForCausalLM (fp32, CPU, eager attention) is loaded with the synthetic
state dict and run greedily; prompt, generated ids and per-step logits are stored.
tests/test_oracle_golden.py requires the CPU oracle to reproduce these files.

Run from the repository root (needs transformers; CPU only):
    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import synth  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))

CASES = {
    "qwen2_tiny_tied": dict(cfg=dict(num_layers=2, hidden=128, q_heads=2, kv_heads=1, intermediate=256,
                                     vocab=1000, tied=True), seed=0, prompt=12, steps=20),
    "qwen2_small_untied": dict(cfg=dict(num_layers=3, hidden=256, q_heads=4, kv_heads=2, intermediate=512,
                                        vocab=2000, tied=False, rope_theta=1e4), seed=1, prompt=33, steps=20),
}


def run_hf(cfg, weights, prompt, steps):
    from transformers import Qwen2Config, Qwen2ForCausalLM
    hf_cfg = Qwen2Config(**{k: v for k, v in cfg.hf_config().items() if k not in ("architectures", "model_type")},
                         attn_implementation="eager")
    model = Qwen2ForCausalLM(hf_cfg).to(torch.float32).eval()
    sd = {k: v.to(torch.float32) for k, v in weights.items()}
    if cfg.tied:
        sd["lm_head.weight"] = sd["model.embed_tokens.weight"]
    missing, unexpected = model.load_state_dict(sd, strict=False)
    assert not unexpected and all("rotary" in m or "inv_freq" in m for m in missing), (missing, unexpected)
    ids = torch.tensor([prompt])
    toks, logits = [], []
    with torch.no_grad():
        out = model(ids, use_cache=True)
        past = out.past_key_values
        for s in range(steps):
            lg = out.logits[0, -1].to(torch.float32)
            logits.append(lg.numpy().copy())
            t = int(torch.argmax(lg))
            toks.append(t)
            if s + 1 < steps:
                out = model(torch.tensor([[t]]), past_key_values=past, use_cache=True)
                past = out.past_key_values
    return toks, np.stack(logits)


def main():
    for name, case in CASES.items():
        cfg = synth.tiny_config(**case["cfg"])
        w = synth.make_weights(cfg, seed=case["seed"])
        prompt = synth.make_token_ids(case["prompt"], seed=case["seed"], vocab=cfg.vocab)
        toks, logits = run_hf(cfg, w, prompt, case["steps"])
        np.savez_compressed(os.path.join(HERE, name + ".npz"), prompt=np.array(prompt, dtype=np.int32),
                            tokens=np.array(toks, dtype=np.int32), logits=logits.astype(np.float32),
                            cfg=np.array(repr(case["cfg"])), seed=np.array(case["seed"]))
        print(name, toks[:8], logits.shape)


if __name__ == "__main__":
    main()
