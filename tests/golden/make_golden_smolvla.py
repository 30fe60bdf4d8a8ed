"""Makes tests/golden/smolvla_vision_tiny.npz: outputs of the public SmolVLM vision tower and connector
(transformers.models.smolvlm.modeling_smolvlm) on a tiny configuration, for pinning oracle/smolvla.py.

Run from the repository root in an environment that has `transformers`:  python tests/golden/make_golden_smolvla.py
"""
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "..", ".."))
from oracle import smolvla  # noqa: E402


def main():
    from transformers.models.smolvlm import modeling_smolvlm as m

    c = smolvla.VlaConfig.tiny()
    w = {k: v.to(torch.float32) for k, v in smolvla.make_weights(c, seed=11).items()}
    vcfg = m.SmolVLMVisionConfig(hidden_size=c.vit_hidden, intermediate_size=c.vit_mlp, num_hidden_layers=c.vit_layers,
                                 num_attention_heads=c.vit_heads, num_channels=3, image_size=c.image_size,
                                 patch_size=c.patch, hidden_act="gelu_pytorch_tanh", layer_norm_eps=c.ln_eps,
                                 attention_dropout=0.0)
    vcfg._attn_implementation = "eager"
    vit = m.SmolVLMVisionTransformer(vcfg).to(torch.float32).eval()
    sd = {"embeddings.patch_embedding.weight": w["vit.patch.weight"].reshape(c.vit_hidden, 3, c.patch, c.patch),
          "embeddings.patch_embedding.bias": w["vit.patch.bias"],
          "embeddings.position_embedding.weight": w["vit.pos"],
          "post_layernorm.weight": w["vit.post_ln.weight"], "post_layernorm.bias": w["vit.post_ln.bias"]}
    for l in range(c.vit_layers):
        p, q = f"encoder.layers.{l}.", f"vit.{l}."
        for a, b in (("self_attn.q_proj", "q"), ("self_attn.k_proj", "k"), ("self_attn.v_proj", "v"),
                     ("self_attn.out_proj", "o"), ("layer_norm1", "ln1"), ("layer_norm2", "ln2"),
                     ("mlp.fc1", "fc1"), ("mlp.fc2", "fc2")):
            sd[p + a + ".weight"] = w[q + b + ".weight"]
            sd[p + a + ".bias"] = w[q + b + ".bias"]
    missing = vit.load_state_dict(sd, strict=True)
    images, _, _, _ = smolvla.make_inputs(c, seed=11)
    mask = torch.ones(c.n_images, c.side, c.side, dtype=torch.bool)
    with torch.no_grad():
        hidden = vit(pixel_values=images, patch_attention_mask=mask).last_hidden_state      # [n, patches, Hv]

        class _Cfg:       # the two fields SmolVLMConnector / SmolVLMSimpleMLP read
            scale_factor = c.shuffle
            vision_config = vcfg
            text_config = type("T", (), {"hidden_size": c.hidden})()
        conn = m.SmolVLMConnector(_Cfg()).to(torch.float32).eval()
        conn.load_state_dict({"modality_projection.proj.weight": w["connector.weight"]}, strict=True)
        out = conn(hidden).reshape(c.n_images * c.image_tokens, c.hidden)

    mine = smolvla.VlaOracle(c, smolvla.make_weights(c, seed=11), mode="exact_fp32").vision(images)
    err = (mine - out).abs().max().item()
    print("max |oracle - transformers| =", err, "scale", out.abs().max().item())
    assert err < 1e-4 * max(1.0, out.abs().max().item())
    np.savez_compressed(os.path.join(os.path.dirname(__file__), "smolvla_vision_tiny.npz"),
                        seed=np.int64(11), expected=out.numpy().astype(np.float32),
                        vit_hidden=hidden.reshape(-1, c.vit_hidden).numpy().astype(np.float32))


if __name__ == "__main__":
    main()
