"""Generates tests/golden/qwen_vit_tiny.npz: outputs of transformers'
Qwen2_5_VisionTransformerPretrainedModel (fp32, CPU, eager attention) on a seeded tiny vision
tower with the real head_dim (80), window size and merge size, for two ragged patch grids and
one two-image batch.  tests/test_oracle_golden.py requires oracle/qwen_vit.py to reproduce it.

Run from the repository root (needs transformers; CPU only):
    python tests/golden/make_golden_vit.py
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import qwen_vit  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))

TINY = dict(depth=4, hidden=160, heads=2, intermediate=344, out_hidden=96, fullatt=(1, 3))
SEED = 3
# (t, h, w) patch grids: one full 8x8-patch window; ragged edges (merged 5x7); video frames + image
CASES = {"one_window": [(1, 8, 8)], "ragged": [(1, 10, 14)], "frames_and_image": [(2, 12, 6), (1, 4, 18)]}


def run_hf(cfg, weights, pixels, grids):
    from transformers.models.qwen2_5_vl.configuration_qwen2_5_vl import Qwen2_5_VLVisionConfig
    from transformers.models.qwen2_5_vl.modeling_qwen2_5_vl import Qwen2_5_VisionTransformerPretrainedModel
    hf_cfg = Qwen2_5_VLVisionConfig(**cfg.hf_config())
    hf_cfg._attn_implementation = "eager"
    model = Qwen2_5_VisionTransformerPretrainedModel(hf_cfg).to(torch.float32).eval()
    sd = {k[len("visual."):]: v.to(torch.float32) for k, v in weights.items()}
    missing, unexpected = model.load_state_dict(sd, strict=False)
    assert not unexpected and all("inv_freq" in m for m in missing), (missing, unexpected)
    with torch.no_grad():
        out = model(pixels.to(torch.float32), grid_thw=torch.tensor(grids))
    out = out.pooler_output if hasattr(out, "pooler_output") else out
    return out.to(torch.float32).numpy()


def main():
    cfg = qwen_vit.VitConfig(**TINY)
    w = qwen_vit.make_weights(cfg, seed=SEED)
    blob = dict(cfg=np.array(repr(TINY)), seed=np.array(SEED))
    for name, grids in CASES.items():
        px = qwen_vit.make_pixels(cfg, grids, seed=SEED)
        out = run_hf(cfg, w, px, grids)
        blob[name + "_grids"] = np.array(grids, dtype=np.int32)
        blob[name + "_out"] = out.astype(np.float32)
        print(name, out.shape, float(np.abs(out).mean()))
    np.savez_compressed(os.path.join(HERE, "qwen_vit_tiny.npz"), **blob)


if __name__ == "__main__":
    main()
