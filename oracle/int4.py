"""Group-wise INT4 (W4A16) weights for the decode pass: quantiser, packer and de-quantiser.  Test / benchmark
infrastructure (the product takes the packed tensors through efm_b200_set_decode_weight).

Weight contract of the reference (src/layers/linear.cu:536-565): per linear ``<name>.qweight`` int8
[out_features / 2, in_features] and ``<name>.scaling_factors`` [in_features / group, out_features], group 128
(src/operators/kernels/int4_groupwise_gemm/int4WoQGemvCuda.cu:228-232), symmetric: w = q * scale with q in [-8, 7].
The reference's kernels read qweight in an interleaved nibble order produced by a packer that is not in its tree
(TensorRT-Edge-LLM); here byte [r][k] simply holds row 2r in its low nibble and row 2r + 1 in its high nibble, each
as q + 8 — parity of the byte layout with the reference is therefore unpinned, the arithmetic (group-wise symmetric
scale, fp16 scale values) follows the contract above.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

GROUP = 128
LINEARS = ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj", "mlp.gate_proj", "mlp.up_proj",
           "mlp.down_proj")


def quantize(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """w [N, K] (any float dtype) -> (q int8 [N, K] in [-8, 7], scales fp16 [K / 128, N]); scale = max|w| / 7 per
    (group of 128 columns, row), rounded to fp16 first so that de-quantisation uses the stored value."""
    N, K = w.shape
    assert K % GROUP == 0 and N % 2 == 0
    wf = w.float().reshape(N, K // GROUP, GROUP)
    s = (wf.abs().amax(dim=2) / 7.0).clamp_min(1e-8).to(torch.float16)           # [N, K / 128]
    q = torch.clamp(torch.round(wf / s.float().unsqueeze(2)), -8, 7).to(torch.int8).reshape(N, K)
    return q, s.T.contiguous()


def pack(q: torch.Tensor) -> torch.Tensor:
    """q int8 [N, K] -> qweight int8 [N / 2, K]: low nibble row 2r, high nibble row 2r + 1, each stored as q + 8."""
    u = (q.to(torch.int16) + 8).to(torch.uint8)
    return (u[0::2] | (u[1::2] << 4)).view(torch.int8).contiguous()


def dequantize(q: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """(q [N, K], scales [K / 128, N]) -> fp32 [N, K] = q * scale."""
    N, K = q.shape
    return (q.float().reshape(N, K // GROUP, GROUP) * scales.T.float().unsqueeze(2)).reshape(N, K)


def quantize_checkpoint(weights: Dict[str, torch.Tensor], num_layers: int, lm_head: bool = True):
    """bf16 checkpoint -> (tensors of the INT4 decode checkpoint: '<linear>.qweight' / '<linear>.scaling_factors';
    the same checkpoint with those linears replaced by their de-quantised fp32 values, for the oracle)."""
    packed, deq = {}, dict(weights)
    names = [f"model.layers.{l}.{n}" for l in range(num_layers) for n in LINEARS]
    if lm_head:
        names.append("lm_head")
    for name in names:
        src = weights.get(name + ".weight")
        if src is None and name == "lm_head":                # tied model: the decode pass gets its own INT4 copy of the table
            src = weights["model.embed_tokens.weight"]
        q, s = quantize(src)
        packed[name + ".qweight"] = pack(q)
        packed[name + ".scaling_factors"] = s
        deq[name + ".weight"] = dequantize(q, s)
    return packed, deq
