"""CPU statement of the INT8 ("SageAttention"-style) prefill attention.  Test infrastructure only.

The reference tree has no source for it (two README mentions, README.md:23,456); the rule below is the
published scheme as the benchmark specification words it:

* per kv head, subtract from every key the mean key over the visible tokens (adds the same constant to all
  scores of a query, so the softmax does not change);
* quantise K (after the subtraction) and Q per block of 128 tokens and per head to INT8 with
  ``scale = max|x| / 127``, ``q = clamp(rint(x / scale), -127, 127)`` (fp32 arithmetic, round half to even);
* ``S = (Qi8 . Ki8^T) * sq * sk / sqrt(D)`` with an exact int32 dot product, causal softmax in fp32;
* ``P`` rounded to fp16, ``V`` taken as fp16 (exact from bf16 in range), ``P . V`` accumulated in fp32 and
  divided by the fp32 row sum of the unrounded ``P``.

Parity unpinned: there is no reference implementation or golden vector to pin this file to; the GPU kernel
is tested against this statement and against exact bf16 attention (error of the INT8 scheme itself).
"""
from __future__ import annotations

import math

import numpy as np
import torch

BLOCK = 128


def quantize_blocks(x: torch.Tensor):
    """x [T, h, D] fp32 -> (int8 [T, h, D], scales [ceil(T/128), h] fp32)."""
    T, h, D = x.shape
    nb = (T + BLOCK - 1) // BLOCK
    q = torch.empty(T, h, D, dtype=torch.int8)
    scales = torch.empty(nb, h, dtype=torch.float32)
    for b in range(nb):
        blk = x[b * BLOCK:(b + 1) * BLOCK]
        amax = blk.abs().amax(dim=(0, 2))                                  # [h]
        s = (amax / np.float32(127.0)).to(torch.float32)
        s = torch.where(s > 0, s, torch.ones_like(s))                      # all-zero block: any scale
        scales[b] = s
        q[b * BLOCK:(b + 1) * BLOCK] = torch.clamp(torch.round(blk / s[None, :, None]), -127, 127).to(torch.int8)
    return q, scales


def key_mean(k: torch.Tensor) -> torch.Tensor:
    """k [T, kvh, D] fp32 -> mean over tokens [kvh, D] (fp32; summation order is not part of the rule)."""
    return k.to(torch.float64).mean(dim=0).to(torch.float32)


def sage_prefill_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, kv_offset: int) -> torch.Tensor:
    """q [S, qh, D], k / v [T, kvh, D] (bf16 values, any float dtype), T = kv_offset + S.
    Query i sees keys [0, kv_offset + i].  Returns fp32 [S, qh, D]."""
    q, k, v = q.to(torch.float32), k.to(torch.float32), v.to(torch.float32)
    S, qh, D = q.shape
    T, kvh, _ = k.shape
    assert T == kv_offset + S
    g = qh // kvh
    qi, sq = quantize_blocks(q)
    ki, sk = quantize_blocks(k - key_mean(k)[None])
    vh = v.to(torch.float16).to(torch.float32)
    out = torch.empty(S, qh, D, dtype=torch.float32)
    qpos = torch.arange(kv_offset, kv_offset + S)
    mask = torch.arange(T)[None, :] <= qpos[:, None]                        # [S, T]
    scale = 1.0 / math.sqrt(D)
    for h in range(qh):
        kh = h // g
        dots = (qi[:, h].to(torch.int32) @ ki[:, kh].to(torch.int32).T).to(torch.float32)      # |dot| <= 127*127*D < 2^24: exact in fp32
        sq_row = sq[torch.arange(S) // BLOCK, h][:, None]
        sk_col = sk[torch.arange(T) // BLOCK, kh][None, :]
        s = dots * (sq_row * sk_col * np.float32(scale))
        s = s.masked_fill(~mask, float("-inf"))
        m = s.max(dim=1, keepdim=True).values
        p = torch.exp(s - m)
        l = p.sum(dim=1, keepdim=True)
        ph = p.to(torch.float16).to(torch.float32)
        out[:, h] = (ph @ vh[:, kh]) / l
    return out


def exact_prefill_attention(q, k, v, kv_offset):
    q, k, v = q.to(torch.float32), k.to(torch.float32), v.to(torch.float32)
    S, qh, D = q.shape
    T, kvh, _ = k.shape
    g = qh // kvh
    K = k.repeat_interleave(g, dim=1)
    V = v.repeat_interleave(g, dim=1)
    s = torch.einsum("shd,thd->hst", q, K) / math.sqrt(D)
    mask = torch.arange(T)[None, :] <= torch.arange(kv_offset, kv_offset + S)[:, None]
    s = s.masked_fill(~mask[None], float("-inf"))
    return torch.einsum("hst,thd->shd", torch.softmax(s, dim=-1), V)
