"""Sampling oracle: greedy, and seeded temperature + top-p.  Test infrastructure only.

The reference samples either by argmax (temperature < 1e-6; ties -> lowest index,
src/layers/sampler.cu:17-35,146-200) or by softmax(logits / T) + inverse-CDF with a
Philox stream whose offset is pinned to 0 (src/layers/sampler.cu:270-296 — the same
uniform every step).  It has no top-p.  Top-p with a per-step counter is therefore
DEFINED here (parity unpinned by the reference) and the CUDA sampler implements
exactly this definition, in integers, so that the result does not depend on how the
vocabulary is split across threads:

1. M = max(logits);  e_i = fp32 exp((l_i - M) * (1/T));  w_i = min(floor(e_i * 2^31), 2^31 - 1).
   All probability mass below is in these integer units (sums are exact in uint64).  W = sum(w_i).
2. Order tokens by (w descending, id ascending).  The nucleus is the shortest prefix of that
   order whose mass reaches target = double(W) * double(top_p); so token j is in the nucleus
   iff the mass E_j strictly before it in that order satisfies double(E_j) < target.
3. Rejection rounds k = 0, 1, ...: the candidates are the tokens before the last rejected token
   in that order (every token with w > 0 in round 0) and Wc is their mass.
   x = first word of Philox4x32-10(key = seed, counter = (step, k, 0, 0));
   r = floor(double(x) * double(Wc) * 2^-32)  (double multiplies, round-to-nearest);
   j = the first candidate, walking candidates in ASCENDING TOKEN ID, whose running candidate mass
   exceeds r.  If j is in the nucleus it is the sample; otherwise j is rejected, which also rules
   out everything after it in the order.  After 32 rejections the argmax is returned.
   An accepted token is distributed exactly as nucleus sampling and a round succeeds with
   probability >= top_p, so there is no sort and rarely a second pass over the vocabulary.
"""
from __future__ import annotations

import numpy as np

PHILOX_M0, PHILOX_M1 = 0xD2511F53, 0xCD9E8D57
PHILOX_W0, PHILOX_W1 = 0x9E3779B9, 0xBB67AE85
MASK32 = 0xFFFFFFFF


def philox4x32_10(counter, key):
    """Philox4x32 with 10 rounds (Salmon et al., SC'11).  counter: 4 words, key: 2 words."""
    c = [int(x) & MASK32 for x in counter]
    k = [int(x) & MASK32 for x in key]
    for _ in range(10):
        p0, p1 = PHILOX_M0 * c[0], PHILOX_M1 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k[0]) & MASK32, p1 & MASK32,
             ((p0 >> 32) ^ c[3] ^ k[1]) & MASK32, p0 & MASK32]
        k = [(k[0] + PHILOX_W0) & MASK32, (k[1] + PHILOX_W1) & MASK32]
    return c


def token_weights(logits: np.ndarray, temperature: float) -> np.ndarray:
    """Step 1: integer probability weights (uint64 array holding values <= 2^31)."""
    l = np.asarray(logits, dtype=np.float32)
    inv_t = np.float32(1.0) / np.float32(temperature)
    e = np.exp(((l - l.max()) * inv_t).astype(np.float32)).astype(np.float32)
    return np.minimum(np.floor(e.astype(np.float64) * float(1 << 31)), float((1 << 31) - 1)).astype(np.uint64)


def uniform_word(seed: int, step: int, round_: int = 0) -> int:
    return philox4x32_10([step & MASK32, round_ & MASK32, 0, 0], [seed & MASK32, (seed >> 32) & MASK32])[0]


def nucleus_size(w: np.ndarray, top_p: float) -> int:
    """Number of tokens in the nucleus (used by tests to describe the workload)."""
    target = float(int(w.sum(dtype=np.uint64))) * float(top_p)
    order = np.lexsort((np.arange(w.size), -w.astype(np.int64)))
    cum = np.cumsum(w[order], dtype=np.uint64)
    return min(int(np.searchsorted(cum.astype(np.float64), target, side="left")) + 1, w.size)


def sample_top_p(logits, temperature: float, top_p: float, seed: int, step: int, return_rounds: bool = False):
    l = np.asarray(logits, dtype=np.float32)
    argmax = int(np.flatnonzero(l == l.max())[0])
    if temperature < 1e-6:
        return (argmax, 0) if return_rounds else argmax
    w = token_weights(l, temperature)
    ids = np.arange(w.size)
    top_p = min(max(float(top_p), 1e-9), 1.0)
    target = float(int(w.sum(dtype=np.uint64))) * top_p
    cand = w > 0
    for k in range(32):
        wc = np.where(cand, w, 0).astype(np.uint64)
        Wc = int(wc.sum(dtype=np.uint64))
        if Wc == 0:
            break
        x = uniform_word(seed, step, k)
        r = int(np.floor(np.float64(x) * np.float64(Wc) * np.float64(2.0 ** -32)))
        run = np.cumsum(wc, dtype=np.uint64)
        j = int(np.searchsorted(run, np.uint64(r), side="right"))
        before = (w > w[j]) | ((w == w[j]) & (ids < j))
        E = int(w[before].sum(dtype=np.uint64))
        if float(E) < target:
            return (j, k + 1) if return_rounds else j
        cand = before
    return (argmax, 32) if return_rounds else argmax


def make_sampler(temperature: float, top_p: float, seed: int):
    def f(logits, step):
        return sample_top_p(logits.detach().cpu().numpy() if hasattr(logits, "detach") else logits,
                            temperature, top_p, seed, step)
    return f
