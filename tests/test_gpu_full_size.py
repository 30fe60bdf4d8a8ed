"""GPU: the benchmark configurations at their full sizes.

Config 0 (Qwen2.5-0.5B shape, 128-token resident prefix + 64-token prompt) is small enough for the CPU
oracle to finish in seconds, so it is checked against it directly: greedy ids for the first 32 steps
(bf16_points oracle, teacher-forced; a differing id must be a tie within the observed logit error) and
logits within 2e-2 relative of the exact fp32 oracle.  Config 1 (1.5B shape, the benchmarked workload) is
checked through size-independent properties: captured graph == plain launches == persistent kernel,
resident prefix == full prefill, run-to-run determinism of the seeded top-p sampler."""
import os

import numpy as np
import pytest
import torch

import cabi
from oracle import qwen_text, synth

pytestmark = pytest.mark.gpu


def rel(a, b):
    return float(np.abs(a - b).max() / np.abs(b).max())


def test_config0_full_size_against_the_oracle():
    cfg = synth.CONFIGS[0]
    prefix_n, prompt_n, _, temp, top_p = synth.WORKLOADS[0]
    w = synth.make_weights(cfg, seed=0)
    ids = synth.make_token_ids(prefix_n + prompt_n, seed=0)
    steps = 32
    be = cabi.Backend(cfg, max_prefill_tokens=256, max_response_tokens=80)
    be.load_weights(w)
    be.alloc_slot(0, prefix_n + prompt_n + 72)
    be.set_sampling(temp, top_p, 0)
    be.prefill(0, ids[:prefix_n], kv_offset=0, sample=False)                       # warmup(): the resident prefix
    toks, logits = cabi.generate(be, 0, ids, steps, prefix_len=prefix_n, collect_logits=True)
    free, _ = cabi.generate(be, 0, ids, steps, prefix_len=prefix_n)               # captured graph, no host interaction
    assert free == toks
    torch.set_num_threads(os.cpu_count() or 8)
    ob = qwen_text.QwenTextOracle(cfg, w, "bf16_points")
    rb = qwen_text.generate(ob, ids, steps, forced=toks)
    del ob
    oe = qwen_text.QwenTextOracle(cfg, w, "exact_fp32")
    re = qwen_text.generate(oe, ids, steps, forced=toks)
    worst, ties = 0.0, 0
    for s in range(steps):
        e = re.logits[s].numpy()
        worst = max(worst, rel(logits[s], e))
        if toks[s] != rb.tokens[s]:
            assert rb.margins[s] <= 2 * np.abs(logits[s] - rb.logits[s].numpy()).max(), f"step {s}"
            ties += 1
    assert worst < 2e-2, worst
    assert ties <= 3
    be.close()


def test_config1_full_size_properties():
    cfg = synth.CONFIGS[1]
    prefix_n, prompt_n, _, temp, top_p = synth.WORKLOADS[1]
    w = synth.make_weights(cfg, seed=0, device="cuda")
    ids = synth.make_token_ids(prefix_n + prompt_n, seed=0)
    steps = 24
    outs = {}
    for name, env in (("phase_per_launch", "0"), ("persistent", "1")):
        os.environ["EFM_B200_MEGA"] = env
        be = cabi.Backend(cfg, max_prefill_tokens=1024, max_response_tokens=64)
        be.load_weights(w)
        for slot in (0, 1):
            be.alloc_slot(slot, prefix_n + prompt_n + 64)
        be.set_sampling(temp, top_p, 0)
        be.prefill(1, ids[:prefix_n], kv_offset=0, sample=False)
        graph, lg = cabi.generate(be, 0, ids, steps, use_graph=True, collect_logits=True)
        eager, _ = cabi.generate(be, 0, ids, steps, use_graph=False)
        again, _ = cabi.generate(be, 0, ids, steps, use_graph=True)
        prefixed, lp = cabi.generate(be, 1, ids, steps, prefix_len=prefix_n, collect_logits=True)
        assert graph == eager == again                          # seeded sampler: same ids every time
        assert rel(lp[0], lg[0]) < 2e-2                          # resident prefix vs one full prefill
        assert len(set(graph)) > steps // 2                      # top-p at T 0.7 actually samples
        outs[name] = (graph, lg)
        be.close()
    os.environ.pop("EFM_B200_MEGA", None)
    # the two decode forms differ only in how the attention partials are merged (cluster exchange vs scratch +
    # ticket), i.e. in fp32 rounding: same first token, logits of the first decode step equal to rounding.  Later
    # sampled ids may part ways once a rounding difference crosses a top-p boundary.
    a, b = outs["phase_per_launch"], outs["persistent"]
    assert a[0][0] == b[0][0]
    assert rel(a[1][0], b[1][0]) < 1e-6                     # prefill: identical kernels
    assert rel(a[1][1], b[1][1]) < 1e-2                     # bf16 rounding points amplify the fp32 merge difference
