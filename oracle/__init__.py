"""CPU oracle for the single-request generate() path.  TEST INFRASTRUCTURE ONLY.

Nothing under this package is shipped or measured as the product: it is the
checker that the tests, the smoke entry and the benchmark's CPU-baseline leg use
to verify (and time beside) the CUDA path.  The product path never imports it.

What it restates
----------------
The reference (windog-labs/edge-fm-x) has no CPU implementation of token
generation (src/engine/engine_factory.cpp:147-149 throws without CUDA) and its
arithmetic lives in third-party libraries that are absent from the checkout
(forked FlashInfer @ a9ffab19, cuBLASLt, CUTLASS @ 418d38a5, TRT-LLM fused MoE).
The oracle therefore restates the published layer math in fp32 torch-CPU,
following the reference's own call sites:

* dataflow and residual handling      src/models/qwen2_5/qwen2_5.cpp:534-930
* RMSNorm / fused add + RMSNorm       tests/operators/test_norm_sampler.py:62-64,82-86
* rotate-half RoPE convention         src/operators/attention_op.cu:327-371
* M-RoPE section selection            src/layers/attention.cu:17-72
* SiLU                                src/operators/activation_op.cu:18-20
* embedding lookup with injection     src/layers/embed_head.cu:63-132
* greedy tie rule (lowest index)      src/layers/sampler.cu:17-35
* generate()/prefix semantics         src/engine/tasks/token_generation/cuda/standard_engine.cpp:872-1094,
                                      src/engine/tasks/token_generation/scheduler.cpp:62-154

Pinning
-------
The reference ships no golden vectors (tests/data is absent); its acceptance
test is exact greedy-token equality with Hugging Face Transformers
(tests/engine/test_qwen2_generate.py:758-1227).  The oracle is pinned the same
way: tests/golden/make_golden.py runs transformers' Qwen2ForCausalLM (fp32, CPU)
on seeded tiny checkpoints and commits ids + logits; tests/test_oracle_golden.py
requires the oracle to reproduce them.  Top-p sampling, which the reference does
not implement, is defined here (oracle/sampling.py): parity unpinned for that
component.
"""
