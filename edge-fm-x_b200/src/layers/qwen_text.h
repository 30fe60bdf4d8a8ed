// Launch sequences of the text tower (definitions in qwen_text.cu).
#pragma once
#include "../backends/b200/ctx.h"

namespace efm {
struct Launcher;
struct GemmParams;
struct SampleParams;
struct SegAttnParams;
enum class GemmEpi : int;

// One decode step: reads the device state (token, kv_len, positions), appends K/V at row
// kv_len-1, samples, advances the state.  All launches go through L (graph-capturable).
void qwen_decode_step(efm_b200_ctx& c, KvSlot& slot, Launcher& L);
// One prefill chunk over c.ids[0:S] (already on the device), KV rows [kv_offset, kv_offset+S).
void qwen_prefill_chunk(efm_b200_ctx& c, KvSlot& slot, int S, int kv_offset, int n_custom, int embed_token_id,
                        bool sample_last, Launcher& L);
// Final norm + lm_head + sampler on one residual row.
void launch_lm_head_and_sample(efm_b200_ctx& c, Launcher& L, const float* resid_row, int advance, bool decode_pass = false);
// Tensor parallel + imported peer buffers + greedy sampling: the sampler exchanges the ranks' maxima itself and the full
// logits vector is not gathered (tp_gather_logits does that on demand).
bool tp_greedy_exchange(const efm_b200_ctx& c);
void tp_gather_logits(efm_b200_ctx& c, Launcher& L);
// Single operators (used by the per-operator C entry points).
void launch_gemm_bf16(Launcher& L, const GemmParams& p);
// C = A . B^T on the tensor cores with the named epilogue; error_word (device int, may be null) is
// raised when a bounded pipeline wait gives up.
void launch_gemm_epi(Launcher& L, GemmEpi epi, const GemmParams& p, int* error_word);
// Attention with per-query key ranges (or the causal prefill rule when p.lo is null).
void launch_seg_attention(Launcher& L, const SegAttnParams& p, int D);
// Same result; picks the all-keys-resident variant when D == 64, S <= 64 and max_keys (largest hi) <= 320.
void launch_seg_attention_short(Launcher& L, const SegAttnParams& p, int D, int max_keys);
// INT8 prefill attention (sage_attention.cuh): pre-pass (key mean, INT8 Q / centred K + scales, fp16 V) into
// `sc`, then the attention kernel.  q: [S, q_heads*D] rotated queries; k/v: cache rows [0, kv_offset + S).
void launch_sage_prefill_attention(Launcher& L, const SageScratch& sc, const __nv_bfloat16* q, const __nv_bfloat16* k,
                                   const __nv_bfloat16* v, __nv_bfloat16* out, int S, int kv_offset, int q_heads,
                                   int kv_heads, int D, int* error = nullptr);
void launch_sample(Launcher& L, const SampleParams& p);
cudaError_t configure_sampler();      // once per device at set-up, never inside a stream capture
// y[r,:] = bf16(rmsnorm(x[r,:]) * w) over `rows` fp32 rows.
void launch_rmsnorm_rows(Launcher& L, const float* x, const __nv_bfloat16* w, __nv_bfloat16* y, int rows, int hidden, float eps);
void launch_prefill_attention(Launcher& L, const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* v,
                              __nv_bfloat16* out, int S, int kv_offset, int q_heads, int kv_heads, int D,
                              int* error = nullptr);
// checkpoint layout -> kernel layout of one INT4 linear (operators/gemv_w4.cuh: w4_repack_kernel)
struct W4RepackParams;
void launch_w4_repack(Launcher& L, const W4RepackParams& p);

}  // namespace efm
