// Host-side state of one backend context: model geometry, device weights, activation
// buffers, KV slots and the captured decode graphs.  Everything is owned per context (the
// reference shares name-keyed buffers process-wide, src/utils/device/memory.h:89-109, which
// makes two engines in one process unsafe; here two contexts never alias).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <map>
#include <string>
#include <vector>

#include "../../../../include/efm_b200.h"
#include "../../operators/common.cuh"

namespace efm {

// One linear of the decode pass in group-wise INT4 (operators/gemv_w4.cuh): kernel-layout weights once `ready`;
// until finalize the checkpoint tensors as they arrived (up to three stacked sources: q | k | v, gate | up).
struct W4Linear {
    uint8_t* q = nullptr;                 // [n_items][K]
    void* s = nullptr;                    // [n_items][K / 128] half2
    int n_items = 0, K = 0;
    bool ready = false;
    void* src_q[3] = {nullptr, nullptr, nullptr};
    void* src_s[3] = {nullptr, nullptr, nullptr};
    int src_s_bf16[3] = {0, 0, 0};
    bool complete(int n_src) const {
        for (int i = 0; i < n_src; ++i)
            if (src_q[i] == nullptr || src_s[i] == nullptr) return false;
        return true;
    }
    bool any() const {
        for (int i = 0; i < 3; ++i)
            if (src_q[i] != nullptr || src_s[i] != nullptr) return true;
        return false;
    }
};

struct LayerWeights {
    __nv_bfloat16* in_norm = nullptr;     // [H]
    __nv_bfloat16* post_norm = nullptr;   // [H]
    __nv_bfloat16* qkv = nullptr;         // [(q+2kv)*D, H] rows: q | k | v
    __nv_bfloat16* qkv_bias = nullptr;    // [(q+2kv)*D]
    __nv_bfloat16* o = nullptr;           // [H, q*D]
    __nv_bfloat16* gate_up = nullptr;     // [2I, H] blocks of 64 gate rows then 64 up rows
    __nv_bfloat16* down = nullptr;        // [H, I]
    uint32_t seen = 0;                    // bit per HF tensor received
    W4Linear w4_qkv, w4_o, w4_gate_up, w4_down;      // decode-only INT4 copies (efm_b200_set_decode_weight)
};

struct KvSlot {
    int max_tokens = 0;
    std::vector<__nv_bfloat16*> k;        // per layer; V block follows K block in the same allocation
    std::vector<__nv_bfloat16*> v;
    cudaGraphExec_t graph = nullptr;      // decode step captured against this slot's pointers
    int graph_nodes = 0;
    int n_splits = 1, chunk_cap = 1, attn_cluster = 0;
};

// Scratch of the INT8 prefill attention (operators/sage_attention.cuh).
struct SageScratch {
    int8_t* q8 = nullptr;      // [q_rows, q_heads*D]
    int8_t* k8 = nullptr;      // [kv_rows, kv_heads*D]
    void* vh = nullptr;        // fp16 [kv_rows, kv_heads*D]
    float* sq = nullptr;       // [q_rows/128 + 1, q_heads]
    float* sk = nullptr;       // [kv_rows/128 + 1, kv_heads]
    float* kmean = nullptr;    // partial key sums [kv_rows/128 + 1, kv_heads, D]
    int q_rows = 0, kv_rows = 0;
};

}  // namespace efm

namespace efm {
// One captured prefill pass: the launch sequence of a single chunk with every shape-dependent argument baked in.
// Valid for exactly the (slot, rows, cache offset, injected-embedding, sampling, attention-kind) combination it
// was captured with; the per-request inputs (ids, positions, embeddings, state) live in stable buffers that are
// refreshed by copies issued before the launch.
struct PrefillGraph {
    int slot = 0, rows = 0, kv_offset = 0, n_embeds = 0, embed_token_id = 0, sample = 0, attention_kind = 0;
    const void* embeds_buf = nullptr;
    cudaGraphExec_t exec = nullptr;
    int nodes = 0;
    uint64_t last_use = 0;
    bool same_key(const PrefillGraph& o) const {
        return slot == o.slot && rows == o.rows && kv_offset == o.kv_offset && n_embeds == o.n_embeds && embed_token_id == o.embed_token_id &&
               sample == o.sample && attention_kind == o.attention_kind && embeds_buf == o.embeds_buf;
    }
};
}  // namespace efm

struct efm_b200_ctx {
    efm_model_desc d{};                   // geometry as THIS RANK sees it (heads / MLP columns already sharded)
    efm_model_desc full{};                // geometry of the whole model (weight slicing)
    // tensor parallel layout: attention is sharded att_shards ways (each shard held by att_rep ranks,
    // which split the o_proj input columns between them); MLP columns and lm_head rows tp_size ways
    int att_shards = 1, att_rep = 1, att_shard = 0, att_rep_idx = 0;
    int o_k = 0;                          // o_proj input columns handled by this rank
    int vocab_l = 0, vocab_off = 0;       // lm_head rows of this rank
    void* nccl_comm = nullptr;
    // Peer exchange of the decode step (row-parallel GEMV fused with its all-reduce): one allocation per rank,
    // [exchange count at byte 64 | block ticket at 68 | receive buffer at 256: 2 x tp x H words {fp32, count}],
    // mapped into every other rank with CUDA IPC.  peer_base[r] is rank r's allocation as seen from here.
    char* tp_xchg = nullptr;
    // prefill exchange (reduce-scatter + all-gather over peer stores): exchange count at byte 96, ticket at 100,
    // scatter flags [2][8] at 128, gather flags [2][8] at 192; receive slots [2][tp][tp_slot_floats] fp32 at
    // tp_prefill_off (one slot = the rows one rank owns: ceil(max_s / tp) x H), gather buffers [2][max_s x H] at tp_gather_off
    // greedy sampling exchange: count at byte 104, receive words [2][tp] of {fp32 maximum, count << 18 | id} at tp_sample_off
    size_t tp_prefill_off = 0, tp_gather_off = 0, tp_slot_floats = 0, tp_sample_off = 0;
    double tp_timeout_s = 300.0;          // host-side limit of a synchronising call on a tensor-parallel context
    unsigned long long peer_wait_ns = 0;  // total wait budget of one kernel on its peers (0 = built-in default)
    int* error_host = nullptr;            // mapped host mirror of DecodeState.error, written by a kernel that gave up a
                                          // wait, polled by decode_steps between graph launches (same address on both sides)
    char* peer_base[8] = {};
    bool peers_ready = false;
    float* ybuf = nullptr;                // [max_s, H] fp32 partial outputs of row-parallel linears
    float* ysum = nullptr;                // [max_s, H] their sum over ranks
    float* logits_l = nullptr;            // [vocab_l]
    int device = 0, tp_rank = 0, tp_size = 1, num_sms = 148;
    cudaStream_t stream = nullptr;
    std::string error;
    bool finalized = false;
    bool pdl = true;

    // weights
    __nv_bfloat16* embed = nullptr;       // [V, H]
    __nv_bfloat16* lm_head = nullptr;     // [V, H] (aliases embed when tied)
    __nv_bfloat16* final_norm = nullptr;
    bool seen_embed = false, seen_lm_head = false, seen_final_norm = false;
    std::vector<efm::LayerWeights> layers;
    efm::W4Linear w4_lm_head;
    bool decode_w4 = false;               // every linear of the decode step has an INT4 copy
    float* inv_freq = nullptr;            // [D/2]

    // activations (prefill rows x width) and decode vectors
    int max_s = 0;
    int32_t* ids = nullptr;               // [max_s]
    int32_t* pos3 = nullptr;              // [3 * max_s]
    float* resid = nullptr;               // [max_s, H] residual stream, fp32
    __nv_bfloat16* norm = nullptr;        // [max_s, H]
    __nv_bfloat16* qkv = nullptr;         // [max_s, (q+2kv)*D]
    __nv_bfloat16* qbuf = nullptr;        // [max_s, q*D]
    __nv_bfloat16* attn = nullptr;        // [max_s, q*D]
    __nv_bfloat16* act = nullptr;         // [max_s, I]
    __nv_bfloat16* custom_embeds = nullptr;
    size_t custom_embeds_cap = 0;
    float* resid_d = nullptr;             // decode residual stream [H], fp32
    float* resid_d2 = nullptr;            // second copy (tensor parallel: the add-and-norm prologue ping-pongs)
    // decode activations stay fp32 from kernel to kernel: a decode step rounds only the K / V rows it appends
    float* q_d = nullptr;                 // [q*D] rotated q
    float* attn_d = nullptr;              // [q*D] attention output
    float* act_d = nullptr;               // [I] silu(gate) * up
    float* logits = nullptr;              // [V]
    float* part_val = nullptr;            // [max gemv grid]
    int* part_idx = nullptr;
    uint32_t* wbuf = nullptr;             // [V] sampler scratch
    float* attn_part_o = nullptr;         // decode attention scratch
    float* attn_part_ml = nullptr;
    unsigned int* attn_counters = nullptr;
    int prefill_attention_kind = 0;       // 0: bf16 flash attention, 1: INT8 Q.K^T / fp16 P.V
    efm::SageScratch sage;
    float* gemm_ws = nullptr;             // split-K workspace of the prefill / vision GEMMs (fp32 partial tiles)
    size_t gemm_ws_floats = 0;
    efm::DecodeState* state = nullptr;
    int32_t* tokens_out = nullptr;        // [max_response_tokens]

    efm_sampling sampling{0.f, 1.f, 1, 0, 0};
    std::map<int, efm::KvSlot> slots;
    int bound_slot = -1;
    // prefill CUDA graphs (short prompts are launch-bound): a shape is launched kernel by kernel the first time it is
    // seen, captured the second time, replayed afterwards; at most kMaxPrefillGraphs shapes are kept (least recently used out)
    bool prefill_graphs = false;
    std::vector<efm::PrefillGraph> prefill_cache;     // exec == nullptr: seen once, not captured yet
    uint64_t prefill_clock = 0;
    int64_t prefill_graph_replays = 0;
    int64_t launches = 0;
    cudaEvent_t events[16] = {};
    std::vector<void*> allocations;
};
