// Launch sequences of the Qwen2.5 / Qwen2.5-VL text tower: one decode step and one prefill
// chunk.  Layer order and residual dataflow follow the reference's forward
// (src/models/qwen2_5/qwen2_5.cpp:534-930); what the reference runs as 9-10 kernels per layer
// at decode is five launches here:
//   [embed +] RMSNorm + QKV GEMV + bias + RoPE + KV append | attention | o_proj + residual |
//   RMSNorm + gate/up GEMV + SiLU*mul | down_proj + residual
// and norm + lm_head + block argmax | sampler + state advance at the end of the step.
#include "qwen_text.h"

#include "../operators/attention_mma.cuh"
#include "../operators/attention_tc.cuh"
#include "../operators/sage_attention.cuh"
#include "../operators/gemm_tc.cuh"
#include "../operators/prefill.cuh"
#include "../operators/sample.cuh"
#include "../backends/b200/nccl_glue.h"
#include "launch.cuh"

namespace efm {

static GemvParams base_gemv(const __nv_bfloat16* W, int N, int K) {
    GemvParams p{};
    p.W = W;
    p.N = N;
    p.K = K;
    p.n_items = N / 2;
    p.prologue = kProPlain;
    return p;
}

// One decode GEMV: the INT4 copy of the linear when the context decodes from INT4 weights, else bf16.
template <Epi EPI>
static void launch_decode_gemv(efm_b200_ctx& c, Launcher& L, const GemvParams& p, const W4Linear* w4, int swiglu_half = 0) {
    if (c.decode_w4 && w4 != nullptr && w4->ready) {
        GemvW4Params q{};
        q.g = p;
        q.g.W = nullptr;
        q.Wq = w4->q;
        q.scales = static_cast<const __half2*>(w4->s);
        q.swiglu_half = swiglu_half;
        launch_gemv_w4<EPI>(L, q, c.num_sms);
        return;
    }
    launch_gemv<EPI>(L, p, c.num_sms);
}

static void tp_all_reduce(efm_b200_ctx& c, Launcher& L, const float* send, float* recv, size_t count);
static void tp_all_gather(efm_b200_ctx& c, Launcher& L, const float* send, float* recv, size_t count);
static void launch_sample_only(efm_b200_ctx& c, Launcher& L, int n_part, int advance);
bool tp_greedy_exchange(const efm_b200_ctx& c);

// Widest cluster the sampler can run with on this device: 16, 8, ... or 1 (single block; also with
// EFM_B200_SAMPLER_CLUSTER=1).  Found once, outside any stream capture.
static int g_sampler_cluster = -1;

cudaError_t configure_sampler() {
    if (g_sampler_cluster >= 0) return cudaSuccess;
    int best = 1;
    const bool wide = cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess;
    for (int cs = wide ? 16 : 8; cs >= 2; cs >>= 1) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(cs, 1, 1);
        cfg.blockDim = dim3(1024);
        cudaLaunchAttribute at;
        at.id = cudaLaunchAttributeClusterDimension;
        at.val.clusterDim.x = (unsigned)cs;
        at.val.clusterDim.y = at.val.clusterDim.z = 1;
        cfg.attrs = &at;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, sample_kernel, &cfg) == cudaSuccess && n >= 1) { best = cs; break; }
    }
    (void)cudaGetLastError();
    if (const char* env = std::getenv("EFM_B200_SAMPLER_CLUSTER")) {
        const int v = std::atoi(env);
        if (v >= 1) { int cs = 1; while (cs * 2 <= v && cs * 2 <= best) cs *= 2; best = cs; }
    }
    g_sampler_cluster = best;
    return cudaSuccess;
}

// Greedy decoding needs one block (the arg-max of the logits pass's partial maxima); top-p sampling
// spreads its passes over the vocabulary across one cluster.
void launch_sample(Launcher& L, const SampleParams& p) {
    if (g_sampler_cluster < 0) (void)configure_sampler();
    const int cs = (p.temperature >= 1e-6f && p.xchg != nullptr) ? g_sampler_cluster : 1;
    L.cluster_x = cs;
    L.launch(sample_kernel, dim3(cs), dim3(1024), 0, p);
}

void launch_lm_head_and_sample(efm_b200_ctx& c, Launcher& L, const float* resid_row, int advance, bool decode_pass) {
    const efm_model_desc& d = c.d;
    GemvParams p = base_gemv(c.lm_head, c.vocab_l, d.hidden);      // this rank's rows (all of them without TP)
    p.prologue = kProRmsNorm;
    p.xr = resid_row;
    p.norm_w = c.final_norm;
    p.eps = d.rms_eps;
    p.logits = c.tp_size > 1 ? c.logits_l : c.logits;
    p.part_val = c.part_val;
    p.part_idx = c.part_idx;
    if (decode_pass) launch_decode_gemv<Epi::Logits>(c, L, p, &c.w4_lm_head);
    else launch_gemv<Epi::Logits>(L, p, c.num_sms);
    if (c.tp_size > 1) {
        const bool pdl = L.pdl;
        if (tp_greedy_exchange(c)) {
            // greedy: the ranks exchange their (maximum, id) as one word each inside the sampler; no collective, no
            // gathered logits (efm_b200_read_logits gathers on demand)
            launch_sample_only(c, L, /*n_part=*/c.num_sms, advance);
        } else {
            tp_all_gather(c, L, c.logits_l, c.logits, (size_t)c.vocab_l);
            launch_sample_only(c, L, /*n_part=*/0, advance);
        }
        L.pdl = pdl;
        return;
    }

    SampleParams s{};
    s.logits = c.logits;
    s.vocab = d.vocab;
    s.part_val = c.part_val;
    s.part_idx = c.part_idx;
    s.n_part = c.num_sms;
    s.temperature = c.sampling.temperature;
    s.top_p = c.sampling.top_p;
    s.seed = c.sampling.seed;
    s.state = c.state;
    s.tokens_out = c.tokens_out;
    s.max_response = d.max_response_tokens;
    s.advance = advance;
    s.wbuf = c.wbuf;
    s.xchg = sample_xchg(c.wbuf, d.vocab);
    launch_sample(L, s);
}

// Tensor parallel with imported peer buffers and greedy sampling: the sampler exchanges the ranks' maxima itself.
bool tp_greedy_exchange(const efm_b200_ctx& c) {
    return c.tp_size > 1 && c.peers_ready && c.sampling.temperature < 1e-6f;
}

static void launch_sample_only(efm_b200_ctx& c, Launcher& L, int n_part, int advance) {
    const efm_model_desc& d = c.d;
    SampleParams s{};
    s.logits = c.logits;
    s.vocab = d.vocab;
    s.part_val = c.part_val;
    s.part_idx = c.part_idx;
    s.n_part = n_part;
    if (n_part > 0 && tp_greedy_exchange(c)) {
        s.tp_n = c.tp_size;
        s.tp_rank = c.tp_rank;
        s.tp_vocab_offset = c.vocab_off;
        s.tp_count = reinterpret_cast<unsigned int*>(c.tp_xchg + 104);
        for (int r = 0; r < c.tp_size; ++r) s.tp_peer_slot[r] = reinterpret_cast<unsigned long long*>(c.peer_base[r] + c.tp_sample_off);
        s.tp_error = &c.state->error;
        s.tp_error_host = c.error_host;
        s.tp_wait_ns = c.peer_wait_ns;
    }
    s.temperature = c.sampling.temperature;
    s.top_p = c.sampling.top_p;
    s.seed = c.sampling.seed;
    s.state = c.state;
    s.tokens_out = c.tokens_out;
    s.max_response = d.max_response_tokens;
    s.advance = advance;
    s.wbuf = c.wbuf;
    s.xchg = sample_xchg(c.wbuf, d.vocab);
    launch_sample(L, s);
}

// Collectives on the context stream (graph-capturable).  A failure is recorded like a launch failure.
static void tp_all_reduce(efm_b200_ctx& c, Launcher& L, const float* send, float* recv, size_t count) {
    if (L.err != cudaSuccess) return;
    const NcclApi& api = nccl_api();
    if (!api.ok || c.nccl_comm == nullptr || api.all_reduce_f32_sum(send, recv, count, c.nccl_comm, L.stream) != 0)
        L.err = cudaErrorUnknown;
    else if (L.counter != nullptr) ++*L.counter;
}
static void tp_all_gather(efm_b200_ctx& c, Launcher& L, const float* send, float* recv, size_t count) {
    if (L.err != cudaSuccess) return;
    const NcclApi& api = nccl_api();
    if (!api.ok || c.nccl_comm == nullptr || api.all_gather_f32(send, recv, count, c.nccl_comm, L.stream) != 0)
        L.err = cudaErrorUnknown;
    else if (L.counter != nullptr) ++*L.counter;
}

void tp_gather_logits(efm_b200_ctx& c, Launcher& L) { tp_all_gather(c, L, c.logits_l, c.logits, (size_t)c.vocab_l); }

// Exchange buffer layout (ctx.h): count at byte 64, ticket at 68, receive buffer [2][tp][H] of {fp32, count} at 256.
static void peers_producer(const efm_b200_ctx& c, GemvParams& p, int parity) {
    const size_t H = (size_t)c.d.hidden;
    p.n_peers = c.tp_size;
    for (int r = 0; r < c.tp_size; ++r)
        p.peer_out[r] = reinterpret_cast<uint2*>(c.peer_base[r] + 256) + ((size_t)parity * c.tp_size + c.tp_rank) * H;
    p.epoch = reinterpret_cast<unsigned int*>(c.tp_xchg + 64);
    p.ticket = reinterpret_cast<unsigned int*>(c.tp_xchg + 68);
}
static void peers_consumer(const efm_b200_ctx& c, GemvParams& p, int parity) {
    p.addend_parts = reinterpret_cast<const uint2*>(c.tp_xchg + 256) + (size_t)parity * c.tp_size * c.d.hidden;
    p.n_parts = c.tp_size;
    p.epoch = reinterpret_cast<unsigned int*>(c.tp_xchg + 64);
    p.error = &c.state->error;
    p.error_host = c.error_host;
    p.wait_ns = c.peer_wait_ns;
}

// Tensor-parallel prefill: sum of the row-parallel partial c.ybuf [S, H] over the ranks, added to the residual.
// With imported peer buffers: reduce-scatter + all-gather over peer stores (operators/prefill.cuh); otherwise
// ncclAllReduce + add.  Header words of the exchange allocation (ctx.h): prefill exchange count at byte 96, ticket at
// 100, scatter flags [2][8] at 128, gather flags [2][8] at 192.
static void tp_prefill_sum(efm_b200_ctx& c, Launcher& L, int S, int parity) {
    const size_t H = (size_t)c.d.hidden, n = (size_t)S * H;
    if (!c.peers_ready) {
        tp_all_reduce(c, L, c.ybuf, c.ysum, n);
        L.launch(add_rows_kernel, dim3(std::min<size_t>((n / 2 + 255) / 256, (size_t)c.num_sms * 8)), dim3(256), 0, c.resid,
                 (const float*)c.ysum, n / 2);
        return;
    }
    const int tp = c.tp_size;
    const size_t slot = c.tp_slot_floats;                                    // floats per (parity, rank) receive slot
    PeerXchgParams pp{};
    pp.src = c.ybuf;
    pp.n_peers = tp;
    pp.rank = c.tp_rank;
    pp.S = S;
    pp.H = (int)H;
    pp.rows_per = (S + tp - 1) / tp;
    pp.slot_floats = slot;
    pp.epoch = reinterpret_cast<unsigned int*>(c.tp_xchg + 96);
    pp.ticket = reinterpret_cast<unsigned int*>(c.tp_xchg + 100);
    pp.error = &c.state->error;
    pp.error_host = c.error_host;
    pp.wait_ns = c.peer_wait_ns;
    pp.recv_local = reinterpret_cast<const float*>(c.tp_xchg + c.tp_prefill_off) + (size_t)parity * tp * slot;
    pp.gather_local = reinterpret_cast<const float*>(c.tp_xchg + c.tp_gather_off) + (size_t)parity * c.max_s * H;
    pp.resid = c.resid;
    for (int r = 0; r < tp; ++r) {
        pp.recv[r] = reinterpret_cast<float*>(c.peer_base[r] + c.tp_prefill_off) + ((size_t)parity * tp + c.tp_rank) * slot;
        pp.gather[r] = reinterpret_cast<float*>(c.peer_base[r] + c.tp_gather_off) + (size_t)parity * c.max_s * H;
    }
    const int grid_all = (int)std::min<size_t>((n / 4 + 255) / 256, (size_t)c.num_sms * 8);
    const int grid_own = (int)std::min<size_t>(((size_t)pp.rows_per * H / 4 + 255) / 256, (size_t)c.num_sms * 8);
    // 1. scatter (publishes this rank's scatter flag on every rank)
    for (int r = 0; r < tp; ++r) pp.flag[r] = reinterpret_cast<unsigned int*>(c.peer_base[r] + 128) + parity * 8 + c.tp_rank;
    L.launch(peer_scatter_rows_kernel, dim3(grid_all), dim3(256), 0, pp);
    // 2. reduce own rows, store them into every rank's gather buffer (waits for the scatter flags, publishes gather flags)
    pp.flags_local = reinterpret_cast<const unsigned int*>(c.tp_xchg + 128) + parity * 8;
    for (int r = 0; r < tp; ++r) pp.flag[r] = reinterpret_cast<unsigned int*>(c.peer_base[r] + 192) + parity * 8 + c.tp_rank;
    L.launch(peer_reduce_gather_kernel, dim3(std::max(1, grid_own)), dim3(256), 0, pp);
    // 3. resid += gathered sum (waits for the gather flags)
    pp.flags_local = reinterpret_cast<const unsigned int*>(c.tp_xchg + 192) + parity * 8;
    L.launch(peer_add_gathered_kernel, dim3(grid_all), dim3(256), 0, pp);
}

// Tensor-parallel decode step: column-parallel QKV / gate-up, row-parallel o_proj / down with an
// all-reduce of the fp32 partial [H]; the residual add moves into the next kernel's norm prologue
// (x = bf16(x + bf16(sum)), ping-ponging between two residual buffers so no block re-reads a row that
// block 0 already updated); lm_head rows are split and the logits all-gathered before sampling.
static void qwen_decode_step_tp(efm_b200_ctx& c, KvSlot& slot, Launcher& L) {
    const efm_model_desc& d = c.d;
    const int H = d.hidden, D = d.head_dim, QD = d.q_heads * D, KVD = d.kv_heads * D, I = d.intermediate;
    float* RA = c.resid_d;
    float* RB = c.resid_d2;
    const bool fused = c.peers_ready;        // exchange inside the GEMVs over peer memory instead of ncclAllReduce
    for (int l = 0; l < d.num_layers; ++l) {
        const LayerWeights& w = c.layers[l];
        {
            GemvParams p = base_gemv(w.qkv, QD + 2 * KVD, H);
            p.prologue = l == 0 ? kProEmbedRmsNorm : kProRmsNorm;
            p.xr = RB;                       // l > 0: residual after the previous layer's attention add
            if (l > 0) { if (fused) peers_consumer(c, p, 1); else p.addend = c.ysum; }
            p.resid_out = RA;
            p.norm_w = w.in_norm; p.eps = d.rms_eps; p.embed_table = c.embed; p.vocab = d.vocab; p.state = c.state;
            p.bias = w.qkv_bias; p.q_out_f = c.q_d; p.k_cache = slot.k[l]; p.v_cache = slot.v[l]; p.inv_freq = c.inv_freq;
            p.q_heads = d.q_heads; p.kv_heads = d.kv_heads; p.head_dim = D; p.use_mrope = d.use_mrope;
            p.sec0 = d.mrope_section[0]; p.sec1 = d.mrope_section[0] + d.mrope_section[1]; p.max_tokens = slot.max_tokens;
            launch_gemv<Epi::QkvRope>(L, p, c.num_sms);
        }
        {
            DecodeAttnParams a{};
            a.qf = c.q_d; a.k_cache = slot.k[l]; a.v_cache = slot.v[l]; a.outf = c.attn_d; a.state = c.state;
            a.q_heads = d.q_heads; a.kv_heads = d.kv_heads; a.group = d.q_heads / d.kv_heads;
            a.n_splits = slot.n_splits; a.chunk_cap = slot.chunk_cap; a.max_tokens = slot.max_tokens; a.cluster = slot.attn_cluster; a.early = l > 0 ? 1 : 0;
            a.scale = 1.0f / sqrtf((float)D);
            a.part_o = c.attn_part_o; a.part_ml = c.attn_part_ml; a.counters = c.attn_counters;
            launch_decode_attention(L, a, D);
        }
        {
            GemvParams p = base_gemv(w.o, H, c.o_k);
            p.xf = c.attn_d + (size_t)c.att_rep_idx * c.o_k;
            if (fused) {
                peers_producer(c, p, 0);
                launch_gemv<Epi::Peers>(L, p, c.num_sms);              // fp32 partial straight into every rank's buffer
            } else {
                p.logits = c.ybuf; p.part_val = c.part_val; p.part_idx = c.part_idx;
                launch_gemv<Epi::Logits>(L, p, c.num_sms);             // fp32 partial output
            }
        }
        if (!fused) tp_all_reduce(c, L, c.ybuf, c.ysum, (size_t)H);
        {
            GemvParams p = base_gemv(w.gate_up, 2 * I, H);
            p.prologue = kProRmsNorm;
            p.xr = RA; p.resid_out = RB;
            if (fused) peers_consumer(c, p, 0); else p.addend = c.ysum;
            p.norm_w = w.post_norm; p.eps = d.rms_eps; p.yf = c.act_d;
            launch_gemv<Epi::SwiGlu>(L, p, c.num_sms);
        }
        {
            GemvParams p = base_gemv(w.down, H, I);
            p.xf = c.act_d;
            if (fused) {
                peers_producer(c, p, 1);
                launch_gemv<Epi::Peers>(L, p, c.num_sms);
            } else {
                p.logits = c.ybuf; p.part_val = c.part_val; p.part_idx = c.part_idx;
                launch_gemv<Epi::Logits>(L, p, c.num_sms);
            }
        }
        if (!fused) tp_all_reduce(c, L, c.ybuf, c.ysum, (size_t)H);
    }
    {
        GemvParams p = base_gemv(c.lm_head, c.vocab_l, H);
        p.prologue = kProRmsNorm;
        p.xr = RB; p.resid_out = RA;
        if (fused) peers_consumer(c, p, 1); else p.addend = c.ysum;
        p.norm_w = c.final_norm; p.eps = d.rms_eps;
        p.logits = c.logits_l; p.part_val = c.part_val; p.part_idx = c.part_idx;
        launch_gemv<Epi::Logits>(L, p, c.num_sms);
    }
    tp_all_gather(c, L, c.logits_l, c.logits, (size_t)c.vocab_l);
    launch_sample_only(c, L, /*n_part=*/0, /*advance=*/1);
}

void launch_w4_repack(Launcher& L, const W4RepackParams& p) {
    const bool pdl = L.pdl;
    L.pdl = false;
    L.launch(w4_repack_kernel<0>, dim3(((p.n_items + 7) / 8) * 8), dim3(256), 0, p);
    L.pdl = pdl;
}

void qwen_decode_step(efm_b200_ctx& c, KvSlot& slot, Launcher& L) {
    if (c.tp_size > 1) {
        qwen_decode_step_tp(c, slot, L);
        return;
    }
    const efm_model_desc& d = c.d;
    const int H = d.hidden, D = d.head_dim, QD = d.q_heads * D, KVD = d.kv_heads * D, I = d.intermediate;
    for (int l = 0; l < d.num_layers; ++l) {
        const LayerWeights& w = c.layers[l];
        {
            GemvParams p = base_gemv(w.qkv, QD + 2 * KVD, H);
            p.prologue = l == 0 ? kProEmbedRmsNorm : kProRmsNorm;
            p.xr = c.resid_d;
            p.norm_w = w.in_norm;
            p.eps = d.rms_eps;
            p.embed_table = c.embed;
            p.vocab = d.vocab;
            p.resid_out = c.resid_d;
            p.state = c.state;
            p.bias = w.qkv_bias;
            p.q_out_f = c.q_d;
            p.k_cache = slot.k[l];
            p.v_cache = slot.v[l];
            p.inv_freq = c.inv_freq;
            p.q_heads = d.q_heads;
            p.kv_heads = d.kv_heads;
            p.head_dim = D;
            p.use_mrope = d.use_mrope;
            p.sec0 = d.mrope_section[0];
            p.sec1 = d.mrope_section[0] + d.mrope_section[1];
            p.max_tokens = slot.max_tokens;
            launch_decode_gemv<Epi::QkvRope>(c, L, p, &w.w4_qkv);
        }
        {
            DecodeAttnParams a{};
            a.qf = c.q_d;
            a.k_cache = slot.k[l];
            a.v_cache = slot.v[l];
            a.outf = c.attn_d;
            a.state = c.state;
            a.q_heads = d.q_heads;
            a.kv_heads = d.kv_heads;
            a.group = d.q_heads / d.kv_heads;
            a.n_splits = slot.n_splits;
            a.chunk_cap = slot.chunk_cap;
            a.cluster = slot.attn_cluster;
            a.early = l > 0 ? 1 : 0;       // layer 0 follows the sampler's state update: wait first
            a.max_tokens = slot.max_tokens;
            a.scale = 1.0f / sqrtf((float)D);
            a.part_o = c.attn_part_o;
            a.part_ml = c.attn_part_ml;
            a.counters = c.attn_counters;
            launch_decode_attention(L, a, D);
        }
        {
            GemvParams p = base_gemv(w.o, H, c.o_k);
            p.xf = c.attn_d;
            p.residual = c.resid_d;
            launch_decode_gemv<Epi::Residual>(c, L, p, &w.w4_o);
        }
        {
            GemvParams p = base_gemv(w.gate_up, 2 * I, H);
            p.prologue = kProRmsNorm;
            p.xr = c.resid_d;
            p.norm_w = w.post_norm;
            p.eps = d.rms_eps;
            p.yf = c.act_d;
            launch_decode_gemv<Epi::SwiGlu>(c, L, p, &w.w4_gate_up, I);
        }
        {
            GemvParams p = base_gemv(w.down, H, I);
            p.xf = c.act_d;
            p.residual = c.resid_d;
            launch_decode_gemv<Epi::Residual>(c, L, p, &w.w4_down);
        }
    }
    launch_lm_head_and_sample(c, L, c.resid_d, /*advance=*/1, /*decode_pass=*/true);
}

// ---- tensor maps for the TMA-fed GEMM --------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult st;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &st) != cudaSuccess ||
            st != cudaDriverEntryPointSuccess)
            f = nullptr;
        return reinterpret_cast<EncodeTiledFn>(f);
    }();
    return fn;
}

// bf16 row-major [rows, cols] tensor, box = 64 columns x box_rows rows, 128-byte swizzle, zero fill
// outside the tensor.
static bool make_tile_map(CUtensorMap* map, const void* ptr, int rows, int cols, int row_stride, int box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return false;
    const cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t gstride[1] = {(cuuint64_t)row_stride * 2};
    const cuuint32_t box[2] = {(cuuint32_t)tc::BK, (cuuint32_t)box_rows};
    const cuuint32_t estride[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), gdim, gstride, box, estride,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// fewest 64-wide k-blocks a split may get (EFM_B200_GEMM_MIN_KB overrides, for measurements)
static int min_kb_per_split() {
    static int v = [] { const char* e = std::getenv("EFM_B200_GEMM_MIN_KB"); const int x = e != nullptr ? std::atoi(e) : 0; return x >= 1 ? x : 4; }();
    return v;
}

// EFM_B200_GEMM_TAIL=0 switches the tail split off (for A/B timing)
static bool tail_split_enabled() {
    static const bool on = [] { const char* e = std::getenv("EFM_B200_GEMM_TAIL"); return e == nullptr || e[0] != '0'; }();
    return on;
}

template <GemmEpi EPI>
static void launch_gemm(Launcher& L, const GemmParams& p, int* error_word = nullptr) {
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(gemm_tc_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tc::SMEM_BYTES);
        attr_set = true;
    }
    CUtensorMap ma, mb;
    if (!make_tile_map(&ma, p.A, p.M, p.K, p.lda > 0 ? p.lda : p.K, tc::BM) || !make_tile_map(&mb, p.B, p.N, p.K, p.K, tc::BN)) {
        if (L.err == cudaSuccess) L.err = cudaErrorInvalidValue;
        return;
    }
    const int tiles = ((p.N + tc::BN - 1) / tc::BN) * ((p.M + tc::BM - 1) / tc::BM);
    const dim3 block(tc::kThreads);
    const bool pdl = L.pdl;
    L.pdl = false;     // prefill kernels do not use the dependent-launch protocol
    // Few output tiles and a long K: split K so that the whole GPU works, fp32 partials to the workspace, then
    // a fixed-order sum with the epilogue.
    if constexpr (EPI == GemmEpi::Bf16Bias || EPI == GemmEpi::Residual || EPI == GemmEpi::F32 || EPI == GemmEpi::SwiGlu) {
        const int KB = (p.K + tc::BK - 1) / tc::BK;
        int splits = std::min(L.num_sms / std::max(1, tiles), KB / min_kb_per_split());
        if (L.gemm_ws != nullptr && splits >= 2 && (p.N & 3) == 0 && (EPI != GemmEpi::SwiGlu || (p.N & 127) == 0) &&
            (size_t)splits * p.M * p.N <= L.gemm_ws_floats) {
            const int per = (KB + splits - 1) / splits;
            splits = (KB + per - 1) / per;                 // no empty split
            GemmParams q = p;
            q.kb_per_split = per;
            q.Cf = L.gemm_ws;
            q.bias = nullptr;
            static bool attr_f32 = false;
            if (!attr_f32) {
                cudaFuncSetAttribute(gemm_tc_kernel<GemmEpi::F32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tc::SMEM_BYTES);
                attr_f32 = true;
            }
            L.launch(gemm_tc_kernel<GemmEpi::F32>, dim3(std::min(L.num_sms, tiles * splits)), block, tc::SMEM_BYTES, ma, mb, q, error_word);
            const size_t total4 = (size_t)p.M * p.N / (EPI == GemmEpi::SwiGlu ? 8 : 4);
            const int fin = (int)std::min<size_t>((total4 + 255) / 256, (size_t)L.num_sms * 4);
            L.launch(gemm_splitk_finish_kernel<EPI>, dim3(fin), dim3(256), 0, (const float*)L.gemm_ws, splits, p);
            L.pdl = pdl;
            return;
        }
    }
    // Tail split: a few tiles more than a multiple of the SM count would cost a whole extra round in which most SMs
    // idle (1324 x 3584 outputs = 154 tiles on 148 SMs: two rounds for 1.04 rounds of work).  The full rounds run as
    // they are; the remaining tiles are cut along K into as many slices as fill the GPU once (compact fp32 slots in
    // the workspace) and a small kernel sums the slices in order with the epilogue.  Worth it only when a tile's K
    // loop is long against the two extra launches (about 12 us).
    if constexpr (EPI == GemmEpi::Bf16Bias || EPI == GemmEpi::Residual || EPI == GemmEpi::F32) {
        const int P = L.num_sms, rounds = tiles / P, rem = tiles % P;
        const int KB = (p.K + tc::BK - 1) / tc::BK;
        if (tail_split_enabled() && L.gemm_ws != nullptr && rounds >= 1 && rem > 0 && rem * 2 <= P && (p.N & 3) == 0 && p.kb_per_split == 0 &&
            p.tile_count == 0) {
            int splits = std::min(P / rem, KB / min_kb_per_split());
            const int per = splits >= 2 ? (KB + splits - 1) / splits : KB;
            splits = (KB + per - 1) / per;
            const double tile_us = KB * 0.45, gain_us = tile_us * (1.0 - 1.0 / std::max(1, splits)) - 12.0;
            if (splits >= 2 && gain_us > 5.0 && (size_t)splits * rem * tc::BM * tc::BN <= L.gemm_ws_floats) {
                GemmParams full = p;
                full.tile_begin = 0;
                full.tile_count = rounds * P;
                L.launch(gemm_tc_kernel<EPI>, dim3(P), block, tc::SMEM_BYTES, ma, mb, full, error_word);
                GemmParams q = p;
                q.tile_begin = rounds * P;
                q.tile_count = rem;
                q.kb_per_split = per;
                q.Cf = L.gemm_ws;
                q.bias = nullptr;
                static bool attr_f32 = false;
                if (!attr_f32) {
                    cudaFuncSetAttribute(gemm_tc_kernel<GemmEpi::F32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tc::SMEM_BYTES);
                    attr_f32 = true;
                }
                L.launch(gemm_tc_kernel<GemmEpi::F32>, dim3(std::min(P, rem * splits)), block, tc::SMEM_BYTES, ma, mb, q, error_word);
                const int per_tile = std::max(1, std::min(32, (P * 4) / rem));
                L.launch(gemm_tail_finish_kernel<EPI>, dim3(per_tile, rem), dim3(256), 0, (const float*)L.gemm_ws, splits, rounds * P, rem, p);
                L.pdl = pdl;
                return;
            }
        }
    }
    L.launch(gemm_tc_kernel<EPI>, dim3(std::min(L.num_sms, tiles)), block, tc::SMEM_BYTES, ma, mb, p, error_word);
    L.pdl = pdl;
}

void launch_gemm_bf16(Launcher& L, const GemmParams& p) { launch_gemm<GemmEpi::Bf16Bias>(L, p); }

void launch_rmsnorm_rows(Launcher& L, const float* x, const __nv_bfloat16* w, __nv_bfloat16* y, int rows, int hidden, float eps) {
    const bool pdl = L.pdl;
    L.pdl = pdl && L.pdl_rows;
    // many short rows (vision tower, action model): one warp per row; otherwise one block per row
    if (hidden <= 2048 && (hidden & 3) == 0 && rows >= 256)
        L.launch(rmsnorm_rows_warp_kernel, dim3((rows + 7) / 8), dim3(256), 0, x, w, y, rows, hidden, eps);
    else
        L.launch(rmsnorm_rows_kernel, dim3(rows), dim3(256), 0, x, w, y, hidden, eps);
    L.pdl = pdl;
}

void launch_gemm_epi(Launcher& L, GemmEpi epi, const GemmParams& p, int* error_word) {
    switch (epi) {
        case GemmEpi::Bf16Bias: launch_gemm<GemmEpi::Bf16Bias>(L, p, error_word); break;
        case GemmEpi::Residual: launch_gemm<GemmEpi::Residual>(L, p, error_word); break;
        case GemmEpi::F32: launch_gemm<GemmEpi::F32>(L, p, error_word); break;
        case GemmEpi::Bf16Gelu: launch_gemm<GemmEpi::Bf16Gelu>(L, p, error_word); break;
        case GemmEpi::Bf16GeluTanh: launch_gemm<GemmEpi::Bf16GeluTanh>(L, p, error_word); break;
        case GemmEpi::SwiGlu: launch_gemm<GemmEpi::SwiGlu>(L, p, error_word); break;
    }
}

template <int D, int NW>
static void launch_seg_attention_dn(Launcher& L, const SegAttnParams& p) {
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(seg_attention_kernel<D, NW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sa::smem_bytes<D, NW>());
        attr_set = true;
    }
    const dim3 grid((p.S + 16 * NW - 1) / (16 * NW), p.q_heads), block(32 * NW);
    const bool pdl = L.pdl;
    L.pdl = pdl && L.pdl_rows;
    L.launch(seg_attention_kernel<D, NW>, grid, block, sa::smem_bytes<D, NW>(), p);
    L.pdl = pdl;
}

template <int D>
static void launch_seg_attention_d(Launcher& L, const SegAttnParams& p) {
    // 64-query blocks: 128-query blocks (NW 8) measured 1-2 % slower on B200 at 1324 and 4784 rows (register-bound
    // occupancy does not improve with them)
    launch_seg_attention_dn<D, 4>(L, p);
}

void launch_seg_attention(Launcher& L, const SegAttnParams& p, int D);
// Head dim 64, at most 64 queries and at most 320 keys per block (the action expert's attention): every key of the
// block is requested at once.  Anything else goes to the streaming kernel.
void launch_seg_attention_short(Launcher& L, const SegAttnParams& p, int D, int max_keys) {
    constexpr int PRE = 5;
    if (D != 64 || p.S <= 0 || p.S > 64 || max_keys > PRE * sa::BKV) { launch_seg_attention(L, p, D); return; }
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(seg_attention_kernel<64, 4, PRE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sa::smem_bytes<64, 4, PRE>());
        attr_set = true;
    }
    const bool pdl = L.pdl;
    L.pdl = pdl && L.pdl_rows;
    L.launch(seg_attention_kernel<64, 4, PRE>, dim3(1, p.q_heads), dim3(128), sa::smem_bytes<64, 4, PRE>(), p);
    L.pdl = pdl;
}

// bf16 tensor of up to three dimensions for TMA: dims / box innermost first, byte strides of dimensions 1 and 2.
static bool make_map_nd(CUtensorMap* map, const void* ptr, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                        const uint32_t* box, CUtensorMapDataType dtype = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return false;
    cuuint64_t gdim[3], gstride[2];
    cuuint32_t bx[3], estride[3] = {1, 1, 1};
    for (int i = 0; i < rank; ++i) { gdim[i] = dims[i]; bx[i] = box[i]; }
    for (int i = 0; i + 1 < rank; ++i) gstride[i] = strides_bytes[i];
    return fn(map, dtype, (cuuint32_t)rank, const_cast<void*>(ptr), gdim, gstride, bx, estride,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static bool attention_tc_enabled() {
    static const bool on = [] { const char* e = std::getenv("EFM_B200_ATTN_TC"); return e == nullptr || e[0] != '0'; }();
    return on;
}

// tcgen05 / TMEM form (attention_tc.cuh).
template <int D>
static bool launch_seg_attention_tc_d(Launcher& L, const SegAttnParams& p0) {
    using C = at::Cfg<D>;
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(seg_attention_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM);
        attr_set = true;
    }
    const SegAttnParams& p = p0;
    CUtensorMap mq, mk, mv;
    const uint64_t qd[3] = {(uint64_t)D, (uint64_t)p.q_heads, (uint64_t)p.S}, qs[2] = {(uint64_t)D * 2, (uint64_t)p.q_stride * 2};
    const uint64_t kd[3] = {(uint64_t)D, (uint64_t)p.kv_heads, (uint64_t)p.kv_rows}, ks[2] = {(uint64_t)D * 2, (uint64_t)p.kv_stride * 2};
    const uint32_t qb[3] = {64, 1, (uint32_t)at::BM}, kb[3] = {64, 1, (uint32_t)at::BN};
    if (!make_map_nd(&mq, p.q, 3, qd, qs, qb) || !make_map_nd(&mk, p.k, 3, kd, ks, kb) || !make_map_nd(&mv, p.v, 3, kd, ks, kb)) return false;
    const bool pdl = L.pdl;
    L.pdl = false;
    L.launch(seg_attention_tc_kernel<D>, dim3((p.S + at::BM - 1) / at::BM, p.q_heads), dim3(at::kThreads), C::SMEM, mq, mk, mv, p, p.error);
    L.pdl = pdl;
    return true;
}

static bool launch_seg_attention_tc(Launcher& L, const SegAttnParams& p, int D) {
    // TMA needs 16-byte aligned bases and strides; anything else stays on the mma.sync kernel
    if (p.kv_rows <= 0 || (p.q_stride & 7) || (p.kv_stride & 7) || (reinterpret_cast<uintptr_t>(p.q) & 15) ||
        (reinterpret_cast<uintptr_t>(p.k) & 15) || (reinterpret_cast<uintptr_t>(p.v) & 15) || (p.out_stride & 7) ||
        (reinterpret_cast<uintptr_t>(p.out) & 15) || !attention_tc_enabled())
        return false;
    if (D == 128) return launch_seg_attention_tc_d<128>(L, p);
    if (D == 80) return launch_seg_attention_tc_d<80>(L, p);
    if (D == 64) return launch_seg_attention_tc_d<64>(L, p);
    return false;
}

void launch_seg_attention(Launcher& L, const SegAttnParams& p, int D) {
    if (p.S <= 0) return;
    if (launch_seg_attention_tc(L, p, D)) return;
    if (D == 128) launch_seg_attention_d<128>(L, p);
    else if (D == 80) launch_seg_attention_d<80>(L, p);
    else if (D == 64) launch_seg_attention_d<64>(L, p);
    else if (L.err == cudaSuccess) L.err = cudaErrorInvalidValue;
}

// Causal GQA attention of a prefill chunk: queries at cache rows [kv_offset, kv_offset + S).
void launch_prefill_attention(Launcher& L, const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* v,
                              __nv_bfloat16* out, int S, int kv_offset, int q_heads, int kv_heads, int D, int* error) {
    SegAttnParams p{};
    p.q = q; p.k = k; p.v = v; p.out = out;
    p.q_stride = q_heads * D; p.kv_stride = kv_heads * D; p.out_stride = q_heads * D;
    p.S = S; p.kv_offset = kv_offset; p.q_heads = q_heads; p.kv_heads = kv_heads;
    p.scale = 1.0f / sqrtf((float)D);
    p.kv_rows = kv_offset + S;
    p.error = error;
    launch_seg_attention(L, p, D);
}

template <int D>
static void launch_sage_d(Launcher& L, const SageAttnParams& p) {
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(sage_attention_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sg::smem_bytes<D>());
        attr_set = true;
    }
    L.launch(sage_attention_kernel<D>, dim3((p.S + sg::BQ - 1) / sg::BQ, p.q_heads), dim3(sg::kThreads), sg::smem_bytes<D>(), p);
}

void launch_sage_prefill_attention(Launcher& L, const SageScratch& sc, const __nv_bfloat16* q, const __nv_bfloat16* k,
                                   const __nv_bfloat16* v, __nv_bfloat16* out, int S, int kv_offset, int q_heads,
                                   int kv_heads, int D, int* error) {
    const int T = kv_offset + S;
    if (S <= 0) return;
    if ((D != 128 && D != 64) || S > sc.q_rows || T > sc.kv_rows) {
        if (L.err == cudaSuccess) L.err = cudaErrorInvalidValue;
        return;
    }
    const bool pdl = L.pdl;
    L.pdl = false;
    const int kvw = kv_heads * D, qw = q_heads * D;
    const int nkb = (T + kSageBlock - 1) / kSageBlock;
    L.launch(sage_ksum_kernel, dim3(nkb, kv_heads), dim3(512), 0, k, kvw, T, kv_heads, D, sc.kmean);
    const dim3 gk(nkb, kv_heads), gq((S + kSageBlock - 1) / kSageBlock, q_heads);
    if (D == 128) {
        L.launch(sage_quant_kernel<128>, gk, dim3(512), 0, k, kvw, T, kv_heads, (const float*)sc.kmean, nkb, sc.k8, sc.sk);
        L.launch(sage_quant_kernel<128>, gq, dim3(512), 0, q, qw, S, q_heads, (const float*)nullptr, 0, sc.q8, sc.sq);
    } else {
        L.launch(sage_quant_kernel<64>, gk, dim3(512), 0, k, kvw, T, kv_heads, (const float*)sc.kmean, nkb, sc.k8, sc.sk);
        L.launch(sage_quant_kernel<64>, gq, dim3(512), 0, q, qw, S, q_heads, (const float*)nullptr, 0, sc.q8, sc.sq);
    }
    L.launch(sage_to_half_kernel, dim3(std::min(((size_t)T * kvw / 2 + 255) / 256, (size_t)L.num_sms * 8)), dim3(256), 0, v, kvw, T,
             kvw, static_cast<__half*>(sc.vh));
    if (D == 128 && attention_tc_enabled()) {
        // tcgen05 form: Qi8 . Ki8^T as kind::i8 into TMEM, P . V in fp16 (attention_tc.cuh, I8 variant)
        using C = at::Cfg<128, true>;
        static bool attr_set = false;
        if (!attr_set) {
            cudaFuncSetAttribute(seg_attention_tc_kernel<128, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM);
            attr_set = true;
        }
        CUtensorMap mq, mk, mv;
        const uint64_t qd[3] = {128, (uint64_t)q_heads, (uint64_t)S}, qs[2] = {128, (uint64_t)q_heads * 128};
        const uint64_t kd[3] = {128, (uint64_t)kv_heads, (uint64_t)T}, ks[2] = {128, (uint64_t)kv_heads * 128};
        const uint64_t vd[3] = {128, (uint64_t)kv_heads, (uint64_t)T}, vs[2] = {256, (uint64_t)kv_heads * 256};
        const uint32_t qb[3] = {128, 1, (uint32_t)at::BM}, kb[3] = {128, 1, (uint32_t)at::BN}, vb[3] = {64, 1, (uint32_t)at::BN};
        if (make_map_nd(&mq, sc.q8, 3, qd, qs, qb, CU_TENSOR_MAP_DATA_TYPE_UINT8) && make_map_nd(&mk, sc.k8, 3, kd, ks, kb, CU_TENSOR_MAP_DATA_TYPE_UINT8) &&
            make_map_nd(&mv, sc.vh, 3, vd, vs, vb, CU_TENSOR_MAP_DATA_TYPE_FLOAT16)) {
            SegAttnParams a{};
            a.out = out; a.out_stride = q_heads * D;
            a.S = S; a.kv_offset = kv_offset; a.q_heads = q_heads; a.kv_heads = kv_heads; a.kv_rows = T;
            a.scale = 1.0f / sqrtf((float)D);
            a.sq = sc.sq; a.sk = sc.sk; a.error = error;
            L.launch(seg_attention_tc_kernel<128, true>, dim3((S + at::BM - 1) / at::BM, q_heads), dim3(at::kThreads), C::SMEM, mq, mk, mv, a, error);
            L.pdl = pdl;
            return;
        }
    }
    SageAttnParams p{};
    p.q = sc.q8; p.k = sc.k8; p.v = static_cast<const __half*>(sc.vh); p.sq = sc.sq; p.sk = sc.sk; p.out = out;
    p.S = S; p.kv_offset = kv_offset; p.q_heads = q_heads; p.kv_heads = kv_heads;
    p.scale = 1.0f / sqrtf((float)D);
    if (D == 128) launch_sage_d<128>(L, p); else launch_sage_d<64>(L, p);
    L.pdl = pdl;
}

void qwen_prefill_chunk(efm_b200_ctx& c, KvSlot& slot, int S, int kv_offset, int n_custom, int embed_token_id,
                        bool sample_last, Launcher& L) {
    const efm_model_desc& d = c.d;
    const int H = d.hidden, D = d.head_dim, QD = d.q_heads * D, KVD = d.kv_heads * D, I = d.intermediate;
    const bool pdl = L.pdl;
    L.pdl = false;
    L.launch(embed_rows_kernel, dim3(S), dim3(128), 0, (const int32_t*)c.ids, (const __nv_bfloat16*)c.embed,
             (const __nv_bfloat16*)(n_custom > 0 ? c.custom_embeds : nullptr), c.resid, d.vocab, H, embed_token_id, n_custom);
    for (int l = 0; l < d.num_layers; ++l) {
        const LayerWeights& w = c.layers[l];
        launch_rmsnorm_rows(L, c.resid, w.in_norm, c.norm, S, H, d.rms_eps);
        {
            GemmParams g{c.norm, w.qkv, w.qkv_bias, c.qkv, nullptr, S, QD + 2 * KVD, H};
            launch_gemm<GemmEpi::Bf16Bias>(L, g, &c.state->error);
        }
        L.launch(rope_scatter_kernel, dim3(S), dim3(256), 0,
                 (const __nv_bfloat16*)c.qkv, c.qbuf, slot.k[l], slot.v[l], (const float*)c.inv_freq,
                 (const int32_t*)c.pos3, S, d.q_heads, d.kv_heads, D, kv_offset, d.use_mrope, d.mrope_section[0],
                 d.mrope_section[0] + d.mrope_section[1]);
        if (c.prefill_attention_kind == 1)
            launch_sage_prefill_attention(L, c.sage, c.qbuf, slot.k[l], slot.v[l], c.attn, S, kv_offset, d.q_heads, d.kv_heads, D, &c.state->error);
        else
            launch_prefill_attention(L, c.qbuf, slot.k[l], slot.v[l], c.attn, S, kv_offset, d.q_heads, d.kv_heads, D, &c.state->error);
        if (c.tp_size == 1) {
            GemmParams g{c.attn, w.o, nullptr, nullptr, c.resid, S, H, QD};
            launch_gemm<GemmEpi::Residual>(L, g, &c.state->error);
        } else {      // row-parallel: this rank's input columns, fp32 partial, all-reduce, then the residual add
            GemmParams g{c.attn + (size_t)c.att_rep_idx * c.o_k, w.o, nullptr, nullptr, c.ybuf, S, H, c.o_k, QD};
            launch_gemm<GemmEpi::F32>(L, g, &c.state->error);
            tp_prefill_sum(c, L, S, 0);
        }
        launch_rmsnorm_rows(L, c.resid, w.post_norm, c.norm, S, H, d.rms_eps);
        {     // gate|up with silu(gate) * up in the epilogue
            GemmParams g{c.norm, w.gate_up, nullptr, c.act, nullptr, S, 2 * I, H};
            launch_gemm<GemmEpi::SwiGlu>(L, g, &c.state->error);
        }
        if (c.tp_size == 1) {
            GemmParams g{c.act, w.down, nullptr, nullptr, c.resid, S, H, I};
            launch_gemm<GemmEpi::Residual>(L, g, &c.state->error);
        } else {
            GemmParams g{c.act, w.down, nullptr, nullptr, c.ybuf, S, H, I};
            launch_gemm<GemmEpi::F32>(L, g, &c.state->error);
            tp_prefill_sum(c, L, S, 1);
        }
    }
    if (sample_last) launch_lm_head_and_sample(c, L, c.resid + (size_t)(S - 1) * H, /*advance=*/0, /*decode_pass=*/false);
    L.pdl = pdl;
}

}  // namespace efm
