// SmolVLA-shaped action chunk behind the C ABI (efm_b200_vla_*): three camera images, a prompt and a
// robot state in, one [chunk, action_dim] action chunk out.  The reference ships no code for this
// model, only its description (doc/smolvla_architecture.md); its flow-matching loop follows the same
// Euler plumbing as src/engine/tasks/trajectory_planning/trajectory_planner_engine.cpp:70-78,298-318.
//
// Phases of one chunk, all on one stream and (from the second call on) replayed as one CUDA graph:
//   vision   patch rows -> patch GEMM onto the position table -> vit_layers x [LayerNorm, q|k|v GEMM,
//            per-image bidirectional attention, out GEMM, LayerNorm, fc1 + tanh-GELU GEMM, fc2 GEMM]
//            -> LayerNorm -> pixel shuffle -> connector GEMM into the prefix rows
//   prefix   [image tokens * sqrt(H) | embed[ids] * sqrt(H) | state_proj(state)] -> layers x Llama block; the
//            q|k|v rows of every layer are kept: their k and v columns are that layer's KV cache
//   bridge   even layers: cache rows copied in front of the expert's own K/V rows; odd layers: the expert's
//            k/v projections of the cache rows (they do not depend on the denoising step: computed once)
//   denoise  steps x [suffix embedding, layers x expert block (self-attention over cache + own rows on
//            even layers, cross-attention over the projected cache on odd ones), norm, output projection,
//            x += dt * v]
// GEMMs: the tcgen05 kernel of gemm_tc.cuh; attention: the mma.sync kernel of attention_mma.cuh with
// per-query key ranges; everything else: vla.cuh.
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <map>
#include <new>
#include <string>
#include <vector>

#include "../../layers/launch.cuh"
#include "../../layers/qwen_text.h"
#include "../../operators/attention_mma.cuh"
#include "../../operators/gemm_tc.cuh"
#include "../../operators/skinny_gemm.cuh"
#include "../../operators/vla.cuh"
#include "efm_b200.h"

using namespace efm;

namespace {

// Where one named tensor goes: `rows` x `cols` bf16 at dst; block > 0: rows are stored in groups of
// `block`, group g at row 2 * g * block + phase * block (the gate | up interleave of the SwiGLU epilogue).
struct Slot {
    __nv_bfloat16* dst = nullptr;
    int64_t rows = 0, cols = 0;
    int block = 0, phase = 0;
    bool seen = false;
};

struct VitLayer {
    __nv_bfloat16 *ln1_w, *ln1_b, *qkv_w, *qkv_b, *o_w, *o_b, *ln2_w, *ln2_b, *fc1_w, *fc1_b, *fc2_w, *fc2_b;
};
struct LlamaLayer {
    __nv_bfloat16 *norm1, *qkv_w, *k_w, *v_w, *o_w, *norm2, *gate_up_w, *down_w;   // k_w / v_w: cross-attention layers only
    __nv_bfloat16* kv = nullptr;     // expert: even layers [P + n, 2 KD] cache rows then own rows; odd [P, 2 KD] projected cache
    __nv_bfloat16* qkv = nullptr;    // backbone: [P, QD + 2 KD] kept for the whole chunk (k | v columns = the KV cache)
};

}  // namespace

struct efm_b200_vla {
    efm_vla_desc d{};
    int device = 0, num_sms = 148;
    cudaStream_t stream = nullptr;
    std::string error;
    bool finalized = false;
    std::map<std::string, Slot> slots;
    std::vector<void*> allocations;
    std::vector<VitLayer> vit;
    std::vector<LlamaLayer> vlm, expert;
    int side = 0, patches = 0, img_tok = 0, P = 0, pd = 0, QD = 0, KD = 0, NV = 0;
    __nv_bfloat16 *patch_w, *patch_b, *pos, *post_w, *post_b, *conn_w, *embed, *state_w, *state_b, *expert_norm;
    __nv_bfloat16 *ain_w, *ain_b, *tin_w, *tin_b, *tout_w, *tout_b, *aout_w, *aout_b;
    // inputs / outputs on the device
    float *images = nullptr, *state = nullptr, *noise = nullptr, *x_t = nullptr, *time_tab = nullptr;
    int32_t* ids = nullptr;
    // vision activations
    __nv_bfloat16 *rows = nullptr, *v_xn = nullptr, *v_qkv = nullptr, *v_attn = nullptr, *v_act = nullptr, *shuf = nullptr;
    float* v_resid = nullptr;
    int32_t *v_lo = nullptr, *v_hi = nullptr, *p_lo = nullptr, *p_hi = nullptr, *s_lo = nullptr, *s_hi = nullptr, *c_hi = nullptr;
    // prefix activations
    float* resid = nullptr;
    __nv_bfloat16 *xn = nullptr, *attn = nullptr, *act = nullptr;
    // expert activations
    float *e_resid = nullptr, *cat = nullptr, *h1 = nullptr, *hf = nullptr;
    __nv_bfloat16 *e_xn = nullptr, *e_qkv = nullptr, *e_attn = nullptr, *e_act = nullptr, *cat16 = nullptr, *h16 = nullptr;
    float* gemm_ws = nullptr;
    size_t gemm_ws_floats = 0;
    int* err_word = nullptr;
    int64_t launches = 0, launches_per_chunk = 0;
    int runs = 0;
    cudaGraphExec_t graph = nullptr;
    cudaEvent_t phase_ev[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};   // set while efm_b200_vla_phase_ms runs
    bool mark_phases = false;
    bool use_pdl = false;            // EFM_B200_VLA_PDL=1: programmatic dependent launches inside the denoising loop.  Measured on
                                     // B200: the kernel-by-kernel run gains 15 % (12.2 -> 10.3 ms), the graph replay loses 1.3 %
                                     // (13.40 -> 13.57 ms per chunk), and the graph is what every call after the first uses
};

namespace {

efm_status vla_fail(efm_b200_vla* v, efm_status st, const std::string& msg) {
    if (v != nullptr) v->error = msg;
    return st;
}
#define VLA_CK(v, call)                                                                             \
    do {                                                                                            \
        cudaError_t e_ = (call);                                                                    \
        if (e_ != cudaSuccess)                                                                      \
            return vla_fail(v, e_ == cudaErrorMemoryAllocation ? EFM_ERR_OUT_OF_MEMORY : EFM_ERR_CUDA, \
                            std::string(#call) + ": " + cudaGetErrorString(e_));                    \
    } while (0)

template <typename T>
cudaError_t vla_alloc(efm_b200_vla* v, T** p, size_t count) {
    void* raw = nullptr;
    const size_t bytes = std::max<size_t>(count * sizeof(T), 16);
    cudaError_t e = cudaMalloc(&raw, bytes);
    if (e != cudaSuccess) return e;
    v->allocations.push_back(raw);
    *p = static_cast<T*>(raw);
    return cudaMemsetAsync(raw, 0, bytes, v->stream);
}

// weight tensor: allocate rows x cols and register it under `name`
cudaError_t vla_weight(efm_b200_vla* v, const std::string& name, __nv_bfloat16** p, int64_t rows, int64_t cols) {
    cudaError_t e = vla_alloc(v, p, (size_t)(rows * cols));
    if (e != cudaSuccess) return e;
    Slot s;
    s.dst = *p; s.rows = rows; s.cols = cols;
    v->slots[name] = s;
    return cudaSuccess;
}
// a named tensor that lands inside an already allocated fused tensor
void vla_part(efm_b200_vla* v, const std::string& name, __nv_bfloat16* dst, int64_t rows, int64_t cols, int block = 0, int phase = 0) {
    Slot s;
    s.dst = dst; s.rows = rows; s.cols = cols; s.block = block; s.phase = phase;
    v->slots[name] = s;
}

}  // namespace

extern "C" {

const char* efm_b200_vla_last_error(const efm_b200_vla* v) { return v != nullptr ? v->error.c_str() : "null handle"; }

efm_status efm_b200_vla_destroy(efm_b200_vla* v) {
    if (v == nullptr) return EFM_OK;
    cudaSetDevice(v->device);
    if (v->stream != nullptr) cudaStreamSynchronize(v->stream);
    if (v->graph != nullptr) cudaGraphExecDestroy(v->graph);
    for (void* p : v->allocations) cudaFree(p);
    if (v->stream != nullptr) cudaStreamDestroy(v->stream);
    delete v;
    return EFM_OK;
}

efm_status efm_b200_vla_create(const efm_vla_desc* desc, int32_t device, efm_b200_vla** out) {
    if (desc == nullptr || out == nullptr) return EFM_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    if (desc->struct_size != (int32_t)sizeof(efm_vla_desc)) return EFM_ERR_INVALID_ARGUMENT;
    const efm_vla_desc& d = *desc;
    const bool geometry_ok =
        d.patch > 0 && d.image_size > 0 && d.image_size % d.patch == 0 && d.shuffle > 0 && (d.image_size / d.patch) % d.shuffle == 0 &&
        d.n_images > 0 && d.vit_layers > 0 && d.vit_heads > 0 && d.vit_hidden == d.vit_heads * 64 && d.vit_mlp > 0 && d.vit_mlp % 8 == 0 &&
        (3 * d.patch * d.patch) % 8 == 0 && d.layers > 0 && d.layers % 2 == 0 && d.head_dim == 64 && d.q_heads > 0 && d.kv_heads > 0 &&
        d.q_heads % d.kv_heads == 0 && d.hidden > 0 && d.hidden % 8 == 0 && d.mlp > 0 && d.mlp % 64 == 0 && d.expert_hidden > 0 &&
        d.expert_hidden % 8 == 0 && d.expert_mlp > 0 && d.expert_mlp % 64 == 0 && d.vocab > 0 && d.lang_tokens >= 0 && d.state_dim > 0 &&
        d.action_dim > 0 && d.chunk > 0 && d.steps > 0 && d.rope_theta > 1.f && d.rms_eps > 0.f && d.ln_eps > 0.f;
    if (!geometry_ok) return EFM_ERR_INVALID_ARGUMENT;
    int n_dev = 0;
    if (cudaGetDeviceCount(&n_dev) != cudaSuccess || n_dev <= 0) return EFM_ERR_CUDA;
    if (device < 0 || device >= n_dev) return EFM_ERR_INVALID_ARGUMENT;
    efm_b200_vla* v = new (std::nothrow) efm_b200_vla();
    if (v == nullptr) return EFM_ERR_OUT_OF_MEMORY;
    v->d = d;
    v->device = device;
    if (const char* env = std::getenv("EFM_B200_VLA_PDL")) v->use_pdl = env[0] != '0';
    auto fail_free = [&](efm_status st) { efm_b200_vla_destroy(v); return st; };
#define VTRY(call) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) return fail_free(e_ == cudaErrorMemoryAllocation ? EFM_ERR_OUT_OF_MEMORY : EFM_ERR_CUDA); } while (0)
    VTRY(cudaSetDevice(device));
    cudaDeviceProp prop;
    VTRY(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) { delete v; return EFM_ERR_CUDA; }      // sm_100a kernels only
    v->num_sms = prop.multiProcessorCount;
    VTRY(cudaStreamCreateWithFlags(&v->stream, cudaStreamNonBlocking));
    v->side = d.image_size / d.patch;
    v->patches = v->side * v->side;
    v->img_tok = v->patches / (d.shuffle * d.shuffle);
    v->P = d.n_images * v->img_tok + d.lang_tokens + 1;
    v->pd = 3 * d.patch * d.patch;
    v->QD = d.q_heads * d.head_dim;
    v->KD = d.kv_heads * d.head_dim;
    v->NV = d.n_images * v->patches;
    const int64_t Hv = d.vit_hidden, H = d.hidden, He = d.expert_hidden, QD = v->QD, KD = v->KD, P = v->P, n = d.chunk, NV = v->NV;
    const int64_t SH = Hv * d.shuffle * d.shuffle;

    // ---- weights ----
    VTRY(vla_weight(v, "vit.patch.weight", &v->patch_w, Hv, v->pd));
    VTRY(vla_weight(v, "vit.patch.bias", &v->patch_b, 1, Hv));
    VTRY(vla_weight(v, "vit.pos", &v->pos, v->patches, Hv));
    v->vit.resize(d.vit_layers);
    for (int l = 0; l < d.vit_layers; ++l) {
        VitLayer& b = v->vit[l];
        const std::string p = "vit." + std::to_string(l) + ".";
        VTRY(vla_weight(v, p + "ln1.weight", &b.ln1_w, 1, Hv));
        VTRY(vla_weight(v, p + "ln1.bias", &b.ln1_b, 1, Hv));
        VTRY(vla_alloc(v, &b.qkv_w, (size_t)(3 * Hv * Hv)));
        VTRY(vla_alloc(v, &b.qkv_b, (size_t)(3 * Hv)));
        const char* names[3] = {"q", "k", "v"};
        for (int i = 0; i < 3; ++i) {
            vla_part(v, p + names[i] + ".weight", b.qkv_w + i * Hv * Hv, Hv, Hv);
            vla_part(v, p + names[i] + ".bias", b.qkv_b + i * Hv, 1, Hv);
        }
        VTRY(vla_weight(v, p + "o.weight", &b.o_w, Hv, Hv));
        VTRY(vla_weight(v, p + "o.bias", &b.o_b, 1, Hv));
        VTRY(vla_weight(v, p + "ln2.weight", &b.ln2_w, 1, Hv));
        VTRY(vla_weight(v, p + "ln2.bias", &b.ln2_b, 1, Hv));
        VTRY(vla_weight(v, p + "fc1.weight", &b.fc1_w, d.vit_mlp, Hv));
        VTRY(vla_weight(v, p + "fc1.bias", &b.fc1_b, 1, d.vit_mlp));
        VTRY(vla_weight(v, p + "fc2.weight", &b.fc2_w, Hv, d.vit_mlp));
        VTRY(vla_weight(v, p + "fc2.bias", &b.fc2_b, 1, Hv));
    }
    VTRY(vla_weight(v, "vit.post_ln.weight", &v->post_w, 1, Hv));
    VTRY(vla_weight(v, "vit.post_ln.bias", &v->post_b, 1, Hv));
    VTRY(vla_weight(v, "connector.weight", &v->conn_w, H, SH));
    VTRY(vla_weight(v, "embed", &v->embed, d.vocab, H));
    VTRY(vla_weight(v, "state_proj.weight", &v->state_w, H, d.state_dim));
    VTRY(vla_weight(v, "state_proj.bias", &v->state_b, 1, H));
    auto llama = [&](std::vector<LlamaLayer>& layers, const std::string& pre, int64_t Hx, int64_t Ix, bool is_expert) -> cudaError_t {
        layers.resize(d.layers);
        for (int l = 0; l < d.layers; ++l) {
            LlamaLayer& b = layers[l];
            const std::string p = pre + std::to_string(l) + ".";
            const bool cross = is_expert && (l % 2 == 1);
            cudaError_t e = vla_weight(v, p + "norm1", &b.norm1, 1, Hx);
            if (e != cudaSuccess) return e;
            if (cross) {
                if ((e = vla_weight(v, p + "q.weight", &b.qkv_w, QD, Hx)) != cudaSuccess) return e;
                if ((e = vla_weight(v, p + "k.weight", &b.k_w, KD, KD)) != cudaSuccess) return e;
                if ((e = vla_weight(v, p + "v.weight", &b.v_w, KD, KD)) != cudaSuccess) return e;
            } else {
                if ((e = vla_alloc(v, &b.qkv_w, (size_t)((QD + 2 * KD) * Hx))) != cudaSuccess) return e;
                vla_part(v, p + "q.weight", b.qkv_w, QD, Hx);
                vla_part(v, p + "k.weight", b.qkv_w + QD * Hx, KD, Hx);
                vla_part(v, p + "v.weight", b.qkv_w + (QD + KD) * Hx, KD, Hx);
                b.k_w = b.v_w = nullptr;
            }
            if ((e = vla_weight(v, p + "o.weight", &b.o_w, Hx, QD)) != cudaSuccess) return e;
            if ((e = vla_weight(v, p + "norm2", &b.norm2, 1, Hx)) != cudaSuccess) return e;
            if ((e = vla_alloc(v, &b.gate_up_w, (size_t)(2 * Ix * Hx))) != cudaSuccess) return e;
            vla_part(v, p + "gate.weight", b.gate_up_w, Ix, Hx, 64, 0);
            vla_part(v, p + "up.weight", b.gate_up_w, Ix, Hx, 64, 1);
            if ((e = vla_weight(v, p + "down.weight", &b.down_w, Hx, Ix)) != cudaSuccess) return e;
            if (is_expert) e = vla_alloc(v, &b.kv, (size_t)((cross ? P : P + n) * 2 * KD));
            else e = vla_alloc(v, &b.qkv, (size_t)(P * (QD + 2 * KD)));
            if (e != cudaSuccess) return e;
        }
        return cudaSuccess;
    };
    VTRY(llama(v->vlm, "vlm.", H, d.mlp, false));
    VTRY(llama(v->expert, "expert.", He, d.expert_mlp, true));
    VTRY(vla_weight(v, "expert.norm", &v->expert_norm, 1, He));
    VTRY(vla_weight(v, "action_in.weight", &v->ain_w, He, d.action_dim));
    VTRY(vla_weight(v, "action_in.bias", &v->ain_b, 1, He));
    VTRY(vla_weight(v, "time_in.weight", &v->tin_w, He, 2 * He));
    VTRY(vla_weight(v, "time_in.bias", &v->tin_b, 1, He));
    VTRY(vla_weight(v, "time_out.weight", &v->tout_w, He, He));
    VTRY(vla_weight(v, "time_out.bias", &v->tout_b, 1, He));
    VTRY(vla_weight(v, "action_out.weight", &v->aout_w, d.action_dim, He));
    VTRY(vla_weight(v, "action_out.bias", &v->aout_b, 1, d.action_dim));

    // ---- inputs, activations ----
    VTRY(vla_alloc(v, &v->images, (size_t)d.n_images * 3 * d.image_size * d.image_size));
    VTRY(vla_alloc(v, &v->ids, (size_t)std::max(1, d.lang_tokens)));
    VTRY(vla_alloc(v, &v->state, (size_t)d.state_dim));
    VTRY(vla_alloc(v, &v->noise, (size_t)(n * d.action_dim)));
    VTRY(vla_alloc(v, &v->x_t, (size_t)(n * d.action_dim)));
    VTRY(vla_alloc(v, &v->time_tab, (size_t)(d.steps * He)));
    VTRY(vla_alloc(v, &v->rows, (size_t)(NV * v->pd)));
    VTRY(vla_alloc(v, &v->v_resid, (size_t)(NV * Hv)));
    VTRY(vla_alloc(v, &v->v_xn, (size_t)(NV * Hv)));
    VTRY(vla_alloc(v, &v->v_qkv, (size_t)(NV * 3 * Hv)));
    VTRY(vla_alloc(v, &v->v_attn, (size_t)(NV * Hv)));
    VTRY(vla_alloc(v, &v->v_act, (size_t)(NV * d.vit_mlp)));
    VTRY(vla_alloc(v, &v->shuf, (size_t)(d.n_images * v->img_tok * SH)));
    VTRY(vla_alloc(v, &v->v_lo, (size_t)NV));
    VTRY(vla_alloc(v, &v->v_hi, (size_t)NV));
    VTRY(vla_alloc(v, &v->p_lo, (size_t)P));
    VTRY(vla_alloc(v, &v->p_hi, (size_t)P));
    VTRY(vla_alloc(v, &v->s_lo, (size_t)n));
    VTRY(vla_alloc(v, &v->s_hi, (size_t)n));
    VTRY(vla_alloc(v, &v->c_hi, (size_t)n));
    VTRY(vla_alloc(v, &v->resid, (size_t)(P * H)));
    VTRY(vla_alloc(v, &v->xn, (size_t)(P * H)));
    VTRY(vla_alloc(v, &v->attn, (size_t)(P * QD)));
    VTRY(vla_alloc(v, &v->act, (size_t)(P * d.mlp)));
    VTRY(vla_alloc(v, &v->e_resid, (size_t)(n * He)));
    VTRY(vla_alloc(v, &v->cat, (size_t)(n * 2 * He)));
    VTRY(vla_alloc(v, &v->h1, (size_t)(n * He)));
    VTRY(vla_alloc(v, &v->hf, (size_t)(n * He)));
    VTRY(vla_alloc(v, &v->e_xn, (size_t)(n * He)));
    VTRY(vla_alloc(v, &v->cat16, (size_t)(n * 2 * He)));
    VTRY(vla_alloc(v, &v->h16, (size_t)(n * He)));
    VTRY(vla_alloc(v, &v->e_qkv, (size_t)(n * (QD + 2 * KD))));
    VTRY(vla_alloc(v, &v->e_attn, (size_t)(n * QD)));
    VTRY(vla_alloc(v, &v->e_act, (size_t)(n * d.expert_mlp)));
    v->gemm_ws_floats = (size_t)v->num_sms * 128 * 256;
    VTRY(vla_alloc(v, &v->gemm_ws, v->gemm_ws_floats));
    VTRY(vla_alloc(v, &v->err_word, 4));

    // ---- constant tables: attention ranges and the time embedding of every step ----
    {
        std::vector<int32_t> lo((size_t)NV), hi((size_t)NV);
        for (int64_t i = 0; i < NV; ++i) { lo[i] = (int32_t)(i / v->patches * v->patches); hi[i] = lo[i] + v->patches; }
        VTRY(cudaMemcpyAsync(v->v_lo, lo.data(), NV * 4, cudaMemcpyHostToDevice, v->stream));
        VTRY(cudaMemcpyAsync(v->v_hi, hi.data(), NV * 4, cudaMemcpyHostToDevice, v->stream));
        std::vector<int32_t> plo((size_t)P, 0), phi((size_t)P, (int32_t)(P - 1)), slo((size_t)n, 0), shi((size_t)n), chi((size_t)n, (int32_t)P);
        phi[(size_t)P - 1] = (int32_t)P;            // the state token sees everything; nothing else sees it
        for (int64_t i = 0; i < n; ++i) shi[i] = (int32_t)(P + i + 1);
        VTRY(cudaMemcpyAsync(v->p_lo, plo.data(), P * 4, cudaMemcpyHostToDevice, v->stream));
        VTRY(cudaMemcpyAsync(v->p_hi, phi.data(), P * 4, cudaMemcpyHostToDevice, v->stream));
        VTRY(cudaMemcpyAsync(v->s_lo, slo.data(), n * 4, cudaMemcpyHostToDevice, v->stream));
        VTRY(cudaMemcpyAsync(v->s_hi, shi.data(), n * 4, cudaMemcpyHostToDevice, v->stream));
        VTRY(cudaMemcpyAsync(v->c_hi, chi.data(), n * 4, cudaMemcpyHostToDevice, v->stream));
        std::vector<float> tt((size_t)(d.steps * He));
        const int half = (int)He / 2;
        for (int s = 0; s < d.steps; ++s) {
            const double t = 1.0 - (double)s / (double)d.steps;
            for (int i = 0; i < half; ++i) {
                const double frac = half > 1 ? (double)i / (double)(half - 1) : 0.0;
                const double period = 4e-3 * std::pow(4.0 / 4e-3, frac);
                const double ang = 2.0 * 3.14159265358979323846 / period * t;
                tt[(size_t)s * He + i] = (float)std::sin(ang);
                tt[(size_t)s * He + half + i] = (float)std::cos(ang);
            }
        }
        VTRY(cudaMemcpyAsync(v->time_tab, tt.data(), tt.size() * 4, cudaMemcpyHostToDevice, v->stream));
        VTRY(cudaStreamSynchronize(v->stream));
    }
#undef VTRY
    *out = v;
    return EFM_OK;
}

efm_status efm_b200_vla_set_weight(efm_b200_vla* v, const char* name, const void* data, const int64_t* shape, int32_t ndim,
                                   int32_t dtype, int32_t mem_kind) {
    if (v == nullptr) return EFM_ERR_INVALID_ARGUMENT;
    if (name == nullptr || data == nullptr || shape == nullptr) return vla_fail(v, EFM_ERR_INVALID_ARGUMENT, "null argument");
    if (v->finalized) return vla_fail(v, EFM_ERR_STATE, "weights are already finalized");
    if (dtype != EFM_BF16) return vla_fail(v, EFM_ERR_UNSUPPORTED, std::string("weights must be bf16: ") + name);
    auto it = v->slots.find(name);
    if (it == v->slots.end()) return vla_fail(v, EFM_ERR_INVALID_ARGUMENT, std::string("unknown tensor: ") + name);
    Slot& s = it->second;
    int64_t elems = 1;
    for (int i = 0; i < ndim; ++i) elems *= shape[i];
    const bool shape_ok = (ndim == 1 && s.rows == 1 && shape[0] == s.cols) ||
                          (ndim >= 2 && shape[0] == s.rows && elems == s.rows * s.cols);
    if (!shape_ok) return vla_fail(v, EFM_ERR_INVALID_ARGUMENT, std::string("unexpected shape for ") + name);
    VLA_CK(v, cudaSetDevice(v->device));
    const cudaMemcpyKind kind = mem_kind == EFM_MEM_DEVICE ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice;
    if (s.block == 0) {
        VLA_CK(v, cudaMemcpyAsync(s.dst, data, (size_t)elems * 2, kind, v->stream));
    } else {
        const size_t group = (size_t)s.block * s.cols * 2;         // bytes of one group of rows
        VLA_CK(v, cudaMemcpy2DAsync(s.dst + (size_t)s.phase * s.block * s.cols, 2 * group, data, group, group,
                                    (size_t)(s.rows / s.block), kind, v->stream));
    }
    VLA_CK(v, cudaStreamSynchronize(v->stream));       // the caller may free `data` on return
    s.seen = true;
    return EFM_OK;
}

efm_status efm_b200_vla_finalize_weights(efm_b200_vla* v) {
    if (v == nullptr) return EFM_ERR_INVALID_ARGUMENT;
    for (const auto& kv : v->slots)
        if (!kv.second.seen) return vla_fail(v, EFM_ERR_STATE, "missing tensor: " + kv.first);
    if (v->finalized) return EFM_OK;
    if (v->d.chunk <= 64) {      // the expert's products run on the skinny kernel: fold its RMSNorm weights into them
        VLA_CK(v, cudaSetDevice(v->device));
        const size_t He = (size_t)v->d.expert_hidden;
        for (int l = 0; l < v->d.layers; ++l) {
            LlamaLayer& e = v->expert[l];
            const size_t qrows = (size_t)(l % 2 == 0 ? v->QD + 2 * v->KD : v->QD), grows = 2 * (size_t)v->d.expert_mlp;
            fold_norm_weight_kernel<<<(unsigned)std::min<size_t>((qrows * He + 255) / 256, 1184), 256, 0, v->stream>>>(e.qkv_w, e.norm1, qrows, (int)He);
            fold_norm_weight_kernel<<<(unsigned)std::min<size_t>((grows * He + 255) / 256, 1184), 256, 0, v->stream>>>(e.gate_up_w, e.norm2, grows, (int)He);
        }
        VLA_CK(v, cudaGetLastError());
        VLA_CK(v, cudaStreamSynchronize(v->stream));
    }
    v->finalized = true;
    return EFM_OK;
}

}  // extern "C"

namespace {

// Every launch of one chunk on L.stream; inputs are already in v->images / ids / state / noise, the result
// lands in v->x_t.
void vla_forward(efm_b200_vla* v, Launcher& L) {
    const efm_vla_desc& d = v->d;
    const int Hv = d.vit_hidden, H = d.hidden, He = d.expert_hidden, QD = v->QD, KD = v->KD, P = v->P, n = d.chunk, NV = v->NV;
    const int D = d.head_dim, QKV = QD + 2 * KD, SH = Hv * d.shuffle * d.shuffle, n_img_tok = d.n_images * v->img_tok;
    int* err = v->err_word;
    const float scale = 1.0f / sqrtf((float)D);
    auto gemm = [&](GemmEpi epi, const __nv_bfloat16* A, int lda, const __nv_bfloat16* B, const __nv_bfloat16* bias, __nv_bfloat16* C,
                    float* Cf, int M, int N, int K) {
        GemmParams g{A, B, bias, C, Cf, M, N, K};
        g.lda = lda;
        launch_gemm_epi(L, epi, g, err);
    };
    auto attend = [&](const __nv_bfloat16* q, int q_stride, const __nv_bfloat16* k, const __nv_bfloat16* vv, int kv_stride,
                      __nv_bfloat16* out, int S, int q_heads, int kv_heads, const int32_t* lo, const int32_t* hi) {
        SegAttnParams a{};
        a.q = q; a.k = k; a.v = vv; a.out = out; a.lo = lo; a.hi = hi;
        a.q_stride = q_stride; a.kv_stride = kv_stride; a.out_stride = q_heads * D;
        a.S = S; a.kv_offset = 0; a.q_heads = q_heads; a.kv_heads = kv_heads; a.scale = scale;
        launch_seg_attention(L, a, D);
    };

    auto mark = [&](int i) { if (v->mark_phases && L.err == cudaSuccess) L.err = cudaEventRecord(v->phase_ev[i], L.stream); };
    mark(0);
    // the action state starts as the noise (copied here, far ahead of the loop that launches with programmatic edges)
    if (L.err == cudaSuccess) L.err = cudaMemcpyAsync(v->x_t, v->noise, (size_t)n * d.action_dim * 4, cudaMemcpyDeviceToDevice, L.stream);
    auto layernorm = [&](const __nv_bfloat16* w, const __nv_bfloat16* b) {       // v_resid -> v_xn
        if (Hv <= 1024 && Hv % 4 == 0)
            L.launch(layernorm_rows_warp_kernel, dim3((NV + 7) / 8), dim3(256), 0, (const float*)v->v_resid, w, b, v->v_xn, NV, Hv, d.ln_eps);
        else
            L.launch(layernorm_rows_kernel, dim3(NV), dim3(256), 0, (const float*)v->v_resid, w, b, v->v_xn, Hv, d.ln_eps);
    };
    // ---- vision tower ----
    L.launch(vla_patch_rows_kernel, dim3(NV), dim3(256), 0, (const float*)v->images, v->rows, d.image_size, d.patch);
    L.launch(vla_tile_rows_kernel, dim3(NV), dim3(256), 0, (const __nv_bfloat16*)v->pos, v->v_resid, v->patches, Hv);
    gemm(GemmEpi::Residual, v->rows, 0, v->patch_w, v->patch_b, nullptr, v->v_resid, NV, Hv, v->pd);
    for (const VitLayer& b : v->vit) {
        layernorm(b.ln1_w, b.ln1_b);
        gemm(GemmEpi::Bf16Bias, v->v_xn, 0, b.qkv_w, b.qkv_b, v->v_qkv, nullptr, NV, 3 * Hv, Hv);
        attend(v->v_qkv, 3 * Hv, v->v_qkv + Hv, v->v_qkv + 2 * Hv, 3 * Hv, v->v_attn, NV, d.vit_heads, d.vit_heads, v->v_lo, v->v_hi);
        gemm(GemmEpi::Residual, v->v_attn, 0, b.o_w, b.o_b, nullptr, v->v_resid, NV, Hv, Hv);
        layernorm(b.ln2_w, b.ln2_b);
        gemm(GemmEpi::Bf16GeluTanh, v->v_xn, 0, b.fc1_w, b.fc1_b, v->v_act, nullptr, NV, d.vit_mlp, Hv);
        gemm(GemmEpi::Residual, v->v_act, 0, b.fc2_w, b.fc2_b, nullptr, v->v_resid, NV, Hv, d.vit_mlp);
    }
    layernorm(v->post_w, v->post_b);
    L.launch(vla_pixel_shuffle_kernel, dim3(n_img_tok), dim3(256), 0, (const __nv_bfloat16*)v->v_xn, v->shuf, v->side, d.shuffle, Hv);
    gemm(GemmEpi::F32, v->shuf, 0, v->conn_w, nullptr, nullptr, v->resid, n_img_tok, H, SH);

    mark(1);
    // ---- prefix through the backbone ----
    L.launch(vla_prefix_rows_kernel, dim3(P), dim3(256), 0, v->resid, (const __nv_bfloat16*)v->embed, (const int32_t*)v->ids,
             (const float*)v->state, (const __nv_bfloat16*)v->state_w, (const __nv_bfloat16*)v->state_b, n_img_tok, d.lang_tokens, H,
             d.state_dim, d.vocab);
    for (LlamaLayer& b : v->vlm) {
        launch_rmsnorm_rows(L, v->resid, b.norm1, v->xn, P, H, d.rms_eps);
        gemm(GemmEpi::Bf16Bias, v->xn, 0, b.qkv_w, nullptr, b.qkv, nullptr, P, QKV, H);
        L.launch(vla_rope_rows_kernel, dim3(P), dim3(256), 0, b.qkv, QKV, d.q_heads, d.kv_heads, D, 0, d.rope_theta,
                 (__nv_bfloat16*)nullptr, 0, 0);
        attend(b.qkv, QKV, b.qkv + QD, b.qkv + QD + KD, QKV, v->attn, P, d.q_heads, d.kv_heads, v->p_lo, v->p_hi);
        gemm(GemmEpi::Residual, v->attn, 0, b.o_w, nullptr, nullptr, v->resid, P, H, QD);
        launch_rmsnorm_rows(L, v->resid, b.norm2, v->xn, P, H, d.rms_eps);
        gemm(GemmEpi::SwiGlu, v->xn, 0, b.gate_up_w, nullptr, v->act, nullptr, P, 2 * d.mlp, H);
        gemm(GemmEpi::Residual, v->act, 0, b.down_w, nullptr, nullptr, v->resid, P, H, d.mlp);
    }

    mark(2);
    // ---- bridge: what the expert reads of the prefix, once per chunk ----
    for (int l = 0; l < d.layers; ++l) {
        LlamaLayer& e = v->expert[l];
        const __nv_bfloat16* cache_k = v->vlm[l].qkv + QD;
        if (l % 2 == 0) {
            L.launch(vla_copy_rows_kernel, dim3(P), dim3(128), 0, cache_k, QKV, e.kv, 2 * KD, 2 * KD);
        } else {
            gemm(GemmEpi::Bf16Bias, cache_k, QKV, e.k_w, nullptr, v->xn, nullptr, P, KD, KD);           // xn: scratch [P, KD]
            L.launch(vla_copy_rows_kernel, dim3(P), dim3(128), 0, (const __nv_bfloat16*)v->xn, KD, e.kv, 2 * KD, KD);
            gemm(GemmEpi::Bf16Bias, cache_k + KD, QKV, e.v_w, nullptr, v->xn, nullptr, P, KD, KD);
            L.launch(vla_copy_rows_kernel, dim3(P), dim3(128), 0, (const __nv_bfloat16*)v->xn, KD, e.kv + KD, 2 * KD, KD);
        }
    }

    mark(3);
    // ---- denoising loop ----
    const float dt = -1.0f / (float)d.steps;
    auto small = [&](int act, const float* x, int ldx, const __nv_bfloat16* W, const __nv_bfloat16* bias, float* y, int ldy, int M, int N,
                     int K, float euler, __nv_bfloat16* y16 = nullptr, int ldy16 = 0) {
        const dim3 grid((M * N + 7) / 8), block(256);
        if (act == 1) L.launch(vla_small_linear_kernel<1>, grid, block, 0, x, ldx, W, bias, y, ldy, M, N, K, euler, y16, ldy16 > 0 ? ldy16 : N);
        else L.launch(vla_small_linear_kernel<0>, grid, block, 0, x, ldx, W, bias, y, ldy, M, N, K, euler, y16, ldy16 > 0 ? ldy16 : N);
    };
    // the expert's products: at most 64 rows -> weights streamed once on mma.sync tiles; more rows -> the tcgen05 GEMM
    const bool skinny = n <= 64;
    auto egemm = [&](GemmEpi epi, const __nv_bfloat16* A, const __nv_bfloat16* B, __nv_bfloat16* C, float* Cf, int N, int K) {
        if (!skinny) { gemm(epi, A, 0, B, nullptr, C, Cf, n, N, K); return; }
        SkinnyParams sp{A, B, C, Cf, n, N, K, K};
        sp.eps = d.rms_eps;
        if (epi == GemmEpi::Residual) sp.x16_out = v->e_xn;      // bf16 copy of the new residual for the NORM product that follows
        if (epi == GemmEpi::SwiGlu) L.launch(skinny_gemm_kernel<SkinnyEpi::SwiGlu, 2, true>, dim3(N / 16), dim3(kSkinnyThreads), 0, sp);
        else if (epi == GemmEpi::Residual && K >= 1024)      // long K: 16 warps share the k-chunks of a tile (+1.8 % on the chunk;
                                                             // 16 warps on the two-tile variants measured 4 % slower: fewer blocks per SM)
            L.launch(skinny_gemm_kernel<SkinnyEpi::Residual, 1, false, 16>, dim3(N / 8), dim3(512), 0, sp);
        else if (epi == GemmEpi::Residual) L.launch(skinny_gemm_kernel<SkinnyEpi::Residual, 1>, dim3(N / 8), dim3(kSkinnyThreads), 0, sp);
        else L.launch(skinny_gemm_kernel<SkinnyEpi::Bf16, 1>, dim3(N / 8), dim3(kSkinnyThreads), 0, sp);
    };
    // the loop's kernels all open with the dependent-launch wait, so they may be launched with programmatic
    // serialization (off by default, see use_pdl; the tcgen05 GEMM of the chunk > 64 fallback has no such wait)
    L.pdl = skinny && v->use_pdl;
    L.pdl_rows = L.pdl;
    for (int s = 0; s < d.steps; ++s) {
        if (skinny) {      // the two wider linears of the suffix embedding on the weight-streaming kernel, bf16 activations
            small(0, v->x_t, d.action_dim, v->ain_w, v->ain_b, v->cat, 2 * He, n, He, d.action_dim, 0.f, v->cat16, 2 * He);
            L.launch(vla_fill_time_kernel, dim3(n), dim3(256), 0, v->cat, 2 * He, He, (const float*)(v->time_tab + (size_t)s * He), He, v->cat16);
            SkinnyParams t1{v->cat16, v->tin_w, v->h16, nullptr, n, He, 2 * He, 2 * He};
            t1.bias = v->tin_b; t1.act = 1;
            L.launch(skinny_gemm_kernel<SkinnyEpi::Bf16, 1>, dim3(He / 8), dim3(kSkinnyThreads), 0, t1);
            SkinnyParams t2{v->h16, v->tout_w, nullptr, v->e_resid, n, He, He, He};
            t2.bias = v->tout_b; t2.assign = 1; t2.x16_out = v->e_xn;
            L.launch(skinny_gemm_kernel<SkinnyEpi::Residual, 1>, dim3(He / 8), dim3(kSkinnyThreads), 0, t2);
        } else {
            small(0, v->x_t, d.action_dim, v->ain_w, v->ain_b, v->cat, 2 * He, n, He, d.action_dim, 0.f);
            L.launch(vla_fill_time_kernel, dim3(n), dim3(256), 0, v->cat, 2 * He, He, (const float*)(v->time_tab + (size_t)s * He), He,
                     (__nv_bfloat16*)nullptr);
            small(1, v->cat, 2 * He, v->tin_w, v->tin_b, v->h1, He, n, He, 2 * He, 0.f);
            small(0, v->h1, He, v->tout_w, v->tout_b, v->e_resid, He, n, He, He, 0.f);
        }
        for (int l = 0; l < d.layers; ++l) {
            LlamaLayer& e = v->expert[l];
            // skinny path: both RMSNorms are folded into the products that follow them (weights folded at load time,
            // e_xn = bf16 copy of the un-normalised residual written by the kernel that produced it)
            if (!skinny) launch_rmsnorm_rows(L, v->e_resid, e.norm1, v->e_xn, n, He, d.rms_eps);
            if (skinny) {          // norm, projection, RoPE and the K / V scatter in one kernel
                const bool self = l % 2 == 0;
                SkinnyParams sp{v->e_xn, e.qkv_w, v->e_qkv, nullptr, n, self ? QKV : QD, He, He};
                sp.q_heads = d.q_heads; sp.kv_heads = self ? d.kv_heads : 0; sp.pos0 = self ? P : 0; sp.theta = d.rope_theta;
                sp.kv_out = self ? e.kv : nullptr; sp.kv_stride = 2 * KD; sp.kv_row0 = P; sp.eps = d.rms_eps;
                L.launch(skinny_gemm_kernel<SkinnyEpi::QkvRope, 2, true>, dim3(sp.N / 16), dim3(kSkinnyThreads), 0, sp);
                SegAttnParams a{};
                a.q = v->e_qkv; a.k = e.kv; a.v = e.kv + KD; a.out = v->e_attn; a.lo = v->s_lo; a.hi = self ? v->s_hi : v->c_hi;
                a.q_stride = self ? QKV : QD; a.kv_stride = 2 * KD; a.out_stride = QD;
                a.S = n; a.kv_offset = 0; a.q_heads = d.q_heads; a.kv_heads = d.kv_heads; a.scale = scale;
                launch_seg_attention_short(L, a, D, self ? P + n : P);
            } else if (l % 2 == 0) {
                egemm(GemmEpi::Bf16Bias, v->e_xn, e.qkv_w, v->e_qkv, nullptr, QKV, He);
                L.launch(vla_rope_rows_kernel, dim3(n), dim3(256), 0, v->e_qkv, QKV, d.q_heads, d.kv_heads, D, P, d.rope_theta, e.kv,
                         2 * KD, P);
                attend(v->e_qkv, QKV, e.kv, e.kv + KD, 2 * KD, v->e_attn, n, d.q_heads, d.kv_heads, v->s_lo, v->s_hi);
            } else {
                egemm(GemmEpi::Bf16Bias, v->e_xn, e.qkv_w, v->e_qkv, nullptr, QD, He);
                L.launch(vla_rope_rows_kernel, dim3(n), dim3(256), 0, v->e_qkv, QD, d.q_heads, 0, D, 0, d.rope_theta,
                         (__nv_bfloat16*)nullptr, 0, 0);
                attend(v->e_qkv, QD, e.kv, e.kv + KD, 2 * KD, v->e_attn, n, d.q_heads, d.kv_heads, v->s_lo, v->c_hi);
            }
            egemm(GemmEpi::Residual, v->e_attn, e.o_w, nullptr, v->e_resid, He, QD);
            if (!skinny) launch_rmsnorm_rows(L, v->e_resid, e.norm2, v->e_xn, n, He, d.rms_eps);
            egemm(GemmEpi::SwiGlu, v->e_xn, e.gate_up_w, v->e_act, nullptr, 2 * d.expert_mlp, He);
            egemm(GemmEpi::Residual, v->e_act, e.down_w, nullptr, v->e_resid, He, d.expert_mlp);
        }
        launch_rmsnorm_rows(L, v->e_resid, v->expert_norm, v->e_xn, n, He, d.rms_eps);
        L.launch(vla_bf16_to_f32_kernel, dim3((n * He + 255) / 256), dim3(256), 0, (const __nv_bfloat16*)v->e_xn, v->hf, n * He);
        small(0, v->hf, He, v->aout_w, v->aout_b, v->x_t, d.action_dim, n, d.action_dim, He, dt);
    }
    L.pdl = false;
    L.pdl_rows = false;
    mark(4);
}

// Runs one chunk on the inputs resident on the device: eagerly the first time (which also sets every
// kernel attribute), then as one captured graph.
efm_status vla_run(efm_b200_vla* v) {
    Launcher L;
    L.stream = v->stream;
    L.pdl = false;
    L.gemm_ws = v->gemm_ws;
    L.gemm_ws_floats = v->gemm_ws_floats;
    L.num_sms = v->num_sms;
    if (v->runs == 0) {
        int64_t count = 0;
        L.counter = &count;
        vla_forward(v, L);
        if (L.err != cudaSuccess) return vla_fail(v, EFM_ERR_CUDA, std::string("chunk launch: ") + cudaGetErrorString(L.err));
        v->launches_per_chunk = count;
    } else {
        if (v->graph == nullptr) {
            cudaGraph_t g = nullptr;
            VLA_CK(v, cudaStreamBeginCapture(v->stream, cudaStreamCaptureModeThreadLocal));
            vla_forward(v, L);
            cudaError_t e = cudaStreamEndCapture(v->stream, &g);
            if (L.err != cudaSuccess || e != cudaSuccess) {
                if (g != nullptr) cudaGraphDestroy(g);
                return vla_fail(v, EFM_ERR_CUDA, std::string("chunk capture: ") + cudaGetErrorString(L.err != cudaSuccess ? L.err : e));
            }
            e = cudaGraphInstantiate(&v->graph, g, 0);
            cudaGraphDestroy(g);
            if (e != cudaSuccess) return vla_fail(v, EFM_ERR_CUDA, std::string("chunk graph: ") + cudaGetErrorString(e));
        }
        VLA_CK(v, cudaGraphLaunch(v->graph, v->stream));
    }
    ++v->runs;
    v->launches += v->launches_per_chunk;
    return EFM_OK;
}

}  // namespace

extern "C" {

efm_status efm_b200_vla_chunk(efm_b200_vla* v, const float* images, const int32_t* lang_ids, const float* state, const float* noise,
                              int32_t mem_kind, float* actions_out) {
    if (v == nullptr) return EFM_ERR_INVALID_ARGUMENT;
    if (!v->finalized) return vla_fail(v, EFM_ERR_STATE, "weights are not finalized");
    const efm_vla_desc& d = v->d;
    VLA_CK(v, cudaSetDevice(v->device));
    const cudaMemcpyKind in = mem_kind == EFM_MEM_DEVICE ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice;
    const cudaMemcpyKind out = mem_kind == EFM_MEM_DEVICE ? cudaMemcpyDeviceToDevice : cudaMemcpyDeviceToHost;
    if (images != nullptr) VLA_CK(v, cudaMemcpyAsync(v->images, images, (size_t)d.n_images * 3 * d.image_size * d.image_size * 4, in, v->stream));
    if (lang_ids != nullptr && d.lang_tokens > 0) VLA_CK(v, cudaMemcpyAsync(v->ids, lang_ids, (size_t)d.lang_tokens * 4, in, v->stream));
    if (state != nullptr) VLA_CK(v, cudaMemcpyAsync(v->state, state, (size_t)d.state_dim * 4, in, v->stream));
    if (noise != nullptr) VLA_CK(v, cudaMemcpyAsync(v->noise, noise, (size_t)d.chunk * d.action_dim * 4, in, v->stream));
    efm_status st = vla_run(v);
    if (st != EFM_OK) return st;
    if (actions_out != nullptr) VLA_CK(v, cudaMemcpyAsync(actions_out, v->x_t, (size_t)d.chunk * d.action_dim * 4, out, v->stream));
    VLA_CK(v, cudaStreamSynchronize(v->stream));
    int flag = 0;
    VLA_CK(v, cudaMemcpy(&flag, v->err_word, 4, cudaMemcpyDeviceToHost));
    if (flag != 0) {
        cudaMemset(v->err_word, 0, 4);
        return vla_fail(v, EFM_ERR_DEVICE_WAIT, "a GEMM pipeline wait ran out inside the chunk");
    }
    return EFM_OK;
}

efm_status efm_b200_vla_stream(efm_b200_vla* v, void** stream_out) {
    if (v == nullptr || stream_out == nullptr) return EFM_ERR_INVALID_ARGUMENT;
    *stream_out = (void*)v->stream;
    return EFM_OK;
}

efm_status efm_b200_vla_enqueue(efm_b200_vla* v) {
    if (v == nullptr) return EFM_ERR_INVALID_ARGUMENT;
    if (!v->finalized) return vla_fail(v, EFM_ERR_STATE, "weights are not finalized");
    VLA_CK(v, cudaSetDevice(v->device));
    return vla_run(v);
}

efm_status efm_b200_vla_phase_ms(efm_b200_vla* v, float* ms4) {
    if (v == nullptr || ms4 == nullptr) return EFM_ERR_INVALID_ARGUMENT;
    if (!v->finalized || v->runs == 0) return vla_fail(v, EFM_ERR_STATE, "run a chunk first");
    VLA_CK(v, cudaSetDevice(v->device));
    for (cudaEvent_t& e : v->phase_ev) VLA_CK(v, cudaEventCreate(&e));
    Launcher L;
    L.stream = v->stream;
    L.pdl = false;
    L.gemm_ws = v->gemm_ws;
    L.gemm_ws_floats = v->gemm_ws_floats;
    L.num_sms = v->num_sms;
    v->mark_phases = true;
    vla_forward(v, L);                 // kernel by kernel, not the graph
    v->mark_phases = false;
    cudaError_t e = L.err != cudaSuccess ? L.err : cudaStreamSynchronize(v->stream);
    if (e == cudaSuccess)
        for (int i = 0; i < 4 && e == cudaSuccess; ++i) e = cudaEventElapsedTime(&ms4[i], v->phase_ev[i], v->phase_ev[i + 1]);
    for (cudaEvent_t& ev : v->phase_ev) { cudaEventDestroy(ev); ev = nullptr; }
    if (e != cudaSuccess) return vla_fail(v, EFM_ERR_CUDA, std::string("phase timing: ") + cudaGetErrorString(e));
    v->launches += v->launches_per_chunk;
    return EFM_OK;
}

efm_status efm_b200_vla_launch_count(const efm_b200_vla* v, int64_t* total, int64_t* per_chunk) {
    if (v == nullptr) return EFM_ERR_INVALID_ARGUMENT;
    if (total != nullptr) *total = v->launches;
    if (per_chunk != nullptr) *per_chunk = v->launches_per_chunk;
    return EFM_OK;
}

}  // extern "C"
