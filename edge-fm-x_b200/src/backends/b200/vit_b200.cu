// Qwen2.5-VL vision encoder behind the C ABI (efm_b200_vit_*): weight ingestion, the host-side
// plan derived from the patch grids (window-major order, attention ranges, 2-D positions) and the
// launch sequence.  The reference has no vision tower; the output is the tensor its callers pass
// through Request.embedding (examples/qwen2.5-vl-3b-instruct/generate.py:3).
//
// Per layer: RMSNorm rows -> qkv GEMM (+bias) -> 2-D rotary -> attention over windows or whole
// frames -> proj GEMM (+bias) into the fp32 residual stream -> RMSNorm rows -> gate|up GEMM with
// silu(gate)*up epilogue -> down GEMM (+bias) into the residual stream.  All GEMMs are the
// tcgen05 kernel of gemm_tc.cuh; the MLP width is zero-padded to a multiple of 64 at load time so
// that every operand row is 16-byte aligned for TMA.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <new>
#include <string>
#include <vector>

#include "../../layers/launch.cuh"
#include "../../layers/qwen_text.h"
#include "../../operators/attention_mma.cuh"
#include "../../operators/gemm_tc.cuh"
#include "../../operators/vit.cuh"
#include "ctx.h"
#include "nccl_glue.h"

using namespace efm;

namespace {

enum : uint32_t { vN1 = 1, vN2 = 2, vQkvW = 4, vQkvB = 8, vProjW = 16, vProjB = 32, vGateW = 64, vGateB = 128,
                  vUpW = 256, vUpB = 512, vDownW = 1024, vDownB = 2048, vAll = 4095 };
enum : uint32_t { gPatch = 1, gLnQ = 2, gM0W = 4, gM0B = 8, gM2W = 16, gM2B = 32, gAll = 63 };

struct VitBlock {
    __nv_bfloat16 *norm1 = nullptr, *norm2 = nullptr;
    __nv_bfloat16 *qkv_w = nullptr, *qkv_b = nullptr;        // [3H, H], [3H]
    __nv_bfloat16 *proj_w = nullptr, *proj_b = nullptr;      // [H, H], [H]
    __nv_bfloat16 *gate_up_w = nullptr, *gate_up_b = nullptr;  // [2 Ip, H], [2 Ip]: 64 gate rows, 64 up rows, ...
    __nv_bfloat16 *down_w = nullptr, *down_b = nullptr;      // [H, Ip], [H]
    uint32_t seen = 0;
};

}  // namespace

struct efm_b200_vit {
    efm_b200_ctx* ctx = nullptr;
    efm_vit_desc d{};
    int head_dim = 0, ipad = 0, patch_dim = 0, unit = 0, merged = 0;
    bool finalized = false;
    uint32_t seen = 0;
    std::vector<VitBlock> blocks;
    __nv_bfloat16 *patch_w = nullptr, *ln_q = nullptr, *m0_w = nullptr, *m0_b = nullptr, *m2_w = nullptr, *m2_b = nullptr;
    // activations for max_patches rows
    __nv_bfloat16 *pixels = nullptr, *xn = nullptr, *qkv = nullptr, *attn = nullptr, *act = nullptr, *h1 = nullptr,
                  *mo = nullptr, *out_dev = nullptr;
    float *pe = nullptr, *resid = nullptr;
    float2* rope_tab = nullptr;          // [N, D/2] (cos, sin)
    int32_t* plan = nullptr;             // order [N/unit] | pos_h | pos_w | lo_win | hi_win | lo_full | hi_full, [N] each
    __nv_bfloat16* qkv_all = nullptr;    // tensor parallel: q|k|v rows of every rank, full-attention layers [N, 3H]
    __nv_bfloat16* mo_all = nullptr;     // tensor parallel: merged tokens of every rank [N/unit, out]
    std::vector<void*> allocations;
};

namespace {

efm_status vfail(efm_b200_vit* v, efm_status st, const std::string& msg) {
    if (v != nullptr && v->ctx != nullptr) v->ctx->error = msg;
    return st;
}
#define VIT_CK(v, call)                                                                           \
    do {                                                                                          \
        cudaError_t e_ = (call);                                                                  \
        if (e_ != cudaSuccess)                                                                    \
            return vfail(v, e_ == cudaErrorMemoryAllocation ? EFM_ERR_OUT_OF_MEMORY : EFM_ERR_CUDA, \
                         std::string(#call) + ": " + cudaGetErrorString(e_));                     \
    } while (0)

template <typename T>
cudaError_t valloc(efm_b200_vit* v, T** p, size_t count) {
    void* raw = nullptr;
    const size_t bytes = std::max<size_t>(count * sizeof(T), 16);
    cudaError_t e = cudaMalloc(&raw, bytes);
    if (e != cudaSuccess) return e;
    v->allocations.push_back(raw);
    *p = static_cast<T*>(raw);
    return cudaMemsetAsync(raw, 0, bytes, v->ctx->stream);
}

bool is_shape(const int64_t* shape, int ndim, std::initializer_list<int64_t> want) {
    if (ndim != (int)want.size()) return false;
    int i = 0;
    for (int64_t w : want) if (shape[i++] != w) return false;
    return true;
}

// Host-side plan of one encode call: see the description of efm_b200_vit_encode.
struct Plan {
    std::vector<int32_t> order, pos_h, pos_w, lo_win, hi_win, lo_full, hi_full;
};

bool build_plan(const efm_vit_desc& d, const int32_t* grids, int n_grids, Plan& P, std::string& why) {
    const int m = d.merge, win = d.window / d.patch / m;
    if (win <= 0) { why = "window smaller than one merged token"; return false; }
    int base = 0, row0 = 0;       // merged tokens / patch rows before this grid
    for (int gi = 0; gi < n_grids; ++gi) {
        const int t = grids[3 * gi], H = grids[3 * gi + 1], W = grids[3 * gi + 2];
        if (t <= 0 || H <= 0 || W <= 0 || H % m != 0 || W % m != 0) { why = "grid rows and columns must be positive multiples of the merge size"; return false; }
        const int h = H / m, w = W / m;
        for (int f = 0; f < t; ++f) {
            const int frame_lo = row0, frame_hi = row0 + H * W;
            for (int wr = 0; wr * win < h; ++wr)
                for (int wc = 0; wc * win < w; ++wc) {
                    const int r1 = std::min(h, (wr + 1) * win), c1 = std::min(w, (wc + 1) * win);
                    const int n = (r1 - wr * win) * (c1 - wc * win) * m * m;
                    const int lo = (int)P.pos_h.size(), hi = lo + n;
                    for (int r = wr * win; r < r1; ++r)
                        for (int c = wc * win; c < c1; ++c) {
                            P.order.push_back(base + (f * h + r) * w + c);
                            for (int dy = 0; dy < m; ++dy)
                                for (int dx = 0; dx < m; ++dx) {
                                    P.pos_h.push_back(r * m + dy);
                                    P.pos_w.push_back(c * m + dx);
                                    P.lo_win.push_back(lo);
                                    P.hi_win.push_back(hi);
                                    P.lo_full.push_back(frame_lo);
                                    P.hi_full.push_back(frame_hi);
                                }
                        }
                }
            row0 = frame_hi;
        }
        base += t * h * w;
    }
    return true;
}

}  // namespace

extern "C" {

efm_status efm_b200_vit_create(efm_b200_ctx* c, const efm_vit_desc* desc, efm_b200_vit** out) {
    if (c == nullptr || desc == nullptr || out == nullptr) return EFM_ERR_INVALID_ARGUMENT;
    auto bad = [&](const char* m) { c->error = m; return (efm_status)EFM_ERR_INVALID_ARGUMENT; };
    if (desc->struct_size != (int32_t)sizeof(efm_vit_desc)) return bad("efm_vit_desc.struct_size mismatch");
    const efm_vit_desc& d = *desc;
    if (d.depth <= 0 || d.heads <= 0 || d.hidden <= 0 || d.hidden % d.heads != 0) return bad("bad vision geometry");
    const int D = d.hidden / d.heads;
    if (D != 64 && D != 80 && D != 128) { c->error = "vision head_dim must be 64, 80 or 128"; return EFM_ERR_UNSUPPORTED; }
    if (d.intermediate <= 0 || d.intermediate % 4 != 0 || d.hidden % 8 != 0 || d.out_hidden <= 0 || d.out_hidden % 8 != 0)
        return bad("vision widths: hidden and out_hidden multiples of 8, intermediate a multiple of 4");
    if (d.merge <= 0 || d.patch <= 0 || d.temporal_patch <= 0 || d.in_channels <= 0 || d.window < d.patch * d.merge)
        return bad("bad patch / merge / window sizes");
    if ((d.in_channels * d.temporal_patch * d.patch * d.patch) % 8 != 0) return bad("patch vector length must be a multiple of 8");
    if (d.n_fullatt < 0 || d.n_fullatt > 8) return bad("n_fullatt out of range");
    if (d.max_patches <= 0 || d.max_patches % (d.merge * d.merge) != 0 || d.max_patches > (1 << 20)) return bad("max_patches out of range");
    efm_b200_vit* v = new (std::nothrow) efm_b200_vit();
    if (v == nullptr) { c->error = "host allocation failed"; return EFM_ERR_OUT_OF_MEMORY; }
    v->ctx = c;
    v->d = d;
    v->head_dim = D;
    v->ipad = (d.intermediate + 63) / 64 * 64;
    v->patch_dim = d.in_channels * d.temporal_patch * d.patch * d.patch;
    v->unit = d.merge * d.merge;
    v->merged = d.hidden * v->unit;
    v->blocks.resize(d.depth);
    auto fail_free = [&](efm_status st) { efm_b200_vit_destroy(v); return st; };
#define VTRY(call) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) { vfail(v, e_ == cudaErrorMemoryAllocation ? EFM_ERR_OUT_OF_MEMORY : EFM_ERR_CUDA, std::string("vision encoder allocation: ") + cudaGetErrorString(e_)); return fail_free(e_ == cudaErrorMemoryAllocation ? EFM_ERR_OUT_OF_MEMORY : EFM_ERR_CUDA); } } while (0)
    VTRY(cudaSetDevice(c->device));
    const size_t H = d.hidden, Ip = v->ipad, N = d.max_patches, M = v->merged, NM = N / v->unit;
    VTRY(valloc(v, &v->patch_w, H * v->patch_dim));
    for (VitBlock& b : v->blocks) {
        VTRY(valloc(v, &b.norm1, H));
        VTRY(valloc(v, &b.norm2, H));
        VTRY(valloc(v, &b.qkv_w, 3 * H * H));
        VTRY(valloc(v, &b.qkv_b, 3 * H));
        VTRY(valloc(v, &b.proj_w, H * H));
        VTRY(valloc(v, &b.proj_b, H));
        VTRY(valloc(v, &b.gate_up_w, 2 * Ip * H));
        VTRY(valloc(v, &b.gate_up_b, 2 * Ip));
        VTRY(valloc(v, &b.down_w, H * Ip));
        VTRY(valloc(v, &b.down_b, H));
    }
    VTRY(valloc(v, &v->ln_q, H));
    VTRY(valloc(v, &v->m0_w, M * M));
    VTRY(valloc(v, &v->m0_b, M));
    VTRY(valloc(v, &v->m2_w, (size_t)d.out_hidden * M));
    VTRY(valloc(v, &v->m2_b, (size_t)d.out_hidden));
    VTRY(valloc(v, &v->pixels, N * v->patch_dim));
    VTRY(valloc(v, &v->pe, N * H));
    VTRY(valloc(v, &v->resid, N * H));
    VTRY(valloc(v, &v->xn, N * H));
    VTRY(valloc(v, &v->qkv, N * 3 * H));
    VTRY(valloc(v, &v->attn, N * H));
    VTRY(valloc(v, &v->act, N * Ip));
    VTRY(valloc(v, &v->h1, NM * M));
    VTRY(valloc(v, &v->mo, NM * d.out_hidden));
    VTRY(valloc(v, &v->out_dev, NM * d.out_hidden));
    VTRY(valloc(v, &v->plan, NM + 6 * N));
    VTRY(valloc(v, &v->rope_tab, N * (size_t)(D / 2)));
#undef VTRY
    *out = v;
    return EFM_OK;
}

efm_status efm_b200_vit_destroy(efm_b200_vit* v) {
    if (v == nullptr) return EFM_OK;
    if (v->ctx != nullptr) {
        cudaSetDevice(v->ctx->device);
        cudaStreamSynchronize(v->ctx->stream);
    }
    for (void* p : v->allocations) cudaFree(p);
    delete v;
    return EFM_OK;
}

efm_status efm_b200_vit_set_weight(efm_b200_vit* v, const char* hf_name, const void* data, const int64_t* shape,
                                   int32_t ndim, int32_t dtype, int32_t mem_kind) {
    if (v == nullptr || hf_name == nullptr || data == nullptr || shape == nullptr) return vfail(v, EFM_ERR_INVALID_ARGUMENT, "null argument");
    if (v->finalized) return vfail(v, EFM_ERR_STATE, "vision weights are already finalized");
    const std::string name(hf_name);
    if (dtype != EFM_BF16) return vfail(v, EFM_ERR_UNSUPPORTED, "weights must be bf16: " + name);
    efm_b200_ctx* c = v->ctx;
    VIT_CK(v, cudaSetDevice(c->device));
    const cudaMemcpyKind kind = mem_kind == EFM_MEM_DEVICE ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice;
    const efm_vit_desc& d = v->d;
    const int64_t H = d.hidden, I = d.intermediate, Ip = v->ipad, M = v->merged;
    auto bad_shape = [&]() { return vfail(v, EFM_ERR_INVALID_ARGUMENT, "unexpected shape for " + name); };
    auto flat = [&](void* dst, size_t elems) -> efm_status {
        VIT_CK(v, cudaMemcpyAsync(dst, data, elems * 2, kind, c->stream));
        return EFM_OK;
    };
    const std::string pre = "visual.";
    if (name.compare(0, pre.size(), pre) != 0) return vfail(v, EFM_ERR_INVALID_ARGUMENT, "not a vision tensor: " + name);
    const std::string n = name.substr(pre.size());
    efm_status st = EFM_OK;
    if (n == "patch_embed.proj.weight") {
        if (!is_shape(shape, ndim, {H, d.in_channels, d.temporal_patch, d.patch, d.patch}) && !is_shape(shape, ndim, {H, v->patch_dim})) return bad_shape();
        st = flat(v->patch_w, (size_t)H * v->patch_dim);
        v->seen |= gPatch;
    } else if (n == "merger.ln_q.weight") {
        if (!is_shape(shape, ndim, {H})) return bad_shape();
        st = flat(v->ln_q, H);
        v->seen |= gLnQ;
    } else if (n == "merger.mlp.0.weight") {
        if (!is_shape(shape, ndim, {M, M})) return bad_shape();
        st = flat(v->m0_w, (size_t)M * M);
        v->seen |= gM0W;
    } else if (n == "merger.mlp.0.bias") {
        if (!is_shape(shape, ndim, {M})) return bad_shape();
        st = flat(v->m0_b, M);
        v->seen |= gM0B;
    } else if (n == "merger.mlp.2.weight") {
        if (!is_shape(shape, ndim, {d.out_hidden, M})) return bad_shape();
        st = flat(v->m2_w, (size_t)d.out_hidden * M);
        v->seen |= gM2W;
    } else if (n == "merger.mlp.2.bias") {
        if (!is_shape(shape, ndim, {d.out_hidden})) return bad_shape();
        st = flat(v->m2_b, d.out_hidden);
        v->seen |= gM2B;
    } else if (n.compare(0, 7, "blocks.") == 0) {
        const size_t dot = n.find('.', 7);
        if (dot == std::string::npos) return vfail(v, EFM_ERR_INVALID_ARGUMENT, "unknown vision tensor: " + name);
        int l = -1;
        try { l = std::stoi(n.substr(7, dot - 7)); } catch (...) { l = -1; }
        if (l < 0 || l >= d.depth) return vfail(v, EFM_ERR_INVALID_ARGUMENT, "block index out of range: " + name);
        VitBlock& b = v->blocks[l];
        const std::string leaf = n.substr(dot + 1);
        // gate / up rows interleaved in blocks of 64: fused rows [128 j, 128 j + 64) = gate rows [64 j, 64 j + 64),
        // the next 64 = the same up rows; rows past I stay zero
        auto interleave = [&](__nv_bfloat16* dst, int64_t width, int which) -> efm_status {
            const char* src = static_cast<const char*>(data);
            for (int64_t j = 0; j * 64 < I; ++j) {
                const int64_t rows = std::min<int64_t>(64, I - j * 64);
                VIT_CK(v, cudaMemcpyAsync(dst + ((size_t)j * 128 + which * 64) * width, src + (size_t)j * 64 * width * 2,
                                          (size_t)rows * width * 2, kind, c->stream));
            }
            return EFM_OK;
        };
        if (leaf == "norm1.weight") { if (!is_shape(shape, ndim, {H})) return bad_shape(); st = flat(b.norm1, H); b.seen |= vN1; }
        else if (leaf == "norm2.weight") { if (!is_shape(shape, ndim, {H})) return bad_shape(); st = flat(b.norm2, H); b.seen |= vN2; }
        else if (leaf == "attn.qkv.weight") { if (!is_shape(shape, ndim, {3 * H, H})) return bad_shape(); st = flat(b.qkv_w, (size_t)3 * H * H); b.seen |= vQkvW; }
        else if (leaf == "attn.qkv.bias") { if (!is_shape(shape, ndim, {3 * H})) return bad_shape(); st = flat(b.qkv_b, 3 * H); b.seen |= vQkvB; }
        else if (leaf == "attn.proj.weight") { if (!is_shape(shape, ndim, {H, H})) return bad_shape(); st = flat(b.proj_w, (size_t)H * H); b.seen |= vProjW; }
        else if (leaf == "attn.proj.bias") { if (!is_shape(shape, ndim, {H})) return bad_shape(); st = flat(b.proj_b, H); b.seen |= vProjB; }
        else if (leaf == "mlp.gate_proj.weight") { if (!is_shape(shape, ndim, {I, H})) return bad_shape(); st = interleave(b.gate_up_w, H, 0); b.seen |= vGateW; }
        else if (leaf == "mlp.up_proj.weight") { if (!is_shape(shape, ndim, {I, H})) return bad_shape(); st = interleave(b.gate_up_w, H, 1); b.seen |= vUpW; }
        else if (leaf == "mlp.gate_proj.bias") { if (!is_shape(shape, ndim, {I})) return bad_shape(); st = interleave(b.gate_up_b, 1, 0); b.seen |= vGateB; }
        else if (leaf == "mlp.up_proj.bias") { if (!is_shape(shape, ndim, {I})) return bad_shape(); st = interleave(b.gate_up_b, 1, 1); b.seen |= vUpB; }
        else if (leaf == "mlp.down_proj.weight") {
            if (!is_shape(shape, ndim, {H, I})) return bad_shape();
            VIT_CK(v, cudaMemcpy2DAsync(b.down_w, (size_t)Ip * 2, data, (size_t)I * 2, (size_t)I * 2, (size_t)H, kind, c->stream));
            b.seen |= vDownW;
        }
        else if (leaf == "mlp.down_proj.bias") { if (!is_shape(shape, ndim, {H})) return bad_shape(); st = flat(b.down_b, H); b.seen |= vDownB; }
        else return vfail(v, EFM_ERR_INVALID_ARGUMENT, "unknown vision tensor: " + name);
    } else {
        return vfail(v, EFM_ERR_INVALID_ARGUMENT, "unknown vision tensor: " + name);
    }
    if (st != EFM_OK) return st;
    if (mem_kind == EFM_MEM_HOST) VIT_CK(v, cudaStreamSynchronize(c->stream));   // the caller may free its buffer
    return EFM_OK;
}

efm_status efm_b200_vit_finalize_weights(efm_b200_vit* v) {
    if (v == nullptr) return EFM_ERR_INVALID_ARGUMENT;
    if ((v->seen & gAll) != gAll) return vfail(v, EFM_ERR_STATE, "vision weights missing: patch embedding or merger tensors");
    for (size_t l = 0; l < v->blocks.size(); ++l)
        if ((v->blocks[l].seen & vAll) != vAll) return vfail(v, EFM_ERR_STATE, "vision weights missing in block " + std::to_string(l));
    VIT_CK(v, cudaStreamSynchronize(v->ctx->stream));
    v->finalized = true;
    return EFM_OK;
}

}  // extern "C"

extern "C" {

efm_status efm_b200_vit_plan(const efm_vit_desc* desc, const int32_t* grid_thw, int32_t n_grids, int32_t* order, int32_t* pos_h,
                             int32_t* pos_w, int32_t* win_lo, int32_t* win_hi, int32_t* full_lo, int32_t* full_hi) {
    if (desc == nullptr || grid_thw == nullptr || n_grids <= 0 || desc->struct_size != (int32_t)sizeof(efm_vit_desc) ||
        desc->merge <= 0 || desc->patch <= 0)
        return EFM_ERR_INVALID_ARGUMENT;
    Plan P;
    std::string why;
    if (!build_plan(*desc, grid_thw, n_grids, P, why)) return EFM_ERR_INVALID_ARGUMENT;
    auto put = [](int32_t* dst, const std::vector<int32_t>& src) {
        if (dst != nullptr) std::memcpy(dst, src.data(), src.size() * sizeof(int32_t));
    };
    put(order, P.order); put(pos_h, P.pos_h); put(pos_w, P.pos_w);
    put(win_lo, P.lo_win); put(win_hi, P.hi_win); put(full_lo, P.lo_full); put(full_hi, P.hi_full);
    return EFM_OK;
}

efm_status efm_b200_vit_encode(efm_b200_vit* v, const void* pixels, int32_t pixels_mem, const int32_t* grid_thw,
                               int32_t n_grids, void* out, int32_t out_mem) {
    if (v == nullptr || pixels == nullptr || grid_thw == nullptr || out == nullptr || n_grids <= 0)
        return vfail(v, EFM_ERR_INVALID_ARGUMENT, "null argument");
    if (!v->finalized) return vfail(v, EFM_ERR_STATE, "vision weights are not finalized");
    efm_b200_ctx* c = v->ctx;
    const efm_vit_desc& d = v->d;
    Plan P;
    std::string why;
    if (!build_plan(d, grid_thw, n_grids, P, why)) return vfail(v, EFM_ERR_INVALID_ARGUMENT, why);
    const int N = (int)P.pos_h.size(), NM = N / v->unit;
    if (N > d.max_patches) return vfail(v, EFM_ERR_INVALID_ARGUMENT, "more patches than max_patches");
    VIT_CK(v, cudaSetDevice(c->device));
    cudaStream_t st = c->stream;
    const int H = d.hidden, D = v->head_dim, Ip = v->ipad;

    // Tensor parallel: the permuted rows are cut at window boundaries into one contiguous share per rank.  The
    // windowed layers then run on the local rows alone; the full-attention layers all-gather the q|k|v rows, and
    // the merged tokens are all-gathered once at the end (every rank ends with the whole output).
    int tp = c->tp_size > 1 && c->nccl_comm != nullptr && std::getenv("EFM_B200_VIT_REPLICATED") == nullptr ? c->tp_size : 1;
    std::vector<int> cut(1, 0);
    if (tp > 1) {
        std::vector<int> bounds;                                   // first row of every window, then N
        for (int i = 0; i < N; ++i)
            if (P.lo_win[i] == i) bounds.push_back(i);
        bounds.push_back(N);
        if ((int)bounds.size() - 1 < tp) tp = 1;                   // fewer windows than ranks: everybody encodes everything
        for (int r = 1; r < tp; ++r) {                             // the window boundary nearest to an even split
            const long long target = (long long)N * r / tp;
            int best = cut.back();
            for (int bnd : bounds)
                if (bnd >= cut.back() && std::llabs(bnd - target) < std::llabs(best - target)) best = bnd;
            cut.push_back(best);
        }
    }
    cut.push_back(N);
    const int rank = tp > 1 ? c->tp_rank : 0;
    const int r0 = cut[rank], n = cut[rank + 1] - r0, nm = n / v->unit;       // this rank's rows
    if (tp > 1 && v->qkv_all == nullptr) {
        VIT_CK(v, valloc(v, &v->qkv_all, (size_t)d.max_patches * 3 * H));
        VIT_CK(v, valloc(v, &v->mo_all, (size_t)(d.max_patches / v->unit) * d.out_hidden));
    }

    // plan and pixels to the device; the windowed ranges are made relative to the local rows
    std::vector<int32_t> lw(P.lo_win.begin() + r0, P.lo_win.begin() + r0 + n), hw(P.hi_win.begin() + r0, P.hi_win.begin() + r0 + n);
    for (int i = 0; i < n; ++i) { lw[i] -= r0; hw[i] -= r0; }
    int32_t* order = v->plan;
    int32_t* pos_h = order + NM;
    int32_t *pos_w = pos_h + N, *lo_win = pos_w + N, *hi_win = lo_win + N, *lo_full = hi_win + N, *hi_full = lo_full + N;
    const std::vector<int32_t>* host[7] = {&P.order, &P.pos_h, &P.pos_w, &lw, &hw, &P.lo_full, &P.hi_full};
    int32_t* dev[7] = {order, pos_h, pos_w, lo_win, hi_win, lo_full, hi_full};
    for (int i = 0; i < 7; ++i)
        if (!host[i]->empty())
            VIT_CK(v, cudaMemcpyAsync(dev[i], host[i]->data(), host[i]->size() * 4, cudaMemcpyHostToDevice, st));
    const __nv_bfloat16* px = static_cast<const __nv_bfloat16*>(pixels);
    if (pixels_mem == EFM_MEM_HOST) {
        VIT_CK(v, cudaMemcpyAsync(v->pixels, pixels, (size_t)N * v->patch_dim * 2, cudaMemcpyHostToDevice, st));
        px = v->pixels;
    }
    // pageable host vectors: the copies above were staged before returning, but keep the plan alive
    // until the stream has consumed it
    VIT_CK(v, cudaStreamSynchronize(st));

    Launcher L;
    L.stream = st;
    L.pdl = false;
    L.counter = &c->launches;
    L.gemm_ws = c->gemm_ws;
    L.gemm_ws_floats = c->gemm_ws_floats;
    L.num_sms = c->num_sms;
    int* err = &c->state->error;
    auto norm_rows = [&](const __nv_bfloat16* w) { if (n > 0) launch_rmsnorm_rows(L, v->resid, w, v->xn, n, H, d.rms_eps); };
    auto gather_v = [&](const void* send, void* recv, size_t row_bytes, int per) {      // rows cut[r]/per .. cut[r+1]/per of every rank
        size_t off[8], cnt[8];
        for (int r = 0; r < tp; ++r) { off[r] = (size_t)(cut[r] / per) * row_bytes; cnt[r] = (size_t)((cut[r + 1] - cut[r]) / per) * row_bytes; }
        if (L.err != cudaSuccess) return;
        const NcclApi& api = nccl_api();
        if (!api.ok || api.all_gather_v_bytes(send, recv, off, cnt, tp, c->nccl_comm, st) != 0) L.err = cudaErrorUnknown;
        else ++c->launches;
    };

    {   // patch embedding (all rows: 1 % of the flops), then this rank's rows in window-major order
        GemmParams g{px, v->patch_w, nullptr, nullptr, v->pe, N, H, v->patch_dim};
        launch_gemm_epi(L, GemmEpi::F32, g, err);
        if (nm > 0)
            L.launch(vit_gather_blocks_f32_kernel, dim3(std::min(nm, c->num_sms * 8)), dim3(256), 0, (const float*)v->pe, v->resid,
                     (const int32_t*)(order + r0 / v->unit), nm, v->unit, H);
    }
    if (n > 0)
        L.launch(vit_rope_table_kernel, dim3((n * (D / 2) + 127) / 128), dim3(128), 0, v->rope_tab, (const int32_t*)(pos_h + r0),
                 (const int32_t*)(pos_w + r0), n, D, d.rope_theta);
    for (int l = 0; l < d.depth; ++l) {
        const VitBlock& b = v->blocks[l];
        bool full = false;
        for (int i = 0; i < d.n_fullatt; ++i) full = full || d.fullatt[i] == l;
        norm_rows(b.norm1);
        if (n > 0) {
            GemmParams g{v->xn, b.qkv_w, b.qkv_b, v->qkv, nullptr, n, 3 * H, H};
            launch_gemm_epi(L, GemmEpi::Bf16Bias, g, err);
            L.launch(vit_rope2d_kernel, dim3(n), dim3(256), 0, v->qkv, (const float2*)v->rope_tab, d.heads, D);
        }
        const __nv_bfloat16* kv_rows = v->qkv;
        if (full && tp > 1) {
            gather_v(v->qkv, v->qkv_all, (size_t)3 * H * 2, 1);
            kv_rows = v->qkv_all;
        }
        if (n > 0) {
            SegAttnParams a{};
            a.q = v->qkv; a.k = kv_rows + H; a.v = kv_rows + 2 * H; a.out = v->attn;
            // windowed ranges are relative to the local rows; full ranges index the gathered (global) rows
            a.lo = full ? lo_full + (tp > 1 ? r0 : 0) : lo_win;
            a.hi = full ? hi_full + (tp > 1 ? r0 : 0) : hi_win;
            a.q_stride = a.kv_stride = 3 * H; a.out_stride = H;
            a.S = n; a.kv_offset = 0; a.q_heads = a.kv_heads = d.heads;
            a.scale = 1.0f / sqrtf((float)D);
            a.kv_rows = full && tp > 1 ? N : n;          // rows behind k / v: the gathered rows of every rank, or the local ones
            a.error = err;
            launch_seg_attention(L, a, D);
            GemmParams g{v->attn, b.proj_w, b.proj_b, nullptr, v->resid, n, H, H};
            launch_gemm_epi(L, GemmEpi::Residual, g, err);
        }
        norm_rows(b.norm2);
        if (n > 0) {
            GemmParams g{v->xn, b.gate_up_w, b.gate_up_b, v->act, nullptr, n, 2 * Ip, H};
            launch_gemm_epi(L, GemmEpi::SwiGlu, g, err);
            GemmParams g2{v->act, b.down_w, b.down_b, nullptr, v->resid, n, H, Ip};
            launch_gemm_epi(L, GemmEpi::Residual, g2, err);
        }
    }
    {   // merger: norm, 4 rows -> one, MLP with exact GELU, back to the original token order
        norm_rows(v->ln_q);
        if (nm > 0) {
            GemmParams g0{v->xn, v->m0_w, v->m0_b, v->h1, nullptr, nm, v->merged, v->merged};
            launch_gemm_epi(L, GemmEpi::Bf16Gelu, g0, err);
            GemmParams g1{v->h1, v->m2_w, v->m2_b, v->mo, nullptr, nm, d.out_hidden, v->merged};
            launch_gemm_epi(L, GemmEpi::Bf16Bias, g1, err);
        }
        const __nv_bfloat16* merged = v->mo;
        if (tp > 1) {
            gather_v(v->mo, v->mo_all, (size_t)d.out_hidden * 2, v->unit);
            merged = v->mo_all;
        }
        __nv_bfloat16* dst = out_mem == EFM_MEM_DEVICE ? static_cast<__nv_bfloat16*>(out) : v->out_dev;
        L.launch(vit_scatter_rows_bf16_kernel, dim3(std::min(NM, c->num_sms * 8)), dim3(128), 0, merged, dst,
                 (const int32_t*)order, NM, d.out_hidden);
    }
    if (L.err != cudaSuccess) return vfail(v, EFM_ERR_CUDA, std::string("vision encoder launch: ") + cudaGetErrorString(L.err));
    if (out_mem == EFM_MEM_HOST) {
        VIT_CK(v, cudaMemcpyAsync(out, v->out_dev, (size_t)NM * d.out_hidden * 2, cudaMemcpyDeviceToHost, st));
        int flag = 0;
        VIT_CK(v, cudaMemcpyAsync(&flag, err, 4, cudaMemcpyDeviceToHost, st));
        VIT_CK(v, cudaStreamSynchronize(st));
        if (flag != 0) {
            cudaMemsetAsync(err, 0, 4, st);
            return vfail(v, EFM_ERR_DEVICE_WAIT, "a GEMM pipeline wait gave up inside the vision encoder");
        }
    }
    return EFM_OK;
}

efm_status efm_b200_op_segment_attention(const void* q, const void* k, const void* vv, void* out_bf16, const int32_t* lo,
                                         const int32_t* hi, int32_t s, int32_t heads, int32_t head_dim, int32_t stride) {
    if (q == nullptr || k == nullptr || vv == nullptr || out_bf16 == nullptr || lo == nullptr || hi == nullptr || s <= 0 || heads <= 0)
        return EFM_ERR_INVALID_ARGUMENT;
    if (head_dim != 64 && head_dim != 80 && head_dim != 128) return EFM_ERR_UNSUPPORTED;
    if (stride % 8 != 0 || stride < heads * head_dim) return EFM_ERR_INVALID_ARGUMENT;
    Launcher L;
    L.pdl = false;
    SegAttnParams a{};
    a.q = static_cast<const __nv_bfloat16*>(q);
    a.k = static_cast<const __nv_bfloat16*>(k);
    a.v = static_cast<const __nv_bfloat16*>(vv);
    a.out = static_cast<__nv_bfloat16*>(out_bf16);
    a.lo = lo; a.hi = hi;
    a.q_stride = a.kv_stride = stride; a.out_stride = heads * head_dim;
    a.S = s; a.q_heads = a.kv_heads = heads;
    a.scale = 1.0f / sqrtf((float)head_dim);
    a.kv_rows = s;                                   // q, k, v are rows of one buffer
    launch_seg_attention(L, a, head_dim);
    cudaError_t e = L.err != cudaSuccess ? L.err : cudaStreamSynchronize(nullptr);
    return e == cudaSuccess ? EFM_OK : EFM_ERR_CUDA;
}

}  // extern "C"
