// Implementation of the C ABI declared in include/efm_b200.h: context lifetime, weight
// ingestion (fusing q|k|v and interleaving gate/up as the kernels expect), KV slots, the
// prefill and decode entry points with CUDA-graph capture of the decode step, and the
// single-operator entry points used by the parity tests.
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <cmath>
#include <new>
#include <string>

#include "../../layers/launch.cuh"
#include "../../layers/qwen_text.h"
#include "../../operators/gemm_tc.cuh"
#define EFM_DECLARATIONS_ONLY
#include "../../operators/sample.cuh"
#undef EFM_DECLARATIONS_ONLY
#include "ctx.h"
#include "nccl_glue.h"

using namespace efm;

namespace {

thread_local std::string g_create_error;

efm_status fail(efm_b200_ctx* c, efm_status st, const std::string& msg) {
    if (c != nullptr) c->error = msg; else g_create_error = msg;
    return st;
}
efm_status cuda_fail(efm_b200_ctx* c, cudaError_t e, const char* what) {
    const efm_status st = e == cudaErrorMemoryAllocation ? EFM_ERR_OUT_OF_MEMORY : EFM_ERR_CUDA;
    return fail(c, st, std::string(what) + ": " + cudaGetErrorString(e));
}
#define EFM_CK(ctx, call)                                              \
    do {                                                               \
        cudaError_t e_ = (call);                                       \
        if (e_ != cudaSuccess) return cuda_fail(ctx, e_, #call);       \
    } while (0)

template <typename T>
cudaError_t dev_alloc(efm_b200_ctx* c, T** p, size_t count, bool zero = true) {
    void* raw = nullptr;
    const size_t bytes = std::max<size_t>(count * sizeof(T), 16);
    cudaError_t e = cudaMalloc(&raw, bytes);
    if (e != cudaSuccess) return e;
    c->allocations.push_back(raw);
    if (zero) e = cudaMemsetAsync(raw, 0, bytes, c->stream);
    *p = static_cast<T*>(raw);
    return e;
}

// a usable sm_100 device, or an error: there is no CPU path behind this library
efm_status require_b200(efm_b200_ctx* c, int device_id) {
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0)
        return fail(c, EFM_ERR_CUDA, std::string("no CUDA device available: ") + cudaGetErrorString(e));
    if (device_id < 0 || device_id >= n) return fail(c, EFM_ERR_INVALID_ARGUMENT, "device_id out of range");
    int major = 0;
    EFM_CK(c, cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device_id));
    if (major != 10) return fail(c, EFM_ERR_CUDA, "device is not sm_100 (this library carries sm_100a code only)");
    EFM_CK(c, cudaSetDevice(device_id));
    EFM_CK(c, configure_decode_attention());
    EFM_CK(c, configure_sampler());
    {
        int optin = 0;
        EFM_CK(c, cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device_id));
        EFM_CK(c, configure_gemv(optin - 2048));        // leave room for the kernels' static shared memory
    }
    return EFM_OK;
}

Launcher make_launcher(efm_b200_ctx* c) {
    Launcher L;
    L.stream = c->stream;
    L.pdl = c->pdl;
    L.counter = &c->launches;
    L.gemm_ws = c->gemm_ws;
    L.gemm_ws_floats = c->gemm_ws_floats;
    L.num_sms = c->num_sms;
    return L;
}

// Stream synchronisation of a context.  Tensor-parallel contexts do not block inside the driver: they poll the stream
// and NCCL's asynchronous error state, and give up after tp_timeout_s (the communicator is then aborted and gone).
int stream_ready(void* stream) { return cudaStreamQuery(static_cast<cudaStream_t>(stream)) != cudaErrorNotReady; }
efm_status ctx_sync(efm_b200_ctx* c) {
    if (c->tp_size > 1 && c->nccl_comm != nullptr) {
        std::string what;
        const int r = tp_host_wait(c->nccl_comm, stream_ready, c->stream, c->tp_timeout_s, &what);
        if (r != 0) {
            c->nccl_comm = nullptr;       // aborted
            return fail(c, r == 2 ? EFM_ERR_DEVICE_WAIT : EFM_ERR_CUDA, what);
        }
    }
    cudaError_t e = cudaStreamSynchronize(c->stream);
    if (e != cudaSuccess) return cuda_fail(c, e, "cudaStreamSynchronize");
    return EFM_OK;
}

constexpr size_t kMaxPrefillGraphs = 8;
void drop_prefill_graphs(efm_b200_ctx* c) {
    for (auto& g : c->prefill_cache)
        if (g.exec != nullptr) cudaGraphExecDestroy(g.exec);
    c->prefill_cache.clear();
}

enum : uint32_t { kQw = 1, kQb = 2, kKw = 4, kKb = 8, kVw = 16, kVb = 32, kO = 64, kGate = 128, kUp = 256,
                  kDown = 512, kInNorm = 1024, kPostNorm = 2048 };
constexpr uint32_t kRequired = kQw | kKw | kVw | kO | kGate | kUp | kDown | kInNorm | kPostNorm;

efm_status copy_rows(efm_b200_ctx* c, void* dst, const void* src, size_t bytes, int mem_kind) {
    EFM_CK(c, cudaMemcpyAsync(dst, src, bytes, mem_kind == EFM_MEM_DEVICE ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, c->stream));
    return EFM_OK;
}

bool shape_is(const int64_t* shape, int ndim, int64_t a, int64_t b = -1) {
    if (b < 0) return ndim == 1 && shape[0] == a;
    return ndim == 2 && shape[0] == a && shape[1] == b;
}

}  // namespace

extern "C" {

const char* efm_b200_version(void) { return "efm_b200 0.1 (sm_100a)"; }

const char* efm_b200_last_error(const efm_b200_ctx* ctx) {
    return ctx != nullptr ? ctx->error.c_str() : g_create_error.c_str();
}

efm_status efm_b200_create(const efm_model_desc* desc, int32_t device_id, int32_t tp_rank, int32_t tp_size,
                           efm_b200_ctx** out) {
    if (desc == nullptr || out == nullptr) return fail(nullptr, EFM_ERR_INVALID_ARGUMENT, "null argument");
    *out = nullptr;
    if (desc->struct_size != (int32_t)sizeof(efm_model_desc))
        return fail(nullptr, EFM_ERR_INVALID_ARGUMENT, "efm_model_desc.struct_size mismatch");
    const efm_model_desc& d = *desc;
    if (d.num_layers <= 0 || d.hidden <= 0 || d.q_heads <= 0 || d.kv_heads <= 0 || d.vocab <= 0 || d.intermediate <= 0)
        return fail(nullptr, EFM_ERR_INVALID_ARGUMENT, "non-positive model dimension");
    if (d.head_dim != 64 && d.head_dim != 128) return fail(nullptr, EFM_ERR_UNSUPPORTED, "head_dim must be 64 or 128");
    if (d.q_heads % d.kv_heads != 0 || d.q_heads / d.kv_heads > kMaxGroup)
        return fail(nullptr, EFM_ERR_UNSUPPORTED, "q_heads / kv_heads must be an integer <= 8");
    if (d.hidden % 32 != 0 || d.intermediate % 64 != 0 || d.vocab % 2 != 0)
        return fail(nullptr, EFM_ERR_UNSUPPORTED, "hidden % 32, intermediate % 64 and vocab % 2 must be 0");
    if (d.use_mrope && d.mrope_section[0] + d.mrope_section[1] + d.mrope_section[2] != d.head_dim / 2)
        return fail(nullptr, EFM_ERR_INVALID_ARGUMENT, "mrope_section must sum to head_dim / 2");
    if (tp_size < 1 || tp_rank < 0 || tp_rank >= tp_size) return fail(nullptr, EFM_ERR_INVALID_ARGUMENT, "bad tensor-parallel coordinates");
    // heads are sharded min(tp, kv_heads) ways; beyond that, ranks pair up on a head shard and split o_proj's input
    const int att_shards = std::min(tp_size, d.kv_heads);
    if (tp_size % att_shards != 0 || d.kv_heads % att_shards != 0 || d.q_heads % att_shards != 0)
        return fail(nullptr, EFM_ERR_UNSUPPORTED, "tensor-parallel size must divide (or be a multiple of) the kv head count");
    const int att_rep = tp_size / att_shards;
    if (d.intermediate % (64 * tp_size) != 0 || d.vocab % (2 * tp_size) != 0 ||
        ((d.q_heads / att_shards) * d.head_dim) % (32 * att_rep) != 0)
        return fail(nullptr, EFM_ERR_UNSUPPORTED, "intermediate / vocab / attention width do not split evenly over the ranks");
    if (d.max_prefill_tokens <= 0 || d.max_response_tokens <= 0)
        return fail(nullptr, EFM_ERR_INVALID_ARGUMENT, "max_prefill_tokens and max_response_tokens must be positive");
    efm_status st = require_b200(nullptr, device_id);
    if (st != EFM_OK) return st;

    efm_b200_ctx* c = new (std::nothrow) efm_b200_ctx();
    if (c == nullptr) return fail(nullptr, EFM_ERR_OUT_OF_MEMORY, "host allocation failed");
    c->full = d;
    c->d = d;
    c->d.q_heads = d.q_heads / att_shards;
    c->d.kv_heads = d.kv_heads / att_shards;
    c->d.intermediate = d.intermediate / tp_size;
    c->att_shards = att_shards;
    c->att_rep = att_rep;
    c->att_shard = tp_rank / att_rep;
    c->att_rep_idx = tp_rank % att_rep;
    c->o_k = c->d.q_heads * d.head_dim / att_rep;
    c->vocab_l = d.vocab / tp_size;
    c->vocab_off = tp_rank * c->vocab_l;
    c->device = device_id;
    c->tp_rank = tp_rank;
    c->tp_size = tp_size;
    c->pdl = std::getenv("EFM_B200_NO_PDL") == nullptr;
    auto bail = [&](cudaError_t e, const char* what) {
        efm_status s = cuda_fail(nullptr, e, what);
        efm_b200_destroy(c);
        return s;
    };
#define EFM_TRY(call) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) return bail(e_, #call); } while (0)
    EFM_TRY(cudaDeviceGetAttribute(&c->num_sms, cudaDevAttrMultiProcessorCount, device_id));
    EFM_TRY(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
    for (auto& ev : c->events) EFM_TRY(cudaEventCreate(&ev));

    const efm_model_desc& dl = c->d;
    const size_t H = dl.hidden, D = dl.head_dim, QD = (size_t)dl.q_heads * D, KVD = (size_t)dl.kv_heads * D, I = dl.intermediate,
                 V = dl.vocab, S = dl.max_prefill_tokens;
    EFM_TRY(dev_alloc(c, &c->embed, V * H, false));
    if (d.tied_lm_head) c->lm_head = c->embed + (size_t)c->vocab_off * H;      // this rank's rows of the shared table
    else EFM_TRY(dev_alloc(c, &c->lm_head, (size_t)c->vocab_l * H, false));
    if (tp_size > 1) {
        EFM_TRY(dev_alloc(c, &c->ybuf, S * H));
        EFM_TRY(dev_alloc(c, &c->ysum, S * H));
        EFM_TRY(dev_alloc(c, &c->logits_l, (size_t)c->vocab_l));
        // zeroed: header (counts, tickets, prefill flags) | decode {value, count} words | prefill receive slots | gather buffers
        c->tp_prefill_off = 256 + (((size_t)2 * tp_size * H * 8 + 255) & ~(size_t)255);
        c->tp_slot_floats = ((S + tp_size - 1) / tp_size) * H;
        c->tp_gather_off = c->tp_prefill_off + (((size_t)2 * tp_size * c->tp_slot_floats * sizeof(float) + 255) & ~(size_t)255);
        c->tp_sample_off = c->tp_gather_off + (((size_t)2 * S * H * sizeof(float) + 255) & ~(size_t)255);
        EFM_TRY(dev_alloc(c, &c->tp_xchg, c->tp_sample_off + 256));
        EFM_TRY(cudaHostAlloc(reinterpret_cast<void**>(&c->error_host), sizeof(int), cudaHostAllocMapped));
        *c->error_host = 0;
        if (const char* ms = std::getenv("EFM_B200_PEER_WAIT_MS")) {
            const long v = std::atol(ms);
            if (v > 0) c->peer_wait_ns = (unsigned long long)v * 1000000ull;
        }
        if (const char* ts = std::getenv("EFM_B200_TP_TIMEOUT_S")) {
            const double v = std::atof(ts);
            if (v > 0) c->tp_timeout_s = v;
        }
    }
    EFM_TRY(dev_alloc(c, &c->final_norm, H));
    c->layers.resize(d.num_layers);
    for (auto& w : c->layers) {
        EFM_TRY(dev_alloc(c, &w.in_norm, H));
        EFM_TRY(dev_alloc(c, &w.post_norm, H));
        EFM_TRY(dev_alloc(c, &w.qkv, (QD + 2 * KVD) * H, false));
        EFM_TRY(dev_alloc(c, &w.qkv_bias, QD + 2 * KVD));
        EFM_TRY(dev_alloc(c, &w.o, H * (size_t)c->o_k, false));
        EFM_TRY(dev_alloc(c, &w.gate_up, 2 * I * H, false));
        EFM_TRY(dev_alloc(c, &w.down, H * I, false));
    }
    {
        std::vector<float> f(D / 2);
        for (size_t i = 0; i < D / 2; ++i) f[i] = (float)std::pow((double)d.rope_theta, -2.0 * (double)i / (double)D);
        EFM_TRY(dev_alloc(c, &c->inv_freq, D / 2));
        EFM_TRY(cudaMemcpyAsync(c->inv_freq, f.data(), f.size() * sizeof(float), cudaMemcpyHostToDevice, c->stream));
        EFM_TRY(cudaStreamSynchronize(c->stream));
    }
    c->max_s = (int)S;
    EFM_TRY(dev_alloc(c, &c->ids, S));
    EFM_TRY(dev_alloc(c, &c->pos3, 3 * S));
    EFM_TRY(dev_alloc(c, &c->resid, S * H));
    EFM_TRY(dev_alloc(c, &c->norm, S * H));
    EFM_TRY(dev_alloc(c, &c->qkv, S * (QD + 2 * KVD)));
    EFM_TRY(dev_alloc(c, &c->qbuf, S * QD));
    EFM_TRY(dev_alloc(c, &c->attn, S * QD));
    EFM_TRY(dev_alloc(c, &c->act, S * I));
    EFM_TRY(dev_alloc(c, &c->resid_d, H));
    EFM_TRY(dev_alloc(c, &c->resid_d2, H));
    EFM_TRY(dev_alloc(c, &c->q_d, QD));
    EFM_TRY(dev_alloc(c, &c->attn_d, QD));
    EFM_TRY(dev_alloc(c, &c->act_d, I));
    EFM_TRY(dev_alloc(c, &c->logits, V));
    EFM_TRY(dev_alloc(c, &c->part_val, 2 * (size_t)c->num_sms + 8));
    EFM_TRY(dev_alloc(c, &c->part_idx, 2 * (size_t)c->num_sms + 8));
    EFM_TRY(dev_alloc(c, &c->wbuf, sample_scratch_words((int)V)));
    EFM_TRY(dev_alloc(c, &c->attn_part_o, (size_t)dl.q_heads * 64 * D));
    EFM_TRY(dev_alloc(c, &c->attn_part_ml, (size_t)dl.q_heads * 64 * 2));
    EFM_TRY(dev_alloc(c, &c->attn_counters, (size_t)dl.kv_heads));
    {   // the longest GEMV input row must fit the kernel's shared memory as fp32
        int optin = 0;
        EFM_TRY(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device_id));
        const size_t need = gemv_w4_smem_bytes((int)std::max(H, std::max(QD, I)));
        if (need + 2048 > (size_t)optin) {
            efm_status s = fail(nullptr, EFM_ERR_UNSUPPORTED, "hidden / intermediate size exceeds what the decode GEMV stages in shared memory");
            efm_b200_destroy(c);
            return s;
        }
    }
    c->gemm_ws_floats = (size_t)c->num_sms * 128 * 256;      // splits x tiles never exceeds the SM count
    EFM_TRY(dev_alloc(c, &c->gemm_ws, c->gemm_ws_floats, false));
    EFM_TRY(dev_alloc(c, &c->state, 1));
    EFM_TRY(dev_alloc(c, &c->tokens_out, (size_t)d.max_response_tokens));
    EFM_TRY(cudaStreamSynchronize(c->stream));
#undef EFM_TRY
    *out = c;
    return EFM_OK;
}

efm_status efm_b200_destroy(efm_b200_ctx* c) {
    if (c == nullptr) return EFM_OK;
    cudaSetDevice(c->device);
    if (c->stream != nullptr) cudaStreamSynchronize(c->stream);
    for (auto& kv : c->slots)      // graphs that hold collective nodes go before their communicator
        if (kv.second.graph != nullptr) cudaGraphExecDestroy(kv.second.graph);
    drop_prefill_graphs(c);
    for (int r = 0; r < 8; ++r)
        if (c->peers_ready && r != c->tp_rank && c->peer_base[r] != nullptr) cudaIpcCloseMemHandle(c->peer_base[r]);
    if (c->nccl_comm != nullptr && nccl_api().ok) nccl_api().comm_destroy(c->nccl_comm);
    if (c->sage.q8 != nullptr) { cudaFree(c->sage.q8); cudaFree(c->sage.k8); cudaFree(c->sage.vh); cudaFree(c->sage.sq); cudaFree(c->sage.sk); cudaFree(c->sage.kmean); }
    for (void* p : c->allocations) cudaFree(p);
    for (auto& ev : c->events)
        if (ev != nullptr) cudaEventDestroy(ev);
    if (c->stream != nullptr) cudaStreamDestroy(c->stream);
    if (c->error_host != nullptr) cudaFreeHost(c->error_host);
    delete c;
    return EFM_OK;
}

efm_status efm_b200_tp_unique_id(void* out128) {
    if (out128 == nullptr) return fail(nullptr, EFM_ERR_INVALID_ARGUMENT, "null argument");
    const NcclApi& api = nccl_api();
    if (!api.ok) return fail(nullptr, EFM_ERR_UNSUPPORTED, api.error);
    const int r = api.get_unique_id(out128);
    if (r != 0) return fail(nullptr, EFM_ERR_CUDA, std::string("ncclGetUniqueId: ") + api.error_string(r));
    return EFM_OK;
}

efm_status efm_b200_tp_init(efm_b200_ctx* c, const void* id128) {
    if (c == nullptr || id128 == nullptr) return fail(c, EFM_ERR_INVALID_ARGUMENT, "null argument");
    if (c->tp_size == 1) return EFM_OK;
    if (c->nccl_comm != nullptr) return fail(c, EFM_ERR_STATE, "communicator already initialised");
    const NcclApi& api = nccl_api();
    if (!api.ok) return fail(c, EFM_ERR_UNSUPPORTED, api.error);
    EFM_CK(c, cudaSetDevice(c->device));
    // In-switch (NVLS) collectives bind this rank's buffers to an NVLink multicast object; a rank that dies while bound
    // can fault its peers' GPUs.  Off unless the caller's environment already decided.
    setenv("NCCL_NVLS_ENABLE", "0", 0);
    const int r = api.comm_init_rank(&c->nccl_comm, c->tp_size, id128, c->tp_rank);
    if (r != 0) { c->nccl_comm = nullptr; return fail(c, EFM_ERR_CUDA, std::string("ncclCommInitRank: ") + api.error_string(r)); }
    return EFM_OK;
}

efm_status efm_b200_tp_set_wait_limit(efm_b200_ctx* c, int64_t device_wait_us, double host_timeout_s) {
    if (c == nullptr) return fail(c, EFM_ERR_INVALID_ARGUMENT, "null context");
    if (device_wait_us < 0 || host_timeout_s < 0) return fail(c, EFM_ERR_INVALID_ARGUMENT, "limits must be >= 0 (0 keeps the current value)");
    bool changed = false;
    if (device_wait_us > 0) { changed = c->peer_wait_ns != (unsigned long long)device_wait_us * 1000ull; c->peer_wait_ns = (unsigned long long)device_wait_us * 1000ull; }
    if (host_timeout_s > 0) c->tp_timeout_s = host_timeout_s;
    if (changed)     // the device limit is a kernel argument baked into the captured step
        for (auto& kv : c->slots)
            if (kv.second.graph != nullptr) { cudaGraphExecDestroy(kv.second.graph); kv.second.graph = nullptr; }
    return EFM_OK;
}

efm_status efm_b200_tp_host_wait(void* nccl_comm, int (*ready)(void*), void* arg, double timeout_s) {
    if (ready == nullptr || !(timeout_s >= 0)) return fail(nullptr, EFM_ERR_INVALID_ARGUMENT, "tp_host_wait: bad arguments");
    std::string what;
    const int r = tp_host_wait(nccl_comm, ready, arg, timeout_s, &what);
    if (r == 0) return EFM_OK;
    return fail(nullptr, r == 2 ? EFM_ERR_DEVICE_WAIT : EFM_ERR_CUDA, what);
}

efm_status efm_b200_tp_peer_export(efm_b200_ctx* c, void* handle64) {
    if (c == nullptr || handle64 == nullptr) return fail(c, EFM_ERR_INVALID_ARGUMENT, "null argument");
    if (c->tp_size == 1 || c->tp_xchg == nullptr) return fail(c, EFM_ERR_STATE, "peer exchange needs tp_size > 1");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    EFM_CK(c, cudaSetDevice(c->device));
    EFM_CK(c, cudaStreamSynchronize(c->stream));            // the buffer's zero fill has landed
    cudaIpcMemHandle_t h;
    EFM_CK(c, cudaIpcGetMemHandle(&h, c->tp_xchg));
    std::memcpy(handle64, &h, 64);
    return EFM_OK;
}

efm_status efm_b200_tp_peer_import(efm_b200_ctx* c, const void* handles, int32_t n_handles) {
    if (c == nullptr || handles == nullptr) return fail(c, EFM_ERR_INVALID_ARGUMENT, "null argument");
    if (c->tp_size == 1 || c->tp_xchg == nullptr) return fail(c, EFM_ERR_STATE, "peer exchange needs tp_size > 1");
    if (n_handles != c->tp_size || c->tp_size > 8) return fail(c, EFM_ERR_INVALID_ARGUMENT, "one handle per rank, at most 8 ranks");
    if (c->peers_ready) return fail(c, EFM_ERR_STATE, "peer buffers are already imported");
    EFM_CK(c, cudaSetDevice(c->device));
    for (int r = 0; r < c->tp_size; ++r) {
        if (r == c->tp_rank) { c->peer_base[r] = c->tp_xchg; continue; }
        cudaIpcMemHandle_t h;
        std::memcpy(&h, static_cast<const char*>(handles) + (size_t)r * 64, 64);
        void* p = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            for (int q = 0; q < r; ++q)
                if (q != c->tp_rank && c->peer_base[q] != nullptr) { cudaIpcCloseMemHandle(c->peer_base[q]); c->peer_base[q] = nullptr; }
            return cuda_fail(c, e, "cudaIpcOpenMemHandle (peer exchange buffer)");
        }
        c->peer_base[r] = static_cast<char*>(p);
    }
    for (auto& kv : c->slots)       // decode graphs captured with the NCCL form are rebuilt on next use
        if (kv.second.graph != nullptr) { cudaGraphExecDestroy(kv.second.graph); kv.second.graph = nullptr; }
    drop_prefill_graphs(c);
    c->peers_ready = true;
    return EFM_OK;
}

efm_status efm_b200_set_weight(efm_b200_ctx* c, const char* hf_name, const void* data, const int64_t* shape,
                               int32_t ndim, int32_t dtype, int32_t mem_kind) {
    if (c == nullptr || hf_name == nullptr || data == nullptr || shape == nullptr)
        return fail(c, EFM_ERR_INVALID_ARGUMENT, "null argument");
    if (c->finalized) return fail(c, EFM_ERR_STATE, "weights are already finalized");
    EFM_CK(c, cudaSetDevice(c->device));
    // The caller always hands over the WHOLE tensor; this rank keeps its slice: q/k/v rows of its head
    // shard, its o_proj input columns, its gate/up rows and down columns, its lm_head rows.
    const efm_model_desc& d = c->d;          // local
    const efm_model_desc& F = c->full;       // whole model
    const int64_t H = d.hidden, D = d.head_dim, I = d.intermediate, V = d.vocab;
    const int64_t QD = d.q_heads * D, KVD = d.kv_heads * D;              // local widths
    const int64_t FQD = F.q_heads * D, FKVD = F.kv_heads * D, FI = F.intermediate;
    const int64_t q_off = (int64_t)c->att_shard * QD, kv_off = (int64_t)c->att_shard * KVD, i_off = (int64_t)c->tp_rank * I;
    const std::string name(hf_name);
    const char* src = static_cast<const char*>(data);
    const cudaMemcpyKind kind = mem_kind == EFM_MEM_DEVICE ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice;
    auto bad_shape = [&]() { return fail(c, EFM_ERR_INVALID_ARGUMENT, "unexpected shape for " + name); };
    auto known = [&]() -> efm_status {
        if (dtype != EFM_BF16) return fail(c, EFM_ERR_UNSUPPORTED, "weights must be bf16: " + name);
        return EFM_OK;
    };
    efm_status st = EFM_OK;
    if (name == "model.embed_tokens.weight") {
        if ((st = known()) != EFM_OK) return st;
        if (!shape_is(shape, ndim, V, H)) return bad_shape();
        st = copy_rows(c, c->embed, data, (size_t)V * H * 2, mem_kind);
        c->seen_embed = true;
    } else if (name == "lm_head.weight") {
        if ((st = known()) != EFM_OK) return st;
        if (!shape_is(shape, ndim, V, H)) return bad_shape();
        if (!d.tied_lm_head) st = copy_rows(c, c->lm_head, src + (size_t)c->vocab_off * H * 2, (size_t)c->vocab_l * H * 2, mem_kind);
        c->seen_lm_head = true;
    } else if (name == "model.norm.weight") {
        if ((st = known()) != EFM_OK) return st;
        if (!shape_is(shape, ndim, H)) return bad_shape();
        st = copy_rows(c, c->final_norm, data, (size_t)H * 2, mem_kind);
        c->seen_final_norm = true;
    } else if (name.rfind("model.layers.", 0) == 0) {
        const size_t dot = name.find('.', 13);
        if (dot == std::string::npos) return EFM_OK;
        const int l = std::atoi(name.substr(13, dot - 13).c_str());
        if (l < 0 || l >= d.num_layers) return EFM_OK;      // e.g. extra layers of a draft model: ignored
        const std::string rest = name.substr(dot + 1);
        LayerWeights& w = c->layers[l];
        if ((st = known()) != EFM_OK) return st;
        const size_t rowb = (size_t)H * 2;
        if (rest == "input_layernorm.weight") {
            if (!shape_is(shape, ndim, H)) return bad_shape();
            st = copy_rows(c, w.in_norm, data, rowb, mem_kind); w.seen |= kInNorm;
        } else if (rest == "post_attention_layernorm.weight") {
            if (!shape_is(shape, ndim, H)) return bad_shape();
            st = copy_rows(c, w.post_norm, data, rowb, mem_kind); w.seen |= kPostNorm;
        } else if (rest == "self_attn.q_proj.weight") {
            if (!shape_is(shape, ndim, FQD, H)) return bad_shape();
            st = copy_rows(c, w.qkv, src + (size_t)q_off * rowb, (size_t)QD * rowb, mem_kind); w.seen |= kQw;
        } else if (rest == "self_attn.k_proj.weight") {
            if (!shape_is(shape, ndim, FKVD, H)) return bad_shape();
            st = copy_rows(c, w.qkv + QD * H, src + (size_t)kv_off * rowb, (size_t)KVD * rowb, mem_kind); w.seen |= kKw;
        } else if (rest == "self_attn.v_proj.weight") {
            if (!shape_is(shape, ndim, FKVD, H)) return bad_shape();
            st = copy_rows(c, w.qkv + (QD + KVD) * H, src + (size_t)kv_off * rowb, (size_t)KVD * rowb, mem_kind); w.seen |= kVw;
        } else if (rest == "self_attn.q_proj.bias") {
            if (!shape_is(shape, ndim, FQD)) return bad_shape();
            st = copy_rows(c, w.qkv_bias, src + (size_t)q_off * 2, (size_t)QD * 2, mem_kind); w.seen |= kQb;
        } else if (rest == "self_attn.k_proj.bias") {
            if (!shape_is(shape, ndim, FKVD)) return bad_shape();
            st = copy_rows(c, w.qkv_bias + QD, src + (size_t)kv_off * 2, (size_t)KVD * 2, mem_kind); w.seen |= kKb;
        } else if (rest == "self_attn.v_proj.bias") {
            if (!shape_is(shape, ndim, FKVD)) return bad_shape();
            st = copy_rows(c, w.qkv_bias + QD + KVD, src + (size_t)kv_off * 2, (size_t)KVD * 2, mem_kind); w.seen |= kVb;
        } else if (rest == "self_attn.o_proj.weight") {
            if (!shape_is(shape, ndim, H, FQD)) return bad_shape();
            // this rank's input columns: its head shard, then its share of the shard when ranks pair up
            const int64_t col0 = q_off + (int64_t)c->att_rep_idx * c->o_k;
            EFM_CK(c, cudaMemcpy2DAsync(w.o, (size_t)c->o_k * 2, src + (size_t)col0 * 2, (size_t)FQD * 2, (size_t)c->o_k * 2,
                                        (size_t)H, kind, c->stream));
            w.seen |= kO;
        } else if (rest == "mlp.gate_proj.weight" || rest == "mlp.up_proj.weight") {
            if (!shape_is(shape, ndim, FI, H)) return bad_shape();
            const bool up = rest[4] == 'u';
            // 64-row blocks: gate block b -> fused rows [128b, 128b+64), up block b -> [128b+64, 128b+128)
            EFM_CK(c, cudaMemcpy2DAsync(w.gate_up + (up ? 64 * H : 0), 128 * rowb, src + (size_t)i_off * rowb, 64 * rowb, 64 * rowb,
                                        (size_t)(I / 64), kind, c->stream));
            w.seen |= up ? kUp : kGate;
        } else if (rest == "mlp.down_proj.weight") {
            if (!shape_is(shape, ndim, H, FI)) return bad_shape();
            EFM_CK(c, cudaMemcpy2DAsync(w.down, (size_t)I * 2, src + (size_t)i_off * 2, (size_t)FI * 2, (size_t)I * 2, (size_t)H, kind,
                                        c->stream));
            w.seen |= kDown;
        } else {
            return EFM_OK;
        }
    } else {
        return EFM_OK;   // visual tower etc.: not part of this path
    }
    if (st != EFM_OK) return st;
    EFM_CK(c, cudaStreamSynchronize(c->stream));   // the caller may release `data` on return
    return EFM_OK;
}

efm_status efm_b200_set_decode_weight(efm_b200_ctx* c, const char* hf_name, const void* data, const int64_t* shape, int32_t ndim,
                                      int32_t dtype, int32_t mem_kind) {
    if (c == nullptr || hf_name == nullptr || data == nullptr || shape == nullptr)
        return fail(c, EFM_ERR_INVALID_ARGUMENT, "null argument");
    if (c->finalized) return fail(c, EFM_ERR_STATE, "weights are already finalized");
    if (c->tp_size > 1) return fail(c, EFM_ERR_UNSUPPORTED, "INT4 decode weights are not sharded: tensor-parallel contexts decode in bf16");
    EFM_CK(c, cudaSetDevice(c->device));
    const efm_model_desc& d = c->d;
    const int64_t H = d.hidden, D = d.head_dim, I = d.intermediate, V = d.vocab, QD = d.q_heads * D, KVD = d.kv_heads * D;
    std::string name(hf_name);
    bool is_q;
    const std::string qs = ".qweight", ss = ".scaling_factors";
    if (name.size() > qs.size() && name.compare(name.size() - qs.size(), qs.size(), qs) == 0) { is_q = true; name.resize(name.size() - qs.size()); }
    else if (name.size() > ss.size() && name.compare(name.size() - ss.size(), ss.size(), ss) == 0) { is_q = false; name.resize(name.size() - ss.size()); }
    else return EFM_OK;                                   // bf16 tensors of a decode checkpoint: the prefill copy serves
    W4Linear* lin = nullptr;
    int src = 0;
    int64_t rows = 0, K = 0;
    if (name == "lm_head") { lin = &c->w4_lm_head; rows = V; K = H; }
    else if (name.rfind("model.layers.", 0) == 0) {
        const size_t dot = name.find('.', 13);
        if (dot == std::string::npos) return EFM_OK;
        const int l = std::atoi(name.substr(13, dot - 13).c_str());
        if (l < 0 || l >= d.num_layers) return EFM_OK;
        const std::string rest = name.substr(dot + 1);
        LayerWeights& w = c->layers[l];
        if (rest == "self_attn.q_proj") { lin = &w.w4_qkv; src = 0; rows = QD; K = H; }
        else if (rest == "self_attn.k_proj") { lin = &w.w4_qkv; src = 1; rows = KVD; K = H; }
        else if (rest == "self_attn.v_proj") { lin = &w.w4_qkv; src = 2; rows = KVD; K = H; }
        else if (rest == "self_attn.o_proj") { lin = &w.w4_o; rows = H; K = QD; }
        else if (rest == "mlp.gate_proj") { lin = &w.w4_gate_up; src = 0; rows = I; K = H; }
        else if (rest == "mlp.up_proj") { lin = &w.w4_gate_up; src = 1; rows = I; K = H; }
        else if (rest == "mlp.down_proj") { lin = &w.w4_down; rows = H; K = I; }
        else return EFM_OK;
    } else {
        return EFM_OK;
    }
    if (K % kW4Group != 0 || rows % 2 != 0)
        return fail(c, EFM_ERR_UNSUPPORTED, "INT4 linear needs in_features % 128 == 0 and even out_features: " + std::string(hf_name));
    size_t bytes;
    if (is_q) {
        if (dtype != EFM_I8 && dtype != EFM_U8) return fail(c, EFM_ERR_UNSUPPORTED, "qweight must be int8 (two 4-bit values per byte): " + std::string(hf_name));
        if (!shape_is(shape, ndim, rows / 2, K)) return fail(c, EFM_ERR_INVALID_ARGUMENT, "unexpected shape for " + std::string(hf_name) + " (want [out_features / 2, in_features])");
        bytes = (size_t)(rows / 2) * K;
    } else {
        if (dtype != EFM_F16 && dtype != EFM_BF16) return fail(c, EFM_ERR_UNSUPPORTED, "scaling_factors must be fp16 or bf16: " + std::string(hf_name));
        if (!shape_is(shape, ndim, K / kW4Group, rows)) return fail(c, EFM_ERR_INVALID_ARGUMENT, "unexpected shape for " + std::string(hf_name) + " (want [in_features / 128, out_features])");
        bytes = (size_t)(K / kW4Group) * rows * 2;
        lin->src_s_bf16[src] = dtype == EFM_BF16;
    }
    void** slot = is_q ? &lin->src_q[src] : &lin->src_s[src];
    if (*slot == nullptr) {
        cudaError_t e = cudaMalloc(slot, bytes);          // released again by finalize_weights
        if (e != cudaSuccess) { *slot = nullptr; return cuda_fail(c, e, "staging an INT4 tensor"); }
    }
    EFM_CK(c, cudaMemcpyAsync(*slot, data, bytes, mem_kind == EFM_MEM_DEVICE ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, c->stream));
    EFM_CK(c, cudaStreamSynchronize(c->stream));
    return EFM_OK;
}

namespace {
// kind: 0 neighbours, 1 rotary partners, 2 gate / up
efm_status finish_w4_linear(efm_b200_ctx* c, W4Linear& lin, int n_src, const int rows[3], int K, int kind, const char* what) {
    if (!lin.any()) return EFM_OK;
    if (!lin.complete(n_src)) return fail(c, EFM_ERR_STATE, std::string("INT4 decode weights incomplete (qweight and scaling_factors of every part): ") + what);
    int total_rows = 0;
    for (int i = 0; i < n_src; ++i) total_rows += rows[i];
    lin.n_items = total_rows / 2;
    lin.K = K;
    if (K % kW4Group != 0) return fail(c, EFM_ERR_UNSUPPORTED, std::string("INT4 decode weights need in_features % 128 == 0: ") + what);
    const size_t padded = (size_t)((lin.n_items + 7) / 8) * 8;          // whole 16-row tiles; the padding holds zeros
    EFM_CK(c, dev_alloc(c, &lin.q, padded * K, false));
    __half2* s = nullptr;
    EFM_CK(c, dev_alloc(c, &s, padded * (K / kW4Group), false));
    lin.s = s;
    W4RepackParams p{};
    int row0 = 0;
    for (int i = 0; i < n_src; ++i) {
        p.q[i] = static_cast<const uint8_t*>(lin.src_q[i]);
        p.s[i] = lin.src_s[i];
        p.row0[i] = row0;
        p.rows[i] = rows[i];
        p.s_is_bf16[i] = lin.src_s_bf16[i];
        row0 += rows[i];
    }
    p.n_src = n_src; p.K = K; p.n_items = lin.n_items; p.kind = kind; p.head_dim = c->d.head_dim; p.half = rows[0];
    p.out_q = lin.q; p.out_s = s;
    Launcher L = make_launcher(c);
    L.counter = nullptr;
    launch_w4_repack(L, p);
    if (L.err != cudaSuccess) return cuda_fail(c, L.err, "INT4 repack launch");
    EFM_CK(c, cudaStreamSynchronize(c->stream));
    for (int i = 0; i < 3; ++i) {
        if (lin.src_q[i] != nullptr) { cudaFree(lin.src_q[i]); lin.src_q[i] = nullptr; }
        if (lin.src_s[i] != nullptr) { cudaFree(lin.src_s[i]); lin.src_s[i] = nullptr; }
    }
    lin.ready = true;
    return EFM_OK;
}
}  // namespace

efm_status efm_b200_finalize_weights(efm_b200_ctx* c) {
    if (c == nullptr) return fail(c, EFM_ERR_INVALID_ARGUMENT, "null context");
    if (!c->seen_embed) return fail(c, EFM_ERR_STATE, "missing model.embed_tokens.weight");
    if (!c->seen_final_norm) return fail(c, EFM_ERR_STATE, "missing model.norm.weight");
    if (!c->d.tied_lm_head && !c->seen_lm_head) return fail(c, EFM_ERR_STATE, "missing lm_head.weight (untied model)");
    for (int l = 0; l < c->d.num_layers; ++l)
        if ((c->layers[l].seen & kRequired) != kRequired)
            return fail(c, EFM_ERR_STATE, "missing weights in layer " + std::to_string(l));
    EFM_CK(c, cudaStreamSynchronize(c->stream));
    {   // INT4 copies of the decode linears, when a decode checkpoint supplied them: all layers or none
        const efm_model_desc& d = c->d;
        const int D = d.head_dim, QD = d.q_heads * D, KVD = d.kv_heads * D;
        bool all = true, any = c->w4_lm_head.any();
        for (auto& w : c->layers) any = any || w.w4_qkv.any() || w.w4_o.any() || w.w4_gate_up.any() || w.w4_down.any();
        if (any) {
            for (int l = 0; l < d.num_layers; ++l) {
                LayerWeights& w = c->layers[l];
                const int r_qkv[3] = {QD, KVD, KVD}, r_o[3] = {d.hidden, 0, 0}, r_gu[3] = {d.intermediate, d.intermediate, 0};
                efm_status st = finish_w4_linear(c, w.w4_qkv, 3, r_qkv, d.hidden, 1, "q/k/v_proj");
                if (st == EFM_OK) st = finish_w4_linear(c, w.w4_o, 1, r_o, QD, 0, "o_proj");
                if (st == EFM_OK) st = finish_w4_linear(c, w.w4_gate_up, 2, r_gu, d.hidden, 2, "gate/up_proj");
                if (st == EFM_OK) st = finish_w4_linear(c, w.w4_down, 1, r_o, d.intermediate, 0, "down_proj");
                if (st != EFM_OK) return st;
                all = all && w.w4_qkv.ready && w.w4_o.ready && w.w4_gate_up.ready && w.w4_down.ready;
            }
            const int r_lm[3] = {d.vocab, 0, 0};
            const efm_status st = finish_w4_linear(c, c->w4_lm_head, 1, r_lm, d.hidden, 0, "lm_head");
            if (st != EFM_OK) return st;
            if (!all) return fail(c, EFM_ERR_STATE, "INT4 decode weights must cover q/k/v/o/gate/up/down_proj of every layer (lm_head is optional)");
            c->decode_w4 = true;
        }
    }
    c->finalized = true;
    return EFM_OK;
}

efm_status efm_b200_alloc_kv_slot(efm_b200_ctx* c, int32_t slot, int32_t max_tokens) {
    if (c == nullptr) return fail(c, EFM_ERR_INVALID_ARGUMENT, "null context");
    if (max_tokens <= 0) return fail(c, EFM_ERR_INVALID_ARGUMENT, "max_tokens must be positive");
    if (c->slots.count(slot)) return fail(c, EFM_ERR_STATE, "slot already allocated");
    EFM_CK(c, cudaSetDevice(c->device));
    KvSlot s;
    s.max_tokens = max_tokens;
    const size_t block = (size_t)max_tokens * c->d.kv_heads * c->d.head_dim;
    for (int l = 0; l < c->d.num_layers; ++l) {
        __nv_bfloat16* base = nullptr;
        EFM_CK(c, dev_alloc(c, &base, 2 * block));
        s.k.push_back(base);
        s.v.push_back(base + block);
    }
    const AttnPlan plan = plan_decode_attention(max_tokens, c->d.kv_heads, c->num_sms);
    s.n_splits = plan.n_splits;
    s.chunk_cap = plan.chunk_cap;
    s.attn_cluster = plan.cluster;
    EFM_CK(c, cudaStreamSynchronize(c->stream));
    c->slots[slot] = s;
    return EFM_OK;
}

efm_status efm_b200_kv_layer_ptr(efm_b200_ctx* c, int32_t slot, int32_t layer, void** k_base, int32_t* max_tokens) {
    if (c == nullptr || k_base == nullptr) return fail(c, EFM_ERR_INVALID_ARGUMENT, "null argument");
    auto it = c->slots.find(slot);
    if (it == c->slots.end() || layer < 0 || layer >= c->d.num_layers) return fail(c, EFM_ERR_INVALID_ARGUMENT, "no such slot/layer");
    *k_base = it->second.k[layer];
    if (max_tokens != nullptr) *max_tokens = it->second.max_tokens;
    return EFM_OK;
}

efm_status efm_b200_set_sampling(efm_b200_ctx* c, const efm_sampling* s) {
    if (c == nullptr || s == nullptr) return fail(c, EFM_ERR_INVALID_ARGUMENT, "null argument");
    if (!(s->temperature >= 0.f)) return fail(c, EFM_ERR_INVALID_ARGUMENT, "temperature must be >= 0");
    const bool changed = std::memcmp(&c->sampling, s, sizeof(*s)) != 0;
    c->sampling = *s;
    if (changed) {   // sampling parameters are baked into the captured step
        for (auto& kv : c->slots)
            if (kv.second.graph != nullptr) { cudaGraphExecDestroy(kv.second.graph); kv.second.graph = nullptr; }
        drop_prefill_graphs(c);
    }
    return EFM_OK;
}

efm_status efm_b200_set_prefill_graph(efm_b200_ctx* c, int32_t enable) {
    if (c == nullptr) return fail(c, EFM_ERR_INVALID_ARGUMENT, "null context");
    c->prefill_graphs = enable != 0;
    if (!c->prefill_graphs) drop_prefill_graphs(c);
    return EFM_OK;
}

efm_status efm_b200_prefill_graph_stats(efm_b200_ctx* c, int32_t* captured, int64_t* replays) {
    if (c == nullptr) return fail(c, EFM_ERR_INVALID_ARGUMENT, "null context");
    int n = 0;
    for (const auto& g : c->prefill_cache) n += g.exec != nullptr ? 1 : 0;
    if (captured != nullptr) *captured = n;
    if (replays != nullptr) *replays = c->prefill_graph_replays;
    return EFM_OK;
}

efm_status efm_b200_prefill(efm_b200_ctx* c, int32_t slot, const int32_t* token_ids, int32_t n_tokens, int32_t kv_offset,
                            const void* embeds, int32_t n_embeds, int32_t embed_token_id, int32_t embeds_mem,
                            const int32_t* pos_ids3, int32_t sample) {
    if (c == nullptr || token_ids == nullptr) return fail(c, EFM_ERR_INVALID_ARGUMENT, "null argument");
    if (!c->finalized) return fail(c, EFM_ERR_STATE, "weights not finalized");
    if (c->tp_size > 1 && c->nccl_comm == nullptr) return fail(c, EFM_ERR_STATE, "tensor-parallel context without efm_b200_tp_init");
    auto it = c->slots.find(slot);
    if (it == c->slots.end()) return fail(c, EFM_ERR_INVALID_ARGUMENT, "unknown KV slot " + std::to_string(slot));
    KvSlot& s = it->second;
    if (n_tokens <= 0 || kv_offset < 0) return fail(c, EFM_ERR_INVALID_ARGUMENT, "n_tokens must be > 0 and kv_offset >= 0");
    if ((int64_t)kv_offset + n_tokens > s.max_tokens)
        return fail(c, EFM_ERR_INVALID_ARGUMENT, "prefill exceeds the slot's max_tokens");
    if (c->d.use_mrope && pos_ids3 == nullptr) return fail(c, EFM_ERR_INVALID_ARGUMENT, "M-RoPE model needs position ids");
    EFM_CK(c, cudaSetDevice(c->device));
    const size_t H = c->d.hidden;
    if (embeds != nullptr && n_embeds > 0) {
        const size_t need = (size_t)n_embeds * H;
        if (need > c->custom_embeds_cap) {
            EFM_CK(c, dev_alloc(c, &c->custom_embeds, need, false));
            c->custom_embeds_cap = need;
        }
        EFM_CK(c, cudaMemcpyAsync(c->custom_embeds, embeds, need * 2,
                                  embeds_mem == EFM_MEM_DEVICE ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, c->stream));
    } else {
        n_embeds = 0;
    }
    Launcher L = make_launcher(c);
    // A sampled prefill runs its LAST token as a decode step (same arithmetic, K / V rows and logits as if it had been
    // a row of the GEMMs, but with the decode kernels' fp32 activations): every logit vector the caller sees then
    // comes from one set of kernels, and the first sample is as accurate as the later ones.  The rows before it go
    // through the tensor-core GEMMs.  Not when the last token is an injected embedding row or outside the vocabulary.
    const int32_t last_id = token_ids[n_tokens - 1];
    const bool tail = sample != 0 && last_id >= 0 && last_id < c->d.vocab &&
                      !(n_embeds > 0 && last_id >= embed_token_id && last_id < embed_token_id + n_embeds);
    const int n_gemm = tail ? n_tokens - 1 : n_tokens;
    if (sample != 0 && !tail) {
        DecodeState st{};
        st.token = -1;
        st.kv_len = (uint32_t)(kv_offset + n_tokens);
        EFM_CK(c, cudaMemcpyAsync(c->state, &st, sizeof(st), cudaMemcpyHostToDevice, c->stream));
    }
    if (tail) {
        DecodeState st{};
        st.token = last_id;
        st.kv_len = (uint32_t)(kv_offset + n_tokens);
        for (int r = 0; r < 3; ++r) st.pos[r] = pos_ids3 != nullptr ? pos_ids3[(size_t)r * n_tokens + n_tokens - 1] : 0;
        EFM_CK(c, cudaMemcpyAsync(c->state, &st, sizeof(st), cudaMemcpyHostToDevice, c->stream));
    }
    auto run_tail = [&](Launcher& LL) {
        if (!tail) return;
        const bool w4 = c->decode_w4;
        c->decode_w4 = false;            // the first token belongs to the prefill pass: bf16 weights even when decode runs on INT4
        qwen_decode_step(*c, s, LL);
        c->decode_w4 = w4;
    };
    // ---- one chunk, graphs on: replay (or capture) the launch sequence of this shape ------------------------------
    if (c->prefill_graphs && n_gemm <= c->max_s) {
        const int S = n_gemm;
        if (S > 0) {
            EFM_CK(c, cudaMemcpyAsync(c->ids, token_ids, (size_t)S * 4, cudaMemcpyHostToDevice, c->stream));
            if (pos_ids3 != nullptr)
                for (int r = 0; r < 3; ++r)
                    EFM_CK(c, cudaMemcpyAsync(c->pos3 + (size_t)r * S, pos_ids3 + (size_t)r * n_tokens, (size_t)S * 4, cudaMemcpyHostToDevice, c->stream));
        }
        PrefillGraph key;
        key.slot = slot; key.rows = n_tokens; key.kv_offset = kv_offset; key.n_embeds = n_embeds; key.embed_token_id = embed_token_id;
        key.sample = (sample != 0 ? 1 : 0) + (tail ? 2 : 0); key.attention_kind = c->prefill_attention_kind;
        key.embeds_buf = n_embeds > 0 ? c->custom_embeds : nullptr;
        PrefillGraph* hit = nullptr;
        for (auto& g : c->prefill_cache)
            if (g.same_key(key)) { hit = &g; break; }
        auto launch_all = [&]() {
            if (S > 0) qwen_prefill_chunk(*c, s, S, kv_offset, n_embeds, embed_token_id, sample != 0 && !tail, L);
            run_tail(L);
        };
        if (hit != nullptr && hit->exec == nullptr) {          // second sighting: capture
            cudaGraph_t g = nullptr;
            const int64_t before = c->launches;
            EFM_CK(c, cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
            launch_all();
            cudaError_t e = cudaStreamEndCapture(c->stream, &g);
            hit->nodes = (int)(c->launches - before);
            c->launches = before;
            if (L.err != cudaSuccess) { if (g) cudaGraphDestroy(g); return cuda_fail(c, L.err, "prefill capture launch"); }
            if (e != cudaSuccess) return cuda_fail(c, e, "cudaStreamEndCapture (prefill)");
            e = cudaGraphInstantiate(&hit->exec, g, 0);
            cudaGraphDestroy(g);
            if (e != cudaSuccess) { hit->exec = nullptr; return cuda_fail(c, e, "cudaGraphInstantiate (prefill)"); }
        }
        if (hit != nullptr) {
            hit->last_use = ++c->prefill_clock;
            EFM_CK(c, cudaGraphLaunch(hit->exec, c->stream));
            c->launches += hit->nodes;
            ++c->prefill_graph_replays;
            return EFM_OK;
        }
        // first sighting: remember the shape (evicting the least recently used one), run kernel by kernel
        if (c->prefill_cache.size() >= kMaxPrefillGraphs) {
            size_t victim = 0;
            for (size_t i = 1; i < c->prefill_cache.size(); ++i)
                if (c->prefill_cache[i].last_use < c->prefill_cache[victim].last_use) victim = i;
            if (c->prefill_cache[victim].exec != nullptr) cudaGraphExecDestroy(c->prefill_cache[victim].exec);
            c->prefill_cache.erase(c->prefill_cache.begin() + (long)victim);
        }
        key.last_use = ++c->prefill_clock;
        c->prefill_cache.push_back(key);
        launch_all();
        if (L.err != cudaSuccess) return cuda_fail(c, L.err, "prefill launch");
        return EFM_OK;
    }
    for (int off = 0; off < n_gemm; off += c->max_s) {
        const int S = std::min(c->max_s, n_gemm - off);
        EFM_CK(c, cudaMemcpyAsync(c->ids, token_ids + off, (size_t)S * 4, cudaMemcpyHostToDevice, c->stream));
        if (pos_ids3 != nullptr)
            for (int r = 0; r < 3; ++r)
                EFM_CK(c, cudaMemcpyAsync(c->pos3 + (size_t)r * S, pos_ids3 + (size_t)r * n_tokens + off, (size_t)S * 4,
                                          cudaMemcpyHostToDevice, c->stream));
        const bool last = off + S >= n_gemm;
        qwen_prefill_chunk(*c, s, S, kv_offset + off, n_embeds, embed_token_id, last && sample != 0 && !tail, L);
        if (L.err != cudaSuccess) return cuda_fail(c, L.err, "prefill launch");
    }
    run_tail(L);
    if (L.err != cudaSuccess) return cuda_fail(c, L.err, "prefill launch (last token)");
    return EFM_OK;
}

efm_status efm_b200_decode_begin(efm_b200_ctx* c, int32_t slot, int32_t kv_len, const int32_t mrope_pos[3], int32_t step) {
    if (c == nullptr) return fail(c, EFM_ERR_INVALID_ARGUMENT, "null context");
    auto it = c->slots.find(slot);
    if (it == c->slots.end()) return fail(c, EFM_ERR_INVALID_ARGUMENT, "unknown KV slot " + std::to_string(slot));
    if (kv_len < 0 || kv_len >= it->second.max_tokens) return fail(c, EFM_ERR_INVALID_ARGUMENT, "kv_len leaves no room in the slot");
    if (step < 0) return fail(c, EFM_ERR_INVALID_ARGUMENT, "step must be >= 0");
    EFM_CK(c, cudaSetDevice(c->device));
    struct { uint32_t kv_len; int32_t pos[3]; int32_t step; int32_t error; } tail;
    tail.kv_len = (uint32_t)kv_len + 1u;      // the step appends its own K/V before attending
    for (int i = 0; i < 3; ++i) tail.pos[i] = mrope_pos != nullptr ? mrope_pos[i] : 0;
    tail.step = step;
    tail.error = 0;
    static_assert(offsetof(DecodeState, kv_len) == 4 && sizeof(tail) == 24, "DecodeState layout");
    EFM_CK(c, cudaMemcpyAsync(reinterpret_cast<char*>(c->state) + 4, &tail, sizeof(tail), cudaMemcpyHostToDevice, c->stream));
    if (c->error_host != nullptr) *reinterpret_cast<volatile int*>(c->error_host) = 0;
    c->bound_slot = slot;
    return EFM_OK;
}

efm_status efm_b200_set_token(efm_b200_ctx* c, int32_t token) {
    if (c == nullptr) return fail(c, EFM_ERR_INVALID_ARGUMENT, "null context");
    EFM_CK(c, cudaMemcpyAsync(&c->state->token, &token, 4, cudaMemcpyHostToDevice, c->stream));
    return EFM_OK;
}

static efm_status ensure_graph(efm_b200_ctx* c, KvSlot& s) {
    if (s.graph != nullptr) return EFM_OK;
    Launcher L = make_launcher(c);
    cudaGraph_t g = nullptr;
    const int64_t before = c->launches;
    EFM_CK(c, cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
    qwen_decode_step(*c, s, L);
    cudaError_t e = cudaStreamEndCapture(c->stream, &g);
    s.graph_nodes = (int)(c->launches - before);
    c->launches = before;                 // capture records, it does not run
    if (L.err != cudaSuccess) { if (g) cudaGraphDestroy(g); return cuda_fail(c, L.err, "decode capture launch"); }
    if (e != cudaSuccess) return cuda_fail(c, e, "cudaStreamEndCapture");
    e = cudaGraphInstantiate(&s.graph, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) { s.graph = nullptr; return cuda_fail(c, e, "cudaGraphInstantiate"); }
    return EFM_OK;
}

efm_status efm_b200_capture_decode(efm_b200_ctx* c, int32_t slot) {
    if (c == nullptr) return fail(c, EFM_ERR_INVALID_ARGUMENT, "null context");
    if (!c->finalized) return fail(c, EFM_ERR_STATE, "weights not finalized");
    auto it = c->slots.find(slot);
    if (it == c->slots.end()) return fail(c, EFM_ERR_INVALID_ARGUMENT, "unknown KV slot " + std::to_string(slot));
    EFM_CK(c, cudaSetDevice(c->device));
    return ensure_graph(c, it->second);
}

efm_status efm_b200_decode_steps(efm_b200_ctx* c, int32_t n_steps, int32_t use_graph) {
    if (c == nullptr) return fail(c, EFM_ERR_INVALID_ARGUMENT, "null context");
    if (c->bound_slot < 0) return fail(c, EFM_ERR_STATE, "decode_begin has not been called");
    if (n_steps <= 0) return EFM_OK;
    KvSlot& s = c->slots[c->bound_slot];
    EFM_CK(c, cudaSetDevice(c->device));
    if (!use_graph) {
        Launcher L = make_launcher(c);
        for (int i = 0; i < n_steps; ++i) qwen_decode_step(*c, s, L);
        if (L.err != cudaSuccess) return cuda_fail(c, L.err, "decode launch");
        return EFM_OK;
    }
    const efm_status st = ensure_graph(c, s);
    if (st != EFM_OK) return st;
    for (int i = 0; i < n_steps; ++i) {
        // a kernel of an earlier step gave up waiting for a peer: queue nothing more behind it
        if (c->error_host != nullptr && *reinterpret_cast<volatile int*>(c->error_host) != 0)
            return fail(c, EFM_ERR_DEVICE_WAIT, "a tensor-parallel peer did not answer within the wait limit; decode stopped after " +
                                                    std::to_string(i) + " queued steps");
        EFM_CK(c, cudaGraphLaunch(s.graph, c->stream));
        c->launches += s.graph_nodes;
    }
    return EFM_OK;
}

static efm_status check_device_state(efm_b200_ctx* c) {
    DecodeState st{};
    EFM_CK(c, cudaMemcpyAsync(&st, c->state, sizeof(st), cudaMemcpyDeviceToHost, c->stream));
    { const efm_status s = ctx_sync(c); if (s != EFM_OK) return s; }
    if (st.error != 0) {
        int zero = 0;
        if (c->error_host != nullptr) *reinterpret_cast<volatile int*>(c->error_host) = 0;
        cudaMemcpyAsync(&c->state->error, &zero, 4, cudaMemcpyHostToDevice, c->stream);
        return fail(c, EFM_ERR_DEVICE_WAIT, "a kernel refused an out-of-range cache row or abandoned a bounded wait (device status " + std::to_string(st.error) + ")");
    }
    return EFM_OK;
}

efm_status efm_b200_read_tokens(efm_b200_ctx* c, int32_t* host_out, int32_t first, int32_t n) {
    if (c == nullptr || host_out == nullptr) return fail(c, EFM_ERR_INVALID_ARGUMENT, "null argument");
    if (first < 0 || n < 0 || first + n > c->d.max_response_tokens) return fail(c, EFM_ERR_INVALID_ARGUMENT, "token range outside the response buffer");
    EFM_CK(c, cudaSetDevice(c->device));
    if (n > 0) EFM_CK(c, cudaMemcpyAsync(host_out, c->tokens_out + first, (size_t)n * 4, cudaMemcpyDeviceToHost, c->stream));
    return check_device_state(c);
}

efm_status efm_b200_read_logits(efm_b200_ctx* c, float* host_out, int32_t n) {
    if (c == nullptr || host_out == nullptr) return fail(c, EFM_ERR_INVALID_ARGUMENT, "null argument");
    if (n < 0 || n > c->d.vocab) return fail(c, EFM_ERR_INVALID_ARGUMENT, "n exceeds vocab");
    EFM_CK(c, cudaSetDevice(c->device));
    if (tp_greedy_exchange(*c)) {       // the step exchanged maxima only: gather the ranks' logits rows now (a collective)
        Launcher L = make_launcher(c);
        L.counter = nullptr;
        tp_gather_logits(*c, L);
        if (L.err != cudaSuccess) return cuda_fail(c, L.err, "gathering the logits of the tensor-parallel ranks");
    }
    EFM_CK(c, cudaMemcpyAsync(host_out, c->logits, (size_t)n * 4, cudaMemcpyDeviceToHost, c->stream));
    return ctx_sync(c);
}

efm_status efm_b200_synchronize(efm_b200_ctx* c) {
    if (c == nullptr) return fail(c, EFM_ERR_INVALID_ARGUMENT, "null context");
    return ctx_sync(c);
}

efm_status efm_b200_event_record(efm_b200_ctx* c, int32_t idx) {
    if (c == nullptr || idx < 0 || idx >= 16) return fail(c, EFM_ERR_INVALID_ARGUMENT, "event index out of range");
    EFM_CK(c, cudaEventRecord(c->events[idx], c->stream));
    return EFM_OK;
}

efm_status efm_b200_event_elapsed_ms(efm_b200_ctx* c, int32_t a, int32_t b, float* ms) {
    if (c == nullptr || ms == nullptr || a < 0 || a >= 16 || b < 0 || b >= 16) return fail(c, EFM_ERR_INVALID_ARGUMENT, "bad event arguments");
    EFM_CK(c, cudaEventSynchronize(c->events[b]));
    EFM_CK(c, cudaEventElapsedTime(ms, c->events[a], c->events[b]));
    return EFM_OK;
}

efm_status efm_b200_launch_count(efm_b200_ctx* c, int64_t* count) {
    if (c == nullptr || count == nullptr) return fail(c, EFM_ERR_INVALID_ARGUMENT, "null argument");
    *count = c->launches;
    return EFM_OK;
}

efm_status efm_b200_decode_breakdown(efm_b200_ctx* c, int32_t n_steps, float* ms_out) {
    if (c == nullptr || ms_out == nullptr) return fail(c, EFM_ERR_INVALID_ARGUMENT, "null argument");
    if (c->bound_slot < 0) return fail(c, EFM_ERR_STATE, "decode_begin has not been called");
    KvSlot& s = c->slots[c->bound_slot];
    EFM_CK(c, cudaSetDevice(c->device));
    for (int i = 0; i < 7; ++i) ms_out[i] = 0.f;
    const int per_step = 5 * c->d.num_layers + 2;
    for (int step = 0; step < n_steps; ++step) {
        std::vector<cudaEvent_t> ev;
        Launcher L = make_launcher(c);
        L.pdl = false;
        L.trace = &ev;
        cudaEvent_t first = nullptr;
        EFM_CK(c, cudaEventCreate(&first));
        EFM_CK(c, cudaEventRecord(first, c->stream));
        qwen_decode_step(*c, s, L);
        cudaError_t e = L.err != cudaSuccess ? L.err : cudaStreamSynchronize(c->stream);
        if (e == cudaSuccess && (int)ev.size() == per_step) {
            cudaEvent_t prev = first;
            for (int i = 0; i < per_step; ++i) {
                float ms = 0.f;
                cudaEventElapsedTime(&ms, prev, ev[i]);
                const int kind = i < 5 * c->d.num_layers ? i % 5 : 5 + (i - 5 * c->d.num_layers);
                ms_out[kind] += ms;
                prev = ev[i];
            }
        }
        cudaEventDestroy(first);
        for (cudaEvent_t x : ev) cudaEventDestroy(x);
        if (e != cudaSuccess) return cuda_fail(c, e, "decode breakdown");
    }
    return EFM_OK;
}

efm_status efm_b200_decode_step_bytes(efm_b200_ctx* c, int32_t kv_len, int64_t* bytes) {
    if (c == nullptr || bytes == nullptr) return fail(c, EFM_ERR_INVALID_ARGUMENT, "null argument");
    const efm_model_desc& d = c->d;
    const int64_t H = d.hidden, D = d.head_dim, q = d.q_heads, kv = d.kv_heads, I = d.intermediate, V = d.vocab, L = d.num_layers;
    // what THIS rank streams: its head shard, its o_proj columns, its MLP columns, its lm_head rows
    const int64_t per_layer = (q + 2 * kv) * D * H + (q + 2 * kv) * D + (int64_t)c->o_k * H + 3 * I * H + 2 * H;
    int64_t w = 2 * (L * per_layer + H + (int64_t)c->vocab_l * H) + 2 * H;      // + final norm, lm_head rows, one embedding row
    if (c->decode_w4) {
        // INT4 linears: half a byte per weight + one fp16 scale per 128 weights; biases, norms, embedding row in bf16
        const int64_t lin = (q + 2 * kv) * D * H + q * D * H + 3 * I * H;
        const int64_t lm = V * H;
        const auto w4 = [](int64_t n) { return n / 2 + n / kW4Group * 2; };
        w = L * (w4(lin) + 2 * ((q + 2 * kv) * D + 2 * H)) + 2 * H + (c->w4_lm_head.ready ? w4(lm) : 2 * lm) + 2 * H;
    }
    *bytes = w + L * 2 * (int64_t)kv_len * kv * D * 2;
    return EFM_OK;
}

// ---------------------------------------------------------------------------------------------
// single operators on caller-provided device buffers (default stream, synchronous)
// ---------------------------------------------------------------------------------------------
static efm_status op_prepare(int* num_sms) {
    int dev = 0;
    efm_status st = EFM_OK;
    if (cudaGetDevice(&dev) != cudaSuccess) return fail(nullptr, EFM_ERR_CUDA, "no CUDA device available");
    if ((st = require_b200(nullptr, dev)) != EFM_OK) return st;
    if (num_sms != nullptr) cudaDeviceGetAttribute(num_sms, cudaDevAttrMultiProcessorCount, dev);
    return EFM_OK;
}
static efm_status op_finish(Launcher& L) {
    if (L.err != cudaSuccess) return cuda_fail(nullptr, L.err, "operator launch");
    cudaError_t e = cudaStreamSynchronize(L.stream);
    if (e != cudaSuccess) return cuda_fail(nullptr, e, "operator execution");
    return EFM_OK;
}

efm_status efm_b200_op_gemv(const void* w, const void* x, const void* norm_w, float eps, void* y_bf16, void* residual,
                            int32_t n, int32_t k) {
    int sms = 148;
    efm_status st = op_prepare(&sms);
    if (st != EFM_OK) return st;
    if (w == nullptr || x == nullptr || (y_bf16 == nullptr && residual == nullptr) || n <= 0 || n % 2 || k <= 0 || k % 8)
        return fail(nullptr, EFM_ERR_INVALID_ARGUMENT, "op_gemv: bad arguments (n even, k % 8 == 0)");
    GemvParams p{};
    p.W = (const __nv_bfloat16*)w; p.N = n; p.K = k; p.n_items = n / 2;
    p.prologue = norm_w != nullptr ? kProRmsNorm : kProPlain;
    p.x = (const __nv_bfloat16*)x; p.xr = (const float*)x; p.norm_w = (const __nv_bfloat16*)norm_w; p.eps = eps;
    p.y = (__nv_bfloat16*)y_bf16; p.residual = (float*)residual;
    Launcher L; L.pdl = false;
    if (residual != nullptr) launch_gemv<Epi::Residual>(L, p, sms); else launch_gemv<Epi::Plain>(L, p, sms);
    return op_finish(L);
}

efm_status efm_b200_op_gemv_peer_consume(const void* w, const void* resid_f32, const void* norm_w, float eps, const void* parts,
                                         int32_t n_parts, uint32_t want_count, int64_t wait_limit_us, void* y_bf16,
                                         void* resid_out_f32, int32_t n, int32_t k) {
    int sms = 148;
    efm_status st = op_prepare(&sms);
    if (st != EFM_OK) return st;
    if (w == nullptr || resid_f32 == nullptr || norm_w == nullptr || parts == nullptr || y_bf16 == nullptr || resid_out_f32 == nullptr ||
        resid_out_f32 == resid_f32 || n_parts < 1 || n_parts > kMaxPeers || want_count == 0 || wait_limit_us <= 0 || n <= 0 || n % 2 ||
        k <= 0 || k % 8)
        return fail(nullptr, EFM_ERR_INVALID_ARGUMENT, "op_gemv_peer_consume: bad arguments");
    int* error = nullptr;
    cudaError_t e = cudaMalloc(&error, sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(error, 0, sizeof(int));
    if (e != cudaSuccess) { cudaFree(error); return cuda_fail(nullptr, e, "op_gemv_peer_consume scratch"); }
    GemvParams p{};
    p.W = (const __nv_bfloat16*)w; p.N = n; p.K = k; p.n_items = n / 2;
    p.prologue = kProRmsNorm;
    p.xr = (const float*)resid_f32; p.norm_w = (const __nv_bfloat16*)norm_w; p.eps = eps;
    p.resid_out = (float*)resid_out_f32;
    p.addend_parts = (const uint2*)parts; p.n_parts = n_parts; p.want_override = want_count;
    p.error = error; p.wait_ns = (unsigned long long)wait_limit_us * 1000ull;
    p.y = (__nv_bfloat16*)y_bf16;
    Launcher L; L.pdl = false;
    launch_gemv<Epi::Plain>(L, p, sms);
    st = op_finish(L);
    int raised = 0;
    if (st == EFM_OK && cudaMemcpy(&raised, error, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) st = fail(nullptr, EFM_ERR_CUDA, "reading the status word");
    cudaFree(error);
    if (st == EFM_OK && raised != 0)
        return fail(nullptr, EFM_ERR_DEVICE_WAIT, "the wait for the peers' words ran out (device status " + std::to_string(raised) + ")");
    return st;
}

efm_status efm_b200_op_gemm(const void* x, const void* w, const void* bias, void* y_bf16, int32_t m, int32_t n, int32_t k) {
    efm_status st = op_prepare(nullptr);
    if (st != EFM_OK) return st;
    if (x == nullptr || w == nullptr || y_bf16 == nullptr || m <= 0 || n <= 0 || n % 2 || k <= 0 || k % 32)
        return fail(nullptr, EFM_ERR_INVALID_ARGUMENT, "op_gemm: bad arguments (n even, k % 32 == 0)");
    GemmParams g{(const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (const __nv_bfloat16*)bias, (__nv_bfloat16*)y_bf16, nullptr, m, n, k};
    Launcher L; L.pdl = false;
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0);
    L.num_sms = sms;
    L.gemm_ws_floats = (size_t)sms * 128 * 256;          // lets skinny products take the split-K path, as inside a context
    if (cudaMalloc(&L.gemm_ws, L.gemm_ws_floats * sizeof(float)) != cudaSuccess) {
        (void)cudaGetLastError();
        L.gemm_ws = nullptr;
    }
    launch_gemm_bf16(L, g);
    const efm_status out = op_finish(L);
    if (L.gemm_ws != nullptr) cudaFree(L.gemm_ws);
    return out;
}

namespace {
// INT8 attention scratch for up to q_rows queries and kv_rows keys (one scale per 128-token block and head);
// plain cudaMalloc, caller frees with free_sage.
cudaError_t alloc_sage(SageScratch& sc, int q_rows, int kv_rows, int q_heads, int kv_heads, int D) {
    cudaError_t e = cudaMalloc(&sc.q8, (size_t)q_rows * q_heads * D);
    if (e == cudaSuccess) e = cudaMalloc(&sc.k8, (size_t)kv_rows * kv_heads * D);
    if (e == cudaSuccess) e = cudaMalloc(&sc.vh, (size_t)kv_rows * kv_heads * D * 2);
    if (e == cudaSuccess) e = cudaMalloc(&sc.sq, (size_t)(q_rows / 128 + 1) * q_heads * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(&sc.sk, (size_t)(kv_rows / 128 + 1) * kv_heads * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(&sc.kmean, (size_t)(kv_rows / 128 + 1) * kv_heads * D * sizeof(float));
    sc.q_rows = q_rows;
    sc.kv_rows = kv_rows;
    return e;
}
void free_sage(SageScratch& sc) {
    cudaFree(sc.q8); cudaFree(sc.k8); cudaFree(sc.vh); cudaFree(sc.sq); cudaFree(sc.sk); cudaFree(sc.kmean);
    sc = SageScratch{};
}
}  // namespace

efm_status efm_b200_set_prefill_attention(efm_b200_ctx* c, int32_t kind) {
    if (c == nullptr) return fail(c, EFM_ERR_INVALID_ARGUMENT, "null argument");
    if (kind != 0 && kind != 1) return fail(c, EFM_ERR_INVALID_ARGUMENT, "prefill attention kind must be 0 (bf16) or 1 (int8)");
    if (kind == 1) {
        int rows = 0;
        for (auto& kv : c->slots) rows = std::max(rows, kv.second.max_tokens);
        if (rows == 0) return fail(c, EFM_ERR_STATE, "allocate the KV slots before selecting the INT8 prefill attention");
        if (c->d.head_dim != 64 && c->d.head_dim != 128) return fail(c, EFM_ERR_UNSUPPORTED, "INT8 prefill attention: head_dim 64 or 128");
        EFM_CK(c, cudaSetDevice(c->device));
        if (rows > c->sage.kv_rows) {
            EFM_CK(c, cudaStreamSynchronize(c->stream));
            free_sage(c->sage);
            cudaError_t e = alloc_sage(c->sage, c->max_s, rows, c->d.q_heads, c->d.kv_heads, c->d.head_dim);
            if (e != cudaSuccess) { free_sage(c->sage); return cuda_fail(c, e, "INT8 attention scratch"); }
        }
    }
    if (c->prefill_attention_kind != kind) drop_prefill_graphs(c);     // the INT8 scratch may have moved as well
    c->prefill_attention_kind = kind;
    return EFM_OK;
}

efm_status efm_b200_op_sage_prefill_attention(const void* q, const void* k_cache, const void* v_cache, void* out_bf16,
                                              int32_t s, int32_t kv_offset, int32_t q_heads, int32_t kv_heads, int32_t head_dim) {
    efm_status st = op_prepare(nullptr);
    if (st != EFM_OK) return st;
    if (q == nullptr || k_cache == nullptr || v_cache == nullptr || out_bf16 == nullptr || s <= 0 || kv_offset < 0 || q_heads <= 0 ||
        kv_heads <= 0 || q_heads % kv_heads != 0)
        return fail(nullptr, EFM_ERR_INVALID_ARGUMENT, "op_sage_prefill_attention: bad arguments");
    if (head_dim != 64 && head_dim != 128) return fail(nullptr, EFM_ERR_UNSUPPORTED, "op_sage_prefill_attention: head_dim 64 or 128");
    SageScratch sc;
    cudaError_t e = alloc_sage(sc, s, kv_offset + s, q_heads, kv_heads, head_dim);
    if (e != cudaSuccess) { free_sage(sc); return cuda_fail(nullptr, e, "INT8 attention scratch"); }
    Launcher L; L.pdl = false;
    launch_sage_prefill_attention(L, sc, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache,
                                  (__nv_bfloat16*)out_bf16, s, kv_offset, q_heads, kv_heads, head_dim);
    st = op_finish(L);
    free_sage(sc);
    return st;
}

efm_status efm_b200_op_decode_attention(const void* q, const void* k_cache, const void* v_cache, void* out_bf16,
                                        int32_t q_heads, int32_t kv_heads, int32_t head_dim, int32_t kv_len, int32_t max_tokens) {
    int sms = 148;
    efm_status st = op_prepare(&sms);
    if (st != EFM_OK) return st;
    if (q == nullptr || k_cache == nullptr || v_cache == nullptr || out_bf16 == nullptr || kv_heads <= 0 || q_heads % kv_heads ||
        q_heads / kv_heads > kMaxGroup || (head_dim != 64 && head_dim != 128) || kv_len <= 0 || kv_len > max_tokens)
        return fail(nullptr, EFM_ERR_INVALID_ARGUMENT, "op_decode_attention: bad arguments");
    const AttnPlan plan = plan_decode_attention(max_tokens, kv_heads, sms);
    float* part_o = nullptr; float* part_ml = nullptr; unsigned int* counters = nullptr;
    cudaError_t e = cudaMalloc(&part_o, (size_t)q_heads * plan.n_splits * head_dim * 4);
    if (e == cudaSuccess) e = cudaMalloc(&part_ml, (size_t)q_heads * plan.n_splits * 2 * 4);
    if (e == cudaSuccess) e = cudaMalloc(&counters, (size_t)kv_heads * 4);
    if (e == cudaSuccess) e = cudaMemset(counters, 0, (size_t)kv_heads * 4);
    if (e == cudaSuccess) {
        DecodeAttnParams a{};
        a.q = (const __nv_bfloat16*)q; a.k_cache = (const __nv_bfloat16*)k_cache; a.v_cache = (const __nv_bfloat16*)v_cache;
        a.out = (__nv_bfloat16*)out_bf16; a.state = nullptr; a.kv_len_static = kv_len;
        a.q_heads = q_heads; a.kv_heads = kv_heads; a.group = q_heads / kv_heads;
        a.n_splits = plan.n_splits; a.chunk_cap = plan.chunk_cap; a.max_tokens = max_tokens; a.cluster = plan.cluster;
        a.scale = 1.0f / sqrtf((float)head_dim);
        a.part_o = part_o; a.part_ml = part_ml; a.counters = counters;
        Launcher L; L.pdl = false;
        launch_decode_attention(L, a, head_dim);
        st = op_finish(L);
    } else {
        st = cuda_fail(nullptr, e, "op_decode_attention scratch");
    }
    cudaFree(part_o); cudaFree(part_ml); cudaFree(counters);
    return st;
}

// ---- decode attention without any allocation -------------------------------------------------
// Scratch for the split-KV partials lives in the library image.  In host code the symbol below is
// only a stand-in for the device array: its device address has to be asked for, per device.
namespace {
constexpr int kNoAllocMaxQD = 4096;       // q_heads * head_dim
constexpr int kNoAllocMaxKvHeads = 16;
constexpr int kNoAllocMaxQHeads = 64;     // head_dim >= 64
// layout in 32-bit words: partial outputs [q_heads][n_splits][D] | (max, sum) pairs
// [q_heads][n_splits][2] | block tickets [kv_heads] (these must read zero when a launch starts)
constexpr size_t kNoAllocPartO = (size_t)kNoAllocMaxQD * kMaxSplits;
constexpr size_t kNoAllocPartMl = (size_t)kNoAllocMaxQHeads * kMaxSplits * 2;
constexpr size_t kNoAllocWords = kNoAllocPartO + kNoAllocPartMl + kNoAllocMaxKvHeads;     // ~1.06 MB
static __device__ __align__(256) float g_noalloc_scratch[kNoAllocWords];
constexpr int kNoAllocMaxDevices = 64;
std::atomic<float*> g_noalloc_ptr[kNoAllocMaxDevices];     // zero-initialised; filled once per device, any thread
}  // namespace

efm_status efm_b200_op_decode_attention_noalloc(const void* q, const void* k_cache, const void* v_cache, void* out_bf16,
                                                int32_t q_heads, int32_t kv_heads, int32_t head_dim, int32_t kv_len,
                                                int32_t max_tokens) {
    int sms = 148;
    efm_status st = op_prepare(&sms);
    if (st != EFM_OK) return st;
    if (q == nullptr || k_cache == nullptr || v_cache == nullptr || out_bf16 == nullptr || kv_heads <= 0 || q_heads % kv_heads ||
        q_heads / kv_heads > kMaxGroup || (head_dim != 64 && head_dim != 128) || kv_len <= 0 || kv_len > max_tokens)
        return fail(nullptr, EFM_ERR_INVALID_ARGUMENT, "op_decode_attention_noalloc: bad arguments");
    if (q_heads * head_dim > kNoAllocMaxQD || kv_heads > kNoAllocMaxKvHeads || q_heads > kNoAllocMaxQHeads)
        return fail(nullptr, EFM_ERR_UNSUPPORTED,
                    "op_decode_attention_noalloc: shape exceeds the built-in scratch (q_heads * head_dim <= 4096, "
                    "q_heads <= 64, kv_heads <= 16); use efm_b200_op_decode_attention");
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(nullptr, e, "cudaGetDevice");
    if (dev < 0 || dev >= kNoAllocMaxDevices) return fail(nullptr, EFM_ERR_UNSUPPORTED, "device index above 63");
    float* scratch = g_noalloc_ptr[dev].load(std::memory_order_acquire);
    if (scratch == nullptr) {      // once per device, with that device current (two threads racing here store the same address)
        float* ptr = nullptr;
        e = cudaGetSymbolAddress((void**)&ptr, g_noalloc_scratch);
        if (e != cudaSuccess || ptr == nullptr) return cuda_fail(nullptr, e, "cudaGetSymbolAddress(scratch)");
        g_noalloc_ptr[dev].store(ptr, std::memory_order_release);
        scratch = ptr;
    }
    unsigned int* tickets = reinterpret_cast<unsigned int*>(scratch + kNoAllocPartO + kNoAllocPartMl);
    const AttnPlan plan = plan_decode_attention(max_tokens, kv_heads, sms);
    e = cudaMemsetAsync(tickets, 0, kNoAllocMaxKvHeads * sizeof(unsigned int), nullptr);
    if (e != cudaSuccess) return cuda_fail(nullptr, e, "clearing the scratch tickets");
    DecodeAttnParams a{};
    a.q = (const __nv_bfloat16*)q; a.k_cache = (const __nv_bfloat16*)k_cache; a.v_cache = (const __nv_bfloat16*)v_cache;
    a.out = (__nv_bfloat16*)out_bf16; a.state = nullptr; a.kv_len_static = kv_len;
    a.q_heads = q_heads; a.kv_heads = kv_heads; a.group = q_heads / kv_heads;
    a.n_splits = plan.n_splits; a.chunk_cap = plan.chunk_cap; a.max_tokens = max_tokens; a.cluster = plan.cluster;
    a.scale = 1.0f / sqrtf((float)head_dim);
    a.part_o = scratch; a.part_ml = scratch + kNoAllocPartO; a.counters = tickets;
    Launcher L; L.pdl = false;
    launch_decode_attention(L, a, head_dim);
    return op_finish(L);
}

efm_status efm_b200_op_prefill_attention(const void* q, const void* k_cache, const void* v_cache, void* out_bf16, int32_t s,
                                         int32_t kv_offset, int32_t q_heads, int32_t kv_heads, int32_t head_dim) {
    efm_status st = op_prepare(nullptr);
    if (st != EFM_OK) return st;
    if (q == nullptr || k_cache == nullptr || v_cache == nullptr || out_bf16 == nullptr || s <= 0 || kv_offset < 0 || kv_heads <= 0 ||
        q_heads % kv_heads || (head_dim != 64 && head_dim != 128))
        return fail(nullptr, EFM_ERR_INVALID_ARGUMENT, "op_prefill_attention: bad arguments");
    Launcher L; L.pdl = false;
    launch_prefill_attention(L, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache,
                             (__nv_bfloat16*)out_bf16, s, kv_offset, q_heads, kv_heads, head_dim);
    return op_finish(L);
}

efm_status efm_b200_op_sample(const float* logits, int32_t vocab, const efm_sampling* s, uint32_t rng_step, int32_t* token_out) {
    efm_status st = op_prepare(nullptr);
    if (st != EFM_OK) return st;
    if (logits == nullptr || s == nullptr || token_out == nullptr || vocab <= 0)
        return fail(nullptr, EFM_ERR_INVALID_ARGUMENT, "op_sample: bad arguments");
    uint32_t* wbuf = nullptr;
    cudaError_t e = cudaMalloc(&wbuf, sample_scratch_words(vocab) * 4);
    if (e != cudaSuccess) return cuda_fail(nullptr, e, "op_sample scratch");
    SampleParams p{};
    p.logits = logits; p.vocab = vocab; p.n_part = 0;
    p.temperature = s->temperature; p.top_p = s->top_p; p.seed = s->seed; p.rng_step = rng_step;
    p.state = nullptr; p.token_single = token_out; p.wbuf = wbuf; p.xchg = sample_xchg(wbuf, vocab);
    Launcher L; L.pdl = false;
    launch_sample(L, p);
    st = op_finish(L);
    cudaFree(wbuf);
    return st;
}

}  // extern "C"
