#include "standard_engine.h"

#include "tp_rendezvous.h"

#include <cuda_runtime.h>
#include <efm_b200.h>

#include <algorithm>
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <unordered_set>

#include "safetensors.h"

namespace edge_fm {

namespace {

double now_ms() {
    using namespace std::chrono;
    return duration<double, std::milli>(steady_clock::now().time_since_epoch()).count();
}

// KV buffers live in the backend; the manager only keeps the bookkeeping and the pointers.
class BackendKVAllocator : public KVBufferAllocator {
public:
    explicit BackendKVAllocator(efm_b200_ctx* ctx) : ctx_(ctx) {}
    Device device() const override { return Device::GPU; }
    std::vector<void*> allocate_slot(int32_t request_id, int32_t max_tokens, size_t, int32_t num_layers) override {
        efm_status st = efm_b200_alloc_kv_slot(ctx_, request_id, max_tokens);
        if (st == EFM_ERR_OUT_OF_MEMORY) throw OutOfMemoryError(efm_b200_last_error(ctx_));
        if (st != EFM_OK) throw DeviceError(efm_b200_last_error(ctx_));
        std::vector<void*> out;
        for (int32_t l = 0; l < num_layers; ++l) {
            void* p = nullptr;
            if (efm_b200_kv_layer_ptr(ctx_, request_id, l, &p, nullptr) != EFM_OK) throw InternalError(efm_b200_last_error(ctx_));
            out.push_back(p);
        }
        return out;
    }

private:
    efm_b200_ctx* ctx_;
};

int32_t dtype_code(const std::string& st) {
    if (st == "BF16") return EFM_BF16;
    if (st == "F16") return EFM_F16;
    if (st == "F32") return EFM_F32;
    if (st == "I32") return EFM_I32;
    if (st == "I64") return EFM_I64;
    if (st == "U8") return EFM_U8;
    if (st == "I8") return EFM_I8;
    return -1;
}

}  // namespace

void StandardEngine::check(int32_t st, const char* what) const {
    if (st == EFM_OK) return;
    const std::string msg = std::string(what) + ": " + efm_b200_last_error(ctx_);
    switch (st) {
        case EFM_ERR_OUT_OF_MEMORY: throw OutOfMemoryError(msg);
        case EFM_ERR_INVALID_ARGUMENT: throw InvalidRequestError(msg);
        case EFM_ERR_UNSUPPORTED: throw ConfigurationError(msg);
        case EFM_ERR_STATE: throw InternalError(msg);
        default: throw DeviceError(msg);
    }
}

StandardEngine::StandardEngine(const EngineConfig& config) : config_(config) {
    if (device_from_string(config_.runtime_device()) != Device::GPU)
        throw ConfigurationError("token generation needs runtime.device = cuda (there is no CPU path)");
    const std::string model = config_.resolved_model_name();
    const json::Value mc = config_.prefill_model_config();
    device_id_ = config_.runtime_device_id();
    use_graph_ = config_.use_cuda_graph();
    if (dtype_from_string(config_.kvcache_dtype()) != DType::BFloat16)
        throw ConfigurationError("kvcache.dtype must be bf16 for this backend");
    const AttentionType attn = attention_type_from_string(config_.kvcache_attention_type());

    efm_model_desc d;
    std::memset(&d, 0, sizeof(d));
    d.struct_size = (int32_t)sizeof(d);
    d.num_layers = (int32_t)mc.get_int("num_hidden_layers", 0);
    d.hidden = (int32_t)mc.get_int("hidden_size", 0);
    d.q_heads = (int32_t)mc.get_int("num_attention_heads", 0);
    d.kv_heads = (int32_t)mc.get_int("num_key_value_heads", d.q_heads);
    d.intermediate = (int32_t)mc.get_int("intermediate_size", 0);
    d.vocab = (int32_t)mc.get_int("vocab_size", 0);
    if (d.num_layers <= 0 || d.hidden <= 0 || d.q_heads <= 0 || d.vocab <= 0 || d.intermediate <= 0)
        throw ConfigurationError("config.json lacks num_hidden_layers / hidden_size / num_attention_heads / vocab_size / intermediate_size");
    d.head_dim = d.hidden / d.q_heads;      // as the reference derives it (kv_manager.cpp:80)
    d.rms_eps = (float)mc.get_double("rms_norm_eps", 1e-6);
    d.rope_theta = (float)mc.get_double("rope_theta", 10000.0);
    const std::string act = mc.get_string("hidden_act", "silu");
    if (act != "silu") throw ConfigurationError("hidden_act must be silu, got " + act);
    const std::string torch_dtype = mc.get_string("torch_dtype", mc.get_string("dtype", "bfloat16"));
    if (torch_dtype != "bfloat16") throw ConfigurationError("checkpoint dtype must be bfloat16, got " + torch_dtype);
    const json::Value* rs = mc.find("rope_scaling");
    if (rs != nullptr && rs->is_object()) {
        const json::Value* sec = rs->find("mrope_section");
        if (sec != nullptr && sec->is_array() && sec->arr.size() == 3) {
            d.use_mrope = 1;
            for (int i = 0; i < 3; ++i) d.mrope_section[i] = (int32_t)sec->arr[i].inum;
        }
    }
    use_mrope_ = d.use_mrope != 0;
    hidden_ = d.hidden;
    vocab_ = d.vocab;
    if (model == "qwen2_5" && use_mrope_) throw ConfigurationError("model_name Qwen2.5 with an mrope checkpoint: use Qwen2.5-VL");

    // tied lm_head <=> the checkpoint carries no lm_head.weight (reference: src/layers/linear.cu:2244-2248)
    const std::vector<std::string> files = collect_safetensors_files(config_.prefill_model_path());
    if (files.empty())
        throw ConfigurationError("No model.safetensors or model-*-of-*.safetensors found in: " + config_.prefill_model_path());
    std::vector<std::unique_ptr<SafeTensorsFile>> maps;
    bool has_lm_head = false;
    const bool vlm = model == "qwen2_5_vl";
    for (const std::string& f : files) {
        maps.emplace_back(new SafeTensorsFile(f));
        for (const SafeTensorEntry& e : maps.back()->entries()) {
            std::string name = e.name;
            if (vlm && !map_vlm_weight_name(e.name, &name)) continue;
            if (name == "lm_head.weight") has_lm_head = true;
        }
    }
    d.tied_lm_head = has_lm_head ? 0 : 1;

    const std::vector<KvRequestConfig> reqs = config_.kv_requests();
    int32_t max_tokens = 1;
    for (const KvRequestConfig& r : reqs) max_tokens = std::max(max_tokens, r.max_tokens);
    d.max_prefill_tokens = std::min(max_tokens, 2048);
    d.max_response_tokens = config_.sampling_max_new_tokens() + 1;

    // Tensor parallel: one process per GPU, every process builds the same engine and issues the same requests.
    // Rank from the environment, device = $LOCAL_RANK (else runtime.device_id + rank), host exchange through files.
    const int32_t tp = config_.tensor_parallel();
    if (tp < 1 || tp > 8) throw ConfigurationError("runtime.tensor_parallel must be between 1 and 8");
    const int32_t tp_rank = tp > 1 ? config_.tp_rank() : 0;
    std::unique_ptr<TpRendezvous> meet;
    if (tp > 1) {
        if (tp_rank < 0 || tp_rank >= tp) throw ConfigurationError("tensor parallel rank (EFM_TP_RANK / RANK) must be in [0, runtime.tensor_parallel)");
        const char* local = std::getenv("LOCAL_RANK");
        device_id_ = local != nullptr && local[0] != 0 ? std::atoi(local) : device_id_ + tp_rank;
        meet.reset(new TpRendezvous(config_.tp_rendezvous(), tp_rank, tp));
    }
    efm_status st = efm_b200_create(&d, device_id_, tp_rank, tp, &ctx_);
    if (st != EFM_OK) {
        const std::string msg = std::string("backend creation failed: ") + efm_b200_last_error(nullptr);
        if (st == EFM_ERR_OUT_OF_MEMORY) throw OutOfMemoryError(msg);
        if (st == EFM_ERR_UNSUPPORTED || st == EFM_ERR_INVALID_ARGUMENT) throw ConfigurationError(msg);
        throw DeviceError(msg);
    }
    try {
        if (tp > 1) {
            std::vector<char> id(128, 0);
            if (tp_rank == 0) check(efm_b200_tp_unique_id(id.data()), "communicator id");
            id = meet->broadcast_from_root("nccl_id", id);
            if (id.size() != 128) throw ConfigurationError("tensor parallel rendezvous: malformed communicator id");
            check(efm_b200_tp_init(ctx_, id.data()), "communicator initialisation");
        }
        for (const auto& m : maps) {
            for (const SafeTensorEntry& e : m->entries()) {
                std::string name = e.name;
                if (vlm && !map_vlm_weight_name(e.name, &name)) continue;
                const int32_t code = dtype_code(e.dtype);
                if (code < 0) continue;
                st = efm_b200_set_weight(ctx_, name.c_str(), e.data, e.shape.data(), (int32_t)e.shape.size(), code, EFM_MEM_HOST);
                if (st != EFM_OK) throw ModelNotLoadedError(std::string("loading ") + name + ": " + efm_b200_last_error(ctx_));
            }
        }
        // Two checkpoints (reference: engine_factory.cpp:64-72): when decode_model_path names another directory, its
        // group-wise INT4 tensors (<linear>.qweight / .scaling_factors) become the decode pass's weights; prefill keeps
        // the bf16 ones.  Tensors of other kinds in that directory are ignored.
        const std::string decode_path = config_.decode_model_path();
        if (!decode_path.empty() && decode_path != config_.prefill_model_path()) {
            const std::vector<std::string> dfiles = collect_safetensors_files(decode_path);
            if (dfiles.empty()) throw ConfigurationError("No model.safetensors or model-*-of-*.safetensors found in decode path");
            for (const std::string& f : dfiles) {
                SafeTensorsFile dm(f);
                for (const SafeTensorEntry& e : dm.entries()) {
                    std::string name = e.name;
                    if (vlm && !map_vlm_weight_name(e.name, &name)) continue;
                    const int32_t code = dtype_code(e.dtype);
                    if (code < 0) continue;
                    st = efm_b200_set_decode_weight(ctx_, name.c_str(), e.data, e.shape.data(), (int32_t)e.shape.size(), code, EFM_MEM_HOST);
                    if (st == EFM_ERR_UNSUPPORTED) throw ConfigurationError(std::string("decode checkpoint, ") + name + ": " + efm_b200_last_error(ctx_));
                    if (st != EFM_OK) throw ModelNotLoadedError(std::string("loading decode weight ") + name + ": " + efm_b200_last_error(ctx_));
                }
            }
        }
        st = efm_b200_finalize_weights(ctx_);
        if (st != EFM_OK) throw ModelNotLoadedError(std::string("checkpoint incomplete: ") + efm_b200_last_error(ctx_));
        maps.clear();

        KVGeometry geo;
        geo.num_layers = d.num_layers;
        geo.kv_heads = d.kv_heads;
        geo.head_dim = d.head_dim;
        geo.dtype = DType::BFloat16;
        kv_manager_ = std::make_shared<KVManager>(reqs, geo, attn, device_id_, std::make_shared<BackendKVAllocator>(ctx_));
        scheduler_.reset(new Scheduler(kv_manager_, config_.sampling_max_new_tokens()));
        if (tp > 1) {      // decode all-reduces inside the GEMVs over peer memory: exchange the buffer handles, then a barrier
            std::vector<char> mine(64, 0);
            check(efm_b200_tp_peer_export(ctx_, mine.data()), "peer buffer export");
            const std::vector<std::vector<char>> all = meet->all_gather("peer", mine);
            std::vector<char> flat;
            for (const auto& h : all) {
                if (h.size() != 64) throw ConfigurationError("tensor parallel rendezvous: malformed peer handle");
                flat.insert(flat.end(), h.begin(), h.end());
            }
            check(efm_b200_tp_peer_import(ctx_, flat.data(), tp), "peer buffer import");
            meet->barrier("ready");
        }

        efm_sampling s;
        std::memset(&s, 0, sizeof(s));
        s.temperature = config_.sampling_temperature();
        s.top_p = config_.sampling_top_p();
        s.top_k = config_.sampling_top_k();
        s.seed = config_.sampling_seed();
        check(efm_b200_set_sampling(ctx_, &s), "sampling configuration");
        // short prompts are launch-bound: one captured graph per (request id, prompt length), as the reference does
        // (standard_engine.cpp:568-770)
        check(efm_b200_set_prefill_graph(ctx_, use_graph_ ? 1 : 0), "prefill graph selection");
        compact_ = CompactVocab(config_);
        const std::string pa = config_.prefill_attention();
        if (pa == "int8") check(efm_b200_set_prefill_attention(ctx_, 1), "prefill attention selection");
        else if (pa != "bf16") throw ConfigurationError("runtime.prefill_attention must be \"bf16\" or \"int8\", got " + pa);
    } catch (...) {
        efm_b200_destroy(ctx_);
        ctx_ = nullptr;
        throw;
    }
}

StandardEngine::~StandardEngine() {
    if (ctx_ != nullptr) efm_b200_destroy(ctx_);
}

void StandardEngine::warmup() {
    const KVManagerStatus st = kv_manager_->get_status();
    for (const KVSlotStatus& slot : st.slots) {
        if (!slot.prefix_token_ids.empty()) {
            const int32_t n = (int32_t)slot.prefix_token_ids.size();
            std::vector<int32_t> pos;
            if (use_mrope_) {       // a text prefix: the same running index on all three axes
                pos.resize(3 * (size_t)n);
                for (int r = 0; r < 3; ++r)
                    for (int32_t i = 0; i < n; ++i) pos[(size_t)r * n + i] = i;
            }
            const std::vector<int32_t> prefix_ids = compact_.remap_required_token_ids(slot.prefix_token_ids, "kvcache prefix_token_ids");
            check(efm_b200_prefill(ctx_, slot.request_id, prefix_ids.data(), n, 0, nullptr, 0, -1, EFM_MEM_HOST,
                                   use_mrope_ ? pos.data() : nullptr, 0),
                  "prefix prefill");
        }
        if (use_graph_) check(efm_b200_capture_decode(ctx_, slot.request_id), "decode graph capture");
    }
    check(efm_b200_synchronize(ctx_), "warmup");
}

void StandardEngine::build_positions(const Request& request, const Context& ctx, std::vector<int32_t>* pos_out, int32_t last_pos[3]) const {
    if (!use_mrope_) return;
    std::vector<int32_t>& pos = *pos_out;
    const int32_t S = ctx.seq_len, P = ctx.prefix_size, n = ctx.prefill_tokens;
    pos.resize(3 * (size_t)n);
    int32_t global_max = 0;
    if (request.has_position_ids()) {
        const Tensor& t = request.position_ids();
        if (t.shape().size() != 2 || t.shape()[0] != 3 || t.shape()[1] != S)
            throw InvalidRequestError("position_ids must have shape [3, seq_len]");
        if (t.dtype() != DType::Int32 && t.dtype() != DType::Int64) throw InvalidRequestError("position_ids must be int32 or int64");
        const size_t esz = get_dtype_size(t.dtype());
        std::vector<char> host(3 * (size_t)S * esz);
        if (std::get<0>(t.device()) == Device::GPU) {
            if (cudaMemcpy(host.data(), t.data_ptr(), host.size(), cudaMemcpyDeviceToHost) != cudaSuccess)
                throw DeviceError("copying position_ids to the host failed");
        } else {
            std::memcpy(host.data(), t.data_ptr(), host.size());
        }
        for (int r = 0; r < 3; ++r)
            for (int32_t i = 0; i < S; ++i) {
                int64_t v;
                if (esz == 4) { int32_t x; std::memcpy(&x, host.data() + ((size_t)r * S + i) * 4, 4); v = x; }
                else std::memcpy(&v, host.data() + ((size_t)r * S + i) * 8, 8);
                global_max = std::max<int32_t>(global_max, (int32_t)v);
                if (i >= P) pos[(size_t)r * n + (i - P)] = (int32_t)v;
            }
    } else {
        for (int r = 0; r < 3; ++r)
            for (int32_t i = 0; i < n; ++i) pos[(size_t)r * n + i] = P + i;
        global_max = S - 1;
    }
    // decode positions start one past the last prefill position on every axis
    // (reference: Qwen2_5::prepare_decode_position_ids, qwen2_5.cpp:932-955)
    for (int r = 0; r < 3; ++r)
        last_pos[r] = request.has_mrope_last_pos() && request.mrope_last_pos().size() >= 3 ? request.mrope_last_pos()[r] : global_max;
}

namespace {
// small integer tensor (int32 / int64, host or device) -> host int32 values
std::vector<int32_t> read_int_tensor(const Tensor& t, const char* what) {
    if (t.dtype() != DType::Int32 && t.dtype() != DType::Int64) throw InvalidRequestError(std::string(what) + " must be int32 or int64");
    size_t n = 1;
    for (int64_t d : t.shape()) n *= (size_t)std::max<int64_t>(d, 0);
    const size_t esz = get_dtype_size(t.dtype());
    std::vector<char> host(n * esz);
    if (n == 0) return {};
    if (std::get<0>(t.device()) == Device::GPU) {
        if (cudaMemcpy(host.data(), t.data_ptr(), host.size(), cudaMemcpyDeviceToHost) != cudaSuccess)
            throw DeviceError(std::string("copying ") + what + " to the host failed");
    } else {
        std::memcpy(host.data(), t.data_ptr(), host.size());
    }
    std::vector<int32_t> out(n);
    for (size_t i = 0; i < n; ++i) {
        if (esz == 4) std::memcpy(&out[i], host.data() + i * 4, 4);
        else { int64_t v; std::memcpy(&v, host.data() + i * 8, 8); out[i] = (int32_t)v; }
    }
    return out;
}
const Tensor* find_input(const TensorRefMap& inputs, const char* name) {
    auto it = inputs.find(name);
    return it != inputs.end() && it->second != nullptr && !it->second->empty() ? it->second : nullptr;
}
}  // namespace

TensorMap StandardEngine::stage_outputs(int32_t response_index) {
    TensorMap out;
    void* lbuf = std::malloc((size_t)vocab_ * sizeof(float));
    void* tbuf = std::malloc(sizeof(int32_t));
    if (lbuf == nullptr || tbuf == nullptr) { std::free(lbuf); std::free(tbuf); throw OutOfMemoryError("stage outputs"); }
    Tensor logits = Tensor::adopt(lbuf, {1, (int64_t)vocab_}, DType::Float32, Device::CPU, 0, MemoryOwnership::OwnCpuMalloc);
    Tensor token = Tensor::adopt(tbuf, {1}, DType::Int32, Device::CPU, 0, MemoryOwnership::OwnCpuMalloc);
    check(efm_b200_read_logits(ctx_, static_cast<float*>(logits.data_ptr()), vocab_), "reading logits");
    check(efm_b200_read_tokens(ctx_, static_cast<int32_t*>(token.data_ptr()), response_index, 1), "reading the sampled token");
    if (compact_.enabled()) {
        std::vector<int32_t> one(1, *static_cast<int32_t*>(token.data_ptr()));
        one = compact_.restore_token_ids(one, "stage next_token");
        *static_cast<int32_t*>(token.data_ptr()) = one[0];
    }
    out.emplace("logits", std::move(logits));
    out.emplace("next_token", std::move(token));
    return out;
}

TensorMap StandardEngine::run_stage(int32_t request_id, const std::string& stage_name, const TensorRefMap& inputs) {
    const double t0 = now_ms();
    stage_metrics_.clear();
    if (stage_name == "prefill") {
        const Tensor* ids_t = find_input(inputs, "token_ids");
        if (ids_t == nullptr) throw InvalidRequestError("prefill stage needs token_ids");
        const std::vector<int32_t> ids = read_int_tensor(*ids_t, "token_ids");
        const Tensor* emb = find_input(inputs, "embedding");
        const Tensor* pid = find_input(inputs, "position_ids");
        const Tensor* eid = find_input(inputs, "embed_token_id");
        const Tensor* mlp = find_input(inputs, "mrope_last_pos");
        const int32_t embed_token_id = eid != nullptr ? read_int_tensor(*eid, "embed_token_id").at(0) : -1;
        std::unique_ptr<Request> req;
        if (emb != nullptr && pid != nullptr && mlp != nullptr)
            req.reset(new Request(request_id, ids, *emb, embed_token_id, *pid, read_int_tensor(*mlp, "mrope_last_pos")));
        else if (emb != nullptr && pid != nullptr) req.reset(new Request(request_id, ids, *emb, embed_token_id, *pid));
        else if (emb != nullptr) req.reset(new Request(request_id, ids, *emb, embed_token_id));
        else req.reset(new Request(request_id, ids));
        const Request& request = *req;
        Context ctx = scheduler_->create_context(request);
        if (ctx.prefill_tokens <= 0) throw InvalidRequestError("prefill stage: nothing beyond the resident prefix");
        const std::vector<int32_t> model_ids = compact_.remap_token_ids(request.token_ids(), "stage token_ids");
        const void* embeds = nullptr;
        int32_t n_embeds = 0, embeds_mem = EFM_MEM_HOST, model_embed_id = request.embed_token_id();
        if (request.has_embedding()) {
            const Tensor& e = request.embedding();
            if (e.dtype() != DType::BFloat16 || e.shape().size() != 2 || e.shape()[1] != hidden_)
                throw InvalidRequestError("embedding must be bf16 [N, hidden_size]");
            if (request.embed_token_id() < 0) throw InvalidRequestError("embedding given without embed_token_id");
            embeds = e.data_ptr();
            n_embeds = (int32_t)e.shape()[0];
            embeds_mem = std::get<0>(e.device()) == Device::GPU ? EFM_MEM_DEVICE : EFM_MEM_HOST;
            model_embed_id = compact_.remap_embed_token_id(request.embed_token_id(), n_embeds);
        }
        std::vector<int32_t> pos;
        int32_t last_pos[3] = {0, 0, 0};
        if (use_mrope_ && !request.has_position_ids() && pid != nullptr) throw InvalidRequestError("position_ids need an embedding tensor in this API");
        build_positions(request, ctx, &pos, last_pos);
        check(efm_b200_prefill(ctx_, ctx.request_id, model_ids.data() + ctx.prefix_size, ctx.prefill_tokens, ctx.prefix_size, embeds,
                               n_embeds, model_embed_id, embeds_mem, use_mrope_ ? pos.data() : nullptr, 1),
              "prefill stage");
        StageState& st = stage_state_[request_id];
        st.kv_len = ctx.seq_len;
        for (int r = 0; r < 3; ++r) st.next_pos[r] = last_pos[r] + 1;
        st.primed = true;
        TensorMap out = stage_outputs(0);
        stage_metrics_ = {{"stage_ms", now_ms() - t0}, {"kv_len", (double)st.kv_len}, {"stage_tokens", (double)ctx.prefill_tokens}};
        return out;
    }
    if (stage_name == "decode") {
        auto it = stage_state_.find(request_id);
        if (it == stage_state_.end() || !it->second.primed) throw InvalidRequestError("decode stage before a prefill stage for request_id " + std::to_string(request_id));
        StageState& st = it->second;
        const KVSlotStatus* slot = kv_manager_->find_slot(request_id);
        if (slot == nullptr || st.kv_len + 1 > slot->max_tokens)
            throw InvalidRequestError("decode stage: the KV slot of request_id " + std::to_string(request_id) + " is full");
        // every call binds the slot afresh and writes its sample to response position 1
        check(efm_b200_decode_begin(ctx_, request_id, st.kv_len, st.next_pos, 1), "decode stage setup");
        if (const Tensor* ids_t = find_input(inputs, "token_ids")) {
            std::vector<int32_t> feed = read_int_tensor(*ids_t, "token_ids");
            if (feed.size() != 1) throw InvalidRequestError("decode stage takes exactly one token");
            feed = compact_.remap_token_ids(feed, "stage token_ids");
            check(efm_b200_set_token(ctx_, feed[0]), "decode stage token");
        }
        check(efm_b200_decode_steps(ctx_, 1, use_graph_ ? 1 : 0), "decode stage");
        st.kv_len += 1;
        for (int r = 0; r < 3; ++r) st.next_pos[r] += 1;
        TensorMap out = stage_outputs(1);
        stage_metrics_ = {{"stage_ms", now_ms() - t0}, {"kv_len", (double)st.kv_len}, {"stage_tokens", 1.0}};
        return out;
    }
    throw ConfigurationError("run_stage('" + stage_name + "'): the token-generation engine serves the stages \"prefill\" and \"decode\"");
}

Response StandardEngine::generate(const Request& request) {
    metrics_.clear();
    Response response;
    const double t_start = now_ms();
    Context ctx = scheduler_->create_context(request);
    if (ctx.prefill_tokens <= 0) return response;       // nothing beyond the resident prefix

    std::unordered_set<int32_t> stop;
    if (!request.ignore_stop_tokens()) {
        for (int32_t id : config_.eos_token_ids()) stop.insert(id);
        for (int32_t id : config_.stop_token_ids()) stop.insert(id);
        for (int32_t id : request.stop_token_ids()) stop.insert(id);
    }

    // compact vocabulary: the model runs on compact ids, callers keep tokenizer ids (identity when disabled)
    const std::vector<int32_t> model_ids = compact_.remap_token_ids(request.token_ids(), "request token_ids");
    if (compact_.enabled() && !request.ignore_stop_tokens())
        (void)compact_.remap_token_ids(request.stop_token_ids(), "request stop_token_ids");      // a pruned stop id is an error
    const int32_t model_embed_token_id = request.has_embedding()
        ? compact_.remap_embed_token_id(request.embed_token_id(), request.embedding().shape().empty() ? -1 : request.embedding().shape()[0])
        : request.embed_token_id();

    // ---- request tensors -> what the backend takes --------------------------------------
    const void* embeds = nullptr;
    int32_t n_embeds = 0, embeds_mem = EFM_MEM_HOST;
    if (request.has_embedding()) {
        const Tensor& e = request.embedding();
        if (e.dtype() != DType::BFloat16) throw InvalidRequestError("embedding must be bf16");
        if (e.shape().size() != 2 || e.shape()[1] != hidden_)
            throw InvalidRequestError("embedding must have shape [N, hidden_size]");
        if (request.embed_token_id() < 0) throw InvalidRequestError("embedding given without embed_token_id");
        embeds = e.data_ptr();
        n_embeds = (int32_t)e.shape()[0];
        embeds_mem = std::get<0>(e.device()) == Device::GPU ? EFM_MEM_DEVICE : EFM_MEM_HOST;
    }
    std::vector<int32_t> pos;          // [3, prefill_tokens]
    int32_t last_pos[3] = {0, 0, 0};
    build_positions(request, ctx, &pos, last_pos);

    // ---- prefill ----------------------------------------------------------------------------
    const double t_prep = now_ms();
    check(efm_b200_event_record(ctx_, 0), "event");
    check(efm_b200_prefill(ctx_, ctx.request_id, model_ids.data() + ctx.prefix_size, ctx.prefill_tokens,
                           ctx.prefix_size, embeds, n_embeds, model_embed_token_id, embeds_mem,
                           use_mrope_ ? pos.data() : nullptr, 1),
          "prefill");
    check(efm_b200_event_record(ctx_, 1), "event");
    ctx.generated_tokens = 1;

    // ---- decode -----------------------------------------------------------------------------
    const int32_t decode_steps = ctx.max_generated_tokens - 1;
    const double t_dec_host = now_ms();
    if (decode_steps > 0) {
        int32_t first_pos[3] = {last_pos[0] + 1, last_pos[1] + 1, last_pos[2] + 1};
        check(efm_b200_decode_begin(ctx_, ctx.request_id, ctx.seq_len, first_pos, 1), "decode setup");
        check(efm_b200_decode_steps(ctx_, decode_steps, use_graph_ ? 1 : 0), "decode");
        ctx.generated_tokens += decode_steps;
    }
    check(efm_b200_event_record(ctx_, 2), "event");
    const double t_dec_host_end = now_ms();

    // ---- one copy back, stop-token cut on the host -------------------------------------------
    std::vector<int32_t> host_tokens((size_t)ctx.generated_tokens);
    const double t_copy = now_ms();
    check(efm_b200_read_tokens(ctx_, host_tokens.data(), 0, ctx.generated_tokens), "reading response tokens");
    const double t_copy_end = now_ms();
    const int32_t executed = ctx.generated_tokens;
    if (compact_.enabled()) host_tokens = compact_.restore_token_ids(host_tokens, "response token_ids");   // stop ids are tokenizer ids
    const double t_stop = now_ms();
    if (!stop.empty())
        for (size_t i = 0; i < host_tokens.size(); ++i)
            if (stop.count(host_tokens[i])) { host_tokens.resize(i + 1); break; }
    const double t_stop_end = now_ms();
    const int32_t returned = (int32_t)host_tokens.size();
    response.token_ids().swap(host_tokens);

    float prefill_ms = 0.f, decode_ms = 0.f;
    check(efm_b200_event_elapsed_ms(ctx_, 0, 1, &prefill_ms), "event");
    check(efm_b200_event_elapsed_ms(ctx_, 1, 2, &decode_ms), "event");
    const double exec_steps = std::max(0, executed - 1), ret_steps = std::max(0, returned - 1);
    const double total = (double)prefill_ms + (double)decode_ms;
    // key set of the reference's make_generate_metrics_map (standard_engine.cpp:462-507)
    metrics_ = {
        {"prefill_ms", prefill_ms},
        {"decode_ms", decode_ms},
        {"total_stage_ms", total},
        {"decode_step_avg_ms", exec_steps > 0 ? decode_ms / exec_steps : 0.0},
        {"generated_tokens_total", (double)returned},
        {"decode_steps", exec_steps},
        {"prefill_prepare_host_ms", t_prep - t_start},
        {"prefill_model_ms", prefill_ms},
        {"prefill_sampler_ms", 0.0},                       // sampled inside the prefill launch sequence
        {"decode_prepare_host_ms", 0.0},
        {"decode_graph_replay_ms", use_graph_ ? (double)decode_ms : 0.0},
        {"decode_model_ms", use_graph_ ? 0.0 : (double)decode_ms},
        {"decode_sampler_ms", 0.0},                        // part of the step
        {"decode_finalize_ms", 0.0},                       // part of the step
        {"decode_launch_host_ms", t_dec_host_end - t_dec_host},
        {"stop_check_host_ms", t_stop_end - t_stop},
        {"response_copy_ms", t_copy_end - t_copy},
        {"tokens_per_second", total > 0 ? returned * 1000.0 / total : 0.0},
        {"decode_tokens_per_second", decode_ms > 0 ? ret_steps * 1000.0 / decode_ms : 0.0},
        {"executed_generated_tokens_total", (double)executed},
        {"returned_generated_tokens_total", (double)returned},
        {"cuda_graph_enabled", use_graph_ ? 1.0 : 0.0},
        {"lm_head_top1_enabled", 1.0},
        {"lm_head_top1_decode_steps", exec_steps},
        {"response_tokens_capacity", (double)ctx.max_generated_tokens},
    };
    return response;
}

}  // namespace edge_fm
