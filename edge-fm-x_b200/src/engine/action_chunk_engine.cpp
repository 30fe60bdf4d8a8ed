#include "action_chunk_engine.h"

#include <cctype>
#include <chrono>
#include <cmath>
#include <random>
#include <vector>

#include "efm_b200.h"
#include "safetensors.h"

namespace edge_fm {

namespace {

int64_t numel(const std::vector<int64_t>& shape) {
    int64_t n = 1;
    for (int64_t d : shape) n *= d;
    return n;
}

const Tensor& require_host(const TensorRefMap& inputs, const std::string& name, DType dtype, int64_t count) {
    auto it = inputs.find(name);
    if (it == inputs.end() || it->second == nullptr) throw InvalidRequestError("plan() input is missing: " + name);
    const Tensor& t = *it->second;
    if (std::get<0>(t.device()) != Device::CPU) throw InvalidRequestError("plan() input must be a host tensor: " + name);
    if (t.dtype() != dtype) throw InvalidRequestError("plan() input has the wrong dtype: " + name);
    if (numel(t.shape()) != count) throw InvalidRequestError("plan() input has the wrong number of elements: " + name);
    return t;
}

std::string lower_alnum(const std::string& raw) {      // the reference's normalize_planner_string (:80-91)
    std::string out;
    for (unsigned char ch : raw) {
        if (std::isalnum(ch)) out.push_back((char)std::tolower(ch));
        else if (ch == '_' || ch == '-' || ch == '.' || ch == ' ' || ch == '/') out.push_back('_');
    }
    return out;
}

}  // namespace

ActionChunkEngine::ActionChunkEngine(const EngineConfig& config) {
    if (config.runtime_device() != "cuda") throw ConfigurationError("trajectory_planning runs on runtime.device = cuda only");
    const json::Value* pl = config.root().find("planner");
    json::Value planner;
    planner.type = json::Value::Object;
    if (pl != nullptr && pl->is_object()) planner = *pl;
    const std::string type = lower_alnum(planner.get_string("type", "iterative_denoise"));
    if (type != "iterative_denoise") throw ConfigurationError("Unsupported planner.type: " + type + " (iterative_denoise only)");
    const std::string sampler = lower_alnum(planner.get_string("sampler", "euler_flow"));
    if (sampler != "euler_flow") throw ConfigurationError("Unsupported iterative_denoise sampler: " + sampler);
    state_name_ = planner.get_string("state_tensor", "current_actions");
    output_name_ = planner.get_string("output_tensor", "trajectory");
    noise_sigma_ = (float)planner.get_double("noise_sigma", 1.0);
    seed_ = (uint32_t)planner.get_int("seed", 0);

    const json::Value m = config.prefill_model_config();          // the checkpoint's config.json
    auto need = [&](const char* key) -> int32_t {
        if (!m.contains(key)) throw ConfigurationError(std::string("config.json of the policy lacks ") + key);
        return (int32_t)m.get_int(key, 0);
    };
    efm_vla_desc d{};
    d.struct_size = (int32_t)sizeof(d);
    d.image_size = need("image_size"); d.patch = need("patch"); d.vit_layers = need("vit_layers"); d.vit_hidden = need("vit_hidden");
    d.vit_heads = need("vit_heads"); d.vit_mlp = need("vit_mlp"); d.shuffle = need("shuffle"); d.n_images = need("n_images");
    d.hidden = need("hidden"); d.layers = need("layers"); d.q_heads = need("q_heads"); d.kv_heads = need("kv_heads");
    d.head_dim = need("head_dim"); d.mlp = need("mlp"); d.vocab = need("vocab"); d.lang_tokens = need("lang_tokens");
    d.expert_hidden = need("expert_hidden"); d.expert_mlp = need("expert_mlp"); d.state_dim = need("state_dim");
    d.action_dim = need("action_dim"); d.chunk = need("chunk");
    d.steps = (int32_t)planner.get_int("num_steps", m.get_int("steps", 10));
    d.rope_theta = (float)m.get_double("rope_theta", 1e5);
    d.rms_eps = (float)m.get_double("rms_eps", 1e-5);
    d.ln_eps = (float)m.get_double("ln_eps", 1e-6);
    // the device loop is x += dt * v with dt = -1 / num_steps from t = 1: refuse a configuration that asks for another schedule
    if (planner.contains("dt") && std::abs(planner.get_double("dt", 0.0) + 1.0 / d.steps) > 1e-6)
        throw ConfigurationError("planner.dt must be -1 / num_steps for this policy");
    if (const json::Value* shape = planner.find("trajectory_shape")) {
        if (!shape->is_array() || shape->arr.size() != 2 || (int64_t)shape->arr[0].num != d.chunk ||
            (int64_t)shape->arr[1].num != d.action_dim)
            throw ConfigurationError("planner.trajectory_shape must be [chunk, action_dim] of the policy");
        has_shape_ = true;
    }
    n_images_ = d.n_images; image_size_ = d.image_size; lang_tokens_ = d.lang_tokens; state_dim_ = d.state_dim;
    chunk_ = d.chunk; action_dim_ = d.action_dim; steps_ = d.steps;

    efm_status st = efm_b200_vla_create(&d, config.runtime_device_id(), &vla_);
    if (st != EFM_OK) throw ModelNotLoadedError("cannot create the action-chunk policy on the GPU (status " + std::to_string((int)st) + ")");
    try {
        for (const std::string& file : collect_safetensors_files(config.prefill_model_path())) {
            SafeTensorsFile f(file);
            for (const SafeTensorEntry& e : f.entries()) {
                if (e.dtype != "BF16") throw ModelNotLoadedError("policy tensors must be bf16: " + e.name);
                st = efm_b200_vla_set_weight(vla_, e.name.c_str(), e.data, e.shape.data(), (int32_t)e.shape.size(), EFM_BF16, EFM_MEM_HOST);
                if (st != EFM_OK) throw ModelNotLoadedError(std::string("policy weight rejected: ") + efm_b200_vla_last_error(vla_));
            }
        }
        st = efm_b200_vla_finalize_weights(vla_);
        if (st != EFM_OK) throw ModelNotLoadedError(std::string("policy checkpoint incomplete: ") + efm_b200_vla_last_error(vla_));
    } catch (...) {
        efm_b200_vla_destroy(vla_);
        vla_ = nullptr;
        throw;
    }
}

ActionChunkEngine::~ActionChunkEngine() {
    if (vla_ != nullptr) efm_b200_vla_destroy(vla_);
}

TensorMap ActionChunkEngine::plan(int32_t, const TensorRefMap& inputs) {
    const auto t0 = std::chrono::steady_clock::now();
    const Tensor& images = require_host(inputs, "images", DType::Float32, (int64_t)n_images_ * 3 * image_size_ * image_size_);
    const Tensor& ids = require_host(inputs, "lang_tokens", DType::Int32, lang_tokens_);
    const Tensor& state = require_host(inputs, "state", DType::Float32, state_dim_);
    const int64_t count = (int64_t)chunk_ * action_dim_;
    std::vector<float> drawn;
    const float* noise = nullptr;
    auto it = inputs.find(state_name_);
    if (it != inputs.end() && it->second != nullptr) {
        noise = static_cast<const float*>(require_host(inputs, state_name_, DType::Float32, count).data_ptr());
    } else {
        if (!has_shape_)
            throw InvalidRequestError("iterative_denoise planner requires input state tensor or planner.trajectory_shape: " + state_name_);
        drawn.assign((size_t)count, 0.0f);
        if (noise_sigma_ != 0.0f) {
            std::mt19937 rng(seed_);
            std::normal_distribution<float> normal(0.0f, noise_sigma_);
            for (float& v : drawn) v = normal(rng);
        }
        noise = drawn.data();
    }
    std::vector<float> actions((size_t)count);
    const efm_status st = efm_b200_vla_chunk(vla_, static_cast<const float*>(images.data_ptr()), static_cast<const int32_t*>(ids.data_ptr()),
                                             static_cast<const float*>(state.data_ptr()), noise, EFM_MEM_HOST, actions.data());
    if (st != EFM_OK) throw InternalError(std::string("action chunk failed: ") + efm_b200_vla_last_error(vla_));
    TensorMap out;
    const std::vector<int64_t> shape{chunk_, action_dim_};
    out[output_name_] = Tensor::clone_from(actions.data(), shape, DType::Float32, Device::CPU, 0, Device::CPU, 0, MemoryOwnership::OwnCpuMalloc);
    if (output_name_ != "trajectory")
        out["trajectory"] = Tensor::clone_from(actions.data(), shape, DType::Float32, Device::CPU, 0, Device::CPU, 0, MemoryOwnership::OwnCpuMalloc);
    metrics_ = {{"stage_calls", (double)(steps_ + 1)}, {"plan_steps", (double)steps_},
                {"plan_ms", std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count()}};
    return out;
}

}  // namespace edge_fm
