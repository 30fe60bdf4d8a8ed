#include "config.h"

#include <cstdlib>

#include <edge-fm/core.h>
#include <sys/stat.h>

#include <algorithm>
#include <cctype>
#include <fstream>
#include <sstream>

namespace edge_fm {

namespace {

// Defaults: the key set and values of the reference's engine_default.json.
const char* kDefaults = R"JSON({
  "model_name": "",
  "runtime": {"num_threads": 0, "use_cuda_graph": false, "device": "cuda", "device_id": 0, "hw_profile": ""},
  "operator_impl_table_path": "",
  "prefill_model_path": "",
  "decode_model_path": null,
  "speculative": {"enabled": false, "algorithm": "EAGLE3", "draft_model": {"path": ""}},
  "kvcache": {"dtype": "fp16", "attention_type": "mha",
              "requests": [{"request_id": 0, "prefix_token_ids": [], "max_tokens": 4096}]},
  "sampling": {"max_new_tokens": 256, "temperature": 1.0, "top_k": 1, "top_p": 1.0, "seed": 0, "stop_token_ids": []},
  "tuning": {"enabled": false},
  "metrics": {"enabled": false, "log_path": null}
})JSON";

json::Value load_json(const std::string& path, const std::string& what) {
    std::ifstream f(path);
    if (!f.is_open()) throw ConfigurationError("Cannot open " + what + ": " + path);
    std::ostringstream ss;
    ss << f.rdbuf();
    try {
        return json::parse(ss.str());
    } catch (const std::exception& e) {
        throw ConfigurationError("Failed to parse " + what + ": " + e.what());
    }
}

bool is_dir(const std::string& p) {
    struct stat st;
    return stat(p.c_str(), &st) == 0 && S_ISDIR(st.st_mode);
}
bool is_file(const std::string& p) {
    struct stat st;
    return stat(p.c_str(), &st) == 0 && S_ISREG(st.st_mode);
}

void validate_model_path(const std::string& path, const std::string& name) {
    if (!is_dir(path)) throw ConfigurationError(name + " does not exist or is not a directory: " + path);
    if (!is_file(path + "/config.json")) throw ConfigurationError("config.json does not exist in " + name + ": " + path);
}

}  // namespace

std::string EngineConfig::normalize_model_name(const std::string& raw) {
    std::string n;
    for (unsigned char ch : raw) {
        if (std::isalnum(ch)) n.push_back((char)std::tolower(ch));
        else if (ch == '_' || ch == '.' || ch == '-' || ch == ' ' || ch == '/') n.push_back('_');
    }
    if (n == "qwen2_5" || n == "qwen25" || n == "qwen2") return "qwen2_5";
    if (n == "qwen2_5_vl" || n == "qwen25_vl" || n == "qwen2_vl" || n == "qwen25vl" || n == "qwen2_5vl" || n == "qwen2vl")
        return "qwen2_5_vl";
    if (n == "smolvla" || n == "smol_vla" || n == "lerobot_smolvla" || n == "lerobot_smol_vla") return "smolvla";
    return n;
}

EngineConfig::EngineConfig(const std::string& config_path) {
    config_ = json::parse(kDefaults);
    {
        const size_t slash = config_path.find_last_of('/');
        config_dir_ = slash == std::string::npos ? std::string(".") : (slash == 0 ? std::string("/") : config_path.substr(0, slash));
    }
    const json::Value user = load_json(config_path, "configuration file");
    if (!user.is_object()) throw ConfigurationError("configuration file must hold a JSON object");
    for (const auto& kv : user.obj) config_.set(kv.first, kv.second);     // shallow: sections replace wholesale

    std::string task = config_.get_string("task", "");
    std::transform(task.begin(), task.end(), task.begin(), [](unsigned char c) { return (char)std::tolower(c); });
    if (!task.empty() && task != "token_generation" && task != "trajectory_planning")
        throw ConfigurationError("Unsupported task in engine config: " + task + " (this build provides token_generation and trajectory_planning)");
    const std::string path = prefill_model_path();
    if (path.empty()) throw ConfigurationError("prefill_model_path is required in configuration");
    validate_model_path(path, "prefill_model_path");
    const json::Value* dec = config_.find("decode_model_path");
    if (dec == nullptr || !dec->is_string() || dec->str.empty()) {
        json::Value v;
        v.type = json::Value::String;
        v.str = path;
        config_.set("decode_model_path", v);
    } else {
        validate_model_path(dec->str, "decode_model_path");
    }
    const json::Value spec = section("speculative");
    if (spec.get_bool("enabled", false)) throw ConfigurationError("speculative decoding is not supported");
}

json::Value EngineConfig::section(const std::string& name) const {
    const json::Value* v = config_.find(name);
    if (v == nullptr || !v->is_object()) { json::Value e; e.type = json::Value::Object; return e; }
    return *v;
}

std::string EngineConfig::task() const {
    std::string t = config_.get_string("task", "");
    std::transform(t.begin(), t.end(), t.begin(), [](unsigned char c) { return (char)std::tolower(c); });
    if (!t.empty()) return t;
    // no task written: a policy model name implies the planner task, as in the reference
    // (tests/engine/test_planner_policy_api.py, "model name without task infers trajectory planning")
    return normalize_model_name(model_name()) == "smolvla" ? std::string("trajectory_planning") : std::string("token_generation");
}
std::string EngineConfig::model_name() const { return config_.get_string("model_name", ""); }
std::string EngineConfig::prefill_model_path() const { return config_.get_string("prefill_model_path", ""); }
std::string EngineConfig::decode_model_path() const { return config_.get_string("decode_model_path", ""); }

std::string EngineConfig::resolved_model_name() const {
    const std::string n = normalize_model_name(model_name());
    if (n == "qwen2_5" || n == "qwen2_5_vl") return n;
    throw ConfigurationError(
        "Unsupported or missing model_name in engine config. Supported values include: Qwen2.5, qwen2_5, "
        "Qwen2.5-VL, qwen2_5_vl");
}

json::Value EngineConfig::prefill_model_config() const {
    json::Value cfg = load_json(prefill_model_path() + "/config.json", "config.json file");
    const json::Value* text = cfg.find("text_config");
    if (text != nullptr && text->is_object()) return *text;
    return cfg;
}

std::string EngineConfig::runtime_device() const { return section("runtime").get_string("device", "cuda"); }
int32_t EngineConfig::runtime_device_id() const { return (int32_t)section("runtime").get_int("device_id", 0); }
bool EngineConfig::use_cuda_graph() const { return section("runtime").get_bool("use_cuda_graph", false); }
std::string EngineConfig::tp_rendezvous() const {
    const std::string v = section("runtime").get_string("tp_rendezvous", "");
    if (!v.empty()) return v;
    const char* e = std::getenv("EFM_TP_RENDEZVOUS");
    return e != nullptr ? std::string(e) : std::string();
}
int32_t EngineConfig::tp_rank() const {
    for (const char* name : {"EFM_TP_RANK", "RANK"}) {
        const char* e = std::getenv(name);
        if (e != nullptr && e[0] != 0) return (int32_t)std::atoi(e);
    }
    return 0;
}
std::string EngineConfig::prefill_attention() const { return section("runtime").get_string("prefill_attention", "bf16"); }
int32_t EngineConfig::tensor_parallel() const { return (int32_t)section("runtime").get_int("tensor_parallel", 1); }
bool EngineConfig::lm_head_top1_enabled() const {
    const json::Value rt = section("runtime");
    const json::Value* v = rt.find("lm_head_top1");
    if (v != nullptr && v->is_bool()) return v->b;
    if (v != nullptr && v->is_object()) return v->get_bool("enabled", false);
    return rt.get_bool("lm_head_top1_enabled", false);
}
std::string EngineConfig::kvcache_dtype() const { return section("kvcache").get_string("dtype", "fp16"); }
std::string EngineConfig::kvcache_attention_type() const { return section("kvcache").get_string("attention_type", "mha"); }

std::vector<KvRequestConfig> EngineConfig::kv_requests() const {
    std::vector<KvRequestConfig> out;
    const json::Value kv = section("kvcache");
    const json::Value* reqs = kv.find("requests");
    if (reqs == nullptr || !reqs->is_array()) return out;
    for (const json::Value& r : reqs->arr) {
        if (!r.is_object()) continue;
        KvRequestConfig k;
        k.request_id = (int32_t)r.get_int("request_id", 0);
        k.max_tokens = (int32_t)r.get_int("max_tokens", 4096);
        const json::Value* p = r.find("prefix_token_ids");
        if (p != nullptr && p->is_array())
            for (const json::Value& e : p->arr)
                if (e.is_number()) k.prefix_token_ids.push_back((int32_t)e.inum);
        out.push_back(std::move(k));
    }
    return out;
}

float EngineConfig::sampling_temperature() const { return (float)section("sampling").get_double("temperature", 1.0); }
float EngineConfig::sampling_top_p() const { return (float)section("sampling").get_double("top_p", 1.0); }
int32_t EngineConfig::sampling_top_k() const { return (int32_t)section("sampling").get_int("top_k", 1); }
uint64_t EngineConfig::sampling_seed() const { return (uint64_t)section("sampling").get_int("seed", 0); }
int32_t EngineConfig::sampling_max_new_tokens() const {
    return std::max<int32_t>(1, (int32_t)section("sampling").get_int("max_new_tokens", 256));
}

std::vector<int32_t> EngineConfig::stop_token_ids() const {
    std::vector<int32_t> ids;
    const json::Value s = section("sampling");
    const json::Value* v = s.find("stop_token_ids");
    if (v != nullptr && v->is_array())
        for (const json::Value& e : v->arr)
            if (e.is_number() && e.is_int) ids.push_back((int32_t)e.inum);
    return ids;
}

std::vector<int32_t> EngineConfig::eos_token_ids() const {
    std::vector<int32_t> ids;
    const std::string p = prefill_model_path() + "/config.json";
    if (!is_file(p)) return ids;
    try {
        const json::Value cfg = load_json(p, "model config");
        const json::Value* v = cfg.find("eos_token_id");
        if (v == nullptr) return ids;
        if (v->is_number() && v->is_int) ids.push_back((int32_t)v->inum);
        else if (v->is_array())
            for (const json::Value& e : v->arr)
                if (e.is_number() && e.is_int) ids.push_back((int32_t)e.inum);
    } catch (...) {
    }
    return ids;
}

}  // namespace edge_fm
