// Engine configuration: built-in defaults shallow-merged with the user's JSON, plus the HF
// config.json of the checkpoint.  Same keys, defaults and normalisation rules as the
// reference's EngineConfig (src/engine/engine.cpp:115-138,202-255,267-277,470-532 and
// examples/config/base/engine_default.json); only the token_generation + cuda branch exists here.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "json.h"

namespace edge_fm {

struct KvRequestConfig {
    int32_t request_id = 0;
    std::vector<int32_t> prefix_token_ids;
    int32_t max_tokens = 4096;
};

class EngineConfig {
public:
    explicit EngineConfig(const std::string& config_path);

    const json::Value& root() const { return config_; }
    const std::string& config_dir() const { return config_dir_; }   // directory of the engine JSON
    json::Value compact_vocab() const { return section("compact_vocab"); }
    std::string task() const;                     // "token_generation" (default) | "trajectory_planning"
    std::string model_name() const;               // as written
    std::string resolved_model_name() const;      // "qwen2_5" | "qwen2_5_vl" (throws otherwise)
    std::string prefill_model_path() const;
    std::string decode_model_path() const;
    json::Value prefill_model_config() const;     // text_config unwrapped for VLM checkpoints

    std::string runtime_device() const;
    int32_t runtime_device_id() const;
    bool use_cuda_graph() const;
    int32_t tensor_parallel() const;              // runtime.tensor_parallel (new key, default 1)
    std::string tp_rendezvous() const;            // runtime.tp_rendezvous (new key) or $EFM_TP_RENDEZVOUS: fresh shared directory
    int32_t tp_rank() const;                      // $EFM_TP_RANK, else $RANK, else 0
    std::string prefill_attention() const;        // runtime.prefill_attention (new key): "bf16" (default) | "int8"
    bool lm_head_top1_enabled() const;            // accepted; the fused argmax is always on here
    std::string kvcache_dtype() const;
    std::string kvcache_attention_type() const;
    std::vector<KvRequestConfig> kv_requests() const;

    float sampling_temperature() const;
    float sampling_top_p() const;
    int32_t sampling_top_k() const;
    uint64_t sampling_seed() const;
    int32_t sampling_max_new_tokens() const;
    std::vector<int32_t> stop_token_ids() const;
    std::vector<int32_t> eos_token_ids() const;   // from the checkpoint's top-level config.json

    static std::string normalize_model_name(const std::string& raw);

private:
    json::Value section(const std::string& name) const;
    json::Value config_;
    std::string config_dir_;
};

}  // namespace edge_fm
