// Token-generation engine over the B200 backend: owns the backend context, the KV manager,
// the scheduler and the generate loop.  Host-side counterpart of the reference's StandardEngine
// (src/engine/tasks/token_generation/cuda/standard_engine.{h,cpp}); all device work goes
// through the C ABI in include/efm_b200.h.
#pragma once
#include <edge-fm/core.h>

#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "compact_vocab.h"
#include "config.h"
#include "kv_manager.h"
#include "scheduler.h"

struct efm_b200_ctx;

namespace edge_fm {

class StandardEngine {
public:
    explicit StandardEngine(const EngineConfig& config);
    ~StandardEngine();
    StandardEngine(const StandardEngine&) = delete;
    StandardEngine& operator=(const StandardEngine&) = delete;

    // Prefill every slot's fixed prefix and capture the decode graph (run by the facade's ctor).
    void warmup();
    Response generate(const Request& request);
    std::unordered_map<std::string, double> last_generate_metrics() const { return metrics_; }

    // Tensor-in / tensor-out stage calls on the token-generation path (the reference declares them on every engine,
    // include/edge-fm/edge-fm.h:57-75; its own token-generation engine leaves them to the refusing base class).
    //   "prefill": token_ids (int32 / int64, [S] or [1, S]; must begin with the slot's fixed prefix), optional
    //              embedding (bf16 [N, hidden]) + embed_token_id (int [1]), position_ids ([3, S]), mrope_last_pos ([3])
    //   "decode" : optional token_ids ([1]: the token to feed; default: the one the previous stage sampled)
    // Both return {"logits": fp32 [1, vocab] (host), "next_token": int32 [1] (host)}; the KV rows of request_id stay
    // in the engine's own slot between calls.
    TensorMap run_stage(int32_t request_id, const std::string& stage_name, const TensorRefMap& inputs);
    std::unordered_map<std::string, double> last_stage_metrics() const { return stage_metrics_; }
    void* backend_handle() const { return ctx_; }

private:
    void load_weights();
    void check(int32_t status, const char* what) const;    // backend status -> edge_fm exception
    // M-RoPE prefill positions [3, prefill_tokens] and the last position per axis (text models: untouched)
    void build_positions(const Request& request, const Context& ctx, std::vector<int32_t>* pos, int32_t last_pos[3]) const;
    TensorMap stage_outputs(int32_t response_index);

    struct StageState { int32_t kv_len = 0; int32_t next_pos[3] = {0, 0, 0}; bool primed = false; };
    std::unordered_map<int32_t, StageState> stage_state_;
    std::unordered_map<std::string, double> stage_metrics_;
    int32_t vocab_ = 0;

    EngineConfig config_;
    efm_b200_ctx* ctx_ = nullptr;
    int32_t device_id_ = 0;
    int32_t hidden_ = 0;
    bool use_mrope_ = false;
    bool use_graph_ = false;
    std::shared_ptr<KVManager> kv_manager_;
    std::unique_ptr<Scheduler> scheduler_;
    CompactVocab compact_;                // identity unless compact_vocab.enabled
    std::unordered_map<std::string, double> metrics_;
};

}  // namespace edge_fm
