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

private:
    void load_weights();
    void check(int32_t status, const char* what) const;    // backend status -> edge_fm exception

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
