// edge_fm::EdgeFM facade: configuration -> engine -> warmup; generate() forwards.
// Reference: src/edge-fm.cpp:12-22 (the constructor runs warmup) and the base Engine's
// refusal of planner calls the configured task does not provide (src/engine/engine.cpp:551-564); the stage calls
// (run_stage / prefill / decode) are served by the token-generation engine.
// task = trajectory_planning builds the action-chunk engine instead and serves plan().
#include <edge-fm/edge-fm.h>

#include "engine/action_chunk_engine.h"
#include "engine/config.h"
#include "engine/standard_engine.h"

namespace edge_fm {

struct EdgeFM::Impl {
    std::unique_ptr<StandardEngine> engine;        // task = token_generation
    std::unique_ptr<ActionChunkEngine> planner;    // task = trajectory_planning
};

EdgeFM::EdgeFM(const std::string& config_path) : impl_(new Impl()) {
    EngineConfig config(config_path);
    if (config.task() == "trajectory_planning") {
        impl_->planner.reset(new ActionChunkEngine(config));
        return;
    }
    impl_->engine.reset(new StandardEngine(config));
    impl_->engine->warmup();
}

EdgeFM::~EdgeFM() noexcept = default;

Response EdgeFM::generate(const Request& request) const {
    if (!impl_->engine) throw ConfigurationError("generate() is not supported by the active engine (task=trajectory_planning)");
    return impl_->engine->generate(request);
}

TensorMap EdgeFM::plan(int32_t request_id, const TensorRefMap& inputs) const {
    if (!impl_->planner) throw ConfigurationError("plan() is not supported by the active engine (task=token_generation)");
    return impl_->planner->plan(request_id, inputs);
}
TensorMap EdgeFM::run_stage(int32_t request_id, const std::string& stage_name, const TensorRefMap& inputs) const {
    if (!impl_->engine) throw ConfigurationError("run_stage('" + stage_name + "') is not supported by the active engine (task=trajectory_planning): use plan()");
    return impl_->engine->run_stage(request_id, stage_name, inputs);
}
// compatibility wrappers, as the reference's base Engine defines them (src/engine/engine.cpp:542-548)
TensorMap EdgeFM::prefill(int32_t request_id, const TensorRefMap& inputs) const { return run_stage(request_id, "prefill", inputs); }
TensorMap EdgeFM::decode(int32_t request_id, const TensorRefMap& inputs) const { return run_stage(request_id, "decode", inputs); }

std::unordered_map<std::string, double> EdgeFM::last_generate_metrics() const {
    if (!impl_->engine) return {};
    return impl_->engine->last_generate_metrics();
}
std::unordered_map<std::string, double> EdgeFM::last_plan_metrics() const {
    if (!impl_->planner) return {};
    return impl_->planner->last_plan_metrics();
}
std::unordered_map<std::string, double> EdgeFM::last_stage_metrics() const {
    if (!impl_->engine) return {};
    return impl_->engine->last_stage_metrics();
}

void EdgeFM::tune() {}

void* EdgeFM::backend_handle() const { return impl_->engine ? impl_->engine->backend_handle() : nullptr; }

}  // namespace edge_fm
