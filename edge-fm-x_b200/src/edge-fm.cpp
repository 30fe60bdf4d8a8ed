// edge_fm::EdgeFM facade: configuration -> engine -> warmup; generate() forwards.
// Reference: src/edge-fm.cpp:12-22 (the constructor runs warmup) and the base Engine's
// refusal of stage / planner calls for a token-generation task (src/engine/engine.cpp:551-564).
#include <edge-fm/edge-fm.h>

#include "engine/config.h"
#include "engine/standard_engine.h"

namespace edge_fm {

struct EdgeFM::Impl {
    std::unique_ptr<StandardEngine> engine;
};

EdgeFM::EdgeFM(const std::string& config_path) : impl_(new Impl()) {
    EngineConfig config(config_path);
    impl_->engine.reset(new StandardEngine(config));
    impl_->engine->warmup();
}

EdgeFM::~EdgeFM() noexcept = default;

Response EdgeFM::generate(const Request& request) const { return impl_->engine->generate(request); }

TensorMap EdgeFM::plan(int32_t, const TensorRefMap&) const {
    throw ConfigurationError("plan() is not supported by the active engine (task=token_generation)");
}
TensorMap EdgeFM::run_stage(int32_t, const std::string& stage_name, const TensorRefMap&) const {
    throw ConfigurationError("run_stage('" + stage_name + "') is not supported by the active engine (task=token_generation)");
}
TensorMap EdgeFM::prefill(int32_t, const TensorRefMap&) const {
    throw ConfigurationError("prefill() stage API is not supported by the active engine; use generate()");
}
TensorMap EdgeFM::decode(int32_t, const TensorRefMap&) const {
    throw ConfigurationError("decode() stage API is not supported by the active engine; use generate()");
}

std::unordered_map<std::string, double> EdgeFM::last_generate_metrics() const {
    return impl_->engine->last_generate_metrics();
}
std::unordered_map<std::string, double> EdgeFM::last_plan_metrics() const { return {}; }
std::unordered_map<std::string, double> EdgeFM::last_stage_metrics() const { return {}; }

void EdgeFM::tune() {}

}  // namespace edge_fm
