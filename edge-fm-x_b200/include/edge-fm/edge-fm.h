// The engine facade.  Source-compatible with the reference's include/edge-fm/edge-fm.h:10-111.
// Behind it: the token-generation path (generate) and, for task = trajectory_planning, the
// action-chunk policy (plan).  The stage entry points exist so that callers link, and throw
// ConfigurationError exactly as the reference's base Engine does when the configured task does
// not provide them (src/engine/engine.cpp:551-564).
#pragma once
#include <edge-fm/core.h>

#include <memory>
#include <string>
#include <unordered_map>

namespace edge_fm {

class EdgeFM {
public:
    // Loads the engine JSON at config_path, the HF checkpoint it points to, allocates the KV
    // slots it declares, prefills each slot's fixed prefix and captures the decode graph.
    explicit EdgeFM(const std::string& config_path);
    ~EdgeFM() noexcept;

    // Prefill the non-prefix part of the request, then decode until max_new_tokens or the
    // slot's capacity; stop tokens cut the returned ids on the host afterwards.
    Response generate(const Request& request) const;

    // task = trajectory_planning: host tensors "images" f32 [n, 3, S, S], "lang_tokens" i32, "state" f32 and optionally
    // the planner's state tensor (default "current_actions", f32 [chunk, action_dim]) -> {"trajectory": f32 [chunk, action_dim]}.
    TensorMap plan(int32_t request_id, const TensorRefMap& inputs) const;
    TensorMap run_stage(int32_t request_id, const std::string& stage_name, const TensorRefMap& inputs) const;
    TensorMap prefill(int32_t request_id, const TensorRefMap& inputs) const;
    TensorMap decode(int32_t request_id, const TensorRefMap& inputs) const;

    // Timing of the most recent generate(): prefill_ms, decode_ms, total_stage_ms,
    // decode_step_avg_ms, generated_tokens_total, decode_steps, ... (same key set as the reference).
    std::unordered_map<std::string, double> last_generate_metrics() const;
    std::unordered_map<std::string, double> last_plan_metrics() const;
    std::unordered_map<std::string, double> last_stage_metrics() const;

    // Accepted for compatibility; there is no operator table to tune in this backend.
    void tune();

    // The device backend of a token-generation engine as an `efm_b200_ctx*` of include/efm_b200.h (nullptr for other
    // tasks): lets a caller put companions of the model -- the vision encoder, efm_b200_vit_create -- on the engine's own
    // device, stream and tensor-parallel communicator instead of a second context.  Not part of the reference's API.
    void* backend_handle() const;

private:
    struct Impl;
    std::unique_ptr<Impl> impl_;
};

}  // namespace edge_fm
