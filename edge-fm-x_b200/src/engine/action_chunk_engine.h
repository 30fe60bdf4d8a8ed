// Engine behind EdgeFM::plan() for task = trajectory_planning: a SmolVLA-shaped policy whose whole
// iterative-denoise loop runs on the device (efm_b200_vla_chunk).  Keeps the request / response
// contract of the reference's planner (src/engine/tasks/trajectory_planning/trajectory_planner_engine.cpp:
// 275-331): planner.type "iterative_denoise" with sampler "euler_flow", planner.num_steps, the state
// tensor named planner.state_tensor (default "current_actions"; when the request has none it is drawn
// from planner.trajectory_shape / noise_sigma / seed with std::mt19937 + std::normal_distribution as
// there, :49-68), the result under planner.output_tensor and under "trajectory", and the metrics
// stage_calls / plan_steps.  The reference runs each step as a run_stage() round trip through host
// tensors; here the context stage, the steps and the Euler updates are one CUDA graph.
#pragma once
#include <edge-fm/core.h>

#include <memory>
#include <string>
#include <unordered_map>

#include "config.h"

struct efm_b200_vla;

namespace edge_fm {

class ActionChunkEngine {
public:
    explicit ActionChunkEngine(const EngineConfig& config);
    ~ActionChunkEngine();
    ActionChunkEngine(const ActionChunkEngine&) = delete;
    ActionChunkEngine& operator=(const ActionChunkEngine&) = delete;

    // inputs: "images" f32 [n_images, 3, S, S], "lang_tokens" i32 [lang_tokens], "state" f32 [state_dim], optionally the
    // state tensor (f32 [chunk, action_dim]); host tensors.  Returns host f32 [chunk, action_dim].
    TensorMap plan(int32_t request_id, const TensorRefMap& inputs);
    std::unordered_map<std::string, double> last_plan_metrics() const { return metrics_; }

private:
    efm_b200_vla* vla_ = nullptr;
    int32_t n_images_ = 0, image_size_ = 0, lang_tokens_ = 0, state_dim_ = 0, chunk_ = 0, action_dim_ = 0, steps_ = 0;
    std::string state_name_, output_name_;
    bool has_shape_ = false;
    float noise_sigma_ = 1.0f;
    uint32_t seed_ = 0;
    std::unordered_map<std::string, double> metrics_;
};

}  // namespace edge_fm
