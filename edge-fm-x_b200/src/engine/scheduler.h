// Per-request admission: slot lookup, fixed-prefix validation and the generated-token cap.
// Same rules and messages as the reference's Scheduler::create_context
// (src/engine/tasks/token_generation/scheduler.cpp:62-154).
#pragma once
#include <edge-fm/core.h>

#include <memory>

#include "kv_manager.h"

namespace edge_fm {

// What generate() needs to know about one admitted request.
struct Context {
    int32_t request_id = 0;
    int32_t prefix_size = 0;           // tokens already resident in the slot
    int32_t seq_len = 0;               // all request tokens (prefix included)
    int32_t prefill_tokens = 0;        // seq_len - prefix_size: what the prefill pass computes
    int32_t max_tokens = 0;            // slot capacity
    int32_t max_generated_tokens = 0;  // min(max_new_tokens, max_tokens - seq_len + 1), at least 1
    int32_t generated_tokens = 0;
    bool is_finished() const { return generated_tokens >= max_generated_tokens; }
};

class Scheduler {
public:
    Scheduler(std::shared_ptr<KVManager> kv_manager, int32_t max_new_tokens);
    // throws InvalidRequestError: unknown request_id, request shorter than or different from
    // the slot's prefix, empty request.
    Context create_context(const Request& request) const;
    int32_t max_new_tokens() const { return max_new_tokens_; }

private:
    std::shared_ptr<KVManager> kv_manager_;
    int32_t max_new_tokens_;
};

}  // namespace edge_fm
