#include "scheduler.h"

#include <algorithm>
#include <string>

namespace edge_fm {

Scheduler::Scheduler(std::shared_ptr<KVManager> kv_manager, int32_t max_new_tokens)
    : kv_manager_(std::move(kv_manager)), max_new_tokens_(std::max(1, max_new_tokens)) {}

Context Scheduler::create_context(const Request& request) const {
    const int32_t id = request.request_id();
    const std::vector<int32_t>& toks = request.token_ids();
    const KVSlotStatus* slot = kv_manager_->find_slot(id);
    if (slot == nullptr) throw InvalidRequestError("Cannot find slot for request_id: " + std::to_string(id));
    if (toks.empty()) throw InvalidRequestError("Request token_ids is empty for request_id: " + std::to_string(id));
    const std::vector<int32_t>& prefix = slot->prefix_token_ids;
    if (!prefix.empty()) {
        if (toks.size() < prefix.size())
            throw InvalidRequestError("Request token_ids length (" + std::to_string(toks.size()) +
                                      ") is less than prefix_token_ids length (" + std::to_string(prefix.size()) +
                                      ") for request_id: " + std::to_string(id));
        for (size_t i = 0; i < prefix.size(); ++i)
            if (toks[i] != prefix[i])
                throw InvalidRequestError("Request token_ids prefix does not match prefix_token_ids for request_id: " +
                                          std::to_string(id) + ". Mismatch at position " + std::to_string(i) +
                                          ": expected " + std::to_string(prefix[i]) + ", got " + std::to_string(toks[i]));
    }
    Context c;
    c.request_id = id;
    c.prefix_size = (int32_t)slot->prefix_size;
    c.seq_len = (int32_t)toks.size();
    c.prefill_tokens = c.seq_len - c.prefix_size;
    c.max_tokens = slot->max_tokens;
    if (c.seq_len > c.max_tokens)
        throw InvalidRequestError("Request sequence length (" + std::to_string(c.seq_len) + ") exceeds max_tokens (" +
                                  std::to_string(c.max_tokens) + ") for request_id: " + std::to_string(id));
    // KV rows used = seq_len + (generated - 1): the prefill sample needs no new row.
    const int32_t capacity = std::max(1, c.max_tokens - c.seq_len + 1);
    c.max_generated_tokens = std::min(max_new_tokens_, capacity);
    return c;
}

}  // namespace edge_fm
