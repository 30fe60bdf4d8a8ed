#include "kv_manager.h"

#include <algorithm>
#include <cstring>

namespace edge_fm {

std::vector<void*> HostKVBufferAllocator::allocate_slot(int32_t, int32_t, size_t layer_bytes, int32_t num_layers) {
    std::vector<void*> out;
    for (int32_t l = 0; l < num_layers; ++l) {
        buffers_.emplace_back(new uint8_t[layer_bytes]);
        std::memset(buffers_.back().get(), 0, layer_bytes);
        out.push_back(buffers_.back().get());
    }
    return out;
}

AttentionType attention_type_from_string(const std::string& s) {
    std::string t = s;
    std::transform(t.begin(), t.end(), t.begin(), [](unsigned char c) { return (char)std::tolower(c); });
    if (t == "mha") return AttentionType::MHA;
    if (t == "gqa") return AttentionType::GQA;
    if (t == "mqa") return AttentionType::MQA;
    throw ConfigurationError("Unsupported kvcache.attention_type: " + s + " (mha, gqa, mqa)");
}

KVManager::KVManager(const std::vector<KvRequestConfig>& requests, const KVGeometry& geometry, AttentionType type,
                     int32_t device_id, std::shared_ptr<KVBufferAllocator> allocator)
    : geo_(geometry), type_(type), device_id_(device_id), allocator_(std::move(allocator)) {
    if (geo_.num_layers <= 0 || geo_.kv_heads <= 0 || geo_.head_dim <= 0)
        throw ConfigurationError("KV geometry must be positive");
    if (requests.empty()) throw ConfigurationError("kvcache.requests must declare at least one slot");
    const size_t k_stride = (size_t)geo_.kv_heads * geo_.head_dim * get_dtype_size(geo_.dtype);
    for (const KvRequestConfig& r : requests) {
        if (slots_.count(r.request_id)) throw ConfigurationError("duplicate request_id in kvcache.requests: " + std::to_string(r.request_id));
        if (r.max_tokens <= 0) throw ConfigurationError("max_tokens must be positive for request_id " + std::to_string(r.request_id));
        if ((int64_t)r.prefix_token_ids.size() >= (int64_t)r.max_tokens)
            throw ConfigurationError("prefix_token_ids does not fit in max_tokens for request_id " + std::to_string(r.request_id));
        Slot s;
        s.status.request_id = r.request_id;
        s.status.prefix_token_ids = r.prefix_token_ids;
        s.status.prefix_size = r.prefix_token_ids.size();
        s.status.max_tokens = r.max_tokens;
        const size_t layer_bytes = 2 * (size_t)r.max_tokens * k_stride;
        s.status.allocated_size = layer_bytes * (size_t)geo_.num_layers;
        s.read_ptrs = allocator_->allocate_slot(r.request_id, r.max_tokens, layer_bytes, geo_.num_layers);
        if ((int32_t)s.read_ptrs.size() != geo_.num_layers) throw InternalError("KV allocator returned a wrong layer count");
        for (void* p : s.read_ptrs)
            s.write_ptrs.push_back(static_cast<uint8_t*>(p) + s.status.prefix_size * k_stride);
        order_.push_back(r.request_id);
        slots_.emplace(r.request_id, std::move(s));
    }
}

size_t KVManager::get_token_stride() const {
    return 2 * (size_t)geo_.kv_heads * geo_.head_dim * get_dtype_size(geo_.dtype);
}

std::vector<void*> KVManager::get_read_kvcache(int32_t request_id) const {
    auto it = slots_.find(request_id);
    if (it == slots_.end()) throw InvalidRequestError("Invalid request_id: " + std::to_string(request_id));
    return it->second.read_ptrs;
}

std::vector<void*> KVManager::get_write_kvcache(int32_t request_id) const {
    auto it = slots_.find(request_id);
    if (it == slots_.end()) throw InvalidRequestError("Invalid request_id: " + std::to_string(request_id));
    return it->second.write_ptrs;
}

KVManagerStatus KVManager::get_status() const {
    KVManagerStatus st;
    st.device = allocator_->device();
    st.device_id = device_id_;
    for (int32_t id : order_) st.slots.push_back(slots_.at(id).status);
    return st;
}

bool KVManager::is_request_valid(int32_t request_id) const { return slots_.count(request_id) > 0; }

const KVSlotStatus* KVManager::find_slot(int32_t request_id) const {
    auto it = slots_.find(request_id);
    return it == slots_.end() ? nullptr : &it->second.status;
}

}  // namespace edge_fm
