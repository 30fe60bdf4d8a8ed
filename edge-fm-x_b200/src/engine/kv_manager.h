// Fixed-prefix KV slots.  One slot per request_id declared in kvcache.requests; per layer one
// buffer laid out [K: max_tokens x kv_heads x head_dim | V: same]; the read pointer is the
// buffer base and the write pointer starts prefix_size tokens into the K block.
// Same bookkeeping and invariants as the reference's KVManager
// (src/engine/tasks/token_generation/kv_manager.cpp:45-272); MLA caches are not built.
#pragma once
#include <edge-fm/core.h>

#include <cstddef>
#include <cstdint>
#include <memory>
#include <unordered_map>
#include <vector>

#include "config.h"

namespace edge_fm {

struct KVSlotStatus {
    int32_t request_id;
    std::vector<int32_t> prefix_token_ids;
    size_t prefix_size;
    int32_t max_tokens;
    size_t allocated_size;     // bytes over all layers
};

struct KVManagerStatus {
    std::vector<KVSlotStatus> slots;
    Device device;
    int32_t device_id;
};

enum class AttentionType { MHA, GQA, MQA };

struct KVGeometry {
    int32_t num_layers = 0, kv_heads = 0, head_dim = 0;
    DType dtype = DType::BFloat16;
};

// Where the per-layer buffers come from.  The engine plugs in the device backend; tests plug
// in host memory (the reference's HostKVBufferAllocator, kv_manager.h:44-56).
class KVBufferAllocator {
public:
    virtual ~KVBufferAllocator() = default;
    virtual Device device() const = 0;
    // Returns num_layers base pointers, each to layer_bytes of zeroed memory.
    virtual std::vector<void*> allocate_slot(int32_t request_id, int32_t max_tokens, size_t layer_bytes,
                                             int32_t num_layers) = 0;
};

class HostKVBufferAllocator : public KVBufferAllocator {
public:
    Device device() const override { return Device::CPU; }
    std::vector<void*> allocate_slot(int32_t request_id, int32_t max_tokens, size_t layer_bytes,
                                     int32_t num_layers) override;

private:
    std::vector<std::unique_ptr<uint8_t[]>> buffers_;
};

class KVManager {
public:
    KVManager(const std::vector<KvRequestConfig>& requests, const KVGeometry& geometry, AttentionType type,
              int32_t device_id, std::shared_ptr<KVBufferAllocator> allocator);
    KVManager(const KVManager&) = delete;
    KVManager& operator=(const KVManager&) = delete;

    size_t get_token_stride() const;       // bytes of K plus V for one token
    AttentionType get_attention_type() const { return type_; }
    std::vector<void*> get_read_kvcache(int32_t request_id) const;
    std::vector<void*> get_write_kvcache(int32_t request_id) const;
    KVManagerStatus get_status() const;
    bool is_request_valid(int32_t request_id) const;
    const KVSlotStatus* find_slot(int32_t request_id) const;

private:
    struct Slot {
        KVSlotStatus status;
        std::vector<void*> read_ptrs, write_ptrs;
    };
    KVGeometry geo_;
    AttentionType type_;
    int32_t device_id_;
    std::shared_ptr<KVBufferAllocator> allocator_;
    std::unordered_map<int32_t, Slot> slots_;
    std::vector<int32_t> order_;
};

AttentionType attention_type_from_string(const std::string& s);

}  // namespace edge_fm
