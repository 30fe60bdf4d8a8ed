// Read-only safetensors access: mmap the file, parse the JSON header, hand out host pointers.
// Replaces the reference's WeightLoader (src/utils/device/weight_loader.cpp:80-171) and the
// file discovery / VLM key mapping of load_cuda_weights (src/engine/engine_factory.cpp:27-110).
#pragma once
#include <cstdint>
#include <functional>
#include <string>
#include <vector>

namespace edge_fm {

struct SafeTensorEntry {
    std::string name;
    std::string dtype;            // "BF16", "F16", "F32", ...
    std::vector<int64_t> shape;
    const void* data = nullptr;   // inside the mapping
    size_t nbytes = 0;
};

class SafeTensorsFile {
public:
    explicit SafeTensorsFile(const std::string& path);   // throws ModelNotLoadedError
    ~SafeTensorsFile();
    SafeTensorsFile(const SafeTensorsFile&) = delete;
    SafeTensorsFile& operator=(const SafeTensorsFile&) = delete;
    const std::vector<SafeTensorEntry>& entries() const { return entries_; }

private:
    void* map_ = nullptr;
    size_t size_ = 0;
    std::vector<SafeTensorEntry> entries_;
};

// model.safetensors, else the sorted model-*-of-*.safetensors shards.
std::vector<std::string> collect_safetensors_files(const std::string& model_dir);
// Key handling for Qwen2.5-VL checkpoints: keep model.* / language_model.* / lm_head.* and strip
// the wrapper prefixes; returns false for tensors that are not part of the text tower.
bool map_vlm_weight_name(const std::string& name, std::string* mapped);

}  // namespace edge_fm
