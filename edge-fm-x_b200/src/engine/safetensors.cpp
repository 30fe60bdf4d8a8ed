#include "safetensors.h"

#include <dirent.h>
#include <edge-fm/core.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstring>

#include "json.h"

namespace edge_fm {

namespace {
// bytes per element of the safetensors dtype names; 0 = unknown (such a tensor is kept, its size is not checked)
size_t dtype_bytes(const std::string& d) {
    if (d == "F64" || d == "I64" || d == "U64") return 8;
    if (d == "F32" || d == "I32" || d == "U32") return 4;
    if (d == "BF16" || d == "F16" || d == "I16" || d == "U16") return 2;
    if (d == "I8" || d == "U8" || d == "BOOL" || d == "F8_E4M3" || d == "F8_E5M2") return 1;
    return 0;
}
// unmaps when the constructor leaves by exception (the destructor does not run then)
struct MapGuard {
    void* map;
    size_t size;
    ~MapGuard() { if (map != nullptr) munmap(map, size); }
};
}  // namespace

SafeTensorsFile::SafeTensorsFile(const std::string& path) {
    const int fd = ::open(path.c_str(), O_RDONLY);
    if (fd < 0) throw ModelNotLoadedError("Cannot open weights file: " + path);
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size < 8) {
        ::close(fd);
        throw ModelNotLoadedError("Weights file is too short to be safetensors: " + path);
    }
    size_ = (size_t)st.st_size;
    map_ = mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd, 0);
    ::close(fd);
    if (map_ == MAP_FAILED) {
        map_ = nullptr;
        throw ModelNotLoadedError("mmap failed for: " + path);
    }
    MapGuard guard{map_, size_};
    const unsigned char* base = static_cast<const unsigned char*>(map_);
    uint64_t header_len = 0;
    for (int i = 7; i >= 0; --i) header_len = (header_len << 8) | base[i];     // little-endian u64
    if (header_len == 0 || header_len > size_ - 8) throw ModelNotLoadedError("Corrupt safetensors header length in: " + path);
    json::Value header;
    try {
        header = json::parse(std::string(reinterpret_cast<const char*>(base + 8), (size_t)header_len));
    } catch (const std::exception& e) {
        throw ModelNotLoadedError("Corrupt safetensors header in " + path + ": " + e.what());
    }
    if (!header.is_object()) throw ModelNotLoadedError("safetensors header is not an object: " + path);
    const size_t data_start = 8 + (size_t)header_len;
    for (const auto& kv : header.obj) {
        if (kv.first == "__metadata__") continue;
        const json::Value& t = kv.second;
        const json::Value* off = t.find("data_offsets");
        const json::Value* shp = t.find("shape");
        if (!t.is_object() || off == nullptr || !off->is_array() || off->arr.size() != 2 || shp == nullptr || !shp->is_array())
            throw ModelNotLoadedError("Malformed tensor record '" + kv.first + "' in " + path);
        SafeTensorEntry e;
        e.name = kv.first;
        e.dtype = t.get_string("dtype", "");
        for (const json::Value& d : shp->arr) e.shape.push_back(d.inum);
        const size_t b = (size_t)off->arr[0].inum, en = (size_t)off->arr[1].inum;
        if (en < b || data_start + en > size_)
            throw ModelNotLoadedError("Tensor '" + kv.first + "' points outside the file (truncated checkpoint?): " + path);
        e.data = base + data_start + b;
        e.nbytes = en - b;
        // the loader copies shape-derived byte counts: a record whose byte range disagrees with its shape would be
        // read past its end
        size_t want = dtype_bytes(e.dtype);
        for (const int64_t d : e.shape) {
            if (d < 0) throw ModelNotLoadedError("Tensor '" + kv.first + "' has a negative dimension in " + path);
            want *= (size_t)d;
        }
        if (dtype_bytes(e.dtype) != 0 && want != e.nbytes)
            throw ModelNotLoadedError("Tensor '" + kv.first + "' spans " + std::to_string(e.nbytes) + " bytes but its shape and dtype need " +
                                      std::to_string(want) + " (malformed or mis-sharded checkpoint): " + path);
        entries_.push_back(std::move(e));
    }
    guard.map = nullptr;      // construction succeeded: the destructor owns the mapping
}

SafeTensorsFile::~SafeTensorsFile() {
    if (map_ != nullptr) munmap(map_, size_);
}

std::vector<std::string> collect_safetensors_files(const std::string& model_dir) {
    std::vector<std::string> out;
    struct stat st;
    const std::string single = model_dir + "/model.safetensors";
    if (stat(single.c_str(), &st) == 0 && S_ISREG(st.st_mode)) {
        out.push_back(single);
        return out;
    }
    DIR* d = opendir(model_dir.c_str());
    if (d == nullptr) return out;
    while (dirent* ent = readdir(d)) {
        const std::string name = ent->d_name;
        const std::string suffix = ".safetensors";
        if (name.size() > 18 && name.compare(0, 6, "model-") == 0 && name.find("-of-") != std::string::npos &&
            name.compare(name.size() - suffix.size(), suffix.size(), suffix) == 0)
            out.push_back(model_dir + "/" + name);
    }
    closedir(d);
    std::sort(out.begin(), out.end());
    return out;
}

bool map_vlm_weight_name(const std::string& name, std::string* mapped) {
    const bool keep = name.rfind("model.", 0) == 0 || name.rfind("language_model.", 0) == 0 || name.rfind("lm_head.", 0) == 0;
    if (!keep) return false;
    if (name.rfind("model.model.", 0) == 0) *mapped = name.substr(6);
    else if (name.rfind("language_model.", 0) == 0) *mapped = name.substr(15);
    else *mapped = name;
    return true;
}

}  // namespace edge_fm
