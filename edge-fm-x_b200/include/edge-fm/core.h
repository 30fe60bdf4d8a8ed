// Public value types of the edge_fm API: errors, enums, Tensor, Request, Response.
// Source-compatible with the reference's include/edge-fm/core.h (same names, signatures,
// defaults and ownership rules), so that callers of the generate() path compile unchanged.
#pragma once
#include <dlpack/dlpack.h>

#include <cstddef>
#include <cstdint>
#include <exception>
#include <memory>
#include <string>
#include <tuple>
#include <unordered_map>
#include <vector>

namespace edge_fm {

// ---- errors: every failure of the library is reported as a subclass of Error ----------------
class Error : public std::exception {
public:
    explicit Error(const std::string& message) : message_(message) {}
    const char* what() const noexcept override { return message_.c_str(); }

protected:
    std::string message_;
};
struct InvalidRequestError : public Error { using Error::Error; };    // bad ids / prefix / shapes in a Request
struct DeviceError : public Error { using Error::Error; };            // CUDA runtime or kernel status
struct InvalidArgumentError : public Error { using Error::Error; };
struct ConfigurationError : public Error { using Error::Error; };     // engine JSON / config.json problems
struct ModelNotLoadedError : public Error { using Error::Error; };    // missing or malformed checkpoint
struct OutOfMemoryError : public Error { using Error::Error; };
struct InternalError : public Error { using Error::Error; };

enum class Device { CPU, GPU };

enum class DType { Float32, Float16, BFloat16, Int32, Int64, UInt8, Int8 };

// Who releases a Tensor's buffer, and how.  Says nothing about who allocated or copied it:
// Tensor::view never frees, Tensor::adopt frees a buffer it was handed, Tensor::clone_from
// frees the buffer it allocated.
// Which of a model's two passes (and weight sets) a call refers to; the reference keeps this enum next to its Engine
// (src/engine/engine.h:16) and exposes it from the Python module.
enum class ModelStage { Prefill, Decode };

enum class MemoryOwnership {
    ViewExternal,    // never freed by the Tensor
    OwnCpuMalloc,    // std::free
    OwnCudaMalloc,   // cudaFree
    OwnCudaPool,     // cudaFreeAsync on the stream given at creation
};

// Dense, contiguous, row-major n-d array on the host or on one GPU.  Move-only.
class Tensor {
public:
    Tensor() noexcept;
    ~Tensor() noexcept;
    Tensor(const Tensor&) = delete;
    Tensor& operator=(const Tensor&) = delete;
    Tensor(Tensor&& other) noexcept;
    Tensor& operator=(Tensor&& other) noexcept;

    // Wraps caller memory; the caller keeps it alive and frees it.
    static Tensor view(void* data, const std::vector<int64_t>& shape, DType dtype, Device device,
                       int32_t device_id = 0);
    // Takes over caller memory; released per `ownership` when the Tensor dies.
    static Tensor adopt(void* data, const std::vector<int64_t>& shape, DType dtype, Device device,
                        int32_t device_id = 0, MemoryOwnership ownership = MemoryOwnership::OwnCudaMalloc,
                        void* stream_handle = nullptr);
    // Allocates on the destination device and copies `src` (host<->device and device<->device).
    static Tensor clone_from(const void* src, const std::vector<int64_t>& shape, DType dtype, Device src_device,
                             int32_t src_device_id, Device dst_device, int32_t dst_device_id = 0,
                             MemoryOwnership ownership = MemoryOwnership::OwnCudaMalloc,
                             void* stream_handle = nullptr);
    // Copies a contiguous row-major DLPack tensor; throws InvalidRequestError otherwise.
    static Tensor from_dlpack(DLManagedTensor* managed_tensor);
    // Shares this tensor's buffer; the caller invokes the returned object's deleter.
    DLManagedTensor* to_dlpack() const;

    bool empty() const noexcept;
    DType dtype() const noexcept;
    const std::vector<int64_t>& shape() const noexcept;
    std::tuple<Device, int32_t> device() const noexcept;
    void* data_ptr() const noexcept;
    bool operator==(const Tensor& other) const noexcept;   // same buffer, not same values
    // Text dump: header lines (shape, dtype, count) then values in row-major order.
    void dump(const std::string& file_path) const;

private:
    struct Impl;
    std::unique_ptr<Impl> impl_;
};

using TensorMap = std::unordered_map<std::string, Tensor>;
using TensorRefMap = std::unordered_map<std::string, const Tensor*>;

// One generation request.  request_id names a pre-declared KV slot; token_ids must start with
// that slot's fixed prefix.  `embedding` rows replace the ids embed_token_id + i; position_ids
// is the [3, S] M-RoPE table.  Tensors passed in are deep-copied to the target device.
struct Request {
    Request(int32_t request_id, const std::vector<int32_t>& token_ids) noexcept
        : request_id_(request_id), token_ids_(token_ids), embed_token_id_(-1) {}

    Request(int32_t request_id, const std::vector<int32_t>& token_ids, const Tensor& embedding,
            int32_t embed_token_id = -1, Device device = Device::GPU, int32_t device_id = 0,
            MemoryOwnership ownership = MemoryOwnership::OwnCudaMalloc, void* stream_handle = nullptr)
        : request_id_(request_id), token_ids_(token_ids), embed_token_id_(embed_token_id) {
        embedding_ = copy_of(embedding, device, device_id, ownership, stream_handle);
    }

    Request(int32_t request_id, const std::vector<int32_t>& token_ids, const Tensor& embedding,
            int32_t embed_token_id, const Tensor& position_ids, const std::vector<int32_t>& mrope_last_pos,
            Device device = Device::GPU, int32_t device_id = 0,
            MemoryOwnership ownership = MemoryOwnership::OwnCudaMalloc, void* stream_handle = nullptr)
        : request_id_(request_id), token_ids_(token_ids), embed_token_id_(embed_token_id) {
        embedding_ = copy_of(embedding, device, device_id, ownership, stream_handle);
        position_ids_ = copy_of(position_ids, device, device_id, ownership, stream_handle);
        mrope_last_pos_ = mrope_last_pos;
    }

    Request(int32_t request_id, const std::vector<int32_t>& token_ids, const Tensor& embedding,
            int32_t embed_token_id, const Tensor& position_ids, Device device = Device::GPU, int32_t device_id = 0,
            MemoryOwnership ownership = MemoryOwnership::OwnCudaMalloc, void* stream_handle = nullptr)
        : Request(request_id, token_ids, embedding, embed_token_id, position_ids, std::vector<int32_t>{}, device,
                  device_id, ownership, stream_handle) {}

    Request(Request&&) noexcept = default;
    Request& operator=(Request&&) noexcept = default;
    Request(const Request&) = delete;
    Request& operator=(const Request&) = delete;

    int32_t request_id() const noexcept { return request_id_; }
    const std::vector<int32_t>& token_ids() const noexcept { return token_ids_; }
    const Tensor& embedding() const noexcept { return embedding_; }
    int32_t embed_token_id() const noexcept { return embed_token_id_; }
    bool has_embedding() const noexcept { return !embedding_.empty(); }
    const Tensor& position_ids() const noexcept { return position_ids_; }
    bool has_position_ids() const noexcept { return !position_ids_.empty(); }
    const std::vector<int32_t>& mrope_last_pos() const noexcept { return mrope_last_pos_; }
    bool has_mrope_last_pos() const noexcept { return !mrope_last_pos_.empty(); }

    void set_stop_token_ids(const std::vector<int32_t>& ids) { stop_token_ids_ = ids; }
    const std::vector<int32_t>& stop_token_ids() const noexcept { return stop_token_ids_; }
    void set_ignore_stop_tokens(bool v) { ignore_stop_tokens_ = v; }
    bool ignore_stop_tokens() const noexcept { return ignore_stop_tokens_; }

private:
    static Tensor copy_of(const Tensor& t, Device device, int32_t device_id, MemoryOwnership ownership,
                          void* stream_handle) {
        return Tensor::clone_from(t.data_ptr(), t.shape(), t.dtype(), std::get<0>(t.device()),
                                  std::get<1>(t.device()), device, device_id, ownership, stream_handle);
    }

    int32_t request_id_;
    std::vector<int32_t> token_ids_;
    int32_t embed_token_id_;
    Tensor embedding_;
    Tensor position_ids_;
    std::vector<int32_t> mrope_last_pos_;
    std::vector<int32_t> stop_token_ids_;
    bool ignore_stop_tokens_ = false;
};

// Generated ids: every sampled token including the one sampled from the prefill, cut after
// the first stop token.
class Response {
public:
    Response() noexcept = default;
    ~Response() noexcept = default;
    Response(Response&&) noexcept = default;
    Response& operator=(Response&&) noexcept = default;
    Response(const Response&) = delete;
    Response& operator=(const Response&) = delete;

    std::vector<int32_t>& token_ids() noexcept { return token_ids_; }
    const std::vector<int32_t>& token_ids() const noexcept { return token_ids_; }

private:
    std::vector<int32_t> token_ids_;
};

inline Device device_from_string(const std::string& s) {
    if (s == "cpu") return Device::CPU;
    if (s == "cuda" || s == "gpu") return Device::GPU;
    throw ConfigurationError("Unsupported device: " + s + ". Expected 'cuda', 'gpu', or 'cpu'");
}

inline DType dtype_from_string(const std::string& s) {
    if (s == "fp32" || s == "float32") return DType::Float32;
    if (s == "fp16" || s == "float16") return DType::Float16;
    if (s == "bf16" || s == "bfloat16") return DType::BFloat16;
    if (s == "int32") return DType::Int32;
    if (s == "int64") return DType::Int64;
    if (s == "int8") return DType::Int8;
    if (s == "uint8") return DType::UInt8;
    throw ConfigurationError("Unsupported dtype: " + s + ". Expected 'fp32', 'fp16', or 'bf16'");
}

inline size_t get_dtype_size(DType dtype) {
    switch (dtype) {
        case DType::Float32: case DType::Int32: return 4;
        case DType::Float16: case DType::BFloat16: return 2;
        case DType::Int64: return 8;
        case DType::UInt8: case DType::Int8: return 1;
    }
    return 0;
}

}  // namespace edge_fm
