// edge_fm::Tensor: a contiguous row-major buffer on the host or one GPU with an explicit
// release policy.  Interface: include/edge-fm/core.h (reference: src/tensor.cpp).
#include <cuda_runtime.h>
#include <edge-fm/core.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iomanip>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace edge_fm {

struct Tensor::Impl {
    void* data = nullptr;
    std::vector<int64_t> shape;
    DType dtype = DType::Float32;
    Device device = Device::CPU;
    int32_t device_id = 0;
    MemoryOwnership ownership = MemoryOwnership::ViewExternal;
    void* stream = nullptr;
};

namespace {

int64_t numel(const std::vector<int64_t>& shape) {
    int64_t n = 1;
    for (int64_t d : shape) n *= d;
    return shape.empty() ? 0 : n;
}

void cuda_check(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return;
    const std::string msg = std::string(what) + ": " + cudaGetErrorString(e);
    if (e == cudaErrorMemoryAllocation) throw OutOfMemoryError(msg);
    throw DeviceError(msg);
}

float half_to_float(uint16_t h) {
    const uint32_t sign = (h & 0x8000u) << 16, exp = (h >> 10) & 0x1f, man = h & 0x3ff;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) bits = sign;
        else {
            int e = -1;
            uint32_t m = man;
            do { ++e; m <<= 1; } while ((m & 0x400) == 0);
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((m & 0x3ff) << 13);
        }
    } else if (exp == 31) bits = sign | 0x7f800000u | (man << 13);
    else bits = sign | ((exp + 112) << 23) | (man << 13);
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

}  // namespace

// Switches the calling thread to a device for the guard's lifetime and puts the caller's device back: copies and frees
// on "the tensor's device" must not move a multi-GPU caller's current device from under it.
struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int device_id) {
        if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
        if (prev != device_id) cuda_check(cudaSetDevice(device_id), "cudaSetDevice");
        else prev = -1;
    }
    ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
};

Tensor::Tensor() noexcept = default;
Tensor::Tensor(Tensor&& other) noexcept = default;

// Device buffers of released OwnCudaMalloc tensors, kept for the next tensor of the same size on the same device: a
// request's embedding tensor is cloned once per request, and cudaMalloc / cudaFree cost milliseconds (and a device
// synchronisation) in a process whose memory is mapped into peers.  At most kCacheSlots buffers / kCacheBytes in total.
namespace {
struct CachedBuffer { void* ptr; size_t bytes; int32_t device_id; };
constexpr size_t kCacheSlots = 8, kCacheBytes = (size_t)256 << 20;
std::mutex g_cache_mutex;
std::vector<CachedBuffer> g_cache;
std::unordered_map<void*, size_t> g_sizes;      // sizes of live buffers that came from device_alloc

void* device_alloc(size_t bytes, int32_t device_id) {
    {
        std::lock_guard<std::mutex> lock(g_cache_mutex);
        for (size_t i = 0; i < g_cache.size(); ++i)
            if (g_cache[i].bytes == bytes && g_cache[i].device_id == device_id) {
                void* p = g_cache[i].ptr;
                g_cache.erase(g_cache.begin() + (long)i);
                g_sizes[p] = bytes;
                return p;
            }
    }
    void* p = nullptr;
    cuda_check(cudaMalloc(&p, bytes), "cudaMalloc");
    std::lock_guard<std::mutex> lock(g_cache_mutex);
    g_sizes[p] = bytes;
    return p;
}

// true: the buffer went into the cache (the caller must not free it)
bool device_release(void* p, int32_t device_id) {
    std::lock_guard<std::mutex> lock(g_cache_mutex);
    auto it = g_sizes.find(p);
    if (it == g_sizes.end()) return false;
    const size_t bytes = it->second;
    g_sizes.erase(it);
    size_t held = 0;
    for (const CachedBuffer& b : g_cache) held += b.bytes;
    if (g_cache.size() >= kCacheSlots || held + bytes > kCacheBytes) return false;
    g_cache.push_back({p, bytes, device_id});
    return true;
}
}  // namespace

static void free_impl(void* data, Device device, int32_t device_id, MemoryOwnership own, void* stream) {
    if (data == nullptr) return;
    switch (own) {
        case MemoryOwnership::ViewExternal: break;
        case MemoryOwnership::OwnCpuMalloc: std::free(data); break;
        case MemoryOwnership::OwnCudaMalloc:
            if (device == Device::GPU) {
                if (device_release(data, device_id)) break;
                int prev = -1;
                if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
                cudaSetDevice(device_id);
                cudaFree(data);
                if (prev >= 0 && prev != device_id) cudaSetDevice(prev);
            } else {
                std::free(data);
            }
            break;
        case MemoryOwnership::OwnCudaPool: {
            int prev = -1;
            if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
            cudaSetDevice(device_id);
            cudaFreeAsync(data, static_cast<cudaStream_t>(stream));
            if (prev >= 0 && prev != device_id) cudaSetDevice(prev);
            break;
        }
    }
}

Tensor::~Tensor() noexcept {
    if (impl_) free_impl(impl_->data, impl_->device, impl_->device_id, impl_->ownership, impl_->stream);
}

Tensor& Tensor::operator=(Tensor&& other) noexcept {
    if (this != &other) {
        if (impl_) free_impl(impl_->data, impl_->device, impl_->device_id, impl_->ownership, impl_->stream);
        impl_ = std::move(other.impl_);
    }
    return *this;
}

Tensor Tensor::view(void* data, const std::vector<int64_t>& shape, DType dtype, Device device, int32_t device_id) {
    Tensor t;
    t.impl_ = std::make_unique<Impl>();
    t.impl_->data = data;
    t.impl_->shape = shape;
    t.impl_->dtype = dtype;
    t.impl_->device = device;
    t.impl_->device_id = device_id;
    return t;
}

Tensor Tensor::adopt(void* data, const std::vector<int64_t>& shape, DType dtype, Device device, int32_t device_id,
                     MemoryOwnership ownership, void* stream_handle) {
    if (ownership == MemoryOwnership::OwnCudaPool && (device != Device::GPU || stream_handle == nullptr))
        throw InvalidArgumentError("OwnCudaPool needs a GPU tensor and a stream");
    if (ownership == MemoryOwnership::OwnCpuMalloc && device != Device::CPU)
        throw InvalidArgumentError("OwnCpuMalloc is for host tensors");
    Tensor t = view(data, shape, dtype, device, device_id);
    t.impl_->ownership = ownership;
    t.impl_->stream = stream_handle;
    return t;
}

Tensor Tensor::clone_from(const void* src, const std::vector<int64_t>& shape, DType dtype, Device src_device,
                          int32_t src_device_id, Device dst_device, int32_t dst_device_id, MemoryOwnership ownership,
                          void* stream_handle) {
    const size_t bytes = (size_t)numel(shape) * get_dtype_size(dtype);
    if (src == nullptr || bytes == 0) return Tensor();
    void* dst = nullptr;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
    if (dst_device == Device::CPU) {
        dst = std::malloc(bytes);
        if (dst == nullptr) throw OutOfMemoryError("host allocation failed");
        if (src_device == Device::CPU) std::memcpy(dst, src, bytes);
        else {
            DeviceGuard guard(src_device_id);
            cuda_check(cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToHost), "copy to host");
        }
        return adopt(dst, shape, dtype, Device::CPU, dst_device_id, MemoryOwnership::OwnCpuMalloc == ownership ? ownership : MemoryOwnership::OwnCpuMalloc);
    }
    DeviceGuard guard(dst_device_id);
    if (ownership == MemoryOwnership::OwnCudaPool) {
        if (stream == nullptr) throw InvalidArgumentError("OwnCudaPool needs a stream");
        cuda_check(cudaMallocAsync(&dst, bytes, stream), "cudaMallocAsync");
    } else {
        ownership = MemoryOwnership::OwnCudaMalloc;
        dst = device_alloc(bytes, dst_device_id);
    }
    cudaError_t e;
    if (src_device == Device::CPU) e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, stream);
    else if (src_device_id == dst_device_id) e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, stream);
    else e = cudaMemcpyPeerAsync(dst, dst_device_id, src, src_device_id, bytes, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);     // the source may be released on return
    if (e != cudaSuccess) {
        if (!device_release(dst, dst_device_id)) cudaFree(dst);
        cuda_check(e, "clone_from copy");
    }
    return adopt(dst, shape, dtype, Device::GPU, dst_device_id, ownership, stream_handle);
}

static DType dtype_from_dl(const DLDataType& t) {
    if (t.lanes != 1) throw InvalidRequestError("vectorised DLPack dtypes are not supported");
    if (t.code == kDLFloat && t.bits == 32) return DType::Float32;
    if (t.code == kDLFloat && t.bits == 16) return DType::Float16;
    if (t.code == kDLBfloat && t.bits == 16) return DType::BFloat16;
    if (t.code == kDLInt && t.bits == 32) return DType::Int32;
    if (t.code == kDLInt && t.bits == 64) return DType::Int64;
    if (t.code == kDLInt && t.bits == 8) return DType::Int8;
    if (t.code == kDLUInt && t.bits == 8) return DType::UInt8;
    throw InvalidRequestError("unsupported DLPack dtype");
}

static DLDataType dtype_to_dl(DType d) {
    switch (d) {
        case DType::Float32: return {kDLFloat, 32, 1};
        case DType::Float16: return {kDLFloat, 16, 1};
        case DType::BFloat16: return {kDLBfloat, 16, 1};
        case DType::Int32: return {kDLInt, 32, 1};
        case DType::Int64: return {kDLInt, 64, 1};
        case DType::Int8: return {kDLInt, 8, 1};
        case DType::UInt8: return {kDLUInt, 8, 1};
    }
    return {kDLFloat, 32, 1};
}

Tensor Tensor::from_dlpack(DLManagedTensor* mt) {
    if (mt == nullptr || mt->dl_tensor.data == nullptr) throw InvalidRequestError("null DLPack tensor");
    const DLTensor& t = mt->dl_tensor;
    std::vector<int64_t> shape(t.shape, t.shape + t.ndim);
    if (t.strides != nullptr) {      // must be contiguous row-major
        int64_t expect = 1;
        for (int i = t.ndim - 1; i >= 0; --i) {
            if (t.shape[i] != 1 && t.strides[i] != expect)
                throw InvalidRequestError("DLPack tensor must be contiguous and row-major");
            expect *= t.shape[i];
        }
    }
    Device dev;
    if (t.device.device_type == kDLCPU || t.device.device_type == kDLCUDAHost) dev = Device::CPU;
    else if (t.device.device_type == kDLCUDA) dev = Device::GPU;
    else throw InvalidRequestError("unsupported DLPack device");
    const char* src = static_cast<const char*>(t.data) + t.byte_offset;
    return clone_from(src, shape, dtype_from_dl(t.dtype), dev, t.device.device_id, dev, t.device.device_id,
                      dev == Device::GPU ? MemoryOwnership::OwnCudaMalloc : MemoryOwnership::OwnCpuMalloc);
}

DLManagedTensor* Tensor::to_dlpack() const {
    if (empty()) throw InvalidRequestError("cannot export an empty tensor");
    struct Holder { DLManagedTensor mt; std::vector<int64_t> shape; };
    Holder* h = new Holder();
    h->shape = impl_->shape;
    h->mt.dl_tensor.data = impl_->data;
    h->mt.dl_tensor.device = {impl_->device == Device::GPU ? kDLCUDA : kDLCPU, impl_->device_id};
    h->mt.dl_tensor.ndim = (int)h->shape.size();
    h->mt.dl_tensor.dtype = dtype_to_dl(impl_->dtype);
    h->mt.dl_tensor.shape = h->shape.data();
    h->mt.dl_tensor.strides = nullptr;
    h->mt.dl_tensor.byte_offset = 0;
    h->mt.manager_ctx = h;
    h->mt.deleter = [](DLManagedTensor* self) { delete static_cast<Holder*>(self->manager_ctx); };
    return &h->mt;
}

bool Tensor::empty() const noexcept { return !impl_ || impl_->data == nullptr || numel(impl_->shape) == 0; }
DType Tensor::dtype() const noexcept { return impl_ ? impl_->dtype : DType::Float32; }
const std::vector<int64_t>& Tensor::shape() const noexcept {
    static const std::vector<int64_t> none;
    return impl_ ? impl_->shape : none;
}
std::tuple<Device, int32_t> Tensor::device() const noexcept {
    return impl_ ? std::make_tuple(impl_->device, impl_->device_id) : std::make_tuple(Device::CPU, 0);
}
void* Tensor::data_ptr() const noexcept { return impl_ ? impl_->data : nullptr; }
bool Tensor::operator==(const Tensor& o) const noexcept { return data_ptr() == o.data_ptr(); }

void Tensor::dump(const std::string& file_path) const {
    if (empty()) throw InvalidRequestError("cannot dump an empty tensor");
    const int64_t n = numel(impl_->shape);
    const size_t esz = get_dtype_size(impl_->dtype);
    std::vector<char> host((size_t)n * esz);
    if (impl_->device == Device::GPU) {
        DeviceGuard guard(impl_->device_id);
        cuda_check(cudaMemcpy(host.data(), impl_->data, host.size(), cudaMemcpyDeviceToHost), "dump copy");
    } else {
        std::memcpy(host.data(), impl_->data, host.size());
    }
    std::ofstream f(file_path);
    if (!f) throw InternalError("cannot open " + file_path);
    static const char* names[] = {"float32", "float16", "bfloat16", "int32", "int64", "uint8", "int8"};
    f << "# shape:";
    for (int64_t d : impl_->shape) f << ' ' << d;
    f << "\n# dtype: " << names[(int)impl_->dtype] << "\n# numel: " << n << "\n";
    f << std::scientific << std::setprecision(9);
    for (int64_t i = 0; i < n; ++i) {
        const char* p = host.data() + (size_t)i * esz;
        switch (impl_->dtype) {
            case DType::Float32: { float v; std::memcpy(&v, p, 4); f << v; break; }
            case DType::Float16: { uint16_t v; std::memcpy(&v, p, 2); f << half_to_float(v); break; }
            case DType::BFloat16: { uint16_t v; std::memcpy(&v, p, 2); uint32_t b = (uint32_t)v << 16; float x; std::memcpy(&x, &b, 4); f << x; break; }
            case DType::Int32: { int32_t v; std::memcpy(&v, p, 4); f << v; break; }
            case DType::Int64: { int64_t v; std::memcpy(&v, p, 8); f << v; break; }
            case DType::UInt8: f << (int)*reinterpret_cast<const uint8_t*>(p); break;
            case DType::Int8: f << (int)*reinterpret_cast<const int8_t*>(p); break;
        }
        f << (i + 1 == n ? '\n' : ' ');
    }
}

}  // namespace edge_fm
