#include "nccl_glue.h"

#include <dlfcn.h>
#include <nccl.h>

#include <cstdlib>
#include <cstring>

namespace efm {

namespace {
decltype(&ncclGetUniqueId) p_get_id = nullptr;
decltype(&ncclCommInitRank) p_init = nullptr;
decltype(&ncclCommDestroy) p_destroy = nullptr;
decltype(&ncclAllReduce) p_all_reduce = nullptr;
decltype(&ncclAllGather) p_all_gather = nullptr;
decltype(&ncclGetErrorString) p_err = nullptr;
decltype(&ncclBroadcast) p_bcast = nullptr;
decltype(&ncclGroupStart) p_group_start = nullptr;
decltype(&ncclGroupEnd) p_group_end = nullptr;

int get_unique_id(void* id128) {
    ncclUniqueId id;
    const ncclResult_t r = p_get_id(&id);
    if (r == ncclSuccess) std::memcpy(id128, &id, sizeof(id));
    return (int)r;
}
int comm_init_rank(void** comm, int nranks, const void* id128, int rank) {
    ncclUniqueId id;
    std::memcpy(&id, id128, sizeof(id));
    ncclComm_t c = nullptr;
    const ncclResult_t r = p_init(&c, nranks, id, rank);
    *comm = c;
    return (int)r;
}
int comm_destroy(void* comm) { return (int)p_destroy(static_cast<ncclComm_t>(comm)); }
int all_reduce_f32_sum(const void* send, void* recv, size_t count, void* comm, cudaStream_t stream) {
    return (int)p_all_reduce(send, recv, count, ncclFloat32, ncclSum, static_cast<ncclComm_t>(comm), stream);
}
int all_gather_f32(const void* send, void* recv, size_t count, void* comm, cudaStream_t stream) {
    return (int)p_all_gather(send, recv, count, ncclFloat32, static_cast<ncclComm_t>(comm), stream);
}
int all_gather_v_bytes(const void* send, void* recv_base, const size_t* offsets, const size_t* counts, int nranks, void* comm,
                       cudaStream_t stream) {
    ncclResult_t r = p_group_start();
    if (r != ncclSuccess) return (int)r;
    for (int root = 0; root < nranks; ++root) {
        const ncclResult_t b = p_bcast(send, static_cast<char*>(recv_base) + offsets[root], counts[root], ncclUint8, root,
                                       static_cast<ncclComm_t>(comm), stream);
        if (b != ncclSuccess) r = b;
    }
    const ncclResult_t e = p_group_end();
    return (int)(r != ncclSuccess ? r : e);
}
const char* error_string(int r) { return p_err != nullptr ? p_err(static_cast<ncclResult_t>(r)) : "nccl error"; }
}  // namespace

const NcclApi& nccl_api() {
    static NcclApi api = [] {
        NcclApi a;
        static_assert(sizeof(ncclUniqueId) == 128, "unique id is 128 bytes in the C ABI");
        const char* override_path = std::getenv("EFM_NCCL_LIB");
        void* h = dlopen(override_path != nullptr ? override_path : "libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (h == nullptr) {
            a.error = std::string("cannot load libnccl.so.2 (set EFM_NCCL_LIB): ") + dlerror();
            return a;
        }
        p_get_id = reinterpret_cast<decltype(p_get_id)>(dlsym(h, "ncclGetUniqueId"));
        p_init = reinterpret_cast<decltype(p_init)>(dlsym(h, "ncclCommInitRank"));
        p_destroy = reinterpret_cast<decltype(p_destroy)>(dlsym(h, "ncclCommDestroy"));
        p_all_reduce = reinterpret_cast<decltype(p_all_reduce)>(dlsym(h, "ncclAllReduce"));
        p_all_gather = reinterpret_cast<decltype(p_all_gather)>(dlsym(h, "ncclAllGather"));
        p_err = reinterpret_cast<decltype(p_err)>(dlsym(h, "ncclGetErrorString"));
        p_bcast = reinterpret_cast<decltype(p_bcast)>(dlsym(h, "ncclBroadcast"));
        p_group_start = reinterpret_cast<decltype(p_group_start)>(dlsym(h, "ncclGroupStart"));
        p_group_end = reinterpret_cast<decltype(p_group_end)>(dlsym(h, "ncclGroupEnd"));
        if (!p_get_id || !p_init || !p_destroy || !p_all_reduce || !p_all_gather || !p_err || !p_bcast || !p_group_start || !p_group_end) {
            a.error = "libnccl.so.2 lacks an expected symbol";
            return a;
        }
        a.get_unique_id = get_unique_id;
        a.comm_init_rank = comm_init_rank;
        a.comm_destroy = comm_destroy;
        a.all_reduce_f32_sum = all_reduce_f32_sum;
        a.all_gather_f32 = all_gather_f32;
        a.all_gather_v_bytes = all_gather_v_bytes;
        a.error_string = error_string;
        a.ok = true;
        return a;
    }();
    return api;
}

}  // namespace efm
