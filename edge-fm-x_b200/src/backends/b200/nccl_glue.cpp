#include "nccl_glue.h"

#include <dlfcn.h>
#include <nccl.h>

#include <chrono>
#include <cstdlib>
#include <cstring>
#include <thread>

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
decltype(&ncclCommGetAsyncError) p_async = nullptr;
decltype(&ncclCommAbort) p_abort = nullptr;

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
int comm_async_error(void* comm, int* async_result) {
    ncclResult_t st = ncclSuccess;
    const ncclResult_t r = p_async(static_cast<ncclComm_t>(comm), &st);
    *async_result = (int)st;
    return (int)r;
}
int comm_abort(void* comm) { return (int)p_abort(static_cast<ncclComm_t>(comm)); }
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
        p_async = reinterpret_cast<decltype(p_async)>(dlsym(h, "ncclCommGetAsyncError"));
        p_abort = reinterpret_cast<decltype(p_abort)>(dlsym(h, "ncclCommAbort"));
        if (!p_get_id || !p_init || !p_destroy || !p_all_reduce || !p_all_gather || !p_err || !p_bcast || !p_group_start || !p_group_end || !p_async ||
            !p_abort) {
            a.error = "libnccl.so.2 lacks an expected symbol";
            return a;
        }
        a.get_unique_id = get_unique_id;
        a.comm_init_rank = comm_init_rank;
        a.comm_destroy = comm_destroy;
        a.comm_async_error = comm_async_error;
        a.comm_abort = comm_abort;
        a.all_reduce_f32_sum = all_reduce_f32_sum;
        a.all_gather_f32 = all_gather_f32;
        a.all_gather_v_bytes = all_gather_v_bytes;
        a.error_string = error_string;
        a.ok = true;
        return a;
    }();
    return api;
}

// Host-side wait of a tensor-parallel context: `ready` about once per millisecond, NCCL's asynchronous error state
// in between, a hard limit on the whole wait.  0 = ready, 1 = NCCL reported an error, 2 = timed out; in both failure
// cases the communicator has been aborted, so that collectives stuck on a lost rank leave the GPU.
int tp_host_wait(void* comm, int (*ready)(void*), void* arg, double timeout_s, std::string* what) {
    const NcclApi& api = nccl_api();
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        if (ready(arg) != 0) return 0;
        if (comm != nullptr && api.ok) {
            int async = 0;
            const int r = api.comm_async_error(comm, &async);
            if (r != 0 || async != 0) {
                if (what != nullptr) *what = std::string("NCCL reported an asynchronous error: ") + api.error_string(r != 0 ? r : async);
                api.comm_abort(comm);
                return 1;
            }
        }
        const double waited = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        if (waited > timeout_s) {
            if (what != nullptr) *what = "tensor-parallel wait timed out after " + std::to_string(timeout_s) + " s (a rank is lost or out of step)";
            if (comm != nullptr && api.ok) api.comm_abort(comm);
            return 2;
        }
        std::this_thread::sleep_for(std::chrono::microseconds(waited < 0.05 ? 50 : 1000));
    }
}

}  // namespace efm
