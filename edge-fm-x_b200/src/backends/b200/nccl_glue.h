// NCCL through dlopen: single-GPU users need no NCCL at link or load time; tensor-parallel
// contexts load libnccl.so.2 (already resident in a torch process, else from the loader path or
// EFM_NCCL_LIB) on first use.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

#include <string>

namespace efm {

struct NcclApi {
    bool ok = false;
    std::string error;
    int (*get_unique_id)(void* id128) = nullptr;
    int (*comm_init_rank)(void** comm, int nranks, const void* id128, int rank) = nullptr;   // wrapper, see .cpp
    int (*comm_destroy)(void* comm) = nullptr;
    int (*comm_async_error)(void* comm, int* async_result) = nullptr;   // ncclCommGetAsyncError
    int (*comm_abort)(void* comm) = nullptr;                            // ncclCommAbort
    int (*all_reduce_f32_sum)(const void* send, void* recv, size_t count, void* comm, cudaStream_t stream) = nullptr;
    int (*all_gather_f32)(const void* send, void* recv, size_t count, void* comm, cudaStream_t stream) = nullptr;
    // all-gather with a different byte count per rank: rank r's `send` (counts[r] bytes) lands at recv_base +
    // offsets[r] on every rank (grouped ncclBroadcast calls)
    int (*all_gather_v_bytes)(const void* send, void* recv_base, const size_t* offsets, const size_t* counts, int nranks,
                              void* comm, cudaStream_t stream) = nullptr;
    const char* (*error_string)(int) = nullptr;
};

const NcclApi& nccl_api();

// Polls ready(arg) (non-zero = done) and the communicator's asynchronous error state until done, error or timeout.
// Returns 0 ready / 1 NCCL error / 2 timeout; on 1 and 2 the communicator was aborted and *what says why.
int tp_host_wait(void* comm, int (*ready)(void*), void* arg, double timeout_s, std::string* what);

}  // namespace efm
