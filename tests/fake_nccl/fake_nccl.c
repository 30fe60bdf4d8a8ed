/* A stand-in for libnccl.so.2 used by the CPU test of the host-side tensor-parallel wait: every symbol the backend
 * binds exists, nothing touches a GPU.  ncclCommGetAsyncError reports success until it has been asked
 * $FAKE_NCCL_FAIL_AFTER times, then ncclSystemError (2); ncclCommAbort counts its calls in $FAKE_NCCL_ABORT_FILE. */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

typedef int ncclResult_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef void* ncclComm_t;
typedef void* cudaStream_t;

static int g_polls = 0;

ncclResult_t ncclGetUniqueId(ncclUniqueId* id) { memset(id, 7, sizeof(*id)); return 0; }
ncclResult_t ncclCommInitRank(ncclComm_t* comm, int n, ncclUniqueId id, int rank) { (void)n; (void)id; (void)rank; *comm = (void*)0x1; return 0; }
ncclResult_t ncclCommDestroy(ncclComm_t comm) { (void)comm; return 0; }
ncclResult_t ncclAllReduce(const void* s, void* r, size_t c, int dt, int op, ncclComm_t comm, cudaStream_t st) {
    (void)s; (void)r; (void)c; (void)dt; (void)op; (void)comm; (void)st; return 0; }
ncclResult_t ncclAllGather(const void* s, void* r, size_t c, int dt, ncclComm_t comm, cudaStream_t st) {
    (void)s; (void)r; (void)c; (void)dt; (void)comm; (void)st; return 0; }
ncclResult_t ncclBroadcast(const void* s, void* r, size_t c, int dt, int root, ncclComm_t comm, cudaStream_t st) {
    (void)s; (void)r; (void)c; (void)dt; (void)root; (void)comm; (void)st; return 0; }
ncclResult_t ncclGroupStart(void) { return 0; }
ncclResult_t ncclGroupEnd(void) { return 0; }
const char* ncclGetErrorString(ncclResult_t r) { return r == 2 ? "unhandled system error (fake)" : "fake nccl"; }
ncclResult_t ncclCommGetAsyncError(ncclComm_t comm, ncclResult_t* async) {
    (void)comm;
    const char* e = getenv("FAKE_NCCL_FAIL_AFTER");
    const int after = e != NULL ? atoi(e) : -1;
    ++g_polls;
    *async = (after >= 0 && g_polls > after) ? 2 : 0;
    return 0;
}
ncclResult_t ncclCommAbort(ncclComm_t comm) {
    (void)comm;
    const char* path = getenv("FAKE_NCCL_ABORT_FILE");
    if (path != NULL) { FILE* f = fopen(path, "a"); if (f != NULL) { fputs("abort\n", f); fclose(f); } }
    return 0;
}
