// Shared device helpers for the sm_100a kernels: bf16 packing, streaming loads, warp
// reductions, programmatic-dependent-launch hooks and the device-side decode state.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace efm {

constexpr int kWarp = 32;

// Device-resident state of one decode stream.  The reference keeps the same words at stable
// addresses so that one captured graph serves every step
// (src/engine/tasks/token_generation/cuda/standard_engine.cpp:128-150).
struct DecodeState {
    int32_t token;      // token fed to the next step (written by the sampler)
    uint32_t kv_len;    // cache rows valid once the current step's K/V are appended
    int32_t pos[3];     // M-RoPE positions of the current step's token (t, h, w)
    int32_t step;       // response index the current step's sample is written to
    int32_t error;      // non-zero: a kernel refused an out-of-range index or gave up a wait
    int32_t pad;
};

// ---- bf16 <-> fp32 ---------------------------------------------------------------------
__device__ __forceinline__ float bf16lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
__device__ __forceinline__ float bf16_to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&p);
}

// 8 bf16 weights (one 128-bit word) dotted with 8 fp32 activations.
__device__ __forceinline__ float dot8(const uint4& w, const float (&x)[8], float acc) {
    acc = fmaf(bf16lo(w.x), x[0], acc);
    acc = fmaf(bf16hi(w.x), x[1], acc);
    acc = fmaf(bf16lo(w.y), x[2], acc);
    acc = fmaf(bf16hi(w.y), x[3], acc);
    acc = fmaf(bf16lo(w.z), x[4], acc);
    acc = fmaf(bf16hi(w.z), x[5], acc);
    acc = fmaf(bf16lo(w.w), x[6], acc);
    acc = fmaf(bf16hi(w.w), x[7], acc);
    return acc;
}
__device__ __forceinline__ void unpack8(const uint4& v, float (&x)[8]) {
    x[0] = bf16lo(v.x); x[1] = bf16hi(v.x); x[2] = bf16lo(v.y); x[3] = bf16hi(v.y);
    x[4] = bf16lo(v.z); x[5] = bf16hi(v.z); x[6] = bf16lo(v.w); x[7] = bf16hi(v.w);
}

// ---- loads -----------------------------------------------------------------------------
// Weights are read exactly once per step: read-only path, no L1 allocation.
__device__ __forceinline__ uint4 ld_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 ld_cached(const void* p) { return *reinterpret_cast<const uint4*>(p); }
// L2-only load for data that another block wrote earlier in the same kernel.
__device__ __forceinline__ uint4 ld_cg(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ float bf16_bits_to_f32(unsigned short v) { return __uint_as_float((uint32_t)v << 16); }

// ---- reductions ------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// ---- programmatic dependent launch -----------------------------------------------------
// Every kernel of the decode step calls pdl_wait() before it touches memory another kernel
// writes, and calls it on every path (a grid that exits without waiting would let ITS
// dependents overtake the grid it skipped).  Both are no-ops when the launch carries no
// programmatic attribute.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- bounded waits on words another GPU writes -------------------------------------------
// Longest a kernel waits for its peers' words, in total over all of its waits (nanoseconds on %globaltimer).  Ranks
// of one request run in lock step, so a healthy wait lasts microseconds; the limit only has to outlast host jitter
// between the ranks' launches.  A context overrides it (efm_b200_tp_set_wait_limit).
constexpr unsigned long long kPeerWaitDefaultNs = 2000ull * 1000ull * 1000ull;
__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ int ld_error_word(const int* p) {
    int v;
    asm volatile("ld.volatile.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Wait budget shared by all waits of one thread in one kernel.  `dead` once the budget ran out here, or once any
// thread of any kernel raised the error word: from then on nothing waits any more (the step's result is void and
// the host reads the status), so a lost peer costs one budget, not one per kernel.
struct PeerWait {
    bool dead;
    unsigned long long deadline;      // 0 until the first poll that had to wait
};
__device__ __forceinline__ PeerWait peer_wait_begin(const int* error) {
    PeerWait w;
    w.dead = error != nullptr && ld_error_word(error) != 0;
    w.deadline = 0ull;
    return w;
}
// Called every few failed polls; true = stop waiting.
__device__ __forceinline__ bool peer_wait_expired(PeerWait& w, int* error, volatile int* error_host, unsigned long long budget_ns) {
    const unsigned long long now = globaltimer_ns();
    if (w.deadline == 0ull) { w.deadline = now + (budget_ns != 0ull ? budget_ns : kPeerWaitDefaultNs); return false; }
    const bool raised = error != nullptr && ld_error_word(error) != 0;
    if (now > w.deadline || raised) {
        if (!raised && error != nullptr) atomicExch(error, 3);
        if (error_host != nullptr) *error_host = 3;
        w.dead = true;
        return true;
    }
    return false;
}

}  // namespace efm
