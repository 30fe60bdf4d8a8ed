// Host-side launch plumbing shared by the layer sequences: a launcher that attaches the
// programmatic-dependent-launch attribute and counts launches, and the shape heuristics that
// pick a GEMV variant and a split count for decode attention.
#pragma once
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <cstdlib>
#include <vector>

#include "../operators/decode_attention.cuh"
#include "../operators/decode_mega.cuh"
#include "../operators/gemv.cuh"

namespace efm {

struct Launcher {
    cudaStream_t stream = nullptr;
    bool pdl = true;                 // programmatic stream serialization between consecutive kernels
    bool cooperative = false;        // next launch only: all blocks co-resident (they wait on each other)
    int64_t* counter = nullptr;
    cudaError_t err = cudaSuccess;   // first failure sticks
    std::vector<cudaEvent_t>* trace = nullptr;   // when set: one event recorded after every launch
    bool phase_timing = false;       // persistent decode kernel: stamp %globaltimer at every phase boundary

    template <typename... KArgs, typename... Args>
    void launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, Args&&... args) {
        if (err != cudaSuccess) return;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = block;
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        if (cooperative) {
            attr[0].id = cudaLaunchAttributeCooperative;
            attr[0].val.cooperative = 1;
        } else {
            attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[0].val.programmaticStreamSerializationAllowed = 1;
        }
        cfg.attrs = (pdl || cooperative) ? attr : nullptr;
        cfg.numAttrs = (pdl || cooperative) ? 1 : 0;
        cooperative = false;
        err = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
        if (counter != nullptr) ++*counter;
        if (trace != nullptr && err == cudaSuccess) {
            cudaEvent_t ev = nullptr;
            if (cudaEventCreate(&ev) == cudaSuccess) { cudaEventRecord(ev, stream); trace->push_back(ev); }
        }
    }
};

// How many of a block's 16 warps share one row pair (ks).  The serial length of a warp's work is
// waves x units per item; the shortest wins, ties go to the smaller split (less reduction).
inline int plan_gemv_ksplit(int n_items, int K, int n_blocks) {
    const int nch = K / 8;
    int best = 1;
    long best_cost = -1;
    for (int ks = 1; ks <= kGemvWarps; ks *= 2) {
        const long slots = (long)n_blocks * (kGemvWarps / ks);
        const long waves = (n_items + slots - 1) / slots;
        const long cpl = (nch + 32 * ks - 1) / (32 * ks);
        const long units = (cpl + kGemvU - 1) / kGemvU;
        const long cost = waves * units * 64 + ks;
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = ks; }
    }
    return best;
}

// One GEMV phase as its own launch: one block per SM.
template <Epi EPI>
inline void launch_gemv(Launcher& L, const GemvParams& p, int num_sms) {
    const int ks = plan_gemv_ksplit(p.n_items, p.K, num_sms);
    L.launch(gemv_kernel<EPI>, dim3(num_sms), dim3(kGemvThreads), gemv_smem_bytes(p.K), p, ks);
}

inline cudaError_t configure_gemv(int max_smem_optin) {
    cudaError_t e = cudaFuncSetAttribute(gemv_kernel<Epi::Plain>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem_optin);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_kernel<Epi::Residual>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem_optin);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_kernel<Epi::QkvRope>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem_optin);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_kernel<Epi::SwiGlu>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem_optin);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_kernel<Epi::Logits>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem_optin);
    return e;
}

inline cudaError_t configure_decode_mega(int max_smem_optin) {
    cudaError_t e = cudaFuncSetAttribute(decode_mega_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem_optin);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(decode_mega_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem_optin);
}

struct AttnPlan { int n_splits, chunk_cap; };
inline AttnPlan plan_decode_attention(int max_tokens, int kv_heads, int num_sms) {
    int n = (max_tokens + kAttnTile - 1) / kAttnTile;
    n = std::min(n, std::max(1, num_sms / std::max(1, kv_heads)));
    n = std::max(1, std::min(n, kMaxSplits));
    return AttnPlan{n, (max_tokens + n - 1) / n};
}

// Opt-in shared-memory sizes; called once per device at set-up, never inside a stream capture.
inline cudaError_t configure_decode_attention() {
    cudaError_t e = cudaFuncSetAttribute(decode_attention_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)decode_attention_smem_bytes(128, 0));
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(decode_attention_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                (int)decode_attention_smem_bytes(64, 0));
}

inline void launch_decode_attention(Launcher& L, const DecodeAttnParams& p, int head_dim) {
    const size_t smem = decode_attention_smem_bytes(head_dim, p.chunk_cap);
    const dim3 grid(p.n_splits, p.kv_heads), block(kAttnThreads);
    if (head_dim == 128) L.launch(decode_attention_kernel<128>, grid, block, smem, p);
    else L.launch(decode_attention_kernel<64>, grid, block, smem, p);
}

}  // namespace efm
