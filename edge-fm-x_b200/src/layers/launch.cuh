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

struct GemvPlan { int items, ksplit, grid; };

// Cost model: a warp's serial work is (128-bit loads per lane) per wave plus a fixed reduce /
// epilogue cost; pick the variant with the shortest critical path and size the grid so that
// every row group slot gets the same number of waves.
inline int gemv_ctas_per_sm() {
    static const int v = [] {
        const char* e = std::getenv("EFM_B200_GEMV_CTAS_PER_SM");     // tuning knob, 1 or 2
        const int x = e != nullptr ? std::atoi(e) : 2;
        return x == 1 ? 1 : 2;
    }();
    return v;
}

inline GemvPlan plan_gemv(int n_items, int K, int num_sms) {
    const int max_ctas = gemv_ctas_per_sm() * num_sms;
    const int nch = K / 8;
    GemvPlan best{2, 1, max_ctas};
    long best_cost = -1;
    for (int items = 2; items >= 1; --items) {
        for (int ks = 1; ks <= 8; ks *= 2) {
            const int gp = 8 / ks;
            const int n_ig = (n_items + items - 1) / items;
            const long slots = (long)max_ctas * gp;
            const long waves = (n_ig + slots - 1) / slots;
            const long per_wave = (long)((nch + 32 * ks - 1) / (32 * ks)) * items * 2 + 8 + (ks > 1 ? 4 : 0);
            const long cost = waves * per_wave;
            if (best_cost < 0 || cost < best_cost) {
                best_cost = cost;
                int grid = (int)((n_ig + waves * gp - 1) / (waves * gp));
                best = GemvPlan{items, ks, std::max(1, std::min(grid, max_ctas))};
            }
        }
    }
    return best;
}

template <Epi EPI>
inline void launch_gemv(Launcher& L, const GemvParams& p, int num_sms) {
    const GemvPlan plan = plan_gemv(p.n_items, p.K, num_sms);
    const size_t smem = gemv_smem_bytes(p.K, plan.items);
    const dim3 grid(plan.grid), block(256);
#define EFM_GEMV_CASE(I, S)                                                                   \
    if (plan.items == I && plan.ksplit == S) {                                                \
        if (smem > 48 * 1024)                                                                 \
            cudaFuncSetAttribute(gemv_kernel<EPI, I, S>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        L.launch(gemv_kernel<EPI, I, S>, grid, block, smem, p);                               \
        return;                                                                               \
    }
    EFM_GEMV_CASE(2, 1) EFM_GEMV_CASE(2, 2) EFM_GEMV_CASE(2, 4) EFM_GEMV_CASE(2, 8)
    EFM_GEMV_CASE(1, 1) EFM_GEMV_CASE(1, 2) EFM_GEMV_CASE(1, 4) EFM_GEMV_CASE(1, 8)
#undef EFM_GEMV_CASE
}

// Persistent decode kernel: how many of a block's 16 warps share one row pair in a phase.
// Fewest dependent load rounds (waves x batches) wins; ties go to the smaller split.
inline int plan_mega_ksplit(int n_items, int K, int n_blocks) {
    const int nch = K / 8;
    int best = 1;
    long best_cost = -1;
    for (int ks = 1; ks <= kMegaWarps; ks *= 2) {
        const long slots = (long)n_blocks * (kMegaWarps / ks);
        const long waves = (n_items + slots - 1) / slots;
        const long batches = (nch + 32 * ks * kMegaU - 1) / (32 * ks * kMegaU);
        const long cost = waves * batches * 64 + ks;
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = ks; }
    }
    return best;
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
    const dim3 grid(p.n_splits, p.kv_heads), block(256);
    if (head_dim == 128) L.launch(decode_attention_kernel<128>, grid, block, smem, p);
    else L.launch(decode_attention_kernel<64>, grid, block, smem, p);
}

}  // namespace efm
