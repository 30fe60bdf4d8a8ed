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
#include "../operators/gemv.cuh"
#include "../operators/gemv_w4.cuh"

namespace efm {

struct Launcher {
    cudaStream_t stream = nullptr;
    bool pdl = true;                 // programmatic stream serialization between consecutive kernels
    bool pdl_rows = false;           // keep `pdl` for the row / attention kernels of the prefill family too (they open with the wait)
    int cluster_x = 0;               // next launch only: thread-block cluster of this many blocks along x
    float* gemm_ws = nullptr;        // split-K workspace of the owning context (nullptr: GEMMs never split)
    size_t gemm_ws_floats = 0;
    int num_sms = 148;
    int64_t* counter = nullptr;
    cudaError_t err = cudaSuccess;   // first failure sticks
    std::vector<cudaEvent_t>* trace = nullptr;   // when set: one event recorded after every launch

    template <typename... KArgs, typename... Args>
    void launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, Args&&... args) {
        if (err != cudaSuccess) return;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = block;
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[2];
        int na = 0;
        if (pdl) {
            attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[na++].val.programmaticStreamSerializationAllowed = 1;
        }
        if (cluster_x > 1) {
            attr[na].id = cudaLaunchAttributeClusterDimension;
            attr[na].val.clusterDim.x = (unsigned)cluster_x;
            attr[na].val.clusterDim.y = 1;
            attr[na++].val.clusterDim.z = 1;
        }
        cfg.attrs = na > 0 ? attr : nullptr;
        cfg.numAttrs = na;
        cluster_x = 0;
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

// INT4 form: `ks` warps share one 16-row tile (8 row pairs), the 128-column groups of K go round-robin over them;
// the split balances (tiles per warp group) x (groups per warp).
inline int plan_gemv_w4_ksplit(int n_items, int K, int n_blocks) {
    const int n_groups = K / 128, tiles = (n_items + 7) / 8;
    int best = 1;
    long best_cost = -1;
    for (int ks = 1; ks <= kGemvWarps; ks *= 2) {
        const long slots = (long)n_blocks * (kGemvWarps / ks);
        const long waves = (tiles + slots - 1) / slots;
        const long gpw = (n_groups + ks - 1) / ks;
        const long cost = waves * gpw * 4 + ks;
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = ks; }
    }
    return best;
}

template <Epi EPI>
inline void launch_gemv_w4(Launcher& L, const GemvW4Params& p, int num_sms) {
    const int ks = plan_gemv_w4_ksplit(p.g.n_items, p.g.K, num_sms);
    L.launch(gemv_w4_kernel<EPI>, dim3(num_sms), dim3(kGemvThreads), gemv_w4_smem_bytes(p.g.K), p, ks);
}

inline cudaError_t configure_gemv(int max_smem_optin) {
    cudaError_t e = cudaFuncSetAttribute(gemv_kernel<Epi::Plain>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem_optin);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_kernel<Epi::Residual>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem_optin);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_kernel<Epi::QkvRope>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem_optin);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_kernel<Epi::SwiGlu>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem_optin);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_kernel<Epi::Logits>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem_optin);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_kernel<Epi::Peers>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem_optin);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_w4_kernel<Epi::Plain>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem_optin);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_w4_kernel<Epi::Residual>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem_optin);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_w4_kernel<Epi::QkvRope>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem_optin);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_w4_kernel<Epi::SwiGlu>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem_optin);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_w4_kernel<Epi::Logits>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem_optin);
    return e;
}

struct AttnPlan { int n_splits, chunk_cap, cluster; };

// Largest cluster the decode attention kernel can run with on this device (16, 8 or 0 = cluster form
// unavailable / switched off with EFM_B200_ATTN_CLUSTER=0); set by configure_decode_attention().
inline int& decode_attention_max_cluster() {
    static int v = 0;
    return v;
}

inline AttnPlan plan_decode_attention(int max_tokens, int kv_heads, int num_sms) {
    int n = (max_tokens + 63) / 64;           // planned in units of 64 rows: as many blocks as that gives, up to the caps
    const int maxc = decode_attention_max_cluster();
    if (maxc > 1 && n <= 2 * maxc) {          // at most one 128-row tile per block: one cluster per kv head
        int cs = 1;
        while (cs < n && cs < maxc) cs <<= 1;
        return AttnPlan{cs, (max_tokens + cs - 1) / cs, cs};
    }
    n = std::min(n, std::max(1, num_sms / std::max(1, kv_heads)));
    n = std::max(1, std::min(n, kMaxSplits));
    return AttnPlan{n, (max_tokens + n - 1) / n, 0};
}

template <int D>
inline cudaError_t configure_decode_attention_d(int& max_cluster) {
    const int smem = (int)decode_attention_smem_bytes(D, 0);
    cudaError_t e = cudaFuncSetAttribute(decode_attention_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(decode_attention_cluster_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    const bool wide = cudaFuncSetAttribute(decode_attention_cluster_kernel<D>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess;
    for (int cs = wide ? 16 : 8; cs >= 2; cs >>= 1) {       // the widest cluster the device can place
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(cs, 1, 1);
        cfg.blockDim = dim3(kAttnThreads);
        cfg.dynamicSmemBytes = smem;
        cudaLaunchAttribute at;
        at.id = cudaLaunchAttributeClusterDimension;
        at.val.clusterDim.x = (unsigned)cs;
        at.val.clusterDim.y = at.val.clusterDim.z = 1;
        cfg.attrs = &at;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, decode_attention_cluster_kernel<D>, &cfg) == cudaSuccess && n >= 1) {
            max_cluster = std::min(max_cluster, cs);
            return cudaSuccess;
        }
    }
    (void)cudaGetLastError();
    max_cluster = 0;
    return cudaSuccess;
}

// Opt-in shared-memory sizes and the cluster width; called once per device at set-up, never inside a
// stream capture.
inline cudaError_t configure_decode_attention() {
    int maxc = 16;
    cudaError_t e = configure_decode_attention_d<128>(maxc);
    if (e == cudaSuccess) e = configure_decode_attention_d<64>(maxc);
    const char* env = std::getenv("EFM_B200_ATTN_CLUSTER");
    if (env != nullptr && env[0] == '0') maxc = 0;
    decode_attention_max_cluster() = maxc;
    return e;
}

inline void launch_decode_attention(Launcher& L, const DecodeAttnParams& p, int head_dim) {
    const size_t smem = decode_attention_smem_bytes(head_dim, p.chunk_cap);
    const dim3 grid(p.n_splits, p.kv_heads), block(kAttnThreads);
    if (p.cluster > 1) {
        L.cluster_x = p.cluster;
        if (head_dim == 128) L.launch(decode_attention_cluster_kernel<128>, grid, block, smem, p);
        else L.launch(decode_attention_cluster_kernel<64>, grid, block, smem, p);
        return;
    }
    if (head_dim == 128) L.launch(decode_attention_kernel<128>, grid, block, smem, p);
    else L.launch(decode_attention_kernel<64>, grid, block, smem, p);
}

}  // namespace efm
