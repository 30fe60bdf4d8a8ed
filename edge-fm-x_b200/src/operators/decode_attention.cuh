// Batch-1 GQA decode attention over the fixed prefix plus the growing KV of one slot.
// Replaces FlashInfer SingleDecodeWithKVCache + MergeStates as the reference calls them
// (src/operators/attention_op.cu:1428-1466): split-KV, kv_len read from a device word so one
// captured graph serves every step.  q arrives rotated and K is cached rotated, so no RoPE here.
//
// Grid (n_splits, kv_heads), 128 threads.  A block owns one contiguous chunk of cache rows of
// one kv head and serves all `group` query heads that share it, so K and V are read once.
//   1. scores: 4 threads per cache row, 128-bit loads, fp32 dot with q held in shared memory;
//   2. chunk-local softmax statistics (max m, sum l) per query head, fp32;
//   3. o = sum_t p_t * v_t with 8 channels per thread, reduced over the row groups;
//   4. the (m, l, o) triple goes to scratch; the last block to finish for a kv head (atomic
//      ticket, no spinning) merges all chunks and writes the bf16 output.
// Bound: HBM (2 * kv_len * kv_heads * D * 2 bytes per layer), in practice launch/latency.
#pragma once
#include "common.cuh"

namespace efm {

constexpr int kMaxGroup = 8;

struct DecodeAttnParams {
    const __nv_bfloat16* q;        // [q_heads, D]
    const __nv_bfloat16* k_cache;  // [max_tokens, kv_heads, D]
    const __nv_bfloat16* v_cache;
    __nv_bfloat16* out;            // [q_heads, D]
    DecodeState* state;            // kv_len source when non-null
    int kv_len_static;
    int q_heads, kv_heads, group, n_splits, max_tokens, chunk_cap;
    float scale;
    float* part_o;                 // [q_heads][n_splits][D]
    float* part_ml;                // [q_heads][n_splits][2]
    unsigned int* counters;        // [kv_heads], zero between launches
};

template <int D>
__global__ void __launch_bounds__(128) decode_attention_kernel(const DecodeAttnParams p) {
    constexpr int NT = 128;
    constexpr int QV = D / 32;            // uint4 loads per thread and row in the score phase
    constexpr int TPR = D / 8;            // threads per V row
    constexpr int TG = NT / TPR;          // row groups in the P.V phase
    extern __shared__ __align__(16) unsigned char attn_smem[];
    constexpr int QP = D / 4 + 4;         // padded quarter-row of q: the 4 threads of a row hit 4 banks
    float* qs = reinterpret_cast<float*>(attn_smem);            // [kMaxGroup][4][QP]
    float* ored = qs + kMaxGroup * 4 * QP;                       // [4][kMaxGroup][D]
    float* ml = ored + 4 * kMaxGroup * D;                        // [kMaxGroup][2]
    float* sc = ml + kMaxGroup * 2;                              // [kMaxGroup][chunk_cap]
    __shared__ unsigned int ticket_s;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int split = blockIdx.x, kvh = blockIdx.y;
    const int G = p.group;
    pdl_launch_dependents();
    pdl_wait();

    int kv_len = p.state != nullptr ? (int)p.state->kv_len : p.kv_len_static;
    if (kv_len > p.max_tokens) {
        if (p.state != nullptr) p.state->error = 2;
        kv_len = p.max_tokens;
    }
    int chunk = (kv_len + p.n_splits - 1) / p.n_splits;
    if (chunk > p.chunk_cap) chunk = p.chunk_cap;     // cannot happen when kv_len <= max_tokens
    const int start = split * chunk;
    int n = kv_len - start;
    n = n < 0 ? 0 : (n > chunk ? chunk : n);
    const size_t row_stride = (size_t)p.kv_heads * D;

    for (int i = tid; i < G * D; i += NT) {
        const int g = i / D, d = i - g * D;
        qs[(g * 4 + d / (D / 4)) * QP + d % (D / 4)] = __bfloat162float(p.q[(size_t)(kvh * G) * D + i]);
    }
    __syncthreads();

    // ---- 1. scores ------------------------------------------------------------------------
    {
        const int tsub = tid >> 2, part = tid & 3;
        for (int t0 = 0; t0 < n; t0 += NT / 4) {
            const int t = t0 + tsub;
            float dot[kMaxGroup];
#pragma unroll
            for (int g = 0; g < kMaxGroup; ++g) dot[g] = 0.f;
            if (t < n) {
                const __nv_bfloat16* kr = p.k_cache + (size_t)(start + t) * row_stride + (size_t)kvh * D + part * (D / 4);
                uint4 kvv[QV];
#pragma unroll
                for (int j = 0; j < QV; ++j) kvv[j] = ld_cached(kr + j * 8);
#pragma unroll
                for (int j = 0; j < QV; ++j) {
                    float kf[8];
                    unpack8(kvv[j], kf);
#pragma unroll
                    for (int g = 0; g < kMaxGroup; ++g) {
                        if (g < G) {
                            const float* qg = qs + (g * 4 + part) * QP + j * 8;
#pragma unroll
                            for (int e = 0; e < 8; ++e) dot[g] = fmaf(kf[e], qg[e], dot[g]);
                        }
                    }
                }
            }
#pragma unroll
            for (int g = 0; g < kMaxGroup; ++g) {
                dot[g] += __shfl_xor_sync(0xffffffffu, dot[g], 1);
                dot[g] += __shfl_xor_sync(0xffffffffu, dot[g], 2);
            }
            if (t < n && part == 0) {
#pragma unroll
                for (int g = 0; g < kMaxGroup; ++g)
                    if (g < G) sc[g * p.chunk_cap + t] = dot[g] * p.scale;
            }
        }
    }
    __syncthreads();

    // ---- 2. chunk-local softmax ---------------------------------------------------------------
    for (int g = warp; g < G; g += 4) {
        float m = -INFINITY;
        for (int t = lane; t < n; t += 32) m = fmaxf(m, sc[g * p.chunk_cap + t]);
        m = warp_max(m);
        float l = 0.f;
        for (int t = lane; t < n; t += 32) {
            const float e = expf(sc[g * p.chunk_cap + t] - m);
            sc[g * p.chunk_cap + t] = e;
            l += e;
        }
        l = warp_sum(l);
        if (lane == 0) { ml[g * 2] = m; ml[g * 2 + 1] = l; }
    }
    __syncthreads();

    // ---- 3. o = P.V ------------------------------------------------------------------------------
    {
        const int dpart = tid % TPR, tg = tid / TPR;
        float acc[kMaxGroup][8];
#pragma unroll
        for (int g = 0; g < kMaxGroup; ++g)
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[g][e] = 0.f;
        for (int t = tg; t < n; t += TG) {
            const uint4 vv = ld_cached(p.v_cache + (size_t)(start + t) * row_stride + (size_t)kvh * D + dpart * 8);
            float vf[8];
            unpack8(vv, vf);
#pragma unroll
            for (int g = 0; g < kMaxGroup; ++g) {
                if (g < G) {
                    const float pg = sc[g * p.chunk_cap + t];
#pragma unroll
                    for (int e = 0; e < 8; ++e) acc[g][e] = fmaf(pg, vf[e], acc[g][e]);
                }
            }
        }
        // fold the row groups that live in the same warp, then the four warps
#pragma unroll
        for (int g = 0; g < kMaxGroup; ++g)
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                float v = acc[g][e];
#pragma unroll
                for (int o = TPR; o < 32; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                acc[g][e] = v;
            }
        if (lane < TPR) {
#pragma unroll
            for (int g = 0; g < kMaxGroup; ++g)
                if (g < G) {
#pragma unroll
                    for (int e = 0; e < 8; ++e) ored[(warp * kMaxGroup + g) * D + lane * 8 + e] = acc[g][e];
                }
        }
    }
    __syncthreads();

    // ---- 4. publish the partial, merge if last ---------------------------------------------------
    for (int i = tid; i < G * D; i += NT) {
        const int g = i / D, d = i - g * D;
        const float o = ored[(0 * kMaxGroup + g) * D + d] + ored[(1 * kMaxGroup + g) * D + d] +
                        ored[(2 * kMaxGroup + g) * D + d] + ored[(3 * kMaxGroup + g) * D + d];
        const int qh = kvh * G + g;
        p.part_o[((size_t)qh * p.n_splits + split) * D + d] = o;
    }
    if (tid < G) {
        const int qh = kvh * G + tid;
        float m = ml[tid * 2], l = ml[tid * 2 + 1];
        if (n == 0) { m = -INFINITY; l = 0.f; }
        p.part_ml[((size_t)qh * p.n_splits + split) * 2] = m;
        p.part_ml[((size_t)qh * p.n_splits + split) * 2 + 1] = l;
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) ticket_s = atomicAdd(&p.counters[kvh], 1u);
    __syncthreads();
    if (ticket_s != (unsigned)(p.n_splits - 1)) return;
    __threadfence();
    for (int i = tid; i < G * D; i += NT) {
        const int g = i / D, d = i - g * D;
        const int qh = kvh * G + g;
        const float* mlp = p.part_ml + (size_t)qh * p.n_splits * 2;
        float M = -INFINITY;
        for (int s = 0; s < p.n_splits; ++s) M = fmaxf(M, __ldcg(mlp + s * 2));
        float L = 0.f, O = 0.f;
        for (int s = 0; s < p.n_splits; ++s) {
            const float ms = __ldcg(mlp + s * 2), ls = __ldcg(mlp + s * 2 + 1);
            if (ls > 0.f) {
                const float w = expf(ms - M);
                L = fmaf(ls, w, L);
                O = fmaf(__ldcg(p.part_o + ((size_t)qh * p.n_splits + s) * D + d), w, O);
            }
        }
        p.out[(size_t)qh * D + d] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
    }
    if (tid == 0) p.counters[kvh] = 0u;
}

inline size_t decode_attention_smem_bytes(int D, int chunk_cap) {
    return (size_t)(kMaxGroup * 4 * (D / 4 + 4) + 4 * kMaxGroup * D + kMaxGroup * 2 + kMaxGroup * chunk_cap) * sizeof(float);
}

}  // namespace efm
