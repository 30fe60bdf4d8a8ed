// Batch-1 GQA decode attention over the fixed prefix plus the growing KV of one slot.
// Replaces FlashInfer SingleDecodeWithKVCache + MergeStates as the reference calls them
// (src/operators/attention_op.cu:1428-1466): split-KV, kv_len read from a device word so one
// captured graph serves every step.  q arrives rotated and K is cached rotated, so no RoPE here.
//
// Grid (n_splits, kv_heads), 256 threads.  A block owns one contiguous chunk of cache rows of one
// kv head and serves all `group` query heads that share it, so K and V are read once.  The chunk
// is walked in tiles of 64 rows (normally exactly one tile):
//   1. every thread issues its quarter-row of K and of V together (one DRAM round trip);
//   2. scores against q (fp32, shared memory), tile max, p = exp(s - max), running (m, l);
//   3. o += P.V from shared memory, 4 channels per thread, folded over the row groups;
//   4. (m, l, o) go to scratch; the last block to finish for a kv head (atomic ticket, nobody
//      spins) computes the merge weights once and folds all chunks with independent loads.
// Bound: HBM (2 * kv_len * kv_heads * D * 2 bytes per layer); in practice latency.
#pragma once
#include "common.cuh"

namespace efm {

constexpr int kMaxGroup = 8;
constexpr int kAttnTile = 64;
constexpr int kMaxSplits = 64;

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
struct DecodeAttnSmem {
    static constexpr int QP = D / 4 + 4;                    // padded quarter-row of q
    float q[kMaxGroup][4][QP];
    float ored[8][kMaxGroup][D];                            // per-warp partial outputs
    float p[kMaxGroup][kAttnTile];
    float wmax[8][kMaxGroup];
    float wsum[8][kMaxGroup];
    float run_m[kMaxGroup], run_l[kMaxGroup], rescale[kMaxGroup];
    float mw[kMaxGroup][kMaxSplits];                        // merge weights
    __nv_bfloat16 v[kAttnTile][D];
    unsigned int ticket;
};

// The 256 threads of one attention work item synchronise either with the whole-block barrier
// (stand-alone kernel) or with named barrier 9 (inside the persistent decode kernel, where the
// block has more warps than the work item uses).
template <bool NAMED>
__device__ __forceinline__ void attn_sync() {
    if constexpr (NAMED) asm volatile("bar.sync 9, 256;" ::: "memory");
    else __syncthreads();
}

// One (chunk, kv head) work item.  Every load of data another block may have written in this
// step (q, the newest cache row, the partials) bypasses L1.
template <int D, bool NAMED>
__device__ __forceinline__ void decode_attention_body(const DecodeAttnParams& p, const int split, const int kvh,
                                                      unsigned char* attn_smem) {
    constexpr int NT = 256;
    constexpr int QV = D / 32;            // uint4 per thread and row (a quarter row)
    constexpr int TPR = D / 4;            // threads per V row in the P.V phase (4 channels each)
    constexpr int TG = NT / TPR;          // row groups in the P.V phase
    DecodeAttnSmem<D>& sm = *reinterpret_cast<DecodeAttnSmem<D>*>(attn_smem);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = p.group;

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

    const int tok = tid >> 2, part = tid & 3;                    // score phase: 4 threads per row
    const int dpart = tid % TPR, tg = tid / TPR;                 // P.V phase
    float acc[kMaxGroup][4];
#pragma unroll
    for (int g = 0; g < kMaxGroup; ++g)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[g][e] = 0.f;

    for (int i = tid; i < G * D; i += NT) {
        const int g = i / D, d = i - g * D;
        sm.q[g][d / (D / 4)][d % (D / 4)] = bf16_bits_to_f32(__ldcg(reinterpret_cast<const unsigned short*>(p.q) + (size_t)(kvh * G) * D + i));
    }
    if (tid < kMaxGroup) { sm.run_m[tid] = -INFINITY; sm.run_l[tid] = 0.f; }

    for (int t0 = 0; t0 < n; t0 += kAttnTile) {
        const int nt = min(kAttnTile, n - t0);
        const bool valid = tok < nt;
        // ---- 1. K and V quarter rows in flight together -------------------------------------
        uint4 kq[QV], vq[QV];
        if (valid) {
            const size_t off = (size_t)(start + t0 + tok) * row_stride + (size_t)kvh * D + part * (D / 4);
#pragma unroll
            for (int j = 0; j < QV; ++j) kq[j] = ld_cg(p.k_cache + off + j * 8);
#pragma unroll
            for (int j = 0; j < QV; ++j) vq[j] = ld_cg(p.v_cache + off + j * 8);
        }
        attn_sync<NAMED>();      // q staged (first tile) / previous tile's p and v fully consumed
        // ---- 2. scores ----------------------------------------------------------------------
        float s[kMaxGroup];
#pragma unroll
        for (int g = 0; g < kMaxGroup; ++g) s[g] = 0.f;
        if (valid) {
#pragma unroll
            for (int j = 0; j < QV; ++j) {
                float kf[8];
                unpack8(kq[j], kf);
#pragma unroll
                for (int g = 0; g < kMaxGroup; ++g) {
                    if (g < G) {
                        const float* qg = &sm.q[g][part][j * 8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) s[g] = fmaf(kf[e], qg[e], s[g]);
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < QV; ++j)
                *reinterpret_cast<uint4*>(&sm.v[tok][part * (D / 4) + j * 8]) = vq[j];
        }
#pragma unroll
        for (int g = 0; g < kMaxGroup; ++g) {
            s[g] += __shfl_xor_sync(0xffffffffu, s[g], 1);
            s[g] += __shfl_xor_sync(0xffffffffu, s[g], 2);
            s[g] = valid ? s[g] * p.scale : -INFINITY;
            float m = s[g];
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 4));
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 8));
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 16));
            if (lane == 0) sm.wmax[warp][g] = m;
        }
        attn_sync<NAMED>();
#pragma unroll
        for (int g = 0; g < kMaxGroup; ++g) {
            if (g < G) {
                float m_new = sm.run_m[g];
#pragma unroll
                for (int w = 0; w < 8; ++w) m_new = fmaxf(m_new, sm.wmax[w][g]);
                const float pv = valid ? expf(s[g] - m_new) : 0.f;
                if (part == 0 && tok < kAttnTile) sm.p[g][tok] = pv;
                float ps = pv;
                ps += __shfl_xor_sync(0xffffffffu, ps, 4);
                ps += __shfl_xor_sync(0xffffffffu, ps, 8);
                ps += __shfl_xor_sync(0xffffffffu, ps, 16);
                if (lane == 0) sm.wsum[warp][g] = ps;
                if (tid == 0) sm.rescale[g] = m_new;      // new running max (read after the barrier)
            }
        }
        attn_sync<NAMED>();
        // ---- 3. o = o * rescale + P.V -----------------------------------------------------------
#pragma unroll
        for (int g = 0; g < kMaxGroup; ++g) {
            if (g < G) {
                const float m_old = sm.run_m[g], m_new = sm.rescale[g];
                const float f = m_old == -INFINITY ? 0.f : expf(m_old - m_new);
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[g][e] *= f;
            }
        }
        for (int t = tg; t < nt; t += TG) {
            const uint2 vv = *reinterpret_cast<const uint2*>(&sm.v[t][dpart * 4]);
            const float vf[4] = {bf16lo(vv.x), bf16hi(vv.x), bf16lo(vv.y), bf16hi(vv.y)};
#pragma unroll
            for (int g = 0; g < kMaxGroup; ++g) {
                if (g < G) {
                    const float pg = sm.p[g][t];
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc[g][e] = fmaf(pg, vf[e], acc[g][e]);
                }
            }
        }
        attn_sync<NAMED>();      // everyone has read run_m / rescale / wsum inputs of this tile
        if (tid < G) {
            const float m_old = sm.run_m[tid], m_new = sm.rescale[tid];
            float l = sm.run_l[tid] * (m_old == -INFINITY ? 0.f : expf(m_old - m_new));
#pragma unroll
            for (int w = 0; w < 8; ++w) l += sm.wsum[w][tid];
            sm.run_l[tid] = l;
            sm.run_m[tid] = m_new;
        }
    }

    // ---- fold the row groups: lanes of a warp first, then the eight warps -----------------------
#pragma unroll
    for (int g = 0; g < kMaxGroup; ++g)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float v = acc[g][e];
#pragma unroll
            for (int o = TPR; o < 32; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            acc[g][e] = v;
        }
    if (lane < TPR) {
#pragma unroll
        for (int g = 0; g < kMaxGroup; ++g)
            if (g < G) *reinterpret_cast<float4*>(&sm.ored[warp][g][lane * 4]) = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
    }
    attn_sync<NAMED>();

    // ---- 4. publish the partial, merge if last -------------------------------------------------
    for (int i = tid; i < G * D; i += NT) {
        const int g = i / D, d = i - g * D;
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) o += sm.ored[w][g][d];
        p.part_o[((size_t)(kvh * G + g) * p.n_splits + split) * D + d] = o;
    }
    if (tid < G) {
        const int qh = kvh * G + tid;
        p.part_ml[((size_t)qh * p.n_splits + split) * 2] = sm.run_m[tid];
        p.part_ml[((size_t)qh * p.n_splits + split) * 2 + 1] = sm.run_l[tid];
    }
    __threadfence();
    attn_sync<NAMED>();
    if (tid == 0) sm.ticket = atomicAdd(&p.counters[kvh], 1u);
    attn_sync<NAMED>();
    if (sm.ticket != (unsigned)(p.n_splits - 1)) return;
    __threadfence();
    // merge weights: warp g handles query head g, lanes over chunks
    for (int g = warp; g < G; g += 8) {
        const float* mlp = p.part_ml + (size_t)(kvh * G + g) * p.n_splits * 2;
        float ms[kMaxSplits / 32], ls[kMaxSplits / 32];
        float M = -INFINITY;
#pragma unroll
        for (int j = 0; j < kMaxSplits / 32; ++j) {
            const int s = lane + j * 32;
            ms[j] = s < p.n_splits ? __ldcg(mlp + s * 2) : -INFINITY;
            ls[j] = s < p.n_splits ? __ldcg(mlp + s * 2 + 1) : 0.f;
            M = fmaxf(M, ms[j]);
        }
        M = warp_max(M);
        float L = 0.f, w[kMaxSplits / 32];
#pragma unroll
        for (int j = 0; j < kMaxSplits / 32; ++j) {
            w[j] = ls[j] > 0.f ? expf(ms[j] - M) : 0.f;
            L = fmaf(ls[j], w[j], L);
        }
        L = warp_sum(L);
        const float inv = L > 0.f ? 1.0f / L : 0.f;
#pragma unroll
        for (int j = 0; j < kMaxSplits / 32; ++j) {
            const int s = lane + j * 32;
            if (s < p.n_splits) sm.mw[g][s] = w[j] * inv;
        }
    }
    attn_sync<NAMED>();
    for (int i = tid; i < G * D; i += NT) {
        const int g = i / D, d = i - g * D;
        const float* po = p.part_o + (size_t)(kvh * G + g) * p.n_splits * D + d;
        float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
        for (int s0 = 0; s0 < p.n_splits; s0 += 16) {          // 16 independent L2 loads per round trip
            float v[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = s0 + j < p.n_splits ? __ldcg(po + (size_t)(s0 + j) * D) : 0.f;
#pragma unroll
            for (int j = 0; j < 16; j += 4) {
                if (s0 + j < p.n_splits) {
                    o0 = fmaf(v[j], sm.mw[g][min(s0 + j, kMaxSplits - 1)], o0);
                    o1 = fmaf(v[j + 1], s0 + j + 1 < p.n_splits ? sm.mw[g][s0 + j + 1] : 0.f, o1);
                    o2 = fmaf(v[j + 2], s0 + j + 2 < p.n_splits ? sm.mw[g][s0 + j + 2] : 0.f, o2);
                    o3 = fmaf(v[j + 3], s0 + j + 3 < p.n_splits ? sm.mw[g][s0 + j + 3] : 0.f, o3);
                }
            }
        }
        p.out[(size_t)(kvh * G + g) * D + d] = __float2bfloat16_rn((o0 + o1) + (o2 + o3));
    }
    if (tid == 0) p.counters[kvh] = 0u;
}

template <int D>
__global__ void __launch_bounds__(256) decode_attention_kernel(const DecodeAttnParams p) {
    extern __shared__ __align__(16) unsigned char attn_smem_raw[];
    pdl_launch_dependents();
    pdl_wait();
    decode_attention_body<D, false>(p, blockIdx.x, blockIdx.y, attn_smem_raw);
}

inline size_t decode_attention_smem_bytes(int D, int /*chunk_cap*/) {
    return D == 128 ? sizeof(DecodeAttnSmem<128>) : sizeof(DecodeAttnSmem<64>);
}

}  // namespace efm
