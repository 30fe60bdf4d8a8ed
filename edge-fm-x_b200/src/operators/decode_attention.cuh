// Batch-1 GQA decode attention over the fixed prefix plus the growing KV of one slot.
// Replaces FlashInfer SingleDecodeWithKVCache + MergeStates as the reference calls them
// (src/operators/attention_op.cu:1428-1466): split-KV, kv_len read from a device word so one
// captured graph serves every step.  q arrives rotated and K is cached rotated, so no RoPE here.
//
// Work item = (chunk of cache rows, kv head), 512 threads; it serves all `group` query heads that
// share the kv head, so K and V are read once.  The chunk is walked in tiles of 128 rows (normally
// exactly one tile):
//   1. every thread issues its eighth of two K rows and of two V rows together (one DRAM round trip);
//   2. scores against q (fp32, shared memory), tile max, p = exp(s - max), running (m, l);
//   3. o += P.V from shared memory, 4 channels per thread, folded over the row groups;
//   4. (m, l, o) go to scratch; the last block to finish for a kv head (atomic ticket, nobody
//      spins) computes the merge weights once and folds all chunks with independent loads.
//   4c. cluster form (short contexts, at most 16 chunks): the chunks of a kv head are the blocks of one
//      thread-block cluster and exchange (m, l, o) through distributed shared memory instead.
// The kernel is latency-bound (about 1 MB of KV per layer): 16 warps per block keep the
// dependent-issue latency covered and the instruction count per warp small.
// Bound: HBM (2 * kv_len * kv_heads * D * 2 bytes per layer); in practice latency.
#pragma once
#include "common.cuh"

namespace efm {

constexpr int kMaxGroup = 8;
constexpr int kAttnTile = 128;
constexpr int kAttnRows = kAttnTile / 64;     // cache rows per thread and tile (512 threads, 8 per row)
constexpr int kMaxSplits = 64;
constexpr int kAttnThreads = 512;
constexpr int kAttnWarps = kAttnThreads / 32;

struct DecodeAttnParams {
    const __nv_bfloat16* q;        // [q_heads, D] bf16 ...
    const float* qf;               // ... or, when non-null, fp32 (the decode step keeps q unrounded)
    const __nv_bfloat16* k_cache;  // [max_tokens, kv_heads, D]
    const __nv_bfloat16* v_cache;
    __nv_bfloat16* out;            // [q_heads, D] bf16 ...
    float* outf;                   // ... or, when non-null, fp32
    DecodeState* state;            // kv_len source when non-null
    int kv_len_static;
    int q_heads, kv_heads, group, n_splits, max_tokens, chunk_cap;
    float scale;
    float* part_o;                 // [q_heads][n_splits][D]
    float* part_ml;                // [q_heads][n_splits][2]
    unsigned int* counters;        // [kv_heads], zero between launches
    int cluster;                   // > 1: the n_splits blocks of a kv head form one thread-block cluster (n_splits == cluster)
    int early;                     // 1: kv_len and every cache row but the newest may be read before the dependency wait
                                   //    (they were written in earlier steps; only q and row kv_len-1 come from the launch before)
};

template <int D>
struct DecodeAttnSmem {
    static constexpr int QP = D / 8 + 4;                    // padded eighth of a q row (bank spread)
    float q[kMaxGroup][8][QP];
    float ored[kAttnWarps][kMaxGroup][D];                   // per-warp partial outputs
    float p[kMaxGroup][kAttnTile];
    float wmax[kAttnWarps][kMaxGroup];
    float wsum[kAttnWarps][kMaxGroup];
    float run_m[kMaxGroup], run_l[kMaxGroup], new_m[kMaxGroup];
    float mw[kMaxGroup][kMaxSplits];                        // merge weights
    __nv_bfloat16 v[kAttnTile][D];
    float fin[kMaxGroup][D];                                // cluster form: this block's un-normalised output
    unsigned int ticket;
};

// One (chunk, kv head) work item, executed by all 512 threads of the block.  Every load of data
// another block may have written in this step (q, the newest cache row, the partials) bypasses L1.
template <int D, bool CLUSTER = false, bool WAIT_INSIDE = false>
__device__ __forceinline__ void decode_attention_body(const DecodeAttnParams& p, const int split, const int kvh,
                                                      unsigned char* attn_smem) {
    constexpr int NT = kAttnThreads, NW = kAttnWarps;
    constexpr int DP = D / 8;             // channels per thread in the score phase
    constexpr int QV = DP / 8;            // uint4 per thread and row
    constexpr int TPR = D / 4;            // threads per V row in the P.V phase (4 channels each)
    constexpr int TG = NT / TPR;          // row groups in the P.V phase
    DecodeAttnSmem<D>& sm = *reinterpret_cast<DecodeAttnSmem<D>*>(attn_smem);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = p.group;

    // WAIT_INSIDE: this body holds the kernel's dependency wait.  With p.early the old cache rows of the first tile
    // are requested before it, so that their DRAM latency runs under the tail of the preceding launch.
    const bool early = WAIT_INSIDE && p.early != 0;
    if (WAIT_INSIDE && !early) pdl_wait();
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

    const int tok = tid >> 3, part = tid & 7;                    // score phase: 8 threads per row
    const int dpart = tid % TPR, tg = tid / TPR;                 // P.V phase
    float acc[kMaxGroup][4];
#pragma unroll
    for (int g = 0; g < kMaxGroup; ++g)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[g][e] = 0.f;

    if (tid < kMaxGroup) { sm.run_m[tid] = -INFINITY; sm.run_l[tid] = 0.f; }

    // ---- 1. K and V slices in flight together; the next tile's are issued as soon as this tile's
    //         registers are free, so that they fly during the softmax and P.V of the current tile
    uint4 kq[kAttnRows][QV], vq[kAttnRows][QV];
    // only_row >= 0: just that cache row (the one the preceding launch appended); skip_row: every row but that one
    auto issue_tile = [&](int t0, int skip_row, int only_row) {
#pragma unroll
        for (int r = 0; r < kAttnRows; ++r) {
            const int row = t0 + tok + 64 * r;
            if (row < n && row < t0 + kAttnTile && start + row != skip_row && (only_row < 0 || start + row == only_row)) {
                const size_t off = (size_t)(start + row) * row_stride + (size_t)kvh * D + part * DP;
#pragma unroll
                for (int j = 0; j < QV; ++j) kq[r][j] = ld_cg(p.k_cache + off + j * 8);
#pragma unroll
                for (int j = 0; j < QV; ++j) vq[r][j] = ld_cg(p.v_cache + off + j * 8);
            }
        }
    };
    if (early) {
        issue_tile(0, kv_len - 1, -1);   // everything but the row the preceding launch appends
        pdl_wait();
    }
    for (int i = tid * 2; i < G * D; i += NT * 2) {              // q: two channels per load
        const int g = i / D, d = i - g * D;
        float q0, q1;
        if (p.qf != nullptr) {
            const float2 two = __ldcg(reinterpret_cast<const float2*>(p.qf + (size_t)(kvh * G) * D + i));
            q0 = two.x;
            q1 = two.y;
        } else {
            const uint32_t two = __ldcg(reinterpret_cast<const unsigned int*>(p.q + (size_t)(kvh * G) * D + i));
            q0 = bf16lo(two);
            q1 = bf16hi(two);
        }
        sm.q[g][d / DP][d % DP] = q0;
        sm.q[g][(d + 1) / DP][(d + 1) % DP] = q1;
    }
    if (early) issue_tile(0, -1, kv_len - 1);
    else issue_tile(0, -1, -1);
    for (int t0 = 0; t0 < n; t0 += kAttnTile) {
        const int nt = min(kAttnTile, n - t0);
        bool valid[kAttnRows];
#pragma unroll
        for (int r = 0; r < kAttnRows; ++r) valid[r] = tok + 64 * r < nt;
        __syncthreads();      // q staged (first tile) / previous tile's p and v fully consumed
        // ---- 2. scores ------------------------------------------------------------------------
        float s[kAttnRows][kMaxGroup];
#pragma unroll
        for (int r = 0; r < kAttnRows; ++r)
#pragma unroll
            for (int g = 0; g < kMaxGroup; ++g) s[r][g] = 0.f;
#pragma unroll
        for (int r = 0; r < kAttnRows; ++r) {
            if (!valid[r]) continue;
#pragma unroll
            for (int j = 0; j < QV; ++j) {
                float kf[8];
                unpack8(kq[r][j], kf);
#pragma unroll
                for (int g = 0; g < kMaxGroup; ++g) {
                    if (g < G) {
                        const float4 qa = *reinterpret_cast<const float4*>(&sm.q[g][part][j * 8]);
                        const float4 qb = *reinterpret_cast<const float4*>(&sm.q[g][part][j * 8 + 4]);
                        s[r][g] = fmaf(kf[0], qa.x, s[r][g]); s[r][g] = fmaf(kf[1], qa.y, s[r][g]);
                        s[r][g] = fmaf(kf[2], qa.z, s[r][g]); s[r][g] = fmaf(kf[3], qa.w, s[r][g]);
                        s[r][g] = fmaf(kf[4], qb.x, s[r][g]); s[r][g] = fmaf(kf[5], qb.y, s[r][g]);
                        s[r][g] = fmaf(kf[6], qb.z, s[r][g]); s[r][g] = fmaf(kf[7], qb.w, s[r][g]);
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < QV; ++j)
                *reinterpret_cast<uint4*>(&sm.v[tok + 64 * r][part * DP + j * 8]) = vq[r][j];
        }
        issue_tile(t0 + kAttnTile, -1, -1);
#pragma unroll
        for (int g = 0; g < kMaxGroup; ++g) {
            float m = -INFINITY;
#pragma unroll
            for (int r = 0; r < kAttnRows; ++r) {
                s[r][g] += __shfl_xor_sync(0xffffffffu, s[r][g], 1);
                s[r][g] += __shfl_xor_sync(0xffffffffu, s[r][g], 2);
                s[r][g] += __shfl_xor_sync(0xffffffffu, s[r][g], 4);
                s[r][g] = valid[r] ? s[r][g] * p.scale : -INFINITY;
                m = fmaxf(m, s[r][g]);
            }
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 8));
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 16));
            if (lane == 0) sm.wmax[warp][g] = m;
        }
        __syncthreads();
#pragma unroll
        for (int g = 0; g < kMaxGroup; ++g) {
            if (g < G) {
                float m_new = sm.run_m[g];
#pragma unroll
                for (int w = 0; w < NW; ++w) m_new = fmaxf(m_new, sm.wmax[w][g]);
                float ps = 0.f;
#pragma unroll
                for (int r = 0; r < kAttnRows; ++r) {
                    const float pv = valid[r] ? expf(s[r][g] - m_new) : 0.f;
                    if (part == 0 && tok + 64 * r < kAttnTile) sm.p[g][tok + 64 * r] = pv;
                    ps += pv;
                }
                ps += __shfl_xor_sync(0xffffffffu, ps, 8);
                ps += __shfl_xor_sync(0xffffffffu, ps, 16);
                if (lane == 0) sm.wsum[warp][g] = ps;
                if (tid == 0) sm.new_m[g] = m_new;        // read after the barrier
            }
        }
        __syncthreads();
        // ---- 3. o = o * rescale + P.V -----------------------------------------------------------
        if (t0 > 0) {
#pragma unroll
            for (int g = 0; g < kMaxGroup; ++g) {
                if (g < G) {
                    const float m_old = sm.run_m[g], m_new = sm.new_m[g];
                    const float f = m_old == -INFINITY ? 0.f : expf(m_old - m_new);
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc[g][e] *= f;
                }
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
        __syncthreads();      // everyone has read run_m / new_m / p / v of this tile
        if (tid < G) {
            const float m_old = sm.run_m[tid], m_new = sm.new_m[tid];
            float l = sm.run_l[tid] * (m_old == -INFINITY ? 0.f : expf(m_old - m_new));
#pragma unroll
            for (int w = 0; w < NW; ++w) l += sm.wsum[w][tid];
            sm.run_l[tid] = l;
            sm.run_m[tid] = m_new;
        }
    }

    // ---- fold the row groups: lanes of a warp first, then the warps ----------------------------
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
            if (g < G)
                *reinterpret_cast<float4*>(&sm.ored[warp][g][(lane % TPR) * 4]) = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
    }
    __syncthreads();

    if constexpr (CLUSTER) {
        // ---- 4c. the blocks of the cluster exchange (m, l, o) through distributed shared memory: no
        //          scratch in global memory, no ticket, one remote round trip
        for (int i = tid; i < G * D; i += NT) {
            const int g = i / D, d = i - g * D;
            float o = 0.f;
#pragma unroll
            for (int w = 0; w < NW; ++w) o += sm.ored[w][g][d];
            sm.fin[g][d] = o;
        }
        asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
        const int CS = p.cluster;
        const uint32_t a_fin = (uint32_t)__cvta_generic_to_shared(&sm.fin[0][0]);
        const uint32_t a_m = (uint32_t)__cvta_generic_to_shared(&sm.run_m[0]);
        const uint32_t a_l = (uint32_t)__cvta_generic_to_shared(&sm.run_l[0]);
        for (int i = split + CS * tid; i < G * D; i += CS * NT) {      // this block's share of the outputs
            const int g = i / D;
            float mr[16], lr[16], orr[16];
#pragma unroll
            for (int r = 0; r < 16; ++r) {
                mr[r] = -INFINITY; lr[r] = 0.f; orr[r] = 0.f;
                if (r < CS) {
                    uint32_t ra;
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(a_m + 4u * g), "r"(r));
                    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(mr[r]) : "r"(ra) : "memory");
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(a_l + 4u * g), "r"(r));
                    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(lr[r]) : "r"(ra) : "memory");
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(a_fin + 4u * i), "r"(r));
                    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(orr[r]) : "r"(ra) : "memory");
                }
            }
            float M = -INFINITY;
#pragma unroll
            for (int r = 0; r < 16; ++r) M = fmaxf(M, mr[r]);
            float Lsum = 0.f, o = 0.f;
#pragma unroll
            for (int r = 0; r < 16; ++r) {
                const float w = lr[r] > 0.f ? expf(mr[r] - M) : 0.f;
                Lsum = fmaf(lr[r], w, Lsum);
                o = fmaf(orr[r], w, o);
            }
            const float res = Lsum > 0.f ? o / Lsum : 0.f;
            if (p.outf != nullptr) p.outf[(size_t)(kvh * G) * D + i] = res;
            else p.out[(size_t)(kvh * G) * D + i] = __float2bfloat16_rn(res);
        }
        // nobody leaves while a neighbour may still read its shared memory
        asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
        return;
    }
    // ---- 4. publish the partial, merge if last -------------------------------------------------
    for (int i = tid; i < G * D; i += NT) {
        const int g = i / D, d = i - g * D;
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) o += sm.ored[w][g][d];
        p.part_o[((size_t)(kvh * G + g) * p.n_splits + split) * D + d] = o;
    }
    if (tid < G) {
        const int qh = kvh * G + tid;
        p.part_ml[((size_t)qh * p.n_splits + split) * 2] = sm.run_m[tid];
        p.part_ml[((size_t)qh * p.n_splits + split) * 2 + 1] = sm.run_l[tid];
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) sm.ticket = atomicAdd(&p.counters[kvh], 1u);
    __syncthreads();
    if (sm.ticket != (unsigned)(p.n_splits - 1)) return;
    __threadfence();
    // merge weights: warp g handles query head g, lanes over chunks
    for (int g = warp; g < G; g += NW) {
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
            sm.mw[g][s] = s < p.n_splits ? w[j] * inv : 0.f;     // zero past n_splits
        }
    }
    __syncthreads();
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
                o0 = fmaf(v[j], sm.mw[g][s0 + j], o0);
                o1 = fmaf(v[j + 1], sm.mw[g][s0 + j + 1], o1);
                o2 = fmaf(v[j + 2], sm.mw[g][s0 + j + 2], o2);
                o3 = fmaf(v[j + 3], sm.mw[g][s0 + j + 3], o3);
            }
        }
        const float res = (o0 + o1) + (o2 + o3);
        if (p.outf != nullptr) p.outf[(size_t)(kvh * G + g) * D + d] = res;
        else p.out[(size_t)(kvh * G + g) * D + d] = __float2bfloat16_rn(res);
    }
    if (tid == 0) p.counters[kvh] = 0u;
}

template <int D>
__global__ void __launch_bounds__(kAttnThreads) decode_attention_kernel(const DecodeAttnParams p) {
    extern __shared__ __align__(16) unsigned char attn_smem_raw[];
    pdl_launch_dependents();
    decode_attention_body<D, false, true>(p, blockIdx.x, blockIdx.y, attn_smem_raw);
}

// Cluster form: grid (cluster, kv_heads) with cluster dimension (cluster, 1, 1).
template <int D>
__global__ void __launch_bounds__(kAttnThreads) decode_attention_cluster_kernel(const DecodeAttnParams p) {
    extern __shared__ __align__(16) unsigned char attn_smem_raw[];
    pdl_launch_dependents();
    decode_attention_body<D, true, true>(p, blockIdx.x, blockIdx.y, attn_smem_raw);
}

inline size_t decode_attention_smem_bytes(int D, int /*chunk_cap*/) {
    return D == 128 ? sizeof(DecodeAttnSmem<128>) : sizeof(DecodeAttnSmem<64>);
}

}  // namespace efm
