// Persistent decode kernel: every layer of one decode step in ONE cooperative launch.
//
// Why: at batch 1 a decode step is a chain of 5 dependent phases per layer (norm+QKV+RoPE+append |
// attention | o_proj+residual | norm+gate/up+SiLU | down+residual).  As separate launches each link
// costs 3.5-5 us of launch / drain / first-load latency on B200 while the weights of a 1.5B model
// stream in ~3.4 us per layer, so the step ends up latency-bound.  Here one block per SM stays
// resident, phases are separated by a grid barrier (atomic arrive + acquire poll, ~1 us), and —
// the point of the design — every warp issues the first batch of the NEXT phase's weight loads
// (16 x 128 bit per lane, ~19 MB chip-wide) before it arrives at the barrier, so HBM keeps
// streaming while the barrier and the activation exchange through L2 are in flight.
//
// Cross-block data (residual stream, q, attention output, SiLU activations, newest cache row,
// split partials) is always read with L2-only loads after a barrier.  Blocks wait on each other, so
// the kernel is launched cooperatively (all blocks co-resident); every wait is bounded: a block
// that gives up raises a global abort flag, all blocks return, and the host reads the status word.
#pragma once
#include "decode_attention.cuh"
#include "gemv.cuh"

namespace efm {

constexpr int kMegaThreads = kGemvThreads, kMegaWarps = kGemvWarps;
constexpr long kMegaSpinLimit = 4L << 20;          // polls of ~0.3-0.5 us: gives up after ~1-2 s

struct MegaLayer {
    const __nv_bfloat16 *in_norm, *post_norm, *qkv, *qkv_bias, *o, *gate_up, *down;
    __nv_bfloat16 *k_cache, *v_cache;
};

struct MegaParams {
    const MegaLayer* layers;           // device array [L]
    int L, H, QD, KVD, I, V, q_heads, kv_heads, vocab;
    float eps;
    int ks_qkv, ks_o, ks_gu, ks_down, ks_lm;     // warps sharing one row pair, per phase
    const __nv_bfloat16 *embed, *final_norm, *lm_head;
    float* resid;                      // residual stream [H] fp32
    __nv_bfloat16 *q, *attn, *act;
    float* logits;
    float* part_val;
    int* part_idx;
    DecodeState* state;
    const float* inv_freq;
    int use_mrope, sec0, sec1, max_tokens;
    int n_splits, chunk_cap;                     // attention work split
    float scale;
    float* part_o;
    float* part_ml;
    unsigned int* attn_counters;
    unsigned int* barrier;                       // [2] alternating by step parity
    int* abort_flag;
    unsigned int gemv_smem_bytes;                // staging area size; attention scratch follows it
    unsigned long long* timing;                  // optional [5L + 2] %globaltimer stamps of block 0 (null: off)
};

// Grid barrier in two halves so that the next phase's weight prefetch sits between them: the
// arrive half publishes this block's writes (its fence must not have to wait for prefetch loads),
// the wait half polls with back-off.  wait returns false when the wait was abandoned.
__device__ __forceinline__ void mega_barrier_arrive(unsigned int* counter) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(counter, 1u);
    }
}
__device__ __forceinline__ bool mega_barrier_wait(unsigned int* counter, unsigned int target, int* abort_flag,
                                                  volatile int* s_abort) {
    if (threadIdx.x == 0) {
        int ok = 1;
        long spins = 0;
        for (;;) {
            unsigned int v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
            if (v >= target) break;
            ++spins;
            if ((spins & 0x3ff) == 0 && *reinterpret_cast<volatile int*>(abort_flag) != 0) { ok = 0; break; }
            if (spins > kMegaSpinLimit) { atomicExch(abort_flag, 1); ok = 0; break; }
            __nanosleep(spins < 64 ? 40 : 400);
        }
        *s_abort = ok ? 0 : 1;
    }
    __syncthreads();
    return *s_abort == 0;
}

template <int D>
__device__ __forceinline__ void mega_attention(const MegaParams& P, const MegaLayer& W, int cta, unsigned char* a_smem) {
    DecodeAttnParams a{};
    a.q = P.q; a.k_cache = W.k_cache; a.v_cache = W.v_cache; a.out = P.attn; a.state = P.state;
    a.q_heads = P.q_heads; a.kv_heads = P.kv_heads; a.group = P.q_heads / P.kv_heads;
    a.n_splits = P.n_splits; a.chunk_cap = P.chunk_cap; a.max_tokens = P.max_tokens; a.scale = P.scale;
    a.part_o = P.part_o; a.part_ml = P.part_ml; a.counters = P.attn_counters;
    decode_attention_body<D>(a, cta % P.n_splits, cta / P.n_splits, a_smem);
}

template <int D>
__global__ void __launch_bounds__(kMegaThreads, 1) decode_mega_kernel(const MegaParams P) {
    extern __shared__ __align__(16) unsigned char mega_smem[];
    __shared__ int s_abort;
    __shared__ float bv[kMegaWarps];
    __shared__ int bi[kMegaWarps];
    unsigned char* a_smem = mega_smem + P.gemv_smem_bytes;
    const int cta = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const unsigned int nblk = gridDim.x;
    const unsigned int xbytes = ((unsigned int)(P.I > P.H ? (P.I > P.QD ? P.I : P.QD) : (P.H > P.QD ? P.H : P.QD)) * 2 + 15) & ~15u;

    const int step = P.state->step;
    unsigned int* bar = P.barrier + (step & 1);
    if (cta == 0 && tid == 0) P.barrier[(step + 1) & 1] = 0u;     // the other counter is idle during this launch
    unsigned int phase = 0;
    auto stamp = [&](unsigned int idx) {
        if (P.timing != nullptr && cta == 0 && tid == 0) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
            P.timing[idx] = t;
        }
    };
    stamp(0);
    GemvRegs regs;
    float best_v = -INFINITY;
    int best_i = 0x7fffffff;

    auto qkv_params = [&](int l) {
        const MegaLayer& W = P.layers[l];
        GemvParams g{};
        g.W = W.qkv; g.N = P.QD + 2 * P.KVD; g.K = P.H; g.n_items = g.N / 2;
        g.prologue = l == 0 ? kProEmbedRmsNorm : kProRmsNorm;
        g.xr = P.resid; g.norm_w = W.in_norm; g.eps = P.eps;
        g.embed_table = P.embed; g.vocab = P.vocab; g.resid_out = P.resid; g.state = P.state;
        g.bias = W.qkv_bias; g.q_out = P.q; g.k_cache = W.k_cache; g.v_cache = W.v_cache;
        g.inv_freq = P.inv_freq; g.q_heads = P.q_heads; g.kv_heads = P.kv_heads; g.head_dim = D;
        g.use_mrope = P.use_mrope; g.sec0 = P.sec0; g.sec1 = P.sec1; g.max_tokens = P.max_tokens;
        return g;
    };
    auto plain_params = [&](const __nv_bfloat16* W, int N, int K, const __nv_bfloat16* x) {
        GemvParams g{};
        g.W = W; g.N = N; g.K = K; g.n_items = N / 2; g.prologue = kProPlain; g.x = x; g.residual = P.resid;
        return g;
    };

    GemvSched sc;
    {
        const GemvParams g = qkv_params(0);
        sc = gemv_sched(g, P.ks_qkv, cta, nblk);
        gemv_prefetch<Epi::QkvRope>(g, sc, regs, mega_smem, xbytes);
    }
    const bool attn_role = cta < P.n_splits * P.kv_heads;      // whole blocks: all 512 threads work on attention
    bool alive = true;
    for (int l = 0; l < P.L && alive; ++l) {
        const MegaLayer& W = P.layers[l];
        // 1. norm + QKV + RoPE + cache append
        {
            const GemvParams g = qkv_params(l);
            gemv_run<Epi::QkvRope>(g, sc, regs, mega_smem, xbytes, best_v, best_i);
        }
        const GemvParams go = plain_params(W.o, P.H, P.QD, P.attn);
        mega_barrier_arrive(bar);
        sc = gemv_sched(go, P.ks_o, cta, nblk);
        if (!attn_role) gemv_prefetch<Epi::Residual>(go, sc, regs, mega_smem, xbytes);
        if (!(alive = mega_barrier_wait(bar, ++phase * nblk, P.abort_flag, &s_abort))) break;
        stamp(phase);
        // 2. attention (the first n_splits * kv_heads blocks)
        if (attn_role) mega_attention<D>(P, W, cta, a_smem);
        mega_barrier_arrive(bar);
        if (attn_role) gemv_prefetch<Epi::Residual>(go, sc, regs, mega_smem, xbytes);
        if (!(alive = mega_barrier_wait(bar, ++phase * nblk, P.abort_flag, &s_abort))) break;
        stamp(phase);
        // 3. o_proj + residual
        gemv_run<Epi::Residual>(go, sc, regs, mega_smem, xbytes, best_v, best_i);
        GemvParams gg{};
        gg.W = W.gate_up; gg.N = 2 * P.I; gg.K = P.H; gg.n_items = P.I; gg.prologue = kProRmsNorm;
        gg.xr = P.resid; gg.norm_w = W.post_norm; gg.eps = P.eps; gg.y = P.act;
        mega_barrier_arrive(bar);
        sc = gemv_sched(gg, P.ks_gu, cta, nblk);
        gemv_prefetch<Epi::SwiGlu>(gg, sc, regs, mega_smem, xbytes);
        if (!(alive = mega_barrier_wait(bar, ++phase * nblk, P.abort_flag, &s_abort))) break;
        stamp(phase);
        // 4. norm + gate/up + SiLU*mul
        gemv_run<Epi::SwiGlu>(gg, sc, regs, mega_smem, xbytes, best_v, best_i);
        const GemvParams gd = plain_params(W.down, P.H, P.I, P.act);
        mega_barrier_arrive(bar);
        sc = gemv_sched(gd, P.ks_down, cta, nblk);
        gemv_prefetch<Epi::Residual>(gd, sc, regs, mega_smem, xbytes);
        if (!(alive = mega_barrier_wait(bar, ++phase * nblk, P.abort_flag, &s_abort))) break;
        stamp(phase);
        // 5. down_proj + residual, then the next layer's (or the lm_head's) first weights
        gemv_run<Epi::Residual>(gd, sc, regs, mega_smem, xbytes, best_v, best_i);
        mega_barrier_arrive(bar);
        if (l + 1 < P.L) {
            const GemvParams g = qkv_params(l + 1);
            sc = gemv_sched(g, P.ks_qkv, cta, nblk);
            gemv_prefetch<Epi::QkvRope>(g, sc, regs, mega_smem, xbytes);
        } else {
            GemvParams g{};
            g.W = P.lm_head; g.N = P.V; g.K = P.H; g.n_items = P.V / 2; g.prologue = kProRmsNorm;
            g.xr = P.resid; g.norm_w = P.final_norm; g.eps = P.eps;
            sc = gemv_sched(g, P.ks_lm, cta, nblk);
            gemv_prefetch<Epi::Logits>(g, sc, regs, mega_smem, xbytes);
        }
        if (!(alive = mega_barrier_wait(bar, ++phase * nblk, P.abort_flag, &s_abort))) break;
        stamp(phase);
    }
    if (!alive) {                             // a wait was abandoned somewhere in the grid
        if (tid == 0) P.state->error = 3;
        return;
    }
    // final norm + lm_head + per-block argmax
    {
        GemvParams g{};
        g.W = P.lm_head; g.N = P.V; g.K = P.H; g.n_items = P.V / 2; g.prologue = kProRmsNorm;
        g.xr = P.resid; g.norm_w = P.final_norm; g.eps = P.eps;
        g.logits = P.logits; g.part_val = P.part_val; g.part_idx = P.part_idx;
        gemv_run<Epi::Logits>(g, sc, regs, mega_smem, xbytes, best_v, best_i);
        gemv_publish_best(g, best_v, best_i, bv, bi);
    }
    stamp(phase + 1);
}

inline size_t mega_gemv_smem_bytes(int H, int QD, int I) { return gemv_smem_bytes(std::max(H, std::max(QD, I))); }

}  // namespace efm
