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

constexpr int kMegaThreads = 512, kMegaWarps = 16, kMegaU = 8;
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
    __nv_bfloat16 *resid, *q, *attn, *act;
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

struct GemvRegs { uint4 wv[kMegaU][2]; };

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

// First batch of weight loads (+ the norm weight into shared memory) for a GEMV phase.  Touches
// weights only, so it may run before the barrier that publishes the phase's activations.
template <Epi EPI>
__device__ __forceinline__ void mega_gemv_prefetch(const GemvParams& p, const int ks, GemvRegs& r, unsigned char* smem,
                                                   const unsigned int xbytes) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int gp = kMegaWarps / ks, gi = warp / ks, wk = warp % ks;
    const int ig = blockIdx.x * gp + gi;
    const int nch = p.K >> 3;
    if (ig < p.n_items) {
        int r0, r1;
        item_rows<EPI>(p, ig, r0, r1);
        const __nv_bfloat16* a = p.W + (size_t)r0 * p.K;
        const __nv_bfloat16* b = p.W + (size_t)r1 * p.K;
        const int stride = ks * 32, gl = wk * 32 + lane;
#pragma unroll
        for (int u = 0; u < kMegaU; ++u) {
            const int c = u * stride + gl;
            if (c < nch) {
                r.wv[u][0] = ld_stream(a + (size_t)c * 8);
                r.wv[u][1] = ld_stream(b + (size_t)c * 8);
            }
        }
    }
    if (p.prologue != kProPlain) {
        uint4* gs = reinterpret_cast<uint4*>(smem + xbytes);
        for (int c = tid; c < nch; c += kMegaThreads) gs[c] = ld_cached(p.norm_w + (size_t)c * 8);
    }
}

// The phase itself: stage activations (with the fused norm), stream the rows, reduce, epilogue.
template <Epi EPI>
__device__ __forceinline__ void mega_gemv_run(const GemvParams& p, const int ks, GemvRegs& r, unsigned char* smem,
                                              const unsigned int xbytes, float& best_v, int& best_i) {
    __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem);
    const uint4* gs = reinterpret_cast<const uint4*>(smem + xbytes);
    float* red = reinterpret_cast<float*>(smem + 2 * xbytes);          // [2][16 warps][2]
    float* misc = red + 2 * kMegaWarps * 2;                             // [16]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int gp = kMegaWarps / ks, gi = warp / ks, wk = warp % ks;
    const int gl = wk * 32 + lane, stride = ks * 32;
    const int nch = p.K >> 3;

    // ---- activations -----------------------------------------------------------------------
    if (p.prologue == kProPlain) {
        for (int c = tid; c < nch; c += kMegaThreads) reinterpret_cast<uint4*>(xs)[c] = ld_cg(p.x + (size_t)c * 8);
    } else {
        const __nv_bfloat16* src = p.x;
        bool zero = false, from_table = false;
        if (p.prologue == kProEmbedRmsNorm) {
            const int tok = p.state->token;
            zero = tok < 0 || tok >= p.vocab;
            src = p.embed_table + (size_t)(zero ? 0 : tok) * p.K;
            from_table = true;
        }
        float ss = 0.f;
        for (int c = tid; c < nch; c += kMegaThreads) {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (!zero) v = from_table ? ld_cached(src + (size_t)c * 8) : ld_cg(src + (size_t)c * 8);
            float f[8];
            unpack8(v, f);
#pragma unroll
            for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
            reinterpret_cast<uint4*>(xs)[c] = v;
            if (from_table && blockIdx.x == 0) reinterpret_cast<uint4*>(p.resid_out)[c] = v;
        }
        ss = warp_sum(ss);
        if (lane == 0) misc[warp] = ss;
        __syncthreads();
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < kMegaWarps; ++w) tot += misc[w];
        const float inv = 1.0f / sqrtf(tot / (float)p.K + p.eps);
        for (int c = tid; c < nch; c += kMegaThreads) {       // same thread, same chunks as above
            float f[8], w[8];
            unpack8(reinterpret_cast<const uint4*>(xs)[c], f);
            unpack8(gs[c], w);
            uint4 o;
            o.x = pack_bf16(f[0] * inv * w[0], f[1] * inv * w[1]);
            o.y = pack_bf16(f[2] * inv * w[2], f[3] * inv * w[3]);
            o.z = pack_bf16(f[4] * inv * w[4], f[5] * inv * w[5]);
            o.w = pack_bf16(f[6] * inv * w[6], f[7] * inv * w[7]);
            reinterpret_cast<uint4*>(xs)[c] = o;
        }
    }
    __syncthreads();

    // ---- rows -------------------------------------------------------------------------------
    const int ig_stride = gridDim.x * gp;
    bool first = true;
    int parity = 0;
    uint32_t old_first = 0u;          // residual pair of the first item, fetched under the weight stream
    if constexpr (EPI == Epi::Residual) {
        const int ig0 = blockIdx.x * gp + gi;
        if (wk == 0 && lane == 0 && ig0 < p.n_items)
            old_first = __ldcg(reinterpret_cast<const unsigned int*>(p.residual + ig0 * 2));
    }
    for (int ig = blockIdx.x * gp + gi; ig < p.n_items; ig += ig_stride) {
        int r0, r1;
        item_rows<EPI>(p, ig, r0, r1);
        const __nv_bfloat16* a = p.W + (size_t)r0 * p.K;
        const __nv_bfloat16* b = p.W + (size_t)r1 * p.K;
        float acc0 = 0.f, acc1 = 0.f;
        for (int cb = 0; cb < nch; cb += kMegaU * stride) {
            if (!(first && cb == 0)) {
#pragma unroll
                for (int u = 0; u < kMegaU; ++u) {
                    const int c = cb + u * stride + gl;
                    if (c < nch) {
                        r.wv[u][0] = ld_stream(a + (size_t)c * 8);
                        r.wv[u][1] = ld_stream(b + (size_t)c * 8);
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < kMegaU; ++u) {
                const int c = cb + u * stride + gl;
                if (c < nch) {
                    float xf[8];
                    unpack8(reinterpret_cast<const uint4*>(xs)[c], xf);
                    acc0 = dot8(r.wv[u][0], xf, acc0);
                    acc1 = dot8(r.wv[u][1], xf, acc1);
                }
            }
        }
        const bool was_first = first;
        first = false;
        acc0 = warp_sum(acc0);
        acc1 = warp_sum(acc1);
        if (ks > 1) {
            float* buf = red + parity * kMegaWarps * 2;
            if (lane == 0) { buf[warp * 2] = acc0; buf[warp * 2 + 1] = acc1; }
            group_barrier(1 + gi, ks * 32);
            if (wk == 0) {
                float t0 = 0.f, t1 = 0.f;
                for (int w = 0; w < ks; ++w) { t0 += buf[(gi * ks + w) * 2]; t1 += buf[(gi * ks + w) * 2 + 1]; }
                acc0 = t0;
                acc1 = t1;
            }
            parity ^= 1;
        }
        if (wk == 0 && lane == 0) {
            if constexpr (EPI == Epi::Residual) {
                const uint32_t old = was_first ? old_first : __ldcg(reinterpret_cast<const unsigned int*>(p.residual + ig * 2));
                *reinterpret_cast<uint32_t*>(p.residual + ig * 2) =
                    pack_bf16(bf16lo(old) + round_bf16(acc0), bf16hi(old) + round_bf16(acc1));
            } else {
                item_epilogue<EPI>(p, ig, acc0, acc1, best_v, best_i);
            }
        }
    }
}

template <int D>
__device__ __forceinline__ void mega_attention(const MegaParams& P, const MegaLayer& W, int cta, unsigned char* a_smem) {
    DecodeAttnParams a{};
    a.q = P.q; a.k_cache = W.k_cache; a.v_cache = W.v_cache; a.out = P.attn; a.state = P.state;
    a.q_heads = P.q_heads; a.kv_heads = P.kv_heads; a.group = P.q_heads / P.kv_heads;
    a.n_splits = P.n_splits; a.chunk_cap = P.chunk_cap; a.max_tokens = P.max_tokens; a.scale = P.scale;
    a.part_o = P.part_o; a.part_ml = P.part_ml; a.counters = P.attn_counters;
    decode_attention_body<D, true>(a, cta % P.n_splits, cta / P.n_splits, a_smem);
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
        g.x = P.resid; g.norm_w = W.in_norm; g.eps = P.eps;
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

    {
        const GemvParams g = qkv_params(0);
        mega_gemv_prefetch<Epi::QkvRope>(g, P.ks_qkv, regs, mega_smem, xbytes);
    }
    const bool attn_role = cta < P.n_splits * P.kv_heads && tid < 256;
    bool alive = true;
    for (int l = 0; l < P.L && alive; ++l) {
        const MegaLayer& W = P.layers[l];
        // 1. norm + QKV + RoPE + cache append
        {
            const GemvParams g = qkv_params(l);
            mega_gemv_run<Epi::QkvRope>(g, P.ks_qkv, regs, mega_smem, xbytes, best_v, best_i);
        }
        const GemvParams go = plain_params(W.o, P.H, P.QD, P.attn);
        mega_barrier_arrive(bar);
        if (!attn_role) mega_gemv_prefetch<Epi::Residual>(go, P.ks_o, regs, mega_smem, xbytes);
        if (!(alive = mega_barrier_wait(bar, ++phase * nblk, P.abort_flag, &s_abort))) break;
        stamp(phase);
        // 2. attention (first n_splits * kv_heads blocks, 256 threads each)
        if (attn_role) mega_attention<D>(P, W, cta, a_smem);
        mega_barrier_arrive(bar);
        if (attn_role) mega_gemv_prefetch<Epi::Residual>(go, P.ks_o, regs, mega_smem, xbytes);
        if (!(alive = mega_barrier_wait(bar, ++phase * nblk, P.abort_flag, &s_abort))) break;
        stamp(phase);
        // 3. o_proj + residual
        mega_gemv_run<Epi::Residual>(go, P.ks_o, regs, mega_smem, xbytes, best_v, best_i);
        GemvParams gg{};
        gg.W = W.gate_up; gg.N = 2 * P.I; gg.K = P.H; gg.n_items = P.I; gg.prologue = kProRmsNorm;
        gg.x = P.resid; gg.norm_w = W.post_norm; gg.eps = P.eps; gg.y = P.act;
        mega_barrier_arrive(bar);
        mega_gemv_prefetch<Epi::SwiGlu>(gg, P.ks_gu, regs, mega_smem, xbytes);
        if (!(alive = mega_barrier_wait(bar, ++phase * nblk, P.abort_flag, &s_abort))) break;
        stamp(phase);
        // 4. norm + gate/up + SiLU*mul
        mega_gemv_run<Epi::SwiGlu>(gg, P.ks_gu, regs, mega_smem, xbytes, best_v, best_i);
        const GemvParams gd = plain_params(W.down, P.H, P.I, P.act);
        mega_barrier_arrive(bar);
        mega_gemv_prefetch<Epi::Residual>(gd, P.ks_down, regs, mega_smem, xbytes);
        if (!(alive = mega_barrier_wait(bar, ++phase * nblk, P.abort_flag, &s_abort))) break;
        stamp(phase);
        // 5. down_proj + residual, then the next layer's (or the lm_head's) first weights
        mega_gemv_run<Epi::Residual>(gd, P.ks_down, regs, mega_smem, xbytes, best_v, best_i);
        mega_barrier_arrive(bar);
        if (l + 1 < P.L) {
            const GemvParams g = qkv_params(l + 1);
            mega_gemv_prefetch<Epi::QkvRope>(g, P.ks_qkv, regs, mega_smem, xbytes);
        } else {
            GemvParams g{};
            g.W = P.lm_head; g.N = P.V; g.K = P.H; g.n_items = P.V / 2; g.prologue = kProRmsNorm;
            g.x = P.resid; g.norm_w = P.final_norm; g.eps = P.eps;
            mega_gemv_prefetch<Epi::Logits>(g, P.ks_lm, regs, mega_smem, xbytes);
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
        g.x = P.resid; g.norm_w = P.final_norm; g.eps = P.eps;
        g.logits = P.logits;
        mega_gemv_run<Epi::Logits>(g, P.ks_lm, regs, mega_smem, xbytes, best_v, best_i);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best_v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best_v || (ov == best_v && oi < best_i)) { best_v = ov; best_i = oi; }
    }
    if (lane == 0) { bv[warp] = best_v; bi[warp] = best_i; }
    __syncthreads();
    if (tid == 0) {
        float v = bv[0];
        int i = bi[0];
        for (int w = 1; w < kMegaWarps; ++w)
            if (bv[w] > v || (bv[w] == v && bi[w] < i)) { v = bv[w]; i = bi[w]; }
        P.part_val[cta] = v;
        P.part_idx[cta] = i;
    }
    stamp(phase + 1);
}

inline size_t mega_gemv_smem_bytes(int H, int QD, int I) {
    const size_t k = (size_t)std::max(H, std::max(QD, I));
    return 2 * ((k * 2 + 15) & ~(size_t)15) + (size_t)(2 * kMegaWarps * 2 + 16) * sizeof(float);
}

}  // namespace efm
