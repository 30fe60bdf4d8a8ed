// Batch-1 weight-streaming GEMV for the decode step, with the neighbouring element-wise work
// fused in so that one launch replaces a chain of the reference's kernels:
//
//   prologue  Plain            x is read as is                      (o_proj, down_proj)
//             RmsNorm          x = rmsnorm(residual) * w, residual stream and x in fp32
//                                                                   (K2/K3 + K4 of the reference:
//                                                                    src/operators/norm_op.cu:20-106)
//             EmbedRmsNorm     residual = embed_table[token] first  (src/layers/embed_head.cu:22-61)
//   epilogue  Plain            y = bf16(W x)
//             Residual         r += W x, r kept in fp32             (fused add of norm_op.cu:64-106; the
//                              reference stores r in bf16, which costs ~2x in logit error on deep stacks)
//             QkvRope          + bias, rotate-half RoPE / M-RoPE on q and k, append k, v to the
//                              cache row kv_len-1                    (linear_impl.cu:90-106,
//                              decode_runtime_kernels.cu:67-225)
//             SwiGlu           act = bf16(silu(gate) * up)          (fused_gate_up_activation_op.cu:198-277)
//             Logits           fp32 logits + per-block (max, argmax) (src/layers/linear.cu:187-270)
//
// Bound: HBM.  One block of 16 warps per SM.  Each weight byte is read once, as 128-bit streaming
// loads.  A warp (or `ks` warps sharing one row pair) walks its rows in units of 8 x 2 loads: 16
// loads of 16 bytes in flight per lane, ~19 MB chip-wide, which is what it takes to cover the
// ~2 us loaded DRAM latency at full bandwidth (halving it to 8 measurably costs 20 %).  Activations
// live in shared memory as fp32 (a decode step rounds nothing to bf16 but the K / V rows it appends: with bf16
// activations the rounding noise of 28-36 layers alone exceeds a 2e-2 logit tolerance on the 3B / 7B shapes);
// dot products reduce with warp shuffles (and a named-barrier exchange
// when ks > 1).  The first unit and the norm weight are fetched BEFORE the dependency wait
// (griddepcontrol.wait, or the grid barrier of the persistent decode kernel), because weights
// do not depend on the previous phase.
#pragma once
#include "common.cuh"

namespace efm {

enum class Epi : int { Plain = 0, Residual = 1, QkvRope = 2, SwiGlu = 3, Logits = 4, Peers = 5 };
constexpr int kMaxPeers = 8;
enum : int { kProPlain = 0, kProRmsNorm = 1, kProEmbedRmsNorm = 2 };

struct GemvParams {
    const __nv_bfloat16* W;   // [N, K] row-major
    int N, K, n_items;        // n_items = N / 2 (every epilogue consumes rows in pairs)
    // prologue
    int prologue;
    const __nv_bfloat16* x;   // Plain: activations [K] bf16 ...
    const float* xf;          // ... or, when non-null, fp32 (the decode step's own activations)
    const float* xr;          // norm prologues: residual stream [K] fp32
    const __nv_bfloat16* norm_w;
    float eps;
    const __nv_bfloat16* embed_table;
    int vocab;
    float* resid_out;         // EmbedRmsNorm / addend: block 0 stores the (updated) residual row here
    const float* addend;      // norm prologues, tensor parallel: x = x + addend first (summed partial output of
                              // the previous row-parallel linear); resid_out must differ from xr
    DecodeState* state;
    // epilogue
    __nv_bfloat16* y;         // Plain: [N]; SwiGlu: [N/2] ...
    float* yf;                // ... or, when non-null, SwiGlu output in fp32
    float* residual;          // Residual: [N] fp32 in/out
    const __nv_bfloat16* bias;
    __nv_bfloat16* q_out;     // QkvRope: rotated q in bf16 (q, k, v rounded to bf16 before the rotation as the prefill does) ...
    float* q_out_f;           // ... or, when non-null, in fp32: then nothing is rounded but the K / V rows written to the cache
    __nv_bfloat16* k_cache;
    __nv_bfloat16* v_cache;
    const float* inv_freq;
    int q_heads, kv_heads, head_dim, use_mrope, sec0, sec1, max_tokens;
    float* logits;            // Logits
    float* part_val;
    int* part_idx;
    // Peers (tensor parallel, row-parallel linear fused with its exchange): every output value travels as one
    // 8-byte word {fp32 value, exchange count} stored into this rank's row of EVERY rank's receive buffer (peer
    // memory over NVLink, own buffer included).  Value and count arrive together, so there is no fence and no
    // separate flag; the last block to finish bumps the local count (local atomics only).
    uint2* peer_out[kMaxPeers];
    int n_peers;
    unsigned int* epoch;      // local: number of exchanges completed by this rank
    unsigned int* ticket;     // local: block ticket, zero between launches
    // consumer side (norm prologues): x = x + sum over ranks, in rank order, of parts[r][:], every word being
    // re-read (bounded) until it carries the local count
    const uint2* addend_parts;            // local receive buffer [n_parts][K] of {value, count}
    int n_parts;
    int* error;               // raised (3) when a wait gives up
    volatile int* error_host; // optional mirror of `error` in mapped host memory (the host stops queueing steps)
    unsigned long long wait_ns;   // total wait budget of one kernel; 0 = kPeerWaitDefaultNs
    unsigned int want_override;   // != 0: wait for this count instead of *epoch (single-GPU test of the wait)
};

// One {value, count} word is ONE 64-bit element (value in the low half), so that value and count are read and
// written together by the memory model's own rule (a 64-bit access is single-copy atomic), not by the accident
// of how a 16-byte store travels.  Two words per access; relaxed, system scope: the consumer needs no ordering
// between words, only each word whole.
__device__ __forceinline__ void ld_peer_words(const uint2* p, unsigned long long& w0, unsigned long long& w1) {
    asm volatile("ld.relaxed.sys.global.v2.b64 {%0,%1}, [%2];" : "=l"(w0), "=l"(w1) : "l"(p) : "memory");
}
__device__ __forceinline__ void st_peer_words(uint2* p, unsigned long long w0, unsigned long long w1) {
    asm volatile("st.relaxed.sys.global.v2.b64 [%0], {%1,%2};" ::"l"(p), "l"(w0), "l"(w1) : "memory");
}
__device__ __forceinline__ unsigned long long peer_word(float v, unsigned int count) {
    return (unsigned long long)__float_as_uint(v) | ((unsigned long long)count << 32);
}
__device__ __forceinline__ void group_barrier(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

template <Epi EPI>
__device__ __forceinline__ void item_rows(const GemvParams& p, int item, int& r0, int& r1) {
    if constexpr (EPI == Epi::QkvRope) {
        const int half = p.head_dim >> 1;
        const int head = item / half, d = item - head * half;
        r0 = head * p.head_dim + d;
        r1 = r0 + half;
    } else if constexpr (EPI == Epi::SwiGlu) {
        // fused weight: blocks of 64 gate rows followed by the 64 matching up rows
        r0 = ((item >> 6) << 7) + (item & 63);
        r1 = r0 + 64;
    } else {
        r0 = item * 2;
        r1 = r0 + 1;
    }
}

template <Epi EPI>
__device__ __forceinline__ void item_epilogue(const GemvParams& p, int item, float a0, float a1,
                                              float& best_v, int& best_i) {
    if constexpr (EPI == Epi::Plain) {
        p.y[item * 2] = __float2bfloat16_rn(a0);
        p.y[item * 2 + 1] = __float2bfloat16_rn(a1);
    } else if constexpr (EPI == Epi::Residual) {
        // L2 load: inside the persistent decode kernel another block wrote this value
        const float2 old = __ldcg(reinterpret_cast<const float2*>(p.residual + item * 2));
        *reinterpret_cast<float2*>(p.residual + item * 2) = make_float2(old.x + a0, old.y + a1);
    } else if constexpr (EPI == Epi::SwiGlu) {
        const float s = a0 / (1.0f + expf(-a0));
        if (p.yf != nullptr) p.yf[item] = s * a1;
        else p.y[item] = __float2bfloat16_rn(s * a1);
    } else if constexpr (EPI == Epi::Peers) {
        const unsigned int e = (unsigned int)best_i;           // exchange count of this launch (see gemv_kernel)
        const unsigned long long w0 = peer_word(a0, e), w1 = peer_word(a1, e);
#pragma unroll
        for (int r = 0; r < kMaxPeers; ++r)
            if (r < p.n_peers) st_peer_words(p.peer_out[r] + item * 2, w0, w1);
    } else if constexpr (EPI == Epi::Logits) {
        *reinterpret_cast<float2*>(p.logits + item * 2) = make_float2(a0, a1);
        if (a0 > best_v) { best_v = a0; best_i = item * 2; }          // ascending ids: strict > keeps
        if (a1 > best_v) { best_v = a1; best_i = item * 2 + 1; }      // the lowest id on ties
    } else {  // QkvRope
        const int D = p.head_dim, half = D >> 1;
        const int head = item / half, d = item - head * half;
        int r0 = head * D + d, r1 = r0 + half;
        float y0 = a0, y1 = a1;
        if (p.bias != nullptr) {
            y0 += __bfloat162float(p.bias[r0]);
            y1 += __bfloat162float(p.bias[r1]);
        }
        const bool full = p.q_out_f != nullptr;
        if (!full) {
            y0 = round_bf16(y0);
            y1 = round_bf16(y1);
        }
        const uint32_t kv_len = p.state->kv_len;
        if (kv_len == 0 || kv_len > (uint32_t)p.max_tokens) {
            p.state->error = 1;   // refuse the out-of-range cache row instead of faulting
            return;
        }
        const size_t row = (size_t)(kv_len - 1) * p.kv_heads * D;
        if (head < p.q_heads + p.kv_heads) {
            int pos;
            if (p.use_mrope) pos = p.state->pos[d < p.sec0 ? 0 : (d < p.sec1 ? 1 : 2)];
            else pos = (int)kv_len - 1;
            float sn, cs;
            sincosf((float)pos * p.inv_freq[d], &sn, &cs);
            const float o0 = y0 * cs - y1 * sn, o1 = y1 * cs + y0 * sn;
            if (head < p.q_heads) {
                if (full) {
                    p.q_out_f[r0] = o0;
                    p.q_out_f[r1] = o1;
                } else {
                    p.q_out[r0] = __float2bfloat16_rn(o0);
                    p.q_out[r1] = __float2bfloat16_rn(o1);
                }
            } else {
                const int kh = head - p.q_heads;
                p.k_cache[row + kh * D + d] = __float2bfloat16_rn(o0);
                p.k_cache[row + kh * D + d + half] = __float2bfloat16_rn(o1);
            }
        } else {
            const int vh = head - p.q_heads - p.kv_heads;
            p.v_cache[row + vh * D + d] = __float2bfloat16_rn(y0);
            p.v_cache[row + vh * D + d + half] = __float2bfloat16_rn(y1);
        }
    }
}

constexpr int kGemvThreads = 512, kGemvWarps = 16, kGemvU = 8;

struct GemvRegs { uint4 a[kGemvU][2]; };

// Per-thread view of the static schedule: which row pairs (items) this warp group walks and in
// how many units.
struct GemvSched {
    int ks, gi, wk, gl, stride, nch, upi, ig0, ig_stride, total;
};

__device__ __forceinline__ GemvSched gemv_sched(const GemvParams& p, const int ks, const int block, const int n_blocks) {
    GemvSched sc;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gp = kGemvWarps / ks;
    sc.ks = ks;
    sc.gi = warp / ks;
    sc.wk = warp % ks;
    sc.gl = sc.wk * 32 + lane;
    sc.stride = ks * 32;
    sc.nch = p.K >> 3;
    const int cpl = (sc.nch + sc.stride - 1) / sc.stride;        // chunks per lane and row
    sc.upi = (cpl + kGemvU - 1) / kGemvU;                         // units per item
    sc.ig0 = block * gp + sc.gi;
    sc.ig_stride = n_blocks * gp;
    const int n_my = sc.ig0 < p.n_items ? (p.n_items - sc.ig0 + sc.ig_stride - 1) / sc.ig_stride : 0;
    sc.total = n_my * sc.upi;
    return sc;
}

template <Epi EPI>
__device__ __forceinline__ void gemv_load_unit(const GemvParams& p, const GemvSched& sc, const int u, uint4 (&buf)[kGemvU][2]) {
    if (u >= sc.total) return;
    const int j = u / sc.upi, part = u - j * sc.upi;
    int r0, r1;
    item_rows<EPI>(p, sc.ig0 + j * sc.ig_stride, r0, r1);
    const __nv_bfloat16* a = p.W + (size_t)r0 * p.K;
    const __nv_bfloat16* b = p.W + (size_t)r1 * p.K;
#pragma unroll
    for (int uu = 0; uu < kGemvU; ++uu) {
        const int c = (part * kGemvU + uu) * sc.stride + sc.gl;
        if (c < sc.nch) {
            buf[uu][0] = ld_stream(a + (size_t)c * 8);
            buf[uu][1] = ld_stream(b + (size_t)c * 8);
        }
    }
}

// Shared memory of one GEMV phase: [xs: fp32 K][norm weight: bf16 K][red: 2 x 16 x 2 floats][misc: 16 floats].
__host__ __device__ inline unsigned int gemv_xbytes(int K) { return ((unsigned int)K * 4u + 15u) & ~15u; }
__host__ __device__ inline unsigned int gemv_wbytes(int K) { return ((unsigned int)K * 2u + 15u) & ~15u; }

// Weights only: the first two units into registers, the norm weight into shared memory.
template <Epi EPI>
__device__ __forceinline__ void gemv_prefetch(const GemvParams& p, const GemvSched& sc, GemvRegs& r, unsigned char* smem,
                                              const unsigned int xbytes) {
    gemv_load_unit<EPI>(p, sc, 0, r.a);
    if (p.prologue != kProPlain) {
        uint4* gs = reinterpret_cast<uint4*>(smem + xbytes);        // xbytes = gemv_xbytes(K)
        for (int c = threadIdx.x; c < sc.nch; c += kGemvThreads) gs[c] = ld_cached(p.norm_w + (size_t)c * 8);
    }
}

// Activations of one GEMV phase into shared memory as fp32 [K], with the fused prologue (embedding row / residual
// stream + tensor-parallel partials -> RMSNorm).  Ends with a block barrier.  xbytes = gemv_xbytes(K).
__device__ __forceinline__ void gemv_stage(const GemvParams& p, const int nch, unsigned char* smem, const unsigned int xbytes) {
    float* xs = reinterpret_cast<float*>(smem);
    const uint4* gs = reinterpret_cast<const uint4*>(smem + xbytes);
    float* red = reinterpret_cast<float*>(smem + xbytes + gemv_wbytes(p.K));
    float* misc = red + 2 * kGemvWarps * 2;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // ---- activations (L2 loads: another block may have produced them) ------------------------
    if (p.prologue == kProPlain) {
        if (p.xf != nullptr) {
            for (int c = tid; c < 2 * nch; c += kGemvThreads)
                reinterpret_cast<float4*>(xs)[c] = __ldcg(reinterpret_cast<const float4*>(p.xf) + c);
        } else {
            for (int c = tid; c < nch; c += kGemvThreads) {
                float f[8];
                unpack8(ld_cg(p.x + (size_t)c * 8), f);
                reinterpret_cast<float4*>(xs)[2 * c] = make_float4(f[0], f[1], f[2], f[3]);
                reinterpret_cast<float4*>(xs)[2 * c + 1] = make_float4(f[4], f[5], f[6], f[7]);
            }
        }
    } else {
        // residual stream in fp32 (or the embedding row); staged unscaled until the norm is known
        const __nv_bfloat16* table_row = nullptr;
        bool zero = false, from_table = false;
        if (p.prologue == kProEmbedRmsNorm) {
            const int tok = p.state->token;
            zero = tok < 0 || tok >= p.vocab;
            table_row = p.embed_table + (size_t)(zero ? 0 : tok) * p.K;
            from_table = true;
        }
        float* xf32 = xs;                                          // normalised in place below
        // count to wait for: bumped by this GPU's producing kernel
        const unsigned int want = p.addend_parts == nullptr ? 0u : (p.want_override != 0u ? p.want_override : __ldcg(p.epoch));
        PeerWait pw = peer_wait_begin(p.addend_parts != nullptr ? p.error : nullptr);
        float ss = 0.f;
        for (int c = tid; c < nch; c += kGemvThreads) {
            float f[8];
            if (from_table) {
                unpack8(zero ? make_uint4(0, 0, 0, 0) : ld_cached(table_row + (size_t)c * 8), f);
            } else {
                const float4 lo = __ldcg(reinterpret_cast<const float4*>(p.xr + (size_t)c * 8));
                const float4 hi = __ldcg(reinterpret_cast<const float4*>(p.xr + (size_t)c * 8 + 4));
                f[0] = lo.x; f[1] = lo.y; f[2] = lo.z; f[3] = lo.w; f[4] = hi.x; f[5] = hi.y; f[6] = hi.z; f[7] = hi.w;
            }
            if (p.addend != nullptr) {
                const float4 a0 = __ldcg(reinterpret_cast<const float4*>(p.addend + (size_t)c * 8));
                const float4 a1 = __ldcg(reinterpret_cast<const float4*>(p.addend + (size_t)c * 8 + 4));
                f[0] += a0.x; f[1] += a0.y; f[2] += a0.z; f[3] += a0.w; f[4] += a1.x; f[5] += a1.y; f[6] += a1.z; f[7] += a1.w;
            }
            if (p.addend_parts != nullptr) {       // (p0 + p1 + ...) + x: the partials first, in rank order, as an all-reduce would
                float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                for (int r = 0; r < p.n_parts; ++r) {
                    const uint2* part = p.addend_parts + (size_t)r * p.K + (size_t)c * 8;
                    unsigned long long w[8];
                    int spins = 0;
                    for (;;) {                     // until all eight words carry this exchange's count
#pragma unroll
                        for (int j = 0; j < 4; ++j) ld_peer_words(part + 2 * j, w[2 * j], w[2 * j + 1]);
                        bool ok = true;
#pragma unroll
                        for (int j = 0; j < 8; ++j) ok = ok && (unsigned int)(w[j] >> 32) == want;
                        if (ok || pw.dead) break;
                        if ((++spins & 15) == 0) {
                            if (peer_wait_expired(pw, p.error, p.error_host, p.wait_ns)) break;
                            __nanosleep(32);
                        }
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) a[j] += __uint_as_float((unsigned int)w[j]);
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] += a[j];
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
            reinterpret_cast<float4*>(xf32)[2 * c] = make_float4(f[0], f[1], f[2], f[3]);
            reinterpret_cast<float4*>(xf32)[2 * c + 1] = make_float4(f[4], f[5], f[6], f[7]);
            if ((from_table || p.addend != nullptr || p.addend_parts != nullptr) && blockIdx.x == 0) {
                reinterpret_cast<float4*>(p.resid_out)[2 * c] = make_float4(f[0], f[1], f[2], f[3]);
                reinterpret_cast<float4*>(p.resid_out)[2 * c + 1] = make_float4(f[4], f[5], f[6], f[7]);
            }
        }
        ss = warp_sum(ss);
        if (lane == 0) misc[warp] = ss;
        __syncthreads();
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < kGemvWarps; ++w) tot += misc[w];
        const float inv = 1.0f / sqrtf(tot / (float)p.K + p.eps);
        for (int c = tid; c < nch; c += kGemvThreads) {       // same thread, same chunks as above
            const float4 lo = reinterpret_cast<const float4*>(xf32)[2 * c], hi = reinterpret_cast<const float4*>(xf32)[2 * c + 1];
            float w[8];
            unpack8(gs[c], w);
            reinterpret_cast<float4*>(xs)[2 * c] = make_float4(lo.x * inv * w[0], lo.y * inv * w[1], lo.z * inv * w[2], lo.w * inv * w[3]);
            reinterpret_cast<float4*>(xs)[2 * c + 1] = make_float4(hi.x * inv * w[4], hi.y * inv * w[5], hi.z * inv * w[6], hi.w * inv * w[7]);
        }
    }
    __syncthreads();
}

// Stage activations (with the fused norm), stream the rows, reduce, epilogue.
template <Epi EPI>
__device__ __forceinline__ void gemv_run(const GemvParams& p, const GemvSched& sc, GemvRegs& r, unsigned char* smem,
                                         const unsigned int xbytes, float& best_v, int& best_i) {
    const float* xs = reinterpret_cast<const float*>(smem);
    float* red = reinterpret_cast<float*>(smem + xbytes + gemv_wbytes(p.K));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nch = sc.nch;

    // residual pair of the first item, fetched under the weight stream
    float2 old_first = make_float2(0.f, 0.f);
    if constexpr (EPI == Epi::Residual) {
        if (sc.wk == 0 && lane == 0 && sc.total > 0)
            old_first = __ldcg(reinterpret_cast<const float2*>(p.residual + sc.ig0 * 2));
    }
    gemv_stage(p, nch, smem, xbytes);
    (void)tid;

    // ---- rows ------------------------------------------------------------------------------------
    float acc0 = 0.f, acc1 = 0.f;
    int parity = 0;
    auto compute_unit = [&](const int u, const uint4 (&buf)[kGemvU][2]) {
        const int j = u / sc.upi, part = u - j * sc.upi;
#pragma unroll
        for (int uu = 0; uu < kGemvU; ++uu) {
            const int c = (part * kGemvU + uu) * sc.stride + sc.gl;
            if (c < nch) {
                const float4 xlo = reinterpret_cast<const float4*>(xs)[2 * c], xhi = reinterpret_cast<const float4*>(xs)[2 * c + 1];
                const float xf[8] = {xlo.x, xlo.y, xlo.z, xlo.w, xhi.x, xhi.y, xhi.z, xhi.w};
                acc0 = dot8(buf[uu][0], xf, acc0);
                acc1 = dot8(buf[uu][1], xf, acc1);
            }
        }
        if (part != sc.upi - 1) return;
        // item complete
        const int ig = sc.ig0 + j * sc.ig_stride;
        float t0 = warp_sum(acc0), t1 = warp_sum(acc1);
        acc0 = 0.f;
        acc1 = 0.f;
        if (sc.ks > 1) {
            float* buf2 = red + parity * kGemvWarps * 2;
            if (lane == 0) { buf2[warp * 2] = t0; buf2[warp * 2 + 1] = t1; }
            group_barrier(1 + sc.gi, sc.ks * 32);
            if (sc.wk == 0) {
                t0 = 0.f;
                t1 = 0.f;
                for (int w = 0; w < sc.ks; ++w) { t0 += buf2[(sc.gi * sc.ks + w) * 2]; t1 += buf2[(sc.gi * sc.ks + w) * 2 + 1]; }
            }
            parity ^= 1;
        }
        if (sc.wk == 0 && lane == 0) {
            if constexpr (EPI == Epi::Residual) {
                const float2 old = j == 0 ? old_first : __ldcg(reinterpret_cast<const float2*>(p.residual + ig * 2));
                *reinterpret_cast<float2*>(p.residual + ig * 2) = make_float2(old.x + t0, old.y + t1);
            } else {
                item_epilogue<EPI>(p, ig, t0, t1, best_v, best_i);
            }
        }
    };
    for (int u = 0; u < sc.total; ++u) {
        if (u > 0) gemv_load_unit<EPI>(p, sc, u, r.a);       // unit 0 was fetched before the dependency wait
        compute_unit(u, r.a);
    }
}

// Per-block (max, argmax) of the Logits epilogue -> part_val / part_idx[block].
__device__ __forceinline__ void gemv_publish_best(const GemvParams& p, float best_v, int best_i, float* bv, int* bi) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
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
        for (int w = 1; w < kGemvWarps; ++w)
            if (bv[w] > v || (bv[w] == v && bi[w] < i)) { v = bv[w]; i = bi[w]; }
        p.part_val[blockIdx.x] = v;
        p.part_idx[blockIdx.x] = i;
    }
}

// One GEMV phase as its own launch (phase-per-launch decode form, prefill lm_head, operator API).
template <Epi EPI>
__global__ void __launch_bounds__(kGemvThreads, 1) gemv_kernel(const GemvParams p, const int ks) {
    extern __shared__ __align__(16) unsigned char gemv_smem[];
    __shared__ float bv[kGemvWarps];
    __shared__ int bi[kGemvWarps];
    const unsigned int xbytes = gemv_xbytes(p.K);
    GemvRegs regs;
    float best_v = -INFINITY;
    int best_i = 0x7fffffff;
    // Let the next kernel of the step start its own weight prefetch as soon as every block of this
    // one is resident, then prefetch (independent of every earlier kernel), then wait.
    pdl_launch_dependents();
    const GemvSched sc = gemv_sched(p, ks, blockIdx.x, gridDim.x);
    gemv_prefetch<EPI>(p, sc, regs, gemv_smem, xbytes);
    pdl_wait();
    if constexpr (EPI == Epi::Peers) best_i = (int)(__ldcg(p.epoch) + 1u);      // this launch's exchange count rides in best_i
    gemv_run<EPI>(p, sc, regs, gemv_smem, xbytes, best_v, best_i);
    if constexpr (EPI == Epi::Logits) gemv_publish_best(p, best_v, best_i, bv, bi);
    if constexpr (EPI == Epi::Peers) {
        // every block has read the count by now; the one that draws the last ticket advances it for the consumer
        __syncthreads();
        if (threadIdx.x == 0) {
            const unsigned int t = atomicAdd(p.ticket, 1u);
            if (t == gridDim.x - 1) {
                *p.ticket = 0u;
                *p.epoch = (unsigned int)best_i;
            }
        }
    }
}

__host__ __device__ inline size_t gemv_smem_bytes(int K) {      // xs (fp32) | norm weight | red + misc
    return (size_t)gemv_xbytes(K) + gemv_wbytes(K) + (size_t)(2 * kGemvWarps * 2 + 16) * sizeof(float);
}

}  // namespace efm
