// Batch-1 weight-streaming GEMV for the decode step, with the neighbouring element-wise work
// fused in so that one launch replaces a chain of the reference's kernels:
//
//   prologue  Plain            x is read as is                      (o_proj, down_proj)
//             RmsNorm          x = bf16(rmsnorm(residual) * w)      (K2/K3 + K4 of the reference:
//                                                                    src/operators/norm_op.cu:20-106)
//             EmbedRmsNorm     residual = embed_table[token] first  (src/layers/embed_head.cu:22-61)
//   epilogue  Plain            y = bf16(W x)
//             Residual         r = bf16(r + bf16(W x))              (fused add of norm_op.cu:64-106)
//             QkvRope          + bias, rotate-half RoPE / M-RoPE on q and k, append k, v to the
//                              cache row kv_len-1                    (linear_impl.cu:90-106,
//                              decode_runtime_kernels.cu:67-225)
//             SwiGlu           act = bf16(silu(gate) * up)          (fused_gate_up_activation_op.cu:198-277)
//             Logits           fp32 logits + per-block (max, argmax) (src/layers/linear.cu:187-270)
//
// Bound: HBM.  Each weight byte is read once, as 128-bit streaming loads, 16 loads in flight per
// lane; activations live in shared memory; dot products reduce with warp shuffles (and, when
// KSPLIT warps share one row group, a shared-memory exchange).  The first batch of weight
// loads is issued BEFORE griddepcontrol.wait, so that it overlaps the tail of the previous
// kernel when launched with programmatic dependent launch.
#pragma once
#include "common.cuh"

namespace efm {

enum class Epi : int { Plain = 0, Residual = 1, QkvRope = 2, SwiGlu = 3, Logits = 4 };
enum : int { kProPlain = 0, kProRmsNorm = 1, kProEmbedRmsNorm = 2 };

struct GemvParams {
    const __nv_bfloat16* W;   // [N, K] row-major
    int N, K, n_items;        // n_items = N / 2 (every epilogue consumes rows in pairs)
    // prologue
    int prologue;
    const __nv_bfloat16* x;   // Plain: [K]; RmsNorm: residual stream [K]
    const __nv_bfloat16* norm_w;
    float eps;
    const __nv_bfloat16* embed_table;
    int vocab;
    __nv_bfloat16* resid_out; // EmbedRmsNorm: block 0 stores the gathered row here
    DecodeState* state;
    // epilogue
    __nv_bfloat16* y;         // Plain: [N]; SwiGlu: [N/2]
    __nv_bfloat16* residual;  // Residual: [N] in/out
    const __nv_bfloat16* bias;
    __nv_bfloat16* q_out;     // QkvRope
    __nv_bfloat16* k_cache;
    __nv_bfloat16* v_cache;
    const float* inv_freq;
    int q_heads, kv_heads, head_dim, use_mrope, sec0, sec1, max_tokens;
    float* logits;            // Logits
    float* part_val;
    int* part_idx;
};

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
        const uint32_t old = __ldcg(reinterpret_cast<const unsigned int*>(p.residual + item * 2));
        *reinterpret_cast<uint32_t*>(p.residual + item * 2) =
            pack_bf16(bf16lo(old) + round_bf16(a0), bf16hi(old) + round_bf16(a1));
    } else if constexpr (EPI == Epi::SwiGlu) {
        const float s = a0 / (1.0f + expf(-a0));
        p.y[item] = __float2bfloat16_rn(s * a1);
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
        y0 = round_bf16(y0);
        y1 = round_bf16(y1);
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
                p.q_out[r0] = __float2bfloat16_rn(o0);
                p.q_out[r1] = __float2bfloat16_rn(o1);
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

// 256 threads; ITEMS row pairs per group iteration; KSPLIT warps share one group.
template <Epi EPI, int ITEMS, int KSPLIT>
__global__ void __launch_bounds__(256, 2) gemv_kernel(const GemvParams p) {
    constexpr int ROWS = ITEMS * 2, U = 8 / ITEMS, GP = 8 / KSPLIT;
    extern __shared__ __align__(16) unsigned char gemv_smem[];
    const size_t xbytes = ((size_t)p.K * 2 + 15) & ~(size_t)15;
    __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(gemv_smem);                 // activations [K]
    __nv_bfloat16* gs = reinterpret_cast<__nv_bfloat16*>(gemv_smem + xbytes);        // norm weight [K]
    float* red = reinterpret_cast<float*>(gemv_smem + 2 * xbytes);                    // [2][8][ROWS]
    float* misc = red + 2 * 8 * ROWS;                                                            // [16]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int gi = warp / KSPLIT, wk = warp % KSPLIT;
    const int gl = wk * 32 + lane, stride = KSPLIT * 32;
    const int nch = p.K >> 3;
    const int n_ig = (p.n_items + ITEMS - 1) / ITEMS;
    const int ig_stride = gridDim.x * GP;
    int ig = blockIdx.x * GP + gi;

    const __nv_bfloat16* rowp[ROWS];
    uint4 wv[U][ROWS];
    auto set_rows = [&](int g) {
#pragma unroll
        for (int it = 0; it < ITEMS; ++it) {
            int item = g * ITEMS + it;
            if (item >= p.n_items) item = p.n_items - 1;   // duplicate work, result discarded
            int r0, r1;
            item_rows<EPI>(p, item, r0, r1);
            rowp[2 * it] = p.W + (size_t)r0 * p.K;
            rowp[2 * it + 1] = p.W + (size_t)r1 * p.K;
        }
    };
    auto load_batch = [&](int cb) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int c = cb + u * stride + gl;
            if (c < nch) {
#pragma unroll
                for (int r = 0; r < ROWS; ++r) wv[u][r] = ld_stream(rowp[r] + (size_t)c * 8);
            }
        }
    };

    // Let the next kernel of the step start its own weight prefetch as soon as every block of
    // this one is resident, then prefetch (independent of every earlier kernel), then wait.
    pdl_launch_dependents();
    if (ig < n_ig) { set_rows(ig); load_batch(0); }
    if (p.prologue != kProPlain)          // the norm weight is a weight too: stage it before waiting
        for (int c = tid; c < nch; c += 256)
            reinterpret_cast<uint4*>(gs)[c] = ld_cached(p.norm_w + (size_t)c * 8);
    pdl_wait();

    // ---- prologue: stage the activation vector in shared memory -------------------------
    if (p.prologue == kProPlain) {
        for (int c = tid; c < nch; c += 256)
            reinterpret_cast<uint4*>(xs)[c] = ld_cached(p.x + (size_t)c * 8);
    } else {
        const __nv_bfloat16* src = p.x;
        bool zero = false;
        if (p.prologue == kProEmbedRmsNorm) {
            const int tok = p.state->token;
            zero = tok < 0 || tok >= p.vocab;
            src = p.embed_table + (size_t)(zero ? 0 : tok) * p.K;
        }
        float ss = 0.f;
        for (int c = tid; c < nch; c += 256) {
            uint4 v = zero ? make_uint4(0, 0, 0, 0) : ld_cached(src + (size_t)c * 8);
            float f[8];
            unpack8(v, f);
#pragma unroll
            for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
            if (p.prologue == kProEmbedRmsNorm && blockIdx.x == 0)
                reinterpret_cast<uint4*>(p.resid_out)[c] = v;
        }
        ss = warp_sum(ss);
        if (lane == 0) misc[warp] = ss;
        __syncthreads();
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) tot += misc[w];
        const float inv = 1.0f / sqrtf(tot / (float)p.K + p.eps);
        for (int c = tid; c < nch; c += 256) {
            uint4 v = zero ? make_uint4(0, 0, 0, 0) : ld_cached(src + (size_t)c * 8);
            const uint4 g = reinterpret_cast<const uint4*>(gs)[c];      // written by this same thread
            float f[8], w[8];
            unpack8(v, f);
            unpack8(g, w);
            uint4 o;
            o.x = pack_bf16(f[0] * inv * w[0], f[1] * inv * w[1]);
            o.y = pack_bf16(f[2] * inv * w[2], f[3] * inv * w[3]);
            o.z = pack_bf16(f[4] * inv * w[4], f[5] * inv * w[5]);
            o.w = pack_bf16(f[6] * inv * w[6], f[7] * inv * w[7]);
            reinterpret_cast<uint4*>(xs)[c] = o;
        }
    }
    __syncthreads();

    // ---- main loop ----------------------------------------------------------------------
    float best_v = -INFINITY;
    int best_i = 0x7fffffff;
    bool first = true;
    int parity = 0;
    for (; ig < n_ig; ig += ig_stride) {
        if (!first) set_rows(ig);
        float acc[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) acc[r] = 0.f;
        for (int cb = 0; cb < nch; cb += U * stride) {
            if (!(first && cb == 0)) load_batch(cb);
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int c = cb + u * stride + gl;
                if (c < nch) {
                    float xf[8];
                    unpack8(reinterpret_cast<const uint4*>(xs)[c], xf);
#pragma unroll
                    for (int r = 0; r < ROWS; ++r) acc[r] = dot8(wv[u][r], xf, acc[r]);
                }
            }
        }
        first = false;
#pragma unroll
        for (int r = 0; r < ROWS; ++r) acc[r] = warp_sum(acc[r]);
        if constexpr (KSPLIT > 1) {
            float* buf = red + parity * 8 * ROWS;
            if (lane == 0) {
#pragma unroll
                for (int r = 0; r < ROWS; ++r) buf[warp * ROWS + r] = acc[r];
            }
            group_barrier(1 + gi, KSPLIT * 32);
            if (wk == 0) {
#pragma unroll
                for (int r = 0; r < ROWS; ++r) {
                    float t = 0.f;
#pragma unroll
                    for (int w = 0; w < KSPLIT; ++w) t += buf[(gi * KSPLIT + w) * ROWS + r];
                    acc[r] = t;
                }
            }
            parity ^= 1;
        }
        if (wk == 0) {
#pragma unroll
            for (int it = 0; it < ITEMS; ++it) {
                const int item = ig * ITEMS + it;
                if (lane == it && item < p.n_items)
                    item_epilogue<EPI>(p, item, acc[2 * it], acc[2 * it + 1], best_v, best_i);
            }
        }
    }

    if constexpr (EPI == Epi::Logits) {
        // lanes 0..ITEMS-1 of the wk==0 warps hold candidates; reduce to one per block
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best_v, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (ov > best_v || (ov == best_v && oi < best_i)) { best_v = ov; best_i = oi; }
        }
        __shared__ float bv[8];
        __shared__ int bi[8];
        if (lane == 0) { bv[warp] = best_v; bi[warp] = best_i; }
        __syncthreads();
        if (tid == 0) {
            float v = bv[0];
            int i = bi[0];
            for (int w = 1; w < 8; ++w)
                if (bv[w] > v || (bv[w] == v && bi[w] < i)) { v = bv[w]; i = bi[w]; }
            p.part_val[blockIdx.x] = v;
            p.part_idx[blockIdx.x] = i;
        }
    }
}

inline size_t gemv_smem_bytes(int K, int items) {
    return 2 * (((size_t)K * 2 + 15) & ~(size_t)15) + (size_t)(2 * 8 * items * 2 + 16) * sizeof(float);
}

}  // namespace efm
