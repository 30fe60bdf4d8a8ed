// Row-wise kernels of the prefill pass (S tokens at once).  The contractions live in the GEMM
// and attention files; these are the HBM-bound glue steps, each one read and one write of an
// [S, *] activation.
#pragma once
#include "common.cuh"

namespace efm {

// Embedding gather with custom-embedding injection.  One block per token.
// Same contract as the reference's embedding_lookup_with_embedding_insertion_kernel
// (src/layers/embed_head.cu:63-132): ids in [embed_token_id, embed_token_id + n_custom) take
// row id - embed_token_id of `custom`; other ids inside the vocabulary take the table row; any
// other id yields zeros.
__global__ void __launch_bounds__(128) embed_rows_kernel(const int32_t* __restrict__ ids,
                                                         const __nv_bfloat16* __restrict__ table,
                                                         const __nv_bfloat16* __restrict__ custom,
                                                         float* __restrict__ out, int vocab, int hidden,
                                                         int embed_token_id, int n_custom) {
    const int t = blockIdx.x;
    const int id = ids[t];
    const __nv_bfloat16* src = nullptr;
    if (custom != nullptr && embed_token_id >= 0 && id >= embed_token_id && id < embed_token_id + n_custom)
        src = custom + (size_t)(id - embed_token_id) * hidden;
    else if (id >= 0 && id < vocab)
        src = table + (size_t)id * hidden;
    float4* dst = reinterpret_cast<float4*>(out + (size_t)t * hidden);      // residual stream: fp32
    for (int c = threadIdx.x; c < hidden / 8; c += blockDim.x) {
        float f[8];
        unpack8(src != nullptr ? ld_cached(src + (size_t)c * 8) : make_uint4(0, 0, 0, 0), f);
        dst[2 * c] = make_float4(f[0], f[1], f[2], f[3]);
        dst[2 * c + 1] = make_float4(f[4], f[5], f[6], f[7]);
    }
}

// y[s,:] = bf16(x[s,:] * rsqrt(mean(x^2) + eps) * w), x = fp32 residual stream, fp32 inside (reference: FlashInfer RMSNorm
// through src/operators/norm_op.cu:20-62; formula pinned by tests/operators/test_norm_sampler.py:62-64).
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(const float* __restrict__ x,
                                                           const __nv_bfloat16* __restrict__ w,
                                                           __nv_bfloat16* __restrict__ y, int hidden, float eps) {
    __shared__ float part[8];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* xr = x + (size_t)blockIdx.x * hidden;
    const int nch = hidden >> 3;
    float ss = 0.f;
    for (int c = tid; c < nch; c += 256) {
        const float4 lo = reinterpret_cast<const float4*>(xr)[2 * c], hi = reinterpret_cast<const float4*>(xr)[2 * c + 1];
        const float f[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
    }
    ss = warp_sum(ss);
    if (lane == 0) part[warp] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += part[i];
    const float inv = 1.0f / sqrtf(tot / (float)hidden + eps);
    uint4* yr = reinterpret_cast<uint4*>(y + (size_t)blockIdx.x * hidden);
    for (int c = tid; c < nch; c += 256) {
        const float4 lo = reinterpret_cast<const float4*>(xr)[2 * c], hi = reinterpret_cast<const float4*>(xr)[2 * c + 1];
        const float f[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
        float g[8];
        unpack8(ld_cached(w + (size_t)c * 8), g);
        uint4 o;
        o.x = pack_bf16(f[0] * inv * g[0], f[1] * inv * g[1]);
        o.y = pack_bf16(f[2] * inv * g[2], f[3] * inv * g[3]);
        o.z = pack_bf16(f[4] * inv * g[4], f[5] * inv * g[5]);
        o.w = pack_bf16(f[6] * inv * g[6], f[7] * inv * g[7]);
        yr[c] = o;
    }
}

// Rotate-half RoPE / M-RoPE on the q and k parts of a fused [S, (q+2kv)*D] projection, then
// scatter: q -> [S, q_heads, D]; rotated k and raw v -> cache rows kv_offset + s.
// Convention of the reference: angle = pos * theta^(-2d/D); o[d] = x0 cos - x1 sin,
// o[d+D/2] = x1 cos + x0 sin (src/operators/attention_op.cu:327-371); M-RoPE picks the position
// row by rotary-pair section (src/layers/attention.cu:17-72).  Grid (S, q+2kv), block D/2.
__global__ void rope_scatter_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ q_out,
                                    __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                                    const float* __restrict__ inv_freq, const int32_t* __restrict__ pos3,
                                    int S, int q_heads, int kv_heads, int D, int kv_offset, int use_mrope,
                                    int sec0, int sec1) {
    const int s = blockIdx.x, head = blockIdx.y, d = threadIdx.x, half = D >> 1;
    if (d >= half) return;
    const int width = (q_heads + 2 * kv_heads) * D;
    const __nv_bfloat16* src = qkv + (size_t)s * width + (size_t)head * D;
    const float x0 = __bfloat162float(src[d]), x1 = __bfloat162float(src[d + half]);
    const size_t row = (size_t)(kv_offset + s) * kv_heads * D;
    if (head < q_heads + kv_heads) {
        int pos;
        if (use_mrope) pos = pos3[(d < sec0 ? 0 : (d < sec1 ? 1 : 2)) * S + s];
        else pos = kv_offset + s;
        float sn, cs;
        sincosf((float)pos * inv_freq[d], &sn, &cs);
        const __nv_bfloat16 o0 = __float2bfloat16_rn(x0 * cs - x1 * sn);
        const __nv_bfloat16 o1 = __float2bfloat16_rn(x1 * cs + x0 * sn);
        if (head < q_heads) {
            __nv_bfloat16* dst = q_out + ((size_t)s * q_heads + head) * D;
            dst[d] = o0;
            dst[d + half] = o1;
        } else {
            __nv_bfloat16* dst = k_cache + row + (size_t)(head - q_heads) * D;
            dst[d] = o0;
            dst[d + half] = o1;
        }
    } else {
        __nv_bfloat16* dst = v_cache + row + (size_t)(head - q_heads - kv_heads) * D;
        dst[d] = src[d];
        dst[d + half] = src[d + half];
    }
}

// act[s, j] = bf16(silu(gate) * up) from the fp32 fused projection [S, 2I] whose columns come in
// blocks of 64 gate values followed by the 64 matching up values
// (reference: act_and_mul, src/operators/activation_op.cu:35-76).
__global__ void __launch_bounds__(256) swiglu_rows_kernel(const float* __restrict__ gu,
                                                          __nv_bfloat16* __restrict__ act, int S, int I) {
    const size_t total = (size_t)S * I;
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (size_t)gridDim.x * 256) {
        const size_t s = i / I;
        const int j = (int)(i - s * I);
        const float* row = gu + s * 2 * (size_t)I + ((j >> 6) << 7) + (j & 63);
        const float g = row[0], u = row[64];
        act[i] = __float2bfloat16_rn(g / (1.0f + expf(-g)) * u);
    }
}

// Tensor parallel prefill: resid += sum, `sum` being the all-reduced fp32 output of a row-parallel linear.
__global__ void __launch_bounds__(256) add_rows_kernel(float* __restrict__ resid, const float* __restrict__ sum,
                                                       size_t n_pairs) {
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n_pairs; i += (size_t)gridDim.x * 256) {
        const float2 old = reinterpret_cast<const float2*>(resid)[i];
        const float2 s = reinterpret_cast<const float2*>(sum)[i];
        reinterpret_cast<float2*>(resid)[i] = make_float2(old.x + s.x, old.y + s.y);
    }
}

// Causal GQA prefill attention on CUDA cores: one warp per (query, q head); the warp is four
// independent 8-lane streams, stream j walking keys j, j+4, ... with its own online-softmax
// state; the four states merge at the end.  Queries sit at cache rows kv_offset + s and see rows
// [0, kv_offset + s] (reference: prefill attention with the q offset, qwen2_5.cpp:812-814;
// FlashInfer SinglePrefillWithKVCache through src/operators/attention_op.cu:1221-1343).
// Grid (ceil(S/4), q_heads), 128 threads.
template <int D>
__global__ void __launch_bounds__(128) prefill_attention_kernel(const __nv_bfloat16* __restrict__ q,
                                                                const __nv_bfloat16* __restrict__ k_cache,
                                                                const __nv_bfloat16* __restrict__ v_cache,
                                                                __nv_bfloat16* __restrict__ out, int S,
                                                                int kv_offset, int q_heads, int kv_heads,
                                                                float scale) {
    constexpr int E = D / 8;                 // channels per lane
    constexpr int NV = E / 8;                // uint4 per lane and row
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int s = blockIdx.x * 4 + warp, h = blockIdx.y;
    if (s >= S) return;
    const int kvh = h / (q_heads / kv_heads);
    const int stream = lane >> 3, part = lane & 7;
    const size_t row_stride = (size_t)kv_heads * D;
    float qf[E];
    {
        const __nv_bfloat16* qr = q + ((size_t)s * q_heads + h) * D + part * E;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            float t[8];
            unpack8(ld_cached(qr + j * 8), t);
#pragma unroll
            for (int e = 0; e < 8; ++e) qf[j * 8 + e] = t[e] * scale;
        }
    }
    float m = -INFINITY, l = 0.f, o[E];
#pragma unroll
    for (int e = 0; e < E; ++e) o[e] = 0.f;
    const int n_keys = kv_offset + s + 1;
    const int n_iter = (n_keys + 3) >> 2;    // every lane runs the same trip count (shuffles inside)
    for (int it = 0; it < n_iter; ++it) {
        const int t = it * 4 + stream;
        const bool valid = t < n_keys;
        const size_t off = (size_t)(valid ? t : 0) * row_stride + (size_t)kvh * D + part * E;
        uint4 kv[NV], vv[NV];
#pragma unroll
        for (int j = 0; j < NV; ++j) { kv[j] = ld_cached(k_cache + off + j * 8); vv[j] = ld_cached(v_cache + off + j * 8); }
        float dot = 0.f;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            float kf[8];
            unpack8(kv[j], kf);
#pragma unroll
            for (int e = 0; e < 8; ++e) dot = fmaf(kf[e], qf[j * 8 + e], dot);
        }
        dot += __shfl_xor_sync(0xffffffffu, dot, 1);
        dot += __shfl_xor_sync(0xffffffffu, dot, 2);
        dot += __shfl_xor_sync(0xffffffffu, dot, 4);
        if (valid) {
            const float mn = fmaxf(m, dot);
            const float corr = expf(m - mn), pj = expf(dot - mn);
            l = l * corr + pj;
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                float vf[8];
                unpack8(vv[j], vf);
#pragma unroll
                for (int e = 0; e < 8; ++e) o[j * 8 + e] = fmaf(pj, vf[e], o[j * 8 + e] * corr);
            }
            m = mn;
        }
    }
    // merge the four streams (lanes with equal `part`)
#pragma unroll
    for (int sh = 8; sh < 32; sh <<= 1) {
        const float mo = __shfl_xor_sync(0xffffffffu, m, sh);
        const float lo = __shfl_xor_sync(0xffffffffu, l, sh);
        const float mn = fmaxf(m, mo);
        const float ca = mn == -INFINITY ? 0.f : expf(m - mn), cb = mn == -INFINITY ? 0.f : expf(mo - mn);
        l = l * ca + lo * cb;
#pragma unroll
        for (int e = 0; e < E; ++e) {
            const float oo = __shfl_xor_sync(0xffffffffu, o[e], sh);
            o[e] = o[e] * ca + oo * cb;
        }
        m = mn;
    }
    if (stream == 0) {
        const float inv = l > 0.f ? 1.0f / l : 0.f;
        __nv_bfloat16* dst = out + ((size_t)s * q_heads + h) * D + part * E;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            uint4 v;
            v.x = pack_bf16(o[j * 8 + 0] * inv, o[j * 8 + 1] * inv);
            v.y = pack_bf16(o[j * 8 + 2] * inv, o[j * 8 + 3] * inv);
            v.z = pack_bf16(o[j * 8 + 4] * inv, o[j * 8 + 5] * inv);
            v.w = pack_bf16(o[j * 8 + 6] * inv, o[j * 8 + 7] * inv);
            reinterpret_cast<uint4*>(dst)[j] = v;
        }
    }
}

}  // namespace efm
