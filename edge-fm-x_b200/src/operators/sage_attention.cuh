// INT8 ("SageAttention"-style) causal prefill attention.
// (The reference tree holds no source for it, only two README mentions, README.md:23,456; the rule is the
//  published one: keys centred per kv head, Q and K quantised to INT8 per block of 128 tokens and head with
//  scale = max|x| / 127, S = (Qi8 . Ki8^T) sq sk / sqrt(D) from an exact int32 dot product, fp32 online
//  softmax, P in fp16, P . V in fp16 with fp32 accumulation.)
//
// Pre-pass (HBM-bound, a few microseconds): per-block key sums; Q and centred K to INT8 + scales; V to fp16.
// Main kernel at head_dim 128: the INT8 variant of seg_attention_tc_kernel (attention_tc.cuh: tcgen05.mma kind::i8 into
// TMEM for Q.K^T, kind::f16 for P.V).  The kernel of this file serves head_dim 64 and EFM_B200_ATTN_TC=0: same tiling as
// seg_attention_kernel (64 queries x 64-key tiles, cp.async double buffer,
// ldmatrix fragments) with mma.sync m16n8k32 s8 for Q.K^T and m16n8k16 f16 for P.V.  Causal rule only:
// query i sees keys [0, kv_offset + i].  Bound: tensor pipe.
#pragma once
#include <cuda_fp16.h>

#include "attention_mma.cuh"
#include "common.cuh"

namespace efm {

constexpr int kSageBlock = 128;      // tokens per quantisation block

// Partial sums for the key mean: block (b, h) adds up the rows of quantisation block b of kv head h,
// part[b][h][:] (fp32).  The consumer adds the partials in block order, so the mean is deterministic.
// 512 threads: warp w takes rows w, w + 16, ... (eight independent loads per lane), lane l the channels 4l .. 4l+3.
__global__ void __launch_bounds__(512) sage_ksum_kernel(const __nv_bfloat16* __restrict__ k, int stride, int T, int heads, int D,
                                                       float* __restrict__ part) {
    __shared__ float red[16][kSageBlock];
    const int b = blockIdx.x, h = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t0 = b * kSageBlock;
    float a[4] = {0.f, 0.f, 0.f, 0.f};
    if (lane * 4 < D) {
        uint2 w[kSageBlock / 16];
#pragma unroll
        for (int i = 0; i < kSageBlock / 16; ++i) {
            const int t = t0 + warp + 16 * i;
            w[i] = t < T ? *reinterpret_cast<const uint2*>(k + (size_t)t * stride + (size_t)h * D + lane * 4) : make_uint2(0u, 0u);
        }
#pragma unroll
        for (int i = 0; i < kSageBlock / 16; ++i) {
            a[0] += bf16lo(w[i].x); a[1] += bf16hi(w[i].x); a[2] += bf16lo(w[i].y); a[3] += bf16hi(w[i].y);
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) red[warp][lane * 4 + e] = a[e];
    }
    __syncthreads();
    if ((int)threadIdx.x < D) {
        float sum = 0.f;
#pragma unroll
        for (int w2 = 0; w2 < 16; ++w2) sum += red[w2][threadIdx.x];
        part[((size_t)b * heads + h) * D + threadIdx.x] = sum;
    }
}

// One block = one quantisation block (128 tokens) of one head, 512 threads: four threads per token row, each
// holding a quarter of the row in registers (max, then quantise, no second read).
// out: int8 [T, heads, D]; scales: [ceil(T/128), heads].  ksum (may be null): the partial key sums of
// sage_ksum_kernel, [n_part][heads][D]; the row mean (sum of the partials in order, divided by T) is subtracted.
template <int D>
__global__ void __launch_bounds__(512) sage_quant_kernel(const __nv_bfloat16* __restrict__ x, int stride, int T, int heads,
                                                        const float* __restrict__ ksum, int n_part, int8_t* __restrict__ out,
                                                        float* __restrict__ scales) {
    constexpr int Q = D / 4;                              // elements per thread (32 or 16)
    __shared__ float wmax[16];
    __shared__ float s_scale;
    __shared__ float s_mean[D];
    const int b = blockIdx.x, h = blockIdx.y, r = threadIdx.x >> 2, part = threadIdx.x & 3;
    const int t = b * kSageBlock + r;
    if (ksum != nullptr && (int)threadIdx.x < D) {
        float a = 0.f;
        for (int i = 0; i < n_part; ++i) a += ksum[((size_t)i * heads + h) * D + threadIdx.x];
        s_mean[threadIdx.x] = a / (float)T;
    }
    __syncthreads();
    float v[Q];
    float amax = 0.f;
    if (t < T) {
        const __nv_bfloat16* src = x + (size_t)t * stride + (size_t)h * D + part * Q;
#pragma unroll
        for (int j = 0; j < Q / 8; ++j) {
            const uint4 w = *reinterpret_cast<const uint4*>(src + j * 8);
            float f[8];
            unpack8(w, f);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                v[j * 8 + e] = ksum != nullptr ? f[e] - s_mean[part * Q + j * 8 + e] : f[e];
                amax = fmaxf(amax, fabsf(v[j * 8 + e]));
            }
        }
    } else {
#pragma unroll
        for (int e = 0; e < Q; ++e) v[e] = 0.f;
    }
    amax = warp_max(amax);
    if ((threadIdx.x & 31) == 0) wmax[threadIdx.x >> 5] = amax;
    __syncthreads();
    if (threadIdx.x == 0) {
        float m = 0.f;
        for (int w = 0; w < 16; ++w) m = fmaxf(m, wmax[w]);
        const float sc = m > 0.f ? m / 127.0f : 1.0f;
        s_scale = sc;
        scales[b * heads + h] = sc;
    }
    __syncthreads();
    if (t >= T) return;
    const float sc = s_scale;
    int8_t* dst = out + ((size_t)t * heads + h) * D + part * Q;
#pragma unroll
    for (int j = 0; j < Q / 16; ++j) {
        uint32_t packed[4];
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            uint32_t word = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int qv = (int)fminf(fmaxf(rintf(v[j * 16 + w * 4 + i] / sc), -127.f), 127.f);
                word |= (uint32_t)(qv & 0xff) << (8 * i);
            }
            packed[w] = word;
        }
        *reinterpret_cast<uint4*>(dst + j * 16) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    }
}

// bf16 rows [T, heads*D] (row stride `stride`) -> contiguous fp16 [T, heads*D].
__global__ void __launch_bounds__(256) sage_to_half_kernel(const __nv_bfloat16* __restrict__ x, int stride, int T, int width,
                                                          __half* __restrict__ out) {
    const size_t total = (size_t)T * width / 2;
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (size_t)gridDim.x * 256) {
        const size_t t = (i * 2) / width, c = (i * 2) % width;
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(x + t * stride + c));
        *reinterpret_cast<__half2*>(out + t * width + c) = __floats2half2_rn(f.x, f.y);
    }
}

struct SageAttnParams {
    const int8_t* q;        // [S, q_heads, D]
    const int8_t* k;        // [T, kv_heads, D] (centred)
    const __half* v;        // [T, kv_heads, D]
    const float* sq;        // [ceil(S/128), q_heads]
    const float* sk;        // [ceil(T/128), kv_heads]
    __nv_bfloat16* out;     // [S, q_heads, D]
    int S, kv_offset, q_heads, kv_heads;
    float scale;            // 1 / sqrt(D)
};

namespace sg {
using namespace sa;
template <int D> constexpr int q_row() { return D + 16; }            // int8 rows, 16 bytes of padding
template <int D> constexpr int v_row() { return (D + 8) * 2; }       // fp16 rows
constexpr int BQ = 64, kThreads = 128;                                 // 4 warps x 16 query rows
template <int D> constexpr size_t smem_bytes() { return (size_t)BQ * q_row<D>() * 3 + (size_t)BKV * v_row<D>() * 2; }

__device__ __forceinline__ void mma_s8(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_half(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}
// 64 rows of ROW_BYTES payload bytes from global (row pitch in bytes) into padded shared rows; rows outside
// [0, row_end) are zero filled.
template <int PAYLOAD, int SROW>
__device__ __forceinline__ void load_rows(uint32_t smem, const unsigned char* base, size_t pitch, int row0, int row_end) {
    constexpr int CH = PAYLOAD / 16;
    for (int idx = threadIdx.x; idx < 64 * CH; idx += kThreads) {
        const int r = idx / CH, ch = idx - r * CH;
        const int row = row0 + r;
        const bool in = row < row_end;
        cp_async16(smem + r * SROW + ch * 16, base + (size_t)(in ? row : 0) * pitch + ch * 16, in ? 16 : 0);
    }
}
}  // namespace sg

template <int D>
__global__ void __launch_bounds__(sg::kThreads) sage_attention_kernel(const SageAttnParams p) {
    using namespace sg;
    constexpr int QR = q_row<D>(), VR = v_row<D>();
    constexpr int KS = D / 32;           // int8 k-steps of Q K^T
    constexpr int DT = D / 8;            // 8-wide output tiles
    extern __shared__ __align__(16) unsigned char sage_smem[];
    const uint32_t sq_ = (uint32_t)__cvta_generic_to_shared(sage_smem);
    const uint32_t sk0 = sq_ + BQ * QR, sv0 = sk0 + 2 * BKV * QR;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int q0 = blockIdx.x * BQ, h = blockIdx.y;
    const int kvh = h / (p.q_heads / p.kv_heads);
    const unsigned char* qbase = reinterpret_cast<const unsigned char*>(p.q) + (size_t)h * D;
    const unsigned char* kbase = reinterpret_cast<const unsigned char*>(p.k) + (size_t)kvh * D;
    const unsigned char* vbase = reinterpret_cast<const unsigned char*>(p.v) + (size_t)kvh * D * 2;
    const size_t qpitch = (size_t)p.q_heads * D, kpitch = (size_t)p.kv_heads * D, vpitch = (size_t)p.kv_heads * D * 2;

    const int last_q = min(q0 + BQ, p.S) - 1;
    const int kend = p.kv_offset + last_q + 1;                         // keys [0, kend) are visible to the block
    const int ntiles = (kend + BKV - 1) / BKV;
    const int i0 = q0 + warp * 16 + g, i1 = i0 + 8;
    const int hi0 = i0 < p.S ? p.kv_offset + i0 + 1 : 0, hi1 = i1 < p.S ? p.kv_offset + i1 + 1 : 0;
    const float qs = p.sq[(q0 / kSageBlock) * p.q_heads + h] * p.scale * 1.4426950408889634f;

    load_rows<D, QR>(sq_, qbase, qpitch, q0, p.S);
    load_rows<D, QR>(sk0, kbase, kpitch, 0, kend);
    load_rows<D * 2, VR>(sv0, vbase, vpitch, 0, kend);
    cp_async_commit();

    uint32_t qf[KS][4];
    float o[DT][4];
#pragma unroll
    for (int d = 0; d < DT; ++d) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    for (int it = 0; it < ntiles; ++it) {
        const int buf = it & 1;
        if (it + 1 < ntiles) {
            load_rows<D, QR>(sk0 + (buf ^ 1) * BKV * QR, kbase, kpitch, (it + 1) * BKV, kend);
            load_rows<D * 2, VR>(sv0 + (buf ^ 1) * BKV * VR, vbase, vpitch, (it + 1) * BKV, kend);
        }
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        if (it == 0) {
#pragma unroll
            for (int ks = 0; ks < KS; ++ks)
                ldsm4(sq_ + (warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * QR + ks * 32 + 16 * (lane >> 4), qf[ks]);
        }
        const uint32_t sk = sk0 + buf * BKV * QR, sv = sv0 + buf * BKV * VR;
        int acc[8][4];
#pragma unroll
        for (int n = 0; n < 8; ++n) { acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0; }
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                uint32_t b[4];
                ldsm4(sk + (np * 16 + (lane & 7) + 8 * (lane >> 4)) * QR + ks * 32 + 16 * ((lane >> 3) & 1), b);
                mma_s8(acc[2 * np], qf[ks], b[0], b[1]);
                mma_s8(acc[2 * np + 1], qf[ks], b[2], b[3]);
            }
        }
        // dequantise (log2 units), mask, running maximum
        const float f = qs * p.sk[((it * BKV) / kSageBlock) * p.kv_heads + kvh];
        const int key0 = it * BKV + 2 * t;
        float s[8][4];
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int n = 0; n < 8; ++n) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int key = key0 + n * 8 + e;
                s[n][e] = key < hi0 ? (float)acc[n][e] * f : -INFINITY;
                s[n][2 + e] = key < hi1 ? (float)acc[n][2 + e] * f : -INFINITY;
                mx0 = fmaxf(mx0, s[n][e]);
                mx1 = fmaxf(mx1, s[n][2 + e]);
            }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const float base0 = mn0 == -INFINITY ? 0.f : mn0, base1 = mn1 == -INFINITY ? 0.f : mn1;
        const float c0 = m0 == -INFINITY ? 0.f : exp2f(m0 - base0), c1 = m1 == -INFINITY ? 0.f : exp2f(m1 - base1);
        m0 = mn0;
        m1 = mn1;
        l0 *= c0;
        l1 *= c1;
#pragma unroll
        for (int d = 0; d < DT; ++d) { o[d][0] *= c0; o[d][1] *= c0; o[d][2] *= c1; o[d][3] *= c1; }
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            s[n][0] = exp2f(s[n][0] - base0);
            s[n][1] = exp2f(s[n][1] - base0);
            s[n][2] = exp2f(s[n][2] - base1);
            s[n][3] = exp2f(s[n][3] - base1);
            l0 += s[n][0] + s[n][1];
            l1 += s[n][2] + s[n][3];
        }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            uint32_t a[4];
            a[0] = pack_half(s[2 * kk][0], s[2 * kk][1]);
            a[1] = pack_half(s[2 * kk][2], s[2 * kk][3]);
            a[2] = pack_half(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            a[3] = pack_half(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int dp = 0; dp < DT / 2; ++dp) {
                uint32_t b[4];
                ldsm4_t(sv + (kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * VR + (dp * 16 + 8 * (lane >> 4)) * 2, b);
                mma_f16(o[2 * dp], a, b[0], b[1]);
                mma_f16(o[2 * dp + 1], a, b[2], b[3]);
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();

    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float r0 = l0 > 0.f ? 1.0f / l0 : 0.f, r1 = l1 > 0.f ? 1.0f / l1 : 0.f;
    if (i0 < p.S) {
        __nv_bfloat16* dst = p.out + ((size_t)i0 * p.q_heads + h) * D + 2 * t;
#pragma unroll
        for (int d = 0; d < DT; ++d) *reinterpret_cast<uint32_t*>(dst + d * 8) = pack_bf16(o[d][0] * r0, o[d][1] * r0);
    }
    if (i1 < p.S) {
        __nv_bfloat16* dst = p.out + ((size_t)i1 * p.q_heads + h) * D + 2 * t;
#pragma unroll
        for (int d = 0; d < DT; ++d) *reinterpret_cast<uint32_t*>(dst + d * 8) = pack_bf16(o[d][2] * r1, o[d][3] * r1);
    }
}

}  // namespace efm
