// Row kernels of the Qwen2.5-VL vision encoder around its GEMMs and attention: the window-major
// re-ordering of the patch rows, the 2-D rotary embedding, and the inverse re-ordering of the
// merged tokens.  (No counterpart in the reference, which receives image embeddings ready-made
// through Request.embedding; the arithmetic follows the published Qwen2.5-VL encoder.)
// All are HBM-bound row copies / elementwise passes.
#pragma once
#include "common.cuh"

namespace efm {

// dst block i (unit rows of `width` floats) = src block order[i].  width % 4 == 0.
__global__ void __launch_bounds__(256) vit_gather_blocks_f32_kernel(const float* __restrict__ src, float* __restrict__ dst,
                                                                   const int32_t* __restrict__ order, int n_blocks,
                                                                   int unit, int width) {
    const int per_block = unit * width / 4;
    for (int b = blockIdx.x; b < n_blocks; b += gridDim.x) {
        const float4* s = reinterpret_cast<const float4*>(src + (size_t)order[b] * unit * width);
        float4* d = reinterpret_cast<float4*>(dst + (size_t)b * unit * width);
        for (int i = threadIdx.x; i < per_block; i += 256) d[i] = s[i];
    }
}

// dst row order[i] = src row i (bf16 rows of `width` elements, width % 8 == 0).
__global__ void __launch_bounds__(128) vit_scatter_rows_bf16_kernel(const __nv_bfloat16* __restrict__ src,
                                                                   __nv_bfloat16* __restrict__ dst,
                                                                   const int32_t* __restrict__ order, int n_rows, int width) {
    for (int r = blockIdx.x; r < n_rows; r += gridDim.x) {
        const uint4* s = reinterpret_cast<const uint4*>(src + (size_t)r * width);
        uint4* d = reinterpret_cast<uint4*>(dst + (size_t)order[r] * width);
        for (int i = threadIdx.x; i < width / 8; i += 128) d[i] = s[i];
    }
}

// cos/sin table of the 2-D rotary embedding, one row of D/2 (cos, sin) pairs per patch: the first D/4
// angles come from the patch's row index, the next D/4 from its column index, both with
// inv_freq[i] = theta^(-2 i / (D/2)).  Computed once per encode call.
__global__ void __launch_bounds__(128) vit_rope_table_kernel(float2* __restrict__ table, const int32_t* __restrict__ pos_h,
                                                            const int32_t* __restrict__ pos_w, int n_patches, int D, float theta) {
    const int half = D / 2, quarter = D / 4;
    const int i = blockIdx.x * 128 + threadIdx.x;
    if (i >= n_patches * half) return;
    const int n = i / half, pair = i - n * half;
    const int f = pair < quarter ? pair : pair - quarter;
    const float inv = 1.0f / powf(theta, (float)(2 * f) / (float)half);
    const float ang = (float)(pair < quarter ? pos_h[n] : pos_w[n]) * inv;
    float sn, cs;
    sincosf(ang, &sn, &cs);
    table[i] = make_float2(cs, sn);
}

// In-place rotary embedding of the q and k parts of qkv [N, 3 * heads * D] (q | k | v along the row):
// element d pairs with d + D/2 (rotate-half); fp32 math, one rounding to bf16.  One block per patch;
// each thread rotates two adjacent pairs of one head (32-bit accesses).
__global__ void __launch_bounds__(256) vit_rope2d_kernel(__nv_bfloat16* __restrict__ qkv, const float2* __restrict__ table,
                                                        int heads, int D) {
    const int n = blockIdx.x;
    const int half = D / 2, hp = half / 2;                   // hp: 2-pair groups per head
    __nv_bfloat16* row = qkv + (size_t)n * 3 * heads * D;
    const float2* tab = table + (size_t)n * half;
    const int total = 2 * heads * hp;
    for (int i = threadIdx.x; i < total; i += 256) {
        const int hh = i / hp, pair = (i - hh * hp) * 2;     // hh in [0, 2*heads): q heads then k heads
        __nv_bfloat162* lo = reinterpret_cast<__nv_bfloat162*>(row + (size_t)hh * D + pair);
        __nv_bfloat162* hi = reinterpret_cast<__nv_bfloat162*>(row + (size_t)hh * D + pair + half);
        const float2 a = __bfloat1622float2(*lo), b = __bfloat1622float2(*hi);
        const float2 t0 = tab[pair], t1 = tab[pair + 1];
        *lo = __floats2bfloat162_rn(a.x * t0.x - b.x * t0.y, a.y * t1.x - b.y * t1.y);
        *hi = __floats2bfloat162_rn(b.x * t0.x + a.x * t0.y, b.y * t1.x + a.y * t1.y);
    }
}

}  // namespace efm
