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

// In-place rotary embedding of the q and k parts of qkv [N, 3 * heads * D] (q | k | v along the row).
// The D/2 rotation angles of a patch are D/4 from its row index and D/4 from its column index, both
// with inv_freq[i] = theta^(-2 i / (D/2)); element d pairs with d + D/2 (rotate-half).  fp32 math,
// one rounding to bf16.  One block per patch; thread = (q|k, head, pair).
__global__ void __launch_bounds__(256) vit_rope2d_kernel(__nv_bfloat16* __restrict__ qkv, const int32_t* __restrict__ pos_h,
                                                        const int32_t* __restrict__ pos_w, int heads, int D, float theta) {
    const int n = blockIdx.x;
    const int half = D / 2, quarter = D / 4;
    const float ph = (float)pos_h[n], pw = (float)pos_w[n];
    __nv_bfloat16* row = qkv + (size_t)n * 3 * heads * D;
    const int total = 2 * heads * half;
    for (int i = threadIdx.x; i < total; i += 256) {
        const int pair = i % half, hh = i / half;            // hh in [0, 2*heads): q heads then k heads
        const int f = pair < quarter ? pair : pair - quarter;
        const float inv = 1.0f / powf(theta, (float)(2 * f) / (float)half);
        const float ang = (pair < quarter ? ph : pw) * inv;
        float sn, cs;
        sincosf(ang, &sn, &cs);
        __nv_bfloat16* x = row + (size_t)hh * D;
        const float a = __bfloat162float(x[pair]), b = __bfloat162float(x[pair + half]);
        x[pair] = __float2bfloat16_rn(a * cs - b * sn);
        x[pair + half] = __float2bfloat16_rn(b * cs + a * sn);
    }
}

}  // namespace efm
