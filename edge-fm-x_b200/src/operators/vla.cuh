// Row kernels of the SmolVLA-shaped action chunk around its GEMMs and attention: patch rows of the
// camera images, LayerNorm, pixel shuffle, prefix assembly, rotate-half RoPE with K/V scatter, the
// small fp32 linears of the flow-matching head and the Euler update.  Every kernel opens with the
// dependent-launch pair (release the next launch, then wait for the previous kernel's writes), so the chunk
// can be launched with programmatic stream serialization; without that attribute both are no-ops.  The reference ships no code
// for this model (only doc/smolvla_architecture.md); the arithmetic follows that description and
// the public SmolVLM vision tower.  All are HBM- or latency-bound elementwise / row passes.
#pragma once
#include "common.cuh"

namespace efm {

// images [n_img, 3, S, S] fp32 -> rows [n_img * side * side, 3 * p * p] bf16, (channel, ky, kx) inside a
// row as in the convolution weight.  One block per patch row.
__global__ void __launch_bounds__(256) vla_patch_rows_kernel(const float* __restrict__ images, __nv_bfloat16* __restrict__ rows,
                                                            int S, int p) {
    pdl_launch_dependents();
    pdl_wait();
    const int side = S / p, patch = blockIdx.x % (side * side), img = blockIdx.x / (side * side);
    const int pr = patch / side, pc = patch % side, pd = 3 * p * p;
    const float* im = images + (size_t)img * 3 * S * S;
    __nv_bfloat16* out = rows + (size_t)blockIdx.x * pd;
    for (int i = threadIdx.x; i < pd; i += 256) {
        const int c = i / (p * p), ky = (i / p) % p, kx = i % p;
        out[i] = __float2bfloat16_rn(im[((size_t)c * S + pr * p + ky) * S + pc * p + kx]);
    }
}

// dst[r, :] = float(src[r % period, :]) -- the learned position table repeated per image, as the start
// value of the residual stream (the patch GEMM then adds onto it).
__global__ void __launch_bounds__(256) vla_tile_rows_kernel(const __nv_bfloat16* __restrict__ src, float* __restrict__ dst,
                                                           int period, int width) {
    pdl_launch_dependents();
    pdl_wait();
    const __nv_bfloat16* s = src + (size_t)(blockIdx.x % period) * width;
    float* d = dst + (size_t)blockIdx.x * width;
    for (int i = threadIdx.x; i < width; i += 256) d[i] = __bfloat162float(s[i]);
}

// y[r, :] = bf16((x - mean) * rsqrt(var + eps) * w + b) over fp32 rows; one block per row, two passes
// over a row held in registers / L1 (width <= 4096).
__global__ void __launch_bounds__(256) layernorm_rows_kernel(const float* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                            const __nv_bfloat16* __restrict__ b, __nv_bfloat16* __restrict__ y,
                                                            int width, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[8];
    __shared__ float stat[2];
    const float* xr = x + (size_t)blockIdx.x * width;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float s = 0.f;
    for (int i = tid; i < width; i += 256) s += xr[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) red[warp] = s;
    __syncthreads();
    if (tid == 0) { float t = 0.f; for (int i = 0; i < 8; ++i) t += red[i]; stat[0] = t / (float)width; }
    __syncthreads();
    const float mu = stat[0];
    float v = 0.f;
    for (int i = tid; i < width; i += 256) { const float d = xr[i] - mu; v += d * d; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (tid == 0) { float t = 0.f; for (int i = 0; i < 8; ++i) t += red[i]; stat[1] = rsqrtf(t / (float)width + eps); }
    __syncthreads();
    const float rs = stat[1];
    __nv_bfloat16* yr = y + (size_t)blockIdx.x * width;
    for (int i = tid; i < width; i += 256)
        yr[i] = __float2bfloat16_rn((xr[i] - mu) * rs * __bfloat162float(w[i]) + __bfloat162float(b[i]));
}

// The same LayerNorm with one warp per row and the row held in registers (width <= 1024, width % 4 == 0): one read of
// x, no block barriers.  Eight rows per 256-thread block.
__global__ void __launch_bounds__(256) layernorm_rows_warp_kernel(const float* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                                 const __nv_bfloat16* __restrict__ b, __nv_bfloat16* __restrict__ y,
                                                                 int rows, int width, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, row = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= rows) return;
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)row * width);
    const int n4 = width >> 2;
    float4 v[8];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int c = lane + 32 * i;
        v[i] = c < n4 ? xr[c] : make_float4(0.f, 0.f, 0.f, 0.f);
        s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const float mu = s / (float)width;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        if (lane + 32 * i < n4) {
            const float a = v[i].x - mu, bb = v[i].y - mu, c = v[i].z - mu, d = v[i].w - mu;
            q += (a * a + bb * bb) + (c * c + d * d);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) q += __shfl_xor_sync(0xffffffffu, q, o);
    const float rs = rsqrtf(q / (float)width + eps);
    uint2* yr = reinterpret_cast<uint2*>(y + (size_t)row * width);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int c = lane + 32 * i;
        if (c < n4) {
            const uint2 wv = *reinterpret_cast<const uint2*>(w + 4 * c), bv = *reinterpret_cast<const uint2*>(b + 4 * c);
            const float w0 = __uint_as_float(wv.x << 16), w1 = __uint_as_float(wv.x & 0xffff0000u);
            const float w2 = __uint_as_float(wv.y << 16), w3 = __uint_as_float(wv.y & 0xffff0000u);
            const float b0 = __uint_as_float(bv.x << 16), b1 = __uint_as_float(bv.x & 0xffff0000u);
            const float b2 = __uint_as_float(bv.y << 16), b3 = __uint_as_float(bv.y & 0xffff0000u);
            yr[c] = make_uint2(pack_bf16((v[i].x - mu) * rs * w0 + b0, (v[i].y - mu) * rs * w1 + b1),
                               pack_bf16((v[i].z - mu) * rs * w2 + b2, (v[i].w - mu) * rs * w3 + b3));
        }
    }
}

// Pixel shuffle by factor s of every image: x [n_img * side * side, d] -> out [n_img * (side/s)^2, s*s*d];
// output token (R, C), channel (ry * s + cx) * d + e  <-  patch (R*s + ry, C*s + cx), channel e.
// One block per output token; d % 8 == 0.
__global__ void __launch_bounds__(256) vla_pixel_shuffle_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out,
                                                               int side, int s, int d) {
    pdl_launch_dependents();
    pdl_wait();
    const int ts = side / s, per = ts * ts;
    const int img = blockIdx.x / per, tok = blockIdx.x % per, R = tok / ts, C = tok % ts;
    const int d8 = d / 8;
    uint4* o = reinterpret_cast<uint4*>(out + (size_t)blockIdx.x * s * s * d);
    for (int i = threadIdx.x; i < s * s * d8; i += 256) {
        const int sub = i / d8, e = i % d8, ry = sub / s, cx = sub % s;
        const size_t row = (size_t)img * side * side + (size_t)(R * s + ry) * side + (C * s + cx);
        o[i] = reinterpret_cast<const uint4*>(x + row * d)[e];
    }
}

// Prefix assembly in the fp32 residual stream [P, H]: rows [0, n_img_tok) (already holding the connector
// output) are scaled by sqrt(H); the next n_lang rows are embed[id] * sqrt(H); the last row is
// state_proj(state).  One block per row.
__global__ void __launch_bounds__(256) vla_prefix_rows_kernel(float* __restrict__ resid, const __nv_bfloat16* __restrict__ embed,
                                                             const int32_t* __restrict__ ids, const float* __restrict__ state,
                                                             const __nv_bfloat16* __restrict__ sw, const __nv_bfloat16* __restrict__ sb,
                                                             int n_img_tok, int n_lang, int H, int state_dim, int vocab) {
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    float* row = resid + (size_t)r * H;
    const float sc = sqrtf((float)H);
    if (r < n_img_tok) {
        for (int i = threadIdx.x; i < H; i += 256) row[i] *= sc;
    } else if (r < n_img_tok + n_lang) {
        int id = ids[r - n_img_tok];
        id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
        const __nv_bfloat16* e = embed + (size_t)id * H;
        for (int i = threadIdx.x; i < H; i += 256) row[i] = __bfloat162float(e[i]) * sc;
    } else {
        for (int i = threadIdx.x; i < H; i += 256) {
            float a = __bfloat162float(sb[i]);
            for (int k = 0; k < state_dim; ++k) a += state[k] * __bfloat162float(sw[(size_t)i * state_dim + k]);
            row[i] = a;
        }
    }
}

// Rotate-half RoPE (inverse frequencies theta^(-2i/D)) on the q and k parts of qkv rows
// [rows, (q_heads + 2 kv_heads) * D] (q | k | v along the row), row r at position pos0 + r; q in place,
// and when kv_out != nullptr the rotated k and the v of row r are written to kv_out row kv_row0 + r
// ([.., 2 * kv_heads * D]: k | v) instead of in place.  kv_heads == 0: q only.  One block per row.
__global__ void __launch_bounds__(256) vla_rope_rows_kernel(__nv_bfloat16* __restrict__ qkv, int row_stride, int q_heads, int kv_heads,
                                                           int D, int pos0, float theta, __nv_bfloat16* __restrict__ kv_out,
                                                           int kv_out_stride, int kv_row0) {
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x, half = D / 2;
    __nv_bfloat16* row = qkv + (size_t)r * row_stride;
    const float pos = (float)(pos0 + r);
    const int heads = q_heads + kv_heads;
    for (int i = threadIdx.x; i < heads * half; i += 256) {
        const int h = i / half, f = i % half;
        const float inv = powf(theta, -(float)(2 * f) / (float)D);
        float sn, cs;
        sincosf(pos * inv, &sn, &cs);
        __nv_bfloat16* x = row + (size_t)h * D;
        const float x1 = __bfloat162float(x[f]), x2 = __bfloat162float(x[f + half]);
        const __nv_bfloat16 o1 = __float2bfloat16_rn(x1 * cs - x2 * sn), o2 = __float2bfloat16_rn(x2 * cs + x1 * sn);
        if (h >= q_heads && kv_out != nullptr) {
            __nv_bfloat16* d = kv_out + (size_t)(kv_row0 + r) * kv_out_stride + (size_t)(h - q_heads) * D;
            d[f] = o1; d[f + half] = o2;
        } else {
            x[f] = o1; x[f + half] = o2;
        }
    }
    if (kv_out != nullptr) {
        const __nv_bfloat16* v = row + (size_t)(q_heads + kv_heads) * D;
        __nv_bfloat16* d = kv_out + (size_t)(kv_row0 + r) * kv_out_stride + (size_t)kv_heads * D;
        for (int i = threadIdx.x; i < kv_heads * D; i += 256) d[i] = v[i];
    }
}

// dst rows [0, rows) of width w (stride dst_stride) = src rows (stride src_stride); w % 8 == 0, bf16.
__global__ void __launch_bounds__(128) vla_copy_rows_kernel(const __nv_bfloat16* __restrict__ src, int src_stride,
                                                           __nv_bfloat16* __restrict__ dst, int dst_stride, int w) {
    pdl_launch_dependents();
    pdl_wait();
    const uint4* s = reinterpret_cast<const uint4*>(src + (size_t)blockIdx.x * src_stride);
    uint4* d = reinterpret_cast<uint4*>(dst + (size_t)blockIdx.x * dst_stride);
    for (int i = threadIdx.x; i < w / 8; i += 128) d[i] = s[i];
}

// Small fp32 linear of the flow-matching head: y[m, n] = act(sum_k x[m, k] * W[n, k] + b[n]) with bf16 weights,
// fp32 input (row stride ldx) and fp32 output (row stride ldy, column offset applied by the caller).
// One warp per output element; ACT 0: none, 1: SiLU.  With `euler` != 0 the result is not stored but
// applied as y[m, n] += euler * value (the flow-matching update x += dt * v).  y16 (optional): bf16 copy of the result.
template <int ACT>
__global__ void __launch_bounds__(256) vla_small_linear_kernel(const float* __restrict__ x, int ldx, const __nv_bfloat16* __restrict__ W,
                                                              const __nv_bfloat16* __restrict__ b, float* __restrict__ y, int ldy,
                                                              int M, int N, int K, float euler, __nv_bfloat16* __restrict__ y16, int ldy16) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int o = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (o >= M * N) return;
    const int m = o / N, n = o % N;
    const float* xr = x + (size_t)m * ldx;
    const __nv_bfloat16* wr = W + (size_t)n * K;
    float a = 0.f;
    for (int k = lane; k < K; k += 32) a += xr[k] * __bfloat162float(wr[k]);
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) a += __shfl_xor_sync(0xffffffffu, a, s);
    if (lane != 0) return;
    if (b != nullptr) a += __bfloat162float(b[n]);
    if (ACT == 1) a = a / (1.0f + __expf(-a));
    if (euler != 0.f) y[(size_t)m * ldy + n] += euler * a;
    else y[(size_t)m * ldy + n] = a;
    if (y16 != nullptr) y16[(size_t)m * ldy16 + n] = __float2bfloat16_rn(a);  // bf16 copy (row stride ldy16) for a skinny product
}

// cat[m, off + i] = emb[i] for every row m: the time embedding of this step beside the action embedding.
__global__ void __launch_bounds__(256) vla_fill_time_kernel(float* __restrict__ cat, int ld, int off, const float* __restrict__ emb,
                                                           int width, __nv_bfloat16* __restrict__ cat16) {
    pdl_launch_dependents();
    pdl_wait();
    float* d = cat + (size_t)blockIdx.x * ld + off;
    for (int i = threadIdx.x; i < width; i += 256) d[i] = emb[i];
    if (cat16 != nullptr) {                 // bf16 copy with the same layout
        __nv_bfloat16* d16 = cat16 + (size_t)blockIdx.x * ld + off;
        for (int i = threadIdx.x; i < width; i += 256) d16[i] = __float2bfloat16_rn(emb[i]);
    }
}

// y (fp32 rows) = float(x) of bf16 rows -- the final expert norm output for the fp32 output projection.
__global__ void __launch_bounds__(256) vla_bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ y, int n) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i < n) y[i] = __bfloat162float(x[i]);
}

}  // namespace efm
