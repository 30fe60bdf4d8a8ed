// C[M, N] = x[M, K] . W[N, K]^T for M <= 64 rows (the action expert's 50-row products): the weights
// are streamed exactly once, 8 rows per warp as 128-bit loads, and multiplied on mma.sync m16n8k16
// tiles against the activation rows, which every warp reads straight from L1 / L2 (they are a few
// hundred KB at most).  A 128 x 256 tcgen05 tile is the wrong tool here: 50 / 128 of it is filled and a
// block that owns a single tile cannot overlap its epilogue.
//
// Work split: an 8-column tile of the output per group of warps (8 warps / TILES tiles per block); the
// warps of a group take the 32-wide k-chunks round-robin and their partial 64 x 8 tiles are summed in
// shared memory in warp order (fixed order: results do not depend on timing).
// RMSNorm in front of a product costs nothing extra (NORM variants): the norm weight is folded into W when the
// weights are loaded, the rows' sums of squares fall out of the activation vectors the warps load anyway, and the
// 1 / rms factor is applied to the finished 64 x 8 tile.
// k-permutation: inside a 32-wide chunk lane t (= lane % 4) owns the 8 consecutive k values 8t .. 8t+7 of
// its row, for both operands, and feeds them to two k16 MMA steps; a dot product does not care in which
// order k is visited as long as both operands agree.
#pragma once
#include "common.cuh"

namespace efm {

enum class SkinnyEpi : int { Bf16 = 0, Residual = 1, SwiGlu = 2, QkvRope = 3 };

struct SkinnyParams {
    const __nv_bfloat16* x;   // [M, K], row stride ldx (elements, multiple of 8)
    const __nv_bfloat16* W;   // [N, K] row-major, K % 8 == 0
    __nv_bfloat16* C;         // Bf16: [M, N]; SwiGlu: [M, N / 2] = silu(gate) * up, W rows interleaved 64 gate | 64 up
    float* Cf;                // Residual: [M, N] fp32, accumulated into
    int M, N, K, ldx;
    // NORM variants: x holds the bf16 copy of the un-normalised residual rows and W already carries the RMSNorm weight
    // (W'[n][k] = W[n][k] * w[k]); the kernel sums x^2 per row on the way and scales its results by
    // rsqrt(mean(x^2) + eps):  rmsnorm(x) . W^T  =  inv_rms(row) * (x . W'^T)
    float eps = 0.f;
    // Residual: when set, the new residual value is also stored as bf16 here ([M, N]) for the next NORM product
    __nv_bfloat16* x16_out = nullptr;
    // Bf16 and Residual: bias[N] added to the sum (nullptr: none); Bf16: act 1 = SiLU; Residual: assign 1 = the fp32
    // destination is overwritten (sum + bias) instead of accumulated into
    const __nv_bfloat16* bias = nullptr;
    int act = 0, assign = 0;
    // QkvRope (head_dim 64): columns are q heads | k heads | v heads; q and k get the rotate-half RoPE at position
    // pos0 + row (inverse frequencies theta^(-2i/64)) on the bf16-rounded projections; q goes to C [M, N] in place
    // of its columns, rotated k and v of row r to kv_out row kv_row0 + r ([.., kv_stride]: k | v) when kv_out is set
    int q_heads = 0, kv_heads = 0, pos0 = 0;
    float theta = 0.f;
    __nv_bfloat16* kv_out = nullptr;
    int kv_stride = 0, kv_row0 = 0;
};

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

constexpr int kSkinnyThreads = 256;

// W[n][k] *= w[k] (bf16, one rounding): folds an RMSNorm weight into the product that follows the norm.
__global__ void __launch_bounds__(256) fold_norm_weight_kernel(__nv_bfloat16* __restrict__ W, const __nv_bfloat16* __restrict__ w, size_t rows,
                                                              int K) {
    const size_t total = rows * (size_t)K;
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (size_t)gridDim.x * 256)
        W[i] = __float2bfloat16_rn(__bfloat162float(W[i]) * __bfloat162float(w[i % (size_t)K]));
}

// TILES: 8-column tiles per block (1 or 2; SwiGlu needs 2: a gate tile and its up tile; QkvRope needs 2: a tile and
// the tile 32 columns further in the same head).
// NWARPS: warps per block (8, or 16 for long K so that a warp's share of the k-chunks fits one batch of requests).
template <SkinnyEpi EPI, int TILES, bool NORM = false, int NWARPS = 8>
__global__ void __launch_bounds__(NWARPS * 32) skinny_gemm_kernel(const SkinnyParams p) {
    constexpr int GROUP = NWARPS / TILES;                  // warps per tile
    constexpr int BATCH = 4;                               // weight vectors requested ahead per warp
    __shared__ float red[NWARPS][64][8];
    __shared__ float ssq[NORM ? NWARPS : 1][64];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    pdl_launch_dependents();
    pdl_wait();            // no-ops unless launched with programmatic stream serialization
    const int tile = warp / GROUP, j = warp % GROUP;
    // first output column (in W's row numbering) of this warp's tile
    int n0;
    if (EPI == SkinnyEpi::SwiGlu) {
        const int blk = blockIdx.x >> 3, j0 = (blockIdx.x & 7) * 8;
        n0 = blk * 128 + tile * 64 + j0;
    } else if (EPI == SkinnyEpi::QkvRope) {
        n0 = (blockIdx.x >> 2) * 64 + (blockIdx.x & 3) * 8 + tile * 32;      // a column tile and its rotation partner
    } else {
        n0 = (blockIdx.x * TILES + tile) * 8;
    }
    const bool tile_ok = n0 < p.N;                          // N % 8 == 0
    float acc[4][4];
#pragma unroll
    for (int mt = 0; mt < 4; ++mt)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[mt][e] = 0.f;
    float ss[4][2];                                         // NORM: sum of squares of rows 16 mt + g (+ 8) over this lane's k
#pragma unroll
    for (int mt = 0; mt < 4; ++mt) ss[mt][0] = ss[mt][1] = 0.f;
    auto sq8 = [](const uint4& v) {
        float a = 0.f;
        const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float lo = __uint_as_float(u[e] << 16), hi = __uint_as_float(u[e] & 0xffff0000u);
            a = fmaf(lo, lo, a);
            a = fmaf(hi, hi, a);
        }
        return a;
    };

    if (tile_ok) {
        const int nchunks = (p.K + 31) >> 5;
        const __nv_bfloat16* wrow = p.W + (size_t)(n0 + g) * p.K + 8 * t;
        const __nv_bfloat16* xcol = p.x + 8 * t;
        for (int c0 = j; c0 < nchunks; c0 += GROUP * BATCH) {
            uint4 w[BATCH];
#pragma unroll
            for (int i = 0; i < BATCH; ++i) {
                const int k0 = (c0 + i * GROUP) << 5;
                w[i] = (k0 + 8 * t + 8 <= p.K) ? ld_stream16(wrow + k0) : make_uint4(0u, 0u, 0u, 0u);   // also false past the last chunk
            }
            // two chunks at a time: all sixteen activation vectors are requested before the first MMA needs one, so a
            // batch costs two memory round trips instead of one per m-tile (rows >= M and k >= K read as zeros)
#pragma unroll
            for (int i = 0; i < BATCH; i += 2) {
                if (((c0 + i * GROUP) << 5) >= p.K) break;
                uint4 xa[2][4], xb[2][4];
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const int k0 = (c0 + (i + u) * GROUP) << 5;
                    const bool kin = k0 + 8 * t + 8 <= p.K;
#pragma unroll
                    for (int mt = 0; mt < 4; ++mt) {
                        const int r0 = 16 * mt + g, r1 = r0 + 8;
                        xa[u][mt] = (kin && r0 < p.M) ? __ldg(reinterpret_cast<const uint4*>(xcol + (size_t)r0 * p.ldx + k0)) : make_uint4(0u, 0u, 0u, 0u);
                        xb[u][mt] = (kin && r1 < p.M) ? __ldg(reinterpret_cast<const uint4*>(xcol + (size_t)r1 * p.ldx + k0)) : make_uint4(0u, 0u, 0u, 0u);
                    }
                }
                if (NORM) {
#pragma unroll
                    for (int u = 0; u < 2; ++u)
#pragma unroll
                        for (int mt = 0; mt < 4; ++mt) { ss[mt][0] += sq8(xa[u][mt]); ss[mt][1] += sq8(xb[u][mt]); }
                }
#pragma unroll
                for (int u = 0; u < 2; ++u)
#pragma unroll
                    for (int mt = 0; mt < 4; ++mt) {
                        mma_bf16_16816(acc[mt], xa[u][mt].x, xb[u][mt].x, xa[u][mt].y, xb[u][mt].y, w[i + u].x, w[i + u].y);
                        mma_bf16_16816(acc[mt], xa[u][mt].z, xb[u][mt].z, xa[u][mt].w, xb[u][mt].w, w[i + u].z, w[i + u].w);
                    }
            }
        }
    }
    // partial tiles -> shared memory: accumulator (row g / g + 8 of m-tile mt, columns 2t, 2t + 1)
#pragma unroll
    for (int mt = 0; mt < 4; ++mt) {
        *reinterpret_cast<float2*>(&red[warp][16 * mt + g][2 * t]) = make_float2(acc[mt][0], acc[mt][1]);
        *reinterpret_cast<float2*>(&red[warp][16 * mt + g + 8][2 * t]) = make_float2(acc[mt][2], acc[mt][3]);
    }
    if (NORM) {          // lanes t = 0..3 of a row hold disjoint k: add them, one value per (warp, row)
#pragma unroll
        for (int mt = 0; mt < 4; ++mt)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float v = ss[mt][h];
                v += __shfl_xor_sync(0xffffffffu, v, 1);
                v += __shfl_xor_sync(0xffffffffu, v, 2);
                if (t == 0) ssq[NORM ? warp : 0][16 * mt + g + 8 * h] = v;
            }
    }
    __syncthreads();
    // 64 x 8 outputs per tile, 4 consecutive columns per thread
    const int idx = tid & 127, row = idx >> 1, c4 = (idx & 1) * 4;
    auto tile_sum = [&](int tl, float (&s)[4]) {
        s[0] = s[1] = s[2] = s[3] = 0.f;
#pragma unroll
        for (int wv = 0; wv < GROUP; ++wv) {
            const float4 v = *reinterpret_cast<const float4*>(&red[tl * GROUP + wv][row][c4]);
            s[0] += v.x; s[1] += v.y; s[2] += v.z; s[3] += v.w;
        }
    };
    if (row >= p.M) return;
    float inv = 1.0f;
    if (NORM) {          // the warps of tile group 0 cover every k exactly once
        float tot = 0.f;
#pragma unroll
        for (int wv = 0; wv < GROUP; ++wv) tot += ssq[NORM ? wv : 0][row];
        inv = rsqrtf(tot / (float)p.K + p.eps);
    }
    if (EPI == SkinnyEpi::SwiGlu) {
        if (tid >= 128) return;
        const int blk = blockIdx.x >> 3, j0 = (blockIdx.x & 7) * 8;
        if (blk * 128 + j0 >= p.N) return;
        float gt[4], up[4];
        tile_sum(0, gt);
        tile_sum(1, up);
        float o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) { const float gv = gt[e] * inv, uv = up[e] * inv; o[e] = gv / (1.0f + __expf(-gv)) * uv; }
        __nv_bfloat16* dst = p.C + (size_t)row * (p.N >> 1) + blk * 64 + j0 + c4;
        *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16(o[0], o[1]), pack_bf16(o[2], o[3]));
    } else if (EPI == SkinnyEpi::QkvRope) {
        if (tid >= 128) return;
        const int head = blockIdx.x >> 2, f0 = (blockIdx.x & 3) * 8 + c4;    // f0: index inside the first half of the head
        if (head * 64 >= p.N) return;
        float x1[4], x2[4];
        tile_sum(0, x1);
        tile_sum(1, x2);
        const bool rotate = head < p.q_heads + p.kv_heads;
        float o1[4], o2[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float a = __bfloat162float(__float2bfloat16_rn(x1[e] * inv)), b = __bfloat162float(__float2bfloat16_rn(x2[e] * inv));
            if (rotate) {
                float sn, cs;
                sincosf((float)(p.pos0 + row) * powf(p.theta, -(float)(2 * (f0 + e)) / 64.0f), &sn, &cs);
                o1[e] = a * cs - b * sn;
                o2[e] = b * cs + a * sn;
            } else {
                o1[e] = a;
                o2[e] = b;
            }
        }
        __nv_bfloat16* dst;
        if (head < p.q_heads || p.kv_out == nullptr) dst = p.C + (size_t)row * p.N + head * 64 + f0;
        else dst = p.kv_out + (size_t)(p.kv_row0 + row) * p.kv_stride + (head - p.q_heads) * 64 + f0;   // k heads, then v heads
        *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16(o1[0], o1[1]), pack_bf16(o1[2], o1[3]));
        *reinterpret_cast<uint2*>(dst + 32) = make_uint2(pack_bf16(o2[0], o2[1]), pack_bf16(o2[2], o2[3]));
    } else {
        const int tl = tid >> 7;
        if (tl >= TILES) return;
        const int n = (blockIdx.x * TILES + tl) * 8 + c4;
        if (n >= p.N) return;
        float s[4];
        tile_sum(tl, s);
        if (p.bias != nullptr) {
#pragma unroll
            for (int e = 0; e < 4; ++e) s[e] += __bfloat162float(p.bias[n + e]);
        }
        if (EPI == SkinnyEpi::Bf16 && p.act == 1) {
#pragma unroll
            for (int e = 0; e < 4; ++e) s[e] = s[e] / (1.0f + __expf(-s[e]));
        }
        if (EPI == SkinnyEpi::Residual) {
            float4* dst = reinterpret_cast<float4*>(p.Cf + (size_t)row * p.N + n);
            const float4 old = p.assign ? make_float4(0.f, 0.f, 0.f, 0.f) : *dst;
            const float4 nv = make_float4(old.x + s[0], old.y + s[1], old.z + s[2], old.w + s[3]);
            *dst = nv;
            if (p.x16_out != nullptr)
                *reinterpret_cast<uint2*>(p.x16_out + (size_t)row * p.N + n) = make_uint2(pack_bf16(nv.x, nv.y), pack_bf16(nv.z, nv.w));
        } else {
            *reinterpret_cast<uint2*>(p.C + (size_t)row * p.N + n) = make_uint2(pack_bf16(s[0], s[1]), pack_bf16(s[2], s[3]));
        }
    }
}

}  // namespace efm
