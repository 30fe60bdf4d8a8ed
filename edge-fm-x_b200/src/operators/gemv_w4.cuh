// Batch-1 GEMV over group-wise INT4 weights (W4A16) for the decode step: the same prologues and epilogues as the
// bf16 kernel (gemv.cuh), a quarter of the weight bytes.  Replaces the reference's INT4 decode kernel
// (src/operators/kernels/int4_groupwise_gemm/int4WoQGemvCuda.cu:93-253: group size 128, fp16 scales
// [K / 128, N], fp16 products).
//
// A CUDA-core version of this kernel (nibble pairs widened to fp16 and multiplied with HFMA2) needs about 4 issue
// slots per weight byte and ran at a third of the HBM bandwidth at the 7B shape's widths.  This one feeds the
// widened nibbles to mma.sync m16n8k16 (f16 inputs, fp32 accumulators), which takes the multiplies off the issue
// slots, and never subtracts the nibble's offset per weight:
//   (word & 0x000F000F) | 0x64006400 = half2(1024 + n_a, 1024 + n_b)          (first row of a pair)
//   (word & 0x00F000F0) | 0x64006400 = half2(1024 + 16 n_a, 1024 + 16 n_b)    (second row of a pair)
// go into the A fragment as they are; the fp32 accumulator then holds sum((1024 + n) x) resp. sum((1024 + 16 n) x)
// over one 128-column scale group (products of two fp16 values are exact in fp32), and with Sx = sum of the group's
// fp16 activations
//   sum(q x) = acc - 1032 Sx          resp.     acc / 16 - 72 Sx            (q = n - 8)
// is scaled by the group's scale and added to the row's fp32 result: 5 issue slots + 1 mma per 8 weights of a lane.
// The B operand carries the activation vector in all 8 columns, so every column of the accumulator is the result.
//
// Weight layout in HBM (built once at load time by w4_repack_kernel from the checkpoint's qweight [N/2, K] /
// scaling_factors [K/128, N]); item i = the row pair (r0, r1) the epilogue consumes together (rotary partners,
// gate / up, neighbours), 8 items = one 16-row mma tile (A rows g and g + 8 = r0 and r1 of item 8 T + g):
//   Wq     [tile T][64-column chunk c][lane = 4 g + t][4 words s]: word s serves the k16 step at column
//          k0 = 64 c + 16 s; its bytes 0..3 hold columns k0 + 2t, k0 + 2t + 8, k0 + 2t + 1, k0 + 2t + 9, each byte =
//          nibble(r0) | nibble(r1) << 4, nibble = q + 8.  One 16-byte load per lane and chunk, 512 contiguous bytes
//          per warp; 8 K bytes per tile.  Items past n_items (last tile) are stored as q = 0 with scale 0.
//   scales [item][K / 128] half2 = (scale of r0, scale of r1);  w[r][k] = q[r][k] * scale[k / 128][r].
// Bound: HBM at K / 2 bytes per row.
//
// Schedule: `ks` warps share one tile (the 128-column groups of K go round-robin over them); a lane keeps
// kW4Batch groups (2 x 16 bytes + the scale word each) in flight.
#pragma once
#include <cuda_fp16.h>

#include "gemv.cuh"

namespace efm {

constexpr int kW4Group = 128;     // columns per scale = two 64-column chunks
constexpr int kW4Batch = 3;       // groups per load buffer (2 x 16 bytes + the scale word each); two buffers alternate, so
                                  // the next batch is in flight while this one goes through the tensor cores

struct GemvW4Params {
    GemvParams g;                 // prologue / epilogue fields; g.W unused, g.N / g.K / g.n_items as for bf16
    const uint8_t* Wq;            // [ceil(n_items / 8)][K / 64][32][16]
    const __half2* scales;        // [ceil(n_items / 8) * 8][K / 128]
    int swiglu_half;              // SwiGlu: rows of the gate block (item i = gate row i, up row i)
};

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));     // (a & mask) | orv
    return r;
}

// One k16 step: the lane's weight word -> A fragment (rows g / g + 8, columns 2t, 2t+1 / 2t+8, 2t+9), times the
// activation fragment (b0, b1), accumulated into c (c[0] = c[1] = row g, c[2] = c[3] = row g + 8).
__device__ __forceinline__ void w4_mma_word(uint32_t w, uint32_t b0, uint32_t b1, float (&c)[4]) {
    const uint32_t u = w >> 8;
    const uint32_t a0 = lop3_and_or(w, 0x000F000Fu, 0x64006400u), a1 = lop3_and_or(w, 0x00F000F0u, 0x64006400u);
    const uint32_t a2 = lop3_and_or(u, 0x000F000Fu, 0x64006400u), a3 = lop3_and_or(u, 0x00F000F0u, 0x64006400u);
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// fp32 activations [K] (staged by gemv_stage) -> B fragments: per 64-column chunk c and t = 0..3 two uint4,
// words (b0, b1) of the k16 steps 0, 1 and 2, 3: b0 = (x[k0 + 2t], x[k0 + 2t + 1]), b1 = (x[k0 + 2t + 8], x[k0 + 2t + 9]);
// and sx[group] = sum of the group's 128 activations as rounded to fp16.
__device__ __forceinline__ void w4_stage_activations(const float* xs, uint4* xh, float* sx, int K) {
    uint32_t* out = reinterpret_cast<uint32_t*>(xh);
    for (int i = threadIdx.x; i < (K >> 2); i += blockDim.x) {
        const int c = i >> 4, t = (i >> 2) & 3, s = i & 3;
        const int k0 = 64 * c + 16 * s + 2 * t;
        const float2 lo = *reinterpret_cast<const float2*>(xs + k0), hi = *reinterpret_cast<const float2*>(xs + k0 + 8);
        const __half2 a = __floats2half2_rn(lo.x, lo.y), b = __floats2half2_rn(hi.x, hi.y);
        out[(c * 4 + t) * 8 + 2 * s] = *reinterpret_cast<const uint32_t*>(&a);
        out[(c * 4 + t) * 8 + 2 * s + 1] = *reinterpret_cast<const uint32_t*>(&b);
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int gidx = warp; gidx < K / kW4Group; gidx += (int)(blockDim.x >> 5)) {
        const float4 v = reinterpret_cast<const float4*>(xs)[gidx * 32 + lane];
        float t = (__half2float(__float2half_rn(v.x)) + __half2float(__float2half_rn(v.y))) +
                  (__half2float(__float2half_rn(v.z)) + __half2float(__float2half_rn(v.w)));
        t = warp_sum(t);
        if (lane == 0) sx[gidx] = t;
    }
}

template <Epi EPI>
__device__ __forceinline__ void w4_item_rows(const GemvW4Params& p, int item, int& r0, int& r1) {
    if constexpr (EPI == Epi::SwiGlu) {
        r0 = item;
        r1 = item + p.swiglu_half;
    } else {
        item_rows<EPI>(p.g, item, r0, r1);
    }
}

// Shared memory: the bf16 kernel's layout (gemv_smem_bytes), then the B fragments (2 K bytes), the group sums and the
// cross-warp reduction buffer (two generations x 16 warps x 8 items x 2 rows).
constexpr int kW4RedFloats = 2 * kGemvWarps * 16;
inline size_t gemv_w4_smem_bytes(int K) {
    return gemv_smem_bytes(K) + 16 + (size_t)K * 2 + (((size_t)(K / kW4Group) * 4 + 15) & ~(size_t)15) + kW4RedFloats * sizeof(float);
}

template <Epi EPI>
__global__ void __launch_bounds__(kGemvThreads, 1) gemv_w4_kernel(const GemvW4Params p, const int ks) {
    extern __shared__ __align__(16) unsigned char gemv_smem[];
    __shared__ float bv[kGemvWarps];
    __shared__ int bi[kGemvWarps];
    const GemvParams& g = p.g;
    const int K = g.K;
    const unsigned int xbytes = gemv_xbytes(K);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int gq = lane >> 2, tq = lane & 3;
    float best_v = -INFINITY;
    int best_i = 0x7fffffff;

    pdl_launch_dependents();
    // ---- static schedule ------------------------------------------------------------------------------
    const int gp = kGemvWarps / ks, gi = warp / ks, wk = warp % ks;
    const int n_groups = K / kW4Group;
    const int gpw = (n_groups + ks - 1) / ks;                 // groups per warp and tile
    const int n_tiles = (g.n_items + 7) >> 3;
    const int tg0 = blockIdx.x * gp + gi, tg_stride = gridDim.x * gp;
    const int n_my = tg0 < n_tiles ? (n_tiles - tg0 + tg_stride - 1) / tg_stride : 0;
    const int total = n_my * gpw;                             // (tile, group) slots of this warp
    const size_t tile_bytes = (size_t)K * 8;

    uint4 buf_a[kW4Batch][2], buf_b[kW4Batch][2];
    uint32_t sc_a[kW4Batch], sc_b[kW4Batch];                  // the groups' scale pairs travel with them
    auto load_batch = [&](uint4 (&buf)[kW4Batch][2], uint32_t (&sbuf)[kW4Batch], const int t0) {
        if (t0 >= total) return;
        int j = t0 / gpw, jg = t0 - j * gpw;                  // one division per batch, then counters
#pragma unroll
        for (int s = 0; s < kW4Batch; ++s) {
            if (t0 + s < total) {
                const int grp = jg * ks + wk;
                if (grp < n_groups) {
                    const int tile = tg0 + j * tg_stride;
                    const uint8_t* src = p.Wq + (size_t)tile * tile_bytes + (size_t)grp * 1024 + lane * 16;
                    buf[s][0] = ld_stream(src);
                    buf[s][1] = ld_stream(src + 512);
                    sbuf[s] = __ldg(reinterpret_cast<const uint32_t*>(p.scales) + (size_t)(tile * 8 + gq) * n_groups + grp);
                }
            }
            if (++jg == gpw) { jg = 0; ++j; }
        }
    };
    load_batch(buf_a, sc_a, 0);                               // weights do not depend on the previous kernel
    load_batch(buf_b, sc_b, kW4Batch);
    if (g.prologue != kProPlain) {
        uint4* gs = reinterpret_cast<uint4*>(gemv_smem + xbytes);
        for (int c = tid; c < (K >> 3); c += kGemvThreads) gs[c] = ld_cached(g.norm_w + (size_t)c * 8);
    }
    pdl_wait();

    gemv_stage(g, K >> 3, gemv_smem, xbytes);
    unsigned char* extra = gemv_smem + ((gemv_smem_bytes(K) + 15) & ~(size_t)15);
    uint4* xh = reinterpret_cast<uint4*>(extra);
    float* sx = reinterpret_cast<float*>(extra + (size_t)K * 2);
    float* red2 = reinterpret_cast<float*>(extra + (size_t)K * 2 + (((size_t)n_groups * 4 + 15) & ~(size_t)15));
    w4_stage_activations(reinterpret_cast<const float*>(gemv_smem), xh, sx, K);
    __syncthreads();

    float res0 = 0.f, res1 = 0.f;
    int parity = 0;
    int cj = 0, cjg = 0;                                      // compute-side counters: tile index, group slot
    auto compute_batch = [&](const uint4 (&buf)[kW4Batch][2], const uint32_t (&sbuf)[kW4Batch], const int t0) {
#pragma unroll
        for (int s = 0; s < kW4Batch; ++s) {
            if (t0 + s >= total) break;                       // warp-uniform, like every branch around the mma
            const int jg = cjg;
            const int tile = tg0 + cj * tg_stride;
            const int grp = jg * ks + wk;
            if (++cjg == gpw) { cjg = 0; ++cj; }
            if (grp < n_groups) {
                float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};      // two chains: the mma latency overlaps
                const uint4* xp = xh + ((size_t)(2 * grp) * 4 + tq) * 2;
                const uint4 xa0 = xp[0], xb0 = xp[1], xa1 = xp[8], xb1 = xp[9];
                w4_mma_word(buf[s][0].x, xa0.x, xa0.y, c0);
                w4_mma_word(buf[s][1].x, xa1.x, xa1.y, c1);
                w4_mma_word(buf[s][0].y, xa0.z, xa0.w, c0);
                w4_mma_word(buf[s][1].y, xa1.z, xa1.w, c1);
                w4_mma_word(buf[s][0].z, xb0.x, xb0.y, c0);
                w4_mma_word(buf[s][1].z, xb1.x, xb1.y, c1);
                w4_mma_word(buf[s][0].w, xb0.z, xb0.w, c0);
                w4_mma_word(buf[s][1].w, xb1.z, xb1.w, c1);
                const float sxg = sx[grp];
                const float2 sf = __half22float2(*reinterpret_cast<const __half2*>(&sbuf[s]));
                res0 = fmaf(sf.x, fmaf(-1032.f, sxg, c0[0] + c1[0]), res0);
                res1 = fmaf(sf.y, fmaf(c0[2] + c1[2], 0.0625f, -72.f * sxg), res1);
            }
            if (jg != gpw - 1) continue;
            // tile complete for this warp: lanes with t == 0 hold the partial results of item 8 tile + g
            float t0s = res0, t1s = res1;
            res0 = 0.f;
            res1 = 0.f;
            if (ks > 1) {
                float* b2 = red2 + parity * (kGemvWarps * 16);
                if (tq == 0) { b2[(warp * 8 + gq) * 2] = t0s; b2[(warp * 8 + gq) * 2 + 1] = t1s; }
                group_barrier(1 + gi, ks * 32);
                if (wk == 0 && tq == 0) {
                    t0s = 0.f;
                    t1s = 0.f;
                    for (int w = 0; w < ks; ++w) { t0s += b2[((gi * ks + w) * 8 + gq) * 2]; t1s += b2[((gi * ks + w) * 8 + gq) * 2 + 1]; }
                }
                parity ^= 1;
            }
            const int ig = tile * 8 + gq;
            if (wk == 0 && tq == 0 && ig < g.n_items) {
                if constexpr (EPI == Epi::SwiGlu) {
                    const float sl = t0s / (1.0f + expf(-t0s));
                    if (g.yf != nullptr) g.yf[ig] = sl * t1s;
                    else g.y[ig] = __float2bfloat16_rn(sl * t1s);
                } else {
                    item_epilogue<EPI>(g, ig, t0s, t1s, best_v, best_i);
                }
            }
        }
    };
    for (int t0 = 0; t0 < total; t0 += 2 * kW4Batch) {
        compute_batch(buf_a, sc_a, t0);
        load_batch(buf_a, sc_a, t0 + 2 * kW4Batch);
        compute_batch(buf_b, sc_b, t0 + kW4Batch);
        load_batch(buf_b, sc_b, t0 + 3 * kW4Batch);
    }
    if constexpr (EPI == Epi::Logits) gemv_publish_best(g, best_v, best_i, bv, bi);
}

// Checkpoint layout -> kernel layout, once per linear at load time.  Up to three source tensors stacked along the
// rows (q | k | v, gate | up): source s covers the fused rows [row0[s], row0[s] + rows[s]).
struct W4RepackParams {
    const uint8_t* q[3];          // [rows / 2][K]: byte = nibble(row 2r) | nibble(row 2r + 1) << 4, nibble = q + 8
    const void* s[3];             // [K / 128][rows] fp16 or bf16
    int row0[3], rows[3], s_is_bf16[3];
    int n_src, K, n_items;
    int kind;                     // 0: neighbours (2i, 2i + 1); 1: rotary partners (QkvRope); 2: (i, i + half)
    int head_dim, half;
    uint8_t* out_q;               // [ceil(n_items / 8)][K / 64][32][16]
    __half2* out_s;               // [ceil(n_items / 8) * 8][K / 128]
};

__device__ __forceinline__ void w4_locate(const W4RepackParams& p, int row, int& src, int& local) {
    src = 0;
    for (int s = 1; s < p.n_src; ++s)
        if (row >= p.row0[s]) src = s;
    local = row - p.row0[src];
}

// grid = ceil(n_items / 8) * 8 blocks, one per (padded) item.
template <int UNUSED = 0>      // a template so that every translation unit including this header may hold a copy
__global__ void __launch_bounds__(256) w4_repack_kernel(const W4RepackParams p) {
    const int item = blockIdx.x;
    const int ng = p.K / kW4Group;
    const int tile = item >> 3, gq = item & 7;
    uint8_t* dst_tile = p.out_q + (size_t)tile * p.K * 8;
    const bool pad = item >= p.n_items;
    int r0 = 0, r1 = 0;
    if (p.kind == 1) {
        const int half = p.head_dim >> 1, head = item / half, d = item - head * half;
        r0 = head * p.head_dim + d;
        r1 = r0 + half;
    } else if (p.kind == 2) {
        r0 = item;
        r1 = item + p.half;
    } else {
        r0 = 2 * item;
        r1 = r0 + 1;
    }
    int s0 = 0, l0 = 0, s1 = 0, l1 = 0;
    const uint8_t *a = nullptr, *b = nullptr;
    if (!pad) {
        w4_locate(p, r0, s0, l0);
        w4_locate(p, r1, s1, l1);
        a = p.q[s0] + (size_t)(l0 >> 1) * p.K;
        b = p.q[s1] + (size_t)(l1 >> 1) * p.K;
    }
    const int sh0 = (l0 & 1) * 4, sh1 = (l1 & 1) * 4;
    for (int k = threadIdx.x; k < p.K; k += 256) {
        const uint8_t byte = pad ? (uint8_t)0x88 : (uint8_t)(((a[k] >> sh0) & 0xF) | (((b[k] >> sh1) & 0xF) << 4));
        const int c = k >> 6, r = k & 63, s = r >> 4, u = r & 15;
        const int t = (u & 7) >> 1, bsel = (u >> 3) | ((u & 1) << 1);        // bytes: 2t, 2t + 8, 2t + 1, 2t + 9
        dst_tile[((size_t)c * 32 + gq * 4 + t) * 16 + s * 4 + bsel] = byte;
    }
    for (int gidx = threadIdx.x; gidx < ng; gidx += 256) {
        float f0 = 0.f, f1 = 0.f;
        if (!pad) {
            if (p.s_is_bf16[s0]) f0 = __bfloat162float(static_cast<const __nv_bfloat16*>(p.s[s0])[(size_t)gidx * p.rows[s0] + l0]);
            else f0 = __half2float(static_cast<const __half*>(p.s[s0])[(size_t)gidx * p.rows[s0] + l0]);
            if (p.s_is_bf16[s1]) f1 = __bfloat162float(static_cast<const __nv_bfloat16*>(p.s[s1])[(size_t)gidx * p.rows[s1] + l1]);
            else f1 = __half2float(static_cast<const __half*>(p.s[s1])[(size_t)gidx * p.rows[s1] + l1]);
        }
        p.out_s[(size_t)item * ng + gidx] = __floats2half2_rn(f0, f1);
    }
}

}  // namespace efm
