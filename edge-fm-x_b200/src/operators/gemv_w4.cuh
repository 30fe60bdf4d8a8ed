// Batch-1 GEMV over group-wise INT4 weights (W4A16) for the decode step: the same prologues and epilogues as the
// bf16 kernel (gemv.cuh), a quarter of the weight bytes.  Replaces the reference's INT4 decode kernel
// (src/operators/kernels/int4_groupwise_gemm/int4WoQGemvCuda.cu:93-253: group size 128, fp16 scales
// [K / 128, N], fp16 products).
//
// Weight layout in HBM (built once at load time by w4_repack_kernel from the checkpoint's qweight [N/2, K] /
// scaling_factors [K/128, N]):
//   Wq     [n_items][K] bytes: byte k of item i = nibble(row r0(i), k) | nibble(row r1(i), k) << 4, nibble = q + 8,
//          (r0, r1) being the row pair the epilogue consumes together (rotary partners, gate / up, neighbours);
//   scales [n_items][K / 128] half2 = (scale of r0, scale of r1);  w[r][k] = q[r][k] * scale[k / 128][r].
// Bound: HBM at K / 2 bytes per row, with about 1.9 issue slots per weight for the nibble -> fp16 conversion, which
// is why the conversion uses the exponent trick on two weights at a time:
//   (word & 0x000F000F) | 0x64006400 = half2(1024 + n_a, 1024 + n_b)            -> minus 1032 = (q_a, q_b)
//   (word & 0x00F000F0) | 0x64006400 = half2(1024 + 16 n_a, 1024 + 16 n_b)      -> times 1/16 minus 72 = (q_a, q_b)
// Products and the sum over one 16-column chunk stay in fp16 (as the reference's kernel keeps its whole row sum);
// chunks are scaled and accumulated in fp32.  Activations are staged as fp16 pairs in the order the conversion
// produces the weights: per 4 columns (x0, x2), (x1, x3).
//
// Schedule: `ks` warps share one row pair (K split over warps, as in the bf16 kernel); a warp walks its (row pair,
// 16-byte chunk) slots in batches of 16 loads in flight.
#pragma once
#include <cuda_fp16.h>

#include "gemv.cuh"

namespace efm {

constexpr int kW4Group = 128;     // columns per scale
constexpr int kW4Batch = 6;       // 16-byte loads (+ their scale words) per buffer; two buffers alternate, so the next
                                  // batch is in flight while this one is converted (the conversion costs about as
                                  // much time as the loads' latency, unlike the bf16 kernel's)

struct GemvW4Params {
    GemvParams g;                 // prologue / epilogue fields; g.W unused, g.N / g.K / g.n_items as for bf16
    const uint8_t* Wq;            // [n_items][K]
    const __half2* scales;        // [n_items][K / 128]
    int swiglu_half;              // SwiGlu: rows of the gate block (item i = gate row i, up row i)
};

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));     // (a & mask) | orv
    return r;
}

// 4 bytes = 4 columns x 2 rows of nibbles against the matching activation pairs x02 = (x0, x2), x13 = (x1, x3).
__device__ __forceinline__ void w4_dot_word(uint32_t w, __half2 x02, __half2 x13, __half2& acc0, __half2& acc1) {
    const __half2 k1032 = __halves2half2(__ushort_as_half(0x6408), __ushort_as_half(0x6408));      // 1032
    const __half2 k16th = __halves2half2(__ushort_as_half(0x2C00), __ushort_as_half(0x2C00));      // 1 / 16
    const __half2 km72 = __halves2half2(__ushort_as_half(0xD480), __ushort_as_half(0xD480));       // -72
    const uint32_t t = w >> 8;
    uint32_t lo02 = lop3_and_or(w, 0x000F000Fu, 0x64006400u), hi02 = lop3_and_or(w, 0x00F000F0u, 0x64006400u);
    uint32_t lo13 = lop3_and_or(t, 0x000F000Fu, 0x64006400u), hi13 = lop3_and_or(t, 0x00F000F0u, 0x64006400u);
    const __half2 q0a = __hsub2(*reinterpret_cast<__half2*>(&lo02), k1032);
    const __half2 q0b = __hsub2(*reinterpret_cast<__half2*>(&lo13), k1032);
    const __half2 q1a = __hfma2(*reinterpret_cast<__half2*>(&hi02), k16th, km72);
    const __half2 q1b = __hfma2(*reinterpret_cast<__half2*>(&hi13), k16th, km72);
    acc0 = __hfma2(q0a, x02, acc0);
    acc0 = __hfma2(q0b, x13, acc0);
    acc1 = __hfma2(q1a, x02, acc1);
    acc1 = __hfma2(q1b, x13, acc1);
}

// fp32 activations [K] (staged by gemv_stage) -> fp16 pairs in conversion order: per 16-column chunk c two uint4,
// words (x[4j], x[4j+2]), (x[4j+1], x[4j+3]) for j = 0..3.  The first uint4 of every chunk (j = 0, 1) lives in
// xh[c], the second (j = 2, 3) in xh[K / 16 + c]: consecutive lanes read consecutive 16-byte words (no bank conflicts).
__device__ __forceinline__ void w4_permute_activations(const float* xs, uint4* xh, int K) {
    const int nq = K >> 2;      // groups of 4 columns
    const int nch = K >> 4;
    uint32_t* out = reinterpret_cast<uint32_t*>(xh);
    for (int q = threadIdx.x; q < nq; q += blockDim.x) {
        const float4 v = reinterpret_cast<const float4*>(xs)[q];
        const __half2 a = __floats2half2_rn(v.x, v.z), b = __floats2half2_rn(v.y, v.w);
        const int c = q >> 2, j = q & 3;
        uint32_t* dst = out + ((j >> 1) * nch + c) * 4 + (j & 1) * 2;
        dst[0] = *reinterpret_cast<const uint32_t*>(&a);
        dst[1] = *reinterpret_cast<const uint32_t*>(&b);
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

// Shared memory: the bf16 kernel's layout (gemv_smem_bytes) followed by the fp16 activation pairs (2 K bytes).
inline size_t gemv_w4_smem_bytes(int K) { return gemv_smem_bytes(K) + (size_t)K * 2 + 16; }

template <Epi EPI>
__global__ void __launch_bounds__(kGemvThreads, 1) gemv_w4_kernel(const GemvW4Params p, const int ks) {
    extern __shared__ __align__(16) unsigned char gemv_smem[];
    __shared__ float bv[kGemvWarps];
    __shared__ int bi[kGemvWarps];
    const GemvParams& g = p.g;
    const int K = g.K;
    const unsigned int xbytes = gemv_xbytes(K);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    float best_v = -INFINITY;
    int best_i = 0x7fffffff;

    pdl_launch_dependents();
    // ---- static schedule ------------------------------------------------------------------------------
    const int gp = kGemvWarps / ks, gi = warp / ks, wk = warp % ks;
    const int nch = K >> 4;                                   // 16-byte chunks per row pair
    const int stride = ks * 32;
    const int cpl = (nch + stride - 1) / stride;              // chunk slots per lane and row pair
    const int ig0 = blockIdx.x * gp + gi, ig_stride = gridDim.x * gp;
    const int n_my = ig0 < g.n_items ? (g.n_items - ig0 + ig_stride - 1) / ig_stride : 0;
    const int total = n_my * cpl;                             // (row pair, chunk slot) slots of this lane
    const int n_groups = K / kW4Group;

    uint4 buf_a[kW4Batch], buf_b[kW4Batch];
    uint32_t sc_a[kW4Batch], sc_b[kW4Batch];                  // the chunks' scale pairs travel with them (no dependent load later)
    auto load_batch = [&](uint4 (&buf)[kW4Batch], uint32_t (&sbuf)[kW4Batch], const int t0) {
        if (t0 >= total) return;
        int j = t0 / cpl, jc = t0 - j * cpl;                  // one division per batch, then counters
#pragma unroll
        for (int s = 0; s < kW4Batch; ++s) {
            if (t0 + s < total) {
                const int c = jc * stride + wk * 32 + lane;
                if (c < nch) {
                    const int ig = ig0 + j * ig_stride;
                    buf[s] = ld_stream(p.Wq + (size_t)ig * K + (size_t)c * 16);
                    sbuf[s] = __ldg(reinterpret_cast<const uint32_t*>(p.scales) + (size_t)ig * n_groups + (c >> 3));
                }
            }
            if (++jc == cpl) { jc = 0; ++j; }
        }
    };
    load_batch(buf_a, sc_a, 0);                               // weights do not depend on the previous kernel
    if (g.prologue != kProPlain) {
        uint4* gs = reinterpret_cast<uint4*>(gemv_smem + xbytes);
        for (int c = tid; c < (K >> 3); c += kGemvThreads) gs[c] = ld_cached(g.norm_w + (size_t)c * 8);
    }
    pdl_wait();

    gemv_stage(g, K >> 3, gemv_smem, xbytes);
    uint4* xh = reinterpret_cast<uint4*>(gemv_smem + ((gemv_smem_bytes(K) + 15) & ~(size_t)15));
    w4_permute_activations(reinterpret_cast<const float*>(gemv_smem), xh, K);
    __syncthreads();

    float* red = reinterpret_cast<float*>(gemv_smem + xbytes + gemv_wbytes(K));
    float acc0 = 0.f, acc1 = 0.f;
    int parity = 0;
    int cj = 0, cjc = 0;                                      // compute-side counters: row pair index, chunk slot
    auto compute_batch = [&](const uint4 (&buf)[kW4Batch], const uint32_t (&sbuf)[kW4Batch], const int t0) {
#pragma unroll
        for (int s = 0; s < kW4Batch; ++s) {
            if (t0 + s >= total) break;
            const int jc = cjc;
            const int ig = ig0 + cj * ig_stride;
            const int c = jc * stride + wk * 32 + lane;
            if (++cjc == cpl) { cjc = 0; ++cj; }
            if (c < nch) {
                const __half2 sc2 = *reinterpret_cast<const __half2*>(&sbuf[s]);
                const uint4 xa = xh[c], xb = xh[nch + c];
                __half2 h0 = __float2half2_rn(0.f), h1 = __float2half2_rn(0.f);
                w4_dot_word(buf[s].x, *reinterpret_cast<const __half2*>(&xa.x), *reinterpret_cast<const __half2*>(&xa.y), h0, h1);
                w4_dot_word(buf[s].y, *reinterpret_cast<const __half2*>(&xa.z), *reinterpret_cast<const __half2*>(&xa.w), h0, h1);
                w4_dot_word(buf[s].z, *reinterpret_cast<const __half2*>(&xb.x), *reinterpret_cast<const __half2*>(&xb.y), h0, h1);
                w4_dot_word(buf[s].w, *reinterpret_cast<const __half2*>(&xb.z), *reinterpret_cast<const __half2*>(&xb.w), h0, h1);
                const float2 f0 = __half22float2(h0), f1 = __half22float2(h1), sf = __half22float2(sc2);
                acc0 = fmaf(f0.x + f0.y, sf.x, acc0);
                acc1 = fmaf(f1.x + f1.y, sf.y, acc1);
            }
            if (jc != cpl - 1) continue;
            // row pair complete
            float t0s = warp_sum(acc0), t1s = warp_sum(acc1);
            acc0 = 0.f;
            acc1 = 0.f;
            if (ks > 1) {
                float* buf2 = red + parity * kGemvWarps * 2;
                if (lane == 0) { buf2[warp * 2] = t0s; buf2[warp * 2 + 1] = t1s; }
                group_barrier(1 + gi, ks * 32);
                if (wk == 0) {
                    t0s = 0.f;
                    t1s = 0.f;
                    for (int w = 0; w < ks; ++w) { t0s += buf2[(gi * ks + w) * 2]; t1s += buf2[(gi * ks + w) * 2 + 1]; }
                }
                parity ^= 1;
            }
            if (wk == 0 && lane == 0) {
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
        load_batch(buf_b, sc_b, t0 + kW4Batch);
        compute_batch(buf_a, sc_a, t0);
        load_batch(buf_a, sc_a, t0 + 2 * kW4Batch);
        compute_batch(buf_b, sc_b, t0 + kW4Batch);
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
    uint8_t* out_q;               // [n_items][K]
    __half2* out_s;               // [n_items][K / 128]
};

__device__ __forceinline__ void w4_locate(const W4RepackParams& p, int row, int& src, int& local) {
    src = 0;
    for (int s = 1; s < p.n_src; ++s)
        if (row >= p.row0[s]) src = s;
    local = row - p.row0[src];
}

template <int UNUSED = 0>      // a template so that every translation unit including this header may hold a copy
__global__ void __launch_bounds__(256) w4_repack_kernel(const W4RepackParams p) {
    const int item = blockIdx.x;
    int r0, r1;
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
    int s0, l0, s1, l1;
    w4_locate(p, r0, s0, l0);
    w4_locate(p, r1, s1, l1);
    const uint8_t* a = p.q[s0] + (size_t)(l0 >> 1) * p.K;
    const uint8_t* b = p.q[s1] + (size_t)(l1 >> 1) * p.K;
    const int sh0 = (l0 & 1) * 4, sh1 = (l1 & 1) * 4;
    for (int k = threadIdx.x; k < p.K; k += 256)
        p.out_q[(size_t)item * p.K + k] = (uint8_t)(((a[k] >> sh0) & 0xF) | (((b[k] >> sh1) & 0xF) << 4));
    const int ng = p.K / kW4Group;
    for (int gidx = threadIdx.x; gidx < ng; gidx += 256) {
        float f0, f1;
        if (p.s_is_bf16[s0]) f0 = __bfloat162float(static_cast<const __nv_bfloat16*>(p.s[s0])[(size_t)gidx * p.rows[s0] + l0]);
        else f0 = __half2float(static_cast<const __half*>(p.s[s0])[(size_t)gidx * p.rows[s0] + l0]);
        if (p.s_is_bf16[s1]) f1 = __bfloat162float(static_cast<const __nv_bfloat16*>(p.s[s1])[(size_t)gidx * p.rows[s1] + l1]);
        else f1 = __half2float(static_cast<const __half*>(p.s[s1])[(size_t)gidx * p.rows[s1] + l1]);
        p.out_s[(size_t)item * ng + gidx] = __floats2half2_rn(f0, f1);
    }
}

}  // namespace efm
