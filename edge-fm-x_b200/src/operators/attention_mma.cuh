// Softmax attention over many query rows on tensor-core tiles (mma.sync m16n8k16, bf16 in, fp32
// accumulate), flash style: the score matrix never leaves registers.
// (reference: the prefill attention of src/operators/attention_op.cu:1305-1338, causal over
//  [fixed prefix | chunk]; the vision tower's bidirectional windowed attention has no counterpart
//  in the reference and follows the published Qwen2.5-VL encoder.)
//
// Each query row i sees the key rows [lo[i], hi[i]).  Without lo/hi the rule is the causal one of
// prefill: [0, kv_offset + i + 1).  One block = 64 or 128 consecutive queries of one head, 4 or 8 warps x 16
// rows; keys and values stream through shared memory in tiles of 64 rows (cp.async, two buffers);
// per tile S = Q K^T (fragments from ldmatrix), online softmax in registers, O += P V (V fragments
// from ldmatrix.trans).  Rows of 16-byte chunks are padded by 16 bytes so that ldmatrix is
// conflict free.  Bound: tensor pipe for long key ranges (4 q D kv flops), otherwise latency.
#pragma once
#include "common.cuh"

namespace efm {

struct SegAttnParams {
    const __nv_bfloat16* q;      // query row i, head h at q + i * q_stride + h * D
    const __nv_bfloat16* k;      // key row j, kv head g at k + j * kv_stride + g * D
    const __nv_bfloat16* v;
    __nv_bfloat16* out;          // out + i * out_stride + h * D
    const int32_t* lo;           // [S] first visible key row (nullptr: causal rule)
    const int32_t* hi;           // [S] one past the last visible key row
    int q_stride, kv_stride, out_stride;
    int S, kv_offset, q_heads, kv_heads;
    float scale;
    // tcgen05 form (attention_tc.cuh) only: number of key / value rows behind k and v (0: the tensor-core-tile kernel of
    // this file)
    int kv_rows;
    const float* sq;             // INT8 variant: scale of each 128-token block and head of q [ceil(S / 128), q_heads] ...
    const float* sk;             // ... and of k [ceil(kv_rows / 128), kv_heads]
    int* error;                  // raised (1) when a bounded pipeline wait of the tcgen05 form gives up; may be null
};

namespace sa {
constexpr int BKV = 64;                                   // key rows per tile
// NW warps per block = 16 * NW query rows (NW 4: short sequences, more blocks; NW 8: long ones, K/V tiles shared
// by twice as many queries and twice the warps per SM)
template <int D> constexpr int row_bytes() { return (D + 8) * 2; }
// PRE = 0: two K / V tile buffers, the next tile streamed in behind the current one.  PRE > 0: room for PRE tiles; all of
// a block's keys are requested at once and the tile loop never waits on memory again (short key ranges, latency-bound).
template <int D, int NW, int PRE = 0> constexpr size_t smem_bytes() { return (size_t)(16 * NW + 2 * (PRE > 0 ? PRE : 2) * BKV) * row_bytes<D>(); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm4_t(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// ROWS rows x D bf16 from global (row stride in elements) into padded shared rows; rows outside
// [row_begin, row_end) are zero filled.
template <int D, int ROWS, int THREADS>
__device__ __forceinline__ void load_tile(uint32_t smem, const __nv_bfloat16* base, int stride, int row0, int row_begin,
                                          int row_end) {
    constexpr int CH = D / 8;
    for (int idx = threadIdx.x; idx < ROWS * CH; idx += THREADS) {
        const int r = idx / CH, ch = idx - r * CH;
        const int row = row0 + r;
        const bool in = row >= row_begin && row < row_end;
        const __nv_bfloat16* src = base + (size_t)(in ? row : row_begin) * stride + ch * 8;
        cp_async16(smem + r * row_bytes<D>() + ch * 16, src, in ? 16 : 0);
    }
}
}  // namespace sa

template <int D, int NW, int PRE = 0>
__global__ void __launch_bounds__(NW * 32) seg_attention_kernel(const SegAttnParams p) {
    using namespace sa;
    pdl_launch_dependents();
    pdl_wait();            // no-ops unless launched with programmatic stream serialization
    constexpr int BQ = 16 * NW, kThreads = 32 * NW;
    constexpr int RB = row_bytes<D>();
    constexpr int KS = D / 16;           // k-steps of Q K^T
    constexpr int DT = D / 8;            // 8-wide output tiles
    extern __shared__ __align__(16) unsigned char seg_attn_smem[];
    __shared__ int s_range[2];
    const uint32_t sq = (uint32_t)__cvta_generic_to_shared(seg_attn_smem);
    constexpr int NBUF = PRE > 0 ? PRE : 2;
    const uint32_t sk0 = sq + BQ * RB, sv0 = sk0 + NBUF * BKV * RB;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int q0 = blockIdx.x * BQ, h = blockIdx.y;
    const int kvh = h / (p.q_heads / p.kv_heads);
    const __nv_bfloat16* kbase = p.k + (size_t)kvh * D;
    const __nv_bfloat16* vbase = p.v + (size_t)kvh * D;

    // key range of the block = union of its queries' ranges
    if (threadIdx.x == 0) { s_range[0] = 0x7fffffff; s_range[1] = 0; }
    __syncthreads();
    if (threadIdx.x < BQ && q0 + threadIdx.x < p.S) {
        const int i = q0 + threadIdx.x;
        const int lo = p.lo != nullptr ? p.lo[i] : 0;
        const int hi = p.hi != nullptr ? p.hi[i] : p.kv_offset + i + 1;
        if (hi > lo) { atomicMin(&s_range[0], lo); atomicMax(&s_range[1], hi); }
    }
    __syncthreads();
    const int kbegin = s_range[0], kend = s_range[1];
    int ntiles = kend > kbegin ? (kend - kbegin + BKV - 1) / BKV : 0;
    if (PRE > 0 && ntiles > PRE) ntiles = PRE;       // never past the buffers; the launcher only picks PRE for ranges that fit

    // per-thread rows: r0 = warp*16 + g, r1 = r0 + 8
    const int i0 = q0 + warp * 16 + g, i1 = i0 + 8;
    int lo0 = 0, hi0 = 0, lo1 = 0, hi1 = 0;
    if (i0 < p.S) { lo0 = p.lo != nullptr ? p.lo[i0] : 0; hi0 = p.hi != nullptr ? p.hi[i0] : p.kv_offset + i0 + 1; }
    if (i1 < p.S) { lo1 = p.lo != nullptr ? p.lo[i1] : 0; hi1 = p.hi != nullptr ? p.hi[i1] : p.kv_offset + i1 + 1; }

    load_tile<D, BQ, kThreads>(sq, p.q + (size_t)h * D, p.q_stride, q0, 0, p.S);
    if (PRE > 0) {
        for (int tl = 0; tl < ntiles; ++tl) {
            load_tile<D, BKV, kThreads>(sk0 + tl * BKV * RB, kbase, p.kv_stride, kbegin + tl * BKV, kbegin, kend);
            load_tile<D, BKV, kThreads>(sv0 + tl * BKV * RB, vbase, p.kv_stride, kbegin + tl * BKV, kbegin, kend);
        }
    } else if (ntiles > 0) {
        load_tile<D, BKV, kThreads>(sk0, kbase, p.kv_stride, kbegin, kbegin, kend);
        load_tile<D, BKV, kThreads>(sv0, vbase, p.kv_stride, kbegin, kbegin, kend);
    }
    cp_async_commit();

    uint32_t qf[KS][4];
    float o[DT][4];
#pragma unroll
    for (int d = 0; d < DT; ++d) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    const float sl2 = p.scale * 1.4426950408889634f;

    for (int it = 0; it < ntiles; ++it) {
        const int buf = PRE > 0 ? it : (it & 1);
        if (PRE > 0) {
            if (it == 0) { cp_async_wait<0>(); __syncthreads(); }
        } else {
            if (it + 1 < ntiles) {
                const int row0 = kbegin + (it + 1) * BKV;
                load_tile<D, BKV, kThreads>(sk0 + (buf ^ 1) * BKV * RB, kbase, p.kv_stride, row0, kbegin, kend);
                load_tile<D, BKV, kThreads>(sv0 + (buf ^ 1) * BKV * RB, vbase, p.kv_stride, row0, kbegin, kend);
            }
            cp_async_commit();
            cp_async_wait<1>();
            __syncthreads();
        }
        if (it == 0) {
#pragma unroll
            for (int ks = 0; ks < KS; ++ks)
                ldsm4(sq + (warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * RB + (ks * 16 + 8 * (lane >> 4)) * 2, qf[ks]);
        }
        const uint32_t sk = sk0 + buf * BKV * RB, sv = sv0 + buf * BKV * RB;
        float s[8][4];
#pragma unroll
        for (int n = 0; n < 8; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                uint32_t b[4];
                ldsm4(sk + (np * 16 + (lane & 7) + 8 * (lane >> 4)) * RB + (ks * 16 + 8 * ((lane >> 3) & 1)) * 2, b);
                mma16816(s[2 * np], qf[ks], b[0], b[1]);
                mma16816(s[2 * np + 1], qf[ks], b[2], b[3]);
            }
        }
        // mask, scale (in log2 units) and running maximum
        const int key0 = kbegin + it * BKV + 2 * t;
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int n = 0; n < 8; ++n) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int key = key0 + n * 8 + e;
                s[n][e] = (key >= lo0 && key < hi0) ? s[n][e] * sl2 : -INFINITY;
                s[n][2 + e] = (key >= lo1 && key < hi1) ? s[n][2 + e] * sl2 : -INFINITY;
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
        // O += P V, 16 keys at a time
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            uint32_t a[4];
            a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int dp = 0; dp < DT / 2; ++dp) {
                uint32_t b[4];
                ldsm4_t(sv + (kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * RB + (dp * 16 + 8 * (lane >> 4)) * 2, b);
                mma16816(o[2 * dp], a, b[0], b[1]);
                mma16816(o[2 * dp + 1], a, b[2], b[3]);
            }
        }
        if (PRE == 0) __syncthreads();          // the next iteration overwrites the other buffer, read one iteration ago
    }
    cp_async_wait<0>();

    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float r0 = l0 > 0.f ? 1.0f / l0 : 0.f, r1 = l1 > 0.f ? 1.0f / l1 : 0.f;
    if (i0 < p.S) {
        __nv_bfloat16* dst = p.out + (size_t)i0 * p.out_stride + (size_t)h * D + 2 * t;
#pragma unroll
        for (int d = 0; d < DT; ++d) *reinterpret_cast<uint32_t*>(dst + d * 8) = pack_bf16(o[d][0] * r0, o[d][1] * r0);
    }
    if (i1 < p.S) {
        __nv_bfloat16* dst = p.out + (size_t)i1 * p.out_stride + (size_t)h * D + 2 * t;
#pragma unroll
        for (int d = 0; d < DT; ++d) *reinterpret_cast<uint32_t*>(dst + d * 8) = pack_bf16(o[d][2] * r1, o[d][3] * r1);
    }
}

}  // namespace efm
