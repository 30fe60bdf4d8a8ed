// Softmax attention over many query rows on the 5th-generation tensor cores (tcgen05.mma, accumulators in tensor
// memory, operands by TMA), flash style: same contract as seg_attention_kernel (attention_mma.cuh) -- query row i
// sees the key rows [lo[i], hi[i]), causal prefill rule when lo / hi are absent -- for the causal prefill of the text
// tower (reference: src/operators/attention_op.cu:1221-1343) and the windowed / full attention of the vision encoder.
//
// One block = 128 consecutive queries of one head, 256 threads; keys in tiles of 64:
//   S = Q K^T     tcgen05.mma kind::f16, M 128 x N 64, K = head_dim in steps of 16; Q and K tiles by TMA (3-D maps
//                 {head_dim, heads, rows}, 128-byte swizzle, zero fill past the rows and past head_dim 80), S in TMEM;
//   softmax       two threads per query row (TMEM lane = row, 32 columns each): mask, running maximum (halves meet
//                 through shared memory), p = exp2(s - m), P written as bf16 in the operand layout of the next MMA;
//   O_tile = P V  tcgen05.mma M 128 x N head_dim, K 64; the V tile [64 keys x head_dim] lands in shared memory exactly
//                 as TMA writes it (rows = keys, 128 bytes = 64 channels per row and box) and is read as an MN-major
//                 B operand: no transposed copy of V is ever made;
//   O += O_tile   each thread reads its half row of the tile from TMEM and folds it into registers with the rescale
//                 exp2(m_old - m_new); the MMA of the next S tile runs meanwhile.
// One elected thread issues every TMA load and MMA; K is double-buffered, V single (its next tile is requested as
// soon as the P V product has read the current one).  Blocks take the query tiles last first: under the causal rule
// the last tiles have the most keys and should start first.  Every mbarrier wait is bounded and raises *error.
// INT8 variant (I8 = true; the "SageAttention"-style prefill attention of sage_attention.cuh, head_dim 128): Q and the
// centred K arrive as int8 with one scale per 128-token block and head, S = Qi8 . Ki8^T is tcgen05.mma kind::i8 (K = 32
// per instruction, exact int32 accumulators in TMEM) scaled by sq * sk / sqrt(D) when it is read; P and V are fp16.
// Bound: tensor pipe / exp throughput (4 q D kv flops, q kv exponentials).
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>

#include "attention_mma.cuh"
#include "gemm_tc.cuh"

namespace efm {

namespace at {

constexpr int BM = 128, BN = 64, kThreads = 256;
constexpr int S_COL = 0, O_COL = 64;

template <int D, bool I8 = false>
struct Cfg {
    static constexpr int DB = (D + 63) / 64;                 // 64-channel boxes per V row (2-byte elements)
    static constexpr int QB = I8 ? (D + 127) / 128 : DB;     // 128-byte boxes per Q / K row
    static constexpr int Q_BYTES = BM * 128 * QB;
    static constexpr int K_BYTES = BN * 128 * QB;
    static constexpr int V_BYTES = BN * 128 * DB;            // V tile: 64 keys x 128 bytes per box of 64 channels
    static constexpr int P_BYTES = BM * 128;
    static constexpr int TMEM_COLS = D == 64 ? 128 : 256;    // S (64 columns) + O tile (head_dim columns), power of two
    static constexpr int HALF = D / 2;                       // output columns per thread
    static constexpr size_t SMEM = (size_t)Q_BYTES + 2 * K_BYTES + V_BYTES + P_BYTES + 2 * BM * 4 + 128 + 1024;
};

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(bar) : "memory");
}
// kind::f16, A = B = bf16, D = fp32, both operands K-major.
__host__ __device__ constexpr uint32_t instr_desc(int M, int N) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
// kind::f16 with A = B = fp16 (format 0), D = fp32.
__host__ __device__ constexpr uint32_t instr_desc_f16(int M, int N) {
    return (1u << 4) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
// kind::i8, A = B = signed 8-bit (format 1), D = int32 (format 2), both operands K-major.
__host__ __device__ constexpr uint32_t instr_desc_i8(int M, int N) {
    return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n"
        "}\n"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_d(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// MN-major operand tile written by TMA with the 128-byte swizzle (rows = K index, 128 bytes = 64 MN elements per row):
// leading byte offset = distance between 64-element blocks along MN, stride byte offset = distance between 8-row groups
// along K.
__device__ __forceinline__ uint64_t umma_desc_mn(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(lbo_bytes >> 4) << 16;
    d |= (uint64_t)(sbo_bytes >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

}  // namespace at

template <int D, bool I8 = false>
__global__ void __launch_bounds__(at::kThreads) seg_attention_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                        const __grid_constant__ CUtensorMap map_k,
                                                                        const __grid_constant__ CUtensorMap map_v,
                                                                        const SegAttnParams p, int* error) {
    using namespace at;
    using tc::mbar_expect_tx;
    using tc::mbar_init;
    using tc::mbar_wait;
    using tc::smem_u32;
    using tc::umma_commit;
    using tc::umma_desc;
    using C = Cfg<D, I8>;
    extern __shared__ unsigned char attn_tc_smem[];
    __shared__ int s_range[4];          // union of the rows' key ranges [0], [1]; largest lo [2] and smallest hi [3] of the rows
    const uint32_t raw = smem_u32(attn_tc_smem);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char* base_ptr = attn_tc_smem + (base - raw);
    const uint32_t sQ = base, sK = sQ + C::Q_BYTES, sV = sK + 2 * C::K_BYTES, sP = sV + C::V_BYTES;
    float* xch = reinterpret_cast<float*>(base_ptr + C::Q_BYTES + 2 * C::K_BYTES + C::V_BYTES + C::P_BYTES);     // [2][BM]
    const uint32_t bars = sP + C::P_BYTES + 2 * BM * 4;
    const uint32_t qfull = bars, kfull0 = bars + 8, vfull = bars + 24, sbar = bars + 32, obar = bars + 40;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + C::Q_BYTES + 2 * C::K_BYTES + C::V_BYTES + C::P_BYTES + 2 * BM * 4 + 48);
    volatile int* abort_s = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int row = (warp & 3) * 32 + lane, hf = warp >> 2;       // TMEM lane = query row; which half of the columns
    const int q0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * BM, h = blockIdx.y;
    const int kvh = h / (p.q_heads / p.kv_heads);
    const int qi = q0 + row;

    if (tid == 0) {
        s_range[0] = 0x7fffffff;
        s_range[1] = 0;
        s_range[2] = 0;
        s_range[3] = 0x7fffffff;
        mbar_init(qfull, 1); mbar_init(kfull0, 1); mbar_init(kfull0 + 8, 1); mbar_init(vfull, 1); mbar_init(sbar, 1); mbar_init(obar, 1);
        *abort_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(C::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    __syncthreads();
    int lo = 0, hi = 0;
    if (qi < p.S) {
        lo = p.lo != nullptr ? p.lo[qi] : 0;
        hi = p.hi != nullptr ? p.hi[qi] : p.kv_offset + qi + 1;
        if (hi > p.kv_rows) hi = p.kv_rows;
        if (hf == 0 && hi > lo) { atomicMin(&s_range[0], lo); atomicMax(&s_range[1], hi); }
        if (hf == 0) { atomicMax(&s_range[2], lo); atomicMin(&s_range[3], hi); }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    const int kend = s_range[1];
    const int lo_max = s_range[2], hi_min = s_range[3];      // rows past S do not count: their output is never stored
    const int kb0 = s_range[0] == 0x7fffffff ? 0 : (s_range[0] & ~7);          // tile origin: a multiple of 8 keys (TMA alignment)
    const int ntiles = kend > kb0 ? (kend - kb0 + BN - 1) / BN : 0;

    // P V: B operand MN-major (bit 16).  Its shared-memory descriptor: 8-key groups 1024 bytes apart along K, boxes of 64
    // channels BN * 128 bytes apart along N.
    constexpr uint32_t kDescS = I8 ? instr_desc_i8(BM, BN) : instr_desc(BM, BN);
    constexpr uint32_t kDescO = (I8 ? instr_desc_f16(BM, D) : instr_desc(BM, D)) | (1u << 16);
    const uint64_t vdesc = umma_desc_mn(sV, (uint32_t)(BN * 128), 1024u);
    const float sl2 = p.scale * 1.4426950408889634f;
    float o[C::HALF];
#pragma unroll
    for (int e = 0; e < C::HALF; ++e) o[e] = 0.f;
    float m = -INFINITY, l = 0.f;

    constexpr int QBOX = I8 ? 128 : 64;                      // elements per 128-byte box of a Q / K row
    constexpr int KSTEP = I8 ? 32 : 16;                      // elements per MMA along head_dim
    auto load_k = [&](int tile, int buf) {
        mbar_expect_tx(kfull0 + 8 * buf, C::K_BYTES);
#pragma unroll
        for (int b = 0; b < C::QB; ++b)
            tma_load_3d(sK + buf * C::K_BYTES + b * (BN * 128), &map_k, b * QBOX, kvh, kb0 + tile * BN, kfull0 + 8 * buf);
    };
    auto load_v = [&](int tile) {
        mbar_expect_tx(vfull, C::V_BYTES);
#pragma unroll
        for (int b = 0; b < C::DB; ++b) tma_load_3d(sV + b * (BN * 128), &map_v, b * 64, kvh, kb0 + tile * BN, vfull);
    };
    auto issue_s = [&](int buf) {
#pragma unroll
        for (int k = 0; k < D / KSTEP; ++k) {                 // one step = 32 bytes of a 128-byte box row, four per box
            const uint64_t da = umma_desc(sQ + (k >> 2) * (BM * 128)) + (uint64_t)((k & 3) * 2);
            const uint64_t db = umma_desc(sK + buf * C::K_BYTES + (k >> 2) * (BN * 128)) + (uint64_t)((k & 3) * 2);
            if constexpr (I8) umma_i8(tmem + S_COL, da, db, kDescS, k != 0 ? 1u : 0u);
            else umma_d(tmem + S_COL, da, db, kDescS, k != 0 ? 1u : 0u);
        }
        umma_commit(sbar);
    };

    if (ntiles > 0 && tid == 0) {
        mbar_expect_tx(qfull, C::Q_BYTES);
#pragma unroll
        for (int b = 0; b < C::QB; ++b) tma_load_3d(sQ + b * (BM * 128), &map_q, b * QBOX, h, q0, qfull);
        load_k(0, 0);
        if (ntiles > 1) load_k(1, 1);
        load_v(0);
        bool ok = mbar_wait(qfull, 0, abort_s) && mbar_wait(kfull0, 0, abort_s);
        if (!ok) *abort_s = 1;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) issue_s(0);
    }

    for (int j = 0; j < ntiles; ++j) {
        if (!mbar_wait(sbar, (uint32_t)j & 1u, abort_s)) *abort_s = 1;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (tid == 0 && j + 2 < ntiles) load_k(j + 2, j & 1);            // S_j has read K buffer j % 2
        // ---- scores of this thread's half row: mask, scale, local maximum -----------------------------------
        uint32_t sr[32];
        tc::tmem_ld32(tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(S_COL + hf * 32), sr);
        const int key0 = kb0 + j * BN + hf * 32;
        float s[32];                                             // unscaled scores (-inf where the key is not visible)
        float mx = -INFINITY;
        float f2 = sl2;
        if constexpr (I8)       // one scale per 128-token block and head on either side (tiles never straddle a block)
            f2 = sl2 * p.sq[(q0 / 128) * p.q_heads + h] * p.sk[((kb0 + j * BN) / 128) * p.kv_heads + kvh];
        // a tile every query row of the block sees completely needs no per-element visibility test
        const bool interior = kb0 + j * BN >= lo_max && kb0 + (j + 1) * BN <= hi_min;
        if (interior) {
#pragma unroll
            for (int e = 0; e < 32; ++e) {
                s[e] = I8 ? (float)(int)sr[e] : __uint_as_float(sr[e]);
                mx = fmaxf(mx, s[e]);
            }
        } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) {
                const int key = key0 + e;
                const float raw = I8 ? (float)(int)sr[e] : __uint_as_float(sr[e]);
                s[e] = (key >= lo && key < hi) ? raw : -INFINITY;
                mx = fmaxf(mx, s[e]);
            }
        }
        xch[hf * BM + row] = mx * f2;                             // f2 > 0: the maximum commutes with the scale
        if (__syncthreads_or(*abort_s != 0)) break;             // every thread takes the same decision
        const float m_new = fmaxf(m, fmaxf(xch[row], xch[BM + row]));
        const float mb = m_new == -INFINITY ? 0.f : m_new;
        const float alpha = m == -INFINITY ? 0.f : ex2(m - mb);
        m = m_new;
        float rs = 0.f;
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
            const float p0 = ex2(fmaf(s[e], f2, -mb)), p1 = ex2(fmaf(s[e + 1], f2, -mb));     // exp2(-inf) = 0 for masked keys
            rs += p0 + p1;
            if constexpr (I8) {
                const __half2 hp = __floats2half2_rn(p0, p1);
                pk[e >> 1] = *reinterpret_cast<const uint32_t*>(&hp);
            } else {
                pk[e >> 1] = pack_bf16(p0, p1);
            }
        }
        l = l * alpha + rs;
        {   // P row into the K-major, 128-byte-swizzled operand layout: chunk c of row r lives at chunk c ^ (r % 8)
            const uint32_t prow = sP + (uint32_t)(row >> 3) * 1024u + (uint32_t)(row & 7) * 128u;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const uint32_t addr = prow + (uint32_t)(((hf * 4 + c) ^ (row & 7)) << 4);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pk[4 * c]), "r"(pk[4 * c + 1]), "r"(pk[4 * c + 2]),
                             "r"(pk[4 * c + 3]) : "memory");
            }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            bool ok = mbar_wait(vfull, (uint32_t)j & 1u, abort_s);
            if (ok) {
                // B = V tile, MN-major: 16 keys (one K step) are two 8-row groups of 1024 bytes
#pragma unroll
                for (int k = 0; k < BN / 16; ++k)
                    umma_d(tmem + O_COL, umma_desc(sP) + (uint64_t)(k * 2), vdesc + (uint64_t)(k * (2048 >> 4)), kDescO, k != 0 ? 1u : 0u);
                umma_commit(obar);
                if (j + 1 < ntiles) {
                    ok = mbar_wait(kfull0 + 8 * ((j + 1) & 1), (uint32_t)((j + 1) >> 1) & 1u, abort_s);
                    if (ok) issue_s((j + 1) & 1);
                }
            }
            if (!ok) *abort_s = 1;
        }
        if (!mbar_wait(obar, (uint32_t)j & 1u, abort_s)) *abort_s = 1;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (tid == 0 && j + 1 < ntiles) load_v(j + 1);                   // P V of tile j has read the V^T buffer
        // ---- O += O_tile (this thread's half row) -------------------------------------------------------------
        const uint32_t orow = tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(O_COL + hf * C::HALF);
#pragma unroll
        for (int c0 = 0; c0 + 32 <= C::HALF; c0 += 32) {
            uint32_t r[32];
            tc::tmem_ld32(orow + (uint32_t)c0, r);
#pragma unroll
            for (int e = 0; e < 32; ++e) o[c0 + e] = fmaf(o[c0 + e], alpha, __uint_as_float(r[e]));
        }
        if constexpr (C::HALF % 32 != 0) {
            constexpr int c0 = (C::HALF / 32) * 32;
            uint32_t r[8];
            tmem_ld8(orow + (uint32_t)c0, r);
#pragma unroll
            for (int e = 0; e < 8; ++e) o[c0 + e] = fmaf(o[c0 + e], alpha, __uint_as_float(r[e]));
        }
    }

    // ---- normalise and store ----------------------------------------------------------------------------------
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    xch[hf * BM + row] = l;
    __syncthreads();
    const float L = xch[row] + xch[BM + row];
    const float inv = L > 0.f ? 1.0f / L : 0.f;
    if (qi < p.S && *abort_s == 0) {
        __nv_bfloat16* dst = p.out + (size_t)qi * p.out_stride + (size_t)h * D + hf * C::HALF;
#pragma unroll
        for (int e = 0; e < C::HALF; e += 8)
            *reinterpret_cast<uint4*>(dst + e) = make_uint4(pack_bf16(o[e] * inv, o[e + 1] * inv), pack_bf16(o[e + 2] * inv, o[e + 3] * inv),
                                                            pack_bf16(o[e + 4] * inv, o[e + 5] * inv), pack_bf16(o[e + 6] * inv, o[e + 7] * inv));
    }
    if (*abort_s != 0 && tid == 0 && error != nullptr) atomicExch(error, 1);
    if (warp == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(C::TMEM_COLS) : "memory");
    }
}

}  // namespace efm
