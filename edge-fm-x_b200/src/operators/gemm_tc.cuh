// Prefill linear on the 5th-generation tensor cores: C[M,N] = A[M,K] . B[N,K]^T, bf16 operands,
// fp32 accumulation in tensor memory.
// (reference: cublasLtMatmul / CUTLASS sm80 prefill linears, src/operators/linear_impl.cu:457-469,482-706;
//  the reference has no sm_100 kernel.)
//
// Persistent blocks (one per SM, 320 threads) walk the 128 x 256 output tiles (and K splits) round-robin:
//   warp 0      one lane issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle, no multicast) of
//               a 128 x 64 A tile and a 256 x 64 B tile per stage into a 4-stage ring;
//   warp 1      owns all 512 TMEM columns = two 128 x 256 fp32 accumulators; one lane issues tcgen05.mma
//               (M 128, N 256, K 16, four per stage) and tcgen05.commit, which releases the stage to the
//               producer, and after the last k-block of a tile marks the accumulator complete;
//   warps 2-9   epilogue of tile j while the MMA warp already fills the other accumulator with tile j+1; two warps
//               per TMEM lane quarter, one per half of the tile's columns (with four warps the drain of a tile took
//               longer than its MMAs whenever K was short):
//               tcgen05.ld (row = TMEM lane, 32 columns at a time), bias / activation, staging through
//               shared memory (XOR-swizzled 16-byte columns) so that global rows are written as contiguous segments:
//               bf16 (+bias, optionally erf-GELU) | fp32 residual add | fp32 | silu(gate)*up in bf16.
// Rows past M and columns past N are zero-filled by TMA on load and masked on store.
// Every mbarrier wait is bounded; a wait that gives up raises *error, all roles leave their loops, the
// block frees its TMEM and returns.  Bound: tensor pipe (2 M N K flops).
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace efm {

enum class GemmEpi : int { Bf16Bias = 0, Residual = 1, F32 = 2, Bf16Gelu = 3, SwiGlu = 4, Bf16GeluTanh = 5 };

struct GemmParams {
    const __nv_bfloat16* A;   // [M, K] (row stride lda)
    const __nv_bfloat16* B;   // [N, K]
    const __nv_bfloat16* bias;
    __nv_bfloat16* C;         // Bf16Bias / Bf16Gelu / Bf16GeluTanh: out [M, N]; SwiGlu: out [M, N/2]
    float* Cf;                // F32: out; Residual: in/out (fp32 residual stream)
    int M, N, K;
    int lda = 0;              // row stride of A in elements (0: K)
    int kb_per_split = 0;     // split-K: split z covers 64-wide k-blocks [z * kb_per_split, (z+1) * kb_per_split) and
                              // writes its raw fp32 partial tile to Cf + z * M * N (F32 epilogue, no bias); 0: no split
    int tile_begin = 0;       // this launch covers the output tiles [tile_begin, tile_begin + tile_count) of the
    int tile_count = 0;       // m-fastest tile order (0: all of them).  With kb_per_split > 0 and tile_count > 0 the
                              // partial of (split z, tile t) goes to the compact slot Cf + (z * tile_count + t -
                              // tile_begin) * 128 * 256, row-major inside the tile ("tail split", see the launcher)
};

namespace tc {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int kThreads = 320;
constexpr int kEpiWarps = 8;
constexpr int TMEM_COLS = 512;                             // two accumulators of BN columns
constexpr int STAGING_BYTES = kEpiWarps * 32 * 32 * 4;     // per epilogue warp: 32 rows x 32 floats, 16-byte columns swizzled
constexpr int kWaitLimit = 1 << 20;                        // try_wait polls before giving up
constexpr size_t SMEM_BYTES = (size_t)STAGES * STAGE_BYTES + STAGING_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait for the phase with the given parity; false when it gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    for (int i = 0; i < kWaitLimit; ++i) {
        if ((i & 0xff) == 0xff && *abort_flag != 0) return false;      // another role already gave up
        uint32_t ok;
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar) : "memory");
}
// K-major operand tile written by TMA with the 128-byte swizzle: rows of 128 bytes, 8-row groups
// 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);        // start address / 16
    d |= (uint64_t)1 << 16;                               // leading byte offset (unused with swizzle)
    d |= (uint64_t)(1024 >> 4) << 32;                     // stride byte offset: 8 rows x 128 B
    d |= (uint64_t)1 << 46;                               // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                               // SWIZZLE_128B
    return d;
}
// kind::f16, A = B = bf16, D = fp32, both operands K-major, M = 128, N = BN.
constexpr uint32_t kInstrDesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(kInstrDesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

}  // namespace tc

template <GemmEpi EPI>
__global__ void __launch_bounds__(tc::kThreads) gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a,
                                                               const __grid_constant__ CUtensorMap map_b,
                                                               const GemmParams p, int* error) {
    using namespace tc;
    extern __shared__ unsigned char gemm_tc_smem[];
    const uint32_t raw = smem_u32(gemm_tc_smem);
    const uint32_t base = (raw + 1023u) & ~1023u;                     // swizzle atoms need 1024-byte alignment
    unsigned char* base_ptr = gemm_tc_smem + (base - raw);
    float* stage_all = reinterpret_cast<float*>(base_ptr + (size_t)STAGES * STAGE_BYTES);
    uint64_t* bars = reinterpret_cast<uint64_t*>(base_ptr + (size_t)STAGES * STAGE_BYTES + STAGING_BYTES);
    const uint32_t full0 = base + STAGES * STAGE_BYTES + STAGING_BYTES;   // full[s]  = full0 + 8 s
    const uint32_t empty0 = full0 + 8 * STAGES;                           // empty[s] = empty0 + 8 s
    const uint32_t accf0 = empty0 + 8 * STAGES;                           // accumulator a complete
    const uint32_t acce0 = accf0 + 16;                                    // accumulator a drained
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_s = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (p.M + BM - 1) / BM, tiles_n = (p.N + BN - 1) / BN;
    const int KB_all = (p.K + BK - 1) / BK;
    const int splits = p.kb_per_split > 0 ? (KB_all + p.kb_per_split - 1) / p.kb_per_split : 1;
    const int n_tiles = p.tile_count > 0 ? p.tile_count : tiles_m * tiles_n;
    const int n_items = n_tiles * splits;                             // item = (split, n tile, m tile), m fastest
    const bool compact = p.tile_count > 0 && p.kb_per_split > 0;      // partial tiles in compact slots

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(accf0 + 8 * a, 1); mbar_init(acce0 + 8 * a, kEpiWarps); }
        *abort_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;

    auto item_coords = [&](int item, int& m0, int& n0, int& kb0, int& kb1, int& z) {
        z = item / n_tiles;
        const int tile = p.tile_begin + (item - z * n_tiles);
        const int mt = tile % tiles_m, nt = tile / tiles_m;
        m0 = mt * BM;
        n0 = nt * BN;
        kb0 = p.kb_per_split > 0 ? z * p.kb_per_split : 0;
        kb1 = p.kb_per_split > 0 ? min(KB_all, kb0 + p.kb_per_split) : KB_all;
    };

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            for (int item = blockIdx.x; item < n_items && *abort_s == 0; item += gridDim.x) {
                int m0, n0, kb0, kb1, z;
                item_coords(item, m0, n0, kb0, kb1, z);
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1u;
                    if (!mbar_wait(empty0 + 8 * s, ph ^ 1u, abort_s)) { *abort_s = 1; break; }
                    mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
                    tma_load_2d(base + s * STAGE_BYTES, &map_a, kb * BK, m0, full0 + 8 * s);
                    tma_load_2d(base + s * STAGE_BYTES + A_BYTES, &map_b, kb * BK, n0, full0 + 8 * s);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            uint32_t it = 0;
            int j = 0;
            for (int item = blockIdx.x; item < n_items && *abort_s == 0; item += gridDim.x, ++j) {
                int m0, n0, kb0, kb1, z;
                item_coords(item, m0, n0, kb0, kb1, z);
                const int a = j & 1;
                const uint32_t use = (uint32_t)(j >> 1) & 1u;
                if (!mbar_wait(acce0 + 8 * a, use ^ 1u, abort_s)) { *abort_s = 1; break; }     // epilogue drained this buffer
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t acc = tmem + (uint32_t)(a * BN);
                bool ok = true;
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1u;
                    if (!mbar_wait(full0 + 8 * s, ph, abort_s)) { *abort_s = 1; ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t da = umma_desc(base + s * STAGE_BYTES), db = umma_desc(base + s * STAGE_BYTES + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)               // 32 bytes further along K inside the swizzle atom
                        umma(acc, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), ((kb - kb0) | k) != 0 ? 1u : 0u);
                    umma_commit(empty0 + 8 * s);                         // stage free once these MMAs have read it
                }
                if (!ok) break;
                umma_commit(accf0 + 8 * a);                              // accumulator complete
            }
        }
    } else {
        // Epilogue warps 2..9: TMEM lane group = warp % 4, column half = (warp - 2) / 4.  Per 32-column chunk: each lane
        // owns one accumulator row (tcgen05.ld), applies bias / activation and parks the row in a staging tile (16-byte
        // column index XOR row & 7: conflict-free both ways); then the warp writes the chunk out four rows per
        // instruction, eight lanes of 16 bytes per row.
        const int q = warp & 3, ch = (warp - 2) >> 2;
        constexpr int LD = 32;
        float* stage = stage_all + (size_t)(warp - 2) * 32 * LD;
        int j = 0;
        for (int item = blockIdx.x; item < n_items; item += gridDim.x, ++j) {
            int m0, n0, kb0, kb1, z;
            item_coords(item, m0, n0, kb0, kb1, z);
            const int a = j & 1;
            const uint32_t use = (uint32_t)(j >> 1) & 1u;
            if (!mbar_wait(accf0 + 8 * a, use, abort_s)) { *abort_s = 1; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t acc = tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(a * BN);
            constexpr int OUT_COLS = EPI == GemmEpi::SwiGlu ? BN / 2 : BN;
            const int ldc = EPI == GemmEpi::SwiGlu ? (p.N >> 1) : p.N;         // output row length
            const int nc0 = EPI == GemmEpi::SwiGlu ? (n0 >> 1) : n0;           // first output column of the tile
            const bool vec = (ldc & 3) == 0;
            const size_t split_off = compact ? (size_t)item * (size_t)(BM * BN)
                                             : (p.kb_per_split > 0 ? (size_t)z * (size_t)p.M * (size_t)p.N : 0);
#pragma unroll 1
            for (int c0 = ch * (OUT_COLS / 2); c0 < (ch + 1) * (OUT_COLS / 2); c0 += 32) {
                if (nc0 + c0 >= ldc) break;                                    // whole chunk outside the matrix
                const int cl = (lane & 7) * 4;
                // residual epilogue: all eight old values of the chunk are requested up front, before the accumulator is
                // read and long before the first store (the
                // compiler may not move a load of Cf above a store to Cf by itself), one round trip per chunk
                float4 prev[8];
                if constexpr (EPI == GemmEpi::Residual) {
#pragma unroll
                    for (int r0 = 0; r0 < 32; r0 += 4) {
                        const int m = m0 + q * 32 + r0 + (lane >> 3), n = nc0 + c0 + cl;
                        prev[r0 >> 2] = (vec && m < p.M && n + 3 < ldc) ? __ldcg(reinterpret_cast<const float4*>(p.Cf + (size_t)m * ldc + n))
                                                                     : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                }
                float o[32];
                if constexpr (EPI == GemmEpi::SwiGlu) {
                    // fused gate|up weight: in every 128 columns the first 64 are gate rows and the last 64 the up
                    // rows of the same channels; out[m, n/2 + j] = silu(gate_j) * up_j
                    const int blk = c0 >> 6, cc = c0 & 63;
                    uint32_t rg[32], ru[32];
                    tmem_ld32(acc + (uint32_t)(blk * 128 + cc), rg);
                    tmem_ld32(acc + (uint32_t)(blk * 128 + 64 + cc), ru);
                    const int n = n0 + blk * 128 + cc;                        // gate column in the fused output
                    const bool in = n0 + blk * 128 + 128 <= p.N;
                    // one gate and one up bias element per lane, handed round by shuffles (64 loads per thread otherwise)
                    const bool has_bias = p.bias != nullptr && in;
                    const float bias_g = has_bias ? __bfloat162float(p.bias[n + lane]) : 0.f;
                    const float bias_u = has_bias ? __bfloat162float(p.bias[n + 64 + lane]) : 0.f;
#pragma unroll
                    for (int e = 0; e < 32; ++e) {
                        float g = __uint_as_float(rg[e]), u = __uint_as_float(ru[e]);
                        if (has_bias) {
                            g += __shfl_sync(0xffffffffu, bias_g, e);
                            u += __shfl_sync(0xffffffffu, bias_u, e);
                        }
                        // four epilogue warps drain a tile while one warp feeds the tensor cores: their issue slots are
                        // the limit when K is short, hence the approximate reciprocal instead of an IEEE division
                        o[e] = __fdividef(g, 1.0f + __expf(-g)) * u;
                    }
                } else {
                    uint32_t r[32];
                    tmem_ld32(acc + (uint32_t)c0, r);
                    const int n = n0 + c0;
                    // one bias element per lane, handed round by shuffles (32 broadcast loads per thread otherwise)
                    const float bias_l = (p.bias != nullptr && n + lane < p.N) ? __bfloat162float(p.bias[n + lane]) : 0.f;
#pragma unroll
                    for (int e = 0; e < 32; ++e) {
                        o[e] = __uint_as_float(r[e]) + __shfl_sync(0xffffffffu, bias_l, e);
                        if constexpr (EPI == GemmEpi::Bf16Gelu) o[e] = 0.5f * o[e] * (1.0f + erff(o[e] * 0.70710678118654752f));
                        if constexpr (EPI == GemmEpi::Bf16GeluTanh)
                        {
                            float th;           // hardware tanh (relative error ~2^-11, below the bf16 rounding of the result)
                            asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(0.7978845608028654f * (o[e] + 0.044715f * o[e] * o[e] * o[e])));
                            o[e] = 0.5f * o[e] * (1.0f + th);
                        }
                    }
                }
                __syncwarp();                                                  // previous chunk fully written out
#pragma unroll
                for (int e = 0; e < 32; e += 4)
                    *reinterpret_cast<float4*>(stage + lane * LD + (((e >> 2) ^ (lane & 7)) << 2)) = make_float4(o[e], o[e + 1], o[e + 2], o[e + 3]);
                __syncwarp();
#pragma unroll
                for (int r0 = 0; r0 < 32; r0 += 4) {
                    const int r = r0 + (lane >> 3);
                    const int m = m0 + q * 32 + r;
                    const int n = nc0 + c0 + cl;
                    if (m >= p.M || n >= ldc) continue;
                    const float4 v = *reinterpret_cast<const float4*>(stage + r * LD + ((((cl >> 2) ^ (r & 7))) << 2));
                    size_t off = (size_t)m * ldc + n;
                    if constexpr (EPI == GemmEpi::F32) {
                        if (compact) off = (size_t)(m - m0) * BN + (size_t)(n - n0);      // slot-local (item = z * n_tiles + t)
                    }
                    if (vec && n + 3 < ldc) {
                        if constexpr (EPI == GemmEpi::F32) {
                            *reinterpret_cast<float4*>(p.Cf + split_off + off) = v;
                        } else if constexpr (EPI == GemmEpi::Residual) {
                            const float4 old = prev[r0 >> 2];
                            *reinterpret_cast<float4*>(p.Cf + off) = make_float4(old.x + v.x, old.y + v.y, old.z + v.z, old.w + v.w);
                        } else {
                            *reinterpret_cast<uint2*>(p.C + off) = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
                        }
                    } else {
                        const float e4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            if (n + i >= ldc) break;
                            if constexpr (EPI == GemmEpi::F32) p.Cf[split_off + off + i] = e4[i];
                            else if constexpr (EPI == GemmEpi::Residual) p.Cf[off + i] += e4[i];
                            else p.C[off + i] = __float2bfloat16_rn(e4[i]);
                        }
                    }
                }
            }
            // every tcgen05.ld of this accumulator has completed: hand the buffer back to the MMA warp
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acce0 + 8 * a) : "memory");
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (*abort_s != 0 && threadIdx.x == 0 && error != nullptr) atomicExch(error, 1);
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

// Second half of a split-K product: out = epilogue(sum over splits, in split order, of the fp32
// partial tiles) -- the order is fixed, so the result does not depend on which block finished first.
template <GemmEpi EPI>
__global__ void __launch_bounds__(256) gemm_splitk_finish_kernel(const float* __restrict__ ws, int splits, const GemmParams p) {
    const size_t plane = (size_t)p.M * p.N;
    if constexpr (EPI == GemmEpi::SwiGlu) {
        // fused gate|up partials [M, N] (64 gate columns, 64 up columns, ...) -> out [M, N / 2] = silu(gate) * up
        const int half = p.N >> 1;
        const size_t out4 = (size_t)p.M * half / 4;        // N % 128 == 0 (checked by the launcher)
        for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < out4; i += (size_t)gridDim.x * 256) {
            const size_t m = (i * 4) / (size_t)half;
            const int j = (int)((i * 4) % (size_t)half), blk = j >> 6, jj = j & 63;
            const size_t goff = m * p.N + (size_t)blk * 128 + jj, uoff = goff + 64;
            float4 g = *reinterpret_cast<const float4*>(ws + goff), u = *reinterpret_cast<const float4*>(ws + uoff);
            for (int z = 1; z < splits; ++z) {
                const float4 g2 = *reinterpret_cast<const float4*>(ws + (size_t)z * plane + goff);
                const float4 u2 = *reinterpret_cast<const float4*>(ws + (size_t)z * plane + uoff);
                g.x += g2.x; g.y += g2.y; g.z += g2.z; g.w += g2.w;
                u.x += u2.x; u.y += u2.y; u.z += u2.z; u.w += u2.w;
            }
            if (p.bias != nullptr) {
                const __nv_bfloat16* bg = p.bias + blk * 128 + jj;
                g.x += __bfloat162float(bg[0]); g.y += __bfloat162float(bg[1]); g.z += __bfloat162float(bg[2]); g.w += __bfloat162float(bg[3]);
                u.x += __bfloat162float(bg[64]); u.y += __bfloat162float(bg[65]); u.z += __bfloat162float(bg[66]); u.w += __bfloat162float(bg[67]);
            }
            const float o0 = g.x / (1.0f + __expf(-g.x)) * u.x, o1 = g.y / (1.0f + __expf(-g.y)) * u.y;
            const float o2 = g.z / (1.0f + __expf(-g.z)) * u.z, o3 = g.w / (1.0f + __expf(-g.w)) * u.w;
            *reinterpret_cast<uint2*>(p.C + m * half + j) = make_uint2(pack_bf16(o0, o1), pack_bf16(o2, o3));
        }
        return;
    }
    const size_t total4 = (size_t)p.M * p.N / 4;           // N % 4 == 0 (checked by the launcher)
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < total4; i += (size_t)gridDim.x * 256) {
        float4 a = *reinterpret_cast<const float4*>(ws + i * 4);
        for (int z = 1; z < splits; ++z) {
            const float4 b = *reinterpret_cast<const float4*>(ws + (size_t)z * plane + i * 4);
            a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        }
        const int n = (int)((i * 4) % (size_t)p.N);
        if (p.bias != nullptr) {
            a.x += __bfloat162float(p.bias[n]); a.y += __bfloat162float(p.bias[n + 1]);
            a.z += __bfloat162float(p.bias[n + 2]); a.w += __bfloat162float(p.bias[n + 3]);
        }
        if constexpr (EPI == GemmEpi::F32) {
            *reinterpret_cast<float4*>(p.Cf + i * 4) = a;
        } else if constexpr (EPI == GemmEpi::Residual) {
            const float4 o = *reinterpret_cast<const float4*>(p.Cf + i * 4);
            *reinterpret_cast<float4*>(p.Cf + i * 4) = make_float4(o.x + a.x, o.y + a.y, o.z + a.z, o.w + a.w);
        } else {
            *reinterpret_cast<uint2*>(p.C + i * 4) = make_uint2(pack_bf16(a.x, a.y), pack_bf16(a.z, a.w));
        }
    }
}

// Second half of a tail split: the last tiles of a product whose tile count is a little more than a multiple of the
// SM count were computed as `splits` K-slices each (compact fp32 slots, see GemmParams::tile_count); sum them in
// split order and apply the epilogue.  grid = (blocks per tile, tile_count).
template <GemmEpi EPI>
__global__ void __launch_bounds__(256) gemm_tail_finish_kernel(const float* __restrict__ ws, int splits, int tile_begin, int tile_count,
                                                               const GemmParams p) {
    constexpr int BM = tc::BM, BN = tc::BN;
    const int tiles_m = (p.M + BM - 1) / BM;
    const int t = blockIdx.y, tile = tile_begin + t;
    const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * BN;
    for (int i = blockIdx.x * 256 + threadIdx.x; i < BM * BN / 4; i += gridDim.x * 256) {
        const int row = i / (BN / 4), c = (i - row * (BN / 4)) * 4;
        const int m = m0 + row, n = n0 + c;
        if (m >= p.M || n >= p.N) continue;                  // N % 4 == 0 (checked by the launcher)
        const float* src = ws + ((size_t)t * BM + row) * BN + c;
        float4 a = *reinterpret_cast<const float4*>(src);
        for (int z = 1; z < splits; ++z) {
            const float4 b = *reinterpret_cast<const float4*>(src + (size_t)z * tile_count * (BM * BN));
            a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        }
        if (p.bias != nullptr) {
            a.x += __bfloat162float(p.bias[n]); a.y += __bfloat162float(p.bias[n + 1]);
            a.z += __bfloat162float(p.bias[n + 2]); a.w += __bfloat162float(p.bias[n + 3]);
        }
        const size_t off = (size_t)m * p.N + n;
        if constexpr (EPI == GemmEpi::F32) {
            *reinterpret_cast<float4*>(p.Cf + off) = a;
        } else if constexpr (EPI == GemmEpi::Residual) {
            const float4 o = *reinterpret_cast<const float4*>(p.Cf + off);
            *reinterpret_cast<float4*>(p.Cf + off) = make_float4(o.x + a.x, o.y + a.y, o.z + a.z, o.w + a.w);
        } else {
            *reinterpret_cast<uint2*>(p.C + off) = make_uint2(pack_bf16(a.x, a.y), pack_bf16(a.z, a.w));
        }
    }
}

}  // namespace efm
