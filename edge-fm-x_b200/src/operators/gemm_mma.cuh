// Prefill linear: C[M,N] = A[M,K] . B[N,K]^T, bf16 operands, fp32 accumulate.
// (reference: cublasLtMatmul / CUTLASS sm80 prefill linears, src/operators/linear_impl.cu:457-469,482-706)
//
// Bring-up tensor-core path: 128x128x32 tiles, 8 warps (2 x 4, 64x32 each), m16n8k16 bf16
// mma.sync fed by ldmatrix from XOR-swizzled shared memory, 3-stage cp.async pipeline.
// Epilogues: bf16 (+bias) | residual add r = bf16(r + bf16(acc)) | fp32.
// Bound: tensor pipe; rows beyond M and columns beyond N are zero-filled on load and masked on store.
#pragma once
#include "common.cuh"

namespace efm {

enum class GemmEpi : int { Bf16Bias = 0, Residual = 1, F32 = 2 };

struct GemmParams {
    const __nv_bfloat16* A;   // [M, K]
    const __nv_bfloat16* B;   // [N, K]
    const __nv_bfloat16* bias;
    __nv_bfloat16* C;         // Bf16Bias: out; Residual: in/out
    float* Cf;                // F32
    int M, N, K;
};

namespace gemm_detail {
constexpr int BM = 128, BN = 128, BK = 32, STAGES = 3, NT = 256;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool pred) {
    const int sz = pred ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// A tile row is 64 bytes = four 16-byte chunks; chunk c of row r is stored at chunk c ^ ((r >> 1) & 3)
// so that the eight rows one ldmatrix phase touches fall in distinct bank groups.
__device__ __forceinline__ uint32_t swz(int row, int chunk) { return (uint32_t)(row * 64 + ((chunk ^ ((row >> 1) & 3)) << 4)); }
}  // namespace gemm_detail

template <GemmEpi EPI>
__global__ void __launch_bounds__(256) gemm_mma_kernel(const GemmParams p) {
    using namespace gemm_detail;
    extern __shared__ __align__(128) unsigned char gemm_smem[];
    const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(gemm_smem);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int wm = warp >> 2, wn = warp & 3;            // 2 x 4 warps
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int KT = p.K / BK;

    auto load_stage = [&](int stage, int kt) {
        const uint32_t sa = smem_base + stage * STAGE_BYTES, sb = sa + A_BYTES;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int idx = tid + i * NT, row = idx >> 2, chunk = idx & 3;
            const int gm = m0 + row, gn = n0 + row;
            cp_async16(sa + swz(row, chunk), p.A + (size_t)(gm < p.M ? gm : 0) * p.K + kt * BK + chunk * 8, gm < p.M);
            cp_async16(sb + swz(row, chunk), p.B + (size_t)(gn < p.N ? gn : 0) * p.K + kt * BK + chunk * 8, gn < p.N);
        }
    };

    float acc[4][4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;

#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < KT) load_stage(s, s);
        cp_async_commit();
    }
    for (int kt = 0; kt < KT; ++kt) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();
        {
            const int nk = kt + STAGES - 1;
            if (nk < KT) load_stage(nk % STAGES, nk);
            cp_async_commit();
        }
        const uint32_t sa = smem_base + (kt % STAGES) * STAGE_BYTES, sb = sa + A_BYTES;
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {                 // two k16 steps per BK = 32
            uint32_t af[4][4], bf[2][4];
#pragma unroll
            for (int mt = 0; mt < 4; ++mt) {
                const int row = wm * 64 + mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                const int chunk = ks * 2 + (lane >> 4);
                ldmatrix_x4(sa + swz(row, chunk), af[mt][0], af[mt][1], af[mt][2], af[mt][3]);
            }
#pragma unroll
            for (int np = 0; np < 2; ++np) {             // each x4 covers two n8 tiles
                const int row = wn * 32 + np * 16 + (lane & 7) + (lane >> 4) * 8;
                const int chunk = ks * 2 + ((lane >> 3) & 1);
                ldmatrix_x4(sb + swz(row, chunk), bf[np][0], bf[np][1], bf[np][2], bf[np][3]);
            }
#pragma unroll
            for (int mt = 0; mt < 4; ++mt)
#pragma unroll
                for (int nt = 0; nt < 4; ++nt)
                    mma_bf16(acc[mt][nt], af[mt], bf[nt >> 1][(nt & 1) * 2], bf[nt >> 1][(nt & 1) * 2 + 1]);
        }
    }
    cp_async_wait<0>();

    // ---- epilogue ------------------------------------------------------------------------
    const int g = lane >> 2, q = lane & 3;
#pragma unroll
    for (int mt = 0; mt < 4; ++mt)
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int hrow = 0; hrow < 2; ++hrow) {
                const int m = m0 + wm * 64 + mt * 16 + g + hrow * 8;
                const int n = n0 + wn * 32 + nt * 8 + q * 2;
                if (m >= p.M || n >= p.N) continue;
                float v0 = acc[mt][nt][hrow * 2], v1 = acc[mt][nt][hrow * 2 + 1];
                const size_t off = (size_t)m * p.N + n;
                if constexpr (EPI == GemmEpi::Bf16Bias) {
                    if (p.bias != nullptr) { v0 += __bfloat162float(p.bias[n]); v1 += __bfloat162float(p.bias[n + 1]); }
                    *reinterpret_cast<uint32_t*>(p.C + off) = pack_bf16(v0, v1);
                } else if constexpr (EPI == GemmEpi::Residual) {
                    const uint32_t r = *reinterpret_cast<const uint32_t*>(p.C + off);
                    *reinterpret_cast<uint32_t*>(p.C + off) = pack_bf16(bf16lo(r) + round_bf16(v0), bf16hi(r) + round_bf16(v1));
                } else {
                    *reinterpret_cast<float2*>(p.Cf + off) = make_float2(v0, v1);
                }
            }
}

inline size_t gemm_mma_smem_bytes() { return (size_t)gemm_detail::STAGES * gemm_detail::STAGE_BYTES; }

}  // namespace efm
