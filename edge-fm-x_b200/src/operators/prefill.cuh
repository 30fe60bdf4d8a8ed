// Row-wise kernels of the prefill pass (S tokens at once).  The contractions live in the GEMM
// and attention files; these are the HBM-bound glue steps, each one read and one write of an
// [S, *] activation.
#pragma once
#include "common.cuh"

namespace efm {

// Embedding gather with custom-embedding injection.  One block per token.
// Same contract as the reference's embedding_lookup_with_embedding_insertion_kernel
// (src/layers/embed_head.cu:63-132): ids in [embed_token_id, embed_token_id + n_custom) take
// row id - embed_token_id of `custom`; other ids inside the vocabulary take the table row; any
// other id yields zeros.
__global__ void __launch_bounds__(128) embed_rows_kernel(const int32_t* __restrict__ ids,
                                                         const __nv_bfloat16* __restrict__ table,
                                                         const __nv_bfloat16* __restrict__ custom,
                                                         float* __restrict__ out, int vocab, int hidden,
                                                         int embed_token_id, int n_custom) {
    const int t = blockIdx.x;
    const int id = ids[t];
    const __nv_bfloat16* src = nullptr;
    if (custom != nullptr && embed_token_id >= 0 && id >= embed_token_id && id < embed_token_id + n_custom)
        src = custom + (size_t)(id - embed_token_id) * hidden;
    else if (id >= 0 && id < vocab)
        src = table + (size_t)id * hidden;
    float4* dst = reinterpret_cast<float4*>(out + (size_t)t * hidden);      // residual stream: fp32
    for (int c = threadIdx.x; c < hidden / 8; c += blockDim.x) {
        float f[8];
        unpack8(src != nullptr ? ld_cached(src + (size_t)c * 8) : make_uint4(0, 0, 0, 0), f);
        dst[2 * c] = make_float4(f[0], f[1], f[2], f[3]);
        dst[2 * c + 1] = make_float4(f[4], f[5], f[6], f[7]);
    }
}

// y[s,:] = bf16(x[s,:] * rsqrt(mean(x^2) + eps) * w), x = fp32 residual stream, fp32 inside (reference: FlashInfer RMSNorm
// through src/operators/norm_op.cu:20-62; formula pinned by tests/operators/test_norm_sampler.py:62-64).
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(const float* __restrict__ x,
                                                           const __nv_bfloat16* __restrict__ w,
                                                           __nv_bfloat16* __restrict__ y, int hidden, float eps) {
    __shared__ float part[8];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    pdl_launch_dependents();
    pdl_wait();            // no-ops unless launched with programmatic stream serialization
    const float* xr = x + (size_t)blockIdx.x * hidden;
    const int nch = hidden >> 3;
    float ss = 0.f;
    for (int c = tid; c < nch; c += 256) {
        const float4 lo = reinterpret_cast<const float4*>(xr)[2 * c], hi = reinterpret_cast<const float4*>(xr)[2 * c + 1];
        const float f[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
    }
    ss = warp_sum(ss);
    if (lane == 0) part[warp] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += part[i];
    const float inv = 1.0f / sqrtf(tot / (float)hidden + eps);
    uint4* yr = reinterpret_cast<uint4*>(y + (size_t)blockIdx.x * hidden);
    for (int c = tid; c < nch; c += 256) {
        const float4 lo = reinterpret_cast<const float4*>(xr)[2 * c], hi = reinterpret_cast<const float4*>(xr)[2 * c + 1];
        const float f[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
        float g[8];
        unpack8(ld_cached(w + (size_t)c * 8), g);
        uint4 o;
        o.x = pack_bf16(f[0] * inv * g[0], f[1] * inv * g[1]);
        o.y = pack_bf16(f[2] * inv * g[2], f[3] * inv * g[3]);
        o.z = pack_bf16(f[4] * inv * g[4], f[5] * inv * g[5]);
        o.w = pack_bf16(f[6] * inv * g[6], f[7] * inv * g[7]);
        yr[c] = o;
    }
}

// The same for rows of at most 2048 channels (hidden % 4 == 0): one warp per row, the row stays in registers between the
// sum of squares and the scaling (one read of x, no block barrier); 8 rows per block.
__global__ void __launch_bounds__(256) rmsnorm_rows_warp_kernel(const float* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                                __nv_bfloat16* __restrict__ y, int rows, int hidden, float eps) {
    constexpr int MAXV = 16;                                   // float4 per lane: 16 x 32 x 4 = 2048 channels
    const int row = blockIdx.x * 8 + (int)(threadIdx.x >> 5), lane = threadIdx.x & 31;
    pdl_launch_dependents();
    pdl_wait();            // no-ops unless launched with programmatic stream serialization
    if (row >= rows) return;
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)row * hidden);
    const int nv = hidden >> 2;
    float4 v[MAXV];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
        const int c = lane + 32 * i;
        if (c < nv) {
            v[i] = xr[c];
            ss = fmaf(v[i].x, v[i].x, ss); ss = fmaf(v[i].y, v[i].y, ss); ss = fmaf(v[i].z, v[i].z, ss); ss = fmaf(v[i].w, v[i].w, ss);
        }
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
    uint2* yr = reinterpret_cast<uint2*>(y + (size_t)row * hidden);
    const uint2* wr = reinterpret_cast<const uint2*>(w);
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
        const int c = lane + 32 * i;
        if (c < nv) {
            const uint2 g = __ldg(wr + c);
            yr[c] = make_uint2(pack_bf16(v[i].x * inv * bf16lo(g.x), v[i].y * inv * bf16hi(g.x)),
                               pack_bf16(v[i].z * inv * bf16lo(g.y), v[i].w * inv * bf16hi(g.y)));
        }
    }
}

// Rotate-half RoPE / M-RoPE on the q and k parts of a fused [S, (q+2kv)*D] projection, then
// scatter: q -> [S, q_heads, D]; rotated k and raw v -> cache rows kv_offset + s.
// Convention of the reference: angle = pos * theta^(-2d/D); o[d] = x0 cos - x1 sin,
// o[d+D/2] = x1 cos + x0 sin (src/operators/attention_op.cu:327-371); M-RoPE picks the position
// row by rotary-pair section (src/layers/attention.cu:17-72).  One block per row: the row's D/2 (sin, cos) pairs are
// computed once and shared by all heads; two channels per thread and access.  head_dim <= 256, even D/2.
__global__ void __launch_bounds__(256) rope_scatter_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ q_out,
                                                           __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                                                           const float* __restrict__ inv_freq, const int32_t* __restrict__ pos3,
                                                           int S, int q_heads, int kv_heads, int D, int kv_offset, int use_mrope,
                                                           int sec0, int sec1) {
    __shared__ float s_sn[128], s_cs[128];
    const int s = blockIdx.x, half = D >> 1;
    for (int d = threadIdx.x; d < half; d += 256) {
        int pos;
        if (use_mrope) pos = pos3[(d < sec0 ? 0 : (d < sec1 ? 1 : 2)) * S + s];
        else pos = kv_offset + s;
        sincosf((float)pos * inv_freq[d], &s_sn[d], &s_cs[d]);
    }
    __syncthreads();
    const int width = (q_heads + 2 * kv_heads) * D, hp = half >> 1;
    const size_t row = (size_t)(kv_offset + s) * kv_heads * D;
    for (int i = threadIdx.x; i < (q_heads + 2 * kv_heads) * hp; i += 256) {
        const int head = i / hp, d = (i - head * hp) * 2;
        const __nv_bfloat16* src = qkv + (size_t)s * width + (size_t)head * D;
        const uint32_t lo = *reinterpret_cast<const uint32_t*>(src + d), hi = *reinterpret_cast<const uint32_t*>(src + d + half);
        if (head < q_heads + kv_heads) {
            const float a0 = bf16lo(lo), a1 = bf16hi(lo), b0 = bf16lo(hi), b1 = bf16hi(hi);
            const uint32_t o_lo = pack_bf16(a0 * s_cs[d] - b0 * s_sn[d], a1 * s_cs[d + 1] - b1 * s_sn[d + 1]);
            const uint32_t o_hi = pack_bf16(b0 * s_cs[d] + a0 * s_sn[d], b1 * s_cs[d + 1] + a1 * s_sn[d + 1]);
            __nv_bfloat16* dst = head < q_heads ? q_out + ((size_t)s * q_heads + head) * D
                                                : k_cache + row + (size_t)(head - q_heads) * D;
            *reinterpret_cast<uint32_t*>(dst + d) = o_lo;
            *reinterpret_cast<uint32_t*>(dst + d + half) = o_hi;
        } else {
            __nv_bfloat16* dst = v_cache + row + (size_t)(head - q_heads - kv_heads) * D;
            *reinterpret_cast<uint32_t*>(dst + d) = lo;
            *reinterpret_cast<uint32_t*>(dst + d + half) = hi;
        }
    }
}

// Tensor parallel prefill: resid += sum, `sum` being the all-reduced fp32 output of a row-parallel linear.
__global__ void __launch_bounds__(256) add_rows_kernel(float* __restrict__ resid, const float* __restrict__ sum,
                                                       size_t n_pairs) {
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n_pairs; i += (size_t)gridDim.x * 256) {
        const float2 old = reinterpret_cast<const float2*>(resid)[i];
        const float2 s = reinterpret_cast<const float2*>(sum)[i];
        reinterpret_cast<float2*>(resid)[i] = make_float2(old.x + s.x, old.y + s.y);
    }
}

// ---- tensor parallel prefill over peer memory: reduce-scatter + all-gather of a row-parallel partial ------------
// Every rank holds an fp32 partial [S, H] of a row-parallel linear and needs resid += sum over ranks.  Rank j owns
// the rows [j * rows_per, (j + 1) * rows_per) of the sum:
//   1. scatter: each rank stores slice j of its partial into its slot of rank j's receive buffer (peer stores over
//      NVLink; (tp - 1) / tp of one copy leaves the GPU instead of tp - 1 whole copies);
//   2. reduce + gather: the owner adds the tp slots in rank order and stores the summed rows into every rank's gather
//      buffer;
//   3. add: resid += gather buffer.
// A step is complete for its readers when the writer's flag word on the reader carries the exchange count: every
// block orders its stores with a system-scope fence and draws a ticket, the block that draws the last one publishes.
// Two buffers used alternately (o_proj, down): a rank can be at most one exchange ahead of a peer.  Every wait is
// bounded (PeerWait) and raises *error = 3.
struct PeerXchgParams {
    const float* src;            // 1: this rank's partial [S, H]
    float* recv[8];              // 1: this rank's slot in rank r's receive buffer [rows_per, H]
    const float* recv_local;     // 2: local receive buffer, tp slots of slot_floats each
    float* gather[8];            // 2: rank r's gather buffer [S, H]
    const float* gather_local;   // 3
    float* resid;                // 3
    unsigned int* flag[8];       // 1, 2: this rank's flag word on rank r (scatter flags in 1, gather flags in 2)
    const unsigned int* flags_local;   // 2, 3: the flag words the ranks publish here
    int n_peers, rank, S, H, rows_per;
    size_t slot_floats;
    unsigned int* epoch;         // local exchange count: advanced by step 1, read by steps 2 and 3
    unsigned int* ticket;        // local, zero between launches
    int* error;
    volatile int* error_host;
    unsigned long long wait_ns;
};

__device__ __forceinline__ void peer_publish(const PeerXchgParams& p, const bool advance) {
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int t = atomicAdd(p.ticket, 1u);
        if (t == gridDim.x - 1) {
            *p.ticket = 0u;
            unsigned int e = *reinterpret_cast<volatile unsigned int*>(p.epoch);
            if (advance) { e += 1u; *p.epoch = e; }
            __threadfence_system();
            for (int r = 0; r < p.n_peers; ++r)
                asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.flag[r]), "r"(e) : "memory");
        }
    }
}

// All ranks' flags have reached the local exchange count (or the wait budget ran out).
__device__ __forceinline__ void peer_await(const PeerXchgParams& p) {
    if ((int)threadIdx.x < p.n_peers) {
        const unsigned int want = __ldcg(p.epoch);
        PeerWait pw = peer_wait_begin(p.error);
        int spins = 0;
        for (;;) {
            unsigned int v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p.flags_local + threadIdx.x) : "memory");
            if ((int)(v - want) >= 0 || pw.dead) break;
            if ((++spins & 15) == 0) {
                if (peer_wait_expired(pw, p.error, p.error_host, p.wait_ns)) break;
                __nanosleep(64);
            }
        }
    }
    __syncthreads();
}

__global__ void __launch_bounds__(256) peer_scatter_rows_kernel(const PeerXchgParams p) {
    const size_t row4 = (size_t)p.H / 4, n4 = (size_t)p.S * row4, per4 = (size_t)p.rows_per * row4;
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n4; i += (size_t)gridDim.x * 256) {
        const int owner = (int)(i / per4);
        reinterpret_cast<float4*>(p.recv[owner])[i - (size_t)owner * per4] = reinterpret_cast<const float4*>(p.src)[i];
    }
    peer_publish(p, /*advance=*/true);
}

__global__ void __launch_bounds__(256) peer_reduce_gather_kernel(const PeerXchgParams p) {
    peer_await(p);
    const size_t row4 = (size_t)p.H / 4, per4 = (size_t)p.rows_per * row4, first4 = (size_t)p.rank * per4;
    const size_t total4 = (size_t)p.S * row4;
    const size_t mine4 = first4 >= total4 ? 0 : (total4 - first4 < per4 ? total4 - first4 : per4);
    const size_t slot4 = p.slot_floats / 4;
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < mine4; i += (size_t)gridDim.x * 256) {
        float4 a = __ldcg(reinterpret_cast<const float4*>(p.recv_local) + i);
        for (int r = 1; r < p.n_peers; ++r) {
            const float4 b = __ldcg(reinterpret_cast<const float4*>(p.recv_local) + (size_t)r * slot4 + i);
            a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        }
        for (int r = 0; r < p.n_peers; ++r) reinterpret_cast<float4*>(p.gather[r])[first4 + i] = a;
    }
    peer_publish(p, /*advance=*/false);
}

__global__ void __launch_bounds__(256) peer_add_gathered_kernel(const PeerXchgParams p) {
    peer_await(p);
    const size_t n4 = (size_t)p.S * p.H / 4;
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n4; i += (size_t)gridDim.x * 256) {
        const float4 a = __ldcg(reinterpret_cast<const float4*>(p.gather_local) + i);
        const float4 o = reinterpret_cast<const float4*>(p.resid)[i];
        reinterpret_cast<float4*>(p.resid)[i] = make_float4(o.x + a.x, o.y + a.y, o.z + a.z, o.w + a.w);
    }
}

}  // namespace efm
