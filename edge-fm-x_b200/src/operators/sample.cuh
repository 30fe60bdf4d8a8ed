// Sampler + decode-state advance, one launch per step.
// Replaces the reference's sampler kernels and its per-step state kernels:
//   greedy   topKStage1Greedy/topKStage2Greedy           src/layers/sampler.cu:38-105
//   sampled  OnlineSoftmax + SamplingFromProb (Philox)    src/layers/sampler.cu:270-296
//   advance  finalize_decode_token / increment_* kernels  decode_runtime_kernels.cu:40-65
// Greedy: argmax, ties -> lowest id.  Temperature > 0: seeded top-p by rejection, in exact
// integer arithmetic (the reference has no top-p; the rule is written out here and restated on
// the CPU by the test oracle):
//   w_i    = min(floor(exp((l_i - max) / T) * 2^31), 2^31 - 1);  W = sum w_i
//   order  = (w descending, id ascending); the nucleus is the shortest prefix of that order
//            whose mass reaches target = double(W) * double(top_p), i.e. token j belongs to it
//            iff the mass E_j strictly before j in that order has double(E_j) < target.
//   round k = 0,1,..: candidates = tokens before the last rejected one in that order (all
//            tokens with w > 0 at k = 0), Wc their mass;
//            x = Philox4x32-10(key = seed, counter = (step, k, 0, 0))[0];
//            r = floor(double(x) * double(Wc) * 2^-32); j = first candidate, in ascending id
//            order, whose running candidate mass exceeds r; accept j if it is in the nucleus,
//            else reject it (which also rules out everything after it in the order).
// Accepted tokens are distributed exactly as nucleus sampling; a round succeeds with
// probability >= top_p, so 1-2 rounds are typical.  Integer mass makes the result independent
// of thread count and summation order.  One block of 1024 threads; the logits (<= 0.6 MB) are
// L2-resident when this runs.
#pragma once
#include "common.cuh"

namespace efm {

struct SampleParams {
    const float* logits;
    int vocab;
    const float* part_val;   // per-block maxima from the logits GEMV (n_part may be 0)
    const int* part_idx;
    int n_part;
    float temperature, top_p;
    unsigned long long seed;
    uint32_t rng_step;       // used when state == nullptr
    DecodeState* state;
    int32_t* tokens_out;     // response buffer, written at state->step
    int max_response;
    int32_t* token_single;   // optional single output
    int advance;             // 1: move kv_len / positions / step on to the next decode step
    uint32_t* wbuf;          // [vocab] scratch: integer weights
};

#ifndef EFM_DECLARATIONS_ONLY   // kernel bodies are compiled in exactly one translation unit
__device__ __forceinline__ uint32_t philox4x32_10_first(uint32_t c0, uint32_t c1, uint32_t k0, uint32_t k1) {
    uint32_t c[4] = {c0, c1, 0u, 0u};
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
        const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
        const uint32_t n0 = hi1 ^ c[1] ^ k0, n2 = hi0 ^ c[3] ^ k1;
        c[0] = n0; c[1] = lo1; c[2] = n2; c[3] = lo0;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    return c[0];
}

// inclusive block scan over 1024 threads (exact 64-bit integers); returns the inclusive prefix,
// total in *total.  `tmp` is a 33-entry shared array.
__device__ __forceinline__ unsigned long long block_scan_u64(unsigned long long v, unsigned long long* tmp,
                                                             unsigned long long* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long u = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += u;
    }
    __syncthreads();                 // tmp may still be read from a previous scan
    if (lane == 31) tmp[warp] = v;
    __syncthreads();
    if (warp == 0) {
        unsigned long long w = tmp[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned long long u = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += u;
        }
        tmp[lane] = w;
        if (lane == 31) tmp[32] = w;
    }
    __syncthreads();
    if (warp > 0) v += tmp[warp - 1];
    *total = tmp[32];
    return v;
}

__global__ void __launch_bounds__(1024) sample_kernel(const SampleParams p) {
    constexpr int NT = 1024;
    __shared__ unsigned long long scan_tmp[33];
    __shared__ float rv[32];
    __shared__ int ri[32];
    __shared__ unsigned int sel_w;
    __shared__ int sel_id;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    pdl_launch_dependents();
    pdl_wait();

    // ---- max / argmax (ties -> lowest id) -------------------------------------------------
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    if (p.n_part > 0) {
        for (int i = tid; i < p.n_part; i += NT) {
            const float v = p.part_val[i];
            const int ix = p.part_idx[i];
            if (v > bv || (v == bv && ix < bi)) { bv = v; bi = ix; }
        }
    } else {
        for (int i = tid; i < p.vocab; i += NT) {
            const float v = p.logits[i];
            if (v > bv) { bv = v; bi = i; }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) { rv[warp] = bv; ri[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        bv = rv[lane];
        bi = ri[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) { rv[0] = bv; ri[0] = bi; }
    }
    __syncthreads();
    const float M = rv[0];
    int token = ri[0];
    if (token < 0 || token >= p.vocab) token = p.vocab - 1;     // all-NaN / empty guard
    if (tid == 0) { sel_id = token; sel_w = 0u; }

    if (p.temperature >= 1e-6f) {
        const float inv_t = 1.0f / p.temperature;
        double top_p = (double)p.top_p;
        top_p = top_p > 1.0 ? 1.0 : (top_p < 1e-9 ? 1e-9 : top_p);
        const uint32_t step = p.state != nullptr ? (uint32_t)p.state->step : p.rng_step;
        const int per = (p.vocab + NT - 1) / NT;          // contiguous id slice per thread
        const int lo = min(p.vocab, tid * per), hi = min(p.vocab, lo + per);
        // integer weights
        for (int i = lo; i < hi; ++i) {
            const float s = expf((p.logits[i] - M) * inv_t) * 2147483648.0f;
            p.wbuf[i] = s >= 2147483648.0f ? 0x7fffffffu : (unsigned int)s;   // NaN -> 0
        }
        unsigned int piv_w = 0u;          // last rejected token (w, id); none yet
        int piv_id = -1;
        double target = 0.0;
        bool accepted = false;
#pragma unroll 1
        for (uint32_t round = 0; round < 32u && !accepted; ++round) {
            // candidate mass of this thread's slice
            unsigned long long mass = 0ull;
            for (int i = lo; i < hi; ++i) {
                const unsigned int w = p.wbuf[i];
                const bool cand = piv_id < 0 ? (w > 0u) : (w > piv_w || (w == piv_w && i < piv_id));
                if (cand) mass += w;
            }
            unsigned long long Wc;
            const unsigned long long incl = block_scan_u64(mass, scan_tmp, &Wc);
            if (round == 0) target = (double)Wc * top_p;
            if (Wc == 0ull) break;
            const uint32_t x = philox4x32_10_first(step, round, (uint32_t)(p.seed & 0xffffffffull),
                                                   (uint32_t)(p.seed >> 32));
            const unsigned long long r =
                __double2ull_rd(__dmul_rn(__dmul_rn((double)x, (double)Wc), 2.3283064365386963e-10));
            const unsigned long long excl = incl - mass;
            if (excl <= r && r < incl) {
                unsigned long long run = excl;
                for (int i = lo; i < hi; ++i) {
                    const unsigned int w = p.wbuf[i];
                    const bool cand = piv_id < 0 ? (w > 0u) : (w > piv_w || (w == piv_w && i < piv_id));
                    if (cand) { run += w; if (run > r) { sel_id = i; sel_w = w; break; } }
                }
            }
            __syncthreads();
            const int j = sel_id;
            const unsigned int wj = sel_w;
            // mass strictly before j in (w desc, id asc) order
            unsigned long long before = 0ull;
            for (int i = lo; i < hi; ++i) {
                const unsigned int w = p.wbuf[i];
                if (w > wj || (w == wj && i < j)) before += w;
            }
            unsigned long long E;
            block_scan_u64(before, scan_tmp, &E);
            if ((double)E < target) { accepted = true; token = j; }
            else { piv_w = wj; piv_id = j; }
            __syncthreads();
        }
    }

    if (tid == 0) {
        if (p.token_single != nullptr) *p.token_single = token;
        if (p.state != nullptr) {
            const int step = p.state->step;
            if (p.tokens_out != nullptr && step >= 0 && step < p.max_response) p.tokens_out[step] = token;
            p.state->token = token;
            if (p.advance) {
                p.state->kv_len += 1u;
                p.state->pos[0] += 1;
                p.state->pos[1] += 1;
                p.state->pos[2] += 1;
            }
            p.state->step = step + 1;
        }
    }
}

#endif  // EFM_DECLARATIONS_ONLY

}  // namespace efm
