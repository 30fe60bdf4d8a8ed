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
// of thread count and summation order.  One block of 1024 threads; each warp owns a contiguous
// id segment and reads it 4 ids per lane, so every pass over the vocabulary is coalesced; the
// logits (<= 0.6 MB) are L2-resident when this runs.
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
    unsigned long long* xchg;  // [1040] scratch of the multi-block form: segment masses [512] | masses before the pick [512] | pick
    // Tensor parallel, greedy only (tp_n > 1): part_val / part_idx are this rank's maxima with row indices local to its
    // vocabulary shard; the ranks exchange one 8-byte word {fp32 maximum, exchange count << 18 | global id} each through
    // peer memory instead of gathering the logits.
    int tp_n, tp_rank, tp_vocab_offset;
    unsigned int* tp_count;                  // exchanges this context has completed (device word, advanced here)
    unsigned long long* tp_peer_slot[8];     // rank r's receive words [2][tp_n] (ours included)
    int* tp_error;                           // DecodeState.error and its host-mapped copy, raised when a wait runs out
    volatile int* tp_error_host;
    unsigned long long tp_wait_ns;
};

__device__ __forceinline__ void st_sys_b64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_sys_b64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.b64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

// Sampler scratch is one allocation of sample_scratch_words(vocab) 32-bit words: the integer weights,
// then (16-byte aligned) the exchange area of the multi-block form.
inline size_t sample_scratch_words(int vocab) { return (size_t)((vocab + 3) & ~3) + 2 * 1040; }
inline unsigned long long* sample_xchg(uint32_t* wbuf, int vocab) {
    return reinterpret_cast<unsigned long long*>(wbuf + ((vocab + 3) & ~3));
}

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

// four 128-id strides of integer weights for one lane (ids past `hi` read as 0)
__device__ __forceinline__ void load_weights16(const uint32_t* wbuf, int base0, int hi, bool vec_ok, unsigned int (&w)[4][4]) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int base = base0 + u * 128;
        if (vec_ok && base < hi) {
            const uint4 v = *reinterpret_cast<const uint4*>(wbuf + base);
            w[u][0] = v.x; w[u][1] = v.y; w[u][2] = v.z; w[u][3] = v.w;
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) w[u][e] = (!vec_ok && base + e < hi) ? wbuf[base + e] : 0u;
        }
    }
}

__global__ void __launch_bounds__(1024) sample_kernel(const SampleParams p) {
    constexpr int NT = 1024;
    __shared__ unsigned long long scan_tmp[33];
    __shared__ float rv[32];
    __shared__ int ri[32];
    __shared__ unsigned long long cta_tot[16];
    __shared__ unsigned long long s_before_seg;
    __shared__ int s_ow;

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
    if (p.tp_n > 1) {
        // every rank publishes its (maximum, global id) into its word of every rank's receive row and reads the others':
        // value and count travel in one 64-bit word, two rows alternate (a rank is never two exchanges ahead: the layers'
        // exchanges lie between two of these).  Waits are limited by time; on expiry the error word is raised.
        __shared__ unsigned int s_epoch;
        if (tid == 0) {
            const unsigned int epoch = *p.tp_count + 1u;
            s_epoch = epoch;
            int gid = ri[0] + p.tp_vocab_offset;
            if (ri[0] < 0 || ri[0] == 0x7fffffff) gid = 0x3ffff;                // nothing found on this rank
            const unsigned long long word = (unsigned long long)__float_as_uint(rv[0]) |
                                            ((unsigned long long)(((epoch & 0x3fffu) << 18) | ((unsigned int)gid & 0x3ffffu)) << 32);
            const int row = (int)(epoch & 1u) * p.tp_n;
            for (int r = 0; r < p.tp_n; ++r) st_sys_b64(p.tp_peer_slot[r] + row + p.tp_rank, word);
        }
        __syncthreads();
        if (tid < p.tp_n) {
            const unsigned int epoch = s_epoch;
            const unsigned long long* src = p.tp_peer_slot[p.tp_rank] + (int)(epoch & 1u) * p.tp_n + tid;
            PeerWait pw = peer_wait_begin(p.tp_error);
            unsigned long long w = 0ull;
            unsigned int spins = 0;
            bool ok = false;
            for (;;) {
                w = ld_sys_b64(src);
                ok = ((unsigned int)(w >> 50) & 0x3fffu) == (epoch & 0x3fffu);
                if (ok || pw.dead) break;
                if ((++spins & 15u) == 0u) {
                    if (peer_wait_expired(pw, p.tp_error, p.tp_error_host, p.tp_wait_ns)) break;
                    __nanosleep(32);
                }
            }
            rv[tid] = ok ? __uint_as_float((unsigned int)w) : -INFINITY;
            ri[tid] = ok ? (int)((unsigned int)(w >> 32) & 0x3ffffu) : 0x7fffffff;
        }
        __syncthreads();
        if (tid == 0) {
            float v = rv[0];
            int ix = ri[0];
            for (int r = 1; r < p.tp_n; ++r)
                if (rv[r] > v || (rv[r] == v && ri[r] < ix)) { v = rv[r]; ix = ri[r]; }
            rv[0] = v;
            ri[0] = ix;
            *p.tp_count = s_epoch;
        }
        __syncthreads();
    }
    const float M = rv[0];
    int token = ri[0];
    if (token < 0 || token >= p.vocab) token = p.vocab - 1;     // all-NaN / empty guard

    if (p.temperature >= 1e-6f) {
        const float inv_t = 1.0f / p.temperature;
        double top_p = (double)p.top_p;
        top_p = top_p > 1.0 ? 1.0 : (top_p < 1e-9 ? 1e-9 : top_p);
        const uint32_t step = p.state != nullptr ? (uint32_t)p.state->step : p.rng_step;
        // The blocks of the launch form one thread-block cluster (1 block: the same code with trivial barriers).
        // Each warp of each block owns one contiguous id segment (a multiple of 128 ids) and walks it 128 ids at a
        // time, 4 consecutive ids per lane: every pass over the vocabulary is coalesced.  All masses are exact
        // integers, so the pick does not depend on how many blocks share the work.
        const int ncta = (int)gridDim.x, cta = (int)blockIdx.x;
        const int nseg = 32 * ncta;
        const int seg = ((p.vocab + nseg * 128 - 1) / (nseg * 128)) * 128;
        const int gs = cta * 32 + warp;
        const int seg_lo = min(p.vocab, gs * seg), seg_hi = min(p.vocab, seg_lo + seg);
        const bool vec_ok = (p.vocab & 3) == 0;
        unsigned long long* xseg = p.xchg;
        unsigned long long* xbefore = p.xchg + 512;
        unsigned int* xsel = reinterpret_cast<unsigned int*>(p.xchg + 1024);
        auto cluster_sync = [&]() {
            if (ncta > 1) asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
            else __syncthreads();
        };
        // sum over all segments of an exchanged array: warp c adds block c's 32 values -> cta_tot[c]
        auto block_totals = [&](const unsigned long long* arr) {
            if (warp < ncta) {
                unsigned long long v = __ldcg(arr + warp * 32 + lane);
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (lane == 0) cta_tot[warp] = v;
            }
            __syncthreads();
        };

        // pass 0: integer weights (four 128-id strides per trip so that the loads overlap); their sum is the
        // candidate mass of round 0 (every token is a candidate then), which saves that round's first scan
        unsigned long long mass0 = 0ull;
        for (int base0 = seg_lo + lane * 4; base0 < seg_hi; base0 += 512) {
            float lg[4][4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int base = base0 + u * 128;
                if (vec_ok && base < seg_hi) {
                    const float4 v = *reinterpret_cast<const float4*>(p.logits + base);
                    lg[u][0] = v.x; lg[u][1] = v.y; lg[u][2] = v.z; lg[u][3] = v.w;
                } else {
#pragma unroll
                    for (int e = 0; e < 4; ++e) lg[u][e] = base + e < seg_hi ? p.logits[base + e] : -INFINITY;
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int base = base0 + u * 128;
                unsigned int w4[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float s = expf((lg[u][e] - M) * inv_t) * 2147483648.0f;
                    w4[e] = s >= 2147483648.0f ? 0x7fffffffu : (unsigned int)s;   // NaN -> 0
                    if (base + e < seg_hi) mass0 += w4[e];
                }
                if (vec_ok) { if (base < seg_hi) *reinterpret_cast<uint4*>(p.wbuf + base) = make_uint4(w4[0], w4[1], w4[2], w4[3]); }
                else {
#pragma unroll
                    for (int e = 0; e < 4; ++e) if (base + e < seg_hi) p.wbuf[base + e] = w4[e];
                }
            }
        }
        __syncthreads();

        unsigned int piv_w = 0u;          // last rejected token (w, id); none yet
        int piv_id = -1;
        double target = 0.0;
        bool accepted = false;
#pragma unroll 1
        for (uint32_t round = 0; round < 32u && !accepted; ++round) {
            // (a) candidate mass per segment
            unsigned long long mass = round == 0 ? mass0 : 0ull;
            for (int base0 = seg_lo + lane * 4; round > 0 && base0 < seg_hi; base0 += 512) {
                unsigned int w4[4][4];
                load_weights16(p.wbuf, base0, seg_hi, vec_ok, w4);
#pragma unroll
                for (int u = 0; u < 4; ++u)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int i = base0 + u * 128 + e;
                        const bool cand = piv_id < 0 ? true : (w4[u][e] > piv_w || (w4[u][e] == piv_w && i < piv_id));
                        if (cand) mass += w4[u][e];
                    }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mass += __shfl_xor_sync(0xffffffffu, mass, o);
            if (lane == 0) xseg[gs] = mass;
            cluster_sync();
            // (b) owner segment of r: first the owning block, then the segment inside it
            block_totals(xseg);
            unsigned long long Wc = 0ull;
            for (int c = 0; c < ncta; ++c) Wc += cta_tot[c];
            if (round == 0) target = (double)Wc * top_p;
            if (Wc == 0ull) break;
            const uint32_t x = philox4x32_10_first(step, round, (uint32_t)(p.seed & 0xffffffffull),
                                                   (uint32_t)(p.seed >> 32));
            const unsigned long long r =
                __double2ull_rd(__dmul_rn(__dmul_rn((double)x, (double)Wc), 2.3283064365386963e-10));
            int oc = 0;
            unsigned long long before_cta = 0ull;
            for (int c = 0; c < ncta; ++c) {
                if (r >= before_cta + cta_tot[c]) before_cta += cta_tot[c]; else { oc = c; break; }
            }
            if (warp == 0) {
                const unsigned long long v = __ldcg(xseg + oc * 32 + lane);
                unsigned long long incl = v;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const unsigned long long u = __shfl_up_sync(0xffffffffu, incl, o);
                    if (lane >= o) incl += u;
                }
                const unsigned long long rr = r - before_cta, excl = incl - v;
                if (lane == 0) { s_ow = oc * 32; s_before_seg = before_cta; }
                __syncwarp();
                if (excl <= rr && rr < incl) { s_ow = oc * 32 + lane; s_before_seg = before_cta + excl; }
            }
            __syncthreads();
            const int ow = s_ow;
            const unsigned long long before_seg = s_before_seg;
            // (c) inside the owner segment: a few consecutive ids per thread, exact block scan
            if (cta == ow / 32) {            // the block that wrote the owner segment's weights
                const int olo = min(p.vocab, ow * seg), ohi = min(p.vocab, olo + seg);
                const int per = (ohi - olo + NT - 1) / NT;
                const int lo = min(ohi, olo + tid * per), hi = min(ohi, lo + per);
                unsigned long long m2 = 0ull;
                for (int i = lo; i < hi; ++i) {
                    const unsigned int w = p.wbuf[i];
                    if (piv_id < 0 || w > piv_w || (w == piv_w && i < piv_id)) m2 += w;
                }
                unsigned long long tot2;
                const unsigned long long incl = block_scan_u64(m2, scan_tmp, &tot2) + before_seg;
                const unsigned long long excl = incl - m2;
                if (excl <= r && r < incl) {
                    unsigned long long run = excl;
                    for (int i = lo; i < hi; ++i) {
                        const unsigned int w = p.wbuf[i];
                        if (piv_id < 0 || w > piv_w || (w == piv_w && i < piv_id)) {
                            run += w;
                            if (run > r) { xsel[0] = (unsigned int)i; xsel[1] = w; break; }
                        }
                    }
                }
            }
            cluster_sync();
            const int j = (int)__ldcg(xsel);
            const unsigned int wj = __ldcg(xsel + 1);
            // (d) mass strictly before j in (w desc, id asc) order
            unsigned long long before = 0ull;
            for (int base0 = seg_lo + lane * 4; base0 < seg_hi; base0 += 512) {
                unsigned int w4[4][4];
                load_weights16(p.wbuf, base0, seg_hi, vec_ok, w4);
#pragma unroll
                for (int u = 0; u < 4; ++u)
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        if (w4[u][e] > wj || (w4[u][e] == wj && base0 + u * 128 + e < j)) before += w4[u][e];
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) before += __shfl_xor_sync(0xffffffffu, before, o);
            if (lane == 0) xbefore[gs] = before;
            cluster_sync();
            block_totals(xbefore);
            unsigned long long E = 0ull;
            for (int c = 0; c < ncta; ++c) E += cta_tot[c];
            if ((double)E < target) { accepted = true; token = j; }
            else { piv_w = wj; piv_id = j; }
            __syncthreads();
        }
    }

    if (tid == 0 && blockIdx.x == 0) {
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
