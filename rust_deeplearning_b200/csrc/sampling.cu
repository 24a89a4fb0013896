// Sampling over float logits, one block per row.
//
// Order of operations (reference: rustml/nlp/main/src/core/generator.rs:176-201):
//   temperature < 1e-7 -> arg max, first maximum wins     sampling.rs:8-18
//   repetition penalty: x > 0 ? x / p : x * p             sampling.rs:23-34
//   x / temperature
//   top-k: keep values >= the k-th largest (ties kept)    sampling.rs:38-52
//   top-p: keep the smallest set of most probable tokens whose mass reaches p   sampling.rs:56-87
//   draw: softmax, first index whose cumulative probability exceeds r           sampling.rs:91-106
// (sampling.rs = rustml/nlp/main/src/core/sampling.rs).  Differences, all by design:
//   - the penalty is applied once per distinct token of the history (the reference applies it
//     once per occurrence);
//   - tokens whose probability ties with the last kept one in top-p are all kept;
//   - r comes from a counter-based generator keyed by (seed, the row's stream id, the row's
//     step), so a row's draw does not depend on what else is in the batch (the reference draws
//     from an unseeded thread-local generator, generator.rs:199).
#include "api.h"
#include "common.cuh"
#include "launch.cuh"

namespace {

constexpr int SAMPLE_THREADS = 1024;

// order-preserving map from float to unsigned
__device__ __forceinline__ unsigned ordered_key(float f) {
    const unsigned u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__host__ __device__ inline unsigned long long splitmix64(unsigned long long x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
// uniform in [0, 1) with 24 bits
__host__ __device__ inline float uniform_from(unsigned long long seed, unsigned long long stream, unsigned long long step) {
    unsigned long long h = splitmix64(seed);
    h = splitmix64(h ^ (stream * 0xD6E8FEB86659FD93ull));
    h = splitmix64(h ^ (step * 0xA5A5A5A5A5A5A5A5ull + 1));
    return (float)(h >> 40) * (1.0f / 16777216.0f);
}

__device__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

__device__ unsigned block_count(unsigned v, unsigned* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        unsigned t = lane < nwarps ? scratch[lane] : 0u;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

__global__ void __launch_bounds__(SAMPLE_THREADS) sample_kernel(int* __restrict__ out_tokens, const float* __restrict__ logits,
                                                                int vocab, SamplingArgs prm,
                                                                const unsigned long long* __restrict__ row_stream,
                                                                const int* __restrict__ row_step,
                                                                const int* __restrict__ history,
                                                                const int* __restrict__ history_start,
                                                                float* __restrict__ work) {
    __shared__ float fscratch[33];
    __shared__ unsigned uscratch[33];
    __shared__ float best_val[32];
    __shared__ int best_idx[32];
    __shared__ float chunk_sum[SAMPLE_THREADS];
    __shared__ int chosen;
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const int row = blockIdx.x, tid = threadIdx.x;
    const float* x = logits + (long long)row * vocab;

    if (prm.temperature < 1e-7f) {
        // ---- arg max, smallest index among equal maxima ----
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
            const float v = x[i];
            if (v > bv) { bv = v; bi = i; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if ((tid & 31) == 0) { best_val[tid >> 5] = bv; best_idx[tid >> 5] = bi; }
        __syncthreads();
        if (tid < 32) {
            bv = best_val[tid];
            bi = best_idx[tid];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
            }
            if (tid == 0) out_tokens[row] = bi == 0x7fffffff ? 0 : bi;
        }
        return;
    }

    float* w = work + (long long)row * vocab;
    // ---- penalty (once per distinct token, from the untouched logits) and temperature ----
    for (int i = tid; i < vocab; i += SAMPLE_THREADS) w[i] = x[i] / prm.temperature;
    __syncthreads();
    if (prm.repetition_penalty != 1.0f && history) {
        const int hb = history_start[row], he = history_start[row + 1];
        for (int i = hb + tid; i < he; i += SAMPLE_THREADS) {
            const int tok = history[i];
            if (tok >= 0 && tok < vocab) {
                const float v = x[tok];
                w[tok] = (v > 0.f ? v / prm.repetition_penalty : v * prm.repetition_penalty) / prm.temperature;  // equal writers
            }
        }
        __syncthreads();
    }
    // ---- top-k: threshold = k-th largest value, found bit by bit on ordered keys ----
    if (prm.top_k > 0 && prm.top_k < vocab) {
        unsigned thr = 0;
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned cand = thr | (1u << bit);
            unsigned c = 0;
            for (int i = tid; i < vocab; i += SAMPLE_THREADS) c += ordered_key(w[i]) >= cand;
            if (block_count(c, uscratch) >= (unsigned)prm.top_k) thr = cand;
        }
        for (int i = tid; i < vocab; i += SAMPLE_THREADS)
            if (ordered_key(w[i]) < thr) w[i] = -INFINITY;
        __syncthreads();
    }
    // ---- maximum and normaliser ----
    float mx = -INFINITY;
    for (int i = tid; i < vocab; i += SAMPLE_THREADS) mx = fmaxf(mx, w[i]);
    mx = block_max(mx, fscratch);
    // ---- top-p: smallest key whose strictly-greater mass stays below p ----
    if (prm.top_p < 1.0f) {
        float z = 0.f;
        for (int i = tid; i < vocab; i += SAMPLE_THREADS) z += expf(w[i] - mx);
        z = block_sum(z, fscratch);
        const float need = prm.top_p * z;
        // mass_gt(key) is non-increasing in key; find the smallest key with mass_gt(key) < need
        unsigned lo_key = 0;  // invariant: mass_gt(lo_key - 1) >= need, built from the top bit down
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned cand = lo_key | (1u << bit);
            // is mass_gt(cand - 1) >= need, i.e. is the mass of keys >= cand still enough?
            float s = 0.f;
            for (int i = tid; i < vocab; i += SAMPLE_THREADS)
                if (ordered_key(w[i]) >= cand) s += expf(w[i] - mx);
            s = block_sum(s, fscratch);
            if (s >= need) lo_key = cand;
        }
        // lo_key is the largest key with mass(keys >= lo_key) >= need: the last value that is kept
        for (int i = tid; i < vocab; i += SAMPLE_THREADS)
            if (ordered_key(w[i]) < lo_key) w[i] = -INFINITY;
        __syncthreads();
    }
    // ---- draw: first index whose cumulative mass exceeds r * total ----
    const int per = (vocab + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    const int b = tid * per, e = min(vocab, b + per);
    float local = 0.f;
    for (int i = b; i < e; ++i) local += expf(w[i] - mx);
    chunk_sum[tid] = local;
    if (tid == 0) chosen = -1;
    __syncthreads();
    if (tid == 0) {
        float total = 0.f;
        for (int i = 0; i < SAMPLE_THREADS; ++i) total += chunk_sum[i];
        const float r = uniform_from(prm.seed, row_stream ? row_stream[row] : (unsigned long long)row,
                                     row_step ? (unsigned long long)row_step[row] : 0ull);
        const float target = r * total;
        float c = 0.f;
        int pick = -1, chunk = -1;
        for (int i = 0; i < SAMPLE_THREADS; ++i) {
            if (target < c + chunk_sum[i]) { chunk = i; break; }
            c += chunk_sum[i];
        }
        if (chunk >= 0) {
            const int cb = chunk * per, ce = min(vocab, cb + per);
            for (int i = cb; i < ce; ++i) {
                c += expf(w[i] - mx);
                if (target < c) { pick = i; break; }
            }
            if (pick < 0) {  // rounding inside the chunk: its last token with mass
                for (int i = ce - 1; i >= cb; --i)
                    if (w[i] != -INFINITY) { pick = i; break; }
            }
        }
        chosen = pick;
    }
    __syncthreads();
    if (chosen < 0) {
        // rounding at the very end of the row: the last token that has mass
        int last = -1;
        for (int i = tid; i < vocab; i += SAMPLE_THREADS)
            if (w[i] != -INFINITY) last = max(last, i);
        const float lf = block_max((float)last, fscratch);
        if (tid == 0) chosen = (int)lf;
        __syncthreads();
    }
    if (tid == 0) out_tokens[row] = chosen < 0 ? 0 : chosen;
}

}  // namespace

extern "C" float rdl_sampling_uniform(unsigned long long seed, unsigned long long stream, unsigned long long step) {
    return uniform_from(seed, stream, step);
}

extern "C" int rdl_sample(int* out_tokens, const float* logits, int n_rows, int vocab, const SamplingArgs* prm,
                          const unsigned long long* row_stream, const int* row_step,
                          const int* history, const int* history_start, float* work, void* stream) {
    RDL_REQUIRE(out_tokens && logits && prm, "sample: missing operand");
    RDL_REQUIRE(n_rows >= 0 && vocab > 0, "sample: bad sizes rows=%d vocab=%d", n_rows, vocab);
    RDL_REQUIRE(vocab < (1 << 24), "sample: vocabulary of %d is too large", vocab);
    RDL_REQUIRE(prm->temperature >= 0.f, "sample: temperature must not be negative");
    if (prm->temperature >= 1e-7f) {
        RDL_REQUIRE(work, "sample: temperature sampling needs a work buffer of rows x vocab floats");
        RDL_REQUIRE(prm->top_k >= 0, "sample: top_k must not be negative");
        RDL_REQUIRE(prm->top_p > 0.f, "sample: top_p must be positive");
        RDL_REQUIRE(prm->repetition_penalty > 0.f, "sample: repetition_penalty must be positive");
        RDL_REQUIRE(prm->repetition_penalty == 1.0f || !history || history_start, "sample: history without offsets");
    }
    if (n_rows == 0) return 0;
    RDL_CHECK_EX(rdl_launch(sample_kernel, dim3(n_rows), dim3(SAMPLE_THREADS), 0, (cudaStream_t)stream, out_tokens, logits, vocab,
                            *prm, row_stream, row_step, history, history_start, work), "sample");
    return 0;
}
