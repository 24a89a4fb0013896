// Sampling over float logits.  Arg max: one block per row.  Temperature sampling: a cluster of up to eight blocks
// per row that keeps the row on the chip (sample_cluster_kernel); rows too long for that, one block per row
// (sample_kernel).
//
// Order of operations (reference: rustml/nlp/main/src/core/generator.rs:176-201):
//   temperature < 1e-7 -> arg max, first maximum wins     sampling.rs:8-18
//   repetition penalty: x > 0 ? x / p : x * p             sampling.rs:23-34
//   x / temperature
//   top-k: keep values >= the k-th largest (ties kept)    sampling.rs:38-52
//   top-p: keep the smallest set of most probable tokens whose mass reaches p   sampling.rs:56-87
//   draw: softmax, first index whose cumulative probability exceeds r           sampling.rs:91-106
// (sampling.rs = rustml/nlp/main/src/core/sampling.rs).  The penalty is applied once per occurrence of a token in
// the history, as the reference's loop over the history does (a token seen n times is penalised n times; every
// application rounds to float like the reference's).  Differences, all by design:
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
    const unsigned u = __float_as_uint(f + 0.0f);          // -0 becomes +0: the two are one value and must have one key
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// One application of the repetition penalty to the logit at `addr`, atomically: the occurrences of a token in the
// history are handled by different threads, and n applications give the same bits in any order.
__device__ __forceinline__ void penalise(float* addr, float penalty) {
    unsigned* bits = reinterpret_cast<unsigned*>(addr);
    unsigned old = *bits, assumed;
    do {
        assumed = old;
        const float v = __uint_as_float(assumed);
        old = atomicCAS(bits, assumed, __float_as_uint(v > 0.f ? v / penalty : v * penalty));
    } while (old != assumed);
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

// The row's token goes to the device vector and, if asked for, straight into pinned host memory as well: the host
// then reads it after the kernel's event, with no copy of its own queued in between.
__device__ __forceinline__ void put_token(int* out_tokens, int* host_tokens, int row, int token) {
    out_tokens[row] = token;
    if (host_tokens) host_tokens[row] = token;
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

__global__ void __launch_bounds__(SAMPLE_THREADS) sample_kernel(int* __restrict__ out_tokens, int* __restrict__ host_tokens, const float* __restrict__ logits,
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
            if (tid == 0) put_token(out_tokens, host_tokens, row, bi == 0x7fffffff ? 0 : bi);
        }
        return;
    }

    float* w = work + (long long)row * vocab;
    // ---- penalty (once per occurrence in the history), then temperature ----
    const bool penalty = prm.repetition_penalty != 1.0f && history;
    for (int i = tid; i < vocab; i += SAMPLE_THREADS) w[i] = penalty ? x[i] : x[i] / prm.temperature;
    __syncthreads();
    if (penalty) {
        const int hb = history_start[row], he = history_start[row + 1];
        for (int i = hb + tid; i < he; i += SAMPLE_THREADS) {
            const int tok = history[i];
            if (tok >= 0 && tok < vocab) penalise(w + tok, prm.repetition_penalty);
        }
        __syncthreads();
        for (int i = tid; i < vocab; i += SAMPLE_THREADS) w[i] = w[i] / prm.temperature;
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
    if (tid == 0) put_token(out_tokens, host_tokens, row, chosen < 0 ? 0 : chosen);
}

// ---------------------------------------------------------------------------------------------
// Temperature sampling with the row on the chip.
//
// The one-block kernel above reads its row from memory once per bit of each threshold search: about 70
// passes over a megabyte at a vocabulary of 256,000 (0.6 ms with top-k, 1.3 ms with top-k and top-p, as
// long as a whole decode step).  Here a cluster of C blocks shares the row: block c holds elements
// [c * 32768, (c + 1) * 32768), thread t of it the 32 consecutive elements from t * 32 on - their ordered keys in
// shared memory, their exp(w - max) in registers.  A round of a threshold search is then 32 compares (and
// adds) per thread, a sum over the block and a sum over the cluster (each block publishes its part in its
// shared memory, a cluster barrier, every block reads all parts in rank order), so every block takes the same
// decisions.  Sums are formed in a fixed order (item, thread tree, rank): a row's result does not depend on
// the run or on the batch.  Same order of operations and same meaning of the options as above.  Measured at
// 256,000 tokens, one row: 34 us plain, 92 us with top-k or top-p, 151 us with both (118 / 606 / 887 / 1,289 us
// in the one-block kernel); two bits a round (three nested candidates) was no faster.
// ---------------------------------------------------------------------------------------------
constexpr int CL_THREADS = 1024, CL_ITEMS = 32, CL_PER_BLOCK = CL_THREADS * CL_ITEMS, CL_MAX_BLOCKS = 8;

__device__ __forceinline__ uint32_t cl_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cl_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cl_map(const void* smem_ptr, uint32_t rank) {
    uint32_t a = (uint32_t)__cvta_generic_to_shared(smem_ptr), r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(rank));
    return r;
}
__device__ __forceinline__ float cl_ld_f32(uint32_t addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ unsigned cl_ld_u32(uint32_t addr) {
    unsigned v;
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}

// Sums over the cluster: the block's value goes into slot[parity], a cluster barrier, all blocks' slots are added (or
// maximised) in rank order.  Two slots alternate so that one barrier a round is enough.
struct ClusterExchange {
    float f[2];
    unsigned u[2];
};
__device__ __forceinline__ float cl_sum_f(float block_value, ClusterExchange* x, int& parity, int n_blocks) {
    if (threadIdx.x == 0) x->f[parity] = block_value;
    cl_sync();
    float t = 0.f;
    for (int r = 0; r < n_blocks; ++r) t += cl_ld_f32(cl_map(&x->f[parity], r));
    parity ^= 1;
    return t;
}
__device__ __forceinline__ float cl_max_f(float block_value, ClusterExchange* x, int& parity, int n_blocks) {
    if (threadIdx.x == 0) x->f[parity] = block_value;
    cl_sync();
    float t = -INFINITY;
    for (int r = 0; r < n_blocks; ++r) t = fmaxf(t, cl_ld_f32(cl_map(&x->f[parity], r)));
    parity ^= 1;
    return t;
}
__device__ __forceinline__ unsigned cl_sum_u(unsigned block_value, ClusterExchange* x, int& parity, int n_blocks) {
    if (threadIdx.x == 0) x->u[parity] = block_value;
    cl_sync();
    unsigned t = 0;
    for (int r = 0; r < n_blocks; ++r) t += cl_ld_u32(cl_map(&x->u[parity], r));
    parity ^= 1;
    return t;
}

// Arg max with the row shared by a cluster: every block takes a contiguous part of the row, the first block picks among
// the blocks' best (the smallest index among equal maxima, as in the one-block kernel).  One block a row reads a
// megabyte through one multiprocessor (14 us at 256,000 tokens); eight read it in 4 us.
__global__ void __launch_bounds__(CL_THREADS, 1) argmax_cluster_kernel(int* __restrict__ out_tokens, int* __restrict__ host_tokens, const float* __restrict__ logits,
                                                                       int vocab, int n_blocks) {
    __shared__ float best_val[32];
    __shared__ int best_idx[32];
    __shared__ float blk_val;
    __shared__ int blk_idx;
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const int row = blockIdx.y, tid = threadIdx.x;
    const int rank = (int)cl_rank();
    const float* x = logits + (long long)row * vocab;
    const int per = (vocab + n_blocks - 1) / n_blocks;
    const int lo = rank * per, hi = min(vocab, lo + per);
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    int i0 = lo;
    if (vocab % 4 == 0 && per % 4 == 0) {
        // sixteen values a thread and round, asked for together (one value at a time is a trip to L2 each: 12 us a row)
        const float4* x4 = reinterpret_cast<const float4*>(x + lo);
        const int n4 = (hi - lo) / 4;
        for (int q = tid; q < n4; q += 4 * CL_THREADS) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                v[u] = q + u * CL_THREADS < n4 ? __ldcg(x4 + q + u * CL_THREADS) : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int at = lo + 4 * (q + u * CL_THREADS);
                if (v[u].x > bv) { bv = v[u].x; bi = at; }
                if (v[u].y > bv) { bv = v[u].y; bi = at + 1; }
                if (v[u].z > bv) { bv = v[u].z; bi = at + 2; }
                if (v[u].w > bv) { bv = v[u].w; bi = at + 3; }
            }
        }
        i0 = lo + 4 * n4;
    }
    for (int i = i0 + tid; i < hi; i += CL_THREADS) {
        const float v = __ldcg(x + i);
        if (v > bv) { bv = v; bi = i; }
    }
    auto better = [](float ov, int oi, float bv, int bi) { return ov > bv || (ov == bv && oi < bi); };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
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
            if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
        }
        if (tid == 0) { blk_val = bv; blk_idx = bi; }
    }
    cl_sync();                 // every block's best is in its shared memory
    if (rank == 0 && tid == 0) {
        for (int r = 1; r < n_blocks; ++r) {
            const float ov = cl_ld_f32(cl_map(&blk_val, r));
            const int oi = (int)cl_ld_u32(cl_map(&blk_idx, r));
            if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
        }
        put_token(out_tokens, host_tokens, row, bi == 0x7fffffff ? 0 : bi);
    }
    cl_sync();                 // no block leaves while the first may still read its shared memory
}

__global__ void __launch_bounds__(CL_THREADS, 1) sample_cluster_kernel(int* __restrict__ out_tokens, int* __restrict__ host_tokens, const float* __restrict__ logits,
                                                                       int vocab, SamplingArgs prm,
                                                                       const unsigned long long* __restrict__ row_stream,
                                                                       const int* __restrict__ row_step,
                                                                       const int* __restrict__ history,
                                                                       const int* __restrict__ history_start,
                                                                       float* __restrict__ work, int n_blocks) {
    extern __shared__ unsigned keys[];                 // [CL_ITEMS][CL_THREADS]: thread t's item i at keys[i * CL_THREADS + t]
    __shared__ float fscratch[33];
    __shared__ unsigned uscratch[33];
    __shared__ float chunk_sum[CL_THREADS];
    __shared__ ClusterExchange xch;
    __shared__ int chosen, s_chunk;
    __shared__ float s_before;
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const int row = blockIdx.y, tid = threadIdx.x;
    const int rank = (int)cl_rank();
    const float* x = logits + (long long)row * vocab;
    const int first = rank * CL_PER_BLOCK + tid * CL_ITEMS;   // this thread's first element
    int parity = 0;

    // ---- penalty (once per occurrence in the history) and temperature ----
    const float* src = x;
    const bool penalty = prm.repetition_penalty != 1.0f && history;
    if (penalty) {
        // the adjusted row goes through memory: a history token may belong to any thread of any block
        float* w = work + (long long)row * vocab;
        for (int i = rank * CL_THREADS + tid; i < vocab; i += n_blocks * CL_THREADS) w[i] = x[i];
        __threadfence();
        cl_sync();
        if (rank == 0) {
            const int hb = history_start[row], he = history_start[row + 1];
            for (int i = hb + tid; i < he; i += CL_THREADS) {
                const int tok = history[i];
                if (tok >= 0 && tok < vocab) penalise(w + tok, prm.repetition_penalty);
            }
            __threadfence();
        }
        cl_sync();
        src = w;
    }
    float e[CL_ITEMS];                                        // the scaled logits first, their exponentials later
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < CL_ITEMS; ++i) {
        const int idx = first + i;
        const float v = idx < vocab ? __ldcg(src + idx) / prm.temperature : -INFINITY;
        e[i] = v;
        keys[i * CL_THREADS + tid] = idx < vocab ? ordered_key(v) : 0u;      // 0 is below every key: "not there"
        mx = fmaxf(mx, v);
    }
    // ---- top-k: threshold = k-th largest value, found bit by bit on ordered keys ----
    if (prm.top_k > 0 && prm.top_k < vocab) {
        unsigned thr = 0;
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned cand = thr | (1u << bit);
            unsigned c = 0;
#pragma unroll
            for (int i = 0; i < CL_ITEMS; ++i) c += keys[i * CL_THREADS + tid] >= cand;
            c = block_count(c, uscratch);
            c = cl_sum_u(c, &xch, parity, n_blocks);
            if (c >= (unsigned)prm.top_k) thr = cand;
            if (c == (unsigned)prm.top_k) break;       // exactly k keys at or above: the lower bits cannot change the set
        }
#pragma unroll
        for (int i = 0; i < CL_ITEMS; ++i)
            if (keys[i * CL_THREADS + tid] < thr) { keys[i * CL_THREADS + tid] = 0u; e[i] = -INFINITY; }
    }
    // ---- maximum, exponentials and normaliser ----
    mx = block_max(mx, fscratch);          // the largest value survives top-k, so the maximum taken before stands
    mx = cl_max_f(mx, &xch, parity, n_blocks);
    float z = 0.f;
#pragma unroll
    for (int i = 0; i < CL_ITEMS; ++i) {
        e[i] = expf(e[i] - mx);            // exp(-inf) = 0 for what is not there
        z += e[i];
    }
    // ---- top-p: the largest key whose own and larger keys' mass reaches p of the whole ----
    if (prm.top_p < 1.0f) {
        z = block_sum(z, fscratch);
        z = cl_sum_f(z, &xch, parity, n_blocks);
        const float need = prm.top_p * z;
        unsigned lo_key = 0;
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned cand = lo_key | (1u << bit);
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < CL_ITEMS; ++i)
                if (keys[i * CL_THREADS + tid] >= cand) s += e[i];
            s = block_sum(s, fscratch);
            if (cl_sum_f(s, &xch, parity, n_blocks) >= need) lo_key = cand;
        }
#pragma unroll
        for (int i = 0; i < CL_ITEMS; ++i)
            if (keys[i * CL_THREADS + tid] < lo_key) { keys[i * CL_THREADS + tid] = 0u; e[i] = 0.f; }
    }
    // ---- draw: first index whose cumulative mass exceeds r * total; a thread's elements are consecutive ----
    float local = 0.f;
#pragma unroll
    for (int i = 0; i < CL_ITEMS; ++i) local += e[i];
    chunk_sum[tid] = local;
    if (tid == 0) chosen = -1;
    const float block_total = block_sum(local, fscratch);     // also orders the writes above before the reads below
    // every block learns every block's total: the totals before this block's, and the whole
    if (tid == 0) xch.f[parity] = block_total;
    cl_sync();
    float before = 0.f, total = 0.f;
    for (int r = 0; r < n_blocks; ++r) {
        const float t = cl_ld_f32(cl_map(&xch.f[parity], r));
        if (r < rank) before += t;
        total += t;
    }
    parity ^= 1;
    const float u = uniform_from(prm.seed, row_stream ? row_stream[row] : (unsigned long long)row,
                                 row_step ? (unsigned long long)row_step[row] : 0ull);
    const float target = u * total;
    // the block in whose range the target falls looks for the thread, that thread for the element
    const bool mine = target >= before && (target < before + block_total);
    if (tid == 0) {
        s_chunk = -1;
        if (mine) {
            float c = before;
            for (int i = 0; i < CL_THREADS; ++i) {
                if (target < c + chunk_sum[i]) { s_chunk = i; s_before = c; break; }
                c += chunk_sum[i];
            }
        }
    }
    __syncthreads();
    if (mine && s_chunk == tid) {
        float c = s_before;
        int pick = -1;
#pragma unroll
        for (int i = 0; i < CL_ITEMS; ++i) {
            c += e[i];
            if (pick < 0 && target < c) pick = first + i;
        }
        if (pick < 0) {        // rounding inside the chunk: its last element with mass
#pragma unroll
            for (int i = 0; i < CL_ITEMS; ++i)
                if (e[i] > 0.f) pick = first + i;
        }
        chosen = pick;
    }
    // the last element with mass, of this block and of the row: where rounding puts the target at or beyond a total
    int last = -1;
#pragma unroll
    for (int i = 0; i < CL_ITEMS; ++i)
        if (e[i] > 0.f) last = first + i;
    const float block_last = block_max((float)last, fscratch);          // also orders the write of `chosen` before the read below
    if (tid == 0 && mine && s_chunk < 0) chosen = (int)block_last;     // the chunks' sum in order fell short of the block's tree sum
    __syncthreads();
    const float found = cl_max_f((float)chosen, &xch, parity, n_blocks);
    const float row_last = cl_max_f(block_last, &xch, parity, n_blocks);
    if (rank == 0 && tid == 0) put_token(out_tokens, host_tokens, row, found >= 0.f ? (int)found : (row_last >= 0.f ? (int)row_last : 0));
    cl_sync();                 // no block leaves while another may still read its shared memory
}

}  // namespace

extern "C" float rdl_sampling_uniform(unsigned long long seed, unsigned long long stream, unsigned long long step) {
    return uniform_from(seed, stream, step);
}

extern "C" int rdl_sample(int* out_tokens, int* host_tokens, const float* logits, int n_rows, int vocab, const SamplingArgs* prm,
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
    if (prm->temperature < 1e-7f && vocab >= 4 * CL_PER_BLOCK && n_rows <= 65535) {
        // arg max of a long row: eight blocks a row
        const int n_blocks = CL_MAX_BLOCKS;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(n_blocks, n_rows);
        cfg.blockDim = dim3(CL_THREADS);
        cfg.stream = (cudaStream_t)stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = n_blocks;
        attr[0].val.clusterDim.y = attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = g_rdl_programmatic_launch ? 2 : 1;
        RDL_CHECK_EX(cudaLaunchKernelEx(&cfg, argmax_cluster_kernel, out_tokens, host_tokens, logits, vocab, n_blocks), "sample");
        return 0;
    }
    if (prm->temperature >= 1e-7f && vocab <= CL_MAX_BLOCKS * CL_PER_BLOCK && n_rows <= 65535) {
        // the row on the chip: 1, 2, 4 or 8 blocks a row
        int n_blocks = 1;
        while (n_blocks * CL_PER_BLOCK < vocab) n_blocks *= 2;
        const size_t smem = (size_t)CL_ITEMS * CL_THREADS * sizeof(unsigned);
        static bool opted = false;
        if (!opted) {
            RDL_CUDA(cudaFuncSetAttribute(sample_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "sample");
            opted = true;
        }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(n_blocks, n_rows);
        cfg.blockDim = dim3(CL_THREADS);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = (cudaStream_t)stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = n_blocks;
        attr[0].val.clusterDim.y = attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = g_rdl_programmatic_launch ? 2 : 1;
        RDL_CHECK_EX(cudaLaunchKernelEx(&cfg, sample_cluster_kernel, out_tokens, host_tokens, logits, vocab, *prm, row_stream, row_step, history,
                                        history_start, work, n_blocks), "sample");
        return 0;
    }
    RDL_CHECK_EX(rdl_launch(sample_kernel, dim3(n_rows), dim3(SAMPLE_THREADS), 0, (cudaStream_t)stream, out_tokens, host_tokens, logits, vocab,
                            *prm, row_stream, row_step, history, history_start, work), "sample");
    return 0;
}
