// Decode attention in bfloat16 over the paged cache: few query tokens, many keys.
//
// The keys a token reads (all earlier positions, or the last `window`) are cut into runs of
// `keys_per_split` positions (a whole number of pages).  One block handles one run for all query
// heads that share a kv head: each page of the run - a contiguous [page_size][head_dim] block of
// keys and one of values - is brought into shared memory by a bulk asynchronous copy (TMA,
// cp.async.bulk + mbarrier) and consumed from there; scores, soft-cap, softmax state and output
// sums are float.  A token with a single run writes its output directly.  Otherwise every block
// writes its unnormalised partial result to scratch and the block that finishes last for a
// (token, kv head) merges the runs in run order and writes the output: one launch, no second
// kernel.  Formulas as in attention_plain.cu; all keys are read from the cache (the step
// writes its new rows first).
//
// Scratch: int counters [tokens * kv_heads] (zero before the launch; the merging block puts its
// counter back to zero), then float partials [token][head][run][head_dim + 2] = sums, maximum,
// normaliser.  Launches that share the scratch must not overlap on the device.
//
// Every wait on a copy is bounded: after about a second without completion the block records
// an error in `status` and leaves.
#include "api.h"
#include "common.cuh"

namespace {

constexpr int DEC_THREADS = 128;
constexpr int DEC_WARPS = DEC_THREADS / 32;
constexpr long long WAIT_CYCLES = 2000000000LL;

__device__ __forceinline__ float tanh_fast(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 t = __bfloat1622float2(p[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}

__host__ __device__ inline int first_key(int p, int window) { return window > 0 ? (p - window + 1 > 0 ? p - window + 1 : 0) : 0; }

__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// false if the copy did not complete within the limit
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity))
        if (clock64() - t0 > WAIT_CYCLES) return false;
    return true;
}

// GP: query heads per kv head, padded to 1, 2, 4 or 8.  LPK: lanes per key (head_dim <= 8 * LPK).
template <int GP, int LPK>
__global__ void __launch_bounds__(DEC_THREADS) attention_decode_kernel(AttentionArgs a) {
    constexpr int KPW = 32 / LPK;                 // keys a warp handles at once
    constexpr int GROUPS = DEC_WARPS * KPW;       // independent softmax states per block
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ __align__(8) unsigned long long bar_storage;
    __shared__ int s_flag;

    const int t = blockIdx.z, g = blockIdx.y, sp = blockIdx.x;
    const int hd = a.head_dim, ps = a.page_size;
    const int G = a.n_heads / a.n_kv_heads;
    const int seq = a.tok_seq[t], p = a.tok_pos[t];
    if (p < 0) return;  // a padding row of a fixed-size batch
    const int lo = first_key(p, a.window);
    const int split0 = lo / a.keys_per_split;
    const int n_splits = p / a.keys_per_split - split0 + 1;
    if (sp >= n_splits) return;
    const int k_begin = max(lo, (split0 + sp) * a.keys_per_split);
    const int k_end = min(p + 1, (split0 + sp + 1) * a.keys_per_split);   // exclusive
    const int* table = a.tables + (long long)seq * a.table_width;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int sub = lane / LPK, li = lane % LPK;
    const int group = warp * KPW + sub;
    const int d0 = li * 8;
    const bool lane_on = d0 < hd;
    const __nv_bfloat16* kcache = (const __nv_bfloat16*)a.k_cache;
    const __nv_bfloat16* vcache = (const __nv_bfloat16*)a.v_cache;
    const uint32_t tile_bytes = (uint32_t)ps * hd * 2;
    unsigned char* k_tile = smem;
    unsigned char* v_tile = smem + tile_bytes;
    const uint32_t k_s = (uint32_t)__cvta_generic_to_shared(k_tile);
    const uint32_t v_s = k_s + tile_bytes;
    const uint32_t bar = (uint32_t)__cvta_generic_to_shared(&bar_storage);

    if (tid == 0) mbar_init(bar, 1);
    __syncthreads();

    float q[GP][8];
#pragma unroll
    for (int h = 0; h < GP; ++h) {
#pragma unroll
        for (int i = 0; i < 8; ++i) q[h][i] = 0.f;
        if (h < G && lane_on) {
            const uint4 v = *(const uint4*)((const __nv_bfloat16*)a.q + (long long)t * a.q_stride + (long long)(g * G + h) * hd + d0);
            unpack8(v, q[h]);
        }
    }
    float acc[GP][8], m[GP], l[GP];
#pragma unroll
    for (int h = 0; h < GP; ++h) {
        m[h] = -INFINITY;
        l[h] = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[h][i] = 0.f;
    }
    const float inv_cap = a.softcap > 0.f ? 1.0f / a.softcap : 0.f;

    uint32_t phase = 0;
    const int page_first = k_begin / ps, page_last = (k_end - 1) / ps;
    for (int lp = page_first; lp <= page_last; ++lp) {
        if (tid == 0) {
            const int page = table[lp % a.ring_pages];
            const long long off = ((long long)page * a.n_kv_heads + g) * ps * hd;
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_expect_tx(bar, 2 * tile_bytes);
            bulk_load(k_s, kcache + off, tile_bytes, bar);
            bulk_load(v_s, vcache + off, tile_bytes, bar);
        }
        if (!mbar_wait_bounded(bar, phase)) {
            if (a.status) atomicExch(a.status, 3);
            return;
        }
        phase ^= 1;
        const int r_begin = max(k_begin, lp * ps) - lp * ps, r_end = min(k_end, (lp + 1) * ps) - lp * ps;
        // the loop bound is the same for every lane of a warp (the shuffles below need all of them)
        for (int base = r_begin + warp * KPW; base < r_end; base += GROUPS) {
            const int r = base + sub;
            const bool valid = r < r_end;
            float s[GP];
            float kf[8];
            {
                uint4 kv = make_uint4(0, 0, 0, 0);
                if (valid && lane_on) kv = *(const uint4*)(k_tile + ((long long)r * hd + d0) * 2);
                unpack8(kv, kf);
            }
#pragma unroll
            for (int h = 0; h < GP; ++h) {
                float d = 0.f;
#pragma unroll
                for (int i = 0; i < 8; ++i) d = fmaf(q[h][i], kf[i], d);
#pragma unroll
                for (int o = LPK / 2; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
                d *= a.score_scale;
                if (a.softcap > 0.f) d = a.softcap * tanh_fast(d * inv_cap);
                s[h] = valid ? d : -INFINITY;
            }
            float vf[8];
            {
                uint4 vv = make_uint4(0, 0, 0, 0);
                if (valid && lane_on) vv = *(const uint4*)(v_tile + ((long long)r * hd + d0) * 2);
                unpack8(vv, vf);
            }
#pragma unroll
            for (int h = 0; h < GP; ++h) {
                const float mn = fmaxf(m[h], s[h]);
                const float ms = mn == -INFINITY ? 0.f : mn;   // a group may have seen no key yet
                const float corr = __expf(m[h] - ms);
                const float pw = __expf(s[h] - ms);
                m[h] = mn;
                l[h] = l[h] * corr + pw;
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[h][i] = fmaf(pw, vf[i], acc[h][i] * corr);
            }
        }
        __syncthreads();   // everyone is done with the tiles before the next copy lands
    }

    // ---- merge the groups of the block through shared memory, in group order ----
    float* sm = reinterpret_cast<float*>(smem);    // [GROUPS][GP][hd_pad + 2], the tiles are no longer needed
    constexpr int hd_pad = LPK * 8;
    constexpr int stride = hd_pad + 2;
#pragma unroll
    for (int h = 0; h < GP; ++h) {
        float* dst = sm + ((long long)group * GP + h) * stride;
#pragma unroll
        for (int i = 0; i < 8; ++i) dst[d0 + i] = acc[h][i];
        if (li == 0) {
            dst[hd_pad] = m[h];
            dst[hd_pad + 1] = l[h];
        }
    }
    __syncthreads();
    __nv_bfloat16* out = (__nv_bfloat16*)a.out + (long long)t * a.out_stride;
    int* counters = (int*)a.scratch;
    float* partials = (float*)((char*)a.scratch + a.counter_bytes);
    for (int idx = tid; idx < G * hd; idx += DEC_THREADS) {
        const int h = idx / hd, d = idx - h * hd;
        float M = -INFINITY;
        for (int gr = 0; gr < GROUPS; ++gr) M = fmaxf(M, sm[((long long)gr * GP + h) * stride + hd_pad]);
        float osum = 0.f, lsum = 0.f;
        for (int gr = 0; gr < GROUPS; ++gr) {
            const float* src = sm + ((long long)gr * GP + h) * stride;
            const float w = src[hd_pad] == -INFINITY ? 0.f : __expf(src[hd_pad] - M);
            osum = fmaf(w, src[d], osum);
            lsum = fmaf(w, src[hd_pad + 1], lsum);
        }
        if (n_splits == 1) {
            out[(long long)(g * G + h) * hd + d] = __float2bfloat16_rn(osum / lsum);
        } else {
            float* dst = partials + (((long long)t * a.n_heads + (g * G + h)) * a.max_splits + sp) * (hd + 2);
            dst[d] = osum;
            if (d == 0) {
                dst[hd] = M;
                dst[hd + 1] = lsum;
            }
        }
    }
    if (n_splits == 1) return;

    // ---- the block that finishes last for this (token, kv head) merges the runs ----
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const int done = atomicAdd(&counters[t * a.n_kv_heads + g], 1);
        s_flag = done == n_splits - 1;
        if (s_flag) counters[t * a.n_kv_heads + g] = 0;    // ready for the next launch
    }
    __syncthreads();
    if (!s_flag) return;
    __threadfence();
    float* w_s = sm;                              // [G][n_splits] weights of the runs
    float* stat = sm + G * n_splits;              // [G] 1 / normaliser
    for (int h = warp; h < G; h += DEC_WARPS) {
        const float* base = partials + ((long long)t * a.n_heads + (g * G + h)) * a.max_splits * (hd + 2);
        float M = -INFINITY;
        for (int s = lane; s < n_splits; s += 32) M = fmaxf(M, base[(long long)s * (hd + 2) + hd]);
        M = warp_max(M);
        float L = 0.f;
        for (int s = lane; s < n_splits; s += 32) {
            const float w = __expf(base[(long long)s * (hd + 2) + hd] - M);
            w_s[h * n_splits + s] = w;
            L = fmaf(w, base[(long long)s * (hd + 2) + hd + 1], L);
        }
        L = warp_sum(L);
        if (lane == 0) stat[h] = 1.0f / L;
    }
    __syncthreads();
    for (int idx = tid; idx < G * hd; idx += DEC_THREADS) {
        const int h = idx / hd, d = idx - h * hd;
        const float* base = partials + ((long long)t * a.n_heads + (g * G + h)) * a.max_splits * (hd + 2) + d;
        float o = 0.f;
#pragma unroll 8
        for (int s = 0; s < n_splits; ++s) o = fmaf(w_s[h * n_splits + s], base[(long long)s * (hd + 2)], o);
        out[(long long)(g * G + h) * hd + d] = __float2bfloat16_rn(o * stat[h]);
    }
}

template <int GP, int LPK>
int launch_decode(const AttentionArgs* a, cudaStream_t st) {
    constexpr int GROUPS = DEC_WARPS * (32 / LPK);
    const int tiles = 2 * a->page_size * a->head_dim * 2;
    const int merge = GROUPS * GP * (LPK * 8 + 2) * (int)sizeof(float);
    const int runs = (GP * a->max_splits + GP) * (int)sizeof(float);
    int smem = tiles > merge ? tiles : merge;
    if (runs > smem) smem = runs;
    RDL_REQUIRE(smem <= 200 * 1024, "attention_decode: page_size %d x head_dim %d needs %d bytes of shared memory, limit is 204800",
                a->page_size, a->head_dim, smem);
    static int granted = 48 * 1024;
    if (smem > granted) {
        RDL_CUDA(cudaFuncSetAttribute(attention_decode_kernel<GP, LPK>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem),
                 "attention_decode");
        granted = smem;
    }
    dim3 grid(a->max_splits, a->n_kv_heads, a->n_tokens);
    attention_decode_kernel<GP, LPK><<<grid, DEC_THREADS, smem, st>>>(*a);
    RDL_CHECK_LAUNCH("attention_decode");
    return 0;
}

template <int GP>
int launch_decode_g(const AttentionArgs* a, cudaStream_t st) {
    if (a->head_dim <= 64) return launch_decode<GP, 8>(a, st);
    if (a->head_dim <= 128) return launch_decode<GP, 16>(a, st);
    return launch_decode<GP, 32>(a, st);
}

}  // namespace

extern "C" long long rdl_attention_decode_counter_bytes(int n_tokens, int n_kv_heads) {
    const long long b = (long long)n_tokens * n_kv_heads * (long long)sizeof(int);
    return (b + 255) / 256 * 256;
}

extern "C" long long rdl_attention_decode_scratch_bytes(int n_tokens, int n_heads, int n_kv_heads, int head_dim, int max_splits) {
    return rdl_attention_decode_counter_bytes(n_tokens, n_kv_heads) +
           (long long)n_tokens * n_heads * max_splits * (head_dim + 2) * (long long)sizeof(float);
}

extern "C" int rdl_attention_decode(const AttentionArgs* a, void* stream) {
    if (int e = rdl_check_attention_args(a, "attention_decode")) return e;
    RDL_REQUIRE(a->dtype == RDL_BF16, "attention_decode: bfloat16 only (the 32-bit path uses attention_plain)");
    RDL_REQUIRE(a->head_dim % 8 == 0 && a->head_dim <= 256, "attention_decode: head_dim %d must be a multiple of 8 and at most 256", a->head_dim);
    const int G = a->n_heads / a->n_kv_heads;
    RDL_REQUIRE(G <= 8, "attention_decode: %d query heads per key/value head, at most 8 are supported", G);
    RDL_REQUIRE(a->tables && a->k_cache && a->v_cache, "attention_decode: needs a cache");
    RDL_REQUIRE(a->keys_per_split > 0 && a->keys_per_split % a->page_size == 0,
                "attention_decode: keys_per_split %d must be a whole number of pages of %d", a->keys_per_split, a->page_size);
    RDL_REQUIRE(a->max_splits > 0 && a->max_splits <= 65535, "attention_decode: bad number of runs %d", a->max_splits);
    RDL_REQUIRE(a->n_kv_heads <= 65535 && a->n_tokens <= 65535, "attention_decode: grid too large");
    RDL_REQUIRE(a->counter_bytes == rdl_attention_decode_counter_bytes(a->n_tokens, a->n_kv_heads),
                "attention_decode: counter_bytes must come from rdl_attention_decode_counter_bytes");
    RDL_REQUIRE(a->scratch && a->scratch_bytes >= rdl_attention_decode_scratch_bytes(a->n_tokens, a->n_heads, a->n_kv_heads, a->head_dim, a->max_splits),
                "attention_decode: scratch of %lld bytes is too small", a->scratch_bytes);
    RDL_REQUIRE(a->q_stride % 8 == 0 && (uintptr_t)a->q % 16 == 0 && (uintptr_t)a->k_cache % 16 == 0 &&
                    (uintptr_t)a->v_cache % 16 == 0 && (uintptr_t)a->scratch % 16 == 0,
                "attention_decode: rows must start on 16-byte boundaries");
    if (a->n_tokens == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    if (G == 1) return launch_decode_g<1>(a, st);
    if (G == 2) return launch_decode_g<2>(a, st);
    if (G <= 4) return launch_decode_g<4>(a, st);
    return launch_decode_g<8>(a, st);
}
