// Decode attention in bfloat16 over the paged cache: few query tokens, many keys.  The keys of
// a (token, kv head) pair are split into runs of `keys_per_split` positions; one block computes
// the unnormalised output, running maximum and sum of a run for all query heads that share the
// kv head, a second kernel merges the runs in a fixed order.  The cache is streamed with 16-byte
// loads; scores, soft-cap, softmax state and the output sums are float.  Formulas as in
// attention_plain.cu; all keys are read from the cache (the step writes its new rows first).
//
// Scratch (float): [token][head][split][head_dim + 2] = partial output, maximum, sum.
#include "api.h"
#include "common.cuh"

namespace {

constexpr int DEC_THREADS = 128;
constexpr int DEC_WARPS = DEC_THREADS / 32;
constexpr int UNROLL = 4;

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

// GP: query heads per kv head, padded to 1, 2, 4 or 8.  LPK: lanes per key (head_dim <= 8 * LPK).
template <int GP, int LPK>
__global__ void __launch_bounds__(DEC_THREADS) attention_decode_kernel(AttentionArgs a) {
    constexpr int KPW = 32 / LPK;                 // keys a warp handles at once
    constexpr int GROUPS = DEC_WARPS * KPW;       // independent softmax states per block
    const int t = blockIdx.z, g = blockIdx.y, sp = blockIdx.x;
    const int hd = a.head_dim;
    const int G = a.n_heads / a.n_kv_heads;
    const int seq = a.tok_seq[t], p = a.tok_pos[t];
    if (p < 0) return;  // a padding row of a fixed-size batch
    const int lo = first_key(p, a.window);
    const int split0 = lo / a.keys_per_split;
    const int k_begin = max(lo, (split0 + sp) * a.keys_per_split);
    const int k_end = min(p + 1, (split0 + sp + 1) * a.keys_per_split);   // exclusive
    if (k_begin >= k_end) return;
    const int* table = a.tables + (long long)seq * a.table_width;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane / LPK, li = lane % LPK;
    const int group = warp * KPW + sub;
    const int d0 = li * 8;
    const bool lane_on = d0 < hd;
    const __nv_bfloat16* kcache = (const __nv_bfloat16*)a.k_cache;
    const __nv_bfloat16* vcache = (const __nv_bfloat16*)a.v_cache;

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
    const uint4 zero4 = make_uint4(0, 0, 0, 0);

    // the loop bound is the same for every lane of a warp (the shuffles below need all of them)
    for (int base = k_begin + warp * KPW; base < k_end; base += GROUPS * UNROLL) {
        const int j0 = base + sub;
        uint4 kv[UNROLL], vv[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int j = j0 + u * GROUPS;
            kv[u] = zero4;
            vv[u] = zero4;
            if (j < k_end && lane_on) {
                const long long off = rdl_cache_offset(table, j, a.page_size, a.ring_pages, a.n_kv_heads, g, hd) + d0;
                kv[u] = *(const uint4*)(kcache + off);
                vv[u] = *(const uint4*)(vcache + off);
            }
        }
        float s[UNROLL][GP];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            float kf[8];
            unpack8(kv[u], kf);
#pragma unroll
            for (int h = 0; h < GP; ++h) {
                float d = 0.f;
#pragma unroll
                for (int i = 0; i < 8; ++i) d = fmaf(q[h][i], kf[i], d);
#pragma unroll
                for (int o = LPK / 2; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
                d *= a.score_scale;
                if (a.softcap > 0.f) d = a.softcap * tanh_fast(d * inv_cap);
                s[u][h] = (j0 + u * GROUPS < k_end) ? d : -INFINITY;
            }
        }
#pragma unroll
        for (int h = 0; h < GP; ++h) {
            float mn = m[h];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) mn = fmaxf(mn, s[u][h]);
            const float ms = mn == -INFINITY ? 0.f : mn;   // a group may have seen no key yet
            const float corr = __expf(m[h] - ms);
            m[h] = mn;
            l[h] *= corr;
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[h][i] *= corr;
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            float vf[8];
            unpack8(vv[u], vf);
#pragma unroll
            for (int h = 0; h < GP; ++h) {
                const float pw = __expf(s[u][h] - (m[h] == -INFINITY ? 0.f : m[h]));
                l[h] += pw;
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[h][i] = fmaf(pw, vf[i], acc[h][i]);
            }
        }
    }

    // ---- merge the groups of the block through shared memory, in group order ----
    extern __shared__ float sm[];                  // [GROUPS][GP][hd_pad + 2]
    const int hd_pad = LPK * 8;
    const int stride = hd_pad + 2;
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
    const int max_splits = a.max_splits;
    float* scratch = (float*)a.scratch;
    for (int idx = threadIdx.x; idx < G * hd; idx += DEC_THREADS) {
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
        float* out = scratch + (((long long)t * a.n_heads + (g * G + h)) * max_splits + sp) * (hd + 2);
        out[d] = osum;
        if (d == 0) {
            out[hd] = M;
            out[hd + 1] = lsum;
        }
    }
}

__global__ void attention_decode_merge_kernel(AttentionArgs a) {
    const int t = blockIdx.x, h = blockIdx.y;
    const int hd = a.head_dim;
    const int p = a.tok_pos[t];
    if (p < 0) return;  // a padding row of a fixed-size batch
    const int lo = first_key(p, a.window);
    const int n_splits = p / a.keys_per_split - lo / a.keys_per_split + 1;
    const float* base = (const float*)a.scratch + ((long long)t * a.n_heads + h) * a.max_splits * (hd + 2);
    float M = -INFINITY;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, base[(long long)s * (hd + 2) + hd]);
    __nv_bfloat16* out = (__nv_bfloat16*)a.out + (long long)t * a.out_stride + (long long)h * hd;
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float osum = 0.f, lsum = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            const float* src = base + (long long)s * (hd + 2);
            const float w = __expf(src[hd] - M);
            osum = fmaf(w, src[d], osum);
            lsum = fmaf(w, src[hd + 1], lsum);
        }
        out[d] = __float2bfloat16_rn(osum / lsum);
    }
}

template <int GP, int LPK>
int launch_decode(const AttentionArgs* a, cudaStream_t st) {
    constexpr int GROUPS = DEC_WARPS * (32 / LPK);
    const int smem = GROUPS * GP * (LPK * 8 + 2) * (int)sizeof(float);
    static bool opted = false;
    if (smem > 48 * 1024 && !opted) {
        RDL_CUDA(cudaFuncSetAttribute(attention_decode_kernel<GP, LPK>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem),
                 "attention_decode");
        opted = true;
    }
    dim3 grid(a->max_splits, a->n_kv_heads, a->n_tokens);
    attention_decode_kernel<GP, LPK><<<grid, DEC_THREADS, smem, st>>>(*a);
    RDL_CHECK_LAUNCH("attention_decode");
    dim3 mgrid(a->n_tokens, a->n_heads);
    attention_decode_merge_kernel<<<mgrid, a->head_dim >= 128 ? 128 : 64, 0, st>>>(*a);
    RDL_CHECK_LAUNCH("attention_decode_merge");
    return 0;
}

template <int GP>
int launch_decode_g(const AttentionArgs* a, cudaStream_t st) {
    if (a->head_dim <= 64) return launch_decode<GP, 8>(a, st);
    if (a->head_dim <= 128) return launch_decode<GP, 16>(a, st);
    return launch_decode<GP, 32>(a, st);
}

}  // namespace

extern "C" long long rdl_attention_decode_scratch_bytes(int n_tokens, int n_heads, int head_dim, int max_splits) {
    return (long long)n_tokens * n_heads * max_splits * (head_dim + 2) * (long long)sizeof(float);
}

extern "C" int rdl_attention_decode(const AttentionArgs* a, void* stream) {
    if (int e = rdl_check_attention_args(a, "attention_decode")) return e;
    RDL_REQUIRE(a->dtype == RDL_BF16, "attention_decode: bfloat16 only (the 32-bit path uses attention_plain)");
    RDL_REQUIRE(a->head_dim % 8 == 0 && a->head_dim <= 256, "attention_decode: head_dim %d must be a multiple of 8 and at most 256", a->head_dim);
    const int G = a->n_heads / a->n_kv_heads;
    RDL_REQUIRE(G <= 8, "attention_decode: %d query heads per key/value head, at most 8 are supported", G);
    RDL_REQUIRE(a->tables && a->k_cache && a->v_cache, "attention_decode: needs a cache");
    RDL_REQUIRE(a->keys_per_split > 0 && a->max_splits > 0 && a->max_splits <= 65535, "attention_decode: bad split sizes");
    RDL_REQUIRE(a->n_kv_heads <= 65535 && a->n_tokens <= 65535, "attention_decode: grid too large");
    RDL_REQUIRE(a->scratch && a->scratch_bytes >= rdl_attention_decode_scratch_bytes(a->n_tokens, a->n_heads, a->head_dim, a->max_splits),
                "attention_decode: scratch of %lld bytes is too small", a->scratch_bytes);
    RDL_REQUIRE(a->q_stride % 8 == 0 && (uintptr_t)a->q % 16 == 0 && (uintptr_t)a->k_cache % 16 == 0 && (uintptr_t)a->v_cache % 16 == 0,
                "attention_decode: rows must start on 16-byte boundaries");
    if (a->n_tokens == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    if (G == 1) return launch_decode_g<1>(a, st);
    if (G == 2) return launch_decode_g<2>(a, st);
    if (G <= 4) return launch_decode_g<4>(a, st);
    return launch_decode_g<8>(a, st);
}
