// Plain attention over new tokens and a paged cache: one warp per (query token, head),
// float arithmetic throughout, a fixed order of operations that depends only on absolute
// positions.  It is the attention of the 32-bit path (prefill and decode alike) and the
// reference the fast kernels are tested against.
//
// For query position p of a sequence and query head h (kv head g = h / (n_heads / n_kv_heads),
// reference: rustml/core/main/src/core/tensor/ops.rs:980-987):
//   s_j = (q_h . k_g,j) * score_scale                    attention.rs:413-416
//   s_j = cap * tanh(s_j / cap)            if cap > 0    attention.rs:419-423
//   keys kept: j <= p and (window == 0 or p - j < window)  ops.rs:905-922, :932-952
//   a = softmax_j(s)                                      ops.rs:598-608
//   o_h = sum_j a_j v_g,j                                 attention.rs:442-446
// (paths within rustml/; attention.rs = nn/main/src/core/attention.rs).  The window holds for
// single-token steps too, which the reference's cached path skips (attention.rs:429).
//
// Keys at positions below seq_cached[s] are read from the cache, later ones from the step's
// own packed key/value rows.
#include "api.h"
#include "common.cuh"

#define PLAIN_MAX_CHUNKS 16  // head_dim <= 512

template <typename T>
__global__ void attention_plain_kernel(AttentionArgs a) {
    const int warps_per_block = blockDim.x >> 5;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * warps_per_block + warp;
    if (item >= (long long)a.n_tokens * a.n_heads) return;
    const int t = (int)(item / a.n_heads), h = (int)(item % a.n_heads);
    const int hd = a.head_dim;
    const int g = h / (a.n_heads / a.n_kv_heads);
    const int seq = a.tok_seq[t], p = a.tok_pos[t];
    if (p < 0) return;  // a padding row of a fixed-size batch
    const int cached = a.seq_cached[seq];
    const int new_row0 = a.seq_start[seq] - a.seq_past[seq];  // packed row of position j is new_row0 + j
    const int* table = a.tables ? a.tables + (long long)seq * a.table_width : nullptr;
    const T* q = (const T*)a.q + (long long)t * a.q_stride + (long long)h * hd;
    const int lo = a.window > 0 ? max(0, p - a.window + 1) : 0;

    float acc[PLAIN_MAX_CHUNKS];
#pragma unroll
    for (int c = 0; c < PLAIN_MAX_CHUNKS; ++c) acc[c] = 0.f;
    float m = -INFINITY, l = 0.f;

    for (int jb = (lo / 32) * 32; jb <= p; jb += 32) {
        const int j = jb + lane;
        const bool valid = j >= lo && j <= p;
        const T* kp = nullptr;
        const T* vp = nullptr;
        float s = -INFINITY;
        int sw = -1;   // place of the row in its cache page (rows there are stored swizzled); -1: a packed new row
        if (valid) {
            if (j < cached) {
                const long long off = rdl_cache_offset(table, j, a.page_size, a.ring_pages, a.n_kv_heads, g, hd);
                kp = (const T*)a.k_cache + off;
                vp = (const T*)a.v_cache + off;
                sw = j % a.page_size;
            } else {
                const long long off = (long long)(new_row0 + j) * a.kv_stride + (long long)g * hd;
                kp = (const T*)a.k_new + off;
                vp = (const T*)a.v_new + off;
            }
            float d = 0.f;
            for (int i = 0; i < hd; ++i) d = fmaf(to_float(q[i]), to_float(kp[sw < 0 ? i : rdl_cache_col<T>(sw, i, hd)]), d);
            d *= a.score_scale;
            if (a.softcap > 0.f) d = a.softcap * tanhf(d / a.softcap);
            s = d;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float corr = expf(m - m_new);   // exp(-inf) = 0 on the first block
        const float pj = valid ? expf(s - m_new) : 0.f;
        l = l * corr + warp_sum(pj);
        m = m_new;
#pragma unroll
        for (int c = 0; c < PLAIN_MAX_CHUNKS; ++c) acc[c] *= corr;
        const unsigned long long vaddr = (unsigned long long)vp;
        for (int jj = 0; jj < 32; ++jj) {
            const int jk = jb + jj;
            if (jk < lo || jk > p) continue;  // uniform over the warp
            const float pw = __shfl_sync(0xffffffffu, pj, jj);
            const unsigned lo32 = __shfl_sync(0xffffffffu, (unsigned)(vaddr & 0xffffffffull), jj);
            const unsigned hi32 = __shfl_sync(0xffffffffu, (unsigned)(vaddr >> 32), jj);
            const int vsw = __shfl_sync(0xffffffffu, sw, jj);
            const T* vrow = (const T*)(((unsigned long long)hi32 << 32) | lo32);
#pragma unroll
            for (int c = 0; c < PLAIN_MAX_CHUNKS; ++c) {
                const int d = c * 32 + lane;
                if (d < hd) acc[c] = fmaf(pw, to_float(vrow[vsw < 0 ? d : rdl_cache_col<T>(vsw, d, hd)]), acc[c]);
            }
        }
    }
    T* o = (T*)a.out + (long long)t * a.out_stride + (long long)h * hd;
    const float inv = 1.0f / l;
#pragma unroll
    for (int c = 0; c < PLAIN_MAX_CHUNKS; ++c) {
        const int d = c * 32 + lane;
        if (d < hd) o[d] = from_float<T>(acc[c] * inv);
    }
}

int rdl_check_attention_args(const AttentionArgs* a, const char* who) {
    RDL_REQUIRE(rdl_valid_dtype(a->dtype), "%s: bad dtype %d", who, a->dtype);
    RDL_REQUIRE(a->n_tokens >= 0 && a->n_seqs >= 0, "%s: bad token or sequence count", who);
    RDL_REQUIRE(a->n_heads > 0 && a->n_kv_heads > 0 && a->n_heads % a->n_kv_heads == 0,
                "%s: %d heads cannot share %d key/value heads", who, a->n_heads, a->n_kv_heads);
    RDL_REQUIRE(a->head_dim > 0, "%s: bad head_dim %d", who, a->head_dim);
    RDL_REQUIRE(a->window >= 0 && a->softcap >= 0.f, "%s: window and soft-cap must not be negative", who);
    RDL_REQUIRE(a->q && a->out && a->tok_seq && a->tok_pos && a->seq_start && a->seq_past && a->seq_cached,
                "%s: missing query, output or batch description", who);
    RDL_REQUIRE(a->q_stride >= (long long)a->n_heads * a->head_dim && a->out_stride >= (long long)a->n_heads * a->head_dim,
                "%s: row strides smaller than a row", who);
    if (a->tables) {
        RDL_REQUIRE(a->k_cache && a->v_cache && a->page_size > 0 && a->ring_pages > 0 && a->ring_pages <= a->table_width,
                    "%s: cache given without storage or with bad paging (page_size=%d ring_pages=%d table_width=%d)", who,
                    a->page_size, a->ring_pages, a->table_width);
    }
    RDL_REQUIRE(a->tables || (a->k_new && a->v_new), "%s: neither a cache nor new keys and values", who);
    return 0;
}

extern "C" int rdl_attention_plain(const AttentionArgs* a, void* stream) {
    if (int e = rdl_check_attention_args(a, "attention_plain")) return e;
    RDL_REQUIRE(a->head_dim <= 32 * PLAIN_MAX_CHUNKS, "attention_plain: head_dim %d exceeds %d", a->head_dim, 32 * PLAIN_MAX_CHUNKS);
    if (a->n_tokens == 0) return 0;
    const int warps = 4;
    const long long items = (long long)a->n_tokens * a->n_heads;
    const unsigned blocks = (unsigned)((items + warps - 1) / warps);
    if (a->dtype == RDL_BF16)
        attention_plain_kernel<__nv_bfloat16><<<blocks, warps * 32, 0, (cudaStream_t)stream>>>(*a);
    else
        attention_plain_kernel<float><<<blocks, warps * 32, 0, (cudaStream_t)stream>>>(*a);
    RDL_CHECK_LAUNCH("attention_plain");
    return 0;
}
