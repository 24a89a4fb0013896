// Rotary position encoding of the query and key heads of a packed [tokens, heads, head_dim]
// buffer, in place, and the write of the new key and value rows into a paged cache.
//
// Rotation (reference: rustml/nn/main/src/core/rope.rs:188-191, half-split pairing):
//   out[i]        = x[i] * cos - x[i + r/2] * sin
//   out[i + r/2]  = x[i] * sin + x[i + r/2] * cos      for i < r/2, r = rotary_dim
// with cos/sin read from float tables [position][r/2]; the product is formed in float.
// The cache write corresponds to rustml/nn/main/src/core/kv_cache.rs:97-109, with pages and a
// length per sequence instead of one shared length.
#include "api.h"
#include "common.cuh"
#include "launch.cuh"

template <typename T>
__global__ void rope_cache_kernel(T* __restrict__ qkv, int n_heads, int n_kv_heads, int head_dim, int rotary_dim,
                                  const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                  const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                  int do_rope, int do_write, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                  const int* __restrict__ tables, int table_width, int page_size, int ring_pages,
                                  const int* __restrict__ seq_end) {
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const int t = blockIdx.x;
    const int head = blockIdx.y;
    const int total_heads = n_heads + 2 * n_kv_heads;
    T* row = qkv + ((long long)t * total_heads + head) * head_dim;
    const int pos = tok_pos[t];
    if (pos < 0) return;  // a padding row of a fixed-size batch
    const bool is_v = head >= n_heads + n_kv_heads;

    if (do_rope && !is_v) {
        const int half = rotary_dim >> 1;
        const float* c = cos_t + (long long)pos * half;
        const float* s = sin_t + (long long)pos * half;
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const float x1 = to_float(row[i]), x2 = to_float(row[i + half]);
            const float cs = c[i], sn = s[i];
            row[i] = from_float<T>(x1 * cs - x2 * sn);
            row[i + half] = from_float<T>(x1 * sn + x2 * cs);
        }
    }
    if (!do_write || head < n_heads) return;
    const int seq = tok_seq[t];
    // In a ring a later token of this step may land on the same row: only the last writer writes.
    const long long ring_rows = (long long)ring_pages * page_size;
    if ((long long)pos + ring_rows < (long long)seq_end[seq]) return;
    __syncthreads();  // the rotated key of this block is complete
    const int kv_head = is_v ? head - n_heads - n_kv_heads : head - n_heads;
    T* dst = (is_v ? v_cache : k_cache) +
             rdl_cache_offset(tables + (long long)seq * table_width, pos, page_size, ring_pages, n_kv_heads, kv_head, head_dim);
    const int r = pos % page_size;   // chunks of a cache row are stored swizzled by its place in the page
    for (int i = threadIdx.x; i < head_dim; i += blockDim.x) dst[rdl_cache_col<T>(r, i, head_dim)] = row[i];
}

// The same work with 16-byte accesses: one block per token, a thread per 16-byte chunk (or pair of
// chunks that rotate together).  Used when head_dim and rotary_dim / 2 are whole numbers of chunks.
template <typename T> struct Chunk;
template <> struct Chunk<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&f)[8]) {
        const uint4 raw = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 v = __bfloat1622float2(h[i]); f[2 * i] = v.x; f[2 * i + 1] = v.y; }
    }
    static __device__ __forceinline__ uint4 pack(const float (&f)[8]) {
        uint4 raw;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
        return raw;
    }
};
template <> struct Chunk<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float (&f)[4]) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
    }
    static __device__ __forceinline__ uint4 pack(const float (&f)[4]) {
        uint4 raw;
        raw.x = __float_as_uint(f[0]); raw.y = __float_as_uint(f[1]); raw.z = __float_as_uint(f[2]); raw.w = __float_as_uint(f[3]);
        return raw;
    }
};

template <typename T>
__global__ void __launch_bounds__(256) rope_cache_vec_kernel(T* __restrict__ qkv, int n_heads, int n_kv_heads, int head_dim, int rotary_dim,
                                                             const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                                             const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                                             int do_rope, int do_write, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                                             const int* __restrict__ tables, int table_width, int page_size,
                                                             int ring_pages, const int* __restrict__ seq_end) {
    constexpr int N = Chunk<T>::N;
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const int t = blockIdx.x;
    const int pos = tok_pos[t];
    if (pos < 0) return;  // a padding row of a fixed-size batch
    const int total_heads = n_heads + 2 * n_kv_heads;
    const int chunks = head_dim / N;
    const int half = rotary_dim >> 1, half_chunks = do_rope ? half / N : 0;
    T* base = qkv + (long long)t * total_heads * head_dim;
    bool write = do_write && n_kv_heads > 0;
    int r = 0;
    long long page_base = 0;
    if (write) {
        const int seq = tok_seq[t];
        // In a ring a later token of this step may land on the same row: only the last writer writes.
        if ((long long)pos + (long long)ring_pages * page_size < (long long)seq_end[seq]) write = false;
        const int logical = pos / page_size;
        r = pos - logical * page_size;
        page_base = (long long)tables[(long long)seq * table_width + logical % ring_pages] * n_kv_heads;
    }
    // Work items, one 16-byte chunk of output pair or chunk each, so that no thread idles: first the rotated
    // pairs (chunk c with chunk c + half) of the query and key heads, then the chunks that are only copied
    // to the cache: the unrotated tail of the key heads and the value heads.
    const int n_pairs = (n_heads + n_kv_heads) * half_chunks;
    const int k_tail = chunks - 2 * half_chunks;                  // unrotated chunks of a key head
    const int n_copy = write ? n_kv_heads * (k_tail + chunks) : 0;
    for (int item = threadIdx.x; item < n_pairs + n_copy; item += blockDim.x) {
        int head, c;
        bool rotated = item < n_pairs;
        if (rotated) {
            head = item / half_chunks;
            c = item - head * half_chunks;
        } else {
            const int rest = item - n_pairs;
            if (rest < n_kv_heads * k_tail) {
                head = n_heads + rest / k_tail;
                c = 2 * half_chunks + rest % k_tail;
            } else {
                const int v = rest - n_kv_heads * k_tail;
                head = n_heads + n_kv_heads + v / chunks;
                c = v % chunks;
            }
        }
        const bool is_q = head < n_heads, is_v = head >= n_heads + n_kv_heads;
        T* row = base + (long long)head * head_dim;
        T* dst = nullptr;
        if (write && !is_q) {
            const int kv_head = is_v ? head - n_heads - n_kv_heads : head - n_heads;
            dst = (is_v ? v_cache : k_cache) + ((page_base + kv_head) * page_size + r) * head_dim;
        }
        float a[N];
        Chunk<T>::load(row + c * N, a);
        if (rotated) {
            float b[N], cs[N], sn[N];
            Chunk<T>::load(row + (c + half_chunks) * N, b);
            const float4* cp = reinterpret_cast<const float4*>(cos_t + (long long)pos * half + c * N);
            const float4* sp = reinterpret_cast<const float4*>(sin_t + (long long)pos * half + c * N);
#pragma unroll
            for (int i = 0; i < N / 4; ++i) {
                const float4 cv = __ldg(cp + i), sv = __ldg(sp + i);
                cs[4 * i] = cv.x; cs[4 * i + 1] = cv.y; cs[4 * i + 2] = cv.z; cs[4 * i + 3] = cv.w;
                sn[4 * i] = sv.x; sn[4 * i + 1] = sv.y; sn[4 * i + 2] = sv.z; sn[4 * i + 3] = sv.w;
            }
            float lo[N], hi[N];
#pragma unroll
            for (int i = 0; i < N; ++i) {
                lo[i] = a[i] * cs[i] - b[i] * sn[i];
                hi[i] = a[i] * sn[i] + b[i] * cs[i];
            }
            const uint4 plo = Chunk<T>::pack(lo), phi = Chunk<T>::pack(hi);
            *reinterpret_cast<uint4*>(row + c * N) = plo;
            *reinterpret_cast<uint4*>(row + (c + half_chunks) * N) = phi;
            if (dst) {
                *reinterpret_cast<uint4*>(dst + rdl_swizzled_chunk(r, c, chunks) * N) = plo;
                *reinterpret_cast<uint4*>(dst + rdl_swizzled_chunk(r, c + half_chunks, chunks) * N) = phi;
            }
        } else if (dst) {
            *reinterpret_cast<uint4*>(dst + rdl_swizzled_chunk(r, c, chunks) * N) = Chunk<T>::pack(a);
        }
    }
}

extern "C" int rdl_rope_cache(void* qkv, int dtype, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                              int rotary_dim, const float* cos_table, const float* sin_table,
                              const int* tok_seq, const int* tok_pos, int do_rope, int do_write,
                              void* k_cache, void* v_cache, const int* tables, int table_width, int page_size,
                              int ring_pages, const int* seq_end, void* stream) {
    RDL_REQUIRE(rdl_valid_dtype(dtype), "rope_cache: bad dtype %d", dtype);
    RDL_REQUIRE(n_tokens >= 0 && n_heads >= 0 && n_kv_heads >= 0 && n_heads + n_kv_heads > 0 && head_dim > 0,
                "rope_cache: bad sizes tokens=%d heads=%d kv_heads=%d head_dim=%d", n_tokens, n_heads, n_kv_heads, head_dim);
    RDL_REQUIRE(!do_rope || (rotary_dim > 0 && rotary_dim % 2 == 0 && rotary_dim <= head_dim && cos_table && sin_table),
                "rope_cache: rotary_dim %d must be even and at most head_dim %d", rotary_dim, head_dim);
    RDL_REQUIRE(!do_write || n_kv_heads == 0 ||
                    (k_cache && v_cache && tables && seq_end && tok_seq && page_size > 0 && ring_pages > 0 && ring_pages <= table_width),
                "rope_cache: cache write needs storage, page tables and lengths (page_size=%d ring_pages=%d table_width=%d)",
                page_size, ring_pages, table_width);
    const int total_heads = n_heads + 2 * n_kv_heads;
    RDL_REQUIRE(total_heads <= 65535, "rope_cache: %d heads exceed the grid limit", total_heads);
    if (n_tokens == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    const int per_chunk = dtype == RDL_BF16 ? 8 : 4;
    const bool aligned = ((uintptr_t)qkv & 15) == 0 && ((uintptr_t)k_cache & 15) == 0 && ((uintptr_t)v_cache & 15) == 0 &&
                         ((uintptr_t)cos_table & 15) == 0 && ((uintptr_t)sin_table & 15) == 0;
    if (aligned && head_dim % per_chunk == 0 && (!do_rope || (rotary_dim / 2) % per_chunk == 0)) {
        // two work items a thread where there are many (the kernel's comment says what an item is)
        const int chunks = head_dim / per_chunk, half_chunks = do_rope ? rotary_dim / 2 / per_chunk : 0;
        const int items = (n_heads + n_kv_heads) * half_chunks + n_kv_heads * (2 * chunks - 2 * half_chunks);
        int vthreads = ((items + 1) / 2 + 31) / 32 * 32;
        vthreads = vthreads < 64 ? 64 : (vthreads > 256 ? 256 : vthreads);
        if (dtype == RDL_BF16)
            e = rdl_launch(rope_cache_vec_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(vthreads), 0, st, (__nv_bfloat16*)qkv, n_heads,
                           n_kv_heads, head_dim, rotary_dim, cos_table, sin_table, tok_seq, tok_pos, do_rope, do_write,
                           (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, tables, table_width, page_size, ring_pages, seq_end);
        else
            e = rdl_launch(rope_cache_vec_kernel<float>, dim3(n_tokens), dim3(vthreads), 0, st, (float*)qkv, n_heads, n_kv_heads,
                           head_dim, rotary_dim, cos_table, sin_table, tok_seq, tok_pos, do_rope, do_write, (float*)k_cache,
                           (float*)v_cache, tables, table_width, page_size, ring_pages, seq_end);
        RDL_CHECK_EX(e, "rope_cache");
        return 0;
    }
    dim3 grid(n_tokens, total_heads);
    const int threads = head_dim >= 256 ? 128 : (head_dim >= 64 ? 64 : 32);
    if (dtype == RDL_BF16)
        e = rdl_launch(rope_cache_kernel<__nv_bfloat16>, grid, dim3(threads), 0, st, (__nv_bfloat16*)qkv, n_heads, n_kv_heads, head_dim,
                       rotary_dim, cos_table, sin_table, tok_seq, tok_pos, do_rope, do_write, (__nv_bfloat16*)k_cache,
                       (__nv_bfloat16*)v_cache, tables, table_width, page_size, ring_pages, seq_end);
    else
        e = rdl_launch(rope_cache_kernel<float>, grid, dim3(threads), 0, st, (float*)qkv, n_heads, n_kv_heads, head_dim,
                       rotary_dim, cos_table, sin_table, tok_seq, tok_pos, do_rope, do_write, (float*)k_cache,
                       (float*)v_cache, tables, table_width, page_size, ring_pages, seq_end);
    RDL_CHECK_EX(e, "rope_cache");
    return 0;
}
