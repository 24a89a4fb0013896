// Shared helpers of the sm_100a kernels: dtype codes, error reporting, loads that
// widen to float, block reductions.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

// dtype codes of the C interface
#define RDL_F32 0
#define RDL_BF16 1

// Launchers return 0 on success.  On failure they return non-zero and leave a message
// that rdl_last_error() hands to the caller.
void rdl_set_error(const char* fmt, ...);

#define RDL_REQUIRE(cond, ...)          \
    do {                                \
        if (!(cond)) {                  \
            rdl_set_error(__VA_ARGS__); \
            return 1;                   \
        }                               \
    } while (0)

#define RDL_CHECK_LAUNCH(name)                                              \
    do {                                                                    \
        cudaError_t e_ = cudaGetLastError();                                \
        if (e_ != cudaSuccess) {                                            \
            rdl_set_error("%s: launch failed: %s", name, cudaGetErrorString(e_)); \
            return 2;                                                       \
        }                                                                   \
    } while (0)

#define RDL_CUDA(call, name)                                                \
    do {                                                                    \
        cudaError_t e_ = (call);                                            \
        if (e_ != cudaSuccess) {                                            \
            rdl_set_error("%s: %s", name, cudaGetErrorString(e_));          \
            return 2;                                                       \
        }                                                                   \
    } while (0)

// About a second of clock cycles: the default limit of a wait inside a kernel.
#define RDL_WAIT_CYCLES 2000000000LL
extern int g_rdl_wait_test_code;
extern long long g_rdl_wait_test_cycles;
extern int g_rdl_wait_test_extra;
// The wait limit of the kernel with fault code `code`, and the extra bytes its first copy announces (0 outside tests).
static inline long long rdl_wait_cycles_for(int code) {
    return (g_rdl_wait_test_code == code && g_rdl_wait_test_cycles > 0) ? g_rdl_wait_test_cycles : RDL_WAIT_CYCLES;
}
static inline int rdl_test_extra_tx_for(int code) { return g_rdl_wait_test_code == code ? g_rdl_wait_test_extra : 0; }

// Multiprocessors of the current device (asked once per device; 1 if the question fails).
int rdl_sm_count();

static inline bool rdl_valid_dtype(int d) { return d == RDL_F32 || d == RDL_BF16; }
static inline size_t rdl_dtype_size(int d) { return d == RDL_BF16 ? 2 : 4; }

__device__ __forceinline__ float rdl_load(const void* p, long long i, int dtype) {
    return dtype == RDL_BF16 ? __bfloat162float(((const __nv_bfloat16*)p)[i]) : ((const float*)p)[i];
}
__device__ __forceinline__ void rdl_store(void* p, long long i, int dtype, float v) {
    if (dtype == RDL_BF16)
        ((__nv_bfloat16*)p)[i] = __float2bfloat16_rn(v);
    else
        ((float*)p)[i] = v;
}

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  `scratch` holds 33 floats.
// The order of additions depends only on the block size.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();  // scratch may still be read from an earlier call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// Where absolute position `pos` of a sequence lies in a paged cache.
// table: the sequence's page list; ring_pages: how many entries of it are in use as a ring
// (a window group), or the table's width (a group that keeps all keys).
// A layer's storage is [page][kv head][row in page][head_dim].
__device__ __forceinline__ long long rdl_cache_offset(const int* __restrict__ table, int pos, int page_size,
                                                      int ring_pages, int n_kv_heads, int kv_head, int head_dim) {
    const int logical = pos / page_size;
    const int page = table[logical % ring_pages];
    const int r = pos - logical * page_size;
    return (((long long)page * n_kv_heads + kv_head) * page_size + r) * head_dim;
}

// Inside a row of a cache page the 16-byte chunks are stored swizzled by the row: chunk c of the row
// at place `r` of its page lies at chunk c ^ (r & 7), for the chunks of the row's last incomplete
// group of eight unchanged.  A whole [page_size][head_dim] block can then be copied to shared
// memory in one piece and still be read by ldmatrix, eight rows at a time, without bank conflicts.
// Rows whose size is no multiple of 16 bytes are stored plainly.
__host__ __device__ __forceinline__ int rdl_swizzled_chunk(int r, int chunk, int chunks_per_row) {
    return ((chunk | 7) < chunks_per_row) ? (chunk ^ (r & 7)) : chunk;
}
// Element i of a cache row of `head_dim` elements of type T -> its place in the stored row.
template <typename T>
__device__ __forceinline__ int rdl_cache_col(int r, int i, int head_dim) {
    constexpr int EPC = 16 / (int)sizeof(T);
    if (head_dim % EPC) return i;
    const int c = i / EPC;
    return rdl_swizzled_chunk(r, c, head_dim / EPC) * EPC + (i - c * EPC);
}
