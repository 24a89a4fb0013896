// Matrix product for few rows (decode): out[m, n] = sum_k x[m, k] * w[n, k] with m <= 16.
// The weight matrix is streamed from HBM exactly once; the few activation rows come through L1/L2.
// bfloat16 operands, float accumulation (mma.sync m16n8k16: 16 weight rows x 8 activation rows per
// instruction).  A unit of work is 16 weight rows (for the gated form: 8 gate rows and the 8 up rows
// of the same outputs, which are the two halves of one 16-row fragment).
//
// Eight warps multiply and a ninth issues the copies: a tile is the unit's 16 weight rows x 768 or 1024 k
// (each row one cp.async.bulk of 1.5 or 2 KB) in a ring of shared-memory tiles, and every multiplying warp
// takes an eighth of its k; the warps' partial sums are added in warp order through shared memory.  The
// copying warp needs nothing an earlier kernel of the step writes, so it never waits for that kernel:
// with programmatic dependent launch a block's ring (about 100 KB) is on its way while the kernel before
// it is still running.  Blocks are persistent (at most two a multiprocessor) and the ring runs on from
// unit to unit, so it never drains.  What is in flight does not live in registers: a multiprocessor has
// about 200 KB on their way, which is what it takes to keep HBM busy when a copy needs about 3 us to
// arrive (with the weights in a ring of registers, 64 KB a multiprocessor, the same products were 15-30 %
// slower).  Every wait is bounded; a block that gives up sets `status`.
//
// Epilogues: plain store (bfloat16 or float), cap * tanh(v / cap) (the output head), and
// act(gate) * up for a row-concatenated [gate; up] matrix (the feed-forward), all in float.
// (y = x W^T, W [out, in]: rustml/nn/main/src/core/linear.rs:12-15; the gated form and the
// activation: rustml/nn/main/src/core/feed_forward.rs:151-161.)
//
// The k index inside a 32-wide step is permuted identically for both operands (a lane's 16
// bytes feed two instructions), which leaves every dot product unchanged.
//
// Deferred norms (MODE; the algebra is in api.h at DeferredNormArgs).  A product whose result is a branch
// of the residual stream (MODE 1) writes, instead of y: a' = y (w1 + off1) and a' (w2 + off2) as bfloat16,
// and for its 16 columns the sums of y^2, h^2, h a' and a'^2 of every row.  The product that follows the two
// norms (MODE 2) multiplies the 16-row operand [h (w2 + off2); a' (w2 + off2)], adds the partial sums up
// (each thread a 32nd of the units, then 32 terms in order), and forms s2 (z_h + s1 z_a) in its epilogue;
// every block also updates a slice of the stream (h' = h + s1 a') and of the next operand's first half.
#include <cstdlib>

#include "activations.cuh"
#include "api.h"
#include "common.cuh"
#include "launch.cuh"

namespace {

constexpr int ROWS = 16;        // weight rows per unit

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct SkinnyArgs {
    const __nv_bfloat16* x;     // [M, K]
    const __nv_bfloat16* w;     // [N, K] (gated: [2 * N, K], gate rows first)
    void* out;                  // [M, N]
    int M, N, K;
    int out_dtype;              // RDL_F32 / RDL_BF16
    int activation;             // of the gated form
    float softcap;              // > 0: cap * tanh(v / cap)
    long long wait_cycles;      // clock cycles after which a wait is given up
    int test_extra_tx;          // tests only: bytes announced beyond what the block's first copy delivers
    DeferredNormArgs d;         // MODE 1 and 2
};

thread_local cudaError_t g_launch_error = cudaSuccess;

constexpr int ST_WARPS = 8;                      // multiplying warps
constexpr int ST_THREADS = (ST_WARPS + 1) * 32;
// KU: steps of 32 k a multiplying warp takes of a tile (4: tiles of 1024 k, 3: of 768 k; the host takes
// the one that leaves less of the last tile of a row empty).
// Rows of a tile lie their length + 64 bytes apart: a quarter warp's eight 16-byte reads (rows g and g + 1,
// four chunks each) then fall into eight different groups of four banks.
__host__ __device__ constexpr int st_kt(int ku) { return ST_WARPS * 32 * ku; }
__host__ __device__ constexpr int st_pitch(int ku) { return st_kt(ku) * 2 + 64; }
__host__ __device__ constexpr int st_tile_bytes(int ku) { return ROWS * st_pitch(ku); }
__host__ __device__ constexpr int st_stages(int ku) { return ku == 4 ? 3 : 4; }      // about 100 KB a block; twice that where one block has a multiprocessor to itself
constexpr int ST_MAX_STAGES = 8;

__device__ __forceinline__ void st_mbar_init(uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void st_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void st_mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// policy: an L2 cache policy (createpolicy); 0: none
__device__ __forceinline__ void st_bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar, unsigned long long policy = 0) {
    if (policy)
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                     ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(policy) : "memory");
    else
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ unsigned long long l2_evict_first_policy() {
    unsigned long long p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ bool st_mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// false if the barrier's phase did not complete within about a second, or if another warp of the block has
// already given up (the block then runs to its end without waiting; its status word says that the result is void)
__device__ __forceinline__ bool st_wait(uint32_t bar, uint32_t parity, long long limit, volatile int* gave_up) {
    if (*gave_up) return false;
    if (st_mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!st_mbar_try_wait(bar, parity)) {
        if (*gave_up) return false;
        if (clock64() - t0 > limit) { *gave_up = 1; return false; }
    }
    return true;
}
// A norm weight's element as raw bits, and its value: a load whose result is not used at once does not hold its
// thread up, so the prologues below ask for everything first and convert afterwards.
__device__ __forceinline__ uint32_t raw_load(const void* p, long long i, int dtype) {
    return dtype == RDL_BF16 ? (uint32_t)((const unsigned short*)p)[i] : ((const uint32_t*)p)[i];
}
__device__ __forceinline__ float raw_value(uint32_t bits, int dtype) {
    return dtype == RDL_BF16 ? __uint_as_float(bits << 16) : __uint_as_float(bits);
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

template <int NT, bool GATED, int KU, int MODE>
__global__ void __launch_bounds__(ST_THREADS, 2) gemm_stream_kernel(const __grid_constant__ SkinnyArgs a, int stages, int* status) {
    // MODE 2 with NT == 1: up to 4 rows; both halves of the operand then share one fragment (rows 0..3 and 4..7)
    static_assert(MODE == 0 || (MODE == 1 && NT == 1 && !GATED) || MODE == 2, "deferred norms: up to 8 rows");
    constexpr bool PACKED = MODE == 2 && NT == 1;
    constexpr int ST_KT = st_kt(KU), ST_PITCH = st_pitch(KU), ST_TILE_BYTES = st_tile_bytes(KU), KW = 32 * KU;
    extern __shared__ __align__(128) unsigned char st_tiles[];
    __shared__ __align__(8) unsigned long long full_bar[ST_MAX_STAGES], empty_bar[ST_MAX_STAGES];
    __shared__ float partial[ST_WARPS][NT][ROWS * 8];
    __shared__ float4 sum_part[MODE == 2 ? 32 : 1][8];     // MODE 2: the partial sums, a 32nd of the units each
    __shared__ float2 row_scale[8];                         // MODE 2: (s1, s2) of every row
    __shared__ int gave_up;
    constexpr int OUT_ROWS = GATED ? 8 : ROWS;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int K = a.K;
    const int n_units = (a.N + OUT_ROWS - 1) / OUT_ROWS;
    const int tiles_per_unit = (K + ST_KT - 1) / ST_KT;
    const uint32_t tiles_s = (uint32_t)__cvta_generic_to_shared(st_tiles);
    const uint32_t full_s = (uint32_t)__cvta_generic_to_shared(full_bar), empty_s = (uint32_t)__cvta_generic_to_shared(empty_bar);
    if (threadIdx.x == 0) {
        gave_up = 0;
        for (int s = 0; s < stages; ++s) {
            st_mbar_init(full_s + 8 * s, 1);
            st_mbar_init(empty_s + 8 * s, ST_WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    volatile int* gave_up_v = &gave_up;

    if (warp == ST_WARPS) {
        // ---- the copying warp: lane r brings row r of every tile ----
        if (lane < ROWS) {
            int s = 0;                                   // place in the ring, and how often it has been gone round
            uint32_t round = 0;
            bool first_copy = true;
            // The weights are read once a step: they pass through L2 marked to be evicted first, so that what the step
            // reads again and again - the rows of activations, the residual stream - stays there.
            const unsigned long long policy = l2_evict_first_policy();
            for (int unit = blockIdx.x; unit < n_units; unit += gridDim.x) {
                long long row;
                bool row_ok;
                if (GATED) {                             // rows 0-7: gate rows of 8 outputs; rows 8-15: their up rows
                    const int o = unit * 8 + (lane & 7);
                    row_ok = o < a.N;
                    row = (long long)(lane < 8 ? 0 : a.N) + o;
                } else {
                    row = (long long)unit * ROWS + lane;
                    row_ok = row < a.N;
                }
                const int n_ok = __popc(__ballot_sync(0xffffu, row_ok));
                for (int tk = 0; tk < tiles_per_unit; ++tk) {
                    // the tile that lay here must have been read by all eight warps
                    if (round > 0 && !st_wait(empty_s + 8 * s, (round & 1) ^ 1, a.wait_cycles, gave_up_v)) break;
                    const int k0 = tk * ST_KT;
                    const uint32_t bytes = (uint32_t)((K - k0 < ST_KT ? K - k0 : ST_KT) * 2);
                    if (lane == 0) {
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        st_mbar_expect_tx(full_s + 8 * s, bytes * (uint32_t)n_ok + (first_copy ? (uint32_t)a.test_extra_tx : 0u));
                    }
                    __syncwarp(0xffffu);
                    if (row_ok) st_bulk_load(tiles_s + (uint32_t)(s * ST_TILE_BYTES + lane * ST_PITCH), a.w + row * K + k0, bytes, full_s + 8 * s, policy);
                    first_copy = false;
                    if (++s == stages) { s = 0; ++round; }
                }
                if (*gave_up_v) break;
            }
        }
    } else {
        // ---- the multiplying warps ----
        const int g = lane >> 2, t = lane & 3;
        const __nv_bfloat16* xrow[NT];
        bool x_ok[NT];
#pragma unroll
        for (int i = 0; i < NT; ++i) {
            // MODE 2: both halves of the operand have M rows (packed: the halves are rows 0..3 and 4..7 of one fragment)
            x_ok[i] = PACKED ? (g & 3) < a.M : (MODE == 2 ? g < a.M : i * 8 + g < a.M);
            xrow[i] = a.x + (long long)(i * 8 + g) * K;
        }
        const uint4 zero4 = make_uint4(0, 0, 0, 0);
        const int kw = warp * KW;                        // this warp's k inside a tile
        auto load_x = [&](int kc, uint4 (&xb)[NT][KU]) {
#pragma unroll
            for (int u = 0; u < KU; ++u) {
                const int k = kc + u * 32 + t * 8;
#pragma unroll
                for (int i = 0; i < NT; ++i)
                    xb[i][u] = (k < K && x_ok[i]) ? __ldg(reinterpret_cast<const uint4*>(xrow[i] + k)) : zero4;
            }
        };
        rdl_grid_wait();
        rdl_grid_launch_dependents();
        // up to 8 rows: the activations of a tile are requested one tile ahead; with 16 rows the registers for
        // that would cost the second block of a multiprocessor
        constexpr bool X_AHEAD = NT == 1;
        uint4 xcur[NT][KU], xnext[X_AHEAD ? NT : 1][KU];
        if (X_AHEAD) load_x(kw, xcur);
        // MODE 2: this block's slice of the stream (one element a thread and round), asked for now, stored once s1 is known
        const DeferredNormArgs& d = a.d;
        const int tid = threadIdx.x;
        long long slice_e = -1;
        float slice_h = 0.f;
        uint32_t slice_a = 0u, slice_w = 0u;               // raw bits until the stores
        bool first_unit = true;
        if constexpr (MODE == 2) {
            if (!X_AHEAD) load_x(kw, xcur);              // the first tile's rows are on their way while the sums are added up
            const long long total = (long long)a.M * K, per = (total + gridDim.x - 1) / gridDim.x;
            if (d.residual_out || d.scaled_next) {
                const long long e = blockIdx.x * per + tid;
                if (tid < per && e < total) {
                    slice_e = e;
                    slice_h = d.residual_in[e];
                    slice_a = raw_load(d.branch_in, e, RDL_BF16);
                    if (d.scaled_next) slice_w = raw_load(d.w_next, e % K, d.w_next_dtype);
                }
            }
            // the partial sums: thread (part, m) adds the units part, part + 32, ... of row m, eight loads in flight at a time
            const int m = tid & 7, part = tid >> 3;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int u0 = part; u0 < d.n_sums; u0 += 8 * 32) {
                float4 v[8];
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    v[i] = u0 + 32 * i < d.n_sums ? __ldcg(reinterpret_cast<const float4*>(d.sums) + (u0 + 32 * i) * 8 + m)
                                                  : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int i = 0; i < 8; ++i) { acc.x += v[i].x; acc.y += v[i].y; acc.z += v[i].z; acc.w += v[i].w; }
            }
            sum_part[part][m] = acc;
            asm volatile("bar.sync 1, %0;" ::"n"(ST_WARPS * 32) : "memory");
            if (tid < 8) {
                float4 t = sum_part[0][tid];
#pragma unroll
                for (int q = 1; q < 32; ++q) {
                    const float4 v = sum_part[q][tid];
                    t.x += v.x; t.y += v.y; t.z += v.z; t.w += v.w;
                }
                const float s1 = rsqrtf(t.x / (float)K + d.eps1);
                const float hh = t.y + 2.f * s1 * t.z + s1 * s1 * t.w;           // sum of (h + s1 a')^2
                row_scale[tid] = make_float2(s1, rsqrtf(fmaxf(hh, 0.f) / (float)K + d.eps2));
            }
            // row_scale is read after the first unit's barrier below
        }
        const uint32_t frag = tiles_s + (uint32_t)(g * ST_PITCH + (kw + t * 8) * 2);
        int s = 0;
        uint32_t round = 0;
        for (int unit = blockIdx.x; unit < n_units; unit += gridDim.x) {
            float acc[NT][4];
#pragma unroll
            for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
            // MODE 1: thread (m, r) of the epilogue asks for its element of the stream and its two norm weights now
            float br_h = 0.f;
            uint32_t br_w1 = 0u, br_w2 = 0u;                 // raw bits until the epilogue
            if constexpr (MODE == 1) {
                const int m = tid >> 4, n = unit * ROWS + (tid & 15);
                if (tid < 8 * ROWS && m < a.M && n < a.N) {
                    br_h = d.residual[(long long)m * a.N + n];
                    br_w1 = raw_load(d.w1, n, d.w1_dtype);
                    br_w2 = raw_load(d.w2, n, d.w2_dtype);
                }
            }
            for (int tk = 0; tk < tiles_per_unit; ++tk) {
                // the activations of the tile after this one (the next unit starts again at k = 0)
                if (X_AHEAD) load_x((tk + 1 < tiles_per_unit ? (tk + 1) * ST_KT : 0) + kw, reinterpret_cast<uint4 (&)[NT][KU]>(xnext));
                else if (!(MODE == 2 && tk == 0 && unit == (int)blockIdx.x)) load_x(tk * ST_KT + kw, xcur);     // (that tile's rows were asked for above)
                st_wait(full_s + 8 * s, round & 1, a.wait_cycles, gave_up_v);
                const int kb = tk * ST_KT + kw;
                if (kb < K) {
                    const uint32_t base = frag + (uint32_t)(s * ST_TILE_BYTES);
#pragma unroll
                    for (int u = 0; u < KU; ++u) {
                        const bool in = kb + u * 32 + t * 8 < K;      // what lies beyond K in the tile is stale
                        const uint4 w0 = in ? lds128(base + u * 64) : zero4;
                        const uint4 w1 = in ? lds128(base + u * 64 + 8 * ST_PITCH) : zero4;
#pragma unroll
                        for (int i = 0; i < NT; ++i) {
                            mma_bf16(acc[i], w0.x, w1.x, w0.y, w1.y, xcur[i][u].x, xcur[i][u].y);
                            mma_bf16(acc[i], w0.z, w1.z, w0.w, w1.w, xcur[i][u].z, xcur[i][u].w);
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) st_mbar_arrive(empty_s + 8 * s);
                if (++s == stages) { s = 0; ++round; }
                if (X_AHEAD) {
#pragma unroll
                    for (int i = 0; i < NT; ++i)
#pragma unroll
                        for (int u = 0; u < KU; ++u) xcur[i][u] = xnext[X_AHEAD ? i : 0][u];
                }
            }
            // accumulator element e of a lane: weight row g + 8 * (e >> 1), activation row 2 t + (e & 1)
#pragma unroll
            for (int i = 0; i < NT; ++i)
#pragma unroll
                for (int e = 0; e < 4; ++e) partial[warp][i][(2 * t + (e & 1)) * ROWS + g + 8 * (e >> 1)] = acc[i][e];
            asm volatile("bar.sync 1, %0;" ::"n"(ST_WARPS * 32) : "memory");
            const int n0 = unit * OUT_ROWS;
            if constexpr (MODE == 1) {
                // the first four warps: thread (m, r) has column n0 + r of row m; 16 neighbouring lanes add up a row's sums
                if (tid < 8 * ROWS) {
                    const int m = tid >> 4, r = tid & 15, n = n0 + r;
                    const bool ok = m < a.M && n < a.N;
                    float y = 0.f;
#pragma unroll
                    for (int w = 0; w < ST_WARPS; ++w) y += partial[w][0][m * ROWS + r];
                    if (!ok) y = 0.f;
                    const float br_g1 = raw_value(br_w1, d.w1_dtype) + d.off1, br_g2 = raw_value(br_w2, d.w2_dtype) + d.off2;
                    const __nv_bfloat16 a1b = __float2bfloat16_rn(y * br_g1);
                    const float a1 = __bfloat162float(a1b);                  // what the stream will add, s1 times
                    float s0 = y * y, s1 = br_h * br_h, s2 = br_h * a1, s3 = a1 * a1;
#pragma unroll
                    for (int o = 8; o > 0; o >>= 1) {
                        s0 += __shfl_xor_sync(0xffffffffu, s0, o);
                        s1 += __shfl_xor_sync(0xffffffffu, s1, o);
                        s2 += __shfl_xor_sync(0xffffffffu, s2, o);
                        s3 += __shfl_xor_sync(0xffffffffu, s3, o);
                    }
                    if (ok) {
                        ((__nv_bfloat16*)d.branch)[(long long)m * a.N + n] = a1b;
                        ((__nv_bfloat16*)d.scaled)[(long long)m * a.N + n] = __float2bfloat16_rn(a1 * br_g2);
                    }
                    if (r == 0) reinterpret_cast<float4*>(d.sums)[unit * 8 + m] = make_float4(s0, s1, s2, s3);   // rows beyond M: zeros
                }
            } else if constexpr (MODE == 2) {
                if (first_unit) {
                    first_unit = false;
                    // the block's slice of the stream and of the next operand
                    const long long total = (long long)a.M * K, per = (total + gridDim.x - 1) / gridDim.x;
                    const long long end = (blockIdx.x + 1) * per < total ? (blockIdx.x + 1) * per : total;
                    for (long long e = slice_e; e >= 0 && e < end;) {
                        const float hn = slice_h + row_scale[e / K].x * raw_value(slice_a, RDL_BF16);
                        if (d.residual_out) d.residual_out[e] = hn;
                        if (d.scaled_next)
                            ((__nv_bfloat16*)d.scaled_next)[e] = __float2bfloat16_rn(hn * (raw_value(slice_w, d.w_next_dtype) + d.off_next));
                        e += ST_WARPS * 32;
                        if (e < end) {
                            slice_h = d.residual_in[e];
                            slice_a = raw_load(d.branch_in, e, RDL_BF16);
                            if (d.scaled_next) slice_w = raw_load(d.w_next, e % K, d.w_next_dtype);
                        }
                    }
                }
                for (int idx = tid; idx < d.n_out * OUT_ROWS; idx += ST_WARPS * 32) {
                    const int j = idx / OUT_ROWS, r = idx - j * OUT_ROWS;
                    const int n = n0 + r;
                    const int m = d.row_index ? d.row_index[j] : j;
                    if (n >= a.N || m < 0 || m >= a.M) continue;
                    const float2 sc = row_scale[m];
                    // the stream's half and the branch's half of the operand: two fragments, or rows m and m + 4 of one
                    const int slot = m * ROWS + r, slot_a = PACKED ? slot + 4 * ROWS : slot;
                    constexpr int IA = PACKED ? 0 : NT - 1;
                    float h0 = 0.f, a0 = 0.f, h1 = 0.f, a1 = 0.f;
#pragma unroll
                    for (int w = 0; w < ST_WARPS; ++w) {
                        h0 += partial[w][0][slot];
                        a0 += partial[w][IA][slot_a];
                        if (GATED) { h1 += partial[w][0][slot + 8]; a1 += partial[w][IA][slot_a + 8]; }
                    }
                    float y = sc.y * (h0 + sc.x * a0);
                    if (GATED) y = rdl_activation(y, a.activation) * (sc.y * (h1 + sc.x * a1));
                    if (a.softcap > 0.f) y = a.softcap * tanhf(y / a.softcap);
                    rdl_store(a.out, (long long)j * a.N + n, a.out_dtype, y);
                }
            } else
            for (int idx = threadIdx.x; idx < NT * 8 * OUT_ROWS; idx += ST_WARPS * 32) {
                const int m = idx / OUT_ROWS, r = idx - m * OUT_ROWS;
                const int n = n0 + r;
                if (m >= a.M || n >= a.N) continue;
                const int i = m >> 3, slot = (m & 7) * ROWS + r;
                float v0 = 0.f, v1 = 0.f;
#pragma unroll
                for (int w = 0; w < ST_WARPS; ++w) {
                    v0 += partial[w][i][slot];
                    if (GATED) v1 += partial[w][i][slot + 8];
                }
                float y = v0;
                if (GATED) y = rdl_activation(v0, a.activation) * v1;
                if (a.softcap > 0.f) y = a.softcap * tanhf(y / a.softcap);
                rdl_store(a.out, (long long)m * a.N + n, a.out_dtype, y);
            }
            asm volatile("bar.sync 1, %0;" ::"n"(ST_WARPS * 32) : "memory");      // the partial sums are free again
        }
    }
    if (*gave_up_v && status && lane == 0) atomicExch(status, RDL_FAULT_GEMM_STREAM);
}

template <int NT, bool GATED, int KU, int MODE>
void launch_stream_ku(const SkinnyArgs& a, int* status, cudaStream_t st) {
    constexpr int smem_max = 2 * st_stages(KU) * st_tile_bytes(KU);
    static_assert(2 * st_stages(KU) <= ST_MAX_STAGES, "the ring's barriers");
    static bool opted = false;
    static int sms = 0;
    if (!opted) {
        g_launch_error = cudaFuncSetAttribute(gemm_stream_kernel<NT, GATED, KU, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_max);
        if (g_launch_error != cudaSuccess) return;
        sms = rdl_sm_count();
        opted = true;
    }
    // What counts is the bytes a multiprocessor has in flight: two blocks with three tiles each, or, where
    // the output is so narrow that there is at most one block a multiprocessor, one block with twice as many.
    const int units = (a.N + (GATED ? 8 : ROWS) - 1) / (GATED ? 8 : ROWS);
    const int stages = units <= sms ? 2 * st_stages(KU) : st_stages(KU);
    const int fit = units <= sms ? sms : 2 * sms;
    g_launch_error = rdl_launch(gemm_stream_kernel<NT, GATED, KU, MODE>, dim3(units < fit ? units : fit), dim3(ST_THREADS), (size_t)stages * st_tile_bytes(KU), st, a, stages, status);
}

template <int NT, bool GATED, int MODE = 0>
void launch_stream(const SkinnyArgs& a, int* status, cudaStream_t st) {
    const int waste4 = (a.K + st_kt(4) - 1) / st_kt(4) * st_kt(4) - a.K, waste3 = (a.K + st_kt(3) - 1) / st_kt(3) * st_kt(3) - a.K;
    // Tiles of 768 k where they divide the row better, unless the output is very wide: there the kernel runs in
    // its steady state, where the larger copies of 1024 k were measured faster (the output head: 162 against 174 us).
    const int units = (a.N + (GATED ? 8 : ROWS) - 1) / (GATED ? 8 : ROWS);
    if (waste3 < waste4 && units <= 4096) launch_stream_ku<NT, GATED, 3, MODE>(a, status, st);
    else launch_stream_ku<NT, GATED, 4, MODE>(a, status, st);
}

}  // namespace

extern "C" int rdl_gemm_skinny(void* out, int out_dtype, const void* x, const void* w, int m, int n, int k,
                               int gated, int activation, float softcap, int* status, void* stream) {
    RDL_REQUIRE(out && x && w, "gemm_skinny: missing operand");
    RDL_REQUIRE(rdl_valid_dtype(out_dtype), "gemm_skinny: bad output dtype %d", out_dtype);
    RDL_REQUIRE(m >= 0 && m <= 16, "gemm_skinny: %d rows, at most 16 are supported", m);
    RDL_REQUIRE(n > 0 && k > 0 && k % 8 == 0, "gemm_skinny: n=%d, k=%d; k must be a multiple of 8", n, k);
    RDL_REQUIRE((uintptr_t)x % 16 == 0 && (uintptr_t)w % 16 == 0, "gemm_skinny: operands must start on 16-byte boundaries");
    RDL_REQUIRE(!gated || rdl_activation_known(activation), "gemm_skinny: unknown activation %d", activation);
    RDL_REQUIRE(softcap >= 0.f, "gemm_skinny: soft-cap must not be negative");
    if (m == 0) return 0;
    SkinnyArgs a{(const __nv_bfloat16*)x, (const __nv_bfloat16*)w, out, m, n, k, out_dtype, activation, softcap,
                 rdl_wait_cycles_for(RDL_FAULT_GEMM_STREAM), rdl_test_extra_tx_for(RDL_FAULT_GEMM_STREAM), DeferredNormArgs{}};
    cudaStream_t st = (cudaStream_t)stream;
    g_launch_error = cudaSuccess;
    if (m <= 8) {
        if (gated) launch_stream<1, true>(a, status, st);
        else launch_stream<1, false>(a, status, st);
    } else {
        if (gated) launch_stream<2, true>(a, status, st);
        else launch_stream<2, false>(a, status, st);
    }
    RDL_CHECK_EX(g_launch_error, "gemm_skinny");
    return 0;
}

extern "C" int rdl_gemm_skinny_norm(void* out, int out_dtype, const void* x, const void* w, int m, int n, int k,
                                    int gated, int activation, float softcap, const DeferredNormArgs* norm, int* status,
                                    void* stream) {
    RDL_REQUIRE(x && w && norm, "gemm_skinny_norm: missing operand");
    RDL_REQUIRE(m >= 0 && m <= 8, "gemm_skinny_norm: %d rows, at most 8 are supported", m);
    RDL_REQUIRE(n > 0 && k > 0 && k % 8 == 0, "gemm_skinny_norm: n=%d, k=%d; k must be a multiple of 8", n, k);
    RDL_REQUIRE((uintptr_t)x % 16 == 0 && (uintptr_t)w % 16 == 0, "gemm_skinny_norm: operands must start on 16-byte boundaries");
    RDL_REQUIRE(norm->sums && (uintptr_t)norm->sums % 16 == 0, "gemm_skinny_norm: the partial sums must lie on a 16-byte boundary");
    if (m == 0) return 0;
    SkinnyArgs a{(const __nv_bfloat16*)x, (const __nv_bfloat16*)w, out, m, n, k, out_dtype, activation, softcap,
                 rdl_wait_cycles_for(RDL_FAULT_GEMM_STREAM), rdl_test_extra_tx_for(RDL_FAULT_GEMM_STREAM), *norm};
    cudaStream_t st = (cudaStream_t)stream;
    g_launch_error = cudaSuccess;
    if (norm->mode == RDL_NORM_BRANCH) {
        RDL_REQUIRE(!gated && softcap == 0.f, "gemm_skinny_norm: a branch's product has the plain epilogue");
        RDL_REQUIRE(norm->residual && norm->w1 && norm->w2 && norm->branch && norm->scaled, "gemm_skinny_norm: a branch needs the stream, both norms' weights and its two outputs");
        RDL_REQUIRE(rdl_valid_dtype(norm->w1_dtype) && rdl_valid_dtype(norm->w2_dtype), "gemm_skinny_norm: bad dtype of a norm's weight");
        launch_stream<1, false, 1>(a, status, st);
    } else if (norm->mode == RDL_NORM_DEFERRED) {
        RDL_REQUIRE(out && rdl_valid_dtype(out_dtype), "gemm_skinny_norm: missing output or bad output dtype %d", out_dtype);
        RDL_REQUIRE(!gated || rdl_activation_known(activation), "gemm_skinny_norm: unknown activation %d", activation);
        RDL_REQUIRE(softcap >= 0.f, "gemm_skinny_norm: soft-cap must not be negative");
        RDL_REQUIRE(norm->n_sums > 0 && norm->n_out >= 0 && norm->n_out <= 8, "gemm_skinny_norm: %d units of sums, %d output rows", norm->n_sums, norm->n_out);
        const bool side = norm->residual_out || norm->scaled_next;
        RDL_REQUIRE(!side || (norm->branch_in && norm->residual_in), "gemm_skinny_norm: the stream's update needs the branch and the stream");
        RDL_REQUIRE(!norm->residual_out || norm->residual_out != norm->residual_in, "gemm_skinny_norm: the updated stream needs a buffer of its own (other blocks still read the old one)");
        RDL_REQUIRE(!norm->scaled_next || (norm->w_next && rdl_valid_dtype(norm->w_next_dtype)), "gemm_skinny_norm: the next operand needs the next norm's weight");
        if (m <= 4) {       // both halves of the operand in one fragment: rows 0..3 and 4..7 of x
            if (gated) launch_stream<1, true, 2>(a, status, st);
            else launch_stream<1, false, 2>(a, status, st);
        } else {
            if (gated) launch_stream<2, true, 2>(a, status, st);
            else launch_stream<2, false, 2>(a, status, st);
        }
    } else {
        RDL_REQUIRE(false, "gemm_skinny_norm: unknown mode %d", norm->mode);
    }
    RDL_CHECK_EX(g_launch_error, "gemm_skinny_norm");
    return 0;
}

// ---------------------------------------------------------------------------------------------
// Rows of a residual stream outside a product: what the deferred-norm products do on the side, for the
// first and the last link of a chain and for a consumer that cannot take the deferred form.  One block a row.
// ---------------------------------------------------------------------------------------------
namespace {
__global__ void stream_rows_kernel(const float* __restrict__ sums, int n_sums, float eps1, const __nv_bfloat16* __restrict__ branch,
                                   const float* __restrict__ residual_in, float* __restrict__ residual_out,
                                   const void* __restrict__ w, int w_dtype, float off, __nv_bfloat16* __restrict__ scaled, int width) {
    __shared__ float scratch[33];
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const int m = blockIdx.x;
    float s1 = 0.f;
    if (sums) {
        float t = 0.f;
        for (int u = threadIdx.x; u < n_sums; u += blockDim.x) t += sums[((long long)u * 8 + m) * 4];
        s1 = rsqrtf(block_sum(t, scratch) / (float)width + eps1);
    }
    for (int k = threadIdx.x; k < width; k += blockDim.x) {
        const long long e = (long long)m * width + k;
        float h = residual_in[e];
        if (sums) h += s1 * __bfloat162float(branch[e]);
        if (residual_out) residual_out[e] = h;
        if (scaled) scaled[e] = __float2bfloat16_rn(h * (rdl_load(w, k, w_dtype) + off));
    }
}
}  // namespace

extern "C" int rdl_stream_rows(const float* sums, int n_sums, float eps1, const void* branch, const float* residual_in,
                               float* residual_out, const void* w, int w_dtype, float off, void* scaled,
                               int n_rows, int width, void* stream) {
    RDL_REQUIRE(residual_in && n_rows >= 0 && n_rows <= 8 && width > 0, "stream_rows: bad sizes rows=%d width=%d (at most 8 rows)", n_rows, width);
    RDL_REQUIRE(!sums || (branch && n_sums > 0), "stream_rows: sums without a branch");
    RDL_REQUIRE(!scaled || (w && rdl_valid_dtype(w_dtype)), "stream_rows: the scaled rows need a norm's weight");
    if (n_rows == 0) return 0;
    RDL_CHECK_EX(rdl_launch(stream_rows_kernel, dim3(n_rows), dim3(256), 0, (cudaStream_t)stream, sums, n_sums, eps1,
                            (const __nv_bfloat16*)branch, residual_in, residual_out, w, w_dtype, off, (__nv_bfloat16*)scaled, width),
                 "stream_rows");
    return 0;
}
