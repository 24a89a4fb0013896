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
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

template <int NT, bool GATED, int KU>
__global__ void __launch_bounds__(ST_THREADS, 2) gemm_stream_kernel(SkinnyArgs a, int stages, int* status) {
    constexpr int ST_KT = st_kt(KU), ST_PITCH = st_pitch(KU), ST_TILE_BYTES = st_tile_bytes(KU), KW = 32 * KU;
    extern __shared__ __align__(128) unsigned char st_tiles[];
    __shared__ __align__(8) unsigned long long full_bar[ST_MAX_STAGES], empty_bar[ST_MAX_STAGES];
    __shared__ float partial[ST_WARPS][NT][ROWS * 8];
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
            x_ok[i] = i * 8 + g < a.M;
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
        const uint32_t frag = tiles_s + (uint32_t)(g * ST_PITCH + (kw + t * 8) * 2);
        int s = 0;
        uint32_t round = 0;
        for (int unit = blockIdx.x; unit < n_units; unit += gridDim.x) {
            float acc[NT][4];
#pragma unroll
            for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
            for (int tk = 0; tk < tiles_per_unit; ++tk) {
                // the activations of the tile after this one (the next unit starts again at k = 0)
                if (X_AHEAD) load_x((tk + 1 < tiles_per_unit ? (tk + 1) * ST_KT : 0) + kw, reinterpret_cast<uint4 (&)[NT][KU]>(xnext));
                else load_x(tk * ST_KT + kw, xcur);
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

template <int NT, bool GATED, int KU>
void launch_stream_ku(const SkinnyArgs& a, int* status, cudaStream_t st) {
    constexpr int smem_max = 2 * st_stages(KU) * st_tile_bytes(KU);
    static_assert(2 * st_stages(KU) <= ST_MAX_STAGES, "the ring's barriers");
    static bool opted = false;
    static int sms = 0;
    if (!opted) {
        g_launch_error = cudaFuncSetAttribute(gemm_stream_kernel<NT, GATED, KU>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_max);
        if (g_launch_error != cudaSuccess) return;
        sms = rdl_sm_count();
        opted = true;
    }
    // What counts is the bytes a multiprocessor has in flight: two blocks with three tiles each, or, where
    // the output is so narrow that there is at most one block a multiprocessor, one block with twice as many.
    const int units = (a.N + (GATED ? 8 : ROWS) - 1) / (GATED ? 8 : ROWS);
    const int stages = units <= sms ? 2 * st_stages(KU) : st_stages(KU);
    const int fit = units <= sms ? sms : 2 * sms;
    g_launch_error = rdl_launch(gemm_stream_kernel<NT, GATED, KU>, dim3(units < fit ? units : fit), dim3(ST_THREADS), (size_t)stages * st_tile_bytes(KU), st, a, stages, status);
}

template <int NT, bool GATED>
void launch_stream(const SkinnyArgs& a, int* status, cudaStream_t st) {
    const int waste4 = (a.K + st_kt(4) - 1) / st_kt(4) * st_kt(4) - a.K, waste3 = (a.K + st_kt(3) - 1) / st_kt(3) * st_kt(3) - a.K;
    // Tiles of 768 k where they divide the row better, unless the output is very wide: there the kernel runs in
    // its steady state, where the larger copies of 1024 k were measured faster (the output head: 162 against 174 us).
    const int units = (a.N + (GATED ? 8 : ROWS) - 1) / (GATED ? 8 : ROWS);
    if (waste3 < waste4 && units <= 4096) launch_stream_ku<NT, GATED, 3>(a, status, st);
    else launch_stream_ku<NT, GATED, 4>(a, status, st);
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
                 rdl_wait_cycles_for(RDL_FAULT_GEMM_STREAM), rdl_test_extra_tx_for(RDL_FAULT_GEMM_STREAM)};
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
