// Matrix product for many rows (prefill) on the fifth-generation tensor cores:
//   out[m, n] = epilogue(sum_k x[m, k] * w[n, k]),  bfloat16 operands, float accumulation in TMEM.
//
// Two kernels.  Where a tile's products are many (the gated form, sums of 4096 terms and more) a pair of
// blocks on two multiprocessors computes a 256 x 256 tile with tcgen05.mma.cta_group::2 (further down).
// Otherwise one block computes a 128 x BN tile (or two of them, one above the other, that share the
// weight tile).  Operand tiles of 64 k (128 bytes a row) are brought into
// shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle) through a ring of stages guarded
// by mbarriers; one thread issues tcgen05.mma (M 128, N BN, K 16) from shared-memory descriptors,
// accumulating in tensor memory; tcgen05.commit hands stages back to the loader and the finished
// accumulator to the epilogue warps, which read it with tcgen05.ld, apply the epilogue in float and
// store.  Warp roles: warp 0 loads, warp 1 allocates tensor memory and issues the products, warps
// 2-9 do the epilogue (two per 32-lane quarter of tensor memory, half of the columns each).
//
// Epilogues: store as bfloat16 or float; cap * tanh(v / cap); and, for a row-concatenated
// [gate; up] matrix, act(gate) * up with both accumulators side by side in tensor memory, which
// saves writing and re-reading the [rows, 2I] intermediate.
// (y = x W^T, W [out, in]: rustml/nn/main/src/core/linear.rs:12-15; the gated form:
// rustml/nn/main/src/core/feed_forward.rs:151-161.)
//
// Every wait is bounded (about a second of clock cycles); a block that gives up sets `status`,
// and every path ends in the common tear-down that frees the tensor memory.
#include <cuda.h>

#include <cstdlib>
#include <map>
#include <mutex>
#include <tuple>

#include "activations.cuh"
#include "api.h"
#include "common.cuh"
#include "launch.cuh"

namespace {

constexpr int BM = 128, BK = 64, TC_THREADS = 320;
constexpr long long WAIT_CYCLES = RDL_WAIT_CYCLES;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity))
        if (clock64() - t0 > WAIT_CYCLES) return false;
    return true;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar) : "memory");
}
// K-major operand tile in shared memory, rows of 128 bytes, 128-byte swizzle: groups of 8 rows are 1024 bytes apart
__device__ __forceinline__ uint64_t umma_desc(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFF) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// kind::f16 instruction descriptor: float accumulator, bfloat16 A and B, both K-major, N >> 3 at bit 17, M >> 4 at bit 24
__host__ __device__ constexpr uint32_t umma_idesc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                   "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
                   "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
                   "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}


struct TcArgs {
    void* out;
    int M, N, K;
    int out_dtype, activation;
    float softcap;
    int* status;
};


// 32 consecutive outputs of one row, from column `col`
__device__ __forceinline__ void store_row_piece(const TcArgs& a, long long base, int col, bool vec, const float (&v)[32]) {
    if (vec && col + 32 <= a.N) {
        if (a.out_dtype == RDL_BF16) {
            __nv_bfloat16* o = (__nv_bfloat16*)a.out + base;
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
                uint4 raw;
                __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
                h[0] = __floats2bfloat162_rn(v[i], v[i + 1]);
                h[1] = __floats2bfloat162_rn(v[i + 2], v[i + 3]);
                h[2] = __floats2bfloat162_rn(v[i + 4], v[i + 5]);
                h[3] = __floats2bfloat162_rn(v[i + 6], v[i + 7]);
                *reinterpret_cast<uint4*>(o + i) = raw;
            }
        } else {
            float* o = (float*)a.out + base;
#pragma unroll
            for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4*>(o + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
        }
    } else {
        for (int i = 0; i < 32; ++i)
            if (col + i < a.N) rdl_store(a.out, base + i, a.out_dtype, v[i]);
    }
}

// ---- the epilogue of a warp: its 32 rows (tensor-memory lanes) of columns [c_begin, c_end) of the tile ----
//
// A thread reads consecutive columns of its own row, so a direct store instruction writes 16 bytes of 32
// different rows: 32 partial lines.  For bfloat16 results the warp therefore passes 32 rows x 64 columns
// (128 bytes a row) through 4 KB of shared memory of its own and writes them out with each instruction
// covering four whole lines.  The 16-byte chunk c of row r lies at chunk c ^ (r & 7), which keeps both
// the writes (a thread a row) and the reads (eight threads a row) free of bank conflicts.
constexpr int EPI_STAGE_BYTES = 32 * 128;                  // a warp's staging area
constexpr int EPI_WARPS = 8;

template <bool GATED>
__device__ __forceinline__ void epilogue_piece(const TcArgs& a, uint32_t taddr, uint32_t up_offset, float (&v)[32]) {
    tmem_ld32(taddr, v);
    if (GATED) {
        float u[32];
        tmem_ld32(taddr + up_offset, u);
        // the gated result is rounded to bfloat16: the fast forms are accurate enough.  The choice is made
        // once a piece, not once a value: otherwise both activations are computed for each.
        if (a.activation == RDL_ACT_GELU_TANH) {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = rdl_activation_fast(v[i], RDL_ACT_GELU_TANH) * u[i];
        } else {
            const int act = a.activation;
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = rdl_activation_fast(v[i], act) * u[i];
        }
    }
    if (a.softcap > 0.f) {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = a.softcap * tanhf(v[i] / a.softcap);
    }
}

// tcol: tensor-memory address of the warp's lanes at column 0 of the tile; row0: the row of lane 0
template <bool GATED>
__device__ __forceinline__ void epilogue_columns(const TcArgs& a, uint32_t tcol, uint32_t up_offset, int c_begin, int c_end,
                                                 int n0, int row0, int lane, unsigned char* stage) {
    const bool vec = (a.N % 8) == 0;
    const bool through_smem = vec && a.out_dtype == RDL_BF16;
#pragma unroll 1
    for (int c0 = c_begin; c0 < c_end; c0 += 64) {
        if (n0 + c0 >= a.N) break;                         // uniform over the warp
        if (through_smem && n0 + c0 + 64 <= a.N) {
#pragma unroll
            for (int p = 0; p < 2; ++p) {
                float v[32];
                epilogue_piece<GATED>(a, tcol + c0 + p * 32, up_offset, v);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    uint4 raw;
                    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
                    h[0] = __floats2bfloat162_rn(v[8 * i], v[8 * i + 1]);
                    h[1] = __floats2bfloat162_rn(v[8 * i + 2], v[8 * i + 3]);
                    h[2] = __floats2bfloat162_rn(v[8 * i + 4], v[8 * i + 5]);
                    h[3] = __floats2bfloat162_rn(v[8 * i + 6], v[8 * i + 7]);
                    *reinterpret_cast<uint4*>(stage + lane * 128 + (((p * 4 + i) ^ (lane & 7)) << 4)) = raw;
                }
            }
            __syncwarp();
            const int c = lane & 7;
            __nv_bfloat16* o = (__nv_bfloat16*)a.out + (long long)row0 * a.N + n0 + c0 + c * 8;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int r = j * 4 + (lane >> 3);
                const uint4 raw = *reinterpret_cast<const uint4*>(stage + r * 128 + ((c ^ (r & 7)) << 4));
                if (row0 + r < a.M) *reinterpret_cast<uint4*>(o + (long long)r * a.N) = raw;
            }
            __syncwarp();                                  // the staging area is free for the next columns
        } else {
#pragma unroll 1
            for (int p = 0; p < 2; ++p) {
                if (n0 + c0 + p * 32 >= a.N) break;
                float v[32];
                epilogue_piece<GATED>(a, tcol + c0 + p * 32, up_offset, v);
                if (row0 + lane < a.M) store_row_piece(a, (long long)(row0 + lane) * a.N + n0 + c0 + p * 32, n0 + c0 + p * 32, vec, v);
            }
        }
    }
}

constexpr int RASTER_GROUP = 8;   // row tiles that share a weight tile and are scheduled together

// MT: row tiles of 128 a block computes (1 or 2).  Two tiles share every weight tile that is loaded,
// which halves the bytes fetched per product: a 256 x 256 tile needs 64 KB of operands for 8.4 MFLOP.
template <int BN, bool GATED, int MT>
__global__ void __launch_bounds__(TC_THREADS, 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap map_x,
                                                                const __grid_constant__ CUtensorMap map_w, TcArgs a) {
    constexpr int NB = GATED ? 2 : 1;
    constexpr int STAGES = MT == 2 ? 3 : 4;
    constexpr int A_BYTES = MT * BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + NB * B_BYTES;
    constexpr int TMEM_COLS = MT * NB * BN;
    static_assert(TMEM_COLS == 32 || TMEM_COLS == 64 || TMEM_COLS == 128 || TMEM_COLS == 256 || TMEM_COLS == 512, "tensor memory is allocated in powers of two");
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) unsigned long long full_bar[STAGES], empty_bar[STAGES], done_bar;
    __shared__ uint32_t tmem_slot;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Blocks are numbered so that up to eight row tiles that share a weight tile follow one another: they
    // run at the same time, the weight tile comes from HBM once and the eight row tiles stay in L2.
    int m0, n0;
    {
        const int tiles_m = (a.M + MT * BM - 1) / (MT * BM), tiles_n = (a.N + BN - 1) / BN;
        const int per_group = RASTER_GROUP * tiles_n;
        const int group = blockIdx.x / per_group, in_group = blockIdx.x - group * per_group;
        const int first_m = group * RASTER_GROUP;
        const int gm = tiles_m - first_m < RASTER_GROUP ? tiles_m - first_m : RASTER_GROUP;
        m0 = (first_m + in_group % gm) * (MT * BM);
        n0 = (in_group / gm) * BN;
    }
    const int kblocks = (a.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        mbar_init(smem_u32(&done_bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_slot;
    bool ok = true;
    // barriers and tensor memory were set up while the kernel before was still running; its results are needed from here on
    rdl_grid_wait();
    rdl_grid_launch_dependents();

    if (warp == 0) {
        if (lane == 0) {
            // ---- loader ----
            for (int kb = 0; kb < kblocks; ++kb) {
                const int s = kb % STAGES;
                const uint32_t parity = ((kb / STAGES) & 1) ^ 1;        // the first pass finds every stage free
                if (!mbar_wait_bounded(smem_u32(&empty_bar[s]), parity)) { ok = false; break; }
                const uint32_t full = smem_u32(&full_bar[s]);
                unsigned char* stage = smem + (size_t)s * STAGE_BYTES;
                mbar_expect_tx(full, STAGE_BYTES);
                tma_load_2d(smem_u32(stage), &map_x, kb * BK, m0, full);
                tma_load_2d(smem_u32(stage + A_BYTES), &map_w, kb * BK, n0, full);
                if (GATED) tma_load_2d(smem_u32(stage + A_BYTES + B_BYTES), &map_w, kb * BK, a.N + n0, full);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- product issuer ----
            constexpr uint32_t idesc = umma_idesc(BM, BN);
            for (int kb = 0; kb < kblocks && ok; ++kb) {
                const int s = kb % STAGES;
                if (!mbar_wait_bounded(smem_u32(&full_bar[s]), (kb / STAGES) & 1)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_addr = smem_u32(smem + (size_t)s * STAGE_BYTES);
                const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
                for (int k = 0; k < BK / 16; ++k) {
                    const uint32_t acc = (kb | k) != 0;
#pragma unroll
                    for (int h = 0; h < MT; ++h) {
                        const uint64_t adesc = umma_desc(a_addr + h * (BM * BK * 2) + k * 32);
                        umma(tmem_base + h * NB * BN, adesc, umma_desc(b_addr + k * 32), idesc, acc);
                        if (GATED) umma(tmem_base + h * NB * BN + BN, adesc, umma_desc(b_addr + B_BYTES + k * 32), idesc, acc);
                    }
                }
                umma_commit(smem_u32(&empty_bar[s]));     // the stage is free once these products have read it
            }
            umma_commit(smem_u32(&done_bar));             // the accumulator is complete
        }
    } else {
        // ---- epilogue: warp q of these four owns tensor-memory lanes [32 q, 32 q + 32) ----
        const int q = warp & 3;
        const int col_half = (warp - 2) >> 2;              // two warps share a quarter: each takes half of the columns
        if (!mbar_wait_bounded(smem_u32(&done_bar), 0)) ok = false;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        unsigned char* stage = smem + (size_t)STAGES * STAGE_BYTES + (size_t)(warp - 2) * EPI_STAGE_BYTES;
#pragma unroll 1
        for (int h = 0; h < MT && ok; ++h) {
            if (m0 + h * BM >= a.M) break;                 // uniform over the block
            const uint32_t tcol = tmem_base + ((uint32_t)(q * 32) << 16) + h * NB * BN;
            epilogue_columns<GATED>(a, tcol, BN, col_half * (BN / 2), (col_half + 1) * (BN / 2), n0, m0 + h * BM + q * 32, lane, stage);
        }
    }
    if (!ok && a.status) atomicExch(a.status, RDL_FAULT_GEMM_TC);
    // ---- tear-down, reached by every thread ----
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
}


// ---- two multiprocessors on one tile (cta_group::2) -------------------------------------------------
//
// A pair of blocks (a cluster of two) computes a 256 x 256 tile: block r of the pair holds rows
// [128 r, 128 r + 128) of the activations and rows [128 r, 128 r + 128) of the weight tile, that is
// half of each operand.  One thread of block 0 issues tcgen05.mma.cta_group::2 (M 256, N 256, K 16):
// the tensor cores of both multiprocessors read both halves of the weight tile, and each writes its
// 128 rows of the result into its own tensor memory.  Per product a multiprocessor then reads 8 KB of
// shared memory for 64 cycles of arithmetic, where a single block that holds both operands whole reads
// 12 KB - more than its shared memory delivers in that time.
// Both blocks load their halves by TMA; all transfers of a stage report to one barrier in block 0,
// and tcgen05.commit with a multicast to both blocks hands the stage back to both loaders.
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_block(uint32_t addr, uint32_t rank) {      // the same place in the shared memory of block `rank`
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.aligned;\nbarrier.cluster.wait.aligned;" ::: "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {        // arrives at `bar` in both blocks of the pair
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((unsigned short)3) : "memory");
}

constexpr int PAIR_BN = 256, PAIR_THREADS = 320, PAIR_STAGES = 6;

__device__ __forceinline__ void mbar_arrive_at(uint32_t cluster_addr) {      // a barrier in any block of the cluster
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// The pair is persistent: it takes tiles pair, pair + pairs, ... of the grouped order.  The loaders run
// ahead into the next tile while the current one is still being multiplied or stored, so a tile's
// first operands are there when its products start.  The accumulator takes half of tensor memory, so
// there can be two: the products of a tile run while the tile before it is stored.  In the main loop a
// block fetches 32 KB of operands for 512 cycles of products; at full rate that is more than the L2 cache
// was seen to deliver to 148 multiprocessors (about 11.6 TB/s), so long sums run at about 80 % of the
// tensor cores' rate.
//
// The gated form is the same product with other weight rows: block 0 of the pair loads 128 gate rows
// and block 1 the 128 up rows of the same outputs, so the accumulator's columns [0, 128) are the gate and
// [128, 256) the up values of a 256 x 128 tile of the result, and the epilogue multiplies them.
template <bool GATED, int NACC>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PAIR_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, TcArgs a) {
    constexpr int HALF = PAIR_BN / 2;                                  // weight rows a block holds
    constexpr int OUT_BN = GATED ? HALF : PAIR_BN;                     // columns of the result a tile covers
    constexpr int A_BYTES = BM * BK * 2, B_BYTES = HALF * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr int STAGES = PAIR_STAGES;
    constexpr int TMEM_COLS = NACC * PAIR_BN;                          // NACC accumulators of 256 columns
    static_assert(TMEM_COLS == 256 || TMEM_COLS == 512, "tensor memory has 512 columns");
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) unsigned long long full_bar[STAGES], empty_bar[STAGES], acc_full[NACC], acc_empty[NACC];
    __shared__ uint32_t tmem_slot;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int tiles_m = (a.M + 2 * BM - 1) / (2 * BM), tiles_n = (a.N + OUT_BN - 1) / OUT_BN;
    const int n_tiles = tiles_m * tiles_n, pairs = gridDim.x >> 1, first_tile = blockIdx.x >> 1;
    auto tile_origin = [&](int tile, int& m0, int& n0) {
        const int per_group = RASTER_GROUP * tiles_n;
        const int group = tile / per_group, in_group = tile - group * per_group;
        const int first_m = group * RASTER_GROUP;
        const int gm = tiles_m - first_m < RASTER_GROUP ? tiles_m - first_m : RASTER_GROUP;
        m0 = (first_m + in_group % gm) * (2 * BM);
        n0 = (in_group / gm) * OUT_BN;
    };
    const int kblocks = (a.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int b = 0; b < NACC; ++b) {
            mbar_init(smem_u32(&acc_full[b]), 1);
            mbar_init(smem_u32(&acc_empty[b]), 16);        // the eight epilogue warps of both blocks (used in block 0)
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {       // the same warp of both blocks: the allocation is made for the pair
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync();        // both blocks have their barriers and their tensor memory before anything crosses
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_slot;
    bool ok = true;
    rdl_grid_wait();
    rdl_grid_launch_dependents();

    if (warp == 0) {
        if (lane == 0) {
            // ---- loader (in both blocks): own half of each operand; every transfer reports to block 0 ----
            int it = 0;                                     // k-blocks loaded so far, over all tiles
            for (int tile = first_tile; tile < n_tiles && ok; tile += pairs) {
                int m0, n0;
                tile_origin(tile, m0, n0);
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait_bounded(smem_u32(&empty_bar[s]), ((it / STAGES) & 1) ^ 1)) { ok = false; break; }
                    const uint32_t full = map_to_block(smem_u32(&full_bar[s]), 0);
                    unsigned char* stage = smem + (size_t)s * STAGE_BYTES;
                    if (rank == 0) mbar_expect_tx(smem_u32(&full_bar[s]), 2 * STAGE_BYTES);
                    tma_load_2d_pair(smem_u32(stage), &map_x, kb * BK, m0 + (int)rank * BM, full);
                    tma_load_2d_pair(smem_u32(stage + A_BYTES), &map_w, kb * BK, GATED ? n0 + (int)rank * a.N : n0 + (int)rank * HALF, full);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // ---- product issuer: one thread for the pair ----
            constexpr uint32_t idesc = umma_idesc(2 * BM, PAIR_BN);
            const uint64_t desc0 = umma_desc(smem_u32(smem));
            int it = 0, lt = 0;
            for (int tile = first_tile; tile < n_tiles && ok; tile += pairs, ++lt) {
                const int buf = lt % NACC;
                // the accumulator must have been read out by the epilogue of the tile that used it last
                if (!mbar_wait_bounded(smem_u32(&acc_empty[buf]), ((lt / NACC) & 1) ^ 1)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t acc_addr = tmem_base + (uint32_t)(buf * PAIR_BN);
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait_bounded(smem_u32(&full_bar[s]), (it / STAGES) & 1)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t adesc = desc0 + (uint32_t)((s * STAGE_BYTES) >> 4);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        const uint32_t acc = (kb | k) != 0;
                        umma_pair(acc_addr, adesc + (uint32_t)(k * 2), adesc + (uint32_t)((A_BYTES >> 4) + k * 2), idesc, acc);
                    }
                    umma_commit_pair(smem_u32(&empty_bar[s]));
                }
                if (ok) umma_commit_pair(smem_u32(&acc_full[buf]));
            }
        }
    } else {
        // ---- epilogue: each block stores its own 128 rows of every tile of the pair ----
        const int q = warp & 3;
        const int col_half = (warp - 2) >> 2;
        unsigned char* stage = smem + (size_t)STAGES * STAGE_BYTES + (size_t)(warp - 2) * EPI_STAGE_BYTES;
        const uint32_t acc_empty_at_leader0 = map_to_block(smem_u32(&acc_empty[0]), 0);
        int lt = 0;
        for (int tile = first_tile; tile < n_tiles && ok; tile += pairs, ++lt) {
            const int buf = lt % NACC;
            int m0, n0;
            tile_origin(tile, m0, n0);
            const int my_m0 = m0 + (int)rank * BM;
            if (!mbar_wait_bounded(smem_u32(&acc_full[buf]), (lt / NACC) & 1)) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t tcol = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * PAIR_BN);
            if (my_m0 < a.M)
                epilogue_columns<GATED>(a, tcol, HALF, col_half * (OUT_BN / 2), (col_half + 1) * (OUT_BN / 2), n0, my_m0 + q * 32, lane, stage);
            // this warp has read its part of the accumulator: tell the issuer in block 0
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_at(acc_empty_at_leader0 + (uint32_t)(buf * 8));
        }
    }
    if (!ok && a.status) atomicExch(a.status, RDL_FAULT_GEMM_TC_PAIR);
    // ---- tear-down, reached by every thread of both blocks ----
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync();        // neither block leaves while the other may still read its shared memory or report to its barriers
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
}

// tensor map of a row-major bfloat16 matrix [rows, cols]: boxes of 64 columns (128 bytes, swizzled) x box_rows rows
int make_map(CUtensorMap* map, const void* ptr, long long rows, long long cols, int box_rows) {
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    // The driver's encoder is looked up at run time, so that the library itself does not link against the
    // driver and loads (for a build check, say) on a machine that has none.
    typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeTiled encode = nullptr;
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult found;
        RDL_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &found), "gemm_tc: looking up cuTensorMapEncodeTiled");
        RDL_REQUIRE(found == cudaDriverEntryPointSuccess && fn, "gemm_tc: this driver has no cuTensorMapEncodeTiled");
        encode = (EncodeTiled)fn;
    }
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    RDL_REQUIRE(r == CUDA_SUCCESS, "gemm_tc: cuTensorMapEncodeTiled failed with driver error %d for a [%lld, %lld] matrix", (int)r, rows, cols);
    return 0;
}

// weight matrices are constant: their maps are made once
std::mutex g_map_mutex;
std::map<std::tuple<const void*, long long, long long, int>, CUtensorMap> g_weight_maps;

template <int BN, bool GATED, int MT>
int launch_tc(const CUtensorMap& mx, const CUtensorMap& mw, const TcArgs& a, cudaStream_t st) {
    constexpr int NB = GATED ? 2 : 1;
    constexpr int STAGES = MT == 2 ? 3 : 4;
    const int smem = STAGES * (MT * BM * BK * 2 + NB * BN * BK * 2) + EPI_WARPS * EPI_STAGE_BYTES + 1024;
    static bool opted = false;
    if (!opted) {
        RDL_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<BN, GATED, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "gemm_tc");
        opted = true;
    }
    const long long tiles = (long long)((a.N + BN - 1) / BN) * ((a.M + MT * BM - 1) / (MT * BM));
    RDL_REQUIRE(tiles <= 0x7fffffffLL, "gemm_tc: %lld tiles exceed the grid limit", tiles);
    dim3 grid((unsigned)tiles);
    RDL_CHECK_EX(rdl_launch(gemm_tc_kernel<BN, GATED, MT>, grid, dim3(TC_THREADS), (size_t)smem, st, mx, mw, a), "gemm_tc");
    return 0;
}

template <bool GATED, int NACC>
int launch_pair(const CUtensorMap& mx, const CUtensorMap& mw, const TcArgs& a, cudaStream_t st) {
    constexpr int OUT_BN = GATED ? PAIR_BN / 2 : PAIR_BN;
    const int smem = PAIR_STAGES * (BM * BK * 2 + (PAIR_BN / 2) * BK * 2) + EPI_WARPS * EPI_STAGE_BYTES + 1024;
    static bool opted = false;
    if (!opted) {
        RDL_CUDA(cudaFuncSetAttribute(gemm_tc_pair_kernel<GATED, NACC>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "gemm_tc");
        opted = true;
    }
    const long long tiles = (long long)((a.N + OUT_BN - 1) / OUT_BN) * ((a.M + 2 * BM - 1) / (2 * BM));
    RDL_REQUIRE(tiles <= 0x3fffffffLL, "gemm_tc: %lld tiles are too many", tiles);
    static int pairs_that_fit = 0;             // one block per multiprocessor: half as many pairs
    if (!pairs_that_fit) {
        const int sms = rdl_sm_count();
        pairs_that_fit = sms / 2 > 0 ? sms / 2 : 1;
    }
    const int pairs = tiles < pairs_that_fit ? (int)tiles : pairs_that_fit;
    RDL_CHECK_EX(rdl_launch(gemm_tc_pair_kernel<GATED, NACC>, dim3((unsigned)(2 * pairs)), dim3(PAIR_THREADS), (size_t)smem, st, mx, mw, a), "gemm_tc");
    return 0;
}

}  // namespace

extern "C" int rdl_gemm_tc(void* out, int out_dtype, const void* x, const void* w, int m, int n, int k,
                           int gated, int activation, float softcap, int* status, void* stream) {
    RDL_REQUIRE(out && x && w, "gemm_tc: missing operand");
    RDL_REQUIRE(rdl_valid_dtype(out_dtype), "gemm_tc: bad output dtype %d", out_dtype);
    RDL_REQUIRE(m >= 0 && n > 0 && k > 0 && k % 8 == 0, "gemm_tc: m=%d n=%d k=%d; k must be a multiple of 8", m, n, k);
    RDL_REQUIRE((uintptr_t)x % 16 == 0 && (uintptr_t)w % 16 == 0 && (uintptr_t)out % 16 == 0,
                "gemm_tc: operands must start on 16-byte boundaries");
    RDL_REQUIRE(!gated || rdl_activation_known(activation), "gemm_tc: unknown activation %d", activation);
    RDL_REQUIRE(softcap >= 0.f, "gemm_tc: soft-cap must not be negative");
    if (m == 0) return 0;
    // Pairs of multiprocessors on 256 x 256 tiles where a tile's products are many (the gated form, or a long
    // sum) or where every pair gets several tiles (its second accumulator then hides the stores): measured 5 to
    // 25 % faster there; with a short sum and few tiles the pair's longer set-up and drain cost more than they
    // bring.  RDL_GEMM_PAIR=0 / 1 forces single blocks / pairs, for comparison.
    static const int pair_mode = getenv("RDL_GEMM_PAIR") ? atoi(getenv("RDL_GEMM_PAIR")) : -1;
    const long long tiles_of_pairs = (long long)((n + 255) / 256) * ((m + 2 * BM - 1) / (2 * BM));
    const bool pair = m > BM && (pair_mode == 1 || (pair_mode != 0 && (gated || k >= 4096 || tiles_of_pairs >= 4 * (rdl_sm_count() / 2))));
    const int bn = pair ? PAIR_BN / 2 : (gated ? 128 : 256);      // weight rows per TMA box
    // two row tiles a block when that still fills most (four in five) of the multiprocessors
    const long long tiles2 = (long long)((n + bn - 1) / bn) * ((m + 2 * BM - 1) / (2 * BM));
    const int mt = pair ? 1 : (tiles2 * 5 >= rdl_sm_count() * 4 ? 2 : 1);
    CUtensorMap mx, mw;
    if (int e = make_map(&mx, x, m, k, mt * BM)) return e;
    {
        std::lock_guard<std::mutex> lock(g_map_mutex);
        const auto key = std::make_tuple(w, (long long)(gated ? 2 * n : n), (long long)k, bn);
        auto it = g_weight_maps.find(key);
        if (it == g_weight_maps.end()) {
            CUtensorMap fresh;
            if (int e = make_map(&fresh, w, gated ? 2LL * n : n, k, bn)) return e;
            it = g_weight_maps.emplace(key, fresh).first;
        }
        mw = it->second;
    }
    TcArgs a{out, m, n, k, out_dtype, activation, softcap, status};
    cudaStream_t st = (cudaStream_t)stream;
    if (pair) {
        // a second accumulator (the products of a tile run while the tile before it is stored) where a pair
        // gets more than one tile and tensor memory has room for it
        const int out_bn = gated ? PAIR_BN / 2 : PAIR_BN;
        const long long pair_tiles = (long long)((n + out_bn - 1) / out_bn) * ((m + 2 * BM - 1) / (2 * BM));
        if (gated) return pair_tiles > rdl_sm_count() / 2 ? launch_pair<true, 2>(mx, mw, a, st) : launch_pair<true, 1>(mx, mw, a, st);
        return pair_tiles > rdl_sm_count() / 2 ? launch_pair<false, 2>(mx, mw, a, st) : launch_pair<false, 1>(mx, mw, a, st);
    }
    if (mt == 2) return gated ? launch_tc<128, true, 2>(mx, mw, a, st) : launch_tc<256, false, 2>(mx, mw, a, st);
    return gated ? launch_tc<128, true, 1>(mx, mw, a, st) : launch_tc<256, false, 1>(mx, mw, a, st);
}
