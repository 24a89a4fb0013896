// Prefill attention on the fifth-generation tensor cores, for prompts that start at position 0
// (all keys and values are this step's packed rows) and head sizes that are multiples of 64.
//
// One block = 128 query rows of one sequence and one head.  Query, key and value tiles come by TMA
// (cp.async.bulk.tensor, 128-byte swizzle) straight out of the packed [tokens, heads * head_dim]
// rows; scores S = Q K^T (128 x 64 a tile) and the output O += P V (128 x head_dim) are tcgen05.mma
// products whose accumulators live in tensor memory; keys and values are double-buffered.
// Warp 0 loads, warp 1 issues products, warps 2-5 do the softmax: each of their 128 threads owns
// one query row, reads its 64 scores with tcgen05.ld, applies scale, soft-cap and masks in float,
// keeps the running maximum and sum, writes the probabilities as bfloat16 into shared memory (the
// A operand of P V) and, at the end, normalises and stores its output row.
//
// The output in tensor memory is rescaled only when a row's maximum has grown by more than 2^8
// since the last rescale (the probabilities are then at most 256, far inside bfloat16's and
// float's range); the final division by the running sum makes the result exact either way.
// Formulas as in attention_plain.cu.  Every wait is bounded; a block that gives up sets `status`.
#include <cuda.h>

#include "api.h"
#include "launch.cuh"
#include "common.cuh"

namespace {

constexpr int QM = 128, KN = 64, ATC_THREADS = 192;
constexpr long long WAIT_CYCLES = RDL_WAIT_CYCLES;
constexpr float RESCALE_STEP = 8.0f;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
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
// K-major tile, rows of 128 bytes, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t desc_k_major(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFF) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// MN-major tile (the contiguous direction is N): blocks of 64 N-elements `lbo` bytes apart, 8-row K groups 1024 bytes apart
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t addr, uint32_t lbo) {
    return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)(lbo >> 4) << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ uint32_t idesc_bf16(int m, int n, int b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
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
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
                 ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
                   "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
                   "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
                   "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
                   "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
                   "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
                   "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
                   "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
                 : "memory");
}
__device__ __forceinline__ float tanh_fast(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float exp2_fast(float x) {      // 2^x, -inf gives 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

struct TcAttnArgs {
    void* out; long long out_stride;
    const int* tile_seq; const int* tile_q0; int n_tiles;
    const int* seq_start;
    int n_heads, n_kv_heads, head_dim;
    float score_scale, softcap;
    int window;
    int* status;
};

// DB: 64-column blocks of a head (head_dim / 64)
template <int DB>
__global__ void __launch_bounds__(ATC_THREADS, 1) attention_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                      const __grid_constant__ CUtensorMap map_kv, TcAttnArgs a) {
    // 64-row tiles come from the host; a block takes two of them, so odd ones have nothing to do
    // later tiles have more keys: they start first, and the heads of a tile follow one another, so that over
    // the whole grid the blocks are handed out from the longest to the shortest
    const int tile = a.n_tiles - 1 - blockIdx.y;
    const int q0 = a.tile_q0[tile];
    if (q0 % QM) return;
    const int seq = a.tile_seq[tile], h = blockIdx.x;
    const int row0 = a.seq_start[seq];
    const int n_new = a.seq_start[seq + 1] - row0;
    const int rows = min(QM, n_new - q0);
    constexpr int hd = DB * 64;
    const int g = h / (a.n_heads / a.n_kv_heads);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t q_bytes = QM * hd * 2, kv_bytes = KN * hd * 2;
    unsigned char* sQ = smem;
    unsigned char* sK = sQ + q_bytes;                  // two stages
    unsigned char* sV = sK + 2 * kv_bytes;             // two stages
    unsigned char* sP = sV + 2 * kv_bytes;             // [128 rows][128 bytes]
    __shared__ __align__(8) unsigned long long q_full, k_full[2], v_full[2], k_empty[2], v_empty[2], s_full, s_empty, p_full, pv_done;
    __shared__ uint32_t tmem_slot;
    const uint32_t tmem_cols = hd <= 64 ? 128 : (hd <= 192 ? 256 : 512);   // 64 for S, head_dim for O, a power of two

    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&q_full), 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&k_full[s]), 1);
            mbar_init(smem_u32(&v_full[s]), 1);
            mbar_init(smem_u32(&k_empty[s]), 1);
            mbar_init(smem_u32(&v_empty[s]), 1);
        }
        mbar_init(smem_u32(&s_full), 1);
        mbar_init(smem_u32(&s_empty), 4);
        mbar_init(smem_u32(&p_full), 4);
        mbar_init(smem_u32(&pv_done), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_s = tmem_slot, tmem_o = tmem_slot + KN;
    // barriers and tensor memory were set up while the kernel before (the rotation) was still running
    rdl_grid_wait();
    rdl_grid_launch_dependents();

    // the tiles of keys this block visits: positions [kv_first, p_last], 64 at a time
    const int p_first = q0, p_last = q0 + rows - 1;
    const int lo_first = a.window > 0 ? max(0, p_first - a.window + 1) : 0;
    const int kv_first = (lo_first / KN) * KN;
    const int n_kv = (p_last - kv_first) / KN + 1;
    bool ok = true;

    if (warp == 0) {
        if (lane == 0) {
            // ---- loader ----
            mbar_expect_tx(smem_u32(&q_full), q_bytes);
            for (int c = 0; c < DB; ++c)
                tma_load_2d(smem_u32(sQ + c * (QM * 128)), &map_q, h * hd + c * 64, row0 + q0, smem_u32(&q_full));
            // A key tile is free again as soon as its scores are computed, a value tile only after P V, one
            // softmax later.  So the keys run one tile further ahead than the values: K(0), K(1), V(0), K(2),
            // V(1), ...; this is also the order in which the buffers become free.
            auto load_k = [&](int j) {
                const int s = j & 1;
                if (!mbar_wait_bounded(smem_u32(&k_empty[s]), ((j >> 1) & 1) ^ 1)) return false;
                mbar_expect_tx(smem_u32(&k_full[s]), kv_bytes);
                for (int c = 0; c < DB; ++c)
                    tma_load_2d(smem_u32(sK + s * kv_bytes + c * (KN * 128)), &map_kv, (a.n_heads + g) * hd + c * 64, row0 + kv_first + j * KN,
                                smem_u32(&k_full[s]));
                return true;
            };
            auto load_v = [&](int j) {
                const int s = j & 1;
                if (!mbar_wait_bounded(smem_u32(&v_empty[s]), ((j >> 1) & 1) ^ 1)) return false;
                mbar_expect_tx(smem_u32(&v_full[s]), kv_bytes);
                for (int c = 0; c < DB; ++c)
                    tma_load_2d(smem_u32(sV + s * kv_bytes + c * (KN * 128)), &map_kv, (a.n_heads + a.n_kv_heads + g) * hd + c * 64,
                                row0 + kv_first + j * KN, smem_u32(&v_full[s]));
                return true;
            };
            ok = load_k(0);
            for (int j = 0; j < n_kv && ok; ++j) {
                if (j + 1 < n_kv) ok = load_k(j + 1);
                if (ok) ok = load_v(j);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- product issuer ----
            const uint32_t idesc_s = idesc_bf16(QM, KN, 0), idesc_o = idesc_bf16(QM, hd, 1);
            // Descriptors are made once; a step along the head dimension adds to the address field (16-byte
            // units): 2 for 16 elements inside a 64-column block, a block's size from one block to the next.
            const uint64_t q_desc = desc_k_major(smem_u32(sQ));
            const uint64_t k_desc0 = desc_k_major(smem_u32(sK)), k_desc1 = desc_k_major(smem_u32(sK + kv_bytes));
            const uint64_t p_desc = desc_k_major(smem_u32(sP));
            const uint64_t v_desc0 = desc_mn_major(smem_u32(sV), KN * 128), v_desc1 = desc_mn_major(smem_u32(sV + kv_bytes), KN * 128);
            auto issue_s = [&](int j) {
                const uint64_t kd = (j & 1) ? k_desc1 : k_desc0;
#pragma unroll
                for (int kk = 0; kk < hd / 16; ++kk) {
                    const uint32_t qo = (uint32_t)((kk >> 2) * (QM * 128) + (kk & 3) * 32) >> 4;
                    const uint32_t ko = (uint32_t)((kk >> 2) * (KN * 128) + (kk & 3) * 32) >> 4;
                    umma(tmem_s, q_desc + qo, kd + ko, idesc_s, kk != 0);
                }
                umma_commit(smem_u32(&s_full));
                umma_commit(smem_u32(&k_empty[j & 1]));
            };
            ok = mbar_wait_bounded(smem_u32(&q_full), 0) && mbar_wait_bounded(smem_u32(&k_full[0]), 0);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (ok) issue_s(0);
            for (int j = 0; j < n_kv && ok; ++j) {
                if (j + 1 < n_kv) {
                    // the scores of the next tile are computed while the softmax of this one runs
                    if (!mbar_wait_bounded(smem_u32(&s_empty), j & 1)) { ok = false; break; }
                    if (!mbar_wait_bounded(smem_u32(&k_full[(j + 1) & 1]), ((j + 1) >> 1) & 1)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    issue_s(j + 1);
                }
                if (!mbar_wait_bounded(smem_u32(&p_full), j & 1)) { ok = false; break; }
                if (!mbar_wait_bounded(smem_u32(&v_full[j & 1]), (j >> 1) & 1)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t vd = (j & 1) ? v_desc1 : v_desc0;
#pragma unroll
                for (int kk = 0; kk < KN / 16; ++kk)
                    umma(tmem_o, p_desc + (uint32_t)(kk * 2), vd + (uint32_t)(kk * 128), idesc_o, (j | kk) != 0);
                umma_commit(smem_u32(&pv_done));
                umma_commit(smem_u32(&v_empty[j & 1]));
            }
        }
    } else {
        // ---- softmax and output: thread = query row ----
        const int q = warp & 3;
        const int r = q * 32 + lane;
        const int pr = q0 + r;                                   // the row's position in its sequence
        const uint32_t lane_base = (uint32_t)(q * 32) << 16;
        const float LOG2E = 1.4426950408889634f;
        // score -> base-2 logit: with a soft-cap, tanh(s * scale / cap) * cap * log2(e); else s * scale * log2(e)
        const bool capped = a.softcap > 0.f;
        const float c_in = capped ? a.score_scale / a.softcap : a.score_scale * LOG2E;
        const float c_out = a.softcap * LOG2E;
        const int pr_warp_first = q0 + q * 32, pr_warp_last = pr_warp_first + 31;
        float m_ref = -INFINITY, l = 0.f;
        for (int j = 0; j < n_kv && ok; ++j) {
            if (!mbar_wait_bounded(smem_u32(&s_full), j & 1)) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float t[KN];
            {
                float half[32];
                tmem_ld32(tmem_s + lane_base, half);
#pragma unroll
                for (int i = 0; i < 32; ++i) t[i] = half[i];
                tmem_ld32(tmem_s + lane_base + 32, half);
#pragma unroll
                for (int i = 0; i < 32; ++i) t[32 + i] = half[i];
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&s_empty));      // the score buffer may be overwritten
            const int key0 = kv_first + j * KN;
            if (capped) {
#pragma unroll
                for (int i = 0; i < KN; ++i) t[i] = tanh_fast(t[i] * c_in) * c_out;
            } else {
#pragma unroll
                for (int i = 0; i < KN; ++i) t[i] *= c_in;
            }
            // tiles that every row of this warp sees whole need no masks (the test is the same for all lanes)
            const bool interior = key0 + KN - 1 <= pr_warp_first && (a.window == 0 || pr_warp_last - key0 < a.window);
            if (!interior) {
                const int hi = pr - key0, lo = a.window > 0 ? pr - a.window + 1 - key0 : -1;   // tile columns [lo, hi] are visible
#pragma unroll
                for (int i = 0; i < KN; ++i)
                    if (i > hi || i < lo) t[i] = -INFINITY;
            }
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < KN; i += 4) {
                mx4[0] = fmaxf(mx4[0], t[i]); mx4[1] = fmaxf(mx4[1], t[i + 1]);
                mx4[2] = fmaxf(mx4[2], t[i + 2]); mx4[3] = fmaxf(mx4[3], t[i + 3]);
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            // P V of the tile before must be finished before its probabilities are overwritten or O is touched
            if (j > 0 && !mbar_wait_bounded(smem_u32(&pv_done), (j - 1) & 1)) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const bool grow = mx > m_ref + RESCALE_STEP || (m_ref == -INFINITY && mx > -INFINITY);
            if (__any_sync(0xffffffffu, grow)) {
                const float m_new = grow ? mx : m_ref;
                const float factor = (grow && m_ref > -INFINITY) ? exp2_fast(m_ref - m_new) : 1.0f;
                if (j > 0) {
                    for (int c = 0; c < hd; c += 32) {
                        float o[32];
                        tmem_ld32(tmem_o + lane_base + c, o);
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] *= factor;
                        tmem_st32(tmem_o + lane_base + c, o);
                    }
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                }
                l *= factor;
                m_ref = m_new;
            }
            const float ms = m_ref == -INFINITY ? 0.f : m_ref;
            float rs4[4] = {0.f, 0.f, 0.f, 0.f};
            unsigned char* prow = sP + r * 128;
#pragma unroll
            for (int c = 0; c < KN / 8; ++c) {
                float e[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) { e[i] = exp2_fast(t[c * 8 + i] - ms); rs4[i & 3] += e[i]; }
                uint4 raw;
                __nv_bfloat162* hp = reinterpret_cast<__nv_bfloat162*>(&raw);
                hp[0] = __floats2bfloat162_rn(e[0], e[1]);
                hp[1] = __floats2bfloat162_rn(e[2], e[3]);
                hp[2] = __floats2bfloat162_rn(e[4], e[5]);
                hp[3] = __floats2bfloat162_rn(e[6], e[7]);
                *reinterpret_cast<uint4*>(prow + ((c ^ (r & 7)) * 16)) = raw;
            }
            l += (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");       // the tensor core reads these writes
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&p_full));
        }
        if (ok && !mbar_wait_bounded(smem_u32(&pv_done), (n_kv - 1) & 1)) ok = false;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // The rows go through shared memory (the query tile is no longer needed) so that the stores to
        // global memory are whole 16-byte chunks of consecutive addresses: thread -> row on the way in
        // (chunks swizzled by the row, no bank conflicts), thread -> chunk on the way out.
        if (ok) {
            const float inv = 1.0f / l;
            unsigned char* srow = sQ + (size_t)r * (hd * 2);
#pragma unroll
            for (int c = 0; c < hd; c += 32) {
                float o[32];
                tmem_ld32(tmem_o + lane_base + c, o);
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    uint4 raw;
                    __nv_bfloat162* hp = reinterpret_cast<__nv_bfloat162*>(&raw);
                    hp[0] = __floats2bfloat162_rn(o[i] * inv, o[i + 1] * inv);
                    hp[1] = __floats2bfloat162_rn(o[i + 2] * inv, o[i + 3] * inv);
                    hp[2] = __floats2bfloat162_rn(o[i + 4] * inv, o[i + 5] * inv);
                    hp[3] = __floats2bfloat162_rn(o[i + 6] * inv, o[i + 7] * inv);
                    *reinterpret_cast<uint4*>(srow + ((((c + i) >> 3) ^ (r & 7)) * 16)) = raw;
                }
            }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");           // the four softmax warps, whatever became of their waits
        {
            constexpr int CHUNKS = hd / 8;                       // 16-byte chunks of a row
            __nv_bfloat16* obase = (__nv_bfloat16*)a.out + (long long)(row0 + q0) * a.out_stride + (long long)h * hd;
            const int tt = threadIdx.x - 64;
#pragma unroll 4
            for (int idx = tt; idx < QM * CHUNKS; idx += 128) {
                const int row = idx / CHUNKS, c = idx - row * CHUNKS;
                if (row < rows)
                    *reinterpret_cast<uint4*>(obase + (long long)row * a.out_stride + c * 8) =
                        *reinterpret_cast<const uint4*>(sQ + (size_t)row * (hd * 2) + ((c ^ (row & 7)) * 16));
            }
        }
    }
    if (!ok && a.status) atomicExch(a.status, RDL_FAULT_ATTENTION_TC);
    // ---- tear-down, reached by every thread ----
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_slot), "r"(tmem_cols) : "memory");
}

int make_map(CUtensorMap* map, const void* ptr, long long rows, long long cols, int box_rows) {
    typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeTiled encode = nullptr;
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult found;
        RDL_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &found), "attention_tc: looking up cuTensorMapEncodeTiled");
        RDL_REQUIRE(found == cudaDriverEntryPointSuccess && fn, "attention_tc: this driver has no cuTensorMapEncodeTiled");
        encode = (EncodeTiled)fn;
    }
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    RDL_REQUIRE(r == CUDA_SUCCESS, "attention_tc: cuTensorMapEncodeTiled failed with driver error %d", (int)r);
    return 0;
}

template <int DB>
int launch_tc(dim3 grid, int smem, cudaStream_t st, const CUtensorMap& map_q, const CUtensorMap& map_kv, const TcAttnArgs& t) {
    static bool opted = false;
    if (!opted) {
        RDL_CUDA(cudaFuncSetAttribute(attention_tc_kernel<DB>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "attention_prefill_tc");
        opted = true;
    }
    RDL_CHECK_EX(rdl_launch(attention_tc_kernel<DB>, grid, dim3(ATC_THREADS), (size_t)smem, st, map_q, map_kv, t), "attention_prefill_tc");
    return 0;
}

}  // namespace

// Prefill attention of sequences that start at position 0, from packed rows [tokens, row_width] that hold
// the rotated query heads, then the key heads, then the value heads.
extern "C" int rdl_attention_prefill_tc(const AttentionArgs* a, long long row_width, void* stream) {
    if (int e = rdl_check_attention_args(a, "attention_prefill_tc")) return e;
    RDL_REQUIRE(a->dtype == RDL_BF16, "attention_prefill_tc: bfloat16 only");
    RDL_REQUIRE(a->head_dim % 64 == 0 && a->head_dim <= 256, "attention_prefill_tc: head_dim %d must be 64, 128, 192 or 256", a->head_dim);
    RDL_REQUIRE(a->tile_seq && a->tile_q0 && a->n_tiles >= 0, "attention_prefill_tc: missing query tiles");
    RDL_REQUIRE(a->k_new && a->v_new && a->q_stride == row_width && a->kv_stride == row_width &&
                    (const char*)a->k_new == (const char*)a->q + 2LL * a->n_heads * a->head_dim &&
                    (const char*)a->v_new == (const char*)a->q + 2LL * (a->n_heads + a->n_kv_heads) * a->head_dim,
                "attention_prefill_tc: queries, keys and values must be the packed rows of one buffer");
    RDL_REQUIRE(row_width >= (long long)(a->n_heads + 2 * a->n_kv_heads) * a->head_dim && row_width % 8 == 0 && (uintptr_t)a->q % 16 == 0,
                "attention_prefill_tc: bad row width or alignment");
    RDL_REQUIRE(a->out_stride % 8 == 0 && (uintptr_t)a->out % 16 == 0, "attention_prefill_tc: output rows must start on 16-byte boundaries");
    RDL_REQUIRE(a->n_tiles <= 65535, "attention_prefill_tc: %d query tiles exceed the grid limit", a->n_tiles);
    if (a->n_tiles == 0 || a->n_tokens == 0) return 0;
    CUtensorMap map_q, map_kv;
    if (int e = make_map(&map_q, a->q, a->n_tokens, row_width, QM)) return e;
    if (int e = make_map(&map_kv, a->q, a->n_tokens, row_width, KN)) return e;
    TcAttnArgs t{a->out, a->out_stride, a->tile_seq, a->tile_q0, a->n_tiles, a->seq_start, a->n_heads, a->n_kv_heads, a->head_dim,
                 a->score_scale, a->softcap, a->window, a->status};
    const int smem = QM * a->head_dim * 2 + 4 * KN * a->head_dim * 2 + QM * 128 + 1024;
    dim3 grid(a->n_heads, a->n_tiles);
    switch (a->head_dim / 64) {
        case 1: return launch_tc<1>(grid, smem, (cudaStream_t)stream, map_q, map_kv, t);
        case 2: return launch_tc<2>(grid, smem, (cudaStream_t)stream, map_q, map_kv, t);
        case 3: return launch_tc<3>(grid, smem, (cudaStream_t)stream, map_q, map_kv, t);
        default: return launch_tc<4>(grid, smem, (cudaStream_t)stream, map_q, map_kv, t);
    }
}
