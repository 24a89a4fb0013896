// Prefill attention in bfloat16: tiled, with an online softmax in float, soft-cap, causal and
// window masks, grouped heads, sequences of unequal length packed in one batch.  Keys and
// values of earlier steps are read from the paged cache, those of this step from the packed
// rows, chosen per key row.  Formulas as in attention_plain.cu.
//
// One block = 64 query rows of one sequence and one head (4 warps, 16 rows each); key tiles of
// 64 positions aligned to absolute multiples of 64; tiles wholly outside the window are skipped.
// Products run on the tensor cores (mma.sync m16n8k16, float accumulators); scores, tanh,
// exponentials, row maxima and row sums are float.
#include "api.h"
#include "common.cuh"
#include "launch.cuh"

namespace {

constexpr int BM = 64, BN = 64, NTHREADS = 128;

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float tanh_fast(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// shared tile [64 rows][HD] of bf16 in 16-byte chunks, chunk index swizzled by the row
template <int HD>
__device__ __forceinline__ int swizzled_chunk(int row, int chunk) {
    constexpr int CH = HD / 8;
    if (CH >= 8) return chunk ^ (row & 7);
    return chunk ^ ((row >> 1) & (CH - 1));
}
template <int HD>
__device__ __forceinline__ uint32_t tile_addr(uint32_t base, int row, int chunk) {
    return base + (uint32_t)((row * (HD / 8) + swizzled_chunk<HD>(row, chunk)) * 16);
}

template <int HD>
__global__ void __launch_bounds__(NTHREADS) attention_prefill_kernel(AttentionArgs a) {
    constexpr int CH = HD / 8;          // 16-byte chunks per row
    extern __shared__ __align__(128) unsigned char smem[];
    const uint32_t sQ = (uint32_t)__cvta_generic_to_shared(smem);
    const uint32_t sK = sQ + BM * HD * 2;
    const uint32_t sV = sK + BN * HD * 2;
    unsigned char* gQ = smem;

    const int tile = a.n_tiles - 1 - blockIdx.x, h = blockIdx.y;   // later tiles of a sequence have more keys: start them first
    const int seq = a.tile_seq[tile], q0 = a.tile_q0[tile];
    const int row0 = a.seq_start[seq];
    const int n_new = a.seq_start[seq + 1] - row0;
    const int rows = min(BM, n_new - q0);
    const int past = a.seq_past[seq];
    const int cached = a.seq_cached[seq];
    const int hd = a.head_dim;
    const int g = h / (a.n_heads / a.n_kv_heads);
    const int* table = a.tables ? a.tables + (long long)seq * a.table_width : nullptr;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int quad = lane >> 2, tq = lane & 3;
    const __nv_bfloat16* qbase = (const __nv_bfloat16*)a.q;
    const __nv_bfloat16* knew = (const __nv_bfloat16*)a.k_new;
    const __nv_bfloat16* vnew = (const __nv_bfloat16*)a.v_new;
    const __nv_bfloat16* kcache = (const __nv_bfloat16*)a.k_cache;
    const __nv_bfloat16* vcache = (const __nv_bfloat16*)a.v_cache;
    const uint4 zero4 = make_uint4(0, 0, 0, 0);

    rdl_grid_wait();               // the batch description above is constant; the rows come from the kernel before
    rdl_grid_launch_dependents();
    // ---- query tile ----
    for (int idx = tid; idx < BM * CH; idx += NTHREADS) {
        const int r = idx / CH, c = idx - r * CH;
        uint4 v = zero4;
        if (r < rows && c * 8 < hd)
            v = *(const uint4*)(qbase + (long long)(row0 + q0 + r) * a.q_stride + (long long)h * hd + c * 8);
        *(uint4*)(gQ + (r * CH + swizzled_chunk<HD>(r, c)) * 16) = v;
    }

    const int p_first = past + q0, p_last = past + q0 + rows - 1;
    const int lo_first = a.window > 0 ? max(0, p_first - a.window + 1) : 0;
    // positions of the two rows this thread holds
    const int pr0 = p_first + warp * 16 + quad, pr1 = pr0 + 8;
    const int pw_first = p_first + warp * 16, pw_last = pw_first + 15;

    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    const float LOG2E = 1.4426950408889634f;
    const float inv_cap = a.softcap > 0.f ? 1.0f / a.softcap : 0.f;
    const int ksteps = (hd + 15) / 16;

    // One tile of keys (which == 0) or values (which == 1) on its way to shared memory: asynchronous
    // 16-byte copies that bypass the registers, rows beyond the sequence and chunks beyond head_dim
    // filled with zeros.  Each call is one commit group.
    auto issue = [&](int kv0, int which) {
        const uint32_t sdst = which ? sV : sK;
        const __nv_bfloat16* cache_base = which ? vcache : kcache;
        const __nv_bfloat16* new_base = which ? vnew : knew;
        for (int idx = tid; idx < BN * CH; idx += NTHREADS) {
            const int r = idx / CH, c = idx - r * CH;
            const int j = kv0 + r;
            const __nv_bfloat16* src = qbase;       // any valid address: nothing is read when the size is 0
            uint32_t bytes = 0;
            if (j <= p_last && c * 8 < hd) {
                bytes = 16;
                if (j < cached)   // chunks of a cache row are stored swizzled by the row's place in its page
                    src = cache_base + rdl_cache_offset(table, j, a.page_size, a.ring_pages, a.n_kv_heads, g, hd) +
                          rdl_swizzled_chunk(j % a.page_size, c, hd / 8) * 8;
                else
                    src = new_base + (long long)(row0 + j - past) * a.kv_stride + (long long)g * hd + c * 8;
            }
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(tile_addr<HD>(sdst, r, c)), "l"(src), "r"(bytes) : "memory");
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };

    const int kv_first = (lo_first / BN) * BN;
    if (kv_first <= p_last) {
        issue(kv_first, 0);
        issue(kv_first, 1);
    }
    for (int kv0 = kv_first; kv0 <= p_last; kv0 += BN) {
        const bool has_next = kv0 + BN <= p_last;
        asm volatile("cp.async.wait_group 1;\n" ::: "memory");   // this tile's keys have landed (its values may be on the way)
        __syncthreads();

        // this warp's rows see nothing of the tile: skip its arithmetic (barriers stay outside)
        const bool warp_active = kv0 <= pw_last && (a.window == 0 || pw_first - (kv0 + BN - 1) < a.window);
        uint32_t pf[BN / 16][4];
        if (warp_active) {
            // ---- S = Q K^T ----
            float s[BN / 8][4];
#pragma unroll
            for (int i = 0; i < BN / 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
            for (int kk = 0; kk < ksteps; ++kk) {
                uint32_t af[4];
                ldmatrix_x4(af, tile_addr<HD>(sQ, warp * 16 + (lane & 15), 2 * kk + (lane >> 4)));
#pragma unroll
                for (int np = 0; np < BN / 16; ++np) {
                    uint32_t bf[4];
                    ldmatrix_x4(bf, tile_addr<HD>(sK, np * 16 + (lane & 7) + 8 * (lane >> 4), 2 * kk + ((lane >> 3) & 1)));
                    mma_bf16(s[2 * np], af, bf[0], bf[1]);
                    mma_bf16(s[2 * np + 1], af, bf[2], bf[3]);
                }
            }
            // ---- scale, soft-cap, mask ----
            const bool need_mask = !(kv0 + BN - 1 <= pw_first && (a.window == 0 || pw_last - kv0 < a.window));
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < BN / 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float v = s[nt][e] * a.score_scale;
                    if (a.softcap > 0.f) v = a.softcap * tanh_fast(v * inv_cap);
                    v *= LOG2E;
                    if (need_mask) {
                        const int key = kv0 + nt * 8 + 2 * tq + (e & 1);
                        const int pr = (e < 2) ? pr0 : pr1;
                        const bool keep = key <= pr && (a.window == 0 || pr - key < a.window);
                        if (!keep) v = -INFINITY;
                    }
                    s[nt][e] = v;
                }
                mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1]));
                mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3]));
            }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
            const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;
            const float c0 = exp2f(m0 - ms0), c1 = exp2f(m1 - ms1);
            m0 = mn0; m1 = mn1;
            float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
            for (int nt = 0; nt < BN / 8; ++nt) {
                const float e0 = exp2f(s[nt][0] - ms0), e1 = exp2f(s[nt][1] - ms0);
                const float e2 = exp2f(s[nt][2] - ms1), e3 = exp2f(s[nt][3] - ms1);
                rs0 += e0 + e1;
                rs1 += e2 + e3;
                pf[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16(e0, e1);
                pf[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(e2, e3);
            }
            rs0 += __shfl_xor_sync(0xffffffffu, rs0, 1);
            rs0 += __shfl_xor_sync(0xffffffffu, rs0, 2);
            rs1 += __shfl_xor_sync(0xffffffffu, rs1, 1);
            rs1 += __shfl_xor_sync(0xffffffffu, rs1, 2);
            l0 = l0 * c0 + rs0;
            l1 = l1 * c1 + rs1;
#pragma unroll
            for (int i = 0; i < HD / 8; ++i) {
                o[i][0] *= c0; o[i][1] *= c0; o[i][2] *= c1; o[i][3] *= c1;
            }
        }
        __syncthreads();                       // every warp is done with the key tile
        if (has_next) issue(kv0 + BN, 0);      // the next keys travel while P V is computed
        if (has_next) asm volatile("cp.async.wait_group 1;\n" ::: "memory");
        else asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        __syncthreads();                       // this tile's values have landed
        if (warp_active) {
            // ---- O += P V ----
#pragma unroll
            for (int kk = 0; kk < BN / 16; ++kk) {
#pragma unroll
                for (int dp = 0; dp < HD / 16; ++dp) {
                    if (dp * 16 < hd) {
                        uint32_t bf[4];
                        ldmatrix_x4_trans(bf, tile_addr<HD>(sV, kk * 16 + (lane & 15), 2 * dp + (lane >> 4)));
                        mma_bf16(o[2 * dp], pf[kk], bf[0], bf[1]);
                        mma_bf16(o[2 * dp + 1], pf[kk], bf[2], bf[3]);
                    }
                }
            }
        }
        __syncthreads();                       // every warp is done with the value tile
        if (has_next) issue(kv0 + BN, 1);      // the next values travel while the next scores are computed
    }

    // ---- normalise and store ----
    const int r0 = warp * 16 + quad, r1 = r0 + 8;
    const float i0 = 1.0f / l0, i1 = 1.0f / l1;
    __nv_bfloat16* out = (__nv_bfloat16*)a.out;
#pragma unroll
    for (int nt = 0; nt < HD / 8; ++nt) {
        const int d = nt * 8 + 2 * tq;
        if (d < hd) {
            if (r0 < rows)
                *(__nv_bfloat162*)(out + (long long)(row0 + q0 + r0) * a.out_stride + (long long)h * hd + d) =
                    __floats2bfloat162_rn(o[nt][0] * i0, o[nt][1] * i0);
            if (r1 < rows)
                *(__nv_bfloat162*)(out + (long long)(row0 + q0 + r1) * a.out_stride + (long long)h * hd + d) =
                    __floats2bfloat162_rn(o[nt][2] * i1, o[nt][3] * i1);
        }
    }
}

template <int HD>
int launch_prefill(const AttentionArgs* a, cudaStream_t st) {
    const int smem = (BM + 2 * BN) * HD * 2;
    static bool opted = false;
    if (smem > 48 * 1024 && !opted) {
        RDL_CUDA(cudaFuncSetAttribute(attention_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem),
                 "attention_prefill");
        opted = true;
    }
    dim3 grid(a->n_tiles, a->n_heads);
    RDL_CHECK_EX(rdl_launch(attention_prefill_kernel<HD>, grid, dim3(NTHREADS), (size_t)smem, st, *a), "attention_prefill");
    return 0;
}

}  // namespace

extern "C" int rdl_attention_prefill(const AttentionArgs* a, void* stream) {
    if (int e = rdl_check_attention_args(a, "attention_prefill")) return e;
    RDL_REQUIRE(a->dtype == RDL_BF16, "attention_prefill: bfloat16 only (the 32-bit path uses attention_plain)");
    RDL_REQUIRE(a->head_dim % 16 == 0 && a->head_dim <= 256,
                "attention_prefill: head_dim %d must be a multiple of 16 and at most 256", a->head_dim);
    RDL_REQUIRE(a->tile_seq && a->tile_q0 && a->n_tiles >= 0, "attention_prefill: missing query tiles");
    RDL_REQUIRE(a->n_heads <= 65535, "attention_prefill: too many heads for the grid");
    RDL_REQUIRE(a->q_stride % 8 == 0 && a->kv_stride % 8 == 0 && a->out_stride % 2 == 0 &&
                    ((uintptr_t)a->q % 16 == 0) && ((uintptr_t)a->k_new % 16 == 0) && ((uintptr_t)a->v_new % 16 == 0) &&
                    ((uintptr_t)a->k_cache % 16 == 0) && ((uintptr_t)a->v_cache % 16 == 0) && ((uintptr_t)a->out % 4 == 0),
                "attention_prefill: rows must start on 16-byte boundaries");
    if (a->n_tiles == 0 || a->n_tokens == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    if (a->head_dim <= 32) return launch_prefill<32>(a, st);
    if (a->head_dim <= 64) return launch_prefill<64>(a, st);
    if (a->head_dim <= 128) return launch_prefill<128>(a, st);
    return launch_prefill<256>(a, st);
}
