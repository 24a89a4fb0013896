// Decode attention in bfloat16 over the paged cache: few query tokens, many keys.
//
// The keys a token reads (all earlier positions, or the last `window`) are cut into runs of
// `keys_per_split` positions (a whole number of pages).  One block handles one run for all query
// heads that share a kv head.  Each page of the run - [page_size][head_dim] keys and as many
// values, each contiguous in the cache - is brought into shared memory by two bulk asynchronous
// copies (TMA, cp.async.bulk + mbarrier).  The cache stores the 16-byte chunks of a row swizzled
// by the row's place in its page (common.cuh), so the copied block is read by ldmatrix without
// bank conflicts as it is.  The heads of the group are the rows of a 16-row query tile:
// scores and P.V run on the tensor cores (mma.sync m16n8k16, float accumulators), each warp
// taking 16 keys of the page; soft-cap, softmax state and output sums are float.
//
// A token with a single run writes its output directly.  Otherwise every block writes its
// unnormalised partial result to scratch and the block that finishes last for a (token, kv head)
// merges the runs in run order and writes the output: one launch, no second kernel.  Formulas as
// in attention_plain.cu; all keys are read from the cache (the step writes its new rows first).
//
// Scratch: int counters [tokens * kv_heads] (zero before the launch; the merging block puts its
// counter back to zero), then float partials [token][head][run][head_dim + 2] = sums, maximum
// (base-2 scale), normaliser.  Launches that share the scratch must not overlap on the device.
//
// Every wait on a copy is bounded: after about a second without completion the block records
// an error in `status` and leaves.
#include "api.h"
#include "common.cuh"
#include "launch.cuh"

namespace {

constexpr int DEC_THREADS = 128;
constexpr int DEC_WARPS = DEC_THREADS / 32;
constexpr int QROWS = 16;                         // rows of the query tile = most heads per kv head
constexpr long long WAIT_CYCLES = 2000000000LL;

__device__ __forceinline__ float tanh_fast(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
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

// HD: head_dim padded to 64, 128 or 256 (head_dim itself is a multiple of 16).
template <int HD>
__global__ void __launch_bounds__(DEC_THREADS) attention_decode_kernel(AttentionArgs a) {
    constexpr int QROWB = HD * 2 + 16;            // bytes between rows of the query tile (padded: no bank conflicts)
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ __align__(8) unsigned long long bar_storage;
    __shared__ float sm_m[DEC_WARPS][QROWS], sm_l[DEC_WARPS][QROWS];
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
    const int quad = lane >> 2, tq = lane & 3;
    const __nv_bfloat16* kcache = (const __nv_bfloat16*)a.k_cache;
    const __nv_bfloat16* vcache = (const __nv_bfloat16*)a.v_cache;
    unsigned char* q_tile = smem;
    unsigned char* k_tile = smem + QROWS * QROWB;                 // [page_size][head_dim] as stored: chunks swizzled by row
    unsigned char* v_tile = k_tile + (size_t)ps * hd * 2;
    const int chunks = hd / 8;
    const uint32_t q_s = (uint32_t)__cvta_generic_to_shared(q_tile);
    const uint32_t k_s = (uint32_t)__cvta_generic_to_shared(k_tile);
    const uint32_t v_s = (uint32_t)__cvta_generic_to_shared(v_tile);
    const uint32_t bar = (uint32_t)__cvta_generic_to_shared(&bar_storage);
    const uint32_t row_bytes = (uint32_t)hd * 2;

    const int page_first = k_begin / ps, page_last = (k_end - 1) / ps;
    // Ask L2 for the run's pages now.  Nothing read up to here was written by an earlier kernel of this
    // step (the batch description and page lists come from the host; the newest row of the last page is
    // written by the kernel before this one, but a prefetch only moves lines into L2, where that write
    // lands too), so this runs while the earlier kernel is still finishing.
    if (tid <= page_last - page_first) {
        const int page = table[(page_first + tid) % a.ring_pages];
        const long long off = ((long long)page * a.n_kv_heads + g) * ps * hd;
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(kcache + off), "r"(ps * row_bytes) : "memory");
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(vcache + off), "r"(ps * row_bytes) : "memory");
    }
    if (tid == 0) mbar_init(bar, 1);
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    // query tile: row h = head g * G + h of this token, rows from G on are zero
    for (int idx = tid; idx < QROWS * (HD / 8); idx += DEC_THREADS) {
        const int r = idx / (HD / 8), c = idx - r * (HD / 8);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < G && c * 8 < hd)
            v = *(const uint4*)((const __nv_bfloat16*)a.q + (long long)t * a.q_stride + (long long)(g * G + r) * hd + c * 8);
        *(uint4*)(q_tile + r * QROWB + c * 16) = v;
    }
    __syncthreads();

    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    const float LOG2E = 1.4426950408889634f;
    const float inv_cap = a.softcap > 0.f ? 1.0f / a.softcap : 0.f;
    const int ksteps = hd / 16;

    uint32_t phase = 0;
    for (int lp = page_first; lp <= page_last; ++lp) {
        if (tid == 0) {
            // the page's keys and its values are each one contiguous block: two copies
            const int page = table[lp % a.ring_pages];
            const long long off = ((long long)page * a.n_kv_heads + g) * ps * hd;
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_expect_tx(bar, 2u * ps * row_bytes);
            bulk_load(k_s, kcache + off, ps * row_bytes, bar);
            bulk_load(v_s, vcache + off, ps * row_bytes, bar);
        }
        if (!mbar_wait_bounded(bar, phase)) {
            if (a.status) atomicExch(a.status, 3);
            return;
        }
        phase ^= 1;
        const int r_begin = max(k_begin, lp * ps) - lp * ps, r_end = min(k_end, (lp + 1) * ps) - lp * ps;
        const int w0 = warp * 16;                  // this warp's 16 keys of the page
        if (w0 < r_end && w0 + 16 > r_begin) {
            if (w0 < r_begin || w0 + 16 > r_end) {
                // value rows outside the run get the weight 0; they may hold anything (rows beyond the
                // sequence's end, an earlier occupant's rows), so make them zero: 0 * NaN is NaN
                for (int idx = lane; idx < 16 * chunks; idx += 32) {
                    const int r = w0 + idx / chunks;
                    if (r < r_begin || r >= r_end) *(uint4*)(v_tile + (size_t)r * row_bytes + (idx % chunks) * 16) = make_uint4(0, 0, 0, 0);
                }
                __syncwarp();
            }
            float s[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
            for (int kk = 0; kk < ksteps; ++kk) {
                uint32_t af[4], bf[4];
                ldmatrix_x4(af, q_s + (lane & 15) * QROWB + (2 * kk + (lane >> 4)) * 16);
                const int kr = w0 + (lane & 7) + 8 * (lane >> 4);
                ldmatrix_x4(bf, k_s + kr * row_bytes + rdl_swizzled_chunk(kr, 2 * kk + ((lane >> 3) & 1), chunks) * 16);
                mma_bf16(s[0], af, bf[0], bf[1]);
                mma_bf16(s[1], af, bf[2], bf[3]);
            }
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float v = s[nt][e] * a.score_scale;
                    if (a.softcap > 0.f) v = a.softcap * tanh_fast(v * inv_cap);
                    v *= LOG2E;
                    const int r = w0 + nt * 8 + 2 * tq + (e & 1);
                    if (r < r_begin || r >= r_end) v = -INFINITY;
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
            const float e00 = exp2f(s[0][0] - ms0), e01 = exp2f(s[0][1] - ms0), e02 = exp2f(s[0][2] - ms1), e03 = exp2f(s[0][3] - ms1);
            const float e10 = exp2f(s[1][0] - ms0), e11 = exp2f(s[1][1] - ms0), e12 = exp2f(s[1][2] - ms1), e13 = exp2f(s[1][3] - ms1);
            float rs0 = e00 + e01 + e10 + e11, rs1 = e02 + e03 + e12 + e13;
            rs0 += __shfl_xor_sync(0xffffffffu, rs0, 1);
            rs0 += __shfl_xor_sync(0xffffffffu, rs0, 2);
            rs1 += __shfl_xor_sync(0xffffffffu, rs1, 1);
            rs1 += __shfl_xor_sync(0xffffffffu, rs1, 2);
            l0 = l0 * c0 + rs0;
            l1 = l1 * c1 + rs1;
            uint32_t pf[4] = {pack_bf16(e00, e01), pack_bf16(e02, e03), pack_bf16(e10, e11), pack_bf16(e12, e13)};
#pragma unroll
            for (int dp = 0; dp < HD / 16; ++dp) {
                if (dp * 16 < hd) {
                    uint32_t bf[4];
                    const int vr = w0 + (lane & 15);
                    ldmatrix_x4_trans(bf, v_s + vr * row_bytes + rdl_swizzled_chunk(vr, 2 * dp + (lane >> 4), chunks) * 16);
                    o[2 * dp][0] *= c0; o[2 * dp][1] *= c0; o[2 * dp][2] *= c1; o[2 * dp][3] *= c1;
                    o[2 * dp + 1][0] *= c0; o[2 * dp + 1][1] *= c0; o[2 * dp + 1][2] *= c1; o[2 * dp + 1][3] *= c1;
                    mma_bf16(o[2 * dp], pf, bf[0], bf[1]);
                    mma_bf16(o[2 * dp + 1], pf, bf[2], bf[3]);
                }
            }
        }
        __syncthreads();   // everyone is done with the tiles before the next copy lands
    }

    // ---- merge the four warps through shared memory, in warp order ----
    float* sm_o = reinterpret_cast<float*>(k_tile);  // [warp][row][HD]; the tiles are no longer needed
    if (tq == 0) {
        sm_m[warp][quad] = m0; sm_m[warp][quad + 8] = m1;
        sm_l[warp][quad] = l0; sm_l[warp][quad + 8] = l1;
    }
#pragma unroll
    for (int nt = 0; nt < HD / 8; ++nt) {
        const int d = nt * 8 + 2 * tq;
        if (d < hd) {
            if (quad < G) *(float2*)(sm_o + ((warp * QROWS + quad) * HD + d)) = make_float2(o[nt][0], o[nt][1]);
            if (quad + 8 < G) *(float2*)(sm_o + ((warp * QROWS + quad + 8) * HD + d)) = make_float2(o[nt][2], o[nt][3]);
        }
    }
    __syncthreads();
    __nv_bfloat16* out = (__nv_bfloat16*)a.out + (long long)t * a.out_stride;
    int* counters = (int*)a.scratch;
    float* partials = (float*)((char*)a.scratch + a.counter_bytes);
    for (int idx = tid; idx < G * hd; idx += DEC_THREADS) {
        const int h = idx / hd, d = idx - h * hd;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, sm_m[w][h]);
        float osum = 0.f, lsum = 0.f;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) {
            const float wt = sm_m[w][h] == -INFINITY ? 0.f : exp2f(sm_m[w][h] - M);
            osum = fmaf(wt, sm_o[(w * QROWS + h) * HD + d], osum);
            lsum = fmaf(wt, sm_l[w][h], lsum);
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
    float* w_s = sm_o;                            // [G][n_splits] weights of the runs
    float* stat = sm_o + G * n_splits;            // [G] 1 / normaliser
    for (int h = warp; h < G; h += DEC_WARPS) {
        const float* base = partials + ((long long)t * a.n_heads + (g * G + h)) * a.max_splits * (hd + 2);
        float M = -INFINITY;
        for (int s = lane; s < n_splits; s += 32) M = fmaxf(M, base[(long long)s * (hd + 2) + hd]);
        M = warp_max(M);
        float L = 0.f;
        for (int s = lane; s < n_splits; s += 32) {
            const float wt = exp2f(base[(long long)s * (hd + 2) + hd] - M);
            w_s[h * n_splits + s] = wt;
            L = fmaf(wt, base[(long long)s * (hd + 2) + hd + 1], L);
        }
        L = warp_sum(L);
        if (lane == 0) stat[h] = 1.0f / L;
    }
    __syncthreads();
    // two outputs per thread and eight runs in flight: the partials are read from L2 in few trips
    for (int idx = tid; idx < G * hd / 2; idx += DEC_THREADS) {
        const int h = (idx * 2) / hd, d = idx * 2 - h * hd;
        const float* base = partials + ((long long)t * a.n_heads + (g * G + h)) * a.max_splits * (hd + 2) + d;
        float ox = 0.f, oy = 0.f;
#pragma unroll 8
        for (int s = 0; s < n_splits; ++s) {
            const float2 v = *(const float2*)(base + (long long)s * (hd + 2));
            const float wt = w_s[h * n_splits + s];
            ox = fmaf(wt, v.x, ox);
            oy = fmaf(wt, v.y, oy);
        }
        *(__nv_bfloat162*)(out + (long long)(g * G + h) * hd + d) = __floats2bfloat162_rn(ox * stat[h], oy * stat[h]);
    }
}

template <int HD>
int launch_decode(const AttentionArgs* a, cudaStream_t st) {
    const int qtile = QROWS * (HD * 2 + 16);
    const int tiles = 2 * a->page_size * a->head_dim * 2;
    const int merge = DEC_WARPS * QROWS * HD * (int)sizeof(float);
    const int runs = (QROWS * a->max_splits + QROWS) * (int)sizeof(float);
    int smem = tiles > merge ? tiles : merge;
    if (runs > smem) smem = runs;
    smem += qtile;
    RDL_REQUIRE(smem <= 200 * 1024, "attention_decode: page_size %d x head_dim %d needs %d bytes of shared memory, limit is 204800",
                a->page_size, a->head_dim, smem);
    static int granted = 48 * 1024;
    if (smem > granted) {
        RDL_CUDA(cudaFuncSetAttribute(attention_decode_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem),
                 "attention_decode");
        granted = smem;
    }
    dim3 grid(a->max_splits, a->n_kv_heads, a->n_tokens);
    RDL_CHECK_EX(rdl_launch(attention_decode_kernel<HD>, grid, dim3(DEC_THREADS), (size_t)smem, st, *a), "attention_decode");
    return 0;
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
    RDL_REQUIRE(a->head_dim % 16 == 0 && a->head_dim <= 256, "attention_decode: head_dim %d must be a multiple of 16 and at most 256", a->head_dim);
    const int G = a->n_heads / a->n_kv_heads;
    RDL_REQUIRE(G <= QROWS, "attention_decode: %d query heads per key/value head, at most %d are supported", G, QROWS);
    RDL_REQUIRE(a->tables && a->k_cache && a->v_cache, "attention_decode: needs a cache");
    RDL_REQUIRE(a->page_size % 16 == 0 && a->page_size <= 16 * DEC_WARPS,
                "attention_decode: page_size %d must be a multiple of 16 and at most %d", a->page_size, 16 * DEC_WARPS);
    RDL_REQUIRE(a->keys_per_split > 0 && a->keys_per_split % a->page_size == 0,
                "attention_decode: keys_per_split %d must be a whole number of pages of %d", a->keys_per_split, a->page_size);
    RDL_REQUIRE(a->max_splits > 0 && a->max_splits <= 65535, "attention_decode: bad number of runs %d", a->max_splits);
    RDL_REQUIRE(a->n_kv_heads <= 65535 && a->n_tokens <= 65535, "attention_decode: grid too large");
    RDL_REQUIRE(a->counter_bytes == rdl_attention_decode_counter_bytes(a->n_tokens, a->n_kv_heads),
                "attention_decode: counter_bytes must come from rdl_attention_decode_counter_bytes");
    RDL_REQUIRE(a->scratch && a->scratch_bytes >= rdl_attention_decode_scratch_bytes(a->n_tokens, a->n_heads, a->n_kv_heads, a->head_dim, a->max_splits),
                "attention_decode: scratch of %lld bytes is too small", a->scratch_bytes);
    RDL_REQUIRE(a->q_stride % 8 == 0 && (uintptr_t)a->q % 16 == 0 && (uintptr_t)a->k_cache % 16 == 0 &&
                    (uintptr_t)a->v_cache % 16 == 0 && (uintptr_t)a->scratch % 16 == 0 && a->out_stride % 2 == 0,
                "attention_decode: rows must start on 16-byte boundaries");
    if (a->n_tokens == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    if (a->head_dim <= 64) return launch_decode<64>(a, st);
    if (a->head_dim <= 128) return launch_decode<128>(a, st);
    return launch_decode<256>(a, st);
}
