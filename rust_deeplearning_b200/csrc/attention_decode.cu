// Decode attention in bfloat16 over the paged cache: few query tokens, many keys.
//
// The keys a token reads (all earlier positions, or the last `window`) are cut into runs of
// `keys_per_split` positions (a whole number of pages).  One block handles one run for all query
// heads that share a kv head.  Each page of the run - [page_size][head_dim] keys and as many
// values, each contiguous in the cache - is brought into shared memory by two bulk asynchronous
// copies (TMA, cp.async.bulk + mbarrier) into a ring of three tiles, so that a copy is requested a
// page and a half before it is read.  The cache stores the 16-byte chunks of a row swizzled
// by the row's place in its page (common.cuh), so the copied block is read by ldmatrix without
// bank conflicts as it is.  The products run on the tensor cores (mma.sync m16n8k16, float
// accumulators) with the keys as rows and the (up to 8) heads of the group as columns:
// S^T = K Q^T and O^T += V^T P^T, each warp taking 16 keys of the page; soft-cap, softmax state
// and output sums are float.
//
// A token with a single run writes its output directly.  Otherwise every block writes its
// unnormalised partial result to scratch and the block that finishes last for a (token, kv head)
// merges the runs in run order and writes the output: one launch, no second kernel.  Formulas as
// in attention_plain.cu; all keys are read from the cache (the step writes its new rows first).
//
// Scratch: int counters [tokens * kv_heads] (zero before the launch; the merging block puts its
// counter back to zero), then float partial sums [token][head][run][head_dim], then per run the
// maximum (base-2 scale) and the normaliser [token][head][run][2].  Launches that share the scratch
// must not overlap on the device.
//
// Optionally (new_rows) the kernel also does what otherwise a kernel of its own does before it: it
// rotates the step's query heads and the new key row by the position's angles (rope_cache.cu has the
// formula), writes the new key and value rows to the cache, and puts them into the copied page in
// shared memory; one launch less per layer of a decode step.
//
// Every wait on a copy is bounded: after about a second without completion the block records
// RDL_FAULT_ATTENTION_DECODE in `status`, stops waiting and issuing, and runs on to its end, so
// that the run counters are left as the next launch needs them; its output is void.
#include "api.h"
#include "common.cuh"
#include "launch.cuh"

namespace {

constexpr int DEC_THREADS = 128;
constexpr int DEC_WARPS = DEC_THREADS / 32;
constexpr int QROWS = 8;                          // most query heads per kv head: the columns of one score product

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
// policy: an L2 cache policy (createpolicy); 0: none
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar, unsigned long long policy = 0) {
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
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// false if the copy did not complete within the limit, or if the block has given up already
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, long long limit, volatile int* gave_up) {
    if (*gave_up) return false;
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (*gave_up) return false;
        if (clock64() - t0 > limit) { *gave_up = 1; return false; }
    }
    return true;
}

// HD: head_dim padded to 64, 128 or 256 (head_dim itself is a multiple of 16).  EXACT: head_dim == HD;
// row sizes and the swizzle are then compile-time constants and a fragment's address is a register
// plus an immediate.
template <int HD, bool EXACT>
__global__ void __launch_bounds__(DEC_THREADS) attention_decode_kernel(AttentionArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ __align__(8) unsigned long long bar_storage[3];     // one per tile of the ring
    __shared__ float sm_m[DEC_WARPS][QROWS], sm_l[DEC_WARPS][QROWS];
    __shared__ int s_flag;
    __shared__ int s_gave_up;      // a wait ran out: the block no longer waits or issues, and its result is void
    // new_rows: the rotated query heads of the group, then the new key row and the new value row
    __shared__ __align__(16) __nv_bfloat16 new_s[(QROWS + 2) * 256];

    const int t = blockIdx.z, g = blockIdx.y, sp = blockIdx.x;
    const int hd = EXACT ? HD : a.head_dim, ps = a.page_size;
    const int G = a.n_heads / a.n_kv_heads;
    // The page list can only be read once the token's sequence and position are known: two trips to memory one
    // after the other, at a time when the kernel before this one keeps the memory system busy.  In a decode
    // step token t usually is sequence t and a run that does not start inside a window begins at page
    // sp * pages-per-run: ask for that line of the page list now (a hint only; the reads below decide).
    if (threadIdx.x == 0) {
        const int guess = (sp * (a.keys_per_split / ps)) % a.ring_pages;
        asm volatile("prefetch.global.L1 [%0];" ::"l"(a.tables + (long long)t * a.table_width + guess));
    }
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
    // Three tiles of [page_size][head_dim] (as stored: chunks swizzled by row) used in turn by the run's
    // key and value pages: K0 V0 K1 V1 ...; tile i of that sequence lives in place i % 3.  While one is read,
    // the next two are on their way, so a copy is asked for a page and a half before it is needed.
    const int chunks = hd / 8;
    const uint32_t row_bytes = (uint32_t)hd * 2;
    const uint32_t tile_bytes = (uint32_t)ps * row_bytes;
    const uint32_t tiles_s = (uint32_t)__cvta_generic_to_shared(smem);
    const uint32_t bars = (uint32_t)__cvta_generic_to_shared(&bar_storage[0]);

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
    if (tid == 0) {
        s_gave_up = 0;
        mbar_init(bars, 1);
        mbar_init(bars + 8, 1);
        mbar_init(bars + 16, 1);
    }
    __syncthreads();   // nobody waits on the barrier before it is initialised
    volatile int* gave_up = &s_gave_up;
    int issued = 0;    // thread 0: tiles asked for so far
    // A page's keys and its values are each one contiguous block: one bulk copy each (issued by thread 0).
    // Tile i of the run is the keys (i even) or the values (i odd) of page page_first + i / 2.
    const int n_tiles = 2 * (page_last - page_first + 1);
    // a step reads every page once: the pages pass through L2 marked to be evicted first and leave the step's
    // activations (and the next kernels' inputs) in place
    const unsigned long long kv_policy = l2_evict_first_policy();
    auto issue = [&](int i) {
        if (*gave_up) return;
        issued = i + 1;
        const int page = table[(page_first + (i >> 1)) % a.ring_pages];
        const long long off = ((long long)page * a.n_kv_heads + g) * ps * hd;
        const uint32_t place = (uint32_t)(i % 3);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_expect_tx(bars + 8 * place, tile_bytes + (i == 0 ? (uint32_t)a.test_extra_tx : 0u));
        bulk_load(tiles_s + place * tile_bytes, ((i & 1) ? vcache : kcache) + off, tile_bytes, bars + 8 * place, kv_policy);
    };
    auto wait_tile = [&](int i) { return mbar_wait_bounded(bars + 8 * (uint32_t)(i % 3), (uint32_t)((i / 3) & 1), a.wait_cycles, gave_up); };
    // The kernel before this one writes the step's new rows: positions from seq_past on.  A first page
    // that lies wholly below seq_past does not change any more and is fetched before that kernel has
    // finished.  (In a ring a new row of a later token of the same sequence could land in this page's
    // place, so there only a sequence's last token does it: the row it overwrites itself lies below
    // every page it reads.)
    // With new_rows no other kernel writes the cache in this step: every first page is fetched early.
    const bool fuse = a.new_rows != 0;
    const bool early = fuse || (a.seq_past != nullptr && (page_first + 1) * ps <= a.seq_past[seq] &&
                                (a.window <= 0 || t == a.seq_start[seq + 1] - 1));
    if (early && tid == 0) {
        issue(0);
        issue(1);
        if (fuse && n_tiles > 2) issue(2);       // with new_rows no page of the run changes any more
    }
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const bool has_new = fuse && sp == n_splits - 1;          // this block's run ends with the token's own position
    if (fuse) {
        // 16-byte chunks of the group's query heads and, in the block that reads position p, of the new key
        // and value rows: rotate (queries and key), keep in shared memory, write the new rows to the cache
        const int half = a.rotary_dim >> 1;
        const float* cs = a.rope_cos + (long long)p * half;
        const float* sn = a.rope_sin + (long long)p * half;
        const int items = (G + (has_new ? 2 : 0)) * chunks;
        for (int idx = tid; idx < items; idx += DEC_THREADS) {
            const int which = idx / chunks, c = idx - which * chunks, d0 = c * 8;
            const __nv_bfloat16* src =
                which < G ? (const __nv_bfloat16*)a.q + (long long)t * a.q_stride + (long long)(g * G + which) * hd
                          : (const __nv_bfloat16*)(which == G ? a.k_new : a.v_new) + (long long)t * a.kv_stride + (long long)g * hd;
            uint4 raw = *reinterpret_cast<const uint4*>(src + d0);
            if (which <= G && d0 < a.rotary_dim) {
                const bool first = d0 < half;                  // x[i] pairs with x[i + half]
                const uint4 other = *reinterpret_cast<const uint4*>(src + (first ? d0 + half : d0 - half));
                const int j = first ? d0 : d0 - half;
                const float4 c0 = *reinterpret_cast<const float4*>(cs + j), c1 = *reinterpret_cast<const float4*>(cs + j + 4);
                const float4 s0 = *reinterpret_cast<const float4*>(sn + j), s1 = *reinterpret_cast<const float4*>(sn + j + 4);
                const float cc[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
                const float ss[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
                const __nv_bfloat162* xo = reinterpret_cast<const __nv_bfloat162*>(&raw);
                const __nv_bfloat162* yo = reinterpret_cast<const __nv_bfloat162*>(&other);
                uint4 res;
                __nv_bfloat162* ro = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 x = __bfloat1622float2(xo[e]), y = __bfloat1622float2(yo[e]);
                    // first half: x cos - y sin; second half (x is x[i + half], y is x[i]): y sin + x cos
                    const float r0 = first ? x.x * cc[2 * e] - y.x * ss[2 * e] : y.x * ss[2 * e] + x.x * cc[2 * e];
                    const float r1 = first ? x.y * cc[2 * e + 1] - y.y * ss[2 * e + 1] : y.y * ss[2 * e + 1] + x.y * cc[2 * e + 1];
                    ro[e] = __floats2bfloat162_rn(r0, r1);
                }
                raw = res;
            }
            *reinterpret_cast<uint4*>(new_s + (which < G ? which : QROWS + which - G) * 256 + d0) = raw;
            if (which >= G) {
                __nv_bfloat16* cache = const_cast<__nv_bfloat16*>(which == G ? kcache : vcache);
                *reinterpret_cast<uint4*>(cache + rdl_cache_offset(table, p, ps, a.ring_pages, a.n_kv_heads, g, hd) +
                                          rdl_swizzled_chunk(p % ps, c, chunks) * 8) = raw;
            }
        }
        __syncthreads();
    }
    // The products are formed with the keys as rows: S^T [16 keys x 8 heads] = K [16 x d] Q^T [d x 8] and
    // O^T [d x 8 heads] += V^T [d x 16 keys] P^T [16 x 8].  Q^T is the B operand of every score product
    // of this block; it stays in registers: for k-step kk, {Q[head quad][16 kk + 2 tq .. +1], Q[..][16 kk + 8 + 2 tq .. +1]}.
    const int ksteps = hd / 16;
    uint32_t qf[HD / 16][2];
    {
        const __nv_bfloat16* qrow = fuse ? new_s + (quad < G ? quad : 0) * 256
                                         : (const __nv_bfloat16*)a.q + (long long)t * a.q_stride + (long long)(g * G + quad) * hd;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
            qf[kk][0] = qf[kk][1] = 0u;
            if (quad < G && kk < ksteps) {
                qf[kk][0] = *reinterpret_cast<const uint32_t*>(qrow + 16 * kk + 2 * tq);
                qf[kk][1] = *reinterpret_cast<const uint32_t*>(qrow + 16 * kk + 8 + 2 * tq);
            }
        }
    }
    // O^T accumulators: block db holds d = 16 db + quad (+ 8) for heads 2 tq, 2 tq + 1
    float o[HD / 16][4];
#pragma unroll
    for (int i = 0; i < HD / 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;      // of heads 2 tq and 2 tq + 1
    const float LOG2E = 1.4426950408889634f;
    const bool capped = a.softcap > 0.f;
    const float c_in = capped ? a.score_scale / a.softcap : a.score_scale * LOG2E;
    const float c_out = a.softcap * LOG2E;

    // Fragment addresses.  Keys (A of the score product): row w0 + (lane & 15), chunk 2 kk + (lane >> 4).
    // Values (A of the output product, transposed on load): row w0 + (lane & 7) + 8 (lane >> 4), chunk
    // 2 db + ((lane >> 3) & 1).  With c = 2 k + hi and the row's swizzle r: (c ^ r) * 16 =
    // 128 (k >> 2) + (((k & 3) << 5) ^ ((hi ^ r) << 4)): four registers and an immediate.
    const int kr = warp * 16 + (lane & 15);
    const int vr = warp * 16 + (lane & 7) + 8 * (lane >> 4);
    uint32_t ka[4], va[4];
    {
        const uint32_t kx = (uint32_t)(((kr & 7) ^ (lane >> 4)) << 4), vx = (uint32_t)(((vr & 7) ^ ((lane >> 3) & 1)) << 4);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            ka[j] = kr * row_bytes + (kx ^ (uint32_t)(j << 5));       // relative to the tile
            va[j] = vr * row_bytes + (vx ^ (uint32_t)(j << 5));
        }
    }
    uint32_t kb[4] = {0, 0, 0, 0}, vb[4] = {0, 0, 0, 0};   // ka, va in the tile that is being read
    auto k_addr = [&](int kk) -> uint32_t {
        if (EXACT) return kb[kk & 3] + (uint32_t)((kk >> 2) * 128);
        return kb[0] - ka[0] + kr * row_bytes + rdl_swizzled_chunk(kr, 2 * kk + (lane >> 4), chunks) * 16;
    };
    auto v_addr = [&](int db) -> uint32_t {
        if (EXACT) return vb[db & 3] + (uint32_t)((db >> 2) * 128);
        return vb[0] - va[0] + vr * row_bytes + rdl_swizzled_chunk(vr, 2 * db + ((lane >> 3) & 1), chunks) * 16;
    };

    if (tid == 0) {
        if (!early) {
            issue(0);
            issue(1);
        }
        if (!(early && fuse) && n_tiles > 2) issue(2);
    }
    for (int lp = page_first; lp <= page_last; ++lp) {
        const int ti = 2 * (lp - page_first);              // the tile of this page's keys; its values: ti + 1
        wait_tile(ti);
        unsigned char* k_tile = smem + (size_t)(ti % 3) * tile_bytes;
        unsigned char* v_tile = smem + (size_t)((ti + 1) % 3) * tile_bytes;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            kb[j] = tiles_s + (uint32_t)(ti % 3) * tile_bytes + ka[j];
            vb[j] = tiles_s + (uint32_t)((ti + 1) % 3) * tile_bytes + va[j];
        }
        if (has_new && lp == page_last) {
            // the copied page holds the row of position p as it was: put the new key there
            const int r = p - lp * ps;
            if (tid < chunks)
                *reinterpret_cast<uint4*>(k_tile + (size_t)r * row_bytes + rdl_swizzled_chunk(r, tid, chunks) * 16) =
                    *reinterpret_cast<const uint4*>(new_s + QROWS * 256 + tid * 8);
            __syncthreads();
        }
        const int r_begin = max(k_begin, lp * ps) - lp * ps, r_end = min(k_end, (lp + 1) * ps) - lp * ps;
        const int w0 = warp * 16;                  // this warp's 16 keys of the page
        const bool active = w0 < r_end && w0 + 16 > r_begin;
        float c0 = 1.f, c1 = 1.f;
        uint32_t pb0 = 0u, pb1 = 0u;
        if (active) {
            // ---- scores: rows = keys w0 + quad (+ 8), columns = heads 2 tq, 2 tq + 1 ----
            // four accumulators: the chain of dependent products is a quarter as long
            float s4[4][4];
#pragma unroll
            for (int j = 0; j < 4; ++j) s4[j][0] = s4[j][1] = s4[j][2] = s4[j][3] = 0.f;
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk) {
                if (EXACT || kk < ksteps) {
                    uint32_t af[4];
                    ldmatrix_x4(af, k_addr(kk));
                    mma_bf16(s4[kk & 3], af, qf[kk][0], qf[kk][1]);
                }
            }
            float s[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) s[e] = (s4[0][e] + s4[1][e]) + (s4[2][e] + s4[3][e]);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float v = capped ? tanh_fast(s[e] * c_in) * c_out : s[e] * c_in;
                const int r = w0 + quad + 8 * (e >> 1);
                if (r < r_begin || r >= r_end) v = -INFINITY;
                s[e] = v;
            }
            // maxima and sums over the 16 keys: over the two rows of a lane and over the lanes that differ in quad
            float mx0 = fmaxf(s[0], s[2]), mx1 = fmaxf(s[1], s[3]);
#pragma unroll
            for (int off = 4; off < 32; off <<= 1) {
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
            }
            const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
            const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;
            c0 = exp2f(m0 - ms0);
            c1 = exp2f(m1 - ms1);
            m0 = mn0; m1 = mn1;
            const float e0 = exp2f(s[0] - ms0), e1 = exp2f(s[1] - ms1), e2 = exp2f(s[2] - ms0), e3 = exp2f(s[3] - ms1);
            float rs0 = e0 + e2, rs1 = e1 + e3;
#pragma unroll
            for (int off = 4; off < 32; off <<= 1) {
                rs0 += __shfl_xor_sync(0xffffffffu, rs0, off);
                rs1 += __shfl_xor_sync(0xffffffffu, rs1, off);
            }
            l0 = l0 * c0 + rs0;
            l1 = l1 * c1 + rs1;
            // P^T as the B operand: the [key][head] fragments transposed to [head][key]
            asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(pb0) : "r"(pack_bf16(e0, e1)));
            asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(pb1) : "r"(pack_bf16(e2, e3)));
        }
        __syncthreads();                                   // every warp is done with the key tile: its place takes tile ti + 3
        if (ti + 3 < n_tiles && tid == 0) issue(ti + 3);
        wait_tile(ti + 1);
        if (has_new && lp == page_last) {
            const int r = p - lp * ps;
            if (tid < chunks)
                *reinterpret_cast<uint4*>(v_tile + (size_t)r * row_bytes + rdl_swizzled_chunk(r, tid, chunks) * 16) =
                    *reinterpret_cast<const uint4*>(new_s + (QROWS + 1) * 256 + tid * 8);
            __syncthreads();
        }
        if (active) {
            if (w0 < r_begin || w0 + 16 > r_end) {
                // value rows outside the run get the weight 0; they may hold anything (rows beyond the
                // sequence's end, an earlier occupant's rows), so make them zero: 0 * NaN is NaN
                for (int idx = lane; idx < 16 * chunks; idx += 32) {
                    const int r = w0 + idx / chunks;
                    if (r < r_begin || r >= r_end) *(uint4*)(v_tile + (size_t)r * row_bytes + (idx % chunks) * 16) = make_uint4(0, 0, 0, 0);
                }
                __syncwarp();
            }
            // ---- O^T += V^T P^T ----
#pragma unroll
            for (int db = 0; db < HD / 16; ++db) {
                if (EXACT || db * 16 < hd) {
                    uint32_t af[4];
                    ldmatrix_x4_trans(af, v_addr(db));
                    o[db][0] *= c0; o[db][1] *= c1; o[db][2] *= c0; o[db][3] *= c1;
                    mma_bf16(o[db], af, pb0, pb1);
                }
            }
        }
        __syncthreads();                                   // every warp is done with the value tile
        if (ti + 4 < n_tiles && tid == 0) issue(ti + 4);
    }

    if (*gave_up) {
        // No copy may still be on its way into this block's shared memory when the block ends: wait once more,
        // again with the limit, for the last tile asked of each place of the ring.
        if (tid == 0) {
            for (int pl = 0; pl < 3; ++pl) {
                int last = -1;
                for (int i = pl; i < issued; i += 3) last = i;
                if (last < 0) continue;
                const long long t0 = clock64();
                while (!mbar_try_wait(bars + 8 * (uint32_t)pl, (uint32_t)((last / 3) & 1)) && clock64() - t0 <= a.wait_cycles) {}
            }
            if (a.status) atomicExch(a.status, RDL_FAULT_ATTENTION_DECODE);
        }
        __syncthreads();
    }
    // ---- merge the four warps through shared memory, in warp order ----
    float* sm_o = reinterpret_cast<float*>(smem);    // [warp][head][HD]; the tiles are no longer needed
    if (quad == 0) {
        sm_m[warp][2 * tq] = m0; sm_m[warp][2 * tq + 1] = m1;
        sm_l[warp][2 * tq] = l0; sm_l[warp][2 * tq + 1] = l1;
    }
#pragma unroll
    for (int db = 0; db < HD / 16; ++db) {
        const int d = db * 16 + quad;
        if (d < hd) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int h = 2 * tq + (e & 1);
                if (h < G) sm_o[(warp * QROWS + h) * HD + d + 8 * (e >> 1)] = o[db][e];
            }
        }
    }
    __syncthreads();
    __nv_bfloat16* out = (__nv_bfloat16*)a.out + (long long)t * a.out_stride;
    int* counters = (int*)a.scratch;
    // partial sums [token][head][run][hd], then (maximum, normaliser) [token][head][run][2]
    float* partials = (float*)((char*)a.scratch + a.counter_bytes);
    float* stats = partials + (long long)a.n_tokens * a.n_heads * a.max_splits * hd;
    // four outputs per thread: the warps' sums weighted by exp2(their maximum - the block's)
    for (int idx = tid; idx < G * hd / 4; idx += DEC_THREADS) {
        const int h = (idx * 4) / hd, d = idx * 4 - h * hd;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, sm_m[w][h]);
        float4 osum = make_float4(0.f, 0.f, 0.f, 0.f);
        float lsum = 0.f;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) {
            const float wt = sm_m[w][h] == -INFINITY ? 0.f : exp2f(sm_m[w][h] - M);
            const float4 v = *reinterpret_cast<const float4*>(sm_o + (w * QROWS + h) * HD + d);
            osum.x = fmaf(wt, v.x, osum.x); osum.y = fmaf(wt, v.y, osum.y);
            osum.z = fmaf(wt, v.z, osum.z); osum.w = fmaf(wt, v.w, osum.w);
            lsum = fmaf(wt, sm_l[w][h], lsum);
        }
        if (n_splits == 1) {
            const float inv = 1.0f / lsum;
            __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(out + (long long)(g * G + h) * hd + d);
            o2[0] = __floats2bfloat162_rn(osum.x * inv, osum.y * inv);
            o2[1] = __floats2bfloat162_rn(osum.z * inv, osum.w * inv);
        } else {
            const long long run = ((long long)t * a.n_heads + (g * G + h)) * a.max_splits + sp;
            *reinterpret_cast<float4*>(partials + run * hd + d) = osum;
            if (d == 0) *reinterpret_cast<float2*>(stats + run * 2) = make_float2(M, lsum);
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
    float* inv_s = sm_o + G * n_splits;           // [G] 1 / normaliser
    const long long run0 = ((long long)t * a.n_heads + g * G) * a.max_splits;
    // The first sixteen runs' sums of this thread's first outputs are requested before the weights are
    // known: the two trips to L2 overlap (with eight, a context of nine runs cost a third trip).
    constexpr int AHEAD = 16;
    float4 ahead[AHEAD];
    {
        const int h = (tid * 4) / hd, d = tid * 4 - h * hd;
        const float* base = partials + (run0 + (long long)h * a.max_splits) * hd + d;
#pragma unroll
        for (int r = 0; r < AHEAD; ++r)
            ahead[r] = (tid < G * hd / 4 && r < n_splits) ? __ldcg(reinterpret_cast<const float4*>(base + (long long)r * hd))
                                                          : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int h = warp; h < G; h += DEC_WARPS) {
        const float2* st = reinterpret_cast<const float2*>(stats + (run0 + (long long)h * a.max_splits) * 2);
        // a lane's first two runs stay in registers: maximum and normaliser come in one trip
        float2 mine[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) mine[i] = lane + 32 * i < n_splits ? __ldcg(st + lane + 32 * i) : make_float2(-INFINITY, 0.f);
        float M = fmaxf(mine[0].x, mine[1].x);
        for (int r = lane + 64; r < n_splits; r += 32) M = fmaxf(M, __ldcg(st + r).x);
        M = warp_max(M);
        float L = 0.f;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            if (lane + 32 * i < n_splits) {
                const float wt = exp2f(mine[i].x - M);
                w_s[h * n_splits + lane + 32 * i] = wt;
                L = fmaf(wt, mine[i].y, L);
            }
        }
        for (int r = lane + 64; r < n_splits; r += 32) {
            const float2 v = __ldcg(st + r);
            const float wt = exp2f(v.x - M);
            w_s[h * n_splits + r] = wt;
            L = fmaf(wt, v.y, L);
        }
        L = warp_sum(L);
        if (lane == 0) inv_s[h] = 1.0f / L;
    }
    __syncthreads();
    for (int idx = tid; idx < G * hd / 4; idx += DEC_THREADS) {
        const int h = (idx * 4) / hd, d = idx * 4 - h * hd;
        const float* base = partials + (run0 + (long long)h * a.max_splits) * hd + d;
        const float* wts = w_s + h * n_splits;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        int r = 0;
        if (idx == tid) {                         // the outputs whose first runs are already here
#pragma unroll
            for (; r < AHEAD; ++r) {
                if (r < n_splits) {
                    const float wt = wts[r];
                    acc.x = fmaf(wt, ahead[r].x, acc.x); acc.y = fmaf(wt, ahead[r].y, acc.y);
                    acc.z = fmaf(wt, ahead[r].z, acc.z); acc.w = fmaf(wt, ahead[r].w, acc.w);
                }
            }
        }
#pragma unroll 8
        for (; r < n_splits; ++r) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(base + (long long)r * hd));
            const float wt = wts[r];
            acc.x = fmaf(wt, v.x, acc.x); acc.y = fmaf(wt, v.y, acc.y);
            acc.z = fmaf(wt, v.z, acc.z); acc.w = fmaf(wt, v.w, acc.w);
        }
        const float inv = inv_s[h];
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(out + (long long)(g * G + h) * hd + d);
        o2[0] = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
        o2[1] = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
    }
}

template <int HD, bool EXACT>
int launch_decode(const AttentionArgs* a, cudaStream_t st) {
    const int tiles = 3 * a->page_size * a->head_dim * 2;
    const int merge = DEC_WARPS * QROWS * HD * (int)sizeof(float);
    const int runs = (QROWS * a->max_splits + QROWS) * (int)sizeof(float);
    int smem = tiles > merge ? tiles : merge;
    if (runs > smem) smem = runs;
    RDL_REQUIRE(smem <= 200 * 1024, "attention_decode: page_size %d x head_dim %d needs %d bytes of shared memory, limit is 204800",
                a->page_size, a->head_dim, smem);
    static int granted = 32 * 1024;      // above this the kernel (which also has a few KB of static shared memory) opts in
    if (smem > granted) {
        RDL_CUDA(cudaFuncSetAttribute(attention_decode_kernel<HD, EXACT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem),
                 "attention_decode");
        granted = smem;
    }
    dim3 grid(a->max_splits, a->n_kv_heads, a->n_tokens);
    AttentionArgs b = *a;
    b.wait_cycles = rdl_wait_cycles_for(RDL_FAULT_ATTENTION_DECODE);
    b.test_extra_tx = rdl_test_extra_tx_for(RDL_FAULT_ATTENTION_DECODE);
    RDL_CHECK_EX(rdl_launch(attention_decode_kernel<HD, EXACT>, grid, dim3(DEC_THREADS), (size_t)smem, st, b), "attention_decode");
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
    if (a->new_rows) {
        RDL_REQUIRE(a->k_new && a->v_new && a->kv_stride % 8 == 0 && (uintptr_t)a->k_new % 16 == 0 && (uintptr_t)a->v_new % 16 == 0,
                    "attention_decode: the step's key and value rows must be given and start on 16-byte boundaries");
        RDL_REQUIRE(a->rotary_dim >= 0 && a->rotary_dim <= a->head_dim && a->rotary_dim % 16 == 0,
                    "attention_decode: rotary_dim %d must be a multiple of 16 and at most head_dim %d", a->rotary_dim, a->head_dim);
        RDL_REQUIRE(a->rotary_dim == 0 || (a->rope_cos && a->rope_sin && (uintptr_t)a->rope_cos % 16 == 0 && (uintptr_t)a->rope_sin % 16 == 0),
                    "attention_decode: rotation tables are missing or not on 16-byte boundaries");
        RDL_REQUIRE(a->n_tokens <= a->n_seqs, "attention_decode: new rows are written for one token per sequence");
    }
    if (a->n_tokens == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    if (a->head_dim == 64) return launch_decode<64, true>(a, st);
    if (a->head_dim == 128) return launch_decode<128, true>(a, st);
    if (a->head_dim == 256) return launch_decode<256, true>(a, st);
    if (a->head_dim < 64) return launch_decode<64, false>(a, st);
    if (a->head_dim < 128) return launch_decode<128, false>(a, st);
    return launch_decode<256, false>(a, st);
}
