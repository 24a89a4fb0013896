// Row-wise kernels: embedding gather, fused RMS norms with the residual sum, gated
// activation, soft-cap.  All statistics and sums are computed in float.
//
// Formulas (reference, paths within rustml/):
//   embedding gather * scale        nn/main/src/core/embedding.rs:50-76, nlp/main/src/core/model.rs:896-900
//   x / sqrt(mean(x^2)+eps) * (w+o) core/main/src/core/tensor/ops.rs:735-743, nn/main/src/core/rms_norm.rs:43-50
//   gelu_tanh(g) * u                nn/main/src/core/feed_forward.rs:151-161, core/main/src/core/tensor/ops.rs:433-438
//   cap * tanh(z / cap)             nn/main/src/core/attention.rs:419-423
#include "activations.cuh"
#include "api.h"
#include "common.cuh"
#include "launch.cuh"

// ---------------------------------------------------------------------------------------------
// embedding
// ---------------------------------------------------------------------------------------------
__global__ void embed_rows_kernel(float* __restrict__ out, const void* __restrict__ table, int table_dtype,
                                  const int* __restrict__ ids, float scale, int hidden, int vocab,
                                  int* __restrict__ status) {
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (long long)t * hidden;
    if (id < 0 || id >= vocab) {
        // never a wrong result: the row is poisoned and the step reports the fault
        for (int j = threadIdx.x; j < hidden; j += blockDim.x) o[j] = __int_as_float(0x7fc00000);
        if (threadIdx.x == 0 && status) atomicExch(status, RDL_FAULT_TOKEN_ID);
        return;
    }
    const long long base = (long long)id * hidden;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) o[j] = rdl_load(table, base + j, table_dtype) * scale;
}

extern "C" int rdl_embed_rows(void* out_f32, const void* table, int table_dtype, const int* ids, float scale,
                              int n_rows, int hidden, int vocab, int* status, void* stream) {
    RDL_REQUIRE(rdl_valid_dtype(table_dtype), "embed_rows: bad table dtype %d", table_dtype);
    RDL_REQUIRE(n_rows >= 0 && hidden > 0 && vocab > 0, "embed_rows: bad sizes rows=%d hidden=%d vocab=%d", n_rows, hidden, vocab);
    if (n_rows == 0) return 0;
    const int threads = hidden >= 1024 ? 256 : 128;
    RDL_CHECK_EX(rdl_launch(embed_rows_kernel, dim3(n_rows), dim3(threads), 0, (cudaStream_t)stream, (float*)out_f32, table,
                            table_dtype, ids, scale, hidden, vocab, status), "embed_rows");
    return 0;
}

// ---------------------------------------------------------------------------------------------
// fused norm / residual / norm
//   t = w1 ? rms_norm(x; w1, eps1, off1) : x
//   h = res ? res + t : t ;  res <- h (float) when res is given
//   y = w2 ? rms_norm(h; w2, eps2, off2) : h          (written when y is given)
// x rows may be gathered through row_index.
// ---------------------------------------------------------------------------------------------
struct NormArgs {
    const void* x; int x_dtype;
    const int* row_index;
    const void* w1; int w1_dtype; float eps1, off1;
    float* res;
    const void* w2; int w2_dtype; float eps2, off2;
    void* y; int y_dtype;
    int hidden;
};

__global__ void norm_residual_norm_kernel(NormArgs a) {
    extern __shared__ float row[];          // hidden floats
    __shared__ float scratch[33];
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const int r = blockIdx.x;
    const int H = a.hidden;
    const long long xin = (long long)(a.row_index ? a.row_index[r] : r) * H;
    const long long out = (long long)r * H;

    float ss = 0.f;
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
        const float v = rdl_load(a.x, xin + j, a.x_dtype);
        row[j] = v;
        ss += v * v;
    }
    if (a.w1) {
        ss = block_sum(ss, scratch);
        const float inv = 1.0f / sqrtf(ss / (float)H + a.eps1);
        for (int j = threadIdx.x; j < H; j += blockDim.x)
            row[j] = row[j] * inv * (rdl_load(a.w1, j, a.w1_dtype) + a.off1);
    }
    if (a.res) {
        for (int j = threadIdx.x; j < H; j += blockDim.x) {
            const float h = a.res[out + j] + row[j];
            a.res[out + j] = h;
            row[j] = h;
        }
    }
    if (!a.y) return;
    if (a.w2) {
        float s2 = 0.f;
        for (int j = threadIdx.x; j < H; j += blockDim.x) s2 += row[j] * row[j];
        s2 = block_sum(s2, scratch);
        const float inv = 1.0f / sqrtf(s2 / (float)H + a.eps2);
        for (int j = threadIdx.x; j < H; j += blockDim.x)
            rdl_store(a.y, out + j, a.y_dtype, row[j] * inv * (rdl_load(a.w2, j, a.w2_dtype) + a.off2));
    } else {
        for (int j = threadIdx.x; j < H; j += blockDim.x) rdl_store(a.y, out + j, a.y_dtype, row[j]);
    }
}

// The same operation with the row held in registers: every load of a row is issued before the
// first reduction, so the kernel's critical path is one trip to memory and two block sums.  Used
// when hidden is a multiple of 4 and at most THREADS * 4 * ITER (ITER <= 8).
__device__ __forceinline__ float4 load4(const void* p, long long i, int dtype) {
    if (dtype == RDL_BF16) {
        const uint2 raw = *reinterpret_cast<const uint2*>((const __nv_bfloat16*)p + i);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    return *reinterpret_cast<const float4*>((const float*)p + i);
}
__device__ __forceinline__ void store4(void* p, long long i, int dtype, float4 v) {
    if (dtype == RDL_BF16) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<uint32_t*>(&a);
        raw.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>((__nv_bfloat16*)p + i) = raw;
    } else {
        *reinterpret_cast<float4*>((float*)p + i) = v;
    }
}

// LATE (many rows): the weights are fetched where they are used (they come from the cache by then) instead of
// being held in registers from the start, and the register count is bounded so that more rows are in
// flight per multiprocessor: with many rows the kernel is bound by the bytes it has in flight.  With few
// rows (decode) everything is requested at once: there the one row's latency is what counts.
constexpr int norm_min_blocks(int iter, int threads, bool late) {
    if (!late) return 1;
    const int by_registers = 65536 / (threads * (8 * iter + (iter >= 4 ? 24 : 16))), by_threads = 2048 / threads;
    const int n = by_registers < by_threads ? by_registers : by_threads;
    return n < 1 ? 1 : n;
}
template <int ITER, int THREADS, bool LATE>
__global__ void __launch_bounds__(THREADS, norm_min_blocks(ITER, THREADS, LATE)) norm_residual_norm_vec_kernel(NormArgs a) {
    __shared__ float scratch[33];
    // Few rows (a decode step): the kernel after this one, a product, is let go before this kernel has waited for
    // its own inputs: its blocks find room as soon as the product before this kernel ends and bring their first
    // weights in meanwhile (its own wait still ends only when this kernel has finished).  Measured: 0.6 to 1 % of a step.
    if (!LATE) rdl_grid_launch_dependents();
    rdl_grid_wait();
    if (LATE) rdl_grid_launch_dependents();
    const int r = blockIdx.x;
    const int H = a.hidden;
    const long long xin = (long long)(a.row_index ? a.row_index[r] : r) * H;
    const long long out = (long long)r * H;
    float4 xv[ITER], rv[ITER], w1v[ITER], w2v[ITER];
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < ITER; ++i) {
        const int j = (i * THREADS + threadIdx.x) * 4;
        const bool on = j < H;
        xv[i] = on ? load4(a.x, xin + j, a.x_dtype) : zero;
        rv[i] = (on && a.res) ? *reinterpret_cast<const float4*>(a.res + out + j) : zero;
        if (!LATE) {
            w1v[i] = (on && a.w1) ? load4(a.w1, j, a.w1_dtype) : zero;
            w2v[i] = (on && a.w2 && a.y) ? load4(a.w2, j, a.w2_dtype) : zero;
        }
    }
    if (a.w1) {
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < ITER; ++i) ss += xv[i].x * xv[i].x + xv[i].y * xv[i].y + xv[i].z * xv[i].z + xv[i].w * xv[i].w;
        ss = block_sum(ss, scratch);
        const float inv = 1.0f / sqrtf(ss / (float)H + a.eps1);
#pragma unroll
        for (int i = 0; i < ITER; ++i) {
            if (LATE) {
                const int j = (i * THREADS + threadIdx.x) * 4;
                w1v[i] = j < H ? load4(a.w1, j, a.w1_dtype) : zero;
            }
            xv[i].x = xv[i].x * inv * (w1v[i].x + a.off1);
            xv[i].y = xv[i].y * inv * (w1v[i].y + a.off1);
            xv[i].z = xv[i].z * inv * (w1v[i].z + a.off1);
            xv[i].w = xv[i].w * inv * (w1v[i].w + a.off1);
        }
    }
    if (a.res) {
#pragma unroll
        for (int i = 0; i < ITER; ++i) {
            const int j = (i * THREADS + threadIdx.x) * 4;
            xv[i].x += rv[i].x; xv[i].y += rv[i].y; xv[i].z += rv[i].z; xv[i].w += rv[i].w;
            if (j < H) *reinterpret_cast<float4*>(a.res + out + j) = xv[i];
        }
    }
    if (!a.y) return;
    float inv2 = 1.f;
    if (a.w2) {
        float s2 = 0.f;
#pragma unroll
        for (int i = 0; i < ITER; ++i) s2 += xv[i].x * xv[i].x + xv[i].y * xv[i].y + xv[i].z * xv[i].z + xv[i].w * xv[i].w;
        s2 = block_sum(s2, scratch);
        inv2 = 1.0f / sqrtf(s2 / (float)H + a.eps2);
    }
#pragma unroll
    for (int i = 0; i < ITER; ++i) {
        const int j = (i * THREADS + threadIdx.x) * 4;
        if (j >= H) continue;
        float4 v = xv[i];
        if (a.w2) {
            if (LATE) w2v[i] = load4(a.w2, j, a.w2_dtype);
            v.x = v.x * inv2 * (w2v[i].x + a.off2);
            v.y = v.y * inv2 * (w2v[i].y + a.off2);
            v.z = v.z * inv2 * (w2v[i].z + a.off2);
            v.w = v.w * inv2 * (w2v[i].w + a.off2);
        }
        store4(a.y, out + j, a.y_dtype, v);
    }
}

static bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

extern "C" int rdl_norm_residual_norm(const void* x, int x_dtype, const int* row_index,
                                      const void* w1, int w1_dtype, float eps1, float off1,
                                      void* res_f32,
                                      const void* w2, int w2_dtype, float eps2, float off2,
                                      void* y, int y_dtype, int n_rows, int hidden, void* stream) {
    if (hidden > 0 && hidden % 4 == 0 && hidden <= 8192 && n_rows > 0 && rdl_valid_dtype(x_dtype) && rdl_valid_dtype(y_dtype) &&
        (!w1 || rdl_valid_dtype(w1_dtype)) && (!w2 || rdl_valid_dtype(w2_dtype)) && !(row_index && res_f32) && (y || res_f32) &&
        aligned16(x) && aligned16(res_f32) && aligned16(w1) && aligned16(w2) && aligned16(y)) {
        NormArgs a{x, x_dtype, row_index, w1, w1_dtype, eps1, off1, (float*)res_f32, w2, w2_dtype, eps2, off2, y, y_dtype, hidden};
        cudaStream_t st = (cudaStream_t)stream;
        cudaError_t e;
        // Threads per row: few rows (decode) want the row spread over many threads; many rows (prefill) want
        // many busy threads and many rows in flight per multiprocessor, so the block is the one of 128, 192 or
        // 256 threads chosen below.  The block size fixes the
        // order in which a row's squares are summed, so the 32-bit path (float results) always takes the one
        // shape that depends on `hidden` alone: a row's result then does not depend on how many rows the
        // step has.  The bfloat16 path rounds its results to 8 bits anyway and keeps the faster choice.
        const bool float_path = y ? y_dtype == RDL_F32 : x_dtype == RDL_F32;
        const bool many_rows = n_rows >= 256 && !float_path;
        const int quads = hidden / 4;
        int threads = 256;
        if (many_rows) {
            // the block that keeps most useful threads resident: threads a multiprocessor holds at this row length (the
            // register bound of the many-row form) times the share of them that have an element.  (Fewest idle lanes
            // alone chose 128 threads x 7 for a width of 3,584: six blocks a multiprocessor, 30.8 us for 2,048 rows
            // against 21.0 with 192 x 5; 4,608: 192 x 6 29.0 us, 256 x 5 27.1.)
            long long best = -1;
            for (int t = 128; t <= 256; t += 64) {
                const int iter = (quads + t - 1) / t;
                if (iter > 8) continue;
                const long long useful = (long long)norm_min_blocks(iter, t, true) * quads / iter;
                if (useful > best) { best = useful; threads = t; }
            }
        }
        const int iter = (quads + threads - 1) / threads;
        const bool late = many_rows;
#define RDL_NORM_CASE(I, T, L) if (iter == I && threads == T && late == L) e = rdl_launch(norm_residual_norm_vec_kernel<I, T, L>, dim3(n_rows), dim3(T), 0, st, a); else
#define RDL_NORM_ITERS(T, L) RDL_NORM_CASE(1, T, L) RDL_NORM_CASE(2, T, L) RDL_NORM_CASE(3, T, L) RDL_NORM_CASE(4, T, L) RDL_NORM_CASE(5, T, L) RDL_NORM_CASE(6, T, L) RDL_NORM_CASE(7, T, L) RDL_NORM_CASE(8, T, L)
        RDL_NORM_ITERS(128, true) RDL_NORM_ITERS(192, true) RDL_NORM_ITERS(256, true) RDL_NORM_ITERS(256, false)
        e = cudaErrorInvalidConfiguration;
#undef RDL_NORM_ITERS
#undef RDL_NORM_CASE
        RDL_CHECK_EX(e, "norm_residual_norm");
        return 0;
    }
    RDL_REQUIRE(rdl_valid_dtype(x_dtype) && rdl_valid_dtype(y_dtype), "norm: bad dtype");
    RDL_REQUIRE(!w1 || rdl_valid_dtype(w1_dtype), "norm: bad dtype of the first weight");
    RDL_REQUIRE(!w2 || rdl_valid_dtype(w2_dtype), "norm: bad dtype of the second weight");
    RDL_REQUIRE(n_rows >= 0 && hidden > 0, "norm: bad sizes rows=%d hidden=%d", n_rows, hidden);
    RDL_REQUIRE(!(row_index && res_f32), "norm: gathered rows cannot be combined with a residual");
    RDL_REQUIRE(y || res_f32, "norm: nothing to write");
    const size_t smem = (size_t)hidden * sizeof(float);
    RDL_REQUIRE(smem <= 200 * 1024, "norm: hidden size %d needs %zu bytes of shared memory, limit is 204800", hidden, smem);
    if (n_rows == 0) return 0;
    if (smem > 48 * 1024) {
        static size_t granted = 0;  // largest size already opted in
        if (smem > granted) {
            RDL_CUDA(cudaFuncSetAttribute(norm_residual_norm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "norm");
            granted = smem;
        }
    }
    NormArgs a{x, x_dtype, row_index, w1, w1_dtype, eps1, off1, (float*)res_f32, w2, w2_dtype, eps2, off2, y, y_dtype, hidden};
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    RDL_CHECK_EX(rdl_launch(norm_residual_norm_kernel, dim3(n_rows), dim3(threads), smem, (cudaStream_t)stream, a), "norm_residual_norm");
    return 0;
}

// ---------------------------------------------------------------------------------------------
// gated activation: out[t, i] = act(gu[t, i]) * gu[t, I + i]
// ---------------------------------------------------------------------------------------------
__global__ void gated_activation_kernel(void* __restrict__ out, const void* __restrict__ gu, int dtype, int act,
                                        long long n_rows, int inter) {
    const long long total = n_rows * inter;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long t = idx / inter;
        const int i = (int)(idx - t * inter);
        const float g = rdl_load(gu, t * 2 * inter + i, dtype);
        const float u = rdl_load(gu, t * 2 * inter + inter + i, dtype);
        const float a = rdl_activation(g, act);
        rdl_store(out, idx, dtype, a * u);
    }
}

// bfloat16 rows whose width is a multiple of 8: eight values (16 bytes) of gate and of up per thread
__global__ void gated_activation_bf16x8_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ gu, int act,
                                               long long n_rows, int inter) {
    const int chunks = inter >> 3;
    const long long total = n_rows * chunks;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long t = idx / chunks;
        const int c = (int)(idx - t * chunks);
        const uint4 graw = *reinterpret_cast<const uint4*>(gu + t * 2 * inter + c * 8);
        const uint4 uraw = *reinterpret_cast<const uint4*>(gu + t * 2 * inter + inter + c * 8);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&graw);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uraw);
        uint4 res;
        __nv_bfloat162* r2 = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 g = __bfloat1622float2(g2[i]), u = __bfloat1622float2(u2[i]);
            const float a0 = rdl_activation(g.x, act);
            const float a1 = rdl_activation(g.y, act);
            r2[i] = __floats2bfloat162_rn(a0 * u.x, a1 * u.y);
        }
        *reinterpret_cast<uint4*>(out + t * inter + c * 8) = res;
    }
}

extern "C" int rdl_gated_activation(void* out, const void* gate_up, int dtype, int activation, int n_rows, int inter,
                                    void* stream) {
    RDL_REQUIRE(rdl_valid_dtype(dtype), "gated_activation: bad dtype %d", dtype);
    RDL_REQUIRE(rdl_activation_known(activation), "gated_activation: unknown activation %d", activation);
    RDL_REQUIRE(n_rows >= 0 && inter > 0, "gated_activation: bad sizes");
    if (n_rows == 0) return 0;
    const long long total = (long long)n_rows * inter;
    const int threads = 256;
    if (dtype == RDL_BF16 && inter % 8 == 0 && ((uintptr_t)out & 15) == 0 && ((uintptr_t)gate_up & 15) == 0) {
        const long long blocks8 = (total / 8 + threads - 1) / threads;
        gated_activation_bf16x8_kernel<<<(unsigned)(blocks8 > rdl_sm_count() * 32 ? rdl_sm_count() * 32 : blocks8), threads, 0, (cudaStream_t)stream>>>(
            (__nv_bfloat16*)out, (const __nv_bfloat16*)gate_up, activation, n_rows, inter);
        RDL_CHECK_LAUNCH("gated_activation");
        return 0;
    }
    const long long blocks = (total + threads - 1) / threads;
    gated_activation_kernel<<<(unsigned)(blocks > rdl_sm_count() * 16 ? rdl_sm_count() * 16 : blocks), threads, 0, (cudaStream_t)stream>>>(
        out, gate_up, dtype, activation, n_rows, inter);
    RDL_CHECK_LAUNCH("gated_activation");
    return 0;
}

// ---------------------------------------------------------------------------------------------
// soft-cap in place on float rows, and residual add
// ---------------------------------------------------------------------------------------------
__global__ void softcap_kernel(float* __restrict__ z, long long total, float cap) {
    const float inv = 1.0f / cap;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x)
        z[i] = cap * tanhf(z[i] * inv);
}

extern "C" int rdl_softcap_inplace(void* z_f32, long long total, float cap, void* stream) {
    RDL_REQUIRE(cap > 0.f, "softcap: cap must be positive, got %g", (double)cap);
    RDL_REQUIRE(total >= 0, "softcap: bad size");
    if (total == 0) return 0;
    const long long blocks = (total + 255) / 256;
    softcap_kernel<<<(unsigned)(blocks > rdl_sm_count() * 16 ? rdl_sm_count() * 16 : blocks), 256, 0, (cudaStream_t)stream>>>((float*)z_f32, total, cap);
    RDL_CHECK_LAUNCH("softcap");
    return 0;
}

__global__ void residual_add_kernel(float* __restrict__ res, const void* __restrict__ x, int dtype, long long total) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x)
        res[i] += rdl_load(x, i, dtype);
}

extern "C" int rdl_residual_add(void* res_f32, const void* x, int x_dtype, long long total, void* stream) {
    RDL_REQUIRE(rdl_valid_dtype(x_dtype), "residual_add: bad dtype");
    if (total <= 0) return 0;
    const long long blocks = (total + 255) / 256;
    residual_add_kernel<<<(unsigned)(blocks > rdl_sm_count() * 16 ? rdl_sm_count() * 16 : blocks), 256, 0, (cudaStream_t)stream>>>(
        (float*)res_f32, x, x_dtype, total);
    RDL_CHECK_LAUNCH("residual_add");
    return 0;
}

// Copies `rows` rows of `width` floats/bf16 chosen by row_index into a dense output, converting dtype.
__global__ void convert_rows_kernel(void* __restrict__ out, int out_dtype, const void* __restrict__ in, int in_dtype,
                                    const int* __restrict__ row_index, int width) {
    const long long src = (long long)(row_index ? row_index[blockIdx.x] : blockIdx.x) * width;
    const long long dst = (long long)blockIdx.x * width;
    for (int j = threadIdx.x; j < width; j += blockDim.x) rdl_store(out, dst + j, out_dtype, rdl_load(in, src + j, in_dtype));
}

extern "C" int rdl_convert_rows(void* out, int out_dtype, const void* in, int in_dtype, const int* row_index,
                                int n_rows, int width, void* stream) {
    RDL_REQUIRE(rdl_valid_dtype(out_dtype) && rdl_valid_dtype(in_dtype), "convert_rows: bad dtype");
    if (n_rows <= 0) return 0;
    convert_rows_kernel<<<n_rows, 256, 0, (cudaStream_t)stream>>>(out, out_dtype, in, in_dtype, row_index, width);
    RDL_CHECK_LAUNCH("convert_rows");
    return 0;
}

// ---------------------------------------------------------------------------------------------
// batch description: pinned host memory -> device, with the ids an earlier sampling left on the device put in place
// ---------------------------------------------------------------------------------------------
__global__ void upload_batch_kernel(int* __restrict__ dst, const int* __restrict__ src, int n, const int* __restrict__ sampled,
                                    int token_src_at, int tokens_at, int n_fed) {
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const int quads = n >> 2;
    for (int q = blockIdx.x * blockDim.x + threadIdx.x; q < quads; q += gridDim.x * blockDim.x) {
        int4 v = reinterpret_cast<const int4*>(src)[q];
        if (sampled) {
            int* e = reinterpret_cast<int*>(&v);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int i = 4 * q + k - tokens_at;
                if (i >= 0 && i < n_fed) e[k] = sampled[src[token_src_at + i]];
            }
        }
        reinterpret_cast<int4*>(dst)[q] = v;
    }
}

extern "C" int rdl_upload_batch(int* dst, const int* src_pinned, int n_ints, const int* sampled, int token_src_at, int tokens_at,
                                int n_fed, void* stream) {
    RDL_REQUIRE(dst && src_pinned && n_ints >= 0 && n_ints % 4 == 0, "upload_batch: %d values (a multiple of 4 is expected)", n_ints);
    RDL_REQUIRE(((uintptr_t)dst & 15) == 0 && ((uintptr_t)src_pinned & 15) == 0, "upload_batch: buffers must start on 16-byte boundaries");
    RDL_REQUIRE(!sampled || (n_fed >= 0 && token_src_at >= 0 && tokens_at >= 0 && token_src_at + n_fed <= n_ints && tokens_at + n_fed <= n_ints),
                "upload_batch: the fed tokens lie outside the description");
    if (n_ints == 0) return 0;
    const int threads = 256, quads = n_ints / 4;
    int blocks = (quads + threads - 1) / threads;
    if (blocks > 64) blocks = 64;
    RDL_CHECK_EX(rdl_launch(upload_batch_kernel, dim3(blocks), dim3(threads), 0, (cudaStream_t)stream, dst, src_pinned, n_ints, sampled,
                            token_src_at, tokens_at, n_fed), "upload_batch");
    return 0;
}
