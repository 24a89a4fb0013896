// Matrix product of the 32-bit path: out[m, n] = sum_k x[m, k] * w[n, k], float operands, fused
// multiply-add in float, no tensor cores and no reduced-precision mode.  Every output element is
// summed over k = 0 .. K-1 in that order, whatever M, N or the element's place in a tile, so a
// row's result does not depend on which other rows are in the batch.
// (The reference's product is an f32 library GEMM: rustml/core/main/src/core/tensor/ops.rs:806-823;
// y = x W^T with W [out, in]: rustml/nn/main/src/core/linear.rs:12-15, :168-169.)
#include "api.h"
#include "common.cuh"

namespace {

constexpr int TM = 64, TN = 64, TK = 16;

__global__ void __launch_bounds__(256) gemm_f32_kernel(float* __restrict__ out, const float* __restrict__ x,
                                                       const float* __restrict__ w, int M, int N, int K) {
    __shared__ float xs[TK][TM + 1];
    __shared__ float ws[TK][TN + 1];
    const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;   // 16 x 16 threads, 4 x 4 outputs each
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += TK) {
        // 64 rows x 16 k of each operand: 1024 values, 4 per thread, k fastest for coalescing
        for (int idx = threadIdx.x; idx < TM * TK; idx += 256) {
            const int r = idx / TK, kk = idx - r * TK;
            const int gm = m0 + r, gn = n0 + r, gk = k0 + kk;
            xs[kk][r] = (gm < M && gk < K) ? x[(long long)gm * K + gk] : 0.f;
            ws[kk][r] = (gn < N && gk < K) ? w[(long long)gn * K + gk] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn < N) out[(long long)gm * N + gn] = acc[i][j];
        }
    }
}

}  // namespace

extern "C" int rdl_gemm_f32(void* out, const void* x, const void* w, int m, int n, int k, void* stream) {
    RDL_REQUIRE(m >= 0 && n > 0 && k > 0, "gemm_f32: bad sizes m=%d n=%d k=%d", m, n, k);
    RDL_REQUIRE(out && x && w, "gemm_f32: missing operand");
    if (m == 0) return 0;
    dim3 grid((n + TN - 1) / TN, (m + TM - 1) / TM);
    RDL_REQUIRE(grid.y <= 65535, "gemm_f32: %d rows exceed the grid limit", m);
    gemm_f32_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((float*)out, (const float*)x, (const float*)w, m, n, k);
    RDL_CHECK_LAUNCH("gemm_f32");
    return 0;
}
