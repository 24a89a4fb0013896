// Counter-based normal random numbers for the random-weights mode.
//
// Element j of a tensor depends only on (key, j): key is formed on the host from the seed and the
// tensor's name, so a tensor's values do not depend on which other tensors a model has, on the
// device that makes them or on how the work is split.  The same numbers are produced on the host
// by `weights/counter_random.py`; both sides use only operations that IEEE 754 rounds identically
// everywhere (add, multiply, divide, square root on doubles, never fused), so the float32 values
// agree bit for bit.  (The reference's random models are unseeded:
// rustml/core/main/src/core/tensor/tensor.rs:217-238.)
//
// Pair i (elements 2i and 2i+1): a = mix(key + 2i), b = mix(key + 2i + 1) with the splitmix64
// finaliser; u1 = ((a >> 12) + 0.5) 2^-52 in (0, 1), u2 = (b >> 11) 2^-53 in [0, 1);
// r = sqrt(-2 ln u1); (z0, z1) = r (cos 2 pi u2, sin 2 pi u2) (Box-Muller); out = float(z * std).
// ln: u1 = m 2^e with m in [sqrt(1/2), sqrt(2)), s = (m - 1) / (m + 1),
//     ln m = 2 s (1 + s^2/3 + ... + s^22/23), all by Horner's rule.
// cos, sin: quadrant q = floor(4 u2), angle t = (4 u2 - q) pi/2 in [0, pi/2), Taylor sums to t^22
//     and t^23 by Horner's rule in t^2, then the quadrant's signs and swap.
#include "api.h"
#include "common.cuh"

namespace {

__device__ __forceinline__ unsigned long long mix64(unsigned long long x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

struct NormalTables {
    double ln_c[12];     // 1 / (2k + 1)
    double sin_c[12];    // (-1)^k / (2k + 1)!
    double cos_c[12];    // (-1)^k / (2k)!
};

__device__ __forceinline__ double mul(double a, double b) { return __dmul_rn(a, b); }
__device__ __forceinline__ double add(double a, double b) { return __dadd_rn(a, b); }

__device__ __forceinline__ void normal_pair(unsigned long long key, unsigned long long i, const NormalTables& tb, double std,
                                            float& z0, float& z1) {
    const unsigned long long a = mix64(key + 2ull * i), b = mix64(key + 2ull * i + 1ull);
    const double u1 = mul(add(__ull2double_rn(a >> 12), 0.5), 2.220446049250313e-16);      // 2^-52
    const double u2 = mul(__ull2double_rn(b >> 11), 1.1102230246251565e-16);               // 2^-53
    int e;
    double m = frexp(u1, &e);                       // m in [0.5, 1), exact
    if (m < 0.7071067811865476) { m = mul(m, 2.0); e -= 1; }
    const double s = __ddiv_rn(add(m, -1.0), add(m, 1.0));
    const double s2 = mul(s, s);
    double p = tb.ln_c[11];
#pragma unroll
    for (int k = 10; k >= 0; --k) p = add(mul(p, s2), tb.ln_c[k]);
    const double ln_u1 = add(mul((double)e, 0.6931471805599453), mul(mul(2.0, s), p));
    const double r = __dsqrt_rn(mul(-2.0, ln_u1));
    const double t4 = mul(u2, 4.0);
    const double q = floor(t4);
    const double t = mul(add(t4, -q), 1.5707963267948966);
    const double t2 = mul(t, t);
    double ps = tb.sin_c[11], pc = tb.cos_c[11];
#pragma unroll
    for (int k = 10; k >= 0; --k) {
        ps = add(mul(ps, t2), tb.sin_c[k]);
        pc = add(mul(pc, t2), tb.cos_c[k]);
    }
    const double sn = mul(t, ps), cs = pc;
    const int qi = (int)q;
    const double c = qi == 0 ? cs : (qi == 1 ? -sn : (qi == 2 ? -cs : sn));
    const double sv = qi == 0 ? sn : (qi == 1 ? cs : (qi == 2 ? -sn : -cs));
    z0 = __double2float_rn(mul(mul(r, c), std));
    z1 = __double2float_rn(mul(mul(r, sv), std));
}

__global__ void random_normal_kernel(void* __restrict__ out, int dtype, long long n, unsigned long long key, double std,
                                     NormalTables tb) {
    const long long pairs = (n + 1) / 2;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < pairs; i += (long long)gridDim.x * blockDim.x) {
        float z0, z1;
        normal_pair(key, (unsigned long long)i, tb, std, z0, z1);
        rdl_store(out, 2 * i, dtype, z0);
        if (2 * i + 1 < n) rdl_store(out, 2 * i + 1, dtype, z1);
    }
}

}  // namespace

extern "C" int rdl_random_normal(void* out, int dtype, long long n, unsigned long long key, double std, void* stream) {
    RDL_REQUIRE(rdl_valid_dtype(dtype), "random_normal: bad dtype %d", dtype);
    RDL_REQUIRE(n >= 0 && out, "random_normal: bad size or missing output");
    if (n == 0) return 0;
    NormalTables tb;
    double f = 1.0;                                   // k!: the same divisions as the host mirror makes
    for (int k = 0; k < 12; ++k) {
        tb.ln_c[k] = 1.0 / (double)(2 * k + 1);
        if (k > 0) f *= (double)(2 * k - 1);
        if (k > 0) f *= (double)(2 * k);              // f = (2k)!
        tb.cos_c[k] = ((k & 1) ? -1.0 : 1.0) / f;
        tb.sin_c[k] = ((k & 1) ? -1.0 : 1.0) / (f * (double)(2 * k + 1));
    }
    const long long pairs = (n + 1) / 2;
    const long long blocks = (pairs + 255) / 256;
    random_normal_kernel<<<(unsigned)(blocks > rdl_sm_count() * 32 ? rdl_sm_count() * 32 : blocks), 256, 0, (cudaStream_t)stream>>>(out, dtype, n, key, std, tb);
    RDL_CHECK_LAUNCH("random_normal");
    return 0;
}
