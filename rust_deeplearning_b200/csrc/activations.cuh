// The activations of gated feed-forwards, in one place.  Codes are the RDL_ACT_* of api.h; the Python
// side maps names to codes (kernels/ops.py: ACTIVATIONS).  Another activation is one more code there
// and one more case in each of the two functions here; every kernel with a gated epilogue (the
// element-wise kernel, the weight-streaming product, the tcgen05 product) goes through these.
//   gelu_tanh(x) = 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3)))   rustml/core/main/src/core/tensor/ops.rs:433-438
//   silu(x) = x / (1 + exp(-x))
#pragma once

#include "api.h"

static inline bool rdl_activation_known(int act) { return act == RDL_ACT_GELU_TANH || act == RDL_ACT_SILU; }

// exact form: library tanh and exp
__device__ __forceinline__ float rdl_activation(float x, int act) {
    switch (act) {
        case RDL_ACT_GELU_TANH: return 0.5f * x * (1.0f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
        default: return x / (1.0f + expf(-x));
    }
}

// Fast form for results that are rounded to bfloat16 (8 bits of mantissa): the hardware tanh (relative error
// about 2^-11) and the fast exponential are accurate enough there and keep an epilogue short.
__device__ __forceinline__ float rdl_activation_fast(float x, int act) {
    switch (act) {
        case RDL_ACT_GELU_TANH: {
            float t;
            asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.7978845608028654f * (x + 0.044715f * x * x * x)));
            return 0.5f * x * (1.0f + t);
        }
        default: return __fdividef(x, 1.0f + __expf(fminf(-x, 80.0f)));     // the divisor stays below 2^126
    }
}
