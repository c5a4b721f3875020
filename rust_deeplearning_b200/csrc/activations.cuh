// The activations of gated feed-forwards, in one place.  Codes are the RDL_ACT_* of api.h; the Python
// side maps names to codes (kernels/ops.py: ACTIVATIONS).  Another activation is one more code there
// and one more case in each of the two functions here; every kernel with a gated epilogue (the
// element-wise kernel, the weight-streaming product, the tcgen05 product) goes through these.
//   gelu_tanh(x) = 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3)))   rustml/core/main/src/core/tensor/ops.rs:433-438
//   silu(x) = x / (1 + exp(-x))
// A gated feed-forward's value is gated(g, u) = act(g) * u for those two.  RDL_ACT_SWISH_LIMIT is a gated
// form with a parameter L: g' = min(g, L), u' = clamp(u, -L, L), value g' sigmoid(1.702 g') (u' + 1).
#pragma once

#include "api.h"

// codes rdl_activation takes (act(g) * u), and codes rdl_gated takes (those, and the forms with a parameter)
static inline bool rdl_activation_known(int act) { return act == RDL_ACT_GELU_TANH || act == RDL_ACT_SILU; }
static inline bool rdl_gated_known(int act) { return rdl_activation_known(act) || act == RDL_ACT_SWISH_LIMIT; }

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

// The value of a gated feed-forward from its two products; `param` is the activation's parameter (the limit of
// RDL_ACT_SWISH_LIMIT; unused by the others).
__device__ __forceinline__ float rdl_gated(float g, float u, int act, float param) {
    if (act == RDL_ACT_SWISH_LIMIT) {
        g = fminf(g, param);
        u = fminf(fmaxf(u, -param), param);
        return g / (1.0f + expf(-1.702f * g)) * (u + 1.0f);
    }
    return rdl_activation(g, act) * u;
}
__device__ __forceinline__ float rdl_gated_fast(float g, float u, int act, float param) {
    if (act == RDL_ACT_SWISH_LIMIT) {
        g = fminf(g, param);
        u = fminf(fmaxf(u, -param), param);
        return __fdividef(g, 1.0f + __expf(fminf(-1.702f * g, 80.0f))) * (u + 1.0f);
    }
    return rdl_activation_fast(g, act) * u;
}

// Element-wise activations of a product that is not gated (codes from 16 on, so that a plain product called with the
// gated forms' default code 0 stays plain): relu2(x) = max(x, 0)^2, silu.
static inline bool rdl_unary_known(int act) { return act == RDL_UNARY_RELU2 || act == RDL_UNARY_SILU; }
__device__ __forceinline__ float rdl_unary(float x, int act) {
    if (act == RDL_UNARY_RELU2) { const float r = fmaxf(x, 0.f); return r * r; }
    return x / (1.0f + expf(-x));
}
__device__ __forceinline__ float rdl_unary_fast(float x, int act) {
    if (act == RDL_UNARY_RELU2) { const float r = fmaxf(x, 0.f); return r * r; }
    return __fdividef(x, 1.0f + __expf(fminf(-x, 80.0f)));
}
