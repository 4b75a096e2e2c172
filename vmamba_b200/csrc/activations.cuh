// Activation functions shared by the elementwise kernels.
#pragma once
#include "common.cuh"

namespace ss2d {

enum { ACT_NONE = 0, ACT_GELU = 1, ACT_SILU = 2 };

template <typename T> __device__ __forceinline__ float round_to(float v) { return to_f<T>(from_f<T>(v)); }

template <int ACT> __device__ __forceinline__ float act_f(float v) {
    if constexpr (ACT == ACT_GELU) return 0.5f * v * (1.0f + erff(v * 0.70710678118654752f));   // exact (erf) GELU
    else if constexpr (ACT == ACT_SILU) return __fdividef(v, 1.0f + ex2_approx(-v * kLog2e));
    else return v;
}

// SiLU on a pair of values for 16-bit storage types: x sigmoid(x) = h + h tanh(h) with h = x / 2, one transcendental
// (tanh.approx, relative error 2^-11, an eighth of a bf16 step) instead of an exponential and a reciprocal.
__device__ __forceinline__ float2 silu_pair_fast(float2 v) {
    const float2 h = __fmul2_rn(v, make_float2(0.5f, 0.5f));
    float2 t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t.x) : "f"(h.x));
    asm("tanh.approx.f32 %0, %1;" : "=f"(t.y) : "f"(h.y));
    return __ffma2_rn(h, t, h);
}

// GELU (erf form) on a pair of values for 16-bit storage types.  erfc(z) = poly(t) * exp(-z^2),
// t = 1 / (1 + p z)  (Abramowitz-Stegun 7.1.26, absolute error 1.5e-7): for v < 0 the factor
// 1 + erf(v / sqrt 2) IS erfc(|v| / sqrt 2), so there is no cancellation and the relative error stays
// below 4e-4 down to v = -3.5, a fifth of a bf16 rounding step; beyond that erff is used (rare).
__device__ __forceinline__ float2 gelu_pair_fast(float2 v) {
    const float2 z = __fmul2_rn(make_float2(fabsf(v.x), fabsf(v.y)), make_float2(0.70710678118654752f, 0.70710678118654752f));
    const float2 den = __ffma2_rn(make_float2(0.3275911f, 0.3275911f), z, make_float2(1.f, 1.f));
    float2 t;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t.x) : "f"(den.x));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t.y) : "f"(den.y));
    float2 pl = __ffma2_rn(make_float2(1.061405429f, 1.061405429f), t, make_float2(-1.453152027f, -1.453152027f));
    pl = __ffma2_rn(pl, t, make_float2(1.421413741f, 1.421413741f));
    pl = __ffma2_rn(pl, t, make_float2(-0.284496736f, -0.284496736f));
    pl = __ffma2_rn(pl, t, make_float2(0.254829592f, 0.254829592f));
    pl = __fmul2_rn(pl, t);
    const float2 arg = __fmul2_rn(__fmul2_rn(z, z), make_float2(-kLog2e, -kLog2e));
    const float2 q = __fmul2_rn(pl, make_float2(ex2_approx(arg.x), ex2_approx(arg.y)));      // erfc(|v| / sqrt 2)
    const float2 cdf2 = make_float2(v.x < 0.f ? q.x : 2.f - q.x, v.y < 0.f ? q.y : 2.f - q.y);   // 1 + erf(v / sqrt 2)
    float2 r = __fmul2_rn(__fmul2_rn(v, make_float2(0.5f, 0.5f)), cdf2);
    if (fminf(v.x, v.y) < -3.5f) {       // far tail (rare): the exact form for whichever value is there
        if (v.x < -3.5f) r.x = act_f<ACT_GELU>(v.x);
        if (v.y < -3.5f) r.y = act_f<ACT_GELU>(v.y);
    }
    return r;
}

// GELU (erf form) on the FMA pipe alone: half the instructions of the form above and no transcendental, at a
// larger absolute error (7.5e-4 against 4e-4 relative): what the 16-bit kernels of the backbone use.
// gelu(v) = v * Phi(v), Phi(v) = 1/2 + z P(z^2) with z = v / sqrt 2 and P an even polynomial of degree 12 fitted to
// erf(z) / (2 z) on |z| <= 3.  The final fused multiply-add saturates to [0, 1], which is Phi's range; beyond the fitted
// range P(t) >= 1 / (2 sqrt t) for every t > 9 (its leading coefficient is positive), so |z P| >= 1/2 there and the result
// is exactly 0 or 1 without a clamp on the argument.  |gelu error| <= 7.5e-4 for every v, a fifth of a bf16 step at 1.
__device__ __forceinline__ float fma_sat(float a, float b, float c) {
    float d;
    asm("fma.rn.sat.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ float2 gelu_pair_poly(float2 v) {
    const float kC = 0.70710678118654752f;
    const float2 z = __fmul2_rn(v, make_float2(kC, kC));
    const float2 t = __fmul2_rn(z, z);
    float2 p = make_float2(1.840303185e-06f, 1.840303185e-06f);
    p = __ffma2_rn(p, t, make_float2(-6.794340152e-05f, -6.794340152e-05f));
    p = __ffma2_rn(p, t, make_float2(1.058246824e-03f, 1.058246824e-03f));
    p = __ffma2_rn(p, t, make_float2(-9.187800810e-03f, -9.187800810e-03f));
    p = __ffma2_rn(p, t, make_float2(4.991913959e-02f, 4.991913959e-02f));
    p = __ffma2_rn(p, t, make_float2(-1.834703386e-01f, -1.834703386e-01f));
    p = __ffma2_rn(p, t, make_float2(5.632318258e-01f, 5.632318258e-01f));
    const float2 phi = make_float2(fma_sat(p.x, z.x, 0.5f), fma_sat(p.y, z.y, 0.5f));
    return __fmul2_rn(v, phi);
}

}  // namespace ss2d
