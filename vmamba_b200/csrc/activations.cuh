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

}  // namespace ss2d
