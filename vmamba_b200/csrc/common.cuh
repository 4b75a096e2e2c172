// Shared device helpers for the SS2D kernels (sm_100a).
#pragma once
#include <cstdlib>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/ss2d_b200.h"

namespace ss2d {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// ---- element <-> float ---------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// ---- VEC consecutive elements <-> float[VEC], one memory transaction when possible -----
// The address must be aligned to VEC * sizeof(T) bytes (callers pick VEC accordingly).
// `Raw` keeps the loaded bits packed so that a prefetched vector costs few registers.
template <typename T> struct Half2Of;
template <> struct Half2Of<__nv_bfloat16> {
    static __device__ __forceinline__ float2 unpack(uint32_t w) {
        // bf16 -> fp32 is a 16-bit shift: exact
        return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
    }
    static __device__ __forceinline__ uint32_t pack(float a, float b) {
        __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&t);
    }
};
template <> struct Half2Of<__half> {
    static __device__ __forceinline__ float2 unpack(uint32_t w) {
        return __half22float2(*reinterpret_cast<const __half2*>(&w));
    }
    static __device__ __forceinline__ uint32_t pack(float a, float b) {
        __half2 t = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&t);
    }
};

template <typename T, int VEC> struct Vec {
    static constexpr int kBytes = VEC * (int)sizeof(T);
    static constexpr int kWords = (kBytes + 3) / 4;
    struct Raw { uint32_t w[kWords]; };

    template <bool kReadOnly = true>
    static __device__ __forceinline__ Raw load_raw(const T* p) {
        Raw r;
        if constexpr (kBytes % 16 == 0) {
#pragma unroll
            for (int i = 0; i < kBytes / 16; ++i) {
                const uint4* q = reinterpret_cast<const uint4*>(p) + i;
                const uint4 t = kReadOnly ? __ldg(q) : *q;
                r.w[4 * i] = t.x; r.w[4 * i + 1] = t.y; r.w[4 * i + 2] = t.z; r.w[4 * i + 3] = t.w;
            }
        } else if constexpr (kBytes == 8) {
            const uint2* q = reinterpret_cast<const uint2*>(p);
            const uint2 t = kReadOnly ? __ldg(q) : *q;
            r.w[0] = t.x; r.w[1] = t.y;
        } else if constexpr (kBytes == 4) {
            const uint32_t* q = reinterpret_cast<const uint32_t*>(p);
            r.w[0] = kReadOnly ? __ldg(q) : *q;
        } else {
            static_assert(kBytes == 2, "unsupported vector width");
            const uint16_t* q = reinterpret_cast<const uint16_t*>(p);
            r.w[0] = kReadOnly ? __ldg(q) : *q;
        }
        return r;
    }
    static __device__ __forceinline__ void store_raw(T* p, const Raw& r) {
        if constexpr (kBytes % 16 == 0) {
#pragma unroll
            for (int i = 0; i < kBytes / 16; ++i)
                reinterpret_cast<uint4*>(p)[i] = make_uint4(r.w[4 * i], r.w[4 * i + 1], r.w[4 * i + 2], r.w[4 * i + 3]);
        } else if constexpr (kBytes == 8) {
            *reinterpret_cast<uint2*>(p) = make_uint2(r.w[0], r.w[1]);
        } else if constexpr (kBytes == 4) {
            *reinterpret_cast<uint32_t*>(p) = r.w[0];
        } else {
            *reinterpret_cast<uint16_t*>(p) = (uint16_t)r.w[0];
        }
    }
    static __device__ __forceinline__ void unpack(const Raw& r, float (&v)[VEC]) {
        if constexpr (sizeof(T) == 4) {
#pragma unroll
            for (int i = 0; i < VEC; ++i) v[i] = __uint_as_float(r.w[i]);
        } else if constexpr (VEC == 1) {
            v[0] = Half2Of<T>::unpack(r.w[0]).x;
        } else {
#pragma unroll
            for (int i = 0; i < VEC / 2; ++i) {
                const float2 f = Half2Of<T>::unpack(r.w[i]);
                v[2 * i] = f.x; v[2 * i + 1] = f.y;
            }
        }
    }
    static __device__ __forceinline__ void load(const T* p, float (&v)[VEC]) { unpack(load_raw(p), v); }
    // for shared memory (or global data written earlier in the same kernel): no read-only path
    static __device__ __forceinline__ void load_plain(const T* p, float (&v)[VEC]) { unpack(load_raw<false>(p), v); }
    static __device__ __forceinline__ void store(T* p, const float (&v)[VEC]) {
        Raw r;
        if constexpr (sizeof(T) == 4) {
#pragma unroll
            for (int i = 0; i < VEC; ++i) r.w[i] = __float_as_uint(v[i]);
        } else if constexpr (VEC == 1) {
            r.w[0] = Half2Of<T>::pack(v[0], 0.f);
        } else {
#pragma unroll
            for (int i = 0; i < VEC / 2; ++i) r.w[i] = Half2Of<T>::pack(v[2 * i], v[2 * i + 1]);
        }
        if constexpr (kBytes % 16 == 0) {
#pragma unroll
            for (int i = 0; i < kBytes / 16; ++i)
                reinterpret_cast<uint4*>(p)[i] = make_uint4(r.w[4 * i], r.w[4 * i + 1], r.w[4 * i + 2], r.w[4 * i + 3]);
        } else if constexpr (kBytes == 8) {
            *reinterpret_cast<uint2*>(p) = make_uint2(r.w[0], r.w[1]);
        } else if constexpr (kBytes == 4) {
            *reinterpret_cast<uint32_t*>(p) = r.w[0];
        } else {
            *reinterpret_cast<uint16_t*>(p) = (uint16_t)r.w[0];
        }
    }
};

// ---- arithmetic of the recurrence -------------------------------------------------------
// softplus with torch's threshold (x > 20 -> x).  exp via ex2.approx; log1p(e) through
// lg2.approx except for small e, where lg2(1+e) would lose the low bits of e and a short
// alternating series is exact to fp32 rounding (e < 2^-6: |error| < e^4/4 < 1.5e-8 * e).
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float lg2_approx(float x) {
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float softplus_fast(float x) {
    const float e = ex2_approx(x * kLog2e);
    const float series = e * fmaf(e, fmaf(e, 0.33333334f, -0.5f), 1.0f);
    const float full = lg2_approx(1.0f + e) * kLn2;
    const float sp = (e < 0.015625f) ? series : full;
    return (x > 20.0f) ? x : sp;
}

// softplus(x) and its derivative sigmoid(x) = e^x / (1 + e^x) from one exponential (threshold 20 as torch:
// above it softplus is x and the derivative 1)
__device__ __forceinline__ void softplus_and_grad(float x, float& sp, float& dsp) {
    const float e = ex2_approx(x * kLog2e);
    const float w = 1.0f + e;
    const float series = e * fmaf(e, fmaf(e, 0.33333334f, -0.5f), 1.0f);
    const float full = lg2_approx(w) * kLn2;
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(w));
    const bool big = x > 20.0f;
    sp = big ? x : ((e < 0.015625f) ? series : full);
    dsp = big ? 1.0f : e * r;
}

// decay exp(dl * A) with A pre-multiplied by log2(e)
__device__ __forceinline__ float decay_fast(float dl, float A_log2e) { return ex2_approx(dl * A_log2e); }

// The recurrence h <- a*h + b composes as (a1,b1) o (a0,b0) = (a1*a0, a1*b0 + b1).
struct AB { float a, b; };
__device__ __forceinline__ AB combine(AB first, AB then) {
    return AB{then.a * first.a, fmaf(then.a, first.b, then.b)};
}

// Inclusive scan of (a, b) across the 32 lanes of a warp, lane 0 first.
__device__ __forceinline__ AB warp_scan_inclusive(AB v, int lane) {
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const float pa = __shfl_up_sync(0xffffffffu, v.a, off);
        const float pb = __shfl_up_sync(0xffffffffu, v.b, off);
        if (lane >= off) { v.b = fmaf(v.a, pb, v.b); v.a *= pa; }
    }
    return v;
}
// Same with lane 31 first (suffix scan): result at lane i covers lanes 31..i.
__device__ __forceinline__ AB warp_scan_inclusive_rev(AB v, int lane) {
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const float pa = __shfl_down_sync(0xffffffffu, v.a, off);
        const float pb = __shfl_down_sync(0xffffffffu, v.b, off);
        if (lane + off < 32) { v.b = fmaf(v.a, pb, v.b); v.a *= pa; }
    }
    return v;
}

// ---- warp-level tensor-core step: D (16 x 8, fp32) += A (16 x 16, row-major) . B (16 x 8, column-major) -------
template <typename T> struct MmaK16;
template <> struct MmaK16<__nv_bfloat16> {
    static __device__ __forceinline__ void run(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
    }
};
template <> struct MmaK16<__half> {
    static __device__ __forceinline__ void run(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
    }
};

// ---- host-side helpers ---------------------------------------------------------------------
inline size_t dtype_size(int dt) { return dt == SS2D_F32 ? 4 : 2; }
inline bool dtype_ok(int dt) { return dt == SS2D_F32 || dt == SS2D_F16 || dt == SS2D_BF16; }
inline bool aligned_to(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

void count_launch(int n = 1);
int check_launch();   // cudaPeekAtLastError -> SS2D_OK / SS2D_ECUDA

// SS2D_SCAN_ROWS=0 keeps the selective-scan operators on their warp-per-row kernels (a switch for comparisons)
inline bool rows_kernels_enabled() {
    static const bool on = [] { const char* e = getenv("SS2D_SCAN_ROWS"); return !(e && e[0] == '0'); }();
    return on;
}

}  // namespace ss2d
