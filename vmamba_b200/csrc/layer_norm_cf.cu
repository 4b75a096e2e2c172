// LayerNorm over the channel axis of a channel-first map (B, D, L), fp32 statistics.
//
// A CTA owns 32 consecutive pixels of one image: threadIdx.x runs along the pixels (every global
// access is a full 128-byte line per channel), threadIdx.y splits the D channels.  Mean and
// variance are the two-pass kind (sum of squared deviations), as the torch operator this replaces.
// Values are kept in registers between the passes when D / NTY fits the cache, else re-read
// (second and third reads come from L1/L2).  Optionally sums n_terms input maps on the way in.
#include "common.cuh"

namespace ss2d {

struct NormArgs {
    const float* in;
    const float *w, *b;
    void* out;
    long long B, D, L, term_stride;
    int n_terms;
    float eps;
};

template <typename Tout, int NTY, int CACHE>
__global__ void __launch_bounds__(32 * NTY) layer_norm_cf_kernel(const NormArgs a) {
    __shared__ float red[NTY][33];
    const int tx = threadIdx.x, ty = threadIdx.y;
    const long long tiles = (a.L + 31) / 32;
    const long long bimg = blockIdx.x / tiles, p = (blockIdx.x % tiles) * 32 + tx;
    const bool in = p < a.L;
    const float* __restrict__ src = a.in + bimg * a.D * a.L + p;
    const int D = (int)a.D;

    auto fetch = [&](int d) -> float {
        float v = 0.f;
        if (in) {
            const float* q = src + (long long)d * a.L;
            v = q[0];
            for (int t = 1; t < a.n_terms; ++t) v += q[t * a.term_stride];
        }
        return v;
    };
    auto reduce_over_ty = [&](float v) -> float {
        red[ty][tx] = v;
        __syncthreads();
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < NTY; ++j) s += red[j][tx];
        __syncthreads();
        return s;
    };

    float cache[CACHE > 0 ? CACHE : 1];
    float s = 0.f;
    if constexpr (CACHE > 0) {
#pragma unroll
        for (int i = 0; i < CACHE; ++i) {
            const int d = ty + i * NTY;
            cache[i] = (d < D) ? fetch(d) : 0.f;
            s += cache[i];
        }
    } else {
        for (int d = ty; d < D; d += NTY) s += fetch(d);
    }
    const float mean = reduce_over_ty(s) / (float)D;
    float q = 0.f;
    if constexpr (CACHE > 0) {
#pragma unroll
        for (int i = 0; i < CACHE; ++i) {
            const int d = ty + i * NTY;
            const float t = cache[i] - mean;
            if (d < D) q = fmaf(t, t, q);
        }
    } else {
        for (int d = ty; d < D; d += NTY) { const float t = fetch(d) - mean; q = fmaf(t, t, q); }
    }
    const float rstd = rsqrtf(reduce_over_ty(q) / (float)D + a.eps);
    if (!in) return;
    Tout* __restrict__ dst = (Tout*)a.out + bimg * a.D * a.L + p;
    auto emit = [&](int d, float v) {
        float t = (v - mean) * rstd;
        if (a.w) t *= __ldg(a.w + d);
        if (a.b) t += __ldg(a.b + d);
        dst[(long long)d * a.L] = from_f<Tout>(t);
    };
    if constexpr (CACHE > 0) {
#pragma unroll
        for (int i = 0; i < CACHE; ++i) {
            const int d = ty + i * NTY;
            if (d < D) emit(d, cache[i]);
        }
    } else {
        for (int d = ty; d < D; d += NTY) emit(d, fetch(d));
    }
}

template <typename Tout>
static void launch_norm(const NormArgs& a, cudaStream_t st) {
    const long long ctas = a.B * ((a.L + 31) / 32);
    const unsigned g = (unsigned)ctas;
    if (a.D <= 8 * 12) layer_norm_cf_kernel<Tout, 8, 12><<<g, dim3(32, 8), 0, st>>>(a);
    else if (a.D <= 8 * 24) layer_norm_cf_kernel<Tout, 8, 24><<<g, dim3(32, 8), 0, st>>>(a);
    else if (a.D <= 16 * 24) layer_norm_cf_kernel<Tout, 16, 24><<<g, dim3(32, 16), 0, st>>>(a);
    else if (a.D <= 32 * 24) layer_norm_cf_kernel<Tout, 32, 24><<<g, dim3(32, 32), 0, st>>>(a);
    else layer_norm_cf_kernel<Tout, 32, 0><<<g, dim3(32, 32), 0, st>>>(a);
}

int layer_norm_cf(const ss2d_norm_params* p, cudaStream_t st) {
    if (!p) return SS2D_EINVAL_NULL;
    if (!p->in || !p->out) return SS2D_EINVAL_NULL;
    if (!dtype_ok(p->out_dtype)) return SS2D_EINVAL_DTYPE;
    if (p->B <= 0 || p->D <= 0 || p->L <= 0 || p->n_terms < 1 || p->n_terms > 8) return SS2D_EINVAL_SHAPE;
    if (!aligned_to(p->in, 4) || !aligned_to(p->out, dtype_size(p->out_dtype)) || !aligned_to(p->weight, 4) ||
        !aligned_to(p->bias, 4))
        return SS2D_EINVAL_ALIGN;
    if (p->B * ((p->L + 31) / 32) > 0x7fffffffLL || p->D > 0x7fffffffLL) return SS2D_EINVAL_SHAPE;
    NormArgs a;
    a.in = (const float*)p->in; a.w = (const float*)p->weight; a.b = (const float*)p->bias; a.out = p->out;
    a.B = p->B; a.D = p->D; a.L = p->L; a.term_stride = p->B * p->D * p->L;
    a.n_terms = p->n_terms; a.eps = p->eps;
    if (p->out_dtype == SS2D_F32) launch_norm<float>(a, st);
    else if (p->out_dtype == SS2D_BF16) launch_norm<__nv_bfloat16>(a, st);
    else launch_norm<__half>(a, st);
    count_launch();
    return check_launch();
}

}  // namespace ss2d
