// Elementwise producers around the SS2D core, channel-first maps, each one pass over HBM:
//   bias_act      y = act(x + bias[d])                       (fc1 bias + GELU of the MLP, in place)
//   dwconv3x3_act y = act(depthwise 3x3 conv of x, pad 1)    (the conv + SiLU in front of the core)
// Rounding follows the chain of separate kernels these replace: the convolution / bias sum is
// formed in fp32, rounded to the storage type, then the activation is evaluated in fp32 on that
// rounded value and rounded again.
#include "common.cuh"

namespace ss2d {

enum { ACT_NONE = 0, ACT_GELU = 1, ACT_SILU = 2 };

template <typename T> __device__ __forceinline__ float round_to(float v) { return to_f<T>(from_f<T>(v)); }

template <int ACT> __device__ __forceinline__ float act_f(float v) {
    if constexpr (ACT == ACT_GELU) return 0.5f * v * (1.0f + erff(v * 0.70710678118654752f));   // exact (erf) GELU
    else if constexpr (ACT == ACT_SILU) return __fdividef(v, 1.0f + ex2_approx(-v * kLog2e));
    else return v;
}

// ------------------------------------------------------------------------------------------------
struct BiasActArgs {
    const void* x;
    const float* bias;
    void* y;
    long long items;     // B * D * (L / PV)
    int D, nv;           // nv = L / PV vectors per row
    int rows_per_channel;   // 1 for (B, D, ...) maps (channel = row % D); B for (D, B, ...) maps (channel = row / B)
};

template <typename T, int PV, int ACT>
__global__ void __launch_bounds__(256) bias_act_kernel(const BiasActArgs a) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long it = (long long)blockIdx.x * blockDim.x + threadIdx.x; it < a.items; it += stride) {
        const long long row = it / a.nv;
        const int d = (int)((row / a.rows_per_channel) % a.D);
        const float b = a.bias ? __ldg(a.bias + d) : 0.f;
        float v[PV];
        Vec<T, PV>::load_plain((const T*)a.x + it * PV, v);      // x may be y: no read-only path
#pragma unroll
        for (int i = 0; i < PV; ++i) v[i] = act_f<ACT>(round_to<T>(v[i] + b));
        Vec<T, PV>::store((T*)a.y + it * PV, v);
    }
}

template <typename T, int PV>
static void launch_bias_act(const BiasActArgs& a, int act, cudaStream_t st) {
    long long ctas = (a.items + 255) / 256;
    const long long cap = 148LL * 8 * 4;          // a few waves of resident CTAs, grid-stride beyond
    if (ctas > cap) ctas = cap;
    const unsigned g = (unsigned)ctas;
    if (act == ACT_GELU) bias_act_kernel<T, PV, ACT_GELU><<<g, 256, 0, st>>>(a);
    else if (act == ACT_SILU) bias_act_kernel<T, PV, ACT_SILU><<<g, 256, 0, st>>>(a);
    else bias_act_kernel<T, PV, ACT_NONE><<<g, 256, 0, st>>>(a);
}

template <typename T>
static void launch_bias_act_v(BiasActArgs a, int pv, long long rows, long long L, int act, cudaStream_t st) {
    a.nv = (int)(L / pv);
    a.items = rows * a.nv;
    if (pv == 8) launch_bias_act<T, 8>(a, act, st);
    else if (pv == 4) launch_bias_act<T, 4>(a, act, st);
    else if (pv == 2) launch_bias_act<T, 2>(a, act, st);
    else launch_bias_act<T, 1>(a, act, st);
}

int bias_act(const ss2d_pointwise_params* p, cudaStream_t st) {
    if (!p) return SS2D_EINVAL_NULL;
    if (!p->x || !p->y) return SS2D_EINVAL_NULL;
    if (!dtype_ok(p->dtype)) return SS2D_EINVAL_DTYPE;
    if (p->act < 0 || p->act > 2) return SS2D_ENOTSUP;
    if (p->B <= 0 || p->D <= 0 || p->H <= 0 || p->W <= 0) return SS2D_EINVAL_SHAPE;
    const size_t s = dtype_size(p->dtype);
    if (!aligned_to(p->x, s) || !aligned_to(p->y, s) || !aligned_to(p->bias, 4)) return SS2D_EINVAL_ALIGN;
    const long long L = p->H * p->W;
    int pv = (s == 2) ? 8 : 4;
    auto fit = [&](long long x) { while (pv > 1 && (x % pv) != 0) pv >>= 1; };
    fit(L);
    fit((long long)(reinterpret_cast<uintptr_t>(p->x) / s));
    fit((long long)(reinterpret_cast<uintptr_t>(p->y) / s));
    BiasActArgs a;
    a.x = p->x; a.bias = (const float*)p->bias; a.y = p->y; a.D = (int)p->D; a.nv = 0; a.items = 0;
    a.rows_per_channel = p->channel_major ? (int)p->B : 1;
    const long long rows = p->B * p->D;
    if (p->dtype == SS2D_F32) launch_bias_act_v<float>(a, pv, rows, L, p->act, st);
    else if (p->dtype == SS2D_BF16) launch_bias_act_v<__nv_bfloat16>(a, pv, rows, L, p->act, st);
    else launch_bias_act_v<__half>(a, pv, rows, L, p->act, st);
    count_launch();
    return check_launch();
}

// ------------------------------------------------------------------------------------------------
// Depthwise 3x3, stride 1, zero padding 1.  A CTA owns PP whole planes: each is staged once in
// shared memory as fp32 inside a one-pixel zero frame (pitch W + 2), then every thread produces
// runs of PV consecutive output pixels of one row from three shared rows.  HBM traffic is the
// minimum: every input element read once, every output written once.
struct DwArgs {
    const void* x;
    const void* w;       // (D, 3, 3) storage type
    const float* bias;   // (D) or null
    void* y;
    int D, H, W, PP, planes, nvw;   // nvw = W / PV runs per row
    int planes_per_channel;         // 1 for (B, D, H, W) maps, B for (D, B, H, W) maps
};

template <typename T, int PV, int ACT>
__global__ void __launch_bounds__(256) dwconv3x3_act_kernel(const DwArgs a) {
    extern __shared__ __align__(16) float sm[];
    const int H = a.H, W = a.W, Wp = W + 2, L = H * W;
    const int plane0 = blockIdx.x * a.PP;
    const int np = min(a.PP, a.planes - plane0);
    const int frame = (H + 2) * Wp;
    // zero the frames, then drop the planes in
    for (int i = threadIdx.x; i < np * frame; i += blockDim.x) sm[i] = 0.f;
    __syncthreads();
    const T* __restrict__ x = (const T*)a.x + (long long)plane0 * L;
    const int nvec = L / PV;
    for (int i = threadIdx.x; i < np * nvec; i += blockDim.x) {
        const int pl = i / nvec, e = (i - pl * nvec) * PV;
        float v[PV];
        Vec<T, PV>::load(x + (long long)pl * L + e, v);
        const int h = e / W, w0 = e - h * W;        // PV divides W: a run never leaves its row
        float* dst = sm + pl * frame + (h + 1) * Wp + w0 + 1;
#pragma unroll
        for (int j = 0; j < PV; ++j) dst[j] = v[j];
    }
    __syncthreads();
    // compute: consecutive threads take consecutive columns w (conflict-free shared reads, 64-byte
    // store runs per warp) and walk kRows rows with the 3x3 window sliding in registers
    constexpr int kRows = 8;
    const int nrb = (H + kRows - 1) / kRows;
    T* __restrict__ y = (T*)a.y + (long long)plane0 * L;
    for (int i = threadIdx.x; i < np * nrb * W; i += blockDim.x) {
        const int w = i % W, t = i / W;
        const int rb = t % nrb, pl = t / nrb;
        const int h0 = rb * kRows, h1 = min(h0 + kRows, H);
        const int d = ((plane0 + pl) / a.planes_per_channel) % a.D;
        const T* __restrict__ wk = (const T*)a.w + d * 9;
        float k[9];
#pragma unroll
        for (int j = 0; j < 9; ++j) k[j] = to_f<T>(wk[j]);
        const float b = a.bias ? __ldg(a.bias + d) : 0.f;
        const float* src = sm + pl * frame + h0 * Wp + w;    // frame row h0 is image row h0 - 1
        float t0 = src[0], t1 = src[1], t2 = src[2];
        float m0 = src[Wp], m1 = src[Wp + 1], m2 = src[Wp + 2];
        T* __restrict__ out = y + (long long)pl * L + w;
        for (int h = h0; h < h1; ++h) {
            const float* bp = src + (h - h0 + 2) * Wp;
            const float b0 = bp[0], b1 = bp[1], b2 = bp[2];
            float acc = b;
            acc = fmaf(k[0], t0, acc); acc = fmaf(k[1], t1, acc); acc = fmaf(k[2], t2, acc);
            acc = fmaf(k[3], m0, acc); acc = fmaf(k[4], m1, acc); acc = fmaf(k[5], m2, acc);
            acc = fmaf(k[6], b0, acc); acc = fmaf(k[7], b1, acc); acc = fmaf(k[8], b2, acc);
            out[h * W] = from_f<T>(act_f<ACT>(round_to<T>(acc)));
            t0 = m0; t1 = m1; t2 = m2; m0 = b0; m1 = b1; m2 = b2;
        }
    }
}

template <typename T, int PV>
static int launch_dw(const DwArgs& a, int act, size_t smem, unsigned grid, cudaStream_t st) {
    if (act == ACT_SILU) {
        auto k = dwconv3x3_act_kernel<T, PV, ACT_SILU>;
        if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return SS2D_ECUDA;
        k<<<grid, 256, smem, st>>>(a);
    } else if (act == ACT_GELU) {
        auto k = dwconv3x3_act_kernel<T, PV, ACT_GELU>;
        if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return SS2D_ECUDA;
        k<<<grid, 256, smem, st>>>(a);
    } else {
        auto k = dwconv3x3_act_kernel<T, PV, ACT_NONE>;
        if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return SS2D_ECUDA;
        k<<<grid, 256, smem, st>>>(a);
    }
    count_launch();
    return check_launch();
}

template <typename T>
static int launch_dw_v(DwArgs a, int pv, int act, size_t smem, unsigned grid, cudaStream_t st) {
    a.nvw = a.W / pv;
    if (pv == 8) return launch_dw<T, 8>(a, act, smem, grid, st);
    if (pv == 4) return launch_dw<T, 4>(a, act, smem, grid, st);
    if (pv == 2) return launch_dw<T, 2>(a, act, smem, grid, st);
    return launch_dw<T, 1>(a, act, smem, grid, st);
}

int dwconv3x3_act(const ss2d_pointwise_params* p, cudaStream_t st) {
    if (!p) return SS2D_EINVAL_NULL;
    if (!p->x || !p->y || !p->weight) return SS2D_EINVAL_NULL;
    if (p->x == p->y) return SS2D_ENOTSUP;       // neighbours are read: not an in-place operation
    if (!dtype_ok(p->dtype)) return SS2D_EINVAL_DTYPE;
    if (p->act < 0 || p->act > 2) return SS2D_ENOTSUP;
    if (p->B <= 0 || p->D <= 0 || p->H <= 0 || p->W <= 0) return SS2D_EINVAL_SHAPE;
    if (p->B * p->D > 0x7fffffffLL || p->H * p->W > 0x3fffffffLL) return SS2D_EINVAL_SHAPE;
    const size_t s = dtype_size(p->dtype);
    if (!aligned_to(p->x, s) || !aligned_to(p->y, s) || !aligned_to(p->weight, s) || !aligned_to(p->bias, 4)) return SS2D_EINVAL_ALIGN;
    const long long L = p->H * p->W;
    int pv = (s == 2) ? 8 : 4;
    auto fit = [&](long long x) { while (pv > 1 && (x % pv) != 0) pv >>= 1; };
    fit(p->W); fit(L);
    fit((long long)(reinterpret_cast<uintptr_t>(p->x) / s));
    fit((long long)(reinterpret_cast<uintptr_t>(p->y) / s));
    const size_t frame = (size_t)(p->H + 2) * (p->W + 2) * sizeof(float);
    if (frame > 200 * 1024) return SS2D_ENOTSUP;     // plane too large for one CTA's shared memory
    // planes per CTA: about 2048 outputs per thread block pass, at most 48 KB of shared memory
    long long PP = (2048 * 4 + L - 1) / L;
    if (PP < 1) PP = 1;
    while (PP > 1 && PP * frame > 48 * 1024) --PP;
    const long long planes = p->B * p->D;
    if (PP > planes) PP = planes;
    DwArgs a;
    a.x = p->x; a.w = p->weight; a.bias = (const float*)p->bias; a.y = p->y;
    a.D = (int)p->D; a.H = (int)p->H; a.W = (int)p->W; a.PP = (int)PP; a.planes = (int)planes; a.nvw = 0;
    a.planes_per_channel = p->channel_major ? (int)p->B : 1;
    const unsigned grid = (unsigned)((planes + PP - 1) / PP);
    const size_t smem = (size_t)PP * frame;
    if (p->dtype == SS2D_F32) return launch_dw_v<float>(a, pv, p->act, smem, grid, st);
    if (p->dtype == SS2D_BF16) return launch_dw_v<__nv_bfloat16>(a, pv, p->act, smem, grid, st);
    return launch_dw_v<__half>(a, pv, p->act, smem, grid, st);
}

}  // namespace ss2d
