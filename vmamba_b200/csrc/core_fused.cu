// Fused SS2D core for scans mode 0, d_state 1: CrossScan folded into the loads, the four-route
// selective scan, and CrossMerge, one CTA pass per group of (image, channel) planes.
//
// Data layout: x is (B, D, H, W); the raw step sizes delta_k and B_k / C_k of route k are stored
// in the ORIENTATION order of the route (row-major for k = 0, 2; column-major for k = 1, 3), so
// every global access of this kernel is a contiguous, 16-byte vectorised stream.  The reversed
// routes 2 and 3 are never materialised: they are the same data scanned from the other end.
//
// Mapping: a plane of L = H*W elements is owned by G = L / VEC consecutive threads, thread v
// holding elements [v*VEC, (v+1)*VEC) of the orientation order in registers.  A CTA handles PP
// planes of one image side by side (PP*G threads).  Per orientation the forward route and the
// backward route are evaluated on the same registers: each thread runs the recurrence over its
// VEC elements in both directions, the thread aggregates (a, b) are combined by one CTA-wide
// scan per direction (warp shuffle scan, then a scan of the warp totals), plane boundaries being
// expressed as a = 0 on the first (last) thread of a plane.  The column-major orientation needs
// x transposed and gives its result transposed: both go through a padded fp32 plane in shared
// memory, which is also where the four routes are summed.  No atomics; output is the merged fp32
// map (B, D, H, W), consumed by the LayerNorm kernel.
//
// HBM traffic per (pixel, channel): x once, four delta values, one fp32 result; B_k/C_k are shared
// by all channels of an image and stay in L1/L2.
#include <mutex>

#include "common.cuh"

namespace ss2d {

struct CoreArgs {
    const void* x;
    const void* delta[4];
    const float* Bm[4];
    const float* Cm[4];
    const float *A, *Dskip, *bias;
    float* merged;
    long long d_bs[4], bc_bs[4];
    int B, D, H, W, L, G, PP, Wp, groups_per_image;
    unsigned magic_G, magic_W, magic_H;   // ceil(2^32 / d): n / d == umulhi(n, magic) for n * d < 2^32
};

struct ScanScratch {
    AB wtot[2][32];
    float wpre[2][32];
};

__device__ __forceinline__ int fast_div(int n, unsigned magic) { return magic ? (int)__umulhi((unsigned)n, magic) : n; }   // magic 0: divisor 1

// CTA-wide scan of per-thread aggregates in thread order (forward) and in reverse thread order
// (backward).  The state before the first thread is zero, so only the state entering each thread
// is needed: hin_f for the forward route, hin_b for the backward route.
__device__ __forceinline__ void cta_scan_pair(AB f, AB bk, int lane, int warp, int nwarps, ScanScratch& s,
                                              float& hin_f, float& hin_b) {
    const AB inc_f = warp_scan_inclusive(f, lane);
    const AB inc_b = warp_scan_inclusive_rev(bk, lane);
    if (lane == 31) s.wtot[0][warp] = inc_f;
    if (lane == 0) s.wtot[1][warp] = inc_b;
    __syncthreads();
    if (warp == 0) {
        const AB t = (lane < nwarps) ? s.wtot[0][lane] : AB{1.f, 0.f};
        const AB sc = warp_scan_inclusive(t, lane);
        float e = __shfl_up_sync(0xffffffffu, sc.b, 1);
        if (lane == 0) e = 0.f;
        s.wpre[0][lane] = e;
    }
    if (warp == (nwarps > 1 ? 1 : 0)) {
        const AB t = (lane < nwarps) ? s.wtot[1][lane] : AB{1.f, 0.f};
        const AB sc = warp_scan_inclusive_rev(t, lane);
        float e = __shfl_down_sync(0xffffffffu, sc.b, 1);
        if (lane == 31) e = 0.f;
        s.wpre[1][lane] = e;
    }
    __syncthreads();
    float ea = __shfl_up_sync(0xffffffffu, inc_f.a, 1), eb = __shfl_up_sync(0xffffffffu, inc_f.b, 1);
    if (lane == 0) { ea = 1.f; eb = 0.f; }
    hin_f = fmaf(ea, s.wpre[0][warp], eb);
    float ra = __shfl_down_sync(0xffffffffu, inc_b.a, 1), rb = __shfl_down_sync(0xffffffffu, inc_b.b, 1);
    if (lane == 31) { ra = 1.f; rb = 0.f; }
    hin_b = fmaf(ra, s.wpre[1][warp], rb);
}

// Per-row constants of one route, pre-scaled for the arithmetic below.
struct RouteConst {
    float A;        // A (negative): decay = 2^(A * log2(1 + e^x))
    float bias2;    // delta_bias * log2(e)
    float bias;     // delta_bias
};

// One direction of one route over the VEC register elements of a thread.
// `ul` holds u * ln2.  With t = log2(1 + e^x), x = delta + bias:  softplus(x) = ln2 * t  and
// exp(softplus(x) * A) = 2^(A t), so one ex2 and one lg2 serve both the step size and the decay.
// Adds C*h_local to ysum, leaves C*prod(a) in cP, returns the thread aggregate.
// kPrecise (fp32 tensors): softplus keeps torch's threshold and a series for small e^x, so that
// the result is accurate to fp32 rounding; otherwise (16-bit tensors, whose own rounding is four
// orders of magnitude coarser) the shortest instruction sequence is used.
template <int VEC, bool kForward, bool kPrecise>
__device__ __forceinline__ AB route_local(const float (&ul)[VEC], const float (&dv)[VEC], const float (&bv)[VEC],
                                          const float (&cv)[VEC], const RouteConst rc, float (&cP)[VEC],
                                          float (&ysum)[VEC]) {
    float p = 1.f, h = 0.f;
#pragma unroll
    for (int ii = 0; ii < VEC; ++ii) {
        const int i = kForward ? ii : VEC - 1 - ii;
        float t, aa;
        if constexpr (kPrecise) {
            const float dl = softplus_fast(dv[i] + rc.bias);
            t = dl * kLog2e;
            aa = ex2_approx(t * rc.A);
        } else {
            // clamp keeps e^x finite; above x = 87 the reference returns x itself
            const float e = ex2_approx(fminf(fmaf(dv[i], kLog2e, rc.bias2), 126.f));
            t = lg2_approx(1.0f + e);
            aa = ex2_approx(t * rc.A);
        }
        h = fmaf(aa, h, t * (bv[i] * ul[i]));
        p *= aa;
        cP[i] = cv[i] * p;
        ysum[i] = fmaf(cv[i], h, ysum[i]);
    }
    return AB{p, h};
}

// Shared-memory word of element i of a VEC-segment that starts at (major0, minor0) of a plane
// walked with `minor` fastest (length n_minor), stored with `minor_stride` / `major_stride`.
// A segment covers at most two lines because VEC <= n_minor.
template <int VEC>
struct SegAddr {
    int a0, n1, jump;
    __device__ __forceinline__ SegAddr(int major0, int minor0, int n_minor, int major_stride, int minor_stride) {
        a0 = major0 * major_stride + minor0 * minor_stride;
        n1 = n_minor - minor0;                                   // elements left in the first line
        jump = major_stride - n_minor * minor_stride;            // extra offset once the line wraps
    }
    __device__ __forceinline__ int at(int i, int minor_stride) const { return a0 + i * minor_stride + (i >= n1 ? jump : 0); }
};

template <typename T, int VEC, int MAXT, int MINB>
__global__ void __launch_bounds__(MAXT, MINB) core_plane_kernel(const CoreArgs a) {
    extern __shared__ __align__(16) float smem[];
    __shared__ ScanScratch scr;
    constexpr bool kPrecise = sizeof(T) == 4;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5, nwarps = (blockDim.x + 31) >> 5;
    const int b = blockIdx.x / a.groups_per_image;
    const int d0 = (blockIdx.x - b * a.groups_per_image) * a.PP;
    const int pp_here = min(a.PP, a.D - d0);
    const int pl = fast_div(t, a.magic_G), v = t - pl * a.G;
    const bool active = pl < pp_here;
    const int d = d0 + pl;
    const int L = a.L, H = a.H, W = a.W, Wp = a.Wp, D = a.D;
    // one padded fp32 plane per channel: first x (for the transposed read), then, once every
    // column-orientation thread has taken its x values, the column-orientation result
    float* plane = smem + (size_t)pl * (H * Wp);
    using VT = Vec<T, VEC>;
    using VF = Vec<float, VEC>;
    const int e0 = v * VEC;   // first element of this thread in either orientation order
    const long long plane_off = (long long)d * L + e0;

    // ---- issue every HBM load of the pass up front: x and the four delta vectors -------------
    typename VT::Raw rx = {}, rd0 = {}, rd1 = {}, rd2 = {}, rd3 = {};
    if (active) {
        rx = VT::load_raw((const T*)a.x + (long long)b * D * L + plane_off);
        rd0 = VT::load_raw((const T*)a.delta[0] + b * a.d_bs[0] + plane_off);
        rd2 = VT::load_raw((const T*)a.delta[2] + b * a.d_bs[2] + plane_off);
        rd1 = VT::load_raw((const T*)a.delta[1] + b * a.d_bs[1] + plane_off);
        rd3 = VT::load_raw((const T*)a.delta[3] + b * a.d_bs[3] + plane_off);
    }
    float ul[VEC], yrow[VEC];
    VT::unpack(rx, ul);

    // ---- x into shared memory (row-major, padded pitch) -------------------------------------
    const int h0 = fast_div(e0, a.magic_W), w0 = e0 - h0 * W;
    const SegAddr<VEC> rs(h0, w0, W, Wp, 1);
    if (active) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) plane[rs.at(i, 1)] = ul[i];
    }
    const int wc = fast_div(e0, a.magic_H), hc = e0 - wc * H;
    const SegAddr<VEC> cs(wc, hc, H, 1, Wp);   // column-major walk: h is the fast index, stride Wp

    // ---- row orientation: routes 0 (forward) and 2 (backward) ---------------------------------
    {
        float dv[VEC], bv[VEC], cv[VEC], cPf[VEC], cPb[VEC];
        AB af{1.f, 0.f}, ab{1.f, 0.f};
        if (active) {
            const float Dsum = (__ldg(a.Dskip + d) + __ldg(a.Dskip + 2 * D + d));
#pragma unroll
            for (int i = 0; i < VEC; ++i) { yrow[i] = Dsum * ul[i]; ul[i] *= kLn2; }
            RouteConst rc;
            rc.A = __ldg(a.A + d); rc.bias = __ldg(a.bias + d); rc.bias2 = rc.bias * kLog2e;
            VT::unpack(rd0, dv);
            VF::load(a.Bm[0] + b * a.bc_bs[0] + e0, bv);
            VF::load(a.Cm[0] + b * a.bc_bs[0] + e0, cv);
            af = route_local<VEC, true, kPrecise>(ul, dv, bv, cv, rc, cPf, yrow);
            if (v == 0) af.a = 0.f;
            rc.A = __ldg(a.A + 2 * D + d); rc.bias = __ldg(a.bias + 2 * D + d); rc.bias2 = rc.bias * kLog2e;
            VT::unpack(rd2, dv);
            VF::load(a.Bm[2] + b * a.bc_bs[2] + e0, bv);
            VF::load(a.Cm[2] + b * a.bc_bs[2] + e0, cv);
            ab = route_local<VEC, false, kPrecise>(ul, dv, bv, cv, rc, cPb, yrow);
            if (v == a.G - 1) ab.a = 0.f;
        } else {
#pragma unroll
            for (int i = 0; i < VEC; ++i) { yrow[i] = 0.f; cPf[i] = 0.f; cPb[i] = 0.f; }
        }
        float hf, hb;
        cta_scan_pair(af, ab, lane, warp, nwarps, scr, hf, hb);   // its barriers also order the x stores before the reads below
        if (v == 0) hf = 0.f;
        if (v == a.G - 1) hb = 0.f;
#pragma unroll
        for (int i = 0; i < VEC; ++i) yrow[i] = fmaf(cPf[i], hf, fmaf(cPb[i], hb, yrow[i]));
    }

    // ---- column orientation: routes 1 (forward) and 3 (backward) -------------------------------
    {
        float dv[VEC], bv[VEC], cv[VEC], cPf[VEC], cPb[VEC], ycol[VEC];
        AB af{1.f, 0.f}, ab{1.f, 0.f};
        if (active) {
#pragma unroll
            for (int i = 0; i < VEC; ++i) ul[i] = plane[cs.at(i, Wp)];
            const float Dsum = (__ldg(a.Dskip + D + d) + __ldg(a.Dskip + 3 * D + d));
#pragma unroll
            for (int i = 0; i < VEC; ++i) { ycol[i] = Dsum * ul[i]; ul[i] *= kLn2; }
            RouteConst rc;
            rc.A = __ldg(a.A + D + d); rc.bias = __ldg(a.bias + D + d); rc.bias2 = rc.bias * kLog2e;
            VT::unpack(rd1, dv);
            VF::load(a.Bm[1] + b * a.bc_bs[1] + e0, bv);
            VF::load(a.Cm[1] + b * a.bc_bs[1] + e0, cv);
            af = route_local<VEC, true, kPrecise>(ul, dv, bv, cv, rc, cPf, ycol);
            if (v == 0) af.a = 0.f;
            rc.A = __ldg(a.A + 3 * D + d); rc.bias = __ldg(a.bias + 3 * D + d); rc.bias2 = rc.bias * kLog2e;
            VT::unpack(rd3, dv);
            VF::load(a.Bm[3] + b * a.bc_bs[3] + e0, bv);
            VF::load(a.Cm[3] + b * a.bc_bs[3] + e0, cv);
            ab = route_local<VEC, false, kPrecise>(ul, dv, bv, cv, rc, cPb, ycol);
            if (v == a.G - 1) ab.a = 0.f;
        } else {
#pragma unroll
            for (int i = 0; i < VEC; ++i) { ycol[i] = 0.f; cPf[i] = 0.f; cPb[i] = 0.f; }
        }
        float hf, hb;
        cta_scan_pair(af, ab, lane, warp, nwarps, scr, hf, hb);   // every x value has been read before these barriers
        if (v == 0) hf = 0.f;
        if (v == a.G - 1) hb = 0.f;
        if (active) {
#pragma unroll
            for (int i = 0; i < VEC; ++i) plane[cs.at(i, Wp)] = fmaf(cPf[i], hf, fmaf(cPb[i], hb, ycol[i]));
        }
    }
    __syncthreads();

    // ---- merge: row result (registers) + column result (transposed read), one vector store ------
    if (active) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) yrow[i] += plane[rs.at(i, 1)];
        VF::store(a.merged + (long long)b * D * L + plane_off, yrow);
    }
}

struct PlaneConfig { int vec, G, PP, threads, Wp; size_t smem; };

static bool plan_planes(const ss2d_core_params* p, PlaneConfig& c) {
    const long long L = p->H * p->W;
    const size_t s = dtype_size(p->act_dtype);
    auto el = [&](const void* q) { return (long long)(reinterpret_cast<uintptr_t>(q) / s); };
    int vec = 8;
    auto fit = [&](long long x) { if (x < 0) x = -x; while (vec > 1 && (x % vec) != 0) vec >>= 1; };
    fit(L); fit(el(p->x));
    for (int k = 0; k < 4; ++k) {
        fit(el(p->delta[k]));
        fit((long long)(reinterpret_cast<uintptr_t>(p->Bm[k]) / 4)); fit((long long)(reinterpret_cast<uintptr_t>(p->Cm[k]) / 4));
        fit(p->delta_batch_stride[k]); fit(p->bc_batch_stride[k]);
    }
    while (vec > 1 && (vec > p->H || vec > p->W)) vec >>= 1;   // a thread's segment spans at most two lines
    // 16-byte loads are enough: an 8-wide fp32 vector is two of them
    // (alignment of the fp32 workspace is checked by the caller)
    const long long G = L / vec;
    if (G > 1024) return false;
    int PP = (int)(448 / G);          // ~14 warps per CTA: two to three CTAs per SM
    if (PP < 1) PP = 1;
    if (PP > p->D) PP = (int)p->D;
    const int Wp = (int)(p->W | 1);   // odd pitch spreads the transposed accesses over banks
    size_t smem = (size_t)PP * p->H * Wp * sizeof(float);
    while (smem > 200 * 1024 && PP > 1) { --PP; smem = (size_t)PP * p->H * Wp * sizeof(float); }
    if (smem > 200 * 1024) return false;
    c.vec = vec; c.G = (int)G; c.PP = PP; c.Wp = Wp; c.smem = smem;
    c.threads = (int)((PP * G + 31) / 32 * 32);
    return true;
}

template <typename T, int VEC>
static int launch_core_t(const CoreArgs& a, const PlaneConfig& c, unsigned grid, cudaStream_t st) {
    cudaError_t e;
    if (c.threads <= 512) {
        auto kern = core_plane_kernel<T, VEC, 512, 2>;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)c.smem);
        if (e != cudaSuccess) return SS2D_ECUDA;
        kern<<<grid, c.threads, c.smem, st>>>(a);
    } else {
        auto kern = core_plane_kernel<T, VEC, 1024, 1>;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)c.smem);
        if (e != cudaSuccess) return SS2D_ECUDA;
        kern<<<grid, c.threads, c.smem, st>>>(a);
    }
    count_launch();
    return check_launch();
}

template <typename T>
static int launch_core_v(const CoreArgs& a, const PlaneConfig& c, unsigned grid, cudaStream_t st) {
    switch (c.vec) {
        case 8: return launch_core_t<T, 8>(a, c, grid, st);
        case 4: return launch_core_t<T, 4>(a, c, grid, st);
        case 2: return launch_core_t<T, 2>(a, c, grid, st);
        default: return launch_core_t<T, 1>(a, c, grid, st);
    }
}

int layer_norm_cf(const ss2d_norm_params* p, cudaStream_t st);

static int validate_core(const ss2d_core_params* p) {
    if (!p) return SS2D_EINVAL_NULL;
    if (!p->x || !p->A || !p->Dskip || !p->delta_bias || !p->y) return SS2D_EINVAL_NULL;
    for (int k = 0; k < 4; ++k)
        if (!p->delta[k] || !p->Bm[k] || !p->Cm[k]) return SS2D_EINVAL_NULL;
    if (!dtype_ok(p->act_dtype) || !dtype_ok(p->y_dtype)) return SS2D_EINVAL_DTYPE;
    if (p->y_dtype != SS2D_F32 && p->y_dtype != p->act_dtype) return SS2D_EINVAL_DTYPE;
    if (p->B <= 0 || p->D <= 0 || p->H <= 0 || p->W <= 0 || p->N <= 0) return SS2D_EINVAL_SHAPE;
    if (p->H * p->W > 0x3fffffffLL || p->B * p->D > 0x7fffffffLL) return SS2D_EINVAL_SHAPE;
    const long long L = p->H * p->W;
    for (int k = 0; k < 4; ++k) {
        if (p->B > 1 && (p->delta_batch_stride[k] < p->D * L || p->bc_batch_stride[k] < p->N * L)) return SS2D_EINVAL_STRIDE;
    }
    const size_t s = dtype_size(p->act_dtype);
    if (!aligned_to(p->x, s) || !aligned_to(p->y, dtype_size(p->y_dtype)) || !aligned_to(p->A, 4) ||
        !aligned_to(p->Dskip, 4) || !aligned_to(p->delta_bias, 4) || !aligned_to(p->ln_weight, 4) ||
        !aligned_to(p->ln_bias, 4))
        return SS2D_EINVAL_ALIGN;
    for (int k = 0; k < 4; ++k)
        if (!aligned_to(p->delta[k], s) || !aligned_to(p->Bm[k], 4) || !aligned_to(p->Cm[k], 4)) return SS2D_EINVAL_ALIGN;
    return SS2D_OK;
}

long long core_workspace_bytes(const ss2d_core_params* p) {
    if (validate_core(p) != SS2D_OK) return -1;
    // the fp32 merged map; not needed when the caller asks for it directly (no norm, fp32 output)
    if (!p->with_norm && p->y_dtype == SS2D_F32) return 0;
    return (long long)(p->B * p->D * p->H * p->W) * 4;
}

int core_fwd(const ss2d_core_params* p, cudaStream_t st) {
    const int rc = validate_core(p);
    if (rc != SS2D_OK) return rc;
    if (p->N != 1) return SS2D_ENOTSUP;          // d_state > 1 runs through the operator-surface kernels
    if (!p->with_norm && p->y_dtype != SS2D_F32) return SS2D_ENOTSUP;
    PlaneConfig c;
    if (!plan_planes(p, c)) return SS2D_ENOTSUP;  // plane too long for one CTA
    const long long need = core_workspace_bytes(p);
    float* merged = (float*)p->y;
    if (need > 0) {
        if (!p->workspace || p->workspace_bytes < need) return SS2D_EWORKSPACE;
        if (!aligned_to(p->workspace, 256)) return SS2D_EINVAL_ALIGN;
        merged = (float*)p->workspace;
    } else if (!aligned_to(p->y, 16)) {
        return SS2D_EINVAL_ALIGN;
    }
    CoreArgs a;
    a.x = p->x;
    for (int k = 0; k < 4; ++k) {
        a.delta[k] = p->delta[k]; a.Bm[k] = (const float*)p->Bm[k]; a.Cm[k] = (const float*)p->Cm[k];
        a.d_bs[k] = p->delta_batch_stride[k]; a.bc_bs[k] = p->bc_batch_stride[k];
    }
    a.A = (const float*)p->A; a.Dskip = (const float*)p->Dskip; a.bias = (const float*)p->delta_bias;
    a.merged = merged;
    a.B = (int)p->B; a.D = (int)p->D; a.H = (int)p->H; a.W = (int)p->W; a.L = (int)(p->H * p->W);
    a.G = c.G; a.PP = c.PP; a.Wp = c.Wp;
    auto magic = [](long long d) { return (unsigned)(((1ULL << 32) + (unsigned long long)d - 1) / (unsigned long long)d); };
    a.magic_G = c.G > 1 ? magic(c.G) : 0; a.magic_W = p->W > 1 ? magic(p->W) : 0; a.magic_H = p->H > 1 ? magic(p->H) : 0;
    a.groups_per_image = (int)((p->D + c.PP - 1) / c.PP);
    const long long grid = (long long)p->B * a.groups_per_image;
    if (grid > 0x7fffffffLL) return SS2D_EINVAL_SHAPE;
    int r;
    if (p->act_dtype == SS2D_F32) r = launch_core_v<float>(a, c, (unsigned)grid, st);
    else if (p->act_dtype == SS2D_BF16) r = launch_core_v<__nv_bfloat16>(a, c, (unsigned)grid, st);
    else r = launch_core_v<__half>(a, c, (unsigned)grid, st);
    if (r != SS2D_OK) return r;
    if (!p->with_norm) return SS2D_OK;
    ss2d_norm_params n;
    n.in = merged; n.weight = p->ln_weight; n.bias = p->ln_bias; n.out = p->y;
    n.B = p->B; n.D = p->D; n.L = p->H * p->W; n.n_terms = 1; n.out_dtype = p->y_dtype; n.eps = p->ln_eps;
    n.reserved0 = 0;
    return layer_norm_cf(&n, st);
}


// ------------------------------------------------------------------------------------------------
// Allocation-free variant of core_fwd.
//
// core_fwd needs the caller to bring one scratch buffer (the fp32 merged map that the scan+merge
// kernel hands to the LayerNorm kernel).  A caller that reaches this library through a bare FFI
// binding -- a custom-operator slot of a serving runtime that passes in only the input and output
// tensors it has already placed, a host program in a language without a CUDA allocator of its own,
// a process whose device memory was carved up once at start-up and is not allowed to grow -- has
// nowhere to get that buffer from.  For those callers the scratch lives in the array below, inside
// the library image: every GPU on which the library is loaded holds kStaticScratchBytes for the
// life of the process.
//
// Rules of use:
//  * capacity: B*D*H*W <= kStaticScratchFloats; larger problems are rejected with SS2D_ETOOBIG
//    before anything is launched;
//  * the first call on each device looks up the device address of the array (cudaGetSymbolAddress,
//    with that device current).  Make that first call outside any stream capture;
//  * all calls on one device share the one array and it keeps whatever the last call left in it.
//    Nothing has to start at zero: the scan+merge kernel overwrites every element the LayerNorm
//    kernel will read.  Two calls that overlap in time on the same GPU (different streams or
//    threads) race on it -- serialise them;
//  * no cudaMalloc / cudaFree / allocating library routine is called here or below.
// ------------------------------------------------------------------------------------------------
constexpr long long kStaticScratchBytes = 32ll << 20;                       // 32 MiB per GPU
constexpr long long kStaticScratchFloats = kStaticScratchBytes / 4;         // 8 388 608 map elements
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];

constexpr int kMaxDevices = 64;
static float* g_static_scratch_addr[kMaxDevices] = {};
static std::mutex g_static_scratch_mutex;

// In host code `g_static_scratch` is only a handle for the runtime, not a device address: the
// address a kernel can use has to be asked for, per device.
static int static_scratch_for_current_device(float** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return SS2D_ECUDA;
    std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
    if (!g_static_scratch_addr[dev]) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || !ptr) return SS2D_ECUDA;
        g_static_scratch_addr[dev] = (float*)ptr;
    }
    *out = g_static_scratch_addr[dev];
    return SS2D_OK;
}

long long core_static_capacity() { return kStaticScratchFloats; }

int core_fwd_static(const ss2d_core_params* p, cudaStream_t st) {
    const int rc = validate_core(p);
    if (rc != SS2D_OK) return rc;
    if (p->N != 1) return SS2D_ENOTSUP;
    if (!p->with_norm && p->y_dtype != SS2D_F32) return SS2D_ENOTSUP;
    PlaneConfig c;
    if (!plan_planes(p, c)) return SS2D_ENOTSUP;
    const long long need = core_workspace_bytes(p);
    float* merged = (float*)p->y;
    if (need > 0) {
        if (need > kStaticScratchBytes) return SS2D_ETOOBIG;
        const int r = static_scratch_for_current_device(&merged);
        if (r != SS2D_OK) return r;
    } else if (!aligned_to(p->y, 16)) {
        return SS2D_EINVAL_ALIGN;
    }
    CoreArgs a;
    a.x = p->x;
    for (int k = 0; k < 4; ++k) {
        a.delta[k] = p->delta[k]; a.Bm[k] = (const float*)p->Bm[k]; a.Cm[k] = (const float*)p->Cm[k];
        a.d_bs[k] = p->delta_batch_stride[k]; a.bc_bs[k] = p->bc_batch_stride[k];
    }
    a.A = (const float*)p->A; a.Dskip = (const float*)p->Dskip; a.bias = (const float*)p->delta_bias;
    a.merged = merged;
    a.B = (int)p->B; a.D = (int)p->D; a.H = (int)p->H; a.W = (int)p->W; a.L = (int)(p->H * p->W);
    a.G = c.G; a.PP = c.PP; a.Wp = c.Wp;
    auto magic = [](long long d) { return (unsigned)(((1ULL << 32) + (unsigned long long)d - 1) / (unsigned long long)d); };
    a.magic_G = c.G > 1 ? magic(c.G) : 0; a.magic_W = p->W > 1 ? magic(p->W) : 0; a.magic_H = p->H > 1 ? magic(p->H) : 0;
    a.groups_per_image = (int)((p->D + c.PP - 1) / c.PP);
    const long long grid = (long long)p->B * a.groups_per_image;
    if (grid > 0x7fffffffLL) return SS2D_EINVAL_SHAPE;
    int r;
    if (p->act_dtype == SS2D_F32) r = launch_core_v<float>(a, c, (unsigned)grid, st);
    else if (p->act_dtype == SS2D_BF16) r = launch_core_v<__nv_bfloat16>(a, c, (unsigned)grid, st);
    else r = launch_core_v<__half>(a, c, (unsigned)grid, st);
    if (r != SS2D_OK) return r;
    if (!p->with_norm) return SS2D_OK;
    ss2d_norm_params n;
    n.in = merged; n.weight = p->ln_weight; n.bias = p->ln_bias; n.out = p->y;
    n.B = p->B; n.D = p->D; n.L = p->H * p->W; n.n_terms = 1; n.out_dtype = p->y_dtype; n.eps = p->ln_eps;
    n.reserved0 = 0;
    return layer_norm_cf(&n, st);
}

}  // namespace ss2d
