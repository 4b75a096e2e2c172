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
// by all channels of an image and stay in L1/L2.  They are read in the activation type (the type
// the projection produced them in): every thread re-reads them for every plane, and with 16-bit
// elements a warp's load is one contiguous 512-byte run instead of two half-used 1 KB runs.
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "common.cuh"
#include "core_routes.cuh"

namespace ss2d {

struct CoreArgs {
    const void* x;
    const void* delta[4];
    const void* Bm[4];   // activation dtype, like delta
    const void* Cm[4];
    const float *A, *Dskip, *bias;
    float* merged;
    long long d_bs[4], d_cs[4], bc_bs[4];
    long long x_bs, x_cs;
    int B, D, H, W, L, G, PP, Wp, groups_per_image;
    unsigned magic_G, magic_W, magic_H;   // ceil(2^32 / d): n / d == umulhi(n, magic) for n * d < 2^32
};

struct ScanScratch {
    AB wtot[4][32];          // [2 * stream + direction][warp]
    float wpre[4][32];
};

__device__ __forceinline__ int fast_div(int n, unsigned magic) { return magic ? (int)__umulhi((unsigned)n, magic) : n; }   // magic 0: divisor 1

// CTA-wide scan of per-thread aggregates in thread order (forward) and in reverse thread order
// (backward), for NS independent streams at once (a thread may hold segments of NS planes: the streams
// share the two barriers).  The state before the first thread is zero, so only the state entering each
// thread is needed: hin_f for the forward route, hin_b for the backward route.
template <int NS>
__device__ __forceinline__ void cta_scan_pair(const AB (&f)[NS], const AB (&bk)[NS], int lane, int warp, int nwarps,
                                              ScanScratch& s, float (&hin_f)[NS], float (&hin_b)[NS]) {
    AB inc_f[NS], inc_b[NS];
#pragma unroll
    for (int q = 0; q < NS; ++q) {
        inc_f[q] = warp_scan_inclusive(f[q], lane);
        inc_b[q] = warp_scan_inclusive_rev(bk[q], lane);
        if (lane == 31) s.wtot[2 * q][warp] = inc_f[q];
        if (lane == 0) s.wtot[2 * q + 1][warp] = inc_b[q];
    }
    __syncthreads();
    for (int job = warp; job < 2 * NS; job += nwarps) {         // one warp per (stream, direction)
        const AB t = (lane < nwarps) ? s.wtot[job][lane] : AB{1.f, 0.f};
        if ((job & 1) == 0) {
            const AB sc = warp_scan_inclusive(t, lane);
            float e = __shfl_up_sync(0xffffffffu, sc.b, 1);
            if (lane == 0) e = 0.f;
            s.wpre[job][lane] = e;
        } else {
            const AB sc = warp_scan_inclusive_rev(t, lane);
            float e = __shfl_down_sync(0xffffffffu, sc.b, 1);
            if (lane == 31) e = 0.f;
            s.wpre[job][lane] = e;
        }
    }
    __syncthreads();
#pragma unroll
    for (int q = 0; q < NS; ++q) {
        float ea = __shfl_up_sync(0xffffffffu, inc_f[q].a, 1), eb = __shfl_up_sync(0xffffffffu, inc_f[q].b, 1);
        if (lane == 0) { ea = 1.f; eb = 0.f; }
        hin_f[q] = fmaf(ea, s.wpre[2 * q][warp], eb);
        float ra = __shfl_down_sync(0xffffffffu, inc_b[q].a, 1), rb = __shfl_down_sync(0xffffffffu, inc_b[q].b, 1);
        if (lane == 31) { ra = 1.f; rb = 0.f; }
        hin_b[q] = fmaf(ra, s.wpre[2 * q + 1][warp], rb);
    }
}

// Per-row constants of one route, pre-scaled for the arithmetic below.
struct RouteConst {
    float A;        // A (negative): decay = 2^(A * log2(1 + e^x))
    float bias2;    // delta_bias * log2(e)
    float bias;     // delta_bias
};

// Packed fp32 pairs: sm_100 executes two independent fp32 operations per FFMA2 / FMUL2 / FADD2
// instruction.  The kernel is bound by instruction issue, so everything elementwise is written on pairs.
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 add2(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 splat(float v) { return make_float2(v, v); }

// One direction of one route over the VEC register elements of a thread (NP = VEC/2 pairs; VEC = 1
// uses the .x half of a single pair).  `ul` holds u * ln2.  With t = log2(1 + e^x), x = delta + bias:
// softplus(x) = ln2 * t and exp(softplus(x) * A) = 2^(A t), so one ex2 and one lg2 serve both the
// step size and the decay.  Adds C*h_local to ysum, leaves C*prod(a) in cP, returns the thread aggregate.
// kPrecise (fp32 tensors): softplus keeps torch's threshold and a series for small e^x, so that the
// result is accurate to fp32 rounding; otherwise (16-bit tensors, whose own rounding is four orders
// of magnitude coarser) the shortest instruction sequence is used.
template <int VEC, bool kForward, bool kPrecise>
__device__ __forceinline__ AB route_local(const float2 (&ul)[(VEC + 1) / 2], const float2 (&dv)[(VEC + 1) / 2],
                                          const float2 (&bv)[(VEC + 1) / 2], const float2 (&cv)[(VEC + 1) / 2],
                                          const RouteConst rc, float2 (&cP)[(VEC + 1) / 2],
                                          float2 (&ysum)[(VEC + 1) / 2]) {
    constexpr int NP = (VEC + 1) / 2;
    float2 aa[NP], bb[NP];
#pragma unroll
    for (int j = 0; j < NP; ++j) {
        float2 t;
        if constexpr (kPrecise) {
            const float2 x = add2(dv[j], splat(rc.bias));
            t = mul2(make_float2(softplus_fast(x.x), softplus_fast(x.y)), splat(kLog2e));
        } else {
            // clamp keeps e^x finite; above x = 87 the reference returns x itself
            float2 arg = fma2(dv[j], splat(kLog2e), splat(rc.bias2));
            arg.x = fminf(arg.x, 126.f); arg.y = fminf(arg.y, 126.f);
            const float2 w = add2(make_float2(ex2_approx(arg.x), ex2_approx(arg.y)), splat(1.0f));
            t = make_float2(lg2_approx(w.x), lg2_approx(w.y));
        }
        const float2 ta = mul2(t, splat(rc.A));
        aa[j] = make_float2(ex2_approx(ta.x), ex2_approx(ta.y));
        bb[j] = mul2(t, mul2(bv[j], ul[j]));
    }
    // the recurrence itself is serial; afterwards aa holds the running product, bb the local state
    float p = 1.f, h = 0.f;
#pragma unroll
    for (int ii = 0; ii < VEC; ++ii) {
        const int i = kForward ? ii : VEC - 1 - ii;
        float& a_i = (i & 1) ? aa[i >> 1].y : aa[i >> 1].x;
        float& b_i = (i & 1) ? bb[i >> 1].y : bb[i >> 1].x;
        h = fmaf(a_i, h, b_i);
        p *= a_i;
        a_i = p; b_i = h;
    }
#pragma unroll
    for (int j = 0; j < NP; ++j) {
        cP[j] = mul2(cv[j], aa[j]);
        ysum[j] = fma2(cv[j], bb[j], ysum[j]);
    }
    return AB{p, h};
}

// Segment lengths that are not a power of two (7: one line of a 7 x 7 or half a line of a 14 x 14 map) cannot
// be moved as one vector; they go element by element.  That is as many load instructions per element as the
// one-element segments such maps would otherwise get, but every per-thread cost (index arithmetic, row
// constants, the two CTA-wide scans) is then shared by seven elements instead of one.
template <typename T, int VEC> struct VecScalar {
    struct Raw { T e[VEC]; };
    template <bool kReadOnly = true>
    static __device__ __forceinline__ Raw load_raw(const T* p) {
        Raw r;
#pragma unroll
        for (int i = 0; i < VEC; ++i) r.e[i] = kReadOnly ? __ldg(p + i) : p[i];
        return r;
    }
    static __device__ __forceinline__ void unpack(const Raw& r, float (&v)[VEC]) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) v[i] = to_f<T>(r.e[i]);
    }
    static __device__ __forceinline__ void store(T* p, const float (&v)[VEC]) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) p[i] = from_f<T>(v[i]);
    }
};
template <typename T, int VEC> struct SegVec { using type = Vec<T, VEC>; };
template <typename T> struct SegVec<T, 7> { using type = VecScalar<T, 7>; };

// VEC consecutive values -> fp32 pairs (odd VEC: the .y half of the last pair is zero)
template <typename T, int VEC>
__device__ __forceinline__ void unpack_pairs(const typename SegVec<T, VEC>::type::Raw& r, float2 (&v)[(VEC + 1) / 2]) {
    float f[VEC];
    SegVec<T, VEC>::type::unpack(r, f);
#pragma unroll
    for (int j = 0; j < VEC / 2; ++j) v[j] = make_float2(f[2 * j], f[2 * j + 1]);
    if constexpr (VEC & 1) v[VEC / 2] = make_float2(f[VEC - 1], 0.f);
}
template <int VEC>
__device__ __forceinline__ void load_pairs(const float* p, float2 (&v)[(VEC + 1) / 2]) {
    float f[VEC];
    Vec<float, VEC>::load(p, f);
    if constexpr (VEC == 1) v[0] = make_float2(f[0], 0.f);
    else {
#pragma unroll
        for (int j = 0; j < VEC / 2; ++j) v[j] = make_float2(f[2 * j], f[2 * j + 1]);
    }
}

// Shared-memory words of a VEC-segment of a plane walked with one index fastest ("minor", line
// length n_minor).  The host picks VEC so that VEC/2 divides n_minor: a segment then either lies
// in one line or wraps exactly at its middle, so the first half is affine from `lo` and the second
// half affine from `hi` (two bases, no per-element test).
template <int VEC>
struct SegAddr {
    int lo, hi;
    __device__ __forceinline__ SegAddr(int major0, int minor0, int n_minor, int major_stride, int minor_stride) {
        lo = major0 * major_stride + minor0 * minor_stride;
        const bool wrap = minor0 + VEC > n_minor;
        hi = wrap ? lo + major_stride - n_minor * minor_stride : lo;
    }
    __device__ __forceinline__ int at(int i, int minor_stride) const { return (i < VEC / 2 || VEC == 1 ? lo : hi) + i * minor_stride; }
};

// NPL = 2 (narrow segments only): a thread holds the same segment of TWO planes of its image, plane pl and plane
// pl + PP/2.  A CTA pass costs about the same whatever the segment width (load, scan, barrier and store latencies in
// sequence), so with four-element segments a pass moved half the pixels of an eight-element pass; two planes per
// thread restore the pixels per pass, share the B / C rows (same image) and the index arithmetic, and the two
// planes' scans share their barriers.
template <typename T, int VEC, int NPL, int MAXT, int MINB>
__global__ void __launch_bounds__(MAXT, MINB) core_plane_kernel(const CoreArgs a) {
    extern __shared__ __align__(16) float smem[];
    __shared__ ScanScratch scr;
    constexpr bool kPrecise = sizeof(T) == 4;
    constexpr int NP = (VEC + 1) / 2;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5, nwarps = (blockDim.x + 31) >> 5;
    const int b = blockIdx.x / a.groups_per_image;
    const int d0 = (blockIdx.x - b * a.groups_per_image) * a.PP;
    const int pp_here = min(a.PP, a.D - d0);
    const int pl0 = fast_div(t, a.magic_G);
    const int v = t - pl0 * a.G;
    const int half = a.PP / NPL;            // planes side by side in thread order
    // Threads past the last plane of the CTA (round-up to a warp, last channel group) run on the
    // last valid plane so that every load below is in range; they take no part in the scans
    // (identity aggregates) and store nothing.
    bool active[NPL];
    int d[NPL];
    float* plane[NPL];
    const int L = a.L, H = a.H, W = a.W, Wp = a.Wp, D = a.D;
#pragma unroll
    for (int s = 0; s < NPL; ++s) {
        int pl = pl0 + s * half;
        active[s] = pl0 < half && pl < pp_here;
        pl = min(pl, pp_here - 1);
        d[s] = d0 + pl;
        // one padded fp32 plane per channel: first x (for the transposed read), then, once every
        // column-orientation thread has taken its x values, the column-orientation result
        plane[s] = smem + (size_t)pl * (H * Wp);
    }
    using VT = typename SegVec<T, VEC>::type;
    const int e0 = v * VEC;   // first element of this thread in either orientation order
    const bool first = v == 0, last = v == a.G - 1;

    // ---- issue every HBM load of the pass up front: x and the four delta vectors -------------
    typename VT::Raw rx[NPL], rd0[NPL], rd1[NPL], rd2[NPL], rd3[NPL];
#pragma unroll
    for (int s = 0; s < NPL; ++s) {
        rx[s] = VT::load_raw((const T*)a.x + b * a.x_bs + d[s] * a.x_cs + e0);
        rd0[s] = VT::load_raw((const T*)a.delta[0] + b * a.d_bs[0] + d[s] * a.d_cs[0] + e0);
        rd2[s] = VT::load_raw((const T*)a.delta[2] + b * a.d_bs[2] + d[s] * a.d_cs[2] + e0);
        rd1[s] = VT::load_raw((const T*)a.delta[1] + b * a.d_bs[1] + d[s] * a.d_cs[1] + e0);
        rd3[s] = VT::load_raw((const T*)a.delta[3] + b * a.d_bs[3] + d[s] * a.d_cs[3] + e0);
    }
    float2 ul[NPL][NP], yrow[NPL][NP];

    // ---- x into shared memory (row-major, padded pitch) -------------------------------------
    const int h0 = fast_div(e0, a.magic_W), w0 = e0 - h0 * W;
    const SegAddr<VEC> rs(h0, w0, W, Wp, 1);
#pragma unroll
    for (int s = 0; s < NPL; ++s) {
        unpack_pairs<T, VEC>(rx[s], ul[s]);
        if (active[s]) {
#pragma unroll
            for (int i = 0; i < VEC; ++i) plane[s][rs.at(i, 1)] = (i & 1) ? ul[s][i >> 1].y : ul[s][i >> 1].x;
        }
    }
    const int wc = fast_div(e0, a.magic_H), hc = e0 - wc * H;
    const SegAddr<VEC> cs(wc, hc, H, 1, Wp);   // column-major walk: h is the fast index, stride Wp

    // ---- row orientation: routes 0 (forward) and 2 (backward) ---------------------------------
    {
        float2 dv[NP], bv[NP], cv[NP], cPf[NPL][NP], cPb[NPL][NP];
        AB af[NPL], ab[NPL];
#pragma unroll
        for (int s = 0; s < NPL; ++s) {
            const float2 Dsum = splat(__ldg(a.Dskip + d[s]) + __ldg(a.Dskip + 2 * D + d[s]));
#pragma unroll
            for (int j = 0; j < NP; ++j) { yrow[s][j] = mul2(Dsum, ul[s][j]); ul[s][j] = mul2(ul[s][j], splat(kLn2)); }
        }
        unpack_pairs<T, VEC>(VT::load_raw((const T*)a.Bm[0] + b * a.bc_bs[0] + e0), bv);      // one image: the planes share B and C
        unpack_pairs<T, VEC>(VT::load_raw((const T*)a.Cm[0] + b * a.bc_bs[0] + e0), cv);
#pragma unroll
        for (int s = 0; s < NPL; ++s) {
            RouteConst rc;
            rc.A = __ldg(a.A + d[s]); rc.bias = __ldg(a.bias + d[s]); rc.bias2 = rc.bias * kLog2e;
            unpack_pairs<T, VEC>(rd0[s], dv);
            af[s] = route_local<VEC, true, kPrecise>(ul[s], dv, bv, cv, rc, cPf[s], yrow[s]);
        }
        unpack_pairs<T, VEC>(VT::load_raw((const T*)a.Bm[2] + b * a.bc_bs[2] + e0), bv);
        unpack_pairs<T, VEC>(VT::load_raw((const T*)a.Cm[2] + b * a.bc_bs[2] + e0), cv);
#pragma unroll
        for (int s = 0; s < NPL; ++s) {
            RouteConst rc;
            rc.A = __ldg(a.A + 2 * D + d[s]); rc.bias = __ldg(a.bias + 2 * D + d[s]); rc.bias2 = rc.bias * kLog2e;
            unpack_pairs<T, VEC>(rd2[s], dv);
            ab[s] = route_local<VEC, false, kPrecise>(ul[s], dv, bv, cv, rc, cPb[s], yrow[s]);
            if (first) af[s].a = 0.f;
            if (last) ab[s].a = 0.f;
            if (!active[s]) { af[s] = AB{1.f, 0.f}; ab[s] = AB{1.f, 0.f}; }
        }
        float hf[NPL], hb[NPL];
        cta_scan_pair<NPL>(af, ab, lane, warp, nwarps, scr, hf, hb);   // its barriers also order the x stores before the reads below
#pragma unroll
        for (int s = 0; s < NPL; ++s) {
            if (first) hf[s] = 0.f;
            if (last) hb[s] = 0.f;
#pragma unroll
            for (int j = 0; j < NP; ++j) yrow[s][j] = fma2(cPf[s][j], splat(hf[s]), fma2(cPb[s][j], splat(hb[s]), yrow[s][j]));
        }
    }

    // ---- column orientation: routes 1 (forward) and 3 (backward) -------------------------------
    {
        float2 dv[NP], bv[NP], cv[NP], cPf[NPL][NP], cPb[NPL][NP], ycol[NPL][NP];
        AB af[NPL], ab[NPL];
#pragma unroll
        for (int s = 0; s < NPL; ++s) {
#pragma unroll
            for (int j = 0; j < NP; ++j) {
                ul[s][j].x = plane[s][cs.at(2 * j, Wp)];
                ul[s][j].y = (2 * j + 1 < VEC) ? plane[s][cs.at(2 * j + 1, Wp)] : 0.f;
            }
            const float2 Dsum = splat(__ldg(a.Dskip + D + d[s]) + __ldg(a.Dskip + 3 * D + d[s]));
#pragma unroll
            for (int j = 0; j < NP; ++j) { ycol[s][j] = mul2(Dsum, ul[s][j]); ul[s][j] = mul2(ul[s][j], splat(kLn2)); }
        }
        unpack_pairs<T, VEC>(VT::load_raw((const T*)a.Bm[1] + b * a.bc_bs[1] + e0), bv);
        unpack_pairs<T, VEC>(VT::load_raw((const T*)a.Cm[1] + b * a.bc_bs[1] + e0), cv);
#pragma unroll
        for (int s = 0; s < NPL; ++s) {
            RouteConst rc;
            rc.A = __ldg(a.A + D + d[s]); rc.bias = __ldg(a.bias + D + d[s]); rc.bias2 = rc.bias * kLog2e;
            unpack_pairs<T, VEC>(rd1[s], dv);
            af[s] = route_local<VEC, true, kPrecise>(ul[s], dv, bv, cv, rc, cPf[s], ycol[s]);
        }
        unpack_pairs<T, VEC>(VT::load_raw((const T*)a.Bm[3] + b * a.bc_bs[3] + e0), bv);
        unpack_pairs<T, VEC>(VT::load_raw((const T*)a.Cm[3] + b * a.bc_bs[3] + e0), cv);
#pragma unroll
        for (int s = 0; s < NPL; ++s) {
            RouteConst rc;
            rc.A = __ldg(a.A + 3 * D + d[s]); rc.bias = __ldg(a.bias + 3 * D + d[s]); rc.bias2 = rc.bias * kLog2e;
            unpack_pairs<T, VEC>(rd3[s], dv);
            ab[s] = route_local<VEC, false, kPrecise>(ul[s], dv, bv, cv, rc, cPb[s], ycol[s]);
            if (first) af[s].a = 0.f;
            if (last) ab[s].a = 0.f;
            if (!active[s]) { af[s] = AB{1.f, 0.f}; ab[s] = AB{1.f, 0.f}; }
        }
        float hf[NPL], hb[NPL];
        cta_scan_pair<NPL>(af, ab, lane, warp, nwarps, scr, hf, hb);   // every x value has been read before these barriers
#pragma unroll
        for (int s = 0; s < NPL; ++s) {
            if (first) hf[s] = 0.f;
            if (last) hb[s] = 0.f;
#pragma unroll
            for (int j = 0; j < NP; ++j) ycol[s][j] = fma2(cPf[s][j], splat(hf[s]), fma2(cPb[s][j], splat(hb[s]), ycol[s][j]));
            if (active[s]) {
#pragma unroll
                for (int i = 0; i < VEC; ++i) plane[s][cs.at(i, Wp)] = (i & 1) ? ycol[s][i >> 1].y : ycol[s][i >> 1].x;
            }
        }
    }
    __syncthreads();

    // ---- merge: row result (registers) + column result (transposed read), one vector store ------
#pragma unroll
    for (int s = 0; s < NPL; ++s) {
        if (active[s]) {
            float out[VEC];
#pragma unroll
            for (int i = 0; i < VEC; ++i) out[i] = ((i & 1) ? yrow[s][i >> 1].y : yrow[s][i >> 1].x) + plane[s][rs.at(i, 1)];
            SegVec<float, VEC>::type::store(a.merged + (long long)b * D * L + (long long)d[s] * L + e0, out);
        }
    }
}


// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per (kernel, device): the attribute only ever has to grow.
static cudaError_t ensure_dynamic_smem(const void* kern, size_t bytes) {
    struct Entry { const void* kern; int dev; size_t bytes; };
    static std::mutex mu;
    static std::vector<Entry> seen;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    std::lock_guard<std::mutex> lock(mu);
    for (Entry& en : seen)
        if (en.kern == kern && en.dev == dev) {
            if (en.bytes >= bytes) return cudaSuccess;
            e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
            if (e == cudaSuccess) en.bytes = bytes;
            return e;
        }
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e == cudaSuccess) seen.push_back(Entry{kern, dev, bytes});
    return e;
}

struct PlaneConfig { int vec, G, PP, threads, Wp, npl; size_t smem; };

static bool plan_planes(const ss2d_core_params* p, PlaneConfig& c) {
    const long long L = p->H * p->W;
    const size_t s = dtype_size(p->act_dtype);
    auto el = [&](const void* q) { return (long long)(reinterpret_cast<uintptr_t>(q) / s); };
    int vec = 8;
    auto fit = [&](long long x) { if (x < 0) x = -x; while (vec > 1 && (x % vec) != 0) vec >>= 1; };
    fit(L); fit(el(p->x)); fit(p->x_batch_stride); fit(p->x_channel_stride);
    for (int k = 0; k < 4; ++k) {
        fit(el(p->delta[k]));
        fit(el(p->Bm[k])); fit(el(p->Cm[k]));
        fit(p->delta_batch_stride[k]); fit(p->bc_batch_stride[k]); fit(p->delta_channel_stride[k]);
    }
    // a thread's segment may wrap to the next line only at its middle: vec/2 divides H and W
    while (vec > 1 && (vec > p->H || vec > p->W || (p->H % (vec / 2)) != 0 || (p->W % (vec / 2)) != 0)) vec >>= 1;
    // odd maps whose sides are multiples of 7 (7 x 7) would get one-element segments: seven-element segments,
    // moved element by element, share the per-thread work of the pass between seven elements instead
    // (234 -> 113 us for the two 7 x 7 launches of a batch-128 VMamba-T forward; for 14 x 14 maps, which get
    // four-element vectors, the same change is 20 % slower)
    if (vec == 1 && p->H % 7 == 0 && p->W % 7 == 0) vec = 7;
    // 16-byte loads are enough: an 8-wide fp32 vector is two of them
    // (alignment of the fp32 workspace is checked by the caller)
    const long long G = L / vec;
    if (G > 1024) return false;
    // ~14 warps per CTA, two CTAs per SM; seven-thread planes (7 x 7) in CTAs of seven warps, four per SM: 61.6 -> 51.4 us
    // per launch at 128 x 768 planes (the 14 x 14 launch takes 84 us with 448, 224 or 160 threads and 98 us with 320)
    int PP = (int)((G <= 8 ? 224 : 448) / G);
    if (PP < 1) PP = 1;
    if (PP > p->D) PP = (int)p->D;
    // segments of at most four elements: two planes per thread (the kernel's NPL = 2), twice the planes per CTA
    // (677 -> 649 us for the eight 14 x 14 launches of a batch-128 VMamba-T forward)
    const int npl = (vec <= 4 && 2 * PP <= p->D) ? 2 : 1;
    PP *= npl;
    const int Wp = (int)(p->W | 1);   // odd pitch spreads the transposed accesses over banks
    size_t smem = (size_t)PP * p->H * Wp * sizeof(float);
    while (smem > 200 * 1024 && PP > npl) { PP -= npl; smem = (size_t)PP * p->H * Wp * sizeof(float); }
    if (smem > 200 * 1024) return false;
    c.vec = vec; c.G = (int)G; c.PP = PP; c.Wp = Wp; c.smem = smem; c.npl = npl;
    c.threads = (int)(((PP / npl) * G + 31) / 32 * 32);
    return true;
}

template <typename T, int VEC, int NPL>
static int launch_core_n(const CoreArgs& a, const PlaneConfig& c, unsigned grid, cudaStream_t st) {
    cudaError_t e;
    if (c.threads <= 448) {           // 72 registers per thread at two CTAs per SM
        auto kern = core_plane_kernel<T, VEC, NPL, 448, 2>;
        e = ensure_dynamic_smem((const void*)kern, c.smem);
        if (e != cudaSuccess) return SS2D_ECUDA;
        kern<<<grid, c.threads, c.smem, st>>>(a);
    } else {
        auto kern = core_plane_kernel<T, VEC, NPL, 1024, 1>;
        e = ensure_dynamic_smem((const void*)kern, c.smem);
        if (e != cudaSuccess) return SS2D_ECUDA;
        kern<<<grid, c.threads, c.smem, st>>>(a);
    }
    count_launch();
    return check_launch();
}

template <typename T, int VEC>
static int launch_core_t(const CoreArgs& a, const PlaneConfig& c, unsigned grid, cudaStream_t st) {
    if constexpr (VEC <= 4) {
        if (c.npl == 2) return launch_core_n<T, VEC, 2>(a, c, grid, st);
    }
    return launch_core_n<T, VEC, 1>(a, c, grid, st);
}

template <typename T>
static int launch_core_v(const CoreArgs& a, const PlaneConfig& c, unsigned grid, cudaStream_t st) {
    switch (c.vec) {
        case 8: return launch_core_t<T, 8>(a, c, grid, st);
        case 7: return launch_core_t<T, 7>(a, c, grid, st);
        case 4: return launch_core_t<T, 4>(a, c, grid, st);
        case 2: return launch_core_t<T, 2>(a, c, grid, st);
        default: return launch_core_t<T, 1>(a, c, grid, st);
    }
}


// ---- route-stream kernel (core_routes.cuh): which planes it takes, and its launch -----------------------------
struct RoutePlan { int S, SV; size_t smem; };

// 0: choose by shape (default), 1: always the plane kernel, 2: the route-stream kernel wherever it applies.
// Read once from SS2D_CORE_KERNEL = plane | routes (a switch for measurements; both kernels pass the same tests).
static int core_kernel_choice() {
    static const int choice = [] {
        const char* v = std::getenv("SS2D_CORE_KERNEL");
        if (!v) return 0;
        if (!std::strcmp(v, "plane")) return 1;
        if (!std::strcmp(v, "routes")) return 2;
        return 0;
    }();
    return choice;
}

static bool plan_routes(const ss2d_core_params* p, RoutePlan& r) {
    const long long L = p->H * p->W;
    const size_t s = dtype_size(p->act_dtype);
    if (L % 4 != 0 || p->W % 4 != 0) return false;
    auto el = [&](const void* q) { return (long long)(reinterpret_cast<uintptr_t>(q) / s); };
    int vec = 8;
    auto fit = [&](long long x) { if (x < 0) x = -x; while (vec > 1 && (x % vec) != 0) vec >>= 1; };
    fit(L); fit(el(p->x)); fit(p->x_batch_stride); fit(p->x_channel_stride);
    for (int k = 0; k < 4; ++k) {
        fit(el(p->delta[k]));
        fit(el(p->Bm[k])); fit(el(p->Cm[k]));
        fit(p->delta_batch_stride[k]); fit(p->bc_batch_stride[k]); fit(p->delta_channel_stride[k]);
    }
    if (vec < 4) return false;
    r.S = vec;
    r.SV = (vec == 8 && p->W % 8 == 0) ? 8 : 4;
    r.smem = (size_t)L * (8 + s);
    return r.smem <= 227 * 1024;
}

template <typename T, int S, int SV, int MINB, int kRoll>
static int launch_routes_k(const RouteArgs& a, const RoutePlan& r, unsigned grid, cudaStream_t st) {
    auto kern = core_route_kernel<T, S, SV, MINB, kRoll>;
    if (ensure_dynamic_smem((const void*)kern, r.smem) != cudaSuccess) return SS2D_ECUDA;
    kern<<<grid, 128, r.smem, st>>>(a);
    count_launch();
    return check_launch();
}

template <typename T, int MINB>
static int launch_routes_t(const RouteArgs& a, const RoutePlan& r, unsigned grid, cudaStream_t st) {
    if (r.S == 8) return r.SV == 8 ? launch_routes_k<T, 8, 8, MINB, 0>(a, r, grid, st) : launch_routes_k<T, 8, 4, MINB, 0>(a, r, grid, st);
    return launch_routes_k<T, 4, 4, MINB, 0>(a, r, grid, st);
}

static int run_routes(const ss2d_core_params* p, const RoutePlan& r, float* merged, cudaStream_t st) {
    RouteArgs a;
    a.x = p->x;
    for (int k = 0; k < 4; ++k) {
        a.delta[k] = p->delta[k]; a.Bm[k] = p->Bm[k]; a.Cm[k] = p->Cm[k];
        a.d_bs[k] = p->delta_batch_stride[k]; a.bc_bs[k] = p->bc_batch_stride[k];
        a.d_cs[k] = p->delta_channel_stride[k] ? p->delta_channel_stride[k] : p->H * p->W;
    }
    a.A = (const float*)p->A; a.Dskip = (const float*)p->Dskip; a.bias = (const float*)p->delta_bias;
    a.merged = merged;
    a.x_bs = p->x_batch_stride ? p->x_batch_stride : p->D * p->H * p->W;
    a.x_cs = p->x_channel_stride ? p->x_channel_stride : p->H * p->W;
    a.B = (int)p->B; a.D = (int)p->D; a.H = (int)p->H; a.W = (int)p->W; a.L = (int)(p->H * p->W);
    a.magic_H = p->H > 1 ? (unsigned)(((1ULL << 32) + (unsigned long long)p->H - 1) / (unsigned long long)p->H) : 0;
    const long long grid = p->B * p->D;
    if (grid > 0x7fffffffLL) return SS2D_EINVAL_SHAPE;
    if (p->act_dtype == SS2D_F32) return launch_routes_t<float, 4>(a, r, (unsigned)grid, st);
    if (p->act_dtype == SS2D_BF16) return launch_routes_t<__nv_bfloat16, 7>(a, r, (unsigned)grid, st);
    return launch_routes_t<__half, 7>(a, r, (unsigned)grid, st);
}

// The scan + merge kernel for this call.  Measured on B200 (bf16, scan + merge alone): the route-stream kernel wins
// where its chunks are well filled and seven CTAs fit an SM (56 x 56: 0.223 against 0.267 ms at batch 128 x 96
// channels; 32 x 32: 0.106 against 0.112 ms), and loses where a quarter of the last chunk's lanes idle (28 x 28:
// 0.148 against 0.141 ms) or shared memory leaves five CTAs per SM (64 x 64: 0.231 against 0.219 ms).
static bool use_routes(const ss2d_core_params* p, RoutePlan& r) {
    const int choice = core_kernel_choice();
    if (choice == 1 || !plan_routes(p, r)) return false;
    if (choice == 2) return true;
    const long long L = p->H * p->W, chunk = 32 * r.S;
    const long long chunks = (L + chunk - 1) / chunk;
    return r.S == 8 && 10 * L >= 9 * chunks * chunk && r.smem <= 32 * 1024;
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
        if (p->B > 1 && (p->delta_batch_stride[k] < L || p->bc_batch_stride[k] < L)) return SS2D_EINVAL_STRIDE;
        if (p->delta_channel_stride[k] && p->delta_channel_stride[k] < L) return SS2D_EINVAL_STRIDE;
    }
    if (p->x_batch_stride < 0 || p->x_channel_stride < 0 || p->y_batch_stride < 0 || p->y_channel_stride < 0) return SS2D_EINVAL_STRIDE;
    if ((p->x_channel_stride && p->x_channel_stride < L) || (p->y_channel_stride && p->y_channel_stride < L)) return SS2D_EINVAL_STRIDE;
    const size_t s = dtype_size(p->act_dtype);
    if (!aligned_to(p->x, s) || !aligned_to(p->y, dtype_size(p->y_dtype)) || !aligned_to(p->A, 4) ||
        !aligned_to(p->Dskip, 4) || !aligned_to(p->delta_bias, 4) || !aligned_to(p->ln_weight, 4) ||
        !aligned_to(p->ln_bias, 4))
        return SS2D_EINVAL_ALIGN;
    for (int k = 0; k < 4; ++k)
        if (!aligned_to(p->delta[k], s) || !aligned_to(p->Bm[k], s) || !aligned_to(p->Cm[k], s)) return SS2D_EINVAL_ALIGN;
    return SS2D_OK;
}

long long core_workspace_bytes(const ss2d_core_params* p) {
    if (validate_core(p) != SS2D_OK) return -1;
    // the fp32 merged map; not needed when the caller asks for it directly (no norm, fp32 output)
    if (!p->with_norm && p->y_dtype == SS2D_F32) return 0;
    return (long long)(p->B * p->D * p->H * p->W) * 4;
}

struct CorePlan { bool routes; RoutePlan r; PlaneConfig c; };

static bool plan_core(const ss2d_core_params* p, CorePlan& plan) {
    plan.routes = use_routes(p, plan.r);
    return plan.routes || plan_planes(p, plan.c);
}

static int run_planes(const ss2d_core_params* p, const PlaneConfig& c, float* merged, cudaStream_t st) {
    CoreArgs a;
    a.x = p->x;
    for (int k = 0; k < 4; ++k) {
        a.delta[k] = p->delta[k]; a.Bm[k] = p->Bm[k]; a.Cm[k] = p->Cm[k];
        a.d_bs[k] = p->delta_batch_stride[k]; a.bc_bs[k] = p->bc_batch_stride[k];
        a.d_cs[k] = p->delta_channel_stride[k] ? p->delta_channel_stride[k] : p->H * p->W;
    }
    a.A = (const float*)p->A; a.Dskip = (const float*)p->Dskip; a.bias = (const float*)p->delta_bias;
    a.merged = merged;
    a.x_bs = p->x_batch_stride ? p->x_batch_stride : p->D * p->H * p->W;
    a.x_cs = p->x_channel_stride ? p->x_channel_stride : p->H * p->W;
    a.B = (int)p->B; a.D = (int)p->D; a.H = (int)p->H; a.W = (int)p->W; a.L = (int)(p->H * p->W);
    a.G = c.G; a.PP = c.PP; a.Wp = c.Wp;
    auto magic = [](long long d) { return (unsigned)(((1ULL << 32) + (unsigned long long)d - 1) / (unsigned long long)d); };
    a.magic_G = c.G > 1 ? magic(c.G) : 0; a.magic_W = p->W > 1 ? magic(p->W) : 0; a.magic_H = p->H > 1 ? magic(p->H) : 0;
    a.groups_per_image = (int)((p->D + c.PP - 1) / c.PP);
    const long long grid = (long long)p->B * a.groups_per_image;
    if (grid > 0x7fffffffLL) return SS2D_EINVAL_SHAPE;
    if (p->act_dtype == SS2D_F32) return launch_core_v<float>(a, c, (unsigned)grid, st);
    if (p->act_dtype == SS2D_BF16) return launch_core_v<__nv_bfloat16>(a, c, (unsigned)grid, st);
    return launch_core_v<__half>(a, c, (unsigned)grid, st);
}

// Scan + merge kernel into `merged`, then (with_norm) the LayerNorm kernel into p->y.  Arguments validated by the caller.
// The merged map goes through memory once between the two kernels.  Walking the batch in groups small enough for
// that map to stay in L2 (scan, LayerNorm, scan, ...) was measured and is slower: a CTA of the scan kernel lives for
// about 20 us, so every extra kernel boundary drains and refills the GPU for longer than the L2 hits save
// (stage 0, batch 128: 0.263 ms in one round, 0.282 / 0.329 / 0.378 ms in rounds of 64 / 32 / 16 images).
static int run_core(const ss2d_core_params* p, const CorePlan& plan, float* merged, cudaStream_t st) {
    const int r = plan.routes ? run_routes(p, plan.r, merged, st) : run_planes(p, plan.c, merged, st);
    if (r != SS2D_OK) return r;
    if (!p->with_norm) return SS2D_OK;
    ss2d_norm_params n = {};
    n.in = merged; n.weight = p->ln_weight; n.bias = p->ln_bias; n.out = p->y;
    n.B = p->B; n.D = p->D; n.L = p->H * p->W; n.io_dtype = p->y_dtype; n.eps = p->ln_eps;
    n.out_batch_stride = p->y_batch_stride; n.out_channel_stride = p->y_channel_stride;
    n.descending = 1;         // the scan kernel wrote `merged` front to back: its end is what L2 still holds
    return layer_norm_cf(&n, st);
}

// Checks shared by the two entry points; on success `plan` is filled and `need` holds the scratch bytes (0: the
// merged map goes straight to p->y).
static int prepare_core(const ss2d_core_params* p, CorePlan& plan, long long& need) {
    const int rc = validate_core(p);
    if (rc != SS2D_OK) return rc;
    if (p->N != 1) return SS2D_ENOTSUP;          // d_state > 1 runs through the operator-surface kernels
    if (!p->with_norm && p->y_dtype != SS2D_F32) return SS2D_ENOTSUP;
    if (!plan_core(p, plan)) return SS2D_ENOTSUP;  // plane too long for one CTA
    need = core_workspace_bytes(p);
    if (need == 0) {
        if (!aligned_to(p->y, 16)) return SS2D_EINVAL_ALIGN;
        if (p->y_batch_stride || p->y_channel_stride) return SS2D_ENOTSUP;     // the un-normalised fp32 map is written dense
    }
    return SS2D_OK;
}

int core_supported(const ss2d_core_params* p) {
    CorePlan plan;
    long long need = 0;
    return prepare_core(p, plan, need);
}

int core_fwd(const ss2d_core_params* p, cudaStream_t st) {
    CorePlan plan;
    long long need = 0;
    const int rc = prepare_core(p, plan, need);
    if (rc != SS2D_OK) return rc;
    float* merged = (float*)p->y;
    if (need > 0) {
        if (!p->workspace || p->workspace_bytes < need) return SS2D_EWORKSPACE;
        if (!aligned_to(p->workspace, 256)) return SS2D_EINVAL_ALIGN;
        merged = (float*)p->workspace;
    }
    return run_core(p, plan, merged, st);
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
    CorePlan plan;
    long long need = 0;
    const int rc = prepare_core(p, plan, need);
    if (rc != SS2D_OK) return rc;
    float* merged = (float*)p->y;
    if (need > 0) {
        if (need > kStaticScratchBytes) return SS2D_ETOOBIG;
        const int r = static_scratch_for_current_device(&merged);
        if (r != SS2D_OK) return r;
    }
    return run_core(p, plan, merged, st);
}

}  // namespace ss2d
