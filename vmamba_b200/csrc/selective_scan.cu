// Selective-scan forward, the operator-surface kernel (one tensor in, one tensor out per row).
//
// Mapping: one warp owns one row (b, r) of length L.  Per step a lane takes VEC consecutive
// elements (one 16-byte load per tensor when alignment allows), runs the recurrence over them
// in registers, the 32 lane aggregates are combined with a shuffle scan of the associative pair
// (a, b) o (a', b') = (a a', a' b + b'), and the carry into the next 32*VEC-element step stays in
// a register (d_state 1) or in shared memory (d_state > 1).  The next step's vectors are
// fetched before the current step's arithmetic.  Traffic per row: u and delta read once, out
// written once; B/C rows are shared by all channels of a group and come from L2.
#include "common.cuh"

namespace ss2d {

struct ScanArgs {
    const void *u, *delta, *B, *C;
    const float *A, *D, *bias;
    void* out;
    int64_t rows, dim, dstate, seqlen, group_size;
    int64_t u_bs, u_ds, d_bs, d_ds, o_bs, o_ds;
    int64_t B_bs, B_gs, B_ss, C_bs, C_gs, C_ss;
    int softplus;
    int64_t dratio;   // channels per delta row
    float* ckpt;      // (rows, nck, dstate) or null
    int64_t nck;
};

constexpr int kWarpsPerCta = 4;

template <typename Tin, typename Tout, int VEC>
__global__ void __launch_bounds__(kWarpsPerCta * 32) selscan_fwd_n1_kernel(const ScanArgs a) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
    if (row >= a.rows) return;
    const int64_t b = row / a.dim, r = row % a.dim, k = r / a.group_size;
    const Tin* __restrict__ u = (const Tin*)a.u + b * a.u_bs + r * a.u_ds;
    const Tin* __restrict__ dt = (const Tin*)a.delta + b * a.d_bs + (r / a.dratio) * a.d_ds;
    const Tin* __restrict__ Bm = (const Tin*)a.B + b * a.B_bs + k * a.B_gs;
    const Tin* __restrict__ Cm = (const Tin*)a.C + b * a.C_bs + k * a.C_gs;
    Tout* __restrict__ out = (Tout*)a.out + b * a.o_bs + r * a.o_ds;
    const float A2 = __ldg(a.A + r) * kLog2e;
    const bool has_D = a.D != nullptr;
    const float Dv = has_D ? __ldg(a.D + r) : 0.f;
    const float bias = a.bias ? __ldg(a.bias + r / a.dratio) : 0.f;
    const bool sp = a.softplus != 0;
    const int L = (int)a.seqlen;
    constexpr int STEP = 32 * VEC;
    using VI = Vec<Tin, VEC>;
    using VO = Vec<Tout, VEC>;

    typename VI::Raw ru = {}, rd = {}, rb = {}, rc = {};
    int pos = lane * VEC;
    if (pos < L) {   // L % VEC == 0: a lane's vector lies wholly inside or outside the row
        ru = VI::load_raw(u + pos); rd = VI::load_raw(dt + pos);
        rb = VI::load_raw(Bm + pos); rc = VI::load_raw(Cm + pos);
    }
    float hc = 0.f;   // state entering this step
    for (int base = 0; base < L; base += STEP) {
        typename VI::Raw nu = {}, nd = {}, nb = {}, nc = {};
        const int npos = pos + STEP;
        if (npos < L) {
            nu = VI::load_raw(u + npos); nd = VI::load_raw(dt + npos);
            nb = VI::load_raw(Bm + npos); nc = VI::load_raw(Cm + npos);
        }
        float uv[VEC], dv[VEC], bv[VEC], cv[VEC], P[VEC], hl[VEC];
        VI::unpack(ru, uv); VI::unpack(rd, dv); VI::unpack(rb, bv); VI::unpack(rc, cv);
        float p = 1.f, h = 0.f;
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            float dl = dv[i] + bias;
            if (sp) dl = softplus_fast(dl);
            const float aa = decay_fast(dl, A2);
            h = fmaf(aa, h, dl * bv[i] * uv[i]);
            p *= aa;
            P[i] = p; hl[i] = h;
        }
        const AB inc = warp_scan_inclusive(AB{p, h}, lane);
        float ea = __shfl_up_sync(0xffffffffu, inc.a, 1);
        float eb = __shfl_up_sync(0xffffffffu, inc.b, 1);
        if (lane == 0) { ea = 1.f; eb = 0.f; }
        const float hin = fmaf(ea, hc, eb);
        if (a.ckpt && (pos & 127) == 0 && pos < L) a.ckpt[row * a.nck + (pos >> 7)] = hin;     // state in front of element pos
        const float ta = __shfl_sync(0xffffffffu, inc.a, 31);
        const float tb = __shfl_sync(0xffffffffu, inc.b, 31);
        hc = fmaf(ta, hc, tb);
        if (pos < L) {
            float ov[VEC];
#pragma unroll
            for (int i = 0; i < VEC; ++i) {
                const float y = cv[i] * fmaf(P[i], hin, hl[i]);
                ov[i] = has_D ? fmaf(Dv, uv[i], y) : y;
            }
            VO::store(out + pos, ov);
        }
        ru = nu; rd = nd; rb = nb; rc = nc;
        pos = npos;
    }
}

// d_state > 1: the carry of each state lives in shared memory (one slot per warp and state).
template <typename Tin, typename Tout, int VEC>
__global__ void __launch_bounds__(kWarpsPerCta * 32) selscan_fwd_nx_kernel(const ScanArgs a) {
    __shared__ float carry_s[kWarpsPerCta][SS2D_MAX_DSTATE];
    __shared__ float A2_s[kWarpsPerCta][SS2D_MAX_DSTATE];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t row = (int64_t)blockIdx.x * kWarpsPerCta + warp;
    if (row >= a.rows) return;
    const int64_t b = row / a.dim, r = row % a.dim, k = r / a.group_size;
    const Tin* __restrict__ u = (const Tin*)a.u + b * a.u_bs + r * a.u_ds;
    const Tin* __restrict__ dt = (const Tin*)a.delta + b * a.d_bs + (r / a.dratio) * a.d_ds;
    const Tin* __restrict__ Bm = (const Tin*)a.B + b * a.B_bs + k * a.B_gs;
    const Tin* __restrict__ Cm = (const Tin*)a.C + b * a.C_bs + k * a.C_gs;
    Tout* __restrict__ out = (Tout*)a.out + b * a.o_bs + r * a.o_ds;
    const int N = (int)a.dstate;
    for (int n = lane; n < N; n += 32) {
        carry_s[warp][n] = 0.f;
        A2_s[warp][n] = __ldg(a.A + r * N + n) * kLog2e;
    }
    __syncwarp();
    const bool has_D = a.D != nullptr;
    const float Dv = has_D ? __ldg(a.D + r) : 0.f;
    const float bias = a.bias ? __ldg(a.bias + r / a.dratio) : 0.f;
    const bool sp = a.softplus != 0;
    const int L = (int)a.seqlen;
    constexpr int STEP = 32 * VEC;
    using VI = Vec<Tin, VEC>;
    using VO = Vec<Tout, VEC>;

    for (int base = 0; base < L; base += STEP) {
        const int pos = base + lane * VEC;
        const bool in = pos < L;
        float uv[VEC], dl[VEC], du[VEC], y[VEC];
        if (in) { VI::load(u + pos, uv); VI::load(dt + pos, dl); }
        else {
#pragma unroll
            for (int i = 0; i < VEC; ++i) { uv[i] = 0.f; dl[i] = 0.f; }
        }
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            float d = dl[i] + bias;
            if (sp) d = softplus_fast(d);
            dl[i] = d; du[i] = d * uv[i];
            y[i] = has_D ? Dv * uv[i] : 0.f;
        }
        for (int n = 0; n < N; ++n) {
            float bv[VEC], cv[VEC], P[VEC], hl[VEC];
            if (in) { VI::load(Bm + n * a.B_ss + pos, bv); VI::load(Cm + n * a.C_ss + pos, cv); }
            else {
#pragma unroll
                for (int i = 0; i < VEC; ++i) { bv[i] = 0.f; cv[i] = 0.f; }
            }
            const float A2 = A2_s[warp][n];
            float p = 1.f, h = 0.f;
#pragma unroll
            for (int i = 0; i < VEC; ++i) {
                const float aa = decay_fast(dl[i], A2);
                h = fmaf(aa, h, du[i] * bv[i]);
                p *= aa;
                P[i] = p; hl[i] = h;
            }
            const AB inc = warp_scan_inclusive(AB{p, h}, lane);
            float ea = __shfl_up_sync(0xffffffffu, inc.a, 1);
            float eb = __shfl_up_sync(0xffffffffu, inc.b, 1);
            if (lane == 0) { ea = 1.f; eb = 0.f; }
            const float hc = carry_s[warp][n];
            const float hin = fmaf(ea, hc, eb);
            if (a.ckpt && (pos & 127) == 0 && in) a.ckpt[(row * a.nck + (pos >> 7)) * N + n] = hin;
            __syncwarp();
            if (lane == 31) carry_s[warp][n] = fmaf(inc.a, hc, inc.b);
#pragma unroll
            for (int i = 0; i < VEC; ++i) y[i] = fmaf(cv[i], fmaf(P[i], hin, hl[i]), y[i]);
        }
        __syncwarp();
        if (in) VO::store(out + pos, y);
    }
}

template <typename Tin, typename Tout, int VEC>
static int launch_scan(const ScanArgs& a, cudaStream_t st) {
    const int64_t ctas = (a.rows + kWarpsPerCta - 1) / kWarpsPerCta;
    if (ctas > 0x7fffffffLL) return SS2D_EINVAL_SHAPE;
    if (a.dstate == 1)
        selscan_fwd_n1_kernel<Tin, Tout, VEC><<<(unsigned)ctas, kWarpsPerCta * 32, 0, st>>>(a);
    else
        selscan_fwd_nx_kernel<Tin, Tout, VEC><<<(unsigned)ctas, kWarpsPerCta * 32, 0, st>>>(a);
    count_launch();
    return check_launch();
}

template <typename Tin, typename Tout>
static int dispatch_vec(const ScanArgs& a, int vec, cudaStream_t st) {
    if constexpr (sizeof(Tin) == 2) {
        if (vec >= 8) return launch_scan<Tin, Tout, 8>(a, st);
    }
    if (vec >= 4) return launch_scan<Tin, Tout, 4>(a, st);
    if (vec >= 2) return launch_scan<Tin, Tout, 2>(a, st);
    return launch_scan<Tin, Tout, 1>(a, st);
}

// largest power of two v <= cap such that every listed quantity is a multiple of v
static int common_pow2(std::initializer_list<int64_t> xs, int cap) {
    int v = cap;
    for (int64_t x : xs) {
        if (x < 0) x = -x;
        while (v > 1 && (x % v) != 0) v >>= 1;
    }
    return v;
}

int selective_scan_fwd(const ss2d_scan_params* p, cudaStream_t st) {
    if (!p) return SS2D_EINVAL_NULL;
    if (!p->u || !p->delta || !p->A || !p->B || !p->C || !p->out) return SS2D_EINVAL_NULL;
    if (!dtype_ok(p->in_dtype) || !dtype_ok(p->out_dtype)) return SS2D_EINVAL_DTYPE;
    if (p->out_dtype != SS2D_F32 && p->out_dtype != p->in_dtype) return SS2D_EINVAL_DTYPE;
    if (p->batch <= 0 || p->dim <= 0 || p->dstate <= 0 || p->seqlen <= 0 || p->n_groups <= 0) return SS2D_EINVAL_SHAPE;
    if (p->dstate > SS2D_MAX_DSTATE) return SS2D_ENOTSUP;
    if (p->dim % p->n_groups != 0) return SS2D_EINVAL_SHAPE;
    if (p->delta_ratio < 0 || (p->delta_ratio > 1 && p->dim % p->delta_ratio != 0)) return SS2D_EINVAL_SHAPE;
    if (p->seqlen > 0x3fffffffLL) return SS2D_ENOTSUP;
    const int64_t L = p->seqlen;
    // rows must not overlap: |stride| >= extent of what it steps over
    if (p->u_dim_stride < L || p->delta_dim_stride < L || p->out_dim_stride < L) return SS2D_EINVAL_STRIDE;
    if (p->B_state_stride < L || p->C_state_stride < L) return SS2D_EINVAL_STRIDE;
    if (p->batch > 1 && (p->u_batch_stride < L || p->delta_batch_stride < L || p->out_batch_stride < L ||
                         p->B_batch_stride < L || p->C_batch_stride < L)) return SS2D_EINVAL_STRIDE;
    if (p->n_groups > 1 && (p->B_group_stride < L || p->C_group_stride < L)) return SS2D_EINVAL_STRIDE;
    const size_t si = dtype_size(p->in_dtype), so = dtype_size(p->out_dtype);
    if (!aligned_to(p->u, si) || !aligned_to(p->delta, si) || !aligned_to(p->B, si) || !aligned_to(p->C, si) ||
        !aligned_to(p->out, so) || !aligned_to(p->checkpoints, 4) || !aligned_to(p->A, 4) || !aligned_to(p->D, 4) || !aligned_to(p->delta_bias, 4))
        return SS2D_EINVAL_ALIGN;

    ScanArgs a;
    a.u = p->u; a.delta = p->delta; a.B = p->B; a.C = p->C;
    a.A = (const float*)p->A; a.D = (const float*)p->D; a.bias = (const float*)p->delta_bias;
    a.out = p->out;
    a.rows = p->batch * p->dim; a.dim = p->dim; a.dstate = p->dstate; a.seqlen = L;
    a.group_size = p->dim / p->n_groups;
    a.u_bs = p->u_batch_stride; a.u_ds = p->u_dim_stride;
    a.d_bs = p->delta_batch_stride; a.d_ds = p->delta_dim_stride;
    a.o_bs = p->out_batch_stride; a.o_ds = p->out_dim_stride;
    a.B_bs = p->B_batch_stride; a.B_gs = p->B_group_stride; a.B_ss = p->B_state_stride;
    a.C_bs = p->C_batch_stride; a.C_gs = p->C_group_stride; a.C_ss = p->C_state_stride;
    a.softplus = p->delta_softplus;
    a.dratio = p->delta_ratio > 1 ? p->delta_ratio : 1;
    a.ckpt = (float*)p->checkpoints; a.nck = (L + 127) / 128;

    // widest vector (in elements) that keeps every row start aligned for every tensor
    const int cap = (si == 2) ? 8 : 4;
    auto ptr_el = [](const void* q, size_t s) { return (int64_t)(reinterpret_cast<uintptr_t>(q) / s); };
    int vec = common_pow2({L, a.u_bs, a.u_ds, a.d_bs, a.d_ds, a.o_bs, a.o_ds, a.B_bs, a.B_gs, a.B_ss, a.C_bs, a.C_gs,
                           a.C_ss, ptr_el(p->u, si), ptr_el(p->delta, si), ptr_el(p->B, si), ptr_el(p->C, si),
                           ptr_el(p->out, so)}, cap);

    const int in = p->in_dtype;
    const bool of32 = p->out_dtype == SS2D_F32;
    if (in == SS2D_F32) return dispatch_vec<float, float>(a, vec, st);
    if (in == SS2D_BF16)
        return of32 ? dispatch_vec<__nv_bfloat16, float>(a, vec, st) : dispatch_vec<__nv_bfloat16, __nv_bfloat16>(a, vec, st);
    return of32 ? dispatch_vec<__half, float>(a, vec, st) : dispatch_vec<__half, __half>(a, vec, st);
}

}  // namespace ss2d
