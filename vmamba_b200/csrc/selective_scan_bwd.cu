// Selective-scan backward, operator surface: gradients of every input of selective_scan_fwd.
//
// With d' = softplus(delta + bias), a = exp(d' A), h_l = a_l h_{l-1} + d'_l B_l u_l and
// y_l = C_l . h_l + D u_l, an upstream gradient g = dout gives
//     dh_l  = C_l g_l + e_{l+1},   e_l = a_l dh_l                  (reverse recurrence, e_L = 0)
//     dC_l  = sum over the channels of a group of g_l h_l
//     dB_l  = sum over the channels of a group of dh_l d'_l u_l
//     du_l  = g_l D + d'_l sum_n B_l dh_l          dD    = sum_{b,l} g_l u_l
//     dd'_l = sum_n dh_l (B_l u_l + A a_l h_{l-1})  dA_n  = sum_{b,l} dh_l d'_l a_l h_{l-1}
//     ddelta_l = dd'_l * sigmoid(delta_l + bias) (1 above softplus' threshold 20),  dbias = sum_{b,l} ddelta_l
//
// Mapping: as in the forward kernel one warp owns one row (b, r) and walks it in steps of 32*VEC
// elements, a lane holding VEC consecutive elements.  The warps of a CTA own rows of the SAME
// (image, group), so that their contributions to dB / dC (which are shared by the channels of a
// group) are summed inside the CTA, in a fixed order, through shared memory.
//   pass 1 (forward over the row): the state entering every step is recomputed and kept in shared
//           memory (nothing is saved by the forward kernel);
//   pass 2 (backward over the steps): within a step the states h come from a forward shuffle scan
//           started at the saved state, e from a backward shuffle scan started at the carry of the
//           step after; every gradient of the step follows elementwise.
// Sums that cross CTAs (dB / dC over the CTAs of a group, dA / dD / dbias over the batch) go to an
// fp32 workspace as partials and are folded by a second kernel in a fixed order: no atomics, the
// result is bit-identical from run to run.
#include <type_traits>

#include "common.cuh"

namespace ss2d {

struct BwdArgs {
    const void *u, *delta, *B, *C, *dout;
    const float *A, *D, *bias;
    void *du, *ddelta;
    float* rowred;      // (batch, dim, N + 2): dA partials, dD, dbias of one row
    float* bcpart;      // (batch, n_groups, parts, 2, N, L): dB then dC partials of one CTA
    int64_t dim, seqlen, group_size;
    int64_t u_bs, u_ds, d_bs, d_ds, g_bs, g_ds;
    int64_t B_bs, B_gs, B_ss, C_bs, C_gs, C_ss;
    int N, n_groups, parts, nsteps, softplus;
    int64_t dratio;   // channels per delta row
    const float* ckpt;   // states in front of every 128th element (rows, nck, N), or null: recompute them
    int64_t nck;
    int64_t rows;        // batch * dim
};

template <typename Tin, typename Tg, int VEC>
__global__ void __launch_bounds__(256) selscan_bwd_kernel(const BwdArgs a) {
    extern __shared__ float sm[];
    constexpr int STEP = 32 * VEC;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, RW = blockDim.x >> 5;
    const int N = a.N, L = (int)a.seqlen, nsteps = a.nsteps;
    int cta = blockIdx.x;
    const int part = cta % a.parts; cta /= a.parts;
    const int k = cta % a.n_groups;
    const int64_t b = cta / a.n_groups;
    const int64_t in_group = (int64_t)part * RW + warp;
    const bool valid = in_group < a.group_size;
    const int64_t r = (int64_t)k * a.group_size + (valid ? in_group : 0);

    float* hstart = sm + (size_t)warp * nsteps * N;                        // [RW][nsteps][N]
    float* carry = sm + (size_t)RW * nsteps * N + (size_t)warp * N;         // [RW][N]
    float* A_s = sm + (size_t)RW * (nsteps + 1) * N + (size_t)warp * N;     // [RW][N]
    float* dA_s = sm + (size_t)RW * (nsteps + 2) * N + (size_t)warp * N;    // [RW][N]
    float* red = sm + (size_t)RW * (nsteps + 3) * N;                        // [RW][2][STEP]

    const Tin* __restrict__ u = (const Tin*)a.u + b * a.u_bs + r * a.u_ds;
    const Tin* __restrict__ dt = (const Tin*)a.delta + b * a.d_bs + (r / a.dratio) * a.d_ds;
    const Tg* __restrict__ gp = (const Tg*)a.dout + b * a.g_bs + r * a.g_ds;
    const Tin* __restrict__ Bm = (const Tin*)a.B + b * a.B_bs + k * a.B_gs;
    const Tin* __restrict__ Cm = (const Tin*)a.C + b * a.C_bs + k * a.C_gs;
    Tin* __restrict__ du = (Tin*)a.du + (b * a.dim + r) * L;
    Tin* __restrict__ dd = (Tin*)a.ddelta + (b * a.dim + r) * L;
    const bool has_D = a.D != nullptr;
    const float Dv = has_D ? __ldg(a.D + r) : 0.f;
    const float bias = a.bias ? __ldg(a.bias + r / a.dratio) : 0.f;
    const bool sp = a.softplus != 0;
    using VI = Vec<Tin, VEC>;
    using VG = Vec<Tg, VEC>;

    for (int n = lane; n < N; n += 32) {
        carry[n] = 0.f; dA_s[n] = 0.f;
        A_s[n] = __ldg(a.A + r * N + n);
    }
    __syncwarp();

    // ---- pass 1: the state entering every step (from the forward call's checkpoints when the steps line up) ------
    const bool have_ckpt = a.ckpt != nullptr && STEP == 128;
    if (have_ckpt) {
        const float* ck = a.ckpt + (b * a.dim + r) * a.nck * N;
        for (int i = lane; i < nsteps * N; i += 32) hstart[i] = valid ? ck[i] : 0.f;
    }
    for (int s = 0; s < (have_ckpt ? 0 : nsteps); ++s) {
        const int pos = s * STEP + lane * VEC;
        const bool in = valid && pos < L;
        float uv[VEC], dl[VEC];
        if (in) { VI::load(u + pos, uv); VI::load(dt + pos, dl); }
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            if (in) { float d = dl[i] + bias; if (sp) d = softplus_fast(d); dl[i] = d; uv[i] *= d; }
            else { dl[i] = 0.f; uv[i] = 0.f; }
        }
        for (int n = 0; n < N; ++n) {
            float bv[VEC];
            if (in) VI::load(Bm + n * a.B_ss + pos, bv);
            const float A2 = A_s[n] * kLog2e;
            float p = 1.f, h = 0.f;
#pragma unroll
            for (int i = 0; i < VEC; ++i) {
                const float aa = in ? decay_fast(dl[i], A2) : 1.f;
                h = fmaf(aa, h, in ? uv[i] * bv[i] : 0.f);
                p *= aa;
            }
            const AB inc = warp_scan_inclusive(AB{p, h}, lane);
            const float ta = __shfl_sync(0xffffffffu, inc.a, 31), tb = __shfl_sync(0xffffffffu, inc.b, 31);
            const float hc = carry[n];
            __syncwarp();
            if (lane == 0) { hstart[s * N + n] = hc; carry[n] = fmaf(ta, hc, tb); }
            __syncwarp();
        }
    }
    for (int n = lane; n < N; n += 32) carry[n] = 0.f;     // from here on: e entering the step from behind
    __syncwarp();

    // ---- pass 2: backwards over the steps ----------------------------------------------------------
    float dD_acc = 0.f, dbias_acc = 0.f;
    float* bc_out = a.bcpart + (((size_t)b * a.n_groups + k) * a.parts + part) * 2 * (size_t)N * L;
    for (int s = nsteps - 1; s >= 0; --s) {
        const int pos = s * STEP + lane * VEC;
        const bool in = valid && pos < L;
        float uv[VEC], dl[VEC], gv[VEC], dsp[VEC], du_acc[VEC], ddl[VEC];
        if (in) { VI::load(u + pos, uv); VI::load(dt + pos, dl); VG::load(gp + pos, gv); }
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            if (in) {
                float x = dl[i] + bias;
                dsp[i] = 1.f;
                if (sp) softplus_and_grad(x, x, dsp[i]);
                dl[i] = x;
            } else { dl[i] = 0.f; uv[i] = 0.f; gv[i] = 0.f; dsp[i] = 0.f; }
            du_acc[i] = has_D ? gv[i] * Dv : 0.f;
            ddl[i] = 0.f;
            dD_acc = fmaf(gv[i], uv[i], dD_acc);
        }
        for (int n = 0; n < N; ++n) {
            float bv[VEC], cv[VEC], av[VEC], P[VEC], hl[VEC], Q[VEC], El[VEC];
            if (in) { VI::load(Bm + n * a.B_ss + pos, bv); VI::load(Cm + n * a.C_ss + pos, cv); }
            else {
#pragma unroll
                for (int i = 0; i < VEC; ++i) { bv[i] = 0.f; cv[i] = 0.f; }
            }
            const float An = A_s[n], A2 = An * kLog2e;
            float p = 1.f, h = 0.f;
#pragma unroll
            for (int i = 0; i < VEC; ++i) {
                av[i] = in ? decay_fast(dl[i], A2) : 1.f;
                h = fmaf(av[i], h, dl[i] * uv[i] * bv[i]);
                p *= av[i];
                P[i] = p; hl[i] = h;
            }
            float q = 1.f, e = 0.f;
#pragma unroll
            for (int i = VEC - 1; i >= 0; --i) {
                e = av[i] * fmaf(cv[i], gv[i], e);
                q *= av[i];
                Q[i] = q; El[i] = e;
            }
            const AB fi = warp_scan_inclusive(AB{p, h}, lane);
            const AB ri = warp_scan_inclusive_rev(AB{q, e}, lane);
            float ea = __shfl_up_sync(0xffffffffu, fi.a, 1), eb = __shfl_up_sync(0xffffffffu, fi.b, 1);
            if (lane == 0) { ea = 1.f; eb = 0.f; }
            float ra = __shfl_down_sync(0xffffffffu, ri.a, 1), rb = __shfl_down_sync(0xffffffffu, ri.b, 1);
            if (lane == 31) { ra = 1.f; rb = 0.f; }
            const float hin = fmaf(ea, hstart[s * N + n], eb);       // h just before this lane's first element
            const float ec = carry[n];
            const float ein = fmaf(ra, ec, rb);                      // e just after this lane's last element
            const float ca = __shfl_sync(0xffffffffu, ri.a, 0), cb = __shfl_sync(0xffffffffu, ri.b, 0);
            __syncwarp();
            if (lane == 0) carry[n] = fmaf(ca, ec, cb);
            float dBv[VEC], dCv[VEC], dA_loc = 0.f;
#pragma unroll
            for (int i = 0; i < VEC; ++i) {
                const float hprev = (i == 0) ? hin : fmaf(P[i > 0 ? i - 1 : 0], hin, hl[i > 0 ? i - 1 : 0]);
                const float hi = fmaf(P[i], hin, hl[i]);
                const float enext = (i + 1 < VEC) ? fmaf(Q[i + 1 < VEC ? i + 1 : i], ein, El[i + 1 < VEC ? i + 1 : i]) : ein;
                const float dh = fmaf(cv[i], gv[i], enext);
                dCv[i] = gv[i] * hi;
                dBv[i] = dh * dl[i] * uv[i];
                du_acc[i] = fmaf(dh * dl[i], bv[i], du_acc[i]);
                const float t = av[i] * hprev;
                ddl[i] = fmaf(dh, fmaf(An, t, bv[i] * uv[i]), ddl[i]);
                dA_loc = fmaf(dh * dl[i], t, dA_loc);
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) dA_loc += __shfl_xor_sync(0xffffffffu, dA_loc, off);
            if (lane == 0) dA_s[n] += dA_loc;
            // sum of the CTA's rows for this (step, state), in warp order
            float* my = red + (size_t)warp * 2 * STEP + lane * VEC;
#pragma unroll
            for (int i = 0; i < VEC; ++i) { my[i] = in ? dBv[i] : 0.f; my[STEP + i] = in ? dCv[i] : 0.f; }
            __syncthreads();
            for (int idx = threadIdx.x; idx < 2 * STEP; idx += blockDim.x) {
                const int which = idx / STEP, el = idx - which * STEP;
                const int gpos = s * STEP + el;
                if (gpos < L) {
                    float acc = 0.f;
                    for (int w = 0; w < RW; ++w) acc += red[(size_t)w * 2 * STEP + idx];
                    bc_out[((size_t)which * N + n) * L + gpos] = acc;
                }
            }
            __syncthreads();
        }
        if (in) {
            float dv[VEC];
#pragma unroll
            for (int i = 0; i < VEC; ++i) { dv[i] = ddl[i] * dsp[i]; dbias_acc += dv[i]; }
            VI::store(du + pos, du_acc);
            VI::store(dd + pos, dv);
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        dD_acc += __shfl_xor_sync(0xffffffffu, dD_acc, off);
        dbias_acc += __shfl_xor_sync(0xffffffffu, dbias_acc, off);
    }
    __syncwarp();
    if (valid) {
        float* rr = a.rowred + (b * a.dim + r) * (N + 2);
        for (int n = lane; n < N; n += 32) rr[n] = dA_s[n];
        if (lane == 0) { rr[N] = dD_acc; rr[N + 1] = dbias_acc; }
    }
}

// d_state 1 (every VMamba backbone): a warp walks R rows of the group per step, so that the B / C
// vectors of the step are loaded once per warp, the dB / dC contributions of its rows are summed in
// registers, and the CTA-wide sum (two barriers) is paid once per step for RW * R rows.  The next
// row's u / delta / dout vectors are fetched before the current row's arithmetic.
template <typename Tin, typename Tg, int VEC>
__global__ void __launch_bounds__(256) selscan_bwd_n1_kernel(const BwdArgs a, const int R) {
    extern __shared__ float sm[];
    constexpr int STEP = 32 * VEC;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, RW = blockDim.x >> 5;
    const int L = (int)a.seqlen, nsteps = a.nsteps;
    int cta = blockIdx.x;
    const int part = cta % a.parts; cta /= a.parts;
    const int k = cta % a.n_groups;
    const int64_t b = cta / a.n_groups;
    const int rows_cta = RW * R;
    // local row lr = i * RW + warp, i < R; row inside the group = part * rows_cta + lr
    float* hstart = sm;                                   // [rows_cta][nsteps]
    float* ecar = sm + (size_t)rows_cta * nsteps;         // [rows_cta]
    float* racc = ecar + rows_cta;                        // [rows_cta][3][32]: per-lane partials of dA, dD, dbias
    float* red = racc + (size_t)rows_cta * 96;            // [RW][2][STEP]
    const bool has_D = a.D != nullptr;
    const bool sp = a.softplus != 0;
    using VI = Vec<Tin, VEC>;
    using VG = Vec<Tg, VEC>;
    const Tin* __restrict__ Bm = (const Tin*)a.B + b * a.B_bs + k * a.B_gs;
    const Tin* __restrict__ Cm = (const Tin*)a.C + b * a.C_bs + k * a.C_gs;
    const int64_t row0 = (int64_t)part * rows_cta;

    // ---- pass 1: the state entering every step, row by row ------------------------------------------
    for (int i = 0; i < R; ++i) {
        const int lr = i * RW + warp;
        const int64_t ig = row0 + lr;
#pragma unroll
        for (int j = 0; j < 3; ++j) racc[lr * 96 + j * 32 + lane] = 0.f;
        if (lane == 0) ecar[lr] = 0.f;
        if (ig >= a.group_size) continue;               // uniform over the warp
        const int64_t r = (int64_t)k * a.group_size + ig;
        if (a.ckpt != nullptr && STEP == 128) {         // the forward call left the step states: no recomputation
            const float* ck = a.ckpt + (b * a.dim + r) * a.nck;
            for (int s = lane; s < nsteps; s += 32) hstart[(size_t)lr * nsteps + s] = ck[s];
            continue;
        }
        const Tin* __restrict__ u = (const Tin*)a.u + b * a.u_bs + r * a.u_ds;
        const Tin* __restrict__ dt = (const Tin*)a.delta + b * a.d_bs + (r / a.dratio) * a.d_ds;
        const float A2 = __ldg(a.A + r) * kLog2e;
        const float bias = a.bias ? __ldg(a.bias + r / a.dratio) : 0.f;
        float hc = 0.f;
        typename VI::Raw ru = {}, rd = {}, rb = {};
        int pos = lane * VEC;
        if (pos < L) { ru = VI::load_raw(u + pos); rd = VI::load_raw(dt + pos); rb = VI::load_raw(Bm + pos); }
        for (int s = 0; s < nsteps; ++s) {
            typename VI::Raw nu = {}, nd = {}, nb = {};
            const int npos = pos + STEP;
            if (npos < L) { nu = VI::load_raw(u + npos); nd = VI::load_raw(dt + npos); nb = VI::load_raw(Bm + npos); }
            const bool in = pos < L;
            float uv[VEC], dl[VEC], bv[VEC];
            VI::unpack(ru, uv); VI::unpack(rd, dl); VI::unpack(rb, bv);
            float p = 1.f, h = 0.f;
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                float d = dl[e] + bias;
                if (sp) d = softplus_fast(d);
                const float aa = in ? decay_fast(d, A2) : 1.f;
                h = fmaf(aa, h, in ? d * uv[e] * bv[e] : 0.f);
                p *= aa;
            }
            const AB inc = warp_scan_inclusive(AB{p, h}, lane);
            const float ta = __shfl_sync(0xffffffffu, inc.a, 31), tb = __shfl_sync(0xffffffffu, inc.b, 31);
            if (lane == 0) hstart[(size_t)lr * nsteps + s] = hc;
            hc = fmaf(ta, hc, tb);
            ru = nu; rd = nd; rb = nb; pos = npos;
        }
    }
    __syncwarp();

    // ---- pass 2: backwards over the steps; inside a step over this warp's rows ------------------------
    float* bc_out = a.bcpart + (((size_t)b * a.n_groups + k) * a.parts + part) * 2 * (size_t)L;
    for (int s = nsteps - 1; s >= 0; --s) {
        const int pos = s * STEP + lane * VEC;
        const bool in_l = pos < L;
        float bv[VEC], cv[VEC], accB[VEC], accC[VEC];
        if (in_l) { VI::load(Bm + pos, bv); VI::load(Cm + pos, cv); }
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            if (!in_l) { bv[e] = 0.f; cv[e] = 0.f; }
            accB[e] = 0.f; accC[e] = 0.f;
        }
        // first row's vectors
        typename VI::Raw ru = {}, rd = {};
        typename VG::Raw rg = {};
        auto fetch = [&](int i, typename VI::Raw& xu, typename VI::Raw& xd, typename VG::Raw& xg) {
            const int64_t ig = row0 + i * RW + warp;
            if (i < R && ig < a.group_size && in_l) {
                const int64_t r = (int64_t)k * a.group_size + ig;
                xu = VI::load_raw((const Tin*)a.u + b * a.u_bs + r * a.u_ds + pos);
                xd = VI::load_raw((const Tin*)a.delta + b * a.d_bs + (r / a.dratio) * a.d_ds + pos);
                xg = VG::load_raw((const Tg*)a.dout + b * a.g_bs + r * a.g_ds + pos);
            }
        };
        fetch(0, ru, rd, rg);
        for (int i = 0; i < R; ++i) {
            typename VI::Raw nu = {}, nd = {};
            typename VG::Raw ng = {};
            fetch(i + 1, nu, nd, ng);
            const int lr = i * RW + warp;
            const int64_t ig = row0 + lr;
            if (ig < a.group_size) {                    // uniform over the warp
                const int64_t r = (int64_t)k * a.group_size + ig;
                const float An = __ldg(a.A + r), A2 = An * kLog2e;
                const float bias = a.bias ? __ldg(a.bias + r / a.dratio) : 0.f;
                const float Dv = has_D ? __ldg(a.D + r) : 0.f;
                float uv[VEC], dl[VEC], gv[VEC], dsp[VEC], av[VEC], P[VEC], hl[VEC], Q[VEC], El[VEC];
                VI::unpack(ru, uv); VI::unpack(rd, dl); VG::unpack(rg, gv);
                float p = 1.f, h = 0.f, dD_loc = 0.f;
#pragma unroll
                for (int e = 0; e < VEC; ++e) {
                    if (in_l) {
                        float x = dl[e] + bias;
                        dsp[e] = 1.f;
                        if (sp) softplus_and_grad(x, x, dsp[e]);
                        dl[e] = x;
                        av[e] = decay_fast(x, A2);
                    } else { dl[e] = 0.f; uv[e] = 0.f; gv[e] = 0.f; dsp[e] = 0.f; av[e] = 1.f; }
                    dD_loc = fmaf(gv[e], uv[e], dD_loc);
                    h = fmaf(av[e], h, dl[e] * uv[e] * bv[e]);
                    p *= av[e];
                    P[e] = p; hl[e] = h;
                }
                float q = 1.f, ee = 0.f;
#pragma unroll
                for (int e = VEC - 1; e >= 0; --e) {
                    ee = av[e] * fmaf(cv[e], gv[e], ee);
                    q *= av[e];
                    Q[e] = q; El[e] = ee;
                }
                const AB fi = warp_scan_inclusive(AB{p, h}, lane);
                const AB ri = warp_scan_inclusive_rev(AB{q, ee}, lane);
                float ea = __shfl_up_sync(0xffffffffu, fi.a, 1), eb = __shfl_up_sync(0xffffffffu, fi.b, 1);
                if (lane == 0) { ea = 1.f; eb = 0.f; }
                float ra = __shfl_down_sync(0xffffffffu, ri.a, 1), rb = __shfl_down_sync(0xffffffffu, ri.b, 1);
                if (lane == 31) { ra = 1.f; rb = 0.f; }
                const float hin = fmaf(ea, hstart[(size_t)lr * nsteps + s], eb);
                const float ec = ecar[lr];
                const float ein = fmaf(ra, ec, rb);
                const float ca = __shfl_sync(0xffffffffu, ri.a, 0), cb = __shfl_sync(0xffffffffu, ri.b, 0);
                __syncwarp();
                if (lane == 0) ecar[lr] = fmaf(ca, ec, cb);
                float duv[VEC], ddv[VEC], dA_loc = 0.f, db_loc = 0.f;
#pragma unroll
                for (int e = 0; e < VEC; ++e) {
                    const float hprev = (e == 0) ? hin : fmaf(P[e > 0 ? e - 1 : 0], hin, hl[e > 0 ? e - 1 : 0]);
                    const float hi = fmaf(P[e], hin, hl[e]);
                    const float enext = (e + 1 < VEC) ? fmaf(Q[e + 1 < VEC ? e + 1 : e], ein, El[e + 1 < VEC ? e + 1 : e]) : ein;
                    const float dh = fmaf(cv[e], gv[e], enext);
                    accC[e] = fmaf(gv[e], hi, accC[e]);
                    const float dhd = dh * dl[e];
                    accB[e] = fmaf(dhd, uv[e], accB[e]);
                    duv[e] = fmaf(dhd, bv[e], has_D ? gv[e] * Dv : 0.f);
                    const float t = av[e] * hprev;
                    ddv[e] = dh * fmaf(An, t, bv[e] * uv[e]) * dsp[e];
                    db_loc += ddv[e];
                    dA_loc = fmaf(dhd, t, dA_loc);
                }
                float* rq = racc + lr * 96 + lane;
                rq[0] += dA_loc; rq[32] += dD_loc; rq[64] += db_loc;
                if (in_l) {
                    VI::store((Tin*)a.du + (b * a.dim + r) * L + pos, duv);
                    VI::store((Tin*)a.ddelta + (b * a.dim + r) * L + pos, ddv);
                }
            }
            ru = nu; rd = nd; rg = ng;
        }
        float* my = red + (size_t)warp * 2 * STEP + lane * VEC;
#pragma unroll
        for (int e = 0; e < VEC; ++e) { my[e] = accB[e]; my[STEP + e] = accC[e]; }
        __syncthreads();
        for (int idx = threadIdx.x; idx < 2 * STEP; idx += blockDim.x) {
            const int which = idx / STEP, el = idx - which * STEP;
            const int gpos = s * STEP + el;
            if (gpos < L) {
                float acc = 0.f;
                for (int w = 0; w < RW; ++w) acc += red[(size_t)w * 2 * STEP + idx];
                bc_out[(size_t)which * L + gpos] = acc;
            }
        }
        __syncthreads();
    }
    // ---- per-row sums ------------------------------------------------------------------------------------
    for (int i = 0; i < R; ++i) {
        const int lr = i * RW + warp;
        const int64_t ig = row0 + lr;
        if (ig >= a.group_size) continue;
        const int64_t r = (int64_t)k * a.group_size + ig;
        float v0 = racc[lr * 96 + lane], v1 = racc[lr * 96 + 32 + lane], v2 = racc[lr * 96 + 64 + lane];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            v0 += __shfl_xor_sync(0xffffffffu, v0, off);
            v1 += __shfl_xor_sync(0xffffffffu, v1, off);
            v2 += __shfl_xor_sync(0xffffffffu, v2, off);
        }
        if (lane == 0) {
            float* rr = a.rowred + (b * a.dim + r) * 3;
            rr[0] = v0; rr[1] = v1; rr[2] = v2;
        }
    }
}

// d_state 1 with many rows and the forward call's checkpoints: LANES ARE ROWS.  A warp owns 32 consecutive rows of one
// (image, group); every lane walks its own row, so the two recurrences are plain fused multiply-adds per element (no
// running products, no shuffle scans, no CTA barrier), the per-row sums (dA, dD, dbias) stay in registers, and the
// sums over the rows of a group (dB, dC) are column sums of a shared tile.  The row is walked chunk by chunk (128
// elements, the checkpoint interval) from its end: a forward sweep over the chunk leaves the state in front of each of
// its eight 16-element tiles, then the tiles are taken in reverse: forward over the tile with the states kept in
// registers, backward over the same 16 elements.  Tiles are staged as in the forward lanes-are-rows kernel: pieces of
// four elements in, fp32 transposed ([element][row], pitch 33) in shared memory, du / ddelta out through the same
// buffers.  The chunk is read twice (sweep, then tiles); the second read finds it in L2.
constexpr int kBwdTile = 16, kBwdRowsWarps = 4, kBwdPitch = 33;
constexpr int kBwdFloatsPerWarp = 4 * kBwdTile * kBwdPitch + 8 * 32 + 2 * kBwdTile;

template <typename Tin, typename Tg>
__global__ void __launch_bounds__(kBwdRowsWarps * 32, 4) selscan_bwd_rows_kernel(const BwdArgs a) {
    extern __shared__ float sm[];
    constexpr int T = kBwdTile, P = kBwdPitch, PE = 4;         // PE: elements per piece (8 bytes of a 16-bit tensor)
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* su = sm + (size_t)warp * kBwdFloatsPerWarp;         // u, then du
    float* sd = su + T * P;                                    // delta, then ddelta
    float* sg = sd + T * P;                                    // dout, then the rows' dB terms
    float* sx = sg + T * P;                                    // the rows' dC terms
    float* hs = sx + T * P;                                    // [tile of the chunk][row]: state in front of the tile
    float* sB = hs + 8 * 32;
    float* sC = sB + T;
    const int64_t row0 = ((int64_t)blockIdx.x * kBwdRowsWarps + warp) * 32;
    const int L = (int)a.seqlen;
    if (row0 >= a.rows) return;
    const int64_t b = row0 / a.dim, r0 = row0 % a.dim, k = r0 / a.group_size, part = (r0 - k * a.group_size) / 32;
    const int64_t r = r0 + lane;
    const Tin* __restrict__ u = (const Tin*)a.u + b * a.u_bs + r0 * a.u_ds;
    const Tin* __restrict__ dt = (const Tin*)a.delta + b * a.d_bs + r0 * a.d_ds;
    const Tg* __restrict__ gp = (const Tg*)a.dout + b * a.g_bs + r0 * a.g_ds;
    const Tin* __restrict__ Bm = (const Tin*)a.B + b * a.B_bs + k * a.B_gs;
    const Tin* __restrict__ Cm = (const Tin*)a.C + b * a.C_bs + k * a.C_gs;
    Tin* __restrict__ du = (Tin*)a.du + (b * a.dim + r0) * L;
    Tin* __restrict__ dd = (Tin*)a.ddelta + (b * a.dim + r0) * L;
    float* __restrict__ bc_out = a.bcpart + (((size_t)b * a.n_groups + k) * a.parts + part) * 2 * (size_t)L;
    const float* __restrict__ ck = a.ckpt + (b * a.dim + r) * a.nck;
    const float An = __ldg(a.A + r), A2 = An * kLog2e;
    const bool has_D = a.D != nullptr;
    const float Dv = has_D ? __ldg(a.D + r) : 0.f;
    const float bias = a.bias ? __ldg(a.bias + r) : 0.f;
    const bool sp = a.softplus != 0;
    using VI = Vec<Tin, PE>;
    using VG = Vec<Tg, PE>;

    // a tile of 32 rows x 16 elements of one tensor: four pieces per lane in, fp32 transposed out
    auto stage_in = [&](auto* src, int64_t stride, int t0, float* dst) {
        using E = std::remove_cv_t<std::remove_pointer_t<decltype(src)>>;
#pragma unroll
        for (int j = 0; j < T / PE; ++j) {
            const int idx = j * 32 + lane, rr = idx / (T / PE), piece = idx - rr * (T / PE);
            const int pos = t0 + piece * PE;
            float v[PE];
            if (pos < L) Vec<E, PE>::load(src + rr * stride + pos, v);
            else {
#pragma unroll
                for (int e = 0; e < PE; ++e) v[e] = 0.f;
            }
#pragma unroll
            for (int e = 0; e < PE; ++e) dst[(piece * PE + e) * P + rr] = v[e];
        }
    };
    auto stage_row = [&](const Tin* src, int t0, float* dst, int first_lane) {     // one row of 16 elements (B or C)
        const int piece = lane - first_lane;
        if (piece >= 0 && piece < T / PE) {
            const int pos = t0 + piece * PE;
            float v[PE];
            if (pos < L) VI::load(src + pos, v);
            else {
#pragma unroll
                for (int e = 0; e < PE; ++e) v[e] = 0.f;
            }
#pragma unroll
            for (int e = 0; e < PE; ++e) dst[piece * PE + e] = v[e];
        }
    };
    auto stage_out = [&](const float* src, Tin* dst_rows, int t0) {
#pragma unroll
        for (int j = 0; j < T / PE; ++j) {
            const int idx = j * 32 + lane, rr = idx / (T / PE), piece = idx - rr * (T / PE);
            const int pos = t0 + piece * PE;
            if (pos < L) {
                float v[PE];
#pragma unroll
                for (int e = 0; e < PE; ++e) v[e] = src[(piece * PE + e) * P + rr];
                VI::store(dst_rows + (int64_t)rr * L + pos, v);
            }
        }
    };

    float e_carry = 0.f, dA_acc = 0.f, dD_acc = 0.f, db_acc = 0.f;
    for (int c = (int)a.nck - 1; c >= 0; --c) {
        const int c0 = c * 128;
        const int ntiles = min(8, (L - c0 + T - 1) / T);
        // ---- forward sweep over the chunk: the state in front of each tile
        float h = ck[c];
        for (int j = 0; j < ntiles; ++j) {
            hs[j * 32 + lane] = h;
            if (j == ntiles - 1) break;
            const int t0 = c0 + j * T;                         // a whole tile: it is not the last of the row
            stage_in(u, a.u_ds, t0, su);
            stage_in(dt, a.d_ds, t0, sd);
            stage_row(Bm, t0, sB, 0);
            __syncwarp();
#pragma unroll 4
            for (int t = 0; t < T; ++t) {
                float d = sd[t * P + lane] + bias;
                if (sp) d = softplus_fast(d);
                h = fmaf(decay_fast(d, A2), h, d * su[t * P + lane] * sB[t]);
            }
            __syncwarp();
        }
        // ---- the tiles of the chunk, last first
        for (int j = ntiles - 1; j >= 0; --j) {
            const int t0 = c0 + j * T;
            stage_in(u, a.u_ds, t0, su);
            stage_in(dt, a.d_ds, t0, sd);
            stage_in(gp, a.g_ds, t0, sg);
            stage_row(Bm, t0, sB, 0);
            stage_row(Cm, t0, sC, 4);
            __syncwarp();
            float av[T], dv[T], hl[T], ds[T];
            const float hstart = hs[j * 32 + lane];
            h = hstart;
#pragma unroll
            for (int t = 0; t < T; ++t) {
                const bool ok = t0 + t < L;                    // beyond the row: a = 1, everything else 0
                float x = sd[t * P + lane] + bias, g1 = 1.f;
                if (sp) softplus_and_grad(x, x, g1);
                x = ok ? x : 0.f;
                ds[t] = ok ? g1 : 0.f;
                dv[t] = x;
                av[t] = decay_fast(x, A2);
                h = fmaf(av[t], h, x * su[t * P + lane] * sB[t]);
                hl[t] = h;
            }
#pragma unroll
            for (int t = T - 1; t >= 0; --t) {
                const float g = sg[t * P + lane], uv = su[t * P + lane], Bt = sB[t], Ct = sC[t];
                const float dh = fmaf(Ct, g, e_carry);
                const float hprev = t == 0 ? hstart : hl[t > 0 ? t - 1 : 0];
                const float dhd = dh * dv[t];
                const float tt = av[t] * hprev;
                const float ddl = dh * fmaf(An, tt, Bt * uv) * ds[t];
                su[t * P + lane] = fmaf(dhd, Bt, has_D ? g * Dv : 0.f);      // du
                sd[t * P + lane] = ddl;                                     // ddelta
                sg[t * P + lane] = dhd * uv;                                // this row's dB term
                sx[t * P + lane] = g * hl[t];                               // this row's dC term
                dA_acc = fmaf(dhd, tt, dA_acc);
                dD_acc = fmaf(g, uv, dD_acc);
                db_acc += ddl;
                e_carry = av[t] * dh;
            }
            __syncwarp();
            {   // sums over the 32 rows: lanes 0..15 the dB of element lane, lanes 16..31 the dC of element lane - 16
                const int el = lane & 15;
                const float* src = (lane < 16 ? sg : sx) + el * P;
                float acc = 0.f;
#pragma unroll
                for (int rr = 0; rr < 32; ++rr) acc += src[rr];
                if (t0 + el < L) bc_out[(size_t)(lane >> 4) * L + t0 + el] = acc;
            }
            stage_out(su, du, t0);
            stage_out(sd, dd, t0);
            __syncwarp();
        }
    }
    float* rr = a.rowred + (b * a.dim + r) * 3;
    rr[0] = dA_acc; rr[1] = dD_acc; rr[2] = db_acc;
}

// d_state 4 / 8 / 16 with many rows and the forward call's checkpoints: lanes are rows, as above, with the NS states of
// a row in registers.  Per chunk of 128 elements a forward sweep leaves the NS states in front of tiles 1..7 in shared
// memory; a tile is then taken state by state (forward over its 16 elements with the decays and states kept in
// registers, then backward), two sums over the states (from which du and ddelta follow) accumulating in registers, the
// rows' dB / dC terms of one state going through two shared tiles whose columns are summed by the warp.  dout, the step
// sizes, their products with u and the two sums of the tile stay in registers, so that the shared-memory traffic per
// (element, state) is the broadcast loads of B and C, two stores and the column sums.  That traffic and the two
// transcendentals per (element, state) bound the kernel: a form with 8-element tiles and twice the warps per SM ran at
// the same speed.
template <int NS> struct BwdRowsN {
    static constexpr int kFloatsPerWarp = 5 * kBwdTile * kBwdPitch + 7 * NS * 32 + 2 * NS * kBwdTile;
};

template <typename Tin, typename Tg, int NS>
__global__ void __launch_bounds__(kBwdRowsWarps * 32, 2) selscan_bwd_rows_nx_kernel(const BwdArgs a) {
    extern __shared__ float sm[];
    constexpr int T = kBwdTile, P = kBwdPitch, PE = 4;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* su = sm + (size_t)warp * BwdRowsN<NS>::kFloatsPerWarp;   // u, then du
    float* sd = su + T * P;                                    // delta, then ddelta
    float* sg = sd + T * P;                                    // dout, then the derivative of the softplus
    float* sb = sg + T * P;                                    // the rows' dB terms of one state
    float* sc = sb + T * P;                                    // the rows' dC terms of one state
    float* hs = sc + T * P;                                    // [tile 1..7 of the chunk][state][row]
    float* sB = hs + 7 * NS * 32;                              // [state][element]
    float* sC = sB + NS * T;
    const int64_t row0 = ((int64_t)blockIdx.x * kBwdRowsWarps + warp) * 32;
    const int L = (int)a.seqlen;
    if (row0 >= a.rows) return;
    const int64_t b = row0 / a.dim, r0 = row0 % a.dim, k = r0 / a.group_size, part = (r0 - k * a.group_size) / 32;
    const int64_t r = r0 + lane;
    const Tin* __restrict__ u = (const Tin*)a.u + b * a.u_bs + r0 * a.u_ds;
    const Tin* __restrict__ dt = (const Tin*)a.delta + b * a.d_bs + r0 * a.d_ds;
    const Tg* __restrict__ gp = (const Tg*)a.dout + b * a.g_bs + r0 * a.g_ds;
    const Tin* __restrict__ Bm = (const Tin*)a.B + b * a.B_bs + k * a.B_gs;
    const Tin* __restrict__ Cm = (const Tin*)a.C + b * a.C_bs + k * a.C_gs;
    Tin* __restrict__ du = (Tin*)a.du + (b * a.dim + r0) * L;
    Tin* __restrict__ dd = (Tin*)a.ddelta + (b * a.dim + r0) * L;
    float* __restrict__ bc_out = a.bcpart + (((size_t)b * a.n_groups + k) * a.parts + part) * 2 * (size_t)NS * L;
    const float* __restrict__ ck = a.ckpt + (b * a.dim + r) * a.nck * NS;
    float A2[NS], e_carry[NS], dA_acc[NS];
#pragma unroll
    for (int n = 0; n < NS; ++n) { A2[n] = __ldg(a.A + r * NS + n) * kLog2e; e_carry[n] = 0.f; dA_acc[n] = 0.f; }
    const bool has_D = a.D != nullptr;
    const float Dv = has_D ? __ldg(a.D + r) : 0.f;
    const float bias = a.bias ? __ldg(a.bias + r) : 0.f;
    const bool sp = a.softplus != 0;
    using VI = Vec<Tin, PE>;

    auto stage_in = [&](auto* src, int64_t stride, int t0, float* dst) {
        using E = std::remove_cv_t<std::remove_pointer_t<decltype(src)>>;
#pragma unroll
        for (int j = 0; j < T / PE; ++j) {
            const int idx = j * 32 + lane, rr = idx / (T / PE), piece = idx - rr * (T / PE);
            const int pos = t0 + piece * PE;
            float v[PE];
            if (pos < L) Vec<E, PE>::load(src + rr * stride + pos, v);
            else {
#pragma unroll
                for (int e = 0; e < PE; ++e) v[e] = 0.f;
            }
#pragma unroll
            for (int e = 0; e < PE; ++e) dst[(piece * PE + e) * P + rr] = v[e];
        }
    };
    // the NS rows of B (and of C) for a tile: 4 pieces of four elements per row
    auto stage_bc = [&](int t0, bool with_c) {
        constexpr int PIECES = NS * (T / PE);
        for (int idx = lane; idx < (with_c ? 2 : 1) * PIECES; idx += 32) {
            const int which = idx / PIECES, rem = idx - which * PIECES, n = rem / (T / PE), piece = rem - n * (T / PE);
            const int pos = t0 + piece * PE;
            const Tin* src = which ? Cm + n * a.C_ss : Bm + n * a.B_ss;
            float v[PE];
            if (pos < L) VI::load(src + pos, v);
            else {
#pragma unroll
                for (int e = 0; e < PE; ++e) v[e] = 0.f;
            }
            float* dst = (which ? sC : sB) + n * T + piece * PE;
#pragma unroll
            for (int e = 0; e < PE; ++e) dst[e] = v[e];
        }
    };
    auto stage_out = [&](const float* src, Tin* dst_rows, int t0) {
#pragma unroll
        for (int j = 0; j < T / PE; ++j) {
            const int idx = j * 32 + lane, rr = idx / (T / PE), piece = idx - rr * (T / PE);
            const int pos = t0 + piece * PE;
            if (pos < L) {
                float v[PE];
#pragma unroll
                for (int e = 0; e < PE; ++e) v[e] = src[(piece * PE + e) * P + rr];
                VI::store(dst_rows + (int64_t)rr * L + pos, v);
            }
        }
    };

    float dD_acc = 0.f, db_acc = 0.f;
    for (int c = (int)a.nck - 1; c >= 0; --c) {
        const int c0 = c * 128;
        const int ntiles = min(8, (L - c0 + T - 1) / T);
        if (c > 0) {     // the chunk in front of this one, on its way into L2 while this one is worked on (a row per lane)
            const char* pu = reinterpret_cast<const char*>(u + lane * a.u_ds + c0 - 128);
            const char* pd = reinterpret_cast<const char*>(dt + lane * a.d_ds + c0 - 128);
            const char* pg = reinterpret_cast<const char*>(gp + lane * a.g_ds + c0 - 128);
#pragma unroll
            for (int i = 0; i < 128 * (int)sizeof(Tin); i += 128) {
                asm volatile("prefetch.global.L2 [%0];" ::"l"(pu + i));
                asm volatile("prefetch.global.L2 [%0];" ::"l"(pd + i));
            }
#pragma unroll
            for (int i = 0; i < 128 * (int)sizeof(Tg); i += 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(pg + i));
        }
        // ---- forward sweep over the chunk: the states in front of tiles 1 .. ntiles-1
        {
            float h[NS];
#pragma unroll
            for (int n = 0; n < NS; ++n) h[n] = ck[c * NS + n];
            for (int j = 0; j + 1 < ntiles; ++j) {
                const int t0 = c0 + j * T;                     // a whole tile: it is not the last of the row
                stage_in(u, a.u_ds, t0, su);
                stage_in(dt, a.d_ds, t0, sd);
                stage_bc(t0, false);
                __syncwarp();
#pragma unroll 2
                for (int t = 0; t < T; ++t) {
                    float d = sd[t * P + lane] + bias;
                    if (sp) d = softplus_fast(d);
                    const float dux = d * su[t * P + lane];
#pragma unroll
                    for (int n = 0; n < NS; ++n) h[n] = fmaf(decay_fast(d, A2[n]), h[n], dux * sB[n * T + t]);
                }
#pragma unroll
                for (int n = 0; n < NS; ++n) hs[(j * NS + n) * 32 + lane] = h[n];
                __syncwarp();
            }
        }
        // ---- the tiles of the chunk, last first
        for (int j = ntiles - 1; j >= 0; --j) {
            const int t0 = c0 + j * T;
            stage_in(u, a.u_ds, t0, su);
            stage_in(dt, a.d_ds, t0, sd);
            stage_in(gp, a.g_ds, t0, sg);
            stage_bc(t0, true);
            __syncwarp();
            // Over the states of an element: S1 = sum of dh B, S2 = sum of dh A a h_prev.  Then du = d' S1 + g D and
            // dd' = S2 + u S1.
            float duv[T], gv[T], dv[T], S1[T], S2[T];
#pragma unroll
            for (int t = 0; t < T; ++t) {
                const bool ok = t0 + t < L;                    // beyond the row: a = 1, everything else 0
                float x = sd[t * P + lane] + bias, g1 = 1.f;
                if (sp) softplus_and_grad(x, x, g1);
                dv[t] = ok ? x : 0.f;
                const float uv = su[t * P + lane];
                duv[t] = dv[t] * uv;
                gv[t] = sg[t * P + lane];
                sg[t * P + lane] = ok ? g1 : 0.f;               // read back when ddelta is complete
                S1[t] = 0.f;
                S2[t] = 0.f;
                dD_acc = fmaf(gv[t], uv, dD_acc);
            }
            // One state per iteration, NOT unrolled (sixteen copies of the body do not fit the instruction cache: the
            // unrolled form ran four times slower).  The per-state registers are used at index 0 and the three arrays
            // rotate by one place per iteration, so that they are back in order after NS iterations.
#pragma unroll 1
            for (int n = 0; n < NS; ++n) {
                const float A2n = A2[0], An = A2n * kLn2;
                const float hstart = j == 0 ? ck[c * NS + n] : hs[((j - 1) * NS + n) * 32 + lane];
                const float* __restrict__ Bn = sB + n * T;
                const float* __restrict__ Cn = sC + n * T;
                float av[T], hl[T];
                float h = hstart;
#pragma unroll
                for (int t = 0; t < T; ++t) {
                    av[t] = decay_fast(dv[t], A2n);
                    h = fmaf(av[t], h, duv[t] * Bn[t]);
                    hl[t] = h;
                }
                float e = e_carry[0], dA_loc = 0.f;
#pragma unroll
                for (int t = T - 1; t >= 0; --t) {
                    const float cg = Cn[t] * gv[t];
                    const float dh = cg + e;
                    e = fmaf(av[t], e, av[t] * cg);               // one fused multiply-add on the chain
                    const float hprev = t == 0 ? hstart : hl[t > 0 ? t - 1 : 0];
                    const float x = dh * (av[t] * hprev);
                    S1[t] = fmaf(dh, Bn[t], S1[t]);
                    S2[t] = fmaf(An, x, S2[t]);
                    dA_loc = fmaf(dv[t], x, dA_loc);
                    sb[t * P + lane] = dh * duv[t];
                    sc[t * P + lane] = gv[t] * hl[t];
                }
                const float dA_n = dA_acc[0] + dA_loc;
#pragma unroll
                for (int i = 0; i + 1 < NS; ++i) { A2[i] = A2[i + 1]; e_carry[i] = e_carry[i + 1]; dA_acc[i] = dA_acc[i + 1]; }
                A2[NS - 1] = A2n; e_carry[NS - 1] = e; dA_acc[NS - 1] = dA_n;
                __syncwarp();
                {   // sums over the 32 rows: lanes 0..15 the dB of element lane, lanes 16..31 the dC of element lane - 16
                    const int el = lane & 15;
                    const float* src = (lane < 16 ? sb : sc) + el * P;
                    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int rr = 0; rr < 32; ++rr) acc[rr & 3] += src[rr];
                    if (t0 + el < L) bc_out[((size_t)(lane >> 4) * NS + n) * L + t0 + el] = (acc[0] + acc[1]) + (acc[2] + acc[3]);
                }
                __syncwarp();
            }
#pragma unroll
            for (int t = 0; t < T; ++t) {
                const float v = fmaf(su[t * P + lane], S1[t], S2[t]) * sg[t * P + lane];
                db_acc += v;
                su[t * P + lane] = fmaf(dv[t], S1[t], has_D ? gv[t] * Dv : 0.f);
                sd[t * P + lane] = v;
            }
            __syncwarp();
            stage_out(su, du, t0);
            stage_out(sd, dd, t0);
            __syncwarp();
        }
    }
    float* rr = a.rowred + (b * a.dim + r) * (NS + 2);
#pragma unroll
    for (int n = 0; n < NS; ++n) rr[n] = dA_acc[n];
    rr[NS] = dD_acc; rr[NS + 1] = db_acc;
}

// Folds the partials: dA / dD / dbias over the batch, dB / dC over the CTAs of a group (and rounds
// them to the storage type).  One thread per output element, fixed summation order.
template <typename Tin>
__global__ void selscan_bwd_fold_kernel(const float* rowred, const float* bcpart, float* dA, float* dD, float* dbias,
                                        Tin* dB, Tin* dC, int64_t batch, int64_t dim, int N, int64_t L,
                                        int n_groups, int parts) {
    const int64_t n_small = dim * (N + 2);
    const int64_t n_bc = batch * n_groups * N * L;       // per tensor
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_small + 2 * n_bc;
         i += (int64_t)gridDim.x * blockDim.x) {
        if (i < n_small) {
            const int64_t r = i / (N + 2);
            const int j = (int)(i - r * (N + 2));
            float acc = 0.f;
            for (int64_t b = 0; b < batch; ++b) acc += rowred[(b * dim + r) * (N + 2) + j];
            if (j < N) dA[r * N + j] = acc;
            else if (j == N) { if (dD) dD[r] = acc; }
            else if (dbias) dbias[r] = acc;
        } else {
            int64_t q = i - n_small;
            const int which = q >= n_bc;
            if (which) q -= n_bc;
            const int64_t l = q % L; int64_t t = q / L;
            const int n = (int)(t % N); t /= N;                 // t = b * n_groups + k
            const float* src = bcpart + ((size_t)t * parts * 2 + which) * (size_t)N * L + (size_t)n * L + l;
            float acc = 0.f;
            for (int pq = 0; pq < parts; ++pq) acc += src[(size_t)pq * 2 * N * L];
            (which ? dC : dB)[q] = from_f<Tin>(acc);
        }
    }
}

struct BwdPlan { int vec, rw, parts, nsteps, R; size_t smem; int64_t ws_floats, rowred_floats; bool rows; };

static int common_pow2b(std::initializer_list<int64_t> xs, int cap) {
    int v = cap;
    for (int64_t x : xs) {
        if (x < 0) x = -x;
        while (v > 1 && (x % v) != 0) v >>= 1;
    }
    return v;
}

static int validate_bwd(const ss2d_scan_bwd_params* p) {
    if (!p) return SS2D_EINVAL_NULL;
    if (!p->u || !p->delta || !p->A || !p->B || !p->C || !p->dout || !p->du || !p->ddelta || !p->dA || !p->dB || !p->dC)
        return SS2D_EINVAL_NULL;
    if ((p->D != nullptr) != (p->dD != nullptr) || (p->delta_bias != nullptr) != (p->ddelta_bias != nullptr)) return SS2D_EINVAL_NULL;
    if (!dtype_ok(p->in_dtype) || !dtype_ok(p->dout_dtype)) return SS2D_EINVAL_DTYPE;
    if (p->dout_dtype != SS2D_F32 && p->dout_dtype != p->in_dtype) return SS2D_EINVAL_DTYPE;
    if (p->batch <= 0 || p->dim <= 0 || p->dstate <= 0 || p->seqlen <= 0 || p->n_groups <= 0) return SS2D_EINVAL_SHAPE;
    if (p->dstate > SS2D_MAX_DSTATE) return SS2D_ENOTSUP;
    if (p->dim % p->n_groups != 0) return SS2D_EINVAL_SHAPE;
    if (p->delta_ratio < 0 || (p->delta_ratio > 1 && p->dim % p->delta_ratio != 0)) return SS2D_EINVAL_SHAPE;
    if (p->seqlen > 0x3fffffffLL) return SS2D_ENOTSUP;
    const int64_t L = p->seqlen;
    if (p->u_dim_stride < L || p->delta_dim_stride < L || p->dout_dim_stride < L) return SS2D_EINVAL_STRIDE;
    if (p->B_state_stride < L || p->C_state_stride < L) return SS2D_EINVAL_STRIDE;
    if (p->batch > 1 && (p->u_batch_stride < L || p->delta_batch_stride < L || p->dout_batch_stride < L ||
                         p->B_batch_stride < L || p->C_batch_stride < L)) return SS2D_EINVAL_STRIDE;
    if (p->n_groups > 1 && (p->B_group_stride < L || p->C_group_stride < L)) return SS2D_EINVAL_STRIDE;
    const size_t si = dtype_size(p->in_dtype), sg = dtype_size(p->dout_dtype);
    if (!aligned_to(p->u, si) || !aligned_to(p->delta, si) || !aligned_to(p->B, si) || !aligned_to(p->C, si) ||
        !aligned_to(p->dout, sg) || !aligned_to(p->du, si) || !aligned_to(p->ddelta, si) || !aligned_to(p->dB, si) ||
        !aligned_to(p->dC, si) || !aligned_to(p->A, 4) || !aligned_to(p->D, 4) || !aligned_to(p->delta_bias, 4) ||
        !aligned_to(p->dA, 4) || !aligned_to(p->dD, 4) || !aligned_to(p->ddelta_bias, 4))
        return SS2D_EINVAL_ALIGN;
    return SS2D_OK;
}

static int plan_bwd(const ss2d_scan_bwd_params* p, BwdPlan& c) {
    const size_t si = dtype_size(p->in_dtype), sg = dtype_size(p->dout_dtype);
    const int64_t L = p->seqlen;
    auto ptr_el = [](const void* q, size_t s) { return (int64_t)(reinterpret_cast<uintptr_t>(q) / s); };
    const int cap = 4;     // four elements per lane: 80 registers, three CTAs per SM; eight-wide was slower (one CTA per SM)
    c.vec = common_pow2b({L, p->u_batch_stride, p->u_dim_stride, p->delta_batch_stride, p->delta_dim_stride,
                          p->dout_batch_stride, p->dout_dim_stride, p->B_batch_stride, p->B_group_stride, p->B_state_stride,
                          p->C_batch_stride, p->C_group_stride, p->C_state_stride, ptr_el(p->u, si), ptr_el(p->delta, si),
                          ptr_el(p->B, si), ptr_el(p->C, si), ptr_el(p->dout, sg), ptr_el(p->du, si), ptr_el(p->ddelta, si)}, cap);
    const int64_t step = 32 * c.vec;
    c.nsteps = (int)((L + step - 1) / step);
    const int64_t gs = p->dim / p->n_groups;
    int rw = 8;
    while (rw > 1 && rw / 2 >= gs) rw >>= 1;
    auto smem_of = [&](int w) { return ((size_t)w * (c.nsteps + 3) * p->dstate + (size_t)w * 2 * step) * sizeof(float); };
    while (rw > 1 && smem_of(rw) > 160 * 1024) rw >>= 1;
    if (smem_of(rw) > 160 * 1024) return SS2D_ENOTSUP;      // row too long for the saved step states
    c.rw = rw; c.smem = smem_of(rw); c.R = 1;
    c.parts = (int)((gs + rw - 1) / rw);
    if (p->dstate == 1) {
        // rows per warp: as many as keep about two CTAs per SM busy and the saved states in shared memory
        auto smem_n1 = [&](int w, int R) { return ((size_t)w * R * (c.nsteps + 1 + 96) + (size_t)w * 2 * step) * sizeof(float); };
        int R = 1;
        while (R < 16 && (int64_t)rw * R < gs) {
            const int R2 = R * 2;
            const int64_t parts2 = (gs + (int64_t)rw * R2 - 1) / ((int64_t)rw * R2);
            if (p->batch * p->n_groups * parts2 < 2 * 148 || smem_n1(rw, R2) > 100 * 1024) break;
            R = R2;
        }
        if (smem_n1(rw, R) > 200 * 1024) return SS2D_ENOTSUP;
        c.R = R; c.smem = smem_n1(rw, R);
        c.parts = (int)((gs + (int64_t)rw * R - 1) / ((int64_t)rw * R));
    }
    // lanes-are-rows kernel: d_state 1, the forward call's checkpoints at hand, rows in whole groups of 32 per
    // (image, group), pieces of four elements everywhere, a delta row per row, enough rows to fill the GPU with warps
    // (measured crossover against the warp-per-row kernel, bf16 with checkpoints: 24 576 rows 0.96 against 0.74 ms at
    // L = 3136, 36 864 rows 0.99 against 1.11 ms; 49 152 rows of 196 elements 0.095 against 0.158 ms)
    c.rows = p->dstate == 1 && p->checkpoints != nullptr && gs % 32 == 0 && p->delta_ratio <= 1 && c.vec >= 4 &&
             p->batch * p->dim >= 32LL * 148 * 7 && rows_kernels_enabled();
    // the same form for d_state 4 / 8 / 16.  Measured (d_state 16, bf16): 15-20 ms against 35-47 ms of the warp-per-row kernel
    // on 2 GB of rows; 57 against 115 ms on 6 528 rows of 65 536 elements, where 1.4 warps per SM walk at their own latency
    const bool rows_nx = (p->dstate == 4 || p->dstate == 8 || p->dstate == 16) && p->checkpoints != nullptr && gs % 32 == 0 &&
                         p->delta_ratio <= 1 && c.vec >= 4 && p->batch * p->dim >= 32LL * 148 && rows_kernels_enabled();
    if (c.rows) {
        c.parts = (int)(gs / 32);
        c.smem = (size_t)kBwdRowsWarps * kBwdFloatsPerWarp * sizeof(float);
    } else if (rows_nx) {
        c.rows = true;
        c.parts = (int)(gs / 32);
        const int per_warp = p->dstate == 16 ? BwdRowsN<16>::kFloatsPerWarp : p->dstate == 8 ? BwdRowsN<8>::kFloatsPerWarp : BwdRowsN<4>::kFloatsPerWarp;
        c.smem = (size_t)kBwdRowsWarps * per_warp * sizeof(float);
    }
    c.rowred_floats = p->batch * p->dim * (p->dstate + 2);
    c.ws_floats = c.rowred_floats + p->batch * p->n_groups * c.parts * 2 * p->dstate * L;
    return SS2D_OK;
}

long long selective_scan_bwd_workspace_bytes(const ss2d_scan_bwd_params* p) {
    if (validate_bwd(p) != SS2D_OK) return -1;
    BwdPlan c;
    if (plan_bwd(p, c) != SS2D_OK) return -1;
    return (long long)c.ws_floats * 4;
}

template <typename Tin, typename Tg, int VEC>
static int launch_bwd(const BwdArgs& a, const BwdPlan& c, int64_t ctas, cudaStream_t st) {
    if (a.N == 1) {
        auto kern = selscan_bwd_n1_kernel<Tin, Tg, VEC>;
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)c.smem) != cudaSuccess) return SS2D_ECUDA;
        kern<<<(unsigned)ctas, c.rw * 32, c.smem, st>>>(a, c.R);
    } else {
        auto kern = selscan_bwd_kernel<Tin, Tg, VEC>;
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)c.smem) != cudaSuccess) return SS2D_ECUDA;
        kern<<<(unsigned)ctas, c.rw * 32, c.smem, st>>>(a);
    }
    count_launch();
    return check_launch();
}

template <typename Tin, typename Tg>
static int launch_bwd_rows(const BwdArgs& a, const BwdPlan& c, cudaStream_t st) {
    void (*kern)(const BwdArgs) = selscan_bwd_rows_kernel<Tin, Tg>;
    if (a.N == 16) kern = selscan_bwd_rows_nx_kernel<Tin, Tg, 16>;
    else if (a.N == 8) kern = selscan_bwd_rows_nx_kernel<Tin, Tg, 8>;
    else if (a.N == 4) kern = selscan_bwd_rows_nx_kernel<Tin, Tg, 4>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)c.smem) != cudaSuccess) return SS2D_ECUDA;
    const int64_t warps = a.rows / 32;
    const int64_t ctas = (warps + kBwdRowsWarps - 1) / kBwdRowsWarps;
    if (ctas > 0x7fffffffLL) return SS2D_EINVAL_SHAPE;
    kern<<<(unsigned)ctas, kBwdRowsWarps * 32, c.smem, st>>>(a);
    count_launch();
    return check_launch();
}

template <typename Tin, typename Tg>
static int dispatch_bwd(const BwdArgs& a, const BwdPlan& c, int64_t ctas, cudaStream_t st) {
    if (c.rows) return launch_bwd_rows<Tin, Tg>(a, c, st);
    if (c.vec >= 4) return launch_bwd<Tin, Tg, 4>(a, c, ctas, st);
    if (c.vec >= 2) return launch_bwd<Tin, Tg, 2>(a, c, ctas, st);
    return launch_bwd<Tin, Tg, 1>(a, c, ctas, st);
}

template <typename Tin>
static int launch_fold(const ss2d_scan_bwd_params* p, const BwdArgs& a, const BwdPlan& c, cudaStream_t st) {
    const int64_t total = p->dim * (p->dstate + 2) + 2 * p->batch * p->n_groups * p->dstate * p->seqlen;
    int64_t blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    selscan_bwd_fold_kernel<Tin><<<(unsigned)blocks, 256, 0, st>>>(a.rowred, a.bcpart, (float*)p->dA, (float*)p->dD,
                                                                  (float*)p->ddelta_bias, (Tin*)p->dB, (Tin*)p->dC, p->batch,
                                                                  p->dim, (int)p->dstate, p->seqlen, (int)p->n_groups, c.parts);
    count_launch();
    return check_launch();
}

int selective_scan_bwd(const ss2d_scan_bwd_params* p, cudaStream_t st) {
    const int rc = validate_bwd(p);
    if (rc != SS2D_OK) return rc;
    BwdPlan c;
    const int pr = plan_bwd(p, c);
    if (pr != SS2D_OK) return pr;
    if (!p->workspace || p->workspace_bytes < (long long)c.ws_floats * 4) return SS2D_EWORKSPACE;
    if (!aligned_to(p->workspace, 16)) return SS2D_EINVAL_ALIGN;
    BwdArgs a;
    a.u = p->u; a.delta = p->delta; a.B = p->B; a.C = p->C; a.dout = p->dout;
    a.A = (const float*)p->A; a.D = (const float*)p->D; a.bias = (const float*)p->delta_bias;
    a.du = p->du; a.ddelta = p->ddelta;
    a.rowred = (float*)p->workspace; a.bcpart = a.rowred + c.rowred_floats;
    a.dim = p->dim; a.seqlen = p->seqlen; a.group_size = p->dim / p->n_groups;
    a.u_bs = p->u_batch_stride; a.u_ds = p->u_dim_stride; a.d_bs = p->delta_batch_stride; a.d_ds = p->delta_dim_stride;
    a.g_bs = p->dout_batch_stride; a.g_ds = p->dout_dim_stride;
    a.B_bs = p->B_batch_stride; a.B_gs = p->B_group_stride; a.B_ss = p->B_state_stride;
    a.C_bs = p->C_batch_stride; a.C_gs = p->C_group_stride; a.C_ss = p->C_state_stride;
    a.N = (int)p->dstate; a.n_groups = (int)p->n_groups; a.parts = c.parts; a.nsteps = c.nsteps; a.softplus = p->delta_softplus;
    a.dratio = p->delta_ratio > 1 ? p->delta_ratio : 1;
    a.ckpt = (const float*)p->checkpoints; a.nck = (p->seqlen + 127) / 128;
    a.rows = p->batch * p->dim;
    const int64_t ctas = p->batch * p->n_groups * c.parts;
    if (ctas > 0x7fffffffLL) return SS2D_EINVAL_SHAPE;
    const bool gf32 = p->dout_dtype == SS2D_F32;
    int r;
    if (p->in_dtype == SS2D_F32) r = dispatch_bwd<float, float>(a, c, ctas, st);
    else if (p->in_dtype == SS2D_BF16)
        r = gf32 ? dispatch_bwd<__nv_bfloat16, float>(a, c, ctas, st) : dispatch_bwd<__nv_bfloat16, __nv_bfloat16>(a, c, ctas, st);
    else
        r = gf32 ? dispatch_bwd<__half, float>(a, c, ctas, st) : dispatch_bwd<__half, __half>(a, c, ctas, st);
    if (r != SS2D_OK) return r;
    if (p->in_dtype == SS2D_F32) return launch_fold<float>(p, a, c, st);
    if (p->in_dtype == SS2D_BF16) return launch_fold<__nv_bfloat16>(p, a, c, st);
    return launch_fold<__half>(p, a, c, st);
}

}  // namespace ss2d
