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

// d_state 4 / 8 / 16 with many rows: LANES ARE ROWS.  A warp owns 32 consecutive rows of one (image, group) and every
// lane walks its own row element by element with all NS states in registers: the recurrence is a plain fused
// multiply-add per (element, state) - no running products, no fix-up, no shuffle scan (the warp-per-row kernel above
// spends 13.7 instructions per (element, state), 2.2 of them in the scans; this form needs 5: scale, ex2, B u, h, y) -
// and the NS states of a lane are NS independent dependency chains.  The B / C values of an element are the same for
// the 32 rows of the warp: they are staged once per tile as fp32 and read as broadcast 16-byte loads.  Tiles of 16
// elements: u and delta (32 rows x 16 elements) and B / C (NS rows x 16 elements) are loaded as 16-byte pieces, unpacked
// and stored transposed ([element][row], pitch 33: conflict-free both ways); the outputs leave through the same buffer
// as 16-byte vectors.  Warps of a CTA never wait for each other.  The kernel is bound by the MUFU pipe (NS + 2
// transcendentals per element and lane).
constexpr int kRowsTile = 16;          // elements per tile: 6.8 KB of shared memory per warp at 16 states, six CTAs per SM
constexpr int kRowsWarps = 4;
template <int NS> struct RowsSmem {
    static constexpr int kPitch = 33;
    static constexpr int kBCPitch = NS >= 4 ? NS + 4 : NS;       // 16-byte aligned rows for the 16-byte reads of four states
    static constexpr int kFloatsPerWarp = 2 * kRowsTile * kPitch + 2 * kRowsTile * kBCPitch;
};

template <typename Tin, typename Tout, int NS, int EPP>
__global__ void __launch_bounds__(kRowsWarps * 32, 6) selscan_fwd_rows_kernel(const ScanArgs a) {
    using S = RowsSmem<NS>;
    // EPP: elements per piece moved by one load (16 bytes; 8 bytes for 16-bit rows whose length is a multiple of 4 only)
    constexpr int PPR = kRowsTile / EPP;                         // pieces per row of a tile
    constexpr int OPP = EPP < 16 / (int)sizeof(Tout) ? EPP : 16 / (int)sizeof(Tout), OPR = kRowsTile / OPP;
    extern __shared__ __align__(16) float rows_sm[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* su = rows_sm + (size_t)warp * S::kFloatsPerWarp;       // [t][row]; overwritten by the outputs
    float* sd = su + kRowsTile * S::kPitch;
    float* sB = sd + kRowsTile * S::kPitch;                      // [t][n]
    float* sC = sB + kRowsTile * S::kBCPitch;
    const int64_t row0 = ((int64_t)blockIdx.x * kRowsWarps + warp) * 32;
    if (row0 >= a.rows) return;
    const int64_t b = row0 / a.dim, r0 = row0 % a.dim, k = r0 / a.group_size;     // 32 rows: one image, one group
    const int64_t r = r0 + lane;
    const Tin* __restrict__ u = (const Tin*)a.u + b * a.u_bs + r0 * a.u_ds;
    const Tin* __restrict__ dt = (const Tin*)a.delta + b * a.d_bs + r0 * a.d_ds;
    const Tin* __restrict__ Bm = (const Tin*)a.B + b * a.B_bs + k * a.B_gs;
    const Tin* __restrict__ Cm = (const Tin*)a.C + b * a.C_bs + k * a.C_gs;
    Tout* __restrict__ out = (Tout*)a.out + b * a.o_bs + r0 * a.o_ds;
    float A2[NS], h[NS];
#pragma unroll
    for (int n = 0; n < NS; ++n) { A2[n] = __ldg(a.A + r * NS + n) * kLog2e; h[n] = 0.f; }
    const bool has_D = a.D != nullptr;
    const float Dv = has_D ? __ldg(a.D + r) : 0.f;
    const float bias = a.bias ? __ldg(a.bias + r) : 0.f;
    const bool sp = a.softplus != 0;
    const int L = (int)a.seqlen;
    using VI = Vec<Tin, EPP>;
    using VO = Vec<Tout, OPP>;

    for (int t0 = 0; t0 < L; t0 += kRowsTile) {
        // ---- stage the tile: 16-byte pieces in, fp32 transposed out (L is a multiple of the piece: a piece is inside or outside)
#pragma unroll
        for (int j = 0; j < PPR; ++j) {
            const int idx = j * 32 + lane, rr = idx / PPR, piece = idx - rr * PPR;
            const int pos = t0 + piece * EPP;
            float uv[EPP], dv[EPP];
            if (pos < L) {
                VI::load(u + rr * a.u_ds + pos, uv);
                VI::load(dt + rr * a.d_ds + pos, dv);
            } else {
#pragma unroll
                for (int e = 0; e < EPP; ++e) { uv[e] = 0.f; dv[e] = 0.f; }
            }
#pragma unroll
            for (int e = 0; e < EPP; ++e) {
                su[(piece * EPP + e) * S::kPitch + rr] = uv[e];
                sd[(piece * EPP + e) * S::kPitch + rr] = dv[e];
            }
        }
#pragma unroll
        for (int j = 0; j < (NS * PPR + 31) / 32; ++j) {
            const int idx = j * 32 + lane, n = idx / PPR, piece = idx - n * PPR;
            const int pos = t0 + piece * EPP;
            if (n < NS) {
                float bv[EPP], cv[EPP];
                if (pos < L) {
                    VI::load(Bm + n * a.B_ss + pos, bv);
                    VI::load(Cm + n * a.C_ss + pos, cv);
                } else {
#pragma unroll
                    for (int e = 0; e < EPP; ++e) { bv[e] = 0.f; cv[e] = 0.f; }
                }
#pragma unroll
                for (int e = 0; e < EPP; ++e) {
                    sB[(piece * EPP + e) * S::kBCPitch + n] = bv[e];
                    sC[(piece * EPP + e) * S::kBCPitch + n] = cv[e];
                }
            }
        }
        __syncwarp();
        // ---- the recurrence: this lane's row, element by element
        const int tn = min(kRowsTile, L - t0);
#pragma unroll 2
        for (int t = 0; t < tn; ++t) {
            const float uv = su[t * S::kPitch + lane];
            float d = sd[t * S::kPitch + lane] + bias;
            if (sp) d = softplus_fast(d);
            const float du = d * uv;
            float y = has_D ? Dv * uv : 0.f, y1 = 0.f;           // two partial sums: half the dependent chain
            if (a.ckpt && ((t0 + t) & 127) == 0) {               // the states in front of element t0 + t
                float* ck = a.ckpt + ((row0 + lane) * a.nck + ((t0 + t) >> 7)) * NS;
                if constexpr (NS >= 4) {
#pragma unroll
                    for (int n = 0; n < NS; n += 4) *reinterpret_cast<float4*>(ck + n) = make_float4(h[n], h[n + 1], h[n + 2], h[n + 3]);
                } else {
#pragma unroll
                    for (int n = 0; n < NS; ++n) ck[n] = h[n];
                }
            }
            if constexpr (NS >= 4) {
#pragma unroll
                for (int n4 = 0; n4 < NS; n4 += 4) {
                    const float4 b4 = *reinterpret_cast<const float4*>(sB + t * S::kBCPitch + n4);
                    const float4 c4 = *reinterpret_cast<const float4*>(sC + t * S::kBCPitch + n4);
                    const float bb[4] = {b4.x, b4.y, b4.z, b4.w}, cc[4] = {c4.x, c4.y, c4.z, c4.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int n = n4 + i;
                        h[n] = fmaf(decay_fast(d, A2[n]), h[n], du * bb[i]);
                        if (i & 1) y1 = fmaf(cc[i], h[n], y1);
                        else y = fmaf(cc[i], h[n], y);
                    }
                }
            } else {
#pragma unroll
                for (int n = 0; n < NS; ++n) {
                    h[n] = fmaf(decay_fast(d, A2[n]), h[n], du * sB[t * S::kBCPitch + n]);
                    y = fmaf(sC[t * S::kBCPitch + n], h[n], y);
                }
            }
            su[t * S::kPitch + lane] = y + y1;
        }
        __syncwarp();
        // ---- outputs: 16-byte pieces along each row
#pragma unroll
        for (int j = 0; j < OPR; ++j) {
            const int idx = j * 32 + lane, rr = idx / OPR, piece = idx - rr * OPR;
            const int pos = t0 + piece * OPP;
            if (pos < L) {
                float ov[OPP];
#pragma unroll
                for (int e = 0; e < OPP; ++e) ov[e] = su[(piece * OPP + e) * S::kPitch + rr];
                VO::store(out + rr * a.o_ds + pos, ov);
            }
        }
        __syncwarp();
    }
}

template <typename Tin, typename Tout, int NS, int EPP>
static int launch_rows(const ScanArgs& a, cudaStream_t st) {
    using S = RowsSmem<NS>;
    const size_t smem = (size_t)kRowsWarps * S::kFloatsPerWarp * sizeof(float);
    auto kern = selscan_fwd_rows_kernel<Tin, Tout, NS, EPP>;
    static bool attr_ok[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_ok[dev & 63]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return SS2D_ECUDA;
        attr_ok[dev & 63] = true;
    }
    const int64_t warps = a.rows / 32;
    const int64_t ctas = (warps + kRowsWarps - 1) / kRowsWarps;
    if (ctas > 0x7fffffffLL) return SS2D_EINVAL_SHAPE;
    kern<<<(unsigned)ctas, kRowsWarps * 32, smem, st>>>(a);
    count_launch();
    return check_launch();
}

// The lanes-are-rows kernel takes a problem when its rows come in whole groups of 32 per (image, group), every tensor
// allows pieces of at least 8 bytes, each row has its own delta row, and there are enough rows (below).
template <typename Tin, typename Tout, int EPP>
static int rows_by_state(const ScanArgs& a, cudaStream_t st) {
    if (a.dstate == 16) return launch_rows<Tin, Tout, 16, EPP>(a, st);
    if (a.dstate == 8) return launch_rows<Tin, Tout, 8, EPP>(a, st);
    if (a.dstate == 4) return launch_rows<Tin, Tout, 4, EPP>(a, st);
    return launch_rows<Tin, Tout, 1, EPP>(a, st);
}
template <typename Tin, typename Tout>
static int try_rows(const ScanArgs& a, int vec, cudaStream_t st, bool& taken) {
    taken = false;
    // d_state 1: short rows only (bf16, fraction of the copy bandwidth, this kernel against the warp-per-row one: 0.42 / 0.35
    // at L = 196, 0.42 / 0.54 at L = 784; the warp-per-row kernel reaches 0.8 from L = 3136 up)
    if (a.dstate == 1 ? a.seqlen > 256 : (a.dstate != 4 && a.dstate != 8 && a.dstate != 16)) return SS2D_OK;
    // enough rows to fill the GPU with warps of 32 rows.  Measured crossover against the warp-per-row kernels (d_state 16,
    // bf16): 12 288 rows tie, 26 112 rows 0.105 against 0.067 of the copy bandwidth, 6 144 rows 0.027 against 0.058
    const long long min_rows = 32LL * 148 * (a.dstate == 1 ? 8 : 3);
    if (vec < 4 || a.dratio != 1 || a.group_size % 32 != 0 || a.rows < min_rows || !rows_kernels_enabled()) return SS2D_OK;
    taken = true;
    if constexpr (sizeof(Tin) == 2) {
        if (vec >= 8) return rows_by_state<Tin, Tout, 8>(a, st);
    }
    return rows_by_state<Tin, Tout, 4>(a, st);
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
    {
        bool taken;
        const int rc = try_rows<Tin, Tout>(a, vec, st, taken);
        if (taken) return rc;
    }
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
