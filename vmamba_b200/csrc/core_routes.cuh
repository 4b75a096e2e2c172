// Route-stream form of the fused SS2D core (scans mode 0, d_state 1): one CTA per (image, channel)
// plane, one warp per route.
//
// A warp walks its route in chunks of 32 * S elements (lane j holds S consecutive elements of the
// route's orientation order), the state of the recurrence crossing from chunk to chunk in a register:
// per chunk one warp-shuffle scan of the lane aggregates, no CTA-wide scan and no barrier inside the
// walk.  The four routes meet in shared memory: the row-major routes 0 / 2 accumulate into an fp32
// plane in row-major order, the column-major routes 1 / 3 into a second fp32 plane in column-major
// order, so every access of the walk is a contiguous 16-byte vector.  The forward warp of an
// orientation walks chunks 0 .. nc-1, the backward warp nc-1 .. 0; each STORES into the half of the
// plane it reaches first and, after one barrier between the two warps, ADDS into the other half:
// every element gets exactly one store and one add in an order fixed by its position (and a two-term
// fp32 sum does not depend on the order anyway), so results are bit-identical run to run without
// atomics and without clearing the planes.  The column-major warps read x from a column-major copy
// of the plane in shared memory, written once by all four warps at the start.  At the end the CTA
// sums the two planes (one transposed read) and writes the merged fp32 plane.
//
// Shared memory per CTA: L * (4 + 4 + sizeof(T)) bytes (31 KB for a 56 x 56 bf16 plane: seven CTAs of
// four warps per SM).
//
// Memory latency: the step sizes are the one stream that comes from HBM and is read once.  A warp
// has a single chunk of loads in flight, far too little to cover the HBM latency (the kernel ran at
// 1.6 TB/s that way), so at its start every warp asks for the whole row of its route with one bulk
// prefetch into L2 (0.240 -> 0.210 ms for the stage-0 launch of a batch-128 VMamba-T forward); the
// loads of the walk then see L2 latency, which the other warps of the scheduler cover.
#pragma once
#include "common.cuh"

namespace ss2d {

struct RouteArgs {
    const void* x;
    const void* delta[4];
    const void* Bm[4];
    const void* Cm[4];
    const float *A, *Dskip, *bias;
    float* merged;
    long long d_bs[4], d_cs[4], bc_bs[4];
    long long x_bs, x_cs;
    int B, D, H, W, L;
    unsigned magic_H;     // ceil(2^32 / H): n / H == umulhi(n, magic_H) for n * H < 2^32 (0 when H == 1)
};

// Barrier between the two warps of an orientation (named barriers 1 and 2; the ids are immediates so that the kernel
// claims three barriers, not all sixteen).
__device__ __forceinline__ void pair_barrier(bool col) {
    if (col) asm volatile("bar.sync 2, 64;" ::: "memory");
    else asm volatile("bar.sync 1, 64;" ::: "memory");
}

// One step of an inclusive (a, b) scan across the lanes: the shuffle's own "source lane in range" predicate guards the
// combine, so a step is two shuffles and two predicated arithmetic instructions (no lane test, no select).
template <int OFF> __device__ __forceinline__ void scan_step_up(float& a, float& b) {
    asm volatile(
        "{\n .reg .pred p;\n .reg .f32 pa, pb;\n"
        " shfl.sync.up.b32 pa|p, %0, %2, 0, 0xffffffff;\n"
        " shfl.sync.up.b32 pb, %1, %2, 0, 0xffffffff;\n"
        " @p fma.rn.f32 %1, %0, pb, %1;\n"
        " @p mul.f32 %0, %0, pa;\n}"
        : "+f"(a), "+f"(b) : "n"(OFF));
}
template <int OFF> __device__ __forceinline__ void scan_step_down(float& a, float& b) {
    asm volatile(
        "{\n .reg .pred p;\n .reg .f32 pa, pb;\n"
        " shfl.sync.down.b32 pa|p, %0, %2, 31, 0xffffffff;\n"
        " shfl.sync.down.b32 pb, %1, %2, 31, 0xffffffff;\n"
        " @p fma.rn.f32 %1, %0, pb, %1;\n"
        " @p mul.f32 %0, %0, pa;\n}"
        : "+f"(a), "+f"(b) : "n"(OFF));
}
// Inclusive state of the neighbouring lane (the lane before, or after when walking backwards); on the first lane of
// the walk, which has no neighbour, the state carried over from the previous chunk.
template <bool kBack> __device__ __forceinline__ float entering_state(float inc_b, float carry) {
    float r;
    if constexpr (kBack)
        asm volatile(
            "{\n .reg .pred p;\n"
            " shfl.sync.down.b32 %0|p, %1, 1, 31, 0xffffffff;\n"
            " @!p mov.f32 %0, %2;\n}"
            : "=&f"(r) : "f"(inc_b), "f"(carry));
    else
        asm volatile(
            "{\n .reg .pred p;\n"
            " shfl.sync.up.b32 %0|p, %1, 1, 0, 0xffffffff;\n"
            " @!p mov.f32 %0, %2;\n}"
            : "=&f"(r) : "f"(inc_b), "f"(carry));
    return r;
}

// One route of one plane (k: route; kBack: routes 2, 3).  `xsrc` is the plane's x in the orientation order of the route
// (global memory for the row-major routes, the shared column-major copy for the others: a generic address); `acc`
// the fp32 plane of the orientation, in orientation order.  kRoll chooses where the loads of the next chunk are issued:
// 0 at the top of that chunk (what is shipped: with the rows already in L2 the seven warps of a scheduler cover the
// wait, 0.223 ms), 1 as soon as the current chunk is unpacked (0.255 ms: 32-byte spill), 2 / 3 after the scan (0.225 ms).
template <typename T, int S, bool kBack, int kRoll>
__device__ __forceinline__ void walk_route(const RouteArgs& a, const int b, const int d, const int k, const int lane,
                                           const T* __restrict__ xsrc, float* __restrict__ acc, const bool col) {
    constexpr int NP = S / 2;
    constexpr int CH = 32 * S;
    constexpr int STEP = kBack ? -CH : CH;
    constexpr bool kPrecise = sizeof(T) == 4;
    using VT = Vec<T, S>;
    using Raw = typename VT::Raw;
    const int L = a.L;
    const T* __restrict__ dp = (const T*)a.delta[k] + b * a.d_bs[k] + d * a.d_cs[k];
    const T* __restrict__ Bp = (const T*)a.Bm[k] + b * a.bc_bs[k];
    const T* __restrict__ Cp = (const T*)a.Cm[k] + b * a.bc_bs[k];
    const float Ak = __ldg(a.A + k * a.D + d) * (kPrecise ? kLog2e : 1.f);
    const float bias = __ldg(a.bias + k * a.D + d) * (kPrecise ? 1.f : kLog2e);
    // 16-bit maps accumulate in units of 1 / ln 2 (the step size stays a base-2 logarithm); the merge rescales
    const float Dk = __ldg(a.Dskip + k * a.D + d) * (kPrecise ? 1.f : 1.f / kLn2);
    const bool first_lane = lane == (kBack ? 31 : 0);
    const bool swap_units = (lane & 4) != 0;
    const int last_seg = L - S;                        // L is a multiple of S
    const int nc = (L + CH - 1) / CH;
    const int half = (nc + 1) >> 1;
    const int nA = kBack ? nc - half : half;           // chunks this warp stores first; into the others it adds
    int e = (kBack ? (nc - 1) * CH : 0) + lane * S;    // first element of this lane's segment in the current chunk
    float carry = 0.f;

    // segments outside the plane (the tail of the last chunk, the chunk after the walk's end) re-read the plane's end
    // or start and are ignored
    auto offset_of = [&](int at) { return max(min(at, last_seg), 0); };
    Raw rd, rb, rx, rc;
    if constexpr (kRoll != 0) {
        const int o = offset_of(e);
        rd = VT::load_raw(dp + o);
        rb = VT::load_raw(Bp + o);
        rx = VT::template load_raw<false>(xsrc + o);
        rc = VT::load_raw(Cp + o);
    }
#pragma unroll 1
    for (int s = 0; s < nc; ++s) {
        if (s == nA) pair_barrier(col);
        const bool active = e < L;
        const int o_next = offset_of(kRoll ? e + STEP : e);
        if constexpr (kRoll == 0) {
            rd = VT::load_raw(dp + o_next);
            rb = VT::load_raw(Bp + o_next);
            rx = VT::template load_raw<false>(xsrc + o_next);
            rc = VT::load_raw(Cp + o_next);
        }
        float2 aa[NP], bb[NP], du[NP];
        {
            float dvf[S], bvf[S], xvf[S];
            VT::unpack(rd, dvf);
            VT::unpack(rb, bvf);
            VT::unpack(rx, xvf);
            if constexpr (kRoll == 1 || kRoll == 3) rd = VT::load_raw(dp + o_next);
            if constexpr (kRoll == 1) {
                // the raw registers of these three streams are free: the next chunk's loads fly during the rest of this one
                rb = VT::load_raw(Bp + o_next);
                rx = VT::template load_raw<false>(xsrc + o_next);
            }
#pragma unroll
            for (int j = 0; j < NP; ++j) {
                const float2 dv = make_float2(dvf[2 * j], dvf[2 * j + 1]);
                float2 t;
                if constexpr (kPrecise) {
                    const float2 xx = __fadd2_rn(dv, make_float2(bias, bias));
                    t = make_float2(softplus_fast(xx.x), softplus_fast(xx.y));     // the step size itself
                } else {
                    // t = log2(1 + e^x), the step size over ln 2.  The clamp keeps e^x finite: exact up to
                    // x = 87 (126 ln 2), constant above.
                    float2 arg = __ffma2_rn(dv, make_float2(kLog2e, kLog2e), make_float2(bias, bias));
                    arg.x = fminf(arg.x, 126.f); arg.y = fminf(arg.y, 126.f);
                    const float2 w = __fadd2_rn(make_float2(ex2_approx(arg.x), ex2_approx(arg.y)), make_float2(1.f, 1.f));
                    t = make_float2(lg2_approx(w.x), lg2_approx(w.y));
                }
                const float2 ta = __fmul2_rn(t, make_float2(Ak, Ak));
                aa[j] = make_float2(ex2_approx(ta.x), ex2_approx(ta.y));
                const float2 xv = make_float2(xvf[2 * j], xvf[2 * j + 1]);
                bb[j] = __fmul2_rn(t, __fmul2_rn(make_float2(bvf[2 * j], bvf[2 * j + 1]), xv));
                du[j] = __fmul2_rn(xv, make_float2(Dk, Dk));
            }
        }
        // the recurrence over the lane's own elements, from state zero: aa becomes the running product, bb the local state
        float p = 1.f, h = 0.f;
#pragma unroll
        for (int ii = 0; ii < S; ++ii) {
            const int i = kBack ? S - 1 - ii : ii;
            float& a_i = (i & 1) ? aa[i >> 1].y : aa[i >> 1].x;
            float& b_i = (i & 1) ? bb[i >> 1].y : bb[i >> 1].x;
            h = fmaf(a_i, h, b_i);
            p *= a_i;
            a_i = p; b_i = h;
        }
        float ia = active ? p : 1.f, ib = active ? h : 0.f;
        // the state left by the chunks before enters through the first lane, so that the scanned b IS the state at the
        // end of every lane's segment
        if (first_lane) ib = fmaf(ia, carry, ib);
        if constexpr (kBack) {
            scan_step_down<1>(ia, ib); scan_step_down<2>(ia, ib); scan_step_down<4>(ia, ib);
            scan_step_down<8>(ia, ib); scan_step_down<16>(ia, ib);
        } else {
            scan_step_up<1>(ia, ib); scan_step_up<2>(ia, ib); scan_step_up<4>(ia, ib);
            scan_step_up<8>(ia, ib); scan_step_up<16>(ia, ib);
        }
        const float hin = entering_state<kBack>(ib, carry);      // state entering this lane's segment
        carry = __shfl_sync(0xffffffffu, ib, kBack ? 0 : 31);    // state leaving the chunk

        if constexpr (kRoll == 2) rd = VT::load_raw(dp + o_next);
        if constexpr (kRoll == 2 || kRoll == 3) {
            rb = VT::load_raw(Bp + o_next);
            rx = VT::template load_raw<false>(xsrc + o_next);
        }
        float2 y[NP];
        {
            float cvf[S];
            VT::unpack(rc, cvf);
            if constexpr (kRoll != 0) rc = VT::load_raw(Cp + o_next);
#pragma unroll
            for (int j = 0; j < NP; ++j) {
                const float2 hh = __ffma2_rn(aa[j], make_float2(hin, hin), bb[j]);
                y[j] = __ffma2_rn(make_float2(cvf[2 * j], cvf[2 * j + 1]), hh, du[j]);
            }
        }
        float* q = acc + min(e, last_seg);
        if constexpr (S == 8) {
            // A lane's eight floats are two 16-byte units, 32 bytes from the next lane's: taken in the same order by every
            // lane, lanes j and j + 4 of a quarter-warp would meet in the same banks on every access.  Lanes 4..7 of each
            // group of eight therefore take their upper unit first.
            const int first = swap_units ? 4 : 0, second = 4 - first;
            float2 u0 = swap_units ? y[2] : y[0], u1 = swap_units ? y[3] : y[1];     // unit accessed first
            float2 v0 = swap_units ? y[0] : y[2], v1 = swap_units ? y[1] : y[3];     // unit accessed second
            if (s >= nA) {                                       // same for the whole warp
                float o[4], w[4];
                Vec<float, 4>::load_plain(q + first, o);
                Vec<float, 4>::load_plain(q + second, w);
                u0 = __fadd2_rn(u0, make_float2(o[0], o[1])); u1 = __fadd2_rn(u1, make_float2(o[2], o[3]));
                v0 = __fadd2_rn(v0, make_float2(w[0], w[1])); v1 = __fadd2_rn(v1, make_float2(w[2], w[3]));
            }
            if (active) {
                const float a0[4] = {u0.x, u0.y, u1.x, u1.y}, a1[4] = {v0.x, v0.y, v1.x, v1.y};
                Vec<float, 4>::store(q + first, a0);
                Vec<float, 4>::store(q + second, a1);
            }
        } else {
            if (s >= nA) {
                float old[S];
                Vec<float, S>::load_plain(q, old);
#pragma unroll
                for (int j = 0; j < NP; ++j) y[j] = __fadd2_rn(y[j], make_float2(old[2 * j], old[2 * j + 1]));
            }
            if (active) {
                float yo[S];
#pragma unroll
                for (int j = 0; j < NP; ++j) { yo[2 * j] = y[j].x; yo[2 * j + 1] = y[j].y; }
                Vec<float, S>::store(q, yo);
            }
        }
        e += STEP;
    }
    if (nA >= nc) pair_barrier(col);
}

// T: element type of x / delta / B / C.  S: elements per lane per chunk (L a multiple of S).  SV: pixels per thread
// in the column-major copy (W a multiple of SV; the merge needs W to be a multiple of 4).
template <typename T, int S, int SV, int MINB, int kRoll>
__global__ void __launch_bounds__(128, MINB) core_route_kernel(const RouteArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int L = a.L, H = a.H, W = a.W, D = a.D;
    float* accR = reinterpret_cast<float*>(smem_raw);          // routes 0, 2: row-major
    float* accC = accR + L;                                    // routes 1, 3: column-major
    T* xT = reinterpret_cast<T*>(accC + L);                    // x, column-major
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int b = blockIdx.x / D, d = blockIdx.x - b * D;
    const T* __restrict__ xg = (const T*)a.x + b * a.x_bs + d * a.x_cs;
    if (lane == 0) {                                           // the row of this warp's route, on its way into L2
        const T* dp = (const T*)a.delta[warp] + b * a.d_bs[warp] + d * a.d_cs[warp];
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(dp), "r"((unsigned)(L * sizeof(T))) : "memory");
    }

    // ---- column-major copy of x: a thread takes SV consecutive pixels of one row; consecutive threads take consecutive
    //      rows, so that the 2- or 4-byte stores of a warp fall into consecutive shared-memory words ----
    {
        const int nvec = (W / SV) * H;
        for (int idx = t; idx < nvec; idx += 128) {
            const int wv = a.magic_H ? (int)__umulhi((unsigned)idx, a.magic_H) : idx;
            const int h = idx - wv * H;
            const typename Vec<T, SV>::Raw r = Vec<T, SV>::load_raw(xg + h * W + wv * SV);
            T* dst = xT + (wv * SV) * H + h;
            if constexpr (sizeof(T) == 4) {
#pragma unroll
                for (int i = 0; i < SV; ++i) reinterpret_cast<uint32_t*>(dst)[i * H] = r.w[i];
            } else {
#pragma unroll
                for (int i = 0; i < SV; ++i)
                    reinterpret_cast<uint16_t*>(dst)[i * H] = (uint16_t)((i & 1) ? (r.w[i >> 1] >> 16) : (r.w[i >> 1] & 0xffffu));
            }
        }
    }
    __syncthreads();

    {
        const bool col = warp & 1;
        const T* xs = col ? xT : xg;
        float* acc = col ? accC : accR;
        if (warp < 2) walk_route<T, S, false, kRoll>(a, b, d, warp, lane, xs, acc, col);
        else walk_route<T, S, true, kRoll>(a, b, d, warp, lane, xs, acc, col);
    }
    __syncthreads();

    // ---- merge: row-major plane + column-major plane (transposed read) -> fp32 merged plane.
    //      A warp takes 16 rows; lane = (row j, half of an 8-column group), four pixels per lane and step.
    {
        const float scale = sizeof(T) == 4 ? 1.f : kLn2;
        float* __restrict__ out = a.merged + ((long long)b * D + d) * L;
        const int j = lane >> 1, wsub = (lane & 1) * 4;
        for (int hb = warp * 16; hb < H; hb += 64) {
            const int h = hb + j;
            if (h < H) {
#pragma unroll 2
                for (int w0 = wsub; w0 < W; w0 += 8) {
                    float r[4], o[4];
                    Vec<float, 4>::load_plain(accR + h * W + w0, r);
#pragma unroll
                    for (int i = 0; i < 4; ++i) o[i] = scale * (r[i] + accC[(w0 + i) * H + h]);
                    Vec<float, 4>::store(out + h * W + w0, o);
                }
            }
        }
    }
}

}  // namespace ss2d
