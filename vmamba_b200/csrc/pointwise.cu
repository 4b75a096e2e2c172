// Elementwise producers around the SS2D core, channel-first maps, each one pass over HBM:
//   bias_act      y = act(x + bias[d])                       (fc1 bias + GELU of the MLP, in place)
//   dwconv3x3_act y = act(depthwise 3x3 conv of x, pad 1)    (the conv + SiLU in front of the core)
// Rounding: the depthwise convolution sum is formed in fp32 and rounded to the storage type before the
// activation (what the stand-alone convolution would hand over); the bias + GELU of 16-bit maps is
// evaluated in fp32 on stored value + bias and rounded once (the reference rounds accumulator + bias
// once inside its GEMM; the accumulator itself is not available here).
#include "activations.cuh"

namespace ss2d {

// ------------------------------------------------------------------------------------------------
struct BiasActArgs {
    const void* x;
    const float* bias;
    void* y;
    long long rows;      // B * D rows of L elements (D rows of B * L for channel-major maps)
    int D, nv;           // nv = L / PV vectors per row
    int rows_per_channel;   // 1 for (B, D, ...) maps (channel = row % D); B for (D, B, ...) maps (channel = row / B)
    int chunks_per_row;     // CTAs per row
};

// A CTA works inside ONE row, so the channel (and its bias) is found once per CTA and the element
// loop has no division.  GELU of 16-bit maps is the polynomial form on the FMA pipe (11 packed instructions per
// pair of values); the rational erfc form with rcp / ex2 took 25 and left the kernel bound by instruction issue.
template <typename T, int PV, int ACT>
__global__ void __launch_bounds__(256) bias_act_kernel(const BiasActArgs a) {
    // x may be y: a store orders every later load behind it, so each pass loads kU vectors first
    constexpr int kU = 4;
    const long long row = blockIdx.x / a.chunks_per_row;
    const int chunk = blockIdx.x - (int)row * a.chunks_per_row;
    const int d = (int)((row / a.rows_per_channel) % a.D);
    const float b = a.bias ? __ldg(a.bias + d) : 0.f;
    const T* __restrict__ xr = (const T*)a.x + row * (long long)a.nv * PV;
    T* __restrict__ yr = (T*)a.y + row * (long long)a.nv * PV;
    for (int it0 = chunk * 256 + threadIdx.x; it0 < a.nv; it0 += kU * 256 * a.chunks_per_row) {
        typename Vec<T, PV>::Raw raw[kU];
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            const int it = it0 + u * 256 * a.chunks_per_row;
            if (it < a.nv) raw[u] = Vec<T, PV>::template load_raw<false>(xr + (long long)it * PV);
        }
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            const int it = it0 + u * 256 * a.chunks_per_row;
            if (it >= a.nv) break;
            float v[PV];
            Vec<T, PV>::unpack(raw[u], v);
            if constexpr (ACT == ACT_GELU && sizeof(T) == 2 && PV >= 2) {
#pragma unroll
                for (int i = 0; i < PV; i += 2) {
                    const float2 r = gelu_pair_poly(make_float2(v[i] + b, v[i + 1] + b));
                    v[i] = r.x; v[i + 1] = r.y;
                }
            } else {
#pragma unroll
                for (int i = 0; i < PV; ++i) v[i] = act_f<ACT>(round_to<T>(v[i] + b));
            }
            Vec<T, PV>::store(yr + (long long)it * PV, v);
        }
    }
}

template <typename T, int PV>
static void launch_bias_act(BiasActArgs a, int act, cudaStream_t st) {
    // about 4 vectors per thread; at least enough CTAs for a few waves
    int chunks = (a.nv + 256 * 4 - 1) / (256 * 4);
    if (chunks < 1) chunks = 1;
    while ((long long)chunks * a.rows > (1LL << 30) && chunks > 1) chunks >>= 1;
    a.chunks_per_row = chunks;
    const unsigned g = (unsigned)(a.rows * chunks);
    if (act == ACT_GELU) bias_act_kernel<T, PV, ACT_GELU><<<g, 256, 0, st>>>(a);
    else if (act == ACT_SILU) bias_act_kernel<T, PV, ACT_SILU><<<g, 256, 0, st>>>(a);
    else bias_act_kernel<T, PV, ACT_NONE><<<g, 256, 0, st>>>(a);
}

template <typename T>
static void launch_bias_act_v(BiasActArgs a, int pv, long long rows, long long L, int act, cudaStream_t st) {
    a.nv = (int)(L / pv);
    a.rows = rows;
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
    a.x = p->x; a.bias = (const float*)p->bias; a.y = p->y; a.D = (int)p->D; a.nv = 0; a.rows = 0; a.chunks_per_row = 1;
    a.rows_per_channel = p->channel_major ? (int)p->B : 1;
    const long long rows = p->B * p->D;
    if (p->dtype == SS2D_F32) launch_bias_act_v<float>(a, pv, rows, L, p->act, st);
    else if (p->dtype == SS2D_BF16) launch_bias_act_v<__nv_bfloat16>(a, pv, rows, L, p->act, st);
    else launch_bias_act_v<__half>(a, pv, rows, L, p->act, st);
    count_launch();
    return check_launch();
}

// ------------------------------------------------------------------------------------------------
// Depthwise 3x3, stride 1, zero padding 1, no shared memory: a thread owns PV neighbouring columns of KR
// consecutive rows.  It reads the KR + 2 input rows of its strip as one vector each (all issued before the
// first result is needed), takes the column to the left and to the right of the strip from the neighbouring
// lanes by shuffle (zero at the image border, a scalar load where the neighbour sits in another warp) and
// slides the 3x3 window down in registers.  Lanes run along a row, then over the row blocks, then over the
// planes, so a warp's loads and stores are contiguous runs.  (An earlier form staged whole planes in shared
// memory as fp32 frames; it issued two to three times the instructions per output and was 25 % slower over a
// backbone forward.)
__device__ __forceinline__ int mdiv(int n, unsigned magic) { return magic ? (int)__umulhi((unsigned)n, magic) : n; }   // magic 0: divisor 1

struct DwStripArgs {
    const void* x;
    const void* w;
    const float* bias;
    void* y;
    int D, H, W, nseg, nrb, total;  // nseg = W / PV strips per row, nrb = row blocks per plane, total threads with work
    unsigned magic_nseg, magic_nrb, magic_ppc;
};

template <typename T, int PV, int KR, int ACT>
__global__ void __launch_bounds__(256, PV == 8 ? 2 : 3) dwconv3x3_strip_kernel(const DwStripArgs a) {
    const int H = a.H, W = a.W;
    const int lane = threadIdx.x & 31;
    const long long gi = (long long)blockIdx.x * 256 + threadIdx.x;
    const bool valid = gi < a.total;
    const int i = valid ? (int)gi : a.total - 1;      // spare threads shadow the last strip (they join the shuffles, store nothing)
    const int t = mdiv(i, a.magic_nseg), seg = i - t * a.nseg;
    const int plane = mdiv(t, a.magic_nrb), rb = t - plane * a.nrb;
    const int d = mdiv(plane, a.magic_ppc) % a.D;
    float k[9];
    {
        const T* __restrict__ wk = (const T*)a.w + d * 9;
#pragma unroll
        for (int j = 0; j < 9; ++j) k[j] = to_f<T>(wk[j]);
    }
    const float b = a.bias ? __ldg(a.bias + d) : 0.f;
    const long long origin = (long long)plane * H * W + seg * PV;
    const T* __restrict__ px = (const T*)a.x + origin;
    T* __restrict__ py = (T*)a.y + origin;
    const bool at_left = seg == 0, at_right = seg == a.nseg - 1;
    const int r0 = rb * KR;

    // the KR + 2 input rows of the strip, kept packed until they are needed (rows outside the image are zero)
    using VT = Vec<T, PV>;
    typename VT::Raw raw[KR + 2];
    float edge_l[KR + 2], edge_r[KR + 2];      // columns next to the strip where the neighbour is in another warp
#pragma unroll
    for (int j = 0; j < KR + 2; ++j) {
        const int h = r0 - 1 + j;
        const bool in = h >= 0 && h < H;
        const T* row = px + (long long)h * W;
        if (in) raw[j] = VT::load_raw(row);
        else {
#pragma unroll
            for (int q = 0; q < VT::kWords; ++q) raw[j].w[q] = 0u;
        }
        edge_l[j] = (in && lane == 0 && !at_left) ? to_f<T>(__ldg(row - 1)) : 0.f;
        edge_r[j] = (in && lane == 31 && !at_right) ? to_f<T>(__ldg(row + PV)) : 0.f;
    }
    // window row: [left neighbour, PV own columns, right neighbour]
    auto open_row = [&](int j, float (&wv)[PV + 2]) {
        float v[PV];
        VT::unpack(raw[j], v);
        float l = __shfl_up_sync(0xffffffffu, v[PV - 1], 1), r = __shfl_down_sync(0xffffffffu, v[0], 1);
        if (at_left) l = 0.f;
        else if (lane == 0) l = edge_l[j];
        if (at_right) r = 0.f;
        else if (lane == 31) r = edge_r[j];
        wv[0] = l; wv[PV + 1] = r;
#pragma unroll
        for (int q = 0; q < PV; ++q) wv[q + 1] = v[q];
    };

    if constexpr (PV >= 2) {
        // Packed form: two neighbouring output columns share every instruction (FFMA2).  A window row is kept as pairs
        // at both alignments - (0,1)(2,3).. for the taps dx = 0 and 2, (1,2)(3,4).. for dx = 1 - so that no pair has to
        // be assembled inside the tap loop; the sums run in the same order as the scalar form (same results).
        constexpr int NE = PV / 2 + 1, NO = PV / 2;
        float2 we[3][NE], wo[3][NO];
        auto open_pairs = [&](int j, int slot) {
            float wv[PV + 2];
            open_row(j, wv);
#pragma unroll
            for (int q = 0; q < NE; ++q) we[slot][q] = make_float2(wv[2 * q], wv[2 * q + 1]);
#pragma unroll
            for (int q = 0; q < NO; ++q) wo[slot][q] = make_float2(wv[2 * q + 1], wv[2 * q + 2]);
        };
        open_pairs(0, 0);
        open_pairs(1, 1);
#pragma unroll
        for (int j = 0; j < KR; ++j) {
            open_pairs(j + 2, (j + 2) % 3);
            if (r0 + j < H && valid) {
                float2 acc[PV / 2];
#pragma unroll
                for (int c = 0; c < PV / 2; ++c) acc[c] = make_float2(b, b);
#pragma unroll
                for (int dy = 0; dy < 3; ++dy) {
                    const int sl = (j + dy) % 3;
#pragma unroll
                    for (int dx = 0; dx < 3; ++dx) {
                        const float2 kk = make_float2(k[dy * 3 + dx], k[dy * 3 + dx]);
#pragma unroll
                        for (int c = 0; c < PV / 2; ++c)
                            acc[c] = __ffma2_rn(kk, dx == 1 ? wo[sl][c] : we[sl][c + dx / 2], acc[c]);
                    }
                }
                float o[PV];
#pragma unroll
                for (int c = 0; c < PV / 2; ++c) {
                    float2 q = acc[c];
                    // conv result rounded to the storage type (as the library convolution returns it), then the activation
                    if constexpr (sizeof(T) == 2) q = Half2Of<T>::unpack(Half2Of<T>::pack(q.x, q.y));
                    if constexpr (ACT == ACT_SILU && sizeof(T) == 2) q = silu_pair_fast(q);
                    else { q.x = act_f<ACT>(q.x); q.y = act_f<ACT>(q.y); }
                    o[2 * c] = q.x; o[2 * c + 1] = q.y;
                }
                VT::store(py + (long long)(r0 + j) * W, o);
            }
        }
    } else {
        float win[3][PV + 2];
        open_row(0, win[0]);
        open_row(1, win[1]);
#pragma unroll
        for (int j = 0; j < KR; ++j) {
            open_row(j + 2, win[(j + 2) % 3]);
            if (r0 + j < H && valid) {
                float o[PV];
#pragma unroll
                for (int c = 0; c < PV; ++c) {
                    float acc = b;
#pragma unroll
                    for (int dy = 0; dy < 3; ++dy)
#pragma unroll
                        for (int dx = 0; dx < 3; ++dx) acc = fmaf(k[dy * 3 + dx], win[(j + dy) % 3][c + dx], acc);
                    o[c] = act_f<ACT>(round_to<T>(acc));
                }
                VT::store(py + (long long)(r0 + j) * W, o);
            }
        }
    }
}

template <typename T, int PV, int KR>
static int launch_dw_strip_a(const DwStripArgs& a, int act, unsigned grid, cudaStream_t st) {
    if (act == ACT_SILU) dwconv3x3_strip_kernel<T, PV, KR, ACT_SILU><<<grid, 256, 0, st>>>(a);
    else if (act == ACT_GELU) dwconv3x3_strip_kernel<T, PV, KR, ACT_GELU><<<grid, 256, 0, st>>>(a);
    else dwconv3x3_strip_kernel<T, PV, KR, ACT_NONE><<<grid, 256, 0, st>>>(a);
    count_launch();
    return check_launch();
}

template <typename T>
static int launch_dw_strip(DwStripArgs a, int pv, int kr, int act, unsigned grid, cudaStream_t st) {
    if (kr == 8) {
        if (pv == 8) return launch_dw_strip_a<T, 8, 8>(a, act, grid, st);
        if (pv == 4) return launch_dw_strip_a<T, 4, 8>(a, act, grid, st);
        if (pv == 2) return launch_dw_strip_a<T, 2, 8>(a, act, grid, st);
        return launch_dw_strip_a<T, 1, 8>(a, act, grid, st);
    }
    if (pv == 8) return launch_dw_strip_a<T, 8, 7>(a, act, grid, st);
    if (pv == 4) return launch_dw_strip_a<T, 4, 7>(a, act, grid, st);
    if (pv == 2) return launch_dw_strip_a<T, 2, 7>(a, act, grid, st);
    return launch_dw_strip_a<T, 1, 7>(a, act, grid, st);
}

int dwconv3x3_act(const ss2d_pointwise_params* p, cudaStream_t st) {
    if (!p) return SS2D_EINVAL_NULL;
    if (!p->x || !p->y || !p->weight) return SS2D_EINVAL_NULL;
    if (p->x == p->y) return SS2D_ENOTSUP;       // neighbours are read: not an in-place operation
    if (!dtype_ok(p->dtype)) return SS2D_EINVAL_DTYPE;
    if (p->act < 0 || p->act > 2) return SS2D_ENOTSUP;
    if (p->B <= 0 || p->D <= 0 || p->H <= 0 || p->W <= 0) return SS2D_EINVAL_SHAPE;
    if (p->H * p->W > 0x3fffffffLL || p->W > 8192) return SS2D_EINVAL_SHAPE;
    const size_t s = dtype_size(p->dtype);
    if (!aligned_to(p->x, s) || !aligned_to(p->y, s) || !aligned_to(p->weight, s) || !aligned_to(p->bias, 4)) return SS2D_EINVAL_ALIGN;
    const long long L = p->H * p->W;
    int pv = (s == 2) ? 8 : 4;
    auto fit = [&](long long x) { while (pv > 1 && (x % pv) != 0) pv >>= 1; };
    fit(p->W); fit(L);
    fit((long long)(reinterpret_cast<uintptr_t>(p->x) / s));
    fit((long long)(reinterpret_cast<uintptr_t>(p->y) / s));
    const int kr = (p->H % 8 == 0 || p->H % 7 != 0) ? 8 : 7;      // rows per thread: whichever divides the map better
    const long long nseg = p->W / pv, nrb = (p->H + kr - 1) / kr, planes = p->B * p->D;
    const long long total = planes * nrb * nseg;
    // every index split inside the kernel is a multiply-shift that needs numerator * divisor < 2^32
    if (total >= (1LL << 31) || total * nseg >= (1LL << 32) || planes * nrb * nrb >= (1LL << 32) || planes * p->B >= (1LL << 32))
        return SS2D_EINVAL_SHAPE;
    auto magic = [](long long d) { return d > 1 ? (unsigned)(((1ULL << 32) + (unsigned long long)d - 1) / (unsigned long long)d) : 0u; };
    DwStripArgs a;
    a.x = p->x; a.w = p->weight; a.bias = (const float*)p->bias; a.y = p->y;
    a.D = (int)p->D; a.H = (int)p->H; a.W = (int)p->W; a.nseg = (int)nseg; a.nrb = (int)nrb; a.total = (int)total;
    a.magic_nseg = magic(nseg); a.magic_nrb = magic(nrb); a.magic_ppc = magic(p->channel_major ? p->B : 1);
    const unsigned grid = (unsigned)((total + 255) / 256);
    if (p->dtype == SS2D_F32) return launch_dw_strip<float>(a, pv, kr, p->act, grid, st);
    if (p->dtype == SS2D_BF16) return launch_dw_strip<__nv_bfloat16>(a, pv, kr, p->act, grid, st);
    return launch_dw_strip<__half>(a, pv, kr, p->act, grid, st);
}

}  // namespace ss2d
