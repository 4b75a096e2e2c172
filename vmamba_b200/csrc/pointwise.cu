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
// loop has no division: the kernel is bound by instruction issue (the erf of GELU), not by HBM.
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
                    const float2 r = gelu_pair_fast(make_float2(v[i] + b, v[i + 1] + b));
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
// Depthwise 3x3, stride 1, zero padding 1.  A work unit is a band of BH rows of one plane (the whole
// plane when it is small); a CTA owns PP units.  Each band is staged once in shared memory as fp32
// with its two halo rows inside a one-pixel zero frame (pitch W + 2); consecutive threads then take
// consecutive columns and walk 8 rows with the 3x3 window sliding in registers.  HBM traffic is the
// minimum for whole planes (every element read once, written once); banded planes re-read two
// halo rows per band.
struct DwArgs {
    const void* x;
    const void* w;       // (D, 3, 3) storage type
    const float* bias;   // (D) or null
    void* y;
    int D, H, W, PP, nvw;           // nvw = W / PV runs per row
    int BH, nb, units;              // rows per band, bands per plane, planes * nb
    int planes_per_channel;         // 1 for (B, D, H, W) maps, B for (D, B, H, W) maps
    int nrb;                        // row blocks of 8 per band
    int krows;                      // rows per thread in the compute phase (7 or 8: whichever divides the band better)
    int flat;                       // bit 0: flat loads, bit 1: flat stores;  whole planes, consecutive in memory and 16-byte aligned per CTA: flat vector loads / stores
    unsigned magic_L;
    unsigned magic_fr, magic_nvw, magic_W, magic_nrb, magic_ppc, magic_nb, magic_frnvw, magic_nrbW, magic_W2, magic_nrbW2;
};

__device__ __forceinline__ int mdiv(int n, unsigned magic) { return magic ? (int)__umulhi((unsigned)n, magic) : n; }   // magic 0: divisor 1

template <typename T, int PV, int ACT>
__global__ void __launch_bounds__(256) dwconv3x3_act_kernel(const DwArgs a) {
    extern __shared__ __align__(16) float sm[];
    const int H = a.H, W = a.W, Wp = W + 2, FR = a.BH + 2;      // frame rows
    const int unit0 = blockIdx.x * a.PP;
    const int np = min(a.PP, a.units - unit0);
    const int frame = FR * Wp;
    // frame cells that no load will write: the left and right columns, and the rows above / below the image
    for (int i = threadIdx.x; i < np * FR; i += blockDim.x) {
        const int pl = mdiv(i, a.magic_fr), fr = i - pl * FR;
        float* row = sm + pl * frame + fr * Wp;
        row[0] = 0.f; row[W + 1] = 0.f;
    }
    const T* __restrict__ x = (const T*)a.x;
    T* obuf = reinterpret_cast<T*>(sm + ((a.PP * frame + 3) & ~3));   // flat mode: the CTA's outputs, np * H * W
    if (a.flat & 1) {
        // whole planes, consecutive in memory: the CTA's input is one run of np * H * W elements, read as
        // 16-byte vectors whatever the row length, and scattered into the frames
        for (int i = threadIdx.x; i < np * 2 * Wp; i += blockDim.x) {       // rows above and below the image
            const int pl = i / (2 * Wp), rem = i - pl * (2 * Wp);
            sm[pl * frame + (rem < Wp ? rem : (H + 1) * Wp + rem - Wp)] = 0.f;
        }
        constexpr int FV = 16 / (int)sizeof(T);
        const int total = np * H * W;
        const T* src = x + (long long)unit0 * H * W;
        for (int e0 = threadIdx.x * FV; e0 < total; e0 += blockDim.x * FV) {
            int pl = mdiv(e0, a.magic_L), rem = e0 - pl * (H * W);
            int h = mdiv(rem, a.magic_W), w = rem - h * W;
            T v[FV];
            if (e0 + FV <= total) *reinterpret_cast<uint4*>(v) = __ldg(reinterpret_cast<const uint4*>(src + e0));
            else {
#pragma unroll
                for (int j = 0; j < FV; ++j) v[j] = (e0 + j < total) ? src[e0 + j] : from_f<T>(0.f);
            }
#pragma unroll
            for (int j = 0; j < FV; ++j) {
                if (e0 + j < total) sm[pl * frame + (h + 1) * Wp + w + 1] = to_f<T>(v[j]);
                if (++w == W) { w = 0; if (++h == H) { h = 0; ++pl; } }
            }
        }
    } else
    for (int i = threadIdx.x; i < np * FR * a.nvw; i += blockDim.x) {
        const int pl = mdiv(i, a.magic_frnvw), rem = i - pl * (FR * a.nvw);
        const int fr = mdiv(rem, a.magic_nvw), v = rem - fr * a.nvw;
        const int u = unit0 + pl;
        const int plane = mdiv(u, a.magic_nb), band = u - plane * a.nb;
        const int h = band * a.BH - 1 + fr;                       // image row held by this frame row
        float val[PV];
        if (h >= 0 && h < H) Vec<T, PV>::load(x + ((long long)plane * H + h) * W + v * PV, val);   // PV divides W
        else {
#pragma unroll
            for (int j = 0; j < PV; ++j) val[j] = 0.f;
        }
        float* dst = sm + pl * frame + fr * Wp + v * PV + 1;
#pragma unroll
        for (int j = 0; j < PV; ++j) dst[j] = val[j];
    }
    __syncthreads();
    const int kRows = a.krows;
    const int nrb = a.nrb;
    if ((W & 1) == 0) {
        // two neighbouring columns per thread: four frame values per row (two 8-byte loads) serve eighteen
        // FMAs, and the two results leave as one store
        const int W2 = W >> 1;
        for (int i = threadIdx.x; i < np * nrb * W2; i += blockDim.x) {
            const int pl = mdiv(i, a.magic_nrbW2), rem = i - pl * (nrb * W2);
            const int rb = mdiv(rem, a.magic_W2), w = (rem - rb * W2) * 2;
            const int u = unit0 + pl;
            const int plane = mdiv(u, a.magic_nb), band = u - plane * a.nb;
            const int r0 = rb * kRows;
            const int rows = min(min(r0 + kRows, a.BH), H - band * a.BH) - r0;
            if (rows <= 0) continue;
            const int d = mdiv(plane, a.magic_ppc) % a.D;
            const T* __restrict__ wk = (const T*)a.w + d * 9;
            float k[9];
#pragma unroll
            for (int j = 0; j < 9; ++j) k[j] = to_f<T>(wk[j]);
            const float b = a.bias ? __ldg(a.bias + d) : 0.f;
            const float* src = sm + pl * frame + r0 * Wp + w;
            float2 ta = *reinterpret_cast<const float2*>(src), tb = *reinterpret_cast<const float2*>(src + 2);
            float2 ma = *reinterpret_cast<const float2*>(src + Wp), mb = *reinterpret_cast<const float2*>(src + Wp + 2);
            T* __restrict__ out = (T*)a.y + ((long long)plane * H + band * a.BH + r0) * W + w;
            for (int r = 0; r < rows; ++r) {
                const float* bp = src + (r + 2) * Wp;
                const float2 ba = *reinterpret_cast<const float2*>(bp), bb = *reinterpret_cast<const float2*>(bp + 2);
                float a0 = b, a1 = b;
                a0 = fmaf(k[0], ta.x, a0); a0 = fmaf(k[1], ta.y, a0); a0 = fmaf(k[2], tb.x, a0);
                a1 = fmaf(k[0], ta.y, a1); a1 = fmaf(k[1], tb.x, a1); a1 = fmaf(k[2], tb.y, a1);
                a0 = fmaf(k[3], ma.x, a0); a0 = fmaf(k[4], ma.y, a0); a0 = fmaf(k[5], mb.x, a0);
                a1 = fmaf(k[3], ma.y, a1); a1 = fmaf(k[4], mb.x, a1); a1 = fmaf(k[5], mb.y, a1);
                a0 = fmaf(k[6], ba.x, a0); a0 = fmaf(k[7], ba.y, a0); a0 = fmaf(k[8], bb.x, a0);
                a1 = fmaf(k[6], ba.y, a1); a1 = fmaf(k[7], bb.x, a1); a1 = fmaf(k[8], bb.y, a1);
                const float o[2] = {act_f<ACT>(round_to<T>(a0)), act_f<ACT>(round_to<T>(a1))};
                if (a.flat & 2) Vec<T, 2>::store(obuf + (pl * H + r0 + r) * W + w, o);
                else Vec<T, 2>::store(out + r * W, o);
                ta = ma; tb = mb; ma = ba; mb = bb;
            }
        }
    } else
    for (int i = threadIdx.x; i < np * nrb * W; i += blockDim.x) {
        const int pl = mdiv(i, a.magic_nrbW), rem = i - pl * (nrb * W);
        const int rb = mdiv(rem, a.magic_W), w = rem - rb * W;
        const int u = unit0 + pl;
        const int plane = mdiv(u, a.magic_nb), band = u - plane * a.nb;
        const int r0 = rb * kRows;                                 // first row of this block inside the band
        const int rows = min(min(r0 + kRows, a.BH), H - band * a.BH) - r0;
        if (rows <= 0) continue;
        const int d = mdiv(plane, a.magic_ppc) % a.D;
        const T* __restrict__ wk = (const T*)a.w + d * 9;
        float k[9];
#pragma unroll
        for (int j = 0; j < 9; ++j) k[j] = to_f<T>(wk[j]);
        const float b = a.bias ? __ldg(a.bias + d) : 0.f;
        const float* src = sm + pl * frame + r0 * Wp + w;        // frame row r0 is the row above output row r0
        float t0 = src[0], t1 = src[1], t2 = src[2];
        float m0 = src[Wp], m1 = src[Wp + 1], m2 = src[Wp + 2];
        T* __restrict__ out = (T*)a.y + ((long long)plane * H + band * a.BH + r0) * W + w;
        for (int r = 0; r < rows; ++r) {
            const float* bp = src + (r + 2) * Wp;
            const float b0 = bp[0], b1 = bp[1], b2 = bp[2];
            float acc = b;
            acc = fmaf(k[0], t0, acc); acc = fmaf(k[1], t1, acc); acc = fmaf(k[2], t2, acc);
            acc = fmaf(k[3], m0, acc); acc = fmaf(k[4], m1, acc); acc = fmaf(k[5], m2, acc);
            acc = fmaf(k[6], b0, acc); acc = fmaf(k[7], b1, acc); acc = fmaf(k[8], b2, acc);
            if (a.flat & 2) obuf[(pl * H + r0 + r) * W + w] = from_f<T>(act_f<ACT>(round_to<T>(acc)));
            else out[r * W] = from_f<T>(act_f<ACT>(round_to<T>(acc)));
            t0 = m0; t1 = m1; t2 = m2; m0 = b0; m1 = b1; m2 = b2;
        }
    }
    if (a.flat & 2) {         // the CTA's outputs leave as one run of 16-byte vectors
        __syncthreads();
        constexpr int FV = 16 / (int)sizeof(T);
        const int total = np * H * W;
        T* dst = (T*)a.y + (long long)unit0 * H * W;
        for (int e0 = threadIdx.x * FV; e0 < total; e0 += blockDim.x * FV) {
            if (e0 + FV <= total) *reinterpret_cast<uint4*>(dst + e0) = *reinterpret_cast<const uint4*>(obuf + e0);
            else for (int j = 0; e0 + j < total; ++j) dst[e0 + j] = obuf[e0 + j];
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
    a.krows = (a.BH % 8 == 0 || a.BH % 7 != 0) ? 8 : 7;
    a.nrb = (a.BH + a.krows - 1) / a.krows;
    auto magic = [](long long d) { return d > 1 ? (unsigned)(((1ULL << 32) + (unsigned long long)d - 1) / (unsigned long long)d) : 0u; };
    const int FR = a.BH + 2;
    a.magic_fr = magic(FR); a.magic_nvw = magic(a.nvw); a.magic_W = magic(a.W); a.magic_nrb = magic(a.nrb);
    a.magic_ppc = magic(a.planes_per_channel); a.magic_nb = magic(a.nb);
    a.magic_frnvw = magic((long long)FR * a.nvw); a.magic_nrbW = magic((long long)a.nrb * a.W);
    a.magic_W2 = magic(a.W / 2); a.magic_nrbW2 = magic((long long)a.nrb * (a.W / 2));
    a.magic_L = magic((long long)a.H * a.W);
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
    if (p->H * p->W > 0x3fffffffLL || p->W > 8192) return SS2D_EINVAL_SHAPE;
    const size_t s = dtype_size(p->dtype);
    if (!aligned_to(p->x, s) || !aligned_to(p->y, s) || !aligned_to(p->weight, s) || !aligned_to(p->bias, 4)) return SS2D_EINVAL_ALIGN;
    const long long L = p->H * p->W;
    int pv = (s == 2) ? 8 : 4;
    auto fit = [&](long long x) { while (pv > 1 && (x % pv) != 0) pv >>= 1; };
    fit(p->W); fit(L);
    fit((long long)(reinterpret_cast<uintptr_t>(p->x) / s));
    fit((long long)(reinterpret_cast<uintptr_t>(p->y) / s));
    // band height: the whole plane if its frame fits in 40 KB, else as many rows as do
    const long long Wp = p->W + 2;
    long long BH = p->H;
    while (BH > 8 && (BH + 2) * Wp * 4 > 40 * 1024) BH = (BH + 1) / 2;
    BH = (BH + 7) / 8 * 8;                      // whole 8-row blocks
    if (BH > p->H) BH = p->H;
    const long long nb = (p->H + BH - 1) / BH;
    const size_t frame = (size_t)(BH + 2) * Wp * sizeof(float);
    if (frame > 160 * 1024) return SS2D_ENOTSUP;
    const long long units = p->B * p->D * nb;
    long long PP = (2048 * 4 + BH * p->W - 1) / (BH * p->W);      // about 8192 outputs per CTA
    if (PP < 1) PP = 1;
    while (PP > 1 && PP * frame > 48 * 1024) --PP;
    if (PP > units) PP = units;
    // flat mode: rows too short for 16-byte vectors, whole-plane bands, planes dense in memory; PP planes must
    // keep every CTA's run 16-byte aligned
    const long long fv = 16 / (long long)s;
    bool flat = nb == 1 && pv == 1 && fv > 1 && aligned_to(p->x, 16) && aligned_to(p->y, 16);   // measured: pays only for odd row lengths
    if (flat) {
        long long step = fv;
        for (long long gcd_a = L, gcd_b = fv; gcd_b; ) { const long long t = gcd_a % gcd_b; gcd_a = gcd_b; gcd_b = t; if (!gcd_b) step = fv / gcd_a; }
        long long PPf = PP / step * step;
        if (PPf < step) PPf = step;
        if (PPf * (frame + L * s) + 32 > 64 * 1024) flat = false; else PP = PPf;
    }
    const long long grid = (units + PP - 1) / PP;
    // every index split inside the kernel is a multiply-shift that needs numerator * divisor < 2^32
    if (units * nb >= (1LL << 32) || p->B * p->D * p->B >= (1LL << 32) || grid > 0x7fffffffLL) return SS2D_EINVAL_SHAPE;
    DwArgs a;
    a.x = p->x; a.w = p->weight; a.bias = (const float*)p->bias; a.y = p->y;
    a.D = (int)p->D; a.H = (int)p->H; a.W = (int)p->W; a.PP = (int)PP; a.nvw = 0;
    a.BH = (int)BH; a.nb = (int)nb; a.units = (int)units;
    a.planes_per_channel = p->channel_major ? (int)p->B : 1;
    a.flat = flat ? 3 : 0;
    const size_t smem = flat ? ((size_t)PP * frame + 15) / 16 * 16 + ((size_t)PP * L * s + 15) / 16 * 16 : (size_t)PP * frame;
    if (p->dtype == SS2D_F32) return launch_dw_v<float>(a, pv, p->act, smem, (unsigned)grid, st);
    if (p->dtype == SS2D_BF16) return launch_dw_v<__nv_bfloat16>(a, pv, p->act, smem, (unsigned)grid, st);
    return launch_dw_v<__half>(a, pv, p->act, smem, (unsigned)grid, st);
}

}  // namespace ss2d
