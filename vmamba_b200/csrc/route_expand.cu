// Per-route expansion of the low-rank projections into the streams the fused scan consumes.
//
// Input: x_dbl = x_proj(x) computed ONCE on the map in its native (row-major) pixel order,
// (B, 4, R+2N, L).  For every route k this kernel writes, in the ORIENTATION order of the route
// (row-major pixels for k = 0, 2; column-major for k = 1, 3):
//   delta_k[b, d, q] = sum_r Wdt[k, d, r] * x_dbl[b, k, r, pix(q)]     (R -> D, rounded to the activation type)
//   bc_k[b, n, q]    = x_dbl[b, k, R + n, pix(q)]   n < 2N            (B then C rows, activation type)
// i.e. dt_projs (a grouped 1x1 convolution with a contraction length of only R = 6..64), the
// split/contiguous copies, and the CrossScan permutation of the projected rows, in one pass whose
// cost is the write of delta.  The contraction is far too short and the output far too large for
// the tensor cores to matter: the kernel is bound by the delta write for R <= 12 and by fp32 FMA
// issue (packed f32x2) for the deep, small stages.
//
// Mapping: an "item" is VEC consecutive pixels q of one (image, route) plane.  A CTA stages the
// R+2N projected rows of NI items in shared memory as fp32 (the column-major gather happens
// here), then thread (item, channel group) accumulates 4 channels x VEC pixels at a time with
// the weights broadcast from shared memory; lanes of a warp hold consecutive items, so every
// delta store is a full 512-byte line per channel.
#include "common.cuh"

namespace ss2d {

struct ExpandArgs {
    const void* xd;      // (B, 4, C, L)
    const void* wdt;     // (4, D, R) activation dtype
    void* delta[4];      // (B, D, L) each
    void* bc[4];         // (B, 2N, L) each, activation dtype
    long long xd_bs, xd_ks, xd_rs;     // element strides of x_dbl: batch, route, row
    long long d_bs[4], d_cs[4], bc_bs[4], bc_rs[4];   // delta: batch / channel strides; B-C rows: batch / row strides
    int B, D, R, N2, C, H, W, L;       // N2 = 2N, C = R + 2N; L = run length (H*W, or B*H*W when images are adjacent)
    int Limg;                          // H * W
    int items_per_plane, items_total;  // L / VEC, B * L / VEC
};

constexpr int kExpThreads = 256;
constexpr int kDChunk = 128;   // channels per CTA (grid.z walks the slices)

template <typename T, int VEC, int NI>
__global__ void __launch_bounds__(kExpThreads) route_expand_kernel(const ExpandArgs a) {
    constexpr int NDG = kExpThreads / NI;   // channel groups working side by side
    constexpr int NP = (VEC + 1) / 2;
    extern __shared__ __align__(16) float sm[];
    float* s_rows = sm;                                  // [C][NI * VEC]
    float* s_w = sm + (size_t)a.C * NI * VEC;            // [R][kDChunk] (transposed: 4 channels = one float4)
    const int k = blockIdx.y;
    const bool col = (k & 1) != 0;
    const int tid = threadIdx.x;
    const int item0 = blockIdx.x * NI;
    const T* __restrict__ xd = (const T*)a.xd + (long long)k * a.xd_ks;

    // ---- stage the projected rows of this CTA's items (gathering column-major pixels for odd k) ----
    const int it = tid % NI, dg = tid / NI;
    const int item = item0 + it;
    const bool live = item < a.items_total;
    const int b = live ? item / a.items_per_plane : 0;
    const int q0 = live ? (item - b * a.items_per_plane) * VEC : 0;
    {
        const int img0 = (q0 / a.Limg) * a.Limg, qi = q0 - img0;     // image of the first pixel, position inside it
        const int w0 = qi / a.H, h0 = qi - w0 * a.H;
        const T* src = xd + (long long)b * a.xd_bs;
        for (int row = dg; row < a.C; row += NDG) {
            float v[VEC];
#pragma unroll
            for (int i = 0; i < VEC; ++i) v[i] = 0.f;
            if (live) {
                const T* rp = src + (long long)row * a.xd_rs;
                if (!col) {
                    Vec<T, VEC>::load(rp + q0, v);
                } else {
                    int w = w0, h = h0, base = img0;      // a run may continue into the next image
#pragma unroll
                    for (int i = 0; i < VEC; ++i) {
                        v[i] = to_f<T>(rp[base + h * a.W + w]);
                        if (++h == a.H) { h = 0; if (++w == a.W) { w = 0; base += a.Limg; } }
                    }
                }
            }
            Vec<float, VEC>::store(s_rows + (size_t)row * (NI * VEC) + it * VEC, v);
        }
    }
    // this CTA's slice of the channels (grid.z splits D so that small maps still fill the GPU)
    const int dc = blockIdx.z * kDChunk;
    const int dn = min(kDChunk, a.D - dc);
    const T* __restrict__ wk = (const T*)a.wdt + (long long)k * a.D * a.R;
    for (int idx = tid; idx < kDChunk * a.R; idx += kExpThreads) {
        const int r = idx / kDChunk, dl = idx - r * kDChunk;
        s_w[idx] = (dl < dn) ? to_f<T>(wk[(long long)(dc + dl) * a.R + r]) : 0.f;
    }
    __syncthreads();

    // ---- B / C rows: pass through (first channel slice only) --------------------------------
    if (live && blockIdx.z == 0) {
        for (int n = dg; n < a.N2; n += NDG) {
            float v[VEC];
            Vec<float, VEC>::load_plain(s_rows + (size_t)(a.R + n) * (NI * VEC) + it * VEC, v);
            Vec<T, VEC>::store((T*)a.bc[k] + b * a.bc_bs[k] + (long long)n * a.bc_rs[k] + q0, v);
        }
    }

    // ---- delta: R -> D expansion for the channels of this slice -------------------------------------
    T* __restrict__ dout = (T*)a.delta[k] + b * a.d_bs[k] + q0;
    for (int dl0 = dg * 4; dl0 < dn; dl0 += NDG * 4) {
        float2 acc[4][NP];
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int j = 0; j < NP; ++j) acc[c][j] = make_float2(0.f, 0.f);
#pragma unroll 2
        for (int r = 0; r < a.R; ++r) {
            float sv[VEC];
            Vec<float, VEC>::load_plain(s_rows + (size_t)r * (NI * VEC) + it * VEC, sv);
            const float4 w4 = *reinterpret_cast<const float4*>(s_w + r * kDChunk + dl0);
            const float wv[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
            for (int c = 0; c < 4; ++c) {
#pragma unroll
                for (int j = 0; j < NP; ++j) {
                    const float2 s2 = make_float2(sv[2 * j], (VEC > 1) ? sv[(2 * j + 1) % VEC] : 0.f);
                    acc[c][j] = __ffma2_rn(make_float2(wv[c], wv[c]), s2, acc[c][j]);
                }
            }
        }
        if (live) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                if (dl0 + c < dn) {
                    float o[VEC];
#pragma unroll
                    for (int i = 0; i < VEC; ++i) o[i] = (i & 1) ? acc[c][i >> 1].y : acc[c][i >> 1].x;
                    Vec<T, VEC>::store(dout + (long long)(dc + dl0 + c) * a.d_cs[k], o);
                }
            }
        }
    }
}

template <typename T, int VEC, int NI>
static int launch_expand(const ExpandArgs& a, cudaStream_t st) {
    const size_t smem = ((size_t)a.C * NI * VEC + (size_t)a.R * kDChunk) * sizeof(float);
    if (smem > 200 * 1024) return SS2D_ENOTSUP;
    auto kern = route_expand_kernel<T, VEC, NI>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return SS2D_ECUDA;
    const dim3 grid((unsigned)((a.items_total + NI - 1) / NI), 4, (unsigned)((a.D + kDChunk - 1) / kDChunk));
    kern<<<grid, kExpThreads, smem, st>>>(a);
    count_launch();
    return check_launch();
}

template <typename T, int VEC>
static int launch_expand_ni(const ExpandArgs& a, cudaStream_t st) {
    // fewer items per CTA when many rows have to be staged
    if ((size_t)a.C * 64 * VEC * 4 <= 56 * 1024) return launch_expand<T, VEC, 64>(a, st);
    return launch_expand<T, VEC, 32>(a, st);
}

template <typename T>
static int launch_expand_v(const ExpandArgs& a, int vec, cudaStream_t st) {
    switch (vec) {
        case 8: return launch_expand_ni<T, 8>(a, st);
        case 4: return launch_expand_ni<T, 4>(a, st);
        case 2: return launch_expand_ni<T, 2>(a, st);
        default: return launch_expand_ni<T, 1>(a, st);
    }
}

int route_expand(const ss2d_expand_params* p, cudaStream_t st) {
    if (!p) return SS2D_EINVAL_NULL;
    if (!p->x_dbl || !p->dt_weight) return SS2D_EINVAL_NULL;
    for (int k = 0; k < 4; ++k)
        if (!p->delta[k] || !p->bc[k]) return SS2D_EINVAL_NULL;
    if (!dtype_ok(p->act_dtype)) return SS2D_EINVAL_DTYPE;
    if (p->B <= 0 || p->D <= 0 || p->R <= 0 || p->N <= 0 || p->H <= 0 || p->W <= 0) return SS2D_EINVAL_SHAPE;
    const long long L = p->H * p->W;
    if (L > 0x3fffffffLL || p->B * L > 0x7fffffffLL || p->R > 1024 || p->N > SS2D_MAX_DSTATE) return SS2D_EINVAL_SHAPE;
    const long long C = p->R + 2 * p->N;
    const long long xd_rs = p->x_dbl_row_stride ? p->x_dbl_row_stride : L;
    if (xd_rs < L || p->x_dbl_route_stride < L || (p->B > 1 && p->x_dbl_batch_stride < L)) return SS2D_EINVAL_STRIDE;
    const size_t s = dtype_size(p->act_dtype);
    if (!aligned_to(p->x_dbl, s) || !aligned_to(p->dt_weight, s)) return SS2D_EINVAL_ALIGN;
    for (int k = 0; k < 4; ++k) {
        if (!aligned_to(p->delta[k], s) || !aligned_to(p->bc[k], s)) return SS2D_EINVAL_ALIGN;
        if (p->B > 1 && (p->delta_batch_stride[k] < L || p->bc_batch_stride[k] < L)) return SS2D_EINVAL_STRIDE;
        if ((p->delta_channel_stride[k] && p->delta_channel_stride[k] < L) || (p->bc_row_stride[k] && p->bc_row_stride[k] < L)) return SS2D_EINVAL_STRIDE;
    }
    // images adjacent in every tensor (channel-major maps): one run of B*L pixels per row, so that the
    // vector width does not depend on the size of a single map
    bool flat = p->B > 1 && p->x_dbl_batch_stride == L;
    for (int k = 0; k < 4; ++k) flat = flat && p->delta_batch_stride[k] == L && p->bc_batch_stride[k] == L;
    const long long run = flat ? p->B * L : L;
    // widest pixel vector that keeps every row start aligned in every tensor
    int vec = 8;
    auto fit = [&](long long x) { if (x < 0) x = -x; while (vec > 1 && (x % vec) != 0) vec >>= 1; };
    fit(run); fit(p->x_dbl_route_stride); fit(xd_rs);
    if (!flat) fit(p->x_dbl_batch_stride);
    fit((long long)(reinterpret_cast<uintptr_t>(p->x_dbl) / s));
    for (int k = 0; k < 4; ++k) {
        if (!flat) { fit(p->delta_batch_stride[k]); fit(p->bc_batch_stride[k]); }
        fit(p->delta_channel_stride[k] ? p->delta_channel_stride[k] : L); fit(p->bc_row_stride[k] ? p->bc_row_stride[k] : L);
        fit((long long)(reinterpret_cast<uintptr_t>(p->delta[k]) / s));
        fit((long long)(reinterpret_cast<uintptr_t>(p->bc[k]) / s));
    }
    // the staged rows (C rows x 64 items x vec floats) should stay near 28 KB so that several CTAs share an SM
    while (vec > 1 && C * 64 * vec * 4 > 28 * 1024) vec >>= 1;
    ExpandArgs a;
    a.xd = p->x_dbl; a.wdt = p->dt_weight;
    for (int k = 0; k < 4; ++k) {
        a.delta[k] = p->delta[k]; a.bc[k] = p->bc[k];
        a.d_bs[k] = p->delta_batch_stride[k]; a.bc_bs[k] = p->bc_batch_stride[k];
        a.d_cs[k] = p->delta_channel_stride[k] ? p->delta_channel_stride[k] : L;
        a.bc_rs[k] = p->bc_row_stride[k] ? p->bc_row_stride[k] : L;
    }
    a.xd_bs = p->x_dbl_batch_stride; a.xd_ks = p->x_dbl_route_stride; a.xd_rs = xd_rs;
    a.B = (int)p->B; a.D = (int)p->D; a.R = (int)p->R; a.N2 = (int)(2 * p->N); a.C = (int)C;
    a.H = (int)p->H; a.W = (int)p->W; a.L = (int)run; a.Limg = (int)L;
    if (flat) a.B = 1;
    a.items_per_plane = (int)(run / vec);
    a.items_total = (int)((flat ? 1 : p->B) * (run / vec));
    if (p->act_dtype == SS2D_F32) return launch_expand_v<float>(a, vec, st);
    if (p->act_dtype == SS2D_BF16) return launch_expand_v<__nv_bfloat16>(a, vec, st);
    return launch_expand_v<__half>(a, vec, st);
}

}  // namespace ss2d
