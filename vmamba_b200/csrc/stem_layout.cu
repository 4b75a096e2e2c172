// The strided 3x3 convolutions of the patch embedding and of the downsampling layers run in the
// library (cuDNN) on pixel-major (B, H, W, C) maps, the layout its tensor-core kernels use; the trunk
// of the backbone keeps channel-major planes (C, B, H, W).  The three kernels here sit on that seam
// and fold the neighbouring elementwise work into the layout change, so that no separate conversion
// pass and no separate LayerNorm / cast pass touches HBM:
//
//   stem_conv_norm_act   image (B, 3, H, W) -> conv 3x3 stride 2 (3 -> C0) + bias -> LayerNorm over C0 -> GELU
//                        -> (B, H/2, W/2, C0).  16-bit images: 16 output pixels x C0 channels x 27 taps as
//                        mma.sync steps, LayerNorm and GELU on the accumulators (stem_mma_kernel); fp32
//                        images: a pair of lanes owns two neighbouring output pixels with the C0 channels
//                        in registers (packed FMAs), one lane exchange for the LayerNorm.
//   pixels_norm_to_planes (N, C) pixel-major rows + bias -> LayerNorm over C -> (C, N) planes (fp32 or 16-bit)
//   planes_to_pixels      (C, N) fp32 planes (+ add + bias, optionally written back) -> (N, C) pixel-major 16-bit
// N counts the pixels of the whole batch (b, h, w): pixel-major row n and element n of every plane
// are the same pixel.
#include "activations.cuh"

namespace ss2d {

// ------------------------------------------------------------------------------------------------
struct StemArgs {
    const void* x;        // (B, 3, H, W)
    const void* w;        // (C0, 3, 3, 3)
    const float *cbias, *lnw, *lnb;
    void* y;              // (B, Ho, Wo, C0)
    int B, H, W, Ho, Wo;
    float eps;
};

template <typename T, int C0>
__global__ void __launch_bounds__(128, 4) stem_conv_norm_act_kernel(const StemArgs a) {
    // weights as [tap][channel] fp32 so that one 16-byte broadcast load brings a tap's weights of four channels
    __shared__ __align__(16) float sw[27 * C0];
    __shared__ float sb[3 * C0];
    constexpr int CH = C0 / 2;                    // two neighbouring lanes share a pixel pair: half of the channels each
    static_assert(CH % 8 == 0, "16-byte stores per half");
    for (int i = threadIdx.x; i < 27 * C0; i += blockDim.x) {
        const int c = i / 27, tap = i - c * 27;
        sw[tap * C0 + c] = to_f<T>(((const T*)a.w)[i]);
    }
    for (int i = threadIdx.x; i < C0; i += blockDim.x) {
        sb[i] = a.cbias ? a.cbias[i] : 0.f;
        sb[C0 + i] = a.lnw ? a.lnw[i] : 1.f;
        sb[2 * C0 + i] = a.lnb ? a.lnb[i] : 0.f;
    }
    __syncthreads();
    const int pairs_per_row = (a.Wo + 1) / 2;
    const long long total = (long long)a.B * a.Ho * pairs_per_row;
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int half = (int)(tid & 1);
    const bool live = (tid >> 1) < total;
    const long long gid = live ? (tid >> 1) : total - 1;      // idle lanes shadow the last pair and store nothing
    const int px = (int)(gid % pairs_per_row);
    const long long rest = gid / pairs_per_row;
    const int oy = (int)(rest % a.Ho);
    const int b = (int)(rest / a.Ho);
    const int ox0 = 2 * px;                       // output pixels (oy, ox0) and (oy, ox0 + 1)
    const bool two = ox0 + 1 < a.Wo;
    // input window: rows 2*oy-1 .. 2*oy+1, columns 2*ox0-1 .. 2*ox0+3 (five columns serve both pixels)
    float in[3][3][5];
    const T* xb = (const T*)a.x + (long long)b * 3 * a.H * a.W;
#pragma unroll
    for (int ky = 0; ky < 3; ++ky) {
        const int iy = 2 * oy - 1 + ky;
        const bool oky = iy >= 0 && iy < a.H;
#pragma unroll
        for (int kx = 0; kx < 5; ++kx) {
            const int ix = 2 * ox0 - 1 + kx;
            const bool ok = oky && ix >= 0 && ix < a.W;
            const int off = iy * a.W + ix;
#pragma unroll
            for (int ci = 0; ci < 3; ++ci) in[ci][ky][kx] = ok ? to_f<T>(xb[ci * a.H * a.W + off]) : 0.f;
        }
    }
    float2 acc0[CH / 2], acc1[CH / 2];            // pixel 0 / pixel 1, channel pairs of this half
#pragma unroll
    for (int c = 0; c < CH / 2; ++c) { acc0[c] = make_float2(0.f, 0.f); acc1[c] = make_float2(0.f, 0.f); }
    const float* swh = sw + half * CH;
#pragma unroll
    for (int ci = 0; ci < 3; ++ci)
#pragma unroll
        for (int ky = 0; ky < 3; ++ky)
#pragma unroll
            for (int kx = 0; kx < 3; ++kx) {
                const int tap = (ci * 3 + ky) * 3 + kx;
                const float2 v0 = make_float2(in[ci][ky][kx], in[ci][ky][kx]);
                const float2 v1 = make_float2(in[ci][ky][kx + 2], in[ci][ky][kx + 2]);
#pragma unroll
                for (int c4 = 0; c4 < CH / 4; ++c4) {
                    const float4 w4 = *reinterpret_cast<const float4*>(swh + tap * C0 + 4 * c4);
                    acc0[2 * c4] = __ffma2_rn(v0, make_float2(w4.x, w4.y), acc0[2 * c4]);
                    acc0[2 * c4 + 1] = __ffma2_rn(v0, make_float2(w4.z, w4.w), acc0[2 * c4 + 1]);
                    acc1[2 * c4] = __ffma2_rn(v1, make_float2(w4.x, w4.y), acc1[2 * c4]);
                    acc1[2 * c4 + 1] = __ffma2_rn(v1, make_float2(w4.z, w4.w), acc1[2 * c4 + 1]);
                }
            }
    // per pixel: conv output rounded to the storage type (as the stand-alone convolution would leave it),
    // + bias, LayerNorm in fp32 over both halves (one exchange with the neighbouring lane), GELU on the fp32
    // value (LayerNorm runs and returns fp32 under autocast), one rounding at the store
    const float* bh = sb + half * CH;
    auto finish = [&](float2 (&acc)[CH / 2], int ox, bool store) {
        float s = 0.f;
#pragma unroll
        for (int c = 0; c < CH / 2; ++c) {
            acc[c].x = round_to<T>(acc[c].x) + bh[2 * c];
            acc[c].y = round_to<T>(acc[c].y) + bh[2 * c + 1];
            s += acc[c].x + acc[c].y;
        }
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        const float mean = s * (1.f / C0);
        float q = 0.f;
#pragma unroll
        for (int c = 0; c < CH / 2; ++c) {
            const float dx = acc[c].x - mean, dy = acc[c].y - mean;
            q = fmaf(dx, dx, q); q = fmaf(dy, dy, q);
        }
        q += __shfl_xor_sync(0xffffffffu, q, 1);
        const float rstd = rsqrtf(q * (1.f / C0) + a.eps);
        T* out = (T*)a.y + (((long long)b * a.Ho + oy) * a.Wo + ox) * C0 + half * CH;
#pragma unroll
        for (int c8 = 0; c8 < CH / 8; ++c8) {
            float o[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int c = 4 * c8 + j;
                float2 v;
                v.x = fmaf((acc[c].x - mean) * rstd, bh[C0 + 2 * c], bh[2 * C0 + 2 * c]);
                v.y = fmaf((acc[c].y - mean) * rstd, bh[C0 + 2 * c + 1], bh[2 * C0 + 2 * c + 1]);
                float2 r;
                if constexpr (sizeof(T) == 2) r = gelu_pair_poly(v);
                else r = make_float2(act_f<ACT_GELU>(v.x), act_f<ACT_GELU>(v.y));
                o[2 * j] = r.x; o[2 * j + 1] = r.y;
            }
            if (store) Vec<T, 8>::store(out + 8 * c8, o);
        }
    };
    finish(acc0, ox0, live);
    finish(acc1, two ? ox0 + 1 : ox0, live && two);
}

// Tensor-core form for 16-bit images: the convolution of 16 output pixels is one 16 x C0 x 32 contraction
// (27 taps, zero-padded) of mma.sync m16n8k16 steps.  A CTA walks output rows: the three input rows of the
// three colour planes are staged in shared memory (zero frame included), warp w takes output pixels
// 16 w .. 16 w + 15 of the row, gathers its im2col fragment from the staged rows (16 two-byte loads) and
// keeps the weight fragments in registers for all its rows.  In the accumulator layout a pixel's C0 channels
// sit in the four lanes of a quad, so the LayerNorm statistics need two shuffles; bias, LayerNorm and GELU
// run on the accumulators and the quad stores 16 contiguous bytes per eight channels.
// The FMA form above issues 61 instructions per output value, 16 of them packed FMAs; here the contraction
// costs 1.5 per output and what remains is the GELU.
template <typename T, int C0>
__global__ void __launch_bounds__(512, 1) stem_mma_kernel(const StemArgs a, int rows_total, int vec_ok) {
    extern __shared__ __align__(16) unsigned char stem_smem[];
    constexpr int NT = C0 / 8;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nthreads = blockDim.x;
    const int g = lane >> 2, t4 = lane & 3;
    const int ntiles = (a.Wo + 15) / 16, nwarps = nthreads >> 5;
    const int XP = 32 * ntiles + 16;                          // staged columns -8 .. 32 * tiles + 7: image column 0 sits 16-byte aligned
    T* xs = reinterpret_cast<T*>(stem_smem);                  // [3 colours][3 rows][XP]
    float* sb = reinterpret_cast<float*>(stem_smem + (((size_t)9 * XP * sizeof(T) + 15) & ~(size_t)15));   // bias, ln weight, ln bias
    for (int i = tid; i < C0; i += nthreads) {
        sb[i] = a.cbias ? a.cbias[i] : 0.f;
        sb[C0 + i] = a.lnw ? a.lnw[i] : 1.f;
        sb[2 * C0 + i] = a.lnb ? a.lnb[i] : 0.f;
    }
    // weight fragments: B[k][n] = w[n][k], k = (colour * 3 + ky) * 3 + kx, zero for k >= 27
    uint32_t bw[NT][2][2];
    {
        const T* __restrict__ w = (const T*)a.w;
        const T zero = from_f<T>(0.f);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int ks = 0; ks < 2; ++ks)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int k = ks * 16 + 8 * h + 2 * t4, co = nt * 8 + g;
                    T lo = k < 27 ? w[co * 27 + k] : zero, hi = k + 1 < 27 ? w[co * 27 + k + 1] : zero;
                    bw[nt][ks][h] = (uint32_t)(*reinterpret_cast<unsigned short*>(&lo)) | ((uint32_t)(*reinterpret_cast<unsigned short*>(&hi)) << 16);
                }
    }
    // shared-memory offsets of this lane's eight taps (pixel 0 of the row; add 2 * ox), -1 for the padding taps
    int toff[2][2][2];
#pragma unroll
    for (int ks = 0; ks < 2; ++ks)
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int k = ks * 16 + 8 * h + 2 * t4 + e;
                const int ci = k / 9, ky = (k - ci * 9) / 3, kx = k - ci * 9 - ky * 3;
                toff[ks][h][e] = k < 27 ? (ci * 3 + ky) * XP + kx + 7 : -1;
            }

    // Input rows: with rows of whole 16-byte pieces the next output row's three input rows per colour are read
    // into registers while the current row is computed, and go to shared memory as 16-byte stores.
    const int W8 = a.W >> 3;
    const bool vec_fill = vec_ok != 0;
    uint4 pre[3];
    auto load_row = [&](int row) {
        const int b = row / a.Ho, oy = row - b * a.Ho;
        const T* __restrict__ xb = (const T*)a.x + (long long)b * 3 * a.H * a.W;
#pragma unroll
        for (int sl = 0; sl < 3; ++sl) {
            const int i = tid + sl * nthreads;
            pre[sl] = make_uint4(0u, 0u, 0u, 0u);
            if (i < 9 * W8) {
                const int r = i / W8, c8 = i - r * W8;
                const int ci = r / 3, ky = r - ci * 3, iy = 2 * oy - 1 + ky;
                if (iy >= 0 && iy < a.H) pre[sl] = __ldg(reinterpret_cast<const uint4*>(xb + ((long long)ci * a.H + iy) * a.W + 8 * c8));
            }
        }
    };
    auto store_row = [&]() {
#pragma unroll
        for (int sl = 0; sl < 3; ++sl) {
            const int i = tid + sl * nthreads;
            if (i < 9 * W8) {
                const int r = i / W8, c8 = i - r * W8;
                *reinterpret_cast<uint4*>(xs + r * XP + 8 + 8 * c8) = pre[sl];
            }
        }
    };
    for (int i = tid; i < 9 * XP; i += nthreads) xs[i] = from_f<T>(0.f);      // the frame around the image stays zero
    if (vec_fill && (int)blockIdx.x < rows_total) load_row(blockIdx.x);
    __syncthreads();
    for (int row = blockIdx.x; row < rows_total; row += gridDim.x) {
        const int b = row / a.Ho, oy = row - b * a.Ho;
        if (vec_fill) store_row();
        else {
            const T* __restrict__ xb = (const T*)a.x + (long long)b * 3 * a.H * a.W;
            for (int i = tid; i < 9 * a.W; i += nthreads) {
                const int r = i / a.W, ix = i - r * a.W;          // r = colour * 3 + ky
                const int ci = r / 3, ky = r - ci * 3, iy = 2 * oy - 1 + ky;
                xs[r * XP + 8 + ix] = (iy >= 0 && iy < a.H) ? xb[((long long)ci * a.H + iy) * a.W + ix] : from_f<T>(0.f);
            }
        }
        __syncthreads();
        if (vec_fill && row + (int)gridDim.x < rows_total) load_row(row + gridDim.x);      // in flight during the contraction
        for (int tile = warp; tile < ntiles; tile += nwarps) {
        const int ox_lo = 16 * tile + g, ox_hi = ox_lo + 8;
        float acc[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) { acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f; }
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
            uint32_t af[4];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                unsigned short v[2][2];                       // [pixel lo / hi][tap e]
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int o = toff[ks][h][e];
                    v[0][e] = o >= 0 ? reinterpret_cast<const unsigned short*>(xs)[o + 2 * ox_lo] : (unsigned short)0;
                    v[1][e] = o >= 0 ? reinterpret_cast<const unsigned short*>(xs)[o + 2 * ox_hi] : (unsigned short)0;
                }
                af[2 * h] = (uint32_t)v[0][0] | ((uint32_t)v[0][1] << 16);          // row g,     k 2t (+8h), 2t+1
                af[2 * h + 1] = (uint32_t)v[1][0] | ((uint32_t)v[1][1] << 16);      // row g + 8
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) MmaK16<T>::run(acc[nt], af, bw[nt][ks]);
        }
        // per pixel (two per lane: rows g and g + 8): conv output rounded to the storage type, + bias, LayerNorm in fp32
        // across the quad, GELU, one rounding at the store
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const int ox = hh ? ox_hi : ox_lo;
            float2 v[NT];
            float s = 0.f;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const float2 bb = *reinterpret_cast<const float2*>(sb + nt * 8 + 2 * t4);
                v[nt].x = round_to<T>(acc[nt][2 * hh]) + bb.x;
                v[nt].y = round_to<T>(acc[nt][2 * hh + 1]) + bb.y;
                s += v[nt].x + v[nt].y;
            }
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            const float mean = s * (1.f / C0);
            float q = 0.f;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const float dx = v[nt].x - mean, dy = v[nt].y - mean;
                q = fmaf(dx, dx, q); q = fmaf(dy, dy, q);
            }
            q += __shfl_xor_sync(0xffffffffu, q, 1);
            q += __shfl_xor_sync(0xffffffffu, q, 2);
            const float rstd = rsqrtf(q * (1.f / C0) + a.eps);
            if (ox < a.Wo) {
                T* out = (T*)a.y + (((long long)b * a.Ho + oy) * a.Wo + ox) * C0 + 2 * t4;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const float2 lw = *reinterpret_cast<const float2*>(sb + C0 + nt * 8 + 2 * t4);
                    const float2 lb = *reinterpret_cast<const float2*>(sb + 2 * C0 + nt * 8 + 2 * t4);
                    float2 n2;
                    n2.x = fmaf((v[nt].x - mean) * rstd, lw.x, lb.x);
                    n2.y = fmaf((v[nt].y - mean) * rstd, lw.y, lb.y);
                    const float2 r = gelu_pair_poly(n2);
                    *reinterpret_cast<uint32_t*>(out + nt * 8) = Half2Of<T>::pack(r.x, r.y);
                }
            }
        }
        }
        __syncthreads();                                      // every fragment of this row has been gathered
    }
}

template <typename T>
static int launch_stem_mma(const StemArgs& a, int C0, cudaStream_t st) {
    const int tiles = (a.Wo + 15) / 16;
    const int threads = 32 * (tiles < 16 ? tiles : 16);
    const int XP = 32 * tiles + 16;
    const int vec_ok = (a.W % 8 == 0 && aligned_to(a.x, 16) && 9 * (a.W / 8) <= 3 * threads) ? 1 : 0;
    const size_t smem = (((size_t)9 * XP * sizeof(T) + 15) & ~(size_t)15) + 3 * (size_t)C0 * sizeof(float);
    const long long rows = (long long)a.B * a.Ho;
    // persistent CTAs, four per SM's worth (224 x 224 images, batch 128: 2 or 4 per SM 164 us, 8: 169, 32: 184)
    const unsigned grid = (unsigned)(rows < 148 * 4 ? rows : 148 * 4);
    if (C0 == 32) stem_mma_kernel<T, 32><<<grid, threads, smem, st>>>(a, (int)rows, vec_ok);
    else if (C0 == 48) stem_mma_kernel<T, 48><<<grid, threads, smem, st>>>(a, (int)rows, vec_ok);
    else stem_mma_kernel<T, 64><<<grid, threads, smem, st>>>(a, (int)rows, vec_ok);
    count_launch();
    return check_launch();
}

int stem_conv_norm_act(const ss2d_stem_params* p, cudaStream_t st) {
    if (!p) return SS2D_EINVAL_NULL;
    if (!p->x || !p->weight || !p->y) return SS2D_EINVAL_NULL;
    if (!dtype_ok(p->dtype)) return SS2D_EINVAL_DTYPE;
    if (p->B <= 0 || p->H <= 0 || p->W <= 0 || p->C0 <= 0) return SS2D_EINVAL_SHAPE;
    if (p->B * p->H * p->W > 0x3fffffffLL) return SS2D_EINVAL_SHAPE;
    const size_t s = dtype_size(p->dtype);
    if (!aligned_to(p->x, s) || !aligned_to(p->weight, s) || !aligned_to(p->y, 16) || !aligned_to(p->conv_bias, 4) ||
        !aligned_to(p->ln_weight, 4) || !aligned_to(p->ln_bias, 4))
        return SS2D_EINVAL_ALIGN;
    if (p->in_channels != 3 || p->act != ACT_GELU) return SS2D_ENOTSUP;
    StemArgs a;
    a.x = p->x; a.w = p->weight; a.cbias = (const float*)p->conv_bias; a.lnw = (const float*)p->ln_weight;
    a.lnb = (const float*)p->ln_bias; a.y = p->y;
    a.B = (int)p->B; a.H = (int)p->H; a.W = (int)p->W; a.Ho = (int)((p->H + 1) / 2); a.Wo = (int)((p->W + 1) / 2);
    a.eps = p->eps;
    if (s == 2 && a.Wo <= 1024 && (long long)a.B * a.Ho <= 0x7fffffffLL && (p->C0 == 32 || p->C0 == 48 || p->C0 == 64)) {
        if (p->dtype == SS2D_BF16) return launch_stem_mma<__nv_bfloat16>(a, (int)p->C0, st);
        return launch_stem_mma<__half>(a, (int)p->C0, st);
    }
    const long long total = 2LL * a.B * a.Ho * ((a.Wo + 1) / 2);      // two threads per pixel pair
    const unsigned grid = (unsigned)((total + 127) / 128);
#define SS2D_STEM_CASE(TT, CC) stem_conv_norm_act_kernel<TT, CC><<<grid, 128, 0, st>>>(a)
#define SS2D_STEM_T(TT) \
    switch (p->C0) { case 32: SS2D_STEM_CASE(TT, 32); break; case 48: SS2D_STEM_CASE(TT, 48); break; \
                     case 64: SS2D_STEM_CASE(TT, 64); break; default: return SS2D_ENOTSUP; }
    if (p->dtype == SS2D_F32) { SS2D_STEM_T(float) }
    else if (p->dtype == SS2D_BF16) { SS2D_STEM_T(__nv_bfloat16) }
    else { SS2D_STEM_T(__half) }
#undef SS2D_STEM_T
#undef SS2D_STEM_CASE
    count_launch();
    return check_launch();
}

// ------------------------------------------------------------------------------------------------
// Pixel-major rows -> LayerNorm -> planes.  A CTA takes TP consecutive pixels (32, or 16 for wide rows):
//   A  all threads bring the rows (+ bias) into a shared fp32 tile [TP][C + 1], 16 bytes per load;
//   B  each warp computes mean and 1/std of TP/8 pixels from the tile (two passes, lanes along C);
//   C  warp w takes channels w, w+8, ...: lane = pixel, so every plane receives its TP pixels as one run
//      (the odd pitch makes the column read conflict-free).
struct RowsArgs {
    const void* in;        // (N, C)
    const float *bias, *lnw, *lnb;
    void* out;             // (C, N) with out_cs between planes
    long long N, out_cs;
    int C;
    float eps;
    unsigned magic_pieces;     // ceil(2^32 / (C / PV)), 0 for one piece per pixel
};

template <typename Tin, typename Tout, int TP>
__global__ void __launch_bounds__(256) pixels_norm_to_planes_kernel(const RowsArgs a) {
    extern __shared__ float tile[];                       // [TP][C + 1], then part[256 / TP][TP], scale[TP], shift[TP]
    const long long n0 = (long long)blockIdx.x * TP;
    const int C = a.C, P = C + 1;
    float* part = tile + TP * P;
    float* stat = part + 256;
    constexpr int PV = sizeof(Tin) == 2 ? 8 : 4;
    const int pieces = C / PV;
    const int live = (int)min((long long)TP, a.N - n0);
    // A: rows (+ bias) -> tile
    for (int idx = threadIdx.x; idx < live * pieces; idx += 256) {
        const int pp = a.magic_pieces ? (int)__umulhi((unsigned)idx, a.magic_pieces) : idx, c = (idx - pp * pieces) * PV;
        float v[PV], bv[PV];
        Vec<Tin, PV>::load((const Tin*)a.in + (n0 + pp) * C + c, v);
        if (a.bias) Vec<float, PV>::load(a.bias + c, bv);
#pragma unroll
        for (int i = 0; i < PV; ++i) tile[pp * P + c + i] = a.bias ? v[i] + bv[i] : v[i];
    }
    __syncthreads();
    // B: statistics.  Thread (pixel pl, slice sl) sums the channels sl, sl + NS, ... of its pixel (the odd
    // pitch keeps the 32 pixels of a warp on different banks); the NS partial sums meet in shared memory.
    constexpr int NS = 256 / TP;
    const int pl = threadIdx.x % TP, sl = threadIdx.x / TP;
    float s = 0.f;
#pragma unroll 4
    for (int c = sl; c < C; c += NS) s += tile[pl * P + c];
    part[sl * TP + pl] = s;
    __syncthreads();
    float mean = 0.f;
#pragma unroll
    for (int k = 0; k < NS; ++k) mean += part[k * TP + pl];
    mean /= C;
    float q = 0.f;
#pragma unroll 4
    for (int c = sl; c < C; c += NS) { const float d = tile[pl * P + c] - mean; q = fmaf(d, d, q); }
    __syncthreads();                                      // every partial sum has been read
    part[sl * TP + pl] = q;
    __syncthreads();
    if (sl == 0) {
        float qq = 0.f;
#pragma unroll
        for (int k = 0; k < NS; ++k) qq += part[k * TP + pl];
        const float rstd = rsqrtf(qq / C + a.eps);
        stat[pl] = rstd; stat[TP + pl] = -mean * rstd;
    }
    __syncthreads();
    // C: thread = four consecutive pixels of one channel -> one 16-byte (fp32) or 8-byte (16-bit) store
    constexpr int Q4 = TP / 4;                            // threads per channel
    const int p4 = (threadIdx.x % Q4) * 4, cw = threadIdx.x / Q4;
    if (p4 < live) {
        float sc[4], sh[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) { sc[i] = stat[p4 + i]; sh[i] = stat[TP + p4 + i]; }
        const bool full = p4 + 4 <= live && ((a.out_cs | n0) & 3) == 0;
#pragma unroll 2
        for (int c = cw; c < C; c += 256 / Q4) {
            const float w = a.lnw ? __ldg(a.lnw + c) : 1.f, bb = a.lnb ? __ldg(a.lnb + c) : 0.f;
            float o[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) o[i] = fmaf(fmaf(tile[(p4 + i) * P + c], sc[i], sh[i]), w, bb);
            Tout* dst = (Tout*)a.out + (long long)c * a.out_cs + n0 + p4;
            if (full) Vec<Tout, 4>::store(dst, o);
            else {
#pragma unroll
                for (int i = 0; i < 4; ++i) if (p4 + i < live) dst[i] = from_f<Tout>(o[i]);
            }
        }
    }
}

int pixels_norm_to_planes(const ss2d_relayout_params* p, cudaStream_t st) {
    if (!p) return SS2D_EINVAL_NULL;
    if (!p->rows || !p->planes) return SS2D_EINVAL_NULL;
    if (!dtype_ok(p->rows_dtype) || !dtype_ok(p->planes_dtype)) return SS2D_EINVAL_DTYPE;
    if (p->N <= 0 || p->C <= 0) return SS2D_EINVAL_SHAPE;
    const size_t sr = dtype_size(p->rows_dtype), sp = dtype_size(p->planes_dtype);
    const int pv = sr == 2 ? 8 : 4;
    if (p->C % pv != 0) return SS2D_ENOTSUP;
    if (!aligned_to(p->rows, 16) || !aligned_to(p->planes, 16) || !aligned_to(p->bias, 16) || !aligned_to(p->ln_weight, 4) ||
        !aligned_to(p->ln_bias, 4))
        return SS2D_EINVAL_ALIGN;
    const long long cs = p->plane_stride ? p->plane_stride : p->N;
    if (cs < p->N) return SS2D_EINVAL_STRIDE;
    if (p->add || p->sum_out) return SS2D_ENOTSUP;
    RowsArgs a;
    a.in = p->rows; a.bias = (const float*)p->bias; a.lnw = (const float*)p->ln_weight; a.lnb = (const float*)p->ln_bias;
    a.out = p->planes; a.N = p->N; a.out_cs = cs; a.C = (int)p->C; a.eps = p->eps;
    a.magic_pieces = (p->C / pv) > 1 ? (unsigned)(((1ULL << 32) + (unsigned long long)(p->C / pv) - 1) / (unsigned long long)(p->C / pv)) : 0u;
    const int tp = p->C <= 512 ? 32 : 16;
    const size_t smem = ((size_t)tp * (p->C + 1) + 256 + 2 * tp) * sizeof(float);
    if (smem > 200 * 1024) return SS2D_ENOTSUP;
    const long long ctas = (p->N + tp - 1) / tp;
    if (ctas > 0x7fffffffLL) return SS2D_EINVAL_SHAPE;
#define SS2D_ROWS_LAUNCH_TP(TI, TO, TPV) { auto kern = pixels_norm_to_planes_kernel<TI, TO, TPV>; \
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return SS2D_ECUDA; \
        kern<<<(unsigned)ctas, 256, smem, st>>>(a); }
#define SS2D_ROWS_LAUNCH(TI, TO) { if (tp == 32) SS2D_ROWS_LAUNCH_TP(TI, TO, 32) else SS2D_ROWS_LAUNCH_TP(TI, TO, 16) }
    const int ri = p->rows_dtype, po = p->planes_dtype;
    if (ri == SS2D_F32 && po == SS2D_F32) SS2D_ROWS_LAUNCH(float, float)
    else if (ri == SS2D_BF16 && po == SS2D_F32) SS2D_ROWS_LAUNCH(__nv_bfloat16, float)
    else if (ri == SS2D_BF16 && po == SS2D_BF16) SS2D_ROWS_LAUNCH(__nv_bfloat16, __nv_bfloat16)
    else if (ri == SS2D_F16 && po == SS2D_F32) SS2D_ROWS_LAUNCH(__half, float)
    else if (ri == SS2D_F16 && po == SS2D_F16) SS2D_ROWS_LAUNCH(__half, __half)
    else return SS2D_EINVAL_DTYPE;
#undef SS2D_ROWS_LAUNCH_TP
#undef SS2D_ROWS_LAUNCH
    count_launch();
    return check_launch();
}

// ------------------------------------------------------------------------------------------------
// Planes -> pixel-major rows, with the residual update in front: v = planes (+ add + bias); v is
// optionally written back to the fp32 planes, and leaves as a 16-bit (or fp32) row per pixel.
struct PlanesArgs {
    float* planes;         // (C, N) fp32, plane stride cs
    const void* add;       // (C, N) rows' dtype, same stride, or NULL
    const float* bias;     // (C) or NULL
    void* rows;            // (N, C)
    long long N, cs;
    int C, write_back;
    int quads;                 // 1: N, cs and the base addresses allow four pixels per load
    unsigned magic_pieces;     // ceil(2^32 / (C / PV)), 0 for one piece per pixel
};

template <typename T, int TP>
__global__ void __launch_bounds__(256) planes_to_pixels_kernel(const PlanesArgs a) {
    extern __shared__ float tile[];                       // [TP][C + 1]
    const long long n0 = (long long)blockIdx.x * TP;
    const int C = a.C, P = C + 1;
    if (a.quads) {
        // thread = four consecutive pixels of one channel: one 16-byte load of the planes, one 8-byte (16-bit) load
        // of `add`; a warp covers 32 pixels of four channels.  Two channels' loads are issued before the first store.
        constexpr int Q = TP / 4, CW4 = 256 / Q;
        const int p4 = (threadIdx.x % Q) * 4, cw = threadIdx.x / Q;
        if (n0 + p4 < a.N) {
            for (int c0 = cw; c0 < C; c0 += 2 * CW4) {
                float v[2][4];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int c = c0 + CW4 * j;
                    if (c < C) {
                        const long long off = (long long)c * a.cs + n0 + p4;
                        Vec<float, 4>::load_plain(a.planes + off, v[j]);
                        if (a.add) {
                            float t[4];
                            Vec<T, 4>::load((const T*)a.add + off, t);
#pragma unroll
                            for (int i = 0; i < 4; ++i) v[j][i] += t[i];
                        }
                    }
                }
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int c = c0 + CW4 * j;
                    if (c < C) {
                        if (a.bias) {
                            const float bb = __ldg(a.bias + c);
#pragma unroll
                            for (int i = 0; i < 4; ++i) v[j][i] += bb;
                        }
                        if (a.write_back) Vec<float, 4>::store(a.planes + (long long)c * a.cs + n0 + p4, v[j]);
#pragma unroll
                        for (int i = 0; i < 4; ++i) tile[(p4 + i) * P + c] = v[j][i];
                    }
                }
            }
        }
    } else {
    const int pl = threadIdx.x % TP, cw = threadIdx.x / TP;
    constexpr int CW = 256 / TP;
    const long long n = n0 + pl;
    if (n < a.N) {
        // the planes may be written back: four channels' loads are issued before the first store
        for (int c0 = cw; c0 < C; c0 += 4 * CW) {
            float v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int c = c0 + CW * j;
                if (c < C) {
                    const long long off = (long long)c * a.cs + n;
                    v[j] = a.planes[off];
                    if (a.add) v[j] += to_f<T>(((const T*)a.add)[off]);
                }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int c = c0 + CW * j;
                if (c < C) {
                    if (a.bias) v[j] += __ldg(a.bias + c);
                    if (a.write_back) a.planes[(long long)c * a.cs + n] = v[j];
                    tile[pl * P + c] = v[j];
                }
            }
        }
    }
    }
    __syncthreads();
    constexpr int PV = sizeof(T) == 2 ? 8 : 4;
    const int pieces = C / PV;
    const int live = (int)min((long long)TP, a.N - n0);
    for (int idx = threadIdx.x; idx < live * pieces; idx += 256) {
        const int pp = a.magic_pieces ? (int)__umulhi((unsigned)idx, a.magic_pieces) : idx, c = (idx - pp * pieces) * PV;
        float v[PV];
#pragma unroll
        for (int i = 0; i < PV; ++i) v[i] = tile[pp * P + c + i];
        Vec<T, PV>::store((T*)a.rows + (n0 + pp) * C + c, v);
    }
}

int planes_to_pixels(const ss2d_relayout_params* p, cudaStream_t st) {
    if (!p) return SS2D_EINVAL_NULL;
    if (!p->rows || !p->planes) return SS2D_EINVAL_NULL;
    if (!dtype_ok(p->rows_dtype) || p->planes_dtype != SS2D_F32) return SS2D_EINVAL_DTYPE;
    if (p->N <= 0 || p->C <= 0) return SS2D_EINVAL_SHAPE;
    const size_t sr = dtype_size(p->rows_dtype);
    const int pv = sr == 2 ? 8 : 4;
    if (p->C % pv != 0) return SS2D_ENOTSUP;
    if (!aligned_to(p->rows, 16) || !aligned_to(p->planes, 4) || !aligned_to(p->add, sr) || !aligned_to(p->bias, 4)) return SS2D_EINVAL_ALIGN;
    const long long cs = p->plane_stride ? p->plane_stride : p->N;
    if (cs < p->N) return SS2D_EINVAL_STRIDE;
    if (p->ln_weight || p->ln_bias) return SS2D_ENOTSUP;
    PlanesArgs a;
    a.planes = (float*)p->planes; a.add = p->add; a.bias = (const float*)p->bias; a.rows = p->rows;
    a.N = p->N; a.cs = cs; a.C = (int)p->C; a.write_back = p->sum_out != nullptr;
    a.quads = (p->N % 4 == 0 && cs % 4 == 0 && aligned_to(p->planes, 16) && aligned_to(p->add, 4 * sr)) ? 1 : 0;
    a.magic_pieces = (p->C / pv) > 1 ? (unsigned)(((1ULL << 32) + (unsigned long long)(p->C / pv) - 1) / (unsigned long long)(p->C / pv)) : 0u;
    if (p->sum_out && p->sum_out != p->planes) return SS2D_ENOTSUP;      // the update is in place
    const int tp = p->C <= 512 ? 32 : 16;
    const size_t smem = (size_t)tp * (p->C + 1) * sizeof(float);
    if (smem > 200 * 1024) return SS2D_ENOTSUP;
    const long long ctas = (p->N + tp - 1) / tp;
    if (ctas > 0x7fffffffLL) return SS2D_EINVAL_SHAPE;
#define SS2D_PLANES_LAUNCH_TP(TT, TPV) { auto kern = planes_to_pixels_kernel<TT, TPV>; \
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return SS2D_ECUDA; \
        kern<<<(unsigned)ctas, 256, smem, st>>>(a); }
#define SS2D_PLANES_LAUNCH(TT) { if (tp == 32) SS2D_PLANES_LAUNCH_TP(TT, 32) else SS2D_PLANES_LAUNCH_TP(TT, 16) }
    if (p->rows_dtype == SS2D_F32) SS2D_PLANES_LAUNCH(float)
    else if (p->rows_dtype == SS2D_BF16) SS2D_PLANES_LAUNCH(__nv_bfloat16)
    else SS2D_PLANES_LAUNCH(__half)
#undef SS2D_PLANES_LAUNCH_TP
#undef SS2D_PLANES_LAUNCH
    count_launch();
    return check_launch();
}

}  // namespace ss2d
