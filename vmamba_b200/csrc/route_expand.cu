// Per-route expansion of the low-rank projections into the streams the fused scan consumes.
//
// Input: x_dbl = x_proj(x) computed ONCE on the map in its native (row-major) pixel order,
// (B, 4, R+2N, L).  For every route k this kernel writes, in the ORIENTATION order of the route
// (row-major pixels for k = 0, 2; column-major for k = 1, 3):
//   delta_k[b, d, q] = sum_r Wdt[k, d, r] * x_dbl[b, k, r, pix(q)]     (R -> D, rounded to the activation type)
//   bc_k[b, n, q]    = x_dbl[b, k, R + n, pix(q)]   n < 2N            (B then C rows, activation type)
// i.e. dt_projs (a grouped 1x1 convolution with a contraction length of only R = 6..64), the
// split/contiguous copies, and the CrossScan permutation of the projected rows, in one pass whose
// cost is the write of delta.  Two kernels: the FMA form below (fp32 maps, unaligned runs) and the
// mma.sync form further down (16-bit maps, every rank), which has no FMA loop and no weight
// broadcasts through shared memory and is 10 to 30 % faster.
//
// Mapping of the FMA form: an "item" is VEC consecutive pixels q of one (image, route) plane.  A CTA stages the
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
    const void* xt;                    // transposed rows of routes 1, 3: (2, C, Btot, Limg), or NULL (gather)
    long long xt_rs;                   // Btot * Limg
    int items_per_plane, items_total;  // L / VEC, B * L / VEC
    int mma_tiles;                     // pixel tiles per CTA of the tensor-core kernel
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
                } else if (a.xt) {
                    Vec<T, VEC>::load((const T*)a.xt + ((long long)(k >> 1) * a.C + row) * a.xt_rs + (long long)b * a.Limg + q0, v);
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

// ------------------------------------------------------------------------------------------------
// Tensor-core variant for 16-bit maps: delta tile (128 channels x 64 pixels) = W (128 x R) . X (R x 64)
// with mma.sync m16n8k16 (fp32 accumulation, R zero-padded to a multiple of 16).  The contraction is
// far too short for the tensor pipe to matter as arithmetic; what it buys is that the shared-memory
// traffic and the issue slots of the FMA loop disappear, leaving the kernel with the write of delta.
// Warp w owns channels [16 w, 16 w + 16) of the CTA's slice and all 64 pixels; the accumulators go
// through a shared tile so that every channel row leaves as 16-byte vectors.
constexpr int kMmaPix = 64;

constexpr int kMmaTilesPerCta = 8;      // most pixel tiles per CTA: the staged weights then serve 512 pixels

// PIX pixels per step.
template <typename T, int KP, int PIX>
__global__ void __launch_bounds__(256) route_expand_mma_kernel(const ExpandArgs a) {
    constexpr int KPAD = KP + 8;                  // row pitch (elements) of the operand tiles: conflict-free fragment loads
    constexpr int OPAD = PIX + 8;
    __shared__ __align__(16) T Ws[kDChunk * KPAD];     // [channel][k]
    __shared__ __align__(16) T Xt[PIX * KPAD];     // [pixel][k]
    __shared__ __align__(16) T Os[kDChunk * OPAD];     // [channel][pixel]
    const int k = blockIdx.y;
    const bool col = (k & 1) != 0;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int tiles_per_run = (a.L + PIX - 1) / PIX;
    const int groups_per_run = (tiles_per_run + a.mma_tiles - 1) / a.mma_tiles;
    const int b = blockIdx.x / groups_per_run;
    const int tile0 = (blockIdx.x - b * groups_per_run) * a.mma_tiles;
    const T* __restrict__ xd = (const T*)a.xd + (long long)k * a.xd_ks + (long long)b * a.xd_bs;
    const int dc = blockIdx.z * kDChunk;
    const int dn = min(kDChunk, a.D - dc);
    const T zero = from_f<T>(0.f);

    // ---- weights of this channel slice, [channel][k], zero beyond R and beyond the slice ----------------
    const T* __restrict__ wk = (const T*)a.wdt + (long long)k * a.D * a.R;
    if ((a.R & 7) == 0 && (reinterpret_cast<uintptr_t>(wk) & 15) == 0) {       // rows of whole 16-byte pieces
        for (int i = tid; i < kDChunk * (KP / 8); i += 256) {
            const int dl = i / (KP / 8), r = (i - dl * (KP / 8)) * 8;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (dl < dn && r < a.R) v = __ldg(reinterpret_cast<const uint4*>(wk + (long long)(dc + dl) * a.R + r));
            *reinterpret_cast<uint4*>(&Ws[dl * KPAD + r]) = v;
        }
    } else {
        for (int i = tid; i < kDChunk * KP; i += 256) {
            const int dl = i / KP, r = i - dl * KP;
            Ws[dl * KPAD + r] = (dl < dn && r < a.R) ? wk[(long long)(dc + dl) * a.R + r] : zero;
        }
    }
    // one projected row of eight pixels, gathered column-major for the odd routes
    auto fetch8 = [&](int row, int q, T (&v)[8]) {
        const T* rp = xd + (long long)row * a.xd_rs;
        if (!col) {
            *reinterpret_cast<uint4*>(v) = __ldg(reinterpret_cast<const uint4*>(rp + q));
        } else if (a.xt) {
            *reinterpret_cast<uint4*>(v) = __ldg(reinterpret_cast<const uint4*>(
                (const T*)a.xt + ((long long)(k >> 1) * a.C + row) * a.xt_rs + (long long)b * a.Limg + q));
        } else {
            const int img0 = (q / a.Limg) * a.Limg, qi = q - img0;
            int w = qi / a.H, h = qi - w * a.H, base = img0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                v[j] = rp[base + h * a.W + w];
                if (++h == a.H) { h = 0; if (++w == a.W) { w = 0; base += a.Limg; } }
            }
        }
    };
    const int g = lane >> 2, t4 = lane & 3;
    const int m0 = warp * 16;
    // X tile, transposed to [pixel][k]; rows R .. KP-1 are zero.  Consecutive threads take consecutive rows of the
    // same eight pixels, so the transposed stores of a warp fall into consecutive words.  The tile is read from
    // global memory into registers one step ahead: the loads of tile t+1 are in flight while tile t is contracted.
    constexpr int NI = (KP * (PIX / 8) + 255) / 256;
    T pre[NI][8];
    auto load_tile = [&](int q0) {
#pragma unroll
        for (int n = 0; n < NI; ++n) {
            const int i = tid + n * 256;
#pragma unroll
            for (int j = 0; j < 8; ++j) pre[n][j] = zero;
            if (i < KP * (PIX / 8)) {
                const int p0 = (i / KP) * 8, r = i - (i / KP) * KP;
                if (r < a.R && q0 + p0 < a.L) fetch8(r, q0 + p0, pre[n]);      // L is a multiple of 8: a chunk is wholly inside or outside
            }
        }
    };
    auto store_tile = [&]() {
#pragma unroll
        for (int n = 0; n < NI; ++n) {
            const int i = tid + n * 256;
            if (i < KP * (PIX / 8)) {
                const int p0 = (i / KP) * 8, r = i - (i / KP) * KP;
#pragma unroll
                for (int j = 0; j < 8; ++j) Xt[(p0 + j) * KPAD + r] = pre[n][j];
            }
        }
    };
    if (tile0 * PIX < a.L) { load_tile(tile0 * PIX); store_tile(); }
    for (int tt = 0; tt < a.mma_tiles; ++tt) {
        const int q0 = (tile0 + tt) * PIX;
        if (q0 >= a.L) break;                        // uniform over the CTA
        const bool has_next = tt + 1 < a.mma_tiles && q0 + PIX < a.L;
        if (has_next) load_tile(q0 + PIX);
        // ---- B / C rows pass through (first channel slice only) ---------------------------------------------
        if (blockIdx.z == 0) {
            for (int i = tid; i < a.N2 * (PIX / 8); i += 256) {
                const int n = i / (PIX / 8), p0 = (i - n * (PIX / 8)) * 8;
                const int q = q0 + p0;
                if (q >= a.L) continue;
                T v[8];
                fetch8(a.R + n, q, v);
                *reinterpret_cast<uint4*>((T*)a.bc[k] + b * a.bc_bs[k] + (long long)n * a.bc_rs[k] + q) = *reinterpret_cast<const uint4*>(v);
            }
        }
        __syncthreads();                             // X tile (and, first time, the weights) in place

        // ---- 16 channels x 64 pixels per warp ---------------------------------------------------------------
        float acc[PIX / 8][4];
#pragma unroll
        for (int nt = 0; nt < PIX / 8; ++nt) { acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f; }
#pragma unroll
        for (int k0 = 0; k0 < KP; k0 += 16) {
            uint32_t af[4];
            af[0] = *reinterpret_cast<const uint32_t*>(&Ws[(m0 + g) * KPAD + k0 + 2 * t4]);
            af[1] = *reinterpret_cast<const uint32_t*>(&Ws[(m0 + g + 8) * KPAD + k0 + 2 * t4]);
            af[2] = *reinterpret_cast<const uint32_t*>(&Ws[(m0 + g) * KPAD + k0 + 2 * t4 + 8]);
            af[3] = *reinterpret_cast<const uint32_t*>(&Ws[(m0 + g + 8) * KPAD + k0 + 2 * t4 + 8]);
#pragma unroll
            for (int nt = 0; nt < PIX / 8; ++nt) {
                uint32_t bf[2];
                bf[0] = *reinterpret_cast<const uint32_t*>(&Xt[(nt * 8 + g) * KPAD + k0 + 2 * t4]);
                bf[1] = *reinterpret_cast<const uint32_t*>(&Xt[(nt * 8 + g) * KPAD + k0 + 2 * t4 + 8]);
                MmaK16<T>::run(acc[nt], af, bf);
            }
        }
        // ---- accumulators -> shared tile -> 16-byte stores along the pixels -----------------------------------
#pragma unroll
        for (int nt = 0; nt < PIX / 8; ++nt) {
            T lo[2] = {from_f<T>(acc[nt][0]), from_f<T>(acc[nt][1])};
            T hi[2] = {from_f<T>(acc[nt][2]), from_f<T>(acc[nt][3])};
            *reinterpret_cast<uint32_t*>(&Os[(m0 + g) * OPAD + nt * 8 + 2 * t4]) = *reinterpret_cast<const uint32_t*>(lo);
            *reinterpret_cast<uint32_t*>(&Os[(m0 + g + 8) * OPAD + nt * 8 + 2 * t4]) = *reinterpret_cast<const uint32_t*>(hi);
        }
        __syncthreads();                             // output tile complete; every read of the X tile is done
        if (has_next) store_tile();                  // next X tile into the same buffer; the barrier at the top of the next step orders it
        T* __restrict__ dout = (T*)a.delta[k] + b * a.d_bs[k] + q0;
        for (int i = tid; i < kDChunk * (PIX / 8); i += 256) {
            const int dl = i / (PIX / 8), p0 = (i - dl * (PIX / 8)) * 8;
            if (dl < dn && q0 + p0 < a.L)
                *reinterpret_cast<uint4*>(dout + (long long)(dc + dl) * a.d_cs[k] + p0) = *reinterpret_cast<const uint4*>(&Os[dl * OPAD + p0]);
        }
        // the barrier at the top of the next step orders the next writes of the output tile behind these reads
    }
}

template <typename T>
static int launch_expand_mma(ExpandArgs a, cudaStream_t st) {
    const int kp = (a.R + 15) / 16 * 16;
    const int pix = kMmaPix;          // 128 pixels per step were measured for the shortest contraction: 4 % slower
    const long long tiles_per_run = (a.L + pix - 1) / pix;
    // Eight pixel tiles per CTA: measured over the ten launches of the 14 x 14 and 7 x 7 stages of a batch-128
    // forward, 4 and 8 tiles are equal (253 / 255 us), 16 and more leave too few CTAs, 1 or 2 re-stage the weights
    // too often.
    const int per = kMmaTilesPerCta;
    a.mma_tiles = per;
    const long long tiles = (long long)a.B * ((tiles_per_run + per - 1) / per);
    if (tiles > 0x7fffffffLL) return SS2D_EINVAL_SHAPE;
    const dim3 grid((unsigned)tiles, 4, (unsigned)((a.D + kDChunk - 1) / kDChunk));
    if (kp == 16) route_expand_mma_kernel<T, 16, kMmaPix><<<grid, 256, 0, st>>>(a);
    else if (kp == 32) route_expand_mma_kernel<T, 32, kMmaPix><<<grid, 256, 0, st>>>(a);
    else if (kp == 48) route_expand_mma_kernel<T, 48, kMmaPix><<<grid, 256, 0, st>>>(a);
    else if (kp == 64) route_expand_mma_kernel<T, 64, kMmaPix><<<grid, 256, 0, st>>>(a);
    else return SS2D_ENOTSUP;
    count_launch();
    return check_launch();
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

// Plane transposes of the projected rows of the two column-major routes: (route 1|3, row c, image b) plane
// H x W (row-major) -> W x H, written as (2, C, Btot, L).  A CTA takes a few planes through shared memory
// (pitch W + 1), reads and writes coalesced.
struct TransArgs {
    const void* xd;
    void* xt;
    long long xd_bs, xd_ks, xd_rs;
    int C, B, H, W, L, planes, vec_ok;  // planes = 2 * C * B; vec_ok: every plane start is 16-byte aligned
};

template <typename T>
__global__ void __launch_bounds__(256) plane_transpose_kernel(const TransArgs a) {
    extern __shared__ __align__(16) unsigned char traw[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int P = a.W + 1, psz = a.H * P;
    T* tile = reinterpret_cast<T*>(traw) + (size_t)warp * psz;     // one plane per warp: no CTA barrier
    constexpr int PV = 16 / (int)sizeof(T);
    const bool vec = (a.L % PV) == 0 && a.vec_ok;
    for (int pid = blockIdx.x * nwarps + warp; pid < a.planes; pid += gridDim.x * nwarps) {
        const int b = pid % a.B, c = (pid / a.B) % a.C, kk = pid / (a.B * a.C);
        const T* src = (const T*)a.xd + (long long)(2 * kk + 1) * a.xd_ks + (long long)b * a.xd_bs + (long long)c * a.xd_rs;
        T* dst = (T*)a.xt + (long long)pid * a.L;
        if (vec) {
            for (int e = lane * PV; e < a.L; e += 32 * PV) {
                T v[PV];
                *reinterpret_cast<uint4*>(v) = __ldg(reinterpret_cast<const uint4*>(src + e));
                int h = e / a.W, w = e - h * a.W;
#pragma unroll
                for (int i = 0; i < PV; ++i) {
                    tile[h * P + w] = v[i];
                    if (++w == a.W) { w = 0; ++h; }
                }
            }
            __syncwarp();
            for (int q = lane * PV; q < a.L; q += 32 * PV) {
                T v[PV];
                int w = q / a.H, h = q - w * a.H;
#pragma unroll
                for (int i = 0; i < PV; ++i) {
                    v[i] = tile[h * P + w];
                    if (++h == a.H) { h = 0; ++w; }
                }
                *reinterpret_cast<uint4*>(dst + q) = *reinterpret_cast<const uint4*>(v);
            }
        } else {
            for (int e = lane; e < a.L; e += 32) { const int h = e / a.W, w = e - h * a.W; tile[h * P + w] = src[e]; }
            __syncwarp();
            for (int q = lane; q < a.L; q += 32) { const int w = q / a.H, h = q - w * a.H; dst[q] = tile[h * P + w]; }
        }
        __syncwarp();
    }
}

static bool transpose_fits(const ss2d_expand_params* p) {
    return (size_t)p->H * (p->W + 1) * dtype_size(p->act_dtype) <= 16 * 1024;
}

long long route_expand_workspace_bytes(const ss2d_expand_params* p) {
    if (!p || !dtype_ok(p->act_dtype) || p->B <= 0 || p->R <= 0 || p->N <= 0 || p->H <= 0 || p->W <= 0) return -1;
    if (!transpose_fits(p)) return 0;
    return 2 * (p->R + 2 * p->N) * p->B * p->H * p->W * (long long)dtype_size(p->act_dtype);
}

template <typename T>
static int launch_transpose(const ss2d_expand_params* p, cudaStream_t st) {
    TransArgs t;
    t.xd = p->x_dbl; t.xt = p->workspace;
    t.xd_bs = p->x_dbl_batch_stride; t.xd_ks = p->x_dbl_route_stride; t.xd_rs = p->x_dbl_row_stride ? p->x_dbl_row_stride : p->H * p->W;
    t.C = (int)(p->R + 2 * p->N); t.B = (int)p->B; t.H = (int)p->H; t.W = (int)p->W; t.L = (int)(p->H * p->W);
    t.planes = 2 * t.C * t.B;
    const size_t pv = 16 / sizeof(T);
    t.vec_ok = (t.xd_bs % pv) == 0 && (t.xd_ks % pv) == 0 && (t.xd_rs % pv) == 0 && aligned_to(p->x_dbl, 16) && aligned_to(p->workspace, 16);
    const size_t plane_bytes = ((size_t)t.H * (t.W + 1) * sizeof(T) + 15) / 16 * 16;
    int warps = (int)(32 * 1024 / plane_bytes);
    if (warps < 1) warps = 1;
    if (warps > 8) warps = 8;
    const size_t smem = plane_bytes * warps;
    auto kern = plane_transpose_kernel<T>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return SS2D_ECUDA;
    long long ctas = (t.planes + warps - 1) / warps;
    if (ctas > 148 * 16) ctas = 148 * 16;
    kern<<<(unsigned)ctas, warps * 32, smem, st>>>(t);
    count_launch();
    return check_launch();
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
    const bool mma_ok = vec == 8 && s == 2 && p->R <= 64 && (run % 8) == 0;
    const int mma_min_r = 1;      // every rank: with the pixel-tile prefetch the tensor-core kernel is 10 % faster than the FMA kernel for R = 6, 12 too
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
    a.xt = nullptr; a.xt_rs = p->B * L;
    if (p->workspace && transpose_fits(p)) {
        if (p->workspace_bytes < route_expand_workspace_bytes(p)) return SS2D_EWORKSPACE;
        if (!aligned_to(p->workspace, 16)) return SS2D_EINVAL_ALIGN;
        int tr;
        if (p->act_dtype == SS2D_F32) tr = launch_transpose<float>(p, st);
        else if (p->act_dtype == SS2D_BF16) tr = launch_transpose<__nv_bfloat16>(p, st);
        else tr = launch_transpose<__half>(p, st);
        if (tr != SS2D_OK) return tr;
        a.xt = p->workspace;
    }
    if (flat) a.B = 1;
    a.items_per_plane = (int)(run / vec);
    a.items_total = (int)((flat ? 1 : p->B) * (run / vec));
    if (mma_ok && p->R >= mma_min_r) {
        if (p->act_dtype == SS2D_BF16) return launch_expand_mma<__nv_bfloat16>(a, st);
        return launch_expand_mma<__half>(a, st);
    }
    if (p->act_dtype == SS2D_F32) return launch_expand_v<float>(a, vec, st);
    if (p->act_dtype == SS2D_BF16) return launch_expand_v<__nv_bfloat16>(a, vec, st);
    return launch_expand_v<__half>(a, vec, st);
}

}  // namespace ss2d
