// LayerNorm over the channel axis of a channel-first map, fp32 statistics, with an optional fused
// residual update:   s = in (+ add) (+ add_bias[d]);   [sum_out = s];   out = LN_D(s) * weight + bias.
//
// An "item" is PV consecutive pixels of one image; items are numbered across the whole batch so
// that every lane of every warp has work whatever the map size (L = 49 or 196 pixels per image
// would otherwise leave most of a tile empty).  threadIdx.x runs along the TX items of a CTA (a
// warp's global access is one contiguous run of PV*TX elements per channel, two channels per
// warp), threadIdx.y splits the D channels.  Mean and variance are the two-pass kind (sum of squared deviations), like the torch
// operator this replaces; values stay in registers between the passes when D / NTY fits, else
// they are re-read (from L1/L2).
#include "common.cuh"

namespace ss2d {

struct NormArgs {
    const float* in;
    const void* add;
    const float* add_bias;
    float* sum_out;
    const float *w, *b;
    void* out;
    long long bs, cs;        // element strides between images and between channels (pixels are contiguous)
    long long obs, ocs;      // the same for `out`
    int D, L, nv, items;     // nv = L / PV items per image, items = B * nv
    float eps;
    int skip_norm;           // 1: out = s converted, no statistics (a fused add + cast + layout change)
    int descending;          // 1: CTAs take the items from the last to the first
};

// MODE picks what the compiler may assume.  0: nothing (every optional pointer is tested, D <= NTY * CACHE).
// 1..3 are the shapes a backbone forward uses, with D == NTY * CACHE, `in`, weight and bias present and the
// normalisation on: 1 = `in` alone; 2 = in + add, sum written back; 3 = in + add + add_bias, sum written back.
// Without the per-channel tests of the general form the kernel issues about half the instructions.
template <typename Tio, int NTY, int CACHE, int PV, int TX, int MODE>
__global__ void __launch_bounds__(TX * NTY, (NTY == 32 && CACHE > 0 && CACHE * PV <= 24) ? 2 : 1) layer_norm_cf_kernel(const NormArgs a) {
    static_assert(TX == 16 && NTY % 4 == 0, "a warp is two channel slices of 16 items");
    constexpr int NP = NTY / 2;                      // partial sums per item after the in-warp step
    __shared__ float red[2][NP][TX][PV];
    const int tx = threadIdx.x, ty = threadIdx.y;
    const int item = (a.descending ? gridDim.x - 1 - blockIdx.x : blockIdx.x) * TX + tx;
    const bool live = item < a.items;
    const int bimg = live ? item / a.nv : 0;
    const long long pix = (long long)(live ? (item - bimg * a.nv) : 0) * PV;
    const long long base = (long long)bimg * a.bs + pix;
    const float* __restrict__ src = a.in + base;
    const int D = a.D;
    const bool has_in = MODE ? true : a.in != nullptr;
    const bool has_add = MODE ? MODE >= 2 : a.add != nullptr;
    const bool has_ab = MODE ? MODE == 3 : a.add_bias != nullptr;
    const bool has_so = MODE ? MODE >= 2 : a.sum_out != nullptr;
    const Tio* __restrict__ addp = has_add ? (const Tio*)a.add + base : nullptr;
    auto in_range = [&](int d) { return MODE ? true : d < D; };

    auto fetch = [&](int d, float (&v)[PV]) {
        if (!live) {
#pragma unroll
            for (int i = 0; i < PV; ++i) v[i] = 0.f;
            return;
        }
        const long long off = (long long)d * a.cs;
        if (has_in) Vec<float, PV>::load_plain(src + off, v);      // `in` may alias `sum_out`: no read-only path
        else {
#pragma unroll
            for (int i = 0; i < PV; ++i) v[i] = 0.f;
        }
        if (has_add) {
            float t[PV];
            Vec<Tio, PV>::load(addp + off, t);
#pragma unroll
            for (int i = 0; i < PV; ++i) v[i] += t[i];
        }
        if (has_ab) {
            const float bb = __ldg(a.add_bias + d);
#pragma unroll
            for (int i = 0; i < PV; ++i) v[i] += bb;
        }
        if (has_so) Vec<float, PV>::store(a.sum_out + base + off, v);
    };
    // Sum over the NTY channel slices of an item.  A warp holds two slices of the same 16 items: one shuffle
    // adds them, the even slice parks the pair sum, and after the barrier each half of the warp adds half of
    // the NP pair sums, a second shuffle joining the halves.  `which` picks one of two buffers, so the
    // second reduction needs no barrier to protect the first one's readers.
    auto reduce_over_ty = [&](float (&v)[PV], int which) {
#pragma unroll
        for (int i = 0; i < PV; ++i) v[i] += __shfl_xor_sync(0xffffffffu, v[i], 16);
        if ((ty & 1) == 0) Vec<float, PV>::store(&red[which][ty >> 1][tx][0], v);
        __syncthreads();
        const int h = ty & 1;
#pragma unroll
        for (int i = 0; i < PV; ++i) v[i] = 0.f;
#pragma unroll
        for (int j = 0; j < NP / 2; ++j) {
            float t[PV];
            Vec<float, PV>::load_plain(&red[which][h * (NP / 2) + j][tx][0], t);
#pragma unroll
            for (int i = 0; i < PV; ++i) v[i] += t[i];
        }
#pragma unroll
        for (int i = 0; i < PV; ++i) v[i] += __shfl_xor_sync(0xffffffffu, v[i], 16);
    };

    float cache[CACHE > 0 ? CACHE : 1][PV];
    float s[PV];
#pragma unroll
    for (int i = 0; i < PV; ++i) s[i] = 0.f;
    if constexpr (CACHE > 0) {
        // All loads are issued before anything is stored: `sum_out` may be the buffer `in`, so a store
        // in between would order every later load behind it and leave one load in flight per warp.
        typename Vec<Tio, PV>::Raw addraw[CACHE];
#pragma unroll
        for (int c = 0; c < CACHE; ++c) {
            const int d = ty + c * NTY;
            if (live && in_range(d) && has_in) Vec<float, PV>::load_plain(src + (long long)d * a.cs, cache[c]);
            else {
#pragma unroll
                for (int i = 0; i < PV; ++i) cache[c][i] = 0.f;
            }
        }
        if (has_add) {
#pragma unroll
            for (int c = 0; c < CACHE; ++c) {
                const int d = ty + c * NTY;
                if (live && in_range(d)) addraw[c] = Vec<Tio, PV>::load_raw(addp + (long long)d * a.cs);
            }
        }
#pragma unroll
        for (int c = 0; c < CACHE; ++c) {
            const int d = ty + c * NTY;
            if (live && in_range(d)) {
                if (has_add) {
                    float tv[PV];
                    Vec<Tio, PV>::unpack(addraw[c], tv);
#pragma unroll
                    for (int i = 0; i < PV; ++i) cache[c][i] += tv[i];
                }
                if (has_ab) {
                    const float bb = __ldg(a.add_bias + d);
#pragma unroll
                    for (int i = 0; i < PV; ++i) cache[c][i] += bb;
                }
            }
#pragma unroll
            for (int i = 0; i < PV; ++i) s[i] += cache[c][i];
        }
        if (has_so && live) {
#pragma unroll
            for (int c = 0; c < CACHE; ++c) {
                const int d = ty + c * NTY;
                if (in_range(d)) Vec<float, PV>::store(a.sum_out + base + (long long)d * a.cs, cache[c]);
            }
        }
    } else {
        for (int d = ty; d < D; d += NTY) {
            float v[PV];
            fetch(d, v);
#pragma unroll
            for (int i = 0; i < PV; ++i) s[i] += v[i];
        }
    }
    const bool norm = MODE ? true : a.skip_norm == 0;      // uniform over the grid
    const float inv_d = 1.0f / (float)D;
    if (norm) reduce_over_ty(s, 0);
    float mean[PV], q[PV];
#pragma unroll
    for (int i = 0; i < PV; ++i) { mean[i] = norm ? s[i] * inv_d : 0.f; q[i] = 0.f; }
    // after the first pass the sum lives in sum_out (if any): re-reads must not add again
    const float* __restrict__ again = has_so ? a.sum_out + base : nullptr;
    auto refetch = [&](int d, float (&v)[PV]) {
        if (!live) {
#pragma unroll
            for (int i = 0; i < PV; ++i) v[i] = 0.f;
            return;
        }
        const long long off = (long long)d * a.cs;
        if (again) { Vec<float, PV>::load_plain(again + off, v); return; }
        if (has_in) Vec<float, PV>::load_plain(src + off, v);
        else {
#pragma unroll
            for (int i = 0; i < PV; ++i) v[i] = 0.f;
        }
        if (has_add) {
            float t[PV];
            Vec<Tio, PV>::load(addp + off, t);
#pragma unroll
            for (int i = 0; i < PV; ++i) v[i] += t[i];
        }
        if (has_ab) {
            const float bb = __ldg(a.add_bias + d);
#pragma unroll
            for (int i = 0; i < PV; ++i) v[i] += bb;
        }
    };
    if (norm) {
        if constexpr (CACHE > 0) {
#pragma unroll
            for (int c = 0; c < CACHE; ++c) {
                if (in_range(ty + c * NTY)) {
#pragma unroll
                    for (int i = 0; i < PV; ++i) { const float t = cache[c][i] - mean[i]; q[i] = fmaf(t, t, q[i]); }
                }
            }
        } else {
            for (int d = ty; d < D; d += NTY) {
                float v[PV];
                refetch(d, v);
#pragma unroll
                for (int i = 0; i < PV; ++i) { const float t = v[i] - mean[i]; q[i] = fmaf(t, t, q[i]); }
            }
        }
        reduce_over_ty(q, 1);
    }
    if (!live) return;
    float rstd[PV];
#pragma unroll
    for (int i = 0; i < PV; ++i) rstd[i] = norm ? rsqrtf(fmaf(q[i], inv_d, a.eps)) : 1.f;
    Tio* __restrict__ dst = (Tio*)a.out + (long long)bimg * a.obs + pix;
    const bool has_w = MODE ? true : (norm && a.w), has_b = MODE ? true : (norm && a.b);
    auto emit = [&](int d, const float (&v)[PV]) {
        const float g = has_w ? __ldg(a.w + d) : 1.f, be = has_b ? __ldg(a.b + d) : 0.f;
        float o[PV];
#pragma unroll
        for (int i = 0; i < PV; ++i) o[i] = fmaf((v[i] - mean[i]) * rstd[i], g, be);
        Vec<Tio, PV>::store(dst + (long long)d * a.ocs, o);
    };
    if constexpr (CACHE > 0) {
#pragma unroll
        for (int c = 0; c < CACHE; ++c) {
            const int d = ty + c * NTY;
            if (in_range(d)) emit(d, cache[c]);
        }
    } else {
        for (int d = ty; d < D; d += NTY) {
            float v[PV];
            refetch(d, v);
            emit(d, v);
        }
    }
}

// 16 items per CTA: CTAs of 128 to 512 threads, several per SM, so that the load phase of one overlaps the
// reduction / store phase of another (32 items per CTA, up to 1024 threads, was 12 % slower over a backbone
// forward); a warp's access is still one run of 16 * PV pixels per channel.
constexpr int kItemsPerCta = 16;

template <typename Tio, int NTY, int CACHE, int PV>
static void launch_one(const NormArgs& a, cudaStream_t st) {
    const dim3 grid((unsigned)((a.items + kItemsPerCta - 1) / kItemsPerCta)), block(kItemsPerCta, NTY);
    int mode = 0;
    if constexpr (CACHE > 0 && CACHE <= 32) {
        if (a.D == NTY * CACHE && a.in && a.w && a.b && !a.skip_norm) {
            if (!a.add && !a.add_bias && !a.sum_out) mode = 1;
            else if (a.add && a.sum_out) mode = a.add_bias ? 3 : 2;
        }
        if (mode == 1) { layer_norm_cf_kernel<Tio, NTY, CACHE, PV, kItemsPerCta, 1><<<grid, block, 0, st>>>(a); return; }
        if (mode == 2) { layer_norm_cf_kernel<Tio, NTY, CACHE, PV, kItemsPerCta, 2><<<grid, block, 0, st>>>(a); return; }
        if (mode == 3) { layer_norm_cf_kernel<Tio, NTY, CACHE, PV, kItemsPerCta, 3><<<grid, block, 0, st>>>(a); return; }
    }
    layer_norm_cf_kernel<Tio, NTY, CACHE, PV, kItemsPerCta, 0><<<grid, block, 0, st>>>(a);
}

template <typename Tio>
static void launch_norm(NormArgs a, int pv, long long B, cudaStream_t st) {
    const int D = a.D;
    // registers hold CACHE * PV values per thread: at most 48 while D <= 192, at most 24 beyond
    // (more threads per CTA: keep about 64 registers per thread so that several CTAs share an SM)
    if (D > 32 * 32) pv = 1;
    else if (D > 16 * 12 && pv > 2) pv = 2;
    a.nv = a.L / pv;
    a.items = (int)(B * a.nv);
    // widths that are 16 per channel slice (128, 256, 512: the VMamba-B dims) get exact shapes of their own,
    // so that the specialised forms apply to them as well
    if (D == 8 * 16 || D == 16 * 16 || D == 32 * 16) {
        if (pv > 2) pv = 2;
        a.nv = a.L / pv;
        a.items = (int)(B * a.nv);
        if (D == 8 * 16) { if (pv == 2) launch_one<Tio, 8, 16, 2>(a, st); else launch_one<Tio, 8, 16, 1>(a, st); }
        else if (D == 16 * 16) { if (pv == 2) launch_one<Tio, 16, 16, 2>(a, st); else launch_one<Tio, 16, 16, 1>(a, st); }
        else { if (pv == 2) launch_one<Tio, 32, 16, 2>(a, st); else launch_one<Tio, 32, 16, 1>(a, st); }
        return;
    }
    if (D <= 8 * 12) {
        if (pv == 4) launch_one<Tio, 8, 12, 4>(a, st); else if (pv == 2) launch_one<Tio, 8, 12, 2>(a, st); else launch_one<Tio, 8, 12, 1>(a, st);
    } else if (D <= 16 * 12) {
        if (pv == 4) launch_one<Tio, 16, 12, 4>(a, st); else if (pv == 2) launch_one<Tio, 16, 12, 2>(a, st); else launch_one<Tio, 16, 12, 1>(a, st);
    } else if (D <= 32 * 12) {
        if (pv == 2) launch_one<Tio, 32, 12, 2>(a, st); else launch_one<Tio, 32, 12, 1>(a, st);
    } else if (D <= 32 * 24) {
        if (pv == 2) launch_one<Tio, 32, 24, 2>(a, st); else launch_one<Tio, 32, 24, 1>(a, st);
    } else if (D <= 32 * 32) {
        if (pv == 2) launch_one<Tio, 32, 32, 2>(a, st); else launch_one<Tio, 32, 32, 1>(a, st);
    } else if (D <= 32 * 48) {
        launch_one<Tio, 32, 48, 1>(a, st);
    } else if (D <= 32 * 64) {
        launch_one<Tio, 32, 64, 1>(a, st);
    } else {      // more channels than 512 threads can keep in registers: statistics pass, then re-read (from L2)
        launch_one<Tio, 32, 0, 1>(a, st);
    }
}

int layer_norm_cf(const ss2d_norm_params* p, cudaStream_t st) {
    if (!p) return SS2D_EINVAL_NULL;
    if ((!p->in && !p->add) || !p->out) return SS2D_EINVAL_NULL;
    if (!dtype_ok(p->io_dtype)) return SS2D_EINVAL_DTYPE;
    if (p->B <= 0 || p->D <= 0 || p->L <= 0) return SS2D_EINVAL_SHAPE;
    if (p->D > 0x7fffffffLL || p->B * p->L > 0x7fffffffLL) return SS2D_EINVAL_SHAPE;
    const long long bs = p->batch_stride ? p->batch_stride : p->D * p->L;
    const long long cs = p->channel_stride ? p->channel_stride : p->L;
    const long long obs = p->out_batch_stride ? p->out_batch_stride : bs;
    const long long ocs = p->out_channel_stride ? p->out_channel_stride : cs;
    if (cs < p->L || (p->B > 1 && bs < p->L) || ocs < p->L || (p->B > 1 && obs < p->L)) return SS2D_EINVAL_STRIDE;
    const size_t so = dtype_size(p->io_dtype);
    if (!aligned_to(p->in, 4) || !aligned_to(p->out, so) || !aligned_to(p->weight, 4) || !aligned_to(p->bias, 4) ||
        !aligned_to(p->add, so) || !aligned_to(p->add_bias, 4) || !aligned_to(p->sum_out, 4))
        return SS2D_EINVAL_ALIGN;
    // channel-major on both sides: the pixels of consecutive images follow one another, so the batch is one
    // long row per channel (wider vectors for odd map sizes such as 7 x 7)
    long long B = p->B, L = p->L;
    if (bs == L && obs == L && B * L <= 0x7fffffffLL) { L *= B; B = 1; }
    int pv = 4;
    auto fit = [&](long long x) { if (x < 0) x = -x; while (pv > 1 && (x % pv) != 0) pv >>= 1; };
    fit(L);
    if (B > 1) { fit(bs); fit(obs); }
    fit(cs); fit(ocs);
    if (p->in) fit((long long)(reinterpret_cast<uintptr_t>(p->in) / 4));
    fit((long long)(reinterpret_cast<uintptr_t>(p->out) / so));
    if (p->add) fit((long long)(reinterpret_cast<uintptr_t>(p->add) / so));
    if (p->sum_out) fit((long long)(reinterpret_cast<uintptr_t>(p->sum_out) / 4));
    NormArgs a;
    a.in = (const float*)p->in; a.add = p->add; a.add_bias = (const float*)p->add_bias; a.sum_out = (float*)p->sum_out;
    a.w = (const float*)p->weight; a.b = (const float*)p->bias; a.out = p->out;
    a.bs = bs; a.cs = cs; a.obs = obs; a.ocs = ocs; a.D = (int)p->D; a.L = (int)L; a.eps = p->eps; a.nv = 0; a.items = 0;
    a.skip_norm = p->skip_norm ? 1 : 0;
    a.descending = p->descending ? 1 : 0;
    if (p->io_dtype == SS2D_F32) launch_norm<float>(a, pv, B, st);
    else if (p->io_dtype == SS2D_BF16) launch_norm<__nv_bfloat16>(a, pv, B, st);
    else launch_norm<__half>(a, pv, B, st);
    count_launch();
    return check_launch();
}

}  // namespace ss2d
